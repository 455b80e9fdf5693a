"""Grouped-query attention with rotary positions on neighbouring pairs, a window that keeps the first tokens,
a softmax with one more (or a learned term) in its denominator, and, as options, a norm per head on q and k,
temperatures on q, and a learned bias by distance."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import PagedKV, PartSpec, TensorSpec


def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of a distance table of `rows` rows that serves the distance n >= 0."""
    half = rows // 2
    if n < half or half == 0:
        return min(n, rows - 1)
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_table(rel: torch.Tensor, rows: int, far: float) -> torch.Tensor:
    """The learned table `rel` [rows, heads] laid out by distance for the attention kernels: [heads, L] 32-bit,
    entry n the bias of distance n; L ends where every later distance reads the last row, so the kernels clamp."""
    if rel.shape[0] != rows or rows < 1 or (rows // 2 >= 1 and not far > rows // 2):
        raise ValueError("pair_rope_attention: dist_bias is (rows of the table, a distance beyond rows // 2)")
    last = 0
    while distance_bucket(last, rows, far) < rows - 1 and last < (1 << 20):
        last += 1
    index = torch.tensor([distance_bucket(n, rows, far) for n in range(last + 1)], dtype=torch.long, device=rel.device)
    return rel.to(torch.float32)[index].t().contiguous()


class PairRopeAttention(Mixer):
    """q = W_q h, k = W_k h, v = W_v h (`bias`: each with a bias, and one on W_o); `heads` query heads and `kv_heads`
    key/value heads of `dim` entries (query head h reads key/value head h // (heads / kv_heads)), values of `vdim`.
    `values_from_keys`: no W_v; the values are the keys as projected, before their rotation (vdim == dim).

    Of every q and k head the first `rot_dims` entries are rotated: entries 2i and 2i + 1 by the angle
    position * `rot_base`^(-2i / rot_dims); the rest pass unchanged.  score = q . k * `scale`.  A query at
    position i sees key j <= i if i - j < `window` or j < `keep_first` (`window` 0: every j <= i); kept keys
    keep their true positions.  `sink_one`: the softmax's denominator holds one more, exp(0), a key without
    a value.  W_o closes.

    Further options, each off unless named:
    `rot_scaling`: every rotation frequency is divided by this factor (positions stretched linearly).
    `head_norm` "unit": after the rotation every q and k head is divided by its root mean square over `dim`
    (`eps` inside the root); "weight": and multiplied by a weight of `dim` entries shared by all heads (tensors
    `q.norm`, `k.norm`).
    `head_temp`: the score of query head h is multiplied by a learned number (tensor `temp` [heads]).
    `q_temp` (coef, every): q at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).
    `sink_learned`: the softmax's denominator holds exp(sink_h), a learned number per head (tensor `sink`): a key
    without a value whose score is not scaled and gets no bias.
    `dist_bias` (rows, far): a learned number per head is added to the scaled score by the distance n = i - j: tensor
    `rel` [rows, heads] (rows -1: as many as the checkpoint stores), row n for n < rows // 2, else min(rows - 1, rows // 2 + floor(ln(n / (rows // 2)) /
    ln(far / (rows // 2)) * (rows - rows // 2))): later rows share distances on a logarithmic scale that reaches
    the last row at `far`.

    One product forms q, k (and v) in 32-bit; one kernel adds the biases, rotates, norms, applies the
    temperatures, rounds q and writes k and v to their page slots.  Heads are cached `ops.padded_head(dim, vdim)`
    wide with zeros beyond their own size.  `forward_inner` leaves the heads' outputs for a caller that owns the
    output projection (mixers side by side)."""
    decode_graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, H, G, D, V, p = spec["hidden"], spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"], spec.prefix
        out = [TensorSpec(p + "q", (H * D, h)), TensorSpec(p + "k", (G * D, h)), TensorSpec(p + "o", (h, H * V))]
        if not spec.get("values_from_keys"):
            out.append(TensorSpec(p + "v", (G * V, h)))
        if spec.get("bias"):
            out += [TensorSpec(p + "q.b", (H * D,), init="bias"), TensorSpec(p + "k.b", (G * D,), init="bias"),
                    TensorSpec(p + "o.b", (h,), init="bias")]
            if not spec.get("values_from_keys"):
                out.append(TensorSpec(p + "v.b", (G * V,), init="bias"))
        if spec.get("head_norm") == "weight":
            out += [TensorSpec(p + "q.norm", (D,), init="norm"), TensorSpec(p + "k.norm", (D,), init="norm")]
        if spec.get("head_temp"):
            out.append(TensorSpec(p + "temp", (H,), init="norm"))
        if spec.get("sink_learned"):
            out.append(TensorSpec(p + "sink", (H,), init="bias"))
        if spec.get("dist_bias"):
            out.append(TensorSpec(p + "rel", (int(spec["dist_bias"][0]), H), init="bias"))
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec):
        window = int(spec.get("window") or 0)
        return PagedKV(spec["kv_heads"], ops.padded_head(spec["dim"], spec["vdim"]), window,
                       int(spec.get("keep_first") or 0) if window else 0)

    @classmethod
    def libraries(cls, spec, dtype):
        out = [("rope_pairs", {})]
        head = ops.padded_head(spec["dim"], spec["vdim"])
        if dtype == torch.bfloat16 and ops.attention_tc_supported(head):
            out.append(("attention_tc", {"LAB_HEAD_DIM": head}))
            if head in (64, 128):
                out.append(("attention_tc05", {"LAB_HEAD_DIM": head}))
        else:
            out.append(("attention_plain", {}))
        return out

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.n_q, self.n_kv, self.dim, self.vdim = (int(spec[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
        if self.n_q % self.n_kv:
            raise ValueError("pair_rope_attention: heads must be a multiple of kv_heads")
        self.from_keys = bool(spec.get("values_from_keys"))
        if self.from_keys and self.vdim != self.dim:
            raise ValueError("pair_rope_attention: values taken from the keys have the keys' size (vdim == dim)")
        self.head = ops.padded_head(self.dim, self.vdim)
        if self.head > 256:
            raise ValueError(f"pair_rope_attention: heads of {max(self.dim, self.vdim)} entries exceed the kernels' 256")
        self.scale = float(spec["scale"])
        self.window, self.keep_first = int(spec.get("window") or 0), int(spec.get("keep_first") or 0)
        self.sink_one = bool(spec.get("sink_one"))
        self.rot_dims = int(spec.get("rot_dims", self.dim))
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dim:
            raise ValueError("pair_rope_attention: rot_dims must be even and at most dim")
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        inv = np.power(float(spec.get("rot_base") or 1.0), -2.0 * i / max(self.rot_dims, 1))
        inv = (inv / float(spec.get("rot_scaling") or 1.0)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(device)
        # the options that take the kernel with a norm per head and temperatures
        self.head_norm = spec.get("head_norm")
        if self.head_norm not in (None, "unit", "weight"):
            raise ValueError(f"pair_rope_attention: head_norm {self.head_norm!r} is not one of 'unit', 'weight'")
        self.eps = float(spec.get("eps") or 0.0)
        if self.head_norm and not self.eps > 0.0:
            raise ValueError("pair_rope_attention: a norm per head needs eps")
        f32 = lambda n: weights[spec.prefix + n].to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        self.head_temp = f32("temp") if spec.get("head_temp") else None
        self.q_temp = tuple(spec["q_temp"]) if spec.get("q_temp") else None
        if self.q_temp is not None and (len(self.q_temp) != 2 or int(self.q_temp[1]) < 1):
            raise ValueError("pair_rope_attention: q_temp is (coef, every) with every >= 1")
        self.sink = f32("sink") if spec.get("sink_learned") else None
        self.dist_bias = None
        if spec.get("dist_bias"):
            rows, far = int(spec["dist_bias"][0]), float(spec["dist_bias"][1])
            rel = f32("rel")
            self.dist_bias = distance_table(rel, rows if rows > 0 else rel.shape[0], far)     # -1: as many as stored
        self.prep = bool(self.head_norm or self.head_temp is not None or self.q_temp is not None)
        w = lambda n: self._weight(weights, n)  # noqa: E731
        names = ("q", "k") if self.from_keys else ("q", "k", "v")
        self.w_in = torch.cat([w(n) for n in names], dim=0).contiguous()
        self.bias_in = torch.cat([w(n + ".b") for n in names], dim=0).contiguous() if spec.get("bias") else None
        self.norm_q = w("q.norm") if self.head_norm == "weight" else None
        self.norm_k = w("k.norm") if self.head_norm == "weight" else None
        self.k_at = self.n_q * self.dim
        self.v_at = self.k_at if self.from_keys else self.k_at + self.n_kv * self.dim
        # the heads' outputs come `head` wide: zero columns of W_o meet the padding
        w_o = torch.zeros((w("o").shape[0], self.n_q, self.head), dtype=dtype, device=w("o").device)
        w_o[:, :, : self.vdim] = w("o").view(-1, self.n_q, self.vdim)
        self.w_o = w_o.view(-1, self.n_q * self.head).contiguous()
        self.bias_o = w("o.b") if spec.get("bias") else None
        self.out_width = self.n_q * self.head

    def forward_inner(self, x: torch.Tensor, ctx: StepContext, cache: CacheView, out=None, mult: float = 1.0, proj=None):
        """The heads' outputs side by side [tokens, heads * padded head] in the storage type: what `w_o` reads.
        `proj`: the 32-bit product of x with `w_in`, where the caller has formed it already (as columns of a wider
        one)."""
        if out is not None or mult != 1.0:
            raise ValueError("pair_rope_attention: the heads' outputs leave unscaled, in a buffer of their own")
        group = ctx.groups[cache.group]
        if proj is None:
            proj = ops.linear(x, self.w_in, None, out_f32=True, allow_partial=True)
        write = cache.write
        slots = group.row_slot if write else None
        if self.prep:
            coef, every = self.q_temp if self.q_temp is not None else (0.0, 0)
            q = ops.head_prep_store(proj, self.bias_in, ctx.row_pos, self.inv_freq, self.rot_dims, slots, cache.k,
                                    cache.v, self.n_q, self.n_kv, self.dim, self.vdim, self.head, self.k_at, self.v_at,
                                    self.dtype, norm_eps=self.eps if self.head_norm else 0.0,
                                    q_norm_w=self.norm_q, k_norm_w=self.norm_k, q_head_scale=self.head_temp,
                                    temp_coef=float(coef), temp_every=int(every))
        else:
            q = ops.rope_pairs_store(proj, self.bias_in, ctx.row_pos, self.inv_freq, self.rot_dims, slots, cache.k,
                                     cache.v, self.n_q, self.n_kv, self.dim, self.vdim, self.head, self.k_at, self.v_at,
                                     self.dtype)
        return ops.attention(q, cache.k, cache.v, ctx, group, self.n_q, self.n_kv, self.head, self.window, self.scale,
                             keep_first=self.keep_first, sink_one=self.sink_one, sink=self.sink,
                             dist_bias=self.dist_bias)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        attn = self.forward_inner(x, ctx, cache)
        if self.bias_o is not None:
            return ops.linear(attn, self.w_o, self.bias_o, out_f32=True)
        return ops.linear(attn, self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "pair_rope_attention", PairRopeAttention)
