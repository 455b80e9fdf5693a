"""Grouped-query attention with rotary positions on neighbouring pairs, a window that keeps the first tokens,
and a softmax with one more in its denominator."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import PagedKV, PartSpec, TensorSpec


class PairRopeAttention(Mixer):
    """q = W_q h, k = W_k h, v = W_v h (`bias`: each with a bias, and one on W_o); `heads` query heads and `kv_heads`
    key/value heads of `dim` entries (query head h reads key/value head h // (heads / kv_heads)), values of `vdim`.
    `values_from_keys`: no W_v; the values are the keys as projected, before their rotation (vdim == dim).

    Of every q and k head the first `rot_dims` entries are rotated: entries 2i and 2i + 1 by the angle
    position * `rot_base`^(-2i / rot_dims); the rest pass unchanged.  score = q . k * `scale`.  A query at
    position i sees key j <= i if i - j < `window` or j < `keep_first` (`window` 0: every j <= i); kept keys
    keep their true positions.  `sink_one`: the softmax's denominator holds one more, exp(0), a key without
    a value.  W_o closes.

    One product forms q, k (and v) in 32-bit; one kernel adds the biases, rotates, rounds q and writes k and v
    to their page slots.  Heads are cached `ops.padded_head(dim, vdim)` wide with zeros beyond their own size."""
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
        inv = np.power(float(spec["rot_base"]), -2.0 * i / max(self.rot_dims, 1)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(device)
        w = lambda n: self._weight(weights, n)  # noqa: E731
        names = ("q", "k") if self.from_keys else ("q", "k", "v")
        self.w_in = torch.cat([w(n) for n in names], dim=0).contiguous()
        self.bias_in = torch.cat([w(n + ".b") for n in names], dim=0).contiguous() if spec.get("bias") else None
        self.k_at = self.n_q * self.dim
        self.v_at = self.k_at if self.from_keys else self.k_at + self.n_kv * self.dim
        # the heads' outputs come `head` wide: zero columns of W_o meet the padding
        w_o = torch.zeros((w("o").shape[0], self.n_q, self.head), dtype=dtype, device=w("o").device)
        w_o[:, :, : self.vdim] = w("o").view(-1, self.n_q, self.vdim)
        self.w_o = w_o.view(-1, self.n_q * self.head).contiguous()
        self.bias_o = w("o.b") if spec.get("bias") else None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        group = ctx.groups[cache.group]
        proj = ops.linear(x, self.w_in, None, out_f32=True, allow_partial=True)
        write = cache.write
        q = ops.rope_pairs_store(proj, self.bias_in, ctx.row_pos, self.inv_freq, self.rot_dims,
                                 group.row_slot if write else None, cache.k, cache.v, self.n_q, self.n_kv, self.dim,
                                 self.vdim, self.head, self.k_at, self.v_at, self.dtype)
        attn = ops.attention(q, cache.k, cache.v, ctx, group, self.n_q, self.n_kv, self.head, self.window, self.scale,
                             keep_first=self.keep_first, sink_one=self.sink_one)
        if self.bias_o is not None:
            return ops.linear(attn, self.w_o, self.bias_o, out_f32=True)
        return ops.linear(attn, self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "pair_rope_attention", PairRopeAttention)
