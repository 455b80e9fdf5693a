"""Attention whose keys and values are read from a cached low-rank latent."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import PagedLatent, PartSpec, TensorSpec


class LatentAttention(Mixer):
    """Queries through a latent: c_q = rmsnorm(W_dq h), q = W_uq c_q, per head [dim plain ; rot_dim rotated]
    (`q_rank` 0: no query latent, q = W_q h directly, tensor `q`).
    Keys and values through another: W_dkv h gives kv_rank numbers, RMS-normed into the latent c, and
    rot_dim more, rotated, one key part shared by all heads.  Per head the plain key is W_uk c and the
    value W_uv c; score = (q_plain . k_plain + q_rot . k_rot) * scale.  Only [c ; k_rot] is cached, one
    vector per position for all heads (`PagedLatent`).

    The key projection is absorbed into the query (q_lat = W_uk^T q_plain, so q_plain . W_uk c = q_lat . c)
    and the value projection applied after the weighted sum of latents, so every step reads the cache as it
    is, for prompts' portions and decoded tokens alike.  Parameters: `window` (0: all keys; else a query at
    p sees the keys j with 0 <= p - j < window), `sink` (a learned number per head that joins the softmax's
    denominator, unscaled, without key or value), rotary base and the number of rotated entries `rot_dims`
    of the rotated part (entry i pairs with i + rot_dims / 2; with `rot_pairs` entry 2i with 2i + 1), `scale`.
    `own_kv` False: the layer has no W_dkv and reads the latents another layer call caches (its cache is the
    other call's, not written here), with its own W_uk, W_uv and queries."""
    decode_graph_safe = True


    @classmethod
    def tensors(cls, spec: PartSpec):
        h, H, D, R, V = spec["hidden"], spec["heads"], spec["dim"], spec["rot_dim"], spec["vdim"]
        Q, C, p = spec["q_rank"], spec["kv_rank"], spec.prefix
        if Q:
            out = [TensorSpec(p + "dq", (Q, h)), TensorSpec(p + "dq.norm", (Q,), init="norm"),
                   TensorSpec(p + "uq", (H * (D + R), Q))]
        else:
            out = [TensorSpec(p + "q", (H * (D + R), h))]
        if spec.get("own_kv", True):
            out += [TensorSpec(p + "dkv", (C + R, h)), TensorSpec(p + "dkv.norm", (C,), init="norm")]
        out += [TensorSpec(p + "uk", (H * D, C)), TensorSpec(p + "uv", (H * V, C)), TensorSpec(p + "o", (h, H * V))]
        if spec.get("sink"):
            out.append(TensorSpec(p + "sink", (H,), init="bias"))
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return PagedLatent(spec["kv_rank"] + spec["rot_dim"], int(spec.get("window") or 0))

    # Requests that bring this many rows or more attend in the plain form on the tensor-core kernel (where it
    # serves: `ops.latent_plain_form_supported`); fewer rows, single decoded tokens above all, read the latents
    # as they are cached (the absorbed form).  0: always the absorbed form.
    PLAIN_FORM_ROWS = 16

    @classmethod
    def libraries(cls, spec, dtype):
        out = [("latent_attention", {})]
        if ops.latent_plain_form_supported(dtype, spec["dim"], spec["rot_dim"], spec["vdim"]):
            out.append(("attention_tc", {"LAB_HEAD_DIM": ops.latent_head_size(spec["dim"], spec["rot_dim"], spec["vdim"])}))
        return out

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.heads, self.dim, self.rot_dim, self.vdim = (int(spec[k]) for k in ("heads", "dim", "rot_dim", "vdim"))
        self.q_rank, self.kv_rank = int(spec["q_rank"]), int(spec["kv_rank"])
        self.window, self.scale, self.eps = int(spec.get("window") or 0), float(spec["scale"]), float(spec["eps"])
        self.rot_dims = int(spec.get("rot_dims", self.rot_dim))
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError("latent_attention: rot_dims must be even and at most rot_dim")
        self.own_kv, self.rot_pairs = bool(spec.get("own_kv", True)), bool(spec.get("rot_pairs"))
        if self.q_rank and not self.own_kv:
            raise ValueError("latent_attention: a layer that borrows its latents projects its queries directly (q_rank 0)")
        w = lambda n: self._weight(weights, n)  # noqa: E731
        # the matrices that read h and leave in 32-bit for the norms: the query's latent, then the keys' and values'
        down = ([w("dq")] if self.q_rank else []) + ([w("dkv")] if self.own_kv else [])
        self.w_down = torch.cat(down, dim=0).contiguous() if down else None
        self.norm_q = w("dq.norm") if self.q_rank else None
        self.norm_c = w("dkv.norm") if self.own_kv else None
        H, D, R, C, V = self.heads, self.dim, self.rot_dim, self.kv_rank, self.vdim
        # A head of q and of the heads' output is HD wide: the plain form's head size where it serves (keys
        # dim + rot_dim, values vdim, padded with zero rows and columns of the matrices around them), else
        # exactly what the design says.
        self.plain_form = ops.latent_plain_form_supported(dtype, D, R, V) and self.PLAIN_FORM_ROWS > 0
        self.hd_q = ops.latent_head_size(D, R, V) if self.plain_form else D + R
        self.hd_o = self.hd_q if self.plain_form else V
        w_q = w("uq") if self.q_rank else w("q")       # what forms q: from the query latent, or from h itself
        w_uq = torch.zeros((H, self.hd_q, w_q.shape[1]), dtype=dtype, device=w_q.device)
        w_uq[:, : D + R] = w_q.view(H, D + R, w_q.shape[1])
        self.w_uq = w_uq.view(H * self.hd_q, w_q.shape[1]).contiguous()
        # per head: the key projection transposed (it meets the query), the value projection as stored
        self.w_uk_t = w("uk").view(H, D, C).transpose(1, 2).contiguous()      # [H, C, D]
        self.w_uv = w("uv").view(H, V, C).contiguous()                        # [H, V, C]
        self.w_up = torch.cat([w("uk"), w("uv")], dim=0).contiguous() if self.plain_form else None
        w_o = torch.zeros((w("o").shape[0], H, self.hd_o), dtype=dtype, device=w("o").device)
        w_o[:, :, :V] = w("o").view(-1, H, V)
        self.w_o = w_o.view(-1, H * self.hd_o).contiguous()
        self.sink = weights[spec.prefix + "sink"].to(torch.float32).contiguous() if spec.get("sink") else None
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        inv = np.power(float(spec["rot_base"]), -2.0 * i / max(self.rot_dims, 1)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(device)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        group = ctx.groups[cache.group]
        H, D, R, C, V = self.heads, self.dim, self.rot_dim, self.kv_rank, self.vdim
        T = x.shape[0]
        write = cache.write and self.own_kv
        cq = x
        if self.w_down is not None:
            proj = ops.linear(x, self.w_down, None, out_f32=True)
            cq = ops.latent_prep(proj, self.q_rank, C, R, self.norm_q, self.norm_c, ctx.row_pos, self.inv_freq,
                                 self.rot_dims, group.row_slot if write else None, cache.k if write else None,
                                 self.eps, pairs=self.rot_pairs)
            if not self.q_rank:
                cq = x
        q = ops.linear(cq, self.w_uq, None)
        rows_plain = self.PLAIN_FORM_ROWS if self.plain_form else 0
        plain = rows_plain > 0 and any(n >= rows_plain for n in ctx.q_lens)
        absorbed = not plain or any(n < rows_plain for n in ctx.q_lens)
        # heads' outputs side by side, HD_o wide each; padding must be zero (it meets zero columns of W_o)
        make = torch.zeros if self.hd_o != V else torch.empty
        attn = make((T, H * self.hd_o), dtype=self.dtype, device=x.device)
        if absorbed:
            q_cat = torch.empty((T, H, C + R), dtype=torch.float32, device=x.device)
            ops.latent_q_rope(q, q_cat, H, D, R, C, ctx.row_pos, self.inv_freq, self.rot_dims, in_place=plain,
                              pairs=self.rot_pairs)
            ops.linear_heads(q.view(T, H, self.hd_q), self.w_uk_t, q_cat)
            mixed = ops.latent_attention(q_cat, cache.k, self.sink, ctx, group, H, C, self.window, self.scale,
                                         below=rows_plain if plain else 0)
            ops.linear_heads(mixed.view(T, H, C), self.w_uv, attn.view(T, H, self.hd_o))
        else:
            ops.latent_q_rope(q, None, H, D, R, C, ctx.row_pos, self.inv_freq, self.rot_dims, in_place=True,
                              pairs=self.rot_pairs)
        if plain:
            ops.latent_attention_plain_form(q, cache.k, self.w_up, self.sink, ctx, group, H, D, R, V, C, self.window,
                                            self.scale, rows_plain, attn)
        return ops.linear(attn, self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "latent_attention", LatentAttention)
