"""A recurrent mixer whose state per head is a matrix memory with exponential gates (the mLSTM cell)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import CacheParts, FixedState, PartSpec, TensorSpec


class MatrixMemory(Mixer):
    """q = W_q h * dim^(-1/2), k = W_k h (`heads` x `dim`), v = W_v h (`heads` x `vdim`); per head a log input gate
    i = cap tanh((W_i h + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f h + b_f) / cap)), cap =
    `gate_cap`.  With a running maximum m that starts at 0 (S and n start at zero):

        m_t = max(f + m_{t-1}, i)
        S_t = exp(f + m_{t-1} - m_t) S_{t-1} + exp(i - m_t) k v^T          n_t likewise with k alone
        o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + `floor`)

    Each head's o is divided by its root mean square (`eps` inside the root); the heads side by side are multiplied
    by a weight (`norm`), by sigmoid(W_g h), and projected by W_o.  Per request the mixer keeps S with n as one
    more column, and m: two fixed-size states (`CacheParts`), 32-bit, zero for a new request.  Everything after
    the input product is 32-bit up to the rounding before W_o; the six matrices that read h are one product.
    The recurrence itself is the framework's `decay_scan` with a decay and a key scale per token and head."""
    decode_graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, H, D, V, p = spec["hidden"], spec["heads"], spec["dim"], spec["vdim"], spec.prefix
        return [TensorSpec(p + "q", (H * D, h)), TensorSpec(p + "k", (H * D, h)), TensorSpec(p + "v", (H * V, h)),
                TensorSpec(p + "g", (H * V, h)), TensorSpec(p + "o", (h, H * V)),
                TensorSpec(p + "norm", (H * V,), init="norm"),
                TensorSpec(p + "i", (H, h)), TensorSpec(p + "i.b", (H,), init="bias"),
                TensorSpec(p + "f", (H, h)), TensorSpec(p + "f.b", (H,), init="bias")]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return CacheParts((FixedState((spec["heads"], spec["dim"], ops.memory_value_width(spec["vdim"]))),
                           FixedState((spec["heads"],))))

    @classmethod
    def libraries(cls, spec, dtype):
        return [("matrix_memory", {}), ("linear_state", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.heads, self.dim, self.vdim = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        if not ops.decay_scan_supported(self.dim):
            raise ValueError(f"matrix_memory: {self.dim} key channels are outside what the recurrence kernel takes")
        self.cap, self.eps = float(spec["gate_cap"]), float(spec["eps"])
        self.floor = float(spec.get("floor", 1e-6))
        if not self.cap > 0.0:
            raise ValueError("matrix_memory: gate_cap must be positive")
        w = lambda n: self._weight(weights, n)  # noqa: E731
        self.w_in = torch.cat([w("q"), w("k"), w("v"), w("g"), w("i"), w("f")], dim=0).contiguous()
        self.b_i, self.b_f = w("i.b").contiguous(), w("f.b").contiguous()
        self.norm_weight = w("norm").contiguous()
        self.w_o = w("o").contiguous()
        self.out_width = self.heads * self.vdim
        self.vpad = ops.memory_value_width(self.vdim)

    def forward_inner(self, x, ctx: StepContext, cache: CacheView, out=None, mult: float = 1.0, proj=None):
        """The normed, gated heads side by side [tokens, heads * vdim], times `mult`, in the storage type.  `proj`:
        the 32-bit product of x with `w_in`, where the caller has formed it already."""
        H, hd, hv = self.heads, self.heads * self.dim, self.heads * self.vdim
        if proj is None:
            proj = ops.linear(x, self.w_in, None, out_f32=True)
        memory, top = cache.part(0), cache.part(1)
        gates, values = ops.memory_gates(proj, 2 * hd, 2 * hd + 2 * hv, 2 * hd + 2 * hv + H, self.b_i, self.b_f, H,
                                         self.vdim, self.cap)
        m = ops.memory_stabilize(gates, top.state, ctx, write=cache.write)
        o = ops.decay_scan(proj[:, :hd], proj[:, hd: 2 * hd], values, memory.state, ctx, H, H, self.dim, self.vpad,
                           a_tok=gates[:, 0, :], s_tok=gates[:, 1, :], write=cache.write)
        return ops.memory_finish(o, m, proj[:, 2 * hd + hv: 2 * hd + 2 * hv], self.norm_weight, ctx, H, self.vdim,
                                 self.dim ** -0.5, self.floor, self.eps, mult=mult, out=out)

    def forward(self, x, ctx, cache):
        return ops.linear(self.forward_inner(x, ctx, cache), self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "matrix_memory", MatrixMemory)
