"""A state-space mixer whose decay differs per channel and per entry of the state (selective scan)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import CacheParts, FixedState, PartSpec, TensorSpec


class SelectiveScanMixer(Mixer):
    """W_in h = [x: inner | z: inner].  x passes a causal convolution per channel over the last `taps` inputs
    (weights [inner, taps], the last column on the current token, zeros before the sequence, a bias) and SiLU.
    W_x x = [dt_low: dt_rank | B: state | C: state]; dt = softplus(W_dt dt_low + dt_bias), one per channel;
    A = -exp(A_log) [inner, state].  Per channel c and state entry n:

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;    y_c = sum_n S[c, n] C_n + D_c x_c

    then y * silu(z) and W_o.  Per request the mixer keeps S (32-bit, zero at the start) and the convolution's
    last taps - 1 inputs: two fixed-size states (`CacheParts`).  Everything between the projections is 32-bit:
    the convolution, step sizes, decays, the state, the skip term and the gate; the projections' inputs are
    rounded to the storage type."""
    decode_graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, I, N, R, K, p = (spec["hidden"], spec["inner"], spec["state"], spec["dt_rank"], spec["taps"], spec.prefix)
        return [TensorSpec(p + "in", (2 * I, h)), TensorSpec(p + "conv", (I, K)),
                TensorSpec(p + "conv.b", (I,), init="bias"), TensorSpec(p + "x", (R + 2 * N, I)),
                TensorSpec(p + "dt", (I, R)), TensorSpec(p + "dt.b", (I,), init="bias"),
                TensorSpec(p + "A_log", (I, N), init="bias"), TensorSpec(p + "D", (I,), init="norm"),
                TensorSpec(p + "o", (h, I))]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return CacheParts((FixedState((spec["inner"], spec["state"])),
                           FixedState((max(spec["taps"] - 1, 0), spec["inner"]))))

    @classmethod
    def libraries(cls, spec, dtype):
        return [("selective_scan", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.inner, self.state, self.rank, self.taps = (int(spec[k]) for k in ("inner", "state", "dt_rank", "taps"))
        if self.state > ops.SELECTIVE_SCAN_MAX_STATE:
            raise ValueError(f"selective_scan: a state of {self.state} entries a channel exceeds what the walk takes "
                             f"({ops.SELECTIVE_SCAN_MAX_STATE})")
        w = lambda n: self._weight(weights, n)  # noqa: E731
        self.w_in = w("in").contiguous()
        self.conv_w, self.conv_b = w("conv").contiguous(), w("conv.b")
        w_x = w("x")
        self.w_x = w_x.contiguous()
        # a 16-bit engine forms the step sizes' low-rank input rounded for its product and B, C in 32-bit: two products
        self.w_x_dt, self.w_x_bc = w_x[: self.rank].contiguous(), w_x[self.rank:].contiguous()
        self.w_dt, self.dt_bias = w("dt").contiguous(), w("dt.b")
        self.a_log, self.skip = w("A_log").contiguous(), w("D")
        self.w_o = w("o").contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        inner, N, R = self.inner, self.state, self.rank
        proj = ops.linear(x, self.w_in, None, out_f32=True)
        state, kept = cache.part(0), cache.part(1)
        x32, xt = ops.conv_silu(proj, 0, inner, self.taps, self.conv_w, self.conv_b, kept.state, ctx, write=cache.write)
        if self.dtype == torch.float32:
            low = ops.linear(xt, self.w_x, None)
            dt_low, bc, b_at = low[:, :R], low, R
        else:
            dt_low = ops.linear(xt, self.w_x_dt, None)
            bc, b_at = ops.linear(xt, self.w_x_bc, None, out_f32=True), 0
        dt_pre = ops.linear(dt_low, self.w_dt, None, out_f32=True)
        y = ops.selective_scan(x32, dt_pre, bc, b_at, b_at + N, proj[:, inner:], self.a_log, self.skip, self.dt_bias,
                               state.state, ctx, write=cache.write)
        return ops.linear(y, self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "selective_scan", SelectiveScanMixer)
