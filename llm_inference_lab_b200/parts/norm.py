"""RMSNorm, fused with the residual add that precedes it."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, register_part
from .spec import PartSpec, TensorSpec


class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w  (rust/engine/src/runner/model/qwen2/kernels.rs:546-582)."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec.prefix + "weight", (spec["hidden"],), init="norm")]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.weight = self._weight(weights, "weight")
        self.eps = float(spec["eps"])

    def forward(self, x, rows=None):
        return ops.add_rmsnorm(x, self.weight, self.eps, rows=rows)

    def forward_add(self, x, delta, rows=None):
        if delta is not None and delta.dim() == 3:      # split-K partial products in 32-bit
            return ops.add_rmsnorm(x, self.weight, self.eps, partial=delta, rows=rows)
        return ops.add_rmsnorm(x, self.weight, self.eps, delta=delta, rows=rows)


class StreamRMSNorm(Norm):
    """RMS norm that reads a residual stream kept in 32-bit: y = x / sqrt(mean(x^2) + eps) * (offset + w),
    rounded to the storage type at the end.  `offset` 1 serves weights stored around zero, 0 plain ones."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec.prefix + spec.get("name", "weight"), (spec["hidden"],),
                           init="around_zero" if spec.get("offset") else "norm")]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.weight = self._weight(weights, spec.get("name", "weight"))
        self.eps = float(spec["eps"])
        self.offset = float(spec.get("offset") or 0.0)

    def forward(self, x, rows=None):
        return ops.norm_stream(x, self.eps, self.offset, weight=self.weight, rows=rows)[1]

    def forward_add(self, x, delta, rows=None):
        if delta is not None and hasattr(delta, "add_norm"):
            # a normed product is owed (`parts.block.PendingNormedAdd`): with all rows wanted, added in this
            # norm's pass; else added first
            if rows is None and delta.eps == self.eps and self.offset == 0.0:
                return delta.add_norm(x, self.weight)
            delta.add_to(x)
            return self.forward(x, rows)
        if delta is None or not hasattr(delta, "a"):      # nothing owed (or rows already rounded: `RoundedStream`)
            return self.forward(x, rows)
        # what the block before still owes the stream (`parts.block.PendingSum`): added here, in the norm's pass
        return ops.stream_add_norm(x, delta.a, delta.scale_a, delta.b, delta.scale_b, delta.mult, self.eps, self.offset,
                                   weight=self.weight, rows=rows)[1]


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "rmsnorm_stream", StreamRMSNorm)
