"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, register_part
from .spec import PartSpec, TensorSpec


class GatedMLP(FeedForward):
    """down( act(x Wg^T) * (x Wu^T) ), no biases; act is SiLU
    (rust/engine/src/runner/model/qwen2/kernels.rs:1469-1486, engine.rs:1242-1293).
    Gate and up matrices are concatenated at load time; the activation and the product are
    the epilogue of their matrix product."""

    ACTS = ("silu",)
    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    @classmethod
    def names(cls, spec: PartSpec) -> dict:
        """Tensor names after the prefix; a model whose checkpoint calls them otherwise says so in `names`."""
        return {**cls.NAMES, **(spec.get("names") or {})}

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, i, p, n = spec["hidden"], spec["intermediate"], spec.prefix, cls.names(spec)
        return [TensorSpec(p + n["gate"], (i, h)), TensorSpec(p + n["up"], (i, h)), TensorSpec(p + n["down"], (h, i))]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        if spec["act"] not in self.ACTS:
            raise ValueError(f"gated_mlp: activation {spec['act']!r} is not built (known: {self.ACTS})")
        n = self.names(spec)
        self.w_gate_up = torch.cat([self._weight(weights, n["gate"]), self._weight(weights, n["up"])],
                                   dim=0).contiguous()
        self.w_down = self._weight(weights, n["down"]).contiguous()
        # True: the product leaves in 32-bit (whole, or as split-K partial sums), for a block whose
        # residual stream is 32-bit
        self.out_f32 = bool(spec.get("out_f32"))

    def forward(self, x, ctx):
        act = ops.linear_gated(x, self.w_gate_up)
        return ops.linear(act, self.w_down, None, out_f32=self.out_f32, allow_partial=True)


register_part("feed_forward", "gated_mlp", GatedMLP)


class DenseMLP(FeedForward):
    """down( act(x Wu^T + bu) ) + bd: one matrix up, an activation, one matrix down, biases optional.  `act`
    is "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) or "relu2" (max(z, 0)^2).  The activation
    is the epilogue of the up product where the product kernel has it."""

    ACTS = ("gelu_tanh", "relu2")
    NAMES = {"up": "up_proj.weight", "down": "down_proj.weight", "bias": ".bias"}

    @classmethod
    def names(cls, spec: PartSpec) -> dict:
        return {**cls.NAMES, **(spec.get("names") or {})}

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, i, p, n = spec["hidden"], spec["intermediate"], spec.prefix, cls.names(spec)
        out = [TensorSpec(p + n["up"], (i, h)), TensorSpec(p + n["down"], (h, i))]
        if spec.get("bias"):
            out += [TensorSpec(p + n["up"] + n["bias"], (i,), init="bias"),
                    TensorSpec(p + n["down"] + n["bias"], (h,), init="bias")]
        return out

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        if spec["act"] not in self.ACTS:
            raise ValueError(f"dense_mlp: activation {spec['act']!r} is not built (known: {self.ACTS})")
        n = self.names(spec)
        self.w_up = self._weight(weights, n["up"]).contiguous()
        self.w_down = self._weight(weights, n["down"]).contiguous()
        self.b_up = self._weight(weights, n["up"] + n["bias"]) if spec.get("bias") else None
        self.b_down = self._weight(weights, n["down"] + n["bias"]) if spec.get("bias") else None
        self.out_f32 = bool(spec.get("out_f32"))
        self.act = spec["act"]

    def forward(self, x, ctx):
        act = ops.linear(x, self.w_up, self.b_up, act=self.act)
        if self.out_f32 and self.b_down is None:      # a 32-bit consumer sums partial products itself
            return ops.linear(act, self.w_down, None, out_f32=True, allow_partial=True)
        return ops.linear(act, self.w_down, self.b_down, out_f32=self.out_f32)

    def forward_open(self, x, ctx):
        """(the down product without its bias, whole or as 32-bit split-K partial products; the bias or None):
        for a consumer that sums partial products and adds the bias in its own pass."""
        act = ops.linear(x, self.w_up, self.b_up, act=self.act)
        return ops.linear(act, self.w_down, None, out_f32=True, allow_partial=True), self.b_down


register_part("feed_forward", "dense_mlp", DenseMLP)
