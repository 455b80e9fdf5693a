"""A routed feed-forward: a mixture of small gated experts, with an optional shared expert."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, register_part
from .spec import PartSpec, TensorSpec


class RoutedExperts(FeedForward):
    """`experts` gated feed-forwards W_down (silu(W_gate h) * (W_up h)) of `expert_ff` rows, without biases, of
    which every token uses `top`: router logits z = W_router h in 32-bit, scores softmax(z) over all experts,
    the `top` largest chosen (ties: the smaller index), weighted by their scores over the sum of the chosen
    scores (+ 1e-20).  `shared_ff` > 0: one more expert of that many rows runs for every token and is added,
    with `shared_gate` multiplied by sigmoid(W_sg h), one number per token.  `renorm` False: the weights are the
    chosen scores as they are.  `limit` > 0 (and `shared_limit` for the shared expert): the experts are of the
    capped form W_down (g' * sigmoid(1.702 g') * (u' + 1)) with g' = min(W_gate h, limit) and u' = clamp(W_up h,
    -limit, limit).

    The router's matrix and the gate's row are one product; one kernel picks, one lays the (token, expert)
    pairs out in rows grouped by expert, two grouped products run the experts, and one kernel forms the weighted
    sum, in the order of each token's choice, with the shared expert's share.  Steps of many pairs in bfloat16
    run the grouped products on the tensor cores over rows gathered into the layout; else the ordinary units
    gather while they load.  The result is 32-bit."""

    NAMES = {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "shared": "shared.",
             "shared_gate": "shared.sg"}

    @classmethod
    def names(cls, spec: PartSpec) -> dict:
        return {**cls.NAMES, **(spec.get("names") or {})}

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, E, F, p, n = spec["hidden"], spec["experts"], spec["expert_ff"], spec.prefix, cls.names(spec)
        out = [TensorSpec(p + n["router"], (E, h))]
        for e in range(E):
            q = p + n["expert"].format(e)
            out += [TensorSpec(q + n["gate"], (F, h)), TensorSpec(q + n["up"], (F, h)), TensorSpec(q + n["down"], (h, F))]
        S = int(spec.get("shared_ff") or 0)
        if S:
            q = p + n["shared"]
            out += [TensorSpec(q + n["gate"], (S, h)), TensorSpec(q + n["up"], (S, h)), TensorSpec(q + n["down"], (h, S))]
            if spec.get("shared_gate"):
                out.append(TensorSpec(p + n["shared_gate"], (1, h)))
        return out

    @classmethod
    def libraries(cls, spec, dtype):
        return [("moe", {})]       # the products' libraries belong to every model

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.experts, self.top, self.ff = int(spec["experts"]), int(spec["top"]), int(spec["expert_ff"])
        if not 0 < self.top <= self.experts:
            raise ValueError("routed_experts: top must lie in 1..experts")
        n = self.names(spec)
        w = lambda name: self._weight(weights, name)  # noqa: E731
        self.shared_ff = int(spec.get("shared_ff") or 0)
        self.gated_share = bool(self.shared_ff and spec.get("shared_gate"))
        self.renorm = bool(spec.get("renorm", True))
        self.limit, self.shared_limit = float(spec.get("limit") or 0.0), float(spec.get("shared_limit") or 0.0)
        rows = [w(n["router"])] + ([w(n["shared_gate"]).reshape(1, -1)] if self.gated_share else [])
        self.w_router = torch.cat(rows, dim=0).contiguous()
        names = [n["expert"].format(e) for e in range(self.experts)]
        self.w_gate_up = torch.stack([torch.cat([w(q + n["gate"]), w(q + n["up"])], dim=0) for q in names]).contiguous()
        self.w_down = torch.stack([w(q + n["down"]) for q in names]).contiguous()
        if self.shared_ff:
            q = n["shared"]
            self.w_shared_gate_up = torch.cat([w(q + n["gate"]), w(q + n["up"])], dim=0).contiguous()
            self.w_shared_down = w(q + n["down"]).contiguous()

    def forward(self, x, ctx):
        E, top = self.experts, self.top
        logits = ops.linear(x, self.w_router, None, out_f32=True)
        chosen, weight, gate = ops.moe_route(logits, E, top, gate_col=E if self.gated_share else -1, renorm=self.renorm)
        lay = ops.moe_layout(chosen, E, x.dtype, x.shape[1], self.ff)
        act = ops.moe_experts_up(x, self.w_gate_up, lay, top, limit=self.limit)
        y = ops.moe_experts_down(act, self.w_down, lay)
        shared = None
        if self.shared_ff:
            shared = ops.linear(ops.linear_gated(x, self.w_shared_gate_up, limit=self.shared_limit), self.w_shared_down,
                                None, out_f32=True)
        return ops.moe_combine(y, lay.pos_of, weight, shared, gate)


register_part("feed_forward", "routed_experts", RoutedExperts)
