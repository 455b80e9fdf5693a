"""Token embedding and output head."""
from __future__ import annotations

from ..kernels import ops
from .base import Embedding, Head, register_part
from .spec import PartSpec, TensorSpec


class TokenEmbedding(Embedding):
    """x[t] = table[id_t], no scaling (rust/engine/src/runner/model/qwen2/kernels.rs:46-57)."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec.prefix + "weight", (spec["vocab"], spec["hidden"]), init="table")]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.table = self._weight(weights, "weight").contiguous()
        weights[spec.prefix + "weight"] = self.table   # a tied head shares this storage

    def forward(self, token_ids, positions=None):
        return ops.embed(token_ids, self.table)


class NormedTokenEmbedding(Embedding):
    """x[t] = norm(table[id_t]) as a 32-bit residual stream: RMS norm with gain (offset + w), for
    models that normalise right after the table and keep the stream in 32-bit."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec["table"], (spec["vocab"], spec["hidden"]), init="table"),
                TensorSpec(spec["norm"], (spec["hidden"],), init="around_zero" if spec.get("offset") else "norm")]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        t = weights[spec["table"]]
        self.table = (t if t.dtype == dtype else t.to(dtype)).contiguous()
        weights[spec["table"]] = self.table
        w = weights[spec["norm"]]
        self.weight = w if w.dtype == dtype else w.to(dtype)
        self.eps, self.offset = float(spec["eps"]), float(spec.get("offset") or 0.0)

    def forward(self, token_ids, positions=None):
        return ops.embed_norm(token_ids, self.table, self.weight, self.eps, self.offset)


class TokenPositionEmbedding(Embedding):
    """x[t] = table[id_t] + positions[p_t] as a 32-bit residual stream: a learned vector per absolute
    position (the table's rows bound the longest sequence), added unscaled."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec["table"], (spec["vocab"], spec["hidden"]), init="table"),
                TensorSpec(spec["positions"], (spec["max_positions"], spec["hidden"]), init="table")]

    @classmethod
    def libraries(cls, spec, dtype):
        return [("stream32", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        t = weights[spec["table"]]
        self.table = (t if t.dtype == dtype else t.to(dtype)).contiguous()
        weights[spec["table"]] = self.table      # a tied head shares this storage
        p = weights[spec["positions"]]
        self.positions = (p if p.dtype == dtype else p.to(dtype)).contiguous()

    def forward(self, token_ids, positions=None):
        if positions is None:
            raise ValueError("token_position_embedding needs the rows' positions")
        return ops.embed_position(token_ids, positions, self.table, self.positions)


class StreamTokenEmbedding(Embedding):
    """x[t] = table[id_t] * `scale` (1 where none is given) as a 32-bit residual stream, no positions."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec["table"], (spec["vocab"], spec["hidden"]), init="table")]

    @classmethod
    def libraries(cls, spec, dtype):
        return [("stream32", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        t = weights[spec["table"]]
        self.table = (t if t.dtype == dtype else t.to(dtype)).contiguous()
        weights[spec["table"]] = self.table      # a tied head shares this storage
        self.scale = float(spec.get("scale", 1.0))

    def forward(self, token_ids, positions=None):
        return ops.embed_position(token_ids, None, self.table, None, scale=self.scale)


class LinearHead(Head):
    """logits = x W^T in 32-bit, no bias; W is the embedding table when tied
    (rust/engine/src/runner/model/qwen2/engine.rs:299-303, 1312-1319).  Options: `softcap` (cap * tanh(logits /
    cap)) and `scale` (logits * scale), both on the 32-bit logits."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        if spec.get("tied_to"):
            return []
        return [TensorSpec(spec.prefix + spec.get("name", "weight"), (spec["vocab"], spec["hidden"]))]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        tied = spec.get("tied_to")
        w = weights[tied] if tied else weights[spec.prefix + spec.get("name", "weight")]
        self.weight = (w if w.dtype == dtype else w.to(dtype)).contiguous()
        # logits <- cap * tanh(logits / cap) where the model caps them (monotonic: the greedy pick is
        # the same, a sampled one is not, so a capped head always forms its logits)
        self.softcap = float(spec.get("softcap") or 0.0)
        self.scale = float(spec.get("scale", 1.0))
        if not self.scale > 0.0:
            raise ValueError("linear_head: the logits' scale must be positive")

    @classmethod
    def libraries(cls, spec, dtype):
        return [("hyper_stream", {})] if float(spec.get("scale", 1.0)) != 1.0 else []

    def forward(self, x):
        logits = ops.linear(x, self.weight, None, out_f32=True)
        if self.scale != 1.0:
            logits = ops.scale_rows(logits, self.scale)
        return ops.softcap(logits, self.softcap) if self.softcap else logits

    def pick(self, x, temperature, seeds, positions, out=None):
        # In one pass where the tensor-core product serves: the [rows, vocab] logits are never written.
        if not self.softcap and self.scale == 1.0 and ops.head_pick_fusable(x, self.weight):
            return ops.head_pick(x, self.weight, temperature, seeds, positions, out=out)
        return super().pick(x, temperature, seeds, positions, out=out)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "normed_token_embedding", NormedTokenEmbedding)
register_part("embedding", "token_position_embedding", TokenPositionEmbedding)
register_part("embedding", "token_embedding_stream", StreamTokenEmbedding)
register_part("head", "linear_head", LinearHead)
