"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..kernels import ops
from ..profiling import scoped_range
from .base import Block, register_part
from .norm import StreamRMSNorm
from .spec import FixedState, TensorSpec


class PreNormBlock(Block):
    """r = x + mixer(norm1(x)); out = r + ffn(norm2(r))
    (rust/engine/src/runner/model/qwen2/engine.rs:1216-1296).

    The add that closes a sub-layer is fused with the norm that opens the next one, so the
    block hands its last product to the next block (or the final norm) as `pending`.
    """
    n_norms = 2

    def forward(self, x, pending, ctx, cache):
        with scoped_range(self.mixer_range):
            h = self.norms[0].forward_add(x, pending)
            a = self.mixer.forward(h, ctx, cache)
        with scoped_range(self.ffn_range):
            h = self.norms[1].forward_add(x, a)
            return x, self.ffn.forward(h, ctx)


register_part("block", "prenorm", PreNormBlock)


@dataclasses.dataclass
class PendingSum:
    """What a block still owes a 32-bit stream: x += mult * (scale_a * a + scale_b * b).  The next block's norms
    (or the final norm) add it in their own pass; whoever needs the stream itself first calls `add_to`."""
    a: torch.Tensor
    scale_a: torch.Tensor
    b: Optional[torch.Tensor]
    scale_b: Optional[torch.Tensor]
    mult: float

    def add_to(self, x):
        return ops.stream_add(x, self.a, self.scale_a, self.b, self.scale_b, self.mult)


class ParallelStreamBlock(Block):
    """Mixer and feed-forward side by side on a 32-bit residual stream, each behind a norm of its own of
    the same x:

        x <- x + mult * (s1 * mixer(shift(norm1(x))) + s2 * ffn(norm2(x)))

    Options, all parameters of the block's spec: `mult` (a constant), per-channel scales s1 and s2 of the
    two results (`scale_names`), and a token shift of the mixer's input (`shift_name`): h[t] + (h[t-1] -
    h[t]) * mix per channel, h[t-1] taken before its own shift, zeros before a sequence's first token.  The
    last unshifted row of every request is fixed-size state of the block, beside the mixer's cache.  A layer
    may have no feed-forward.  The sum is 32-bit; both results arrive as 32-bit products (or split-K partial
    products, summed in order).  As in the pre-norm block, the sum that closes a block is fused with the
    norms that open the next one: the block hands it on as `pending` (`PendingSum`)."""
    decode_graph_safe = True

    n_norms = 2

    @classmethod
    def tensors(cls, spec):
        out = []
        if spec is None:
            return out
        h, p = spec["hidden"], spec.prefix
        for name in spec.get("scale_names") or ():
            out.append(TensorSpec(p + name, (h,), init="norm"))
        if spec.get("shift_name"):
            out.append(TensorSpec(p + spec["shift_name"], (h,), init="fraction"))
        return out

    @classmethod
    def cache_need(cls, spec):
        if spec is not None and spec.get("shift_name"):
            return FixedState((spec["hidden"],))
        return None

    @classmethod
    def libraries(cls, spec, dtype):
        return [("stream32", {})]

    def __init__(self, mixer, ffn, norms, spec=None, weights=None, dtype=None, device=None):
        super().__init__(mixer, ffn, norms, spec, weights, dtype, device)
        if spec is None:
            raise ValueError("parallel_stream: the block needs a spec (hidden, mult)")
        h = spec["hidden"]

        def get(name):
            t = weights[spec.prefix + name]
            return t if t.dtype == dtype else t.to(dtype)

        names = tuple(spec.get("scale_names") or ())
        if names and len(names) < (2 if ffn is not None else 1):
            raise ValueError("parallel_stream: one scale per result")
        ones = None
        if not names:
            ones = torch.ones((h,), dtype=dtype, device=device)
        self.scale_mixer = get(names[0]) if names else ones
        self.scale_ffn = (get(names[1]) if names else ones) if ffn is not None else None
        self.mix = get(spec["shift_name"]) if spec.get("shift_name") else None
        self.mult = float(spec.get("mult", 1.0))
        n1 = norms[0]
        for n in norms[: 2 if ffn is not None else 1]:
            if type(n) is not StreamRMSNorm or (n.eps, n.offset) != (n1.eps, n1.offset):
                raise ValueError("parallel_stream: both norms are rmsnorm_stream with the same constants")

    def forward(self, x, pending, ctx, cache):
        if pending is not None and not isinstance(pending, PendingSum):
            raise ValueError("parallel_stream follows a block that leaves a sum of another kind to the next norm")
        n1 = self.norms[0]
        w2 = self.norms[1].weight if self.ffn is not None else None
        with scoped_range(self.mixer_range):
            if self.mix is not None:
                if pending is not None:
                    normed, h2 = ops.stream_add_norm(x, pending.a, pending.scale_a, pending.b, pending.scale_b,
                                                     pending.mult, n1.eps, n1.offset, weight_f32=n1.weight, weight=w2)
                else:
                    normed, h2 = ops.norm_stream(x, n1.eps, n1.offset, weight_f32=n1.weight, weight=w2)
                h1 = ops.token_shift(normed, self.mix, cache.block_state, ctx, write=cache.write)
            else:
                if pending is not None:
                    pending.add_to(x)
                h1 = ops.norm_stream(x, n1.eps, n1.offset, weight=n1.weight)[1]
                h2 = ops.norm_stream(x, n1.eps, n1.offset, weight=w2)[1] if w2 is not None else None
            a = self.mixer.forward(h1, ctx, cache)
        f = None
        if self.ffn is not None:
            with scoped_range(self.ffn_range):
                f = self.ffn.forward(h2, ctx)
        return x, PendingSum(a, self.scale_mixer, f, self.scale_ffn, self.mult)


register_part("block", "parallel_stream", ParallelStreamBlock)


@dataclasses.dataclass
class RoundedStream:
    """What a block that owes the stream nothing hands on: the rows of the stream as it left them, already
    rounded to the storage type, for a next block whose sublayers read the stream itself."""
    rows: torch.Tensor

    def add_to(self, x):      # nothing is owed
        return x


class NormedSublayersBlock(Block):
    """Each sublayer reads the 32-bit residual stream itself and its *output* is normed before the sum:

        x <- x + norm1(mixer(x));   x <- x + norm2(ffn(x))

    (RMS norms with plain weights; a layer may have no feed-forward.)  The sublayers' products arrive in
    32-bit, whole or as split-K partial products; one kernel sums them, norms, adds to the stream and leaves
    the new rows rounded for the product that reads them next, so the block hands the next one those rows
    as `pending` (`RoundedStream`) and owes the stream nothing."""
    decode_graph_safe = True

    n_norms = 2

    @classmethod
    def libraries(cls, spec, dtype):
        return [("stream32", {})]

    def __init__(self, mixer, ffn, norms, spec=None, weights=None, dtype=None, device=None):
        super().__init__(mixer, ffn, norms, spec, weights, dtype, device)
        self.dtype = dtype
        for n in norms[: 2 if ffn is not None else 1]:
            if type(n) is not StreamRMSNorm or n.offset != 0.0:
                raise ValueError("normed_sublayers_stream: the norms are rmsnorm_stream with plain weights")

    def forward(self, x, pending, ctx, cache):
        if isinstance(pending, RoundedStream):
            h = pending.rows
        else:
            if pending is not None:
                if not hasattr(pending, "add_to"):
                    raise ValueError("normed_sublayers_stream follows a block whose sum it cannot take")
                pending.add_to(x)
            h = ops.stream_round(x, self.dtype)
        n1 = self.norms[0]
        with scoped_range(self.mixer_range):
            a = self.mixer.forward(h, ctx, cache)
            h = ops.stream_norm_add(x, a, n1.weight, n1.eps, copy=self.dtype != torch.float32)
        if self.ffn is not None:
            n2 = self.norms[1]
            with scoped_range(self.ffn_range):
                if hasattr(self.ffn, "forward_open"):      # the bias joins the partial products' sum here
                    f, bias = self.ffn.forward_open(x if h is None else h, ctx)
                else:
                    f, bias = self.ffn.forward(x if h is None else h, ctx), None
                h = ops.stream_norm_add(x, f, n2.weight, n2.eps, bias=bias, copy=self.dtype != torch.float32)
        return x, RoundedStream(x if h is None else h)


register_part("block", "normed_sublayers_stream", NormedSublayersBlock)


@dataclasses.dataclass
class PendingNormedAdd:
    """What a block whose sublayers' outputs are normed still owes a 32-bit stream: x += rmsnorm(a + bias) * weight,
    `a` a 32-bit product or split-K partial products.  The norm that reads the stream next adds it in its own pass
    (`add_norm`); whoever needs the stream itself first calls `add_to`."""
    a: torch.Tensor
    weight: torch.Tensor
    eps: float
    bias: Optional[torch.Tensor] = None

    def add_to(self, x):
        ops.stream_norm_add(x, self.a, self.weight, self.eps, bias=self.bias)
        return x

    def add_norm(self, x, next_weight):
        """x += what is owed; returns rmsnorm(x) * next_weight with the same eps, rounded to the storage type."""
        return ops.stream_norm_add(x, self.a, self.weight, self.eps, bias=self.bias, next_weight=next_weight)


class SandwichStreamBlock(Block):
    """Every sublayer between two norms on a 32-bit residual stream:

        x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ffn(norm2(x)))

    (RMS norms with plain weights and one eps; a layer may have no feed-forward: two norms then.)  The
    sublayers' products arrive in 32-bit, whole or as split-K partial products; one kernel sums them, norms
    them, adds to the stream and, in the same pass, norms the new row for the sublayer that reads it next.
    The last sum of a block is left to the norm that opens the next block (or to the final norm):
    `PendingNormedAdd`."""
    decode_graph_safe = True

    n_norms = 4

    @classmethod
    def libraries(cls, spec, dtype):
        return [("stream32", {})]

    def __init__(self, mixer, ffn, norms, spec=None, weights=None, dtype=None, device=None):
        super().__init__(mixer, ffn, norms, spec, weights, dtype, device)
        want = 4 if ffn is not None else 2
        if len(norms) < want:
            raise ValueError(f"sandwich_stream: {want} norms (before and after each sublayer), got {len(norms)}")
        for n in norms[:want]:
            if type(n) is not StreamRMSNorm or n.offset != 0.0 or n.eps != norms[0].eps:
                raise ValueError("sandwich_stream: the norms are rmsnorm_stream with plain weights and one eps")

    def forward(self, x, pending, ctx, cache):
        before, after = self.norms[0], self.norms[1]
        with scoped_range(self.mixer_range):
            if pending is not None and hasattr(pending, "add_norm") and pending.eps == before.eps:
                h = pending.add_norm(x, before.weight)
            else:
                if pending is not None:
                    if not hasattr(pending, "add_to"):
                        raise ValueError("sandwich_stream follows a block whose sum it cannot take")
                    pending.add_to(x)
                h = ops.norm_stream(x, before.eps, 0.0, weight=before.weight)[1]
            a = self.mixer.forward(h, ctx, cache)
        if self.ffn is None:
            return x, PendingNormedAdd(a, after.weight, after.eps)
        before2, after2 = self.norms[2], self.norms[3]
        with scoped_range(self.ffn_range):
            h = ops.stream_norm_add(x, a, after.weight, after.eps, next_weight=before2.weight)
            f = self.ffn.forward(h, ctx)
        return x, PendingNormedAdd(f, after2.weight, after2.eps)


register_part("block", "sandwich_stream", SandwichStreamBlock)
