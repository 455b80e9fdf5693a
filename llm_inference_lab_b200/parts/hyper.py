"""A residual made of several streams (hyper-connections): the block arrangement and the norms that read it."""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..kernels import ops
from ..profiling import scoped_range
from .base import Block, Norm, register_part
from .spec import PartSpec, TensorSpec


class HyperStreamNorm(Norm):
    """RMS norm that reads a residual of `streams` 32-bit streams X [tokens, streams, hidden]:
    u = sum_s c[s] X[s] with the coefficients of the sublayer that reads (the plain sum where none are given: the
    model's last norm), then u / sqrt(mean(u^2) + eps) * w, rounded to the storage type.  `scalar`: the weight is
    one number for all coordinates (a tensor without dimensions), else one per coordinate."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        shape = () if spec.get("scalar") else (spec["hidden"],)
        return [TensorSpec(spec.prefix + spec.get("name", "weight"), shape, init="norm")]

    @classmethod
    def libraries(cls, spec, dtype):
        return [("hyper_stream", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.weight = self._weight(weights, spec.get("name", "weight")).reshape(-1).contiguous()
        self.eps = float(spec["eps"])
        self.streams = int(spec.get("streams") or 1)

    def _streams(self, x):
        return x if x.dim() == 3 else x.view(x.shape[0], 1, x.shape[1])

    def forward(self, x, rows=None, c_in=None):
        return ops.hyper_read_norm(self._streams(x), c_in, self.weight, self.eps, rows=rows)

    def forward_add(self, x, delta, rows=None):
        if delta is not None:
            if not hasattr(delta, "add_to"):
                raise ValueError("rmsnorm_hyper follows a block whose sum it cannot take")
            x = delta.add_to(x)
        return self.forward(x, rows)


register_part("norm", "rmsnorm_hyper", HyperStreamNorm)


@dataclasses.dataclass
class PendingHyperWrite:
    """What a block still owes a residual of several streams: X[r] <- sum_s mix[s, r] X[s] + out[r] * y for all
    streams at once, y a 32-bit result or split-K partial products.  The block that follows writes it in the pass
    of its first norm (`write_read`); whoever needs the streams themselves first calls `add_to`."""
    y: torch.Tensor
    mix: torch.Tensor
    out: torch.Tensor

    def add_to(self, X):
        ops.hyper_write(X, self.y, self.mix, self.out)
        return X

    def write_read(self, X, c_in, weight, eps):
        return ops.hyper_write(X, self.y, self.mix, self.out, c_in, weight, eps)


class HyperStreamBlock(Block):
    """Pre-norm sublayers on a residual of `streams` 32-bit streams X[1..S], all equal to the embedding output at
    the start.  For sublayer q (the mixer, then the feed-forward), with coefficients in[S], out[S] and mix[S, S]
    (indexed [from, to]) of its own:

        u = sum_s in[s] X[s];   y = sublayer(norm_q(u));   X[r] <- sum_s mix[s, r] X[s] + out[r] * y

    `streams` 0 is the plain pre-norm residual x <- x + sublayer(norm(x)): one stream whose coefficients are all
    one and that names no tensors.  The write that closes a sublayer runs in the pass of the norm that opens the
    next one (the block's own second norm, the next block's first, or the model's last norm, which reads the sum
    of the streams): the block hands it on as `pending`.  All of it is 32-bit; a layer may have no feed-forward."""
    decode_graph_safe = True
    n_norms = 2

    @classmethod
    def tensors(cls, spec):
        S = int(spec.get("streams") or 0)
        if not S:
            return []
        out = []
        names = spec.get("names") or ("hc1.", "hc2.")
        for q in names[: 2 if spec.get("ffn", True) else 1]:
            p = spec.prefix + q
            out += [TensorSpec(p + "in", (S,), init="fraction", keep_f32=True),
                    TensorSpec(p + "out", (S,), init="fraction", keep_f32=True),
                    TensorSpec(p + "mix", (S, S), init="fraction", keep_f32=True)]
        return out

    @classmethod
    def libraries(cls, spec, dtype):
        return [("hyper_stream", {})]

    def __init__(self, mixer, ffn, norms, spec=None, weights=None, dtype=None, device=None):
        super().__init__(mixer, ffn, norms, spec, weights, dtype, device)
        if spec is None:
            raise ValueError("hyper_stream: the block needs a spec (streams)")
        S = int(spec.get("streams") or 0)
        self.streams = max(S, 1)
        if self.streams > ops.hyper_max_streams():
            raise ValueError(f"hyper_stream: at most {ops.hyper_max_streams()} streams, got {self.streams}")
        n_sub = 2 if ffn is not None else 1
        if len(norms) < n_sub or any(type(n) is not HyperStreamNorm for n in norms[:n_sub]):
            raise ValueError("hyper_stream: one rmsnorm_hyper per sublayer")
        names = spec.get("names") or ("hc1.", "hc2.")
        self.coef = []
        for q in names[:n_sub]:
            if S:
                get = lambda n: weights[spec.prefix + q + n].to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
                self.coef.append((get("in").reshape(-1), get("out").reshape(-1), get("mix").reshape(S, S)))
            else:
                one = torch.ones((1,), dtype=torch.float32, device=device)
                self.coef.append((one, one, one.view(1, 1)))

    def forward(self, x, pending, ctx, cache):
        if x.dim() == 2:       # the embedding output: every stream starts as a copy of it
            if pending is not None:
                raise ValueError("hyper_stream: a sum is owed to rows that are not streams yet")
            x = ops.hyper_expand(x, self.streams)
        elif x.shape[1] != self.streams:
            raise ValueError("hyper_stream: the number of streams changed between layers")
        (in1, out1, mix1), n1 = self.coef[0], self.norms[0]
        with scoped_range(self.mixer_range):
            if pending is None:
                h = n1.forward(x, c_in=in1)
            elif isinstance(pending, PendingHyperWrite):
                h = pending.write_read(x, in1, n1.weight, n1.eps)
            else:
                raise ValueError("hyper_stream follows a block whose sum it cannot take")
            a = self.mixer.forward(h, ctx, cache)
        if self.ffn is None:
            return x, PendingHyperWrite(a, mix1, out1)
        (in2, out2, mix2), n2 = self.coef[1], self.norms[1]
        with scoped_range(self.ffn_range):
            h = ops.hyper_write(x, a, mix1, out1, in2, n2.weight, n2.eps)
            f = self.ffn.forward(h, ctx)
        return x, PendingHyperWrite(f, mix2, out2)


register_part("block", "hyper_stream", HyperStreamBlock)
