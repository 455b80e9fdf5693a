"""Recurrent mixers whose state per head is a matrix with a scalar decay, and mixers side by side."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, lookup, register_part
from .spec import CacheParts, FixedState, PartSpec, TensorSpec


class DecayLinearAttention(Mixer):
    """Linear attention with one fixed decay per head: q = silu(W_q h), k = silu(W_k h) (`heads` x `dim`),
    v = silu(W_v h) (`heads` x `vdim`); per head S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, no other
    scale.  The heads side by side are RMS-normed together with a plain weight, multiplied by sigmoid(W_g h)
    and projected by W_o.  S starts at zero, is 32-bit and is carried from token to token per request
    (`FixedState`); the recurrence, the norm and the gate are 32-bit.  The four matrices that read h are one
    product.  `decay` is a tuple with one number per head."""
    decode_graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, H, D, V, p = spec["hidden"], spec["heads"], spec["dim"], spec["vdim"], spec.prefix
        return [TensorSpec(p + "q", (H * D, h)), TensorSpec(p + "k", (H * D, h)), TensorSpec(p + "v", (H * V, h)),
                TensorSpec(p + "g", (H * V, h)), TensorSpec(p + "norm", (H * V,), init="norm"),
                TensorSpec(p + "o", (h, H * V))]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return FixedState((spec["heads"], spec["dim"], spec["vdim"]))

    @classmethod
    def libraries(cls, spec, dtype):
        return [("linear_state", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.heads, self.dim, self.vdim = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        if not ops.decay_scan_supported(self.dim):
            raise ValueError(f"decay_linear_attention: {self.dim} key channels are outside what the recurrence kernel takes")
        if len(spec["decay"]) != self.heads:
            raise ValueError("decay_linear_attention: one decay per head")
        w = lambda n: self._weight(weights, n)  # noqa: E731
        self.w_in = torch.cat([w("q"), w("k"), w("v"), w("g")], dim=0).contiguous()
        self.norm_weight = w("norm")
        self.w_o = w("o").contiguous()
        self.decay = torch.tensor([float(d) for d in spec["decay"]], dtype=torch.float32, device=device)
        self.eps = float(spec["eps"])
        self.out_width = self.heads * self.vdim

    def forward_inner(self, x, ctx: StepContext, cache: CacheView, out=None, mult: float = 1.0, proj=None):
        """The normed, gated heads side by side [tokens, heads * vdim], times `mult`, in the storage type.  `proj`:
        the whole 32-bit product of x with `w_in`, where the caller has formed it already."""
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        if proj is None:
            proj = ops.linear(x, self.w_in, None, out_f32=True)
        o = ops.decay_scan(proj[:, :hd], proj[:, hd: 2 * hd], proj[:, 2 * hd: 2 * hd + hv], cache.state, ctx, self.heads,
                           self.heads, self.dim, self.vdim, a_head=self.decay, silu=True, write=cache.write)
        return ops.gated_norm(o, proj[:, 2 * hd + hv:], self.norm_weight, self.eps, mult=mult, out=out)

    def forward(self, x, ctx, cache):
        return ops.linear(self.forward_inner(x, ctx, cache), self.w_o, None, out_f32=True, allow_partial=True)


class StateSpaceMixer(Mixer):
    """A state-space mixer with a scalar decay per head and token.  inner = heads * vdim, N = `state`,
    G = `groups`; W_in h = [z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C pass a causal
    convolution per channel over the last `taps` inputs (weights [channels, taps], the last column on the
    current token, zeros before the sequence, a bias) and SiLU.  dt <- softplus(dt + dt_bias); per head (head h
    reads group h // (heads / G)): S_t = exp(-exp(A_log_h) dt) S_{t-1} + dt B_t x_t^T (S is N x vdim),
    y_t = S_t^T C_t + D_h x_t.  y is multiplied by silu(z), RMS-normed in `norm_groups` equal parts (each by
    its own root mean square) with a weight, and projected by W_o.  Per request the mixer keeps S (32-bit)
    and the convolution's last taps - 1 inputs: two fixed-size states (`CacheParts`).  Everything after the
    input projection is 32-bit up to the rounding before W_o."""
    decode_graph_safe = True

    @classmethod
    def _sizes(cls, spec):
        inner, gn = spec["heads"] * spec["vdim"], spec["groups"] * spec["state"]
        return inner, gn, inner + 2 * gn      # inner, one of B / C, channels of the convolution

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, H, p = spec["hidden"], spec["heads"], spec.prefix
        inner, gn, channels = cls._sizes(spec)
        return [TensorSpec(p + "in", (2 * inner + 2 * gn + H, h)), TensorSpec(p + "conv", (channels, spec["taps"])),
                TensorSpec(p + "conv.b", (channels,), init="bias"), TensorSpec(p + "dt_bias", (H,), init="bias"),
                TensorSpec(p + "A_log", (H,), init="bias"), TensorSpec(p + "D", (H,), init="norm"),
                TensorSpec(p + "norm", (inner,), init="norm"), TensorSpec(p + "o", (h, inner))]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        _, _, channels = cls._sizes(spec)
        return CacheParts((FixedState((spec["heads"], spec["state"], spec["vdim"])),
                           FixedState((max(spec["taps"] - 1, 0), channels))))

    @classmethod
    def libraries(cls, spec, dtype):
        return [("linear_state", {})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.heads, self.vdim, self.state, self.groups = (int(spec[k]) for k in ("heads", "vdim", "state", "groups"))
        self.taps, self.parts, self.eps = int(spec["taps"]), int(spec["norm_groups"]), float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError("state_space: heads must be a multiple of groups")
        if not ops.decay_scan_supported(self.state):
            raise ValueError(f"state_space: a state of {self.state} is outside what the recurrence kernel takes")
        self.inner, self.gn, self.channels = self._sizes(spec)
        if self.inner % self.parts:
            raise ValueError("state_space: norm_groups must divide heads * vdim")
        w = lambda n: self._weight(weights, n)  # noqa: E731
        self.w_in = w("in").contiguous()
        self.conv_w, self.conv_b = w("conv").contiguous(), w("conv.b")
        self.dt_bias, self.a_log, self.skip = w("dt_bias"), w("A_log"), w("D")
        self.norm_weight = w("norm")
        self.w_o = w("o").contiguous()
        self.out_width = self.inner

    def forward_inner(self, x, ctx: StepContext, cache: CacheView, out=None, mult: float = 1.0, proj=None):
        inner, gn = self.inner, self.gn
        if proj is None:
            proj = ops.linear(x, self.w_in, None, out_f32=True)
        state, kept = cache.part(0), cache.part(1)
        conv, dt, decay = ops.ssm_prepare(proj, inner, 2 * inner + 2 * gn, self.channels, self.taps, self.heads,
                                          self.conv_w, self.conv_b, self.dt_bias, self.a_log, kept.state, ctx,
                                          write=cache.write)
        xs = conv[:, :inner]
        y = ops.decay_scan(conv[:, inner + gn:], conv[:, inner: inner + gn], xs, state.state, ctx, self.heads,
                           self.groups, self.state, self.vdim, a_tok=decay, s_tok=dt, write=cache.write)
        return ops.gated_norm(y, proj[:, :inner], self.norm_weight, self.eps, parts=self.parts, gate_first=True,
                              skip=self.skip, x=xs, head_size=self.vdim, mult=mult, out=out)

    def forward(self, x, ctx, cache):
        return ops.linear(self.forward_inner(x, ctx, cache), self.w_o, None, out_f32=True, allow_partial=True)


class SideBySide(Mixer):
    """Several mixers that read the same input, their results summed with a constant each:
    sum_i c_i * mixer_i(h).  `parts` is a tuple of (mixer spec, c_i).  Each mixer keeps its own cache
    (`CacheParts`, in the order of `parts`).  Mixers that take the product of the input with their `w_in` from
    the caller and leave the input of their output projection in a caller's buffer (`forward_inner`, `w_in`,
    `w_o`, `out_width`) share both products: one matrix of all their input rows meets h once, and their inner
    results, each times its constant, lie side by side and meet the output matrices side by side, so the
    weighted sum is formed inside one product.

    `out_norms` (tensor names, one per mixer) with `eps`: every mixer's result is first RMS-normed over the model
    width with a plain weight of its own, sum_i c_i * rmsnorm_i(mixer_i(h)); the mixers then share the input
    product only, each keeps its output product, and one kernel norms and sums (one or two mixers)."""

    @classmethod
    def _children(cls, spec):
        return [(lookup("mixer", part.kind), part, float(c)) for part, c in spec["parts"]]

    @classmethod
    def tensors(cls, spec: PartSpec):
        out = [t for klass, part, _ in cls._children(spec) for t in klass.tensors(part)]
        for name in spec.get("out_norms") or ():
            out.append(TensorSpec(spec.prefix + name, (spec["hidden"],), init="norm"))
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return CacheParts(tuple(klass.cache_need(part) for klass, part, _ in cls._children(spec)))

    @classmethod
    def libraries(cls, spec, dtype):
        return ([job for klass, part, _ in cls._children(spec) for job in klass.libraries(part, dtype)]
                + [("hyper_stream" if spec.get("out_norms") else "stream32", {})])

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.mixers = [(klass(part, weights, dtype, device), c) for klass, part, c in self._children(spec)]
        if not self.mixers:
            raise ValueError("side_by_side: at least one mixer")
        self.decode_graph_safe = all(getattr(m, "decode_graph_safe", False) for m, _ in self.mixers)
        self.shared = all(hasattr(m, "forward_inner") for m, _ in self.mixers)
        self.out_norms = None
        if spec.get("out_norms"):
            names = tuple(spec["out_norms"])
            if len(names) != len(self.mixers) or not 1 <= len(names) <= 2:
                raise ValueError("side_by_side: out_norms names one weight per mixer, for one or two mixers")
            self.out_norms = [self._weight(weights, n).contiguous() for n in names]
            self.eps = float(spec["eps"])
            if self.shared:
                self.w_in = torch.cat([m.w_in for m, _ in self.mixers], dim=0).contiguous()
                self.in_widths = [m.w_in.shape[0] for m, _ in self.mixers]
        elif self.shared:
            self.w_in = torch.cat([m.w_in for m, _ in self.mixers], dim=0).contiguous()
            self.in_widths = [m.w_in.shape[0] for m, _ in self.mixers]
            self.w_o = torch.cat([m.w_o for m, _ in self.mixers], dim=1).contiguous()
            self.widths = [m.out_width for m, _ in self.mixers]

    def _forward_normed(self, x, ctx: StepContext, cache: CacheView):
        results = []
        if self.shared:
            proj = ops.linear(x, self.w_in, None, out_f32=True)
            at = 0
            for i, (mixer, _) in enumerate(self.mixers):
                inner = mixer.forward_inner(x, ctx, cache.part(i), proj=proj[:, at: at + self.in_widths[i]])
                results.append(ops.linear(inner, mixer.w_o, None, out_f32=True, allow_partial=True))
                at += self.in_widths[i]
        else:
            results = [mixer.forward(x, ctx, cache.part(i)) for i, (mixer, _) in enumerate(self.mixers)]
        second = len(results) > 1
        return ops.normed_sum(results[0], self.out_norms[0], self.mixers[0][1], results[1] if second else None,
                              self.out_norms[1] if second else None, self.mixers[1][1] if second else 0.0, self.eps)

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if self.out_norms is not None:
            return self._forward_normed(x, ctx, cache)
        if self.shared:
            proj = ops.linear(x, self.w_in, None, out_f32=True)
            inner = torch.empty((x.shape[0], sum(self.widths)), dtype=self.dtype, device=x.device)
            at = at_in = 0
            for i, (mixer, c) in enumerate(self.mixers):
                mixer.forward_inner(x, ctx, cache.part(i), out=inner[:, at: at + self.widths[i]], mult=c,
                                    proj=proj[:, at_in: at_in + self.in_widths[i]])
                at, at_in = at + self.widths[i], at_in + self.in_widths[i]
            return ops.linear(inner, self.w_o, None, out_f32=True, allow_partial=True)
        total, c_total = None, 1.0
        for i, (mixer, c) in enumerate(self.mixers):
            result = mixer.forward(x, ctx, cache.part(i))
            if total is None:
                total, c_total = result, c
            else:
                total, c_total = ops.weighted_sum(total, c_total, result, c), 1.0
        if c_total != 1.0 or total.dim() == 3:
            total = ops.weighted_sum(total, c_total, total, 0.0)
        return total


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "side_by_side", SideBySide)
