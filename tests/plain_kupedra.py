"""A plain, slow NumPy implementation of the Kupedra design: whole sequences, no cache, one
function per mechanism, 64-bit floats.  It shares no code with the engine; the tests hold the
engine against it.

Notation: X[t, s] is stream s of the residual at token t (positions count from 0), h a sublayer's
input, W_name the matrix stored [out, in] and applied as W h.  A model folder's config.json gives
every size and constant; what the design fixes (1.702, 1e-6 in the memory's denominator, the
pairing of rotated entries) stands here as a literal.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------
# reading a model folder (safetensors: 8-byte length, JSON header, data)
# ---------------------------------------------------------------------------------------------
def read_folder(folder):
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(info["dtype"])
        w[name] = a.reshape(info["shape"])
    return cfg, w


# ---------------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def unit_rms(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return unit_rms(x, eps) * float(np.asarray(g).reshape(-1)[0])


def rotate_pairs(v, positions, base, dims, factor=1.0):
    """Entries (2i, 2i + 1), i < dims / 2, of the last axis of v [tokens, heads, n] turn by the angle
    position * base^(-2i / dims) / factor; entries from `dims` on stay."""
    out = np.array(v, dtype=np.float64, copy=True)
    half = dims // 2
    if half == 0:
        return out
    freq = float(base) ** (-2.0 * np.arange(half) / dims) / float(factor)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    cs, sn = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
    return out


def sink_softmax(scores, seen, sink):
    """Softmax over the seen keys of scores [heads, queries, keys] whose denominator also holds
    exp(sink[head]): a key without a value.  sink 0 is 'one more in the denominator'."""
    s = np.where(seen, scores, -np.inf)
    sink = np.asarray(sink, dtype=np.float64).reshape(-1, 1, 1)
    top = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - top)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - top))


def distance_bucket(n, rows, far):
    """The row of a distance table with `rows` rows for the distance n >= 0: the first rows / 2 distances have
    a row each, larger ones share rows on a logarithmic scale that reaches the last row at `far`."""
    half = rows // 2
    if n < half:
        return n
    if half == 0:            # a table of one row serves every distance
        return 0
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def grouped_scores(q, k, heads, kv_heads):
    """q [tokens, heads, d], k [tokens, kv_heads, d] -> [heads, queries, keys]; query head h reads key head
    h // (heads / kv_heads)."""
    per = heads // kv_heads
    return np.stack([q[:, h, :] @ k[:, h // per, :].T for h in range(heads)])


def weighted_values(p, v, heads, kv_heads):
    per = heads // kv_heads
    return np.stack([p[h] @ v[:, h // per, :] for h in range(heads)], axis=1)      # [tokens, heads, vdim]


# ---------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------
def rotary_attention(h, w, p, m, eps):
    """Mixer 'attention': rotated q and k, each head then over its own root mean square, a temperature per
    head on the scaled score, causal, one more in the denominator."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, V)
    rot = m.get("rot")
    if rot is not None:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_pairs(q, pos, rot["base"], rot["dims"], factor)
        k = rotate_pairs(k, pos, rot["base"], rot["dims"], factor)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    s = grouped_scores(q, k, H, G) * m["scale"] * w[p + "temp"].reshape(H, 1, 1)
    seen = pos[None, :] <= pos[:, None]
    out = weighted_values(sink_softmax(s, seen[None], np.zeros(H)), v, H, G)
    return out.reshape(T, H * V) @ w[p + "o"].T


def biased_attention(h, w, p, m, eps):
    """Left half of mixer 'parallel': q and k normed per head with a weight shared by the heads, no rotation,
    q grown with its position, a learned bias by distance on the scaled score, causal, a learned sink."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = unit_rms((h @ w[p + "q"].T).reshape(T, H, D), eps) * w[p + "q.norm"]
    k = unit_rms((h @ w[p + "k"].T).reshape(T, G, D), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(T, G, V)
    qt = m.get("q_temp")
    if qt is not None:
        grow = 1.0 + qt["coef"] * np.log(np.floor((pos + 1) / qt["every"]) + 1.0)
        q = q * grow[:, None, None]
    s = grouped_scores(q, k, H, G) * m["scale"]
    rel = w[p + "rel"]                                          # [rows, heads]
    rows = rel.shape[0]
    bucket = np.array([distance_bucket(n, rows, m["bias_max"]) for n in range(T)])
    dist = np.maximum(pos[:, None] - pos[None, :], 0)
    s = s + np.transpose(rel[bucket[dist]], (2, 0, 1))
    seen = pos[None, :] <= pos[:, None]
    out = weighted_values(sink_softmax(s, seen[None], w[p + "sink"]), v, H, G)
    return out.reshape(T, H * V) @ w[p + "o"].T


def matrix_memory(h, w, p, m, eps):
    """Right half of mixer 'parallel': a matrix memory per head with exponential input gate, sigmoid forget
    gate in the log domain, and a running maximum that keeps the exponentials in range."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                 # [T, H] log input gate
    gf = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))    # [T, H] log forget gate
    S = np.zeros((H, D, V))
    n = np.zeros((H, D))
    top = np.zeros(H)
    out = np.zeros((T, H, V))
    for t in range(T):
        new = np.maximum(gf[t] + top, gi[t])
        keep, take = np.exp(gf[t] + top - new), np.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        top = new
        num = np.einsum("hdv,hd->hv", S, q[t])
        den = np.maximum(np.abs(np.einsum("hd,hd->h", n, q[t])), np.exp(-top)) + 1e-6
        out[t] = num / den[:, None]
    out = unit_rms(out, eps).reshape(T, H * V) * w[p + "norm"]
    out = out * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    """Both halves read the same h; each result is RMS-normed over the width with its weight; half the sum."""
    left = unit_rms(biased_attention(h, w, p + "left.", m["left"], eps), eps) * w[p + "left.out"]
    right = unit_rms(matrix_memory(h, w, p + "right.", m["right"], eps), eps) * w[p + "right.out"]
    return 0.5 * (left + right)


# ---------------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------------
def capped_expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routed_experts(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    out = np.zeros_like(h)
    each = [capped_expert(h, w, f"{p}e{e}.", mlp["expert"]["limit"]) for e in range(E)]
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-s[t, e], e))[:top]
        for e in order:
            out[t] += s[t, e] * each[e][t]            # the scores as they are: not renormalised
    shared = mlp.get("shared")
    if shared is not None:
        out = out + capped_expert(h, w, p + "shared.", shared["limit"]) * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer(X, w, p, q, eps, fn):
    """One sublayer on the streams X [tokens, streams, width]: read a mix of the streams, run, write back."""
    if f"{p}hc{q}.in" in w:
        c_in, c_out, c_mix = w[f"{p}hc{q}.in"], w[f"{p}hc{q}.out"], w[f"{p}hc{q}.mix"]
    else:                      # no streams configured: the plain residual x + sublayer(norm(x))
        c_in, c_out, c_mix = np.ones(1), np.ones(1), np.ones((1, 1))
    u = np.einsum("s,tsw->tw", c_in, X)
    y = fn(scalar_norm(u, w[f"{p}norm{q}"], eps))
    return np.einsum("sr,tsw->trw", c_mix, X) + c_out[None, :, None] * y[:, None, :]


def forward(cfg, w, tokens, layers_out=None):
    """Logits [tokens, vocab] of one sequence; `layers_out` (a list) receives the sum of the streams after
    every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    X = np.repeat(x[:, None, :], int(cfg.get("streams") or 1), axis=1)
    for i in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            mix = lambda h: rotary_attention(h, w, p + "mix.", m, eps)  # noqa: E731
        else:
            mix = lambda h: parallel_mixer(h, w, p + "mix.", m, eps)  # noqa: E731
        X = sublayer(X, w, p, 1, eps, mix)
        if layer.get("mlp") is not None:
            X = sublayer(X, w, p, 2, eps, lambda h: routed_experts(h, w, p + "mlp.", layer["mlp"]))
        if layers_out is not None:
            layers_out.append(X.sum(axis=1))
    x = scalar_norm(X.sum(axis=1), w["final.norm"], eps)
    return (x @ w["head"].T) * cfg["logit_scale"]
