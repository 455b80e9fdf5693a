"""A plain, slow NumPy implementation of the Bukatar design: whole sequences, no cache, one
function per mechanism, 64-bit floats.  It shares no code with the engine; the tests hold the
engine against it.

Notation: x[t] is the residual stream at token t (positions count from 0), h a sublayer's input,
W_name the matrix stored [out, in] and applied as W h.  Every sublayer sits between two norms:
x <- x + norm_after(sublayer(norm_before(x))).
"""
from __future__ import annotations

import json
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


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def relu_squared(z):
    return np.maximum(z, 0.0) ** 2


def rms_norm(x, weight, eps):
    """x over its root mean square along the last axis (eps inside the root), times a plain weight."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def rotate_pairs(v, positions, base, dims):
    """Rotary positions on neighbouring pairs: entries (2i, 2i + 1), i < dims / 2, of the last axis of
    v [tokens, ..., n] turn by the angle position * base^(-2i / dims); entries from `dims` on stay."""
    out = np.array(v, dtype=np.float64, copy=True)
    half = dims // 2
    freq = float(base) ** (-2.0 * np.arange(half) / dims)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]           # [tokens, half]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    cs, sn = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
    return out


def visible_keys(n, window=0, keep_first=0):
    """[query i, key j]: j <= i, and with a window only the last `window` keys or the first `keep_first`."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    seen = j <= i
    if window > 0:
        seen &= (i - j < window) | (j < keep_first)
    return seen


def softmax_weights(scores, seen, extra_one=False):
    """Softmax over the seen keys of scores [..., queries, keys]; `extra_one` adds 1 to the denominator
    (a key with score 0 and no value)."""
    s = np.where(seen, scores, -np.inf)
    top = s.max(axis=-1, keepdims=True)
    if extra_one:
        top = np.maximum(top, 0.0)
    e = np.exp(s - top)
    den = e.sum(axis=-1, keepdims=True)
    if extra_one:
        den = den + np.exp(-top)
    return e / den


# ---------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------
def causal_conv(x, weight, bias):
    """Per channel: out[t] = bias + sum_j weight[:, taps - 1 - j] * x[t - j], zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    out = np.tile(bias[None, :], (T, 1)).astype(np.float64)
    for j in range(taps):
        shifted = np.zeros_like(x)
        if j < T:
            shifted[j:] = x[: T - j]
        out += shifted * weight[None, :, taps - 1 - j]
    return out


def selective_scan_mixer(h, w, p, m):
    """State-space mixer with a decay per channel and state entry, token by token."""
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[p + "conv"], w[p + "conv.b"]))
    low = x @ w[p + "x"].T
    dt_low, B, C = low[:, :R], low[:, R: R + N], low[:, R + N: R + 2 * N]
    dt = softplus(dt_low @ w[p + "dt"].T + w[p + "dt.b"])            # [T, inner]
    A = -np.exp(w[p + "A_log"])                                      # [inner, N]
    S = np.zeros((inner, N))
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


def window_attention_mixer(h, w, p, m, positions=None):
    """Grouped-query attention whose values are the keys as projected (before the rotation), with a window
    that keeps the first tokens and a softmax with one more in the denominator."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, D)
    v = k
    q = rotate_pairs(q, pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_pairs(k, pos, m["rot"]["base"], m["rot"]["dims"])
    seen = visible_keys(T, m["mask"]["size"], m["mask"]["keep_first"])
    out = np.zeros((T, H, m["vdim"]))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        out[:, head] = softmax_weights(s, seen, extra_one=True) @ v[:, g]
    return out.reshape(T, -1) @ w[p + "o"].T + w[p + "o.b"]


def latent_of(h, w, p, m, eps):
    """What a latent-attention layer caches: the normed latent c and the rotated key part shared by all heads."""
    C, R = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = rms_norm(d[:, :C], w[p + "dkv.norm"], eps)
    kr = rotate_pairs(d[:, C: C + R], np.arange(h.shape[0]), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention_mixer(h, w, p, m, latent):
    """Causal softmax attention whose keys and values are projected per head from the latent `latent` = (c, kr)
    (this layer's, or the one of the layer it borrows from)."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = latent
    q = (h @ w[p + "q"].T).reshape(T, H, D + R)
    q_plain = q[:, :, :D]
    q_rot = rotate_pairs(q[:, :, D:], np.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    seen = visible_keys(T)
    out = np.zeros((T, H, V))
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ kr.T) * m["scale"]
        out[:, head] = softmax_weights(s, seen) @ v[:, head]
    return out.reshape(T, -1) @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return relu_squared(h @ w[p + "up"].T) @ w[p + "down"].T


def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h, w, p, mlp):
    """Every token's `top` best experts, weighted by their softmax scores over their sum, plus a shared
    expert behind a sigmoid gate of one number per token."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        chosen = np.argsort(-s[t], kind="stable")[:top]
        total = s[t, chosen].sum() + 1e-20
        for e in chosen:
            out[t] += s[t, e] / total * gated_expert(h[t: t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        gate = sigmoid(h @ w[p + "shared.sg"].T)                      # [T, 1]
        out += gate * gated_expert(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layer_outputs=None):
    """Logits [tokens, vocab] of one whole sequence.  `layer_outputs`: a list that receives the residual stream
    after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if kind == "mamba1":
            a = selective_scan_mixer(h, w, p + "mix.", m)
        elif kind == "attention":
            a = window_attention_mixer(h, w, p + "mix.", m)
        elif kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, p + "mix.", m, eps)
                src = i
            a = latent_attention_mixer(h, w, p + "mix.", m, latents[src])
        else:
            raise ValueError(kind)
        x = x + rms_norm(a, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            f = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp)
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    x = rms_norm(x, w["final.norm"], eps)
    return x @ w["embed"].T
