"""Small Bukatar configurations for the tests.  Every size differs from one configuration to the next; none
has the sizes of a published model."""
from __future__ import annotations

import numpy as np


def _mlp(ff):
    """None: no feed-forward; an int: dense; a tuple (experts, top, expert_ff, shared_ff or None): routed."""
    if ff is None:
        return None
    if isinstance(ff, int):
        return {"kind": "dense", "ff": ff}
    experts, top, eff, shared = ff
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": eff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def mamba1(inner, state, dt_rank, conv, ff=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv},
            "mlp": _mlp(ff)}


def attention(heads, kv_heads, dim, window, keep_first, rot_dims, base=10000.0, scale=None, ff=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                      "scale": float(scale if scale is not None else dim ** -0.5),
                      "mask": {"size": window, "keep_first": keep_first}, "rot": {"base": base, "dims": rot_dims}},
            "mlp": _mlp(ff)}


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None, kv_from=None, rot_dims=None, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5),
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": _mlp(ff)}


def config(layers, vocab=97, width=48, eps=1e-5):
    return {"architecture": "Bukatar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}


# A: every mixer and both feed-forwards; a layer that borrows latents; a window that is no multiple of a page;
# several key/value heads; a layer without a feed-forward
SMALL_A = config([mamba1(80, 12, 6, 4, ff=88), attention(6, 3, 16, 21, 3, 8, ff=(5, 2, 24, 40)),
                  latent(3, 16, 8, 24, 40, ff=56), mamba1(80, 12, 6, 4), latent(3, 16, 8, 24, 40, kv_from=2, scale=0.3,
                                                                               ff=(5, 2, 24, None))],
                 vocab=101, width=72)
# B: the attention opens the model; as many key/value heads as query heads; every entry rotated; no first tokens
# kept; one expert of one chosen (the weights are 1); two taps; a state of one lane's worth
SMALL_B = config([attention(2, 2, 32, 9, 0, 32, base=500.0, scale=0.2, ff=(1, 1, 16, 8)),
                  mamba1(48, 5, 3, 2, ff=40), latent(5, 8, 16, 8, 24, base=2000.0, ff=(7, 7, 8, 16))],
                 vocab=89, width=56, eps=1e-6)
# C: a width that is no multiple of 8 (the products leave the tensor cores), one head everywhere, a convolution
# of one tap (no kept inputs), nothing rotated in the attention, a window of one page, more kept tokens than a page
SMALL_C = config([mamba1(30, 40, 2, 1, ff=30), attention(1, 1, 48, 32, 37, 0), latent(1, 24, 4, 12, 10, ff=70),
                  latent(1, 24, 4, 12, 10, kv_from=2), attention(1, 1, 48, 32, 37, 0, ff=(3, 2, 10, 6))],
                 vocab=67, width=50, eps=3e-6)
# D: heads of 64 entries with long portions, a state of 64 entries, many experts
SMALL_D = config([attention(4, 2, 64, 100, 5, 32, ff=(16, 4, 32, 32)), mamba1(128, 64, 8, 4, ff=64),
                  latent(2, 64, 32, 64, 96, ff=64)],
                 vocab=113, width=64)
SMALL = {"A": (SMALL_A, dict(seed=11, page_size=16)), "B": (SMALL_B, dict(seed=12, page_size=4)),
         "C": (SMALL_C, dict(seed=13, page_size=32)), "D": (SMALL_D, dict(seed=14, page_size=16))}

# Random N(0, std) weights give nearly uniform attention and a router without preferences: queries, keys and
# the router are scaled up so that scores spread; the state-space mixer's step sizes so that its state forgets
# at a visible pace.
SPREAD = {".q": 2.0, ".k": 2.0, ".router": 6.0, "dt.b": 10.0, "A_log": 8.0}


def sequences(rng, vocab, lengths):
    return {f"s{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def plain_logits(folder, seqs):
    import plain_bukatar as pb
    cfg, w = pb.read_folder(folder)
    return {name: np.asarray(pb.forward(cfg, w, ids), dtype=np.float64) for name, ids in seqs.items()}


def random_config(rng):
    """A random Bukatar configuration and page size: one to five layers in any order of the three mixers and the
    three kinds of feed-forward, sizes that are multiples of 8 or only of 2, any number of heads and groups,
    windows from one key to longer than the sequences, kept first tokens from none to more than a window, one to
    five taps, layers that borrow the latents of an earlier layer."""
    def size(lo, hi):
        return int(rng.choice([8, 8, 16, 2])) * int(rng.integers(lo, hi))

    def ff():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.55:
            return size(2, 20)
        experts = int(rng.integers(1, 10))
        return (experts, int(rng.integers(1, experts + 1)), size(1, 8), size(1, 8) if rng.random() < 0.6 else None)

    layers, owners = [], []
    for i in range(int(rng.integers(1, 6))):
        kind = rng.choice(["mamba1", "attention", "latent_attention", "latent_attention"])
        if kind == "mamba1":
            layer = mamba1(size(2, 20), int(rng.choice([1, 4, 8, 12, 16, 33, 70])), int(rng.choice([1, 2, 8, 16])),
                           int(rng.integers(1, 6)), ff=ff())
        elif kind == "attention":
            G = int(rng.choice([1, 1, 2, 3]))
            dim = min(size(1, 12), 160)
            layer = attention(G * int(rng.choice([1, 2, 4, 5])), G, dim, int(rng.choice([1, 2, 7, 16, 40, 64, 500])),
                              int(rng.choice([0, 0, 1, 4, 19, 70])), 2 * int(rng.integers(0, dim // 2 + 1)),
                              base=float(rng.choice([100.0, 10000.0, 250000.0])),
                              scale=float(rng.uniform(0.5, 2.0)) * dim ** -0.5, ff=ff())
        else:
            if owners and rng.random() < 0.4:
                src = int(rng.choice(owners))
                m = layers[src]["mixer"]
                layer = latent(int(rng.choice([1, 2, 3])), size(1, 6), m["rot_dim"], size(1, 6), m["kv_rank"],
                               base=m["rot"]["base"], rot_dims=m["rot"]["dims"], kv_from=src, ff=ff())
            else:
                rot_dim = 2 * int(rng.integers(1, 17))
                layer = latent(int(rng.choice([1, 2, 3, 6])), size(1, 6), rot_dim, size(1, 6), size(1, 12),
                               base=float(rng.choice([100.0, 10000.0, 250000.0])),
                               rot_dims=2 * int(rng.integers(1, rot_dim // 2 + 1)), ff=ff())
                owners.append(i)
        layers.append(layer)
    cfg = config(layers, vocab=int(rng.integers(30, 400)), width=size(3, 16), eps=float(rng.choice([1e-6, 1e-5])))
    return cfg, int(rng.choice([16, 16, 4, 8, 32, 64]))
