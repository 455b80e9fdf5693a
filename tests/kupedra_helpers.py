"""Small Kupedra configurations for the tests.  Every size differs from one configuration to the next; none
has the sizes of a published model."""
from __future__ import annotations

import numpy as np


def moe(experts, top, ff, limit, shared=None):
    """shared: (ff, limit) or None."""
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, factor=None, scale=None, ff=None):
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot,
                      "scale": float(scale if scale is not None else 1.0)},
            "mlp": ff}


def parallel(left, right, ff=None):
    """left: (heads, kv_heads, dim, vdim, scale, (coef, every) or None, rows of the distance table, far);
    right: (heads, dim, vdim, gate cap)."""
    H, G, D, V, scale, qt, rows, far = left
    lm = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": float(scale), "bias_max": far, "bias_rows": rows}
    if qt is not None:
        lm["q_temp"] = {"coef": qt[0], "every": qt[1]}
    rh, rd, rv, cap = right
    return {"type": "parallel", "mixer": {"left": lm, "right": {"heads": rh, "dim": rd, "vdim": rv, "gate_cap": cap}},
            "mlp": ff}


def config(layers, vocab=97, width=48, eps=1e-5, streams=2, loop=None, embed_scale=1.0, logit_scale=1.0):
    out = {"architecture": "Kupedra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale}, "logit_scale": logit_scale}
    if streams:
        out["streams"] = streams
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# A: both mixers, a loop over the first two layers, three streams, a distance table whose shared rows are reached
# inside the test's sequences, a temperature that grows every few positions, a layer without a feed-forward
SMALL_A = config([parallel((4, 2, 16, 24, 0.3, (0.4, 7), 10, 30), (3, 16, 8, 9.0), ff=moe(5, 2, 24, 1.2, (40, 1.7))),
                  attention(6, 3, 16, 16, 8, base=500.0, factor=1.5, scale=0.3, ff=moe(4, 1, 16, 0.8)),
                  parallel((2, 1, 32, 16, 0.2, None, 6, 12), (2, 24, 20, 5.0))],
                 vocab=101, width=72, streams=3, loop=(0, 2, 2), embed_scale=0.7, logit_scale=1.5)
# B: the attention opens the model; as many key/value heads as query heads; every entry rotated, no scaling of
# the frequencies; one stream with coefficients; one expert of one chosen; no loop; an odd number of table rows
SMALL_B = config([attention(2, 2, 32, 8, 32, base=2000.0, scale=0.2, ff=moe(1, 1, 16, 2.5, (8, 0.6))),
                  parallel((3, 3, 8, 8, 0.5, (0.2, 3), 7, 40), (1, 32, 40, 15.0), ff=moe(7, 7, 8, 1.0))],
                 vocab=89, width=56, eps=1e-6, streams=1, embed_scale=2.0, logit_scale=0.5)
# C: a width that is no multiple of 8 (the products leave the tensor cores), no streams (the plain residual),
# nothing rotated, one head everywhere, the loop over the last layer alone and three times, a distance table
# that is never exhausted (far beyond the sequences)
SMALL_C = config([attention(1, 1, 40, 20, 0, scale=0.15, ff=moe(3, 2, 10, 1.6)),
                  parallel((1, 1, 24, 12, 0.25, (1.0, 16), 12, 5000), (1, 8, 12, 11.0), ff=moe(2, 1, 6, 3.0, (10, 3.0)))],
                 vocab=67, width=50, eps=3e-6, streams=0, loop=(1, 2, 3))
# D: heads of 64 entries with long portions, many experts, four streams
SMALL_D = config([parallel((4, 2, 64, 64, 0.125, (0.35, 50), 32, 200), (2, 64, 64, 10.0), ff=moe(16, 4, 32, 1.4, (32, 2.2))),
                  attention(4, 1, 64, 64, 32, base=500000.0, factor=4.0, scale=0.11, ff=moe(8, 2, 64, 1.0))],
                 vocab=113, width=64, streams=4)
SMALL = {"A": (SMALL_A, dict(seed=21, page_size=16)), "B": (SMALL_B, dict(seed=22, page_size=4)),
         "C": (SMALL_C, dict(seed=23, page_size=32)), "D": (SMALL_D, dict(seed=24, page_size=16))}

# Random N(0, std) weights give nearly uniform attention, a router without preferences and gates that never
# close: queries, keys, the router, the distance table, the sinks and the gates' biases are scaled up.
SPREAD = {"mix.q": 2.0, "mix.k": 2.0, "left.q": 1.5, "left.k": 1.5, ".router": 6.0, ".rel": 30.0, ".sink": 20.0,
          "right.i.b": 40.0, "right.f.b": 40.0}


def sequences(rng, vocab, lengths):
    return {f"s{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def plain_logits(folder, seqs):
    import plain_kupedra as pk
    cfg, w = pk.read_folder(folder)
    return {name: np.asarray(pk.forward(cfg, w, ids), dtype=np.float64) for name, ids in seqs.items()}


def random_config(rng):
    """A random Kupedra configuration and page size: one to four layers of both mixers in any order, sizes that are
    multiples of 8 or only of 2, any number of heads and groups, zero to five streams, a loop anywhere or none,
    distance tables of 1 to 40 rows that end before or beyond the sequences."""
    def size(lo, hi):
        return int(rng.choice([8, 8, 16, 2])) * int(rng.integers(lo, hi))

    def ff():
        if rng.random() < 0.2:
            return None
        experts = int(rng.integers(1, 10))
        shared = (size(1, 8), float(rng.uniform(0.5, 3.0))) if rng.random() < 0.6 else None
        return moe(experts, int(rng.integers(1, experts + 1)), size(1, 8), float(rng.uniform(0.5, 3.0)), shared)

    layers = []
    for _ in range(int(rng.integers(1, 5))):
        G = int(rng.choice([1, 1, 2, 3]))
        H = G * int(rng.choice([1, 2, 4, 5]))
        dim, vdim = min(size(1, 12), 160), min(size(1, 12), 160)
        if rng.random() < 0.45:
            layers.append(attention(H, G, dim, vdim, 2 * int(rng.integers(0, dim // 2 + 1)),
                                    base=float(rng.choice([100.0, 10000.0, 500000.0])),
                                    factor=float(rng.choice([1.0, 2.0, 8.0])) if rng.random() < 0.7 else None,
                                    scale=float(rng.uniform(0.5, 2.0)) * dim ** -0.5, ff=ff()))
        else:
            rows = int(rng.choice([1, 2, 5, 8, 16, 40]))
            far = float(rows // 2 + int(rng.choice([1, 3, 20, 400])))
            qt = (float(rng.uniform(0.0, 1.0)), int(rng.choice([1, 4, 30, 1000]))) if rng.random() < 0.7 else None
            layers.append(parallel((H, G, dim, vdim, float(rng.uniform(0.5, 2.0)) * dim ** -0.5, qt, rows, far),
                                   (int(rng.integers(1, 5)), size(1, 9), size(1, 9), float(rng.choice([3.0, 11.0, 30.0]))),
                                   ff=ff()))
    n = len(layers)
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n))
        loop = (a, int(rng.integers(a, n + 1)), int(rng.integers(1, 4)))
    cfg = config(layers, vocab=int(rng.integers(30, 400)), width=size(3, 16), eps=float(rng.choice([1e-6, 1e-5])),
                 streams=int(rng.integers(0, 6)), loop=loop, embed_scale=float(rng.uniform(0.3, 3.0)),
                 logit_scale=float(rng.uniform(0.3, 3.0)))
    return cfg, int(rng.choice([16, 16, 4, 8, 32, 64]))
