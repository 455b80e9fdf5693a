"""Kupedra on the CPU: configuration, registry, blueprint, tensor names, random-weights mode, and properties of the
plain mechanisms the GPU tests hold the engine against."""
import copy
import json
import os

import numpy as np
import pytest

import plain_kupedra as pk
from helpers import make_model_folder
from kupedra_helpers import SMALL, SPREAD, attention, config, moe, parallel


def _resolve(cfg):
    from llm_inference_lab_b200.registry import resolve
    arch = resolve(cfg)
    return arch, arch.config_class.from_dict(cfg)


def test_registry_and_round_trip(tmp_path):
    cfg, _ = SMALL["A"]
    arch, typed = _resolve(cfg)
    assert arch.name == "Kupedra" and typed.streams == 3 and typed.loop == {"start": 0, "stop": 2, "times": 2}
    typed.save(str(tmp_path))
    with open(os.path.join(str(tmp_path), "config.json")) as fh:
        again = json.load(fh)
    assert again["architecture"] == "Kupedra" and again["layers"] == cfg["layers"]
    assert _resolve(again)[1].to_dict() == typed.to_dict()
    plain, _ = SMALL["C"]
    assert "streams" not in _resolve(plain)[1].to_dict()       # the plain residual names no streams


def test_run_order_caches_and_state():
    from llm_inference_lab_b200.models.builder import cache_plan
    from llm_inference_lab_b200.parts.spec import CacheParts, FixedState, PagedKV
    cfg, _ = SMALL["A"]
    arch, typed = _resolve(cfg)
    bp = arch.blueprint(typed)
    # layers 0 and 1 run twice in a row, then layer 2; every run has a cache of its own
    assert [c.layer for c in bp.order] == [0, 1, 0, 1, 2] == pk.run_order(cfg)
    assert [c.cache for c in bp.order] == [0, 1, 2, 3, 4] and all(c.write for c in bp.order)
    plan = cache_plan(bp)
    assert len(plan.group_keys) == 1 and plan.group_windows == (0,)      # every attention keeps all its keys
    side = plan.needs[0]
    assert isinstance(side, CacheParts) and isinstance(side.parts[0], PagedKV) and isinstance(side.parts[1], CacheParts)
    memory, top = side.parts[1].parts
    assert isinstance(memory, FixedState) and memory.shape[:2] == (3, 16) and memory.shape[2] > 8
    assert isinstance(top, FixedState) and top.shape == (3,)
    assert isinstance(plan.needs[1], PagedKV) and plan.needs[1].n_kv_heads == 3
    loop_last, _ = SMALL["C"]
    arch, typed = _resolve(loop_last)
    assert [c.layer for c in arch.blueprint(typed).order] == [0, 1, 1, 1]
    assert bp.stream_f32 and bp.head.get("scale") == 1.5 and bp.embedding.get("scale") == 0.7


def test_tensor_names_and_shapes():
    from llm_inference_lab_b200.models.builder import expected_tensors
    cfg, _ = SMALL["A"]
    arch, typed = _resolve(cfg)
    got = {t.name: tuple(t.shape) for t in expected_tensors(arch.blueprint(typed))}
    W = 72
    want = {"embed": (101, W), "head": (101, W), "final.norm": (), "l0.norm1": (), "l0.norm2": (), "l2.norm1": (),
            "l0.hc1.in": (3,), "l0.hc1.out": (3,), "l0.hc1.mix": (3, 3), "l0.hc2.mix": (3, 3), "l2.hc1.mix": (3, 3),
            "l0.mix.left.q": (64, W), "l0.mix.left.k": (32, W), "l0.mix.left.v": (48, W), "l0.mix.left.o": (W, 96),
            "l0.mix.left.q.norm": (16,), "l0.mix.left.k.norm": (16,), "l0.mix.left.rel": (10, 4), "l0.mix.left.sink": (4,),
            "l0.mix.left.out": (W,), "l0.mix.right.out": (W,),
            "l0.mix.right.q": (48, W), "l0.mix.right.k": (48, W), "l0.mix.right.v": (24, W), "l0.mix.right.g": (24, W),
            "l0.mix.right.o": (W, 24), "l0.mix.right.norm": (24,), "l0.mix.right.i": (3, W), "l0.mix.right.i.b": (3,),
            "l0.mix.right.f": (3, W), "l0.mix.right.f.b": (3,),
            "l1.mix.q": (96, W), "l1.mix.k": (48, W), "l1.mix.v": (48, W), "l1.mix.o": (W, 96), "l1.mix.temp": (6,),
            "l0.mlp.router": (5, W), "l0.mlp.e4.gate": (24, W), "l0.mlp.e0.down": (W, 24), "l0.mlp.shared.up": (40, W),
            "l0.mlp.shared.sg": (1, W), "l1.mlp.e3.up": (16, W)}
    for name, shape in want.items():
        assert got.get(name) == shape, (name, got.get(name), shape)
    for absent in ("l2.norm2", "l2.hc2.in", "l1.mlp.shared.sg", "l1.mix.sink", "l0.mix.left.temp", "l0.mlp.e5.gate"):
        assert absent not in got, absent
    plain, _ = SMALL["C"]
    arch, typed = _resolve(plain)
    assert not any(".hc" in t.name for t in expected_tensors(arch.blueprint(typed)))
    # a distance table whose rows the configuration does not name takes them from the checkpoint
    free = copy.deepcopy(cfg)
    del free["layers"][0]["mixer"]["left"]["bias_rows"]
    arch, typed = _resolve(free)
    shapes = {t.name: tuple(t.shape) for t in expected_tensors(arch.blueprint(typed))}
    assert shapes["l0.mix.left.rel"] == (-1, 4)


@pytest.mark.parametrize("path,value,needle", [
    (("vocab",), None, "vocab"), (("norm",), {}, "norm.eps"), (("layers",), [], "layers"),
    (("layers", 0, "type"), "mamba", "type"), (("layers", 0, "mixer", "left", "heads"), 5, "kv_heads"),
    (("layers", 0, "mixer", "left", "bias_max"), None, "bias_max"), (("layers", 0, "mixer", "right", "gate_cap"), -1.0, "gate_cap"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "rot", "scaling"), {"factor": 0}, "factor"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"), (("layers", 0, "mlp", "expert"), {"ff": 8}, "limit"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"), (("loop",), {"start": 2, "stop": 1, "times": 2}, "loop"),
    (("loop",), {"start": 0, "stop": 2, "times": 0}, "times"), (("streams",), -1, "streams"),
    (("embedding",), {"scale": -2.0}, "embedding.scale"),
])
def test_configurations_that_are_refused(path, value, needle):
    from llm_inference_lab_b200.config.base import ConfigError
    cfg = copy.deepcopy(SMALL["A"][0])
    at = cfg
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as err:
        _resolve(cfg)
    assert needle in str(err.value)


def test_random_weights_mode_is_read_by_the_plain_model(tmp_path):
    cfg, opt = SMALL["B"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, opt["seed"], "float32", std=0.08, scales=SPREAD)
    pcfg, w = pk.read_folder(folder)
    assert w["final.norm"].shape == () and w["l1.hc1.mix"].shape == (1, 1) and w["l1.mix.left.rel"].shape == (7, 3)
    logits = pk.forward(pcfg, w, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, cfg["vocab"]) and np.isfinite(logits).all()


# ---------------------------------------------------------------------------------------------
# properties of the plain mechanisms
# ---------------------------------------------------------------------------------------------
def test_streams_reduce_to_the_plain_residual():
    """One stream whose coefficients are all one is x + sublayer(norm(x)); several equal streams read with
    coefficients that sum to one see the same input."""
    rng = np.random.default_rng(0)
    T, W = 5, 12
    x = rng.standard_normal((T, W))
    w = {"p.norm1": np.array(1.3), "p.hc1.in": np.ones(1), "p.hc1.out": np.ones(1), "p.hc1.mix": np.ones((1, 1))}
    fn = lambda h: np.tanh(h)  # noqa: E731
    got = pk.sublayer(x[:, None, :], w, "p.", 1, 1e-6, fn)
    assert np.allclose(got[:, 0], x + fn(pk.scalar_norm(x, 1.3, 1e-6)))
    w3 = {"p.norm1": np.array(1.3), "p.hc1.in": np.array([0.2, 0.5, 0.3]), "p.hc1.out": np.array([1.0, 0.0, -1.0]),
          "p.hc1.mix": np.eye(3)}
    got3 = pk.sublayer(np.repeat(x[:, None, :], 3, axis=1), w3, "p.", 1, 1e-6, fn)
    y = fn(pk.scalar_norm(x, 1.3, 1e-6))
    assert np.allclose(got3[:, 0], x + y) and np.allclose(got3[:, 1], x) and np.allclose(got3[:, 2], x - y)
    # the mix matrix is indexed [from, to]
    w3["p.hc1.mix"] = np.array([[0.0, 1.0, 0.0], [0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    X = rng.standard_normal((T, 3, W))
    w3["p.hc1.out"] = np.zeros(3)
    moved = pk.sublayer(X, w3, "p.", 1, 1e-6, fn)
    assert np.allclose(moved[:, 1], X[:, 0]) and np.allclose(moved[:, 2], X[:, 1]) and np.allclose(moved[:, 0], X[:, 2])


def test_distance_rows():
    """The first half of the rows serves a distance each; from `far` on (at the latest) the last row serves; rows
    never go back."""
    for rows, far in ((16, 200.0), (10, 30.0), (6, 12.0), (7, 40.0)):
        half = rows // 2
        got = [pk.distance_bucket(n, rows, far) for n in range(int(far) + 50)]
        assert got[:half] == list(range(half)) and got[half] == half
        assert all(b >= a for a, b in zip(got, got[1:])) and max(got) == rows - 1
        assert got[int(far)] == rows - 1
    assert [pk.distance_bucket(n, 1, 5.0) for n in range(4)] == [0, 0, 0, 0]


def test_sink_takes_weight_and_memory_forgets():
    rng = np.random.default_rng(1)
    s = rng.standard_normal((2, 3, 3))
    seen = np.tril(np.ones((3, 3), dtype=bool))[None]
    free = pk.sink_softmax(s, seen, np.array([-np.inf, -np.inf]))
    assert np.allclose(free.sum(-1), 1.0) and np.allclose(free[:, 0, 1:], 0.0)
    one = pk.sink_softmax(s, seen, np.zeros(2))
    assert np.allclose(one.sum(-1), 1.0 - 1.0 / (1.0 + np.where(seen, np.exp(s), 0).sum(-1)))
    assert pk.sink_softmax(s, seen, np.array([50.0, 50.0])).max() < 1e-18
    # a forget gate that closes at token t wipes what came before; an input gate that closes keeps the memory as it is
    T, W, H, D, V = 6, 8, 1, 4, 4
    w = {"m." + n: rng.standard_normal(shape) for n, shape in
         {"q": (H * D, W), "k": (H * D, W), "v": (H * V, W), "g": (H * V, W), "o": (W, H * V), "i": (H, W), "f": (H, W)}.items()}
    w["m.norm"], w["m.i"], w["m.f"] = np.ones(H * V), np.zeros((H, W)), np.zeros((H, W))
    w["m.i.b"], w["m.f.b"] = np.zeros(H), np.full(H, -1e4)            # forget everything at every token
    m = {"heads": H, "dim": D, "vdim": V, "gate_cap": 40.0}
    h = rng.standard_normal((T, W))
    each = np.concatenate([pk.matrix_memory(h[t: t + 1], w, "m.", m, 1e-6) for t in range(T)])
    assert np.allclose(pk.matrix_memory(h, w, "m.", m, 1e-6), each, atol=1e-9)


def test_prefix_does_not_depend_on_what_follows():
    cfg, opt = SMALL["A"]
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_model_folder(os.path.join(tmp, "m"), cfg, opt["seed"], "float32", std=0.08, scales=SPREAD)
        pcfg, w = pk.read_folder(folder)
    ids = [int(t) for t in np.random.default_rng(2).integers(0, cfg["vocab"], size=40)]
    whole = pk.forward(pcfg, w, ids)
    assert np.allclose(pk.forward(pcfg, w, ids[:25]), whole[:25], atol=1e-9)
    one_layer = config([parallel((2, 1, 8, 8, 0.3, (0.5, 3), 6, 10), (1, 8, 8, 5.0), ff=moe(3, 1, 8, 1.0)),
                        attention(2, 2, 8, 8, 4, ff=None)], vocab=31, width=16, streams=2)
    assert pk.run_order(one_layer) == [0, 1]
