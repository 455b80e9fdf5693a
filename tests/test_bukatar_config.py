"""Bukatar on the CPU: configuration, blueprint, caches, page groups that keep first tokens, random-weights mode,
and properties of the plain implementation's mechanisms."""
import copy

import numpy as np
import pytest

import plain_bukatar as pb
from bukatar_helpers import SMALL, attention, config, latent, mamba1


def _cfg(raw):
    from llm_inference_lab_b200.registry import resolve
    arch = resolve(raw)
    return arch, arch.config_class.from_dict(raw)


def test_registry_resolves_and_round_trips():
    arch, cfg = _cfg(SMALL["A"][0])
    assert arch.name == "Bukatar" and cfg.width == 72 and cfg.vocab == 101
    again = arch.config_class.from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and cfg.to_dict()["architecture"] == "Bukatar"


def test_blueprint_layers_caches_and_tensors():
    from llm_inference_lab_b200.config.bukatar import bukatar_blueprint
    from llm_inference_lab_b200.models.builder import cache_plan, expected_tensors
    from llm_inference_lab_b200.parts.spec import CacheParts, FixedState, PagedKV, PagedLatent
    _, cfg = _cfg(SMALL["A"][0])
    bp = bukatar_blueprint(cfg)
    assert bp.stream_f32 and bp.head.get("tied_to") == "embed"
    # the layer that borrows latents reads the third layer's cache and owns none
    assert [(c.layer, c.cache, c.write) for c in bp.order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 3, True),
                                                               (4, 2, False)]
    plan = cache_plan(bp)
    assert plan.needs[0] == CacheParts((FixedState((80, 12)), FixedState((3, 80))))
    assert plan.needs[1] == PagedKV(3, 16, 21, 3) and plan.needs[2] == PagedLatent(40 + 8, 0)
    assert plan.group_windows == (21, 0) and plan.group_keeps == (3, 0)
    shapes = {t.name: t.shape for t in expected_tensors(bp)}
    assert shapes["embed"] == (101, 72) and "head" not in shapes
    assert shapes["l0.mix.in"] == (160, 72) and shapes["l0.mix.x"] == (6 + 24, 80) and shapes["l0.mix.A_log"] == (80, 12)
    assert shapes["l1.mix.q"] == (96, 72) and shapes["l1.mix.k.b"] == (48,) and "l1.mix.v" not in shapes
    assert shapes["l1.mlp.router"] == (5, 72) and shapes["l1.mlp.e4.down"] == (72, 24)
    assert shapes["l1.mlp.shared.sg"] == (1, 72) and shapes["l1.mlp.shared.up"] == (40, 72)
    assert shapes["l2.mix.dkv"] == (48, 72) and shapes["l2.mix.q"] == (3 * 24, 72) and shapes["l2.mix.uk"] == (48, 40)
    assert "l4.mix.dkv" not in shapes and "l4.mlp.shared.sg" not in shapes and "l3.norm2" not in shapes
    assert all(f"l{i}.norm1b" in shapes for i in range(5)) and "l0.norm2b" in shapes


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="mamba3"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("dt_rank"), "dt_rank"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["mask"].pop("keep_first"), "keep_first"),
    (lambda c: c["layers"][1]["mixer"].update(heads=4), "heads"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(kv_rank=41), "kv_rank"),
    (lambda c: c["layers"][4]["mixer"]["rot"].update(base=3.0), "rot"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_configurations_that_are_refused(change, word):
    from llm_inference_lab_b200.config.base import ConfigError
    raw = copy.deepcopy(SMALL["A"][0])
    change(raw)
    with pytest.raises(ConfigError) as err:
        _cfg(raw)
    assert word in str(err.value)


def test_page_groups_keep_the_first_pages():
    """A windowed page group that keeps first tokens never gives their pages back; the others return as the
    window passes, and everything returns when the request ends."""
    from llm_inference_lab_b200.cache import CacheManager, GroupConfig
    c = CacheManager([GroupConfig(4, 6, 32, 5), GroupConfig(4, 6, 32)], 2)
    c.open(7)
    for _ in range(10):
        c.reserve(7, 3)
        c.commit(7, 3)
    # positions 0..4 lie on two pages; a query at 30 reads keys from 25 on: pages 6 and 7 (and 8 once reserved)
    assert 32 - c.free_pages(0) == 2 + 2 and 32 - c.free_pages(1) == 2
    table = list(c.block_table(7, 0))
    assert table[0] >= 0 and table[1] >= 0 and all(p < 0 for p in table[2:6]) and all(p >= 0 for p in table[6:8])
    assert c.pages_at_peak(0, 100, 3) == c.pages_at_peak(1, 100, 3) + 2
    c.check_consistency()
    c.close(7)
    assert c.free_pages(0) == 32 and c.free_pages(1) == 32


def test_random_weights_mode_is_read_by_the_plain_model(tmp_path):
    from helpers import make_model_folder
    cfg = SMALL["B"][0]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 3, "float32", std=0.08)
    pcfg, w = pb.read_folder(folder)
    logits = pb.forward(pcfg, w, [1, 5, 2, 8, 13])
    assert logits.shape == (5, cfg["vocab"]) and np.isfinite(logits).all()


def test_properties_of_the_plain_mechanisms():
    rng = np.random.default_rng(0)
    # rotation by pairs keeps norms, leaves entries beyond `dims` alone, and scores depend on distance only
    v = rng.standard_normal((6, 2, 12))
    r = pb.rotate_pairs(v, np.arange(6), 100.0, 8)
    assert np.allclose((r ** 2).sum(-1), (v ** 2).sum(-1)) and np.array_equal(r[..., 8:], v[..., 8:])
    a, b = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    s1 = (pb.rotate_pairs(a, [9], 50.0, 8) * pb.rotate_pairs(b, [4], 50.0, 8)).sum()
    s2 = (pb.rotate_pairs(a, [25], 50.0, 8) * pb.rotate_pairs(b, [20], 50.0, 8)).sum()
    assert abs(s1 - s2) < 1e-9
    # the mask: the window's last place is seen, the next is not, unless it is one of the kept first tokens
    seen = pb.visible_keys(20, window=5, keep_first=2)
    assert seen[10, 6] and not seen[10, 5] and seen[10, 1] and not seen[10, 2] and not seen[3, 4]
    # one more in the denominator: weights sum to less than one, and to nearly nothing where scores are low
    w = pb.softmax_weights(np.array([[0.0, 0.0]]), np.array([[True, True]]), extra_one=True)
    assert np.allclose(w, 1 / 3)
    assert pb.softmax_weights(np.array([[-40.0]]), np.array([[True]]), extra_one=True)[0, 0] < 1e-15
    # the convolution's last tap meets the current token; zeros before the start
    x = rng.standard_normal((5, 3))
    taps = np.zeros((3, 4)); taps[:, -1] = 2.0
    assert np.allclose(pb.causal_conv(x, taps, np.zeros(3)), 2 * x)
    taps = np.zeros((3, 4)); taps[:, 0] = 1.0
    out = pb.causal_conv(x, taps, np.zeros(3))
    assert np.allclose(out[3:], x[:2]) and not out[:3].any()
    # a routed layer with one expert of one gives that expert; the selective scan is causal
    cfg = config([mamba1(16, 4, 2, 3, ff=(1, 1, 8, None))], vocab=31, width=16)
    from helpers import make_model_folder  # noqa: F401
    assert attention(2, 1, 8, 4, 1, 4)["mixer"]["vdim"] == 8 and latent(1, 8, 4, 8, 8)["mixer"]["rot"]["dims"] == 4
    assert cfg["layers"][0]["mlp"]["router"] == {"experts": 1, "top": 1}
