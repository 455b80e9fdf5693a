"""Bukatar: a decoder that puts every sublayer between two norms on a 32-bit residual stream and mixes three
kinds of token mixers with dense and routed feed-forwards, layer by layer.

config.json keys: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list whose entries give ``type`` (the
mixer), ``mixer`` (its sizes and constants) and ``mlp`` (or null for a layer without a feed-forward):

``mamba1``
    a state-space mixer with a decay per channel and state entry (``inner``, ``state``, ``dt_rank``, ``conv`` taps).
``attention``
    grouped-query softmax attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) with biases on q, k
    and the output; the values are the keys as projected; rotary positions on neighbouring pairs of the first
    ``rot.dims`` entries of a head (``rot.base``); a window of ``mask.size`` keys that also keeps the first
    ``mask.keep_first`` tokens; one more in the softmax's denominator.
``latent_attention``
    causal attention over a cached latent (``heads``, ``dim`` plain and ``rot_dim`` rotated entries per head,
    ``vdim``, ``kv_rank``, ``scale``, ``rot.base``, ``rot.dims``), queries projected directly.  ``kv_from``: j makes
    the layer read the latents layer j caches.

``mlp.kind`` is ``dense`` (``ff``; W_down relu(W_up h)^2) or ``moe`` (``router.experts``, ``router.top``,
``expert.ff``, optional ``shared.ff`` behind a sigmoid gate).  Each layer is x <- x + norm1b(mixer(norm1(x))),
then x <- x + norm2b(ff(norm2(x))).  The head is the embedding table.  Tensor names: ``embed``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

import dataclasses
from typing import Any

from .base import ConfigError, ModelConfig, finite_positive, optional, positive, required
from ..parts.spec import LayerCall, LayerSpec, ModelBlueprint, PartSpec

MIXER_TYPES = ("mamba1", "attention", "latent_attention")


def _need(obj: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"config.json of Bukatar lacks {where}.{key}")
    value = obj[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config key {where}.{key} has the wrong type: {value!r}")
    return value


def _positive_int(obj, key, where) -> int:
    value = _need(obj, key, where, (int,))
    if value <= 0:
        raise ConfigError(f"config key {where}.{key} must be positive, got {value!r}")
    return int(value)


def _check_rot(m, where, most: int) -> None:
    rot = _need(m, "rot", where, (dict,))
    finite_positive(where + ".rot.base", _need(rot, "base", where + ".rot"))
    dims = _need(rot, "dims", where + ".rot", (int,))
    if dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot.dims must be even and at most {most}, got {dims!r}")


@dataclasses.dataclass
class BukatarConfig(ModelConfig):
    architecture = "Bukatar"

    vocab: int = required(int, positive)
    width: int = required(int, positive)
    layers: Any = required("any")
    norm: Any = required("any")
    max_positions: int = optional(int, 1 << 17, positive, doc="longest sequence the engine plans for")

    def validate(self) -> None:
        finite_positive("norm.eps", _need(self.norm, "eps", "norm"))
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}.type must be one of {MIXER_TYPES}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m, kind = layer.get("mixer"), layer["type"]
            where += ".mixer"
            if not isinstance(m, dict):
                raise ConfigError(f"config.json of Bukatar lacks {where}")
            if kind == "mamba1":
                for key in ("inner", "state", "dt_rank", "conv"):
                    _positive_int(m, key, where)
            elif kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(m, key, where)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.heads must be a multiple of {where}.kv_heads")
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"{where}.vdim must equal {where}.dim: the values are the keys")
                finite_positive(where + ".scale", _need(m, "scale", where))
                _check_rot(m, where, m["dim"])
                mask = _need(m, "mask", where, (dict,))
                _positive_int(mask, "size", where + ".mask")
                if _need(mask, "keep_first", where + ".mask", (int,)) < 0:
                    raise ConfigError(f"{where}.mask.keep_first must not be negative")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _positive_int(m, key, where)
                finite_positive(where + ".scale", _need(m, "scale", where))
                _check_rot(m, where, m["rot_dim"])
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"{where}.kv_from must name an earlier layer, got {src!r}")
                    other = self.layers[src]
                    if other["type"] != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.kv_from must name a latent_attention layer with latents of its own")
                    for key in ("kv_rank", "rot_dim"):
                        if other["mixer"][key] != m[key]:
                            raise ConfigError(f"{where}.{key} differs from layer {src}'s, whose latents it reads")
                    if other["mixer"]["rot"] != m["rot"]:
                        raise ConfigError(f"{where}.rot differs from layer {src}'s, whose rotated key part it reads")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            where = f"layers[{i}].mlp"
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"{where}.kind must be 'dense' or 'moe' (or mlp null)")
            if mlp["kind"] == "dense":
                _positive_int(mlp, "ff", where)
            else:
                router = _need(mlp, "router", where, (dict,))
                experts, top = _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router")
                if top > experts:
                    raise ConfigError(f"{where}.router.top must not exceed {where}.router.experts")
                _positive_int(_need(mlp, "expert", where, (dict,)), "ff", where + ".expert")
                if mlp.get("shared") is not None:
                    _positive_int(_need(mlp, "shared", where, (dict,)), "ff", where + ".shared")

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture}
        out.update(dataclasses.asdict(self))
        return out


def bukatar_blueprint(cfg: BukatarConfig) -> ModelBlueprint:
    """The design's layers as data: every size and constant comes from `cfg`; what the design fixes (which
    mixer has biases, the pairing of the rotation, the activations, the extra one in the attention's
    denominator) is set here as parameters of the parts."""
    eps, width = float(cfg.norm["eps"]), cfg.width
    layers, calls, cache_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        cache, write = i, True
        if kind == "mamba1":
            mixer = PartSpec("selective_scan", {"hidden": width, "inner": m["inner"], "state": m["state"],
                                                "dt_rank": m["dt_rank"], "taps": m["conv"]}, prefix=p + "mix.")
        elif kind == "attention":
            mixer = PartSpec("pair_rope_attention", {
                "hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                "scale": float(m["scale"]), "window": int(m["mask"]["size"]), "keep_first": int(m["mask"]["keep_first"]),
                "sink_one": True, "rot_base": float(m["rot"]["base"]), "rot_dims": int(m["rot"]["dims"]), "bias": True,
                "values_from_keys": True}, prefix=p + "mix.")
        else:
            src = m.get("kv_from")
            mixer = PartSpec("latent_attention", {
                "hidden": width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "q_rank": 0, "kv_rank": m["kv_rank"], "window": 0, "sink": False, "rot_base": float(m["rot"]["base"]),
                "rot_dims": int(m["rot"]["dims"]), "rot_pairs": True, "scale": float(m["scale"]), "eps": eps,
                "own_kv": src is None}, prefix=p + "mix.")
            if src is not None:
                cache, write = cache_of[src], False
        cache_of[i] = cache
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None and mlp["kind"] == "dense":
            ffn = PartSpec("dense_mlp", {"hidden": width, "intermediate": mlp["ff"], "act": "relu2", "bias": False,
                                         "out_f32": True, "names": {"up": "up", "down": "down"}}, prefix=p + "mlp.")
        elif mlp is not None:
            shared = mlp.get("shared")
            ffn = PartSpec("routed_experts", {
                "hidden": width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_ff": mlp["expert"]["ff"], "shared_ff": shared["ff"] if shared is not None else 0,
                "shared_gate": shared is not None}, prefix=p + "mlp.")
        names = ("norm1", "norm1b", "norm2", "norm2b") if mlp is not None else ("norm1", "norm1b")
        norms = tuple(PartSpec("rmsnorm_stream", {"hidden": width, "eps": eps, "offset": 0.0, "name": name}, prefix=p)
                      for name in names)
        layers.append(LayerSpec("sandwich_stream", mixer, ffn, norms, hidden=width))
        calls.append(LayerCall(layer=i, cache=cache, write=write))
    # cache ids are dense: layers that borrow another layer's latents own none
    ids = {c: n for n, c in enumerate(sorted({c.cache for c in calls}))}
    calls = tuple(LayerCall(c.layer, ids[c.cache], c.write) for c in calls)
    return ModelBlueprint(
        hidden=width, vocab=cfg.vocab,
        embedding=PartSpec("token_embedding_stream", {"vocab": cfg.vocab, "hidden": width, "table": "embed"}),
        layers=tuple(layers), order=calls,
        final_norm=PartSpec("rmsnorm_stream", {"hidden": width, "eps": eps, "offset": 0.0, "name": "norm"},
                            prefix="final."),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": width, "tied_to": "embed"}),
        max_positions=cfg.max_positions, eos_token_ids=(), stream_f32=True)
