"""Kupedra: a decoder on a residual of several 32-bit streams (hyper-connections) that mixes two kinds of token
mixers with routed feed-forwards, layer by layer, and may run a span of its layers several times.

config.json keys: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale``, ``streams`` (absent:
the plain pre-norm residual), ``loop`` (``start``, ``stop``, ``times``: layers start .. stop - 1 run that many times
in a row with the same weights, every pass with caches and state of its own; absent: every layer once) and
``layers``, a list whose entries give ``type`` (the mixer), ``mixer`` (its sizes and constants) and ``mlp`` (or
null for a layer without a feed-forward):

``attention``
    grouped-query softmax attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``), no biases; rotary
    positions on neighbouring pairs of the first ``rot.dims`` entries of a head (``rot.base``, frequencies divided
    by ``rot.scaling.factor``); q and k then divided by their root mean square per head; a learned temperature
    per head on the score (``temp``); causal; one more in the softmax's denominator.
``parallel``
    two mixers on the same input, ``left`` and ``right``; each result is RMS-normed over the width with a weight
    (``left.out``, ``right.out``) and half their sum is the result.  Left: grouped-query attention without rotation,
    q and k normed per head with a weight shared by the heads (``q.norm``, ``k.norm``), q multiplied by 1 +
    ``q_temp.coef`` * ln(floor((p + 1) / ``q_temp.every``) + 1) at position p, a learned bias by distance (``rel``,
    its last row reached at ``bias_max``; its rows are the checkpoint's, ``bias_rows`` names them for random
    weights), a learned term per head in the softmax's denominator (``sink``).  Right: a
    matrix memory with exponential gates (``heads``, ``dim``, ``vdim``, ``gate_cap``).

``mlp.kind`` is ``moe``: ``router.experts`` experts of ``expert.ff`` rows of which a token uses ``router.top``,
weighted by their softmax scores as they are; experts of the capped form with ``expert.limit``; an optional
``shared`` expert (``ff``, ``limit``) behind a sigmoid gate of one number per token.  Norms have one number as their
weight.  Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import dataclasses
from typing import Any

from .base import ConfigError, ModelConfig, finite_positive, optional, positive, required
from ..parts.spec import LayerCall, LayerSpec, ModelBlueprint, PartSpec

MIXER_TYPES = ("attention", "parallel")


def _need(obj: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"config.json of Kupedra lacks {where}.{key}")
    value = obj[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config key {where}.{key} has the wrong type: {value!r}")
    return value


def _positive_int(obj, key, where) -> int:
    value = _need(obj, key, where, (int,))
    if value <= 0:
        raise ConfigError(f"config key {where}.{key} must be positive, got {value!r}")
    return int(value)


def _check_heads(m, where, grouped: bool) -> None:
    for key in ("heads", "dim", "vdim") + (("kv_heads",) if grouped else ()):
        _positive_int(m, key, where)
    if grouped and m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}.heads must be a multiple of {where}.kv_heads")


def _check_expert(e, where) -> None:
    _positive_int(e, "ff", where)
    finite_positive(where + ".limit", _need(e, "limit", where))


@dataclasses.dataclass
class KupedraConfig(ModelConfig):
    architecture = "Kupedra"

    vocab: int = required(int, positive)
    width: int = required(int, positive)
    layers: Any = required("any")
    norm: Any = required("any")
    embedding: Any = optional("any", None, doc="{'scale': s}: the embedding output is table[token] * s")
    logit_scale: float = optional(float, 1.0, finite_positive)
    streams: int = optional(int, 0, doc="streams of the residual; 0 or absent: the plain pre-norm residual")
    loop: Any = optional("any", None)
    max_positions: int = optional(int, 1 << 17, positive, doc="longest sequence the engine plans for")

    def validate(self) -> None:
        finite_positive("norm.eps", _need(self.norm, "eps", "norm"))
        if self.embedding is not None:
            finite_positive("embedding.scale", _need(self.embedding, "scale", "embedding"))
        if self.streams < 0:
            raise ConfigError("'streams' must not be negative")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        if self.loop is not None:
            start, stop = _need(self.loop, "start", "loop", (int,)), _need(self.loop, "stop", "loop", (int,))
            _positive_int(self.loop, "times", "loop")
            if not 0 <= start <= stop <= len(self.layers):
                raise ConfigError(f"loop.start .. loop.stop must lie within the {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}.type must be one of {MIXER_TYPES}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m, kind = layer.get("mixer"), layer["type"]
            where += ".mixer"
            if not isinstance(m, dict):
                raise ConfigError(f"config.json of Kupedra lacks {where}")
            if kind == "attention":
                _check_heads(m, where, True)
                finite_positive(where + ".scale", _need(m, "scale", where))
                if m.get("rot") is not None:
                    rot = _need(m, "rot", where, (dict,))
                    finite_positive(where + ".rot.base", _need(rot, "base", where + ".rot"))
                    dims = _need(rot, "dims", where + ".rot", (int,))
                    if dims < 0 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{where}.rot.dims must be even and at most {where}.dim, got {dims!r}")
                    if rot.get("scaling") is not None:
                        finite_positive(where + ".rot.scaling.factor",
                                        _need(rot["scaling"], "factor", where + ".rot.scaling"))
            else:
                left, right = _need(m, "left", where, (dict,)), _need(m, "right", where, (dict,))
                _check_heads(left, where + ".left", True)
                finite_positive(where + ".left.scale", _need(left, "scale", where + ".left"))
                if left.get("q_temp") is not None:
                    _need(left["q_temp"], "coef", where + ".left.q_temp")
                    _positive_int(left["q_temp"], "every", where + ".left.q_temp")
                finite_positive(where + ".left.bias_max", _need(left, "bias_max", where + ".left"))
                _check_heads(right, where + ".right", False)
                finite_positive(where + ".right.gate_cap", _need(right, "gate_cap", where + ".right"))
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            where = f"layers[{i}].mlp"
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"{where}.kind must be 'moe' (or mlp null)")
            router = _need(mlp, "router", where, (dict,))
            experts, top = _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"{where}.router.top must not exceed {where}.router.experts")
            _check_expert(_need(mlp, "expert", where, (dict,)), where + ".expert")
            if mlp.get("shared") is not None:
                _check_expert(_need(mlp, "shared", where, (dict,)), where + ".shared")

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture}
        out.update(dataclasses.asdict(self))
        for key in ("embedding", "loop"):
            if out[key] is None:
                del out[key]
        if not out["streams"]:
            del out["streams"]
        return out


def run_order(n_layers: int, loop) -> list[int]:
    """The layers in the order they run: layers start .. stop - 1 `times` times in a row, the rest once."""
    if not loop:
        return list(range(n_layers))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n_layers))


def kupedra_blueprint(cfg: KupedraConfig) -> ModelBlueprint:
    """The design's layers as data: every size and constant comes from `cfg` (the rows of a distance table from the
    checkpoint); what the design fixes (the pairing of the rotation, which norm a mixer has, the form of the
    softmax's extra term, the experts' form, weights that are not renormalised) is set here as parameters of the
    parts."""
    eps, width, S = float(cfg.norm["eps"]), cfg.width, int(cfg.streams or 0)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]

        def attention(a, prefix, **more):
            return PartSpec("pair_rope_attention", {
                "hidden": width, "heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"], "vdim": a["vdim"],
                "scale": float(a["scale"]), "window": 0, "keep_first": 0, "bias": False, "values_from_keys": False,
                "eps": eps, **more}, prefix=prefix)

        if layer["type"] == "attention":
            rot = m.get("rot")
            mixer = attention(m, p + "mix.", sink_one=True, head_norm="unit", head_temp=True,
                              rot_base=float(rot["base"]) if rot else 1.0, rot_dims=int(rot["dims"]) if rot else 0,
                              rot_scaling=float((rot.get("scaling") or {}).get("factor", 1.0)) if rot else 1.0)
        else:
            left, right = m["left"], m["right"]
            qt = left.get("q_temp")
            left_spec = attention(left, p + "mix.left.", sink_one=False, sink_learned=True, head_norm="weight",
                                  rot_dims=0, q_temp=(float(qt["coef"]), int(qt["every"])) if qt else None,
                                  dist_bias=(int(left.get("bias_rows") or -1), float(left["bias_max"])))
            right_spec = PartSpec("matrix_memory", {"hidden": width, "heads": right["heads"], "dim": right["dim"],
                                                    "vdim": right["vdim"], "gate_cap": float(right["gate_cap"]),
                                                    "eps": eps, "floor": 1e-6}, prefix=p + "mix.right.")
            mixer = PartSpec("side_by_side", {"hidden": width, "parts": ((left_spec, 0.5), (right_spec, 0.5)),
                                              "out_norms": ("left.out", "right.out"), "eps": eps}, prefix=p + "mix.")
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            shared = mlp.get("shared")
            ffn = PartSpec("routed_experts", {
                "hidden": width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_ff": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]), "renorm": False,
                "shared_ff": shared["ff"] if shared is not None else 0, "shared_gate": shared is not None,
                "shared_limit": float(shared["limit"]) if shared is not None else 0.0}, prefix=p + "mlp.")
        names = ("norm1", "norm2") if mlp is not None else ("norm1",)
        norms = tuple(PartSpec("rmsnorm_hyper", {"hidden": width, "eps": eps, "scalar": True, "streams": S, "name": n},
                               prefix=p) for n in names)
        block = PartSpec("hyper_stream", {"hidden": width, "streams": S, "ffn": mlp is not None}, prefix=p)
        layers.append(LayerSpec("hyper_stream", mixer, ffn, norms, hidden=width, block_spec=block))
    # every run of a layer has a cache of its own, also the runs of a looped layer
    calls = tuple(LayerCall(layer=i, cache=n, write=True) for n, i in enumerate(run_order(len(cfg.layers), cfg.loop)))
    scale = float(cfg.embedding["scale"]) if cfg.embedding is not None else 1.0
    return ModelBlueprint(
        hidden=width, vocab=cfg.vocab,
        embedding=PartSpec("token_embedding_stream", {"vocab": cfg.vocab, "hidden": width, "table": "embed",
                                                      "scale": scale}),
        layers=tuple(layers), order=calls,
        final_norm=PartSpec("rmsnorm_hyper", {"hidden": width, "eps": eps, "scalar": True, "streams": S, "name": "norm"},
                            prefix="final."),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": width, "name": "head", "scale": float(cfg.logit_scale)}),
        max_positions=cfg.max_positions, eos_token_ids=(), stream_f32=True)
