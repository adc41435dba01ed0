"""Typed configuration of the Girelix decoder, read from its own config.json keys.

A Girelix layer norms the float32 residual stream once and hands the result to two sublayers at the same time: a
mixer made of two mixers side by side (causal softmax attention whose values are its keys and whose softmax has a
learned sink per head, with rotary pairs of neighbouring channels; and linear attention with a constant decay per
head) and a mixture of SwiGLU experts with identity experts and a grouped, corrected choice. Their results, each
through a learned scale per channel, are added to the stream times a constant. config.json lists the layers one by
one (``layers[i] = {"type", "mixer", "mlp"}``), so every layer may have sizes of its own and a layer may have no
feed-forward.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.mix.left.{q,k,sink,o}``,
``l<i>.mix.right.{q,k,v,g,o,norm}``, ``l<i>.mlp.{router,correction}``, ``l<i>.mlp.e<j>.{gate,up,down}``,
``final.norm``, ``head``.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .specs import (
    AttentionSpec,
    DecayedLinearAttentionSpec,
    LayerSpec,
    ModelSpec,
    ParallelMixerSpec,
    RMSNormSpec,
    RopeSpec,
    RoutedExpertsSpec,
)

ARCHITECTURE = "Girelix"
LAYER_TYPES = ("parallel",)


def _int(where: str, data: Mapping[str, Any], key: str, least: int = 1) -> int:
    value = data.get(key) if isinstance(data, Mapping) else None
    if type(value) is not int or value < least:
        raise ConfigError(f"{where}.{key} must be an integer of at least {least}, got {value!r}")
    return value


def _number(where: str, data: Mapping[str, Any], key: str, positive: bool = True) -> float:
    value = data.get(key) if isinstance(data, Mapping) else None
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"{where}.{key} must be a {'positive ' if positive else ''}finite number, got {value!r}")
    return float(value)


def _freeze(value):
    if isinstance(value, Mapping):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    if isinstance(value, (list, tuple)):
        return ("__list__", tuple(_freeze(v) for v in value))
    return value


def _thaw(value):
    if isinstance(value, tuple) and len(value) == 2 and value[0] == "__list__":
        return [_thaw(v) for v in value[1]]
    if isinstance(value, tuple):
        return {k: _thaw(v) for k, v in value}
    return value


@dataclass(frozen=True)
class GirelixLayer:
    """One entry of ``layers``: its type and what config.json gives for its mixer and its feed-forward (None: none),
    kept as nested tuples so that the layer can be hashed."""

    type: str
    mixer: tuple
    mlp: Optional[tuple]

    @property
    def mixer_options(self) -> dict:
        return _thaw(self.mixer)

    @property
    def mlp_options(self) -> Optional[dict]:
        return None if self.mlp is None else _thaw(self.mlp)


@dataclass(frozen=True)
class GirelixConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[GirelixLayer, ...]
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "GirelixConfig":
        if data.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {ARCHITECTURE!r}")
        width = _int("config", data, "width")
        vocab = _int("config", data, "vocab")
        eps = _number("norm", data.get("norm") or {}, "eps")
        mult = _number("config", data, "residual_mult", positive=False)
        listed = data.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = entry.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{where}.type {kind!r} is none of {list(LAYER_TYPES)}")
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}.mixer must be an object")
            cls._check_mixer(where + ".mixer", m)
            mlp = entry.get("mlp")
            if mlp is not None:
                cls._check_mlp(where + ".mlp", mlp)
            layers.append(GirelixLayer(kind, _freeze(m), None if mlp is None else _freeze(mlp)))
        eos = data.get("eos_token_id")
        return cls(width=width, vocab=vocab, norm_eps=eps, residual_mult=mult, layers=tuple(layers),
                   eos_token_id=eos if type(eos) is int else None)

    @staticmethod
    def _check_mixer(where: str, m: Mapping[str, Any]) -> None:
        left, right = m.get("left"), m.get("right")
        if not isinstance(left, Mapping) or not isinstance(right, Mapping):
            raise ConfigError(f"{where} must hold the objects 'left' and 'right'")
        _number(where, m, "left_scale", positive=False)
        _number(where, m, "right_scale", positive=False)
        w = where + ".left"
        heads, dim = _int(w, left, "heads"), _int(w, left, "dim")
        if heads % _int(w, left, "kv_heads"):
            raise ConfigError(f"{w}: {heads} heads are not a multiple of {left['kv_heads']} kv_heads")
        if _int(w, left, "vdim") != dim:
            raise ConfigError(f"{w}: the values are the keys, so vdim {left['vdim']} must equal dim {dim}")
        _number(w, left, "scale")
        rot = left.get("rot")
        dims = _int(w + ".rot", rot, "dims", least=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{w}.rot.dims {dims} must be even and at most dim {dim}")
        _number(w + ".rot", rot, "base")
        w = where + ".right"
        heads = _int(w, right, "heads")
        _int(w, right, "dim"), _int(w, right, "vdim")
        decay = right.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or not all(
                isinstance(d, (int, float)) and not isinstance(d, bool) and math.isfinite(d) for d in decay):
            raise ConfigError(f"{w}.decay must list one finite number for each of the {heads} heads")

    @staticmethod
    def _check_mlp(where: str, mlp: Mapping[str, Any]) -> None:
        if mlp.get("kind") != "moe":
            raise ConfigError(f"{where}.kind {mlp.get('kind')!r} is not 'moe'")
        _int(where + ".expert", mlp.get("expert"), "ff")
        r = mlp.get("router")
        w = where + ".router"
        outputs = _int(w, r, "experts") + _int(w, r, "identity", least=0)
        top = _int(w, r, "top")
        groups = r.get("groups")
        count, keep = _int(w + ".groups", groups, "count"), _int(w + ".groups", groups, "keep")
        if outputs % count or keep > count:
            raise ConfigError(f"{w}: {outputs} router outputs do not form {count} equal groups of which {keep} stay")
        if top > keep * (outputs // count):
            raise ConfigError(f"{w}.top {top} exceeds what {keep} groups of {outputs // count} offer")

    @classmethod
    def from_json(cls, path) -> "GirelixConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        """A config.json that reads back as this configuration."""
        data = dict(
            architecture=ARCHITECTURE,
            layers=[dict(type=l.type, mixer=l.mixer_options, mlp=l.mlp_options) for l in self.layers],
            norm=dict(eps=self.norm_eps),
            residual_mult=self.residual_mult,
            vocab=self.vocab,
            width=self.width,
        )
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # ------------------------------------------------------------------ the model it describes

    def mixer_spec(self, layer: GirelixLayer) -> ParallelMixerSpec:
        m, c = layer.mixer_options, self.width
        left, right = m["left"], m["right"]
        rot = left["rot"]
        attention = AttentionSpec(
            c, left["heads"], left["kv_heads"], left["dim"],
            position=RopeSpec(left["dim"], float(rot["base"]), rot["dims"], interleaved=True) if rot["dims"] else None,
            scale=float(left["scale"]), v_head_dim=left["dim"], sink="learned", values_are_keys=True,
            names={"q_proj.weight": "q", "k_proj.weight": "k", "out_proj.weight": "o", "sink": "sink"},
        )
        linear = DecayedLinearAttentionSpec(
            c, right["heads"], right["dim"], right["vdim"], tuple(float(d) for d in right["decay"]), self.norm_eps,
            activation="silu", whole_norm=True, gate_activation="sigmoid", q_scale=1.0,
        )
        return ParallelMixerSpec(c, (("left.", attention, float(m["left_scale"])), ("right.", linear, float(m["right_scale"]))))

    def ffn_spec(self, layer: GirelixLayer) -> Optional[RoutedExpertsSpec]:
        f = layer.mlp_options
        if f is None:
            return None
        r = f["router"]
        return RoutedExpertsSpec(self.width, f["expert"]["ff"], r["experts"], r["identity"], r["top"], r["groups"]["count"],
                                 r["groups"]["keep"])

    def model_spec(self) -> ModelSpec:
        norm = RMSNormSpec(self.width, self.norm_eps)
        layers = []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            layers.append(LayerSpec(
                mixer=self.mixer_spec(layer),
                ffn=self.ffn_spec(layer),
                mixer_norm=norm,
                ffn_norm=None,
                mixer_prefix=prefix + "mix.",
                ffn_prefix=prefix + "mlp.",
                mixer_norm_name=prefix + "norm1",
                ffn_norm_name=None,
                arrangement="parallel",
                residual_multiplier=self.residual_mult,
                mixer_scale_name=prefix + "ls1",
                ffn_scale_name=prefix + "ls2",
            ))
        return ModelSpec(
            architecture=ARCHITECTURE,
            hidden_size=self.width,
            vocab_size=self.vocab,
            layers=tuple(layers),
            final_norm=norm,
            embedding_name="embed",
            final_norm_name="final.norm",
            head_name="head",
            head_optional=False,
        )
