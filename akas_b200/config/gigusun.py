"""Typed configuration of the Gigusun decoder, read from its own config.json keys.

A Gigusun model is a list of layers, each with one of three mixers (softmax attention over a sliding
window with kept first tokens, gated linear attention, the gated delta rule) and an optional dense
feed-forward with a PolyNorm activation, around a float32 residual stream with one-plus RMS norms.
Token embeddings get a learned position vector and a norm before the first layer; the head is a
tensor of its own. config.json lists the layers one by one (``layers[i] = {"type", "mixer", "mlp"}``),
so every layer may have sizes of its own; what the file does not give (the rank of the decay's
low-rank pair) is taken from the checkpoint's tensor shapes.

Checkpoint names: ``embed``, ``pos``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
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
    GatedDeltaSpec,
    GatedLinearAttentionSpec,
    LayerSpec,
    ModelSpec,
    PolyNormMLPSpec,
    RMSNormSpec,
)

ARCHITECTURE = "Gigusun"
MIXER_TYPES = ("attention", "gla", "delta")


def _int(where: str, data: Mapping[str, Any], key: str, least: int = 1) -> int:
    value = data.get(key)
    if type(value) is not int or value < least:
        raise ConfigError(f"{where}.{key} must be an integer of at least {least}, got {value!r}")
    return value


def _number(where: str, data: Mapping[str, Any], key: str) -> float:
    value = data.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value <= 0:
        raise ConfigError(f"{where}.{key} must be a positive finite number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class GigusunLayer:
    """One entry of ``layers``: the mixer's type and sizes as config.json gives them, and the feed-forward's width
    (None: the layer has none)."""

    type: str
    mixer: Tuple[Tuple[str, Any], ...]  # the mixer's keys, sorted, as a tuple so that the layer can be hashed
    ff: Optional[int]

    @property
    def options(self) -> dict:
        return {k: (dict(v) if isinstance(v, tuple) else v) for k, v in self.mixer}


@dataclass(frozen=True)
class GigusunConfig:
    width: int
    vocab: int
    max_positions: int
    norm_eps: float
    layers: Tuple[GigusunLayer, ...]
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "GigusunConfig":
        if data.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {ARCHITECTURE!r}")
        width = _int("config", data, "width")
        vocab = _int("config", data, "vocab")
        positions = _int("config", data, "max_positions")
        eps = _number("norm", data.get("norm") or {}, "eps")
        listed = data.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}.type {kind!r} is none of {list(MIXER_TYPES)}")
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}.mixer must be an object")
            where += ".mixer"
            heads = _int(where, m, "heads")
            _int(where, m, "dim")
            _int(where, m, "vdim")
            if kind in ("attention", "delta"):
                if heads % _int(where, m, "kv_heads"):
                    raise ConfigError(f"{where}: {heads} heads are not a multiple of {m['kv_heads']} kv_heads")
            if kind == "attention":
                mask = m.get("mask")
                if not isinstance(mask, Mapping):
                    raise ConfigError(f"{where}.mask must be an object")
                _int(where + ".mask", mask, "size")
                _int(where + ".mask", mask, "keep_first", least=0)
                _number(where, m, "scale")
                _number(where, m, "softcap")
            elif kind == "gla":
                _number(where, m, "tau")
                if "rank" in m:
                    _int(where, m, "rank")
            else:
                _int(where, m, "conv")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind {mlp.get('kind')!r} is not 'dense'")
                ff = _int(f"layers[{i}].mlp", mlp, "ff")
            frozen = tuple(sorted((k, tuple(sorted(v.items())) if isinstance(v, Mapping) else v) for k, v in m.items()))
            layers.append(GigusunLayer(kind, frozen, ff))
        eos = data.get("eos_token_id")
        return cls(width=width, vocab=vocab, max_positions=positions, norm_eps=eps, layers=tuple(layers),
                   eos_token_id=eos if type(eos) is int else None)

    @classmethod
    def from_json(cls, path) -> "GigusunConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        """A config.json that reads back as this configuration."""
        data = dict(
            architecture=ARCHITECTURE,
            layers=[dict(type=l.type, mixer=l.options, mlp=None if l.ff is None else dict(ff=l.ff, kind="dense"))
                    for l in self.layers],
            max_positions=self.max_positions,
            norm=dict(eps=self.norm_eps),
            vocab=self.vocab,
            width=self.width,
        )
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # ------------------------------------------------------------------ the model it describes

    def mixer_spec(self, layer: GigusunLayer):
        m, c, eps = layer.options, self.width, self.norm_eps
        if layer.type == "attention":
            return AttentionSpec(
                c, m["heads"], m["kv_heads"], m["dim"],
                qk_norm=RMSNormSpec(m["dim"], eps), position=None, window=m["mask"]["size"], scale=float(m["scale"]),
                v_head_dim=m["vdim"], softcap=float(m["softcap"]), distance_bias=True, keep_first=m["mask"]["keep_first"],
                sink=True, gate="head",
                names={"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "out_proj.weight": "o",
                       "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "gate.weight": "g"},
            )
        if layer.type == "gla":
            return GatedLinearAttentionSpec(c, m["heads"], m["dim"], m["vdim"], m.get("rank"), float(m["tau"]), eps)
        return GatedDeltaSpec(c, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], eps)

    def model_spec(self) -> ModelSpec:
        norm = RMSNormSpec(self.width, self.norm_eps, zero_centered=True)
        layers = []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            has_ff = layer.ff is not None
            layers.append(LayerSpec(
                mixer=self.mixer_spec(layer),
                ffn=PolyNormMLPSpec(self.width, layer.ff, self.norm_eps) if has_ff else None,
                mixer_norm=norm,
                ffn_norm=norm if has_ff else None,
                mixer_prefix=prefix + "mix.",
                ffn_prefix=prefix + "mlp.",
                mixer_norm_name=prefix + "norm1",
                ffn_norm_name=prefix + "norm2",
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
            max_context=self.max_positions,
            position_table_name="pos",
            embedding_norm=norm,
            embedding_norm_name="embed.norm",
        )
