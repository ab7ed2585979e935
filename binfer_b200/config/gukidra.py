"""Typed configuration of the Gukidra hybrid decoder, read from its config.json keys.

Gukidra alternates two kinds of mixer, listed layer by layer under ``layers``: a matrix
memory with exponential gates (``type: mlstm``) and windowed grouped attention with pooled
blocks of older keys (``type: attention``).  Each entry carries its mixer's sizes under
``mixer`` and its feed-forward under ``mlp`` (``null``: the layer has none).  A sublayer
reads the residual stream itself; the norm, whose checkpoint weight is the deviation from one, sits on the
sublayer's output.  The embedding is scaled by ``embedding.scale`` and tied to the output
head (which uses the table unscaled).

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``layers``;
of an mlstm mixer ``heads``, ``dim``, ``vdim``, ``gate_cap``; of an attention mixer
``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot.base``, ``rot.dims``,
``mask.size``, ``mask.pool`` and optionally ``kv_from`` (the index of the layer whose keys
and values it reads); of a feed-forward ``kind`` (``dense``) and ``ff``.  Tensors are named
``embed``, ``final.norm`` and ``l<i>.{norm1,norm2,mix.*,mlp.*}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .specs import (ConfigError, GatedMLPSpec, LayerSpec, MLSTMSpec, ModelSpec, NameLayout,
                    NormSpec, PooledWindowAttentionSpec, RopeSpec, ScheduleEntry)

# constants that the design fixes
SINK_LOGIT = 0.0            # the softmax's denominator holds exp(0) beside the keys
NORM_WEIGHT_OFFSET = 1.0    # checkpoints hold w - 1 for a norm weight w

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g"),
                    ("q_norm", "q.norm"), ("k_norm", "k.norm"))
_MLSTM_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"),
                ("i", "i"), ("i_bias", "i.b"), ("f", "f"), ("f_bias", "f.b"))
_MLP_NAMES = ("gate", "up", "down")


def _need(d: Dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Missing required config key: {where}{key}")
    return d[key]


def _positive(v: Any, what: str) -> int:
    if int(v) != v or int(v) <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class GukidraConfig:
    raw: Dict[str, Any]
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LayerSpec, ...]
    cache_from: Tuple[Optional[int], ...]
    architectures: Tuple[str, ...] = ("Gukidra",)

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GukidraConfig":
        width = _positive(_need(raw, "width", ""), "width")
        vocab = _positive(_need(raw, "vocab", ""), "vocab")
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        scale = float((raw.get("embedding") or {}).get("scale", 1.0))
        entries = _need(raw, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        norm = NormSpec(eps=eps, offset=NORM_WEIGHT_OFFSET)
        layers: List[LayerSpec] = []
        cache_from: List[Optional[int]] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            kind = _need(entry, "type", where)
            mx = _need(entry, "mixer", where)
            src = None
            if kind == "mlstm":
                mixer = cls._mlstm(mx, eps, where + "mixer.")
            elif kind == "attention":
                mixer, src = cls._attention(mx, eps, where + "mixer.")
            else:
                raise ConfigError(f"{where}type {kind!r} is not supported "
                                  f"(supported: 'mlstm', 'attention')")
            ffn = cls._mlp(entry.get("mlp"), where + "mlp.")
            layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm=norm, block="sublayer_norm"))
            cache_from.append(src)
        for i, src in enumerate(cache_from):
            if src is None:
                continue
            a = layers[i].mixer
            b = layers[src].mixer if 0 <= src < i else None
            if (not isinstance(b, PooledWindowAttentionSpec) or cache_from[src] is not None):
                raise ConfigError(f"layers[{i}].mixer.kv_from must name an earlier attention "
                                  f"layer with keys and values of its own, got {src}")
            if (a.num_kv_heads, a.head_dim, a.value_dim) != (b.num_kv_heads, b.head_dim,
                                                             b.value_dim):
                raise ConfigError(f"layers[{i}] reads the keys and values of layers[{src}], "
                                  f"whose head count or sizes differ")
        cfg = cls(raw=copy.deepcopy(raw), vocab_size=vocab, hidden_size=width, norm_eps=eps,
                  embedding_scale=scale, layers=tuple(layers), cache_from=tuple(cache_from),
                  architectures=(str(raw.get("architecture", "Gukidra")),))
        return cfg

    @staticmethod
    def _mlstm(mx: Dict[str, Any], eps: float, where: str) -> MLSTMSpec:
        return MLSTMSpec(
            num_heads=_positive(_need(mx, "heads", where), where + "heads"),
            qk_dim=_positive(_need(mx, "dim", where), where + "dim"),
            v_dim=_positive(_need(mx, "vdim", where), where + "vdim"),
            gate_cap=float(mx.get("gate_cap") or 0.0), norm_eps=eps, names=_MLSTM_NAMES)

    @staticmethod
    def _attention(mx: Dict[str, Any], eps: float, where: str):
        heads = _positive(_need(mx, "heads", where), where + "heads")
        kv_heads = _positive(mx.get("kv_heads") or heads, where + "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive(_need(mx, "dim", where), where + "dim")
        vdim = _positive(mx.get("vdim") or dim, where + "vdim")
        rot, mask = mx.get("rot"), mx.get("mask") or {}
        position = value_rotation = None
        interleaved = False
        if rot:
            base = float(_need(rot, "base", where + "rot."))
            dims = _positive(rot.get("dims") or dim, where + "rot.dims")
            if dims % 2 or dims > dim:
                raise ConfigError(f"{where}rot.dims must be even and at most dim, got {dims}")
            if vdim % 2:
                raise ConfigError(f"{where}vdim must be even for rotated values, got {vdim}")
            layout = str(rot.get("layout", "half"))
            if layout not in ("half", "halves", "interleaved"):
                raise ConfigError(f"{where}rot.layout {layout!r} is not supported")
            interleaved = layout == "interleaved"
            position = RopeSpec(theta=base, rotary_dim=dims)
            value_rotation = RopeSpec(theta=base, rotary_dim=vdim)
        window = mask.get("size")
        pool = int(mask.get("pool") or 0)
        if window is not None:
            window = _positive(window, where + "mask.size")
        if pool < 0:
            raise ConfigError(f"{where}mask.pool must not be negative")
        src = mx.get("kv_from")
        spec = PooledWindowAttentionSpec(
            num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim, qk_norm=True,
            qk_norm_eps=eps, window=window, pool=pool if window is not None else 0,
            scale=None if mx.get("scale") is None else float(mx["scale"]), position=position,
            value_rotation=value_rotation, interleaved=interleaved, sink=SINK_LOGIT,
            head_gate=True, own_cache=src is None, names=_ATTENTION_NAMES)
        return spec, (None if src is None else int(src))

    @staticmethod
    def _mlp(mlp: Optional[Dict[str, Any]], where: str) -> Optional[GatedMLPSpec]:
        if mlp is None:
            return None
        kind = mlp.get("kind", "dense")
        if kind != "dense":
            raise ConfigError(f"{where}kind {kind!r} is not supported (supported: 'dense')")
        return GatedMLPSpec(intermediate_size=_positive(_need(mlp, "ff", where), where + "ff"),
                            activation="silu", names=_MLP_NAMES)

    # ------------------------------------------------------------- derivation
    def to_spec(self) -> ModelSpec:
        norm = NormSpec(eps=self.norm_eps, offset=NORM_WEIGHT_OFFSET)
        names = NameLayout(embed="embed", layer_prefix="l{i}.", input_norm="norm0",
                           post_mixer_norm="norm1", mixer="mix", ffn="mlp",
                           final_norm="final.norm", lm_head="head",
                           more_norms=(("post_ffn", "norm2"),), norm_suffix="")
        return ModelSpec(
            architecture=self.architectures[0], hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, layers=self.layers,
            schedule=tuple(ScheduleEntry(i, src) for i, src in enumerate(self.cache_from)),
            final_norm=norm, tie_word_embeddings=True,
            max_position_embeddings=1 << 30, eos_token_ids=(), bos_token_id=None,
            pad_token_id=None, embedding_scale=self.embedding_scale, names=names)

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that :meth:`from_dict` reads back to this object."""
        return copy.deepcopy(self.raw)

    # ---------------------------------------------------------------- memory
    def num_parameters(self) -> int:
        from ..parts.model import param_specs_for
        total = 0
        for s in param_specs_for(self.to_spec()):
            n = 1
            for d in s.shape:
                n *= d
            total += n
        return total
