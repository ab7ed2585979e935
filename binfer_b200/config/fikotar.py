"""Typed configuration of the Fikotar decoder, read from its config.json keys.

Every Fikotar layer is *parallel*: one layer norm (weight and bias) whose output both
sublayers read, ``x += mixer(norm(x)) + ff(norm(x))``.  The mixer is itself two mixers side
by side on the same input, combined as ``left_scale * left + right_scale * right``:

* left: grouped softmax attention whose q, k and v projections pass a short causal
  convolution, with partial rotary positions (frequencies stretched by wavelength), q and k
  heads divided by their root mean square after the rotation, a sliding window that keeps
  the first tokens, and a learned sink logit per head in the softmax's denominator;
* right: retention, linear attention with a fixed decay per head, rotary positions, a head
  norm without weight and a ``silu`` gate.

The feed-forward is a mixture of experts with a shared expert behind a sigmoid gate, or
absent (``mlp: null``).  The model ends in a layer norm and an output head of its own,
whose logits are multiplied by ``logit_scale``.

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, ``layers``; of a
layer ``type`` (``parallel``), ``mixer.{left, right, left_scale, right_scale}``, ``mlp``; of
the left mixer ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``, ``scale``, ``rot.{base,
dims, scaling.{factor, low, high, original}}``, ``mask.{size, keep_first}``; of the right
mixer ``heads``, ``dim``, ``vdim``, ``decay``, ``rot.{base, dims}``; of a feed-forward ``kind``
(``moe``), ``router.{experts, top}``, ``expert.ff``, ``shared.ff``.  Tensors are named
``embed``, ``head``, ``final.norm`` (``.b``: bias) and ``l<i>.{norm1, mix.left.*,
mix.right.*, mlp.*}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .specs import (ConfigError, ConvWindowAttentionSpec, LayerSpec, MixerBranch, ModelSpec,
                    MoESpec, NameLayout, NormSpec, ParallelMixersSpec, RetentionSpec, RopeSpec,
                    ScheduleEntry, WavelengthScaling)

NORM_BIAS_SUFFIX = ".b"      # a norm's bias is the tensor of the same name with this added


def _need(d: Dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Missing required config key: {where}{key}")
    return d[key]


def _positive(v: Any, what: str) -> int:
    if isinstance(v, bool) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return int(v)


def _rope(rot: Optional[Dict[str, Any]], dim: int, where: str) -> Optional[RopeSpec]:
    if not rot:
        return None
    base = float(_need(rot, "base", where))
    dims = _positive(rot.get("dims") or dim, where + "dims")
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}dims must be even and at most dim, got {dims}")
    sc = rot.get("scaling")
    scaling = None
    if sc:
        w = where + "scaling."
        scaling = WavelengthScaling(
            factor=float(_need(sc, "factor", w)), low=float(_need(sc, "low", w)),
            high=float(_need(sc, "high", w)), original=float(_need(sc, "original", w)))
        if scaling.high == scaling.low or scaling.factor <= 0:
            raise ConfigError(f"{w}high must differ from low, and factor be positive")
    return RopeSpec(theta=base, rotary_dim=dims, wavelength_scaling=scaling)


@dataclass(frozen=True)
class FikotarConfig:
    raw: Dict[str, Any]
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[LayerSpec, ...]
    architectures: Tuple[str, ...] = ("Fikotar",)

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FikotarConfig":
        width = _positive(_need(raw, "width", ""), "width")
        vocab = _positive(_need(raw, "vocab", ""), "vocab")
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        entries = _need(raw, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        norm = NormSpec(kind="layernorm", eps=eps, bias_suffix=NORM_BIAS_SUFFIX)
        layers: List[LayerSpec] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            kind = _need(entry, "type", where)
            if kind != "parallel":
                raise ConfigError(f"{where}type {kind!r} is not supported (supported: "
                                  f"'parallel')")
            mx = _need(entry, "mixer", where)
            m = where + "mixer."
            mixer = ParallelMixersSpec(branches=(
                MixerBranch(cls._left(_need(mx, "left", m), eps, m + "left."), "left.",
                            float(mx.get("left_scale", 1.0))),
                MixerBranch(cls._right(_need(mx, "right", m), eps, m + "right."), "right.",
                            float(mx.get("right_scale", 1.0)))))
            ffn = cls._mlp(entry.get("mlp"), where + "mlp.")
            layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm=norm, block="parallel"))
        return cls(raw=copy.deepcopy(raw), vocab_size=vocab, hidden_size=width, norm_eps=eps,
                   logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(layers),
                   architectures=(str(raw.get("architecture", "Fikotar")),))

    @staticmethod
    def _left(mx: Dict[str, Any], eps: float, where: str) -> ConvWindowAttentionSpec:
        heads = _positive(_need(mx, "heads", where), where + "heads")
        kv_heads = _positive(mx.get("kv_heads") or heads, where + "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive(_need(mx, "dim", where), where + "dim")
        vdim = _positive(mx.get("vdim") or dim, where + "vdim")
        taps = int(mx.get("conv") or 0)
        if taps < 0:
            raise ConfigError(f"{where}conv must not be negative")
        mask = mx.get("mask") or {}
        window = mask.get("size")
        if window is not None:
            window = _positive(window, where + "mask.size")
        keep = int(mask.get("keep_first") or 0)
        if keep < 0:
            raise ConfigError(f"{where}mask.keep_first must not be negative")
        return ConvWindowAttentionSpec(
            num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
            conv_taps=taps, position=_rope(mx.get("rot"), dim, where + "rot."), unit_norm=True,
            norm_eps=eps, scale=None if mx.get("scale") is None else float(mx["scale"]),
            window=window, keep_first=keep if window is not None else 0, sinks=True)

    @staticmethod
    def _right(mx: Dict[str, Any], eps: float, where: str) -> RetentionSpec:
        heads = _positive(_need(mx, "heads", where), where + "heads")
        dim = _positive(_need(mx, "dim", where), where + "dim")
        vdim = _positive(mx.get("vdim") or dim, where + "vdim")
        decay = _need(mx, "decay", where)
        if not isinstance(decay, list) or len(decay) != heads:
            raise ConfigError(f"{where}decay must list one number per head ({heads})")
        return RetentionSpec(num_heads=heads, qk_dim=dim, v_dim=vdim,
                             decays=tuple(float(d) for d in decay),
                             position=_rope(mx.get("rot"), dim, where + "rot."), norm_eps=eps)

    @staticmethod
    def _mlp(mlp: Optional[Dict[str, Any]], where: str) -> Optional[MoESpec]:
        if mlp is None:
            return None
        kind = mlp.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}kind {kind!r} is not supported (supported: 'moe')")
        router = _need(mlp, "router", where)
        experts = _positive(_need(router, "experts", where + "router."), where + "router.experts")
        top = _positive(_need(router, "top", where + "router."), where + "router.top")
        if top > experts:
            raise ConfigError(f"{where}router.top ({top}) exceeds router.experts ({experts})")
        ff = _positive(_need(_need(mlp, "expert", where), "ff", where + "expert."),
                       where + "expert.ff")
        shared = mlp.get("shared")
        ff_sh = _positive(_need(shared, "ff", where + "shared."), where + "shared.ff") if shared else 0
        return MoESpec(num_experts=experts, top=top, expert_size=ff, shared_size=ff_sh,
                       shared_gate=bool(ff_sh))

    # ------------------------------------------------------------- derivation
    def to_spec(self) -> ModelSpec:
        norm = NormSpec(kind="layernorm", eps=self.norm_eps, bias_suffix=NORM_BIAS_SUFFIX)
        names = NameLayout(embed="embed", layer_prefix="l{i}.", input_norm="norm1",
                           post_mixer_norm="norm2", mixer="mix", ffn="mlp",
                           final_norm="final.norm", lm_head="head", norm_suffix="")
        return ModelSpec(
            architecture=self.architectures[0], hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, layers=self.layers,
            schedule=tuple(ScheduleEntry(i) for i in range(len(self.layers))),
            final_norm=norm, tie_word_embeddings=False, max_position_embeddings=1 << 30,
            eos_token_ids=(), bos_token_id=None, pad_token_id=None,
            logit_scale=self.logit_scale, names=names)

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
