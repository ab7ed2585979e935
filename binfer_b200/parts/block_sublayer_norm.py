"""Arrangement of a layer's parts with the norm on each sublayer's output.

``x += norm1(mixer(x))`` and, where the layer has a feed-forward, ``x += norm2(ffn(x))``:
both sublayers read the residual stream itself (in the activation type), and what they
return is normed before it is added.  The norm, the add into the float stream and the
rounding of the new stream for the next sublayer's products are one kernel
(``Norm.add_normed``); only the first sublayer of a model pays for a rounding pass of its
own.
"""
from __future__ import annotations

from typing import List

from ..config.specs import LayerSpec, NameLayout
from .base import (BuildEnv, EntryView, Part, ResidualStream, StepContext, build_ffn,
                   build_mixer, build_norm, register_block)


class SublayerNormBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int, names: NameLayout, index: int,
                 env: BuildEnv):
        p = names.layer_prefix.format(i=index)
        sfx = names.norm_suffix
        self.index, self.env = index, env
        self.mixer = build_mixer(spec.mixer, hidden_size, f"{p}{names.mixer}.", env)
        self.mixer_norm = build_norm(spec.norm, hidden_size,
                                     f"{p}{names.norm('post_mixer')}{sfx}", env)
        self.ffn = self.ffn_norm = None
        if spec.ffn is not None:
            self.ffn = build_ffn(spec.ffn, hidden_size, f"{p}{names.ffn}.", env)
            self.ffn_norm = build_norm(spec.norm, hidden_size,
                                       f"{p}{names.norm('post_ffn')}{sfx}", env)

    def parts(self) -> List[Part]:
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm)
                if p is not None]

    def param_specs(self):
        return [s for part in self.parts() for s in part.param_specs()]

    def load(self, get) -> None:
        for part in self.parts():
            part.load(get)

    def forward(self, stream: ResidualStream, ctx: StepContext, view: EntryView) -> None:
        h = stream.read(self.env.dtype)
        self.mixer_norm.add_normed(stream, self.mixer.forward(h, ctx, view))
        if self.ffn is not None:
            h = stream.read(self.env.dtype)
            self.ffn_norm.add_normed(stream, self.ffn.forward(h, ctx))


register_block("sublayer_norm", SublayerNormBlock)
