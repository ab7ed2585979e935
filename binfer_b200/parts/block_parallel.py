"""Arrangement of a layer's parts with one norm that both sublayers read.

``h = norm(x);  x += mixer(h) + ffn(h)`` (a layer may have no feed-forward).  The mixer's
output is left pending on the residual stream and the feed-forward's rides beside it as a
second pending add; the next norm (this arrangement's, or the model's final one) folds
both into the float stream in the pass that norms it.
"""
from __future__ import annotations

from typing import List

from ..config.specs import LayerSpec, NameLayout
from .base import (BuildEnv, EntryView, Part, ResidualStream, StepContext, build_ffn,
                   build_mixer, build_norm, register_block)


class ParallelBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int, names: NameLayout, index: int,
                 env: BuildEnv):
        p = names.layer_prefix.format(i=index)
        self.index, self.env = index, env
        self.norm = build_norm(spec.norm, hidden_size,
                               f"{p}{names.norm('input')}{names.norm_suffix}", env)
        self.mixer = build_mixer(spec.mixer, hidden_size, f"{p}{names.mixer}.", env)
        self.ffn = (build_ffn(spec.ffn, hidden_size, f"{p}{names.ffn}.", env)
                    if spec.ffn is not None else None)

    def parts(self) -> List[Part]:
        return [p for p in (self.norm, self.mixer, self.ffn) if p is not None]

    def param_specs(self):
        return [s for part in self.parts() for s in part.param_specs()]

    def load(self, get) -> None:
        for part in self.parts():
            part.load(get)

    def forward(self, stream: ResidualStream, ctx: StepContext, view: EntryView) -> None:
        h = stream.norm_input(self.norm)
        y = self.mixer.forward(h, ctx, view)
        if self.ffn is not None:
            stream.add_pair(y, self.ffn.forward(h, ctx))
        else:
            stream.add(y)


register_block("parallel", ParallelBlock)
