"""Several mixers side by side on the same input: ``sum_i scale_i mixer_i(h)``.

The branches are ordinary mixers that also offer the branch interface: ``in_rows`` /
``w_in [in_rows, width]`` (their stacked input projections), ``out_cols`` / ``w_out [width,
out_cols]`` and ``run(proj, ctx, view, out, out_scale)``, which turns the branch's block of
projections into its block of pre-output activations times ``out_scale``.  This part stacks
the branches' input weights into one product and their output weights, side by side, into
another, so the sum over the branches is that product's own accumulation and the branch
factors ride on the activations.

Cache and state: at most one branch may keep pages (its need is this mixer's); the
branches' fixed-size states are laid side by side in one flat float state per request, and
each branch sees its own columns.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional

import torch

from ..cache.manager import KVNeed, StateNeed
from ..config.specs import ParallelMixersSpec
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, build_mixer, register_mixer
from .linear import linear


class ParallelMixers(Mixer):
    def __init__(self, spec: ParallelMixersSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if not spec.branches:
            raise ValueError("parallel mixers need at least one branch")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.branches = [build_mixer(b.spec, hidden_size, prefix + b.prefix, env)
                         for b in spec.branches]
        self.scales = [float(b.scale) for b in spec.branches]
        for m in self.branches:
            if not all(hasattr(m, a) for a in ("in_rows", "out_cols", "run")):
                raise ValueError(f"{type(m).__name__} cannot run as a branch: it lacks the "
                                 f"interface in_rows / out_cols / w_in / w_out / run")
        if sum(m.kv_need() is not None for m in self.branches) > 1:
            raise ValueError("at most one branch of parallel mixers may keep cache pages")
        self.state_cols = []
        off = 0
        for m in self.branches:
            need = m.state_need()
            n = 0
            if need is not None:
                if need.dtype != "float32":
                    raise ValueError("branches of parallel mixers keep float32 state")
                n = 1
                for d in need.shape:
                    n *= int(d)
            self.state_cols.append((off, n))
            off += n
        self.state_size = off
        self.in_off, self.out_off = [], []
        a = b = 0
        for m in self.branches:
            self.in_off.append(a)
            self.out_off.append(b)
            a += m.in_rows
            b += m.out_cols
        self.in_rows, self.out_cols = a, b
        self.w_in = self.w_out = None

    def param_specs(self) -> List[ParamSpec]:
        return [s for m in self.branches for s in m.param_specs()]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        for m in self.branches:
            m.load(get)
        self.w_in = torch.cat([m.w_in for m in self.branches], dim=0).contiguous()
        self.w_out = torch.cat([m.w_out for m in self.branches], dim=1).contiguous()
        for m in self.branches:          # the stacked copies are the ones that are read
            m.w_in = m.w_out = None

    def kv_need(self) -> Optional[KVNeed]:
        for m in self.branches:
            need = m.kv_need()
            if need is not None:
                return need
        return None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.state_size,), "float32") if self.state_size else None

    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        T = x.shape[0]
        proj = linear(x, self.w_in)
        acts = torch.empty((T, self.out_cols), dtype=x.dtype, device=x.device)
        for m, scale, a, b, (so, sn) in zip(self.branches, self.scales, self.in_off, self.out_off,
                                            self.state_cols):
            sub = dataclasses.replace(
                view, state=view.state[:, so:so + sn] if sn else None)
            m.run(proj[:, a:a + m.in_rows], ctx, sub, acts[:, b:b + m.out_cols], scale)
        return linear(acts, self.w_out)


register_mixer("parallel_mixers", ParallelMixers)
