"""Retention (linear attention with a fixed decay per head) as a mixer part with
per-request state.

Per head, with a state ``S [dk, dv]`` that starts at zero for a new request::

    q = rot(W_q h)      k = rot(W_k h) / sqrt(dk)      v = W_v h
    S <- decay_h S + k v^T          o = S^T q

and the mixer returns ``W_o (o / rms_head(o) * silu(W_g h))``.  There is no softmax and no
denominator.  The q, k, v and gate projections are one product against the stacked weight;
rotation, recurrence and the head norm are float whatever the engine's precision; the state
lives in the cache manager's slots and is carried from step to step, so a prompt can be cut
anywhere and a request can share a step with others.  ``w_in`` / ``w_out`` /
``run(proj, ctx, view, out, out_scale)`` let ``ParallelMixers`` run it as a branch.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..cache.manager import StateNeed
from ..config.specs import RetentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, build_position, register_mixer
from .linear import linear


class RetentionMixer(Mixer):
    def __init__(self, spec: RetentionSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.qk_dim > ops.RETENTION_MAX_QK_DIM:
            raise ValueError(f"retention: a key size of {spec.qk_dim} is not supported "
                             f"(at most {ops.RETENTION_MAX_QK_DIM})")
        if len(spec.decays) != spec.num_heads:
            raise ValueError("retention: one decay per head is needed")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.heads, self.dk, self.dv = spec.num_heads, spec.qk_dim, spec.v_dim
        self.qk_size, self.v_size = self.heads * self.dk, self.heads * self.dv
        self.position = (build_position(spec.position, self.dk, env)
                         if spec.position is not None else None)
        if self.position is not None and self.position.inv_freq is None:
            raise ValueError("retention takes rotary encodings only")
        self.decays = torch.tensor(spec.decays, dtype=torch.float64).to(torch.float32).to(env.device)
        self.names = dict(spec.names)
        self.in_rows, self.out_cols = 2 * self.qk_size + 2 * self.v_size, self.v_size
        self.w_in = self.w_out = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        shape = {"q": (self.qk_size, self.hidden), "k": (self.qk_size, self.hidden),
                 "v": (self.v_size, self.hidden), "g": (self.v_size, self.hidden),
                 "o": (self.hidden, self.v_size)}[role]
        return ParamSpec(self.prefix + self.names[role], shape)

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in ("q", "k", "v", "g", "o")]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        self.w_in = torch.cat([g("q"), g("k"), g("v"), g("g")], dim=0).contiguous()
        self.w_out = g("o")

    # ------------------------------------------------------------------- state
    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads * self.dk * self.dv,), "float32")

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.out_cols), dtype=x.dtype, device=x.device)
        self.run(linear(x, self.w_in), ctx, view, out, 1.0)
        return linear(out, self.w_out)

    def run(self, proj: torch.Tensor, ctx: StepContext, view: EntryView, out: torch.Tensor,
            out_scale: float) -> None:
        T = proj.shape[0]
        o_raw = torch.empty((T, self.v_size), dtype=torch.float32, device=proj.device)
        inv = self.position.inv_freq if self.position is not None else None
        ops.retention_scan(proj, 0, self.qk_size, 2 * self.qk_size, self.decays, inv,
                           ctx.positions, view.state, ctx.q_start, ctx.state_slots, o_raw, ctx.B,
                           self.heads, self.dk, self.dv, self.dk ** -0.5, ctx.err,
                           max_q=1 if ctx.decode_only else ctx.max_q_len)
        ops.retention_out(o_raw, proj, 2 * self.qk_size + self.v_size, out, self.heads, self.dv,
                          self.spec.norm_eps, out_scale)


register_mixer("retention", RetentionMixer)
