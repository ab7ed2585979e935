"""Mixture of gated feed-forward experts, with an optional shared expert.

A token's router logits ``z = W_router h`` are taken in float; the ``top`` experts with the
largest logits run, weighted by the softmax over those logits alone; the shared expert runs
for every token, times ``sigmoid(w_sg . h)`` when it has a gate.  Expert: ``W_down
(silu(W_gate h) * (W_up h))``.

How it runs here: the gate and up projections of all experts (and the shared one) are one
stacked weight, so one product gives every expert's pre-activations; a kernel applies the
activation and multiplies each expert's block by the token's weight for it (zero when not
chosen); one product with the down projections laid side by side then sums the weighted
experts in its own accumulation.  Unchosen experts cost arithmetic but no extra pass over
memory, no token is moved, and a token's result does not depend on what else is in the
batch.

A step of very few tokens in bfloat16 (a request that decodes alone) would read every expert
for nothing; there the chosen experts' rows alone are read, a warp per output row
(``ops.moe_sparse``).  The float32 engine keeps the one path, so that its sums have one order.
"""
from __future__ import annotations

import os
from typing import Callable, List

import torch

from ..config.specs import MoESpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, FeedForward, StepContext, register_ffn
from .linear import linear


# BINFER_B200_MOE_SPARSE=0: every step computes every expert
SPARSE = os.environ.get("BINFER_B200_MOE_SPARSE", "1") != "0"


class MoEFeedForward(FeedForward):
    def __init__(self, spec: MoESpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (supported: 'silu')")
        if not 1 <= spec.top <= spec.num_experts:
            raise ValueError("moe: top must be between 1 and the number of experts")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.E, self.top, self.ff, self.ff_sh = (spec.num_experts, spec.top, spec.expert_size,
                                                 spec.shared_size)
        self.F = self.E * self.ff + self.ff_sh
        self.gated_shared = bool(spec.shared_gate and self.ff_sh)
        self.w_gate_up = self.w_down = self.w_router = None

    def _expert_specs(self, p: str, ff: int) -> List[ParamSpec]:
        gate, up, down = self.spec.names
        return [ParamSpec(p + gate, (ff, self.hidden)), ParamSpec(p + up, (ff, self.hidden)),
                ParamSpec(p + down, (self.hidden, ff))]

    def _groups(self) -> List[List[ParamSpec]]:
        s = self.spec
        groups = [self._expert_specs(self.prefix + s.expert_prefix.format(e=e), self.ff)
                  for e in range(self.E)]
        if self.ff_sh:
            groups.append(self._expert_specs(self.prefix + s.shared_prefix, self.ff_sh))
        return groups

    def _router_specs(self) -> List[ParamSpec]:
        s = self.spec
        specs = [ParamSpec(self.prefix + s.router_name, (self.E, self.hidden), init="router",
                           role="vector")]
        if self.gated_shared:
            specs.append(ParamSpec(self.prefix + s.shared_prefix + s.shared_gate_name,
                                   (1, self.hidden), role="vector"))
        return specs

    def param_specs(self) -> List[ParamSpec]:
        return [x for g in self._groups() for x in g] + self._router_specs()

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        groups = self._groups()
        self.w_gate_up = torch.cat([get(g[0]) for g in groups] + [get(g[1]) for g in groups],
                                   dim=0).contiguous()
        self.w_down = torch.cat([get(g[2]) for g in groups], dim=1).contiguous()
        # the router (and the shared expert's gate as one more row) in float
        self.w_router = torch.cat([get(s) for s in self._router_specs()], dim=0).contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = x.shape[0]
        cols = self.E + (1 if self.gated_shared else 0)
        route_w = torch.empty((T, cols), dtype=torch.float32, device=x.device)
        top_ids = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        top_w = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        ops.moe_route(x, self.w_router, self.E, self.top, self.gated_shared, route_w, top_ids,
                      top_w)
        if (SPARSE and x.dtype == torch.bfloat16 and 2 * T * self.top <= self.E
                and ops.moe_sparse_takes(self.hidden, self.ff, self.ff_sh, self.top)):
            # so few tokens that most experts are chosen by none: read the chosen ones alone
            out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
            ops.moe_sparse(x, self.w_gate_up, self.w_down, top_ids, top_w, route_w, out, self.E,
                           self.ff, self.ff_sh, self.top)
            return out
        gu = linear(x, self.w_gate_up)
        act = torch.empty((T, self.F), dtype=x.dtype, device=x.device)
        ops.moe_act(gu, route_w, act, self.E, self.ff)
        return linear(act, self.w_down)


register_ffn("moe", MoEFeedForward)
