"""The matrix memory with exponential gates (mLSTM) as a mixer part with per-request state.

Per head, with a state ``S [dk, dv]``, ``n [dk]`` and a running maximum ``m`` that start at
zero for a new request, a token with input ``h`` does::

    q = W_q h / sqrt(dk)      k = W_k h      v = W_v h
    i = cap tanh((W_i h + b_i) / cap)        f = logsigmoid(cap tanh((W_f h + b_f) / cap))
    m' = max(f + m, i)
    S' = exp(f + m - m') S + exp(i - m') k v^T        n' = exp(f + m - m') n + exp(i - m') k
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

and the mixer returns ``W_o (o / rms_head(o) * w_norm * sigmoid(W_g h))``.  The q, k, v and
output-gate projections are one product against the stacked weight; the two gate
projections are a kernel of their own that leaves the log gates in float; the state lives
in the cache manager's slots (float, whatever the engine's precision) and is carried from
step to step, so a prompt can be cut anywhere and a request can share a step with others.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..cache.manager import StateNeed
from ..config.specs import MLSTMSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, register_mixer
from .linear import linear


class MLSTMMixer(Mixer):
    def __init__(self, spec: MLSTMSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.qk_dim > ops.MLSTM_MAX_QK_DIM:
            raise ValueError(f"mlstm: a key size of {spec.qk_dim} is not supported "
                             f"(at most {ops.MLSTM_MAX_QK_DIM})")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.heads, self.dk, self.dv = spec.num_heads, spec.qk_dim, spec.v_dim
        self.qk_size, self.v_size = self.heads * self.dk, self.heads * self.dv
        self.names = dict(spec.names)
        self.w_proj = self.w_gates = self.gate_bias = self.norm_w = self.w_o = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        n = self.prefix + self.names[role]
        H = self.heads
        shape, kind, init = {
            "q": ((self.qk_size, self.hidden), "matrix", "matrix"),
            "k": ((self.qk_size, self.hidden), "matrix", "matrix"),
            "v": ((self.v_size, self.hidden), "matrix", "matrix"),
            "g": ((self.v_size, self.hidden), "matrix", "matrix"),
            "o": ((self.hidden, self.v_size), "matrix", "matrix"),
            "norm": ((self.v_size,), "vector", "norm"),
            "i": ((H, self.hidden), "matrix", "matrix"),
            "f": ((H, self.hidden), "matrix", "matrix"),
            "i_bias": ((H,), "vector", "around_zero"),
            "f_bias": ((H,), "vector", "norm"),
        }[role]
        return ParamSpec(n, shape, init=init, role=kind)

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in ("q", "k", "v", "g", "o", "norm", "i", "i_bias", "f",
                                        "f_bias")]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        # one [2 H dk + 2 H dv, width] weight: q, k, v and the output gate of a token side by side
        self.w_proj = torch.cat([g("q"), g("k"), g("v"), g("g")], dim=0).contiguous()
        self.w_gates = torch.cat([g("i"), g("f")], dim=0).contiguous()
        self.gate_bias = torch.cat([g("i_bias"), g("f_bias")], dim=0).float().contiguous()
        self.norm_w = g("norm")
        self.w_o = g("o")

    # ------------------------------------------------------------------- state
    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads, ops.mlstm_state_size(self.dk, self.dv)), "float32")

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        T = x.shape[0]
        proj = linear(x, self.w_proj)
        gates = torch.empty((T, 2 * self.heads), dtype=torch.float32, device=x.device)
        ops.mlstm_gates(x, self.w_gates, self.gate_bias, gates, self.heads, self.spec.gate_cap)
        o_raw = torch.empty((T, self.v_size), dtype=torch.float32, device=x.device)
        ops.mlstm_scan(proj, gates, view.state, ctx.q_start, ctx.state_slots, o_raw, ctx.B,
                       self.heads, self.dk, self.dv, self.dk ** -0.5, ctx.err)
        out = torch.empty((T, self.v_size), dtype=x.dtype, device=x.device)
        ops.mlstm_out(o_raw, proj, 2 * self.qk_size + self.v_size, self.norm_w, out, self.heads,
                      self.dv, self.spec.norm_eps)
        return linear(out, self.w_o)


register_mixer("mlstm", MLSTMMixer)
