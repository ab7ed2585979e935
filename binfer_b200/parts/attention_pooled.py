"""Windowed grouped-query attention with pooled blocks behind the window, as a mixer part.

A query at position p sees the tokens ``p - window < j <= p`` of its request and one mean
key and value per block of ``pool`` tokens that lies wholly before the window.  Tokens live
in the mixer's paged cache, the blocks' means in a *summary* cache with one entry per block
(``KVNeed.pools``), which the step that completes a block fills.  Order of operations:
one product for q, (k, v) and the heads' gates; per-head RMSNorm and rotation of q and k,
rotation of v by its own position, k and v into the pages; means of completed blocks; the
attention (one softmax over tokens and blocks, a constant sink in its denominator), whose
output is turned back by the query's position and multiplied by the head's gate; the output
projection.  A layer that reads another layer's cache projects only q and the gates.

Every key, also those of the step's own tokens, is read from the pages, so a prompt can
be cut anywhere and portions can share a step with decoded tokens.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

from ..cache.manager import KVNeed
from ..config.specs import PooledWindowAttentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, build_position, register_mixer
from .linear import linear


# BINFER_B200_PWA_TENSOR_CORES=0: the one-warp-per-row kernel also in bfloat16 (the float32
# engine always runs it: its sums have one fixed order per position)
TENSOR_CORES = os.environ.get("BINFER_B200_PWA_TENSOR_CORES", "1") != "0"


class PooledWindowAttention(Mixer):
    def __init__(self, spec: PooledWindowAttentionSpec, hidden_size: int, prefix: str,
                 env: BuildEnv):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.value_dim > 256 or spec.value_dim % 2:
            raise ValueError(f"value_dim {spec.value_dim} is not supported (even, at most 256)")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.H, self.G, self.dk, self.dv = (spec.num_heads, spec.num_kv_heads, spec.head_dim,
                                            spec.value_dim)
        self.q_size, self.k_size, self.v_size = self.H * self.dk, self.G * self.dk, self.G * self.dv
        self.pool = spec.pool if spec.window is not None else 0
        self.position = (build_position(spec.position, self.dk, env)
                         if spec.position is not None else None)
        self.value_position = (build_position(spec.value_rotation, self.dv, env)
                               if spec.value_rotation is not None else None)
        for pos in (self.position, self.value_position):
            if pos is not None and pos.inv_freq is None:
                raise ValueError("pooled window attention takes rotary encodings only")
        self.names = dict(spec.names)
        self.w_proj = self.w_o = self.q_norm = self.k_norm = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        n = self.prefix + self.names[role]
        shape = {"q": (self.q_size, self.hidden), "k": (self.k_size, self.hidden),
                 "v": (self.v_size, self.hidden), "g": (self.H, self.hidden),
                 "o": (self.hidden, self.H * self.dv), "q_norm": (self.dk,),
                 "k_norm": (self.dk,)}[role]
        if role in ("q_norm", "k_norm"):
            return ParamSpec(n, shape, init="norm", role="vector")
        return ParamSpec(n, shape)

    def _roles(self) -> List[str]:
        s = self.spec
        roles = ["q"] + (["k", "v"] if s.own_cache else []) + (["g"] if s.head_gate else []) + ["o"]
        if s.qk_norm:
            roles += ["q_norm"] + (["k_norm"] if s.own_cache else [])
        return roles

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in self._roles()]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        s = self.spec
        g = lambda role: get(self._spec(role))          # noqa: E731
        rows = [g("q")] + ([g("k"), g("v")] if s.own_cache else []) + \
            ([g("g")] if s.head_gate else [])
        self.w_proj = torch.cat(rows, dim=0).contiguous()
        self.gate_off = self.q_size + (self.k_size + self.v_size if s.own_cache else 0)
        self.w_o = g("o")
        if s.qk_norm:
            self.q_norm = g("q_norm")
            self.k_norm = g("k_norm") if s.own_cache else None

    # ------------------------------------------------------------------- cache
    def kv_need(self) -> Optional[KVNeed]:
        s = self.spec
        return KVNeed(self.G, self.dk, s.window, None if self.dv == self.dk else self.dv,
                      (self.pool,) if self.pool else ())

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        s, T = self.spec, x.shape[0]
        if view.writes_cache != s.own_cache:
            raise ValueError("a layer with key and value tensors keeps a cache of its own, "
                             "one without reads another's")
        proj = linear(x, self.w_proj)
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=x.device)
        inv = self.position.inv_freq if self.position is not None else None
        v_inv = self.value_position.inv_freq if self.value_position is not None else None
        g = view.group
        writes = view.writes_cache
        ops.apw_encode(proj, self.q_norm, self.k_norm, inv, v_inv, s.interleaved, ctx.positions,
                       ctx.slots[g] if writes else None, q, view.k_cache if writes else None,
                       view.v_cache if writes else None, self.H, self.G, self.dk, self.dv,
                       s.qk_norm_eps, ctx.err)
        if writes:
            for P, (ks, vs, sg) in view.summaries.items():
                n_new = self._new_blocks(ctx, P)
                if n_new:
                    ops.apw_pool_blocks(view.k_cache, view.v_cache, ks, vs, ctx.q_start,
                                        ctx.ctx_lens, ctx.block_tables[g], ctx.block_tables[sg],
                                        ctx.B, n_new, self.G, self.dk, self.dv, P, ctx.err)
        ks = vs = s_tables = None
        if self.pool:
            ks, vs, sg = view.summaries[self.pool]
            s_tables = ctx.block_tables[sg]
        gate = proj[:, self.gate_off:self.gate_off + self.H] if s.head_gate else None
        out = torch.empty((T, self.H * self.dv), dtype=x.dtype, device=x.device)
        if (TENSOR_CORES and s.softmax_scale > 0
                and ops.pwm_attention_takes(x.dtype, self.H, self.G, self.dk, self.dv)):
            # bfloat16: tiles of (token, head of a group) rows on the tensor cores, prompt
            # portions and single tokens alike
            ops.pwm_attention(q, view.k_cache, view.v_cache, ks, vs, ctx.q_start, ctx.positions,
                              ctx.block_tables[g], s_tables, gate, v_inv, s.interleaved, out,
                              ctx.B, 1 if ctx.decode_only else ctx.max_q_len, self.H, self.G,
                              self.dk, self.dv, s.window, self.pool, s.softmax_scale, s.sink,
                              ctx.err, max_ctx=ctx.max_ctx_len)
            return linear(out, self.w_o)
        ops.apw_attention(q, view.k_cache, view.v_cache, ks, vs, ctx.seq_of_token, ctx.positions,
                          ctx.block_tables[g], s_tables, gate, v_inv, s.interleaved, out, self.H,
                          self.G, self.dk, self.dv, s.window, self.pool, s.softmax_scale, s.sink,
                          ctx.err)
        return linear(out, self.w_o)

    @staticmethod
    def _new_blocks(ctx: StepContext, P: int) -> int:
        """Most blocks of ``P`` tokens that this step completes for one request.  A step of
        single tokens always answers 1: its launches may be replayed from a graph."""
        if ctx.decode_only or not ctx.ctx_lens_host:
            return 1
        return max(end // P - (end - n) // P for end, n in zip(ctx.ctx_lens_host, ctx.q_lens))


register_mixer("pooled_window_attention", PooledWindowAttention)
