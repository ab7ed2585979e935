"""A plain, slow Gukidra decoder: whole sequences, no cache, one function per mechanism.

The tests' oracle for the hybrid design.  It shares no code with ``binfer_b200``: it
reads the raw config.json dictionary and a name -> tensor dictionary itself and runs on
the CPU with ordinary tensor arithmetic, token by token where the design is a recurrence.

The design in this file's notation (``D`` width, ``t`` a position counted from 0):

* embedding: ``x_t = E[token_t] * embedding.scale``;
* a layer: ``x += N1(mixer(x))`` and, if it has a feed-forward, ``x += N2(ff(x))``; both
  sublayers read the stream itself, the norm sits on their output;
* ``N(y) = y / sqrt(mean(y^2) + eps) * (1 + w)``;
* mixers ``mlstm`` (a matrix memory with exponential gates, stabilised by a running maximum)
  and ``attention`` (windowed, grouped, with mean-pooled blocks of older keys, a unit sink,
  rotated values and a gate per head), see the functions below;
* output: ``N_final(x) E^T`` (the table without the embedding's scale).

``dtype`` is the working precision (float64 gives an oracle whose own rounding is
negligible).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------- small parts
def unit_offset_rms_norm(y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``y / sqrt(mean(y^2) + eps) * (1 + w)`` over the last axis."""
    ms = (y * y).mean(dim=-1, keepdim=True)
    return y / torch.sqrt(ms + eps) * (1.0 + w)


def plain_rms_norm(y: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """``y / sqrt(mean(y^2) + eps)``, times ``w`` if there is one (the weight as stored)."""
    ms = (y * y).mean(dim=-1, keepdim=True)
    out = y / torch.sqrt(ms + eps)
    return out if w is None else out * w


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int,
                 interleaved: bool = False, sign: float = 1.0) -> torch.Tensor:
    """Turn pair ``m`` of the first ``dims`` entries of the last axis by
    ``sign * pos * base^(-2m/dims)``.  Pairs are ``(m, m + dims/2)``, or ``(2m, 2m+1)`` when
    ``interleaved``.  ``x`` is ``[T, ..., d]`` and ``pos`` ``[T]``."""
    half = dims // 2
    m = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(base, dtype=torch.float64) ** (-2.0 * m / dims)
    ang = sign * pos.to(torch.float64)[:, None] * freq[None, :]            # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).to(x.dtype).view(shape), torch.sin(ang).to(x.dtype).view(shape)
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# ------------------------------------------------------------------------------ mixers
def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: dict, eps: float
                ) -> torch.Tensor:
    """The matrix memory, one token after the other.  Per head, with ``S`` ``[dim, vdim]``,
    ``n`` ``[dim]`` and ``m`` all starting at zero::

        i = cap tanh((W_i h + b_i) / cap)         f = logsigmoid(cap tanh((W_f h + b_f) / cap))
        m' = max(f + m, i)
        S' = exp(f + m - m') S + exp(i - m') k v^T         n' likewise with k
        o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)     q = W_q h / sqrt(dim)

    then each head's ``o`` over its root mean square, all heads times the weight ``norm``,
    times ``sigmoid(W_g h)``, and the output projection."""
    T = h.shape[0]
    H, dk, dv, cap = cfg["heads"], cfg["dim"], cfg["vdim"], float(cfg["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    ig = capped(h @ w[p + "i"].T + w[p + "i.b"], cap)                       # [T, H]
    fg = F.logsigmoid(capped(h @ w[p + "f"].T + w[p + "f.b"], cap))
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    n = torch.zeros(H, dk, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)
    outs = []
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a = torch.exp(fg[t] + m - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        outs.append(num / den[:, None])
    o = torch.stack(outs)                                                   # [T, H, dv]
    o = plain_rms_norm(o, None, eps).reshape(T, H * dv) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def visible(i: int, window: Optional[int], pool: int):
    """What a query at position ``i`` sees: ``(blocks, first)``: the pooled blocks
    ``0 .. blocks-1`` and the tokens ``first .. i``."""
    if window is None:
        return 0, 0
    first = max(0, i - window + 1)
    blocks = 0 if pool <= 0 else max(0, (i - window + 1) // pool)
    return blocks, first


def attention_keys_values(h, w, p, cfg, eps):
    """Keys after head norm and rotation, values after their rotation, as a cache holds them:
    ``[T, G, dim]`` and ``[T, G, vdim]``."""
    T = h.shape[0]
    G, dk, dv = cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    rot = cfg.get("rot")
    pos = torch.arange(T)
    k = plain_rms_norm((h @ w[p + "k"].T).view(T, G, dk), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    if rot:
        il = rot.get("layout", "half") == "interleaved"
        k = rotate_pairs(k, pos, rot["base"], rot["dims"], il)
        v = rotate_pairs(v, pos, rot["base"], dv, il)
    return k, v


def attention_mixer(h, w, p, cfg, eps, k, v):
    """Windowed grouped attention over ``k``/``v`` (this layer's or another's)."""
    T = h.shape[0]
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    rot, mask = cfg.get("rot"), cfg.get("mask") or {}
    window, pool = mask.get("size"), int(mask.get("pool") or 0)
    pos = torch.arange(T)
    q = plain_rms_norm((h @ w[p + "q"].T).view(T, H, dk), w[p + "q.norm"], eps)
    il = bool(rot) and rot.get("layout", "half") == "interleaved"
    if rot:
        q = rotate_pairs(q, pos, rot["base"], rot["dims"], il)
    gate = torch.sigmoid(h @ w[p + "g"].T)                                  # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        blocks, first = visible(i, window, pool)
        ks = [k[b * pool:(b + 1) * pool].mean(0) for b in range(blocks)] + list(k[first:i + 1])
        vs = [v[b * pool:(b + 1) * pool].mean(0) for b in range(blocks)] + list(v[first:i + 1])
        K, V = torch.stack(ks), torch.stack(vs)                             # [n, G, d]
        for hh in range(H):
            g = hh // (H // G)
            s = (K[:, g] @ q[i, hh]) * cfg["scale"]
            mx = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - mx)
            pr = e / (torch.exp(-mx) + e.sum())            # one more in the denominator
            out[i, hh] = pr @ V[:, g]
    if rot:
        out = rotate_pairs(out, pos, rot["base"], dv, il, sign=-1.0)
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h, w, p):
    return (F.silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ------------------------------------------------------------------------------- model
def forward(raw: dict, w: Dict[str, torch.Tensor], tokens: List[int],
            dtype: torch.dtype = torch.float64, layers_out: Optional[list] = None
            ) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence.  ``layers_out``: a list that receives the
    residual stream after every layer."""
    w = {n: (t.to(dtype) if t.dtype.is_floating_point else t) for n, t in w.items()}
    eps = float(raw["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(raw["embedding"]["scale"])
    kv = {}
    for i, layer in enumerate(raw["layers"]):
        p, cfg = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "mlstm":
            y = mlstm_mixer(x, w, p, cfg, eps)
        elif layer["type"] == "attention":
            src = cfg.get("kv_from")
            if src is None:
                kv[i] = attention_keys_values(x, w, p, cfg, eps)
                src = i
            y = attention_mixer(x, w, p, cfg, eps, *kv[src])
        else:
            raise ValueError(layer["type"])
        x = x + unit_offset_rms_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + unit_offset_rms_norm(dense_ff(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return unit_offset_rms_norm(x, w["final.norm"], eps) @ w["embed"].T


def greedy_generate(raw: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int,
                    dtype: torch.dtype = torch.float64) -> List[int]:
    """``n`` tokens after ``prompt``, each the largest logit's (the lowest id on a tie); the
    whole sequence is run again for every token."""
    toks, out = list(prompt), []
    for _ in range(n):
        row = forward(raw, w, toks, dtype)[-1]
        out.append(int(torch.argmax(row)))
        toks.append(out[-1])
    return out
