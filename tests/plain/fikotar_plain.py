"""A plain, slow implementation of the Fikotar design from its equations: one function per
mechanism, float64 on the CPU, every sequence walked as whole matrices (or token by token,
for the recurrence).  It shares no code with the engine; the tests hold the engine to it.

Notation: T tokens of one sequence at positions 0..T-1, h [T, width] a layer's normed input.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ----------------------------------------------------------------------- small pieces
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i/dims); with ``scaling``, by wavelength l = 2 pi / f: kept below
    original/high, divided by factor above original/low, blended between."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = []
    for fi in f.tolist():
        wave = 2 * math.pi / fi
        if wave < sc["original"] / sc["high"]:
            out.append(fi)
        elif wave > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1 - s) * fi / sc["factor"] + s * fi)
    return torch.tensor(out, dtype=F64)


def rotate(x, rot: Optional[dict]):
    """x [T, heads, d]: pairs (i, i + dims/2) of the first ``dims`` sizes turn by p f_i."""
    if not rot:
        return x
    dims, half = rot["dims"], rot["dims"] // 2
    f = rotary_frequencies(rot)
    ang = torch.arange(x.shape[0], dtype=F64)[:, None, None] * f[None, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_{t - taps + 1 + j}, zeros before 0."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    if j > i:
        return False
    if not mask or mask.get("size") is None:
        return True
    return i - j < mask["size"] or j < int(mask.get("keep_first") or 0)


# ---------------------------------------------------------------------------- mixers
def conv_window_attention(h, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, G = mx["heads"], mx.get("kv_heads") or mx["heads"]
    d, dv = mx["dim"], mx.get("vdim") or mx["dim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if int(mx.get("conv") or 0) >= 1:
        q, k, v = (causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]),
                   causal_conv(v, w[p + "v.conv"]))
    q = unit_rms(rotate(q.view(T, H, d), mx.get("rot")), eps)
    k = unit_rms(rotate(k.view(T, G, d), mx.get("rot")), eps)
    v = v.view(T, G, dv)
    scale = mx["scale"] if mx.get("scale") is not None else d ** -0.5
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        sink = w[p + "sink"][hd]
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, mx.get("mask"))]
            s = (k[js, g] @ q[i, hd]) * scale
            m = torch.maximum(s.max(), sink)
            e = torch.exp(s - m)
            den = e.sum() + torch.exp(sink - m)
            out[i, hd] = ((e / den)[:, None] * v[js, g]).sum(0)
    return out.reshape(T, H * dv) @ w[p + "o"].T


def retention(h, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, d, dv = mx["heads"], mx["dim"], mx.get("vdim") or mx["dim"]
    q = rotate((h @ w[p + "q"].T).view(T, H, d), mx.get("rot"))
    k = rotate((h @ w[p + "k"].T).view(T, H, d), mx.get("rot")) * d ** -0.5
    v = (h @ w[p + "v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = mx["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = unit_rms(o, eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side(h, w, p: str, mx: dict, eps: float):
    return (mx.get("left_scale", 1.0) * conv_window_attention(h, w, p + "left.", mx["left"], eps)
            + mx.get("right_scale", 1.0) * retention(h, w, p + "right.", mx["right"], eps))


# ---------------------------------------------------------------------- feed-forward
def gated_expert(h, w, p: str):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def chosen_experts(h, w, p: str, mlp: dict):
    """Per token: the ids of the ``top`` largest router logits and their softmax weights."""
    z = h @ w[p + "router"].T
    top = mlp["router"]["top"]
    vals, ids = torch.sort(z, dim=-1, descending=True, stable=True)
    vals, ids = vals[:, :top], ids[:, :top]
    return ids, torch.softmax(vals, dim=-1)


def mixture_of_experts(h, w, p: str, mlp: dict):
    ids, wts = chosen_experts(h, w, p, mlp)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wts[t]):
            out[t] += a * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(h, w, p + "shared.")
    return out


# ------------------------------------------------------------------------- the model
def forward(raw: dict, weights: Dict[str, torch.Tensor], tokens: List[int],
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence."""
    w = {n: t.to(F64) for n, t in weights.items()}
    eps = raw["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(raw["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        y = side_by_side(h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + mixture_of_experts(h, w, p + "mlp.", layer["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return (x @ w["head"].T) * raw.get("logit_scale", 1.0)
