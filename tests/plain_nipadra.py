"""A plain, slow implementation of the Nipadra design: whole sequences, no cache, no batching, one
function per mechanism, on the CPU. It is the oracle of the Nipadra tests and shares no code with
the engine (its own reading of config.json, its own loops).

Notation. h: the input of a sublayer [T, width]. A layer is ``x <- N1(alpha x + mixer(x))`` and,
when it has a feed-forward, ``x <- N2(alpha x + ff(x))`` with N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).
Every function takes ``dt``, the torch dtype it computes in (float32, or float64 for an oracle
with no rounding of its own), and ``rnd``, applied where a bfloat16 engine stores an operand of a
matrix product in 16 bits.
"""
from __future__ import annotations

import json
import math
from typing import Dict, Optional, Sequence

import torch

import plain_model as pm


def ident(t):
    return t


def bf16(t):
    return t.to(torch.bfloat16).to(t.dtype)


def load(model_dir: str):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return pm.read_safetensors_f32(f"{model_dir}/model.safetensors"), cfg


# ------------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layer and model norm: weight stored around zero."""
    return unit_rms(x, eps) * (1.0 + w.to(x.dtype))


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w.to(x.dtype)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


ACTS = {"relu": torch.relu, "silu": silu, "gelu_tanh": gelu_tanh}


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ------------------------------------------------------------------------------------ lightning
def lightning_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, dt=torch.float32, rnd=ident):
    """Three activated projections feed a fading outer-product memory per head (S <- decay * S + k (x) v, read out
    as S^T q); all heads' read-outs are normed as one vector, weighted, gated by a fourth projection's sigmoid."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    hb = rnd(h)
    q = rnd(silu(hb @ w[p + "q"].to(dt).T)).reshape(T, H, dk)
    k = rnd(silu(hb @ w[p + "k"].to(dt).T)).reshape(T, H, dk)
    v = rnd(silu(hb @ w[p + "v"].to(dt).T)).reshape(T, H, dv)
    g = hb @ w[p + "g"].to(dt).T
    o = torch.zeros(T, H, dv, dtype=dt)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=dt)
        a = float(m["decay"][hd])
        for t in range(T):
            S = a * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    y = norm_plain(o.reshape(T, H * dv), w[p + "norm"], eps) * torch.sigmoid(g)
    return rnd(y) @ w[p + "o"].to(dt).T


# ------------------------------------------------------------------------------------ windowed attention
def rotate_interleaved(v, positions, base: float, dims: int):
    """Pairs (2i, 2i+1) of the first ``dims`` dimensions turned by the angle p * base^(-2i/dims)."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(v.dtype)
    ang = torch.tensor(list(positions), dtype=v.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def sink_window_attention(q, k, v, scale: float, window: int, rnd=ident):
    """Query i looks back over at most ``window`` keys, itself included; the weights' denominator carries an extra 1
    (a phantom key of score 0 that contributes no value). q [T, H, d]; k, v [T, G, d]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale
            mx = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - mx)
            out[i, hd] = (rnd(e) @ v[lo:i + 1, g]) / (torch.exp(-mx) + e.sum())
    return out


def left_mixer(h, w, p: str, m: dict, eps: float, dt=torch.float32, rnd=ident):
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    hb = rnd(h)
    q = (hb @ w[p + "q"].to(dt).T).reshape(T, H, d)
    k = (hb @ w[p + "k"].to(dt).T).reshape(T, G, d)
    v = rnd(k)                                             # values: the key projection's raw output
    q = norm_plain(q, w[p + "q.norm"], eps)
    kn = norm_plain(k, w[p + "k.norm"], eps)
    pos = range(T)
    q = rnd(rotate_interleaved(q, pos, m["rot"]["base"], m["rot"]["dims"]))
    kn = rnd(rotate_interleaved(kn, pos, m["rot"]["base"], m["rot"]["dims"]))
    att = sink_window_attention(q, kn, v, float(m["scale"]), int(m["mask"]["size"]), rnd)
    gate = torch.sigmoid(hb @ w[p + "g"].to(dt).T)         # [T, H]
    att = att * gate[:, :, None]
    return att.reshape(T, -1)


# ------------------------------------------------------------------------------------ state-space side
def causal_conv(u, weight, bias):
    """Depthwise filter over time. u [T, C]; weight [C, taps] with column taps-1 on the newest token; the sequence is
    padded with zeros on the left."""
    T, C = u.shape
    taps = weight.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u])
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + pad[j:j + T] * weight[:, j].to(u.dtype)[None, :]
    return out + bias.to(u.dtype)[None, :]


def right_mixer(h, w, p: str, m: dict, eps: float, dt=torch.float32, rnd=ident):
    T = h.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    hb = rnd(h)
    proj = hb @ w[p + "in"].to(dt).T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    step = proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    xs = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    step = softplus(step + w[p + "dt_bias"].to(dt)[None, :])
    A = -torch.exp(w[p + "A_log"].to(dt))
    D = w[p + "D"].to(dt)
    y = torch.zeros(T, Hh, P, dtype=dt)
    for hd in range(Hh):
        g = hd // (Hh // G)
        S = torch.zeros(N, P, dtype=dt)
        for t in range(T):
            S = torch.exp(A[hd] * step[t, hd]) * S + step[t, hd] * torch.outer(B[t, g], xs[t, hd])
            y[t, hd] = S.T @ C[t, g] + D[hd] * xs[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"].to(dt)
    return y


def parallel_mixer(h, w, p: str, m: dict, eps: float, dt=torch.float32, rnd=ident):
    left = rnd(left_mixer(h, w, p + "left.", m["left"], eps, dt, rnd)) @ w[p + "left.o"].to(dt).T
    right = rnd(right_mixer(h, w, p + "right.", m["right"], eps, dt, rnd)) @ w[p + "right.o"].to(dt).T
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ------------------------------------------------------------------------------------ feed-forward, model
def dense_ff(h, w, p: str, mlp: dict, dt=torch.float32, rnd=ident):
    act = ACTS[mlp.get("act", "relu")]
    hb = rnd(h)
    return rnd(act(hb @ w[p + "gate"].to(dt).T) * (hb @ w[p + "up"].to(dt).T)) @ w[p + "down"].to(dt).T


MIXERS = {"lightning": lightning_mixer, "parallel": parallel_mixer}


def forward(w, cfg, tokens: Sequence[int], dt=torch.float32, rnd=ident, positions: Optional[Sequence[int]] = None,
            layers_out: Optional[list] = None):
    """Logits [T, vocab] (or at ``positions``); ``layers_out`` collects the stream after every layer."""
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    emb = w["embed"].to(dt)
    x = emb[torch.tensor(list(tokens), dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](x, w, p + "mix.", layer["mixer"], eps, dt, rnd)
        x = norm_one_plus(alpha * x + y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = dense_ff(x, w, p + "mlp.", layer["mlp"], dt, rnd)
            x = norm_one_plus(alpha * x + y, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    if positions is not None:
        x = x[torch.tensor(list(positions), dtype=torch.long)]
    return rnd(norm_one_plus(x, w["final.norm"], eps)) @ emb.T
