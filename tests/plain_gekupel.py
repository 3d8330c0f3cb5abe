"""A plain, slow implementation of the Gekupel design: one function per mechanism, whole sequences at once,
no cache, no batching, torch on the CPU in float64 (angles of the rotation in 32-bit, as the design computes them).

It takes the configuration as the dictionary that config.json holds and the weights by their checkpoint names,
and shares no code with the engine. Notation: h is a sublayer's input [n, width], n tokens at positions 0..n-1.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def ident(x: torch.Tensor) -> torch.Tensor:
    return x


def bf16(x: torch.Tensor) -> torch.Tensor:
    """Rounds to bfloat16 and back: what an engine that keeps the operands of its matrix products and its cache in
    bfloat16 does to them (the functions below take it as ``rnd`` and apply it at those places)."""
    return x.to(torch.bfloat16).to(F)


# ---------------------------------------------------------------------------------------------- small pieces
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------------------------- rotation
def rotation_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[torch.Tensor, float]:
    """(frequency of each pair [dims / 2], factor on cos and sin). Without scaling f_i = base^(-2i/dims) and 1.
    With the long-context scaling {factor, original, fast, slow}: pairs that turn more than ``fast`` times within
    ``original`` positions keep f_i, pairs that turn fewer than ``slow`` times get f_i / factor, a linear ramp over
    the pair index between; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, amplitude: float) -> torch.Tensor:
    """Rotates the first 2 * len(freq) values of the last dimension of x [n, ..., d]: (x[2i], x[2i+1]) turn by the
    angle position * freq[i] (taken in 32-bit); the rest passes."""
    n, r = x.shape[0], 2 * freq.numel()
    angle = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(F)       # [n, r/2]
    shape = [n] + [1] * (x.dim() - 2) + [r // 2]
    c, s = (torch.cos(angle) * amplitude).view(shape), (torch.sin(angle) * amplitude).view(shape)
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out = x.clone()
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


# ---------------------------------------------------------------------------------------------- who sees whom
def window_mask(positions: torch.Tensor, size: int) -> torch.Tensor:
    """[n, n] True where query i sees key j: 0 <= i - j < size."""
    d = positions[:, None] - positions[None, :]
    return (d >= 0) & (d < size)


def chunk_mask(positions: torch.Tensor, size: int) -> torch.Tensor:
    """[n, n] True where j <= i and both lie in the same block of ``size`` positions counted from 0."""
    i, j = positions[:, None], positions[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def softmax_rows(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """Softmax over the visible keys of scores [H, n, n]; with ``sink`` [H] the denominator holds exp(sink_h) too."""
    scores = scores.masked_fill(~mask[None], -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.view(-1, 1, 1))
    e = torch.exp(scores - top)
    total = e.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink.view(-1, 1, 1) - top)
    return e / total


# ---------------------------------------------------------------------------------------------- mixers
def attention_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], eps: float, positions: torch.Tensor, rnd=ident) -> torch.Tensor:
    """Grouped-query attention without rotation: queries and keys brought to unit RMS per head, a bias that grows
    with the distance, blocks of positions that do not see each other, a sink per head."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = rnd(h)
    q = rnd(unit_rms((h @ w["q"].T).view(n, H, d), eps))
    k = rnd(unit_rms((h @ w["k"].T).view(n, G, d), eps))
    v = rnd((h @ w["v"].T).view(n, G, dv))
    per = H // G
    k = k.repeat_interleave(per, dim=1)
    v = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    slope = torch.tensor([2.0 ** (-8.0 * (x + 1) / H) for x in range(H)], dtype=F)
    scores = scores - slope.view(H, 1, 1) * (positions[:, None] - positions[None, :]).to(F)[None]
    p = softmax_rows(scores, chunk_mask(positions, m["mask"]["size"]), w["sink"])
    out = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    return rnd(out) @ w["o"].T


def latent_attention_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], eps: float, positions: torch.Tensor,
                           second: bool, rnd=ident) -> torch.Tensor:
    """Attention whose queries, keys and values are made from low-rank latents; one rotated key part is shared by
    the heads; a sliding window; the second kind scales the rotation for long contexts and has one more term in the
    softmax's denominator."""
    n = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    freq, amp = rotation_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"]["scaling"] if second else None)
    h = rnd(h)
    cq = rnd(rms_norm(h @ w["dq"].T, w["dq.norm"], eps))
    q = (cq @ w["uq"].T).view(n, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], positions, freq, amp)
    ckv = h @ w["dkv"].T
    c = rnd(rms_norm(ckv[:, :rank], w["dkv.norm"], eps))
    k_rot = rnd(rotate_pairs(ckv[:, rank:], positions, freq, amp))               # [n, r], one for all heads
    k_plain = (c @ w["uk"].T).view(n, H, d)
    v = (c @ w["uv"].T).view(n, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    p = softmax_rows(scores, window_mask(positions, m["mask"]["size"]), w["sink"] if second else None)
    out = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    return rnd(out) @ w["o"].T


# ---------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], rnd=ident) -> torch.Tensor:
    h = rnd(h)
    return rnd(gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [n, top], their weights [n, top]): the experts with the largest sigmoid(router h) + correction;
    the weights are the sigmoids themselves, not renormalised."""
    s = torch.sigmoid(h @ router.T)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def moe_ff(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], rnd=ident) -> torch.Tensor:
    h = rnd(h)
    chosen, weight = route(h, w["router"], w["correction"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            x = h[t]
            y = (silu(w[f"e{e}.gate"] @ x) * (w[f"e{e}.up"] @ x))
            out[t] += g * (w[f"e{e}.down"] @ y)
    return out


# ---------------------------------------------------------------------------------------------- the model
def _sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], rnd=ident) -> Tuple[torch.Tensor, torch.Tensor]:
    """(logits [n, vocab], the residual stream after every layer run [runs, n, width])."""
    eps = config["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = weights["embed"].to(F)[torch.tensor(tokens)] * config["embedding"]["scale"]
    after = []
    for i, layer in enumerate(config["layers"]):
        owner = layer.get("weights_of", i)
        w = _sub(weights, f"l{owner}.")
        mix = _sub(w, "mix.")
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = attention_mixer(x, m, mix, eps, positions, rnd)
        elif kind in ("latent_attention", "latent_attention_2"):
            y = latent_attention_mixer(x, m, mix, eps, positions, kind == "latent_attention_2", rnd)
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, w["norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = _sub(w, "mlp.")
            y = dense_ff(x, ff, rnd) if mlp["kind"] == "dense" else moe_ff(x, mlp, ff, rnd)
            x = x + rms_norm(y, w["norm2"], eps)
        after.append(x)
    logits = rnd(rms_norm(x, weights["final.norm"].to(F), eps)) @ weights["head"].to(F).T
    return logits, torch.stack(after)


def load(folder: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """(config.json as a dictionary, the tensors of model.safetensors by name), read with a reader of its own."""
    import json
    import os
    import struct
    import numpy as np
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        if e["dtype"] == "BF16":
            bits = np.frombuffer(data[a:b], dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        else:
            t = torch.from_numpy(np.frombuffer(data[a:b], dtype="<f4").copy())
        out[name] = t.view(e["shape"])
    return config, out
