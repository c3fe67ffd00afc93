"""Plain, slow implementation of the Sukisun decoder, used only as the oracle of the tests.

Whole sequences, no cache, one function per mechanism, float64 tensor arithmetic on the CPU.  It
shares no code with the `beglin_b200` package: the model folder is read with the `json` module and
the `safetensors` library, and everything is computed position by position or with plain matrix
products, so that a fault of the engine's loader, cache, state slots, batching or kernels cannot be
mirrored here.

The design in this file's notation.  A layer maps the stream x to x + M(LN(x)) and then, when it has a
feed-forward, to x + F(LN(x)); after layer i the stream that goes on is a weighted sum of the embedding
output and of all layer results so far.  M is either attention through a low-rank latent with an output
gate, or a Mamba-2 recurrence.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def read_folder(folder: str, dtype: torch.dtype = torch.float64):
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


# ----------------------------------------------------------------------------- small functions
def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Mean taken off, divided by the root of (variance + eps), times w; no bias."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """A parabola through the origin above zero, a scaled exponential below; both branches have slope 1/2 at 0."""
    ap = softplus(p)
    an = 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [T, ..., n]: the first `dims` features are rotated in neighbouring pairs (2i, 2i+1) by the angle
    position * base^(-2i/dims); the rest pass unchanged."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]                # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape).to(v.dtype), torch.sin(ang).reshape(shape).to(v.dtype)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- feed-forward
def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    act = w[p + "mlp.act"]
    return xielu(h @ w[p + "mlp.up"].t(), act[0], act[1]) @ w[p + "mlp.down"].t()


# ----------------------------------------------------------------------------- attention through a latent
def latent_of(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """What a layer with a down-projection of its own leaves for the keys and values: the normed latent
    [T, kv_rank] and the one rotated key part [T, rot_dim] that all heads share."""
    T = h.shape[0]
    kv_rank, rot = m["kv_rank"], m["rot_dim"]
    dkv = h @ w[p + "mix.dkv"].t()
    c = rms_unit(dkv[:, :kv_rank], eps) * w[p + "mix.dkv.norm"]
    kr = rotate_pairs(dkv[:, kv_rank:kv_rank + rot], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, c: torch.Tensor,
                     kr: torch.Tensor) -> torch.Tensor:
    """h [T, width] of ONE sequence from its position 0; c, kr as `latent_of` returns them (this layer's
    or another's).  Position by position, head by head."""
    T = h.shape[0]
    H, dim, rot, vd, kv_rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_unit(h @ w[p + "mix.dq"].t(), eps) * w[p + "mix.dq.norm"]
    q = (cq @ w[p + "mix.uq"].t()).reshape(T, H, dim + rot)
    q_plain = q[..., :dim]
    q_rot = rotate_pairs(q[..., dim:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "mix.uk"].t()).reshape(T, H, dim)
    v = (c @ w[p + "mix.uv"].t()).reshape(T, H, vd)
    gate = torch.sigmoid(h @ w[p + "mix.g"].t())                                # [T, H]
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            s = (k_plain[:t + 1, hh] @ q_plain[t, hh] + kr[:t + 1] @ q_rot[t, hh]) * m["scale"]
            pr = torch.softmax(s, dim=0)
            out[t, hh] = (pr[:, None] * v[:t + 1, hh]).sum(0) * gate[t, hh]
    return out.reshape(T, H * vd) @ w[p + "mix.o"].t()


# ----------------------------------------------------------------------------- Mamba-2
def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """h [T, width] of ONE sequence from its position 0, with S = 0 before the first token."""
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = h @ w[p + "mix.in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    # causal convolution per channel: tap j multiplies the input taps-1-j tokens back; nothing precedes token 0
    cw, cb = w[p + "mix.conv"], w[p + "mix.conv.b"]
    conv = torch.zeros_like(xbc)
    for t in range(T):
        acc = cb.clone()
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                acc = acc + cw[:, j] * xbc[src]
        conv[t] = acc
    conv = silu(conv)
    x = conv[:, :inner].reshape(T, H, P)
    B = conv[:, inner:inner + G * N].reshape(T, G, N)
    C = conv[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "mix.dt_bias"])                                    # [T, H]
    a = torch.exp(w[p + "mix.A_log"])                                           # [H]
    D = w[p + "mix.D"]
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    per_group = H // G
    for t in range(T):
        for hh in range(H):
            g = hh // per_group
            S[hh] = torch.exp(-a[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].t() @ C[t, g] + D[hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_unit(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * w[p + "mix.norm"]
    return y @ w[p + "mix.o"].t()


# ----------------------------------------------------------------------------- the whole model
def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], return_layers: bool = False):
    """float64 logits [T, vocab] of one sequence; with `return_layers` also the stream after every layer."""
    eps = cfg["norm"]["eps"]
    ids_t = torch.tensor(list(ids), dtype=torch.long)
    x = w["embed"][ids_t] * cfg["embedding"]["scale"]
    history: List[torch.Tensor] = [x]
    latents = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, p, m, eps)
                src = i
            x = x + latent_attention(h, w, p, m, eps, *latents[src])
        elif layer["type"] == "mamba2":
            x = x + mamba2(h, w, p, m, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            x = x + dense_feed_forward(layer_norm(x, w[p + "norm2"], eps), w, p)
        history.append(x)
        mix = w[p + "dwa"]
        x = sum(mix[j] * history[j] for j in range(i + 2))
        streams.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["embed"].t()
    if return_layers:
        return logits, torch.stack(streams)
    return logits
