"""Plain, slow implementation of the Nadilorn decoder, used only as the oracle of the tests.

Whole sequences, no cache, one function per mechanism, float64 tensor arithmetic on the CPU.  It shares no code
with the `beglin_b200` package: the model folder is read with the `json` module and the `safetensors` library,
and attention is computed query by query over explicit lists of visible keys, so that a fault of the engine's
loader, cache, batching or kernels cannot be mirrored here.

The design in this file's notation.  The stream x of a token passes layers of two sublayers each.  A sublayer S
reads x as it is and its result is normed before it is added: x <- x + N(S(x)), with N an RMS norm with a weight.
The first sublayer is attention; the second, which a layer may lack, is a gated feed-forward or a sum over routed
experts.  Attention: queries, keys and values are products of x; the whole query row and the whole key row are
RMS-normed (over all heads at once) with weights; the leading features of every head are turned by position;
a query sees itself and the w - 1 positions before it; the softmax has a denominator enlarged by one (a key of
score nought that carries no value); the joined heads are multiplied by sigmoid of another product of x before the
output product.
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
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def turn_halves(v: torch.Tensor, positions: Sequence[int], base: float, dims: int, divisor: float) -> torch.Tensor:
    """v [T, heads, n]: of every head the first `dims` features turn, feature i together with feature i + dims/2, by
    the angle position * base^(-2i/dims) / divisor; the rest pass unchanged."""
    out = v.clone()
    half = dims // 2
    pos = torch.tensor(list(positions), dtype=torch.float64)
    for i in range(half):
        a = pos * (base ** (-2.0 * i / dims)) / divisor
        c, s = torch.cos(a)[:, None].to(v.dtype), torch.sin(a)[:, None].to(v.dtype)
        lo, hi = v[:, :, i], v[:, :, i + half]
        out[:, :, i] = lo * c - hi * s
        out[:, :, i + half] = hi * c + lo * s
    return out


def sink_softmax(scores: torch.Tensor) -> torch.Tensor:
    """exp(s_j) / (1 + sum_j exp(s_j)): the weights add up to less than one."""
    m = max(float(scores.max()), 0.0)
    e = torch.exp(scores - m)
    return e / (math.exp(-m) + e.sum())


# ----------------------------------------------------------------------------- mixer
def attention(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, m: dict, eps: float,
              positions: Optional[Sequence[int]] = None) -> torch.Tensor:
    """h [T, width] -> [T, width].  `p` is the prefix of the mixer's tensors ("l3.mix.")."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T)) if positions is None else list(positions)
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(T, H, dim)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(T, G, dim)
    v = (h @ w[p + "v"].T).reshape(T, G, vdim)
    rot = m.get("rot")
    if rot and rot.get("dims", 0) > 0:
        divisor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = turn_halves(q, positions, float(rot["base"]), int(rot["dims"]), divisor)
        k = turn_halves(k, positions, float(rot["base"]), int(rot["dims"]), divisor)
    window = (m.get("mask") or {}).get("size")
    per = H // G
    joined = torch.zeros(T, H * vdim, dtype=h.dtype)
    for t in range(T):
        first = 0 if window is None else max(0, t - window + 1)
        seen = list(range(first, t + 1))
        for head in range(H):
            g = head // per
            scores = (k[seen, g] @ q[t, head]) * m["scale"]
            weights = sink_softmax(scores)
            joined[t, head * vdim:(head + 1) * vdim] = (weights[:, None] * v[seen, g]).sum(0)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (joined * gate) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def gated_feed_forward(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_experts(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, experts: int, top: int) -> torch.Tensor:
    """Every token goes to the `top` experts of largest sigmoid(router logit); its input to an expert is scaled by that
    score as it is (the scores of the chosen are not made to add up to one), and the experts' results are added."""
    out = torch.zeros_like(h)
    scores = torch.sigmoid(h @ w[p + "router"].T)                       # [T, experts]
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(scores[t, e]), e))
        for e in order[:top]:
            z = (scores[t, e] * h[t]) @ w[f"{p}e{e}.up"].T
            out[t] += relu_squared(z) @ w[f"{p}e{e}.down"].T
    return out


def feed_forward(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_feed_forward(w, p, h)
    if mlp["kind"] == "moe":
        return routed_experts(w, p, h, int(mlp["router"]["experts"]), int(mlp["router"]["top"]))
    raise ValueError(mlp["kind"])


# ----------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], taps: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  `taps`, when a list, receives the stream behind every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][list(ids)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        x = x + rms_norm(attention(w, p + "mix.", x, layer["mixer"], eps), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(w, p + "mlp.", x, layer["mlp"]), w[p + "norm2"], eps)
        if taps is not None:
            taps.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
