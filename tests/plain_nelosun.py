"""Nelosun, plainly: one function per mechanism, loops over tokens, float64 by default.

Nothing here is shared with the package: the folder is read with a few lines of its own, the model is
a function of (configuration, weights, tokens) without cache or state, and every mechanism is
written from its equations.

The model.  ``x = embed[token] * embedding.scale``.  ``layers`` lists the layers; those from ``loop.start`` to
``loop.stop - 1`` run ``loop.times`` times in a row with the same weights, and right before the first layer
of every such pass ``x <- W_in [x; x0]`` with x0 the embedding's output.  A layer is parallel:
``h = rmsnorm(x)``, ``x <- x + ls1 * mixer(h) + ls2 * ff(h)``.  Its mixer is grouped-query attention
without rotation (biases, a query temperature that grows with the logarithm of the position, a sink of
score zero in the softmax's denominator, a sigmoid gate per head), latent attention (queries through a
normed latent, keys and values expanded from a normed latent that is all the cache has to keep, one
rotated key part shared by the heads) or a recurrent block around the real-gated linear recurrent unit.
Its feed-forward is a mixture of clamped gated experts chosen by a table over the token ids, or absent.
The model ends on an RMS norm and the embedding table as the head.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Any, Dict, List, Sequence

import torch

_DT = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32,
       "I64": torch.int64}


def read_config(folder: str) -> Dict[str, Any]:
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    """Eight bytes of length, that much json (name -> dtype, shape, data_offsets), then the data."""
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in head.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=_DT[e["dtype"]]).reshape(e["shape"])
        out[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return out


# ---- small functions ----------------------------------------------------------------------------------

def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# ---- attention with a sink of score zero ----------------------------------------------------------------

def query_temperature(p: int, coef: float, every: int) -> float:
    """What the query at position p is multiplied by."""
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sink_attention(w: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor) -> torch.Tensor:
    """h [T, width], one sequence from position 0.  Every token's softmax has one more term, exp(0), that
    carries no value."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).reshape(T, H, d)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).reshape(T, G, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).reshape(T, G, dv)
    gate = sigmoid(h @ w[pre + "g"].T)                                   # [T, H]
    qt = m.get("q_temp")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        f = query_temperature(t, float(qt["coef"]), int(qt["every"])) if qt else 1.0
        for a in range(H):
            g = a // (H // G)
            s = torch.stack([(q[t, a] * f) @ k[j, g] for j in range(t + 1)]) * m["scale"]
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[t, a] = gate[t, a] * (p[:, None] * v[: t + 1, g]).sum(0)
    return out.reshape(T, H * dv) @ w[pre + "o"].T + w[pre + "o.b"]


# ---- latent attention ---------------------------------------------------------------------------------------

def rotate_half(x: torch.Tensor, p: int, dims: int, base: float) -> torch.Tensor:
    """x [..., n]: its first ``dims`` elements turn, element i with element i + dims/2, by p * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = p * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def latent_attention(w: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    cq = rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).reshape(T, H, d + r)
    kv = h @ w[pre + "dkv"].T                                              # [T, R + r]
    c = rms_norm(kv[:, :R], w[pre + "dkv.norm"], eps)
    kr = kv[:, R:]
    kn = (c @ w[pre + "uk"].T).reshape(T, H, d)
    v = (c @ w[pre + "uv"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    krot = torch.stack([rotate_half(kr[j], j, dims, base) for j in range(T)])
    for t in range(T):
        for a in range(H):
            qn, qr = q[t, a, :d], rotate_half(q[t, a, d:], t, dims, base)
            s = torch.stack([qn @ kn[j, a] + qr @ krot[j] for j in range(t + 1)]) * m["scale"]
            p = torch.softmax(s, 0)
            out[t, a] = (p[:, None] * v[: t + 1, a]).sum(0)
    return out.reshape(T, H * dv) @ w[pre + "o"].T


# ---- the recurrent block ------------------------------------------------------------------------------------

def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, L]: the last column is the current token's; zeros before the start."""
    T, C = x.shape
    L = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        acc = bias.clone()
        for j in range(L):
            s = t - (L - 1) + j
            if s >= 0:
                acc = acc + taps[:, j] * x[s]
        out[t] = acc
    return out


def rglru_block(w: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, decay_c: float = 8.0) -> torch.Tensor:
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    bs = C // B
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    u = causal_conv(h @ w[pre + "x"].T + w[pre + "x.b"], w[pre + "conv"], w[pre + "conv.b"])
    sp = softplus(w[pre + "lam"])
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        r = torch.zeros(C, dtype=h.dtype)
        i = torch.zeros(C, dtype=h.dtype)
        for b in range(B):
            ub = u[t, b * bs:(b + 1) * bs]
            r[b * bs:(b + 1) * bs] = sigmoid(w[pre + "ra"][b] @ ub + w[pre + "ra.b"][b])
            i[b * bs:(b + 1) * bs] = sigmoid(w[pre + "ri"][b] @ ub + w[pre + "ri.b"][b])
        a = torch.exp(-decay_c * r * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * (i * u[t])
        out[t] = S * y[t]
    return out @ w[pre + "o"].T


# ---- the feed-forward ---------------------------------------------------------------------------------------

def clamped_expert(w: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def table_moe(w: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    top, limit = int(m["router"]["top"]), float(m["expert"]["limit"])
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for e in w[pre + "table"][tok].tolist():
            out[t] = out[t] + clamped_expert(w, f"{pre}e{int(e)}.", h[t], limit) / top
    return out


# ---- the model ------------------------------------------------------------------------------------------------

def run_order(cfg: Dict[str, Any]) -> List[tuple]:
    """(layer, whether the loop's input product comes right before it) for every layer run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def layer(cfg, w, i: int, x: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    e, eps, pre = cfg["layers"][i], float(cfg["norm"]["eps"]), f"l{i}."
    h = rms_norm(x, w[pre + "norm1"], eps)
    if e["type"] == "attention":
        mix = sink_attention(w, pre + "mix.", e["mixer"], h)
    elif e["type"] == "latent_attention":
        mix = latent_attention(w, pre + "mix.", e["mixer"], h, eps)
    elif e["type"] == "rglru":
        mix = rglru_block(w, pre + "mix.", e["mixer"], h)
    else:
        raise ValueError(e["type"])
    x = x + mix * w[pre + "ls1"]
    if e.get("mlp") is not None:
        x = x + table_moe(w, pre + "mlp.", e["mlp"], h, tokens) * w[pre + "ls2"]
    return x


def forward(cfg: Dict[str, Any], w: Dict[str, torch.Tensor], tokens: Sequence[int], keep_layers: bool = False):
    """Logits [T, vocab] of one sequence from position 0; with ``keep_layers`` also the stream after every layer run."""
    tok = torch.tensor(list(tokens), dtype=torch.long)
    x0 = w["embed"][tok] * float(cfg.get("embedding", {}).get("scale", 1.0))
    x, kept = x0, []
    for i, inject in run_order(cfg):
        if inject:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        x = layer(cfg, w, i, x, tokens)
        kept.append(x)
    logits = rms_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["embed"].T
    return (logits, torch.stack(kept)) if keep_layers else logits
