"""The Demazen model, plainly: one function per mechanism, float64 by default, token by token where the
design is a recurrence.  Shares no code with the package; reads a model folder with its own few lines."""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch

MLSTM_FLOOR_EPS = 1e-6          # added to the denominator of the matrix memory's read-out


# ---- files ---------------------------------------------------------------------------------------
def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


_DT = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in head.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=_DT[e["dtype"]]).reshape(e["shape"])
        out[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return out


# ---- small pieces ----------------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w when given."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * w if w is not None else y


def silu(z):
    return z * torch.sigmoid(z)


def logsigmoid(z):
    return -torch.nn.functional.softplus(-z)


def embed(w, tokens: Sequence[int], first: int = 0) -> torch.Tensor:
    idx = torch.tensor(list(tokens), dtype=torch.long)
    pos = torch.arange(first, first + len(tokens))
    return w["embed"][idx] + w["pos"][pos]


# ---- the matrix memory -------------------------------------------------------------------------------
def mlstm(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """h [T, width] -> [T, width]; the whole sequence from an empty memory."""
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                 # [T, H] log input gate
    gf = logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))     # [T, H] log forget gate
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        n = torch.zeros(dk, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new = torch.maximum(gf[t, a] + mx, gi[t, a])
            keep, take = torch.exp(gf[t, a] + mx - new), torch.exp(gi[t, a] - new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            mx = new
            den = torch.maximum(torch.abs(n @ q[t, a]), torch.exp(-mx)) + MLSTM_FLOOR_EPS
            out[t, a] = (S.T @ q[t, a]) / den
    o = rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---- attention over a sliding window -----------------------------------------------------------------
def window_attention(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = (m.get("mask") or {}).get("size")
    T = h.shape[0]
    q = rms(h @ w[p + "q"].T, eps, w[p + "q.norm"]).reshape(T, H, dk)
    k = rms(h @ w[p + "k"].T, eps, w[p + "k.norm"]).reshape(T, G, dk)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if not size else (j <= i) & (i - j < size)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~seen, float("-inf"))
        out[:, a] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- gated linear attention --------------------------------------------------------------------------
def gated_linear_attention(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.exp(logsigmoid(z) / tau).reshape(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = alpha[t, a][:, None] * S + torch.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    o = (rms(out, eps) * w[p + "norm"]).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    a = window_attention(w, p + "left.", m["left"], h, eps)
    b = gated_linear_attention(w, p + "right.", m["right"], h, eps)
    return 0.5 * (rms(a, eps, w[p + "left.out"]) + rms(b, eps, w[p + "right.out"]))


# ---- feed-forward --------------------------------------------------------------------------------------
def gated_ff(w, p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def experts(w, p: str, m: dict, h: torch.Tensor, margins: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    top = m["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    if margins is not None and top < z.shape[-1]:
        # how far the last chosen logit stands above the first one left out, as a part of the logits' spread
        zs = torch.sort(z, -1, descending=True).values
        margins.append((zs[:, top - 1] - zs[:, top]) / (zs[:, 0] - zs[:, -1]).clamp_min(1e-30))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        val, idx = torch.topk(z[t], top)
        wt = torch.softmax(val, -1)
        for c in range(top):
            out[t] += wt[c] * gated_ff(w, f"{p}e{int(idx[c])}.", h[t:t + 1])[0]
    return out


def feed_forward(w, p: str, m: dict, h: torch.Tensor, margins: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    return gated_ff(w, p, h) if m["kind"] == "dense" else experts(w, p, m, h, margins)


# ---- the model -------------------------------------------------------------------------------------------
def forward(cfg: dict, w, tokens: Sequence[int], layers_out: Optional[List[torch.Tensor]] = None,
            margins: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence from position 0.  ``layers_out`` receives the stream after every layer,
    ``margins`` every routed layer's margin of choice per token."""
    eps = float(cfg["norm"]["eps"])
    x = embed(w, tokens)
    for i, e in enumerate(cfg["layers"]):
        p = f"l{e.get('weights_of', i)}."
        mix = mlstm if e["type"] == "mlstm" else parallel
        x = x + rms(mix(w, p + "mix.", e["mixer"], x, eps), eps, w[p + "norm1"])
        if e.get("mlp") is not None:
            x = x + rms(feed_forward(w, p + "mlp.", e["mlp"], x, margins), eps, w[p + "norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rms(x, eps, w["final.norm"]) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
