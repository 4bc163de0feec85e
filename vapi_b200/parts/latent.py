"""Latent attention: keys and values are made from one small normed vector per token, which is all the cache keeps."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, Mixer, PagedBuffer, PagedSpec, TensorSpec, register_mixer


class LatentAttention(Mixer):
    """Causal attention of ``heads`` heads whose per-head query and key have ``dim`` unrotated and ``rot_dim``
    rotated elements (laid out in that order) and whose value has ``vdim``.

    Queries: ``c_q = rmsnorm(W_dq x) * w_q`` (``q_rank`` wide), ``q = W_uq c_q``.  Keys and values:
    ``W_dkv x`` has ``kv_rank + rot_dim`` rows; ``c = rmsnorm(first kv_rank) * w_c`` is the latent and the last
    ``rot_dim`` (not normed) are one rotated key part that every head shares.  Head h's unrotated key is
    ``W_uk[h] c``, its value ``W_uv[h] c``, and its score
    ``(q_unrotated . k_unrotated + rot(q_rotated) . rot(k_rotated)) * scale``; softmax over the visible keys;
    ``W_o`` on the concatenated heads.  ``pos`` names the rotary tables (pairs (i, i + rot/2) over the first
    ``rot`` elements of the rotated part; ``rot`` defaults to ``rot_dim``).

    What runs is the same sum in another order, so that nothing but ``c | rot(k_rotated)`` is ever cached or
    expanded: ``q_unrotated . (W_uk[h] c) = (W_uk[h]^T q_unrotated) . c``, so the head's query is carried through
    the key up-projection once (a batched product over the heads), a score is one dot product of
    ``[W_uk[h]^T q_unrotated | rot(q_rotated)]`` with a token's cached row, the softmax's weighted sum is taken over
    the cached latents themselves (every head reads the one cached row per token: the attention kernel's key and
    value are the same memory), and the value up-projection ``W_uv[h]`` is applied to that sum (a second batched
    product).  The three down-projections are one product whose float32 result feeds the norms unrounded.
    """

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, *,
                 scale: float, norm_eps: float, pos: Optional[str] = "rope", rot: Optional[int] = None,
                 names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight"):
        if heads <= 0 or dim <= 0 or rot_dim < 0 or vdim <= 0 or kv_rank <= 0 or q_rank <= 0:
            raise ValueError(f"latent attention of {heads} heads, {dim} + {rot_dim} / {vdim}, ranks {q_rank} / {kv_rank}")
        if kv_rank % 4 or rot_dim % 4 or not 4 <= kv_rank + rot_dim <= 640 or kv_rank > 512:
            raise ValueError(f"a cached row of {kv_rank} + {rot_dim}: both multiples of 4, at most 640 together, 512 the latent")
        self.hidden, self.H, self.d, self.r, self.dv = int(hidden), int(heads), int(dim), int(rot_dim), int(vdim)
        self.R, self.Q = int(kv_rank), int(q_rank)
        self.rot = int(rot) if rot is not None else self.r
        if pos is None or self.r == 0:
            self.rot, pos = 0, None
        if self.rot < 0 or self.rot > self.r or self.rot % 2:
            raise ValueError(f"{self.rot} rotated elements of a part of {self.r}")
        self.scale, self.eps, self.pos, self.sfx = float(scale), float(norm_eps), pos, weight_suffix
        self.names = {"dq": "q_down", "dq_norm": "q_down_norm", "uq": "q_up", "dkv": "kv_down", "dkv_norm": "kv_down_norm",
                      "uk": "k_up", "uv": "v_up", "o": "out_proj"}
        if names:
            self.names.update(names)
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.q_w = self.c_w = None

    def cache_spec(self):
        return PagedSpec((PagedBuffer("latent", 1, self.R + self.r),), 0)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, x, H = self.names, self.sfx, self.H
        return [TensorSpec(f"{prefix}{n['dq']}{x}", (self.Q, self.hidden)),
                TensorSpec(f"{prefix}{n['dq_norm']}", (self.Q,), role="vector", init="ones"),
                TensorSpec(f"{prefix}{n['uq']}{x}", (H * (self.d + self.r), self.Q)),
                TensorSpec(f"{prefix}{n['dkv']}{x}", (self.R + self.r, self.hidden)),
                TensorSpec(f"{prefix}{n['dkv_norm']}", (self.R,), role="vector", init="ones"),
                TensorSpec(f"{prefix}{n['uk']}{x}", (H * self.d, self.R)),
                TensorSpec(f"{prefix}{n['uv']}{x}", (H * self.dv, self.R)),
                TensorSpec(f"{prefix}{n['o']}{x}", (self.hidden, H * self.dv))]

    def bind(self, tensors, prefix, dtype):
        n, x = self.names, self.sfx
        dq, dkv = tensors[f"{prefix}{n['dq']}{x}"], tensors[f"{prefix}{n['dkv']}{x}"]
        wd = dq.dtype if dq.dtype == dkv.dtype else torch.float32
        self.w_down = torch.cat([dq.to(wd), dkv.to(wd)], 0).contiguous()                 # query latent | latent | key part
        self.w_uq = tensors[f"{prefix}{n['uq']}{x}"].contiguous()
        # [heads, dim, kv_rank]: a head's query times this is its query in the latent's coordinates
        self.w_uk = tensors[f"{prefix}{n['uk']}{x}"].to(dtype).reshape(self.H, self.d, self.R).contiguous()
        # [heads, kv_rank, vdim]
        self.w_uv = tensors[f"{prefix}{n['uv']}{x}"].to(dtype).reshape(self.H, self.dv, self.R).transpose(1, 2).contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}{x}"].contiguous()
        self.q_w = tensors[f"{prefix}{n['dq_norm']}"].contiguous()
        self.c_w = tensors[f"{prefix}{n['dkv_norm']}"].contiguous()

    def decode_splits(self, batch: int, max_context: int, page_size: int, dtype: torch.dtype) -> int:
        return ops.masked_attention_splits(batch, 1, max_context, self.H, 1)

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        H, d, r, R, dv = self.H, self.d, self.r, self.R, self.dv
        n = a.shape[0]
        cos = sin = None
        if self.pos is not None:
            cos, sin = ctx.pos[self.pos]
        grp = cache.group
        pages = cache.tensor                                         # flat [pages, page_size * (R + r)]
        page_size = pages.shape[1] // (R + r)
        down = ops.linear(a, self.w_down, None, torch.float32)
        cq = ops.latent_prepare(down, self.Q, R, r, self.q_w, self.c_w, self.eps, cos, sin, self.rot,
                                pages if cache.write else None, page_size, grp.slot_mapping, a.dtype, ctx.status)
        q = ops.linear(cq, self.w_uq)                                # [n, H * (d + r)]
        if q.dtype != a.dtype:
            q = q.to(a.dtype)
        qfull = torch.empty((n, H, R + r), dtype=a.dtype, device=a.device)
        ops.head_products(q.view(n, H, d + r)[:, :, :d], self.w_uk, qfull[:, :, :R])
        if r:
            ops.latent_rotate_q(q, qfull, H, d, r, R, cos, sin, self.rot)
        splits = grp.splits if getattr(grp, "splits", None) is not None else ctx.attention_splits
        max_k = getattr(grp, "max_k", None) or ctx.max_k
        o = ops.latent_attention(qfull.view(n, H * (R + r)), pages, page_size, grp.block_table, ctx.cu_q, ctx.seqlens_k,
                                 ctx.n, ctx.num_seqs, ctx.max_q, max_k, H, R, r, self.scale, splits=splits,
                                 status=ctx.status)                                          # [n, H * R]
        y = ops.head_products(o.view(n, H, R), self.w_uv)                                    # [n, H, dv]
        return ops.linear(y.view(n, H * dv), self.w_o)


register_mixer("latent_attention", LatentAttention)
