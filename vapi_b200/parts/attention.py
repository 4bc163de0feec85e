"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, Mixer, PagedBuffer, PagedSpec, StreamState, TensorSpec, register_mixer


class GQAttention(Mixer):
    """q/k/v projection, optional per-head RMSNorm of q and k, optional rotary encoding,
    cache write, causal attention over the block table (optionally windowed), out
    projection (crates/vapi-backend-candle/src/models/lfm2.rs:343-406; attention semantics
    crates/vapi-backend-candle/src/attention.rs:90-163).

    The three projections are fused into one matrix at bind time.  ``names`` maps the roles
    ``q k v o q_norm k_norm`` to checkpoint sub-names, so another architecture's naming is a
    parameter, not a subclass.  ``pos`` names the position encoding whose ``(cos, sin)`` to
    apply (None: no rotation).

    Options beyond the plain form, each a parameter: ``v_head_dim`` (values of another width than
    queries and keys), ``chunk`` (a query sees only keys of its own block of ``chunk`` positions,
    counted from position 0), ``sink`` (a learned number per head whose exponential joins the
    softmax's denominator), ``head_gate`` (head h's output times ``sigmoid(W_g x)_h``, the gate's
    rows riding on the fused projection), ``keep_first`` (with a window: the first ``keep_first`` tokens of a
    sequence stay visible to every later query, at their true positions; the pages are then all kept),
    ``qk_norm`` ("head": the q/k norms run per head with a weight of ``head_dim``; "projection": over a token's
    whole q, and whole k, before they are split into heads, with a weight per element of the projection),
    ``out_gate`` (the concatenated heads times ``sigmoid(W_g x)`` element by element, a gate as wide as the
    heads' output, its rows riding on the fused projection too), ``rope_layout`` ("half": pairs (i, i + rot/2);
    "interleaved": pairs (2i, 2i+1)) and ``weight_suffix`` (what follows a projection's name in the
    checkpoint), ``bias_suffix`` (what follows it for its bias), ``fixed_sink`` (a sink whose score is this number
    for every head, with no tensor: 0.0 puts a plain one into the denominator) and ``q_temp`` = (coef, every) (the
    query at position p is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``).  Any of these but the
    suffixes sends the mixer to the general kernels
    (``ops.qk_norm_rope_write_split``, ``ops.masked_attention``); the plain form keeps the
    specialised ones.
    """

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, *,
                 qk_norm_eps: Optional[float] = None, pos: Optional[str] = "rope",
                 rot_dim: Optional[int] = None, window: int = 0, bias: bool = False,
                 scale: Optional[float] = None, names: Optional[Dict[str, str]] = None,
                 v_head_dim: Optional[int] = None, chunk: int = 0, sink: bool = False, head_gate: bool = False,
                 rope_layout: str = "half", weight_suffix: str = ".weight", keep_first: int = 0, out_gate: bool = False,
                 qk_norm: str = "head", bias_suffix: str = ".bias", fixed_sink: Optional[float] = None,
                 q_temp: Optional[Any] = None):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if rope_layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout `{rope_layout}` is not one of half, interleaved")
        self.dv = int(v_head_dim) if v_head_dim is not None else int(head_dim)
        self.chunk, self.sink, self.head_gate = int(chunk), bool(sink), bool(head_gate)
        self.interleaved = rope_layout == "interleaved"
        self.keep_first, self.out_gate = max(int(keep_first), 0) if int(window) > 0 else 0, bool(out_gate)
        if qk_norm not in ("head", "projection"):
            raise ValueError(f"q/k norm `{qk_norm}` is not one of head, projection")
        self.whole_norm = qk_norm == "projection" and qk_norm_eps is not None
        if self.head_gate and self.out_gate:
            raise ValueError("a gate per head and a gate per element exclude one another")
        if fixed_sink is not None and self.sink:
            raise ValueError("a learned sink and a fixed one exclude one another")
        self.fixed_sink = float(fixed_sink) if fixed_sink is not None else None
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else None
        if self.q_temp is not None and (self.q_temp[1] < 1 or self.whole_norm):
            raise ValueError("a query temperature needs `every` >= 1 and q/k norms per head")
        self.general = bool(self.dv != int(head_dim) or self.chunk > 0 or self.sink or self.head_gate or self.interleaved
                            or self.keep_first > 0 or self.out_gate or self.whole_norm or self.fixed_sink is not None
                            or self.q_temp is not None)
        if self.general:
            if head_dim % 4 or self.dv % 4 or not (4 <= head_dim <= 256 and 4 <= self.dv <= 256):
                raise ValueError(f"head sizes {head_dim} / {self.dv} must be multiples of 4 in 4..256")
        elif head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim} must be a multiple of 16 in 16..256")
        self.sfx, self.bsfx = weight_suffix, bias_suffix
        self.hidden, self.nh, self.nkv, self.d = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.qk_norm_eps = qk_norm_eps
        self.pos = pos
        self.rot_dim = int(rot_dim) if rot_dim is not None else self.d
        self.window = int(window)
        self.bias = bool(bias)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.d)
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "out_proj",
                      "q_norm": "q_layernorm", "k_norm": "k_layernorm", "sink": "sinks", "gate": "gate_proj"}
        if names:
            self.names.update(names)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_w = self.k_w = self.sinks = None

    def cache_spec(self):
        # (for equal widths this is PagedSpec.kv: keys [nkv, page, d], then values [nkv, page, dv])
        # (kept first tokens are read for as long as the request lives: nothing is given back early)
        return PagedSpec((PagedBuffer("k", self.nkv, self.d), PagedBuffer("v", self.nkv, self.dv)),
                         0 if self.keep_first > 0 else self.window)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, (h, nh, nkv, d), x = self.names, (self.hidden, self.nh, self.nkv, self.d), self.sfx
        specs = [TensorSpec(f"{prefix}{n['q']}{x}", (nh * d, h)),
                 TensorSpec(f"{prefix}{n['k']}{x}", (nkv * d, h)),
                 TensorSpec(f"{prefix}{n['v']}{x}", (nkv * self.dv, h)),
                 TensorSpec(f"{prefix}{n['o']}{x}", (h, nh * self.dv))]
        if self.head_gate or self.out_gate:
            specs.append(TensorSpec(f"{prefix}{n['gate']}{x}", (nh if self.head_gate else nh * self.dv, h)))
        if self.sink:
            specs.append(TensorSpec(f"{prefix}{n['sink']}", (nh,), role="vector", init="normal"))
        if self.bias:
            b = self.bsfx
            specs += [TensorSpec(f"{prefix}{n['q']}{b}", (nh * d,), role="vector"),
                      TensorSpec(f"{prefix}{n['k']}{b}", (nkv * d,), role="vector"),
                      TensorSpec(f"{prefix}{n['v']}{b}", (nkv * self.dv,), role="vector"),
                      TensorSpec(f"{prefix}{n['o']}{b}", (h,), role="vector")]
        if self.qk_norm_eps is not None:
            specs += [TensorSpec(f"{prefix}{n['q_norm']}{x}", (nh * d if self.whole_norm else d,), role="vector", init="ones"),
                      TensorSpec(f"{prefix}{n['k_norm']}{x}", (nkv * d if self.whole_norm else d,), role="vector", init="ones")]
        return specs

    def bind(self, tensors, prefix, dtype):
        n, x = self.names, self.sfx
        parts = [tensors[f"{prefix}{n[r]}{x}"] for r in ("q", "k", "v")]
        if self.head_gate or self.out_gate:
            parts.append(tensors[f"{prefix}{n['gate']}{x}"])
        wd = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        if self.general:
            # rows of the fused product stay 16-byte aligned whatever the gate adds
            rows = sum(p.shape[0] for p in parts)
            if rows % 8:
                parts.append(torch.zeros((8 - rows % 8, self.hidden), dtype=wd, device=parts[0].device))
        self.w_qkv = torch.cat([p.to(wd) for p in parts], 0).contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}{x}"].contiguous()
        if self.sink:
            self.sinks = tensors[f"{prefix}{n['sink']}"].contiguous()
        elif self.fixed_sink is not None:
            self.sinks = torch.full((self.nh,), self.fixed_sink, dtype=torch.float32, device=self.w_o.device)
        if self.bias:
            self.b_qkv = torch.cat([tensors[f"{prefix}{n[r]}{self.bsfx}"] for r in ("q", "k", "v")], 0).contiguous()
            if self.b_qkv.numel() < self.w_qkv.shape[0]:       # the gate's rows and the padding have no bias
                self.b_qkv = torch.cat([self.b_qkv, self.b_qkv.new_zeros(self.w_qkv.shape[0] - self.b_qkv.numel())])
            self.b_o = tensors[f"{prefix}{n['o']}{self.bsfx}"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_w = tensors[f"{prefix}{n['q_norm']}{x}"].contiguous()
            self.k_w = tensors[f"{prefix}{n['k_norm']}{x}"].contiguous()

    def decode_splits(self, batch: int, max_context: int, page_size: int, dtype: torch.dtype) -> int:
        keys = min(max_context, self.window + self.keep_first) if self.window > 0 else max_context
        if self.general:
            if self.chunk > 0:
                keys = min(keys, self.chunk)
            return ops.masked_attention_splits(batch, 1, keys, self.nh, self.nkv)
        dec = ops.decode_attention_applies(dtype, self.d, page_size, self.nh // self.nkv)
        return ops.attention_splits(batch, 1, keys, self.nh, self.nkv, dec)

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        qkv = ops.linear(a, self.w_qkv, self.b_qkv)
        return ops.linear(self._attend(qkv, ctx, cache), self.w_o, self.b_o)

    def forward_stream(self, a, ctx, cache, x, next_weight):
        n = x.shape[0]
        if not (ops.few_rows_applies(n, self.w_qkv) and ops.few_rows_applies(n, self.w_o)):
            return NotImplemented
        qkv = ops.few_rows_linear(self.w_qkv, xw=a.xw, ss_in=a.ss, eps=a.eps, epilogue="bf16", bias=self.b_qkv)
        y = self._attend(qkv, ctx, cache)
        ss, xw = ops.few_rows_linear(self.w_o, act=y, epilogue="resid", resid=x, bias=self.b_o, next_weight=next_weight)
        return StreamState(xw, ss)

    def _attend(self, qkv: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        nh, nkv, d = self.nh, self.nkv, self.d
        cos = sin = None
        if self.pos is not None:
            cos, sin = ctx.pos[self.pos]
        grp = cache.group
        if self.general:
            return self._attend_general(qkv, ctx, cache, cos, sin)
        n_rep = nh // nkv
        kv = cache.stacked() if cache.tensor is not None else None      # [pages, 2, n_kv, page_size, head_dim]
        splits = grp.splits if getattr(grp, "splits", None) is not None else ctx.attention_splits
        max_k = getattr(grp, "max_k", None) or ctx.max_k
        if self.window > 0:
            max_k = min(max_k, self.window + ctx.max_q - 1)      # a query reads at most `window` keys
        if (ops.FUSED_DECODE_ROPE and qkv.is_cuda and kv is not None
                and ops.decode_attention_fused_applies(qkv.dtype, d, kv.shape[3], ctx.max_q * n_rep,
                                                       self.rot_dim if cos is not None else None)
                and (cos is None or (cos.is_contiguous() and sin.is_contiguous()))):
            # a decode step: norm, rotation and the cache write ride in the attention kernel
            return ops.decode_attention_fused(qkv, nh, nkv, d, self.q_w, self.k_w,
                                              self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin,
                                              kv, cache.write, grp.block_table, ctx.cu_q, ctx.seqlens_k,
                                              ctx.n, ctx.num_seqs, ctx.max_q, max_k, self.scale, self.window,
                                              splits, ctx.status)
        ops.qk_norm_rope_write(qkv, nh, nkv, d, self.q_w, self.k_w,
                               self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                               cos, sin, self.rot_dim,
                               kv if cache.write else None, grp.slot_mapping, ctx.status)
        y = ops.paged_attention(qkv, qkv.stride(0), kv, grp.block_table, ctx.cu_q,
                                ctx.seqlens_k, ctx.n, ctx.num_seqs, ctx.max_q, max_k, nh, nkv, d,
                                self.scale, self.window, splits, ctx.status)
        return y


    def _attend_general(self, qkv, ctx, cache, cos, sin):
        """Unlike key and value widths, a chunked mask, a sink, a head gate or interleaved pairs."""
        nh, nkv, d, dv = self.nh, self.nkv, self.d, self.dv
        grp = cache.group
        pages = cache.tensor                                    # flat [pages, page_size * nkv * (d + dv)]
        page_size = pages.shape[1] // (nkv * (d + dv))
        ops.qk_norm_rope_write_split(qkv, nh, nkv, d, dv, self.q_w, self.k_w,
                                     self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin, self.rot_dim,
                                     self.interleaved, pages if cache.write else None, page_size, grp.slot_mapping,
                                     ctx.status, whole=self.whole_norm,
                                     positions=ctx.positions if self.q_temp is not None else None, q_temp=self.q_temp)
        gate = None
        if self.head_gate:
            off = (nh + nkv) * d + nkv * dv
            gate = qkv[:, off:off + nh]
        splits = grp.splits if getattr(grp, "splits", None) is not None else ctx.attention_splits
        max_k = getattr(grp, "max_k", None) or ctx.max_k
        y = ops.masked_attention(qkv, qkv.stride(0), pages, page_size, grp.block_table, ctx.cu_q, ctx.seqlens_k,
                                 ctx.n, ctx.num_seqs, ctx.max_q, max_k, nh, nkv, d, dv, self.scale,
                                 window=self.window, chunk=self.chunk, sinks=self.sinks, gate=gate, splits=splits,
                                 status=ctx.status, keep=self.keep_first)
        if self.out_gate:
            off = (nh + nkv) * d + nkv * dv
            y = ops.sigmoid_gate(y, qkv[:, off:off + nh * dv])
        return y


register_mixer("gqa_attention", GQAttention)
