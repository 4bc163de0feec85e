"""Token embedding and the output head."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from .. import ops
from .base import Part, TensorSpec


class TokenEmbedding(Part):
    """Row gather from a [vocab, hidden] table, no scaling
    (crates/vapi-backend-candle/src/models/lfm2.rs:675, 808).  Starts the float32 stream."""

    def __init__(self, vocab: int, hidden: int, name: str = "model.embed_tokens.weight", *,
                 sinusoid_base: Optional[float] = None, streams: Optional[int] = None,
                 position_table: Optional[str] = None, positions: int = 0, scale: float = 1.0):
        self.vocab, self.hidden, self.name = int(vocab), int(hidden), name
        #: every row is multiplied by this number (a float32 product) on its way into the stream
        self.scale = float(scale)
        #: with ``sinusoid_base`` a position vector is added: entry 2i is sin(p * base^(-2i/hidden)), entry
        #: 2i+1 the cosine of the same angle (positions and angles in float32)
        self.sinusoid_base = float(sinusoid_base) if sinusoid_base is not None else None
        #: with ``streams`` the stream starts as that many equal copies, [n, streams, hidden]
        self.streams = int(streams) if streams is not None else None
        #: with ``position_table`` (a tensor name) row p of that [positions, hidden] table is added at position p
        self.position_table, self.positions = position_table, int(positions)
        if position_table is not None and self.positions <= 0:
            raise ValueError("a position table needs its number of rows")
        self.table: Optional[torch.Tensor] = None
        self.freq: Optional[torch.Tensor] = None
        self.pos_rows: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str = "") -> List[TensorSpec]:
        specs = [TensorSpec(self.name, (self.vocab, self.hidden))]
        if self.position_table is not None:
            specs.append(TensorSpec(self.position_table, (self.positions, self.hidden)))
        return specs

    def bind(self, tensors, prefix, dtype):
        self.table = tensors[self.name].contiguous()
        if self.position_table is not None:
            self.pos_rows = tensors[self.position_table].to(self.table.dtype).contiguous()
        if self.sinusoid_base is not None:
            i = torch.arange((self.hidden + 1) // 2, dtype=torch.float64)
            freq = torch.pow(torch.tensor(self.sinusoid_base, dtype=torch.float64), -2.0 * i / self.hidden)
            self.freq = freq.to(torch.float32).to(self.table.device)      # rounded once, from the exact value

    def forward(self, ctx: Any, next_weight: Optional[torch.Tensor] = None):
        """The stream; with ``next_weight`` also what a deferred norm needs: ``(x, ss, xw)``."""
        if self.sinusoid_base is not None or self.streams is not None or self.pos_rows is not None:
            if next_weight is not None or self.scale != 1.0:
                raise ValueError("an embedding with positions or several streams has no deferred-norm form and no scale")
            x = ops.embed_sinusoid(self.table, ctx.tokens, ctx.positions, self.freq, self.streams or 1, ctx.status,
                                   pos_table=self.pos_rows)
            return x if self.streams is not None else x.view(x.shape[0], self.hidden)
        return ops.embed(self.table, ctx.tokens, ctx.status, next_weight, self.scale)


class OutputHead(Part):
    """Logits in float32 for the wanted rows: ``norm(x)[rows] @ W.T``.

    ``tied`` (or a checkpoint without the head's tensor) reuses the embedding table
    (crates/vapi-backend-candle/src/models/lfm2.rs:676-680, 803-818)."""

    def __init__(self, vocab: int, hidden: int, tied: bool, embedding: TokenEmbedding,
                 name: str = "lm_head.weight", scale: float = 1.0, softcap: Optional[float] = None):
        self.vocab, self.hidden, self.tied, self.embedding, self.name = int(vocab), int(hidden), bool(tied), embedding, name
        #: the logits are multiplied by this number (in float32, after the product)
        self.scale = float(scale)
        #: then ``logits <- softcap * tanh(logits / softcap)`` (None: not at all)
        self.softcap = float(softcap) if softcap else None
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str = "") -> List[TensorSpec]:
        if self.tied:
            return []
        # optional: a checkpoint that leaves it out falls back to the embedding table
        return [TensorSpec(self.name, (self.vocab, self.hidden), optional=True)]

    def bind(self, tensors, prefix, dtype):
        w = None if self.tied else tensors.get(self.name)
        self.weight = (w if w is not None else tensors[self.embedding.name]).contiguous()

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(xn, self.weight, None, torch.float32)
        if self.scale != 1.0:
            logits = ops.scale_rows(logits, self.scale)
        return logits if self.softcap is None else ops.softcap(logits.contiguous(), self.softcap)

    def forward_stream(self, a):
        """Logits of every row of a lazily normed stream (decode steps), or NotImplemented."""
        if not ops.few_rows_applies(a.xw.shape[0], self.weight):
            return NotImplemented
        logits = ops.few_rows_linear(self.weight, xw=a.xw, ss_in=a.ss, eps=a.eps, epilogue="f32")
        if self.scale != 1.0:
            logits = ops.scale_rows(logits, self.scale)
        return logits if self.softcap is None else ops.softcap(logits, self.softcap)
