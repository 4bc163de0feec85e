"""Small Demazen configurations and model folders whose small parameters make faults show."""
from __future__ import annotations

import zlib
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_demazen as plain


def memory(heads=2, dim=16, vdim=24, gate_cap=8.0) -> dict:
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}


def left(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size: Optional[int] = 20) -> dict:
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    return m


def right(heads=2, dim=16, vdim=16, tau=8.0, rank=8) -> dict:
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def dense(ff=96) -> dict:
    return {"kind": "dense", "ff": ff}


def moe(ff=40, experts=6, top=2) -> dict:
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def mlstm(mixer: dict, mlp: Optional[dict], weights_of: Optional[int] = None) -> dict:
    e = {"type": "mlstm", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def parallel(l: dict, r: dict, mlp: Optional[dict], weights_of: Optional[int] = None) -> dict:
    e = {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def config(layers: Sequence[dict], width=64, vocab=200, softcap: Optional[float] = 20.0, eps=1e-5, max_positions=512) -> dict:
    c = {"architecture": "Demazen", "layers": list(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width,
         "max_positions": max_positions}
    if softcap is not None:
        c["logit_softcap"] = softcap
    return c


#: both mixers, sizes that all differ from one another, every kind of feed-forward, a layer without one, shared key
#: heads, windows that end inside pages of 16, layers that run another layer's weights (a parallel one and a memory)
MIXED = config([mlstm(memory(), dense()),
                parallel(left(), right(), moe()),
                parallel(left(heads=3, kv_heads=3, dim=24, vdim=16, size=33), right(heads=3, dim=8, vdim=24, tau=4.0, rank=4), None),
                mlstm(memory(heads=1, dim=40, vdim=12, gate_cap=15.0), moe(ff=24, experts=5, top=1)),
                parallel(left(), right(), moe(), weights_of=1),
                mlstm(memory(), dense(), weights_of=0)])
#: tiny, for runs where plain Python stands in for the kernels
TINY = config([mlstm(memory(heads=2, dim=8, vdim=12, gate_cap=6.0), moe(ff=12, experts=3, top=2)),
               parallel(left(heads=2, kv_heads=1, dim=8, vdim=12, size=6), right(heads=2, dim=8, vdim=8, tau=5.0, rank=3), dense(40)),
               mlstm(memory(heads=2, dim=8, vdim=12, gate_cap=6.0), moe(ff=12, experts=3, top=2), weights_of=0)],
              width=32, vocab=61, max_positions=64)
#: keys and values of 64 and of 128, the widths of the tensor-core attention kernels; windows that end inside pages of 64;
#: memories of 64 x 64 and 128 x 64
SERVING_HEADS = config([parallel(left(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=100), right(heads=2, dim=64, vdim=64, tau=16.0, rank=16), dense(128)),
                        mlstm(memory(heads=2, dim=128, vdim=64, gate_cap=10.0), moe(ff=64, experts=8, top=3)),
                        parallel(left(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, size=70), right(heads=1, dim=128, vdim=32, tau=2.0, rank=8), None)],
                       width=128, max_positions=1024)
#: sizes that fit no vector width: a model width of 100, heads of 12 and 20, a window of one token, no mask at all, keys
#: of 36, 132 and 200 channels (every shape of the recurrences' kernel), all experts chosen, one expert, no cap on the logits
ODD = config([parallel(left(heads=5, kv_heads=5, dim=12, vdim=20, scale=0.4, size=1), right(heads=1, dim=132, vdim=12, tau=1.0, rank=5), moe(ff=10, experts=7, top=7)),
              mlstm(memory(heads=3, dim=36, vdim=20, gate_cap=3.0), dense(34)),
              parallel(left(heads=6, kv_heads=2, dim=20, vdim=12, scale=0.2, size=None), right(heads=5, dim=12, vdim=4, tau=30.0, rank=1), moe(ff=6, experts=1, top=1)),
              mlstm(memory(heads=1, dim=200, vdim=28, gate_cap=25.0), None)],
             width=100, vocab=133, softcap=None, eps=1e-6, max_positions=300)


#: one layer of one mechanism each, so that a fault names its mixer or its feed-forward
ONE = {
    "memory": config([mlstm(memory(heads=3, dim=20, vdim=12, gate_cap=5.0), None)]),
    "memory_wide": config([mlstm(memory(heads=1, dim=72, vdim=40, gate_cap=9.0), None)]),
    "window": config([parallel(left(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.5, size=19), right(heads=1, dim=4, vdim=4, rank=2), None)]),
    "shared_keys": config([parallel(left(heads=6, kv_heads=1, dim=8, vdim=8, scale=0.7, size=50), right(heads=1, dim=4, vdim=4, rank=2), None)]),
    "linear": config([parallel(left(heads=1, kv_heads=1, dim=4, vdim=4, size=3), right(heads=3, dim=24, vdim=20, tau=3.0, rank=6), None)]),
    "linear_wide": config([parallel(left(heads=1, kv_heads=1, dim=4, vdim=4, size=3), right(heads=2, dim=136, vdim=8, tau=40.0, rank=2), None)]),
    "experts": config([mlstm(memory(heads=1, dim=8, vdim=8), moe(ff=20, experts=9, top=4))]),
    "dense": config([mlstm(memory(heads=1, dim=8, vdim=8), dense(70))]),
}


def planted_cache(klen: int, qlen: int, j_star: int, dk: int, dv: int, page: int, nh: int = 2, nkv: int = 1, device="cuda",
                  dtype=torch.float32):
    """Queries, a paged cache and its page table in which key ``j_star`` matches every query far better than any
    other key and carries the value 1 where all others carry 0; the pages are taken in a scrambled order."""
    g = torch.Generator().manual_seed(klen * 131 + j_star)
    pages = -(-klen // page)
    order = torch.randperm(pages + 3, generator=g)[:pages].to(torch.int32)
    cache = torch.randn((pages + 3, page * nkv * (dk + dv)), generator=g) * 0.01
    direction = torch.randn(dk, generator=g)
    direction /= direction.norm()
    for j in range(klen):
        pg, off = int(order[j // page]), j % page
        cache[pg, off * dk:(off + 1) * dk] = direction * (30.0 if j == j_star else 0.0) + 0.01 * torch.randn(dk, generator=g)
        v0 = page * nkv * dk + off * dv
        cache[pg, v0:v0 + dv] = 1.0 if j == j_star else 0.0
    q = (direction[None, :] + 0.01 * torch.randn((qlen * nh, dk), generator=g)).reshape(qlen, nh * dk)
    return q.to(device, dtype).contiguous(), cache.to(device, dtype).contiguous(), order[None, :].to(device).contiguous()


def write_model(folder: str, cfg: dict, seed: int = 0, dtype=torch.float32, std: float = 0.12) -> str:
    """A model folder whose small parameters are far from their neutral values: gates that move and reach their cap,
    decays from fast to slow, router biases of both signs, position vectors as large as the embeddings."""
    from vapi_b200.config.model import resolve_architecture
    from vapi_b200.weights import write_random_model
    arch = resolve_architecture(cfg)
    specs = arch.plan(arch.parse(cfg)).tensor_specs()
    over = {}
    for s in specs:
        g = torch.Generator().manual_seed(seed * 7919 + zlib.crc32(s.name.encode()) % 100003)
        parts = s.name.split(".")
        tail = ".".join(parts[2:])
        if tail in ("mix.i", "mix.f"):
            over[s.name] = 0.6 * torch.randn(s.shape, generator=g)
        elif tail == "mix.i.b":
            over[s.name] = 1.5 * torch.randn(s.shape, generator=g)
        elif tail == "mix.f.b":
            over[s.name] = 2.0 + 1.5 * torch.randn(s.shape, generator=g)
        elif tail in ("mix.right.a1", "mix.right.a2"):
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif tail == "mix.right.a2.b":
            over[s.name] = 2.0 * torch.randn(s.shape, generator=g) + 1.0
        elif tail == "mlp.router":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif tail == "mlp.router.b":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
    return write_random_model(folder, cfg, seed, std=std, norm_init="perturbed", dtype=dtype, overrides=over)


class Oracle:
    """The plain model on a folder, float64."""

    def __init__(self, folder: str):
        self.cfg = plain.read_config(folder)
        self.w = plain.read_weights(folder, torch.float64)
        self._memo: Dict[Tuple[int, ...], torch.Tensor] = {}
        self.w32 = None

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.w, tokens)
        return self._memo[key]

    def rounding(self, tokens: Sequence[int]) -> np.ndarray:
        """What 32-bit arithmetic alone does to each position's logits: the plain model in float32 against itself
        in float64, as a part of the logits' range.  (Where a memory's read-out is small beside its terms, or a norm
        divides by little, a position is ill-conditioned, and no order of summation is exact there.)"""
        key = ("f32",) + tuple(tokens)
        if key not in self._memo:
            if self.w32 is None:
                self.w32 = {k: (v.float() if v.is_floating_point() else v) for k, v in self.w.items()}
            want = self.logits(tokens)
            got = plain.forward(self.cfg, self.w32, tokens).double()
            self._memo[key] = ((got - want).abs().amax(-1) / float(want.max() - want.min())).numpy()
        return self._memo[key]

    def greedy(self, tokens: Sequence[int], n: int):
        toks, out = list(tokens), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(toks)[-1]))
            out.append(t)
            toks.append(t)
        return out
