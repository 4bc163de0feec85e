"""Small Nelosun configurations and model folders whose small parameters make faults show."""
from __future__ import annotations

import zlib
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_nelosun as plain


def attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, coef: Optional[float] = 0.4, every=5) -> dict:
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=28, scale=0.25, base=100.0, dims: Optional[int] = None) -> dict:
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def rglru(width=48, blocks=3, conv=4) -> dict:
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def moe(ff=24, experts=5, top=2, limit=0.8) -> dict:
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(mixer: dict, mlp: Optional[dict]) -> dict:
    return {**mixer, "mlp": mlp}


def config(layers: Sequence[dict], width=64, vocab=200, loop: Optional[Tuple[int, int, int]] = None, scale: Optional[float] = 3.0,
           eps=1e-5) -> dict:
    c = {"architecture": "Nelosun", "layers": list(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if scale is not None:
        c["embedding"] = {"scale": scale}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


#: sizes that all differ from one another; the loop starts behind the first layer and runs three times; a layer
#: without a feed-forward; a temperature that steps every five positions; two experts a token; clamps that bite
MIXED = config([layer(attention(), moe()),
                layer(latent(), moe(ff=16, experts=4, top=1, limit=0.5)),
                layer(rglru(), None),
                layer(attention(heads=3, kv_heads=3, dim=24, vdim=16, scale=0.2, coef=0.7, every=16), moe(ff=32, experts=3, top=3)),
                layer(latent(heads=2, dim=16, rot_dim=12, vdim=16, kv_rank=40, q_rank=20, dims=8, base=7.0), moe())],
               loop=(1, 4, 3))
#: tiny, for runs where plain Python stands in for the kernels
TINY = config([layer(latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=12, q_rank=8), moe(ff=8, experts=3, top=2)),
               layer(attention(heads=2, kv_heads=1, dim=8, vdim=12, every=3), moe(ff=8, experts=2, top=1)),
               layer(rglru(width=16, blocks=2, conv=3), None)], width=32, vocab=64, loop=(0, 2, 2))
#: values that a model may happen to make equal or one: no loop, no scale, no temperature, one expert, one part, one tap,
#: one head, equal key and value widths
PLAIN = config([layer(attention(heads=1, kv_heads=1, dim=16, vdim=16, coef=None), moe(ff=16, experts=1, top=1, limit=50.0)),
                layer(latent(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=16, q_rank=16), None),
                layer(rglru(width=64, blocks=1, conv=1), moe(ff=64, experts=2, top=2))], width=64, vocab=90, scale=None)
#: the head sizes of the serving kernels (keys and values of 64: tensor cores for bfloat16), a loop over everything, once
SERVING_HEADS = config([layer(attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.11, every=40), moe(ff=64, experts=6, top=2, limit=2.0)),
                        layer(latent(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=64, q_rank=48, scale=0.12), moe(ff=64, experts=6, top=2)),
                        layer(rglru(width=128, blocks=2, conv=4), moe(ff=32, experts=4, top=1))], width=128, vocab=300, loop=(0, 3, 1))
#: one kind of mixer alone, with a feed-forward and a loop of two passes
ONE = {"attention": config([layer(attention(), moe())] * 2, loop=(0, 1, 2)),
       "latent": config([layer(latent(), moe())] * 2, loop=(1, 2, 2)),
       "rglru": config([layer(rglru(), moe())] * 2, loop=(0, 2, 2))}


def write_model(folder: str, cfg: dict, seed: int = 0, dtype=torch.float32, std: float = 0.12) -> str:
    """A model folder whose small parameters are far from their neutral values: layer scales and norm weights that
    differ, biases and gates that matter, decays from fast to slow, convolutions with a bias, an input product as
    strong as the identity."""
    from vapi_b200.config.model import resolve_architecture
    from vapi_b200.weights import write_random_model
    arch = resolve_architecture(cfg)
    specs = arch.plan(arch.parse(cfg)).tensor_specs()
    over = {}
    W = cfg["width"]
    for s in specs:
        g = torch.Generator().manual_seed(seed * 7919 + zlib.crc32(s.name.encode()) % 100003)
        tail = ".".join(s.name.split(".")[1:])
        if tail in ("ls1", "ls2"):
            over[s.name] = 0.7 + 0.5 * torch.rand(s.shape, generator=g)
        elif tail == "mix.lam":
            over[s.name] = torch.linspace(-4.0, 2.0, s.shape[0])[torch.randperm(s.shape[0], generator=g)]
        elif tail in ("mix.ra", "mix.ri"):
            over[s.name] = 0.4 * torch.randn(s.shape, generator=g)
        elif tail == "mix.conv":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif tail.endswith(".b"):
            over[s.name] = 0.3 * torch.randn(s.shape, generator=g)
        elif tail == "mix.g":
            over[s.name] = 0.5 * torch.randn(s.shape, generator=g)
        elif s.name == "loop.in":
            over[s.name] = torch.cat([torch.eye(W), 0.5 * torch.eye(W)], 1) + 0.05 * torch.randn(s.shape, generator=g)
    return write_random_model(folder, cfg, seed, std=std, norm_init="perturbed", dtype=dtype, overrides=over)


def prompt(cfg: dict, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


class Oracle:
    """The plain model on a folder, float64."""

    def __init__(self, folder: str):
        self.cfg = plain.read_config(folder)
        self.w = plain.read_weights(folder, torch.float64)
        self._memo: Dict[tuple, object] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.w, tokens)
        return self._memo[key]

    def rounding(self, tokens: Sequence[int], dtype: str = "float32") -> np.ndarray:
        """What reduced precision alone does to each position's logits, as a part of the logits' range.  float32: the
        plain model in float32 against itself in float64, the largest of three draws (the weights as they are, and
        twice with every element moved by up to 2^-23 of itself).  bfloat16: the plain model with every matrix moved
        by up to 2^-8 of each element against itself."""
        key = (dtype,) + tuple(tokens)
        if key not in self._memo:
            want = self.logits(tokens)
            g = torch.Generator().manual_seed(99)

            def moved(by, to):
                return {k: (v * (1.0 + by * (2.0 * torch.rand(v.shape, generator=g, dtype=v.dtype) - 1.0))).to(to)
                        if v.is_floating_point() and (v.dim() >= 2 or to == torch.float32) else v for k, v in self.w.items()}
            if dtype == "float32":
                draws = [plain.forward(self.cfg, moved(by, torch.float32), tokens).double() for by in (0.0, 2.0 ** -23, 2.0 ** -23)]
            else:
                draws = [plain.forward(self.cfg, moved(2.0 ** -8, torch.float64), tokens)]
            err = torch.stack([(got - want).abs().amax(-1) for got in draws]).amax(0)
            self._memo[key] = (err / float(want.max() - want.min())).numpy()
        return self._memo[key]

    def greedy(self, tokens: Sequence[int], n: int):
        toks, out = list(tokens), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(toks)[-1]))
            out.append(t)
            toks.append(t)
        return out


def planted_latent(klen: int, j_star: int, qlen: int, heads: int, rank: int, rot: int, page: int, device: str, dtype=torch.float32):
    """Queries, a paged cache of rows ``[latent | key part]`` and its page table in which row ``j_star`` matches every
    query far better than any other row; its latent is all ones where the others' are near zero, so that a head's
    output says whether that row was seen.  The pages are taken in a scrambled order."""
    g = torch.Generator().manual_seed(klen * 131 + j_star)
    width = rank + rot
    pages = -(-klen // page)
    order = torch.randperm(pages + 3, generator=g)[:pages].to(torch.int32)
    cache = torch.randn((pages + 3, page * width), generator=g) * 0.01
    direction = torch.randn(rot, generator=g)
    direction /= direction.norm()
    for j in range(klen):
        pg, off = int(order[j // page]), j % page
        row = 0.01 * torch.randn(width, generator=g)
        if j == j_star:
            row[:rank] = 1.0
            row[rank:] = direction * 30.0
        cache[pg, off * width:(off + 1) * width] = row
    q = torch.zeros((qlen, heads, width))
    q[:, :, rank:] = direction[None, None, :] + 0.01 * torch.randn((qlen, heads, rot), generator=g)
    return (q.reshape(qlen, heads * width).to(device, dtype).contiguous(), cache.to(device, dtype).contiguous(),
            order[None, :].to(device).contiguous())
