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


def write_model(folder: str, cfg: dict, seed: int = 0, dtype=torch.float32, std: float = 0.12, planted_routes: bool = False) -> str:
    """A model folder whose small parameters are far from their neutral values: gates that move and reach their cap,
    decays from fast to slow, router biases of both signs, position vectors as large as the embeddings.

    With ``planted_routes`` no router's choice is a close call, so that a model in reduced precision chooses as the
    plain one does: the last channels of the width carry a code of the token (the embedding writes it, the position
    vectors and every norm weight are zero there, so no sublayer adds to it), each expert's router row reads one of
    these channels with a large weight, and two experts' logits are at least 2 apart whatever the other channels hold.
    The chosen experts' weights still move with the random part of the rows and with the biases."""
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
    if planted_routes:
        W, V = cfg["width"], cfg["vocab"]
        most = max([e["mlp"]["router"]["experts"] for e in cfg["layers"] if e.get("mlp") and e["mlp"]["kind"] == "moe"] or [0])
        chan = list(range(W - most, W))
        shape = {s.name: tuple(s.shape) for s in specs}

        def drawn(name, scale, mean=0.0):
            g = torch.Generator().manual_seed(seed * 104729 + zlib.crc32(name.encode()) % 100003)
            return mean + scale * torch.randn(shape[name], generator=g)
        emb, pos = drawn("embed", std), drawn("pos", std)
        for j, c in enumerate(chan):                      # channel j of token t holds ((t + j) mod most) / 4: exact in bfloat16
            emb[:, c] = ((torch.arange(V) + j) % most).float() * 0.25
            pos[:, c] = 0.0
        over["embed"], over["pos"] = emb, pos
        for name in shape:
            parts = name.split(".")
            if len(parts) == 2 and parts[1] in ("norm1", "norm2"):
                over[name] = drawn(name, 0.1, 1.0)
                over[name][chan] = 0.0
            elif name.endswith("mlp.router"):
                r = drawn(name, 0.004)
                for e in range(r.shape[0]):
                    r[e, chan[(e + int(parts[0][1:])) % most]] = 8.0
                over[name] = r
            elif name.endswith("mlp.router.b"):
                over[name] = drawn(name, 0.2)
    return write_random_model(folder, cfg, seed, std=std, norm_init="perturbed", dtype=dtype, overrides=over)


class Oracle:
    """The plain model on a folder, float64."""

    def __init__(self, folder: str):
        self.cfg = plain.read_config(folder)
        self.w = plain.read_weights(folder, torch.float64)
        self._memo: Dict[Tuple[int, ...], torch.Tensor] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.w, tokens)
        return self._memo[key]

    def rounding(self, tokens: Sequence[int], dtype: str = "float32") -> np.ndarray:
        """What reduced precision alone does to each position's logits, as a part of the logits' range.  float32: the
        plain model in float32 against itself in float64, the largest of three draws (the weights as they are, and
        twice with every element moved by up to 2^-23 of itself, so that the roundings fall otherwise): one draw of
        an ill-conditioned position's error may be small by chance.  bfloat16: the plain model with every matrix and
        table moved by up to 2^-8 of each element (as much as rounding its operands to bfloat16 moves a product)
        against itself.  Where a memory's read-out is small beside its terms, a norm divides by little or a gate sits
        on its steep part, a position is ill-conditioned, and no order of summation is exact there."""
        key = (dtype,) + tuple(tokens)
        if key not in self._memo:
            want = self.logits(tokens)
            g = torch.Generator().manual_seed(99)

            def moved(by, to):
                return {k: (v * (1.0 + by * (2.0 * torch.rand(v.shape, generator=g, dtype=v.dtype) - 1.0))).to(to)
                        if v.is_floating_point() and (v.dim() == 2 or to == torch.float32) else v for k, v in self.w.items()}
            if dtype == "float32":
                draws = [plain.forward(self.cfg, moved(by, torch.float32), tokens).double() for by in (0.0, 2.0 ** -23, 2.0 ** -23)]
            else:
                draws = [plain.forward(self.cfg, moved(2.0 ** -8, torch.float64), tokens)]
            err = torch.stack([(got - want).abs().amax(-1) for got in draws]).amax(0)
            self._memo[key] = (err / float(want.max() - want.min())).numpy()
        return self._memo[key]

    def close_calls(self, tokens: Sequence[int], least: float = 0.02) -> np.ndarray:
        """Positions at which some router's choice hangs on less than ``least`` of its logits' spread: reduced
        precision may choose otherwise there, and nothing can be asked of such a position's logits."""
        key = ("margin",) + tuple(tokens)
        if key not in self._memo:
            m: list = []
            plain.forward(self.cfg, self.w, tokens, margins=m)
            self._memo[key] = torch.stack(m).amin(0).numpy() if m else np.full(len(tokens), np.inf)
        return self._memo[key] < least

    def greedy(self, tokens: Sequence[int], n: int):
        toks, out = list(tokens), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(toks)[-1]))
            out.append(t)
            toks.append(t)
        return out
