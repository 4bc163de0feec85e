"""Nelosun (``"architecture": "Nelosun"``) as a plan of parts.

A decoder-only model.  The embedding's rows are multiplied by ``embedding.scale``.  Every layer is parallel: one RMS
norm, and the mixer and the feed-forward both read its output; each result is multiplied column by column by a
stored vector (layer scale) before both are added to the stream.  A layer's mixer is one of

* ``attention``: grouped-query attention without rotation, with biases on all four projections, a query temperature
  (the query at position p times ``1 + coef * ln(floor((p + 1) / every) + 1)``), a free ``scale``, a sink of score
  zero in the softmax's denominator (``p_j = exp(s_j) / (1 + sum exp(s))``) and a sigmoid gate per head;
* ``latent_attention``: queries through a normed latent, keys and values expanded from a normed latent that is all the
  cache keeps, beside one rotated key part that the heads share (rotate-half pairs over ``rot.dims`` elements,
  frequencies ``rot.base^(-2i / dims)``);
* ``rglru``: a recurrent block around the real-gated linear recurrent unit behind a short causal convolution.

Its feed-forward is a mixture of gated experts with clamped activations, chosen not by a router but by a stored table
over the token ids (``top`` experts a token, each with weight ``1 / top``), or absent.  ``loop`` = {start, stop, times}
runs layers start .. stop-1 that many times in a row with the same weights, every pass with caches and states of its
own, and right before the first layer of every pass the stream becomes ``W_in [x; x0]`` with x0 the embedding's output.
The model ends on an RMS norm and the embedding table as the head.  Everything here is data handed to parameterised
parts.

config.json keys: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``loop{start stop times}`` and
``layers[i] = {type, mixer, mlp}`` with ``mixer`` = ``{heads kv_heads dim vdim scale q_temp{coef every}}`` |
``{heads dim rot_dim vdim kv_rank q_rank scale rot{base dims}}`` | ``{width blocks conv}`` and ``mlp`` = null |
``{kind: moe, expert{ff limit}, router{experts top}}``.
Tensors: ``embed``, ``loop.in``, ``l<i>.norm1 ls1 ls2``, ``l<i>.mix.{q,k,v,o}(.b) g`` | ``l<i>.mix.{dq, dq.norm, uq, dkv,
dkv.norm, uk, uv, o}`` | ``l<i>.mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}``, ``l<i>.mlp.{e<j>.gate, e<j>.up,
e<j>.down, table}``, ``final.norm``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model import Architecture, ConfigError, register_architecture, require_int
from ..parts import (GQAttention, LatentAttention, OutputHead, ParallelBlock, RGLRUMixer, RMSNorm, ScaledRotaryEncoding,
                     SparseMoE, StreamInjection, TokenEmbedding)
from .plan import LayerCall, ModelPlan

#: positions are counted in float32, which holds integers exactly up to here
MAX_POSITIONS = 1 << 24
#: log a = -DECAY_C * r * softplus(lam)
DECAY_C = 8.0
#: an expert's gate passes g * sigmoid(GATE_ALPHA * g), and its up branch is shifted by UP_SHIFT before the product
GATE_ALPHA = 1.702
UP_SHIFT = 1.0
#: the score of the sink that joins every softmax's denominator
SINK_SCORE = 0.0

MIXER_TYPES = ("attention", "latent_attention", "rglru")


def _num(v: Any, key: str, where: str) -> float:
    x = v.get(key) if isinstance(v, dict) else None
    if isinstance(x, bool) or not isinstance(x, (int, float)):
        raise ConfigError(f"config.json: {where} needs the number `{key}`")
    return float(x)


def _int(v: Any, key: str, where: str, least: int = 1) -> int:
    x = v.get(key) if isinstance(v, dict) else None
    if isinstance(x, bool) or not isinstance(x, int) or x < least:
        raise ConfigError(f"config.json: {where} needs the integer `{key}` >= {least}")
    return int(x)


@dataclass(frozen=True)
class NelosunLayer:
    kind: str                                    # attention | latent_attention | rglru
    mixer: Tuple[Tuple[str, Any], ...]           # the mixer's sizes and constants, as sorted items
    mlp: Optional[Tuple[Tuple[str, Any], ...]]   # None: no feed-forward


@dataclass(frozen=True)
class NelosunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    loop: Optional[Tuple[int, int, int]]         # (start, stop, times); None: every layer runs once
    layers: Tuple[NelosunLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_json(cls, v: Dict[str, Any]) -> "NelosunConfig":
        norm = v.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: missing `norm`")
        raw = v.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = []
        for i, e in enumerate(raw):
            where = f"layer {i}"
            if not isinstance(e, dict) or e.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}: type must be one of {', '.join(MIXER_TYPES)}")
            kind, mx = e["type"], e.get("mixer")
            if not isinstance(mx, dict):
                raise ConfigError(f"config.json: {where} needs `mixer`")
            m: Dict[str, Any] = {}
            if kind == "attention":
                m = {k: _int(mx, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {where}: {m['heads']} heads over {m['kv_heads']} kv heads")
                m["scale"] = _num(mx, "scale", where)
                qt = mx.get("q_temp")
                if qt is not None:
                    m["q_temp"] = (_num(qt, "coef", where + " q_temp"), _int(qt, "every", where + " q_temp"))
            elif kind == "latent_attention":
                m = {k: _int(mx, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
                m["scale"] = _num(mx, "scale", where)
                rot = mx.get("rot")
                m["rot_base"] = _num(rot, "base", where + " rot")
                m["rot_dims"] = _int(rot, "dims", where + " rot")
                if m["rot_dims"] % 2 or m["rot_dims"] > m["rot_dim"]:
                    raise ConfigError(f"config.json: {where}: {m['rot_dims']} rotated elements of a part of {m['rot_dim']}")
            else:
                m = {k: _int(mx, k, where) for k in ("width", "blocks", "conv")}
                if m["width"] % m["blocks"]:
                    raise ConfigError(f"config.json: {where}: {m['width']} channels in {m['blocks']} parts")
            mlp = e.get("mlp")
            f: Optional[Dict[str, Any]] = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {where}: the feed-forward kind must be `moe`")
                f = {"ff": _int(mlp.get("expert"), "ff", where + " mlp.expert"),
                     "limit": _num(mlp.get("expert"), "limit", where + " mlp.expert"),
                     "experts": _int(mlp.get("router"), "experts", where + " mlp.router"),
                     "top": _int(mlp.get("router"), "top", where + " mlp.router")}
                if f["top"] > f["experts"] or f["limit"] <= 0:
                    raise ConfigError(f"config.json: {where}: top {f['top']} of {f['experts']} experts, limit {f['limit']}")
            layers.append(NelosunLayer(kind, tuple(sorted(m.items())), tuple(sorted(f.items())) if f is not None else None))
        loop = None
        lp = v.get("loop")
        if lp is not None:
            a, b, t = _int(lp, "start", "loop", 0), _int(lp, "stop", "loop"), _int(lp, "times", "loop")
            if not a < b <= len(layers):
                raise ConfigError(f"config.json: loop from {a} to {b} over {len(layers)} layers")
            loop = (a, b, t)
        emb = v.get("embedding")
        scale = _num(emb, "scale", "embedding") if isinstance(emb, dict) and emb.get("scale") is not None else 1.0
        eos = v.get("eos_token_id")
        eos_ids = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos if isinstance(x, int)) if isinstance(eos, list) else ()
        return cls(vocab=require_int(v, "vocab"), width=require_int(v, "width"), norm_eps=_num(norm, "eps", "norm"),
                   embedding_scale=scale, loop=loop, layers=tuple(layers), eos_token_ids=tuple(sorted(set(eos_ids))))


def run_order(n_layers: int, loop: Optional[Tuple[int, int, int]], inject: str) -> List[LayerCall]:
    """Every layer once, but those of the loop ``times`` times in a row, each pass led by the stream part."""
    if loop is None:
        return [LayerCall(i) for i in range(n_layers)]
    a, b, times = loop
    order = [LayerCall(i) for i in range(a)]
    for _ in range(times):
        order += [LayerCall(i, before=inject if i == a else None) for i in range(a, b)]
    return order + [LayerCall(i) for i in range(b, n_layers)]


def nelosun_plan(cfg: NelosunConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    emb = TokenEmbedding(cfg.vocab, W, "embed", scale=cfg.embedding_scale)
    layers, prefixes = [], []
    ropes: Dict[Any, ScaledRotaryEncoding] = {}
    for i, layer in enumerate(cfg.layers):
        m = dict(layer.mixer)
        if layer.kind == "attention":
            mixer = GQAttention(W, m["heads"], m["kv_heads"], m["dim"], qk_norm_eps=None, pos=None, scale=m["scale"],
                                v_head_dim=m["vdim"], bias=True, bias_suffix=".b", weight_suffix="", head_gate=True,
                                fixed_sink=SINK_SCORE, q_temp=m.get("q_temp"),
                                names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g"})
        elif layer.kind == "latent_attention":
            key = (m["rot_dims"], m["rot_base"])
            if key not in ropes:          # layers that agree share one pair of tables
                ropes[key] = ScaledRotaryEncoding(m["rot_dims"], m["rot_base"], None, name=f"rope{len(ropes)}")
            mixer = LatentAttention(W, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"],
                                    scale=m["scale"], norm_eps=eps, pos=ropes[key].name, rot=m["rot_dims"], weight_suffix="",
                                    names={"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                                           "uk": "uk", "uv": "uv", "o": "o"})
        else:
            mixer = RGLRUMixer(W, m["width"], m["blocks"], m["conv"], decay_c=DECAY_C, weight_suffix="", bias_suffix=".b",
                               names={"y": "y", "x": "x", "conv": "conv", "a": "ra", "i": "ri", "lam": "lam", "o": "o"})
        ffn = None
        if layer.mlp is not None:
            f = dict(layer.mlp)
            ffn = SparseMoE(W, f["ff"], f["experts"], f["top"], gated=True, route="table", vocab=cfg.vocab,
                            act=(f["limit"], GATE_ALPHA, UP_SHIFT), weight_suffix="",
                            names={"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "table": "table"})
        layers.append(ParallelBlock(RMSNorm(W, eps, "norm1"), mixer, ffn, {"mixer": "mix.", "ffn": "mlp."},
                                    scales=("ls1", "ls2"), hidden=W))
        prefixes.append(f"l{i}.")
    stream_parts = {"loop_in": StreamInjection(W, "loop.in")} if cfg.loop is not None else {}
    return ModelPlan(
        architecture="Nelosun", vocab_size=cfg.vocab, hidden_size=W, max_positions=MAX_POSITIONS, embedding=emb,
        layers=layers, layer_prefixes=prefixes, order=run_order(len(layers), cfg.loop, "loop_in"),
        final_norm=RMSNorm(W, eps, "norm"), final_norm_prefix="final.",
        head=OutputHead(cfg.vocab, W, True, emb, "head"),
        position_encodings=list(ropes.values()), eos_token_ids=cfg.eos_token_ids, config=cfg, stream_parts=stream_parts)


register_architecture(Architecture(name="Nelosun", model_types=("nelosun",), parse=NelosunConfig.from_json, plan=nelosun_plan))
