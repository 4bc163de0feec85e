"""Demazen (``"architecture": "Demazen"``) as a plan of parts.

A decoder-only model.  The embedding adds a learned position vector (row p of a table).  A layer's sublayers read
the residual stream as it is, without a norm in front, and what they return is RMS-normed on its way into the
stream: ``x <- x + norm1(mixer(x))``, ``x <- x + norm2(ff(x))``.  A layer's mixer is either the matrix memory of the
xLSTM (``type`` ``mlstm``) or two mixers side by side on the same input, each RMS-normed over the width and the two
averaged (``type`` ``parallel``): grouped-query attention without rotation over a sliding window, with q and k
normed over their whole projections (``left``), and gated linear attention with a low-rank decay (``right``).  Its
feed-forward is a dense SwiGLU, a mixture of SwiGLU experts whose weights are the softmax over the chosen logits,
or absent.  A layer may run another layer's weights with a state and cache of its own (``weights_of``).  The
model ends on an RMS norm, the embedding table as the head, and ``cap * tanh(logits / cap)``.  Everything here is
data handed to parameterised parts.

config.json keys: ``vocab``, ``width``, ``max_positions``, ``norm.eps``, ``logit_softcap`` and ``layers[i] = {type,
weights_of?, mixer, mlp}`` with ``mixer = {heads dim vdim gate_cap}`` (mlstm) or ``{left: {heads kv_heads dim vdim
scale mask{size}}, right: {heads dim vdim tau}}`` (parallel) and ``mlp = null | {kind: dense, ff} | {kind: moe,
expert{ff}, router{experts top}}``.  ``right.rank`` may name the width of the decay's low-rank pair; a checkpoint's
shapes give it otherwise.
Tensors: ``embed``, ``pos``, ``l<i>.norm1 norm2``, ``l<i>.mix.{q,k,v,g,o,norm,i,i.b,f,f.b}`` or
``l<i>.mix.left.{q,k,v,o,q.norm,k.norm,out}`` and ``l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b,out}``,
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{e<j>.gate, e<j>.up, e<j>.down, router, router.b}``, ``final.norm``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..config.model import Architecture, ConfigError, register_architecture, require_int
from ..parts import (GatedLinearAttentionMixer, GQAttention, MatrixMemoryMixer, NoNorm, OutputHead, ParallelMixer, RMSNorm,
                     SandwichBlock, SparseMoE, SwiGLU, TokenEmbedding)
from .plan import LayerCall, ModelPlan

#: added to the denominator of the matrix memory's read-out
MEMORY_FLOOR_EPS = 1e-6


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


Items = Tuple[Tuple[str, Any], ...]


@dataclass(frozen=True)
class DemazenLayer:
    kind: str                               # "mlstm" | "parallel"
    mixer: Items                            # mlstm: the memory's sizes and cap; parallel: unused
    left: Optional[Items]                   # parallel: the attention's sizes and constants
    right: Optional[Items]                  # parallel: the linear attention's
    mlp: Optional[Items]                    # None: no feed-forward
    weights_of: Optional[int]               # None: tensors of its own


@dataclass(frozen=True)
class DemazenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[DemazenLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_json(cls, v: Dict[str, Any]) -> "DemazenConfig":
        norm = v.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: missing `norm`")
        raw = v.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = []
        for i, e in enumerate(raw):
            where = f"layer {i}"
            if not isinstance(e, dict) or e.get("type") not in ("mlstm", "parallel"):
                raise ConfigError(f"config.json: {where}: type must be `mlstm` or `parallel`")
            mx = e.get("mixer")
            mixer: Dict[str, Any] = {}
            left = right = None
            if e["type"] == "mlstm":
                mixer = {k: _int(mx, k, where) for k in ("heads", "dim", "vdim")}
                mixer["gate_cap"] = _num(mx, "gate_cap", where)
                if not mixer["gate_cap"] > 0:
                    raise ConfigError(f"config.json: {where}: gate_cap must be positive")
            else:
                if not isinstance(mx, dict) or not isinstance(mx.get("left"), dict) or not isinstance(mx.get("right"), dict):
                    raise ConfigError(f"config.json: {where} needs `mixer.left` and `mixer.right`")
                le, ri = mx["left"], mx["right"]
                left = {k: _int(le, k, where + " left") for k in ("heads", "kv_heads", "dim", "vdim")}
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config.json: {where}: {left['heads']} heads over {left['kv_heads']} kv heads")
                left["scale"] = _num(le, "scale", where + " left")
                mask = le.get("mask")
                left["window"] = _int(mask, "size", where + " mask") if isinstance(mask, dict) and mask.get("size") is not None else 0
                right = {k: _int(ri, k, where + " right") for k in ("heads", "dim", "vdim")}
                right["tau"] = _num(ri, "tau", where + " right")
                if not right["tau"] > 0:
                    raise ConfigError(f"config.json: {where}: tau must be positive")
                right["rank"] = _int(ri, "rank", where + " right") if ri.get("rank") is not None else None
            mlp = e.get("mlp")
            m: Optional[Dict[str, Any]] = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {where}: the feed-forward kind must be `dense` or `moe`")
                m = {"kind": mlp["kind"]}
                if mlp["kind"] == "dense":
                    m["ff"] = _int(mlp, "ff", where + " mlp")
                else:
                    m["ff"] = _int(mlp.get("expert"), "ff", where + " mlp.expert")
                    m["experts"] = _int(mlp.get("router"), "experts", where + " mlp.router")
                    m["top"] = _int(mlp.get("router"), "top", where + " mlp.router")
                    if m["top"] > m["experts"]:
                        raise ConfigError(f"config.json: {where}: top {m['top']} of {m['experts']} experts")
            wo = e.get("weights_of")
            if wo is not None:
                if isinstance(wo, bool) or not isinstance(wo, int) or not 0 <= wo < len(raw) or wo == i:
                    raise ConfigError(f"config.json: {where}: `weights_of` must name another layer")
                if raw[wo].get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}: `weights_of` names a layer without tensors of its own")
            layers.append(DemazenLayer(e["type"], tuple(sorted(mixer.items())),
                                       tuple(sorted(left.items())) if left is not None else None,
                                       tuple(sorted(right.items())) if right is not None else None,
                                       tuple(sorted(m.items())) if m is not None else None, wo))
        cap = v.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap <= 0):
            raise ConfigError("config.json: `logit_softcap` must be a positive number")
        eos = v.get("eos_token_id")
        eos_ids = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos if isinstance(x, int)) if isinstance(eos, list) else ()
        return cls(vocab=require_int(v, "vocab"), width=require_int(v, "width"), max_positions=_int(v, "max_positions", "the model"),
                   norm_eps=_num(norm, "eps", "norm"), logit_softcap=float(cap) if cap is not None else None,
                   layers=tuple(layers), eos_token_ids=tuple(sorted(set(eos_ids))))


def _block(cfg: DemazenConfig, layer: DemazenLayer) -> SandwichBlock:
    W, eps = cfg.width, cfg.norm_eps
    if layer.kind == "mlstm":
        m = dict(layer.mixer)
        mixer = MatrixMemoryMixer(W, m["heads"], m["dim"], m["vdim"], m["gate_cap"], eps, floor_eps=MEMORY_FLOOR_EPS,
                                  weight_suffix="", bias_suffix=".b",
                                  names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "i": "i", "f": "f", "norm": "norm"})
    else:
        le, ri = dict(layer.left), dict(layer.right)
        attn = GQAttention(W, le["heads"], le["kv_heads"], le["dim"], qk_norm_eps=eps, qk_norm="projection", pos=None,
                           scale=le["scale"], v_head_dim=le["vdim"], window=le["window"], weight_suffix="",
                           names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"})
        gla = GatedLinearAttentionMixer(W, ri["heads"], ri["dim"], ri["vdim"], ri["tau"], eps, weight_suffix="", bias_suffix=".b",
                                        names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a1": "a1", "a2": "a2",
                                               "norm": "norm"})
        if ri["rank"] is not None:
            gla.with_rank(ri["rank"])
        # (the two branch norms and their mean ride on the kernel that norms the mixer's output into the stream)
        mixer = ParallelMixer(W, [("left.", attn), ("right.", gla)], eps, norm_name="out", deferred=True)
    ffn = ffn_norm = ffn_post = None
    if layer.mlp is not None:
        m = dict(layer.mlp)
        ffn_norm, ffn_post = NoNorm(W), RMSNorm(W, eps, "norm2")
        if m["kind"] == "dense":
            ffn = SwiGLU(W, m["ff"], {"gate": "gate", "up": "up", "down": "down"}, weight_suffix="")
        else:
            ffn = SparseMoE(W, m["ff"], m["experts"], m["top"], weight_suffix="", gated=True, router_bias=True, score="chosen",
                            names={"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "router": "router",
                                   "router_bias": "router.b"})
    return SandwichBlock(NoNorm(W), mixer, RMSNorm(W, eps, "norm1"), ffn_norm, ffn, ffn_post,
                         {"mixer": "mix.", "ffn": "mlp."})


def demazen_plan(cfg: DemazenConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    emb = TokenEmbedding(cfg.vocab, W, "embed", position_table="pos", positions=cfg.max_positions)
    layers, prefixes, index_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is None:
            index_of[i] = len(layers)
            layers.append(_block(cfg, layer))
            prefixes.append(f"l{i}.")
    # a layer that names another layer's weights runs that block again, with a cache and a state of its own
    order = [LayerCall(index_of[i if layer.weights_of is None else layer.weights_of]) for i, layer in enumerate(cfg.layers)]
    return ModelPlan(
        architecture="Demazen", vocab_size=cfg.vocab, hidden_size=W, max_positions=cfg.max_positions, embedding=emb,
        layers=layers, layer_prefixes=prefixes, order=order,
        final_norm=RMSNorm(W, eps, "norm"), final_norm_prefix="final.",
        head=OutputHead(cfg.vocab, W, True, emb, softcap=cfg.logit_softcap),
        position_encodings=[], eos_token_ids=cfg.eos_token_ids, config=cfg)


register_architecture(Architecture(name="Demazen", model_types=("demazen",), parse=DemazenConfig.from_json, plan=demazen_plan))
