"""Demazen through the framework's own step function, cache manager, scheduler and kernels, against the plain
model of ``plain_demazen.py``.  Model-level cases run twice: on the host with plain Python standing in for the
kernels (what is under test there is the plan, the parts' wiring, layers that run another layer's weights, the cache
manager and the packer), and on a GPU with the kernels themselves.  Kernel-level cases compare each new kernel with
its restatement in ``plain_ops.py`` at sizes of their own, or with a value that is known by construction."""
import math

import numpy as np
import pytest
import torch

import demazen_util as du
import plain_demazen as plain
import plain_ops
import vukavik_util as vu           # the schedule runner and the error measures are not tied to a model


@pytest.fixture()
def kernels(request, monkeypatch):
    """On the host the plain restatements stand in for the kernels; on a GPU nothing is replaced."""
    def use(device):
        if device == "cpu":
            from vapi_b200 import ops
            for name in plain_ops.ALL:
                monkeypatch.setattr(ops, name, getattr(plain_ops, name))
    return use


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg, seed in [("mixed", du.MIXED, 1), ("tiny", du.TINY, 2), ("serving_heads", du.SERVING_HEADS, 3), ("odd", du.ODD, 4)] + \
            [(k, v, 10 + i) for i, (k, v) in enumerate(du.ONE.items())]:
        out[name] = du.write_model(str(tmp_path_factory.mktemp(name)), cfg, seed)
        out[name + "/bf16"] = du.write_model(str(tmp_path_factory.mktemp(name + "bf16")), cfg, seed, torch.bfloat16, std=0.05,
                                             planted_routes=True)
    return out


def _judge(e, slack, dtype, what):
    """``e``: errors as parts of the logit range; ``slack``: what reduced precision alone does to the plain model at
    the same positions.  An error counts as far as it exceeds three times that."""
    e, slack = np.asarray(e, dtype=np.float64), np.asarray(slack, dtype=np.float64)
    assert np.isfinite(e).all(), what
    if dtype == "bfloat16":
        ex = np.maximum(0.0, e - 3.0 * slack)
        assert ex.mean() <= 0.02 and np.percentile(ex, 95) <= vu.limit(dtype) and ex.max() <= 0.15, \
            f"{what}: mean {ex.mean():.3e}, 95th percentile {np.percentile(ex, 95):.3e}, worst {ex.max():.3e} at {int(ex.argmax())}"
    else:
        over = e - np.maximum(vu.limit(dtype), 3.0 * slack)
        pos = int(over.argmax())
        assert over[pos] <= 0, f"{what}: {e[pos]:.3e} of the logit range at {pos} of {len(e)}"


def _check(runner, oracle, requests, schedule, dtype):
    got = vu.run_schedule(runner, requests, schedule)
    for rid, toks in requests.items():
        want = oracle.logits(toks)
        e = np.abs(got[rid] - want.numpy()).max(-1) / float(want.max() - want.min())
        _judge(e, oracle.rounding(toks, dtype), dtype, f"request {rid}")


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.isfinite(a).all()
    assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max())), f"{float((a - b).abs().max()):.3e}"


def _step_meta(lens, starts, slots, device):
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    pos = torch.cat([torch.arange(s, s + q, dtype=torch.int32) for s, q in zip(starts, lens)])
    return cu.to(device), pos.to(device), torch.tensor(slots, dtype=torch.int32).to(device)


# ---- configuration and registry --------------------------------------------------------------------------
def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_configuration():
    from vapi_b200.config.model import ConfigError, resolve_architecture
    from vapi_b200.parts import GatedLinearAttentionMixer, GQAttention, MatrixMemoryMixer
    arch = resolve_architecture(du.MIXED)
    assert arch.name == "Demazen"
    cfg = arch.parse(du.MIXED)
    plan = arch.plan(cfg)
    shapes = {s.name: tuple(s.shape) for s in plan.tensor_specs()}
    assert shapes["embed"] == (200, 64) and shapes["pos"] == (512, 64) and shapes["final.norm"] == (64,)
    assert "head" not in shapes, "the embedding table is the head"
    assert shapes["l0.mix.q"] == (32, 64) and shapes["l0.mix.v"] == (48, 64) and shapes["l0.mix.g"] == (48, 64)
    assert shapes["l0.mix.o"] == (64, 48) and shapes["l0.mix.norm"] == (48,) and shapes["l0.mix.i"] == (2, 64)
    assert shapes["l0.mix.f.b"] == (2,) and shapes["l0.norm1"] == (64,) and shapes["l0.mlp.down"] == (64, 96)
    assert shapes["l1.mix.left.q"] == (64, 64) and shapes["l1.mix.left.k"] == (32, 64) and shapes["l1.mix.left.v"] == (48, 64)
    assert shapes["l1.mix.left.q.norm"] == (64,) and shapes["l1.mix.left.k.norm"] == (32,), "one weight over the whole projection"
    assert shapes["l1.mix.left.o"] == (64, 96) and shapes["l1.mix.left.out"] == (64,) and shapes["l1.mix.right.out"] == (64,)
    assert shapes["l1.mix.right.a1"] == (8, 64) and shapes["l1.mix.right.a2"] == (32, 8) and shapes["l1.mix.right.a2.b"] == (32,)
    assert shapes["l1.mix.right.norm"] == (16,), "one weight of the value size, shared by the heads"
    assert shapes["l1.mlp.router"] == (6, 64) and shapes["l1.mlp.router.b"] == (6,) and shapes["l1.mlp.e5.gate"] == (40, 64)
    assert "l2.norm2" not in shapes and not any(k.startswith("l2.mlp") for k in shapes), "a layer without a feed-forward"
    assert shapes["l3.mix.q"] == (40, 64) and shapes["l3.mlp.e4.down"] == (64, 24)
    assert not any(k.startswith(("l4.", "l5.")) for k in shapes), "a layer that names another layer's weights has no tensors"
    # six layer runs over four blocks, each run with a cache or a state of its own
    assert [c.layer for c in plan.order] == [0, 1, 2, 3, 1, 0] and len(plan.layers) == 4
    sites = plan.cache_sites()
    kinds = [type(s).__name__ for _, s in sites]
    assert kinds.count("PagedSpec") == 3 and kinds.count("StateSpec") == 6 and len({site for site, _ in sites}) == 9
    members = [type(m) for blk in plan.layers for m in blk.mixer.members()]
    assert members == [MatrixMemoryMixer, GQAttention, GatedLinearAttentionMixer, GQAttention, GatedLinearAttentionMixer, MatrixMemoryMixer]
    att = plan.layers[2].mixer.members()[0]
    assert (att.nh, att.nkv, att.d, att.dv, att.window, att.scale) == (3, 3, 24, 16, 33, 0.3)
    assert plan.layers[0].mixer.cap == 8.0 and plan.layers[3].mixer.cap == 15.0 and plan.layers[2].mixer.members()[1].tau == 4.0
    odd = arch.plan(arch.parse(du.ODD))
    assert odd.layers[2].mixer.members()[0].window == 0 and odd.head.softcap is None
    # without `rank` the decay's pair takes the size that the checkpoint's shapes give
    free = du.config([du.parallel(du.left(), {k: v for k, v in du.right().items() if k != "rank"}, None)])
    assert {s.name: tuple(s.shape) for s in arch.plan(arch.parse(free)).tensor_specs()}["l0.mix.right.a1"][0] == -1
    lay = du.MIXED["layers"]
    for bad in ({**du.MIXED, "layers": [{"type": "attention", "mixer": {}, "mlp": None}]},
                {**du.MIXED, "layers": [du.mlstm(du.memory(), {"kind": "sparse", "ff": 8})]},
                {**du.MIXED, "layers": [du.mlstm(du.memory(gate_cap=0.0), None)]},
                {**du.MIXED, "layers": [du.parallel(du.left(heads=3, kv_heads=2), du.right(), None)]},
                {**du.MIXED, "layers": [du.parallel(du.left(), du.right(tau=0.0), None)]},
                {**du.MIXED, "layers": [du.mlstm(du.memory(), du.moe(experts=2, top=3))]},
                {**du.MIXED, "layers": [lay[0], du.mlstm(du.memory(), du.dense(), weights_of=1)]},
                {**du.MIXED, "layers": [lay[0], du.mlstm(du.memory(), du.dense(), weights_of=0), du.mlstm(du.memory(), du.dense(), weights_of=1)]},
                {k: v for k, v in du.MIXED.items() if k != "norm"},
                {k: v for k, v in du.MIXED.items() if k != "max_positions"}):
        with pytest.raises(ConfigError):
            arch.parse(bad)


# ---- the plain model itself ----------------------------------------------------------------------------
def test_the_plain_model_is_causal_and_its_recurrences_run_by_hand():
    from vapi_b200.config.model import resolve_architecture
    cfg = du.TINY
    arch = resolve_architecture(cfg)
    g = torch.Generator().manual_seed(0)
    w = {s.name: torch.randn(s.shape, generator=g, dtype=torch.float64) * 0.3 for s in arch.plan(arch.parse(cfg)).tensor_specs()}
    toks = vu.prompt(cfg, 25, 0)
    a, b = plain.forward(cfg, w, toks), plain.forward(cfg, w, toks[:13])
    assert torch.allclose(a[:13], b, atol=1e-12)
    # the matrix memory, one head of 1 x 1, two tokens, identity-like weights: gates, running maximum and read-out by hand
    one = {"q": torch.tensor([[1.0]]), "k": torch.tensor([[1.0]]), "v": torch.tensor([[2.0]]), "g": torch.tensor([[0.0]]),
           "o": torch.tensor([[1.0]]), "norm": torch.tensor([1.0]), "i": torch.tensor([[1.0]]), "i.b": torch.tensor([0.5]),
           "f": torch.tensor([[0.0]]), "f.b": torch.tensor([3.0])}
    one = {"m." + k: v.double() for k, v in one.items()}
    cap = 4.0
    x = torch.tensor([[1.0], [-2.0]], dtype=torch.float64)
    got = plain.mlstm(one, "m.", {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": cap}, x, 0.0)
    li = [cap * math.tanh((xi + 0.5) / cap) for xi in (1.0, -2.0)]
    lf = -math.log1p(math.exp(-cap * math.tanh(3.0 / cap)))
    m1 = max(lf + 0.0, li[0])
    S1 = math.exp(li[0] - m1) * 1.0 * 2.0
    n1 = math.exp(li[0] - m1) * 1.0
    o1 = S1 * 1.0 / (max(abs(n1 * 1.0), math.exp(-m1)) + 1e-6)
    m2 = max(lf + m1, li[1])
    S2 = math.exp(lf + m1 - m2) * S1 + math.exp(li[1] - m2) * (-2.0) * (-4.0)
    n2 = math.exp(lf + m1 - m2) * n1 + math.exp(li[1] - m2) * (-2.0)
    o2 = S2 * (-2.0) / (max(abs(n2 * -2.0), math.exp(-m2)) + 1e-6)
    # a head of one channel divided by its root mean square is its sign; the output gate is sigmoid(0)
    want = [0.5 * math.copysign(1.0, o) for o in (o1, o2)]
    assert got.reshape(-1).tolist() == pytest.approx(want, abs=1e-9)
    # gated linear attention, one head of 1 x 1: S2 = alpha2 S1 + k2 v2, alpha = sigmoid(z)^(1/tau)
    lin = {"q": [[1.0]], "k": [[1.0]], "v": [[3.0]], "g": [[1.0]], "o": [[1.0]], "norm": [2.0], "a1": [[1.0]], "a2": [[0.5]], "a2.b": [0.25]}
    lin = {"r." + k: torch.tensor(v, dtype=torch.float64) for k, v in lin.items()}
    got = plain.gated_linear_attention(lin, "r.", {"heads": 1, "dim": 1, "vdim": 1, "tau": 2.0}, x, 0.0)
    alpha2 = (1.0 / (1.0 + math.exp(-(0.5 * -2.0 + 0.25)))) ** 0.5
    s1 = 1.0 * 3.0
    s2 = alpha2 * s1 + (-2.0) * (-6.0)
    silu = lambda z: z / (1.0 + math.exp(-z))
    want = [math.copysign(2.0, s1 * 1.0) * silu(1.0), math.copysign(2.0, s2 * -2.0) * silu(-2.0)]
    assert got.reshape(-1).tolist() == pytest.approx(want, abs=1e-9)
    # the window: with a mask of one token every position sees itself alone, so the mixer is W_o W_v on each token
    g = torch.Generator().manual_seed(3)
    att = {"a." + k: torch.randn(sh, generator=g, dtype=torch.float64) for k, sh in
           (("q", (4, 5)), ("k", (4, 5)), ("v", (6, 5)), ("o", (5, 6)), ("q.norm", (4,)), ("k.norm", (4,)))}
    h = torch.randn((7, 5), generator=g, dtype=torch.float64)
    got = plain.window_attention(att, "a.", {"heads": 2, "kv_heads": 2, "dim": 2, "vdim": 3, "scale": 0.3, "mask": {"size": 1}}, h, 1e-5)
    assert torch.allclose(got, h @ att["a.v"].T @ att["a.o"].T, atol=1e-12)
    # the experts: all chosen, a router of zeros and no bias give the mean of all experts
    ex = {"e.router": torch.zeros((3, 5), dtype=torch.float64), "e.router.b": torch.zeros(3, dtype=torch.float64)}
    for j in range(3):
        ex.update({f"e.e{j}.gate": torch.randn((4, 5), generator=g, dtype=torch.float64), f"e.e{j}.up": torch.randn((4, 5), generator=g, dtype=torch.float64),
                   f"e.e{j}.down": torch.randn((5, 4), generator=g, dtype=torch.float64)})
    got = plain.experts(ex, "e.", {"router": {"experts": 3, "top": 3}}, h)
    assert torch.allclose(got, sum(plain.gated_ff(ex, f"e.e{j}.", h) for j in range(3)) / 3.0, atol=1e-12)


# ---- each mechanism alone: one layer of it ---------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("kind", list(du.ONE))
def test_one_layer_of_each_mechanism(kind, folders, kernels):
    kernels("cuda")
    oracle = du.Oracle(folders[kind])
    runner = vu.make_runner(folders[kind], "float32", "cuda", num_pages=12)
    toks = vu.prompt(oracle.cfg, 150, 11)
    _check(runner, oracle, {"a": toks}, [[("a", 150)]], "float32")
    _check(runner, oracle, {"b": toks}, [[("b", q)] for q in vu.cuts(150, [37, 2, 1, 64, 3])], "float32")


# ---- prompts, decoding, portions ---------------------------------------------------------------------------
@pytest.mark.parametrize("device,name,length", [pytest.param("cpu", "tiny", 24, id="host"),
                                                pytest.param("cuda", "mixed", 140, marks=pytest.mark.gpu, id="gpu"),
                                                pytest.param("cuda", "odd", 90, marks=pytest.mark.gpu, id="gpu-odd-sizes"),
                                                pytest.param("cuda", "serving_heads", 230, marks=pytest.mark.gpu, id="gpu-wide-heads")])
def test_whole_prompt_token_by_token_and_portions_agree_with_the_plain_model(device, name, length, folders, kernels):
    kernels(device)
    oracle = du.Oracle(folders[name])
    runner = vu.make_runner(folders[name], "float32", device, num_pages=16)
    toks = vu.prompt(oracle.cfg, length, 21)
    _check(runner, oracle, {"w": toks}, [[("w", length)]], "float32")
    _check(runner, oracle, {"d": toks}, [[("d", 1)]] * length, "float32")          # the first tokens, long decoding
    for sizes in ([2], [5, 3, 2, 1, 17], [16, 1, 15, 33], [64, 7]):
        _check(runner, oracle, {"p": toks}, [[("p", q)] for q in vu.cuts(length, sizes)], "float32")


@pytest.mark.parametrize("device,name,lengths", [pytest.param("cpu", "tiny", [20, 3, 11], id="host"),
                                                 pytest.param("cuda", "mixed", [130, 9, 71, 40, 1, 100], marks=pytest.mark.gpu, id="gpu")])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(device, name, lengths, folders, kernels):
    """Portions of some requests beside single tokens of others; more requests than slots and a pool smaller than all
    of them together, so that pages and state slots that were written are handed out again (nothing clears them)."""
    kernels(device)
    oracle = du.Oracle(folders[name])
    page = 16
    runner = vu.make_runner(folders[name], "float32", device, page_size=page, max_requests=3,
                            num_pages=sum(sorted(-(-n // page) for n in lengths)[-3:]))
    reqs = {f"r{i}": vu.prompt(oracle.cfg, n, 30 + i) for i, n in enumerate(lengths)}
    rng = np.random.RandomState(5)
    waiting, live, at, schedule = list(reqs), [], {k: 0 for k in reqs}, []
    while waiting or live:
        while waiting and len(live) < 3:
            live.append(waiting.pop(0))
        step = []
        for rid in list(live):
            rest = len(reqs[rid]) - at[rid]
            if len(live) > 1 and rng.rand() < 0.25:
                continue                                    # a request may sit out a step
            q = 1 if rest <= 6 else int(min(rest - 6, rng.choice([2, 3, 16, 17, 40])))
            step.append((rid, q))
            at[rid] += q
            if at[rid] == len(reqs[rid]):
                live.remove(rid)
        if step:
            schedule.append(step)
    assert any(len(s) > 1 and {q for _, q in s} != {1} and 1 in {q for _, q in s} for s in schedule)
    _check(runner, oracle, reqs, schedule, "float32")
    # and once more on the same runner: every page and slot has been used before
    _check(runner, oracle, reqs, schedule, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("name,page", [("mixed", 16), ("serving_heads", 64), ("odd", 16)])
def test_bfloat16_serving_path(name, page, folders, kernels):
    """(`serving_heads`: keys and values of 64 and of 128 on pages of 64 tokens, the shapes that the tensor-core
    attention kernels take.)  The residual stream, the recurrences' states and the gates stay float32."""
    kernels("cuda")
    oracle = du.Oracle(folders[name + "/bf16"])
    runner = vu.make_runner(folders[name + "/bf16"], "bfloat16", "cuda", num_pages=24, max_tokens=512, page_size=page)
    n = min(280, oracle.cfg["max_positions"])
    reqs = {"a": vu.prompt(oracle.cfg, n, 41), "b": vu.prompt(oracle.cfg, 45, 42)}
    _check(runner, oracle, reqs, [[("a", n)], [("b", 45)]], "bfloat16")
    _check(runner, oracle, reqs, [[("a", n - 30), ("b", 2)], [("a", 1), ("b", 20)]] + [[("a", 1), ("b", 1)]] * 23 + [[("a", 1)]] * 6,
           "bfloat16")


# ---- the window's edges and far keys: inputs made so that one key decides -------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv,page", [(16, 8, 16), (24, 40, 16), (64, 64, 64), (128, 128, 64)])
@pytest.mark.parametrize("qlen", [1, 2, 40, 100])
def test_a_planted_key_is_seen_exactly_while_the_window_holds_it(qlen, dk, dv, page, dtype):
    """A query at p sees key j iff 0 <= p - j < window; the windows end inside pages.  One token alone is a decode
    step, more are a prompt's portion whose first queries look back into what earlier steps wrote."""
    from vapi_b200 import ops
    klen = 150
    cu = torch.tensor([0, qlen], dtype=torch.int32, device="cuda")
    kl = torch.tensor([klen], dtype=torch.int32, device="cuda")
    for window in (1, 37, 64, 0):
        edges = {0, 3, klen - 1, klen - qlen, max(klen - qlen - 1, 0)}
        if window:
            edges |= {max(p - window + d, 0) for p in (klen - qlen, klen - 1) for d in (0, 1)}     # just outside, just inside
        for j_star in sorted(edges):
            q, cache, table = du.planted_cache(klen, qlen, j_star, dk, dv, page, dtype=dtype)
            for splits in (1, 3):
                out = ops.masked_attention(q, q.stride(0), cache, page, table, cu, kl, qlen, 1, qlen, klen, 2, 1, dk, dv, 1.0,
                                           window=window, splits=splits).float().cpu()
                for i in range(qlen):
                    p = klen - qlen + i
                    seen = j_star <= p and (window == 0 or p - j_star < window)
                    assert abs(float(out[i].mean()) - (1.0 if seen else 0.0)) < 0.02, \
                        f"key {j_star}, query at {p}, window {window}, {splits} slices: {out[i].mean():.3f}, seen={seen}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv", [(16, 24), (64, 64), (136, 8)])
def test_the_memories_keep_a_token_from_far_back_across_steps(dk, dv, dtype):
    """One token among hundreds carries a key along e_0 and a marked value; every later query along e_0 must read it
    back, whether the steps between were long portions or single tokens.  Gated linear attention: with a constant
    decay a per step the read-out at distance d is a^d times the value.  The matrix memory: the marked token's input
    gate is open and every other one shut, so the normalised read-out is the marked value itself."""
    from vapi_b200 import ops
    nh, T, j_star, slots = 2, 400, 5, 3
    steps = vu.cuts(T, [7, 130, 1, 1, 64, 2])
    g = torch.Generator().manual_seed(dk)
    qkv = torch.zeros((T, 2 * nh * dk + nh * dv))
    qkv[:, 0:dk] = 0.0
    for h in range(nh):
        qkv[:, h * dk] = 1.0                                   # q = e_0 in every head
        qkv[j_star, nh * dk + h * dk] = 2.0                    # the marked key
        qkv[j_star, 2 * nh * dk + h * dv:2 * nh * dk + (h + 1) * dv] = torch.arange(1, dv + 1, dtype=torch.float32) / dv
    qkv[:, nh * dk + 1:nh * dk + dk] += 0.5 * torch.randn((T, dk - 1), generator=g)      # other keys avoid e_0
    others = torch.arange(T) != j_star
    qkv[others, 2 * nh * dk:] = torch.randn((int(others.sum()), nh * dv), generator=g)
    qkv = qkv.to(dtype).cuda()
    marked = (torch.arange(1, dv + 1, dtype=torch.float32) / dv).to(dtype).float()
    # gated linear attention
    tau, z0 = 4.0, 6.0
    a = torch.sigmoid(torch.tensor(z0, dtype=torch.float64)) ** (1.0 / tau)
    z = torch.full((T, nh * dk), z0, device="cuda")
    state = torch.randn((slots, nh * dk * dv + 5), generator=g).cuda()           # never cleared: position 0 starts fresh
    got, at = [], 0
    for n in steps:
        cu, pos, sl = _step_meta([n], [at], [1], "cuda")
        got.append(ops.gated_linear_attention(qkv[at:at + n], z[at:at + n], tau, state, sl, cu, pos, nh, dk, dv, 1.0, max_q=n))
        at += n
    got = torch.cat(got).cpu().double()
    for t in (j_star, j_star + 1, 140, 141, 142, 399):
        want = 2.0 * float(a ** (t - j_star)) * marked.double()
        for h in range(nh):
            assert torch.allclose(got[t, h * dv:(h + 1) * dv], want, rtol=2e-3, atol=1e-5), f"token {t}, head {h}"
    assert float(got[:j_star].abs().max()) < 1e-5, "before the marked token nothing lies along e_0"
    # the matrix memory
    cap = 12.0
    gates = torch.full((T, 2 * nh), -50.0)
    gates[:, nh:] = 50.0                                        # the forget gates stay open
    gates[j_star, :nh] = 50.0
    gates = gates.cuda()
    state = torch.randn((slots, nh * dk * dv + nh * dk + nh + 3), generator=g).cuda()
    got, at = [], 0
    for n in steps:
        cu, pos, sl = _step_meta([n], [at], [2], "cuda")
        got.append(ops.matrix_memory(qkv[at:at + n], gates[at:at + n], None, cap, state, sl, cu, pos, nh, dk, dv, 1.0, 1e-6, max_q=n))
        at += n
    got = torch.cat(got).cpu()
    for t in (j_star, j_star + 1, 140, 141, 142, 399):
        for h in range(nh):
            assert torch.allclose(got[t, h * dv:(h + 1) * dv], marked, rtol=1e-3, atol=1e-3), f"token {t}, head {h}"
    # the running maximum ends at the open gate's value less what the forget gates took since
    m = state[2, nh * dk * dv + nh * dk:nh * dk * dv + nh * dk + nh].cpu()
    lf = -math.log1p(math.exp(-cap * math.tanh(50.0 / cap)))
    assert torch.allclose(m, torch.full((nh,), cap * math.tanh(50.0 / cap) + (T - 1 - j_star) * lf), atol=1e-3)


# ---- the engine: scheduler, batching, sampling, entry point -----------------------------------------------------
@pytest.mark.parametrize("device,name,lens,new", [pytest.param("cpu", "tiny", [1, 9, 20], 5, id="host"),
                                                  pytest.param("cuda", "mixed", [1, 33, 150, 7, 64, 90], 24, marks=pytest.mark.gpu, id="gpu")])
def test_greedy_generation_through_the_entry_point(device, name, lens, new, folders, kernels):
    """More requests than slots, prompts cut into portions of 16 beside other requests' decoding; on a GPU pure
    decode steps run as captured graphs.  The memories' slots pass from finished requests to waiting ones."""
    kernels(device)
    from vapi_b200 import LLM, SamplingParams
    oracle = du.Oracle(folders[name])
    llm = LLM(folders[name], dtype="f32", device=device, num_blocks=40, page_size=16, max_concurrent_seqs=4,
              max_batched_tokens=64, prefill_chunk_tokens=16, max_context=256, cuda_graphs=device == "cuda")
    prompts = [vu.prompt(oracle.cfg, n, 50 + i) for i, n in enumerate(lens)]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    for p, c in zip(prompts, out):
        want = oracle.greedy(p, new)
        if c.tokens != want:                 # only a near-tie of the plain model's own logits may part them
            i = next(k for k in range(new) if c.tokens[k] != want[k])
            top = torch.topk(oracle.logits(list(p) + want[:i])[-1], 2).values
            assert float(top[0] - top[1]) < 1e-3, f"prompt of {len(p)}: token {i} differs without a tie"
    llm.runner.cache.check_invariants()


# ---- trace replay: the program a user replays a trace with ----------------------------------------------------------
def _trace(cfg):
    import replay_util as rp
    reqs = {f"r{i}": vu.prompt(cfg, n, 70 + i) for i, n in enumerate([1, 70, 40, 90, 66])}
    tr = rp.Trace()
    rp.whole(tr, "w", reqs["r1"])
    rp.tail_decode(tr, "t", reqs["r2"], tail=5)
    rp.portions(tr, "p", reqs["r3"], sizes=[2, 3, 61, 2, 1])
    mix = {f"m{k}": v for k, v in reqs.items()}
    rp.mixed(tr, mix, seed=5, decode_tail=3)
    return tr, {"w": reqs["r1"], "t": reqs["r2"], "p": reqs["r3"], **mix}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(dtype, folders, tmp_path):
    """The replay program as a child process: four state slots and a pool for the live requests only."""
    import replay_util as rp
    name = "mixed" if dtype == "float32" else "mixed/bf16"
    oracle = du.Oracle(folders[name])
    tr, tokens = _trace(oracle.cfg)
    got = rp.run_trace(folders[name], dtype, tr, str(tmp_path / "out"))
    ref = {k: oracle.logits(v).float() for k, v in tokens.items()}
    span = max(float(r.max() - r.min()) for r in ref.values())
    where = [(step, i, rid, pos) for step, rows in tr.rows.items() for i, (rid, pos) in enumerate(rows)]
    e = [np.abs(got[step][i] - ref[rid][pos].numpy()).max() / span for step, i, rid, pos in where]
    slack = [oracle.rounding(tokens[rid], dtype)[pos] for _, _, rid, pos in where]
    _judge(e, slack, dtype, "replay")


# ---- the recurrences' kernel against its restatements, at sizes that are not powers of two -----------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_memory_kernels_continue_from_their_state_and_start_fresh_at_position_zero(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(7)
    lens, starts, slots = [1, 9, 2, 70, 1], [0, 5, 0, 1, 33], [3, 0, 2, 1, 4]
    cu, pos, sl = _step_meta(lens, starts, slots, "cuda")
    n = sum(lens)
    # (65 to 128 rows: few blocks take the finer split of the rows, many the ordinary one)
    for nh, dk, dv in ((3, 20, 12), (2, 32, 48), (1, 72, 40), (1, 100, 24), (8, 128, 128), (2, 136, 8), (1, 200, 28), (5, 12, 4), (1, 1, 1),
                       (2, 64, 64)):
        cols = 2 * nh * dk + nh * dv
        qkv = torch.randn((n, cols + 9), generator=g).to(dtype)
        pre = torch.randn((n, 2 * nh), generator=g) * 3.0
        pre[:, nh:] += 2.0
        bias = torch.randn(2 * nh, generator=g)
        need = nh * dk * dv + nh * dk + nh
        state = torch.randn((6, need + 5), generator=g)
        state[:, nh * dk * dv + nh * dk:need] = torch.rand((6, nh), generator=g) * 3.0     # maxima of earlier steps
        want_state = state.clone()
        want = plain_ops.matrix_memory(qkv[:, :cols], pre, bias, 6.0, want_state, sl.cpu(), cu.cpu(), pos.cpu(), nh, dk, dv, dk ** -0.5, 1e-6)
        dstate = state.cuda()
        got = ops.matrix_memory(qkv.cuda()[:, :cols], pre.cuda(), bias.cuda(), 6.0, dstate, sl, cu, pos, nh, dk, dv, dk ** -0.5, 1e-6,
                                max_q=max(lens))
        _close(got, want, 2e-4)
        _close(dstate, want_state, 2e-4)
        assert torch.equal(dstate[5].cpu(), state[5]) and torch.equal(dstate[:, need:].cpu(), state[:, need:]), "rows of no request"
        z = torch.randn((n, nh * dk), generator=g) * 3.0
        state = torch.randn((6, nh * dk * dv + 2), generator=g)
        want_state = state.clone()
        want = plain_ops.gated_linear_attention(qkv[:, :cols], z, 3.0, want_state, sl.cpu(), cu.cpu(), pos.cpu(), nh, dk, dv, dk ** -0.5)
        dstate = state.cuda()
        got = ops.gated_linear_attention(qkv.cuda()[:, :cols], z.cuda(), 3.0, dstate, sl, cu, pos, nh, dk, dv, dk ** -0.5, max_q=max(lens))
        _close(got, want, 2e-4)
        _close(dstate, want_state, 2e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [99, 324, 2048, 4100])
def test_two_raw_branches_ride_on_the_post_norm(hidden, dtype):
    """``x += rmsnorm(mean of the two branch norms) * w`` in one kernel against its restatement: every row, selected
    rows (the stream untouched), with a following norm and with the stream's rows handed on as they are."""
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    n = 37
    x = torch.randn((n, hidden), generator=g)
    ya, yb = (torch.randn((n, hidden), generator=g) * s for s in (3.0, 0.02))
    ya, yb = ya.to(dtype), yb.to(dtype)
    wa, wb, wp, w = (torch.randn(hidden, generator=g) for _ in range(4))
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for r in (None, rows):
        for weight, copy in ((w, False), (None, True)):
            xr, xd = x.clone(), x.clone().cuda()
            want = plain_ops.postnorm_add_rmsnorm(xr, ya, wp, 1e-5, 0.7, weight, 1e-6, dtype, r, copy=copy, branches=(yb, wa, wb, 1e-4, 0.5))
            got = ops.postnorm_add_rmsnorm(xd, ya.cuda(), wp.cuda(), 1e-5, 0.7, None if weight is None else weight.cuda(), 1e-6, dtype,
                                           None if r is None else r.cuda(), copy=copy, branches=(yb.cuda(), wa.cuda(), wb.cuda(), 1e-4, 0.5))
            _close(got.float(), want.float(), tol)
            _close(xd, xr, 2e-5)
            assert (r is None) != torch.equal(xd.cpu(), x), "selected rows leave the stream as it was"
