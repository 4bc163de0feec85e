"""Nelosun through the framework's own step function, cache manager, scheduler and kernels, against the plain
model of ``plain_nelosun.py``.  Model-level cases run twice: on the host with plain Python standing in for the
kernels (what is under test there is the plan, the parts' wiring, the looped stack, the cache manager and the
packer), and on a GPU with the kernels themselves.  Kernel-level cases compare each new kernel with its restatement
in ``plain_ops.py`` at sizes of their own, or with a value that is known by construction."""
import math

import numpy as np
import pytest
import torch

import nelosun_util as nu
import plain_nelosun as plain
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
    for name, cfg, seed in [("mixed", nu.MIXED, 1), ("tiny", nu.TINY, 2), ("plain", nu.PLAIN, 3), ("serving_heads", nu.SERVING_HEADS, 4)] + \
            [(k, v, 10 + i) for i, (k, v) in enumerate(nu.ONE.items())]:
        out[name] = nu.write_model(str(tmp_path_factory.mktemp(name)), cfg, seed)
        out[name + "/bf16"] = nu.write_model(str(tmp_path_factory.mktemp(name + "bf16")), cfg, seed, torch.bfloat16, std=0.05)
    return out


def _within(e, slack, dtype, what):
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
        _within(e, oracle.rounding(toks, dtype), dtype, f"request {rid}")


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.isfinite(a).all()
    assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max())), f"{float((a - b).abs().max()):.3e}"


# ---- configuration and registry --------------------------------------------------------------------------
def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_configuration():
    from vapi_b200.config.model import ConfigError, resolve_architecture
    from vapi_b200.parts import GQAttention, LatentAttention, RGLRUMixer
    arch = resolve_architecture(nu.MIXED)
    assert arch.name == "Nelosun"
    cfg = arch.parse(nu.MIXED)
    plan = arch.plan(cfg)
    shapes = {s.name: tuple(s.shape) for s in plan.tensor_specs()}
    assert shapes["embed"] == (200, 64) and shapes["final.norm"] == (64,) and shapes["loop.in"] == (64, 128)
    assert "head" not in shapes, "the embedding table is the head"
    assert shapes["l0.mix.q"] == (64, 64) and shapes["l0.mix.k"] == (32, 64) and shapes["l0.mix.v"] == (48, 64)
    assert shapes["l0.mix.q.b"] == (64,) and shapes["l0.mix.o.b"] == (64,) and shapes["l0.mix.g"] == (4, 64)
    assert shapes["l0.mix.o"] == (64, 96) and shapes["l0.ls1"] == (64,) and shapes["l0.ls2"] == (64,)
    assert shapes["l0.mlp.table"] == (200, 2) and shapes["l0.mlp.e4.gate"] == (24, 64) and shapes["l0.mlp.e4.down"] == (64, 24)
    assert shapes["l1.mix.dq"] == (28, 64) and shapes["l1.mix.dq.norm"] == (28,) and shapes["l1.mix.uq"] == (3 * 20, 28)
    assert shapes["l1.mix.dkv"] == (32, 64) and shapes["l1.mix.dkv.norm"] == (24,) and shapes["l1.mix.uk"] == (36, 24)
    assert shapes["l1.mix.uv"] == (60, 24) and shapes["l1.mix.o"] == (64, 60) and shapes["l1.mlp.table"] == (200, 1)
    assert shapes["l2.mix.ra"] == (3, 16, 16) and shapes["l2.mix.conv"] == (48, 4) and shapes["l2.mix.lam"] == (48,)
    assert "l2.ls2" not in shapes and not any(k.startswith("l2.mlp") for k in shapes), "a layer without a feed-forward"
    # layers 1..3 run three times, each pass led by the input product; every run has a cache or a state of its own
    assert [c.layer for c in plan.order] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert [c.before is not None for c in plan.order] == [False, True, False, False, True, False, False, True, False, False, False]
    sites = plan.cache_sites()
    kinds = [type(s).__name__ for _, s in sites]
    assert kinds.count("PagedSpec") == 8 and kinds.count("StateSpec") == 3 and len({site for site, _ in sites}) == 11
    assert [type(b.mixer) for b in plan.layers] == [GQAttention, LatentAttention, RGLRUMixer, GQAttention, LatentAttention]
    att = plan.layers[3].mixer
    assert (att.nh, att.nkv, att.d, att.dv, att.scale, att.q_temp, att.fixed_sink) == (3, 3, 24, 16, 0.2, (0.7, 16), 0.0)
    lat = plan.layers[4].mixer
    assert (lat.H, lat.d, lat.r, lat.dv, lat.R, lat.Q, lat.rot, lat.scale) == (2, 16, 12, 16, 40, 20, 8, 0.25)
    assert len(plan.position_encodings) == 2, "rotary tables are shared only by layers that agree on them"
    assert plan.layers[1].ffn.act == (0.5, 1.702, 1.0) and plan.layers[0].ffn.top == 2 and plan.embedding.scale == 3.0
    free = arch.plan(arch.parse(nu.PLAIN))
    assert not free.stream_parts and [c.layer for c in free.order] == [0, 1, 2] and free.embedding.scale == 1.0
    assert free.layers[0].mixer.q_temp is None
    for bad in ({**nu.MIXED, "layers": [{"type": "window", "mixer": {}, "mlp": None}]},
                {**nu.MIXED, "layers": [nu.layer(nu.attention(heads=3, kv_heads=2), None)], "loop": None},
                {**nu.MIXED, "layers": [nu.layer(nu.rglru(width=50), None)], "loop": None},
                {**nu.MIXED, "layers": [nu.layer(nu.latent(dims=10), None)], "loop": None},
                {**nu.MIXED, "layers": [nu.layer(nu.rglru(), nu.moe(experts=2, top=3))], "loop": None},
                {**nu.MIXED, "loop": {"start": 2, "stop": 9, "times": 2}},
                {**nu.MIXED, "loop": {"start": 2, "stop": 2, "times": 2}}):
        with pytest.raises(ConfigError):
            arch.parse(bad)


def test_random_tables_name_distinct_experts_and_the_loader_keeps_them_integers(folders):
    from vapi_b200.config.model import load_config_json, resolve_architecture
    from vapi_b200.weights.loader import load_tensors
    cfg = load_config_json(folders["mixed"])
    arch = resolve_architecture(cfg)
    t = load_tensors(folders["mixed"], arch.plan(arch.parse(cfg)).tensor_specs(), torch.bfloat16, "cpu")
    tab = t["l3.mlp.table"]
    assert tab.dtype == torch.int32 and tab.shape == (200, 3) and int(tab.min()) == 0 and int(tab.max()) == 2
    assert all(len(set(r)) == 3 for r in tab.tolist()) and len({tuple(r) for r in tab.tolist()}) > 1
    assert t["l0.ls1"].dtype == torch.float32 and t["l0.mix.q"].dtype == torch.float32, "what is stored in 32 bits stays so"
    t = load_tensors(folders["mixed/bf16"], arch.plan(arch.parse(cfg)).tensor_specs(), torch.bfloat16, "cpu")
    assert t["l0.ls1"].dtype == torch.float32 and t["l0.mix.q"].dtype == torch.bfloat16 and t["l3.mlp.table"].dtype == torch.int32


# ---- the plain model itself, by hand -------------------------------------------------------------------------
def test_the_plain_mechanisms_by_hand():
    # the temperature steps when p + 1 reaches a multiple of `every`
    assert plain.query_temperature(3, 0.5, 5) == 1.0 and plain.query_temperature(4, 0.5, 5) == pytest.approx(1 + 0.5 * math.log(2))
    assert plain.query_temperature(13, 0.5, 5) == pytest.approx(1 + 0.5 * math.log(3)) and plain.query_temperature(14, 0.5, 5) == pytest.approx(1 + 0.5 * math.log(4))
    # a sink of score zero: one key of score s gets exp(s) / (1 + exp(s)), so the first token does not pass unchanged
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0}
    eye = torch.eye(2, dtype=torch.float64)
    w = {"q": eye, "k": eye, "v": eye, "o": eye, "g": torch.zeros((1, 2), dtype=torch.float64),
         "q.b": torch.zeros(2, dtype=torch.float64), "k.b": torch.zeros(2, dtype=torch.float64),
         "v.b": torch.zeros(2, dtype=torch.float64), "o.b": torch.zeros(2, dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    out = plain.sink_attention(w, "", m, h)
    s = 5.0
    assert torch.allclose(out, 0.5 * h * math.exp(s) / (1 + math.exp(s)))         # the gate's sigmoid(0) is a half
    # rotate-half pairs element i with i + dims/2 and leaves the rest
    x = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], dtype=torch.float64)
    r = plain.rotate_half(x, 3, 4, 10.0)
    a0, a1 = 3.0, 3.0 * 10.0 ** -0.5
    assert r[0] == pytest.approx(math.cos(a0) - 3 * math.sin(a0)) and r[2] == pytest.approx(3 * math.cos(a0) + math.sin(a0))
    assert r[1] == pytest.approx(2 * math.cos(a1) - 4 * math.sin(a1)) and r[4] == 5.0 and r[5] == 6.0
    # an expert: clamps before the gate, the up branch shifted by one
    we = {"gate": torch.tensor([[2.0]], dtype=torch.float64), "up": torch.tensor([[-3.0]], dtype=torch.float64),
          "down": torch.tensor([[1.0]], dtype=torch.float64)}
    y = plain.clamped_expert(we, "", torch.tensor([1.0], dtype=torch.float64), 1.5)
    assert float(y) == pytest.approx(1.5 / (1 + math.exp(-1.702 * 1.5)) * (-1.5 + 1.0))
    # the recurrence from zero: the first token is not passed through, it is scaled by sqrt(1 - a^2) like any other
    wr = {"y": torch.zeros((1, 1), dtype=torch.float64), "y.b": torch.tensor([10.0], dtype=torch.float64),
          "x": torch.ones((1, 1), dtype=torch.float64), "x.b": torch.zeros(1, dtype=torch.float64),
          "conv": torch.tensor([[0.0, 1.0]], dtype=torch.float64), "conv.b": torch.zeros(1, dtype=torch.float64),
          "ra": torch.zeros((1, 1, 1), dtype=torch.float64), "ra.b": torch.zeros((1, 1), dtype=torch.float64),
          "ri": torch.zeros((1, 1, 1), dtype=torch.float64), "ri.b": torch.zeros((1, 1), dtype=torch.float64),
          "lam": torch.zeros(1, dtype=torch.float64), "o": torch.ones((1, 1), dtype=torch.float64)}
    out = plain.rglru_block(wr, "", {"width": 1, "blocks": 1, "conv": 2}, torch.tensor([[2.0], [0.0]], dtype=torch.float64))
    a = math.exp(-8 * 0.5 * math.log(2.0))
    s0 = math.sqrt(1 - a * a) * 0.5 * 2.0
    assert float(out[0]) == pytest.approx(s0 * 10.0, rel=1e-6) and float(out[1]) == pytest.approx(a * s0 * 10.0, rel=1e-6)
    # the run order of a loop
    assert plain.run_order({"layers": [0] * 4, "loop": {"start": 1, "stop": 3, "times": 2}}) == \
        [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]


# ---- the model against the plain one: whole prompts, decoding, portions ---------------------------------------
WHOLE = [pytest.param("cpu", "tiny", [19], id="host"),
         pytest.param("cuda", "mixed", [150, 1, 37], marks=pytest.mark.gpu, id="gpu-mixed"),
         pytest.param("cuda", "plain", [70, 2], marks=pytest.mark.gpu, id="gpu-plain"),
         pytest.param("cuda", "serving_heads", [100], marks=pytest.mark.gpu, id="gpu-serving-heads"),
         pytest.param("cuda", "attention", [40], marks=pytest.mark.gpu, id="gpu-attention-alone"),
         pytest.param("cuda", "latent", [40], marks=pytest.mark.gpu, id="gpu-latent-alone"),
         pytest.param("cuda", "rglru", [40], marks=pytest.mark.gpu, id="gpu-rglru-alone")]


@pytest.mark.parametrize("device,name,lens", WHOLE)
def test_whole_prompt_token_by_token_and_portions_agree_with_the_plain_model(device, name, lens, folders, kernels):
    """Each request alone: its whole prompt in one step; a prompt and then single tokens; portions of changing size
    down to two tokens, cut inside pages and across the temperature's steps."""
    kernels(device)
    oracle = nu.Oracle(folders[name])
    runner = vu.make_runner(folders[name], "float32", device, num_pages=12)
    for i, n in enumerate(lens):
        toks = nu.prompt(oracle.cfg, n, 20 + i)
        _check(runner, oracle, {"a": toks}, [[("a", n)]], "float32")
        head = max(1, n - 12) if device == "cuda" else max(1, n - 4)
        _check(runner, oracle, {"b": toks}, [[("b", head)]] + [[("b", 1)]] * (n - head), "float32")
        if n > 2:
            _check(runner, oracle, {"c": toks}, [[("c", q)] for q in vu.cuts(n, [2, 3, 17, 5, 64, 2, 16, 1])], "float32")
            _check(runner, oracle, {"d": toks}, [[("d", q)] for q in vu.cuts(n, [16, 15, 2, 31])], "float32")


@pytest.mark.gpu
def test_long_decoding_one_token_at_a_time(folders):
    """Every token alone from the first: 170 steps through the caches, the convolution's taps and the recurrent state."""
    oracle = nu.Oracle(folders["mixed"])
    runner = vu.make_runner(folders["mixed"], "float32", "cuda", num_pages=12)
    toks = nu.prompt(oracle.cfg, 170, 5)
    _check(runner, oracle, {"a": toks}, [[("a", 1)]] * 170, "float32")


BATCH = [pytest.param("cpu", "tiny", "float32", [7, 1, 12, 3, 9], id="host"),
         pytest.param("cuda", "mixed", "float32", [70, 1, 33, 150, 2, 64, 17], marks=pytest.mark.gpu, id="gpu-f32"),
         pytest.param("cuda", "mixed/bf16", "bfloat16", [70, 1, 33, 150, 2, 64, 17], marks=pytest.mark.gpu, id="gpu-bf16"),
         pytest.param("cuda", "serving_heads/bf16", "bfloat16", [130, 40, 3, 66], marks=pytest.mark.gpu, id="gpu-bf16-tensor-cores"),
         pytest.param("cuda", "plain/bf16", "bfloat16", [60, 5, 31], marks=pytest.mark.gpu, id="gpu-bf16-plain")]


@pytest.mark.parametrize("device,name,dtype,lens", BATCH)
def test_unequal_requests_in_one_batch_match_each_alone(device, name, dtype, lens, folders, kernels):
    """More requests than state slots and a pool smaller than their sum: portions of some beside single tokens of
    others, requests that pause, pages and slots that pass from finished requests to new ones; then the same
    schedule once more on the same runner, over whatever the first pass left in pages and slots."""
    kernels(device)
    oracle = nu.Oracle(folders[name.split("/")[0]] if dtype == "float32" else folders[name])
    page = 16
    need = sorted((-(-n // page) for n in lens), reverse=True)
    runner = vu.make_runner(folders[name], dtype, device, num_pages=sum(need[:4]) + 1, page_size=page, max_requests=4)
    reqs = {f"r{i}": nu.prompt(oracle.cfg, n, 40 + i) for i, n in enumerate(lens)}
    g = torch.Generator().manual_seed(3)
    left = {k: len(v) for k, v in reqs.items()}
    waiting, live, schedule = list(reqs), [], []
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        step = []
        for rid in list(live):
            if len(live) > 1 and float(torch.rand(1, generator=g)) < 0.2:
                continue                                        # left out of this step, goes on later
            q = min(left[rid], int(torch.tensor([1, 1, 2, 3, 16, 29])[torch.randint(0, 6, (1,), generator=g)]))
            step.append((rid, q))
            left[rid] -= q
            if left[rid] == 0:
                live.remove(rid)
        if step:
            schedule.append(step)
    for _ in range(2):
        _check(runner, oracle, reqs, schedule, dtype)


# ---- the new kernels against their restatements -------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [99, 324, 2048, 4100])
def test_two_scaled_sublayers_ride_on_the_norm(hidden, dtype):
    """``x += s1 * y1 + s2 * y2`` and the norm in one kernel: every row, selected rows (the stream untouched), with a
    norm and with the stream's rows handed on as they are, into an output of its own and into the left half of a
    wider buffer; one sublayer alone; nothing pending."""
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    n = 37
    x = torch.randn((n, hidden), generator=g)
    ya, yb = (torch.randn((n, hidden), generator=g) * s for s in (3.0, 0.2))
    ya, yb = ya.to(dtype), yb.to(dtype)
    sa, sb, w = (torch.randn(hidden, generator=g) for _ in range(3))
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    dev = lambda t: None if t is None else t.cuda()
    for r in (None, rows):
        for a, s1, b, s2 in ((ya, sa, yb, sb), (ya, sa, None, None), (ya, None, yb, sb), (None, None, None, None)):
            for weight, copy in ((w, False), (None, True)):
                xr, xd = x.clone(), x.clone().cuda()
                want = plain_ops.scaled_add_rmsnorm(xr, a, s1, b, s2, weight, 1e-6, dtype, r, copy=copy)
                got = ops.scaled_add_rmsnorm(xd, dev(a), dev(s1), dev(b), dev(s2), dev(weight), 1e-6, dtype, dev(r), copy=copy)
                _close(got.float(), want.float(), tol)
                _close(xd, xr, 2e-5)
                assert (r is None and a is not None) != torch.equal(xd.cpu(), x), "selected rows leave the stream as it was"
    wide = torch.full((n, 2 * hidden + 4), 7.0, dtype=dtype).cuda()
    xr, xd = x.clone(), x.clone().cuda()
    want = plain_ops.scaled_add_rmsnorm(xr, ya, sa, yb, sb, None, 0.0, dtype, copy=True)
    ops.scaled_add_rmsnorm(xd, ya.cuda(), sa.cuda(), yb.cuda(), sb.cuda(), None, 0.0, dtype, copy=True, out=wide[:, :hidden])
    _close(wide[:, :hidden].float(), want.float(), tol)
    assert bool((wide[:, hidden:] == 7.0).all()), "the rest of the buffer is someone else's"
    assert ops.scaled_add_rmsnorm(xd, ya.cuda(), sa.cuda(), None, None, None, 0.0, dtype) is None      # the update alone
    xr += ya.float() * sa
    _close(xd, xr, 2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_cache_write_and_query_rotation(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(11)
    for n, Q, R, r, rot, H, d, page in ((9, 20, 24, 8, 8, 3, 12, 4), (70, 136, 200, 64, 32, 5, 40, 16), (1, 4, 4, 4, 2, 1, 4, 8),
                                        (33, 300, 512, 64, 64, 2, 128, 64), (5, 12, 36, 0, 0, 2, 8, 4)):
        down = torch.randn((n, Q + R + r + 3), generator=g) * 2.0
        wq, wc = torch.randn(Q, generator=g), torch.randn(R, generator=g)
        pos = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32)
        freq = torch.tensor([50.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32)
        cos, sin = (torch.cos(pos[:, None].float() * freq), torch.sin(pos[:, None].float() * freq)) if rot else (None, None)
        pages = -(-n // page) + 2
        slots = torch.randperm(pages * page, generator=g)[:n].to(torch.int32)
        cache = torch.randn((pages, page * (R + r)), generator=g).to(dtype)
        want_cache = cache.clone()
        want_cq = plain_ops.latent_prepare(down, Q, R, r, wq, wc, 1e-5, cos, sin, rot, want_cache, page, slots, dtype)
        dcache = cache.cuda()
        c = lambda t: None if t is None else t.cuda()
        got_cq = ops.latent_prepare(down.cuda(), Q, R, r, wq.cuda(), wc.cuda(), 1e-5, c(cos), c(sin), rot, dcache, page, slots.cuda(), dtype)
        tol = 2e-5 if dtype == torch.float32 else 1e-2
        _close(got_cq, want_cq, tol)
        _close(dcache, want_cache, tol)
        untouched = torch.ones(pages * page, dtype=torch.bool)
        untouched[slots.long()] = False
        assert torch.equal(dcache.cpu().view(pages * page, R + r)[untouched], cache.view(pages * page, R + r)[untouched]), "rows of no token"
        if r:
            q = torch.randn((n, H * (d + r) + 8), generator=g).to(dtype)
            qfull = torch.zeros((n, H, R + r), dtype=dtype)
            want = qfull.clone()
            plain_ops.latent_rotate_q(q[:, :H * (d + r)], want, H, d, r, R, cos, sin, rot)
            dq = qfull.cuda()
            ops.latent_rotate_q(q.cuda()[:, :H * (d + r)], dq, H, d, r, R, c(cos), c(sin), rot)
            _close(dq, want, tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_temperature_at_its_steps(dtype):
    """Positions just below and at every multiple of `every`, far positions, beside keys and values that it leaves alone."""
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(5)
    nh, nkv, dk, dv, page = 3, 1, 20, 12, 8
    pos = torch.tensor([0, 1, 5, 6, 7, 13, 14, 20, 21, 699, 700, 7000 * 7 - 2, 7000 * 7 - 1], dtype=torch.int32)
    n = pos.numel()
    qkv = torch.randn((n, (nh + nkv) * dk + nkv * dv + 4), generator=g).to(dtype)
    cache = torch.zeros((4, page * nkv * (dk + dv)), dtype=dtype)
    slots = torch.randperm(4 * page, generator=g)[:n].to(torch.int32)
    want, want_cache = qkv.clone(), cache.clone()
    plain_ops.qk_norm_rope_write_split(want, nh, nkv, dk, dv, None, None, 0.0, None, None, 0, False, want_cache, page, slots,
                                       positions=pos, q_temp=(0.37, 7))
    got, dcache = qkv.cuda(), cache.cuda()
    ops.qk_norm_rope_write_split(got, nh, nkv, dk, dv, None, None, 0.0, None, None, 0, False, dcache, page, slots.cuda(),
                                 positions=pos.cuda(), q_temp=(0.37, 7))
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    _close(got, want, tol)
    _close(dcache, want_cache, tol)
    for t, steps in ((0, 0), (2, 0), (3, 1), (5, 2), (6, 2), (7, 3), (9, 100), (10, 100), (11, 6999), (12, 7000)):
        f = 1 + 0.37 * math.log(steps + 1)
        assert torch.allclose(got[t, :nh * dk].float().cpu(), qkv[t, :nh * dk].float() * f, rtol=1e-2 if dtype == torch.bfloat16 else 1e-6)
    assert torch.equal(got[:, nh * dk:].cpu(), qkv[:, nh * dk:]), "keys, values and what follows them are left alone"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_table_choice_and_clamped_experts(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(9)
    for n, W, ff, E, top, V in ((70, 64, 24, 5, 2, 50), (1, 40, 8, 3, 3, 7), (300, 136, 72, 9, 1, 300), (17, 32, 16, 1, 1, 4)):
        h = torch.randn((n, W), generator=g).to(dtype)
        toks = torch.randint(0, V, (n,), generator=g, dtype=torch.int32)
        table = torch.rand((V, E), generator=g).argsort(1)[:, :top].to(torch.int32).contiguous()
        w_up = (torch.randn((E, 2 * ff, W), generator=g) * 0.3).to(dtype)
        w_down = (torch.randn((E, W, ff), generator=g) * 0.3).to(dtype)
        act = (0.9, 1.702, 1.0)
        ids, wts, _ = plain_ops.moe_table_route(toks, table, E)
        want = plain_ops.moe_experts(h, ids, wts, None, w_up, w_down, None, gated=True, act=act)
        dids, dwts, plan = ops.moe_table_route(toks.cuda(), table.cuda(), E)
        assert torch.equal(dids.cpu(), ids) and torch.allclose(dwts.cpu(), wts)
        got = ops.moe_experts(h.cuda(), dids, dwts, plan, w_up.cuda(), w_down.cuda(), None, gated=True, act=act)
        _close(got, want, 2e-5 if dtype == torch.float32 else 3e-2)
        # the constants of plain SiLU gating give what the gated form gave before it had constants
        want = plain_ops.moe_experts(h, ids, wts, None, w_up, w_down, None, gated=True)
        got = ops.moe_experts(h.cuda(), dids, dwts, plan, w_up.cuda(), w_down.cuda(), None, gated=True)
        _close(got, want, 2e-5 if dtype == torch.float32 else 3e-2)


def _shared_attention(ops_mod, q, cache, table, qlen, klen, H, R, r, page, splits, device):
    cu = torch.tensor([0, qlen], dtype=torch.int32).to(device)
    sk = torch.tensor([klen], dtype=torch.int32).to(device)
    return ops_mod.masked_attention(q, H * (R + r), cache, page, table, cu, sk, qlen, 1, qlen, klen, H, 1, R + r, R, 1.0,
                                    splits=splits, shared_kv=True)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_row_is_found_in_the_shared_cache(dtype):
    """One cached row that matches among hundreds: far back, at page borders, the newest row, with and without split
    keys, for single tokens and portions.  Its latent comes out of every head; a row behind the query does not."""
    from vapi_b200 import ops
    # (widths that are multiples of 16 take the tensor-core kernel in bfloat16, the others the general one)
    for H, R, r, page in ((3, 24, 8, 16), (5, 32, 16, 16), (2, 128, 32, 64)):
      for klen, j_star, qlen, splits in ((900, 3, 1, 1), (900, 3, 1, 4), (900, 15, 7, 1), (900, 16, 7, 3), (641, 640, 1, 2), (640, 639, 1, 1),
                                         (333, 0, 40, 1), (48, 47, 48, 1), (2, 0, 2, 1), (1, 0, 1, 1), (100, 63, 100, 1), (100, 64, 100, 2),
                                         (130, 31, 99, 1), (130, 32, 99, 1), (97, 96, 33, 2)):
        q, cache, table = nu.planted_latent(klen, j_star, qlen, H, R, r, page, "cuda", dtype)
        out = _shared_attention(ops, q, cache, table, qlen, klen, H, R, r, page, splits, "cuda").float().cpu().view(qlen, H, R)
        for j in range(qlen):
            p = klen - qlen + j
            seen = j_star <= p
            assert bool(((out[j] - (1.0 if seen else 0.0)).abs() < 0.05).all()), \
                f"heads {H} of {R} + {r}: keys {klen}, planted {j_star}, query at {p}, splits {splits}"
    # against the restatement, at sizes that fit no vector width but four: a mixed batch
    g = torch.Generator().manual_seed(2)
    for H, R, r, page in ((5, 36, 4, 8), (2, 260, 64, 16), (1, 4, 0, 4), (3, 512, 64, 16), (4, 96, 16, 16), (2, 256, 32, 8), (3, 64, 64, 64),
                          (5, 48, 0, 16), (7, 144, 16, 16)):
        lens, klens = [1, 9, 30, 2], [70, 9, 41, 33]
        pages = sum(-(-k // page) for k in klens)
        cache = (torch.randn((pages + 2, page * (R + r)), generator=g) * 0.5).to(dtype)
        order = torch.randperm(pages + 2, generator=g).to(torch.int32)
        width = max(-(-k // page) for k in klens)
        table = torch.zeros((4, width), dtype=torch.int32)
        at = 0
        for s, k in enumerate(klens):
            np_ = -(-k // page)
            table[s, :np_] = order[at:at + np_]
            at += np_
        n = sum(lens)
        q = (torch.randn((n, H * (R + r)), generator=g) * 0.3).to(dtype)
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        sk = torch.tensor(klens, dtype=torch.int32)
        want = plain_ops.masked_attention(q, H * (R + r), cache, page, table, cu, sk, n, 4, max(lens), max(klens), H, 1, R + r, R, 0.2,
                                          shared_kv=True)
        for splits in (1, 3):
            got = ops.masked_attention(q.cuda(), H * (R + r), cache.cuda(), page, table.cuda(), cu.cuda(), sk.cuda(), n, 4, max(lens),
                                       max(klens), H, 1, R + r, R, 0.2, splits=splits, shared_kv=True)
            _close(got, want, 2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dk,dv", [(torch.float32, 20, 12), (torch.bfloat16, 20, 12), (torch.bfloat16, 64, 64), (torch.bfloat16, 128, 128)])
def test_a_sink_of_score_zero_by_hand(dtype, dk, dv):
    """One key of score s and value one: the head returns exp(s) / (1 + exp(s)), on every attention kernel (the general
    one, and for keys and values of 64 or 128 in bfloat16 the tensor-core ones); without the sink it returns one."""
    from vapi_b200 import ops
    page, nh = 64, 2
    for s in (-2.0, 0.0, 3.0):
        cache = torch.zeros((2, page * (dk + dv)), dtype=torch.float32)
        cache[1, 0] = 1.0                       # key 0 of the page: first element one
        cache[1, page * dk:page * dk + dv] = 1.0
        q = torch.zeros((1, nh * dk))
        q[0, 0], q[0, dk] = s, 2 * s
        args = (q.to(dtype).cuda(), nh * dk, cache.to(dtype).cuda(), page, torch.tensor([[1]], dtype=torch.int32).cuda(),
                torch.tensor([0, 1], dtype=torch.int32).cuda(), torch.tensor([1], dtype=torch.int32).cuda(), 1, 1, 1, 1, nh, 1, dk, dv, 1.0)
        with_sink = ops.masked_attention(*args, sinks=torch.zeros(nh).cuda()).float().cpu().view(nh, dv)
        without = ops.masked_attention(*args).float().cpu().view(nh, dv)
        for h, sc in enumerate((s, 2 * s)):
            assert torch.allclose(with_sink[h], torch.full((dv,), math.exp(sc) / (1 + math.exp(sc))), atol=1e-2 if dtype == torch.bfloat16 else 1e-6)
        assert torch.allclose(without, torch.ones((nh, dv)))


@pytest.mark.gpu
def test_a_slow_decay_keeps_its_digits():
    """Decays close to one over a thousand tokens: what the recurrence feels is 1 - a, so a has to be the float nearest
    to exp(log a).  Float32 in, float64 as the measure; two ulps of a would show a hundred times over."""
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(4)
    n, C, B = 1200, 64, 2
    bs = C // B
    u = torch.randn((n, C), generator=g)
    y = torch.randn((n, C), generator=g)
    wa, wi = torch.randn((B, bs, bs), generator=g) * 0.1, torch.randn((B, bs, bs), generator=g) * 0.1
    ba, bi = torch.randn(C, generator=g), torch.randn(C, generator=g)
    lam = torch.linspace(-9.0, -5.0, C)                              # log a from a few parts in a hundred down to a few in ten thousand
    state = torch.zeros((1, C))
    cu, pos, sl = torch.tensor([0, n], dtype=torch.int32), torch.arange(n, dtype=torch.int32), torch.zeros(1, dtype=torch.int32)
    want = plain_ops.rglru(u.double(), y.double(), wa.double(), ba.double(), wi.double(), bi.double(), lam.double(), 8.0, state.double(), 0,
                           sl, cu, pos)
    got = ops.rglru(u.cuda(), y.cuda(), wa.cuda(), ba.cuda(), wi.cuda(), bi.cuda(), lam.cuda(), 8.0, state.cuda(), 0, sl.cuda(), cu.cuda(),
                    pos.cuda(), max_q=n)
    err = float((got.double().cpu() - want).abs().max()) / float(want.abs().max())
    assert err < 2e-5, f"{err:.3e}"


# ---- the engine: scheduler, batching, sampling, entry point -----------------------------------------------------
@pytest.mark.parametrize("device,name,lens,new", [pytest.param("cpu", "tiny", [1, 9, 20], 5, id="host"),
                                                  pytest.param("cuda", "mixed", [1, 33, 80, 7, 64, 40], 10, marks=pytest.mark.gpu, id="gpu")])
def test_greedy_generation_through_the_entry_point(device, name, lens, new, folders, kernels):
    """More requests than slots, prompts cut into portions of 16 beside other requests' decoding; on a GPU pure
    decode steps run as captured graphs.  Slots and pages pass from finished requests to waiting ones."""
    kernels(device)
    from vapi_b200 import LLM, SamplingParams
    oracle = nu.Oracle(folders[name])
    llm = LLM(folders[name], dtype="f32", device=device, num_blocks=40, page_size=16, max_concurrent_seqs=4,
              max_batched_tokens=64, prefill_chunk_tokens=16, max_context=256, cuda_graphs=device == "cuda")
    prompts = [nu.prompt(oracle.cfg, n, 50 + i) for i, n in enumerate(lens)]
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
    reqs = {f"r{i}": nu.prompt(cfg, n, 70 + i) for i, n in enumerate([1, 70, 40, 90, 66])}
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
    oracle = nu.Oracle(folders[name])
    tr, tokens = _trace(oracle.cfg)
    got = rp.run_trace(folders[name], dtype, tr, str(tmp_path / "out"))
    ref = {k: oracle.logits(v).float() for k, v in tokens.items()}
    span = max(float(r.max() - r.min()) for r in ref.values())
    where = [(step, i, rid, pos) for step, rows in tr.rows.items() for i, (rid, pos) in enumerate(rows)]
    e = [np.abs(got[step][i] - ref[rid][pos].numpy()).max() / span for step, i, rid, pos in where]
    slack = [oracle.rounding(tokens[rid], dtype)[pos] for _, _, rid, pos in where]
    _within(e, slack, dtype, "replay")
