"""Fidasun on the GPU against the plain restatement in tests/fidasun_ref.py: each mechanism alone, whole prompts against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, pages and slots
that are used again, window / page edges with inputs made so that one key stands out, the first tokens of a sequence,
long decoding, several sizes, and greedy generation through LLMEngine.  fp32 runs are held to 2e-4 of the logits'
spread, bf16 runs to 6e-2."""
import numpy as np
import pytest
import torch

import fidasun_ref as R
from fidasun_util import Driver, full_cfg, layer, make_cfg, mixer_cfg, mlp_cfg, random_tensors, rel_err

pytestmark = pytest.mark.gpu
F32_TOL, BF16_TOL = 2e-4, 6e-2


def ref_logits(cfg, tensors, tokens):
    return R.forward(cfg, tensors, tokens, torch.float64).numpy()


def toks(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


# ------------------------------------------------------------------ each mechanism alone (one-layer models)
@pytest.mark.parametrize("kind,kw", [
    ("latent_attention", {}),
    ("latent_attention", dict(heads=5, dim=8, rot_dim=12, vdim=8, kv_rank=24, mask=None,
                              rot={"base": 500.0, "dims": 12, "scaling": None})),
    ("latent_attention", dict(heads=9, mask={"size": 64}, rot={"base": 10000.0, "dims": 8, "scaling": None})),
    ("latent_attention", dict(heads=3, dim=16, rot_dim=16, vdim=24, kv_rank=64, mask={"size": 37})),   # tensor-core form
    ("latent_attention", dict(heads=2, dim=8, rot_dim=32, vdim=40, kv_rank=128, mask=None)),
    ("delta", {}),
    ("delta", dict(heads=2, kv_heads=2, dim=40, vdim=70, conv=4)),
    ("mamba2", {}),
    ("mamba2", dict(heads=6, groups=3, vdim=36, state=70, conv=1, norm_groups=3)),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_mixer_alone(lib, kind, kw, dtype):
    cfg = make_cfg([layer(kind, mlp=False, **kw)])
    w = random_tensors(cfg, seed=3)
    t = toks(90, cfg["vocab"], 1)
    d = Driver(cfg, w, dtype, trace=True)
    d.step([("a", t)])
    tr = []
    want = R.forward(cfg, w, t, torch.float64, tr).numpy()
    resid = d.runner.trace[0, :len(t)].cpu().numpy()
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    assert np.abs(resid - tr[0].numpy()).max() <= tol * np.abs(tr[0].numpy()).max()
    assert rel_err(d.result("a"), want) <= tol


@pytest.mark.parametrize("mlp", [mlp_cfg(), mlp_cfg(experts=5, top=5, ff=17, shared_ff=0, scale=0.5),
                                 mlp_cfg(experts=33, top=1, ff=8, shared_ff=9, scale=1.0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_alone(lib, mlp, dtype):
    cfg = make_cfg([layer("delta", mlp=mlp)])
    w = random_tensors(cfg, seed=5)
    t = toks(70, cfg["vocab"], 2)
    d = Driver(cfg, w, dtype)
    d.step([("a", t)])
    if dtype == torch.float32:
        assert rel_err(d.result("a"), ref_logits(cfg, w, t)) <= F32_TOL
    else:
        assert rel_err(d.result("a"), ref_logits(cfg, w, t), q=0.9) <= BF16_TOL


def test_expert_ops_against_the_plain_form(lib):
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(0)
    T, D, E, F, top = 37, 40, 7, 24, 3
    h = torch.randn(T, D, generator=g)
    router = torch.randn(E, D, generator=g) / D ** 0.5
    wts = {"router": router}
    for e in range(E):
        wts[f"e{e}.gate"], wts[f"e{e}.up"], wts[f"e{e}.down"] = (torch.randn(F, D, generator=g) / D ** 0.5,
                                                                 torch.randn(F, D, generator=g) / D ** 0.5,
                                                                 torch.randn(D, F, generator=g) / F ** 0.5)
    mlp = {"router": {"experts": E, "top": top, "scale": 1.3}, "expert": {"ff": F}, "shared": None}
    want = R.moe_ffn(h.double(), {k: v.double() for k, v in wts.items()}, mlp).numpy()
    idx, w = ops.moe_route((h @ router.T).cuda().contiguous(), top, 1.3)
    s = torch.softmax((h @ router.T).double(), -1)
    v, i = torch.topk(s, top, -1)
    assert idx.cpu().tolist() == i.tolist()
    assert np.allclose(w.cpu().numpy(), (v * 1.3).numpy(), rtol=1e-5)
    gu = torch.stack([torch.cat([wts[f"e{e}.gate"], wts[f"e{e}.up"]]) for e in range(E)]).cuda().contiguous()
    dn = torch.stack([wts[f"e{e}.down"] for e in range(E)]).cuda().contiguous()
    x = torch.zeros(T, D, device="cuda")
    ops.moe_experts(x, h.cuda(), idx, w, gu, dn)
    assert np.abs(x.cpu().numpy() - want).max() <= 1e-4 * np.abs(want).max()


def test_norm_ops(lib):
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 52, generator=g) * 3
    w = torch.randn(52, generator=g) * 0.2
    got = ops.resid_rmsnorm(x.cuda(), w.cuda(), 1e-5, 1.0, torch.float32).cpu()
    assert torch.allclose(got, R.norm_zero_centred(x.double(), w.double(), 1e-5).float(), atol=1e-5)
    got = ops.resid_rmsnorm(x.cuda(), w.cuda(), 1e-5, 0.0, torch.float32).cpu()
    assert torch.allclose(got, R.norm_plain(x.double(), w.double(), 1e-5).float(), atol=1e-5)
    y, gate = torch.randn(9, 48, generator=g), torch.randn(9, 48, generator=g)
    wn = torch.randn(48, generator=g)
    u = (y * torch.nn.functional.silu(gate)).double()
    want = R.rms_unit(u.reshape(9, 4, 12), 1e-5).reshape(9, 48) * wn.double()
    got = ops.gated_group_norm(y.cuda(), gate.cuda(), wn.cuda(), 12, 1e-5, True, torch.float32).cpu()
    assert torch.allclose(got, want.float(), atol=2e-5)
    wh = torch.randn(12, generator=g)
    want = R.rms_unit(y.double().reshape(9, 4, 12), 1e-5) * wh.double() * torch.nn.functional.silu(gate.double()).reshape(9, 4, 12)
    got = ops.gated_group_norm(y.cuda(), gate.cuda(), wh.cuda(), 12, 1e-5, False, torch.float32).cpu()
    assert torch.allclose(got, want.reshape(9, 48).float(), atol=2e-5)


def _i32(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


def test_short_conv_carries_its_last_inputs(lib):
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(2)
    for taps in (1, 2, 4, 7):
        C, T = 150, 23
        x, w, b = torch.randn(T, C, generator=g), torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
        want = R.short_conv_silu(x.double(), w.double(), b.double()).float()
        state = torch.full((3, max(taps - 1, 1), C), 7.0, device="cuda")        # stale contents of a used slot
        got = []
        for lo, hi in ((0, 1), (1, 3), (3, 4), (4, 16), (16, 23)):               # the first portion is one token
            got.append(ops.short_conv_silu(x[lo:hi].cuda().contiguous(), w.cuda(), b.cuda(), state, _i32([2]),
                                           _i32([0, hi - lo]), _i32([hi])).cpu())
        assert torch.allclose(torch.cat(got), want, atol=1e-5), taps


def test_delta_rule_and_ssd_ops_in_portions(lib):
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(4)
    T, H, Hk, dk, dv = 41, 4, 2, 20, 50
    q, k = torch.randn(T, Hk, dk, generator=g), torch.randn(T, Hk, dk, generator=g)
    v, b, a = torch.randn(T, H, dv, generator=g), torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    a_log, dtb = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g)
    qn = q.double() / torch.sqrt((q.double() ** 2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kn = k.double() / torch.sqrt((k.double() ** 2).sum(-1, keepdim=True) + 1e-6)
    gt = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(a.double() + dtb.double()))
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=torch.float64)
        for t in range(T):
            S = gt[t, h] * S
            u = torch.sigmoid(b[t, h].double()) * (v[t, h].double() - S.T @ kn[t, h // 2])
            S = S + torch.outer(kn[t, h // 2], u)
            want[t, h] = S.T @ qn[t, h // 2]
    state = torch.full((2, H, dk, dv), 3.0, device="cuda")
    got = []
    for lo, hi in ((0, 2), (2, 3), (3, 30), (30, 41)):
        c = lambda z: z[lo:hi].cuda().contiguous()                             # noqa: E731
        got.append(ops.delta_rule(c(q), c(k), c(v), c(b), c(a), a_log.cuda(), dtb.cuda(), state, _i32([1]),
                                  _i32([0, hi - lo]), _i32([hi])).cpu())
    assert np.abs(torch.cat(got).numpy() - want.numpy()).max() <= 2e-5 * want.abs().max().item()
    # SSD
    G, N, P = 2, 28, 36
    x, Bm, Cm = torch.randn(T, H, P, generator=g), torch.randn(T, G, N, generator=g), torch.randn(T, G, N, generator=g)
    dt, dsk = torch.randn(T, H, generator=g), torch.randn(H, generator=g)
    dts = torch.nn.functional.softplus(dt.double() + dtb.double())
    want = torch.zeros(T, H, P, dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(N, P, dtype=torch.float64)
        for t in range(T):
            S = torch.exp(-torch.exp(a_log[h].double()) * dts[t, h]) * S + dts[t, h] * torch.outer(Bm[t, h // 2].double(), x[t, h].double())
            want[t, h] = S.T @ Cm[t, h // 2].double() + dsk[h].double() * x[t, h].double()
    state = torch.full((2, H, N, P), -2.0, device="cuda")
    got = []
    for lo, hi in ((0, 1), (1, 9), (9, 41)):
        c = lambda z: z[lo:hi].cuda().contiguous()                             # noqa: E731
        got.append(ops.ssd_scan(c(x), c(Bm), c(Cm), c(dt), a_log.cuda(), dtb.cuda(), dsk.cuda(), state, _i32([0]),
                                _i32([0, hi - lo]), _i32([hi])).cpu())
    assert np.abs(torch.cat(got).numpy() - want.numpy()).max() <= 2e-5 * want.abs().max().item()


# ------------------------------------------------------------------ window and page edges, made to show
@pytest.mark.parametrize("window", [0, 5, 64, 70, 130])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("r,dr", [(12, 4), (64, 16)])        # the second shape takes the tensor-core form for many rows
def test_latent_attention_sees_exactly_its_window(lib, window, dtype, split, r, dr):
    """Every cached latent is a distinct random vector and the query is made to score the EARLIEST visible key far
    above all others: the output must be the latent at the window's far edge, never the one just outside it; checked
    for prompt rows and for single decoded rows, with edges at page borders and far back, on a shuffled block table."""
    from vllm_rs_b200 import ops
    H, n = 2, 200
    R_ = r + dr
    pages = [5, 2, 7, 0]                                               # shuffled physical pages
    cache = torch.zeros(8, 64, R_, dtype=dtype, device="cuda")
    lat = torch.randn(n, r, generator=torch.Generator().manual_seed(0))
    for j in range(n):
        row = torch.cat([lat[j], torch.full((dr,), j / n)])            # rotated part: a position tag in every entry
        cache[pages[j // 64], j % 64] = row.to(dtype).cuda()
    bt = _i32([pages])

    def first_visible(i):
        return 0 if window <= 0 else max(0, i - window + 1)

    # the rotated query part is a steep NEGATIVE ramp over the position tag: the earliest visible key outweighs all
    # later ones by e^-20 per position, so the output is the latent at the window's far edge (or key 0 without a
    # window), and a key one place outside the window would have won had it been seen
    for rows_pos in ([199], [64], [63], list(range(100, 200)), list(range(120, 200)), list(range(0, 70)), list(range(0, 129))):
        T = len(rows_pos)
        q = torch.zeros(T, H, R_)
        q[:, :, r:] = -4000.0 / dr                                     # prefers the earliest visible key
        out = ops.latent_attn(q.cuda().contiguous(), cache, torch.full((H,), -1e4, device="cuda"), _i32([0, T]),
                              _i32([rows_pos[-1] + 1]), bt, kv_rank=r, rot_dim=dr, window=window, scale=1.0,
                              split=split).float().cpu()
        tol = 2e-3 if dtype == torch.float32 else 3e-2
        for i, p in enumerate(rows_pos):
            j = first_visible(p)
            want = lat[j].to(dtype).float()
            assert (out[i, 0] - want).abs().max() <= tol, (window, p, j)
            assert (out[i, 1] - want).abs().max() <= tol
    # the sink takes its share: with a sink as large as the best score the output halves
    q = torch.zeros(1, H, R_)
    out = ops.latent_attn(q.cuda(), cache, torch.tensor([0.0, -1e4], device="cuda"), _i32([0, 1]), _i32([1]), bt,
                          kv_rank=r, rot_dim=dr, window=window, scale=1.0, split=split).float().cpu()
    assert (out[0, 0] - 0.5 * lat[0].to(dtype).float()).abs().max() <= 2e-2
    assert (out[0, 1] - lat[0].to(dtype).float()).abs().max() <= 2e-2


@pytest.mark.parametrize("window", [3, 64, 65])
def test_model_window_edge_shows_in_logits(lib, window):
    """A one-layer model: replacing the token at one place changes the last row's logits exactly while that place is
    inside the last row's window (the plain model gives identical logits otherwise), by far more than the tolerance."""
    cfg = make_cfg([layer("latent_attention", mlp=False, mask={"size": window}, heads=2)])
    w = random_tensors(cfg, seed=11)
    n = window + 70
    base = toks(n, cfg["vocab"] - 1, 5)
    special = cfg["vocab"] - 1
    for pos_x in (n - 1 - window, n - window):                        # just outside / just inside the last row's window
        t = list(base)
        t[pos_x] = special
        want = ref_logits(cfg, w, t)
        d = Driver(cfg, w, torch.float32)
        d.step([("a", t[:n - 1])])
        d.step([("a", t[n - 1:])])                                    # the last row is decoded alone
        got = d.result("a")
        assert rel_err(got, want) <= F32_TOL
        other = ref_logits(cfg, w, base)
        visible = pos_x == n - window
        diff = np.abs(want[-1] - other[-1]).max()
        assert (diff > 5 * F32_TOL * want.std()) if visible else diff == 0.0


# ------------------------------------------------------------------ schedules
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_decode_and_portions_agree_with_the_plain_model(lib, dtype):
    cfg = full_cfg()
    w = random_tensors(cfg, seed=7)
    t = toks(150, cfg["vocab"], 3)
    want = ref_logits(cfg, w, t)
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    q = 1.0 if dtype == torch.float32 else 0.8       # bf16: a near-tied expert choice may flip at single rows
    d = Driver(cfg, w, dtype)
    d.step([("whole", t)])
    assert rel_err(d.result("whole"), want, q) <= tol
    d.close("whole")
    d.step([("dec", t[:60])])
    for x in t[60:]:
        d.step([("dec", [x])])
    assert rel_err(d.result("dec"), want, q) <= tol
    d.close("dec")
    cuts = [2, 1, 2, 61, 2, 3, 64, 2, 13]                            # 150 tokens; cuts inside pages and windows
    at = 0
    for c in cuts:
        d.step([("cut", t[at:at + c])])
        at += c
    assert at == len(t)
    assert rel_err(d.result("cut"), want, q) <= tol
    if dtype == torch.float32:                                       # the cut must not matter beyond rounding
        assert rel_err(d.result("cut"), d.result("dec")) <= 2e-5


def test_unequal_batches_and_reuse_of_pages_and_slots(lib):
    cfg = full_cfg()
    w = random_tensors(cfg, seed=9)
    V = cfg["vocab"]
    reqs = {"a": toks(130, V, 1), "b": toks(3, V, 2), "c": toks(70, V, 3), "d": toks(65, V, 4), "e": toks(40, V, 5),
            "f": toks(129, V, 6)}
    want = {k: ref_logits(cfg, w, v) for k, v in reqs.items()}
    d = Driver(cfg, w, torch.float32, num_blocks=7, max_seqs=4, slots=4)      # 7 pages: a(3) + c(2) + d(2) fill it
    at = {k: 0 for k in reqs}

    def portion(k, n):
        p = (k, reqs[k][at[k]:at[k] + n])
        at[k] += n
        return p

    d.step([portion("a", 64), portion("b", 2)])
    d.step([portion("a", 1), portion("b", 1), portion("c", 30)])
    d.close("b")                                                      # its page and slot go back
    d.step([portion("c", 40), portion("a", 2), portion("d", 65)])
    d.step([portion("a", 63)])
    d.close("a"), d.close("c")
    assert d.sched.num_free_blocks == 5 and d.sched.num_free_state_slots == 3
    d.step([portion("e", 39), portion("f", 128)])                     # reuses a's and c's pages and slots
    d.step([portion("f", 1), portion("e", 1)])
    for k in "abcdef":
        assert at[k] == len(reqs[k])
        assert rel_err(d.result(k), want[k]) <= F32_TOL, k


def test_first_tokens_and_long_decoding(lib):
    cfg = full_cfg()
    w = random_tensors(cfg, seed=13)
    t = toks(260, cfg["vocab"], 8)
    want = ref_logits(cfg, w, t)
    d = Driver(cfg, w, torch.float32)
    for x in t:                                                       # every token alone, from the very first
        d.step([("a", [x])])
    got = d.result("a")
    assert rel_err(got[:6], want[:6]) <= F32_TOL
    assert rel_err(got, want) <= F32_TOL


def test_other_sizes(lib):
    cfg = make_cfg([layer("delta", heads=3, kv_heads=1, dim=17, vdim=33, conv=2, mlp=mlp_cfg(4, 3, 10, 6, 0.7)),
                    layer("latent_attention", heads=1, dim=4, rot_dim=2, vdim=5, kv_rank=9, mask={"size": 1},
                          rot={"base": 77.0, "dims": 2, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}},
                          mlp=False),
                    layer("mamba2", heads=2, groups=2, vdim=130, state=5, conv=8, norm_groups=4, mlp=mlp_cfg(3, 1, 5, 0, 2.0))],
                   width=24, vocab=50, eps=1e-3)
    w = random_tensors(cfg, seed=17)
    t = toks(80, cfg["vocab"], 9)
    want = ref_logits(cfg, w, t)
    d = Driver(cfg, w, torch.float32)
    d.step([("a", t[:7])]), d.step([("a", t[7:9])]), d.step([("a", t[9:])])
    assert rel_err(d.result("a"), want) <= F32_TOL


def test_greedy_generation_through_the_engine(lib):
    """LLMEngine (schedule -> chunked prefill -> decode, state slots from the scheduler) against greedy decoding with
    the plain model."""
    from vllm_rs_b200 import engine, models
    cfg = full_cfg()
    w = random_tensors(cfg, seed=21)
    V = cfg["vocab"]
    prompts = [toks(75, V, 1), toks(5, V, 2), toks(40, V, 3)]
    new = 12
    runner = models.build_runner(cfg, w, dtype=torch.float32, device="cuda", num_blocks=12, max_blocks_per_seq=4,
                                 max_seqs=5, max_tokens=64, num_state_slots=5)
    eng = engine.LLMEngine(runner, 12, 3, chunk_size=32)              # prompts longer than a chunk are cut
    sids = [eng.add_request(p, new) for p in prompts]
    out = eng.run_to_completion()
    for sid, p in zip(sids, prompts):
        seq, want = list(p), []
        for _ in range(new):
            lg = ref_logits(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            nxt = int(lg.argmax())
            want.append(nxt)
            seq.append(nxt)
            if top2[1] - top2[0] < 1e-3:                              # a near tie may flip in fp32: stop comparing there
                break
        assert out[sid][:len(want)] == want
    assert eng.sched.num_free_state_slots == 5


# ------------------------------------------------------------------ random configurations under random schedules
def _random_layer(rng, kind):
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    if kind == "latent_attention":
        rd = pick(8, 16, 32, 64)
        m = dict(heads=pick(2, 4, 6, 16), dim=pick(16, 24, 64, 128), rot_dim=rd, vdim=pick(32, 48, 128),
                 kv_rank=pick(64, 96, 192, 256, 512), scale=pick(0.125, 0.07), mask={"size": pick(1, 17, 64, 100, 200, 1000)},
                 rot={"base": pick(1e4, 5e5), "dims": rd, "scaling": {"factor": pick(4.0, 40.0), "original": pick(64, 4096),
                                                                       "fast": pick(32.0, 8.0), "slow": pick(1.0, 2.0)}})
    elif kind == "delta":
        kvh = pick(1, 2, 4)
        m = dict(heads=kvh * pick(1, 2, 3), kv_heads=kvh, dim=pick(32, 48, 128, 130, 256), vdim=pick(8, 64, 80, 200),
                 conv=pick(2, 3, 4, 7))
    else:
        g = pick(1, 2, 4)
        h, vd = g * pick(1, 2, 4), pick(32, 48, 64)
        m = dict(heads=h, groups=g, vdim=vd, state=pick(16, 48, 128, 129, 256), conv=pick(2, 4, 6),
                 norm_groups=pick(*[x for x in (1, 2, 4, h) if (h * vd) % x == 0]))
    E = pick(2, 4, 7, 16)
    mlp = None if rng.random() < 0.15 else {
        "kind": "moe", "router": {"experts": E, "top": int(rng.integers(1, min(E, 6) + 1)), "scale": pick(1.0, 2.5, 0.5)},
        "expert": {"ff": pick(20, 32, 96)}, "shared": {"ff": pick(48, 128)} if rng.random() < 0.8 else None}
    return {"type": kind, "mixer": m, "mlp": mlp}


def _random_schedule(rng, reqs):
    """[(portions, requests that end)]: at most four live, portions of 2 .. 300 tokens, the last 20 tokens one by one,
    a live request is sometimes left out of a step."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    pending, live, at, steps = list(reqs), [], {}, []
    while pending or live:
        while pending and len(live) < 4 and (not live or rng.random() < 0.6):
            live.append(pending.pop(0))
            at[live[-1]] = 0
        st, ends = [], []
        for k in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            left = len(reqs[k]) - at[k]
            n = 1 if left <= 20 else max(1, min(left - 20, pick(2, 2, 3, 7, 31, 64, 65, 130, 300)))
            st.append((k, reqs[k][at[k]:at[k] + n]))
            at[k] += n
            if at[k] == len(reqs[k]):
                ends.append(k)
                live.remove(k)
        if st:
            steps.append((st, ends))
    return steps


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_random_configurations_under_random_schedules(lib, seed):
    """Sizes, layer orders and constants drawn at random (also key / state sizes above 128 and odd ones); five requests
    of 5 .. 420 tokens share four state slots and just enough pages, so both are used again.  fp32 only: with bf16
    operands a near-tied expert choice may flip and a recurrent layer then carries the difference along."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    kinds = [pick("latent_attention", "delta", "mamba2") for _ in range(int(rng.integers(2, 6)))]
    cfg = make_cfg([_random_layer(rng, k) for k in kinds], width=pick(128, 192, 320), vocab=pick(300, 512),
                   eps=pick(1e-6, 1e-5))
    w = random_tensors(cfg, seed=seed)
    reqs = {f"r{i}": toks(pick(5, 40, 150, 260, 420), cfg["vocab"], seed + i) for i in range(5)}
    pages = sum(sorted((len(v) + 63) // 64 for v in reqs.values())[-4:])
    d = Driver(cfg, w, torch.float32, num_blocks=pages, max_seqs=4, slots=4)
    for st, ends in _random_schedule(rng, reqs):
        d.step(st)
        for k in ends:
            d.close(k)
    for k, v in reqs.items():
        assert rel_err(d.result(k), ref_logits(cfg, w, v)) <= F32_TOL, (k, kinds)
