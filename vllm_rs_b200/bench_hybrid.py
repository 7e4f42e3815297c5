"""Throughput of the Fidasun hybrid decoder at layer sizes that resemble a real model (random weights), next to the
dense fp16 LLaMA plan at equal width, depth and active feed-forward size: `python bench.py --config fidasun`.

Per size: prefill tokens/s (one prompt of `prefill` tokens in one step) and decode tokens/s (`batch` sequences at
context `ctx`, one token each), CUDA events after warm-up, and a table of the new design's own kernels timed alone
at the same shapes with their algorithmic bytes / flops against the measured copy bandwidth and cuBLAS bf16 peak."""
from __future__ import annotations

import numpy as np
import torch

from . import ops, synthetic
from .hybrid import MIXER_DELTA_RULE, MIXER_LATENT_ATTN, MIXER_SSD

SIZES = {
    # width, per-mixer sizes, experts; `dense` = (heads, kv heads, head dim, inter) of the LLaMA plan of equal width
    "w2048": dict(width=2048, vocab=32000, latent=dict(heads=16, dim=64, rot_dim=32, vdim=64, kv_rank=256, window=1024),
                  delta=dict(heads=16, kv_heads=8, dim=128, vdim=128, conv=4),
                  ssd=dict(heads=32, groups=1, vdim=64, state=128, conv=4, norm_groups=1),
                  moe=dict(experts=16, top=4, ff=512, shared=1024), dense=(16, 4, 128, 3072)),
    "w4096": dict(width=4096, vocab=32000, latent=dict(heads=32, dim=64, rot_dim=32, vdim=64, kv_rank=512, window=2048),
                  delta=dict(heads=32, kv_heads=16, dim=128, vdim=128, conv=4),
                  ssd=dict(heads=64, groups=1, vdim=64, state=128, conv=4, norm_groups=1),
                  moe=dict(experts=32, top=4, ff=1024, shared=2048), dense=(32, 8, 128, 6144)),
}
ORDER = ["mamba2", "latent_attention", "latent_attention", "delta"]


def config(size, layers):
    s = SIZES[size]
    la, de, sd, mo = s["latent"], s["delta"], s["ssd"], s["moe"]
    mlp = {"kind": "moe", "router": {"experts": mo["experts"], "top": mo["top"], "scale": 1.0},
           "expert": {"ff": mo["ff"]}, "shared": {"ff": mo["shared"]}}
    mix = {"latent_attention": dict(heads=la["heads"], dim=la["dim"], rot_dim=la["rot_dim"], vdim=la["vdim"],
                                    kv_rank=la["kv_rank"], scale=(la["dim"] + la["rot_dim"]) ** -0.5,
                                    mask={"size": la["window"]}, rot={"base": 10000.0, "dims": la["rot_dim"], "scaling": None}),
           "delta": dict(heads=de["heads"], kv_heads=de["kv_heads"], dim=de["dim"], vdim=de["vdim"], conv=de["conv"]),
           "mamba2": dict(heads=sd["heads"], groups=sd["groups"], vdim=sd["vdim"], state=sd["state"], conv=sd["conv"],
                          norm_groups=sd["norm_groups"])}
    return {"architecture": "Fidasun", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6},
            "layers": [{"type": ORDER[i % 4], "mixer": mix[ORDER[i % 4]], "mlp": mlp} for i in range(layers)]}


def random_tensors(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}
    lin = lambda n, k: (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)         # noqa: E731
    vec = lambda n, m=0.0, s=0.1: (m + s * torch.randn(n, generator=g)).to(torch.bfloat16)   # noqa: E731
    out["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(torch.bfloat16)
    out["head"], out["final.norm"] = lin(cfg["vocab"], D), vec(D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = vec(D)
        if L["type"] == "latent_attention":
            H = m["heads"]
            out.update({p + "mix.q": lin(H * (m["dim"] + m["rot_dim"]), D), p + "mix.dkv": lin(m["kv_rank"] + m["rot_dim"], D),
                        p + "mix.dkv.norm": vec(m["kv_rank"], 1.0), p + "mix.uk": lin(H * m["dim"], m["kv_rank"]),
                        p + "mix.uv": lin(H * m["vdim"], m["kv_rank"]), p + "mix.sink": vec(H),
                        p + "mix.o": lin(D, H * m["vdim"])})
        elif L["type"] == "delta":
            H, Hk = m["heads"], m["kv_heads"]
            for n, rows in (("q", Hk * m["dim"]), ("k", Hk * m["dim"]), ("v", H * m["vdim"])):
                out[p + f"mix.{n}"] = lin(rows, D)
                out[p + f"mix.{n}.conv"] = vec(rows * m["conv"], 0.0, 0.5).reshape(rows, m["conv"])
            out.update({p + "mix.b": lin(H, D), p + "mix.a": lin(H, D), p + "mix.A_log": vec(H, -0.5, 0.5),
                        p + "mix.dt_bias": vec(H, -1.0, 0.5), p + "mix.norm": vec(m["vdim"], 1.0),
                        p + "mix.g": lin(H * m["vdim"], D), p + "mix.o": lin(D, H * m["vdim"])})
        else:
            H, inner, GN = m["heads"], m["heads"] * m["vdim"], m["groups"] * m["state"]
            out.update({p + "mix.in": lin(2 * inner + 2 * GN + H, D),
                        p + "mix.conv": vec((inner + 2 * GN) * m["conv"], 0.0, 0.5).reshape(inner + 2 * GN, m["conv"]),
                        p + "mix.conv.b": vec(inner + 2 * GN), p + "mix.dt_bias": vec(H, -1.0, 0.5),
                        p + "mix.A_log": vec(H, -0.5, 0.5), p + "mix.D": vec(H, 1.0), p + "mix.norm": vec(inner, 1.0),
                        p + "mix.o": lin(D, inner)})
        mlp = L["mlp"]
        E, F, Fs = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["shared"]["ff"]
        out[p + "mlp.router"] = lin(E, D)
        for e in range(E):
            out.update({p + f"mlp.e{e}.gate": lin(F, D), p + f"mlp.e{e}.up": lin(F, D), p + f"mlp.e{e}.down": lin(D, F)})
        out.update({p + "mlp.shared.gate": lin(Fs, D), p + "mlp.shared.up": lin(Fs, D), p + "mlp.shared.down": lin(D, Fs)})
    return out


def _say(msg):
    import sys
    print(f"[bench_hybrid] {msg}", file=sys.stderr, flush=True)


def _time(fn, reps, warm=3):
    """ms per call on the current stream: warm-up, then CUDA events around `reps` calls."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _meta(B, q_len, ctx, blocks_per_seq, vocab, seed=0):
    """Hand-made step metadata: B sequences, each bringing q_len tokens that end at context ctx; sequence b owns the
    pages [b * blocks_per_seq, ...) and state slot b."""
    rng = np.random.default_rng(seed)
    T = B * q_len
    pos = np.tile(np.arange(ctx - q_len, ctx, dtype=np.int64), B)
    seq = np.repeat(np.arange(B, dtype=np.int64), q_len)
    bt = (np.arange(B * blocks_per_seq, dtype=np.uint32)).reshape(B, blocks_per_seq)
    slot = (seq * blocks_per_seq + pos // 64) * 64 + pos % 64
    return dict(input_ids=rng.integers(0, vocab, size=T).astype(np.uint32), positions=pos, slot_mapping=slot,
                cu_seqlens_q=(np.arange(B + 1) * q_len).astype(np.uint32), context_lens=np.full(B, ctx, np.uint32),
                block_tables=np.ascontiguousarray(bt.reshape(-1)), state_slots=np.arange(B, dtype=np.int32),
                num_seqs=B, num_tokens=T, max_blocks=blocks_per_seq)


def kernel_table(size, prefill, batch, ctx, peaks):
    """Each new kernel alone at the prefill shape (one sequence of `prefill` tokens) and the decode shape (`batch`
    sequences at context `ctx`): ms, achieved and the fraction of the bound it should sit on."""
    s, dev = SIZES[size], "cuda"
    hbm, tc = float(peaks["hbm_gbs"]) * 1e9, float(peaks["bf16_tflops"]) * 1e12
    fma = 148 * 128 * 2 * 1.9e9                      # fp32 FMA peak of the CUDA cores (nominal clocks)
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *sh: torch.randn(*sh, generator=g, device=dev)          # noqa: E731
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)       # noqa: E731
    rows = []

    def add(name, phase, ms, flops=0.0, nbytes=0.0, bound="hbm", note=""):
        _say(f"{name} {phase}: {ms:.3f} ms")
        ach_f, ach_b = flops / (ms * 1e-3), nbytes / (ms * 1e-3)
        frac = {"hbm": ach_b / hbm, "tensor": ach_f / tc, "fp32": ach_f / fma}[bound]
        rows.append(dict(kernel=name, phase=phase, ms=round(ms, 4), tflops=round(ach_f / 1e12, 3),
                         gbs=round(ach_b / 1e9, 1), bound=bound, frac=round(frac, 4), note=note))

    for phase, B, q_len, cx_len in (("prefill", 1, prefill, prefill), ("decode", batch, 1, ctx)):
        T, nblk = B * q_len, (cx_len + 63) // 64
        cu, cl = i32((np.arange(B + 1) * q_len).tolist()), i32([cx_len] * B)
        slots = i32(list(range(B)))
        # latent attention
        la = s["latent"]
        H, r, dr, W = la["heads"], la["kv_rank"], la["rot_dim"], la["window"]
        cache = (rnd(B * nblk, 64, r + dr) * 0.3).to(torch.bfloat16)
        bt = i32(np.arange(B * nblk).reshape(B, nblk).tolist())
        q = rnd(T, H, r + dr) * 0.1
        sink = torch.zeros(H, device=dev)
        ms = _time(lambda: ops.latent_attn(q, cache, sink, cu, cl, bt, kv_rank=r, rot_dim=dr, window=W, scale=0.1), 3)
        keys = sum(min(p + 1, W) for p in range(cx_len - q_len, cx_len)) * B
        if phase == "decode":
            add("latent_attn", phase, ms, 2.0 * H * keys * (2 * r + dr), keys * (r + dr) * 2.0, "hbm",
                "bytes = visible cache rows, read once for all heads")
        else:
            add("latent_attn", phase, ms, 2.0 * H * keys * (2 * r + dr), 0.0, "tensor")
        # short convolution + gated delta rule
        de = s["delta"]
        Hd, Hk, dk, dv = de["heads"], de["kv_heads"], de["dim"], de["vdim"]
        C = 2 * Hk * dk + Hd * dv
        x = rnd(T, C)
        st = torch.zeros(B, de["conv"] - 1, C, device=dev)
        tw, tb = rnd(C, de["conv"]), rnd(C)
        ms = _time(lambda: ops.short_conv_silu(x, tw, tb, st, slots, cu, cl), 3)
        add("short_conv_silu", phase, ms, 0.0, T * C * 8.0 + B * (de["conv"] - 1) * C * 8.0, "hbm")
        qd, kd, vd = rnd(T, Hk, dk), rnd(T, Hk, dk), rnd(T, Hd, dv)
        bb, aa, al, db = rnd(T, Hd), rnd(T, Hd), rnd(Hd) * 0.3, rnd(Hd)
        sd_ = torch.zeros(B, Hd, dk, dv, device=dev)
        ms = _time(lambda: ops.delta_rule(qd, kd, vd, bb, aa, al, db, sd_, slots, cu, cl), 3)
        if phase == "decode":
            add("delta_rule", phase, ms, 6.0 * T * Hd * dk * dv, B * Hd * dk * dv * 8.0, "hbm", "bytes = state read + write")
        else:
            add("delta_rule", phase, ms, 6.0 * T * Hd * dk * dv, 0.0, "fp32", "token-serial recurrence")
        # SSD scan
        ss = s["ssd"]
        Hs, G, N, P = ss["heads"], ss["groups"], ss["state"], ss["vdim"]
        xs, Bm, Cm, dt = rnd(T, Hs, P), rnd(T, G, N), rnd(T, G, N), rnd(T, Hs)
        als, dbs, dsk = rnd(Hs) * 0.3, rnd(Hs), rnd(Hs)
        sst = torch.zeros(B, Hs, N, P, device=dev)
        ms = _time(lambda: ops.ssd_scan(xs, Bm, Cm, dt, als, dbs, dsk, sst, slots, cu, cl), 3)
        if phase == "decode":
            add("ssd_scan", phase, ms, 4.0 * T * Hs * N * P, B * Hs * N * P * 8.0, "hbm", "bytes = state read + write")
        else:
            add("ssd_scan", phase, ms, 4.0 * T * Hs * N * P, 0.0, "fp32", "token-serial recurrence")
        # routed experts (sort + grouped gate|up + grouped down + combine)
        mo, D = s["moe"], s["width"]
        E, top, F = mo["experts"], mo["top"], mo["ff"]
        h = (rnd(T, D) * 0.5).to(torch.bfloat16)
        gu = (rnd(E, 2 * F, D) / D ** 0.5).to(torch.bfloat16)
        dn = (rnd(E, D, F) / F ** 0.5).to(torch.bfloat16)
        idx, w = ops.moe_route(rnd(T, E), top, 1.0)
        xo = torch.zeros(T, D, device=dev)
        ms = _time(lambda: ops.moe_experts(xo, h, idx, w, gu, dn), 3)
        fl = 2.0 * T * top * 3 * F * D
        if phase == "decode":
            add("moe_experts", phase, ms, fl, min(E, T * top) * 3.0 * F * D * 2, "hbm", "bytes = weights of the experts hit")
        else:
            add("moe_experts", phase, ms, fl, 0.0, "tensor", "mma.sync grouped GEMM")
        del cache, q, x, gu, dn, h
        torch.cuda.empty_cache()
    return rows


def run(size="w2048", layers=4, prefill=4096, batch=32, ctx=2048, reps=5, dense=False):
    from . import models
    import json
    from pathlib import Path
    pk = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    peaks = json.loads(pk.read_text()) if pk.exists() else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    s = SIZES[size]
    cfg = config(size, layers)
    res = {"size": size, "layers": layers, "order": ORDER[:layers], "prefill_tokens": prefill, "decode_batch": batch,
           "decode_context": ctx}
    nblk = (max(prefill, ctx) + 63) // 64
    # ---- the hybrid decoder
    r = models.build_runner(cfg, random_tensors(cfg), dtype=torch.bfloat16, device="cuda", num_blocks=batch * nblk,
                            max_blocks_per_seq=nblk, max_seqs=batch, max_tokens=max(prefill, batch),
                            num_state_slots=batch)
    _say("hybrid runner built")
    for c in r.kv_cache.values():
        c.normal_(std=0.3)
    mp = _meta(1, prefill, prefill, nblk, s["vocab"])
    ms = _time(lambda: r.step(mp, [prefill - 1]), 1, warm=1)
    _say(f"first prefill steps: {ms:.2f} ms")
    ms = _time(lambda: r.step(mp, [prefill - 1]), reps, warm=1)
    res["fidasun"] = {"prefill_ms": ms, "prefill_tok_s": prefill * 1e3 / ms, "launches": int(r.launches_per_step)}
    md = _meta(batch, 1, ctx, nblk, s["vocab"])
    ms = _time(lambda: r.step(md, list(range(batch))), reps * 4, warm=3)
    res["fidasun"].update(decode_ms=ms, decode_tok_s=batch * 1e3 / ms)
    _say(f"fidasun: {res['fidasun']}")
    del r
    torch.cuda.empty_cache()
    # ---- the dense fp16 LLaMA plan at equal width / depth / active feed-forward size.  At these shapes that plan did
    # not return in three of eight runs (in this process or one of its own; the GPU kept answering, the cause is not
    # found), so it runs only when asked for (--dense-arm), in a process of its own with a time limit; otherwise the
    # line carries the numbers of a run in which it answered (profiles/hy_b_bench_fidasun_<size>.json).
    import subprocess
    import sys
    root = Path(__file__).resolve().parent.parent
    if dense:
        try:
            out = subprocess.run([sys.executable, "-m", "vllm_rs_b200.bench_hybrid", size, str(layers), str(prefill),
                                  str(batch), str(ctx), str(reps)], capture_output=True, text=True, timeout=180,
                                 cwd=str(root))
            line = [x for x in out.stdout.splitlines() if x.startswith("{")]
            res["llama_fp16"] = json.loads(line[-1]) if line else {"unavailable": f"exit {out.returncode}: {out.stderr[-300:]}"}
        except subprocess.TimeoutExpired:
            res["llama_fp16"] = {"unavailable": "no answer within 180 s"}
    else:
        res["llama_fp16"] = {"unavailable": "not run (ask with --dense-arm): this arm has stalled at these shapes"}
    if "unavailable" in res["llama_fp16"]:
        rec = root / "profiles" / f"hy_b_bench_fidasun_{size}.json"
        if rec.exists() and (layers, prefill, batch, ctx) == (4, 4096, 32, 2048):
            res["llama_fp16"]["recorded"] = json.loads(rec.read_text())["sizes"][0]["llama_fp16"]
            res["llama_fp16"]["recorded_in"] = f"profiles/{rec.name}"
    _say(f"llama fp16: {res['llama_fp16']}")
    res["kernels"] = kernel_table(size, prefill, batch, ctx, peaks)
    return res


def dense_arm(size, layers, prefill, batch, ctx, reps):
    """Prefill and decode of the dense fp16 LLaMA plan at the width / depth / active feed-forward size of `size`, on a
    stream of its own as the other benches run it."""
    s = SIZES[size]
    nblk = (max(prefill, ctx) + 63) // 64
    H, Hkv, Dh, inter = s["dense"]
    name = f"dense-{size}"
    synthetic.SHAPES[name] = (s["width"], layers, H, Hkv, Dh, inter, s["vocab"], 10000.0)
    lr = synthetic.build_runner(name, "fp16", num_blocks=batch * nblk, max_blocks_per_seq=nblk, max_batch=batch,
                                num_layers=layers, max_prefill_tokens=prefill)
    synthetic.fill_kv_random(lr)
    mp, md = _meta(1, prefill, prefill, nblk, s["vocab"]), _meta(batch, 1, ctx, nblk, s["vocab"])
    meta = dict(input_ids=mp["input_ids"], positions=mp["positions"], slot_mapping=mp["slot_mapping"],
                cu_seqlens_q=mp["cu_seqlens_q"], context_lens=None, block_tables=mp["block_tables"].reshape(1, nblk),
                max_seqlen_q=prefill)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        ms = _time(lambda: lr.prefill_device(meta, want_logits=False), reps, warm=2)
        res = {"prefill_ms": ms, "prefill_tok_s": prefill * 1e3 / ms}
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).astype(dt)).to("cuda")          # noqa: E731
        ids, pos, slot = t(md["input_ids"], np.int32), t(md["positions"], np.int64), t(md["slot_mapping"], np.int64)
        bt, cl = t(md["block_tables"].reshape(batch, nblk), np.int32), t(md["context_lens"], np.int32)
        ms = _time(lambda: lr.decode_device(ids, pos, slot, bt, cl, want_logits=False), reps * 4, warm=3)
        res.update(decode_ms=ms, decode_tok_s=batch * 1e3 / ms, launches=int(lr.launches_per_step))
    return res


if __name__ == "__main__":
    import json as _json
    import sys as _sys
    a = _sys.argv[1:]
    print(_json.dumps(dense_arm(a[0], int(a[1]), int(a[2]), int(a[3]), int(a[4]), int(a[5]))), flush=True)
