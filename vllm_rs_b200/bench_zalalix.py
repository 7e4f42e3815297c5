"""Throughput of the Zalalix decoder at layer sizes that resemble a real model (random weights), next to the closest
existing model of the framework, the Fidasun hybrid decoder, at equal width and depth: `python bench.py --config zalalix`.

Per size: prefill tokens/s (one prompt of `prefill` tokens in one step) and decode tokens/s (`batch` sequences at
context `ctx`, one token each) of both models, CUDA events after warm-up, and a table of the new design's own kernels
timed alone at the same shapes with their algorithmic bytes / flops against the measured copy bandwidth and cuBLAS bf16
peak (the like kernels of the Fidasun plan come from bench_hybrid.kernel_table at the same shapes)."""
from __future__ import annotations

import numpy as np
import torch

from . import bench_hybrid, ops
from .bench_hybrid import _meta, _say, _time

SIZES = {
    # window attention (left) and gated linear attention (right) of a parallel layer, the fixed-decay layers, ff
    "w2048": dict(width=2048, vocab=32000, ff=5632,
                  left=dict(heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep_first=4, rot_dims=64),
                  right=dict(heads=8, dim=128, vdim=256, tau=16.0, rank=16),
                  lightning=dict(heads=16, dim=128, vdim=128), retention=dict(heads=8, dim=128, vdim=256)),
    "w4096": dict(width=4096, vocab=32000, ff=11008,
                  left=dict(heads=32, kv_heads=8, dim=128, vdim=128, window=2048, keep_first=4, rot_dims=64),
                  right=dict(heads=16, dim=128, vdim=256, tau=16.0, rank=32),
                  lightning=dict(heads=32, dim=128, vdim=128), retention=dict(heads=16, dim=128, vdim=256)),
}
ORDER = ["parallel", "parallel", "lightning", "retention"]


def config(size, layers):
    s = SIZES[size]
    le, ri = s["left"], s["right"]
    mix = {"parallel": {"left": dict(heads=le["heads"], kv_heads=le["kv_heads"], dim=le["dim"], vdim=le["vdim"],
                                     scale=le["dim"] ** -0.5, softcap=30.0,
                                     mask={"size": le["window"], "keep_first": le["keep_first"]},
                                     rot={"base": 10000.0, "dims": le["rot_dims"],
                                          "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}),
                        "right": dict(heads=ri["heads"], dim=ri["dim"], vdim=ri["vdim"], tau=ri["tau"]),
                        "left_scale": 1.0, "right_scale": 1.0},
           "lightning": dict(heads=s["lightning"]["heads"], dim=s["lightning"]["dim"], vdim=s["lightning"]["vdim"],
                             decay=[1.0 - 2.0 ** -(5 + i % 4) for i in range(s["lightning"]["heads"])]),
           "retention": dict(heads=s["retention"]["heads"], dim=s["retention"]["dim"], vdim=s["retention"]["vdim"],
                             decay=[1.0 - 2.0 ** -(5 + i % 4) for i in range(s["retention"]["heads"])])}
    mlp = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Zalalix", "width": s["width"], "vocab": s["vocab"], "embedding": {"scale": s["width"] ** 0.5},
            "norm": {"eps": 1e-6},
            "layers": [{"type": ORDER[i % 4], "mixer": mix[ORDER[i % 4]], "mlp": mlp} for i in range(layers)]}


def random_tensors(cfg, size, seed=0):
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}
    lin = lambda n, k: (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)         # noqa: E731
    vec = lambda n, m=0.0, s=0.1: (m + s * torch.randn(n, generator=g)).to(torch.bfloat16)   # noqa: E731
    rank = SIZES[size]["right"]["rank"]

    def decay_attn(p, m, gated):
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        out.update({p + "q": lin(H * dk, D), p + "k": lin(H * dk, D), p + "v": lin(H * dv, D), p + "g": lin(H * dv, D),
                    p + "o": lin(D, H * dv)})
        if gated:
            out.update({p + "a1": lin(rank, D), p + "a2": lin(H * dk, rank), p + "a2.b": vec(H * dk, 3.0, 1.0)})

    out["embed"] = (torch.randn(cfg["vocab"], D, generator=g) / D ** 0.5).to(torch.bfloat16)
    out["head"], out["final.norm"] = lin(cfg["vocab"], D), vec(D, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            out[p + n] = vec(D, 1.0)
        if L["type"] == "lightning":
            decay_attn(p + "mix.", m, False)
            out[p + "mix.norm"] = vec(m["heads"] * m["vdim"], 1.0)
        elif L["type"] == "retention":
            decay_attn(p + "mix.", m, False)
        else:
            a, q = m["left"], p + "mix.left."
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                out[q + n], out[q + n + ".b"] = lin(rows, D), vec(rows)
            out.update({q + "q.norm": vec(H * dk, 1.0), q + "k.norm": vec(G * dk, 1.0), q + "g": lin(H, D),
                        q + "o": lin(D, H * dv), q + "o.b": vec(D)})
            decay_attn(p + "mix.right.", m["right"], True)
            out[p + "mix.right.norm"] = vec(m["right"]["vdim"], 1.0)
        F = L["mlp"]["ff"]
        out.update({p + "mlp.gate": lin(F, D), p + "mlp.up": lin(F, D), p + "mlp.down": lin(D, F)})
    return out


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
        # windowed attention with grouped heads
        le = s["left"]
        H, G, dk, dv, W, K0 = le["heads"], le["kv_heads"], le["dim"], le["vdim"], le["window"], le["keep_first"]
        kc = (rnd(B * nblk, 64, G, dk) * 0.3).to(torch.bfloat16)
        vc = (rnd(B * nblk, 64, G, dv) * 0.3).to(torch.bfloat16)
        bt = i32(np.arange(B * nblk).reshape(B, nblk).tolist())
        q, gate, sink = rnd(T, H, dk) * 0.3, rnd(T, H), torch.zeros(H, device=dev)
        ms = _time(lambda: ops.window_attn(q, kc, vc, sink, gate, cu, cl, bt, window=W, keep_first=K0, scale=dk ** -0.5,
                                           softcap=30.0), 3)
        keys = sum(min(p + 1, W + min(K0, max(0, p + 1 - W))) for p in range(cx_len - q_len, cx_len)) * B
        if phase == "decode":
            add("window_attn", phase, ms, 2.0 * H * keys * (dk + dv), keys * G * (dk + dv) * 2.0, "hbm",
                "bytes = visible K and V rows, read once per key / value head")
        else:
            add("window_attn", phase, ms, 2.0 * H * keys * (dk + dv), 0.0, "tensor", "mma.sync form")
        n_in = H * dk + G * (dk + dv) + H
        proj, bias = rnd(T, n_in), rnd(H * dk + G * (dk + dv))
        qn, kn = rnd(H * dk), rnd(G * dk)
        freq = torch.from_numpy(np.power(10000.0, -np.arange(le["rot_dims"] // 2) * 2.0 / le["rot_dims"])).to(dev)
        pos = torch.arange(cx_len - q_len, cx_len, device=dev).repeat(B)
        slot = ((torch.arange(B, device=dev) * nblk).repeat_interleave(q_len) + pos // 64) * 64 + pos % 64
        ms = _time(lambda: ops.window_attn_prep(proj, bias, qn, kn, freq, pos, slot, kc, vc, heads=H,
                                                rot_dims=le["rot_dims"], eps=1e-6), 3)
        add("window_attn_prep", phase, ms, 0.0, T * (n_in * 4.0 + H * dk * 4.0 + G * (dk + dv) * 2.0), "hbm")
        # decayed linear attention: per-channel decay (the parallel layer's right side) and fixed decay
        for name, m, chan in (("decay_attn (channel decay)", s["right"], True), ("decay_attn (head decay)", s["lightning"], False)):
            Hd, ddk, ddv = m["heads"], m["dim"], m["vdim"]
            qd, kd, vd = rnd(T, Hd, ddk) * 0.3, rnd(T, Hd, ddk) * 0.3, rnd(T, Hd, ddv)
            cd = torch.rand(T, Hd, ddk, generator=g, device=dev) * 0.1 + 0.9 if chan else None
            hd = None if chan else torch.full((Hd,), 0.97, device=dev)
            st = torch.zeros(B, Hd, ddk, ddv, device=dev)
            ms = _time(lambda: ops.decay_attn(qd, kd, vd, st, slots, cu, cl, head_decay=hd, chan_decay=cd), 3)
            if phase == "decode":
                add(name, phase, ms, 4.0 * T * Hd * ddk * ddv, B * Hd * ddk * ddv * 8.0, "hbm", "bytes = state read + write")
            else:
                add(name, phase, ms, 4.0 * T * Hd * ddk * ddv, 0.0, "fp32", "token-serial recurrence")
        ri = s["right"]
        C, rk = ri["heads"] * ri["dim"], ri["rank"]
        low, w2, b2 = rnd(T, rk), rnd(C, rk), rnd(C)
        ms = _time(lambda: ops.lowrank_decay(low, w2, b2, ri["tau"]), 3)
        add("lowrank_decay", phase, ms, 2.0 * T * C * rk, T * (C + rk) * 4.0 + C * rk * 4.0, "hbm")
        x, y, w = rnd(T, s["width"]), rnd(T, s["width"]), rnd(s["width"])
        ms = _time(lambda: ops.resid_add_rmsnorm(x, y, w, 1e-6), 3)
        add("resid_add_rmsnorm", phase, ms, 0.0, T * s["width"] * 12.0, "hbm")
        del kc, vc, q, proj
        torch.cuda.empty_cache()
    return rows


def run(size="w2048", layers=4, prefill=4096, batch=32, ctx=2048, reps=5):
    import json
    from pathlib import Path

    from . import models
    pk = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    peaks = json.loads(pk.read_text()) if pk.exists() else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    s = SIZES[size]
    res = {"size": size, "layers": layers, "order": ORDER[:layers], "prefill_tokens": prefill, "decode_batch": batch,
           "decode_context": ctx}
    nblk = (max(prefill, ctx) + 63) // 64
    mp, md = _meta(1, prefill, prefill, nblk, s["vocab"]), _meta(batch, 1, ctx, nblk, s["vocab"])
    arms = (("zalalix", config(size, layers), lambda c: random_tensors(c, size)),
            ("fidasun", bench_hybrid.config(size, layers), bench_hybrid.random_tensors))
    for name, cfg, make in arms:
        r = models.build_runner(cfg, make(cfg), dtype=torch.bfloat16, device="cuda", num_blocks=batch * nblk,
                                max_blocks_per_seq=nblk, max_seqs=batch, max_tokens=max(prefill, batch),
                                num_state_slots=batch)
        for c in list(r.kv_cache.values()) + list(r.v_cache.values()):
            c.normal_(std=0.3)
        ms = _time(lambda: r.step(mp, [prefill - 1]), 1, warm=1)
        ms = _time(lambda: r.step(mp, [prefill - 1]), reps, warm=1)
        res[name] = {"prefill_ms": ms, "prefill_tok_s": prefill * 1e3 / ms, "launches": int(r.launches_per_step)}
        ms = _time(lambda: r.step(md, list(range(batch))), reps * 4, warm=3)
        res[name].update(decode_ms=ms, decode_tok_s=batch * 1e3 / ms)
        _say(f"{name}: {res[name]}")
        del r
        torch.cuda.empty_cache()
    res["kernels"] = kernel_table(size, prefill, batch, ctx, peaks)
    res["kernels_fidasun"] = bench_hybrid.kernel_table(size, prefill, batch, ctx, peaks)
    return res
