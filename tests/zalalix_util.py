"""Small Zalalix configurations with random weights, and random schedules of portions.  Test infrastructure; the driver
that feeds portions through the scheduler and the runner is fidasun_util.Driver (it is model-agnostic)."""
from __future__ import annotations

import numpy as np
import torch


def window_cfg(**kw):
    m = dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, softcap=5.0, mask={"size": 11, "keep_first": 3},
             rot={"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}})
    m.update(kw)
    return m


def gla_cfg(**kw):
    m = dict(heads=3, dim=12, vdim=20, tau=8.0)
    m.update(kw)
    return m


def mixer_cfg(kind, **kw):
    if kind == "lightning":
        m = dict(heads=3, dim=20, vdim=24, decay=[0.6, 0.9, 0.99])
    elif kind == "retention":
        m = dict(heads=2, dim=24, vdim=40, decay=[0.95, 0.98])
    else:
        m = dict(left=window_cfg(), right=gla_cfg(), left_scale=1.3, right_scale=0.7)
    m.update(kw)
    return m


def layer(kind, mlp=True, **kw):
    return {"type": kind, "mixer": mixer_cfg(kind, **kw),
            "mlp": ({"kind": "dense", "ff": 40} if mlp is True else (mlp or None))}


def make_cfg(layers, width=48, vocab=96, eps=1e-5, embed_scale=3.0):
    return {"architecture": "Zalalix", "width": width, "vocab": vocab, "embedding": {"scale": embed_scale},
            "norm": {"eps": eps}, "layers": layers}


def full_cfg(**kw):
    """All three layer types, with and without a feed-forward, sizes pairwise different."""
    return make_cfg([layer("parallel"), layer("lightning", mlp=False), layer("retention"),
                     layer("parallel", mlp=False, left=window_cfg(heads=6, kv_heads=1, dim=8, vdim=16,
                                                                  mask={"size": 70, "keep_first": 0}, softcap=None),
                           right=gla_cfg(heads=2, dim=40, vdim=8, tau=3.0), left_scale=0.5, right_scale=2.0)], **kw)


def random_tensors(cfg, seed=0, rank=5):
    """name -> CPU tensor; everything is bf16 (exact in both operand dtypes)."""
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(n, k, gain=1.0):
        return (torch.randn(n, k, generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.2):
        return (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def decay_attn(p, m, gated_decay):
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        out[p + "q"], out[p + "k"], out[p + "v"] = lin(H * dk, D, 2.0), lin(H * dk, D, 2.0), lin(H * dv, D, 2.0)
        out[p + "g"], out[p + "o"] = lin(H * dv, D, 2.0), lin(D, H * dv)
        if gated_decay:
            out[p + "a1"], out[p + "a2"] = lin(rank, D, 2.0), lin(H * dk, rank, 3.0)
            out[p + "a2.b"] = vec(H * dk, 2.0, 1.5)

    out["embed"] = (torch.randn(cfg["vocab"], D, generator=g)).to(torch.bfloat16)
    out["head"] = lin(cfg["vocab"], D)
    out["final.norm"] = vec(D, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"], out[p + "norm1b"] = vec(D, 1.0), vec(D, 1.0)
        if L["type"] == "lightning":
            decay_attn(p + "mix.", m, False)
            out[p + "mix.norm"] = vec(m["heads"] * m["vdim"], 1.0)
        elif L["type"] == "retention":
            decay_attn(p + "mix.", m, False)
        else:
            a, q = m["left"], p + "mix.left."
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                out[q + n] = lin(rows, D, 2.0)
                out[q + n + ".b"] = vec(rows, 0.0, 0.5)
            out[q + "q.norm"], out[q + "k.norm"] = vec(H * dk, 1.0, 0.4), vec(G * dk, 1.0, 0.4)
            out[q + "g"], out[q + "o"], out[q + "o.b"] = lin(H, D, 3.0), lin(D, H * dv), vec(D, 0.0, 0.3)
            decay_attn(p + "mix.right.", m["right"], True)
            out[p + "mix.right.norm"] = vec(m["right"]["vdim"], 1.0)
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            out[p + "norm2"], out[p + "norm2b"] = vec(D, 1.0), vec(D, 1.0)
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = lin(F, D, 2.0), lin(F, D, 2.0), lin(D, F)
    return out


def random_layer(rng, kind):
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]              # noqa: E731
    if kind in ("lightning", "retention"):
        H = pick(1, 2, 5)
        m = dict(heads=H, dim=pick(16, 40, 64, 130), vdim=pick(8, 48, 80), decay=[float(pick(0.5, 0.9, 0.97, 0.999, 1.0)) for _ in range(H)])
    else:
        G = pick(1, 2, 3)
        dk = pick(16, 32, 48, 64)
        rd = pick(0, 2, 8, dk)
        left = dict(heads=G * pick(1, 2, 4, 9), kv_heads=G, dim=dk, vdim=pick(8, 32, 64, 96), scale=pick(0.125, 0.3),
                    softcap=pick(None, 2.0, 30.0),
                    mask=pick(None, {"size": pick(1, 17, 64, 100, 200), "keep_first": pick(0, 1, 5, 64, 70)}),
                    rot=None if rd == 0 else {"base": pick(1e4, 5e5), "dims": rd,
                                              "scaling": pick(None, {"factor": pick(2.0, 8.0), "low": 1.0, "high": pick(2.0, 4.0),
                                                                     "original": pick(16, 64, 4096)})})
        right = dict(heads=pick(1, 2, 4), dim=pick(16, 24, 64, 136), vdim=pick(16, 40, 64), tau=pick(1.0, 4.0, 16.0))
        m = dict(left=left, right=right, left_scale=pick(1.0, 0.7, 1.5), right_scale=pick(1.0, 0.4, 1.1))
    mlp = None if rng.random() < 0.3 else {"kind": "dense", "ff": pick(24, 64, 100)}
    return {"type": kind, "mixer": m, "mlp": mlp}


def random_schedule(rng, reqs):
    """[(portions, requests that end)]: at most four live, portions of 2 .. 300 tokens, the last 20 tokens one by one,
    a live request is sometimes left out of a step."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]              # noqa: E731
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
