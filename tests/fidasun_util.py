"""Small Fidasun configurations with random weights, and a driver that feeds token portions through the framework's
scheduler (streamed sequences), block manager, state slots and runner.  Test infrastructure."""
from __future__ import annotations

import numpy as np
import torch


def mixer_cfg(kind, **kw):
    if kind == "latent_attention":
        m = dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, mask={"size": 11},
                 rot={"base": 10000.0, "dims": 6,
                      "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}})
    elif kind == "delta":
        m = dict(heads=4, kv_heads=2, dim=24, vdim=40, conv=3)
    else:
        m = dict(heads=4, groups=2, vdim=24, state=20, conv=5, norm_groups=2)
    m.update(kw)
    return m


def mlp_cfg(experts=6, top=2, ff=24, shared_ff=40, scale=1.75):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff},
            "shared": {"ff": shared_ff} if shared_ff else None}


def make_cfg(layers, width=48, vocab=96, eps=1e-5):
    return {"architecture": "Fidasun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def layer(kind, mlp=True, **kw):
    return {"type": kind, "mixer": mixer_cfg(kind, **kw), "mlp": (mlp_cfg() if mlp is True else (mlp or None))}


def full_cfg(**kw):
    """All three mixers, each with experts, sizes pairwise different."""
    return make_cfg([layer("mamba2"), layer("latent_attention"), layer("delta"), layer("latent_attention", mlp=False),
                     layer("mamba2", groups=1, norm_groups=1, conv=2)], **kw)


def random_tensors(cfg, seed=0):
    """name -> CPU tensor; matrix weights are bf16 (exact in both operand dtypes), integer-free."""
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(n, k, gain=1.0):
        return (torch.randn(n, k, generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.2):
        return (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    out["embed"] = (torch.randn(cfg["vocab"], D, generator=g)).to(torch.bfloat16)
    out["head"] = lin(cfg["vocab"], D)
    out["final.norm"] = vec(D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = vec(D)
        if L["type"] == "latent_attention":
            H = m["heads"]
            out[p + "mix.q"] = lin(H * (m["dim"] + m["rot_dim"]), D, 2.0)
            out[p + "mix.dkv"] = lin(m["kv_rank"] + m["rot_dim"], D, 2.0)
            out[p + "mix.dkv.norm"] = vec(m["kv_rank"], 1.0)
            out[p + "mix.uk"] = lin(H * m["dim"], m["kv_rank"], 2.0)
            out[p + "mix.uv"] = lin(H * m["vdim"], m["kv_rank"])
            out[p + "mix.sink"] = vec(H, 0.0, 1.0)
            out[p + "mix.o"] = lin(D, H * m["vdim"])
        elif L["type"] == "delta":
            H, Hk = m["heads"], m["kv_heads"]
            for n, rows in (("q", Hk * m["dim"]), ("k", Hk * m["dim"]), ("v", H * m["vdim"])):
                out[p + f"mix.{n}"] = lin(rows, D, 2.0)
                out[p + f"mix.{n}.conv"] = vec(rows * m["conv"], 0.0, 0.6).reshape(rows, m["conv"])
            out[p + "mix.b"] = lin(H, D, 2.0)
            out[p + "mix.a"] = lin(H, D, 2.0)
            out[p + "mix.A_log"] = vec(H, -0.5, 0.7)
            out[p + "mix.dt_bias"] = vec(H, -1.0, 0.7)
            out[p + "mix.norm"] = vec(m["vdim"], 1.0)
            out[p + "mix.g"] = lin(H * m["vdim"], D, 2.0)
            out[p + "mix.o"] = lin(D, H * m["vdim"])
        else:
            H, inner, GN = m["heads"], m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + "mix.in"] = lin(2 * inner + 2 * GN + H, D, 2.0)
            out[p + "mix.conv"] = vec((inner + 2 * GN) * m["conv"], 0.0, 0.6).reshape(inner + 2 * GN, m["conv"])
            out[p + "mix.conv.b"] = vec(inner + 2 * GN, 0.0, 0.3)
            out[p + "mix.dt_bias"] = vec(H, -1.0, 0.7)
            out[p + "mix.A_log"] = vec(H, -0.5, 0.7)
            out[p + "mix.D"] = vec(H, 1.0, 0.3)
            out[p + "mix.norm"] = vec(inner, 1.0)
            out[p + "mix.o"] = lin(D, inner)
        mlp = L.get("mlp")
        if mlp:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            out[p + "mlp.router"] = lin(E, D, 3.0)
            for e in range(E):
                out[p + f"mlp.e{e}.gate"] = lin(F, D, 2.0)
                out[p + f"mlp.e{e}.up"] = lin(F, D, 2.0)
                out[p + f"mlp.e{e}.down"] = lin(D, F)
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                out[p + "mlp.shared.gate"] = lin(Fs, D, 2.0)
                out[p + "mlp.shared.up"] = lin(Fs, D, 2.0)
                out[p + "mlp.shared.down"] = lin(D, Fs)
    return out


class Driver:
    """Feeds portions of requests through Scheduler (open / feed / prepare_ragged / close) and HybridRunner.step,
    as the trace runner and the engine do; collects the logits of every fed position."""

    def __init__(self, cfg, tensors, dtype=torch.float32, num_blocks=16, max_seqs=4, slots=4, trace=False):
        from vllm_rs_b200 import engine, models
        self.runner = models.build_runner(cfg, tensors, dtype=dtype, device="cuda", num_blocks=num_blocks,
                                          max_blocks_per_seq=num_blocks, max_seqs=max_seqs,
                                          max_tokens=num_blocks * 64, num_state_slots=slots, layer_trace=trace)
        self.sched = engine.Scheduler(num_blocks, 64, max_seqs, 0, num_blocks * 64)
        self.sched.enable_state_slots(slots)
        self.num_blocks = num_blocks
        self.live, self.logits = {}, {}

    def step(self, portions):
        """portions: [(request name, token list)]; every fed position's logits are kept in self.logits[name]."""
        ids, rows = [], 0
        for name, toks in portions:
            if name not in self.live:
                sid = self.sched.open()
                assert sid >= 0, "no free state slot"
                self.live[name] = sid
                self.logits[name] = []
            assert self.sched.feed(self.live[name], toks) == 0, "out of pages"
            ids.append(self.sched.running_index(self.live[name]))
            rows += len(toks)
        meta = self.sched.prepare_ragged(ids, None, 2, self.runner.cfg.max_tokens, self.num_blocks,
                                         pinned=self.runner.pinned)
        lg, _ = self.runner.step(meta, list(range(rows)), want_logits=True, want_ids=False)
        at = 0
        for name, toks in portions:
            self.logits[name].append(lg[at:at + len(toks)].copy())
            at += len(toks)

    def close(self, name):
        self.sched.close(self.live.pop(name))

    def result(self, name):
        return np.concatenate(self.logits[name], 0)


def rel_err(got, want, q=1.0):
    """Row error (root mean square over the vocabulary) relative to the spread of the expected logits: the largest
    over the rows, or their q-quantile (bf16 runs with a top-1 router may flip a near-tied choice at single rows)."""
    want = np.asarray(want, dtype=np.float64)
    d = np.asarray(got, dtype=np.float64) - want
    return float(np.quantile(np.sqrt((d ** 2).mean(-1)), q) / want.std())
