"""Plain, slow restatement of the Fidasun decoder, one function per mechanism, token by token where the
mechanism is a recurrence.  Test infrastructure only: it shares no code with the product path and is written
for clarity, not speed.  Everything runs on the CPU in the dtype of the tensors it is given (tests use
float64 or float32).

Notation: T tokens of ONE sequence, positions 0 .. T-1, width D.  `w` maps tensor names (without the layer
prefix) to tensors; `m` is the layer's `mixer` dictionary of the configuration.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_zero_centred(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


# ----------------------------------------------------------------------------------------------- rotary
def rotary_table(rot, positions, dtype=torch.float64):
    """cos / sin [len(positions), dims/2] for interleaved pairs, with optional YaRN frequency blending."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(ang) * mag).to(dtype), (torch.sin(ang) * mag).to(dtype)


def rotate_pairs(x, cos, sin, dims):
    """x [T, ..., n]; the first `dims` entries are rotated as pairs (2i, 2i+1), the rest pass."""
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = cos.reshape(shape), sin.reshape(shape)
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def latent_attention(h, w, m, eps):
    """Attention over a compressed latent: every head's keys and values are expansions of one cached vector
    per token, plus one rotated key part shared by the heads; sliding window; a per-head sink in the
    softmax denominator."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w["q"].T).reshape(T, H, dn + dr)
    qn, qr = q[..., :dn], q[..., dn:]
    ckr = h @ w["dkv"].T
    c = norm_plain(ckr[:, :r], w["dkv.norm"], eps)
    kr = ckr[:, r:]
    cos, sin = rotary_table(m["rot"], range(T), h.dtype)
    rd = int(m["rot"]["dims"])
    qr = rotate_pairs(qr, cos, sin, rd)
    kr = rotate_pairs(kr, cos, sin, rd)
    kn = (c @ w["uk"].T).reshape(T, H, dn)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    win = m.get("mask", {}).get("size") if m.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = 0 if not win else max(0, i - int(win) + 1)
        for hh in range(H):
            s = (kn[lo:i + 1, hh] @ qn[i, hh] + kr[lo:i + 1] @ qr[i, hh]) * m["scale"]
            sink = w["sink"][hh] if "sink" in w else None
            mx = s.max() if sink is None else torch.maximum(s.max(), sink)
            e = torch.exp(s - mx)
            den = e.sum() + (0.0 if sink is None else torch.exp(sink - mx))
            out[i, hh] = (e / den) @ v[lo:i + 1, hh]
    return out.reshape(T, H * dv) @ w["o"].T


def short_conv_silu(x, taps_w, bias=None):
    """Causal per-channel convolution over time (the last column of taps_w meets the current token;
    zeros before the start) followed by SiLU.  x [T, C], taps_w [C, K]."""
    T, C = x.shape
    K = taps_w.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + pad[j:j + T] * taps_w[:, j][None, :]
    if bias is not None:
        y = y + bias[None, :]
    return F.silu(y)


def delta_mixer(h, w, m, eps):
    """Gated delta rule: a per-head matrix memory that decays, is corrected toward the new value along the
    new key, and is read with the query after the write."""
    T = h.shape[0]
    H, Hk, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w["q"].T, w["q.conv"]).reshape(T, Hk, dk)
    k = short_conv_silu(h @ w["k"].T, w["k.conv"]).reshape(T, Hk, dk)
    v = short_conv_silu(h @ w["v"].T, w["v.conv"]).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)
    g = torch.exp(-torch.exp(w["A_log"]) * F.softplus(h @ w["a"].T + w["dt_bias"]))
    gate = F.silu(h @ w["g"].T).reshape(T, H, dv)
    rep = H // Hk
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        kk, qq = k[:, hh // rep], q[:, hh // rep]
        for t in range(T):
            S = g[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ kk[t])
            S = S + torch.outer(kk[t], u)
            o[t, hh] = S.T @ qq[t]
    o = rms_unit(o, eps) * w["norm"][None, None, :] * gate
    return o.reshape(T, H * dv) @ w["o"].T


def mamba2_mixer(h, w, m, eps):
    """Selective state space with one scalar decay per head (the SSD form of Mamba-2)."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zxbcdt = h @ w["in"].T
    z = zxbcdt[:, :inner]
    xbc = short_conv_silu(zxbcdt[:, inner:2 * inner + 2 * G * N], w["conv"], w["conv.b"])
    dt = F.softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + w["dt_bias"])
    x = xbc[:, :inner].reshape(T, H, P)
    Bm = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    rep = H // G
    y = torch.zeros(T, H, P, dtype=h.dtype)
    A = -torch.exp(w["A_log"])
    for hh in range(H):
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(A[hh] * dt[t, hh]) * S + dt[t, hh] * torch.outer(Bm[t, hh // rep], x[t, hh])
            y[t, hh] = S.T @ Cm[t, hh // rep] + w["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * F.silu(z)
    ng = m["norm_groups"]
    y = rms_unit(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * w["norm"][None, :]
    return y @ w["o"].T


# ----------------------------------------------------------------------------------------------- feed-forward
def gated_ffn(h, gate, up, down):
    return (F.silu(h @ gate.T) * (h @ up.T)) @ down.T


def moe_ffn(h, w, mlp):
    """Softmax router over all experts, the `top` largest scores kept as they are (times a constant, not
    renormalised), plus an always-on shared expert."""
    E, top, scale = mlp["router"]["experts"], mlp["router"]["top"], mlp["router"]["scale"]
    s = torch.softmax(h @ w["router"].T, -1)
    val, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += val[t, j] * scale * gated_ffn(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + gated_ffn(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


# ----------------------------------------------------------------------------------------------- model
MIXERS = {"latent_attention": latent_attention, "delta": delta_mixer, "mamba2": mamba2_mixer}


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, dtype=torch.float64, trace=None):
    """Logits [T, vocab] of one sequence; `trace`, if a list, receives the residual stream after every layer."""
    tn = {k: v.to(dtype) if v.is_floating_point() else v for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = tn["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_zero_centred(x, tn[p + "norm1"], eps)
        y = MIXERS[layer["type"]](h, sub(tn, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp"):
            y = y + moe_ffn(h, sub(tn, p + "mlp."), layer["mlp"])
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    return norm_zero_centred(x, tn["final.norm"], eps) @ tn["head"].T
