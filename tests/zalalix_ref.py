"""Plain, slow restatement of the Zalalix decoder, one function per mechanism, token by token where the mechanism
is a recurrence and key by key where it is attention.  Test infrastructure only: it shares no code with the product
path and is written for clarity, not speed.  Everything runs on the CPU in the dtype it is asked for (tests use
float64).

Notation: T tokens of ONE sequence at positions 0 .. T-1, width D.  `w` maps tensor names without the layer / mixer
prefix to tensors ([out, in] for matrices); `m` is the mixer's dictionary of the configuration.

The layer:   x <- x + N1b(mixer(N1(x)));   x <- x + N2b(ff(N2(x)))  (second line only with a feed-forward),
N(y) = y / sqrt(mean(y^2) + eps) * weight.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------------------------- rotary
def scaled_frequencies(rot):
    """f[i] = base^(-2i/dims); with `scaling` (factor, low, high, original): a pair whose wavelength 2 pi / f is
    shorter than original / high keeps f, one longer than original / low gets f / factor, and in between the two are
    blended with weight s = (original / wavelength - low) / (high - low) on the unscaled one."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x, pos, rot):
    """x [..., n]: vectors at position pos; pairs (2i, 2i+1) of the first rot.dims entries turn by pos * f[i]."""
    f = torch.tensor(scaled_frequencies(rot), dtype=torch.float64)
    dims = 2 * len(f)
    c, s = torch.cos(pos * f).to(x.dtype), torch.sin(pos * f).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def windowed_attention(h, w, m, eps):
    """Softmax attention with grouped key / value heads, biases, a norm over the whole q and k projections, rotary
    on part of each head, capped scores, a sliding window that keeps the first tokens, a unit sink in the
    denominator and a per-head sigmoid gate on the output."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = norm(h @ w["q"].T + w["q.b"], w["q.norm"], eps).reshape(T, H, dk)
    k = norm(h @ w["k"].T + w["k.b"], w["k.norm"], eps).reshape(T, G, dk)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, dv)
    gate = torch.sigmoid(h @ w["g"].T)                                   # [T, H]
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = torch.stack([rotate(q[t], t, rot) for t in range(T)])
        k = torch.stack([rotate(k[t], t, rot) for t in range(T)])
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first", 0))
    cap = m.get("softcap")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        seen = [j for j in range(i + 1) if size is None or i - j < size or j < keep]
        for a in range(H):
            g = a // (H // G)
            s = (k[seen, g] @ q[i, a]) * m["scale"]                      # one score per visible key
            if cap:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s)
            p = e / (1.0 + e.sum())                                      # the sink: score 0, no value
            out[i, a] = (p[:, None] * v[seen, g]).sum(0) * gate[i, a]
    return out.reshape(T, H * dv) @ w["o"].T + w["o.b"]


def decayed_state_readout(q, k, v, decay):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T (the decay multiplies the rows of S, one per key channel),
    o_t = S_t^T q_t, for one head.  q, k [T, dk], v [T, dv], decay [T, dk]."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out)


def lightning(h, w, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q, k, v = silu(h @ w["q"].T).reshape(T, H, dk), silu(h @ w["k"].T).reshape(T, H, dk), silu(h @ w["v"].T).reshape(T, H, dv)
    o = torch.stack([decayed_state_readout(q[:, a], k[:, a], v[:, a],
                                           torch.full((T, dk), float(m["decay"][a]), dtype=h.dtype)) for a in range(H)], 1)
    o = norm(o.reshape(T, H * dv), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def retention(h, w, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w["q"].T).reshape(T, H, dk), (h @ w["k"].T).reshape(T, H, dk) * dk ** -0.5, (h @ w["v"].T).reshape(T, H, dv)
    o = torch.stack([decayed_state_readout(q[:, a], k[:, a], v[:, a],
                                           torch.full((T, dk), float(m["decay"][a]), dtype=h.dtype)) for a in range(H)], 1)
    o = rms_unit(o, eps).reshape(T, H * dv) * silu(h @ w["g"].T)
    return o @ w["o"].T


def gated_linear_attention(h, w, m, eps):
    """Decay per key channel and token: sigmoid(z)^(1/tau), z from a low-rank projection with a bias."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w["q"].T).reshape(T, H, dk) * dk ** -0.5, (h @ w["k"].T).reshape(T, H, dk), (h @ w["v"].T).reshape(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).reshape(T, H, dk)
    o = torch.stack([decayed_state_readout(q[:, a], k[:, a], v[:, a], alpha[:, a]) for a in range(H)], 1)
    o = (rms_unit(o, eps) * w["norm"]).reshape(T, H * dv) * silu(h @ w["g"].T)
    return o @ w["o"].T


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def parallel(h, w, m, eps):
    return (float(m["left_scale"]) * windowed_attention(h, sub(w, "left."), m["left"], eps)
            + float(m["right_scale"]) * gated_linear_attention(h, sub(w, "right."), m["right"], eps))


MIXERS = {"lightning": lightning, "retention": retention, "parallel": parallel}


def dense_ffn(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


# ----------------------------------------------------------------------------------------------- the model
def forward(cfg, tensors, tokens, dtype=torch.float64, trace=None):
    """Logits [T, vocab] of one sequence; `trace` (a list) receives the stream after every layer."""
    W = {k: v.to(dtype) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, L in enumerate(cfg["layers"]):
        w = sub(W, f"l{i}.")
        y = MIXERS[L["type"]](norm(x, w["norm1"], eps), sub(w, "mix."), L["mixer"], eps)
        x = x + norm(y, w["norm1b"], eps)
        if L.get("mlp"):
            if L["mlp"].get("kind", "dense") != "dense":
                raise ValueError("unknown feed-forward kind")
            x = x + norm(dense_ffn(norm(x, w["norm2"], eps), sub(w, "mlp.")), w["norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["head"].T
