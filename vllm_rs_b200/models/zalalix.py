"""Zalalix checkpoints -> hybrid.HybridRunner.

config.json: {"architecture": "Zalalix", "width", "vocab", "embedding": {"scale"}, "norm": {"eps"}, "layers": [{"type",
"mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}, ...]}; tensors are named "embed", "l<i>.norm1", "l<i>.norm1b",
"l<i>.norm2", "l<i>.norm2b", "l<i>.mix.*", "l<i>.mlp.{gate,up,down}", "final.norm", "head", linear weights [out, in].
Every sublayer has a plain RMS norm before and after it (sandwich layout).  Mixer types:
  lightning : decayed linear attention, one fixed decay per head, SiLU on q / k / v, one RMS norm over all heads with a
              weight, sigmoid gate
  retention : decayed linear attention, fixed decays, k scaled by dim^-1/2, weightless RMS norm per head, SiLU gate
  parallel  : two mixers side by side -- `left`: softmax attention with grouped K / V heads, biases, whole-projection
              q / k norms, partial interleaved rotary with banded frequency scaling, capped scores, a sliding window
              that keeps the first tokens, a unit sink and a per-head sigmoid gate; `right`: gated linear attention (a
              decay per key channel and token from a low-rank projection), per-head RMS norm with a shared weight, SiLU
              gate -- summed with `left_scale` / `right_scale`.
This file only arranges weights for the launch plan (fused input projections, fp32 small parameters, rotary
frequencies); the arithmetic is in the CUDA kernels."""
from __future__ import annotations

import torch

from ..hybrid import LAYOUT_SANDWICH, MIXER_DECAY_ATTN, MIXER_WINDOW_ATTN, HybridRunner, LayerSpec
from ..rotary import banded_rotary_frequencies
from . import register

_ZERO = dict(heads=0, kv_heads=0, dim=0, rot_dim=0, rot_dims=0, vdim=0, kv_rank=0, window=0, state=0, conv_taps=0,
             norm_groups=0, scale=0.0, rot_mag=1.0, experts=0, top=0, expert_ff=0, shared_ff=0, route_scale=0.0,
             layout=LAYOUT_SANDWICH, keep_first=0, qkv_act=0, gate_act=0, decay_rank=0, out_norm_period=0, softcap=0.0,
             q_scale=1.0, k_scale=1.0, decay_tau=0.0, out_scale=1.0, gated=0)


@register("Zalalix")
def build(cfg, tensors, *, dtype=torch.bfloat16, device="cuda", num_blocks, max_blocks_per_seq, max_seqs, max_tokens,
          num_state_slots=None, layer_trace=False, **_):
    dtype = dtype or torch.bfloat16
    dev = torch.device(device)

    def mat(*names):                      # matrix-product operand(s), fused along the output rows
        ts = [tensors[n] for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).to(dtype).contiguous().to(dev)

    def vec(*names):                      # small parameters stay fp32
        ts = [tensors[n].to(torch.float32).reshape(-1) for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).contiguous().to(dev)

    def decay_attention(p, m, *, qkv_act, gate_act, q_scale, k_scale, groups, norm, out_scale=1.0):
        """Decayed linear attention under prefix p.  `decay` in the mixer's config: one constant per head; otherwise
        (`tau`): per-channel decays from the low-rank pair a1 / a2."""
        H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        d, t = dict(_ZERO), {}
        d.update(heads=H, dim=dk, vdim=dv, qkv_act=qkv_act, gate_act=gate_act, q_scale=q_scale, k_scale=k_scale,
                 norm_groups=groups, out_scale=float(out_scale))
        names = [p + "q", p + "k", p + "v", p + "g"]
        if "decay" in m:
            if len(m["decay"]) != H:
                raise ValueError(f"{p}: {len(m['decay'])} decays for {H} heads")
            t["head_decay"] = torch.tensor([float(x) for x in m["decay"]], dtype=torch.float32, device=dev)
        else:
            d.update(decay_rank=int(tensors[p + "a1"].shape[0]), decay_tau=float(m["tau"]))
            names.append(p + "a1")
            t.update(w_decay2=tensors[p + "a2"].to(torch.float32).contiguous().to(dev), decay_bias=vec(p + "a2.b"))
        if norm:
            t["out_norm_w"] = vec(norm)
            d["out_norm_period"] = int(t["out_norm_w"].numel())
        t.update(w_in=mat(*names), w_o=mat(p + "o"))
        return LayerSpec(MIXER_DECAY_ATTN, d, t)

    def window_attention(p, m, out_scale):
        H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        mask, rot = m.get("mask") or {}, m.get("rot") or {}
        rot_dims = int(rot.get("dims", 0))
        d, t = dict(_ZERO), {}
        d.update(heads=H, kv_heads=G, dim=dk, vdim=dv, rot_dims=rot_dims, window=int(mask.get("size") or 0),
                 keep_first=int(mask.get("keep_first", 0)), scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                 gated=1, out_scale=float(out_scale))
        if rot_dims:
            freq = banded_rotary_frequencies(rot_dims, rot["base"], rot.get("scaling"))
            t["rot_freq"] = torch.from_numpy(freq).to(torch.float64).contiguous().to(dev)
        t.update(w_in=mat(p + "q", p + "k", p + "v", p + "g"), w_o=mat(p + "o"),
                 in_bias=vec(p + "q.b", p + "k.b", p + "v.b"), o_bias=vec(p + "o.b"),
                 q_norm_w=vec(p + "q.norm"), k_norm_w=vec(p + "k.norm"),
                 sink=torch.zeros(H, dtype=torch.float32, device=dev))       # sink logit 0: a unit term in the softmax denominator
        return LayerSpec(MIXER_WINDOW_ATTN, d, t)

    specs = []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        if kind == "lightning":
            spec = decay_attention(p, m, qkv_act=1, gate_act=1, q_scale=1.0, k_scale=1.0, groups=1, norm=p + "norm")
        elif kind == "retention":
            spec = decay_attention(p, m, qkv_act=0, gate_act=0, q_scale=1.0, k_scale=float(m["dim"]) ** -0.5,
                                   groups=int(m["heads"]), norm=None)
        elif kind == "parallel":
            spec = window_attention(p + "left.", m["left"], m.get("left_scale", 1.0))
            r = m["right"]
            spec.side = decay_attention(p + "right.", r, qkv_act=0, gate_act=0, q_scale=float(r["dim"]) ** -0.5,
                                        k_scale=1.0, groups=int(r["heads"]), norm=p + "right.norm",
                                        out_scale=m.get("right_scale", 1.0))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        spec.tensors.update(norm_w=vec(f"l{i}.norm1"), post_norm_w=vec(f"l{i}.norm1b"))
        mlp = layer.get("mlp")
        if mlp:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            q = f"l{i}.mlp."
            spec.dims["shared_ff"] = int(mlp["ff"])
            spec.tensors.update(w_shared_gate_up=mat(q + "gate", q + "up"), w_shared_down=mat(q + "down"),
                                ff_norm_w=vec(f"l{i}.norm2"), ff_post_norm_w=vec(f"l{i}.norm2b"))
        specs.append(spec)
    return HybridRunner(width=cfg["width"], vocab=cfg["vocab"], layers=specs, embed=mat("embed"),
                        final_norm=vec("final.norm"), lm_head=mat("head"), norm_eps=float(cfg["norm"]["eps"]),
                        norm_weight_offset=0.0, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                        dtype=dtype, num_blocks=num_blocks, max_blocks_per_seq=max_blocks_per_seq, max_seqs=max_seqs,
                        max_tokens=max_tokens, num_state_slots=num_state_slots or max_seqs, device=device,
                        layer_trace=layer_trace)
