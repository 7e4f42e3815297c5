"""Fidasun checkpoints -> hybrid.HybridRunner.

config.json: {"architecture": "Fidasun", "width", "vocab", "norm": {"eps"}, "layers": [{"type", "mixer": {...},
"mlp": {...} | null}, ...]}; tensors are named "embed", "l<i>.norm1", "l<i>.mix.*", "l<i>.mlp.*", "final.norm", "head",
linear weights [out, in].  Every layer is parallel: the mixer and the feed-forward read one zero-centred RMS norm of
the stream.  This file only arranges weights for the launch plan (fused input projections, stacked experts, fp32
small parameters, rotary frequencies); the arithmetic is in the CUDA kernels."""
from __future__ import annotations

import torch

from ..hybrid import MIXER_DELTA_RULE, MIXER_LATENT_ATTN, MIXER_SSD, HybridRunner, LayerSpec
from ..rotary import rotary_frequencies
from . import register

_ZERO = dict(heads=0, kv_heads=0, dim=0, rot_dim=0, rot_dims=0, vdim=0, kv_rank=0, window=0, state=0, conv_taps=0,
             norm_groups=0, scale=0.0, rot_mag=1.0, experts=0, top=0, expert_ff=0, shared_ff=0, route_scale=0.0)


@register("Fidasun")
def build(cfg, tensors, *, dtype=torch.bfloat16, device="cuda", num_blocks, max_blocks_per_seq, max_seqs, max_tokens,
          num_state_slots=None, layer_trace=False, **_):
    dtype = dtype or torch.bfloat16
    dev = torch.device(device)

    def mat(*names):                      # matrix-product operand(s), fused along the output rows
        ts = [tensors[n] for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).to(dtype).contiguous().to(dev)

    def vec(*names):                      # small parameters stay fp32
        ts = [tensors[n].to(torch.float32) for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).contiguous().to(dev)

    specs = []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        d, t = dict(_ZERO), {"norm_w": vec(f"l{i}.norm1")}
        if kind == "latent_attention":
            mixer = MIXER_LATENT_ATTN
            rot = m.get("rot") or {}
            rot_dims = int(rot.get("dims", 0))
            d.update(heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], rot_dims=rot_dims, vdim=m["vdim"],
                     kv_rank=m["kv_rank"], window=int((m.get("mask") or {}).get("size", 0)), scale=float(m["scale"]))
            if rot_dims:
                freq, mag = rotary_frequencies(rot_dims, rot["base"], rot.get("scaling"))
                d["rot_mag"] = float(mag)
                t["rot_freq"] = torch.from_numpy(freq).to(torch.float64).contiguous().to(dev)
            t.update(w_in=mat(p + "q", p + "dkv"), w_uk=mat(p + "uk"), w_uv=mat(p + "uv"), w_o=mat(p + "o"),
                     latent_norm_w=vec(p + "dkv.norm"), sink=vec(p + "sink") if p + "sink" in tensors else None)
        elif kind == "delta":
            mixer = MIXER_DELTA_RULE
            d.update(heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), dim=m["dim"], vdim=m["vdim"],
                     conv_taps=m["conv"])
            t.update(w_in=mat(p + "q", p + "k", p + "v", p + "b", p + "a", p + "g"), w_o=mat(p + "o"),
                     conv_w=vec(p + "q.conv", p + "k.conv", p + "v.conv"), a_log=vec(p + "A_log"),
                     dt_bias=vec(p + "dt_bias"), out_norm_w=vec(p + "norm"))
        elif kind == "mamba2":
            mixer = MIXER_SSD
            d.update(heads=m["heads"], kv_heads=m.get("groups", 1), vdim=m["vdim"], state=m["state"],
                     conv_taps=m["conv"], norm_groups=m.get("norm_groups", 1))
            t.update(w_in=mat(p + "in"), w_o=mat(p + "o"), conv_w=vec(p + "conv"), conv_b=vec(p + "conv.b"),
                     a_log=vec(p + "A_log"), dt_bias=vec(p + "dt_bias"), d_skip=vec(p + "D"), out_norm_w=vec(p + "norm"))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = layer.get("mlp")
        if mlp:
            if mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            q, E = f"l{i}.mlp.", int(mlp["router"]["experts"])
            d.update(experts=E, top=int(mlp["router"]["top"]), expert_ff=int(mlp["expert"]["ff"]),
                     route_scale=float(mlp["router"].get("scale", 1.0)))
            t.update(w_router=mat(q + "router"),
                     w_gate_up=torch.stack([mat(f"{q}e{e}.gate", f"{q}e{e}.up") for e in range(E)]).contiguous(),
                     w_down=torch.stack([mat(f"{q}e{e}.down") for e in range(E)]).contiguous())
            if mlp.get("shared"):
                d["shared_ff"] = int(mlp["shared"]["ff"])
                t.update(w_shared_gate_up=mat(q + "shared.gate", q + "shared.up"), w_shared_down=mat(q + "shared.down"))
        specs.append(LayerSpec(mixer, d, t))
    return HybridRunner(width=cfg["width"], vocab=cfg["vocab"], layers=specs, embed=mat("embed"),
                        final_norm=vec("final.norm"), lm_head=mat("head"), norm_eps=float(cfg["norm"]["eps"]),
                        norm_weight_offset=1.0, dtype=dtype, num_blocks=num_blocks,
                        max_blocks_per_seq=max_blocks_per_seq, max_seqs=max_seqs, max_tokens=max_tokens,
                        num_state_slots=num_state_slots or max_seqs, device=device, layer_trace=layer_trace)
