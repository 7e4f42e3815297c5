"""Dense LLaMA / Qwen2 checkpoints (HuggingFace names, fp16 weights) -> engine.ModelRunner (the fp16 launch plan of
csrc/host/model_runner.cpp with `bits = 16`)."""
from __future__ import annotations

import numpy as np
import torch

from .. import engine
from . import register


@register("LlamaForCausalLM", "Qwen2ForCausalLM")
def build(cfg, tensors, *, dtype=torch.float16, device="cuda", num_blocks, max_blocks_per_seq, max_seqs,
          max_tokens=0, **_):
    if dtype not in (torch.float16, None):
        raise ValueError("the dense LLaMA / Qwen2 plan runs in float16")
    H, Hkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    D = cfg.get("head_dim", cfg["hidden_size"] // H)
    bias = "model.layers.0.self_attn.q_proj.bias" in tensors
    r = engine.ModelRunner(hidden=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=H,
                           num_kv_heads=Hkv, head_dim=D, inter=cfg["intermediate_size"], vocab=cfg["vocab_size"],
                           num_blocks=num_blocks, max_blocks_per_seq=max_blocks_per_seq, max_batch=max(max_seqs, 5),
                           bits=16, rms_eps=cfg.get("rms_norm_eps", 1e-5), qkv_bias=bias,
                           max_pos=cfg.get("max_position_embeddings", 8192), max_prefill_tokens=max_tokens,
                           device=device)

    def w(name):
        return tensors[name].to(torch.float16)

    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        kn = lambda n: w(p + n + ".weight").t().contiguous()        # noqa: E731  ([N, K] -> the [K, N] fuse_dense takes)
        qkv_b = None
        if bias:
            qkv_b = torch.cat([w(p + f"self_attn.{n}_proj.bias") for n in "qkv"]).to(device)
        r.set_layer(i, input_norm=w(p + "input_layernorm.weight").to(device),
                    post_norm=w(p + "post_attention_layernorm.weight").to(device),
                    qkv=engine.fuse_dense([kn(f"self_attn.{n}_proj") for n in "qkv"], device),
                    o=engine.fuse_dense([kn("self_attn.o_proj")], device),
                    gate_up=engine.fuse_dense([kn("mlp.gate_proj"), kn("mlp.up_proj")], device),
                    down=engine.fuse_dense([kn("mlp.down_proj")], device), qkv_bias=qkv_b)
    theta = float(cfg.get("rope_theta", 10000.0))
    inv = 1.0 / theta ** (np.arange(0, D, 2, dtype=np.float64) / D)
    ang = np.arange(r.cfg.max_pos, dtype=np.float64)[:, None] * inv[None, :]
    head = tensors.get("lm_head.weight", tensors["model.embed_tokens.weight"])
    r.set_globals(w("model.embed_tokens.weight").to(device), w("model.norm.weight").to(device),
                  head.to(torch.float16).to(device), torch.from_numpy(np.cos(ang)).to(torch.float16).to(device),
                  torch.from_numpy(np.sin(ang)).to(torch.float16).to(device))
    return r
