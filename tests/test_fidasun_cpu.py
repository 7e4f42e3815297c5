"""Host-side pieces behind the hybrid decoders: safetensors reading, rotary frequencies, the model registry, state
slots and host-driven (streamed) sequences of the scheduler, and the plain restatement's own invariants."""
import json
import struct

import numpy as np
import pytest
import torch

import fidasun_ref as R
from fidasun_util import full_cfg, layer, make_cfg, random_tensors


def test_safetensors_reader(tmp_path):
    from vllm_rs_b200.weights import read_model_dir
    a = torch.randn(5, 7).to(torch.bfloat16)
    b = torch.arange(6, dtype=torch.int32).reshape(2, 3)
    c = torch.randn(4)
    blobs, header, at = [], {}, 0
    for name, t, dt in (("w.a", a, "BF16"), ("idx", b, "I32"), ("c", c, "F32")):
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else \
            t.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    header["__metadata__"] = {"format": "pt"}
    h = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Fidasun", "width": 7}))
    cfg, ts = read_model_dir(tmp_path)
    assert cfg["width"] == 7
    assert torch.equal(ts["w.a"], a) and torch.equal(ts["idx"], b) and torch.equal(ts["c"], c)


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0},
                                     {"factor": 3.0, "original": 4096, "fast": 32.0, "slow": 1.0}])
def test_rotary_frequencies_match_the_plain_table(scaling):
    from vllm_rs_b200.rotary import rotary_frequencies
    rot = {"base": 5000.0, "dims": 14, "scaling": scaling}
    f, mag = rotary_frequencies(14, 5000.0, scaling)
    pos = [0, 1, 17, 300]
    cos, sin = R.rotary_table(rot, pos)
    assert np.allclose(np.cos(np.outer(pos, f)) * mag, cos.numpy(), atol=1e-12)
    assert np.allclose(np.sin(np.outer(pos, f)) * mag, sin.numpy(), atol=1e-12)
    if scaling is None:
        assert mag == 1.0 and np.allclose(f, 5000.0 ** (-np.arange(7) / 7.0))


def test_registry_knows_the_families():
    from vllm_rs_b200 import models
    names = models.registered()
    assert "Fidasun" in names and "LlamaForCausalLM" in names and "Qwen2ForCausalLM" in names
    assert models.architecture_of({"architectures": ["Qwen2ForCausalLM"]}) == "Qwen2ForCausalLM"
    with pytest.raises(ValueError):
        models.build_runner({"architecture": "Nope"}, {})


def test_streamed_sequences_pages_and_state_slots(lib):
    from vllm_rs_b200 import engine
    s = engine.Scheduler(8, 64, 4, 0, 512)
    assert s.enable_state_slots(3) == 3
    a, b = s.open(), s.open()
    assert (a, b) == (0, 1) and s.num_free_state_slots == 1
    assert s.feed(a, list(range(70))) == 0 and s.feed(b, [5, 6, 7]) == 0
    assert s.num_free_blocks == 5
    m = s.prepare_ragged([s.running_index(a), s.running_index(b)], None, 2, 1024, 8)
    assert m["num_tokens"] == 73 and m["cu_seqlens_q"][:3].tolist() == [0, 70, 73]
    assert m["context_lens"][:2].tolist() == [70, 3] and m["state_slots"][:2].tolist() == [0, 1]
    ta, tb = s.block_table(s.running_index(a)), s.block_table(s.running_index(b))
    assert m["slot_mapping"][63] == ta[0] * 64 + 63 and m["slot_mapping"][64] == ta[1] * 64
    assert m["slot_mapping"][70] == tb[0] * 64 and m["positions"][68:73].tolist() == [68, 69, 0, 1, 2]
    assert s.feed(a, [1]) == 0 and s.feed(b, [9, 9]) == 0
    m = s.prepare_ragged([s.running_index(b), s.running_index(a)], None, 2, 1024, 8)      # other order, only new tokens
    assert m["num_tokens"] == 3 and m["context_lens"][:2].tolist() == [5, 71]
    assert m["positions"][:3].tolist() == [3, 4, 70] and m["input_ids"][:3].tolist() == [9, 9, 1]
    assert s.feed(a, list(range(64 * 7))) == -1 and s.num_free_blocks == 5                # refused: nothing is taken
    c = s.open()
    assert c >= 0 and s.open() == -1                                                      # three slots, all in use
    assert s.close(a) == 0 and s.num_free_blocks == 7 and s.num_free_state_slots == 1
    d = s.open()
    assert s.state_slot(s.running_index(d)) == 0                                          # a's slot, used again
    assert s.feed(d, list(range(64 * 7))) == 0 and s.num_free_blocks == 0
    assert set(s.block_table(s.running_index(d))) >= set(ta)                              # and a's pages


def test_scheduled_sequences_wait_for_a_state_slot(lib):
    from vllm_rs_b200 import engine
    s = engine.Scheduler(16, 64, 8, 0, 32)
    s.enable_state_slots(2)
    for n in (40, 3, 5):
        s.add(list(range(n)), 4)
    ids, pf = s.schedule()
    assert pf and len(ids) == 2 and sorted(s.state_slot(i) for i in ids) == [0, 1]        # the third has no slot yet
    m = s.prepare_ragged(ids, None, 0, 256, 4)
    assert m["num_tokens"] == 32 + 3 and m["context_lens"][:2].tolist() == [32, 3]        # first chunk of 32
    pos, fin = s.filter_prefill_finished(ids)
    assert pos == [1]
    s.postprocess(fin, [7])
    ids, pf = s.schedule()                       # prefill and decode steps alternate: the short one decodes
    assert not pf and len(ids) == 1
    s.postprocess(ids, [8])
    ids, pf = s.schedule()                       # the long prompt's second chunk passes the request that has no slot
    assert pf and len(ids) == 1 and s.num_waiting == 1
    m = s.prepare_ragged(ids, None, 0, 256, 4)
    assert m["num_tokens"] == 8 and m["positions"][:2].tolist() == [32, 33] and m["state_slots"][0] == 0


def test_plain_model_invariants():
    """The restatement itself: causal (a later token cannot change earlier logits), the window forgets, and a
    sequence's logits do not depend on what follows."""
    cfg = make_cfg([layer("latent_attention", mlp=False, mask={"size": 4}), layer("delta"), layer("mamba2")])
    w = random_tensors(cfg, seed=1)
    t = np.random.default_rng(0).integers(0, cfg["vocab"], size=30).tolist()
    full = R.forward(cfg, w, t).numpy()
    part = R.forward(cfg, w, t[:17]).numpy()
    assert np.abs(full[:17] - part).max() < 1e-9
    one = make_cfg([layer("latent_attention", mlp=False, mask={"size": 4})])
    w1 = random_tensors(one, seed=2)
    t2 = list(t)
    t2[10] = (t2[10] + 1) % one["vocab"]
    a, b = R.forward(one, w1, t).numpy(), R.forward(one, w1, t2).numpy()
    assert np.abs(a[13] - b[13]).max() > 1e-6 and np.abs(a[14] - b[14]).max() == 0.0      # 13 sees 10, 14 does not
    assert len(full_cfg()["layers"]) == 5


def test_command_line_lists_the_architectures(capsys):
    from vllm_rs_b200.__main__ import main
    assert main(["models"]) == 0
    assert "Fidasun" in capsys.readouterr().out.split()
