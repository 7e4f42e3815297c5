"""Host-side pieces behind the Zalalix decoder: banded rotary frequencies, the model registry, and the plain
restatement's own invariants."""
import numpy as np
import pytest
import torch

import zalalix_ref as R
from zalalix_util import full_cfg, gla_cfg, layer, make_cfg, random_tensors, window_cfg


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64},
                                     {"factor": 3.0, "low": 2.0, "high": 16.0, "original": 4096}])
def test_banded_rotary_frequencies_match_the_plain_table(scaling):
    from vllm_rs_b200.rotary import banded_rotary_frequencies
    f = banded_rotary_frequencies(14, 5000.0, scaling)
    want = R.scaled_frequencies({"base": 5000.0, "dims": 14, "scaling": scaling})
    assert np.allclose(f, want, rtol=1e-13, atol=0)
    if scaling is None:
        assert np.allclose(f, 5000.0 ** (-np.arange(7) / 7.0))
    else:                                                            # all three bands occur
        plain = 5000.0 ** (-np.arange(7) / 7.0)
        assert f[0] == plain[0] and np.isclose(f[-1], plain[-1] / scaling["factor"])
        assert any(plain[i] / scaling["factor"] < f[i] < plain[i] for i in range(7))


def test_registry_knows_the_family():
    from vllm_rs_b200 import models
    assert "Zalalix" in models.registered() and "Zalalix" in models.HYBRID_ARCHITECTURES
    assert models.architecture_of({"architecture": "Zalalix"}) == "Zalalix"


def test_plain_model_invariants():
    """The restatement itself: causal, and with the recurrent side off a token outside the window and the kept first
    tokens cannot change the logits while one inside either can."""
    cfg = full_cfg()
    w = random_tensors(cfg, seed=1)
    t = np.random.default_rng(0).integers(0, cfg["vocab"], size=30).tolist()
    full = R.forward(cfg, w, t).numpy()
    part = R.forward(cfg, w, t[:17]).numpy()
    assert np.abs(full[:17] - part).max() < 1e-9
    one = make_cfg([layer("parallel", mlp=False, left=window_cfg(mask={"size": 4, "keep_first": 2}), right=gla_cfg(),
                          left_scale=1.0, right_scale=0.0)])
    w1 = random_tensors(one, seed=2)
    base = R.forward(one, w1, t).numpy()

    def changed(pos):
        t2 = list(t)
        t2[pos] = (t2[pos] + 1) % one["vocab"]
        return np.abs(R.forward(one, w1, t2).numpy()[-1] - base[-1]).max()

    assert changed(29 - 4) == 0.0 and changed(2) == 0.0              # just outside the window / the kept tokens
    assert changed(29 - 3) > 1e-6 and changed(1) > 1e-6              # just inside


def test_sink_takes_its_share():
    """One visible key whose score is 0: the unit sink halves its weight."""
    m = window_cfg(heads=1, kv_heads=1, dim=2, vdim=3, softcap=None, rot=None, mask=None, scale=1.0)
    w = {"q": torch.zeros(2, 4), "q.b": torch.zeros(2), "k": torch.zeros(2, 4), "k.b": torch.zeros(2),
         "v": torch.zeros(3, 4), "v.b": torch.tensor([2.0, 4.0, 6.0]), "q.norm": torch.ones(2), "k.norm": torch.ones(2),
         "g": torch.zeros(1, 4), "o": torch.eye(3), "o.b": torch.zeros(3)}
    out = R.windowed_attention(torch.ones(1, 4), w, m, 1e-6)
    assert torch.allclose(out, torch.tensor([[0.5, 1.0, 1.5]]))      # softmax share 1/2, gate sigmoid(0) = 1/2
