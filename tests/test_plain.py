"""The plain implementation: against logits of the reference's own CPU forward (tests/golden), and its parts
against closed forms."""
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import qwen2_plain as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_forward_matches_the_reference_cpu_forward():
    cfg, w = P.load(os.path.join(GOLDEN, "model"))
    with open(os.path.join(GOLDEN, "ids.json")) as f:
        ids = json.load(f)
    mine = P.forward(cfg, w, ids).numpy()
    whole = np.load(os.path.join(GOLDEN, "logits_whole.npy"))
    chunked = np.load(os.path.join(GOLDEN, "logits_chunk5.npy"))
    assert whole.shape == mine.shape == (24, 64)
    assert float(np.abs(whole).max()) > 1.0                     # logits far from zero: the comparison means something
    assert float(np.abs(mine - whole).max()) < 1e-5
    assert float(np.abs(mine - chunked).max()) < 1e-5
    assert (mine.argmax(axis=1) == whole.argmax(axis=1)).all()


def test_rope_is_a_rotation_by_position_times_frequency():
    x = torch.randn(5, 3, 16)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = P.rope(x, pos, 10000.0)
    assert torch.equal(y[0], x[0])                               # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    k = 3
    ang = 7 * (10000.0 ** (-2 * k / 16))
    a, b = x[2, 1, k], x[2, 1, k + 8]
    assert math.isclose(float(y[2, 1, k]), float(a) * math.cos(ang) - float(b) * math.sin(ang), abs_tol=1e-5)
    assert math.isclose(float(y[2, 1, k + 8]), float(b) * math.cos(ang) + float(a) * math.sin(ang), abs_tol=1e-5)


def test_attention_mask_groups_and_window():
    t, nh, nkv, hd = 9, 4, 2, 8
    q, k, v = torch.randn(t, nh, hd), torch.randn(t, nkv, hd), torch.randn(t, nkv, hd)
    out = P.attention(q, k, v, 0.5)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])      # first token sees itself
    i, h = 6, 2
    s = torch.tensor([float(q[i, h] @ k[j, 1]) * 0.5 for j in range(i + 1)])
    p = torch.softmax(s, 0)
    assert torch.allclose(out[i, h], (p[:, None] * v[:i + 1, 1]).sum(0), atol=1e-5)
    win = P.attention(q, k, v, 0.5, window=3)
    s = torch.tensor([float(q[i, h] @ k[j, 1]) * 0.5 for j in range(i - 2, i + 1)])
    p = torch.softmax(s, 0)
    assert torch.allclose(win[i, h], (p[:, None] * v[i - 2:i + 1, 1]).sum(0), atol=1e-5)
    assert torch.allclose(win[:3], out[:3], atol=1e-6)            # the window has not started to cut yet


def test_norm_activation_and_sampling():
    x, w = torch.randn(4, 10), torch.randn(10)
    y = P.rms_norm(x, w, 1e-3)
    assert torch.allclose(y, w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3), atol=1e-6)
    g, u = torch.randn(6), torch.randn(6)
    assert torch.allclose(P.swiglu(g, u), u * torch.nn.functional.silu(g), atol=1e-6)
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert P.greedy(logits) == 1
    d = P.sampling_distribution(logits, 1.0, 2, 1.0)
    assert torch.allclose(d, torch.tensor([0.0, 0.5, 0.5, 0.0, 0.0]))
    d = P.sampling_distribution(torch.tensor([0.0, math.log(3.0), math.log(6.0)]), 1.0, 0, 0.65)
    assert torch.allclose(d, torch.tensor([0.0, 1 / 3, 2 / 3]), atol=1e-6)      # 0.6 < 0.65: the second one is needed
    d = P.sampling_distribution(torch.tensor([2.0, 1.0]), 1.0, 0, 1.0, recent=[0], repetition_penalty=2.0)
    assert torch.allclose(d, torch.tensor([0.5, 0.5]))
    assert P.pick_from(torch.tensor([0.25, 0.25, 0.5]), 0.3) == 1 and P.pick_from(torch.tensor([0.25, 0.25, 0.5]), 0.0) == 0


def test_bfloat16_rounding_points_change_little():
    cfg, w = P.load(os.path.join(GOLDEN, "model"))
    with open(os.path.join(GOLDEN, "ids.json")) as f:
        ids = json.load(f)
    a, b = P.forward(cfg, w, ids), P.forward(cfg, w, ids, torch.bfloat16)
    assert 0 < float((a - b).abs().max()) < 0.15


def test_sampling_distribution_matches_the_reference_sampler():
    """``tests/golden/sampler_cases.json``: what tianyuxbear/zedinfer's own GeneralSampler::truncatedDist keeps of a
    row of logits (src/frontend/sampler/sampler.cpp:195-247, compiled unmodified by tests/golden/make_golden.py):
    the same tokens survive top-k and top-p here, with the same renormalised probabilities, after the same
    repetition penalty (applied once per listed token, twice for one that is listed twice) and temperature."""
    with open(os.path.join(GOLDEN, "sampler_cases.json")) as f:
        gold = json.load(f)
    assert len(gold["cases"]) >= 8
    for c in gold["cases"]:
        logits = torch.tensor(c["logits"], dtype=torch.float32)
        d = P.sampling_distribution(logits, c["temperature"], c["top_k"], c["top_p"], recent=c["recent"],
                                    repetition_penalty=c["repetition_penalty"])
        kept = torch.nonzero(d > 0).flatten().tolist()
        assert sorted(kept) == sorted(c["kept_tokens"]), (c["temperature"], c["top_k"], c["top_p"])
        ref = torch.zeros_like(d)
        ref[torch.tensor(c["kept_tokens"])] = torch.tensor(c["kept_probs"], dtype=torch.float32)
        assert float((d - ref).abs().max()) < 1e-6
        # the reference lists what it keeps by falling probability
        assert all(a >= b for a, b in zip(c["kept_probs"], c["kept_probs"][1:]))
