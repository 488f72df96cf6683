"""The plain implementation itself (no GPU): properties each of its functions must have."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import TINY, tokens_for

GOLDEN = Path(__file__).parent / "golden"


def test_rms_norm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = plain.rms_norm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    g, u = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64), torch.tensor([5.0, 2.0, 3.0], dtype=torch.float64)
    assert torch.allclose(plain.swiglu(g, u), torch.tensor([0.0, 2 / (1 + math.exp(-1)), -6 / (1 + math.exp(2))], dtype=torch.float64))


def test_rope_is_a_rotation_that_depends_on_the_distance_only():
    torch.manual_seed(0)
    q, k = torch.randn(1, 1, 32, dtype=torch.float64), torch.randn(1, 1, 32, dtype=torch.float64)
    assert torch.allclose(plain.rope(q, [0], 1e4), q)
    assert torch.allclose(plain.rope(q, [37], 1e4).norm(), q.norm())
    d1 = (plain.rope(q, [10], 1e4) * plain.rope(k, [3], 1e4)).sum()
    d2 = (plain.rope(q, [57], 1e4) * plain.rope(k, [50], 1e4)).sum()
    assert abs(d1 - d2) < 1e-5
    # halves are paired: element i with element i + d/2
    x = torch.zeros(1, 1, 8, dtype=torch.float64); x[0, 0, 1] = 1.0
    y = plain.rope(x, [1], 100.0)
    assert y[0, 0, [0, 2, 3, 4, 6, 7]].abs().max() == 0 and abs(y[0, 0, 1] ** 2 + y[0, 0, 5] ** 2 - 1) < 1e-12


def test_attention_mask_window_and_groups():
    torch.manual_seed(1)
    T, nq, nkv, d = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    pos = list(range(T))
    o = plain.attention(q, k, v, pos, pos, 0.3)
    assert torch.allclose(o[0], v[0].repeat_interleave(2, dim=0))                   # the first token sees itself only
    assert torch.allclose(plain.attention(q, k, v, pos, pos, 0.3, window=1), v.repeat_interleave(2, dim=1))
    k2, v2 = k.clone(), v.clone(); k2[5:] += 1.0; v2[5:] -= 2.0
    assert torch.allclose(plain.attention(q, k2, v2, pos, pos, 0.3)[:5], o[:5])     # later keys do not reach earlier queries
    ow = plain.attention(q, k, v, pos, pos, 0.3, window=3)
    k3, v3 = k.clone(), v.clone(); k3[:6] += 5.0; v3[:6] += 5.0
    assert torch.allclose(plain.attention(q, k3, v3, pos, pos, 0.3, window=3)[8], ow[8])  # position 8 sees 6, 7, 8
    # query heads 0, 1 read kv head 0; 2, 3 read kv head 1
    v4 = v.clone(); v4[:, 1] += 1.0
    o4 = plain.attention(q, k, v4, pos, pos, 0.3)
    assert torch.allclose(o4[:, :2], o[:, :2]) and torch.allclose(o4[:, 2:], o[:, 2:] + 1.0)
    # by hand for one query
    s = (q[4, 3] @ k[:5, 1].t()) * 0.3
    assert torch.allclose(o[4, 3], torch.softmax(s, 0) @ v[:5, 1])


@pytest.mark.parametrize("name", list(TINY))
def test_forward_is_causal_and_honours_every_option(name, tiny_models):
    cfg, w = plain.read_model(tiny_models[name])
    ids = tokens_for(name, 40)
    full = plain.forward(cfg, w, ids)
    assert full.shape == (40, cfg["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(plain.forward(cfg, w, ids[:17]), full[:17], atol=1e-9)
    for key, val in (("rms_norm_eps", 0.1), ("rope_theta", 77.0)):
        assert not torch.allclose(plain.forward(dict(cfg, **{key: val}), w, ids), full, atol=1e-4)
    if cfg.get("use_sliding_window"):
        off = dict(cfg, use_sliding_window=False, layer_types=None)
        other = plain.forward(off, w, ids)
        w_ = cfg["sliding_window"]
        assert torch.allclose(other[:w_], full[:w_], atol=1e-9) and not torch.allclose(other[w_ + 8:], full[w_ + 8:], atol=1e-4)


def test_layer_order_as_data(tiny_models):
    cfg, w = plain.read_model(tiny_models["A"])
    ids = tokens_for("A", 12)
    base = plain.forward(cfg, w, ids)
    assert torch.equal(plain.forward(cfg, w, ids, calls=[(0, 0, True), (1, 1, True)]), base)
    twice = plain.forward(cfg, w, ids, calls=[(0, 0, True), (0, 1, True), (1, 2, True)])
    shared = plain.forward(cfg, w, ids, calls=[(0, 0, True), (1, 0, False)])
    assert not torch.allclose(twice, base, atol=1e-4) and not torch.allclose(shared, base, atol=1e-4)


def test_greedy_tie_and_sampler_hash():
    assert plain.greedy(torch.tensor([1.0, 7.0, 7.0, 3.0])) == 1
    from lucciola_b200 import ops
    from lucciola_b200.sampling.sampler import sampling_key
    for key, counter, i in [(0, 0, 0), (12345678901234567890, 7, 151935), (sampling_key(7), 3, 99), ((1 << 64) - 1, 2 ** 31, 1)]:
        assert float(plain.hash_uniform(key, counter, i)) == ops.hash_uniform(key, counter, i)
        assert 0.0 < plain.hash_uniform(key, counter, i) < 1.0
    u = np.array([plain.hash_uniform(sampling_key(1), 0, i) for i in range(4000)])
    assert abs(u.mean() - 0.5) < 0.03 and abs((u < 0.25).mean() - 0.25) < 0.03


def test_every_hash_value_maps_strictly_inside_the_unit_interval():
    """All 2^23 values of the hash's top bits: none maps to 0 or to 1 in float32 (u = 1 would score +infinity in
    -log(-log u) and win whatever the logits are), the Gumbel score of each is finite, and the library's mapping of
    the two extreme inputs is the plain one's."""
    from lucciola_b200.csrc import library
    import ctypes
    u = plain.bits_to_uniform(np.arange(1 << 23, dtype=np.uint32))
    assert u.dtype == np.float32 and u.min() > 0.0 and u.max() < 1.0
    assert u[0] == np.float32(2.0 ** -24) and u[-1] == np.float32(1.0 - 2.0 ** -24)
    assert (np.diff(u) > 0).all()                                       # exact: no two inputs share a value
    score = -np.log(-np.log(u))
    assert np.isfinite(score).all()
    f = library().lb_bits_to_uniform
    f.argtypes, f.restype = [ctypes.c_uint], ctypes.c_float
    for b in (0, 1, (1 << 22), (1 << 23) - 2, (1 << 23) - 1):
        assert f(b) == float(u[b])


def test_temperature_sampling_follows_the_softmax():
    logits = np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    T = 0.8
    p = np.exp(logits / T); p /= p.sum()
    draws = np.bincount([plain.temperature_sample(logits, T, 99, n) for n in range(3000)], minlength=4) / 3000
    assert np.abs(draws - p).max() < 0.03
    assert plain.temperature_sample(logits, 0.0, 99, 5) == 0


def test_golden_outputs_of_the_plain_implementation(tiny_models):
    """Small outputs committed with the script that made them (tests/golden/make_golden.py): a change
    of the plain implementation shows here."""
    gold = json.loads((GOLDEN / "plain_tiny.json").read_text())
    for name in TINY:
        cfg, w = plain.read_model(tiny_models[name])
        ids = tokens_for(name, 24)
        out = plain.forward(cfg, w, ids)
        g = gold[name]
        assert ids == g["tokens"]
        assert np.allclose(out[-1, :8].numpy(), np.array(g["last_row_first8"]), rtol=1e-9, atol=1e-12)
        assert [int(r.argmax()) for r in out[-4:]] == g["argmax_last4"]
