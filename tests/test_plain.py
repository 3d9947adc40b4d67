"""The plain implementation checked against itself and against hand cases (no GPU)."""
import math

import numpy as np
import torch

import helpers
import plain_llama as P
from llama_rs_metal_b200.parts.rope import RotaryEmbedding

F64 = torch.float64


def test_rms_norm_hand_case():
    # x = 1..8, w = 1, eps = 1e-5: first and last values from the reference's own check
    y = P.rms_norm(torch.arange(1, 9, dtype=F64)[None], torch.ones(8, dtype=F64), 1e-5)[0]
    assert abs(y[0].item() - 0.198029) < 1e-6 and abs(y[7].item() - 1.584236) < 1e-6


def test_attention_matches_a_scalar_loop_with_groups_and_window():
    torch.manual_seed(0)
    T, Hq, Hk, d, window = 9, 4, 2, 6, 4
    q, k, v = torch.randn(T, Hq, d, dtype=F64), torch.randn(T, Hk, d, dtype=F64), torch.randn(T, Hk, d, dtype=F64)
    for w in (None, window):
        got = P.attention(q, k, v, window=w)
        for t in range(T):
            for h in range(Hq):
                kh = h // (Hq // Hk)
                keys = [j for j in range(t + 1) if w is None or j > t - w]
                s = [sum(q[t, h, i].item() * k[j, kh, i].item() for i in range(d)) / math.sqrt(d) for j in keys]
                m = max(s)
                p = [math.exp(x - m) for x in s]
                for i in range(d):
                    want = sum(pj * v[j, kh, i].item() for pj, j in zip(p, keys)) / sum(p)
                    assert abs(got[t, h, i].item() - want) < 1e-12


def test_attention_with_zero_keys_is_the_mean_of_values():
    # crates/metal-backend/tests/operations.rs:30-44
    T, d = 5, 4
    v = torch.arange(T * d, dtype=F64).view(T, 1, d)
    out = P.attention(torch.randn(T, 2, d, dtype=F64), torch.zeros(T, 1, d, dtype=F64), v)
    for t in range(T):
        assert torch.allclose(out[t, 0], v[: t + 1, 0].mean(dim=0))


def test_rope_rotates_pairs_split_half_and_keeps_norms():
    x = torch.randn(3, 2, 8, dtype=F64)
    inv = np.array([1.0, 0.1, 0.01], dtype=np.float32)          # rotary 6 of 8: dims 6, 7 pass through
    y = P.rope(x, [0, 5, 9], inv, 6)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 6:], x[..., 6:])
    a = np.float32(5.0) * np.float32(0.1)
    assert abs(y[1, 0, 1].item() - (x[1, 0, 1].item() * math.cos(a) - x[1, 0, 4].item() * math.sin(a))) < 1e-12
    assert abs(y[1, 0, 4].item() - (x[1, 0, 1].item() * math.sin(a) + x[1, 0, 4].item() * math.cos(a))) < 1e-12
    assert torch.allclose(y[..., :6].norm(dim=-1), x[..., :6].norm(dim=-1))


def test_llama3_factors_hit_all_three_branches_and_match_the_engine_table():
    cfg = helpers.TINY["B"]["config"]
    inv = P.rope_inverse_frequencies(cfg, 32)
    base = np.array([500000.0 ** (-2.0 * i / 32) for i in range(16)])
    ratio = base / inv
    assert np.isclose(ratio[0], 1.0) and np.isclose(ratio[-1], 8.0)      # high and low frequency ends
    assert np.any((ratio > 1.0 + 1e-6) & (ratio < 8.0 - 1e-6))           # and the smooth middle
    s = cfg["rope_scaling"]
    part = RotaryEmbedding(32, 32, 500000.0, "llama3", s["factor"], s["low_freq_factor"],
                           s["high_freq_factor"], s["original_max_position_embeddings"])
    assert np.array_equal(np.asarray(part.inverse_frequencies(), dtype=np.float64).astype(np.float32), inv)
    lin = helpers.TINY["C"]["config"]
    assert np.allclose(P.rope_inverse_frequencies(lin, 48),
                       [0.5 * 1000.0 ** (-2.0 * i / 48) for i in range(24)])


def test_forward_is_causal_and_greedy_continuation_is_consistent(plain_models):
    cfg, tensors = plain_models["A"]
    tokens = helpers.random_tokens(1, 12, 256)
    full = P.forward(cfg, tensors, tokens)
    assert full.shape == (12, 256)
    assert torch.allclose(P.forward(cfg, tensors, tokens[:7]), full[:7], atol=1e-12)
    out = P.greedy_continue(cfg, tensors, tokens[:5], 3)
    assert out[0] == P.argmax_lowest(P.forward(cfg, tensors, tokens[:5])[-1])
    cut = out.index(out[-1])                  # the stop id's first appearance ends the sequence
    assert P.greedy_continue(cfg, tensors, tokens[:5], 3, stop_ids=[out[-1]]) == out[:cut]


def test_untied_head_and_norm_weights_matter(plain_models):
    cfg, tensors = plain_models["B"]
    tokens = helpers.random_tokens(8, 6, 512)
    a = P.forward(cfg, tensors, tokens)
    changed = dict(tensors)
    changed["lm_head.weight"] = tensors["lm_head.weight"] * 2
    assert torch.allclose(P.forward(cfg, changed, tokens), a * 2)
    changed = dict(tensors)
    changed["model.layers.1.post_attention_layernorm.weight"] = torch.ones(96, dtype=F64)
    assert not torch.allclose(P.forward(cfg, changed, tokens), a)


def test_argmax_prefers_the_lowest_id():
    assert P.argmax_lowest([1.0, 3.0, 3.0]) == 1
