"""The plain implementation against the reference's own shader arithmetic.

tests/golden/reference_shaders.npz holds inputs and outputs of the reference's Metal kernels
compiled as plain C++ on the CPU (tests/golden/make_golden.py made it). The shaders compute in
float32, the plain implementation in float64: they must agree to float32 rounding.
"""
import os

import numpy as np
import pytest
import torch

import plain_llama as P

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_shaders.npz"))


def case(name):
    prefix = name + "."
    return {key[len(prefix):]: GOLDEN[key] for key in GOLDEN.files if key.startswith(prefix)}


def bf16_values(bits):
    return torch.from_numpy((bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64))


def close(got, want, tol=2e-5):
    got, want = np.asarray(got, dtype=np.float64).reshape(-1), np.asarray(want, dtype=np.float64).reshape(-1)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("name", ["norm_f32", "norm_bf16"])
def test_rms_norm(name):
    c = case(name)
    rows, width, eps, kind = c["args"]
    x = torch.from_numpy(c["x"].astype(np.float64)).view(int(rows), int(width))
    w = bf16_values(c["w"]) if kind == 30 else torch.from_numpy(c["w"].astype(np.float64))
    close(P.rms_norm(x, w, float(np.float32(eps))), c["y"])


def test_gate_add_embedding():
    c = case("activation")
    close(P.silu(torch.from_numpy(c["a"].astype(np.float64))) * torch.from_numpy(c["b"].astype(np.float64)), c["y"])
    c = case("add")
    close(c["a"].astype(np.float64) + c["b"], c["y"], tol=1e-7)
    c = case("embedding")
    width, row, _ = (int(v) for v in c["args"])
    close(P.embedding(bf16_values(c["w"]).view(-1, width), [row]), c["y"], tol=0.0)


@pytest.mark.parametrize("name", ["gemv_f32", "gemv_bf16"])
def test_linear(name):
    c = case(name)
    tokens, rows, cols = (int(v) for v in c["args"])
    w = bf16_values(c["w"]) if name == "gemv_bf16" else torch.from_numpy(c["w"].astype(np.float64))
    x = torch.from_numpy(c["x"].astype(np.float64)).view(tokens, cols)
    close(P.linear(x, w.view(rows, cols)), c["y"], tol=2e-6 * cols)


@pytest.mark.parametrize("name", ["rope_split", "rope_partial", "rope_adjacent"])
def test_rope(name):
    c = case(name)
    tokens, heads, d, rotary, split, start, theta, scale = c["args"]
    tokens, heads, d, rotary, start = int(tokens), int(heads), int(d), int(rotary), int(start)
    assert (split == 0) == (name == "rope_adjacent")
    # the shader's angle: float(position) * scale * theta^(-2 pair / R) / factors[pair]
    pairs = np.arange(rotary // 2, dtype=np.float64)
    inv = (scale * theta ** (-2.0 * pairs / rotary) / c["factors"].astype(np.float64)).astype(np.float32)
    x = torch.from_numpy(c["x"].astype(np.float64)).view(tokens, heads, d)
    got = P.rope(x, [start + t for t in range(tokens)], inv, rotary, adjacent=split == 0)
    # float32 pow/cos/sin of angles up to a few units: agree to a few float32 ulps of the angle
    close(got, c["y"], tol=5e-5)


def test_prompt_attention():
    c = case("attention_prompt")
    tokens, heads, kv, d, start, scale = c["args"]
    tokens, heads, kv, d = int(tokens), int(heads), int(kv), int(d)
    q = torch.from_numpy(c["q"].astype(np.float64)).view(tokens, heads, d)
    k = torch.from_numpy(c["k"].astype(np.float64)).view(tokens, kv, d)
    v = torch.from_numpy(c["v"].astype(np.float64)).view(tokens, kv, d)
    close(P.attention(q, k, v, scale=float(scale)), c["y"])


def test_attention_over_earlier_keys():
    c = case("attention_continued")
    tokens, heads, kv, d, start, scale = c["args"]
    tokens, heads, kv, d, start = int(tokens), int(heads), int(kv), int(d), int(start)
    total = start + tokens
    q = torch.zeros(total, heads, d, dtype=torch.float64)
    q[start:] = torch.from_numpy(c["q"].astype(np.float64)).view(tokens, heads, d)
    k = torch.from_numpy(c["k"].astype(np.float64)).view(total, kv, d)
    v = torch.from_numpy(c["v"].astype(np.float64)).view(total, kv, d)
    close(P.attention(q, k, v, scale=float(scale))[start:], c["y"])


def test_split_decode_attention():
    c = case("attention_decode")
    heads, kv, d, keys, chunk, scale = c["args"]
    heads, kv, d, keys = int(heads), int(kv), int(d), int(keys)
    q = torch.zeros(keys, heads, d, dtype=torch.float64)
    q[-1] = torch.from_numpy(c["q"].astype(np.float64)).view(heads, d)
    k = torch.from_numpy(c["k"].astype(np.float64)).view(keys, kv, d)
    v = torch.from_numpy(c["v"].astype(np.float64)).view(keys, kv, d)
    close(P.attention(q, k, v, scale=float(scale))[-1], c["y"])


def test_greedy_pick():
    c = case("argmax_tie")
    assert int(c["y"][0]) == 41 == P.argmax_lowest(torch.from_numpy(c["x"]))
    c = case("argmax_nonfinite")
    assert int(c["y"][0]) == -1 == P.argmax_lowest(torch.from_numpy(c["x"]))   # a non-finite logit is flagged
