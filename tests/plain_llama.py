"""A plain, slow Llama 3 decoder: whole sequences, no cache, float64 on the CPU.

This file rests on the reference's formulas, read from its sources: the Rust
crates cannot be compiled or run here (no Rust toolchain, no Metal), so the
model as a whole is not run. Its Metal shaders, however, compile as plain C++
on the CPU with a few definitions; tests/golden/make_golden.py does that and
tests/test_golden.py checks the functions below (norm, products, rotation,
attention, gate, embedding, greedy pick) against the shaders' own arithmetic.
Each function cites the file and lines it restates. It shares no code with the
package: it reads model folders with the `safetensors` library and plain
`json`, and computes with basic torch CPU tensor arithmetic.

Precision: weights are taken as stored and widened to float64; every sum,
softmax and norm is float64. The rotation angle is the one exception by
design: it is `float32(position) * float32(inverse frequency)` as one float32
product, the 32-bit angle the engine's kernels use, so that engine and oracle
rotate by the same angle and differ only by the accuracy of cos/sin.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
def read_model(model_dir):
    """(config dict, {tensor name: float64 tensor}) of a model folder."""
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as handle:
        config = json.load(handle)
    tensors = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name).to(F64)
    return config, tensors


class LazyTensors:
    """Tensors of a model folder read one at a time when asked for, in their stored precision
    (the functions below widen what they use): for models too large to hold in float64 at once."""

    def __init__(self, model_dir):
        from safetensors import safe_open
        self._handle = safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt")
        self._names = set(self._handle.keys())

    def __getitem__(self, name):
        return self._handle.get_tensor(name)

    def __contains__(self, name):
        return name in self._names


def read_model_lazily(model_dir):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as handle:
        return json.load(handle), LazyTensors(model_dir)


# --------------------------------------------------------------------------- parts
def embedding(table, ids):
    """hidden[t,:] = E[ids[t],:]  (crates/metal-backend/src/shaders/matrix.metal:94-103)."""
    return table[torch.as_tensor(ids, dtype=torch.long)].to(F64)


def rms_norm(x, weight, eps):
    """inv = rsqrt(mean(x^2) + eps); y = x * inv * w, row by row
    (crates/metal-backend/src/shaders/elementwise.metal:31-46;
    crates/tensor-core/src/lib.rs:64-70)."""
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * weight.to(F64)


def linear(x, weight):
    """y[t,o] = sum_k W[o,k] x[t,k], no bias
    (crates/metal-backend/src/shaders/matrix.metal:10-37)."""
    return x @ weight.to(F64).T


def rope_scaling_fields(config):
    """theta and the scaling dict as the reference reads them
    (crates/model-format/src/mlx/config.rs:74-92,157-197)."""
    rope = config.get("rope_parameters")
    if rope is None:
        rope = config.get("rope_scaling")
    theta = config.get("rope_theta", 10000.0)
    if isinstance(rope, dict) and "rope_theta" in rope:
        theta = rope["rope_theta"]
    return float(theta), rope if isinstance(rope, dict) else None


def rope_inverse_frequencies(config, rotary):
    """Per pair i: scale * theta^(-2i/R) / factor[i] as a float32 table.

    factor[i] is the llama3 rule (crates/model-format/src/mlx/config.rs:174-194):
    wavelen = 2*pi*theta^(2i/R); wavelen < orig/high -> 1; wavelen > orig/low ->
    factor; else s = (orig/wavelen - low)/(high - low), 1/((1-s)/factor + s).
    The factor divides the angle (crates/metal-backend/src/shaders/attention.metal:18-20);
    `linear` scaling multiplies it by 1/factor (mlx/config.rs:166-172).
    """
    theta, rope = rope_scaling_fields(config)
    kind = "default"
    if rope is not None:
        kind = rope.get("rope_type", rope.get("type", "default"))
    out = []
    for i in range(rotary // 2):
        freq = theta ** (-2.0 * i / rotary)
        if kind == "linear":
            freq *= 1.0 / float(rope.get("factor", 1.0))
        elif kind == "llama3":
            factor = float(rope.get("factor", 1.0))
            low = float(rope.get("low_freq_factor", 1.0))
            high = float(rope.get("high_freq_factor", 4.0))
            orig = float(rope["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi * theta ** (2.0 * i / rotary)
            if wavelen < orig / high:
                f = 1.0
            elif wavelen > orig / low:
                f = factor
            else:
                s = (orig / wavelen - low) / (high - low)
                f = 1.0 / ((1.0 - s) / factor + s)
            freq /= f
        out.append(freq)
    return np.asarray(out, dtype=np.float64).astype(np.float32)


def rope(x, positions, inv_freq, rotary, adjacent=False):
    """Rotation of x [T, heads, d] at the given positions
    (crates/metal-backend/src/shaders/attention.metal:3-25). Split-half (the default):
    pair = j mod R/2; y[pair] = x[pair] cos - x[pair+R/2] sin;
    y[pair+R/2] = x[pair] sin + x[pair+R/2] cos. Adjacent (config key rope_traditional,
    crates/model-format/src/mlx/config.rs:222-226): pair i is (2i, 2i+1), same angles.
    Dims >= R are copied."""
    half = rotary // 2
    pos32 = np.asarray(positions, dtype=np.float32)
    angle = (pos32[:, None] * inv_freq[None, :]).astype(np.float32)  # one float32 product
    angle = torch.from_numpy(angle.astype(np.float64))
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    if adjacent:
        first, second = x[..., 0:rotary:2], x[..., 1:rotary:2]
        out[..., 0:rotary:2] = first * cos - second * sin
        out[..., 1:rotary:2] = first * sin + second * cos
    else:
        first, second = x[..., :half], x[..., half:rotary]
        out[..., :half] = first * cos - second * sin
        out[..., half:rotary] = first * sin + second * cos
    return out


def attention(q, k, v, window=None, scale=None):
    """Causal grouped-query attention of one sequence that starts at position 0.

    q [T,Hq,d], k,v [T,Hk,d]; query t sees keys 0..t, query head h uses key head
    h // (Hq/Hk), score = q.k / sqrt(d), softmax, weighted sum of v
    (crates/metal-backend/src/shaders/attention.metal:28-57; scale at
    crates/metal-backend/src/apple/ops/attention.rs:232). With `window` w a
    query sees only the last w keys (itself included); the reference has no
    window, the parameter serves the library's windowed cache group.
    """
    T, Hq, d = q.shape
    Hk = k.shape[1]
    group = Hq // Hk
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = torch.zeros_like(q)
    t_idx = torch.arange(T)
    allowed = t_idx[None, :] <= t_idx[:, None]
    if window is not None:
        allowed &= t_idx[None, :] > t_idx[:, None] - window
    for h in range(Hq):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].T) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ v[:, kh, :]
    return out


def silu(x):
    """x / (1 + exp(-x))  (crates/tensor-core/src/lib.rs:86-88)."""
    return x / (1.0 + torch.exp(-x))


def gated_mlp(x, gate, up, down):
    """down( silu(x Wg^T) * (x Wu^T) )  (crates/model-runtime/src/execute.rs:251-267;
    crates/metal-backend/src/shaders/elementwise.metal:8-17)."""
    return linear(silu(linear(x, gate)) * linear(x, up), down)


# --------------------------------------------------------------------------- the model
def forward(config, tensors, tokens, window=None, rows=None):
    """Logits [T, vocab] (float64) at every position of one whole sequence, or with `rows` at
    those positions only (the head is the one part whose cost the positions asked for decide).

    Order of operations of crates/model-runtime/src/execute.rs:3-249 (Llama
    branch): embedding; per layer norm -> q,k,v -> rope(q), rope(k) ->
    attention -> o_proj -> add; norm -> gated MLP -> add; final norm; head
    (the embedding again when tie_word_embeddings is true,
    crates/model-runtime/src/loader.rs:64-75). The reference computes the head
    for the last token only; here every position gets logits.
    """
    cfg = config.get("text_config", config)
    h = cfg["hidden_size"]
    Hq = cfg["num_attention_heads"]
    Hk = cfg.get("num_key_value_heads", Hq)
    d = cfg.get("head_dim", h // Hq)
    eps = cfg.get("rms_norm_eps", 1e-5)
    rotary = int(d * cfg.get("partial_rotary_factor", 1.0))
    inv_freq = rope_inverse_frequencies(cfg, rotary)
    adjacent = cfg.get("rope_traditional") is True  # crates/model-format/src/mlx/config.rs:222-226
    T = len(tokens)
    positions = list(range(T))
    hidden = embedding(tensors["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        x = rms_norm(hidden, tensors[p + "input_layernorm.weight"], eps)
        q = linear(x, tensors[p + "self_attn.q_proj.weight"]).view(T, Hq, d)
        k = linear(x, tensors[p + "self_attn.k_proj.weight"]).view(T, Hk, d)
        v = linear(x, tensors[p + "self_attn.v_proj.weight"]).view(T, Hk, d)
        q = rope(q, positions, inv_freq, rotary, adjacent)
        k = rope(k, positions, inv_freq, rotary, adjacent)
        a = attention(q, k, v, window=window).reshape(T, Hq * d)
        hidden = hidden + linear(a, tensors[p + "self_attn.o_proj.weight"])
        x = rms_norm(hidden, tensors[p + "post_attention_layernorm.weight"], eps)
        hidden = hidden + gated_mlp(x, tensors[p + "mlp.gate_proj.weight"],
                                    tensors[p + "mlp.up_proj.weight"],
                                    tensors[p + "mlp.down_proj.weight"])
    if rows is not None:
        hidden = hidden[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rms_norm(hidden, tensors["model.norm.weight"], eps)
    tied = cfg.get("tie_word_embeddings", False)
    head = tensors["model.embed_tokens.weight"] if tied else tensors["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------------------- sampling
def argmax_lowest(logits):
    """Greedy pick, lowest id on ties, -1 when any logit is not finite
    (crates/metal-backend/src/shaders/sampling.metal:39-80; crates/llama-rs/src/sampling.rs:41-48)."""
    values = [float(v) for v in logits]
    if not all(math.isfinite(v) for v in values):
        return -1
    best = max(values)
    return values.index(best)


class SplitMix64:
    """crates/llama-rs/src/sampling.rs:108-120."""

    MASK = (1 << 64) - 1

    def __init__(self, seed):
        self.state = seed & self.MASK

    def uniform(self):
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.MASK
        z ^= z >> 31
        return (z >> 11) / float(1 << 53)


def sample(logits, history, rng, temperature=0.8, top_k=40, top_p=0.95,
           repeat_penalty=1.0, repeat_last_n=64):
    """The reference's sampler, step by step (crates/llama-rs/src/sampling.rs:37-106):
    penalty over the distinct ids of the last `repeat_last_n` history tokens
    (v <= 0 ? v*p : v/p); keep the top_k; sort descending, ties by lower id;
    temperature 0 -> first; p_i = exp((v_i - max)/T) in float64; cut at the
    shortest prefix with cumulative mass >= top_p; r = u * total; first i with
    r < cumulative sum."""
    values = [float(v) for v in logits]
    if not values or any(not math.isfinite(v) for v in values):
        raise ValueError("empty or non-finite logits")
    if temperature == 0.0 and repeat_penalty == 1.0:
        return argmax_lowest(values)
    cand = list(enumerate(values))
    if repeat_penalty != 1.0:
        seen = set()
        for t in list(reversed(history))[:repeat_last_n]:
            if t not in seen:
                seen.add(t)
                if 0 <= t < len(cand):
                    i, v = cand[t]
                    cand[t] = (i, v * repeat_penalty if v <= 0.0 else v / repeat_penalty)
    cand.sort(key=lambda iv: (-iv[1], iv[0]))
    if 0 < top_k < len(cand):
        cand = cand[:top_k]
    if temperature == 0.0:
        return cand[0][0]
    mx = cand[0][1]
    probs = [math.exp((v - mx) / temperature) for _, v in cand]
    total = 0.0
    for p in probs:
        total += p
    acc, keep = 0.0, len(cand)
    for i, p in enumerate(probs):
        acc += p
        if acc / total >= top_p:
            keep = i + 1
            break
    cand, probs = cand[:keep], probs[:keep]
    total = 0.0
    for p in probs:
        total += p
    r = rng.uniform() * total
    acc = 0.0
    for (i, _), p in zip(cand, probs):
        acc += p
        if r < acc:
            return i
    return cand[-1][0]


# --------------------------------------------------------------------------- generation
def greedy_continue(config, tensors, prompt, steps, stop_ids=()):
    """Greedy decoding by recomputing the whole sequence at every step."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(config, tensors, tokens)[-1]
        nxt = argmax_lowest(logits)
        if nxt in stop_ids:
            break
        out.append(nxt)
        tokens.append(nxt)
    return out
