"""Grouped-query attention over the paged key/value cache."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..errors import InvalidError
from ..kernels import ops
from ..registry import POSITION_ENCODINGS, build_part, register_mixer
from ..weights.loader import TensorSpec
from .base import KeyValueRequest, Mixer, PartSpec
from .linear import LinearWeight


@register_mixer("attention")
class Attention(Mixer):
    """q, k, v projections -> position encoding of q and k -> cache write ->
    causal attention with scale head_dim^-1/2 -> output projection, added to
    the residual stream (crates/model-runtime/src/execute.rs:45-112,196).

    A prompt attends to its own freshly projected keys; a decoded token
    attends to the cache. `window` limits a query to the last `window` keys.
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, window: Optional[int] = None,
                 scale: Optional[float] = None):
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise InvalidError("attention heads must be a multiple of key/value heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.window = head_dim, window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = build_part(POSITION_ENCODINGS, position, "position encoding") \
            if position is not None else None
        self.qkv: Optional[LinearWeight] = None
        self.q_only: Optional[LinearWeight] = None
        self.out: Optional[LinearWeight] = None

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def tensors(self) -> Dict[str, TensorSpec]:
        q, kv, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.hidden_size
        out = {"q_proj.weight": TensorSpec((q, h)), "k_proj.weight": TensorSpec((kv, h)),
               "v_proj.weight": TensorSpec((kv, h)), "o_proj.weight": TensorSpec((h, q))}
        if self.position is not None:
            out.update({"position." + n: s for n, s in self.position.tensors().items()})
        return out

    def bind(self, weights, runtime) -> None:
        # One [q + 2kv, h] matrix: rows of the three projections one after another,
        # so each output element is the same dot product as with separate matrices.
        q_weight, k_weight = weights["q_proj.weight"], weights["k_proj.weight"]
        order = self.position.head_permutation() if self.position is not None else None
        if order is not None:
            # the position scheme wants each head's dimensions reordered: the same reordering of
            # the rows of the query and key projections leaves every score q.k as it was
            index = torch.tensor(order, dtype=torch.long, device=q_weight.device)
            q_weight = q_weight.view(self.num_heads, self.head_dim, -1)[:, index].reshape(q_weight.shape)
            k_weight = k_weight.view(self.num_kv_heads, self.head_dim, -1)[:, index].reshape(k_weight.shape)
        fused = torch.cat([q_weight, k_weight, weights["v_proj.weight"]], dim=0).contiguous()
        self.qkv = LinearWeight(fused)
        self.q_only = LinearWeight(fused[: self.num_heads * self.head_dim])
        self.out = LinearWeight(weights["o_proj.weight"])
        if self.position is not None:
            self.position.bind({n[len("position."):]: t for n, t in weights.items()
                                if n.startswith("position.")}, runtime)

    def cache_request(self):
        return KeyValueRequest(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache, residual):
        entry = ctx.entry
        table = self.position.rotary_table() if self.position is not None else None
        inv_freq, rotary = table if table is not None else (None, 0)
        prefill = ctx.phase == "prefill"
        if entry.writes_cache:
            qkv = self.qkv(x)
            if self.position is not None and table is None:
                qkv = self._apply_other_position(qkv, ctx)
            if (not prefill and cache is not None and qkv.dtype == torch.bfloat16
                    and ops.attention_decode_fused_supported(qkv.dtype, self.head_dim, cache.page_size,
                                                             rotary if inv_freq is not None else 0,
                                                             self.window or cache.window)
                    and ops.attention_decode_prefers_fused(qkv.shape[0], self.num_kv_heads,
                                                           self.num_heads // self.num_kv_heads, self.head_dim,
                                                           ctx.max_kv_len)):
                # rotation, cache write, attention and the merge of the splits in one launch
                mixed = ops.attention_decode_fused(qkv, self.num_heads, inv_freq, rotary, ctx.positions, cache,
                                                   ctx.dest_rows[cache.group], ctx.slots, ctx.kv_lens,
                                                   ctx.max_kv_len, self.scale)
                return self.out(mixed, epilogue=ops.ADD, out=residual)
            q, k, v = ops.rope_store(qkv, self.num_heads, self.num_kv_heads, self.head_dim, inv_freq,
                                     rotary, ctx.positions, kv=cache,
                                     dest_rows=ctx.dest_rows[cache.group] if cache is not None else None,
                                     keep_packed=prefill)
            if prefill:
                ctx.fresh_kv[entry.cache] = (k, v)
        else:
            # this layer reads keys and values another layer stored
            q_proj = self.q_only(x)
            q, _, _ = ops.rope_store(q_proj, self.num_heads, 0, self.head_dim, inv_freq, rotary,
                                     ctx.positions, keep_packed=False)
            if prefill:
                k, v = ctx.fresh_kv[entry.cache]
        if prefill:
            mixed = ops.attention_prefill(q, k, v, ctx.cu_seqlens, ctx.seq_of_token, ctx.max_seq_len,
                                          self.scale, self.window)
        else:
            mixed = ops.attention_decode(q, cache, ctx.slots, ctx.kv_lens, ctx.max_kv_len,
                                         self.scale, self.window)
        return self.out(mixed, epilogue=ops.ADD, out=residual)

    def _apply_other_position(self, qkv, ctx):
        T = qkv.shape[0]
        nq, nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        q = qkv[:, :nq].reshape(T, self.num_heads, self.head_dim)
        k = qkv[:, nq:nq + nk].reshape(T, self.num_kv_heads, self.head_dim)
        q, k = self.position.apply(q, k, ctx)
        return torch.cat([q.reshape(T, nq), k.reshape(T, nk), qkv[:, nq + nk:]], dim=1).contiguous()
