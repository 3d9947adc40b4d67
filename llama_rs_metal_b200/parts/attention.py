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

    A prompt attends to its own freshly projected keys; a decoded token, or a
    portion of several tokens appended to a started sequence, attends to the
    cache. `window` limits a query to the last `window` keys. Which kernels run
    is decided in kernels/attention_dispatch.py (`attend`); a variant mixer
    overrides `before_rotation` to transform q and k per head.
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
        weight = self.qkv if entry.writes_cache else self.q_only
        rotary = self.position.rotary_table() if self.position is not None else None
        # Nothing stands between projection and rotation unless a variant mixer overrides the hook
        # or the position scheme is no rotary table: the kernels may then do both in one launch.
        direct = (type(self).before_rotation is Attention.before_rotation
                  and (self.position is None or rotary is not None) and x.dtype == weight.weight.dtype)
        projected = None if direct else self.before_rotation(weight(x), ctx, entry.writes_cache)
        mixed = ops.attend(projected, q_heads=self.num_heads, kv_heads=self.num_kv_heads,
                           head_dim=self.head_dim, rotary=rotary, ctx=ctx, cache=cache,
                           writes_cache=entry.writes_cache, cache_entry=entry.cache, scale=self.scale,
                           window=self.window, projection=(x, weight.weight) if direct else None)
        return self.out(mixed, epilogue=ops.ADD, out=residual, ctx=ctx)

    def before_rotation(self, projected, ctx, has_keys: bool):
        """Hook between the projection and the kernels: [T, (Hq + 2 Hk) d] when `has_keys`, else
        [T, Hq d] queries. A variant mixer transforms q and k per head here (a norm of each
        head, a bias) and returns the same layout. As built: a position scheme that is not a
        rotary table transforms q and k here."""
        if self.position is None or self.position.rotary_table() is not None:
            return projected
        T = projected.shape[0]
        nq, nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        q = projected[:, :nq].reshape(T, self.num_heads, self.head_dim)
        if not has_keys:
            q, _ = self.position.apply(q, q[:, :0], ctx)
            return q.reshape(T, nq).contiguous()
        k = projected[:, nq:nq + nk].reshape(T, self.num_kv_heads, self.head_dim)
        q, k = self.position.apply(q, k, ctx)
        return torch.cat([q.reshape(T, nq), k.reshape(T, nk), projected[:, nq + nk:]], dim=1).contiguous()
