"""The Llama 3 dense decoder's configuration, read from its own config.json keys.

Defaults and rejections follow the reference's parser
(crates/model-format/src/mlx/config.rs:26-239); the llama3 frequency factors
are built in parts/rope.py from the fields kept here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from ..errors import InvalidError, UnsupportedError
from .base import normalize_token_ids, read_bool, read_int, read_real


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` / `rope_parameters` of config.json (mlx/config.rs:157-197)."""

    kind: str = "default"  # "default" | "linear" | "llama3"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    def to_dict(self) -> Optional[dict]:
        if self.kind == "default":
            return None
        out = {"rope_type": self.kind, "factor": self.factor}
        if self.kind == "llama3":
            out.update(
                low_freq_factor=self.low_freq_factor,
                high_freq_factor=self.high_freq_factor,
                original_max_position_embeddings=self.original_max_position_embeddings,
            )
        return out


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rotary_dim: int = 0  # head_dim * partial_rotary_factor
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    rope_adjacent_pairs: bool = False  # config key rope_traditional
    tie_word_embeddings: bool = False
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = "LlamaForCausalLM"
    model_type: str = "llama"

    # -- reading ---------------------------------------------------------------
    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "LlamaConfig":
        text = root.get("text_config", root)  # mlx/config.rs:27
        if not isinstance(text, Mapping):
            raise InvalidError("config.text_config must be an object")
        for flag in ("attention_bias", "mlp_bias"):  # mlx/config.rs:46-50
            if text.get(flag) is True:
                raise UnsupportedError(f"{flag}=true")
        window = text.get("sliding_window")
        if isinstance(window, int) and not isinstance(window, bool) and window > 0:
            raise UnsupportedError("sliding-window attention")  # mlx/config.rs:51-57
        act = text.get("hidden_act")
        if isinstance(act, str) and act != "silu":
            raise UnsupportedError("activation other than SiLU")  # mlx/config.rs:58-64
        # rope_traditional=true pairs adjacent elements (2i, 2i+1); otherwise the halves of a head
        # pair up, as in Hugging Face checkpoints (mlx/config.rs:222-226)
        adjacent = text.get("rope_traditional") is True

        hidden = read_int(text, "hidden_size")
        heads = read_int(text, "num_attention_heads")
        if hidden == 0 or heads == 0 or heads > 1024:
            raise InvalidError("attention dimensions")
        head_dim = read_int(text, "head_dim", hidden // heads)
        kv_heads = read_int(text, "num_key_value_heads", heads)
        layers = read_int(text, "num_hidden_layers")
        vocab = read_int(text, "vocab_size")
        intermediate = read_int(text, "intermediate_size")

        rope = text.get("rope_parameters")
        if rope is None:
            rope = text.get("rope_scaling")
        if not isinstance(rope, Mapping):
            rope = None
        theta = read_real(rope if rope is not None else text, "rope_theta",
                          read_real(text, "rope_theta", 10000.0))
        partial = read_real(rope if rope is not None else text, "partial_rotary_factor",
                            read_real(text, "partial_rotary_factor", 1.0))
        rotary = int(head_dim * partial)
        eps = read_real(text, "rms_norm_eps", 1e-5)
        if (layers == 0 or layers > 1024 or vocab == 0 or head_dim == 0 or head_dim > 512
                or kv_heads == 0 or heads % kv_heads != 0 or rotary == 0 or rotary > head_dim
                or rotary % 2 != 0 or eps <= 0.0 or theta <= 0.0 or intermediate == 0):
            raise InvalidError("invalid model dimensions or normalization")
        types = text.get("layer_types")
        if isinstance(types, list):  # mlx/config.rs:109-119; only full attention is built
            if len(types) != layers or any(t != "full_attention" for t in types):
                raise UnsupportedError("layer_types must be full_attention for every layer")

        scaling = RopeScaling()
        if rope is not None:
            kind = rope.get("rope_type", rope.get("type", "default"))
            if not isinstance(kind, str):
                kind = "default"
            if kind in ("default", "none"):
                pass
            elif kind == "linear":
                factor = read_real(rope, "factor", 1.0)
                if factor <= 0.0:
                    raise InvalidError("RoPE factor")
                scaling = RopeScaling(kind="linear", factor=factor)
            elif kind == "llama3":
                factor = read_real(rope, "factor", 1.0)
                low = read_real(rope, "low_freq_factor", 1.0)
                high = read_real(rope, "high_freq_factor", 4.0)
                original = read_int(rope, "original_max_position_embeddings")
                if factor <= 0.0 or low <= 0.0 or high <= low or original <= 0:
                    raise InvalidError("Llama3 RoPE parameters")
                scaling = RopeScaling("llama3", factor, low, high, original)
            else:
                raise UnsupportedError(f"RoPE type {kind}")

        context = read_int(text, "max_position_embeddings", 8192)
        if context == 0:
            raise InvalidError("zero context capacity")
        archs = root.get("architectures")
        arch = archs[0] if isinstance(archs, list) and archs and isinstance(archs[0], str) \
            else "LlamaForCausalLM"
        bos = text.get("bos_token_id")
        return cls(
            hidden_size=hidden, intermediate_size=intermediate, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            vocab_size=vocab, max_position_embeddings=context, rms_norm_eps=eps,
            rope_theta=theta, rotary_dim=rotary, rope_scaling=scaling, rope_adjacent_pairs=adjacent,
            tie_word_embeddings=read_bool(text, "tie_word_embeddings", False),
            eos_token_ids=normalize_token_ids(text.get("eos_token_id")),
            bos_token_id=bos if isinstance(bos, int) and not isinstance(bos, bool) else None,
            architecture=arch, model_type=str(root.get("model_type", "llama")),
        )

    # -- writing (random-weights mode writes a loadable config.json) ---------
    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict(),
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rotary_dim != self.head_dim:
            out["partial_rotary_factor"] = self.rotary_dim / self.head_dim
        if self.rope_adjacent_pairs:
            out["rope_traditional"] = True
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out
