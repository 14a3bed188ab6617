"""`LlamaConfig`: the dense Llama decoder's `config.json`, typed and checked.

Key names are the ones a Llama model folder carries.  The reference's eleven
numbers (include/model.h:58-81: vocab_size, dim, hidden_dim, layers, n_heads,
n_kv_heads, head_dim, max_seq_len, rope_theta, rms_norm_eps, rope_type) map to
vocab_size, hidden_size, intermediate_size, num_hidden_layers,
num_attention_heads, num_key_value_heads, head_dim, max_position_embeddings,
rope_theta, rms_norm_eps and rope_interleaved.  Its checks (src/load.cc:315-363)
are repeated in `validate`; `rope_scaling`, `tie_word_embeddings` and
`attention_bias` go beyond it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, take_bool, take_float, take_int


@dataclass
class RopeScaling:
    """`rope_scaling` of type llama3: frequencies whose wavelength exceeds
    original_max_position_embeddings / low_freq_factor are divided by `factor`,
    those shorter than original / high_freq_factor are kept, the band between
    is blended linearly."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, raw: Any) -> Optional["RopeScaling"]:
        if raw is None:
            return None
        if not isinstance(raw, dict):
            raise ConfigError("config.json: 'rope_scaling' must be an object or null")
        kind = raw.get("rope_type", raw.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(
                f"config.json: rope_scaling type {kind!r} is not supported (known: llama3, default)")
        scaling = cls(
            rope_type="llama3",
            factor=take_float(raw, "factor"),
            low_freq_factor=take_float(raw, "low_freq_factor"),
            high_freq_factor=take_float(raw, "high_freq_factor"),
            original_max_position_embeddings=take_int(raw, "original_max_position_embeddings", minimum=1),
        )
        if scaling.factor < 1.0:
            raise ConfigError("config.json: rope_scaling.factor must be >= 1")
        if not scaling.high_freq_factor > scaling.low_freq_factor > 0:
            raise ConfigError(
                "config.json: rope_scaling needs high_freq_factor > low_freq_factor > 0")
        return scaling

    def to_dict(self) -> Dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass
class LlamaConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    max_position_embeddings: int = 0
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    rope_interleaved: bool = False
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self):
        if not self.architecture:
            self.architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LlamaConfig":
        heads = take_int(raw, "num_attention_heads", minimum=1)
        hidden = take_int(raw, "hidden_size", minimum=1)
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: List[int] = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = [eos]
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = list(eos)
        else:
            raise ConfigError("config.json: 'eos_token_id' must be an integer, a list of integers or null")
        bos = raw.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError("config.json: 'bos_token_id' must be an integer or null")
        if take_bool(raw, "mlp_bias", False):
            raise ConfigError("config.json: mlp_bias=true is not supported (the feed-forward has no bias)")
        dtype = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            # the dtype the folder's tensors are stored in (the reference reads F32 and F16 tensors,
            # include/quantized_tensor.h:37-81); a run converts them to its own dtype when it loads them
            raise ConfigError(f"config.json: torch_dtype {dtype!r} not supported (bfloat16, float16 or float32)")
        act = raw.get("hidden_act", "silu")
        return cls(
            vocab_size=take_int(raw, "vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=take_int(raw, "intermediate_size", minimum=1),
            num_hidden_layers=take_int(raw, "num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            num_key_value_heads=take_int(raw, "num_key_value_heads", default=heads, minimum=1),
            head_dim=take_int(raw, "head_dim", default=max(hidden // heads, 1), minimum=1),
            max_position_embeddings=take_int(raw, "max_position_embeddings", minimum=1),
            rope_theta=take_float(raw, "rope_theta", 10000.0),
            rope_scaling=RopeScaling.from_dict(raw.get("rope_scaling")),
            rope_interleaved=take_bool(raw, "rope_interleaved", False),
            rms_norm_eps=take_float(raw, "rms_norm_eps", 1e-5),
            tie_word_embeddings=take_bool(raw, "tie_word_embeddings", False),
            attention_bias=take_bool(raw, "attention_bias", False),
            hidden_act=act,
            torch_dtype=dtype,
            bos_token_id=bos,
            eos_token_ids=eos_ids,
        )

    def validate(self) -> None:
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act {self.hidden_act!r} not supported (silu)")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not self.rope_theta > 0:
            raise ConfigError("config.json: rope_theta must be > 0")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: rms_norm_eps must be > 0")
        for token in ([self.bos_token_id] if self.bos_token_id is not None else []) + self.eos_token_ids:
            if not 0 <= token < self.vocab_size:
                raise ConfigError(f"config.json: special token id {token} outside the vocabulary")

    def to_dict(self) -> Dict[str, Any]:
        eos: Any = None
        if len(self.eos_token_ids) == 1:
            eos = self.eos_token_ids[0]
        elif self.eos_token_ids:
            eos = list(self.eos_token_ids)
        return {
            "architectures": [self.architecture or "LlamaForCausalLM"],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "rope_interleaved": self.rope_interleaved,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": False,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": eos,
        }
