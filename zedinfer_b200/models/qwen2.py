"""Qwen2 dense: config.json → typed configuration → :class:`ModelSpec`.

The architecture as the reference runs it (src/frontend/models/transformer_forward.cpp:63-156,
src/frontend/models/qwen2.hpp:29-34): pre-RMSNorm decoder blocks; attention with
grouped KV heads, bias on the q/k/v projections and none on the output projection,
no per-head q/k norm, rotate-half RoPE over the whole head; a SwiGLU feed-forward
without biases; a final RMSNorm; an output head that is the embedding table when
``tie_word_embeddings`` is set (src/frontend/models/base.cpp:411-416).

Keys and defaults follow src/frontend/models/base.cpp:683-720 and :807-813.  The
reference parses ``sliding_window`` / ``max_window_layers`` / ``use_sliding_window``
and then never reads them; here ``use_sliding_window=true`` gives the layers with
index >= ``max_window_layers`` a window of ``sliding_window`` keys (the query's own
position included), which is what the three keys say.  ``rope_scaling`` is refused.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

_REQUIRED = ("hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers",
             "num_attention_heads", "max_position_embeddings")


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    hidden_act: str = "silu"
    bos_token_id: int = 151643
    eos_token_ids: Tuple[int, ...] = (151643,)
    sliding_window: int = 4096
    max_window_layers: int = 21
    use_sliding_window: bool = False

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def to_json_dict(self) -> dict:
        eos = list(self.eos_token_ids)
        return {
            "architectures": ["Qwen2ForCausalLM"],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": self.hidden_act,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": eos[0] if len(eos) == 1 else eos,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "use_sliding_window": self.use_sliding_window,
        }


def _as_int(raw: Mapping[str, Any], key: str, default=None) -> int:
    v = raw.get(key, default)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    return v


def _as_float(raw: Mapping[str, Any], key: str, default: float) -> float:
    v = raw.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


def _as_bool(raw: Mapping[str, Any], key: str, default: bool) -> bool:
    v = raw.get(key, default)
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
    return v


def parse_qwen2_config(raw: Mapping[str, Any]) -> Qwen2Config:
    missing = [k for k in _REQUIRED if k not in raw]
    if missing:
        raise ConfigError("config.json: missing required key(s): " + ", ".join(missing))
    hidden = _as_int(raw, "hidden_size")
    nh = _as_int(raw, "num_attention_heads")
    for key in _REQUIRED:
        if _as_int(raw, key) <= 0:
            raise ConfigError(f"config.json: '{key}' must be positive, got {raw[key]!r}")
    nkv = _as_int(raw, "num_key_value_heads", nh)
    if nkv <= 0 or nh % nkv != 0:
        raise ConfigError(f"config.json: num_attention_heads={nh} must be a positive multiple of "
                          f"num_key_value_heads={nkv}")
    if raw.get("head_dim") is None:
        if hidden % nh != 0:
            raise ConfigError(f"config.json: no 'head_dim', and hidden_size={hidden} is not a multiple of "
                              f"num_attention_heads={nh}")
        head_dim = hidden // nh
    else:
        head_dim = _as_int(raw, "head_dim")
    if head_dim <= 0 or head_dim % 2 != 0:
        raise ConfigError(f"config.json: head_dim={head_dim} must be positive and even (rotate-half RoPE)")
    eps = _as_float(raw, "rms_norm_eps", 1e-6)
    if not eps > 0.0:
        raise ConfigError(f"config.json: rms_norm_eps={eps} must be positive")
    theta = _as_float(raw, "rope_theta", 10000.0)
    if not theta > 0.0:
        raise ConfigError(f"config.json: rope_theta={theta} must be positive")
    if raw.get("rope_scaling") is not None:
        raise ConfigError("config.json: 'rope_scaling' is not supported (the engine rotates with "
                          "unscaled positions only)")
    act = raw.get("hidden_act", "silu")
    if act != "silu":
        raise ConfigError(f"config.json: hidden_act={act!r} is not supported (only 'silu')")
    dtype = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
    if dtype not in ("bfloat16", "float32", "float16"):
        raise ConfigError(f"config.json: torch_dtype={dtype!r} is not one of bfloat16, float16, float32")
    eos_raw = raw.get("eos_token_id", 151643)
    if isinstance(eos_raw, list):
        if not all(isinstance(e, int) and not isinstance(e, bool) for e in eos_raw):
            raise ConfigError(f"config.json: eos_token_id={eos_raw!r} must be an integer or a list of integers")
        eos = tuple(eos_raw)
    elif isinstance(eos_raw, int) and not isinstance(eos_raw, bool):
        eos = (eos_raw,)
    else:
        raise ConfigError(f"config.json: eos_token_id={eos_raw!r} must be an integer or a list of integers")
    use_window = _as_bool(raw, "use_sliding_window", False)
    window_raw = raw.get("sliding_window")
    window = window_raw if isinstance(window_raw, int) and not isinstance(window_raw, bool) else 4096
    if use_window and window <= 0:
        raise ConfigError(f"config.json: sliding_window={window} must be positive when use_sliding_window is true")
    max_window_layers = _as_int(raw, "max_window_layers", 21)
    if max_window_layers < 0:
        raise ConfigError(f"config.json: max_window_layers={max_window_layers} must not be negative")
    return Qwen2Config(
        hidden_size=hidden,
        intermediate_size=_as_int(raw, "intermediate_size"),
        vocab_size=_as_int(raw, "vocab_size"),
        num_hidden_layers=_as_int(raw, "num_hidden_layers"),
        num_attention_heads=nh,
        num_key_value_heads=nkv,
        head_dim=head_dim,
        max_position_embeddings=_as_int(raw, "max_position_embeddings"),
        rms_norm_eps=eps,
        rope_theta=theta,
        tie_word_embeddings=_as_bool(raw, "tie_word_embeddings", False),
        torch_dtype=dtype,
        hidden_act=act,
        bos_token_id=_as_int(raw, "bos_token_id", 151643),
        eos_token_ids=eos,
        sliding_window=window,
        max_window_layers=max_window_layers,
        use_sliding_window=use_window,
    )


def build_qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    ffn = PartSpec("gated_mlp", {"hidden_size": cfg.hidden_size,
                                 "intermediate_size": cfg.intermediate_size,
                                 "activation": cfg.hidden_act, "bias": False})
    layers = []
    for i in range(cfg.num_hidden_layers):
        window = cfg.sliding_window if (cfg.use_sliding_window and i >= cfg.max_window_layers) else None
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qkv_bias": True,
            "out_bias": False,
            "scale": None,           # None: 1/sqrt(head_dim), transformer_forward.cpp:31
            "window": window,
            "position": position,
        })
        layers.append(LayerSpec(
            block="pre_norm", mixer=mixer, ffn=ffn,
            norms={"norm1": norm, "norm2": norm},
            prefixes={"mixer": "self_attn.", "ffn": "mlp.",
                      "norm1": "input_layernorm.", "norm2": "post_attention_layernorm."}))
    return ModelSpec(
        architecture="Qwen2ForCausalLM",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        tie_word_embeddings=cfg.tie_word_embeddings,
        max_position_embeddings=cfg.max_position_embeddings,
        bos_token_id=cfg.bos_token_id,
        eos_token_ids=cfg.eos_token_ids,
    )


QWEN2 = register_architecture("Qwen2ForCausalLM", model_types=("qwen2",),
                              parse=parse_qwen2_config, build_spec=build_qwen2_spec)
