"""Typed configuration of the Llama dense decoder, read from config.json keys.

Key ↔ reference equivalent (the reference fills ``ModelConfig`` from GGUF
metadata, include/cuinfer/model.h:60-74, src/model.cu:536-548):

=========================  ===================================================
config.json key            reference
=========================  ===================================================
hidden_size                ``{arch}.embedding_length``
num_hidden_layers          ``{arch}.block_count``
num_attention_heads        ``{arch}.attention.head_count``
num_key_value_heads        ``{arch}.attention.head_count_kv`` (default: heads)
head_dim                   fixed ``dim / n_heads`` at src/model.cu:541
intermediate_size          ``{arch}.feed_forward_length``
vocab_size                 ``{arch}.vocab_size`` (src/gguf_parser.cpp:742-759)
max_position_embeddings    ``{arch}.context_length``
rms_norm_eps               default 1e-5 (src/gguf_parser.cpp:730-736)
rope_theta                 default 10000 (src/gguf_parser.cpp:722-728)
tie_word_embeddings        ``output.weight`` absent (src/gguf_parser.cpp:761-765)
eos_token_id/bos_token_id  ``tokenizer.ggml.{eos,bos}_token_id``
sliding_window             none (the reference attends to every earlier key); an
                           integer W lets a query see the last W keys only
layer_types                none; with ``sliding_window``, a list that names each
                           layer ``"sliding_attention"`` or ``"full_attention"``
=========================  ===================================================

Validation follows src/attention.cu:517-540 (heads > 0, even head size, heads
divisible by key/value heads).  The reference has no bias, no rope scaling and
only SiLU; a config that asks for any of these is refused rather than run wrong.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .spec import ModelSpec, PartSpec, ScheduleEntry, prenorm_layer

_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads",
             "intermediate_size", "vocab_size")


@dataclass
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_interleaved: bool = False
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    sliding_window: Optional[int] = None
    layer_types: Optional[List[str]] = None
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architecture: str = "LlamaForCausalLM"

    # derived sizes (include/cuinfer/attention.h:27-34)
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def n_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def validate(self) -> None:
        def positive(name):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size",
                     "max_position_embeddings"):
            positive(name)
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        w = self.sliding_window
        if w is not None and (not isinstance(w, int) or isinstance(w, bool) or w <= 0):
            raise ConfigError(f"sliding_window must be a positive integer or null, got {w!r}")
        if self.layer_types is not None:
            kinds = ("full_attention", "sliding_attention")
            if (not isinstance(self.layer_types, (list, tuple))
                    or len(self.layer_types) != self.num_hidden_layers
                    or any(t not in kinds for t in self.layer_types)):
                raise ConfigError(f"layer_types must name each of the {self.num_hidden_layers} "
                                  f"layers one of {kinds}, got {self.layer_types!r}")
            if w is None and "sliding_attention" in self.layer_types:
                raise ConfigError("layer_types asks for sliding_attention but sliding_window "
                                  "is not given")

    def window_of(self, layer: int) -> int:
        """Keys a query of this layer sees (0: all of them)."""
        if self.sliding_window is None:
            return 0
        if self.layer_types is not None and self.layer_types[layer] != "sliding_attention":
            return 0
        return int(self.sliding_window)

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope_interleaved:
            d["rope_interleaved"] = True
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d


def _as_int(raw, key):
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{key} must be an integer, got {v!r}")
    return v


def llama_config_from_dict(raw: Dict[str, Any]) -> LlamaConfig:
    missing = [k for k in _REQUIRED if k not in raw]
    if missing:
        raise ConfigError(f"config.json lacks required keys: {missing}")
    nh = _as_int(raw, "num_attention_heads")
    hidden = _as_int(raw, "hidden_size")
    if nh <= 0:
        raise ConfigError(f"num_attention_heads must be positive, got {nh}")
    if raw.get("head_dim") is not None:
        hd = _as_int(raw, "head_dim")
    else:
        if hidden % nh:
            raise ConfigError(f"hidden_size {hidden} is not divisible by num_attention_heads "
                              f"{nh} and no head_dim is given")
        hd = hidden // nh
    nkv = raw.get("num_key_value_heads")
    nkv = nh if nkv is None else _as_int(raw, "num_key_value_heads")
    if raw.get("rope_scaling") not in (None, {}):
        raise ConfigError("rope_scaling is not supported (the engine computes plain rotary "
                          f"angles only), got {raw['rope_scaling']!r}")
    for key in ("attention_bias", "mlp_bias"):
        if raw.get(key):
            raise ConfigError(f"{key}=true is not supported (projections have no bias)")
    eos = raw.get("eos_token_id")
    if eos is None:
        eos_ids: List[int] = []
    elif isinstance(eos, int) and not isinstance(eos, bool):
        eos_ids = [eos]
    elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
        eos_ids = list(eos)
    else:
        raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
    cfg = LlamaConfig(
        hidden_size=hidden,
        num_hidden_layers=_as_int(raw, "num_hidden_layers"),
        num_attention_heads=nh,
        num_key_value_heads=nkv,
        head_dim=hd,
        intermediate_size=_as_int(raw, "intermediate_size"),
        vocab_size=_as_int(raw, "vocab_size"),
        max_position_embeddings=int(raw.get("max_position_embeddings", 2048)),
        rms_norm_eps=float(raw.get("rms_norm_eps", 1e-5)),
        rope_theta=float(raw.get("rope_theta", 10000.0)),
        rope_interleaved=bool(raw.get("rope_interleaved", False)),
        tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
        hidden_act=str(raw.get("hidden_act", "silu")),
        sliding_window=raw.get("sliding_window"),
        layer_types=raw.get("layer_types"),
        eos_token_ids=eos_ids,
        bos_token_id=raw.get("bos_token_id"),
        torch_dtype=raw.get("torch_dtype"),
        architecture=(raw.get("architectures") or ["LlamaForCausalLM"])[0],
    )
    cfg.validate()
    for t in cfg.eos_token_ids:
        if not 0 <= t < cfg.vocab_size:
            raise ConfigError(f"eos_token_id {t} is outside the vocabulary [0, {cfg.vocab_size})")
    return cfg


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    """Every layer: RMSNorm → rotary GQA attention → RMSNorm → SwiGLU (src/model.cu:887-1018)."""
    norm = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps})
    position = {"kind": "rotary", "theta": cfg.rope_theta, "rotary_dim": cfg.head_dim,
                "pairing": "interleaved" if cfg.rope_interleaved else "half"}
    def mixer(i: int) -> PartSpec:
        return PartSpec("attention", {
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "scale": cfg.head_dim ** -0.5,       # 1/sqrt(hd), src/attention.cu:690-692
            "window": cfg.window_of(i),          # 0: causal over all keys, as the reference
            "position": position,
            "names": {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                      "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight"},
        })
    ffn = PartSpec("gated_mlp", {
        "intermediate_size": cfg.intermediate_size,
        "activation": cfg.hidden_act,
        "names": {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
                  "down": "mlp.down_proj.weight"},
    })
    layers = [
        prenorm_layer(f"model.layers.{i}.", mixer(i), ffn,
                      PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps,
                                           "name": "input_layernorm.weight"}),
                      PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps,
                                           "name": "post_attention_layernorm.weight"}))
        for i in range(cfg.num_hidden_layers)
    ]
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        embedding=PartSpec("token_embedding", {"name": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"eps": norm.params["eps"], "name": "model.norm.weight"}),
        head=PartSpec("linear_head", {"tied": cfg.tie_word_embeddings,
                                      "name": "lm_head.weight",
                                      "tied_to": "model.embed_tokens.weight"}),
        max_positions=cfg.max_position_embeddings,
        stop_token_ids=list(cfg.eos_token_ids),
        bos_token_id=cfg.bos_token_id,
    )


register_architecture("LlamaForCausalLM", llama_config_from_dict, build_llama_spec)
