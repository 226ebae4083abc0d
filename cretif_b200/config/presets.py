"""Named configurations (config.json contents) for the random-weights mode.

Sizes are those the reference's documentation and tests quote for the models it runs
(SmolLM2-135M: tests/test_model.cu:212-235; docs/smollm2_gguf_mapping.md), plus the two tiny
shapes the tests use.  A preset is only a config.json as a dict; nothing else in the library
knows these numbers.
"""
from __future__ import annotations

from typing import Any, Dict


def _llama(**kw) -> Dict[str, Any]:
    base = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
            "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "rope_scaling": None,
            "attention_bias": False, "mlp_bias": False}
    base.update(kw)
    return base


PRESETS: Dict[str, Dict[str, Any]] = {
    "tiny-a": _llama(hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, intermediate_size=176, vocab_size=256,
                     rope_theta=10000.0, max_position_embeddings=128),
    "tiny-b": _llama(hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
                     num_key_value_heads=1, intermediate_size=256, vocab_size=384,
                     rope_theta=100000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                     max_position_embeddings=256),
    "smollm2-135m": _llama(hidden_size=576, num_hidden_layers=30, num_attention_heads=9,
                           num_key_value_heads=3, head_dim=64, intermediate_size=1536,
                           vocab_size=49152, rope_theta=100000.0, max_position_embeddings=8192,
                           bos_token_id=1, eos_token_id=2),
    "smollm2-360m": _llama(hidden_size=960, num_hidden_layers=32, num_attention_heads=15,
                           num_key_value_heads=5, head_dim=64, intermediate_size=2560,
                           vocab_size=49152, rope_theta=100000.0, max_position_embeddings=8192,
                           bos_token_id=1, eos_token_id=2),
    "smollm2-1.7b": _llama(hidden_size=2048, num_hidden_layers=24, num_attention_heads=32,
                           num_key_value_heads=32, head_dim=64, intermediate_size=8192,
                           vocab_size=49152, rope_theta=130000.0, max_position_embeddings=8192,
                           bos_token_id=1, eos_token_id=2),
}


def preset(name: str) -> Dict[str, Any]:
    try:
        return dict(PRESETS[name.lower()])
    except KeyError:
        raise KeyError(f"unknown preset {name!r}; there are {sorted(PRESETS)}") from None
