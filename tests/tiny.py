"""Tiny configurations of the architecture; they differ in every size and option."""
import numpy as np

# 2 layers, 4 heads sharing 2 key/value heads, head size 16, tied head.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 176,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "eos_token_id": 7,
}
# 3 layers, 3 heads on 1 key/value head, head size 32, untied head, other theta and eps.
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "intermediate_size": 256,
    "vocab_size": 384, "rope_theta": 100000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "eos_token_id": [3, 5],
}
# 1 layer, 5 heads with their own key/value heads, an explicit head size (48) that does
# not divide the width (104), odd vocabulary, interleaved rotary pairs, long context.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 104, "num_hidden_layers": 1,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 333, "rope_theta": 500000.0, "rms_norm_eps": 3e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "rope_interleaved": True,
}
# 4 layers of which the first and third see only the last 24 keys (a cache group of their
# own, whose blocks are given back behind the window), 5 heads on 1 key/value head.
TINY_W = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 80, "num_hidden_layers": 4,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 16,
    "intermediate_size": 112, "vocab_size": 200, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "sliding_window": 24,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "W": TINY_W}
SEEDS = {"A": 11, "B": 22, "C": 33, "W": 44}


def tokens(name: str, length: int, seed: int):
    """Uniform token ids for configuration ``name``."""
    rng = np.random.default_rng(1000 * seed + length)
    return rng.integers(0, CONFIGS[name]["vocab_size"], size=length).tolist()
