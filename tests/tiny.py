"""Tiny Qwen2 configurations for the tests.  They differ in every size and option: head counts
and groups, head sizes, widths that are no power of two, number of layers, vocabulary, eps,
theta, tied or separate head, and (C) a window on some layers."""
import os

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 512, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "use_sliding_window": False,
    "max_position_embeddings": 256,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 512,
}
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 80, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 777, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-4, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 24, "max_window_layers": 1, "max_position_embeddings": 384,
}
# group of 6 with head_dim 128, the shape family of the benchmark model, at a small width
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 12, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 328, "vocab_size": 1311, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 1024,
}
# every K of a product a multiple of 32 (the decode step's weight-streaming kernel takes all four products of a
# layer), head_dim 64, group 4, tied head
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 352, "vocab_size": 1500, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "use_sliding_window": False,
    "max_position_embeddings": 1024,
}
# a window on the upper layers with head_dim 128: windowed layers on the tensor-core attention kernels, with
# pages given back behind the window while a request still runs
TINY_F = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 2, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 224, "vocab_size": 901, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 40, "max_window_layers": 1, "max_position_embeddings": 1024,
}
CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 7), "D": (TINY_D, 9), "E": (TINY_E, 12), "F": (TINY_F, 13)}
INIT_SCALE = 4.0
# The tolerances of the engine tests are absolute, for logits of magnitude about 3; E is wider than the others and
# takes a smaller scale to land there.
INIT_SCALES = {"E": 2.8}


def make_model_dir(tmp_root, name, dtype="bfloat16"):
    from zedinfer_b200.weights import write_random_model
    cfg, seed = CONFIGS[name]
    out = os.path.join(str(tmp_root), f"tiny_{name}_{dtype}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(cfg, seed, out, dtype=dtype, init_scale=INIT_SCALES.get(name, INIT_SCALE))
    return out
