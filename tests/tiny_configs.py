"""The tests' own small configurations of the architecture.  A and B differ in every
size and option: layers, width, head counts and groups, head size, inner width (no
power of two), vocabulary, rotary base, the norms' eps, tied or own head, window."""
import torch

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 512, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 128,
    "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 0,
    "max_position_embeddings": 256, "torch_dtype": "bfloat16",
}
# Wider heads, more groups, a window on the upper layers only (two cache groups), a head
# size that is no power of two, a long context for far keys.
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 4, "hidden_size": 120, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 777, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 80, "max_window_layers": 2,
    "max_position_embeddings": 1024, "torch_dtype": "bfloat16",
}
# Head size 64 with a width that differs from heads * head_dim; no window; an own head.
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 136, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 328, "vocab_size": 300, "rope_theta": 20000.0, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": False, "use_sliding_window": False, "max_position_embeddings": 512,
    "torch_dtype": "bfloat16",
}
CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3)}


def make_model_dir(path, cfg_dict, seed, dtype="BF16", shards=1):
    """Writes a model folder with the library's random-weights mode."""
    from friday_inference_engine_b200 import write_model_dir
    return write_model_dir(path, cfg_dict, seed, dtype=dtype, shards=shards)


def random_prompts(lengths, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
