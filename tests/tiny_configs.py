"""The tiny configurations the tests run: they differ in every size and option.

A and B are the two tiny models of the build's baseline description; C adds what the architecture's
checkpoint format allows beyond the reference (an explicit head_dim that is not hidden/heads, a
sliding window on the upper layers, no QKV bias). D has heads of 64, three to a key/value head: in
bfloat16 its prompt portions and decoded tokens go through the tensor-core attention kernels.
"""

def _base(**kw):
    d = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "use_sliding_window": False}
    d.update(kw)
    return d


TINY_A = _base(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
               max_position_embeddings=128)
TINY_B = _base(vocab_size=320, hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=3,
               num_key_value_heads=1, rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=False,
               max_position_embeddings=256)
TINY_C = _base(vocab_size=131, hidden_size=80, intermediate_size=72, num_hidden_layers=4, num_attention_heads=6,
               num_key_value_heads=3, head_dim=48, rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=True,
               attention_bias=False, max_position_embeddings=512, use_sliding_window=True, sliding_window=24,
               max_window_layers=2)

TINY_D = _base(vocab_size=200, hidden_size=96, intermediate_size=160, num_hidden_layers=2, num_attention_heads=6,
               num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False,
               max_position_embeddings=256)

SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}
PAGE_SIZES = {"A": 16, "B": 8, "C": 16, "D": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
