"""The tiny Qwen3 configurations the tests use: A and B differ in every size and option;
C adds a sliding window on its upper layers (cache groups of two kinds in one model); D and E
have the served head size of 128 (E with five heads a group and a window)."""

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=128,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
    max_position_embeddings=512, hidden_act="silu",
)  # fmt: skip
BLOCK_SIZE_A = 16

TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=512, hidden_size=96, intermediate_size=224,
    num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
    rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
    max_position_embeddings=1024, hidden_act="silu",
)  # fmt: skip
BLOCK_SIZE_B = 8

# No power of two anywhere; one kv head serving five query heads; a window of 24 on layers 1..3.
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=331, hidden_size=80, intermediate_size=176,
    num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=1, head_dim=48,
    rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=False,
    max_position_embeddings=2048, hidden_act="silu",
    use_sliding_window=True, sliding_window=24, max_window_layers=1,
)  # fmt: skip
BLOCK_SIZE_C = 16

# Head size 128 with four query heads per kv head, as the served models have it: the shapes that
# run the tensor-core kernels (tcgen05 GEMM and prefill attention, mma.sync decode attention).
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=640, hidden_size=256, intermediate_size=704,
    num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
    max_position_embeddings=4096, hidden_act="silu",
)  # fmt: skip
BLOCK_SIZE_D = 16

# Head size 128 with five query heads per kv head (a group that does not divide the attention
# kernels' 128-row tile, as Qwen3-14B has it) and a window of 40 on layers 1 and 2: the window's
# edges and the released pages through the tensor-core attention kernels.
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=777, hidden_size=320, intermediate_size=528,
    num_hidden_layers=3, num_attention_heads=10, num_key_value_heads=2, head_dim=128,
    rms_norm_eps=2e-6, rope_theta=500000.0, tie_word_embeddings=True,
    max_position_embeddings=4096, hidden_act="silu",
    use_sliding_window=True, sliding_window=40, max_window_layers=1,
)  # fmt: skip
BLOCK_SIZE_E = 8
TINY = {
    "a": (TINY_A, BLOCK_SIZE_A), "b": (TINY_B, BLOCK_SIZE_B), "c": (TINY_C, BLOCK_SIZE_C),
    "d": (TINY_D, BLOCK_SIZE_D), "e": (TINY_E, BLOCK_SIZE_E),
}  # fmt: skip
