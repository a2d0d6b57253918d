"""The small configurations the tests run on.  A and B differ in every size and option; C adds a
sliding window on some layers; D has head size 64, which with pages of 64 tokens takes the engine
through the TMA decode kernel and the tcgen05 prefill kernel, with a window on its second layer; E
has head size 128 and room for prompts of more than a thousand tokens; all have sizes that are no
power of two somewhere."""

TINY_A = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
  num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
  rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=128, tie_word_embeddings=True,
  attention_bias=False, use_sliding_window=False, hidden_act="silu", initializer_range=0.02)

TINY_B = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
  num_attention_heads=8, num_key_value_heads=1, head_dim=32, intermediate_size=160, vocab_size=512,
  rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=256, tie_word_embeddings=False,
  attention_bias=False, use_sliding_window=False, hidden_act="silu", initializer_range=0.02)

# windowed layers beside full ones, 3 query heads per kv head, head_dim 48, vocabulary 1000
TINY_C = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
  num_attention_heads=6, num_key_value_heads=2, head_dim=48, intermediate_size=176, vocab_size=1000,
  rope_theta=50000.0, rms_norm_eps=1e-5, max_position_embeddings=512, tie_word_embeddings=True,
  attention_bias=False, use_sliding_window=True, sliding_window=40, max_window_layers=2,
  hidden_act="silu", initializer_range=0.02)

# head size 64, two query heads per kv head, a window of 100 on the second of two layers
TINY_D = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=72,
  num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=144, vocab_size=333,
  rope_theta=20000.0, rms_norm_eps=1e-6, max_position_embeddings=512, tie_word_embeddings=False,
  attention_bias=False, use_sliding_window=True, sliding_window=100, max_window_layers=1,
  hidden_act="silu", initializer_range=0.02)

# head size 128 and room for prompts of more than a thousand tokens: what a step of many rows runs
# through (the tcgen05 gate-and-up product, the many-token form of the QK-norm/rotation kernel)
TINY_E = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=136,
  num_attention_heads=2, num_key_value_heads=1, head_dim=128, intermediate_size=200, vocab_size=300,
  rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=2048, tie_word_embeddings=True,
  attention_bias=False, use_sliding_window=False, hidden_act="silu", initializer_range=0.02)

# eight query heads per kv head (the grouping of the Qwen3-32B shape, 64 / 8) with head size 128 on a narrow model
TINY_F = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=264,
  num_attention_heads=16, num_key_value_heads=2, head_dim=128, intermediate_size=520, vocab_size=1003,
  rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=False,
  attention_bias=False, use_sliding_window=False, hidden_act="silu", initializer_range=0.02)

# the layer sizes of Qwen3-0.6B (the shape the benchmark times), two of its 28 layers
QWEN3_06B_2_OF_28_LAYERS = dict(
  architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=1024,
  num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
  rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=True,
  attention_bias=False, use_sliding_window=False, hidden_act="silu", initializer_range=0.02)

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F, "R": QWEN3_06B_2_OF_28_LAYERS}
