"""Tiny Qwen3 configurations for the tests.  They differ in every size and option:
layers, width, heads and groups (GQA 2, MQA 6, MHA), head size (16, 32, 48),
feed-forward width, vocabulary (a power of two, an even and an odd non-power),
rope base, norm eps, tied or untied output, and the key window (none; some layers)."""
import os
import tempfile

from arle_b200.weights import write_random_model

TINY_A = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512, hidden_act="silu",
              bos_token_id=1, eos_token_id=2)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, intermediate_size=176, vocab_size=500, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024, hidden_act="silu",
              bos_token_id=0, eos_token_id=3)
TINY_C = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=4, hidden_size=72, num_attention_heads=3,
              num_key_value_heads=3, head_dim=48, intermediate_size=100, vocab_size=301, rope_theta=500000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=768, hidden_act="silu",
              use_sliding_window=True, sliding_window=21, max_window_layers=2, bos_token_id=0, eos_token_id=5)
# D has a head size the tensor-core attention kernels take (64), so the engine-level
# tests in bfloat16 run those kernels; one of its layers has a window.
TINY_D = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=136, num_attention_heads=6,
              num_key_value_heads=2, head_dim=64, intermediate_size=200, vocab_size=384, rope_theta=50000.0,
              rms_norm_eps=2e-6, tie_word_embeddings=True, max_position_embeddings=2048, hidden_act="silu",
              sliding_window=70, layer_types=["full_attention", "sliding_attention", "full_attention"],
              bos_token_id=0, eos_token_id=4)
# E has the head size of the large models (128) and widths that are multiples of 32,
# so in bfloat16 every projection of a decode step runs the weight-streaming kernel.
TINY_E = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=192, num_attention_heads=2,
              num_key_value_heads=1, head_dim=128, intermediate_size=320, vocab_size=1000, rope_theta=1000000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu",
              bos_token_id=0, eos_token_id=1)
# F is wider and deeper than the others (a width that is a multiple of 128, four layers, GQA 2, head 64).
TINY_F = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=4, hidden_size=256, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, intermediate_size=416, vocab_size=777, rope_theta=300000.0,
              rms_norm_eps=5e-6, tie_word_embeddings=True, max_position_embeddings=2048, hidden_act="silu",
              bos_token_id=0, eos_token_id=2)
INIT = {"A": dict(sigma=0.02, gain_jitter=0.1), "B": dict(sigma=0.03, gain_jitter=0.2),
        "C": dict(sigma=0.05, gain_jitter=0.15),
        "D": dict(sigma=0.04, gain_jitter=0.1), "E": dict(sigma=0.03, gain_jitter=0.1),
        "F": dict(sigma=0.03, gain_jitter=0.2)}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}
PAGE_SIZES = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 16, "F": 16}
# With small weights a tied model repeats one token for ever, and a test of generation that
# compares such outputs passes for any decode path that gets the first token right.  The
# generation tests therefore use weights large enough that the greedy continuation keeps
# changing, and check that it does (``assert_varied``).
VARIED_INIT = {"A": dict(sigma=0.15), "B": dict(sigma=0.1), "C": dict(sigma=0.15), "D": dict(sigma=0.15),
               "E": dict(sigma=0.06), "F": dict(sigma=0.08)}


def make_model_dir(name: str, seed: int = 0, root: str = None, **init) -> str:
    """Writes the tiny model into a fresh temporary folder and returns it."""
    root = root or tempfile.mkdtemp(prefix=f"arle_tiny_{name}_")
    kw = dict(INIT[name])
    kw.update(init)
    return write_random_model(os.path.join(root, name), CONFIGS[name], seed, **kw)


def make_varied_model_dir(name: str, seed: int = 0, root: str = None) -> str:
    """Like ``make_model_dir`` with the larger weights of ``VARIED_INIT``."""
    return make_model_dir(name, seed, root, **VARIED_INIT[name])


def assert_varied(sequences, least: int = 4) -> None:
    """Every reference continuation must hold at least ``least`` different tokens."""
    for s in sequences:
        assert len(set(s)) >= min(least, len(s)), f"reference continuation {s} is too uniform to test anything"
