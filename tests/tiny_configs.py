"""The tiny configurations that the tests run: two of the architecture that
differ in every size and option, and helpers to draw prompts."""
import torch

ARCH = ["Lfm2ForCausalLM"]

TINY_A = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
    num_key_value_heads=2, vocab_size=256, block_ff_dim=192, block_auto_adjust_ff_dim=False,
    layer_types=["conv", "full_attention", "conv", "full_attention"], rope_theta=10000.0, norm_eps=1e-5,
    conv_L_cache=3, conv_bias=False, tie_embedding=True)

TINY_B = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=96, num_hidden_layers=6, num_attention_heads=3,
    num_key_value_heads=1, vocab_size=384, block_ff_dim=384, block_auto_adjust_ff_dim=True,
    block_multiple_of=64, block_ffn_dim_multiplier=1.0,
    layer_types=["full_attention", "conv", "conv", "full_attention", "conv", "full_attention"],
    rope_theta=1000000.0, norm_eps=1e-6, conv_L_cache=4, conv_bias=True, tie_embedding=False)

# sizes that are no power of two anywhere: width 80 = 5 heads of 16, 5:1 groups... ff 144, vocab 301
TINY_C = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=240, num_hidden_layers=3, num_attention_heads=5,
    num_key_value_heads=5, vocab_size=301, block_ff_dim=200, block_auto_adjust_ff_dim=False,
    layer_types=["full_attention", "conv", "full_attention"], rope_theta=50000.0, norm_eps=1e-5,
    conv_L_cache=2, conv_bias=False, tie_embedding=True, rope_style="half_split")

# awkward sizes: a feed-forward width (100) and a vocabulary (131) that are multiples of nothing, as many kv
# heads as heads, a wide convolution, one layer kind only at the start
TINY_D = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=112, num_hidden_layers=3, num_attention_heads=7,
    num_key_value_heads=7, vocab_size=131, block_ff_dim=100, block_auto_adjust_ff_dim=False,
    layer_types=["conv", "conv", "full_attention"], rope_theta=777.0, norm_eps=3e-5,
    conv_L_cache=5, conv_bias=True, tie_embedding=False)

# a convolution of width 1 (no state at all), one kv head for five heads, the adjusted width rounded to 8
TINY_E = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=160, num_hidden_layers=2, num_attention_heads=5,
    num_key_value_heads=1, vocab_size=1000, block_ff_dim=301, block_auto_adjust_ff_dim=True, block_multiple_of=8,
    block_ffn_dim_multiplier=1.3, layer_types=["full_attention", "conv"], rope_theta=1000000.0, norm_eps=1e-5,
    conv_L_cache=1, conv_bias=False, tie_embedding=True)

# heads of 64, the size that the tcgen05 attention kernel of long prompts takes; 3 heads on one kv head
TINY_F = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=192, num_hidden_layers=3, num_attention_heads=3,
    num_key_value_heads=1, vocab_size=500, block_ff_dim=256, block_auto_adjust_ff_dim=False,
    layer_types=["full_attention", "conv", "full_attention"], rope_theta=10000.0, norm_eps=1e-5,
    conv_L_cache=3, conv_bias=False, tie_embedding=False)

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4),
           "F": (TINY_F, 5)}

# The same configurations with every part loud (``init="loud"``: matrices with standard deviation
# 1/sqrt(columns)): with N(0, 0.02) matrices at these widths a gated convolution moves the logits by less
# than a bfloat16 run's rounding, so a fault in one would pass unseen.
LOUD_CONFIGS = {"AL": (TINY_A, 0), "BL": (TINY_B, 1), "FL": (TINY_F, 5)}


def all_folders(root):
    """Model folders for every configuration above: name -> folder."""
    from helpers import write_model
    out = {k: write_model(root, cfg, seed) for k, (cfg, seed) in CONFIGS.items()}
    out.update({k: write_model(root, cfg, seed, init="loud") for k, (cfg, seed) in LOUD_CONFIGS.items()})
    return out


def config_of(name: str) -> dict:
    return (CONFIGS.get(name) or LOUD_CONFIGS[name])[0]


def prompts(vocab: int, lengths, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
