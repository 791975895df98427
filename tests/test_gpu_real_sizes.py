"""The bfloat16 path against the 32-bit path at the layer sizes of Qwen3-8B (GPU).

Every other comparison of logits in this suite runs at widths of up to 168. Here the products sum over 4,096
and 12,288 terms, the head has 151,936 rows and the attention 32 query heads over 8 kv heads of size 128: the
sizes that are benchmarked. Two layers instead of 36 (the sizes of a layer are what matters; both numbers are
named). The 32-bit path is the one the plain implementation pins at small sizes.

The bounds are wider than those of the tiny models, and for a reason that is a model of the error, not a guess:
with 4,096 inputs of N(0, 0.02) weights the layers' outputs dwarf the embedding (which is exact in both paths and
dominates the residual stream of a tiny model), so the logits carry the bfloat16 roundings of the activations
undiluted. One layer measured stage by stage: q, k and v 2.6e-3 of their rms (two roundings of 2^-8 / sqrt(3)
each), the attention's output 4.6e-3 (scores from 128 products of twice-rounded values, P and the output rounded
once more), the feed-forward's hidden values 7.8e-3 (gate and up both inherit the attention's error), the logits
7.9e-3; two layers 9.8e-3. With 151,936 random logits a row's two best are often closer than that, so the best
token is not always the same one; where it differs the 32-bit path must hold the other choice for nearly as good.
"""
import pytest

pytestmark = pytest.mark.gpu

QWEN3_8B_LAYERS = 36
CONFIG = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=2,
              num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
              vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
              attention_bias=False, use_sliding_window=False, max_position_embeddings=40960, hidden_act="silu")


# the layer sizes of the other two configurations that are benchmarked (Qwen3-14B, Qwen3-32B: 5,120 wide, 40 or 64 query
# heads, 17,408 or 25,600 hidden units: 272 and 400 k blocks for the down product)
OTHER_SIZES = {"14b": dict(CONFIG, hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
               "32b": dict(CONFIG, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)}


def test_bfloat16_follows_float32_at_8b_layer_sizes():
    from jllm_serve_b200.precision_check import compare_precisions
    got = compare_precisions(CONFIG, seed=3)
    print(f"layers {CONFIG['num_hidden_layers']} of {QWEN3_8B_LAYERS}: {got}")
    for name in ("alone", "mixed"):
        s = got[name]
        assert s["rows"] >= 316
        assert s["max_rel"] <= 1.5e-2, (name, s)
        assert s["rms_rel"] <= 1.3e-2, (name, s)
        assert s["argmax_agree"] >= 0.96, (name, s)
        # where the two paths choose differently, the 32-bit path holds the other choice for almost as good
        assert s["worst_choice_gap_rel"] <= 1e-2, (name, s)


def test_bfloat16_follows_float32_with_a_prompt_of_many_rows():
    """The same with 1,280 rows in one step and portions of 1,024: the products then run two SMs to a tile, with
    float32 outputs by tiled bulk copies, and the attention two query tiles to a block."""
    from jllm_serve_b200.csrc import ops
    from jllm_serve_b200.precision_check import compare_precisions
    for rows in (1280, 1024):
        assert ops.gemm_kernel_for(rows, 24576, 4096, sms=ops.sm_count(), pairs=ops.resident_pairs()) == "pair"
    got = compare_precisions(CONFIG, seed=5, prompt=1280, tail=4, portion=1024)
    print(f"layers {CONFIG['num_hidden_layers']} of {QWEN3_8B_LAYERS}: {got}")
    for name in ("alone", "mixed"):
        s = got[name]
        assert s["rows"] >= 1284
        assert s["max_rel"] <= 1.5e-2, (name, s)
        assert s["rms_rel"] <= 1.3e-2, (name, s)
        assert s["argmax_agree"] >= 0.96, (name, s)
        assert s["worst_choice_gap_rel"] <= 1e-2, (name, s)


@pytest.mark.parametrize("size", ["14b", "32b"])
def test_bfloat16_follows_float32_at_other_layer_sizes(size):
    """The same at the layer sizes of Qwen3-14B and Qwen3-32B, with a short prompt (128-row tiles, the weight-stream
    products) and with one of 1,280 rows (two SMs to a tile)."""
    from jllm_serve_b200.precision_check import compare_precisions
    for kw in (dict(prompt=300, tail=16, portion=256), dict(prompt=1280, tail=4, portion=1024)):
        got = compare_precisions(OTHER_SIZES[size], seed=1, **kw)
        print(f"{size}, two layers, {kw}: {got}")
        for name in ("alone", "mixed"):
            s = got[name]
            assert s["rows"] >= kw["prompt"] + kw["tail"]
            assert s["max_rel"] <= 1.5e-2, (size, name, s)
            assert s["rms_rel"] <= 1.3e-2, (size, name, s)
            assert s["argmax_agree"] >= 0.96, (size, name, s)
            assert s["worst_choice_gap_rel"] <= 1e-2, (size, name, s)


def test_bfloat16_follows_float32_far_into_a_long_prompt():
    """A prompt of 9,000 tokens, whole and in portions of 2,048 beside two requests that decode at 5,000 and 3,000
    tokens of context: the last rows of every portion and every decoded row. The flash attention then runs portions
    whose keys begin thousands of positions back, the decode attention many splits, the products two SMs to a tile."""
    from jllm_serve_b200.precision_check import compare_precisions
    got = compare_precisions(CONFIG, seed=7, prompt=9000, tail=6, portion=2048, others=(5000, 3000), want_last=4)
    print(f"layers {CONFIG['num_hidden_layers']} of {QWEN3_8B_LAYERS}: {got}")
    assert got["alone"]["rows"] == 10 and got["mixed"]["rows"] == 8 + 5 * 6 + 6 * 3
    for name in ("alone", "mixed"):
        s = got[name]
        assert s["max_rel"] <= 1.5e-2, (name, s)
        assert s["rms_rel"] <= 1.3e-2, (name, s)
        assert s["argmax_agree"] >= 0.85, (name, s)          # (ten rows: one other choice is a tenth)
        assert s["worst_choice_gap_rel"] <= 1e-2, (name, s)


def test_bfloat16_follows_float32_with_portions_of_some_hundred_rows():
    """Steps of 129 to 512 rows (portions of 150, 220 and 440 rows beside two decoding requests). Up to 256 rows the
    tokens are still one N side of the weight-stream product, which takes the down product there, and up to 160 rows
    the others too; from 257 to 512 rows the down product's 256 x 256 tiles are cut up over all pairs of SMs."""
    from jllm_serve_b200.csrc import ops
    from jllm_serve_b200.precision_check import compare_precisions
    assert ops.gemm_kernel_for(222, 4096, 12288) == "swap" and ops.gemm_kernel_for(152, 6144, 4096) == "swap"
    if ops.resident_pairs() > 0:       # 442 rows: the down product's tiles cut up over all pairs
        assert ops.gemm_kernel_for(442, 4096, 12288, pairs=ops.resident_pairs()) == "pair-streamed"
    for portion in (150, 220, 440):
        got = compare_precisions(CONFIG, seed=9, prompt=2 * portion, tail=4, portion=portion)
        print(f"portions of {portion}, layers {CONFIG['num_hidden_layers']} of {QWEN3_8B_LAYERS}: {got}")
        for name in ("alone", "mixed"):
            s = got[name]
            assert s["rows"] >= 2 * portion + 4
            assert s["max_rel"] <= 1.5e-2, (name, s)
            assert s["rms_rel"] <= 1.3e-2, (name, s)
            assert s["argmax_agree"] >= 0.96, (name, s)
            assert s["worst_choice_gap_rel"] <= 1e-2, (name, s)
