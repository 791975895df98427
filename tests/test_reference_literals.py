"""The numbers the reference's own test suite writes down, as anchors of BOTH the plain implementation and the product.

The reference (Java, no JDK where these tests run) cannot be executed here, but its tests state results as
literals (src/test/java/org/robomiri/jllm/SmokeTest.java). Each is checked against the plain implementation of
`tests/plain` and against the product's own code, so the two are never only compared with one another.

What stays pinned by reading alone, because no literal of the reference fixes it for a whole qwen3 model: the
rotate-half pairing across a whole head of more than one pair, the order "per-head norm, then rotation", and the
map from query head to kv head.
"""
import math

import pytest
import torch

from jllm_serve_b200.config import RopeScaling, RopeTableSpec, parse_config
from jllm_serve_b200.parts.rope import RotaryTable, amplitude, inverse_frequencies
from tests.plain import qwen3_plain as P

YARN_40 = {"rope_type": "yarn", "factor": 40.0, "original_max_position_embeddings": 4096, "beta_fast": 32, "beta_slow": 1}


def product_frequencies(rotary_dim, theta, scaling: RopeScaling, max_positions=4096):
    return inverse_frequencies(RopeTableSpec(rotary_dim, theta, scaling, "half"), max_positions).tolist()


def yarn(factor, orig, mscale=1.0, all_dim=0.0, attention=0.0, truncate=True):
    return RopeScaling(kind="yarn", factor=factor, original_max_positions=orig, beta_fast=32.0, beta_slow=1.0,
                       mscale=mscale, mscale_all_dim=all_dim, attention_factor=attention, truncate=truncate)


@pytest.mark.parametrize("which", ["plain", "product"])
def test_plain_rope_frequencies(which):
    # SmokeTest.java:652-653: invFreq(8, 1e4) = {1, 0.1, 0.01, 0.001}
    f = P.rope_inverse_frequencies(8, 1e4, None, 4096) if which == "plain" else product_frequencies(8, 1e4, RopeScaling())
    assert f[0] == 1.0 and all(abs(a - b) < 1e-15 for a, b in zip(f, [1.0, 0.1, 0.01, 0.001]))
    # SmokeTest.java:645-648 (plain part): head size 64, theta 5e5: first, second and last of 32 frequencies
    h = P.rope_inverse_frequencies(64, 5e5, None, 4096) if which == "plain" else product_frequencies(64, 5e5, RopeScaling())
    assert h[0] == 1.0 and abs(h[1] - 0.6636012376960885) < 1e-12 and len(h) == 32


@pytest.mark.parametrize("which", ["plain", "product"])
def test_rope_table_covers_the_rotary_dims_only(which):
    # SmokeTest.java:676-677: rotary_dim 4 of theta 1e4 has frequencies (1, 0.01): sin[position 2, pair 1] = sin(0.02)
    if which == "plain":
        cos, sin = P.rope_table(range(3), 4, 1e4)
    else:
        t = RotaryTable(RopeTableSpec(4, 1e4, RopeScaling(), "half"), 3, "cpu")
        cos, sin = t.cos, t.sin
    assert tuple(cos.shape) == (3, 2) and abs(float(sin[2, 1]) - float(torch.tensor(math.sin(0.02), dtype=torch.float32))) < 1e-7


@pytest.mark.parametrize("which", ["plain", "product"])
def test_yarn_frequencies(which):
    """SmokeTest.java:1491-1509: rotary dim 64, theta 1e4, factor 40 over 4,096 positions, beta 32 / 1. Correction
    dims 10.47 -> 10 and 22.51 -> 23: pairs up to 10 keep theta^(-i/32), pairs from 23 on are divided by 40, between
    them a ramp: pair 16 gives 0.00025 * 6/13 + 0.01 * 7/13 = 0.0055."""
    f = P.rope_inverse_frequencies(64, 1e4, YARN_40, 4096) if which == "plain" else \
        product_frequencies(64, 1e4, yarn(40.0, 4096))
    assert len(f) == 32 and f[0] == 1.0
    assert abs(f[5] - math.pow(1e4, -5.0 / 32)) < 1e-15 and abs(f[10] - 0.056234132519034905) < 1e-15
    assert abs(f[16] - 0.0055) < 1e-15
    assert abs(f[22] - 0.0001778279410038922) < 1e-15
    assert abs(f[23] - 3.33380358040831e-05) < 1e-18 and abs(f[23] - math.pow(1e4, -23.0 / 32) / 40) < 1e-18
    assert abs(f[31] - math.pow(1e4, -31.0 / 32) / 40) < 1e-18


@pytest.mark.parametrize("which", ["plain", "product"])
def test_yarn_amplitude(which):
    """SmokeTest.java:1507-1520: mscale(40, 0.707) = 1.2608037774058554, mscale(40, 1) = 1.3688879454113936; the
    table is multiplied by mscale / mscale_all_dim (1 when they are equal); attention_factor overrides both."""
    m = 1.3688879454113936 / 1.2608037774058554
    if which == "plain":
        amp = lambda **kw: P.rope_amplitude(dict(YARN_40, **kw))
        table = lambda **kw: P.rope_table(range(4), 64, 1e4, dict(YARN_40, **kw), 4096)
    else:
        amp = lambda mscale=0.0, mscale_all_dim=0.0, attention_factor=0.0: amplitude(
            yarn(40.0, 4096, *((mscale, mscale_all_dim) if mscale and mscale_all_dim else (1.0, 0.0)), attention_factor))

        def table(mscale=0.0, mscale_all_dim=0.0):
            t = RotaryTable(RopeTableSpec(64, 1e4, yarn(40.0, 4096, *((mscale, mscale_all_dim) if mscale and mscale_all_dim
                                                                       else (1.0, 0.0))), "half"), 4, "cpu")
            return t.cos, t.sin
    assert abs(amp(mscale=0.707, mscale_all_dim=0.707) - 1.0) < 1e-12
    assert abs(amp(mscale=1.0, mscale_all_dim=0.707) - m) < 1e-12
    assert amp(mscale=1.0, mscale_all_dim=0.707, attention_factor=1.5) == 1.5
    # one argument of the pair alone: the paper's 0.1 ln(factor) + 1 (the numerator with mscale 1, the denominator 1)
    assert abs(amp() - (0.1 * math.log(40) + 1)) < 1e-12 and abs(0.1 * math.log(40) + 1 - 1.3688879454113936) < 1e-12
    cos, sin = table(mscale=0.707, mscale_all_dim=0.707)
    assert float(cos[0, 0]) == 1.0 and float(sin[0, 0]) == 0.0 and abs(float(cos[1, 16]) - math.cos(0.0055)) < 1e-6
    cos, sin = table(mscale=1.0, mscale_all_dim=0.707)
    assert abs(float(cos[0, 0]) - m) < 1e-6 and abs(float(sin[1, 16]) - math.sin(0.0055) * m) < 1e-6


def test_qwen3_yarn_config():
    """SmokeTest.java:1522-1556: the long-context recipe in a qwen3 config.json; the same frequencies as computed
    from the parameters directly; amplitude 0.1 ln 4 + 1; the defaults of the other keys."""
    base = dict(model_type="qwen3", hidden_size=1024, intermediate_size=3072, num_hidden_layers=2, num_attention_heads=16,
                num_key_value_heads=8, head_dim=128, vocab_size=1000, rope_theta=1000000, max_position_embeddings=40960)
    q = parse_config(dict(base, rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}))
    s = q.rope_tables[0].scaling
    assert (s.kind, s.factor, s.original_max_positions, s.beta_fast, s.beta_slow) == ("yarn", 4.0, 32768, 32.0, 1.0)
    assert q.core.description.endswith(" rope=yarnx4")
    got = inverse_frequencies(q.rope_tables[0], 40960).tolist()
    assert got == product_frequencies(128, 1e6, yarn(4.0, 32768), 40960)
    assert got == P.rope_inverse_frequencies(128, 1e6, {"rope_type": "yarn", "factor": 4.0,
                                                        "original_max_position_embeddings": 32768}, 40960)
    amp = 0.1 * math.log(4) + 1
    assert abs(amplitude(s) - amp) < 1e-15
    t = RotaryTable(q.rope_tables[0], 3, "cpu")
    assert abs(float(t.cos[0, 0]) - amp) < 1e-6 and abs(float(t.sin[2, 63]) - math.sin(2 * got[63]) * amp) < 1e-6
    a = parse_config(dict(base, rope_scaling={"type": "yarn", "factor": 2.0, "attention_factor": 1.25})).rope_tables[0].scaling
    assert a.original_max_positions == 40960 and amplitude(a) == 1.25
    ms = parse_config(dict(base, rope_scaling={"type": "yarn", "factor": 40, "mscale": 1.0, "mscale_all_dim": 0.707,
                                               "beta_fast": 16})).rope_tables[0].scaling
    assert ms.beta_fast == 16 and abs(amplitude(ms) - 1.3688879454113936 / 1.2608037774058554) < 1e-12
    ntt = parse_config(dict(base, rope_scaling={"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768,
                                                "truncate": False})).rope_tables[0]
    assert not ntt.scaling.truncate and s.truncate and inverse_frequencies(ntt, 40960).tolist() != got
    from jllm_serve_b200.config import ConfigError
    with pytest.raises(ConfigError, match="yarn"):
        parse_config(dict(base, rope_scaling={"type": "yarn", "factor": -1}))


def test_qwen3_config_cases():
    """SmokeTest.java:841-857: the window from `max_window_layers` on only with `use_sliding_window`; a qwen3 config
    gets the q/k norm; `attention_bias` biases q, k, v AND o_proj and the description says " bias obias"."""
    windowed = parse_config(dict(model_type="qwen3", hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                                 num_attention_heads=12, vocab_size=151936, sliding_window=4096, use_sliding_window=True,
                                 max_window_layers=21))
    assert windowed.layers[20].mixer.window == 0 and windowed.layers[21].mixer.window == 4096
    off = parse_config(dict(model_type="qwen3", hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                            num_attention_heads=12, num_key_value_heads=2, vocab_size=151936, sliding_window=32768,
                            use_sliding_window=False, max_window_layers=21, tie_word_embeddings=True,
                            eos_token_id=[151645, 151643]))
    assert off.layers[27].mixer.window == 0 and off.layers[0].mixer.head_dim == 128 and off.core.eos == (151645, 151643)
    q3 = parse_config(dict(model_type="qwen3", hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                           num_attention_heads=16, num_key_value_heads=8, head_dim=128, vocab_size=151936))
    assert q3.layers[0].mixer.qk_norm
    biased = parse_config(dict(model_type="qwen3", hidden_size=1024, intermediate_size=3072, num_hidden_layers=2,
                               num_attention_heads=16, num_key_value_heads=8, head_dim=64, vocab_size=1000,
                               attention_bias=True))
    assert biased.layers[1].mixer.bias and biased.layers[1].mixer.out_bias and " bias obias" in biased.core.description
