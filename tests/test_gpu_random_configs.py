"""Configurations drawn at random (seeded) through the engine, under every way of cutting the work, against the plain
implementation (GPU): sizes and options in combinations that the five fixed tiny configurations do not hold, with page
sizes that are no powers of two among them."""
import random

import pytest

from tests import traces
from tests.helpers import RowChecker, replay
from tests.tiny import make_model_folder, random_config, random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [9004, 9011, 9033, 9036, 9040, 9057])
def test_a_random_configuration_under_every_cut(seed, tmp_path):
    from jllm_serve_b200.engine import ModelRunner
    cfg = random_config(seed)
    rng = random.Random(seed + 1)
    page = rng.choice([1, 2, 3, 4, 8, 12, 16, 32, 64, 128])
    lengths = [rng.randint(1, 40), rng.randint(30, 140), rng.randint(100, 330), rng.randint(2, 90),
               rng.randint(120, 300), rng.randint(1, 20)]
    if seed % 2:
        lengths[2] = rng.randint(400, 900)                 # portions of several 128-row tiles
    folder = make_model_folder(cfg, seed, tmp_path / "model")
    reqs = {f"r{j}": random_tokens(n, cfg["vocab_size"], 1000 * seed + j) for j, n in enumerate(lengths)}
    cuts = {"whole": traces.whole(reqs), "decode tail": traces.prompt_then_decode(reqs, 24),
            "portions": traces.changing_portions(reqs), "mixed": traces.mixed(reqs, max_live=4),
            "side by side": traces.all_together(reqs, tail=6)}
    shape = (f"seed {seed}: head size {cfg['head_dim']}, heads {cfg['num_attention_heads']}/{cfg['num_key_value_heads']}, "
             f"width {cfg['hidden_size']}/{cfg['intermediate_size']}, vocabulary {cfg['vocab_size']}, page {page}")
    for dtype in ("float32", "bfloat16"):
        for cut, steps in cuts.items():
            tokens = traces.peak_tokens(steps, max(64, page))
            runner = ModelRunner(folder, dtype=dtype, page_size=page, num_pages=-(-tokens // page) + 2,
                                 max_batch_tokens=1024, max_requests=8, ctx=1024, poison_freed_pages=True)
            got = replay(runner, steps)
            checker = RowChecker(folder, reqs, dtype, None, f"{shape}, {cut}")
            for (rid, position), row in got.items():
                checker.row(rid, position, row)
            checker.finish()
            runner.close()


EDGE = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
            rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False,
            use_sliding_window=False, max_position_embeddings=512, hidden_act="silu")


@pytest.mark.parametrize("what,change", [
    ("24 query heads to a kv head, head size 128", dict(num_attention_heads=24, num_key_value_heads=1, head_dim=128)),
    ("17 query heads to a kv head", dict(num_attention_heads=17, num_key_value_heads=1, head_dim=32)),
    ("a width that is no multiple of 4", dict(hidden_size=50, intermediate_size=70)),
    ("widths that are multiples of 4, not of 8", dict(hidden_size=100, intermediate_size=36)),
    ("a vocabulary of 7", dict(vocab_size=7)),
    ("a prime vocabulary", dict(vocab_size=100003)),
    ("head size 24 (no multiple of 16)", dict(head_dim=24)),
    ("head size 272 (beyond the tensor-core attention kernels)", dict(head_dim=272)),
    ("eight hidden units", dict(intermediate_size=8))])
def test_sizes_at_the_edge_of_what_the_kernels_take(what, change, tmp_path):
    """Sizes that the fast kernels do not take fall to the plain ones (or are taken after all): never a wrong result.
    Whole, mixed with pages used again, and a tail decoded one by one, in both precisions, against the plain model."""
    from jllm_serve_b200.engine import ModelRunner
    cfg = dict(EDGE, **change)
    folder = make_model_folder(cfg, 5, tmp_path / "model")
    reqs = {f"r{j}": random_tokens(n, cfg["vocab_size"], 50 + j) for j, n in enumerate((3, 70, 150, 33))}
    for dtype in ("float32", "bfloat16"):
        for cut, steps in (("whole", traces.whole(reqs)), ("mixed", traces.mixed(reqs, max_live=3)),
                           ("decode tail", traces.prompt_then_decode(reqs, 20))):
            runner = ModelRunner(folder, dtype=dtype, page_size=16, num_pages=traces.peak_tokens(steps, 64) // 16 + 2,
                                 max_batch_tokens=512, max_requests=8, ctx=256, poison_freed_pages=True)
            got = replay(runner, steps)
            checker = RowChecker(folder, reqs, dtype, None, f"{what}, {cut}")
            for (rid, position), row in got.items():
                checker.row(rid, position, row)
            checker.finish()
            runner.close()
