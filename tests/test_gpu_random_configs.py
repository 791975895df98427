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
