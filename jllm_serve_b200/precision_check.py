"""The 32-bit path as a check of the bfloat16 path at a model's real layer sizes.

The tiny test models have widths of a hundred or two; the products of a real model sum over 4,096 or 12,288
terms and its head has 151,936 rows. This check runs the same random model (same seed, the same bfloat16 weight
values, widened exactly for the 32-bit path) through both precisions of the engine's own step function and
compares the logits place by place: a prompt whole and then some tokens one by one, and the same tokens again
as portions beside two other requests that are decoding. The reference does the like with a real checkpoint
and an outside implementation (scripts/real-weights-check.sh:1-20, scripts/real_ref.py:16-18 there); here both
sides are this engine, the 32-bit side being the one that the plain implementation pins at small sizes.

    python -m jllm_serve_b200.precision_check [--layers 2]
"""
from __future__ import annotations

import argparse
import json
import math
from typing import Dict, List, Sequence

import torch


def _tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _rows_of(runner, trace) -> Dict[tuple, torch.Tensor]:
    """Runs [(entries, ends)] with entries [(request, tokens, want)], want = True (every row's logits), False (none) or
    a number (those of the last so many rows); {(request, position): logits row}."""
    from .engine import Segment

    def wanted(toks, want):
        n = len(toks)
        return list(range(n)) if want is True else list(range(max(0, n - int(want)), n))

    fed, out = {}, {}
    for entries, ends in trace:
        segs = [Segment(rid, toks, fed.get(rid, 0), wanted(toks, want)) for rid, toks, want in entries]
        rows = runner.step(segs).clone()
        r = 0
        for rid, toks, want in entries:
            base = fed.get(rid, 0)
            for k in wanted(toks, want):
                out[(rid, base + k)] = rows[r]
                r += 1
            fed[rid] = base + len(toks)
        for rid in ends:
            runner.finish(rid)
            fed.pop(rid, None)
    return out


class _Stats:
    def __init__(self):
        self.rows = self.same = self.near = 0
        self.err2 = self.ref2 = self.worst = self.scale = self.far = 0.0

    def add(self, got: torch.Tensor, want: torch.Tensor) -> None:
        d = (got - want).double()
        self.err2 += float((d * d).sum())
        self.ref2 += float((want.double() ** 2).sum())
        self.worst = max(self.worst, float(d.abs().max()))
        self.scale = max(self.scale, float(want.abs().max()))
        choice = int(got.argmax())
        self.same += choice == int(want.argmax())
        self.far = max(self.far, float(want.max() - want[choice]))      # how much worse the other choice is
        self.rows += 1

    def summary(self) -> dict:
        return {"rows": self.rows, "max_rel": self.worst / max(self.scale, 1e-30),
                "rms_rel": math.sqrt(self.err2 / max(self.ref2, 1e-300)), "argmax_agree": self.same / max(1, self.rows),
                "worst_choice_gap_rel": self.far / max(self.scale, 1e-30)}


def compare_precisions(config: dict, seed: int = 0, prompt: int = 300, tail: int = 16, portion: int = 256,
                       others: Sequence[int] = (40, 90), page_size: int = 16, device: str = "cuda:0",
                       want_last: int = 0) -> dict:
    """Logits of the bfloat16 path against the 32-bit path of the same random model. Returns, for the request
    alone ("alone") and for the same request in portions beside two decoding requests ("mixed", all three
    requests' rows): rows compared, the largest difference as a share of the largest |logit|, the rms error as a
    share of the rms logit, the share of rows with the same best token, and the largest gap (same unit as the
    first) between the 32-bit path's best logit and its logit of the bfloat16 path's choice.
    `want_last` > 0 (long prompts: the logits of thousands of rows would fill the device): only the last so many
    rows of every portion are compared, and the 32-bit path runs the very same steps."""
    from .engine import ModelRunner
    vocab = config["vocab_size"]
    main = _tokens(prompt + tail, vocab, seed + 1)
    steps_beside = max(2, -(-prompt // portion))
    side = {f"side{i}": _tokens(n + steps_beside + tail, vocab, seed + 2 + i) for i, n in enumerate(others)}
    ctx = 64 * (-(-(prompt + tail + max(others) + steps_beside) // 64))
    kw = dict(config=config, seed=seed, device=device, page_size=page_size, max_batch_tokens=prompt + tail + len(others),
              max_requests=len(others) + 1, ctx=ctx, num_pages=(len(others) + 1) * (ctx // page_size + 1))

    every = want_last if want_last > 0 else True
    alone = [([("main", main[:prompt], every)], [])]
    alone += [([("main", main[p:p + 1], True)], ["main"] if p == prompt + tail - 1 else []) for p in range(prompt, prompt + tail)]
    whole_sides = [([(rid, toks, True)], [rid]) for rid, toks in side.items()]
    mixed = [([(rid, toks[:n], every)], []) for (rid, toks), n in zip(side.items(), others)]
    at = {rid: n for rid, n in zip(side, others)}

    def beside(entry):
        rows = [entry] + [(rid, side[rid][at[rid]:at[rid] + 1], True) for rid in side]
        for rid in side:
            at[rid] += 1
        return rows

    for lo in range(0, prompt, portion):
        mixed.append((beside(("main", main[lo:min(prompt, lo + portion)], every)), []))
    for p in range(prompt, prompt + tail):
        mixed.append((beside(("main", main[p:p + 1], True)), []))
    mixed[-1] = (mixed[-1][0], ["main"] + list(side))

    exact = ModelRunner(dtype="float32", **kw)
    want = _rows_of(exact, alone + whole_sides) if want_last <= 0 else {**_rows_of(exact, alone), **_rows_of(exact, mixed)}
    exact.close()
    del exact
    torch.cuda.empty_cache()
    fast = ModelRunner(dtype="bfloat16", **kw)
    got_alone = _rows_of(fast, alone)
    got_mixed = _rows_of(fast, mixed)
    from .csrc import ops
    ops.check_kernel_errors()
    out = {}
    for name, got in (("alone", got_alone), ("mixed", got_mixed)):
        st = _Stats()
        for key, row in got.items():
            st.add(row, want[key])
        out[name] = st.summary()
    out["mixed"]["largest_step_rows"] = portion + len(others)
    fast.close()
    del fast
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    config = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=args.layers,
                  num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                  vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                  max_position_embeddings=40960)
    print(json.dumps(compare_precisions(config, args.seed)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
