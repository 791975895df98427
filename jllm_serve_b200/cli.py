"""The command line, in the reference's manner: `jllm <command> [--key value | --key=value | --flag]`.

Settings are layered as in the reference (src/main/java/org/robomiri/jllm/config/Settings.java:
88-127,156-202): built-in defaults < a properties file (`--config FILE`, `$JLLM_CONFIG`, or
`./jllm.properties`) < flags. A flag is either an alias (`--temp` = `sampling.temperature`,
:31-75) or a property key itself (`--sampling.top-k 40`). An unknown option is an error and
exits with 2 (Main.java:44-50). Every typed value is checked before the weights load.

Commands in scope: `run` (one completion), `bench` (prefill / decode throughput) and `config`
(every key, its value and where it came from). Prompts are token ids: `--tokens 1,2,3` or
`--random-prompt N`; the engine carries no tokenizer, chat template, downloader or server.
"""
from __future__ import annotations

import os
import sys
import time
from pathlib import Path
from typing import Dict, List, Tuple

DEFAULTS: Dict[str, Tuple[str, str]] = {
    # key: (default, meaning)
    "model.dir": ("", "folder with config.json and model.safetensors"),
    "model.random-weights": ("", "seed: make random weights for --model-config instead of reading a folder"),
    "model.config": ("", "a config.json to use with model.random-weights"),
    "backend.dtype": ("bf16", "bf16 | fp32 (true 32-bit, no tensor cores)"),
    "backend.ctx": ("0", "context length; 0 = the model's max_position_embeddings"),
    "backend.batch": ("512", "rows of one prompt portion (the reference's backend.batch)"),
    "backend.kv-block": ("16", "positions per cache page"),
    "backend.num-pages": ("auto", "pages of the cache pool; auto = backend.kv-share of the free device memory; "
                                  "0 = enough for ctx x 4 tokens"),
    "backend.kv-share": ("0.6", "auto: the part of the free device memory the cache pool may take"),
    "engine.pass-budget": ("0", "most rows in one step; 0 = backend.batch + engine.mixed-reserve"),
    "engine.mixed-reserve": ("32", "rows kept for decoding requests beside a prompt portion"),
    "engine.min-chunk": ("16", "a portion is trimmed to the room left only down to this many rows"),
    "engine.max-running": ("64", "most requests generating at a time"),
    "engine.cuda-graphs": ("true", "replay captured decode steps"),
    "engine.overlap": ("true", "plan and launch a step while the one before still runs (its tokens are read a step later)"),
    "engine.fill-portions": ("true", "a step with room left takes the next prompts' portions too (false: one portion a step)"),
    "sampling.temperature": ("0.6", "0 means greedy"),
    "sampling.top-k": ("20", "0 disables"),
    "sampling.top-p": ("0.95", "1 disables"),
    "sampling.min-p": ("0", "0 disables"),
    "sampling.seed": ("-1", "-1 = random"),
    "sampling.max-tokens": ("1024", "most generated tokens"),
    "sampling.ignore-eos": ("false", "keep generating past a stop token"),
    "bench.max-tokens": ("128", "tokens decoded per bench round"),
    "bench.rounds": ("3", "bench rounds; the best is reported"),
    "bench.prompt-tokens": ("413", "length of the synthetic bench prompt"),
}

ALIASES = {
    "model": "model.dir", "dir": "model.dir", "random-weights": "model.random-weights", "model-config": "model.config",
    "dtype": "backend.dtype", "ctx": "backend.ctx", "batch": "backend.batch", "chunk": "backend.batch",
    "page-size": "backend.kv-block", "num-pages": "backend.num-pages", "kv-share": "backend.kv-share",
    "max-batch-tokens": "engine.pass-budget",
    "max-running": "engine.max-running", "temp": "sampling.temperature", "temperature": "sampling.temperature",
    "top-k": "sampling.top-k", "top-p": "sampling.top-p", "min-p": "sampling.min-p", "seed": "sampling.seed",
    "max-tokens": "sampling.max-tokens", "ignore-eos": "sampling.ignore-eos",
}
CLI_ONLY = {"tokens", "random-prompt", "config", "prompt-seed"}
BOOLEAN_KEYS = {"sampling.ignore-eos", "engine.cuda-graphs", "engine.overlap", "engine.fill-portions"}


class SettingsError(ValueError):
    pass


class Settings:
    def __init__(self, values: Dict[str, str], sources: Dict[str, str], cli: Dict[str, str]):
        self.values, self.sources, self.cli = values, sources, cli

    @classmethod
    def load(cls, args: List[str], env=os.environ, cwd=".") -> "Settings":
        values = {k: v[0] for k, v in DEFAULTS.items()}
        sources = {k: "default" for k in DEFAULTS}
        flags, cli = cls.parse_args(args)
        path = cli.get("config") or env.get("JLLM_CONFIG") or (
            str(Path(cwd) / "jllm.properties") if (Path(cwd) / "jllm.properties").is_file() else None)
        if path:
            if not Path(path).is_file():
                raise SettingsError(f"config file not found: {path}")
            for n, line in enumerate(Path(path).read_text().splitlines(), 1):
                line = line.strip()
                if not line or line[0] in "#!":
                    continue
                if "=" not in line:
                    raise SettingsError(f"{path}:{n}: expected key=value, got {line!r}")
                k, v = (s.strip() for s in line.split("=", 1))
                if k not in DEFAULTS:
                    raise SettingsError(f"{path}:{n}: unknown setting '{k}'")
                values[k], sources[k] = v, path
        for k, v in flags.items():
            values[k], sources[k] = v, "flag"
        return cls(values, sources, cli)

    @staticmethod
    def parse_args(args: List[str]):
        """`--k v`, `--k=v`, and bare booleans (Settings.java:156-187)."""
        flags, cli = {}, {}
        i = 0
        while i < len(args):
            a = args[i]
            if not a.startswith("--"):
                raise SettingsError(f"unexpected argument '{a}' (options start with --)")
            name, eq, val = a[2:].partition("=")
            key = ALIASES.get(name, name)
            if key not in DEFAULTS and name not in CLI_ONLY:
                raise SettingsError(f"unknown option --{name}")
            if not eq:
                if key in BOOLEAN_KEYS and (i + 1 >= len(args) or args[i + 1].startswith("--")):
                    val = "true"
                elif i + 1 < len(args):
                    i += 1
                    val = args[i]
                else:
                    raise SettingsError(f"option --{name} needs a value")
            (cli if name in CLI_ONLY else flags)[name if name in CLI_ONLY else key] = val
            i += 1
        return flags, cli

    def get(self, key: str) -> str:
        return self.values[key]

    def integer(self, key: str, low=None) -> int:
        try:
            v = int(self.values[key])
        except ValueError:
            raise SettingsError(f"{key} must be an integer, got '{self.values[key]}'") from None
        if low is not None and v < low:
            raise SettingsError(f"{key} must be at least {low}, got {v}")
        return v

    def number(self, key: str) -> float:
        try:
            return float(self.values[key])
        except ValueError:
            raise SettingsError(f"{key} must be a number, got '{self.values[key]}'") from None

    def boolean(self, key: str) -> bool:
        v = self.values[key].lower()
        if v not in ("true", "false"):
            raise SettingsError(f"{key} must be true or false, got '{self.values[key]}'")
        return v == "true"

    def validate(self) -> "Settings":
        if self.get("backend.dtype") not in ("bf16", "fp32", "bfloat16", "float32"):
            raise SettingsError(f"backend.dtype must be bf16 or fp32, got '{self.get('backend.dtype')}'")
        self.integer("backend.ctx", 0)
        self.integer("backend.batch", 1)
        self.integer("backend.kv-block", 1)
        if self.get("backend.num-pages") != "auto":
            self.integer("backend.num-pages", 0)
        if not 0 < self.number("backend.kv-share") <= 1:
            raise SettingsError(f"backend.kv-share must be in (0, 1], got '{self.get('backend.kv-share')}'")
        self.integer("engine.pass-budget", 0)
        self.integer("engine.mixed-reserve", 0)
        self.integer("engine.min-chunk", 1)
        self.integer("engine.max-running", 1)
        self.integer("bench.max-tokens", 1)
        self.integer("bench.rounds", 1)
        self.integer("bench.prompt-tokens", 1)
        self.boolean("engine.cuda-graphs")
        self.boolean("engine.overlap")
        self.boolean("engine.fill-portions")
        self.sampling()
        return self

    def sampling(self):
        from .sampling import SamplingParams
        try:
            return SamplingParams(temperature=self.number("sampling.temperature"), top_k=self.integer("sampling.top-k"),
                                  top_p=self.number("sampling.top-p"), min_p=self.number("sampling.min-p"),
                                  seed=self.integer("sampling.seed"), max_tokens=self.integer("sampling.max-tokens"),
                                  ignore_eos=self.boolean("sampling.ignore-eos"))
        except ValueError as e:
            raise SettingsError(str(e)) from None

    def describe(self) -> str:
        """Every key, its value and its source (Settings.java:460-465)."""
        return "".join(f"{k} = {self.values[k]}    # {self.sources[k]}: {DEFAULTS[k][1]}\n" for k in DEFAULTS)


USAGE = """usage: jllm <command> [options]
  run        single completion of a token prompt (--tokens 1,2,3 | --random-prompt N)
  bench      measure prefill/decode throughput on a synthetic prompt
  config     print the effective configuration and where each value comes from
options (override with --config <file> or flags):
  --model <dir>   --random-weights <seed> --model-config <config.json>   --dtype bf16|fp32
  --ctx <n>  --batch <n>  --page-size <n>  --num-pages <n|auto>  --kv-share <0..1>  --max-batch-tokens <n>
  --max-running <n>
  --temp <t> --top-k <k> --top-p <p> --min-p <p> --seed <s> --max-tokens <n> --ignore-eos
  any property key directly, e.g. --bench.rounds=5
"""


def build_engine(s: Settings):
    import json

    from .engine import Engine
    batch = s.integer("backend.batch")
    budget = s.integer("engine.pass-budget") or batch + s.integer("engine.mixed-reserve")
    kw = dict(dtype=s.get("backend.dtype"), ctx=s.integer("backend.ctx") or None,
              page_size=s.integer("backend.kv-block"), kv_share=s.number("backend.kv-share"),
              num_pages="auto" if s.get("backend.num-pages") == "auto" else (s.integer("backend.num-pages") or None),
              max_batch_tokens=budget, chunk=batch, min_chunk=s.integer("engine.min-chunk"),
              max_running=s.integer("engine.max-running"), cuda_graphs=s.boolean("engine.cuda-graphs"),
              overlap=s.boolean("engine.overlap"), fill_portions=s.boolean("engine.fill-portions"))
    if s.get("model.random-weights"):
        if not s.get("model.config"):
            raise SettingsError("--random-weights needs --model-config <config.json>")
        config = json.loads(Path(s.get("model.config")).read_text())
        return Engine(config=config, seed=int(s.get("model.random-weights")), **kw)
    if not s.get("model.dir"):
        raise SettingsError("no model: give --model <dir>, or --random-weights <seed> --model-config <config.json>")
    return Engine(s.get("model.dir"), **kw)


def _prompt(s: Settings, vocab: int, default_len=None) -> List[int]:
    import torch
    if "tokens" in s.cli:
        try:
            return [int(t) for t in s.cli["tokens"].replace(" ", "").split(",") if t]
        except ValueError:
            raise SettingsError(f"--tokens must be integers separated by commas, got '{s.cli['tokens']}'") from None
    n = int(s.cli.get("random-prompt", default_len or 0))
    if n < 1:
        raise SettingsError("no prompt: give --tokens 1,2,3 or --random-prompt N")
    g = torch.Generator().manual_seed(int(s.cli.get("prompt-seed", 0)))
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _describe(engine) -> None:
    print(f"Model: {engine.describe()}", file=sys.stderr)
    for note in engine.runner.notes:
        print(f"note: {note}", file=sys.stderr)


def cmd_run(s: Settings) -> int:
    engine = build_engine(s)
    _describe(engine)
    res = engine.generate([_prompt(s, engine.runner.vocab)], s.sampling())[0]
    print(",".join(str(t) for t in res.tokens))
    print(f"[{res.finish_reason}] {res.stats.line()}", file=sys.stderr)
    return 0


def cmd_bench(s: Settings) -> int:
    """Prefill and decode throughput of one request, the best of `bench.rounds` (Main.java:363-382)."""
    from .sampling import SamplingParams
    engine = build_engine(s)
    _describe(engine)
    prompt = _prompt(s, engine.runner.vocab, s.integer("bench.prompt-tokens"))
    params = SamplingParams.greedy_params(max_tokens=s.integer("bench.max-tokens"), ignore_eos=True)
    best = None
    for _ in range(s.integer("bench.rounds")):
        st = engine.generate([prompt], params)[0].stats
        if best is None or st.decode_ms < best.decode_ms:
            best = st
    print(f"prefill {best.prompt_tokens} tok in {best.prefill_ms:.0f} ms ({best.prompt_tokens / best.prefill_ms * 1e3:.1f}"
          f" tok/s), decode {best.generated} tok in {best.decode_ms:.0f} ms ({best.tok_per_sec:.1f} tok/s)")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        sys.stderr.write(USAGE)
        return 0
    cmd, rest = argv[0], argv[1:]
    try:
        s = Settings.load(rest).validate()
    except SettingsError as e:
        print(e, file=sys.stderr)
        return 2
    try:
        if cmd == "config":
            sys.stdout.write(s.describe())
            return 0
        if cmd == "run":
            return cmd_run(s)
        if cmd == "bench":
            return cmd_bench(s)
    except SettingsError as e:
        print(e, file=sys.stderr)
        return 2
    print(f"unknown command: {cmd}", file=sys.stderr)
    sys.stderr.write(USAGE)
    return 2


if __name__ == "__main__":
    sys.exit(main())
