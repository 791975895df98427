"""The command line: settings in layers (defaults < properties file < flags), aliases, checks before anything loads
(no GPU), and `bin/jllm run` on a tiny random model against the plain implementation (GPU).

The layering, the forms of a flag and the exit code of an unknown option follow the reference
(src/main/java/org/robomiri/jllm/config/Settings.java:88-127,156-202; Main.java:44-50).
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from jllm_serve_b200.cli import DEFAULTS, Settings, SettingsError, main

ROOT = Path(__file__).resolve().parent.parent


def load(args, env=None, cwd="."):
    return Settings.load(list(args), env=env or {}, cwd=cwd).validate()


def test_defaults_flags_and_aliases(tmp_path):
    s = load([], cwd=tmp_path)
    assert {k: s.get(k) for k in DEFAULTS} == {k: v[0] for k, v in DEFAULTS.items()}
    assert set(s.sources.values()) == {"default"}
    # the three forms of a flag; an alias and the key itself are the same setting; a bare boolean is true
    s = load(["--temp", "0", "--sampling.top-k=7", "--ignore-eos", "--page-size", "8", "--engine.overlap=false"], cwd=tmp_path)
    assert s.number("sampling.temperature") == 0 and s.integer("sampling.top-k") == 7
    assert s.boolean("sampling.ignore-eos") and s.integer("backend.kv-block") == 8 and not s.boolean("engine.overlap")
    assert s.sources["sampling.temperature"] == "flag" and s.sources["sampling.top-p"] == "default"
    p = s.sampling()
    assert p.temperature == 0 and p.top_k == 7 and p.ignore_eos
    # a boolean before another option takes no value; before a value it takes that value
    assert load(["--ignore-eos", "--temp", "1"], cwd=tmp_path).boolean("sampling.ignore-eos")
    assert not load(["--ignore-eos", "false"], cwd=tmp_path).boolean("sampling.ignore-eos")
    # what the command line alone knows is kept apart from the settings
    s = load(["--tokens", "1,2,3", "--random-prompt", "5"], cwd=tmp_path)
    assert s.cli == {"tokens": "1,2,3", "random-prompt": "5"}


def test_properties_file_lies_between_defaults_and_flags(tmp_path):
    (tmp_path / "jllm.properties").write_text("# a comment\n! another\n\nsampling.top-k = 11\nbackend.ctx=2048\n")
    s = load(["--ctx", "512"], cwd=tmp_path)                      # found in the working directory
    assert s.integer("sampling.top-k") == 11 and s.integer("backend.ctx") == 512
    assert s.sources["sampling.top-k"].endswith("jllm.properties") and s.sources["backend.ctx"] == "flag"
    other = tmp_path / "other.properties"
    other.write_text("sampling.top-k=3\n")
    assert load([], env={"JLLM_CONFIG": str(other)}, cwd=tmp_path).integer("sampling.top-k") == 3     # the environment's file
    (tmp_path / "third.properties").write_text("sampling.top-k=4\n")
    assert load(["--config", str(tmp_path / "third.properties")], env={"JLLM_CONFIG": str(other)},
                cwd=tmp_path).integer("sampling.top-k") == 4                                          # --config wins
    text = load(["--top-k", "9"], cwd=tmp_path).describe()
    assert "sampling.top-k = 9    # flag" in text and "backend.ctx = 2048" in text and text.count("\n") == len(DEFAULTS)
    for bad, what in (("sampling.topk=1\n", "unknown setting 'sampling.topk'"), ("just a line\n", "expected key=value")):
        other.write_text(bad)
        with pytest.raises(SettingsError, match=what):
            load(["--config", str(other)], cwd=tmp_path)
    with pytest.raises(SettingsError, match="config file not found"):
        load(["--config", str(tmp_path / "missing")], cwd=tmp_path)


@pytest.mark.parametrize("args,what", [
    (["--nonsense", "1"], "unknown option --nonsense"),
    (["stray"], "unexpected argument 'stray'"),
    (["--top-k"], "needs a value"),
    (["--dtype", "fp16"], "backend.dtype must be bf16 or fp32"),
    (["--ctx", "many"], "backend.ctx must be an integer"),
    (["--page-size", "0"], "backend.kv-block must be at least 1"),
    (["--kv-share", "1.5"], "backend.kv-share must be in"),
    (["--num-pages", "-3"], "backend.num-pages must be at least 0"),
    (["--engine.cuda-graphs", "perhaps"], "engine.cuda-graphs must be true or false"),
    (["--engine.overlap", "perhaps"], "engine.overlap must be true or false"),
    (["--top-p", "0"], "top_p"),
    (["--temp", "-1"], "temperature"),
    (["--bench.rounds", "0"], "bench.rounds must be at least 1"),
])
def test_wrong_settings_are_refused_before_anything_loads(args, what, tmp_path, capsys):
    with pytest.raises(SettingsError, match=what):
        load(args, cwd=tmp_path)
    assert main(["config", *args]) == 2                            # and the program exits with 2, saying why
    assert what.split("'")[0].split(" must")[0] in capsys.readouterr().err


def test_commands(capsys, tmp_path):
    assert main([]) == 0 and "usage: jllm" in capsys.readouterr().err
    assert main(["config", "--top-k", "5"]) == 0
    assert "sampling.top-k = 5    # flag" in capsys.readouterr().out
    assert main(["dance"]) == 2 and "unknown command: dance" in capsys.readouterr().err
    assert main(["run", "--tokens", "1,2"]) == 2 and "no model" in capsys.readouterr().err
    assert main(["run", "--random-weights", "1"]) == 2 and "--model-config" in capsys.readouterr().err


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_run_generates_the_plain_implementation_s_tokens(dtype, tmp_path):
    """`bin/jllm run` as a user starts it: a model folder, a token prompt, greedy; and a random model from a config."""
    from tests.plain import qwen3_plain as plain
    from tests.tiny import TINY_B, make_model_folder, random_tokens
    folder = make_model_folder(TINY_B, 5, tmp_path / "m")
    cfg, weights = plain.load_plain(folder)
    prompt = random_tokens(23, TINY_B["vocab_size"], 3)
    want = plain.greedy_generate(cfg, weights, prompt, 6)
    cmd = [sys.executable, str(ROOT / "bin" / "jllm"), "run", "--model", str(folder), "--dtype", dtype, "--temp", "0",
           "--max-tokens", "6", "--ignore-eos", "--ctx", "128", "--page-size", "8", "--num-pages", "64", "--batch", "16",
           "--tokens", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().split(",")]
    if dtype == "fp32":
        assert got == want
    else:
        logits = plain.forward(cfg, weights, prompt + got[:-1])
        scale = float(logits.abs().max())
        assert all(float(logits[len(prompt) - 1 + i].max() - logits[len(prompt) - 1 + i][t]) <= 1.2e-2 * scale
                   for i, t in enumerate(got))
    assert "Model: Qwen3ForCausalLM" in proc.stderr and "[length]" in proc.stderr
    # the same architecture with random weights from a config.json and a seed; the overlap switched off gives the same tokens
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    outs = []
    for overlap in ("true", "false"):
        cmd = [sys.executable, str(ROOT / "bin" / "jllm"), "run", "--random-weights", "5", "--model-config",
               str(tmp_path / "config.json"), "--dtype", dtype, "--temp", "0", "--max-tokens", "6", "--ignore-eos", "--ctx",
               "128", "--page-size", "8", "--num-pages", "64", "--engine.overlap", overlap, "--tokens", ",".join(map(str, prompt))]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=tmp_path)
        assert proc.returncode == 0, proc.stderr[-2000:]
        outs.append(proc.stdout.strip())
    assert outs[0] == outs[1] and len(outs[0].split(",")) == 6
