"""What stands in for a memory checker on the device (GPU): the library built with bounds checks, and a bounded wait
that is made to run out.

compute-sanitizer cannot be used where these tests run. Instead the kernels can be built a second time with
-DJLLM_CHECK_BOUNDS (JLLM_B200_CHECK_BOUNDS=1 chooses that library): every table index, page id, cache slot and
token id is then compared with its limit, an access outside is skipped and recorded, and
`ops.check_kernel_errors()` raises. The replay traces run once under it; and kernels that are handed bad tables
on purpose must skip, report and go on. A step of the reference that fails likewise reports and the others go on
(src/main/java/org/robomiri/jllm/engine/BatchGroup.java:396-402).
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"


def checked_env():
    env = dict(os.environ)
    env["JLLM_B200_CHECK_BOUNDS"] = "1"
    return env


def test_bad_tables_slots_and_tokens_are_skipped_and_reported():
    proc = subprocess.run([sys.executable, str(ROOT / "tests" / "bounds_cases.py")], env=checked_env(),
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, (proc.stdout[-3000:], proc.stderr[-3000:])
    assert proc.stdout.count("ok:") == 10, proc.stdout


def test_replay_traces_run_clean_under_the_checked_library():
    """The mixed traces (pages used again, windows releasing pages, portions beside decoding rows) and the steps of
    the scheduler's form, with every paged access checked: nothing is caught, and the logits are right."""
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "tests/test_gpu_replay.py", "tests/test_gpu_scheduled.py",
           "-k", "mixed_batches or four_live or hundred"]
    proc = subprocess.run(cmd, env=checked_env(), cwd=ROOT, capture_output=True, text=True, timeout=1800)
    assert proc.returncode == 0, (proc.stdout[-3000:], proc.stderr[-3000:])
    assert " passed" in proc.stdout and "failed" not in proc.stdout


def test_a_wait_that_runs_out_returns_and_is_reported():
    """One 128 x 128 x 64 tile whose barrier expects more bytes than arrive, with waits that give up after 1,024
    tries: the kernel returns, the error word is raised, and the next product is right."""
    from jllm_serve_b200.csrc import ops
    ops.require_device()
    ops.check_kernel_errors()
    g = torch.Generator().manual_seed(3)
    a = torch.randn(128, 64, generator=g).bfloat16().to(DEV)
    w = (torch.randn(128, 64, generator=g) * 0.05).bfloat16().to(DEV)
    out = torch.zeros(128, 128, device=DEV)
    ops.gemm_tcgen05_starve_next()
    ops.gemm_tcgen05(a, w, out, tile_width=128)
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelError, match="bounded wait ran out inside gemm_tcgen05"):
        ops.check_kernel_errors()
    ops.check_kernel_errors()                                   # read once, cleared
    again = torch.zeros(128, 128, device=DEV)
    ops.gemm_tcgen05(a, w, again, tile_width=128)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    want = a.double().cpu() @ w.double().cpu().t()
    assert torch.allclose(again.cpu().double(), want, rtol=1e-4, atol=1e-4)
