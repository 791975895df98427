"""Builds the kernel library from the .cu files beside this file, in-tree, with nvcc for sm_100a, and the
host library (csrc/host/*.cpp: pools, block tables, batch tables) with the system's C++ compiler.

The library is compiled at the first call that needs it and again whenever a source, a
header or a flag changes (a hash of all of them is kept beside the library). Each .cu
file becomes one object, compiled in parallel; a line is printed when each finishes, so a
first call in a fresh checkout shows progress. Nothing is written outside the build
folder: `csrc/_build/` by default, or `$JLLM_B200_BUILD_DIR`, or a folder under the
system's temporary directory if the tree is read-only.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libjllm_b200.so"
CHECKED_LIB_NAME = "libjllm_b200_checked.so"      # the same sources with -DJLLM_CHECK_BOUNDS
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("JLLM_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found (looked at $JLLM_B200_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels cannot be built, and there is no other path")


def sources() -> list:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def checked_build_wanted() -> bool:
    """JLLM_B200_CHECK_BOUNDS=1 chooses the library whose kernels check every table index, page id, cache slot and
    token id before they use it (slower; for tests and for hunting a fault)."""
    return os.environ.get("JLLM_B200_CHECK_BOUNDS", "0") not in ("", "0")


def _fingerprint(nvcc: str, extra=()) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + list(extra)).encode())
    h.update(nvcc.encode())
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build_dir() -> Path:
    env = os.environ.get("JLLM_B200_BUILD_DIR")
    if env:
        d = Path(env)
    else:
        d = CSRC / "_build"
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"jllm_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[jllm-b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool, extra=()) -> str:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def ensure_built(force: bool = False, verbose: bool = False, checked: bool | None = None) -> Path:
    """Returns the path of an up-to-date library, compiling it first if need be. `checked` (default: what
    JLLM_B200_CHECK_BOUNDS says) chooses the variant with bounds checks, which is built beside the ordinary one."""
    checked = checked_build_wanted() if checked is None else checked
    extra = ["-DJLLM_CHECK_BOUNDS"] if checked else []
    tag = "checked_" if checked else ""
    with _lock:
        nvcc = None
        out_dir = build_dir()
        lib, stamp = out_dir / (CHECKED_LIB_NAME if checked else LIB_NAME), out_dir / f"{tag}stamp.json"
        try:
            nvcc = find_nvcc()
        except BuildError:
            if lib.is_file() and not force:
                return lib  # a prebuilt library travels with the tree; without nvcc it cannot be checked
            raise
        want = _fingerprint(nvcc, extra)
        if not force and lib.is_file() and stamp.is_file():
            try:
                if json.loads(stamp.read_text()).get("fingerprint") == want:
                    return lib
            except (json.JSONDecodeError, OSError):
                pass
        srcs = sources()
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call, or a source changed)"
             + (", with bounds checks" if checked else ""))
        t0 = time.time()
        done = []
        stop = threading.Event()

        def heartbeat():
            while not stop.wait(10.0):
                _say(f"... still compiling, {len(done)}/{len(srcs)} files done after {time.time() - t0:.0f} s")

        hb = threading.Thread(target=heartbeat, daemon=True)
        hb.start()
        logs = {}
        try:
            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
                futures = {}
                for s in srcs:
                    obj = out_dir / (tag + s.stem + ".o")
                    futures[pool.submit(_compile_one, nvcc, s, obj, verbose, extra)] = s
                for fut, s in futures.items():
                    logs[s.name] = fut.result()
                    done.append(s)
                    _say(f"compiled {s.name} ({len(done)}/{len(srcs)}, {time.time() - t0:.0f} s)")
            tmp = out_dir / (lib.name + f".tmp{os.getpid()}")
            link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp)] + [str(out_dir / (tag + s.stem + ".o")) for s in srcs]
            proc = subprocess.run(link, capture_output=True, text=True)
            if proc.returncode != 0:
                raise BuildError(f"linking {lib.name} failed:\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp, lib)
            stamp.write_text(json.dumps({"fingerprint": want, "seconds": round(time.time() - t0, 1)}))
        finally:
            stop.set()
        _say(f"built {lib.name} in {time.time() - t0:.0f} s")
        if verbose:
            for name, log in logs.items():
                print(f"---- {name}\n{log}", file=sys.stderr)
        return lib


# ---- the host library: plain C++, no CUDA ---------------------------------------------------------------------------

HOST_LIB_NAME = "libjllm_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


def find_cxx() -> str:
    for cand in (os.environ.get("JLLM_B200_CXX"), os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"),
                 shutil.which("clang++")):
        if cand and (Path(cand).is_file() or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler found (looked at $JLLM_B200_CXX, $CXX, g++, c++, clang++): the host side of the "
                     "engine (page pools, block tables, batch tables) cannot be built")


def host_sources() -> list:
    return sorted((CSRC / "host").glob("*.cpp"))


def ensure_host_built(force: bool = False) -> Path:
    """The C++ library of the host-side bookkeeping (csrc/host/*.cpp), built with the system's C++ compiler; it needs
    neither nvcc nor a GPU."""
    with _lock:
        out_dir = build_dir()
        lib, stamp = out_dir / HOST_LIB_NAME, out_dir / "host_stamp.json"
        try:
            cxx = find_cxx()
        except BuildError:
            if lib.is_file() and not force:
                return lib
            raise
        h = hashlib.sha256()
        h.update((cxx + " ".join(HOST_FLAGS)).encode())
        for p in host_sources():
            h.update(p.name.encode())
            h.update(p.read_bytes())
        want = h.hexdigest()
        if not force and lib.is_file() and stamp.is_file():
            try:
                if json.loads(stamp.read_text()).get("fingerprint") == want:
                    return lib
            except (json.JSONDecodeError, OSError):
                pass
        t0 = time.time()
        tmp = out_dir / (HOST_LIB_NAME + f".tmp{os.getpid()}")
        proc = subprocess.run([cxx, *HOST_FLAGS, "-o", str(tmp), *[str(p) for p in host_sources()]],
                              capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"{cxx} failed on the host library:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, lib)
        stamp.write_text(json.dumps({"fingerprint": want, "seconds": round(time.time() - t0, 1)}))
        _say(f"built {lib.name} in {time.time() - t0:.0f} s")
        return lib


if __name__ == "__main__":
    print(ensure_host_built(force="--force" in sys.argv))
    print(ensure_built(force="--force" in sys.argv, verbose="-v" in sys.argv))
