"""The decode attention entry point that brings its own scratch memory (GPU).

`jllm_attention_decode_static` is for programs that cannot give the library scratch memory: a server
that has handed all device memory to its cache pool, or a host that forbids allocation after start-up.
The test calls it the way such a program would, through the exported C symbol with raw device pointers,
twice in a row (the second call meets the first call's leftovers in the built-in array), and checks
each result against the ordinary entry point, which gets scratch from the caller.

The file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _library():
    from jllm_serve_b200.csrc.build import ensure_built
    lib = ctypes.CDLL(str(ensure_built()))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.jllm_attention_decode_static.argtypes = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P]
    lib.jllm_attention_decode_static.restype = I
    lib.jllm_attention_decode.argtypes = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P, P]
    lib.jllm_attention_decode.restype = I
    lib.jllm_attention_decode_static_capacity.restype = ctypes.c_longlong
    lib.jllm_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed, lens, H, Hkv, hd, page):
    """Requests of `lens` cached positions in a shuffled pool whose unused rows are NaN; one query row each."""
    g = torch.Generator().manual_seed(seed)
    pool = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(pool, generator=g).tolist()
    kc = torch.full((pool, Hkv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    tables = torch.full((len(lens), max(-(-n // page) for n in lens)), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        k = torch.randn(n, Hkv, hd, generator=g).bfloat16()
        v = torch.randn(n, Hkv, hd, generator=g).bfloat16()
        for b in range(-(-n // page)):
            pg = perm.pop()
            tables[s, b] = pg
            m = min(page, n - b * page)
            kc[pg, :, :m] = k[b * page:b * page + m].transpose(0, 1).to(DEV)
            vc[pg, :, :m] = v[b * page:b * page + m].transpose(0, 1).to(DEV)
    q = torch.randn(len(lens), H * hd, generator=g).bfloat16().to(DEV)
    seg = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    return q, kc, vc, seg, pos, tables.to(DEV)


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    H, Hkv, hd, page = 8, 2, 128, 16
    scale = 1.0 / math.sqrt(hd)
    for call, (lens, splits) in enumerate([((700, 1, 300, 1100), 4), ((90, 2000, 513), 7)]):
        q, kc, vc, seg, pos, tables = _case(100 + call, lens, H, Hkv, hd, page)
        rows = len(lens)
        args = (q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr())
        tail = (seg.data_ptr(), pos.data_ptr(), tables.data_ptr(), tables.stride(0), rows, H, Hkv, hd, page, 0, scale,
                splits)
        got = torch.full_like(q, float("nan"))
        rc = lib.jllm_attention_decode_static(*args, got.data_ptr(), got.stride(0), *tail, stream)
        assert rc == 0, lib.jllm_last_error().decode()
        want = torch.full_like(q, float("nan"))
        scratch = torch.empty(rows * H * splits * (hd + 2), dtype=torch.float32, device=DEV)
        rc = lib.jllm_attention_decode(*args, want.data_ptr(), want.stride(0), *tail, scratch.data_ptr(), stream)
        assert rc == 0, lib.jllm_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), \
            f"call {call}: differs by {float((got.float() - want.float()).abs().max())}"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    cap = lib.jllm_attention_decode_static_capacity()
    assert cap == 2 * 1024 * 1024
    q, kc, vc, seg, pos, tables = _case(7, (40, 50), 8, 2, 128, 16)
    out = torch.zeros_like(q)
    # rows * heads * splits * (head_dim + 2) floats: claim far more rows than the array can serve; the size
    # check comes before anything is launched, so the short tensors are never touched
    rows, splits = 4096, 32
    assert rows * 8 * splits * 130 > cap
    rc = lib.jllm_attention_decode_static(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                          out.stride(0), seg.data_ptr(), pos.data_ptr(), tables.data_ptr(),
                                          tables.stride(0), rows, 8, 2, 128, 16, 0, 0.1, splits,
                                          torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"built-in array holds" in lib.jllm_last_error()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0
