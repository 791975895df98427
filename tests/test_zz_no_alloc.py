"""The decode attention entry point that brings its own scratch memory (GPU).

`jllm_attention_decode_static` is for programs that cannot give the library scratch memory: a server
that has handed all device memory to its cache pool, or a host that forbids allocation after start-up.
The test calls it the way such a program would, through the exported C symbol with raw device pointers,
twice in a row for every case (the second call meets the first call's leftovers in the built-in array), and
checks each result against the plain attention of the test suite and against the ordinary entry point, which
gets scratch from the caller. Head sizes of both decode kernels (128: keys staged through shared memory; 48:
straight from global memory) and a window are driven through it, and the device's free memory is read before and
after the calls: it does not change.

The file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes
import math

import pytest
import torch

from tests.test_gpu_kernels import attention_case, rows_close

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


CASES = [  # heads, kv heads, head size, window, (lengths, splits) of the two calls in a row
    (8, 2, 128, 0, (((700, 1, 300, 1100), 4), ((90, 2000, 513), 7))),
    (6, 2, 48, 0, (((300, 17, 1000), 3), ((64, 131, 2, 700), 5))),
    (8, 2, 128, 100, (((700, 50, 300, 1100), 5), ((101, 99, 1500), 2))),
]


@pytest.mark.parametrize("H, Hkv, hd, window, calls", CASES)
def test_static_scratch_entry_point_is_right_twice_in_a_row_and_allocates_nothing(H, Hkv, hd, window, calls):
    from jllm_serve_b200.csrc import ops
    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    page, scale = 16, 1.0 / math.sqrt(hd)
    prepared = []
    for lens, splits in calls:
        for mode in ("far", "planted"):
            q, kc, vc, out, seg, pos, tables, want, _ = attention_case(ops, torch.bfloat16, H, Hkv, hd, page, list(lens), window,
                                                                       scale, mode, [1] * len(lens))
            got, same = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
            scratch = torch.empty(len(lens) * H * splits * (hd + 2), dtype=torch.float32, device=DEV)
            prepared.append((q, kc, vc, seg, pos, tables, want, got, same, scratch, len(lens), splits, mode))
    # one warm call first: the entry point looks its array's address up at its first call on a device
    q, kc, vc, seg, pos, tables, want, got, same, scratch, rows, splits, mode = prepared[0]
    rc = lib.jllm_attention_decode_static(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), got.data_ptr(), got.stride(0),
                                          seg.data_ptr(), pos.data_ptr(), tables.data_ptr(), tables.stride(0), rows, H, Hkv, hd,
                                          page, window, scale, splits, stream)
    assert rc == 0, lib.jllm_last_error().decode()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for q, kc, vc, seg, pos, tables, want, got, same, scratch, rows, splits, mode in prepared:
        args = (q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr())
        tail = (seg.data_ptr(), pos.data_ptr(), tables.data_ptr(), tables.stride(0), rows, H, Hkv, hd, page, window, scale,
                splits)
        rc = lib.jllm_attention_decode_static(*args, got.data_ptr(), got.stride(0), *tail, stream)
        assert rc == 0, lib.jllm_last_error().decode()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the entry point took device memory"
    for q, kc, vc, seg, pos, tables, want, got, same, scratch, rows, splits, mode in prepared:
        args = (q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr())
        tail = (seg.data_ptr(), pos.data_ptr(), tables.data_ptr(), tables.stride(0), rows, H, Hkv, hd, page, window, scale,
                splits)
        rc = lib.jllm_attention_decode(*args, same.data_ptr(), same.stride(0), *tail, scratch.data_ptr(), stream)
        assert rc == 0, lib.jllm_last_error().decode()
        torch.cuda.synchronize()
        rows_close(got, want, f"static entry, head size {hd}, window {window}, {splits} splits, {mode}")
        assert torch.equal(got, same), "the two entry points run the same kernels: their results are the same bits"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from jllm_serve_b200.csrc import ops
    lib = _library()
    cap = lib.jllm_attention_decode_static_capacity()
    assert cap == 2 * 1024 * 1024
    q, kc, vc, out, seg, pos, tables, want, _ = attention_case(ops, torch.bfloat16, 8, 2, 128, 16, [40, 50], 0, 0.1, False, [1, 1])
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
