"""Run by tests/test_gpu_bounds.py in a process of its own, with JLLM_B200_CHECK_BOUNDS=1 (the library with bounds
checks is chosen when the process loads it). Hands every paged kernel a table, a slot list or token ids that point
outside their arrays and checks that the library SKIPS those accesses, says what it caught, and computes the right
thing again afterwards. Refuses to run on the ordinary library, where such inputs would be read.
"""
import math
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from jllm_serve_b200.csrc import ops  # noqa: E402
from tests.test_gpu_kernels import attention_case  # noqa: E402

DEV = "cuda:0"


def main() -> int:
    ops.require_device()
    if not ops.checks_bounds():
        print("the library was built without bounds checks: nothing is run")
        return 3
    assert ops.bounds_errors() == {}
    H, Hkv, page = 4, 2, 16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)

    def spoil(tables, pool):
        bad = tables.clone()
        bad[1, 0] = pool + 7          # a page beyond the pool
        bad[2, 1] = -1                # a page that was given back
        return bad

    def caught(file, *whats):
        got = ops.bounds_errors()
        assert set(got) == {file}, (file, got)
        assert got[file][0] in whats and got[file][3] >= 1, got
        assert ops.bounds_errors() == {}                         # reading clears

    # ---- attention over the cache: every kernel, a clean run after the spoilt one ---------------------------------
    for name, hd, dtype in (("plain", 48, torch.float32), ("decode", 48, torch.bfloat16), ("decode", 128, torch.bfloat16),
                            ("flat", 128, torch.bfloat16), ("mma", 64, torch.bfloat16), ("tc", 128, torch.bfloat16),
                            ("pair", 128, torch.bfloat16)):
        scale = 1.0 / math.sqrt(hd)
        lens = [40, 300, 200, 70]
        q_lens = [1, 1, 1, 1] if name in ("decode", "flat") else [3, 260, 150, 2]
        q, kc, vc, out, rseg, rpos, tables, want, q_lens = attention_case(ops, dtype, H, Hkv, hd, page, lens, 0, scale, False,
                                                                          q_lens)
        pool = kc.shape[0]
        ops.set_pool_pages(pool)
        rows = q.shape[0]
        starts = [sum(q_lens[:i]) for i in range(len(lens))]
        scratch = torch.empty(1 << 20, device=DEV)

        def run(tab, name=name, hd=hd):
            out.fill_(float("nan"))
            if name == "plain":
                ops.attention_plain(q, q.stride(0), kc, vc, out, rseg, rpos, tab, rows, H, Hkv, hd, page, 0, scale)
            elif name == "decode":
                ops.attention_decode(q, kc, vc, out, rseg, rpos, tab, rows, H, Hkv, hd, page, 0, scale, 3, scratch)
            elif name == "flat":
                ops.attention_decode_flat(q, kc, vc, out, rseg, rpos, tab, rows, H, Hkv, hd, page, 0, scale, 5, scratch)
            else:
                ops.attention_prefill(q, kc, vc, out, i32(starts), i32(q_lens), i32(lens), tab, rows, H, Hkv, hd, page, 0,
                                      scale, kernel=name)
            torch.cuda.synchronize()

        run(spoil(tables, pool))
        file = {"plain": "attention_plain", "decode": "attention_decode", "flat": "attention_decode",
                "mma": "attention_prefill", "tc": "attention_prefill_tc", "pair": "attention_prefill_pair"}[name]
        caught(file, "a page id")
        # a table whose row is shorter than the keys need: the index past its end is caught, not read
        short = tables[:, :3].contiguous()
        run(short)
        caught(file, "a block-table index", "a page id")
        run(tables)
        assert ops.bounds_errors() == {}
        tol = dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        assert torch.allclose(out.float().cpu(), want, **tol), (name, hd)
        ops.check_kernel_errors()
        print(f"ok: {name} head size {hd}")

    # ---- the decode attention that makes its own rows' keys and values: a spoilt page of the newest position is neither
    # read nor written; afterwards the same bits as the row-wise kernel followed by the attention ----------------------
    hd, scale, eps = 128, 1.0 / math.sqrt(128), 1e-6
    lens = [40, 300, 200, 70]
    pool = sum(-(-n // page) for n in lens) + 3
    ops.set_pool_pages(pool)
    tables = torch.full((4, 20), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(lens):
        k = -(-n // page)
        tables[r, :k] = torch.arange(at, at + k, dtype=torch.int32)
        at += k
    tables = tables.to(DEV)
    kc0 = (torch.randn(pool, Hkv, page, hd, device=DEV) * 0.5).to(torch.bfloat16)
    vc0 = torch.randn(pool, Hkv, page, hd, device=DEV).to(torch.bfloat16)
    qkv = torch.randn(4, (H + 2 * Hkv) * hd, device=DEV).to(torch.bfloat16)
    gain = torch.ones(hd, dtype=torch.bfloat16, device=DEV)
    ang = torch.outer(torch.arange(301, dtype=torch.float64), 1e4 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    seg, pos = i32([0, 1, 2, 3]), i32([n - 1 for n in lens])
    scratch = torch.empty(1 << 20, device=DEV)

    def fresh(tab, kc, vc, out):
        ops._call("jllm_attention_decode_fresh", qkv.data_ptr(), qkv.stride(0), gain.data_ptr(), gain.data_ptr(),
                  ops._DT[gain.dtype], 1, eps, cos.data_ptr(), sin.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                  out.stride(0), seg.data_ptr(), pos.data_ptr(), tab.data_ptr(), tab.stride(0), 4, H, Hkv, hd, page, 0,
                  scale, 0, 3, scratch.data_ptr(), ops._stream())
        torch.cuda.synchronize()

    bad = tables.clone()
    bad[3, (lens[3] - 1) // page] = pool + 9          # the page of request 3's newest position
    kc, vc, out = kc0.clone(), vc0.clone(), torch.empty(4, H * hd, dtype=torch.bfloat16, device=DEV)
    fresh(bad, kc, vc, out)
    caught("attention_decode", "a page id")
    rest = [r for r in range(pool) if r != int(tables[3, (lens[3] - 1) // page])]
    slots = i32([int(tables[r, (n - 1) // page]) * page + (n - 1) % page for r, n in enumerate(lens)])
    work, kc_a, vc_a, out_a = qkv.clone(), kc0.clone(), vc0.clone(), torch.empty_like(out)
    ops.qk_norm_rope_store(work, gain, gain, eps, cos, sin, hd, pos, slots, kc_a, vc_a, H, Hkv, hd, page)
    ops.attention_decode(work, kc_a, vc_a, out_a, seg, pos, tables, 4, H, Hkv, hd, page, 0, scale, 3, scratch)
    assert torch.equal(kc[rest].view(torch.int16), kc_a[rest].view(torch.int16))      # requests 0 to 2 were written as always
    assert torch.equal(out[:3], out_a[:3])
    kc, vc = kc0.clone(), vc0.clone()
    fresh(tables, kc, vc, out)
    assert ops.bounds_errors() == {}
    assert torch.equal(out, out_a) and torch.equal(kc.view(torch.int16), kc_a.view(torch.int16)) and \
        torch.equal(vc.view(torch.int16), vc_a.view(torch.int16))
    print("ok: decode attention that makes its own rows")

    # ---- the cache write: a slot beyond the pool is dropped, the others are written --------------------------------
    for dtype, hd in ((torch.float32, 48), (torch.bfloat16, 128)):
        R, pages = 40, 6
        ops.set_pool_pages(pages)
        qkv = torch.randn(R, (H + 2 * Hkv) * hd, device=DEV).to(dtype)
        kc = torch.zeros(pages, Hkv, page, hd, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        slots = torch.arange(R, dtype=torch.int32, device=DEV)
        slots[5] = pages * page + 3
        slots[9] = -4
        pos = torch.arange(R, dtype=torch.int32, device=DEV)
        ops.qk_norm_rope_store(qkv, None, None, 1e-6, None, None, 0, pos, slots, kc, vc, H, Hkv, hd, page)
        torch.cuda.synchronize()
        caught("rowwise", "a cache slot")
        flat = vc.permute(0, 2, 1, 3).reshape(pages * page, Hkv * hd)
        v_in = qkv[:, (H + Hkv) * hd:]
        good = [r for r in range(R) if r not in (5, 9)]
        assert torch.equal(flat[good], v_in[good]) and float(flat[5].abs().max()) == 0 and float(flat[9].abs().max()) == 0
        print(f"ok: cache write head size {hd}")

    # ---- token ids: clamped as always, and reported here ----------------------------------------------------------
    table = torch.randn(50, 24, device=DEV)
    out = torch.empty(3, 24, device=DEV)
    ops.embed_rows(i32([1, 50, -2]), table, out)
    torch.cuda.synchronize()
    caught("rowwise", "a token id")
    assert torch.equal(out[0], table[1])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
