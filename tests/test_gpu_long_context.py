"""The attention kernels over tens of thousands of cached keys (GPU).

Among so many keys a tile of 64 that is dropped, doubled or read from the wrong page moves an average by less than
bfloat16's rounding, so here every (query row, head) is AIMED: its query is a multiple of ONE key of its own, chosen at
random among those it may see (and often at an edge: the first one, its own position, the two sides of a 64-key tile or
of a page), so that its softmax is all but that key and its result is that key's value. A key that is not where the
block table says, a tile that a split or an evenly dealt run loses, a window that is off by one: each gives some row a
wholly different value. The reference is the plain float32 formula on the same bfloat16-rounded numbers, computed for
the step's rows only (q . k * scale, softmax over the visible keys, weighted sum of the values; the formulas of
src/main/java/org/robomiri/jllm/cpu/KvCache.java:455-464,595-623 and model/Attention.java:68-71).
"""
import math
import random

import pytest
import torch

from tests.test_gpu_kernels import DEV, rows_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from jllm_serve_b200.csrc import ops as module
    module.require_device()
    return module


def aimed_case(H, Hkv, hd, page, lens, q_lens, window, scale, seed):
    """Requests of `lens` cached positions in a shuffled pool of pages (unused slots NaN); the last `q_lens[s]` positions
    of each are the step's rows. Returns q, caches, row tables, block tables, the wanted [rows, H * hd] and the share
    of a row's softmax weight that lies on its aimed key (smallest over all rows and heads)."""
    rng = random.Random(seed)
    gen = torch.Generator(device=DEV).manual_seed(seed)
    G = H // Hkv
    pages_of = [-(-L // page) for L in lens]
    pool = sum(pages_of) + 7
    perm = torch.randperm(pool, generator=torch.Generator().manual_seed(seed)).tolist()
    kc = torch.full((pool, Hkv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    tables = torch.full((len(lens), max(pages_of) + 2), -1, dtype=torch.int32)
    qs, wants, row_seg, row_pos, sure = [], [], [], [], 1.0
    for s, (L, n) in enumerate(zip(lens, q_lens)):
        k = torch.randn(L, Hkv, hd, device=DEV, generator=gen).bfloat16()
        v = (3 * torch.randn(L, Hkv, hd, device=DEV, generator=gen)).bfloat16()
        ids = [perm.pop() for _ in range(pages_of[s])]
        tables[s, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        pad = pages_of[s] * page - L
        for cache, x in ((kc, k), (vc, v)):
            x = torch.cat([x, torch.full((pad, Hkv, hd), float("nan"), dtype=x.dtype, device=DEV)]) if pad else x
            cache[torch.tensor(ids, device=DEV)] = x.view(pages_of[s], page, Hkv, hd).transpose(1, 2)
        positions = list(range(L - n, L))
        aim = torch.empty(n, H, dtype=torch.long)
        for i, p in enumerate(positions):
            lo = max(0, p + 1 - window) if window > 0 else 0
            for h in range(H):
                edges = [lo, p, min(p, lo + 1), max(lo, p - 1)]
                for unit in (64, page, 128):
                    b = rng.randint(lo // unit, p // unit) * unit
                    edges += [min(max(b, lo), p), min(max(b - 1, lo), p)]
                aim[i, h] = rng.choice(edges) if rng.random() < 0.5 else rng.randint(lo, p)
        kf = k.float()
        target = kf[aim.to(DEV), (torch.arange(H, device=DEV) // G)[None, :]]             # [n, H, hd]
        q = (target * (30.0 / scale / (target * target).sum(-1, keepdim=True))).bfloat16()
        qf, vf = q.float(), v.float()
        want = torch.empty(n, H, hd, device=DEV)
        pos_t = torch.tensor(positions, device=DEV)
        keys = torch.arange(L, device=DEV)
        visible = keys[None, :] <= pos_t[:, None]
        if window > 0:
            visible &= keys[None, :] >= pos_t[:, None] + 1 - window
        for h in range(H):
            scores = (qf[:, h] @ kf[:, h // G].t()) * scale
            scores = scores.masked_fill(~visible, float("-inf"))
            e = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
            prob = e * (1.0 / e.sum(dim=-1, keepdim=True))
            want[:, h] = prob @ vf[:, h // G]
            sure = min(sure, float(prob.gather(1, aim[:, h:h + 1].to(DEV)).min()))
        qs.append(q.reshape(n, H * hd))
        wants.append(want.reshape(n, H * hd).cpu())
        row_seg += [s] * n
        row_pos += positions
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return torch.cat(qs).contiguous(), kc, vc, i32(row_seg), i32(row_pos), tables.to(DEV), torch.cat(wants), sure


@pytest.mark.parametrize("H,Hkv,hd,page,window", [(16, 2, 128, 16, 0), (8, 1, 128, 64, 0), (8, 2, 128, 16, 5000),
                                                   (12, 3, 64, 16, 0), (4, 2, 256, 32, 0), (6, 2, 80, 8, 0)])
def test_decode_attention_finds_its_key_among_tens_of_thousands(ops, H, Hkv, hd, page, window):
    """One row per request, 3 to 40 thousand keys each: one block per pair, splits, and the evenly dealt kernel."""
    lens = [40000, 33001, 20480, 12345, 8191, 4097, 3000, 36000, 25000, 16385]
    scale = 1.0 / math.sqrt(hd)
    q, kc, vc, rseg, rpos, tables, want, sure = aimed_case(H, Hkv, hd, page, lens, [1] * len(lens), window, scale, 3 + hd)
    assert sure > 0.99, "the queries do not single out their keys: the test would see nothing"
    rows = len(lens)
    for splits in (1, 4, 13, 32):
        out = torch.full_like(q, float("nan"))
        scratch = torch.full((ops.attention_decode_scratch_floats(rows, H, hd, splits) + 1,), float("nan"), device=DEV)
        ops.attention_decode(q, kc, vc, out, rseg, rpos, tables, rows, H, Hkv, hd, page, window, scale, splits, scratch)
        rows_close(out, want, f"decode, {splits} splits")
    if hd in (64, 128, 256):
        for blocks in (296, 37, 62 * Hkv):
            blocks = min(blocks, 62 * Hkv)
            out = torch.full_like(q, float("nan"))
            scratch = torch.full((ops.attention_decode_flat_scratch_floats(rows, H, Hkv, hd, blocks),), float("nan"),
                                 device=DEV)
            ops.attention_decode_flat(q, kc, vc, out, rseg, rpos, tables, rows, H, Hkv, hd, page, window, scale, blocks,
                                      scratch)
            rows_close(out, want, f"decode dealt out over {blocks} blocks")
    ops.check_kernel_errors()


@pytest.mark.parametrize("kernel,H,Hkv,hd,page,window", [("pair", 8, 2, 128, 16, 0), ("tc", 8, 2, 128, 16, 0),
                                                          ("pair", 4, 1, 128, 64, 7000), ("tc", 6, 3, 128, 8, 129),
                                                          ("mma", 6, 2, 64, 16, 0), ("mma", 2, 1, 256, 32, 3000)])
def test_prefill_attention_finds_its_keys_among_tens_of_thousands(ops, kernel, H, Hkv, hd, page, window):
    """Portions of prompts far into long requests (the portion a scheduler cuts at position 30 thousand), beside a
    short one and a single row: every row and head has a key of its own to find."""
    lens, q_lens = [33000, 20001, 300, 12345, 9000], [300, 129, 300, 1, 513]
    scale = 1.0 / math.sqrt(hd)
    q, kc, vc, rseg, rpos, tables, want, sure = aimed_case(H, Hkv, hd, page, lens, q_lens, window, scale, 11 + hd + page)
    assert sure > 0.99, "the queries do not single out their keys: the test would see nothing"
    out = torch.full_like(q, float("nan"))
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    starts = [sum(q_lens[:i]) for i in range(len(lens))]
    ops.attention_prefill(q, kc, vc, out, i32(starts), i32(q_lens), i32(lens), tables, q.shape[0], H, Hkv, hd, page, window,
                          scale, kernel=kernel)
    assert ops.attention_prefill_tc_error() == 0
    rows_close(out, want, f"prefill {kernel}")
    ops.check_kernel_errors()
