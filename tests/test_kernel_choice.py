"""Which kernel a step's work goes to: decisions taken on the host from sizes alone (no GPU, nothing launched)."""
import torch

from jllm_serve_b200.csrc import ops


def test_product_kernel_by_rows_and_shape():
    k = ops.gemm_kernel_for
    assert k(1, 4096, 4096) == "rows"
    assert k(8, 24576, 4096) == "rows"                     # few rows: even the widest matrix goes row by row
    assert k(16, 24576, 4096) == "tiles"                   # 16 rows against gate_up: tcgen05 tiles
    assert k(16, 6144, 4096) == "rows"
    assert k(17, 6144, 4096) == "swap"                     # QKV (50 MB) from 17 rows: weight rows as the MMA's M side
    assert k(64, 6144, 4096) == "swap" and k(128, 6144, 4096) == "swap" and k(160, 6144, 4096) == "swap"
    assert k(161, 6144, 4096) == "tiles" and k(161, 4096, 4096) == "tiles"      # above 160 rows its parked parts cost too much
    # ... except against matrices much longer than high (down), up to the 256 tokens of one tcgen05 N side
    assert k(64, 4096, 12288) == "swap" and k(128, 4096, 12288) == "swap" and k(256, 4096, 12288) == "swap"
    assert k(256, 5120, 17408) == "swap" and k(200, 24576, 4096) == "tiles"
    # 257 to 512 rows against such a matrix: its few 256 x 256 tiles cut up over all pairs
    assert k(257, 4096, 12288) == "pair-streamed" and k(512, 5120, 17408) == "pair-streamed"
    assert k(513, 4096, 12288) == "tiles" and k(400, 6144, 4096) == "tiles" and k(400, 4096, 12288, pairs=0) == "tiles"
    assert k(40, 4096, 4096) == "rows" and k(41, 4096, 4096) == "swap"         # O (34 MB): from 41 rows
    assert k(64, 24576, 4096) == "tiles"                                       # gate_up: whole tiles fill the SMs
    # many rows: two SMs to a 256 x 256 tile where such tiles keep the pairs busy in no more rounds than one-SM tiles
    assert k(2048, 4096, 4096) == "pair" and k(2048, 6144, 4096) == "pair" and k(2048, 24576, 4096) == "pair"
    assert k(1024, 4096, 12288) == "pair" and k(512, 24576, 4096) == "pair"
    assert k(512, 6144, 4096) == "tiles"                   # 48 tiles for 74 pairs
    assert k(300, 24576, 4096) == "tiles"                  # 300 rows: three 128-row tiles, not two of 256
    assert k(1024, 6144, 4096) == "tiles"                  # the one-SM kernel would take 192-wide tiles: 2 rounds of 0.83
    assert k(544, 5120, 5120) == "tiles" and k(544, 5120, 17408) == "tiles"     # a third pair tile an eighth full
    assert k(2048, 4096, 4096, pairs=0) == "tiles"         # a device that runs no pairs
    assert k(16, 24576, 4096, tiles_fit=False) == "rows"
    assert k(8, 4096, 4096, rows_fit=False) == "tiles"
    assert k(8, 4096, 4096, rows_fit=False, tiles_fit=False) == ""


def test_decode_attention_splits_fill_the_gpu_once():
    scratch = torch.empty(2 << 20)
    # 8 rows x 8 kv heads = 64 pairs for 296 places: 4 blocks per pair; 16 keys-of-256 allow up to 32
    assert ops.decode_splits(8, 8, 16, 32, 128, scratch, places=296) == 4
    assert ops.decode_splits(1, 8, 16, 32, 128, scratch, places=296) == 32      # one row: as many as the keys allow, 32 at most
    assert ops.decode_splits(1, 8, 2, 32, 128, scratch, places=296) == 4        # 512 keys: blocks of at least 128
    assert ops.decode_splits(64, 8, 16, 32, 128, scratch, places=296) == 1
    assert ops.decode_splits(8, 8, 16, 32, 128, None, places=296) == 1          # no scratch, no partial results
    tiny = torch.empty(8 * 32 * 2 * (128 + 2))                      # room for two splits only
    assert ops.decode_splits(8, 8, 16, 32, 128, tiny, places=296) == 2


def test_decode_attention_is_dealt_out_evenly_only_where_that_pays():
    scratch = torch.empty(2 << 20)
    assert ops.decode_plan(8, 8, 16, 32, 128, scratch, places=296) == ("split", 4)          # fewer pairs than places
    assert ops.decode_plan(37, 8, 16, 32, 128, scratch, places=296) == ("split", 1)         # 296 pairs: one full round
    how, blocks = ops.decode_plan(64, 8, 16, 32, 128, scratch, places=296)                  # 512 pairs: 1.73 rounds
    assert how == "flat" and blocks == 296
    how, blocks = ops.decode_plan(104, 3, 1, 6, 64, scratch, places=296)                    # few kv heads bound the blocks
    assert how == "flat" and blocks == 62 * 3
    assert ops.decode_plan(64, 8, 16, 32, 80, scratch, places=296)[0] == "split"            # a head size the flat kernel lacks
    assert ops.decode_plan(64, 8, 16, 32, 128, torch.empty(1000), places=296)[0] == "split"  # no room for its partial results


def test_a_decode_steps_bucket_is_clamped_where_it_stops_mattering():
    """`decode_bucket_cap`: from that bucket on the plan of a decode step is the same for every longer context, so the
    step function may clamp the bucket there (and a growing context does not ask for a new captured step every 256
    tokens); below it the bucket is rounded down to one of sixteen levels, each a valid plan for fewer keys."""
    import torch
    from jllm_serve_b200.csrc import ops
    scratch = torch.empty(2 << 20)
    for rows, heads, kv_heads, hd, window in [(1, 32, 8, 128, 0), (8, 32, 8, 128, 0), (64, 32, 8, 128, 0), (3, 40, 8, 128, 0),
                                              (8, 64, 8, 128, 0), (200, 6, 3, 64, 0), (2, 16, 1, 256, 0), (8, 32, 8, 128, 700),
                                              (1, 4, 4, 64, 5000), (37, 8, 2, 64, 0)]:
        cap = ops.decode_bucket_cap(rows, kv_heads, heads, hd, window, scratch, places=296)
        assert 1 <= cap <= ops.KV_BUCKET_MAX

        def plan(b):
            return ops.decode_plan(rows, kv_heads, ops._windowed_bucket(b, window), heads, hd, scratch, 296)
        for b in range(1, ops.KV_BUCKET_MAX + 1):
            assert plan(min(b, cap)) == plan(b), (rows, heads, kv_heads, hd, window, b, cap)
        assert cap == 1 or plan(cap - 1) != plan(cap)
    assert ops.decode_bucket_cap(8, 8, 32, 128, 0, scratch, places=296) == 2       # four splits from 512 keys on
    assert ops.decode_bucket_cap(1, 8, 32, 128, 0, scratch, places=296) == 16      # 32 splits from 4,096 keys on
    levels = [ops.bucket_level(b) for b in range(0, 40)]
    assert levels[:9] == [1, 1, 2, 3, 4, 5, 6, 7, 8] and levels[32:] == [32] * 8
    assert all(l <= max(1, b) and l in ops.KV_BUCKET_LEVELS for b, l in enumerate(levels))
    assert all(4 * b <= 5 * l + 4 for b, l in enumerate(levels[:33]))                # never more than a quarter below
    assert len(set(levels)) == 16
