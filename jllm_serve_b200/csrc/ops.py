"""Python face of the kernel library: loads it (building it first if need be) and wraps each launcher.

The launchers are plain C functions taking device pointers, sizes and a stream; tensors are
torch tensors used as typed device memory only. There is no other implementation behind
these functions: without the library or without a B200 they raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_void_p

import torch

from .build import ensure_built

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None
_device_ok = False


def library():
    global _lib
    if _lib is None:
        path = ensure_built()
        lib = ctypes.CDLL(str(path))
        lib.jllm_last_error.restype = c_char_p
        for name in dir(_Signatures):
            if name.startswith("jllm_"):
                fn = getattr(lib, name)
                fn.argtypes = getattr(_Signatures, name)
                fn.restype = c_int
        _lib = lib
    return _lib


def require_device() -> None:
    """Raises unless a B200 is current and the library can run on it."""
    global _device_ok
    if _device_ok:
        return
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine runs on a B200 (sm_100a) only, it has no CPU path")
    _call("jllm_check_device")
    _device_ok = True


_sm_count = 0


def sm_count() -> int:
    """SMs of the current device, asked of the library once (it asks the driver)."""
    global _sm_count
    if not _sm_count:
        n = library().jllm_sm_count()
        if n <= 0:
            raise KernelError("the device does not say how many SMs it has")
        _sm_count = n
    return _sm_count


def resident_blocks() -> int:
    """Places for blocks of the decode attention on the device: two per SM."""
    return 2 * sm_count()


launch_count = 0   # kernels of this library launched (or captured into a graph) by this process


_functions = {}


def _call(name, *args):
    global launch_count
    fn = _functions.get(name)
    if fn is None:
        fn = _functions[name] = getattr(library(), name)
    launch_count += 1
    code = fn(*args)
    if code != 0:
        raise KernelError(f"{name} failed ({code}): {library().jllm_last_error().decode(errors='replace')}")


def set_dependent_launch(on: bool) -> None:
    """Programmatic dependent launch of the step's kernels on (default) or off."""
    library().jllm_set_pdl(int(on))


def launch_plan(dynamic_smem: int, how: int) -> bool:
    """What the library's launcher decides for a kernel of `dynamic_smem` bytes launched plainly (how 0), as a
    programmatic dependent (1) or as one that wants L1 (2): whether it may overlap its predecessor. Keeps the same
    record as a launch does; launches nothing (a test's view of the rule)."""
    return bool(library().jllm_launch_plan(int(dynamic_smem), int(how)))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle (asked for at every launch: the quick way if torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return 0 if t is None else t.data_ptr()


class _Signatures:
    P, I, F = c_void_p, c_int, c_float
    jllm_check_device = []
    jllm_sm_count = []
    jllm_checks_bounds = []
    jllm_set_pool_pages = [I]
    jllm_bounds_error_attention_plain = [P]
    jllm_bounds_error_attention_decode = [P]
    jllm_bounds_error_attention_prefill = [P]
    jllm_bounds_error_attention_prefill_tc = [P]
    jllm_bounds_error_attention_prefill_pair = [P]
    jllm_bounds_error_rowwise = [P]
    jllm_set_pdl = [I]
    jllm_launch_plan = [ctypes.c_longlong, I]
    jllm_embed_rows = [P, P, I, P, I, I, I, P]
    jllm_feed_tokens = [P, P, I, I, P]
    jllm_rmsnorm = [P, P, I, P, I, P, I, I, F, P]
    jllm_swiglu = [P, P, I, I, I, P]
    jllm_qk_norm_rope_store = [P, I, P, P, I, I, F, P, P, I, P, P, P, P, I, I, I, I, I, I, I, P]
    jllm_gemm_plain = [P, I, I, P, I, P, I, P, I, I, I, I, I, I, P]
    jllm_gemm_small_m = [P, I, P, I, P, I, P, I, I, I, I, I, I, I, P]
    jllm_gemm_tcgen05 = [P, I, P, I, P, I, P, I, I, I, I, I, I, I, I, P, ctypes.c_longlong, I, I, P]
    jllm_gemm_pair = [P, I, P, I, P, I, P, I, I, I, I, I, I, I, I, P, ctypes.c_longlong, I, P]
    jllm_gemm_pair_resident = []
    jllm_gemm_plain_stores = [I]
    jllm_gemm_stream = [P, I, P, I, P, I, P, I, I, I, I, I, I, I, P, ctypes.c_longlong, I, P]
    jllm_gemm_tcgen05_error = []
    jllm_gemm_tcgen05_starve_next = []
    jllm_attention_plain = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P]
    jllm_attention_decode = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P, P]
    jllm_attention_decode_flat = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P, P]
    jllm_attention_prefill = [P, I, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P]
    jllm_attention_prefill_tc = [P, I, P, P, ctypes.c_longlong, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P]
    jllm_attention_prefill_tc_error = []
    jllm_attention_prefill_pair = [P, I, P, P, ctypes.c_longlong, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P]
    jllm_attention_decode_separate_combine = [I]
    jllm_attention_decode_fresh = [P, I, P, P, I, I, F, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P]
    jllm_argmax = [P, I, I, I, P, P]
    jllm_sample = [P, I, I, I, P, P, P, P, P, P, P]


# ---------------------------------------------------------------------------------------------------------

def embed_rows(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = table[ids[r]] as float32; ids int32 [rows]."""
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.dim() == 2
    _call("jllm_embed_rows", ids.data_ptr(), table.data_ptr(), _DT[table.dtype], out.data_ptr(), ids.numel(),
          table.shape[1], table.shape[0], _stream())


def feed_tokens(ids: torch.Tensor, sampled: torch.Tensor) -> None:
    """ids[r] < 0 becomes sampled[-ids[r] - 1]: tokens that the step before sampled go into this step's rows on the
    device, before the host has read them."""
    assert ids.dtype == torch.int32 and sampled.dtype == torch.int32
    _call("jllm_feed_tokens", ids.data_ptr(), sampled.data_ptr(), ids.numel(), sampled.numel(), _stream())


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor, row_index: torch.Tensor | None = None,
            rows: int | None = None) -> None:
    """out[r] = rmsnorm(x[row_index[r] or r]) * gain; x float32 [*, dim]; out float32 or bfloat16."""
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n = (row_index.numel() if row_index is not None else x.shape[0]) if rows is None else rows
    _call("jllm_rmsnorm", x.data_ptr(), gain.data_ptr(), _DT[gain.dtype], out.data_ptr(), _DT[out.dtype],
          _p(row_index), n, x.shape[-1], float(eps), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, j] = silu(gate_up[r, j]) * gate_up[r, hidden + j]."""
    assert gate_up.dtype == out.dtype and gate_up.is_contiguous() and out.is_contiguous()
    _call("jllm_swiglu", gate_up.data_ptr(), out.data_ptr(), _DT[out.dtype], out.shape[0], out.shape[1], _stream())


def qk_norm_rope_store(qkv, q_gain, k_gain, eps, cos, sin, rotary_dim, positions, slots, k_cache, v_cache,
                       heads, kv_heads, head_dim, page_size, write_kv=True) -> None:
    """In place on the queries of qkv [rows, stride]; keys and values go to the cache rows `slots`."""
    use_norm = q_gain is not None
    _call("jllm_qk_norm_rope_store", qkv.data_ptr(), _DT[qkv.dtype], _p(q_gain), _p(k_gain),
          _DT[q_gain.dtype] if use_norm else F32, int(use_norm), float(eps), _p(cos), _p(sin), int(rotary_dim),
          positions.data_ptr(), _p(slots), _p(k_cache), _p(v_cache), int(write_kv), qkv.shape[0], qkv.stride(0),
          heads, kv_heads, head_dim, page_size, _stream())


def gemm_plain(a, w, out, bias=None, accumulate=False) -> None:
    """out (+)= a @ w.T (+ bias) on the CUDA cores with float32 accumulation in ascending k."""
    assert a.dtype == w.dtype and a.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    _call("jllm_gemm_plain", a.data_ptr(), _DT[a.dtype], a.stride(0), w.data_ptr(), w.stride(0), _p(bias),
          _DT[bias.dtype] if bias is not None else F32, out.data_ptr(), _DT[out.dtype], out.stride(0),
          int(accumulate), a.shape[0], w.shape[0], a.shape[1], _stream())


def attention_plain(q, q_stride, k_cache, v_cache, out, row_seg, row_pos, block_tables, rows, heads, kv_heads,
                    head_dim, page_size, window, scale) -> None:
    _call("jllm_attention_plain", q.data_ptr(), q_stride, k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
          out.stride(0), row_seg.data_ptr(), row_pos.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
          rows, heads, kv_heads, head_dim, page_size, int(window), float(scale), _DT[q.dtype], _stream())


def argmax(logits: torch.Tensor, out: torch.Tensor, vocab: int | None = None) -> None:
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    _call("jllm_argmax", logits.data_ptr(), logits.stride(0), logits.shape[0], vocab or logits.shape[1],
          out.data_ptr(), _stream())


def sample(logits, temperature, top_k, top_p, min_p, uniform, out, vocab: int | None = None) -> None:
    assert logits.dtype == torch.float32 and uniform.dtype == torch.float64 and out.dtype == torch.int32
    _call("jllm_sample", logits.data_ptr(), logits.stride(0), logits.shape[0], vocab or logits.shape[1],
          temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(),
          out.data_ptr(), _stream())


def _packed(w) -> "PackedWeight":
    """The weight in the packed layout: as given, or packed now (tests and one-off calls hand in plain matrices; a
    model packs its weights once at load)."""
    return w if isinstance(w, PackedWeight) else pack_weight(w)


def _rows_fit(a, w) -> bool:
    """Whether the weight-row kernel (`gemm_small_m`) takes this product."""
    M, K = a.shape
    return (1 <= M <= 64 and K >= 8 and K % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
            and a.data_ptr() % 16 == 0)


def _tcgen05_fits(a, w) -> bool:
    M, K = a.shape
    return M >= 1 and K >= 8 and K % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1 and a.data_ptr() % 16 == 0


def gemm_bf16_fits(a, w, out) -> bool:
    """Whether the tensor-core kernels take this product; otherwise the CUDA-core kernel runs it."""
    return a.dtype == torch.bfloat16 and (isinstance(w, PackedWeight) or w.dtype == torch.bfloat16) and _tcgen05_fits(a, w)


# Which kernel takes a bfloat16 product of M rows (measured on the layer shapes of an 8B model; the figures are in the
# design notes):
#   "rows"   gemm_small_m: weight rows as the M side of mma.sync, tokens register-blocked; the fastest up to 16 rows
#            and for small matrices up to 64 rows;
#   "swap"   gemm_stream: tcgen05 with the weight rows as the M side, one 16 KB bulk copy per tile, the k blocks dealt
#            out evenly over the SMs; from 17 to 128 rows for matrices of 40 MB or more (QKV, down), from 41 rows for
#            smaller ones (O), where the row kernel's time grows with the rows; up to 160 rows for all of these and up to
#            256 for matrices much longer than high (down); not for very wide matrices (gate_up), which whole tiles of
#            the tiles kernel fill the SMs with;
#   "tiles"  gemm_tcgen05: tokens as the M side, 128 x BN tiles; above that, and from 16 rows for very wide matrices.
SWAP_MAX_ROWS = 256      # gemm_stream: the tokens are the N side of one tcgen05.mma
TILE_ROWS = 128          # rows of a tcgen05 product tile (BM in gemm_tcgen05.cu): a step of 129 rows pays for 256
SMALL_M_ROWS = int(os.environ.get("JLLM_B200_SMALL_M_ROWS", "64"))
WIDE_ROWS = int(os.environ.get("JLLM_B200_WIDE_ROWS", "16384"))
SWAP_MIN_BYTES = int(os.environ.get("JLLM_B200_SWAP_MIN_BYTES", str(40_000_000)))
_workspaces = {}
# counters of up to 65,536 tiles, then one parked 128 x 256 partial tile for each of up to 160 blocks
STREAM_WORKSPACE_FLOATS = 65536 + 160 * 128 * 256
SWAP_WORKSPACE_FLOATS = 2 * 65536 + 160 * 2 * 256 * 128       # gemm_stream: two counters per tile, then the parts
PAIR_WORKSPACE_FLOATS = 2 * 65536 + 160 * 128 * 256           # gemm_pair: two counters per tile, a part per block


def gemm_workspace(key, floats: int = 8 << 20) -> torch.Tensor:
    """Zero-initialised workspace of a streamed product (tile counters, then parked partial tiles), one per `key` (a
    device, or (device, kernel) for a kernel that keeps its own), grown when a product needs more; earlier ones stay
    alive because captured graphs may point at them."""
    held = _workspaces.setdefault(key, [])
    if not held or held[-1].numel() < floats:
        device = key[0] if isinstance(key, tuple) else key
        held.append(torch.zeros(max(floats, 8 << 20), dtype=torch.float32, device=device))
    return held[-1]


def gemm_kernel_for(rows: int, out_features: int, in_features: int = 4096, rows_fit: bool = True,
                    tiles_fit: bool = True, sms: int = 148, pairs: int = 74) -> str:
    """"rows", "swap", "tiles", "pair", "pair-streamed" or "" for a bfloat16 product of `rows` rows against a [out_features, in_features]
    weight, given which kernels take its strides and alignment, the SMs and the pairs of them the device runs at a time."""
    # 16 or more rows against a wide matrix (gate_up): 128 or more 192-wide tcgen05 tiles stream it faster than the
    # weight-row kernel, whose blocks have half their loads in flight once they hold more than two token tiles
    wide = rows >= 16 and out_features >= WIDE_ROWS and tiles_fit
    if tiles_fit and not wide and 16 < rows <= 128 and (out_features * in_features * 2 >= SWAP_MIN_BYTES or rows > 40):
        return "swap"
    # 129 to 256 rows (the tokens are still one tcgen05 N side): the parked parts grow with the rows, so it keeps only
    # what the tiles kernel is worst at, matrices much longer than high (down: 12,288 k for 4,096 rows; 31 to 41 us
    # against 58), and everything up to 160 rows (QKV 20 to 22 us against 23, O 19 to 20 against 22)
    if tiles_fit and not wide and 128 < rows <= SWAP_MAX_ROWS and (rows <= 160 or in_features >= 2 * out_features):
        return "swap"
    if rows <= min(SMALL_M_ROWS, 64) and rows_fit and not wide:
        return "rows"
    if not tiles_fit:
        return ""
    # 257 to 512 rows against a matrix much longer than high (down): its few 256 x 256 tiles cut up over ALL pairs, the
    # parts of a tile meeting in a workspace (8B shape, 384 rows: 49 us against 59 on one-SM tiles; 512 rows: 52 against
    # 67; the shorter matrices lose that way, and above 512 rows the whole tiles are enough)
    if pairs > 0 and tiles_fit and 256 < rows <= 512 and in_features >= 2 * out_features:
        return "pair-streamed"
    # Many rows: two SMs to a 256 x 256 tile take in a third less per multiply-add than one SM with a 128 x 256 tile,
    # which is what bounds these products. It pays where its tiles keep three quarters of the pairs busy or more and its
    # rounds of tiles, each about a tenth shorter than a round of one-SM tiles of the same width, take less than the
    # one-SM kernel's rounds at the tile width that kernel would choose (rounds x (rows + width) of a tile, as it does).
    col_tiles = -(-out_features // 256)
    pair_tiles = -(-rows // 256) * col_tiles
    if pairs > 0 and pair_tiles * 4 >= pairs * 3:
        row_tiles, tile_rows = -(-rows // 128), min(rows, 128)
        single = min(-(-(row_tiles * -(-out_features // w)) // sms) * (tile_rows + w) for w in (256, 192, 128, 64, 32))
        if -(-pair_tiles // pairs) * 0.9 * (128 + 256) <= single:
            return "pair"
    return "tiles"


def gemm_bf16(a, w, out, bias=None, accumulate=False, swiglu=False) -> None:
    """out (+)= a @ w.T (+ bias) on the tensor cores: bfloat16 operands, float32 accumulation; `w` a PackedWeight (a
    plain [out, in] matrix is packed on the spot). With `swiglu` the rows of w are blocks of 8 gate rows followed by
    their 8 up rows and out[m, j] = silu(gate_j) * up_j."""
    w = _packed(w)
    rows = a.shape[0]
    kernel = gemm_kernel_for(rows, w.rows, w.cols, _rows_fit(a, w), _tcgen05_fits(a, w), sm_count(),
                             resident_pairs() if rows > 128 else 0)
    if kernel == "rows":
        return gemm_small_m(a, w, out, bias, accumulate, swiglu=swiglu)
    if kernel == "swap":
        return gemm_stream(a, w, out, bias, accumulate, swiglu=swiglu)
    if kernel == "pair":
        return gemm_pair(a, w, out, bias, accumulate, swiglu=swiglu)
    if kernel == "pair-streamed":
        return gemm_pair(a, w, out, bias, accumulate, swiglu=swiglu, stream_mode=1)
    if kernel == "tiles":
        return gemm_tcgen05(a, w, out, bias, accumulate, swiglu=swiglu)
    raise KernelError("the tensor-core matrix product is not built for this shape")


def gemm_tcgen05(a, w, out, bias=None, accumulate=False, max_blocks: int = 0, swiglu=False, stream_mode: int = 0,
                 tile_width: int = 0) -> None:
    """The prefill product: tcgen05.mma tiles of 128 x `tile_width` (0: chosen from the shape, 256 for big products,
    down to 32 when the rows are few) with the accumulator in tensor memory; the activations' tiles come by TMA, the
    packed weight's by contiguous bulk copies. `stream_mode` 1: the tiles of a last, partly filled round are
    streamed (stream-K: equal runs of (tile, k block) pairs per block, walked before the block's whole tiles; partial
    tiles meet in a workspace); not the default (it gains little where the SMs share one memory system and one power
    limit)."""
    w = _packed(w)
    assert a.dtype == torch.bfloat16 and out.stride(-1) == 1 and a.shape[1] == w.cols
    ws = gemm_workspace(a.device, STREAM_WORKSPACE_FLOATS) if stream_mode == 1 else None
    _call("jllm_gemm_tcgen05", a.data_ptr(), a.stride(0), w.data.data_ptr(), w.k_blocks, _p(bias),
          _DT[bias.dtype] if bias is not None else F32, out.data_ptr(), _DT[out.dtype], out.stride(0),
          int(accumulate), a.shape[0], w.rows, w.cols, int(max_blocks), int(swiglu), _p(ws),
          ws.numel() if ws is not None else 0, int(stream_mode), int(tile_width), _stream())


def gemm_pair(a, w, out, bias=None, accumulate=False, swiglu=False, max_pairs: int = 0, stream_mode: int = 0) -> None:
    """The product of a prefill with many rows: two SMs to a 256 x 256 tile (tcgen05 cta_group::2), each bringing half of
    the tile's rows of A and of W; epilogues as `gemm_tcgen05`. `stream_mode` 1: the tiles of a last, partly filled
    round are cut up over all pairs (stream-K: equal runs of (tile, k block) pairs, walked before the whole tiles; partial
    tiles meet in a workspace); not the default (the busy pairs win back what the idle ones of a last round lose)."""
    w = _packed(w)
    assert a.dtype == torch.bfloat16 and out.stride(-1) == 1 and a.shape[1] == w.cols
    ws = gemm_workspace((a.device, "pair"), PAIR_WORKSPACE_FLOATS) if stream_mode == 1 else None
    _call("jllm_gemm_pair", a.data_ptr(), a.stride(0), w.data.data_ptr(), w.k_blocks, _p(bias),
          _DT[bias.dtype] if bias is not None else F32, out.data_ptr(), _DT[out.dtype], out.stride(0),
          int(accumulate), a.shape[0], w.rows, w.cols, int(max_pairs), int(swiglu), _p(ws),
          ws.numel() if ws is not None else 0, int(stream_mode), _stream())


_resident_pairs = None


def resident_pairs() -> int:
    """How many clusters of two blocks of the paired product the device runs at a time (0: it is not offered)."""
    global _resident_pairs
    if _resident_pairs is None:
        _resident_pairs = max(0, int(library().jllm_gemm_pair_resident()))
    return _resident_pairs


class PackedWeight:
    """A [rows, cols] bfloat16 weight in the layout the tensor cores stream: tiles of 128 rows x 64 k, each tile the
    16 KB image of its 128-byte-swizzled shared-memory form (row r of a tile is 128 bytes; its 16-byte chunk c lies at
    chunk position c ^ (r & 7)), tile (t, kb) at (t * k_blocks + kb) * 16 KB. Rows are padded to a multiple of 128 and
    k to a multiple of 64 with zeros. One tile is one contiguous bulk copy."""

    def __init__(self, data: torch.Tensor, rows: int, cols: int):
        self.data, self.rows, self.cols = data, rows, cols
        self.tiles, self.k_blocks = data.shape[0], data.shape[1]

    @property
    def shape(self):
        return (self.rows, self.cols)

    def unpack(self) -> torch.Tensor:
        """The [rows, cols] matrix again (tests)."""
        T, KB = self.tiles, self.k_blocks
        idx = _swizzle_index(self.data.device).expand(T, KB, 128, 8, 8)
        plain = self.data.view(T, KB, 128, 8, 8).gather(3, idx).permute(0, 2, 1, 3, 4).reshape(T * 128, KB * 64)
        return plain[:self.rows, :self.cols].contiguous()


_swizzle = {}


def _swizzle_index(device) -> torch.Tensor:
    idx = _swizzle.get(device)
    if idx is None:
        r, c = torch.arange(128, device=device), torch.arange(8, device=device)
        idx = (c[None, :] ^ (r[:, None] & 7))[None, None, :, :, None]          # [1, 1, 128, 8, 1]
        _swizzle[device] = idx
    return idx


def pack_weight(w: torch.Tensor) -> PackedWeight:
    """Packs a [rows, cols] bfloat16 weight for `gemm_stream` (done once, at load)."""
    assert w.dim() == 2 and w.dtype == torch.bfloat16
    N, K = w.shape
    T, KB = -(-N // 128), -(-K // 64)
    if T * 128 != N or KB * 64 != K:
        padded = torch.zeros((T * 128, KB * 64), dtype=w.dtype, device=w.device)
        padded[:N, :K] = w
    else:
        padded = w
    tiles = padded.view(T, 128, KB, 8, 8).permute(0, 2, 1, 3, 4)                   # [T, KB, 128 rows, 8 chunks, 8]
    data = tiles.gather(3, _swizzle_index(w.device).expand(T, KB, 128, 8, 8)).contiguous().view(T, KB, 128, 64)
    return PackedWeight(data, N, K)


def gemm_stream_fits(a, packed: PackedWeight) -> bool:
    M, K = a.shape
    return (1 <= M <= SWAP_MAX_ROWS and K == packed.cols and K >= 8 and K % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
            and a.data_ptr() % 16 == 0)


def gemm_stream(a, packed: PackedWeight, out, bias=None, accumulate=False, swiglu=False, max_blocks: int = 0) -> None:
    """out (+)= a @ W^T (+ bias) for at most 256 rows: the packed weight streamed once through tcgen05.mma with the
    weight rows as the M side (see gemm_stream.cu). With `swiglu` the rows of W are blocks of 8 gate rows followed by
    their 8 up rows and out[m, j] = silu(gate_j) * up_j. A tile's parts (its k blocks may fall to several blocks) are
    added in k order: two runs give the same bits."""
    packed = _packed(packed)
    assert a.dtype == torch.bfloat16 and out.stride(-1) == 1 and a.shape[1] == packed.cols
    ws = gemm_workspace((a.device, "stream"), SWAP_WORKSPACE_FLOATS)     # its own: it keeps counters of its own there
    _call("jllm_gemm_stream", a.data_ptr(), a.stride(0), packed.data.data_ptr(), packed.k_blocks, _p(bias),
          _DT[bias.dtype] if bias is not None else F32, out.data_ptr(), _DT[out.dtype], out.stride(0), int(accumulate),
          a.shape[0], packed.rows, packed.cols, int(swiglu), ws.data_ptr(), ws.numel(), int(max_blocks), _stream())


BOUNDS_FILES = ("attention_plain", "attention_decode", "attention_prefill", "attention_prefill_tc",
                "attention_prefill_pair", "rowwise")
BOUNDS_WHAT = {1: "a block-table index", 2: "a page id", 3: "a cache slot", 4: "a token id", 5: "a row"}


def checks_bounds() -> bool:
    """Whether the loaded library is the one built with bounds checks (JLLM_B200_CHECK_BOUNDS=1)."""
    return bool(library().jllm_checks_bounds())


def set_pool_pages(pages: int) -> None:
    """Tells the library how many pages the cache pool has that the next launches read and write. Only the library
    with bounds checks uses it (page ids and cache slots are compared with it)."""
    library().jllm_set_pool_pages(int(pages))


def bounds_errors() -> dict:
    """{file: (what, index, limit, how many)} for every file of kernels whose checks caught something since the last
    call (only the library built with bounds checks ever reports any). Synchronises."""
    out = {}
    lib = library()
    word = (c_int * 4)()
    for name in BOUNDS_FILES:
        code = getattr(lib, "jllm_bounds_error_" + name)(word)
        if code:
            raise KernelError(f"reading the bounds word of {name} failed ({code})")
        if word[3]:
            out[name] = (BOUNDS_WHAT.get(word[0], str(word[0])), word[1], word[2], word[3])
    return out


def check_kernel_errors() -> None:
    """Raises if a tcgen05 kernel gave up on one of its bounded waits since the last check (its results are then
    not to be trusted), or, in the build with bounds checks, if a kernel was handed a table index, page id, cache
    slot or token id outside its array (the access was skipped). Reads a few words from the device, so it
    synchronises."""
    lib = library()
    raised = {name: code for name, code in (("gemm_tcgen05", lib.jllm_gemm_tcgen05_error()),
                                            ("attention_prefill_tc", lib.jllm_attention_prefill_tc_error())) if code}
    if raised:
        raise KernelError("a bounded wait ran out inside " + ", ".join(f"{k} (code {v})" for k, v in raised.items()))
    if checks_bounds():
        caught = bounds_errors()
        if caught:
            raise KernelError("out of bounds (the accesses were skipped): " + "; ".join(
                f"{name}: {what} {index} with limit {limit}, {n} in all" for name, (what, index, limit, n) in caught.items()))


def gemm_plain_stores(on: bool) -> None:
    """A test's switch: the tcgen05 products store float32 outputs (and add into them) with the epilogue warps' own loads
    and stores, as where the output's rows allow no tensor map, instead of by tiled bulk copies."""
    library().jllm_gemm_plain_stores(int(bool(on)))


def attention_decode_separate_combine(on: bool) -> None:
    """A test's switch: the partial results of split or dealt-out decode attention are added up by a combine kernel of
    their own (as where the library's pair counters do not reach) instead of by the last block of every pair."""
    library().jllm_attention_decode_separate_combine(int(bool(on)))


def gemm_tcgen05_starve_next() -> None:
    """A test of the bounded waits: the next tcgen05 product (one tile) is given a barrier that never completes and
    waits that give up after 1,024 tries; it returns and raises the error word that `check_kernel_errors` reads."""
    library().jllm_gemm_tcgen05_starve_next()


def gemm_tcgen05_error() -> int:
    """0, or the code a tcgen05 kernel raised because one of its bounded waits ran out (synchronises)."""
    return library().jllm_gemm_tcgen05_error()


def gemm_small_m(a, w, out, bias=None, accumulate=False, swiglu=False) -> None:
    """The decode-step product (at most 64 rows): the packed weight's rows as the M side of mma.sync, tokens as N."""
    w = _packed(w)
    assert a.dtype == torch.bfloat16 and out.stride(-1) == 1 and a.shape[1] == w.cols
    _call("jllm_gemm_small_m", a.data_ptr(), a.stride(0), w.data.data_ptr(), w.k_blocks, _p(bias),
          _DT[bias.dtype] if bias is not None else F32, out.data_ptr(), _DT[out.dtype], out.stride(0),
          int(accumulate), a.shape[0], w.rows, w.cols, int(swiglu), _stream())


def attention_decode_fits(dtype, heads, kv_heads, head_dim) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and heads // kv_heads <= 16


def attention_decode_scratch_floats(rows, heads, head_dim, splits) -> int:
    return 0 if splits <= 1 else rows * heads * splits * (head_dim + 2)


def attention_decode(q, k_cache, v_cache, out, row_seg, row_pos, block_tables, rows, heads, kv_heads, head_dim,
                     page_size, window, scale, splits=1, scratch=None) -> None:
    """One query position per row; the key range of a row may be split over `splits` blocks (needs scratch)."""
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32 and \
            scratch.numel() >= attention_decode_scratch_floats(rows, heads, head_dim, splits)
    global launch_count
    launch_count += _combine_launches("split", splits, rows, kv_heads, head_dim)
    _call("jllm_attention_decode", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
          out.stride(0), row_seg.data_ptr(), row_pos.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
          rows, heads, kv_heads, head_dim, page_size, int(window), float(scale), int(splits), _p(scratch), _stream())


def attention_decode_flat_scratch_floats(rows, heads, kv_heads, head_dim, blocks) -> int:
    return (rows * kv_heads + blocks) * (heads // kv_heads) * (head_dim + 2)


def attention_decode_flat(q, k_cache, v_cache, out, row_seg, row_pos, block_tables, rows, heads, kv_heads, head_dim,
                          page_size, window, scale, blocks, scratch) -> None:
    """One query position per row, the key tiles of all (row, kv head) pairs dealt out evenly over `blocks` blocks."""
    assert scratch.dtype == torch.float32 and \
        scratch.numel() >= attention_decode_flat_scratch_floats(rows, heads, kv_heads, head_dim, blocks)
    global launch_count
    launch_count += _combine_launches("flat", blocks, rows, kv_heads, head_dim)
    _call("jllm_attention_decode_flat", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
          out.stride(0), row_seg.data_ptr(), row_pos.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
          rows, heads, kv_heads, head_dim, page_size, int(window), float(scale), int(blocks), scratch.data_ptr(), _stream())


FLAT_DECODE = int(os.environ.get("JLLM_B200_FLAT_DECODE", "1"))


def decode_plan(rows, kv_heads, kv_bucket, heads, head_dim, scratch, places: int = 0):
    """("flat", blocks) or ("split", splits) for a decode step's attention: one block per (row, kv head, split), or,
    when there are more (row, kv head) pairs than places for blocks (`places`, by default two per SM of the device)
    and they would fill the last round of places
    badly (by less than 93 %), the key tiles of all pairs dealt out evenly over as many blocks as there are places
    (with fewer pairs than places the even deal is the slower one). `kv_bucket` = the longest request's keys in
    units of 256."""
    places = places or resident_blocks()
    splits = decode_splits(rows, kv_heads, kv_bucket, heads, head_dim, scratch, places)
    uniform = rows * kv_heads * splits
    rounds = -(-uniform // places)
    if (not FLAT_DECODE or scratch is None or head_dim not in (64, 128, 256) or rows > 1024
            or rows * kv_heads <= places or uniform * 100 >= rounds * places * 93):
        return "split", splits
    tiles = rows * kv_heads * kv_bucket * 4                    # 64 keys a tile; an upper bound, like the bucket
    blocks = max(1, min(places, 62 * kv_heads, tiles // 2))
    if attention_decode_flat_scratch_floats(rows, heads, kv_heads, head_dim, blocks) > scratch.numel():
        return "split", splits
    return "flat", blocks


KV_BUCKET_MAX = 32
# the buckets a decode step is planned for: a step's bucket is rounded down to one of them, so that a context that grows
# asks for a new plan (and a newly captured step) sixteen times in its life and not every 256 tokens
KV_BUCKET_LEVELS = (1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16, 20, 24, 28, 32)


def bucket_level(kv_bucket: int) -> int:
    """`kv_bucket` rounded down to the nearest of KV_BUCKET_LEVELS (a plan for fewer keys is always a valid one)."""
    return max(l for l in KV_BUCKET_LEVELS if l <= max(1, kv_bucket))


def _windowed_bucket(kv_bucket: int, window: int) -> int:
    return kv_bucket if window <= 0 else max(1, min(kv_bucket, window // 256))


def decode_bucket_cap(rows, kv_heads, heads, head_dim, window, scratch, places: int = 0) -> int:
    """The smallest bucket from which on `decode_plan` says the same for every larger one: with so many keys the split is
    bounded by the places for blocks, not by the keys, and a step's launches no longer change as its context grows."""
    def plan(b):
        return decode_plan(rows, kv_heads, _windowed_bucket(b, window), heads, head_dim, scratch, places)
    cap, top = KV_BUCKET_MAX, plan(KV_BUCKET_MAX)
    while cap > 1 and plan(cap - 1) == top:
        cap -= 1
    return cap


def _attention_decode_rows(q, k_cache, v_cache, out, row_seg, positions, table, rows, heads, kv_heads, head_dim, page_size,
                           window, scale, kv_bucket, scratch):
    bucket = _windowed_bucket(kv_bucket, window)
    how, n = decode_plan(rows, kv_heads, bucket, heads, head_dim, scratch)
    if how == "flat":
        return attention_decode_flat(q, k_cache, v_cache, out, row_seg, positions, table, rows, heads, kv_heads, head_dim,
                                     page_size, window, scale, n, scratch)
    return attention_decode(q, k_cache, v_cache, out, row_seg, positions, table, rows, heads, kv_heads, head_dim, page_size,
                            window, scale, n, scratch)


def attention_decode_fresh_fits(dtype, heads, kv_heads, head_dim, rotary_dim) -> bool:
    """Whether the decode attention can finish its own rows (norm, rotation, cache write) instead of a kernel in front."""
    return (FRESH_DECODE and dtype == torch.bfloat16 and head_dim in (64, 128, 256) and rotary_dim == head_dim
            and heads % kv_heads == 0 and heads // kv_heads <= 16)


FRESH_DECODE = int(os.environ.get("JLLM_B200_FRESH_DECODE", "1"))      # 0: never; 2: also where the key tiles are dealt out


def attention_decode_fresh(qkv, q_gain, k_gain, eps, cos, sin, k_cache, v_cache, out, row_seg, positions, table, rows,
                           heads, kv_heads, head_dim, page_size, window, scale, kv_bucket, scratch) -> bool:
    """Decode attention over rows whose queries, key and value lie in `qkv` as the QKV product left them: the kernel norms
    and rotates them itself and writes the key and value of every row's newest position to the cache (what
    `qk_norm_rope_store` does in a launch of its own). Taken, and True returned, where `decode_plan` gives every (row, kv
    head) pair blocks of its own: a step of 8 rows 4.17 ms against 4.24, of one row 3.38 against 3.43; where the key tiles
    are dealt out over the blocks (64 rows: 10.46 against 10.44 ms) nothing is launched and the caller takes the two
    kernels."""
    bucket = _windowed_bucket(kv_bucket, window)
    how, n = decode_plan(rows, kv_heads, bucket, heads, head_dim, scratch)
    if how == "flat" and FRESH_DECODE != 2:
        return False
    use_norm = q_gain is not None
    global launch_count
    launch_count += _combine_launches(how, n, rows, kv_heads, head_dim)
    _call("jllm_attention_decode_fresh", qkv.data_ptr(), qkv.stride(0), _p(q_gain), _p(k_gain),
          _DT[q_gain.dtype] if use_norm else F32, int(use_norm), float(eps), cos.data_ptr(), sin.data_ptr(),
          k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), out.stride(0), row_seg.data_ptr(), positions.data_ptr(),
          table.data_ptr(), table.stride(0), rows, heads, kv_heads, head_dim, page_size, int(window), float(scale),
          int(how == "flat"), int(n), _p(scratch), _stream())
    return True


PAIR_COUNTERS = 1 << 16      # the library's counters of (row, kv head) pairs: within them no combine kernel follows


def _combine_launches(how, n, rows, kv_heads, head_dim) -> int:
    """Kernels that a decode attention launches besides the attention itself (the count `bench.py` reports)."""
    within = rows * kv_heads <= PAIR_COUNTERS and head_dim in (64, 128, 256)
    if how == "flat":
        return 0 if within and rows * kv_heads >= n else 1
    return 0 if n == 1 or (within and n <= 8) else 1


def attention(q, k_cache, v_cache, out, batch, group, heads, kv_heads, head_dim, page_size, window, scale,
              scratch=None) -> None:
    """Causal attention of every row of the batch over its own request's cached keys and values."""
    if batch.decode_only and attention_decode_fits(q.dtype, heads, kv_heads, head_dim):
        return _attention_decode_rows(q, k_cache, v_cache, out, batch.row_seg, batch.positions, batch.block_tables[group],
                                      batch.rows, heads, kv_heads, head_dim, page_size, window, scale, batch.kv_bucket,
                                      scratch)
    if q.dtype == torch.bfloat16 and attention_prefill_fits(head_dim):
        # prompt portions through the flash kernel; the single rows riding beside them (the scheduler puts them
        # last) through the decode kernel, which shares every key among the query heads of a kv head
        ms, mr = batch.multi_segments, batch.multi_rows
        if ms < 0 or mr == batch.rows or not attention_decode_fits(q.dtype, heads, kv_heads, head_dim):
            ms, mr = batch.seg_start.numel(), batch.rows
        if mr > 0:
            attention_prefill(q[:mr], k_cache, v_cache, out[:mr], batch.seg_start[:ms], batch.seg_len[:ms],
                              batch.seg_kv_len[:ms], batch.block_tables[group], mr, heads, kv_heads, head_dim, page_size,
                              window, scale)
        if mr < batch.rows:
            n = batch.rows - mr
            _attention_decode_rows(q[mr:], k_cache, v_cache, out[mr:], batch.row_seg[mr:], batch.positions[mr:],
                                   batch.block_tables[group], n, heads, kv_heads, head_dim, page_size, window, scale,
                                   batch.kv_bucket, scratch)
        return
    attention_plain(q, q.stride(0), k_cache, v_cache, out, batch.row_seg, batch.positions, batch.block_tables[group],
                    batch.rows, heads, kv_heads, head_dim, page_size, window, scale)


def attention_prefill_fits(head_dim) -> bool:
    return head_dim in (64, 128, 256)


PREFILL_TC = int(os.environ.get("JLLM_B200_PREFILL_TC", "1"))


def attention_prefill_tc_fits(q, out, k_cache, head_dim, page_size) -> bool:
    return (head_dim == 128 and 1 <= page_size <= 128 and page_size & (page_size - 1) == 0 and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and k_cache.is_contiguous())


def attention_prefill(q, k_cache, v_cache, out, seg_start, seg_len, seg_kv_len, block_tables, rows, heads, kv_heads,
                      head_dim, page_size, window, scale, kernel: str = "auto") -> None:
    """Flash attention of prompt portions: segments of consecutive rows, each over its own request's pages.
    Head size 128 runs on tcgen05 (both products, accumulators in tensor memory; kernel "pair" or "tc"), other
    sizes on mma.sync ("mma")."""
    if kernel == "auto" and PREFILL_TC and attention_prefill_tc_fits(q, out, k_cache, head_dim, page_size):
        # two query tiles per block where the portions are long enough to fill them (the tiles take turns on the
        # tensor cores); one tile per block, with two S buffers, for short portions
        kernel = "pair" if rows > 128 * seg_start.numel() and PREFILL_TC != 3 else "tc"
    if kernel in ("tc", "pair"):
        return _call("jllm_attention_prefill_tc" if kernel == "tc" else "jllm_attention_prefill_pair", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                     k_cache.shape[0], out.data_ptr(), out.stride(0), seg_start.data_ptr(), seg_len.data_ptr(),
                     seg_kv_len.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), seg_start.numel(), rows,
                     heads, kv_heads, head_dim, page_size, int(window), float(scale), _stream())
    _call("jllm_attention_prefill", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
          out.stride(0), seg_start.data_ptr(), seg_len.data_ptr(), seg_kv_len.data_ptr(), block_tables.data_ptr(),
          block_tables.stride(0), seg_start.numel(), rows, heads, kv_heads, head_dim, page_size, int(window),
          float(scale), _stream())


def attention_prefill_tc_error() -> int:
    """0, or the code the tcgen05 attention kernel raised because a bounded wait ran out (synchronises)."""
    return library().jllm_attention_prefill_tc_error()


def decode_splits(rows, kv_heads, kv_bucket, heads, head_dim, scratch, places: int = 0) -> int:
    """How many blocks share one row's keys: as many as fit on the GPU at once (two blocks per SM; one block
    more than that would cost a whole second wave), each with at least 128 keys (`kv_bucket` = the longest
    request's keys in units of 256)."""
    want = (places or resident_blocks()) // max(1, rows * kv_heads)
    splits = max(1, min(want, 2 * kv_bucket, 32))
    if scratch is None:
        return 1
    while splits > 1 and attention_decode_scratch_floats(rows, heads, head_dim, splits) > scratch.numel():
        splits -= 1
    return splits
