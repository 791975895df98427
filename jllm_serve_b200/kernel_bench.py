"""Times the hand-written kernels alone on the layer shapes of a model, against their rooflines.

    python -m jllm_serve_b200.kernel_bench [--rows 8] [--prompt 2048] [--context 4096] [--repeat 20] [--only NAME] [--eager]

Every kernel runs on random tensors of the shapes one layer of the Qwen3-8B configuration gives it
(hidden 4096, 32/8 heads of 128, intermediate 12288), timed with CUDA events over `--repeat` calls (replayed
as one CUDA graph unless `--eager`) that rotate through several copies of the weights, so every call streams
them from HBM. It prints, per kernel,
microseconds per call and the achieved GB/s (weight or cache bytes, the decode kernels) or TFLOP/s (the
prefill kernels). With `--repeat 1` it is the small workload that profilers are pointed at.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--rows", type=int, default=8, help="rows of a decode step")
    ap.add_argument("--prompt", type=int, default=2048, help="rows of a prefill step")
    ap.add_argument("--context", type=int, default=4096, help="cached positions per request in the decode attention")
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--only", default="", help="run only the kernels whose name contains this")
    ap.add_argument("--eager", action="store_true", help="launch from the host call by call instead of replaying a graph")
    ap.add_argument("--all-kernels", action="store_true",
                    help="the products of the prefill step also on every product kernel that takes their shape, not only "
                         "on the one the dispatch chooses")
    args = ap.parse_args()

    from .csrc import ops
    ops.require_device()
    dev = torch.device("cuda:0")
    D, H, Hkv, hd, F, page = 4096, 32, 8, 128, 12288, 16
    M, T, ctx = args.rows, args.prompt, args.context
    bf = torch.bfloat16

    def weights(n, k):
        copies = max(2, int(300e6 // (n * k * 2)) + 1) if args.repeat > 1 else 1
        return [ops.pack_weight((torch.randn(n, k, device=dev) * 0.02).to(bf)) for _ in range(copies)]

    def interleaved(n_hidden, k):
        return weights(2 * n_hidden, k)      # the SwiGLU epilogue only needs the row count to be a multiple of 16

    cases = []

    def case(name, fn, copies, bytes_=0, flops=0):
        if args.only in name:
            cases.append((name, fn, copies, bytes_, flops))

    # ---- decode: M rows ----
    a_d, a_f = torch.randn(M, D, device=dev).to(bf), torch.randn(M, F, device=dev).to(bf)
    x = torch.randn(M, D, device=dev)
    qkv_d, h_d = torch.empty(M, (H + 2 * Hkv) * hd, device=dev, dtype=bf), torch.empty(M, F, device=dev, dtype=bf)
    w_qkv, w_o, w_gu, w_down = weights((H + 2 * Hkv) * hd, D), weights(D, H * hd), interleaved(F, D), weights(D, F)
    case("decode gemm qkv", lambda i: ops.gemm_bf16(a_d, w_qkv[i], qkv_d), len(w_qkv), w_qkv[0].rows * w_qkv[0].cols * 2)
    case("decode gemm o (+= residual)", lambda i: ops.gemm_bf16(a_d, w_o[i], x, None, True), len(w_o), w_o[0].rows * w_o[0].cols * 2)
    case("decode gemm gate_up + swiglu", lambda i: ops.gemm_bf16(a_d, w_gu[i], h_d, swiglu=True), len(w_gu),
         w_gu[0].rows * w_gu[0].cols * 2)
    case("decode gemm down (+= residual)", lambda i: ops.gemm_bf16(a_f, w_down[i], x, None, True), len(w_down),
         w_down[0].rows * w_down[0].cols * 2)
    pages = M * (ctx // page + 1)
    n_caches = max(2, int(300e6 // (pages * Hkv * page * hd * 4)) + 1) if args.repeat > 1 else 1
    caches = [(torch.randn(pages, Hkv, page, hd, device=dev).to(bf), torch.randn(pages, Hkv, page, hd, device=dev).to(bf))
              for _ in range(n_caches)]
    tables = torch.arange(pages, dtype=torch.int32, device=dev).reshape(M, -1).contiguous()
    q = torch.randn(M, H * hd, device=dev).to(bf)
    out = torch.empty_like(q)
    seg = torch.arange(M, dtype=torch.int32, device=dev)
    pos = torch.full((M,), ctx - 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 << 20, device=dev)
    how, n = ops.decode_plan(M, Hkv, max(1, min(32, ctx // 256, -(-ops.resident_blocks() // M))), H, hd, scratch)
    if how == "flat":
        case(f"decode attention (dealt out over {n} blocks)",
             lambda i: ops.attention_decode_flat(q, caches[i][0], caches[i][1], out, seg, pos, tables, M, H, Hkv, hd, page, 0,
                                                 1 / math.sqrt(hd), n, scratch), n_caches, M * ctx * Hkv * hd * 4)
    else:
        case(f"decode attention ({n} splits)",
             lambda i: ops.attention_decode(q, caches[i][0], caches[i][1], out, seg, pos, tables, M, H, Hkv, hd, page, 0,
                                            1 / math.sqrt(hd), n, scratch), n_caches, M * ctx * Hkv * hd * 4)
    if how != "flat":
        # the same with the rows' own norm, rotation and cache write done by the attention (what a decode step takes)
        ang_d = torch.outer(torch.arange(ctx + 1, dtype=torch.float64),
                            1e6 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))
        cos_d, sin_d = ang_d.cos().float().to(dev), ang_d.sin().float().to(dev)
        gains = torch.ones(hd, device=dev, dtype=bf)
        qkv_raw = torch.randn(M, (H + 2 * Hkv) * hd, device=dev).to(bf)
        case(f"decode attention, finishing its own rows ({n} splits)",
             lambda i: ops.attention_decode_fresh(qkv_raw, gains, gains, 1e-6, cos_d, sin_d, caches[i][0], caches[i][1], out, seg,
                                                  pos, tables, M, H, Hkv, hd, page, 0, 1 / math.sqrt(hd), max(1, ctx // 256),
                                                  scratch), n_caches, M * ctx * Hkv * hd * 4)
    ctx_pad = max(ctx, T) + page
    ang = torch.outer(torch.arange(ctx_pad, dtype=torch.float64), 1e6 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))
    cos_t, sin_t = ang.cos().float().to(dev), ang.sin().float().to(dev)
    hg = torch.ones(hd, device=dev, dtype=bf)
    slots_d = (tables[:, -1].long() * page + (ctx - 1) % page).to(torch.int32)
    case("decode q/k norm + rope + cache write",
         lambda i: ops.qk_norm_rope_store(qkv_d, hg, hg, 1e-6, cos_t, sin_t, hd, pos, slots_d, caches[0][0], caches[0][1],
                                          H, Hkv, hd, page), 1, M * (H + 2 * Hkv) * hd * 4)
    gain = torch.ones(D, device=dev, dtype=bf)
    xb = torch.empty(M, D, device=dev, dtype=bf)
    case("decode rmsnorm", lambda i: ops.rmsnorm(x, gain, 1e-6, xb), 1, M * D * 6)

    # ---- prefill: T rows of one request ----
    a_p = torch.randn(T, D, device=dev).to(bf)
    h_p = torch.empty(T, F, device=dev, dtype=bf)
    qkv_p = torch.empty(T, (H + 2 * Hkv) * hd, device=dev, dtype=bf)
    x_p = torch.randn(T, D, device=dev)
    products = [("qkv", a_p, w_qkv, qkv_p, False, False, 2 * T * D * qkv_p.shape[1]),
                ("o (+= residual)", a_p, w_o, x_p, True, False, 2 * T * D * D),
                ("gate_up + swiglu", a_p, w_gu, h_p, False, True, 2 * T * D * 2 * F),
                ("down (+= residual)", h_p, w_down, x_p, True, False, 2 * T * D * F)]
    pairs = ops.resident_pairs() if T > 128 else 0
    for what, a_, ws_, out_, acc_, glu_, flops_ in products:
        chosen = ops.gemm_kernel_for(T, ws_[0].rows, ws_[0].cols, T <= 64, True, ops.sm_count(), pairs)
        case(f"prefill gemm {what} [{chosen}]",
             lambda i, a_=a_, ws_=ws_, out_=out_, acc_=acc_, glu_=glu_: ops.gemm_bf16(a_, ws_[i], out_, None, acc_, glu_),
             len(ws_), flops=flops_)
        if not args.all_kernels:
            continue
        # every product kernel that takes this shape, side by side on the same packed weights
        kernels = {"tiles": lambda i, a_=a_, ws_=ws_, out_=out_, acc_=acc_, glu_=glu_: ops.gemm_tcgen05(a_, ws_[i], out_, None, acc_, swiglu=glu_)}
        if pairs > 0:
            kernels["pair"] = lambda i, a_=a_, ws_=ws_, out_=out_, acc_=acc_, glu_=glu_: ops.gemm_pair(a_, ws_[i], out_, None, acc_, swiglu=glu_)
            kernels["pair-streamed"] = lambda i, a_=a_, ws_=ws_, out_=out_, acc_=acc_, glu_=glu_: ops.gemm_pair(a_, ws_[i], out_, None, acc_, swiglu=glu_, stream_mode=1)
        if T <= ops.SWAP_MAX_ROWS:
            kernels["swap"] = lambda i, a_=a_, ws_=ws_, out_=out_, acc_=acc_, glu_=glu_: ops.gemm_stream(a_, ws_[i], out_, None, acc_, swiglu=glu_)
        if T <= 64:
            kernels["rows"] = lambda i, a_=a_, ws_=ws_, out_=out_, acc_=acc_, glu_=glu_: ops.gemm_small_m(a_, ws_[i], out_, None, acc_, swiglu=glu_)
        for kernel, fn in kernels.items():
            if kernel != chosen:
                case(f"prefill gemm {what} on {kernel}", fn, len(ws_), flops=flops_)
    pp = T // page + 1
    kc, vc = torch.randn(pp, Hkv, page, hd, device=dev).to(bf), torch.randn(pp, Hkv, page, hd, device=dev).to(bf)
    tp = torch.arange(pp, dtype=torch.int32, device=dev).reshape(1, -1).contiguous()
    qp = torch.randn(T, H * hd, device=dev).to(bf)
    op = torch.empty_like(qp)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    s0, s1, s2 = i32([0]), i32([T]), i32([T])
    case("prefill attention (causal)",
         lambda i: ops.attention_prefill(qp, kc, vc, op, s0, s1, s2, tp, T, H, Hkv, hd, page, 0, 1 / math.sqrt(hd)), 1,
         flops=4 * (T * (T + 1) // 2) * H * hd)
    pos_p = torch.arange(T, dtype=torch.int32, device=dev)
    case("prefill q/k norm + rope + cache write",
         lambda i: ops.qk_norm_rope_store(qkv_p, hg, hg, 1e-6, cos_t, sin_t, hd, pos_p, pos_p, kc, vc, H, Hkv, hd, page), 1,
         T * (H + 2 * Hkv) * hd * 4)
    gp = torch.ones(D, device=dev, dtype=bf)
    xbp = torch.empty(T, D, device=dev, dtype=bf)
    case("prefill rmsnorm", lambda i: ops.rmsnorm(x_p, gp, 1e-6, xbp), 1, T * D * 6)

    for name, fn, copies, bytes_, flops in cases:
        for i in range(3 if args.repeat > 1 else 0):
            fn(i % copies)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.eager or args.repeat == 1:
            s.record()
            for i in range(args.repeat):
                fn(i % copies)
            e.record()
        else:
            # the calls as one CUDA graph: what is timed is the device, not the host's launches
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(args.repeat):
                    fn(i % copies)
            graph.replay()
            torch.cuda.synchronize()
            s.record()
            graph.replay()
            e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) / args.repeat * 1e3
        rate = f"{bytes_ / us / 1e3:8.0f} GB/s" if bytes_ else f"{flops / us / 1e6:8.0f} TFLOP/s"
        print(f"{name:36s} {us:9.1f} us {rate}", flush=True)
    ops.check_kernel_errors()
    return 0


if __name__ == "__main__":
    sys.exit(main())
