"""Kernel micro-benchmarks: ``python -m lm_engine.ops.microbench {gemm,attention,moe,elementwise} [options]``.

Every case is timed with CUDA events around single launches after warm-up, with a write larger than L2 between
launches, and reports the median. ``--profile`` runs each case exactly ``--iters`` times with no comparison library and
no flush kernel in between, which is the form to put under a profiler (small, few launches, ends by itself).
"""

from __future__ import annotations

import argparse
import json

import torch

from . import native, status_word

L2_FLUSH_BYTES = 256 * 1024 * 1024


def _time(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]


def _emit(record: dict) -> None:
    print(json.dumps(record), flush=True)


def bench_gemm(args) -> None:
    C, st = native(), status_word(torch.device("cuda"))
    flush = None if args.profile else torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device="cuda")
    shapes = [tuple(int(v) for v in s.split("x")) for s in args.shapes] if args.shapes else [
        (8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336), (8192, 8192, 8192), (4096, 128256, 4096)]
    trace = torch.zeros(8 * 148, dtype=torch.int64, device="cuda") if args.trace else None
    if args.swiglu_only or args.swiglu_bwd:
        shapes = []
    for M, N, K in shapes:
        flops = 2.0 * M * N * K
        for layout in args.layouts:
            a_mn, b_mn = layout[0] == "t", layout[1] == "n"
            a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
            b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
            out = torch.empty(M, N, device="cuda", dtype=torch.float32 if args.accumulate else torch.bfloat16)
            record = dict(op="gemm", layout=layout, m=M, n=N, k=K, accumulate=args.accumulate)
            if args.variant in ("all", "cta1"):
                ms = _time(lambda: C.gemm(a, b, out, a_mn, b_mn, args.accumulate, 1.0, st, 0, 1), args.iters, args.warmup, flush)
                record["cta1_ms"], record["cta1_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
            if args.variant in ("all", "cta_pair"):
                # knobs of the CTA-pair kernel: raster group (0 = built-in choice), k skew, register-store epilogue
                configs = [(group, skew, direct, split) for group in args.groups for skew in args.k_skew
                           for direct in ([False, True] if args.direct_store else [False]) for split in args.split_k]

                def key_of(group, skew, direct, split=0):
                    return ("cta_pair" + (f"_g{group}" if group else "") + (f"_s{skew}" if skew else "") + ("_direct" if direct else "")
                            + (f"_k{split}" if split else ""))

                def run_pair(group, skew, direct, split=0):
                    C.gemm_tuning(group, skew, direct, trace, split)
                    C.gemm(a, b, out, a_mn, b_mn, args.accumulate, 1.0, st, 0, 2)

                if args.interleave:
                    # all candidates (and the library) take turns launch by launch after a warm-up long enough to reach the
                    # power-capped clock, so that clock drift during the sweep hits every candidate alike
                    am, bm = (a.t() if a_mn else a), (b if b_mn else b.t())
                    out_lib = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
                    end = torch.cuda.Event(enable_timing=True)
                    begin = torch.cuda.Event(enable_timing=True)
                    begin.record()
                    while True:
                        for _ in range(20):
                            run_pair(0, 0, False)
                        end.record()
                        end.synchronize()
                        if begin.elapsed_time(end) > args.heat_ms:
                            break
                    samples: dict[str, list[float]] = {}
                    for _ in range(args.iters):
                        for cfg in configs + ["cublas"]:
                            flush.zero_() if flush is not None else None
                            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                            e0.record()
                            if cfg == "cublas":
                                torch.matmul(am, bm, out=out_lib)
                            else:
                                run_pair(*cfg)
                            e1.record()
                            e1.synchronize()
                            samples.setdefault(cfg if cfg == "cublas" else key_of(*cfg), []).append(e0.elapsed_time(e1))
                    for key, values in samples.items():
                        values.sort()
                        ms = values[len(values) // 2]
                        record[f"{key}_ms"], record[f"{key}_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
                    C.gemm_tuning(0, 0, False, None)
                    record["status"] = int(st.item())
                    _emit(record)
                    continue
                for group, skew, direct, split in configs:
                    ms = _time(lambda: run_pair(group, skew, direct, split), args.iters, args.warmup, flush)
                    key = key_of(group, skew, direct, split)
                    record[f"{key}_ms"], record[f"{key}_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
                    if trace is not None:
                        # cycle counters of the last launch, averaged over the leader CTAs: share of the MMA
                        # thread's time spent waiting for operands / for a free accumulator, and of the
                        # epilogue's time spent waiting for a finished accumulator / for its store boxes
                        t = trace.view(148, 8)[0::2].double()
                        total, epi_total = t[:, 3].clamp(min=1), t[:, 5].clamp(min=1)
                        record[f"{key}_trace"] = dict(
                            mma_wait_operands=round((t[:, 1] / total).mean().item(), 3),
                            mma_wait_accumulator=round((t[:, 2] / total).mean().item(), 3),
                            producer_wait_stage=round((t[:, 0] / total).mean().item(), 3),
                            epilogue_wait_accumulator=round((t[:, 4] / epi_total).mean().item(), 3),
                            epilogue_wait_store=round((t[:, 7] / epi_total).mean().item(), 3),
                            mma_cycles=int(total.mean().item()), tiles_per_pair=round(t[:, 6].mean().item(), 2))
                C.gemm_tuning(0, 0, False, None)
            if not args.profile:
                am, bm = (a.t() if a_mn else a), (b if b_mn else b.t())
                out_lib = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
                ms = _time(lambda: torch.matmul(am, bm, out=out_lib), args.iters, args.warmup, flush)
                record["cublas_ms"], record["cublas_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
            record["status"] = int(st.item())
            _emit(record)
    if args.swiglu or args.swiglu_only:
        # c_fc GEMM with the SwiGLU activation in its epilogue against GEMM followed by the stand-alone kernel
        T, H, I = args.tokens, args.hidden, args.intermediate
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.02
        fc = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        act = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * T * 2 * I * H

        def unfused():
            C.gemm(x, w, fc, False, False, False, 1.0, st, 0, 2)
            return C.swiglu_fwd(fc)

        ms_f = _time(lambda: C.gemm_swiglu(x, w, fc, act, st), args.iters, args.warmup, flush)
        ms_u = ms_f if args.swiglu_only else _time(unfused, args.iters, args.warmup, flush)
        _emit(dict(op="gemm_swiglu", tokens=T, hidden=H, intermediate=I, fused_ms=round(ms_f, 4), fused_tflops=round(flops / ms_f / 1e9, 1),
                   gemm_then_swiglu_ms=round(ms_u, 4), status=int(st.item())))
    if args.swiglu_bwd:
        # data gradient of the down-projection with the SwiGLU backward in its epilogue against GEMM + stand-alone kernel
        T, H, I = args.tokens, args.hidden, args.intermediate
        dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(H, I, device="cuda", dtype=torch.bfloat16) * 0.02
        fc = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        dfc = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        act = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
        dact = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * T * I * H

        def unfused():
            C.gemm(dy, w, dact, False, True, False, 1.0, st, 0, 2)
            return C.swiglu_bwd(dact, fc, True)

        record = dict(op="gemm_swiglu_bwd", tokens=T, hidden=H, intermediate=I)
        samples = {"fused": [], "gemm_then_swiglu_bwd": [], "gemm_alone": []}
        calls = {"fused": lambda: C.gemm_swiglu_bwd(dy, w, fc, dfc, act, st), "gemm_then_swiglu_bwd": unfused,
                 "gemm_alone": lambda: C.gemm(dy, w, dact, False, True, False, 1.0, st, 0, 2)}
        for _ in range(args.warmup):
            for fn in calls.values():
                fn()
        for _ in range(args.iters):  # the three take turns, so that clock drift under the power cap hits them alike
            for key, fn in calls.items():
                flush.zero_() if flush is not None else None
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                e1.synchronize()
                samples[key].append(e0.elapsed_time(e1))
        for key, values in samples.items():
            values.sort()
            record[f"{key}_ms"] = round(values[len(values) // 2], 4)
        record["fused_tflops"] = round(flops / record["fused_ms"] / 1e9, 1)
        if trace is not None:
            C.gemm_tuning(0, 0, False, trace, 0)
            C.gemm_swiglu_bwd(dy, w, fc, dfc, act, st)
            torch.cuda.synchronize()
            C.gemm_tuning(0, 0, False, None, 0)
            t = trace.view(148, 8)[0::2].double()
            total, epi_total = t[:, 3].clamp(min=1), t[:, 5].clamp(min=1)
            record["trace"] = dict(mma_wait_operands=round((t[:, 1] / total).mean().item(), 3),
                                   mma_wait_accumulator=round((t[:, 2] / total).mean().item(), 3),
                                   epilogue_wait_accumulator=round((t[:, 4] / epi_total).mean().item(), 3),
                                   epilogue_wait_store=round((t[:, 7] / epi_total).mean().item(), 3),
                                   mma_cycles=int(total.mean().item()), tiles_per_pair=round(t[:, 6].mean().item(), 2))
        record["status"] = int(st.item())
        _emit(record)


def bench_mxfp8(args) -> None:
    """Block-scaled MXFP8 GEMM and its quantisation kernels; denominators: this library's bf16 GEMM on the same shape and
    ``torch._scaled_mm`` (the library's tensor-scaled fp8 GEMM) as the measured fp8 rate of the machine."""
    C, st = native(), status_word(torch.device("cuda"))
    flush = None if args.profile else torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device="cuda")
    shapes = [tuple(int(v) for v in s.split("x")) for s in args.shapes] if args.shapes else [
        (8192, 6144, 4096), (8192, 28672, 4096), (8192, 4096, 14336), (8192, 8192, 8192)]
    for M, N, K in shapes:
        flops = 2.0 * M * N * K
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        aq, asf = C.quantize_mx(a, False, 0)
        bq, bsf = C.quantize_mx(b, False, 0)
        record = dict(op="gemm_mxfp8", layout="nt", m=M, n=N, k=K)
        ms = _time(lambda: C.gemm_mxfp8(aq, asf, bq, bsf, out, False, False, 0, 0, False, 1.0, st), args.iters, args.warmup, flush)
        record["mxfp8_ms"], record["mxfp8_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
        ms = _time(lambda: C.gemm(a, b, out, False, False, False, 1.0, st, 0, 2), args.iters, args.warmup, flush)
        record["bf16_pair_ms"], record["bf16_pair_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
        ms = _time(lambda: C.quantize_mx(a, False, 0), args.iters, args.warmup, flush)
        record["quantize_along_columns_ms"], record["quantize_along_columns_gbs"] = round(ms, 4), round(M * K * 3.03 / ms / 1e6, 1)
        if M % 128 == 0:
            ms = _time(lambda: C.quantize_mx(a, True, 0), args.iters, args.warmup, flush)
            record["quantize_along_rows_ms"], record["quantize_along_rows_gbs"] = round(ms, 4), round(M * K * 3.03 / ms / 1e6, 1)
        if not args.profile and hasattr(torch, "_scaled_mm"):
            try:
                a8, b8 = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)
                one = torch.ones((), device="cuda")
                ms = _time(lambda: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), args.iters, args.warmup, flush)
                record["library_fp8_ms"], record["library_fp8_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
            except Exception as error:  # the library call is only a yardstick
                record["library_fp8_error"] = f"{type(error).__name__}: {error}"[:200]
        record["status"] = int(st.item())
        _emit(record)


def bench_attention(args) -> None:
    C, st = native(), status_word(torch.device("cuda"))
    flush = None if args.profile else torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device="cuda")
    groups, qpg, d = args.kv_heads, args.heads // args.kv_heads, args.head_dim
    for spec in args.shapes or ["2x4096", "1x8192"]:
        nseq, L = (int(v) for v in spec.split("x"))
        T = nseq * L
        cu = torch.arange(0, T + 1, L, dtype=torch.int32, device="cuda")
        qkv = torch.randn(T, groups * (qpg + 2) * d, device="cuda", dtype=torch.bfloat16)
        out, lse = C.attn_fwd(qkv, cu, L, groups, qpg, d, d**-0.5, True, st)
        dout = torch.randn_like(out)
        flops = 4.0 * L * L * d * groups * qpg * nseq / 2
        record = dict(op="attention", causal=True, sequences=nseq, seq_len=L, heads=args.heads, kv_heads=groups, head_dim=d)
        if args.direction in ("all", "fwd"):
            ms = _time(lambda: C.attn_fwd(qkv, cu, L, groups, qpg, d, d**-0.5, True, st), args.iters, args.warmup, flush)
            record["fwd_ms"], record["fwd_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
        if args.direction in ("all", "bwd"):
            ms = _time(lambda: C.attn_bwd(dout, qkv, out, lse, cu, L, groups, qpg, d, d**-0.5, True, st), args.iters, args.warmup, flush)
            record["bwd_ms"], record["bwd_tflops"] = round(ms, 4), round(2.5 * flops / ms / 1e9, 1)
            if args.trace:
                # cycle counters of the backward kernel's first CTA (the one with the most query tiles): clocks per
                # (head, query tile) step that its arithmetic threads and its MMA thread spend in each phase / wait
                words = torch.zeros(16, dtype=torch.int64, device="cuda")
                C.attn_bwd_trace(words)
                C.attn_bwd(dout, qkv, out, lse, cu, L, groups, qpg, d, d**-0.5, True, st)
                torch.cuda.synchronize()
                C.attn_bwd_trace(None)
                w = words.tolist()
                steps = max(w[15], 1)
                names = ["wait_S", "P_from_S", None, None, None, "wait_dP", None, "dS_from_dP", "arithmetic_total",
                         "mma_wait_P", "mma_wait_Q", "mma_wait_dS", "mma_wait_dQ_drained", "mma_wait_dO", "mma_total"]
                record["bwd_trace_clocks_per_step"] = {name: round(w[i] / steps, 1) for i, name in enumerate(names) if name}
                record["bwd_trace_steps"] = steps
        if not args.profile and not args.trace:
            try:
                from flash_attn import flash_attn_varlen_func

                x = qkv.view(T, groups, qpg + 2, d)
                q = x[:, :, :qpg].reshape(T, groups * qpg, d).contiguous().requires_grad_(True)
                k = x[:, :, qpg].contiguous().requires_grad_(True)
                v = x[:, :, qpg + 1].contiguous().requires_grad_(True)
                o = flash_attn_varlen_func(q, k, v, cu, cu, L, L, causal=True)
                ms = _time(lambda: flash_attn_varlen_func(q, k, v, cu, cu, L, L, causal=True), args.iters, args.warmup, flush)
                record["flash_attn2_fwd_ms"], record["flash_attn2_fwd_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
                do = dout.view(T, groups * qpg, d)
                ms = _time(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True), args.iters, args.warmup, flush)
                record["flash_attn2_bwd_ms"], record["flash_attn2_bwd_tflops"] = round(ms, 4), round(2.5 * flops / ms / 1e9, 1)
            except ImportError:
                pass
        if hasattr(C, "sb_attn_bwd") and (args.stickbreaking or (not args.profile and not args.trace)):
            # stick-breaking attention on the same buffer (strictly causal, same matrix products as the softmax kernels)
            sb_out, sb_rem = C.sb_attn_fwd(qkv, cu, groups, qpg, d, d**-0.5, st)
            d_rem = torch.randn_like(sb_rem)
            ms = _time(lambda: C.sb_attn_fwd(qkv, cu, groups, qpg, d, d**-0.5, st), args.iters, args.warmup, flush)
            record["stickbreaking_fwd_ms"], record["stickbreaking_fwd_tflops"] = round(ms, 4), round(flops / ms / 1e9, 1)
            ms = _time(lambda: C.sb_attn_bwd(dout, d_rem, qkv, sb_out, sb_rem, cu, groups, qpg, d, d**-0.5, st), args.iters, args.warmup, flush)
            record["stickbreaking_bwd_ms"], record["stickbreaking_bwd_tflops"] = round(ms, 4), round(2.5 * flops / ms / 1e9, 1)
        record["status"] = int(st.item())
        _emit(record)


def bench_moe(args) -> None:
    from .moe import build_grouped_layout

    C, st = native(), status_word(torch.device("cuda"))
    flush = None if args.profile else torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device="cuda")
    T, H, I, E, k = args.tokens, args.hidden, args.intermediate, args.experts, args.top_k
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w_fc = torch.randn(E, 2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.02
    w_proj = torch.randn(E, H, I, device="cuda", dtype=torch.bfloat16) * 0.02
    selected = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]) if T <= 4096 else torch.randint(0, E, (T, k), device="cuda")
    layout = build_grouped_layout(selected.reshape(-1), E)
    xg = C.moe_gather([x.data_ptr()], [], layout.src_entry, H, T * k, k, x)
    record = dict(op="moe_grouped_gemm", tokens=T, hidden=H, intermediate=I, experts=E, top_k=k, rows=layout.rows)
    ms = _time(lambda: C.grouped_rows(xg, w_fc, layout.tile_expert, False, st), args.iters, args.warmup, flush)
    record["c_fc_ms"], record["c_fc_tflops_useful"] = round(ms, 4), round(2.0 * T * k * 2 * I * H / ms / 1e9, 1)
    act = torch.randn(layout.rows, I, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: C.grouped_rows(act, w_proj, layout.tile_expert, False, st), args.iters, args.warmup, flush)
    record["c_proj_ms"], record["c_proj_tflops_useful"] = round(ms, 4), round(2.0 * T * k * I * H / ms / 1e9, 1)
    dw = torch.zeros(E, 2 * I, H, device="cuda", dtype=torch.float32)
    dfc = torch.randn(layout.rows, 2 * I, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: C.grouped_wgrad(dfc, xg, dw, layout.padded_offsets, True, st), args.iters, args.warmup, flush)
    record["wgrad_fc_ms"], record["wgrad_fc_tflops_useful"] = round(ms, 4), round(2.0 * T * k * 2 * I * H / ms / 1e9, 1)
    ms = _time(lambda: C.moe_gather([x.data_ptr()], [], layout.src_entry, H, T * k, k, x), args.iters, args.warmup, flush)
    record["gather_ms"], record["gather_gbs"] = round(ms, 4), round(2.0 * layout.rows * H * 2 / ms / 1e6, 1)
    if hasattr(C, "grouped_rows_dispatch") and H * 2 <= 16384:
        # dispatch fused into the c_fc GEMM, with two buffers of this GPU standing in for the token buffers of two ranks
        # (on one GPU this shows the cost of running the gather inside the GEMM kernel, not the NVLink overlap it is for)
        x2 = torch.randn_like(x)
        both = torch.cat([selected.reshape(-1), selected.flip(0).reshape(-1)]).to(torch.int32)
        layout2 = build_grouped_layout(both, E)
        ptrs = [x.data_ptr(), x2.data_ptr()]

        def separate():
            rows = C.moe_gather(ptrs, [], layout2.src_entry, H, T * k, k, x, layout2.tile_expert, E)
            return C.grouped_rows(rows, w_fc, layout2.tile_expert, False, st)

        record["dispatch_rows"] = layout2.rows
        record["gather_then_c_fc_ms"] = round(_time(separate, args.iters, args.warmup, flush), 4)
        for ctas in (16, 32):
            ms = _time(lambda: C.grouped_rows_dispatch(ptrs, layout2.src_entry, T * k, k, w_fc, layout2.tile_expert, False, st, ctas), args.iters, args.warmup, flush)
            record[f"fused_dispatch_c_fc_ms_{ctas}_gather_ctas"] = round(ms, 4)
    record["status"] = int(st.item())
    _emit(record)


def bench_elementwise(args) -> None:
    C = native()
    flush = None if args.profile else torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device="cuda")
    T, H, I, V = args.tokens, args.hidden, args.intermediate, args.vocab
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    res = torch.randn_like(x)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: C.rmsnorm_fwd(x, res, w, 1e-5, True), args.iters, args.warmup, flush)
    _emit(dict(op="rmsnorm_fwd_residual", tokens=T, hidden=H, ms=round(ms, 4), gbs=round(4.0 * T * H * 2 / ms / 1e6, 1)))
    fc = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: C.swiglu_fwd(fc), args.iters, args.warmup, flush)
    _emit(dict(op="swiglu_fwd", tokens=T, intermediate=I, ms=round(ms, 4), gbs=round(3.0 * T * I * 2 / ms / 1e6, 1)))
    rows = min(T, 4096)
    logits = torch.randn(rows, V, device="cuda", dtype=torch.bfloat16)
    labels = torch.randint(0, V, (rows,), device="cuda")
    ms = _time(lambda: C.cross_entropy_(logits, labels, 1.0, 1.0, -100, True), args.iters, args.warmup, flush)
    _emit(dict(op="cross_entropy_inplace", rows=rows, vocab=V, ms=round(ms, 4), gbs=round(2.0 * rows * V * 2 / ms / 1e6, 1)))
    n = 256 * 1024 * 1024
    p32, g32 = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros_like(p32), torch.zeros_like(p32)
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    # reads p, m, v, g (fp32); writes p, m, v, g (zeroed) and the bf16 copy
    ms = _time(lambda: C.adamw_step(p32, m, v, g32, p16, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, None, 1.0, True), args.iters, args.warmup, flush)
    _emit(dict(op="adamw_step", elements=n, ms=round(ms, 4), gbs=round(n * (4 * 4 + 4 * 4 + 2) / ms / 1e6, 1)))


def bench_scans(args) -> None:
    """State-resident scans: Mamba-2 SSD (against the chunked PyTorch formulation) and the GRU scan."""
    from ..hf_models.layers.mamba2 import ssd_chunk_scan
    from .recurrent import recurrent_scan
    from .ssd import ssd_scan

    flush = None if args.profile else torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device="cuda")
    B, L, H, G, P, N = 4, 4096, 32, 1, 64, 128
    x = torch.randn(B, L, H, P, device="cuda", requires_grad=True)
    a = (-torch.rand(B, L, H, device="cuda") * 0.2).requires_grad_(True)
    b = (torch.randn(B, L, G, N, device="cuda") * 0.3).requires_grad_(True)
    c = (torch.randn(B, L, G, N, device="cuda") * 0.3).requires_grad_(True)
    dy = torch.randn(B, L, H, P, device="cuda")

    def native_step():
        y, _ = ssd_scan(x, a, b, c)
        y.backward(dy)

    def torch_step():
        y, _ = ssd_chunk_scan(x, a, b.repeat_interleave(H // G, dim=2), c.repeat_interleave(H // G, dim=2), 256)
        y.backward(dy)

    record = dict(op="ssd_scan", batch=B, seq_len=L, heads=H, head_dim=P, state=N)
    record["fwd_ms"] = round(_time(lambda: ssd_scan(x.detach(), a.detach(), b.detach(), c.detach()), args.iters, args.warmup, flush), 4)
    record["fwd_bwd_ms"] = round(_time(native_step, args.iters, args.warmup, flush), 4)
    record["torch_chunked_fwd_bwd_ms"] = round(_time(torch_step, max(2, args.iters // 4), 1, flush), 4)
    _emit(record)

    n, d = 16, 64
    tokens = 4 * 4096
    cu = torch.arange(0, tokens + 1, 4096, dtype=torch.int32, device="cuda")
    xr = (torch.randn(tokens, 3 * n * d, device="cuda", dtype=torch.bfloat16) * 0.5).requires_grad_(True)
    wr = (torch.randn(3 * n, d, d, device="cuda") / d**0.5).requires_grad_(True)
    dout = torch.randn(tokens, n, d, device="cuda", dtype=torch.bfloat16)

    def gru_step():
        recurrent_scan(xr, wr, cu, n, d, True, None).backward(dout)

    record = dict(op="gru_scan", sequences=4, seq_len=4096, heads=n, head_dim=d)
    record["fwd_ms"] = round(_time(lambda: recurrent_scan(xr.detach(), wr.detach(), cu, n, d, True, None), args.iters, args.warmup, flush), 4)
    record["fwd_bwd_ms"] = round(_time(gru_step, args.iters, args.warmup, flush), 4)
    _emit(record)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("op", choices=["gemm", "mxfp8", "attention", "moe", "elementwise", "scans"])
    parser.add_argument("--shapes", nargs="*", help="gemm: MxNxK ...; attention: SEQUENCESxLENGTH ...")
    parser.add_argument("--layouts", nargs="*", default=["nt"], help="gemm: nt (y = x w^T), nn (dgrad), tn (wgrad)")
    parser.add_argument("--variant", default="all", choices=["all", "cta1", "cta_pair"])
    parser.add_argument("--direction", default="all", choices=["all", "fwd", "bwd"])
    parser.add_argument("--groups", nargs="*", type=int, default=[0], help="gemm: raster groups of the CTA-pair kernel to sweep (0 = built-in)")
    parser.add_argument("--k-skew", nargs="*", type=int, default=[0], help="gemm: k-block skews of the CTA-pair kernel to sweep")
    parser.add_argument("--split-k", nargs="*", type=int, default=[0], help="gemm --accumulate: splits of K to sweep (0 = built-in, 1 = none)")
    parser.add_argument("--direct-store", action="store_true", help="gemm: also time the register-store epilogue")
    parser.add_argument("--accumulate", action="store_true", help="gemm: fp32 accumulate into the output (weight-gradient form)")
    parser.add_argument("--stickbreaking", action="store_true", help="attention: run the stick-breaking kernels also under --profile / --trace")
    parser.add_argument("--trace", action="store_true", help="gemm: report where the MMA and epilogue threads of the CTA-pair kernel wait")
    parser.add_argument("--interleave", action="store_true", help="gemm: candidates and the library take turns launch by launch after heating the GPU to its power-capped clock")
    parser.add_argument("--heat-ms", type=float, default=1500.0, help="gemm --interleave: length of the warm-up under load")
    parser.add_argument("--swiglu-only", action="store_true", help="gemm: run nothing but the c_fc GEMM with the SwiGLU epilogue (the form to put under a profiler)")
    parser.add_argument("--swiglu-bwd", action="store_true", help="gemm: time only the down-projection data gradient with the SwiGLU backward in its epilogue")
    parser.add_argument("--swiglu", action="store_true", help="gemm: also time the c_fc GEMM with the SwiGLU epilogue")
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--profile", action="store_true", help="no comparison library, no L2 flush kernel")
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--tokens", type=int, default=8192)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--intermediate", type=int, default=14336)
    parser.add_argument("--experts", type=int, default=40)
    parser.add_argument("--top-k", type=int, default=8)
    parser.add_argument("--vocab", type=int, default=128256)
    args = parser.parse_args()
    {"gemm": bench_gemm, "mxfp8": bench_mxfp8, "attention": bench_attention, "moe": bench_moe, "elementwise": bench_elementwise, "scans": bench_scans}[args.op](args)


if __name__ == "__main__":
    main()
