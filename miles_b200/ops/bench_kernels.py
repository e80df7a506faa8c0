"""Device-timed micro-benchmarks of the hot kernels against the measured machine peaks.

    python -m miles_b200.ops.bench_kernels gemm [--m 8192 --n 8192 --k 8192] [--iters 20]
    python -m miles_b200.ops.bench_kernels attention [--seqlen 4096 --batch 8]
    python -m miles_b200.ops.bench_kernels decode [--batch 64 --context 4096]
    python -m miles_b200.ops.bench_kernels elementwise
    python -m miles_b200.ops.bench_kernels all --json out.json

Timing: CUDA events on the launching stream after 3 warm-up launches, synchronised on both sides; a 256 MiB buffer is
written between timed launches to flush L2 (126 MB).  Roofline fractions are reported "of measured" against
MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 burst throughput) when that file is present, otherwise "of fallback"
(6.65 TB/s, 1.59 PFLOP/s).  cuBLAS (torch.matmul) is timed alongside the GEMM as the library baseline.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def timeit(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def bench_gemm(a):
    from miles_b200.ops import cuda as K

    hbm, tf, tag = peaks()
    out = []
    shapes = [(a.m, a.n, a.k)] if a.m else [(8192, 8192, 8192), (16384, 5120, 2048), (16384, 2048, 4096), (16384, 1536, 2048),
                                           (16384, 151936 // 8, 2048), (64, 5120, 2048), (64, 2048, 4096)]
    for (M, N, Kd) in shapes:
        x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: K.gemm_nt(x, w, out=y), a.iters)
        ms_lib = timeit(lambda: torch.matmul(x, w.t(), out=y), a.iters)
        flops = 2.0 * M * N * Kd
        byts = 2.0 * (M * Kd + N * Kd + M * N)
        t_roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3
        out.append({"kernel": "gemm_bf16_nt", "M": M, "N": N, "K": Kd, "ms": ms, "tflops": flops / ms / 1e9, "cublas_ms": ms_lib,
                    "cublas_tflops": flops / ms_lib / 1e9, "vs_cublas": ms_lib / ms, "roofline_frac": t_roof / ms, "roofline": tag})
    return out


def bench_attention(a):
    from miles_b200.ops import cuda as K

    hbm, tf, tag = peaks()
    B, L, Hq, Hkv, D = a.batch, a.seqlen, 32, 4, 128
    T = B * L
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu = torch.arange(0, T + 1, L, dtype=torch.int32, device="cuda")
    fwd = timeit(lambda: K.attention_varlen(q.detach(), k.detach(), v.detach(), cu, L), a.iters)
    o = K.attention_varlen(q, k, v, cu, L)
    g = torch.randn_like(o)
    bwd = timeit(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True), a.iters)
    f_fwd = 4.0 * B * Hq * L * L * D / 2
    return [{"kernel": "flash_fwd", "batch": B, "seqlen": L, "ms": fwd, "tflops": f_fwd / fwd / 1e9, "roofline_frac": f_fwd / (tf * 1e12) * 1e3 / fwd,
             "roofline": tag, "ctas_per_sm": K.C.flash_fwd_tc_ctas_per_sm()},
            {"kernel": "flash_bwd", "batch": B, "seqlen": L, "ms": bwd, "tflops": 2.5 * f_fwd / bwd / 1e9,
             "roofline_frac": 2.5 * f_fwd / (tf * 1e12) * 1e3 / bwd, "roofline": tag}]


def bench_decode(a):
    from miles_b200.ops import cuda as K

    hbm, tf, tag = peaks()
    B, L, Hq, Hkv, D, bs = a.batch, a.context, 32, 4, 128, 64
    nb = (L + bs - 1) // bs
    kc = torch.randn(B * nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.arange(B * nb, dtype=torch.int32, device="cuda").view(B, nb)
    sl = torch.full((B,), L, dtype=torch.int32, device="cuda")
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.paged_attention(q, kc, vc, bt, sl), a.iters)
    byts = 2.0 * B * L * Hkv * D * 2
    return [{"kernel": "paged_decode_mma", "batch": B, "context": L, "ms": ms, "gbs": byts / ms / 1e6, "roofline_frac": byts / (hbm * 1e9) * 1e3 / ms,
             "roofline": tag}]


def bench_elementwise(a):
    from miles_b200.ops import cuda as K

    hbm, tf, tag = peaks()
    T, H = 32768, 2048
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    out = []
    ms = timeit(lambda: K.add_rmsnorm(x, r, w, 1e-6), a.iters)
    out.append({"kernel": "add_rmsnorm", "T": T, "H": H, "ms": ms, "gbs": 4 * T * H * 2 / ms / 1e6, "roofline_frac": 4 * T * H * 2 / (hbm * 1e9) * 1e3 / ms, "roofline": tag})
    gu = torch.randn(T, 2 * 768 * 8, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.swiglu(gu), a.iters)
    b = gu.numel() * 2 * 1.5
    out.append({"kernel": "swiglu", "T": T, "F": 768 * 8, "ms": ms, "gbs": b / ms / 1e6, "roofline_frac": b / (hbm * 1e9) * 1e3 / ms, "roofline": tag})
    n = 1 << 28
    master, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
    po = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.adamw_step_masked(master, g, m, v.abs_(), None, 1e-3, 0.9, 0.98, 1e-8, 0.0, 1, 1.0, po), a.iters)
    b = n * (4 * 4 + 3 * 4 + 2)
    out.append({"kernel": "adamw", "n": n, "ms": ms, "gbs": b / ms / 1e6, "roofline_frac": b / (hbm * 1e9) * 1e3 / ms, "roofline": tag})
    xq = torch.randn(16384, 4096, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.mxfp8_quant(xq), a.iters)
    b = xq.numel() * (2 + 1 + 1 / 32)
    out.append({"kernel": "mxfp8_quant", "numel": xq.numel(), "ms": ms, "gbs": b / ms / 1e6, "roofline_frac": b / (hbm * 1e9) * 1e3 / ms, "roofline": tag})
    ms = timeit(lambda: K.nvfp4_qdq(xq, torch.ones(1, device="cuda")), a.iters)
    b = xq.numel() * 4
    out.append({"kernel": "nvfp4_qdq", "numel": xq.numel(), "ms": ms, "gbs": b / ms / 1e6, "roofline_frac": b / (hbm * 1e9) * 1e3 / ms, "roofline": tag})
    for mode in (0, 1, 2):                      # MXFP8 / MXFP4 / compressed-KV style fake quantisation: read 2 B, write 2 B per element
        ms = timeit(lambda: K.C.block_fake_quant(xq, mode), a.iters)
        out.append({"kernel": f"block_fake_quant<{mode}>", "numel": xq.numel(), "ms": ms, "gbs": b / ms / 1e6,
                    "roofline_frac": b / (hbm * 1e9) * 1e3 / ms, "roofline": tag})
    return out


def bench_mxfp8(a):
    """Block-scaled MXFP8 GEMM against the bf16 GEMM on the same shapes (fp8 peak is twice the bf16 peak)."""
    from miles_b200.ops import cuda as K
    from miles_b200.ops import extra as X

    hbm, tf, tag = peaks()
    out = []
    shapes = [(a.m, a.n, a.k)] if a.m else [(8192, 8192, 8192), (16384, 5120, 2048), (16384, 2048, 4096)]
    for M, N, Kd in shapes:
        x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16)
        xq, xs = K.mxfp8_quant(x)
        wq, ws = K.mxfp8_quant(w)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: X.gemm_mxfp8(xq, xs, wq, ws, out=y), a.iters)
        ms_q = timeit(lambda: K.mxfp8_quant(x), a.iters)
        ms_bf16 = timeit(lambda: K.gemm_nt(x, w, out=y), a.iters)
        flops = 2.0 * M * N * Kd
        out.append({"kernel": "gemm_mxfp8_block_scaled", "M": M, "N": N, "K": Kd, "ms": ms, "tflops": flops / ms / 1e9,
                    "bf16_gemm_ms": ms_bf16, "vs_bf16_gemm": ms_bf16 / ms, "quant_activation_ms": ms_q,
                    "roofline_frac": flops / (2 * tf * 1e12) * 1e3 / ms, "roofline": tag + " (2 × bf16 peak)"})
    return out


def bench_moe_gemv(a):
    """Decode-time MoE FFN for a handful of tokens (matrix-vector kernels, gemv.cu): 16 local experts of the Qwen3-30B-A3B
    shape, top-8 routing; three weight sets are rotated so that no call finds its 151 MB of weights in L2."""
    from . import cuda as K
    from . import reference as ref

    hbm, _, tag = peaks()
    T, k, E, H, F = max(1, min(a.batch, 8)), 8, 16, 2048, 768
    torch.manual_seed(0)
    sets = [((0.02 * torch.randn(E, 2 * F, H, device="cuda")).bfloat16(), (0.02 * torch.randn(E, H, F, device="cuda")).bfloat16())
            for _ in range(3)]
    x = torch.randn(T, H, device="cuda").bfloat16()
    tw, ti, _ = ref.router_topk(torch.randn(T, E, device="cuda"), k, True)
    ti32, twf = ti.to(torch.int32).contiguous(), tw.float().contiguous()
    act = torch.empty(T * k, F, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(x)
    state = {"i": 0}

    def run():
        w13, w2 = sets[state["i"] % 3]
        state["i"] += 1
        K.C.moe_gemv(x, w13, w2, ti32, twf, act, out, 0)

    ms = timeit(run, iters=a.iters, flush=False)
    w13, w2 = sets[(state["i"] - 1) % 3]
    want = ref.moe_ffn(x.float(), w13.float(), w2.float(), tw.float(), ti)
    rel = ((out.float() - want).norm() / want.norm()).item()
    touched = int(torch.unique(ti).numel())
    gb = touched * 3 * F * H * 2 / 1e9
    return [{"op": "moe_gemv up+down", "tokens": T, "experts_touched": touched, "us": ms * 1e3, "weight_MB": gb * 1e3,
             "GBps": gb / (ms * 1e-3), "frac_hbm": gb / (ms * 1e-3) / hbm, "peak": tag, "rel_err_vs_fp32": rel}]


def main():
    p = argparse.ArgumentParser()
    p.add_argument("what", choices=["gemm", "mxfp8", "attention", "decode", "elementwise", "moe_gemv", "all"])
    p.add_argument("--m", type=int, default=0)
    p.add_argument("--n", type=int, default=8192)
    p.add_argument("--k", type=int, default=8192)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--seqlen", type=int, default=4096)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--json", type=str, default=None)
    a = p.parse_args()
    torch.cuda.set_device(0)
    rows = []
    if a.what in ("gemm", "all"):
        rows += bench_gemm(a)
    if a.what in ("mxfp8", "all"):
        rows += bench_mxfp8(a)
    if a.what in ("attention", "all"):
        rows += bench_attention(a)
    if a.what in ("decode", "all"):
        a2 = argparse.Namespace(**vars(a))
        a2.batch = max(a.batch, 64) if a.what == "all" else a.batch
        rows += bench_decode(a2)
    if a.what in ("elementwise", "all"):
        rows += bench_elementwise(a)
    if a.what in ("moe_gemv", "all"):
        rows += bench_moe_gemv(a)
    for r in rows:
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
