"""Device-timed benchmark of the fused tensor-parallel paths against the NCCL + GEMM path, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m miles_b200.parallel.bench_tp [--shape qwen3-32b|qwen3-4b] [--tokens 8192] [--iters 10] [--json out.json]

For the model shape and TP = N it times, per op, `iters` launches after 3 warm-ups with CUDA events on the launching
stream (a host barrier and a device synchronise on both sides, a 256 MiB write between launches to flush L2) and takes the
MAX over ranks:

  ag_gemm     sequence-parallel all-gather → column GEMM   (QKV and FC1 of the shape)   fused kernel  vs  NCCL all-gather + GEMM
  gemm_rs     row GEMM → reduce-scatter                    (O-proj and FC2)             fused kernel  vs  GEMM + NCCL reduce-scatter
  ar_rmsnorm  all-reduce + residual add + RMSNorm          (decode 64 rows, prefill T)  fused kernel(s) vs NCCL all-reduce + add-RMSNorm

Roofline per op = the slower of FLOPs ÷ measured bf16 GEMM peak and the bytes that must cross NVLink ÷ 770 GB/s per
direction (the measured peer-copy rate of this pool; 900 nominal); the table prints achieved ÷ that.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

SHAPES = {
    # hidden, q heads, kv heads, head_dim, ffn
    "qwen3-32b": dict(H=5120, hq=64, hkv=8, d=128, F=25600),
    "qwen3-4b": dict(H=2560, hq=32, hkv=8, d=128, F=9728),
}
NVLINK_GBS = 770.0


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], "of measured"
    return 1590.0, "of fallback"


_flush = None


def _timeit(fn, iters, group):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        _flush.fill_(1)
        dist.barrier(group=group)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    t = torch.tensor([tot / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="qwen3-32b", choices=sorted(SHAPES))
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()

    from ..ops import add_rmsnorm
    from ..ops import cuda as K
    from . import tp as tpmod
    from .fabric import Fabric
    from .state import ParallelState, init_distributed

    rank, world, local = init_distributed()
    torch.cuda.set_device(local)
    ps = ParallelState.build(tp=world, sequence_parallel=True)
    ps.fabric = Fabric.create(ps)
    sh = SHAPES[a.shape]
    H, F = sh["H"], sh["F"]
    qkv = (sh["hq"] + 2 * sh["hkv"]) * sh["d"]
    T = a.tokens // (128 * world) * (128 * world)
    n = T // world
    peak, label = _peaks()
    g = torch.Generator(device="cuda").manual_seed(5 + rank)
    rows = []

    def rnd(*shape):
        return (0.05 * torch.randn(*shape, device="cuda", generator=g)).bfloat16()

    def report(op, name, M, N, Kd, nvl_bytes, t_fused, t_nccl):
        flops = 2.0 * M * N * Kd
        ideal_ms = max(flops / (peak * 1e12), nvl_bytes / (NVLINK_GBS * 1e9)) * 1e3
        rows.append(dict(op=op, layer=name, M=M, N=N, K=Kd, fused_ms=round(t_fused, 4), nccl_ms=round(t_nccl, 4),
                         speedup=round(t_nccl / t_fused, 3), roofline_ms=round(ideal_ms, 4),
                         frac_of_roofline=round(ideal_ms / t_fused, 3),
                         bound="compute" if flops / (peak * 1e12) >= nvl_bytes / (NVLINK_GBS * 1e9) else "nvlink"))

    with torch.no_grad():
        # ---- all-gather → column GEMM --------------------------------------------------------------------------------
        for name, N_full in (("qkv", qkv), ("fc1", 2 * F)):
            Nl = N_full // world
            x, w = rnd(n, H), rnd(Nl, H)
            ps.fused = True
            tf = _timeit(lambda: ps.fabric.ag_gemm(x, w, ps), a.iters, ps.tp_group)
            tn = _timeit(lambda: K.gemm_nt(tpmod._all_gather_dim0(x, ps), w), a.iters, ps.tp_group)
            report("ag_gemm", name, T, Nl, H, (world - 1) * n * H * 2, tf, tn)
        # ---- row GEMM → reduce-scatter --------------------------------------------------------------------------------
        for name, K_full in (("o_proj", sh["hq"] * sh["d"]), ("fc2", F)):
            Kl = K_full // world
            x, w = rnd(T, Kl), rnd(H, Kl)
            tf = _timeit(lambda: ps.fabric.gemm_rs(x, w, ps), a.iters, ps.tp_group)
            tn = _timeit(lambda: tpmod._reduce_scatter_dim0(K.gemm_nt(x, w), ps), a.iters, ps.tp_group)
            report("gemm_rs", name, T, H, Kl, (world - 1) * n * H * 2, tf, tn)
        # ---- all-reduce + add + RMSNorm (engine path: replicated activations) --------------------------------------------
        ps.sequence_parallel = False
        wn = rnd(H) + 1
        for name, rows_ in (("decode64", 64), ("prefill", T)):
            part, res = rnd(rows_, H), rnd(rows_, H)
            tf = _timeit(lambda: ps.fabric.allreduce_add_rmsnorm(part, res, wn, 1e-6, ps), a.iters, ps.tp_group)
            tn = _timeit(lambda: add_rmsnorm(tpmod._all_reduce(part, ps), res, wn, 1e-6), a.iters, ps.tp_group)
            two_shot = world >= 4 and rows_ % world == 0 and rows_ * H * 2 >= (1 << 20)
            nvl = (2 * (world - 1) / world if two_shot else (world - 1)) * rows_ * H * 2
            ideal_ms = nvl / (NVLINK_GBS * 1e9) * 1e3
            rows.append(dict(op="ar_rmsnorm", layer=name, M=rows_, N=H, K=0, fused_ms=round(tf, 4), nccl_ms=round(tn, 4),
                             speedup=round(tn / tf, 3), roofline_ms=round(ideal_ms, 4), frac_of_roofline=round(ideal_ms / tf, 3),
                             bound="nvlink", schedule="two-shot" if two_shot else "one-shot"))
    ps.fabric.check()
    if rank == 0:
        print(f"# {a.shape}, TP = {world}, T = {T} tokens; bf16 peak {peak} TFLOP/s ({label}), NVLink {NVLINK_GBS} GB/s per direction")
        print("| op | layer | M×N×K | fused ms | NCCL path ms | speed-up | roofline ms | achieved ÷ roofline | bound |")
        print("|---|---|---|---|---|---|---|---|---|")
        for r in rows:
            print(f"| {r['op']} | {r['layer']} | {r['M']}×{r['N']}×{r['K']} | {r['fused_ms']} | {r['nccl_ms']} | {r['speedup']} | "
                  f"{r['roofline_ms']} | {r['frac_of_roofline']} | {r['bound']}{' ' + r['schedule'] if 'schedule' in r else ''} |")
        if a.json:
            json.dump({"shape": a.shape, "tp": world, "tokens": T, "rows": rows}, open(a.json, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
