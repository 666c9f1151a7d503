"""Device-timed comparison of the fused compute+collective kernels with their NCCL arms.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m plow_b200.parallel.bench_collectives [--iters 50]

Every case is captured in a CUDA graph of ``reps`` back-to-back calls (so Python launch cost is out of the number),
replayed after 3 warm-up replays, timed with CUDA events on the launching stream and reduced with MAX over ranks.
Rank 0 prints one JSON line per case with the roofline of the fused op:
    t_roof = max(FLOPs / measured GEMM peak, bytes over NVLink per GPU / 770 GB/s, weight bytes / measured HBM copy rate)
(the decode shapes are weight-streaming bound, so the HBM term is the binding one) and achieved = t_roof / t.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peaks(path):
    """(HBM GB/s, sustained bf16 TFLOP/s, source) from the measured-peaks JSON named on the command line."""
    try:
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops_sustained"], "measured"
    except Exception:
        return 6650.0, 1400.0, "fallback"


def _graph_time(fn, reps, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) * 1e3 / (iters * reps)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--reps", type=int, default=8)
    ap.add_argument("--peaks", default="", help="JSON file of measured peaks (hbm_gbs, bf16_tflops_sustained) for the roofline column")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ..ops import native, quant
    from .tp import TpComm
    hbm, tflops, src = _peaks(a.peaks)
    fused = TpComm(rank, world, impl="fused", max_rows=128, max_n=8192, max_k=8192, form="oneshot")
    fused2 = TpComm(rank, world, impl="fused", max_rows=128, max_n=8192, max_k=8192, form="twoshot")
    fused3 = TpComm(rank, world, impl="fused", max_rows=128, max_n=8192, max_k=8192, form="nvls") if fused.mc_ptr else None
    nccl = TpComm(rank, world, impl="nccl")
    # row-parallel projections of the dense 8B shape (o_proj, down) and of the MLA shape (o_proj), K sharded over ranks
    for name, M, N, Kfull, fp8 in (("dense8b_o_proj", 64, 4096, 4096, False), ("dense8b_down", 64, 4096, 14336, False),
                                   ("mla_o_proj_fp8", 64, 7168, 16384, True)):
        K = max(128, Kfull // world // 128 * 128)
        x = torch.randn(M, K, device="cuda")
        w = torch.randn(N, K, device="cuda") * 0.05
        if fp8:
            xq, sx = quant.quant_act_1x128(x)
            wq, sw = quant.quant_weight_128x128(w)
        else:
            xq, wq, sx, sw = x.bfloat16(), w.bfloat16(), None, None
        tf = _graph_time(lambda: fused.gemm_allreduce(xq, wq, N, sx=sx, sw=sw), a.reps, a.iters)
        t2 = _graph_time(lambda: fused2.gemm_allreduce(xq, wq, N, sx=sx, sw=sw), a.reps, a.iters)
        t3 = _graph_time(lambda: fused3.gemm_allreduce(xq, wq, N, sx=sx, sw=sw), a.reps, a.iters) if fused3 else None
        tn = _graph_time(lambda: nccl.gemm_allreduce(xq, wq, N, sx=sx, sw=sw), a.reps, a.iters)
        native.check_status()
        es = 1 if fp8 else 2
        link = float(world - 1) * M * N * 2                     # one-shot: this rank's partial to every peer
        roof = max(2.0 * M * N * K / (tflops * 1e6), link / (NVLINK_GBS * 1e3), N * K * es / (hbm * 1e3))
        if rank == 0:
            print(json.dumps(dict(case=f"gemm_allreduce/{name}", world=world, M=M, N=N, K_per_rank=K, fused_us=round(tf, 2),
                                  fused_twoshot_us=round(t2, 2), fused_nvls_us=(round(t3, 2) if t3 else None), nccl_us=round(tn, 2), roofline_us=round(roof, 2),
                                  achieved=round(roof / min(x for x in (tf, t2, t3) if x), 3), peaks=src)))
    # column-parallel projections behind a sequence-parallel seam: gather the row bands, then GEMM
    for name, M, Nfull, K in (("dense8b_qkv", 64, 6144, 4096), ("dense8b_gate_up", 64, 28672, 4096)):
        N = Nfull // world // 128 * 128
        band = M // world
        xb = torch.randn(band, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        tf = _graph_time(lambda: (fused.allgather_gemm(xb, w, N), fused.allgather_gemm(xb, w, N)), a.reps // 2, a.iters) / 2
        tn = _graph_time(lambda: nccl.allgather_gemm(xb, w, N), a.reps, a.iters)
        native.check_status()
        link = (world - 1) * band * K * 2.0
        roof = max(2.0 * M * N * K / (tflops * 1e6), link / (NVLINK_GBS * 1e3), N * K * 2.0 / (hbm * 1e3))
        if rank == 0:
            print(json.dumps(dict(case=f"allgather_gemm/{name}", world=world, M=M, N_per_rank=N, K=K, fused_us=round(tf, 2),
                                  nccl_us=round(tn, 2), roofline_us=round(roof, 2), achieved=round(roof / tf, 3), peaks=src)))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
