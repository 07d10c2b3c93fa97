#!/usr/bin/env python
"""Row-parallel GEMM -> reduce -> residual + RMSNorm -> (all-gather) -> column-parallel GEMM on N GPUs:
the communication-bound half of a tensor-parallel decoder layer, timed on the device per variant.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29500 \
        benchmark/kernels/bench_fused_comm.py [--tokens 128 1152 8192] [--iters 30]

Variants (same inputs, same outputs):
  nccl      library GEMM kernel of this repo + NCCL all-reduce + fused add-RMSNorm kernel + GEMM
  two       GEMM with reduce-scatter push epilogue + reduce/norm/all-gather kernel (two barriers) + GEMM
  one       one launch: GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather (waits for its peers) + GEMM
  one+ag    the same launch without the final wait + the consumer GEMM that waits per chunk of rows
  gemms     the two GEMMs alone (no reduction, no norm): the floor of this repo's GEMM kernels

Shapes are Qwen3-32B's at tensor-parallel size N: hidden 5120; o_proj (K = 8192 / N) feeding gate_up
(N2 = 51200 / N), and down_proj (K = 25600 / N) feeding qkv (N2 = 10240 / N).  Every iteration uses another copy
of the weights (more than L2 in total).  Times are CUDA-event means over `iters` launches, max over ranks.  The
NVLink floor of the reduce + gather is 2 * (N - 1) / N * T * hidden * 2 bytes per rank and direction at the
measured 770 GB/s peer-copy bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="*", default=[128, 1152, 8192])
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    from sglang_jax_b200 import ops
    from sglang_jax_b200.ops import native
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.parallel.fused_comm import FusedComm
    ps.init_distributed(rank, world, "cuda", init_method="env://" if world > 1 else None,
                        local_rank=int(os.environ.get("LOCAL_RANK", rank)))
    st = ps.get_state()
    dev = st.device
    H = 5120
    comm = FusedComm.create(st, H, torch.bfloat16, max_tokens=max(args.tokens) + 128) if world > 1 else \
        FusedComm.create_loopback(H, dev, max_tokens=max(args.tokens) + 128)
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    copies = 6
    rows = []
    peak = 1.59e15          # fallback cuBLAS bf16 burst figure; the measured one when the driver's file is present
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] * 1e12
    except Exception:
        pass
    for name, K, N2 in (("o_proj->gate_up", 8192 // world, 51200 // world), ("down_proj->qkv", 25600 // world, 10240 // world)):
        ws = [(torch.randn(H, K, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        w2s = [(torch.randn(N2, H, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
        for T in args.tokens:
            x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
            res = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)

            def nccl(i):
                y = ops.linear(x, ws[i % copies])
                if world > 1:
                    dist.all_reduce(y, group=st.tp.device_group)
                h, _ = native.fused_add_rmsnorm(y, res, nw, 1e-6)
                return ops.linear(h, w2s[i % copies])

            def fused(one_kernel, defer):
                def run(i):
                    comm.one_kernel = one_kernel
                    h, _ = comm.gemm_allreduce_add_rmsnorm(x, ws[i % copies], res, nw, 1e-6, defer=defer)
                    return comm.consume_linear(h, w2s[i % copies]) if defer else native.linear(h, w2s[i % copies])
                return run

            def gemms_only(i):
                y = ops.linear(x, ws[i % copies])
                return ops.linear(y, w2s[i % copies])

            for label, fn in (("gemms", gemms_only), ("nccl", nccl), ("two", fused(False, False)),
                              ("one", fused(True, False)), ("one+ag", fused(True, True))):
                for i in range(3):
                    fn(i)
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier(group=st.tp.cpu_group)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                if T <= 256:
                    # decode-sized: the launches of a step run from a captured graph in serving, so time them that way
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(side):
                        fn(0)
                        with torch.cuda.graph(graph, stream=side):
                            for i in range(args.iters):
                                fn(i)
                    torch.cuda.current_stream().wait_stream(side)
                    graph.replay()
                    torch.cuda.synchronize()
                    if world > 1:
                        dist.barrier(group=st.tp.cpu_group)
                    e0.record()
                    graph.replay()
                    e1.record()
                else:
                    e0.record()
                    for i in range(args.iters):
                        fn(i)
                    e1.record()
                torch.cuda.synchronize()
                native.check_status()
                us = e0.elapsed_time(e1) * 1e3 / args.iters
                t = torch.tensor([us], dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=st.tp.cpu_group)
                link_us = 2 * (world - 1) / world * T * H * 2 / 770e9 * 1e6
                flops = 2.0 * T * H * K + 2.0 * T * H * N2
                rows.append({"pair": name, "tokens": T, "variant": label, "us": round(float(t.item()), 1),
                             "nvlink_floor_us": round(link_us, 1), "gemm_floor_us": round(flops / peak * 1e6, 1)})
                if rank == 0:
                    print(json.dumps(rows[-1]), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
