#!/usr/bin/env python
"""Bandwidth and latency of the NVLink collectives of this package against NCCL, on the GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 benchmark/comm_bench.py [--max-mb 256]

For every message size (per-rank bytes) and collective - all-gather, all-to-all, reduce-scatter, axis switch + LayerNorm -
the script times the one-kernel push collective (csrc/comm_p2p.cu ``symm_xchg_k`` / ``symm_xchg_ln_k``), the
two-kernel publish + pull form it replaced, and the NCCL call the reference uses, as CUDA-graph replays timed with CUDA
events, maximum over ranks.  Reported per row: microseconds per call and the NVLink bytes this rank must send divided
by that time (GB/s), to be read against the measured peer-copy bandwidth of the pool (770 GB/s per direction) - the
roofline of a collective is bytes over link bandwidth.  The 16-byte row is the flag round trip: the latency floor of
a collective.  Rank 0 prints one JSON line per row.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters=20, warmup=3):
    """Mean microseconds of ``fn()`` replayed from a CUDA graph (``iters`` calls per replay), max over ranks."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=128, help="largest per-rank message in MiB")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    os.environ.setdefault("FASTFOLD_SYMM_HEAP_MB", str(16 * 1024))
    from fastfold_b200.parallel import core, init_dap, symm
    world = int(os.environ.get("WORLD_SIZE", 1))
    init_dap(world)
    P, rank = core.get_dap_size(), core.get_dap_rank()
    assert P > 1, "needs at least 2 ranks"
    symm.request_message_bytes(args.max_mb * (1 << 20) * P)
    h = symm.get_heap("dap")
    dev = torch.device("cuda", torch.cuda.current_device())
    group = core.get_dap_group()
    sizes = [16 * P]
    mb = 1
    while mb <= args.max_mb:
        sizes.append(mb << 20)
        mb *= 4
    rows = []

    def report(name, nbytes, sent, variants):
        row = {"collective": name, "ranks": P, "bytes_per_rank": nbytes, "nvlink_bytes_sent_per_rank": sent}
        for k, us in variants.items():
            row[k + "_us"] = round(us, 2)
            row[k + "_GBps"] = round(sent / us / 1e3, 1)
        rows.append(row)
        if core.get_rank() == 0:
            print(json.dumps(row), flush=True)

    for nb in sizes:
        n = nb // 2
        x = torch.randn(n, device=dev).to(torch.bfloat16)
        frac = (P - 1) / P
        # all-gather: every rank sends its nb bytes to P - 1 peers
        out = torch.empty(P * n, device=dev, dtype=torch.bfloat16)
        v = {"push": timed(lambda: h.gather_dim(x.view(1, n), 0), args.iters)}
        symm.PUSH = False
        v["publish_pull"] = timed(lambda: h.all_gather(None, x), args.iters)
        symm.PUSH = True
        v["nccl"] = timed(lambda: dist.all_gather_into_tensor(out, x, group=group), args.iters)
        report("all_gather", nb, nb * (P - 1), v)
        # all-to-all: (P - 1) / P of the message leaves the GPU
        send = x.view(P, n // P)
        recv = torch.empty_like(send)
        v = {"push": timed(lambda: h.all_to_all(None, send), args.iters)}
        symm.PUSH = False
        v["publish_pull"] = timed(lambda: h.all_to_all(None, send), args.iters)
        symm.PUSH = True
        v["nccl"] = timed(lambda: dist.all_to_all_single(recv, send, group=group), args.iters)
        report("all_to_all", nb, int(nb * frac), v)
        # reduce-scatter (sum in fp32 at the destination)
        rs_out = torch.empty(n // P, device=dev, dtype=torch.bfloat16)
        v = {"push": timed(lambda: h.reduce_scatter_dim(x.view(P, n // P), 0), args.iters)}
        v["nccl"] = timed(lambda: dist.reduce_scatter_tensor(rs_out, x, group=group), args.iters)
        report("reduce_scatter", nb, int(nb * frac), v)
        # axis switch + LayerNorm of a [A/P, B, 128] shard (the pair tensor around the triangle modules)
        C = 128
        rows_total = n // C
        if rows_total >= P * P and rows_total % (P * P) == 0:
            B = P
            while B * B * 4 <= rows_total * P and (rows_total * P) % (B * 2) == 0 and B * 2 <= 8192:
                B *= 2
            A = rows_total * P // B
            if A % P == 0 and B % P == 0 and (A // P) * B == rows_total:
                shard = x.view(A // P, B, C)
                gamma = torch.ones(C, device=dev, dtype=torch.bfloat16)
                beta = torch.zeros(C, device=dev, dtype=torch.bfloat16)
                v = {"push": timed(lambda: h.a2a_layer_norm(None, shard, 0, A, B, C, gamma, beta, 1e-5), args.iters)}
                symm.PUSH = False
                v["publish_pull"] = timed(lambda: h.a2a_layer_norm(None, shard, 0, A, B, C, gamma, beta, 1e-5), args.iters)
                symm.PUSH = True

                def nccl_form():
                    r = torch.empty_like(send)
                    dist.all_to_all_single(r, send, group=group)
                    return torch.nn.functional.layer_norm(r.view(-1, C), (C,), gamma, beta, 1e-5)
                v["nccl_plus_layernorm"] = timed(nccl_form, args.iters)
                report("axis_switch_layernorm", nb, int(nb * frac), v)
    from fastfold_b200.ops import _lib
    st = _lib.read_status()
    if core.get_rank() == 0:
        print(json.dumps({"device_status": st[0], "rows": len(rows)}), flush=True)
    core.shutdown()


if __name__ == "__main__":
    main()
