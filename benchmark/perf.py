#!/usr/bin/env python
"""Stand-alone Evoformer forward / backward timing (flags of the reference's benchmark/perf.py:13-35).

    python benchmark/perf.py --msa-length 128 --res-length 256
    torchrun --nproc_per_node=2 benchmark/perf.py --msa-length 128 --res-length 256 --dap-size 2

CUDA-event timing with a barrier + synchronise before every trial; prints mean forward and backward milliseconds
per layer (max over ranks).  bf16 at every DAP size (the reference falls back to fp16 for DAP > 1).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    p = argparse.ArgumentParser(description="Evoformer stand-alone perf benchmark")
    p.add_argument("--dap-size", default=1, type=int)
    p.add_argument("--msa-length", default=132, type=int)
    p.add_argument("--res-length", default=256, type=int)
    p.add_argument("--trials", default=50, type=int)
    p.add_argument("--warmup-trials", default=5, type=int)
    p.add_argument("--layers", default=12, type=int)
    p.add_argument("--cm", default=256, type=int)
    p.add_argument("--cz", default=128, type=int)
    p.add_argument("--heads", default=8, type=int)
    p.add_argument("--openfold", action="store_true", help="time the OpenFold-layout reference modules instead of the fast ones")
    p.add_argument("--fwd", action="store_true", help="forward only")
    p.add_argument("--prof", action="store_true", help="record a torch.profiler trace under ./log/fastfold")
    p.add_argument("--nvtx", action="store_true", help="one NVTX range per sub-module call (for a timeline viewer)")
    p.add_argument("--module-times", action="store_true",
                   help="after the run, print device time per module class over the timed trials (forward only; max over ranks)")
    args = p.parse_args()
    from fastfold_b200.parallel import init_dap, barrier, core
    from fastfold_b200.models.fastnn import Evoformer
    init_dap(args.dap_size)
    if not torch.cuda.is_available():
        raise NotImplementedError("Running on CPU is not supported")
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(42)
    layers = []
    for i in range(args.layers):
        if args.openfold:
            from fastfold_b200.models.nn.evoformer import EvoformerBlock
            layer = EvoformerBlock(args.cm, args.cz, args.cm // 8, 32, args.cz, args.cz // 4, 8, 4, 4, 0.15, 0.25, 1e9, 1e-10)
        else:
            layer = Evoformer(c_m=args.cm, c_z=args.cz, first_block=(i == 0), last_block=(i == args.layers - 1))
        layers.append(layer.to(dev, torch.bfloat16))
    m = torch.randn(args.msa_length, args.res_length, args.cm, dtype=torch.bfloat16, device=dev, requires_grad=True)
    z = torch.randn(args.res_length, args.res_length, args.cz, dtype=torch.bfloat16, device=dev, requires_grad=True)
    mm = torch.ones(args.msa_length, args.res_length, dtype=torch.bfloat16, device=dev)
    pm = torch.ones(args.res_length, args.res_length, dtype=torch.bfloat16, device=dev)
    gz = torch.randn_like(z)
    prof = None
    if args.prof:
        prof = torch.profiler.profile(schedule=torch.profiler.schedule(wait=1, warmup=args.warmup_trials, active=args.trials, repeat=1),
                                      on_trace_ready=torch.profiler.tensorboard_trace_handler("./log/fastfold"))
        prof.start()
    from fastfold_b200.utils import tracing
    stack = torch.nn.ModuleList(layers)
    ranges = tracing.annotate(stack, max_depth=3) if args.nvtx else None
    timer = None
    f_ms = b_ms = 0.0
    for t in range(args.trials + args.warmup_trials):
        if args.module_times and t == args.warmup_trials:
            timer = tracing.ModuleTimer(stack, max_depth=3)
        barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        x = (m, z)
        for layer in layers:
            x = layer(x[0], x[1], mm, pm)
        e1.record()
        if not args.fwd:
            x[1].backward(gz)
        e2.record()
        torch.cuda.synchronize()
        if t >= args.warmup_trials:
            f_ms += e0.elapsed_time(e1)
            b_ms += e1.elapsed_time(e2)
        if prof:
            prof.step()
    if prof:
        prof.stop()
    if ranges:
        ranges.remove()
    if timer:
        table = timer.table(by="class")
        timer.remove()
        if core.get_rank() == 0:
            print(table)
    vals = torch.tensor([f_ms, b_ms], device=dev, dtype=torch.float64) / (args.trials * args.layers)
    if core.get_world_size() > 1:
        torch.distributed.all_reduce(vals, op=torch.distributed.ReduceOp.MAX)
    if core.get_rank() == 0:
        print("[ MSA Attn ] Input: %4d, %4d, %4d, (%4d %4d) Fwd Time / Layer: %.3f ms Bwd Time / Layer: %.3f ms" % (
            1, args.msa_length, args.res_length, args.cm, args.cz, vals[0].item(), vals[1].item()))
    core.shutdown()


if __name__ == "__main__":
    main()
