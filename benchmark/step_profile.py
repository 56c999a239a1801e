"""Kernel-level breakdown of the headline training step (Evoformer stack, bf16, CUDA-graph replay).

    python benchmark/step_profile.py [--blocks 2] [--msa 128] [--res 256] [--rows 45] [--eager]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 benchmark/step_profile.py ...

Builds the same model / inputs / trainer as ``bench.py`` with ``--blocks`` Evoformer blocks, warms the step up, and
prints the PyTorch profiler's table of CUDA kernels for ONE step, sorted by device time.  The figures are kernel
durations seen by the profiler (the timed ``bench.py`` number is taken without it).  Under ``torch.distributed.run`` the
P ranks form one DAP group and rank 0 prints its table.  With programmatic dependent launch a kernel's duration includes
the time it waits for its predecessor, so set ``FFB_PDL=0`` for per-kernel durations that add up.  ``--summary`` prints
launch counts and time per kernel family instead of the raw table.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402
from fastfold_b200.models.fastnn import EvoformerStack  # noqa: E402
from fastfold_b200.runtime import FlatAdamTrainer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, default=2)
    ap.add_argument("--msa", type=int, default=128)
    ap.add_argument("--res", type=int, default=256)
    ap.add_argument("--rows", type=int, default=45)
    ap.add_argument("--eager", action="store_true", help="profile eager launches instead of the captured graph")
    ap.add_argument("--summary", action="store_true", help="launch count and device time per kernel family")
    args = ap.parse_args()
    from torch.profiler import ProfilerActivity, profile
    from fastfold_b200.parallel import core, init_dap
    init_dap(int(os.environ.get("WORLD_SIZE", 1)))
    dev = torch.device("cuda", torch.cuda.current_device())
    model = EvoformerStack(256, 128, 384, args.blocks, blocks_per_ckpt=1)
    bench.randomize_zero_weights(torch, model, 99)
    model = model.to(dev, torch.bfloat16).train()
    inp = [t.to(dev) for t in bench.make_inputs(torch, args.msa, args.res, dev, torch.bfloat16, 7)]

    def loss_fn(mod, m, z, mm, pm, tm, tz, ts):
        return bench.mse_loss(mod(m, z, mm, pm, None), tm, tz, ts)

    trainer = FlatAdamTrainer(model, loss_fn, use_graph=not args.eager)
    for _ in range(4):
        trainer.step(*inp)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        trainer.step(*inp)
        torch.cuda.synchronize()
    if core.get_rank() == 0:
        if args.summary:
            print(summary(prof.key_averages()))
        else:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.rows, max_name_column_width=90))
    core.shutdown()


FAMILIES = [("gemm_bf16_kernel", "tcgen05 GEMM"), ("attn_fwd", "attention forward"), ("attn_bwd", "attention backward"),
            ("symm_", "NVLink collectives (own kernels)"), ("nccl", "NCCL"), ("ln_", "LayerNorm forward / backward"), ("ltb_", "LayerNorm forward / backward"),
            ("colsum", "bias-gradient column sums"), ("glu_", "triangle gating (channel-major)"), ("adam", "Adam"),
            ("ffb::", "other own kernels (epilogue-less elementwise, softmax, masks)"), ("at::native", "PyTorch elementwise / reductions / copies"),
            ("Memcpy", "memcpy / memset"), ("memcpy", "memcpy / memset"), ("Memset", "memcpy / memset"),
            ("cutlass", "library GEMM (narrow shapes)"), ("nvjet", "library GEMM (narrow shapes)"), ("cublas", "library GEMM (narrow shapes)")]


def summary(events):
    fam = {}
    for e in events:
        t = getattr(e, "self_device_time_total", 0) or getattr(e, "self_cuda_time_total", 0)
        if not t:
            continue
        name = next((label for key, label in FAMILIES if key in e.key), "other")
        n, tot = fam.get(name, (0, 0.0))
        fam[name] = (n + e.count, tot + t)
    total = sum(t for _, t in fam.values())
    calls = sum(n for n, _ in fam.values())
    lines = ["| kernel family | launches | device time | average | share |", "|---|---|---|---|---|"]
    for name, (n, t) in sorted(fam.items(), key=lambda kv: -kv[1][1]):
        lines.append("| %s | %d | %.2f ms | %.1f us | %.1f %% |" % (name, n, t / 1e3, t / n, 100 * t / total))
    lines.append("| all | %d | %.2f ms | %.1f us | 100 %% |" % (calls, total / 1e3, total / calls))
    return "\n".join(lines)


if __name__ == "__main__":
    main()
