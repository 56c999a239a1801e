"""Kernel-level breakdown of the headline training step (Evoformer stack, bf16, CUDA-graph replay).

    python benchmark/step_profile.py [--blocks 2] [--msa 128] [--res 256] [--rows 45] [--eager]

Builds the same model / inputs / trainer as ``bench.py`` with ``--blocks`` Evoformer blocks, warms the step up, and
prints the PyTorch profiler's table of CUDA kernels for ONE step, sorted by device time.  The figures are kernel
durations seen by the profiler (the timed ``bench.py`` number is taken without it).
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
    args = ap.parse_args()
    from torch.profiler import ProfilerActivity, profile
    dev = torch.device("cuda", 0)
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
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.rows, max_name_column_width=90))


if __name__ == "__main__":
    main()
