#!/usr/bin/env python
"""Full-model inference on synthetic features (no databases needed).

    python demo.py --gpus 2 --n_res 512 --chunk_size 64 --inplace

Same flags as the reference's demo.py:143-153, plus the MSA sizes.  Prints the device-timed latency and peak memory.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--n_res", type=int, default=256)
    ap.add_argument("--n_seq", type=int, default=128)
    ap.add_argument("--n_extra", type=int, default=1024)
    ap.add_argument("--n_templ", type=int, default=0)
    ap.add_argument("--recycles", type=int, default=3)
    ap.add_argument("--model_name", type=str, default="model_3")
    ap.add_argument("--param_path", type=str, default=None)
    ap.add_argument("--chunk_size", type=int, default=None)
    ap.add_argument("--inplace", default=False, action="store_true")
    ap.add_argument("--shard_pair", default=False, action="store_true",
                    help="with --gpus > 1: keep the pair tensor row-sharded from the embedders to the heads (long sequences)")
    ap.add_argument("--output", type=str, default=None, help="write the prediction as PDB")
    args = ap.parse_args()
    from fastfold_b200.common import protein
    from fastfold_b200.runtime.inference import run_inference
    from fastfold_b200.utils.synthetic import random_features
    batch = random_features(args.n_res, args.n_seq, args.n_extra, n_templ=args.n_templ, n_recycle=args.recycles, seed=0)
    out = run_inference(batch, gpus=args.gpus, model_name=args.model_name, param_path=args.param_path, chunk_size=args.chunk_size,
                        inplace=args.inplace, shard_pair=args.shard_pair)
    print("Inference time: %.3f s   peak memory: %.2f GiB   mean pLDDT: %.1f" % (out["_seconds"], out["_peak_gib"], float(out["plddt"].mean())))
    if args.output:
        feats = {"aatype": batch["aatype"][..., 0].numpy(), "residue_index": batch["residue_index"][..., 0].numpy()}
        b = out["plddt"][:, None] * out["final_atom_mask"]
        with open(args.output, "w") as fh:
            fh.write(protein.to_pdb(protein.from_prediction(feats, out, b_factors=b)))


if __name__ == "__main__":
    main()
