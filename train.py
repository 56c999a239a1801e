#!/usr/bin/env python
"""Training entry point.

    torchrun --nproc_per_node=8 train.py --dap_size 2 --config_preset initial_training --synthetic --max_steps 100 \
        --save_ckpt_path ./ckpt --save_ckpt_interval 50

Flags follow the reference's train.py:37-159 (``--from_torch --dap_size --config_preset --seed --max_epochs
--log_interval --log_path --save_ckpt_path --save_ckpt_interval`` + data paths).  World = DAP x DP: ranks of one DAP
group share a sample, different groups get different samples.  Differences on purpose: the optimizer, gradient
reduction and (optionally) CUDA-graph replay come from ``FlatAdamTrainer`` instead of ColossalAI's engine; a
checkpoint holds model, optimizer moments, scheduler, step and RNG state and ``--resume`` continues from it (the
reference pickles the bare module and cannot resume, train.py:253-254); the schedule advances per step.
``--synthetic`` trains on generated features (no databases); otherwise ``--train_data_dir`` must hold ``<tag>.pdb``
structures with optional alignments under ``--train_alignment_dir/<tag>``.
"""
import argparse
import logging
import os
import random
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--from_torch", default=False, action="store_true")
    p.add_argument("--dap_size", type=int, default=1)
    p.add_argument("--config_preset", type=str, default="initial_training")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--max_epochs", type=int, default=10000)
    p.add_argument("--max_steps", type=int, default=None)
    p.add_argument("--train_epoch_len", type=int, default=64)
    p.add_argument("--log_interval", type=int, default=1)
    p.add_argument("--log_path", type=str, default="train_log")
    p.add_argument("--save_ckpt_path", type=str, default=None)
    p.add_argument("--save_ckpt_interval", type=int, default=1)
    p.add_argument("--resume", type=str, default=None)
    p.add_argument("--synthetic", default=False, action="store_true")
    p.add_argument("--train_data_dir", type=str, default=None)
    p.add_argument("--train_alignment_dir", type=str, default=None)
    p.add_argument("--val_data_dir", type=str, default=None)
    p.add_argument("--val_alignment_dir", type=str, default=None)
    p.add_argument("--template_mmcif_dir", type=str, default=None)
    p.add_argument("--train_chain_data_cache_path", type=str, default=None, help="chain-level cache (resolution, cluster size, sequence) "
                   "for the stochastic training filters")
    p.add_argument("--distillation_data_dir", type=str, default=None, help="directory of self-distillation PDB files")
    p.add_argument("--distillation_alignment_dir", type=str, default=None)
    p.add_argument("--distillation_chain_data_cache_path", type=str, default=None)
    p.add_argument("--kalign_binary_path", type=str, default="/usr/bin/kalign")
    p.add_argument("--train_filter_path", type=str, default=None, help="text file with the names of the training examples to use, one per line")
    p.add_argument("--distillation_filter_path", type=str, default=None, help="as --train_filter_path, for the distillation set")
    p.add_argument("--obsolete_pdbs_file_path", type=str, default=None)
    p.add_argument("--template_release_dates_cache_path", type=str, default=None)
    p.add_argument("--_alignment_index_path", type=str, default=None)
    p.add_argument("--_distillation_structure_index_path", type=str, default=None)
    p.add_argument("--distillation_alignment_index_path", type=str, default=None)
    p.add_argument("--plain_dataset", default=False, action="store_true", help="read --train_data_dir file by file in order "
                   "(no stochastic filtering, no distillation mix, no template search) instead of the filtered mixture dataset")
    p.add_argument("--max_template_date", type=str, default="2021-10-10")
    p.add_argument("--n_res", type=int, default=None, help="(synthetic) crop size; default from the preset")
    p.add_argument("--n_seq", type=int, default=None)
    p.add_argument("--n_extra", type=int, default=None)
    p.add_argument("--blocks", type=int, default=None, help="override the number of Evoformer blocks (debugging)")
    p.add_argument("--recycles", type=int, default=None, help="(synthetic) fixed number of recycling iterations per step instead of a uniform draw")
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--no_graph", default=False, action="store_true", help="run every step eagerly instead of replaying captured CUDA graphs")
    p.add_argument("--val_interval", type=int, default=1, help="epochs between validation passes")
    p.add_argument("--val_epoch_len", type=int, default=2, help="(synthetic) validation samples per pass; 0 disables")
    return p.parse_args()


class _LoaderDataset:
    """``len`` / ``get(epoch, i)`` over an ``OpenFoldDataLoader``: a new pass over the loader (and a re-draw of the
    filtered training mixture) whenever the epoch changes."""

    def __init__(self, loader):
        self.loader, self._it, self._epoch = loader, None, None

    def __len__(self):
        return len(self.loader)

    def get(self, epoch, i):
        if self._it is None or epoch != self._epoch or i == 0:
            if self._epoch is not None and epoch != self._epoch and hasattr(self.loader.dataset, "reroll"):
                self.loader.dataset.reroll()
            self._it, self._epoch = iter(self.loader), epoch
        return dict(next(self._it))


def main():
    args = parse()
    from fastfold_b200.config import model_config
    from fastfold_b200.models.hub import AlphaFold, AlphaFoldLoss, AlphaFoldLRScheduler
    from fastfold_b200.parallel import core, init_dap
    from fastfold_b200.runtime import FlatAdamTrainer
    from fastfold_b200.runtime.trainer import default_replicated_param_filter
    from fastfold_b200.runtime.checkpoint import load_checkpoint, save_checkpoint
    from fastfold_b200.utils.inject_fastnn import inject_fastnn
    from fastfold_b200.utils.tensor_utils import tensor_tree_map
    from fastfold_b200.utils.validation_utils import validation_metrics
    init_dap(args.dap_size)
    rank = core.get_rank()
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    # every rank seeds alike: DAP ranks must draw identical dropout masks
    random.seed(args.seed)
    np.random.seed(args.seed)
    torch.manual_seed(args.seed)
    logging.basicConfig(level=logging.INFO if rank == 0 else logging.WARNING, format="%(asctime)s %(message)s",
                        handlers=[logging.StreamHandler()] + ([logging.FileHandler(args.log_path + ".log")] if rank == 0 else []))
    log = logging.getLogger("train")
    config = model_config(args.config_preset, train=True)
    if args.blocks:
        config.model.evoformer_stack.no_blocks = args.blocks
    for mode_cfg in (config.data.train, config.data.eval):          # the size overrides apply to real data as well
        if args.n_res:
            mode_cfg.crop_size = args.n_res
        if args.n_seq:
            mode_cfg.max_msa_clusters = args.n_seq
        if args.n_extra:
            mode_cfg.max_extra_msa = args.n_extra
    model = inject_fastnn(AlphaFold(config))
    model = model.to(device=device, dtype=torch.bfloat16 if cuda else torch.float32).train()
    criterion = AlphaFoldLoss(config.loss)

    tc = config.data.train
    n_res, n_seq, n_extra = args.n_res or tc.crop_size, args.n_seq or tc.max_msa_clusters, args.n_extra or tc.max_extra_msa
    if args.synthetic or not args.train_data_dir:
        from fastfold_b200.data.data_modules import SyntheticDataset
        dataset = SyntheticDataset(n_res, n_seq, n_extra, n_recycle=config.data.common.max_recycling_iters if args.recycles is None else args.recycles,
                                   length=args.train_epoch_len, seed=args.seed, dp_rank=core.get_dp_rank(), dp_size=core.get_dp_size(),
                                   n_templ=tc.max_templates if config.model.template.enabled else 0, uniform_recycling=args.recycles is None)
    elif args.plain_dataset:
        from fastfold_b200.data.data_modules import StructureDataset
        dataset = StructureDataset(args.train_data_dir, args.train_alignment_dir, config.data, mode="train", seed=args.seed,
                                   dp_rank=core.get_dp_rank(), dp_size=core.get_dp_size())
    else:
        # the reference's data path (train.py:177-203): filtered mixture of PDB and distillation chains, template search
        # with the date / identity filters, per-batch clamping and recycling draws, one share of the epoch per DP replica
        from fastfold_b200.data.data_modules import SetupTrainDataset, TrainDataLoader
        train_set, val_set = SetupTrainDataset(
            config=config.data, template_mmcif_dir=args.template_mmcif_dir, max_template_date=args.max_template_date,
            train_data_dir=args.train_data_dir, train_alignment_dir=args.train_alignment_dir,
            train_chain_data_cache_path=args.train_chain_data_cache_path, distillation_data_dir=args.distillation_data_dir,
            distillation_alignment_dir=args.distillation_alignment_dir,
            distillation_chain_data_cache_path=args.distillation_chain_data_cache_path, val_data_dir=args.val_data_dir,
            val_alignment_dir=args.val_alignment_dir, kalign_binary_path=args.kalign_binary_path, train_mapping_path=args.train_filter_path,
            distillation_mapping_path=args.distillation_filter_path, obsolete_pdbs_file_path=args.obsolete_pdbs_file_path,
            template_release_dates_cache_path=args.template_release_dates_cache_path, train_epoch_len=args.train_epoch_len,
            _alignment_index_path=args._alignment_index_path)
        train_loader, val_loader = TrainDataLoader(config=config.data, train_dataset=train_set, test_dataset=val_set, batch_seed=args.seed)
        dataset = _LoaderDataset(train_loader)
        loader_val_dataset = _LoaderDataset(val_loader) if val_loader is not None else None

    def loss_fn(mod, *tensors):
        batch = dict(zip(loss_fn.keys, tensors))
        out = mod(batch)
        last = tensor_tree_map(lambda t: t[..., -1], batch)
        loss, parts = criterion(out, last, _return_breakdown=True)
        loss_fn.last = (out, last, parts)
        return loss

    # With fixed feature shapes (synthetic data, or cropped + padded training features) the whole step - all recycling
    # iterations, loss, backward with recomputation, gradient reduction, Adam - is captured as one CUDA graph per number
    # of recycling iterations and replayed, exactly what bench.py measures on the Evoformer stack.  A capture that fails
    # (an op that needs a host read) falls back to eager steps.
    use_graph = cuda and not args.no_graph
    trainer = FlatAdamTrainer(model, loss_fn, lr=args.lr, eps=1e-8, use_graph=use_graph,
                              replicated_param_filter=default_replicated_param_filter)
    trainer.graph_fallback = True
    trainer.aux_getter = lambda: getattr(loss_fn, "last", None)
    sched = AlphaFoldLRScheduler(trainer, max_lr=args.lr)
    start_epoch = 0
    if args.resume:
        start_epoch = load_checkpoint(args.resume, model, trainer, sched, device)
        log.info("resumed from %s at step %d (epoch %d)", args.resume, trainer.step_count, start_epoch)

    val_dataset = None
    if args.val_data_dir and not args.synthetic and not args.plain_dataset and args.train_data_dir:
        val_dataset = loader_val_dataset
    elif args.val_data_dir:
        from fastfold_b200.data.data_modules import StructureDataset
        val_dataset = StructureDataset(args.val_data_dir, args.val_alignment_dir, config.data, mode="eval", seed=args.seed,
                                       dp_rank=core.get_dp_rank(), dp_size=core.get_dp_size())
    elif (args.synthetic or not args.train_data_dir) and args.val_epoch_len > 0:      # same condition as the synthetic training set
        from fastfold_b200.data.data_modules import SyntheticDataset
        val_dataset = SyntheticDataset(n_res, n_seq, n_extra, n_recycle=config.data.common.max_recycling_iters, length=args.val_epoch_len,
                                       seed=args.seed + 7919, dp_rank=core.get_dp_rank(), dp_size=core.get_dp_size(), uniform_recycling=False,
                                       n_templ=tc.max_templates if config.model.template.enabled else 0)

    def validate(epoch):
        """Validation pass of the reference's train.py:240-251: eval mode, no gradients, unclamped FAPE, superposition
        metrics; averages over this replica's samples and over the data-parallel replicas."""
        bad = [n for n, p_ in model.named_parameters() if not bool(torch.isfinite(p_).all())]
        if bad:
            raise RuntimeError("non-finite parameters before validation: %s%s" % (", ".join(bad[:5]), " ..." if len(bad) > 5 else ""))
        model.eval()
        sums, count = {}, 0
        with torch.no_grad():
            for i in range(len(val_dataset)):
                batch = val_dataset.get(0, i)
                batch.pop("no_recycling_iters", None)
                batch = {k: v.to(device, non_blocking=True) for k, v in batch.items()}
                batch["use_clamped_fape"] = torch.zeros_like(batch["use_clamped_fape"]) if "use_clamped_fape" in batch else torch.zeros(
                    batch["aatype"].shape[-1], device=device)
                out = model(batch)
                last = tensor_tree_map(lambda t: t[..., -1], batch)
                _, parts = criterion(out, last, _return_breakdown=True)
                parts.update(validation_metrics(out, last, superimposition_metrics=True))
                for k, v in parts.items():
                    sums[k] = sums.get(k, 0.0) + float(v)
                count += 1
        model.train()
        keys = sorted(sums)
        t = torch.tensor([sums[k] for k in keys] + [float(count)], device=device, dtype=torch.float64)
        if core.get_world_size() > 1:
            torch.distributed.all_reduce(t)
        means = {k: float(t[j] / t[-1].clamp(min=1)) for j, k in enumerate(keys)}
        if rank == 0:
            # the sum runs over the whole world; the ranks of one DAP group hold the same samples
            log.info("validation epoch %d (%d samples) | %s", epoch, int(t[-1]) // core.get_dap_size(), " ".join("%s %.4f" % (k, v) for k, v in means.items()))
        return means

    steps_done = 0
    for epoch in range(start_epoch, args.max_epochs):
        t_epoch = time.time()
        epoch_steps = 0
        for i in range(len(dataset)):
            batch = dataset.get(epoch, i)
            n_iter = int(batch.pop("no_recycling_iters", torch.tensor(batch["aatype"].shape[-1] - 1)).reshape(-1)[0]) + 1
            batch = {k: v[..., :n_iter].to(device, non_blocking=True) for k, v in batch.items()}
            loss_fn.keys = sorted(batch)
            t_step = time.time()
            loss = trainer.step(*[batch[k] for k in loss_fn.keys], graph_key=(n_iter,) + tuple(loss_fn.keys))
            loss_fn.last = trainer.aux if trainer.aux is not None else loss_fn.last      # the replayed graph's own output tensors
            sched.step()
            steps_done += 1
            epoch_steps += 1
            if (i + 1) % args.log_interval == 0:
                trainer.check_status()       # every rank: a kernel that gave up on a wait must stop the run, not train on garbage
                if rank == 0:
                    out, last, parts = loss_fn.last
                    with torch.no_grad():
                        metrics = validation_metrics(out, last)
                    loss_value = float(loss)                      # synchronises: the step's kernels have finished
                    log.info("epoch %d step %d (%.3f s) lr %.2e loss %.4f | %s | %s", epoch, trainer.step_count, time.time() - t_step, trainer.lr, loss_value,
                             " ".join("%s %.3f" % (k, float(v)) for k, v in parts.items() if k not in ("loss", "unscaled_loss")),
                             " ".join("%s %.3f" % (k, float(v)) for k, v in metrics.items()))
            if args.max_steps and steps_done >= args.max_steps:
                break
        if device.type == "cuda":
            torch.cuda.synchronize()
        dt = max(time.time() - t_epoch, 1e-9)
        # throughput over the whole job: every data-parallel replica trains one sample per step
        log.info("epoch %d done in %.1f s: %d steps, %.3f samples/s over %d replica(s)%s", epoch, dt, epoch_steps,
                 epoch_steps * core.get_dp_size() / dt, core.get_dp_size(),
                 ", peak device memory %.2f GiB" % (torch.cuda.max_memory_allocated() / 2 ** 30) if device.type == "cuda" else "")
        if val_dataset is not None and (epoch + 1) % args.val_interval == 0:
            validate(epoch)
        if args.save_ckpt_path and (epoch + 1) % args.save_ckpt_interval == 0:
            trainer.check_status()
            save_checkpoint(os.path.join(args.save_ckpt_path, "checkpoint.pt"), model, trainer, sched, epoch + 1)
            if rank == 0:
                log.info("checkpoint written to %s", args.save_ckpt_path)
        if args.max_steps and steps_done >= args.max_steps:
            break
    core.shutdown()


if __name__ == "__main__":
    main()
