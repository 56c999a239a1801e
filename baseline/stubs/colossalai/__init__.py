"""Minimal stand-in for the ColossalAI runtime that the reference imports.

Only the process bootstrap and the parallel-context queries that
``fastfold/distributed/core.py`` and ``fastfold/distributed/comm*.py`` use are
provided, implemented directly on ``torch.distributed``.  It exists so that the
unmodified reference package can be imported and benchmarked on a machine
where ColossalAI is not installed; nothing in ``fastfold_b200`` imports it.
"""
import os

import torch
import torch.distributed as dist

from . import logging  # noqa: F401
from .context.parallel_mode import ParallelMode
from .core import global_context


def launch_from_torch(config=None, backend=None, seed=1024, verbose=False, **_):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda:
        torch.cuda.set_device(local)
    if not dist.is_initialized():
        kw = {}
        if use_cuda:
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    tp = 1
    if config and "parallel" in config:
        tp = int(config["parallel"].get("tensor", {}).get("size", 1))
    global_context._build(rank, world, local, tp)
    torch.manual_seed(seed)


launch = launch_from_torch
