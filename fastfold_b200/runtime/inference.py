"""Multi-GPU inference driver shared by ``inference.py`` and ``demo.py``.

One process per GPU (``torch.multiprocessing.spawn``); every process calls ``init_dap`` (the DAP group spans all
``--gpus``), builds the model, optionally imports an AlphaFold parameter archive, swaps in the fast trunk, and runs
the full feature dict; rank 0 returns the outputs to the parent through a queue.  The model call is timed on the
device (CUDA events between synchronisations), unlike the reference's ``perf_counter`` without a synchronise
(inference.py:150-152).
"""
import os
import time

import numpy as np
import torch


def _worker(rank, world, port, batch, opts, queue):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from ..config import model_config
    from ..models.fastnn import set_chunk_size
    from ..models.hub import AlphaFold
    from ..parallel import init_dap, shutdown
    from ..utils.import_weights import import_jax_weights_
    from ..utils.inject_fastnn import inject_fastnn
    init_dap()
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    config = model_config(opts["model_name"])
    config.globals.chunk_size = opts.get("chunk_size")
    config.globals.inplace = bool(opts.get("inplace", False))
    for k, v in (opts.get("overrides") or {}).items():
        node = config
        parts = k.split(".")
        for p in parts[:-1]:
            node = node[p]
        node[parts[-1]] = v
    torch.manual_seed(opts.get("seed", 0))
    model = AlphaFold(config)
    if opts.get("param_path") and os.path.exists(opts["param_path"]):
        import_jax_weights_(model, opts["param_path"], version=opts["model_name"])
    model = inject_fastnn(model).eval()
    model = model.to(device=device, dtype=torch.bfloat16 if (cuda and opts.get("bf16", True)) else torch.float32)
    set_chunk_size(config.globals.chunk_size)
    batch = {k: torch.as_tensor(v).to(device) for k, v in batch.items()}
    with torch.no_grad():
        if cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        out = model(batch)
        if cuda:
            e1.record()
            torch.cuda.synchronize()
            seconds = e0.elapsed_time(e1) / 1e3
            from .trainer import check_device_status
            check_device_status()        # a kernel that gave up on a wait leaves unwritten outputs: fail on every rank
        else:
            seconds = time.perf_counter() - t0
    peak = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0
    if rank == 0:
        res = {k: v.float().cpu().numpy() for k, v in out.items() if isinstance(v, torch.Tensor)}
        res["_seconds"] = seconds
        res["_peak_gib"] = peak
        queue.put(res)
    from ..parallel import barrier
    barrier()
    shutdown()


def run_inference(batch, gpus=1, model_name="model_1", param_path=None, chunk_size=None, inplace=False, seed=0, overrides=None, port=None):
    """Runs the model on ``batch`` (features with the recycling dimension last) over ``gpus`` DAP ranks; returns numpy outputs."""
    import torch.multiprocessing as mp
    opts = {"model_name": model_name, "param_path": param_path, "chunk_size": chunk_size, "inplace": inplace, "seed": seed, "overrides": overrides}
    batch = {k: (v.cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in batch.items()}
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    queue = manager.Queue()
    port = port or int(os.environ.get("MASTER_PORT", 18417))
    mp.spawn(_worker, args=(gpus, port, batch, opts, queue), nprocs=gpus, join=True)
    return queue.get()
