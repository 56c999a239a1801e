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


def load_model(model_name="model_1", param_path=None, chunk_size=None, inplace=False, overrides=None, seed=0, device=None, bf16=True,
               shard_pair=False):
    """Builds the model a prediction runs: ``AlphaFold(model_config(model_name))`` (+ an AlphaFold parameter archive when
    ``param_path`` exists), fast trunk swapped in, eval mode, on ``device`` in bf16 (GPU) or fp32 (CPU).  ``init_dap`` must
    have been called.  Sets the process-wide chunk size, as the reference's inference.py:129-145 does."""
    from ..config import model_config
    from ..models.fastnn import set_chunk_size
    from ..models.hub import AlphaFold
    from ..utils.import_weights import import_jax_weights_
    from ..utils.inject_fastnn import inject_fastnn
    cuda = torch.cuda.is_available()
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    config = model_config(model_name)
    config.globals.chunk_size = chunk_size
    config.globals.inplace = bool(inplace)
    config.globals.shard_pair = bool(shard_pair)      # long sequences under DAP: the pair tensor stays a row shard end to end
    for k, v in (overrides or {}).items():
        node = config
        parts = k.split(".")
        for p in parts[:-1]:
            node = node[p]
        node[parts[-1]] = v
    torch.manual_seed(seed)
    model = AlphaFold(config)
    if param_path and os.path.exists(param_path):
        import_jax_weights_(model, param_path, version=model_name)
    model = inject_fastnn(model).eval()
    model = model.to(device=device, dtype=torch.bfloat16 if (device.type == "cuda" and bf16) else torch.float32)
    set_chunk_size(config.globals.chunk_size)
    return model


def predict(model, batch, module_times=None):
    """One prediction: ``batch`` (features with the recycling dimension last; host or device tensors / arrays) is moved
    to the model's device, the model runs without gradients, and the outputs come back as device tensors together with
    the device-timed seconds of the model call.  Raises on every rank if a kernel reported a failed wait.
    ``module_times``: a dict that receives ``{"table": str, "summary": dict}`` - device time per top-level module of the
    model (max over ranks, ``utils.tracing.ModuleTimer``); the hooks add a few event records per module call."""
    device = next(model.parameters()).device
    cuda = device.type == "cuda"
    if cuda:
        # size the symmetric heap (created at the first collective) from the shapes, so that every axis switch and
        # gather of this call runs on the package's own NVLink kernels instead of falling back to NCCL
        from ..parallel import core, symm
        P = core.get_dap_size()
        if P > 1:
            symm.request_message_bytes(symm.ring_bytes_for(int(batch["aatype"].shape[0]), int(batch["msa_feat"].shape[0]),
                                                           int(batch["extra_msa"].shape[0]) if "extra_msa" in batch else 0, P))
    batch = {k: torch.as_tensor(v).to(device, non_blocking=True) for k, v in batch.items()}
    with torch.no_grad():
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        timer = None
        if module_times is not None:
            from ..utils import tracing
            timer = tracing.ModuleTimer(model, max_depth=1)
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
        if timer is not None:
            module_times["summary"] = timer.summary(by="path")
            module_times["table"] = timer.table(by="path")
            timer.remove()
    return out, seconds


def _worker(rank, world, port, batch, opts, queue):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from ..parallel import init_dap, shutdown
    init_dap()
    cuda = torch.cuda.is_available()
    model = load_model(opts["model_name"], opts.get("param_path"), opts.get("chunk_size"), opts.get("inplace", False), opts.get("overrides"),
                       opts.get("seed", 0), bf16=opts.get("bf16", True), shard_pair=opts.get("shard_pair", False))
    if cuda:
        torch.cuda.synchronize()
    times = {} if opts.get("module_times") else None
    out, seconds = predict(model, batch, module_times=times)
    peak = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0
    if rank == 0:
        res = {k: v.float().cpu().numpy() for k, v in out.items() if isinstance(v, torch.Tensor)}
        res["_seconds"] = seconds
        res["_peak_gib"] = peak
        if times:
            res["_module_times"] = times["table"]
        queue.put(res)
    from ..parallel import barrier
    barrier()
    shutdown()


def run_inference(batch, gpus=1, model_name="model_1", param_path=None, chunk_size=None, inplace=False, seed=0, overrides=None, port=None,
                  shard_pair=False, module_times=False):
    """Runs the model on ``batch`` (features with the recycling dimension last) over ``gpus`` DAP ranks; returns numpy outputs."""
    import torch.multiprocessing as mp
    opts = {"model_name": model_name, "param_path": param_path, "chunk_size": chunk_size, "inplace": inplace, "seed": seed, "overrides": overrides,
            "shard_pair": shard_pair, "module_times": module_times}
    batch = {k: (v.cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in batch.items()}
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    queue = manager.Queue()
    port = port or int(os.environ.get("MASTER_PORT", 18417))
    mp.spawn(_worker, args=(gpus, port, batch, opts, queue), nprocs=gpus, join=True)
    return queue.get()
