"""Training checkpoints: model (OpenFold-named ``state_dict``), optimizer state, schedule, step counter and RNG state.

Rank 0 writes atomically (temporary file + rename); every rank loads.  The model part uses the OpenFold /
AlphaFold-archive naming (``utils.inject_fastnn.extract_fastnn``), so a checkpoint can also be loaded into the
un-injected model or exported to an ``.npz`` archive.  The reference saves ``torch.save(engine.model)`` only and has
no load path (train.py:253-254).
"""
import os
import random

import numpy as np
import torch

from ..parallel import core


def save_checkpoint(path, model, trainer, scheduler, epoch):
    from ..utils.inject_fastnn import extract_fastnn
    core.barrier()
    if core.get_rank() == 0:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        state = {
            "model": {k: v.detach().float().cpu() for k, v in extract_fastnn(model).items()},
            "trainer": {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in trainer.state_dict().items()},
            "scheduler": scheduler.state_dict() if scheduler is not None else None,
            "epoch": epoch,
            "rng": {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state(),
                    "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None},
        }
        tmp = path + ".tmp"
        torch.save(state, tmp)
        os.replace(tmp, path)
    core.barrier()


def load_checkpoint(path, model, trainer, scheduler, device):
    state = torch.load(path, map_location="cpu", weights_only=False)
    if state.get("trainer") is not None and trainer is not None:
        if state["trainer"]["names"] != trainer.names:
            raise RuntimeError("checkpoint was written for a different parameter list")
        trainer.load_state_dict({k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in state["trainer"].items()})
    else:
        from ..utils.inject_fastnn import inject_fastnn  # noqa: F401  (the model arrives already injected)
        _load_openfold_named(model, state["model"])
    if scheduler is not None and state.get("scheduler"):
        scheduler.load_state_dict(state["scheduler"])
    rng = state.get("rng")
    if rng:
        random.setstate(rng["python"])
        np.random.set_state(rng["numpy"])
        torch.set_rng_state(rng["torch"])
        if rng.get("cuda") is not None and torch.cuda.is_available() and len(rng["cuda"]) == torch.cuda.device_count():
            torch.cuda.set_rng_state_all(rng["cuda"])
    return int(state.get("epoch", 0))


def _load_openfold_named(model, sd):
    """Loads OpenFold-named tensors into an injected model by building an un-injected twin, loading, re-injecting."""
    from ..models.hub import AlphaFold
    from ..utils.inject_fastnn import copy_evoformer_block, copy_extra_msa_block, copy_template_pair_block, _copy_linear
    import copy
    twin = AlphaFold(_config_of(model))
    twin.load_state_dict(sd, strict=True)
    with torch.no_grad():
        for fb, ob in zip(model.evoformer.blocks, twin.evoformer.blocks):
            copy_evoformer_block(fb, ob)
        _copy_linear(model.evoformer.linear, twin.evoformer.linear)
        for fb, ob in zip(model.extra_msa_stack.blocks, twin.extra_msa_stack.blocks):
            copy_extra_msa_block(fb, ob)
        tps = getattr(getattr(model, "template_embedder", None), "template_pair_stack", None)
        skip = ("evoformer.", "extra_msa_stack.")
        if tps is not None and hasattr(tps.blocks[0], "TriangleAttentionStartingNode"):
            # injected template stack: fast parameter names, filled through the same copy helpers as ``inject_fastnn``
            otps = twin.template_embedder.template_pair_stack
            for fb, ob in zip(tps.blocks, otps.blocks):
                copy_template_pair_block(fb, ob)
            tps.layer_norm.load_state_dict(otps.layer_norm.state_dict())
            skip = skip + ("template_embedder.template_pair_stack.",)
        own = model.state_dict()
        for k, v in twin.state_dict().items():
            if not k.startswith(skip):
                if k not in own:
                    raise KeyError("checkpoint tensor %r has no counterpart in the model" % k)
                own[k].copy_(v)


def _config_of(model):
    from ..config import ConfigDict
    return ConfigDict({"globals": model.globals, "model": model.config})
