"""Stand-in for ``colossalai.utils``: the one query the reference's data modules import."""
import torch.distributed as dist


def is_using_ddp():
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
