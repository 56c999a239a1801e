"""Process bootstrap and the DAP x DP device mesh.

``init_dap(size)`` is the one call a program makes instead of
``torch.distributed.init_process_group``: it creates the world group (NCCL on
GPUs, Gloo on CPU), and splits the world into *Dynamic Axial Parallelism*
groups of ``size`` consecutive ranks (NVLink neighbours on one box) and the
orthogonal data-parallel groups.  With no launcher environment it sets up a
single-process world, exactly like the reference, whose ``init_dap`` delegates
to ``colossalai.launch_from_torch`` (fastfold/distributed/core.py:17-40); no
ColossalAI is involved here.

rank = dp_rank * dap_size + dap_rank.
"""
import datetime
import os
import warnings

import torch
import torch.distributed as dist


class _Mesh:
    def __init__(self):
        self.reset()

    def reset(self):
        self.initialized = False
        self.world_size = 1
        self.rank = 0
        self.local_rank = 0
        self.dap_size = 1
        self.dap_rank = 0
        self.dp_size = 1
        self.dp_rank = 0
        self.dap_group = None
        self.dp_group = None
        self.dap_ranks = [0]
        self.owns_pg = False


_MESH = _Mesh()


def ensure_divisibility(numerator, denominator):
    assert numerator % denominator == 0, "{} is not divisible by {}".format(numerator, denominator)


def set_missing_distributed_environ(key, value):
    if key not in os.environ:
        os.environ[str(key)] = str(value)


def init_dap(tensor_model_parallel_size_=None, *, backend=None, timeout_s=None, adopt_existing=False):
    """Initialises the process group and the DAP/DP mesh.

    ``tensor_model_parallel_size_`` is the DAP group size; ``None`` means the
    whole world (``WORLD_SIZE`` or 1).  Refuses to run when
    ``torch.distributed`` was already initialised by someone else (pass
    ``adopt_existing=True`` to build the mesh on the existing world group).
    ``timeout_s`` bounds every collective so that a rank that never joins ends
    the others with an error instead of a hang.
    """
    m = _MESH
    world = int(os.environ.get("WORLD_SIZE", 1))
    if tensor_model_parallel_size_ is None:
        tensor_model_parallel_size_ = world
    size = int(tensor_model_parallel_size_)
    if m.initialized:
        if m.dap_size == size:
            return m
        raise RuntimeError("init_dap was already called with DAP size %d" % m.dap_size)
    if dist.is_initialized() and not adopt_existing:
        raise RuntimeError("use fastfold.distributed.init_dap instead of torch.distributed.init_process_group!")

    set_missing_distributed_environ("WORLD_SIZE", 1)
    set_missing_distributed_environ("RANK", 0)
    set_missing_distributed_environ("LOCAL_RANK", 0)
    set_missing_distributed_environ("MASTER_ADDR", "127.0.0.1")
    set_missing_distributed_environ("MASTER_PORT", 18417)
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    ensure_divisibility(world, size)
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local % torch.cuda.device_count())
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if use_cuda else "gloo"
        kw = {}
        if timeout_s is not None:
            kw["timeout"] = datetime.timedelta(seconds=float(timeout_s))
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
        m.owns_pg = True
    m.world_size, m.rank, m.local_rank = world, rank, local
    m.dap_size = size
    m.dp_size = world // size
    m.dp_rank, m.dap_rank = divmod(rank, size)
    m.dap_ranks = list(range(m.dp_rank * size, (m.dp_rank + 1) * size))
    m.dap_group = None
    m.dp_group = None
    if world > 1:
        if size == world:
            m.dap_group = dist.group.WORLD
        elif size > 1:
            for d in range(m.dp_size):
                ranks = list(range(d * size, (d + 1) * size))
                g = dist.new_group(ranks)
                if d == m.dp_rank:
                    m.dap_group = g
        if m.dp_size == world:
            m.dp_group = dist.group.WORLD
        elif m.dp_size > 1:
            for t in range(size):
                ranks = list(range(t, world, size))
                g = dist.new_group(ranks)
                if t == m.dap_rank:
                    m.dp_group = g
    m.initialized = True
    return m


def shutdown():
    """Destroys the process group created by ``init_dap`` (tests, repeated launches)."""
    m = _MESH
    try:
        from . import symm
        symm.release_all()
    except Exception:
        pass
    if m.owns_pg and dist.is_initialized():
        dist.destroy_process_group()
    m.reset()


def mesh():
    return _MESH


def get_dap_size():
    return _MESH.dap_size


def get_dap_rank():
    return _MESH.dap_rank


def get_dap_group():
    return _MESH.dap_group


def get_dp_size():
    return _MESH.dp_size


def get_dp_rank():
    return _MESH.dp_rank


def get_dp_group():
    return _MESH.dp_group


def get_world_size():
    return _MESH.world_size


def get_rank():
    return _MESH.rank


def barrier():
    if dist.is_initialized() and _MESH.world_size > 1:
        dist.barrier()


def warn_once(msg, _seen=set()):
    if msg not in _seen:
        _seen.add(msg)
        warnings.warn(msg)
