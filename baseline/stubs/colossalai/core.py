"""``colossalai.core.global_context`` stand-in: TENSOR (=DAP) and DATA groups."""
import torch.distributed as dist

from .context.parallel_mode import ParallelMode


class _GlobalContext:
    def __init__(self):
        self._rank = 0
        self._world = 1
        self._local = 0
        self._tp = 1
        self._groups = {}
        self._local_ranks = {ParallelMode.GLOBAL: 0, ParallelMode.TENSOR: 0, ParallelMode.DATA: 0}

    def _build(self, rank, world, local, tp):
        assert world % tp == 0, "world size must be divisible by the tensor-parallel size"
        self._rank, self._world, self._local, self._tp = rank, world, local, tp
        dp = world // tp
        self._groups[ParallelMode.GLOBAL] = dist.group.WORLD
        self._local_ranks[ParallelMode.GLOBAL] = rank
        if tp == world:
            self._groups[ParallelMode.TENSOR] = dist.group.WORLD
            self._local_ranks[ParallelMode.TENSOR] = rank
        else:
            for d in range(dp):
                ranks = list(range(d * tp, (d + 1) * tp))
                g = dist.new_group(ranks) if tp > 1 else None
                if rank in ranks:
                    self._groups[ParallelMode.TENSOR] = g
                    self._local_ranks[ParallelMode.TENSOR] = ranks.index(rank)
        if dp == world:
            self._groups[ParallelMode.DATA] = dist.group.WORLD
            self._local_ranks[ParallelMode.DATA] = rank
        else:
            for t in range(tp):
                ranks = list(range(t, world, tp))
                g = dist.new_group(ranks) if dp > 1 else None
                if rank in ranks:
                    self._groups[ParallelMode.DATA] = g
                    self._local_ranks[ParallelMode.DATA] = ranks.index(rank)

    def get_world_size(self, mode=ParallelMode.GLOBAL):
        if mode == ParallelMode.TENSOR:
            return self._tp
        if mode == ParallelMode.DATA:
            return self._world // self._tp
        return self._world

    def get_group(self, mode=ParallelMode.GLOBAL):
        return self._groups.get(mode)

    def get_local_rank(self, mode=ParallelMode.GLOBAL):
        return self._local_ranks.get(mode, 0)

    def get_global_rank(self):
        return self._rank

    def is_initialized(self, mode):
        return mode in self._groups


global_context = _GlobalContext()
