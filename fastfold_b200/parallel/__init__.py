"""Dynamic Axial Parallelism runtime: mesh bootstrap, collectives, fused P2P kernels, DP gradient reduction."""
from .core import (init_dap, shutdown, mesh, get_dap_size, get_dap_rank, get_dap_group, get_dp_size, get_dp_rank,
                   get_dp_group, ensure_divisibility, barrier)
from .comm import (_reduce, _split, _gather, copy, scatter, reduce, gather, col_to_row, row_to_col)

__all__ = [
    "init_dap", "shutdown", "mesh", "get_dap_size", "get_dap_rank", "get_dap_group", "get_dp_size", "get_dp_rank",
    "get_dp_group", "ensure_divisibility", "barrier", "_reduce", "_split", "_gather", "copy", "scatter", "reduce",
    "gather", "col_to_row", "row_to_col",
]
