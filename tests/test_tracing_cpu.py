"""utils/tracing.py on CPU: module selection, timing hooks, max-over-ranks reduction on Gloo ranks."""
import os
import socket
import sys
import time

import torch
import torch.multiprocessing as mp
from torch import nn

from fastfold_b200.utils import tracing

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _Slow(nn.Module):
    def __init__(self, ms):
        super().__init__()
        self.ms = ms
        self.lin = nn.Linear(4, 4)

    def forward(self, x):
        time.sleep(self.ms / 1e3)
        return self.lin(x)


def _model(ms=(5, 10)):
    return nn.Sequential(_Slow(ms[0]), _Slow(ms[1]), nn.ReLU())


def test_select_modules_by_depth_class_and_predicate():
    m = _model()
    assert [p for p, _ in tracing.select_modules(m, max_depth=1)] == ["0", "1", "2"]
    assert [p for p, _ in tracing.select_modules(m, classes=("Linear",))] == ["0.lin", "1.lin"]
    assert [p for p, _ in tracing.select_modules(m, classes=(nn.ReLU,), include_root=True)] == ["Sequential", "2"]
    assert [p for p, _ in tracing.select_modules(m, predicate=lambda path, mod: path.startswith("1"))] == ["1", "1.lin"]


def test_module_timer_counts_and_times_on_the_host_clock():
    m = _model()
    x = torch.randn(3, 4)
    with tracing.ModuleTimer(m, max_depth=1) as timer:
        for _ in range(3):
            m(x)
        s = timer.summary(by="path")
        assert [s[k]["calls"] for k in ("0", "1", "2")] == [3, 3, 3]
        assert s["0"]["total_ms"] >= 15 and s["1"]["total_ms"] >= 30 and s["2"]["total_ms"] < 15
        by_cls = timer.summary(by="class")
        assert by_cls["_Slow"]["calls"] == 6 and by_cls["_Slow"]["total_ms"] >= 45
        assert "_Slow" in timer.table() and timer.table(top=1).count("\n") == 1
        timer.reset()
        assert timer.summary()["0"]["calls"] == 0
    m(x)                                    # hooks removed: nothing is recorded any more
    assert all(len(v) == 0 for v in timer.spans.values())


def test_timer_survives_a_module_that_raises():
    class Boom(nn.Module):
        def forward(self, x):
            raise RuntimeError("boom")
    m = nn.Sequential(nn.Linear(4, 4), Boom())
    with tracing.ModuleTimer(m, max_depth=1) as timer:
        for _ in range(2):
            try:
                m(torch.randn(1, 4))
            except RuntimeError:
                pass
        s = timer.summary()
    assert s["0"]["calls"] == 2 and s["1"]["calls"] == 2 and not any(timer._open.values())


def test_annotate_and_regions_are_harmless_without_a_gpu():
    m = _model((0, 0))
    with tracing.annotate(m, max_depth=2) as a:
        assert "1.lin [Linear]" in a.names and (a.active or not a._handles)
        m(torch.randn(2, 4))
    with tracing.nvtx_range("outer"):
        pass
    d = {}
    with tracing.timed_region(d):
        time.sleep(0.002)
    assert d["ms"] >= 2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_path):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m = _model((5, 5 if rank == 0 else 40))          # rank 1 is the slow one on module "1"
    timer = tracing.ModuleTimer(m, max_depth=1)
    m(torch.randn(2, 4))
    s = timer.summary(by="path")
    if rank == 0:
        torch.save({k: v["total_ms"] for k, v in s.items()}, out_path)
    dist.destroy_process_group()


def test_summary_is_the_maximum_over_ranks(tmp_path):
    out = str(tmp_path / "s.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    s = torch.load(out)
    assert s["1"] >= 40 and s["0"] < 40       # rank 0 reports rank 1's time for the module that was slow there
