"""Dynamic Axial Parallelism on CPU ranks (Gloo): outputs and gradients for P in {2, 4} must equal P = 1.

The reference tests DAP only in forward and only on GPUs (tests/test_fastnn/test_evoformer.py:49-62); backward
under DAP is what exposes a missing reduce-scatter in the gradient of the gathered operands.
"""
import os
import socket
import sys
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _build(seed, c_m, c_z, n_blocks):
    from fastfold_b200.models.fastnn import EvoformerStack
    torch.manual_seed(seed)
    model = EvoformerStack(c_m, c_z, 24, n_blocks, blocks_per_ckpt=1).double()
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float64) * 0.1)
    return model


def _inputs(seed, S, N, c_m, c_z):
    g = torch.Generator().manual_seed(seed)
    m = torch.randn(S, N, c_m, generator=g, dtype=torch.float64)
    z = torch.randn(N, N, c_z, generator=g, dtype=torch.float64)
    msa_mask = (torch.rand(S, N, generator=g) > 0.1).double()
    pair_mask = (torch.rand(N, N, generator=g) > 0.1).double()
    return m, z, msa_mask, pair_mask


def _run(model, m, z, mm, pm, train):
    model.train(train)
    m = m.clone().requires_grad_(True)
    z = z.clone().requires_grad_(True)
    om, oz, s = model(m, z, mm, pm, None)
    loss = (om ** 2).mean() + (oz ** 2).mean() + (s ** 2).mean()
    loss.backward()
    grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    return om.detach(), oz.detach(), s.detach(), m.grad, z.grad, grads


def _worker(rank, world, port, S, N, train, out_path):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from fastfold_b200.parallel import init_dap, shutdown
    init_dap(world, backend="gloo", timeout_s=120)
    model = _build(3, 16, 8, 2)
    m, z, mm, pm = _inputs(5, S, N, 16, 8)
    torch.manual_seed(11)           # identical dropout masks on every rank (and in the P = 1 run)
    om, oz, s, gm, gz, grads = _run(model, m, z, mm, pm, train)
    # weights are replicated over the DAP group: sum gradients of sharded computation, average the replicated projection
    for n, g in grads.items():
        dist.all_reduce(g)
        if n.startswith("linear."):
            g /= world
    # input gradients need no reduction: the backward of the first block's scatter is an all-gather
    if rank == 0:
        torch.save({"om": om, "oz": oz, "s": s, "gm": gm, "gz": gz, "grads": grads}, out_path)
    shutdown()


@pytest.mark.parametrize("world,S,N,train", [(2, 4, 6, False), (2, 4, 7, True), (4, 8, 9, True)])
def test_dap_matches_single_rank(world, S, N, train):
    sys.path.insert(0, ROOT)
    from fastfold_b200.parallel import core
    assert core.get_dap_size() == 1
    model = _build(3, 16, 8, 2)
    m, z, mm, pm = _inputs(5, S, N, 16, 8)
    torch.manual_seed(11)
    ref = _run(model, m, z, mm, pm, train)
    with tempfile.TemporaryDirectory() as d:
        out_path = os.path.join(d, "out.pt")
        mp.spawn(_worker, args=(world, _free_port(), S, N, train, out_path), nprocs=world, join=True)
        got = torch.load(out_path)
    tol = 1e-9
    assert (got["om"] - ref[0]).abs().max() < tol
    assert (got["oz"] - ref[1]).abs().max() < tol
    assert (got["s"] - ref[2]).abs().max() < tol
    assert (got["gm"] - ref[3]).abs().max() < tol
    assert (got["gz"] - ref[4]).abs().max() < tol
    for n, g in ref[5].items():
        assert (got["grads"][n] - g).abs().max() < tol * max(1.0, g.abs().max().item()), n
