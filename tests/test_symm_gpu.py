"""P2P collective kernels over the symmetric heap (2 GPUs): all-gather, all-to-all, fused all-to-all + LayerNorm,
two-shot all-reduce, CUDA-graph replay of a collective, and the bounded wait (a flag nobody raises must time out
with a status code, not hang).  NVLS is switched off for NCCL; the kernels use plain peer loads and stores."""
import os
import socket
import sys
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_path):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0", FASTFOLD_SYMM_HEAP_MB="256", FASTFOLD_SYMM_WAIT_S="1.0")
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from fastfold_b200.parallel import init_dap, shutdown, symm
    from fastfold_b200.ops import _lib
    init_dap(world, timeout_s=60)
    dev = torch.device("cuda", rank)
    h = symm.get_heap("dap")
    h.poison()                       # every slot starts as NaN: reading a slot before it is written cannot pass
    import time
    res = {}
    skew = lambda k: time.sleep(0.02 * ((rank * 7 + k) % world))     # ranks reach each collective at different times
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    # all-gather
    x = torch.randn(64, 40, generator=g).to(dev, torch.bfloat16)
    skew(0)
    got = h.all_gather(None, x)
    ref = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(ref, x)
    res["all_gather"] = float((got.float() - torch.stack(ref).float()).abs().max())
    # all-to-all (several rounds so that ring slots are reused)
    worst = 0.0
    for it in range(30):
        send = torch.randn(world, 33, 16, generator=g).to(dev, torch.bfloat16)
        if it % 7 == 0:
            skew(it)
        recv = h.all_to_all(None, send)
        ref = torch.empty_like(send)
        dist.all_to_all_single(ref, send)
        worst = max(worst, float((recv.float() - ref.float()).abs().max()))
    res["all_to_all"] = worst
    # fused axis switch + LayerNorm, both directions, with and without transposed output
    A, B, C = 8 * world // 2, 12 * world // 2, 128
    gamma = (torch.randn(C, generator=torch.Generator().manual_seed(1)) * 0.3 + 1).to(dev, torch.bfloat16)
    beta = (torch.randn(C, generator=torch.Generator().manual_seed(2)) * 0.1).to(dev, torch.bfloat16)
    full = torch.randn(A, B, C, generator=torch.Generator().manual_seed(3)).to(dev, torch.bfloat16)
    a2a_err = 0.0
    for mode in (0, 1):
        for tr in (False, True):
            if mode == 0:
                shard = full[rank * (A // world):(rank + 1) * (A // world)]
                want = full[:, rank * (B // world):(rank + 1) * (B // world)]
            else:
                shard = full[:, rank * (B // world):(rank + 1) * (B // world)]
                want = full[rank * (A // world):(rank + 1) * (A // world)]
            skew(mode * 2 + int(tr))
            raw, norm = h.a2a_layer_norm(None, shard, mode, A, B, C, gamma, beta, 1e-5, True, tr)
            wn = torch.nn.functional.layer_norm(want.float(), (C,), gamma.float(), beta.float(), 1e-5)
            if tr:
                wn = wn.transpose(0, 1)
            a2a_err = max(a2a_err, float((raw.float() - want.float()).abs().max()), float((norm.float() - wn).abs().max()))
    res["a2a_ln"] = a2a_err
    # one-kernel push collectives against compositions of NCCL calls
    push_err = 0.0
    for dim in (0, 1, 2):
        x = torch.randn(6, 10, 16, generator=g).to(dev, torch.bfloat16)
        skew(dim)
        got = h.gather_dim(x, dim)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        push_err = max(push_err, float((got.float() - torch.cat(parts, dim=dim).float()).abs().max()))
    for in_dim, out_dim in ((1, 2), (2, 1), (0, 2)):
        shape = [2 * world, 4 * world, 4 * world, 16]          # every split dimension divides by the world size
        x = torch.randn(*shape, generator=g).to(dev, torch.bfloat16)
        in_d, out_d = in_dim + (0 if in_dim == 0 else 0), out_dim
        skew(in_dim + out_dim)
        got = h.all_to_all_dims(x, in_d, out_d)
        send = list(x.chunk(world, dim=in_d))
        recv = [torch.empty_like(send[0]) for _ in range(world)]
        dist.all_to_all(recv, [t.contiguous() for t in send])
        push_err = max(push_err, float((got.float() - torch.cat(recv, dim=out_d).float()).abs().max()))
    res["push_copy"] = push_err
    rs_err = 0.0
    for dim in (0, 1):
        x = torch.randn(8 * world // 2, 4 * world, 24, generator=g).to(dev, torch.bfloat16)
        skew(dim)
        got = h.reduce_scatter_dim(x, dim)
        full = x.float().clone()
        dist.all_reduce(full)
        want = full.chunk(world, dim=dim)[rank]
        rs_err = max(rs_err, float((got.float() - want).abs().max() / (want.abs().max() + 1e-6)))
    res["push_reduce_scatter"] = rs_err
    # all-reduce of a vector living in the heap, replayed from a CUDA graph
    n = 8 * 1000
    slot = h.slot("t_grads", n * 2)
    v = h.view(slot, (n,), torch.bfloat16)
    base = torch.randn(n, generator=g).to(dev, torch.bfloat16)
    allv = [torch.empty_like(base) for _ in range(world)]
    dist.all_gather(allv, base)
    want = torch.stack(allv).float().sum(0)
    v.copy_(base)
    h.all_reduce_(slot, n)
    res["all_reduce"] = float((v.float() - want).abs().max() / (want.abs().max() + 1e-6))
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        v.copy_(base)
        h.all_reduce_(slot, n)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        v.copy_(base)
        h.all_reduce_(slot, n)
    worst = 0.0
    for _ in range(5):
        graph.replay()
        torch.cuda.synchronize()
        worst = max(worst, float((v.float() - want).abs().max() / (want.abs().max() + 1e-6)))
    res["all_reduce_graph"] = worst
    torch.cuda.synchronize()
    res["status_before"] = _lib.read_status()[0]
    dist.barrier()
    # bounded wait: must come back with ST_TIMEOUT_PEER (4) after about a second
    t0 = time.time()
    h.wait_never(h.slot("never", 1024))
    torch.cuda.synchronize()
    res["timeout_s"] = time.time() - t0
    res["status_after"] = _lib.read_status()[0]
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    shutdown()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_symm_collectives(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    with tempfile.TemporaryDirectory() as d:
        out_path = os.path.join(d, "o.pt")
        mp.spawn(_worker, args=(world, _free_port(), out_path), nprocs=world, join=True)
        res = torch.load(out_path)
    assert res["all_gather"] == 0.0
    assert res["all_to_all"] == 0.0
    assert res["a2a_ln"] < 5e-2
    assert res["push_copy"] == 0.0
    assert res["push_reduce_scatter"] < 1e-2
    assert res["all_reduce"] < 1e-2 and res["all_reduce_graph"] < 1e-2
    assert res["status_before"] == 0
    assert res["status_after"] == 4 and 0.5 < res["timeout_s"] < 10
