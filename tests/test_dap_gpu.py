"""DAP on real GPUs (NCCL / fused P2P kernels): a 2-rank Evoformer stack must reproduce the 1-rank result."""
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


def _model():
    from fastfold_b200.models.fastnn import EvoformerStack
    torch.manual_seed(3)
    model = EvoformerStack(256, 128, 384, 2, blocks_per_ckpt=1)
    g = torch.Generator().manual_seed(4)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
    return model


def _inputs(S, N):
    g = torch.Generator().manual_seed(5)
    m = torch.randn(S, N, 256, generator=g)
    z = torch.randn(N, N, 128, generator=g)
    mm = (torch.rand(S, N, generator=g) > 0.1).float()
    pm = (torch.rand(N, N, generator=g) > 0.1).float()
    return m, z, mm, pm


def _run(dev, S, N, train):
    model = _model().to(dev, torch.bfloat16).train(train)
    m, z, mm, pm = (t.to(dev, torch.bfloat16) for t in _inputs(S, N))
    torch.manual_seed(11)
    if train:
        m.requires_grad_(True)
        z.requires_grad_(True)
        om, oz, s = model(m, z, mm, pm, None)
        (om.float().pow(2).mean() + oz.float().pow(2).mean() + s.float().pow(2).mean()).backward()
        return om.detach().float().cpu(), oz.detach().float().cpu(), m.grad.float().cpu(), z.grad.float().cpu()
    with torch.no_grad():
        om, oz, s = model(m, z, mm, pm, None)
    return om.float().cpu(), oz.float().cpu(), s.float().cpu(), None


def _worker(rank, world, port, S, N, train, out_path):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    import time
    from fastfold_b200.parallel import init_dap, shutdown, symm
    from fastfold_b200.ops import _lib
    init_dap(world, timeout_s=120)
    h = symm.get_heap("dap")
    if h is not None:
        h.poison()                   # peer slots start as NaN
    time.sleep(0.05 * rank)          # ranks start the model at different times
    out = _run(torch.device("cuda", rank), S, N, train)
    if not train:
        # determinism: two more runs of the inference path must reproduce the first one bit for bit
        for _ in range(2):
            again = _run(torch.device("cuda", rank), S, N, train)
            for a, b in zip(out, again):
                if a is not None and not torch.equal(a, b):
                    raise AssertionError("inference under DAP is not bitwise reproducible")
    torch.cuda.synchronize()
    st = _lib.read_status()
    if rank == 0:
        torch.save({"out": out, "status": st}, out_path)
    shutdown()


@pytest.mark.parametrize("world,S,N,train", [(2, 32, 64, False), (2, 32, 72, False), (2, 32, 64, True), (2, 16, 256, False), (2, 16, 256, True),
                                             (4, 32, 512, False), (4, 32, 512, True), (8, 32, 1024, False), (8, 32, 1024, True)])
def test_ranks_match_one(world, S, N, train):
    """Outputs (and, in training, input gradients) of a 2-block stack on ``world`` DAP ranks against one rank.  The
    larger worlds use lengths at which every rank's slab is a whole number of 128-wide tiles, so the GEMMs that read
    their gathered operand straight from the peers' memory run."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    ref = _run(torch.device("cuda", 0), S, N, train)
    with tempfile.TemporaryDirectory() as d:
        out_path = os.path.join(d, "o.pt")
        mp.spawn(_worker, args=(world, _free_port(), S, N, train, out_path), nprocs=world, join=True)
        got = torch.load(out_path)
    assert got["status"][0] == 0, got["status"]
    for a, b in zip(got["out"], ref):
        if b is None:
            continue
        err = (a - b).abs().mean().item()
        scale = b.abs().mean().item() + 1e-6
        assert err < 3e-2 * max(1.0, scale), "mean abs err %g (scale %g)" % (err, scale)


def test_inference_is_bitwise_reproducible(device_status):
    """Three runs of the inference path on one GPU give identical bits (no atomics, no order-dependent reductions)."""
    dev = torch.device("cuda", 0)
    first = _run(dev, 32, 64, False)
    for _ in range(2):
        again = _run(dev, 32, 64, False)
        for a, b in zip(first, again):
            if a is not None:
                assert torch.equal(a, b)


def _full_model_worker(rank, world, port, shard, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    from fastfold_b200.ops import _lib
    from fastfold_b200.parallel import init_dap, shutdown
    from fastfold_b200.runtime.inference import load_model, predict
    from fastfold_b200.utils.synthetic import random_features
    init_dap(world, timeout_s=120)
    model = load_model("model_3", None, chunk_size=None, inplace=True, seed=5, shard_pair=shard,
                       overrides={"model.evoformer_stack.no_blocks": 2, "model.extra_msa.extra_msa_stack.no_blocks": 1})
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.normal_(0.0, 0.05)
    batch = random_features(128, 16, 32, n_templ=0, n_recycle=1, seed=2)
    out, _ = predict(model, batch)
    torch.cuda.synchronize()
    st = _lib.read_status()
    torch.save({"pos": out["final_atom_positions"].float().cpu(), "single": out["single"].float().cpu(), "pair": out["pair"].float().cpu(),
                "dist": out["distogram_logits"].float().cpu(), "status": st}, os.path.join(out_dir, "r%d.pt" % rank))
    shutdown()


def test_full_model_with_row_sharded_pair_tensor():
    """Full (reduced-depth) model over two GPUs, in place, with the pair tensor kept as row shards from the embedders to the
    heads (row-parallel invariant point attention kernel, sharded recycling and distogram head) against the run that
    gathers the pair tensor after every stack."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = {}
    for shard in (False, True):
        with tempfile.TemporaryDirectory() as d:
            mp.spawn(_full_model_worker, args=(2, _free_port(), shard, d), nprocs=2, join=True)
            res[shard] = [torch.load(os.path.join(d, "r%d.pt" % r)) for r in range(2)]
    full, sh = res[False], res[True]
    assert all(r["status"][0] == 0 for r in full + sh)
    assert sh[0]["pair"].shape[0] * 2 == full[0]["pair"].shape[0]
    pair = torch.cat([sh[0]["pair"], sh[1]["pair"]], dim=0)
    dist = torch.cat([sh[0]["dist"], sh[1]["dist"]], dim=0)
    scale = lambda t: max(1.0, t.abs().mean().item())
    assert (pair - full[0]["pair"]).abs().mean().item() < 3e-2 * scale(full[0]["pair"])
    assert (dist - full[0]["dist"]).abs().mean().item() < 3e-2 * scale(full[0]["dist"])
    assert (sh[0]["single"] - full[0]["single"]).abs().mean().item() < 3e-2 * scale(full[0]["single"])
    assert torch.isfinite(sh[0]["pos"]).all() and torch.isfinite(full[0]["pos"]).all()
