"""Full model over two CPU ranks (Gloo) with the pair tensor kept row-sharded from the embedders to the heads: final
coordinates, single representation and (after concatenating the ranks' shards) the pair tensor and distogram logits
must equal the run that gathers the pair tensor at the end of every stack."""
import os
import socket
import sys
import tempfile

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, shard, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    from fastfold_b200.config import model_config
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.parallel import init_dap, shutdown
    from fastfold_b200.utils.inject_fastnn import inject_fastnn
    from fastfold_b200.utils.synthetic import random_features
    init_dap(world)
    cfg = model_config("model_3")
    cfg.model.evoformer_stack.no_blocks = 2
    cfg.model.extra_msa.extra_msa_stack.no_blocks = 1
    cfg.globals.shard_pair = shard
    torch.manual_seed(0)
    model = AlphaFold(cfg)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.normal_(0.0, 0.05)
    model = inject_fastnn(model).eval()
    batch = random_features(24, 6, 8, n_templ=0, n_recycle=1, seed=2)
    with torch.no_grad():
        out = model(batch)
    torch.save({k: out[k] for k in ("final_atom_positions", "single", "pair", "distogram_logits", "plddt")}, os.path.join(out_dir, "r%d.pt" % rank))
    shutdown()


def _run(shard):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, _free_port(), shard, d), nprocs=2, join=True)
        return [torch.load(os.path.join(d, "r%d.pt" % r)) for r in range(2)]


def test_pair_tensor_stays_sharded_end_to_end():
    full = _run(False)
    shard = _run(True)
    assert full[0]["pair"].shape == (24, 24, 128)
    assert shard[0]["pair"].shape == (12, 24, 128) and shard[1]["pair"].shape == (12, 24, 128)
    pair = torch.cat([shard[0]["pair"], shard[1]["pair"]], dim=0)
    dist = torch.cat([shard[0]["distogram_logits"], shard[1]["distogram_logits"]], dim=0)
    assert torch.allclose(pair, full[0]["pair"], atol=1e-4)
    assert torch.allclose(dist, full[0]["distogram_logits"], atol=1e-4)
    for r in range(2):
        assert torch.allclose(shard[r]["final_atom_positions"], full[0]["final_atom_positions"], atol=1e-3)
        assert torch.allclose(shard[r]["single"], full[0]["single"], atol=1e-4)
        assert torch.allclose(shard[r]["plddt"], full[0]["plddt"], atol=1e-3)
