"""Invariant point attention kernel (csrc/ipa.cu) against its fp32 PyTorch statement, and the module that calls it."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(N, seed=0, masked=True):
    g = torch.Generator().manual_seed(seed)
    H, C, PQ, PV, CZ = 12, 16, 4, 8, 128
    r = lambda *s: torch.randn(*s, generator=g)
    q, k, v = r(N, H, C), r(N, H, C), r(N, H, C)
    q_pts, k_pts, v_pts = r(N, H, PQ, 3) * 8, r(N, H, PQ, 3) * 8, r(N, H, PV, 3) * 8
    z = r(N, N, CZ).to(torch.bfloat16)
    wb, bb = r(H, CZ) * 0.1, r(H) * 0.1
    gamma = torch.nn.functional.softplus(r(H)) * math.sqrt(1.0 / (3 * (PQ * 9.0 / 2)))
    mask = (torch.rand(N, generator=g) > 0.15).float() if masked else torch.ones(N)
    return [t.to(DEV) for t in (q, k, v, q_pts, k_pts, v_pts, z, wb, bb, gamma, mask)]


@pytest.mark.parametrize("N", [64, 200, 333])
def test_ipa_core_matches_reference(N, device_status):
    from fastfold_b200.ops.ipa import ipa_core, ipa_core_ref
    args = _inputs(N)
    w_c, w_b, inf = math.sqrt(1.0 / 48), math.sqrt(1.0 / 3), 1e5
    with torch.no_grad():
        o, o_pt, o_pair = ipa_core(*args, w_c, w_b, inf)
        ro, ro_pt, ro_pair = ipa_core_ref(*args, w_c, w_b, inf)
    for a, b, tol in ((o, ro, 2e-3), (o_pt, ro_pt, 2e-2), (o_pair, ro_pair, 2e-3)):
        assert a.shape == b.shape
        assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item())


def test_ipa_core_row_block(device_status):
    """A rank that holds rows [64, 128) of the pair tensor computes exactly those query rows."""
    from fastfold_b200.ops.ipa import ipa_core
    args = _inputs(192, seed=3)
    w_c, w_b, inf = math.sqrt(1.0 / 48), math.sqrt(1.0 / 3), 1e5
    with torch.no_grad():
        full = ipa_core(*args, w_c, w_b, inf)
        shard = list(args)
        shard[6] = args[6][64:128].contiguous()
        part = ipa_core(*shard, w_c, w_b, inf, row0=64)
    for a, b in zip(part, full):
        assert torch.equal(a, b[64:128])


def test_ipa_module_uses_kernel_and_matches_cpu(device_status):
    from fastfold_b200.models.nn.structure_module import InvariantPointAttention
    from fastfold_b200.ops import _lib
    from fastfold_b200.utils.rigid_utils import Rigid, Rotation
    torch.manual_seed(0)
    N = 96
    ipa = InvariantPointAttention(384, 128, 16, 12, 4, 8).eval()
    with torch.no_grad():
        for p in ipa.parameters():
            if float(p.abs().sum()) == 0.0:
                p.normal_(0, 0.05)
    s, z = torch.randn(N, 384), torch.randn(N, N, 128)
    quats, trans = torch.randn(N, 4), torch.randn(N, 3) * 5
    mask = torch.ones(N)
    with torch.no_grad():
        ref = ipa(s, z, Rigid(Rotation(quats=quats, normalize_quats=True), trans), mask)
        ipa_g = ipa.to(DEV, torch.bfloat16)
        n0 = _lib.LAUNCHES[0]
        got = ipa_g(s.to(DEV, torch.bfloat16), z.to(DEV, torch.bfloat16), Rigid(Rotation(quats=quats.to(DEV), normalize_quats=True), trans.to(DEV)),
                    mask.to(DEV, torch.bfloat16))
        assert _lib.LAUNCHES[0] > n0            # the native kernel ran
    err = (got.float().cpu() - ref).abs().mean().item()
    assert err <= 5e-2 * max(1.0, ref.abs().mean().item()), err
