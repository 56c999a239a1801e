"""Struct-of-arrays geometry against the tensor-based rigid utilities."""
import torch

from fastfold_b200.utils.geometry import QuatRigid, Rigid3Array, Rot3Array, Vec3Array, dihedral_angle
from fastfold_b200.utils.rigid_utils import Rigid


def test_rigid_composition_and_inverse():
    torch.manual_seed(0)
    a, b, c = (torch.randn(5, 3) for _ in range(3))
    r1 = Rigid.from_3_points(a, b, c)
    m = r1.to_tensor_4x4()
    s = Rigid3Array.from_tensor_4x4(m)
    p = torch.randn(5, 3)
    assert torch.allclose(s.apply_to_point(Vec3Array.from_array(p)).to_tensor(), r1.apply(p), atol=1e-5)
    assert torch.allclose(s.apply_inverse_to_point(Vec3Array.from_array(p)).to_tensor(), r1.invert_apply(p), atol=1e-5)
    ident = (s @ s.inverse()).to_tensor_4x4()
    assert torch.allclose(ident, torch.eye(4).expand(5, 4, 4), atol=1e-5)


def test_two_vector_frame_and_dihedral():
    e0, e1 = Vec3Array.from_array(torch.tensor([[2.0, 0, 0]])), Vec3Array.from_array(torch.tensor([[1.0, 3.0, 0]]))
    rot = Rot3Array.from_two_vectors(e0, e1).to_tensor()
    assert torch.allclose(rot, torch.eye(3)[None], atol=1e-6)
    pts = [Vec3Array.from_array(torch.tensor([v])) for v in ([1.0, 0, 0], [0.0, 0, 0], [0.0, 0, 1], [0.0, 1, 1])]
    ang = dihedral_angle(*pts)
    assert abs(abs(float(ang)) - torch.pi / 2) < 1e-5


def test_quat_rigid_starts_at_identity():
    q = QuatRigid(8)
    out = q(torch.randn(3, 8))
    assert torch.allclose(out.rotation.to_tensor(), torch.eye(3).expand(3, 3, 3), atol=1e-6)
    assert torch.allclose(out.translation.to_tensor(), torch.zeros(3, 3))


def test_atom14_atom37_round_trip():
    from fastfold_b200.utils import all_atom_multimer as aam
    torch.manual_seed(1)
    aatype = torch.randint(0, 20, (7,))
    x14 = torch.randn(7, 14, 3) * aam.get_atom14_mask(aatype)[..., None]
    x37 = aam.atom14_to_atom37(x14, aatype)
    assert x37.shape == (7, 37, 3)
    back = aam.atom37_to_atom14(x37, aatype)
    assert torch.allclose(back, x14)
    pos = Vec3Array.from_array(x37)
    frames, fmask = aam.make_backbone_affine(pos, aam.get_atom37_mask(aatype), aatype)
    assert fmask.shape == (7,) and frames.rotation.xx.shape == (7,)
    chi, chi_mask = aam.compute_chi_angles(pos, aam.get_atom37_mask(aatype), aatype)
    assert chi.shape == (7, 4) and chi_mask.shape == (7, 4) and torch.isfinite(chi).all()


def test_multimer_all_atom_helpers_match_monomer_code():
    """The struct-of-arrays (multimer) frame / torsion / placement helpers agree with the quaternion-free monomer ones."""
    import torch
    from fastfold_b200.common import residue_constants as rc
    from fastfold_b200.data import data_transforms as dt
    from fastfold_b200.utils import all_atom_multimer as aam, feats
    from fastfold_b200.utils.geometry import Rigid3Array, Vec3Array
    from fastfold_b200.utils.rigid_utils import Rigid, Rotation
    from fastfold_b200.utils.synthetic import random_ground_truth
    g = torch.Generator().manual_seed(0)
    aatype = torch.randint(0, 20, (24,), generator=g)
    gt = random_ground_truth(aatype, g)
    pos37, mask37 = gt["all_atom_positions"], gt["all_atom_mask"]
    # frames from atom37 coordinates
    fr = aam.atom37_to_frames(aatype, Vec3Array.from_array(pos37), mask37)
    ref = dt.atom37_to_frames({"aatype": aatype, "all_atom_positions": pos37, "all_atom_mask": mask37})
    ex = ref["rigidgroups_gt_exists"]
    assert torch.equal(fr["rigidgroups_gt_exists"], ex)
    assert torch.equal(fr["rigidgroups_group_is_ambiguous"], ref["rigidgroups_group_is_ambiguous"])
    got4 = fr["rigidgroups_gt_frames"].to_tensor_4x4()
    assert torch.allclose(got4 * ex[..., None, None], ref["rigidgroups_gt_frames"] * ex[..., None, None], atol=1e-4)
    alt4 = fr["rigidgroups_alt_gt_frames"].to_tensor_4x4()
    assert torch.allclose(alt4 * ex[..., None, None], ref["rigidgroups_alt_gt_frames"] * ex[..., None, None], atol=1e-4)
    # torsions -> frames -> atom14 positions
    quats = torch.randn(24, 4, generator=g)
    trans = torch.randn(24, 3, generator=g) * 5
    bb = Rigid(Rotation(quats=quats, normalize_quats=True), trans)
    ang = torch.randn(24, 7, 2, generator=g)
    ang = ang / ang.norm(dim=-1, keepdim=True)
    rrgdf = torch.tensor(rc.restype_rigid_group_default_frame, dtype=torch.float32)
    ref_frames = feats.torsion_angles_to_frames(bb, ang, aatype, rrgdf)
    ref_pos = feats.frames_and_literature_positions_to_atom14_pos(ref_frames, aatype, rrgdf, torch.tensor(rc.restype_atom14_to_rigid_group),
                                                                  torch.tensor(rc.restype_atom14_mask), torch.tensor(rc.restype_atom14_rigid_group_positions, dtype=torch.float32))
    bb3 = Rigid3Array.from_tensor_4x4(bb.to_tensor_4x4())
    frames = aam.torsion_angles_to_frames(aatype, bb3, ang)
    assert torch.allclose(frames.to_tensor_4x4(), ref_frames.to_tensor_4x4(), atol=1e-4)
    pos = aam.frames_and_literature_positions_to_atom14_pos(aatype, frames)
    assert torch.allclose(pos.to_tensor(), ref_pos, atol=1e-4)
    # renamed ground truth and chain-break statistic
    p14 = aam.atom37_to_atom14(pos37, aatype)
    alt_pos, alt_mask = aam.get_alt_atom14(aatype, Vec3Array.from_array(p14), aam.get_atom14_mask(aatype))
    ref_alt = dt.make_atom14_positions(dt.make_atom14_masks({"aatype": aatype, "all_atom_positions": pos37, "all_atom_mask": mask37}))
    assert torch.allclose(alt_pos.to_tensor(), ref_alt["atom14_alt_gt_positions"], atol=1e-5)
    v = aam.extreme_ca_ca_distance_violations(Vec3Array.from_array(p14), aam.get_atom14_mask(aatype), torch.arange(24))
    assert 0.0 <= float(v) <= 1.0
    assert aam.get_chi_atom_indices().shape == (21, 4, 4)
