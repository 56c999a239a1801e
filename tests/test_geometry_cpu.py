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
