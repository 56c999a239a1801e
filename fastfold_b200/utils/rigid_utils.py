"""Rotations and rigid transforms on batched tensors (fp32 islands inside a bf16 model).

``Rotation`` (rotation matrix or unit quaternion) and ``Rigid`` (rotation + translation) with the operations the
structure module, the feature builders and the FAPE loss need: composition, inversion, application to points,
quaternion updates from a 6-vector, construction from three points, 4x4 / 7-vector conversions.  All maths runs
in fp32 whatever the activation dtype, and ``rot_matmul`` / ``rot_vec_mul`` are written as explicit sums so that
no reduced-precision matmul path is ever taken.  Same role as fastfold/utils/rigid_utils.py.
"""
from __future__ import annotations

from typing import Any, Callable, Optional, Sequence, Tuple

import numpy as np
import torch


def rot_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[*, 3, 3] x [*, 3, 3] with explicit products and sums."""
    rows = []
    for i in range(3):
        rows.append(torch.stack([a[..., i, 0] * b[..., 0, j] + a[..., i, 1] * b[..., 1, j] + a[..., i, 2] * b[..., 2, j]
                                 for j in range(3)], dim=-1))
    return torch.stack(rows, dim=-2)


def rot_vec_mul(r: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
    """[*, 3, 3] applied to [*, 3]."""
    x, y, z = torch.unbind(t, dim=-1)
    return torch.stack([r[..., 0, 0] * x + r[..., 0, 1] * y + r[..., 0, 2] * z,
                        r[..., 1, 0] * x + r[..., 1, 1] * y + r[..., 1, 2] * z,
                        r[..., 2, 0] * x + r[..., 2, 1] * y + r[..., 2, 2] * z], dim=-1)


def identity_rot_mats(batch_dims, dtype=None, device=None, requires_grad=True):
    rots = torch.eye(3, dtype=dtype, device=device, requires_grad=requires_grad)
    rots = rots.view(*((1,) * len(batch_dims)), 3, 3).expand(*batch_dims, -1, -1)
    return rots.contiguous()


def identity_trans(batch_dims, dtype=None, device=None, requires_grad=True):
    return torch.zeros((*batch_dims, 3), dtype=dtype, device=device, requires_grad=requires_grad)


def identity_quats(batch_dims, dtype=None, device=None, requires_grad=True):
    quat = torch.zeros((*batch_dims, 4), dtype=dtype, device=device, requires_grad=requires_grad)
    with torch.no_grad():
        quat[..., 0] = 1
    return quat


def quat_to_rot(quat: torch.Tensor) -> torch.Tensor:
    """Unit (or unnormalised: the result is scaled by |q|^2) quaternion [*, 4] (w, x, y, z) -> rotation matrix."""
    w, x, y, z = torch.unbind(quat, dim=-1)
    return torch.stack([
        torch.stack([w * w + x * x - y * y - z * z, 2 * (x * y - w * z), 2 * (x * z + w * y)], dim=-1),
        torch.stack([2 * (x * y + w * z), w * w - x * x + y * y - z * z, 2 * (y * z - w * x)], dim=-1),
        torch.stack([2 * (x * z - w * y), 2 * (y * z + w * x), w * w - x * x - y * y + z * z], dim=-1),
    ], dim=-2)


def rot_to_quat(rot: torch.Tensor) -> torch.Tensor:
    """Rotation matrix -> unit quaternion via the largest-eigenvalue eigenvector of the 4x4 K matrix."""
    if rot.shape[-2:] != (3, 3):
        raise ValueError("Input rotation is incorrectly shaped")
    [[xx, xy, xz], [yx, yy, yz], [zx, zy, zz]] = [[rot[..., i, j] for j in range(3)] for i in range(3)]
    k = [[xx + yy + zz, zy - yz, xz - zx, yx - xy],
         [zy - yz, xx - yy - zz, xy + yx, xz + zx],
         [xz - zx, xy + yx, yy - xx - zz, yz + zy],
         [yx - xy, xz + zx, yz + zy, zz - xx - yy]]
    k = (1.0 / 3.0) * torch.stack([torch.stack(t, dim=-1) for t in k], dim=-2)
    _, vectors = torch.linalg.eigh(k)
    return vectors[..., -1]


def quat_multiply(q1: torch.Tensor, q2: torch.Tensor) -> torch.Tensor:
    w1, x1, y1, z1 = torch.unbind(q1, dim=-1)
    w2, x2, y2, z2 = torch.unbind(q2, dim=-1)
    return torch.stack([w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2,
                        w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2,
                        w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2,
                        w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2], dim=-1)


def quat_multiply_by_vec(quat: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
    """Quaternion times the pure-imaginary quaternion (0, vec)."""
    w, x, y, z = torch.unbind(quat, dim=-1)
    a, b, c = torch.unbind(vec, dim=-1)
    return torch.stack([-x * a - y * b - z * c, w * a + y * c - z * b, w * b - x * c + z * a, w * c + x * b - y * a], dim=-1)


def invert_rot_mat(rot_mat: torch.Tensor) -> torch.Tensor:
    return rot_mat.transpose(-1, -2)


def invert_quat(quat: torch.Tensor) -> torch.Tensor:
    quat_prime = quat.clone()
    quat_prime[..., 1:] *= -1
    return quat_prime / torch.sum(quat ** 2, dim=-1, keepdim=True)


class Rotation:
    """A batch of 3D rotations held either as matrices ``[*, 3, 3]`` or as quaternions ``[*, 4]``."""

    def __init__(self, rot_mats: Optional[torch.Tensor] = None, quats: Optional[torch.Tensor] = None, normalize_quats: bool = True):
        if (rot_mats is None) == (quats is None):
            raise ValueError("Exactly one input argument must be specified")
        if (rot_mats is not None and rot_mats.shape[-2:] != (3, 3)) or (quats is not None and quats.shape[-1] != 4):
            raise ValueError("Incorrectly shaped rotation matrix or quaternion")
        if quats is not None:
            quats = quats.to(dtype=torch.float32)
        if rot_mats is not None:
            rot_mats = rot_mats.to(dtype=torch.float32)
        if quats is not None and normalize_quats:
            quats = quats / torch.linalg.norm(quats, dim=-1, keepdim=True)
        self._rot_mats = rot_mats
        self._quats = quats

    @staticmethod
    def identity(shape, dtype=None, device=None, requires_grad=True, fmt="quat") -> "Rotation":
        if fmt == "rot_mat":
            return Rotation(rot_mats=identity_rot_mats(shape, dtype, device, requires_grad))
        if fmt == "quat":
            return Rotation(quats=identity_quats(shape, dtype, device, requires_grad), normalize_quats=False)
        raise ValueError("Invalid format: %s" % fmt)

    def __getitem__(self, index: Any) -> "Rotation":
        if type(index) != tuple:
            index = (index,)
        if self._rot_mats is not None:
            return Rotation(rot_mats=self._rot_mats[index + (slice(None), slice(None))])
        return Rotation(quats=self._quats[index + (slice(None),)], normalize_quats=False)

    def __mul__(self, right: torch.Tensor) -> "Rotation":
        if self._rot_mats is not None:
            return Rotation(rot_mats=self._rot_mats * right[..., None, None])
        return Rotation(quats=self._quats * right[..., None], normalize_quats=False)

    __rmul__ = __mul__

    @property
    def shape(self) -> torch.Size:
        return self._rot_mats.shape[:-2] if self._rot_mats is not None else self._quats.shape[:-1]

    @property
    def dtype(self):
        return self._rot_mats.dtype if self._rot_mats is not None else self._quats.dtype

    @property
    def device(self):
        return self._rot_mats.device if self._rot_mats is not None else self._quats.device

    @property
    def requires_grad(self) -> bool:
        return self._rot_mats.requires_grad if self._rot_mats is not None else self._quats.requires_grad

    def get_rot_mats(self) -> torch.Tensor:
        return self._rot_mats if self._rot_mats is not None else quat_to_rot(self._quats)

    def get_quats(self) -> torch.Tensor:
        return self._quats if self._quats is not None else rot_to_quat(self._rot_mats)

    def get_cur_rot(self) -> torch.Tensor:
        return self._rot_mats if self._rot_mats is not None else self._quats

    def compose_q_update_vec(self, q_update_vec: torch.Tensor, normalize_quats: bool = True) -> "Rotation":
        """New rotation = this one composed with the quaternion (1, b, c, d)."""
        quats = self.get_quats()
        return Rotation(quats=quats + quat_multiply_by_vec(quats, q_update_vec), normalize_quats=normalize_quats)

    def compose_r(self, r: "Rotation") -> "Rotation":
        return Rotation(rot_mats=rot_matmul(self.get_rot_mats(), r.get_rot_mats()))

    def compose_q(self, r: "Rotation", normalize_quats: bool = True) -> "Rotation":
        return Rotation(quats=quat_multiply(self.get_quats(), r.get_quats()), normalize_quats=normalize_quats)

    def apply(self, pts: torch.Tensor) -> torch.Tensor:
        return rot_vec_mul(self.get_rot_mats(), pts)

    def invert_apply(self, pts: torch.Tensor) -> torch.Tensor:
        return rot_vec_mul(invert_rot_mat(self.get_rot_mats()), pts)

    def invert(self) -> "Rotation":
        if self._rot_mats is not None:
            return Rotation(rot_mats=invert_rot_mat(self._rot_mats))
        return Rotation(quats=invert_quat(self._quats), normalize_quats=False)

    def _map(self, fn: Callable[[torch.Tensor], torch.Tensor], n_rot: int, n_quat: int) -> "Rotation":
        if self._rot_mats is not None:
            return Rotation(rot_mats=fn(self._rot_mats, n_rot))
        return Rotation(quats=fn(self._quats, n_quat), normalize_quats=False)

    def unsqueeze(self, dim: int) -> "Rotation":
        if dim >= len(self.shape):
            raise ValueError("Invalid dimension")
        return self._map(lambda t, k: t.unsqueeze(dim if dim >= 0 else dim - k), 2, 1)

    @staticmethod
    def cat(rs: Sequence["Rotation"], dim: int) -> "Rotation":
        rot_mats = torch.cat([r.get_rot_mats() for r in rs], dim=dim if dim >= 0 else dim - 2)
        return Rotation(rot_mats=rot_mats)

    def map_tensor_fn(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "Rotation":
        """Applies ``fn`` (a function of one tensor that keeps the batch layout) to every scalar channel."""
        if self._rot_mats is not None:
            m = self._rot_mats.view(self._rot_mats.shape[:-2] + (9,))
            m = torch.stack(list(map(fn, torch.unbind(m, dim=-1))), dim=-1)
            return Rotation(rot_mats=m.view(m.shape[:-1] + (3, 3)))
        q = torch.stack(list(map(fn, torch.unbind(self._quats, dim=-1))), dim=-1)
        return Rotation(quats=q, normalize_quats=False)

    def cuda(self) -> "Rotation":
        return self.to(device="cuda", dtype=None)

    def to(self, device=None, dtype=None) -> "Rotation":
        if self._rot_mats is not None:
            return Rotation(rot_mats=self._rot_mats.to(device=device, dtype=dtype))
        return Rotation(quats=self._quats.to(device=device, dtype=dtype), normalize_quats=False)

    def detach(self) -> "Rotation":
        if self._rot_mats is not None:
            return Rotation(rot_mats=self._rot_mats.detach())
        return Rotation(quats=self._quats.detach(), normalize_quats=False)


class Rigid:
    """A batch of rigid transforms: ``x -> R x + t``."""

    def __init__(self, rots: Optional[Rotation], trans: Optional[torch.Tensor]):
        batch_dims, dtype, device, requires_grad = None, None, None, None
        if trans is not None:
            batch_dims, dtype, device, requires_grad = trans.shape[:-1], trans.dtype, trans.device, trans.requires_grad
        elif rots is not None:
            batch_dims, dtype, device, requires_grad = rots.shape, rots.dtype, rots.device, rots.requires_grad
        else:
            raise ValueError("At least one input argument must be specified")
        if rots is None:
            rots = Rotation.identity(batch_dims, dtype, device, requires_grad)
        elif trans is None:
            trans = identity_trans(batch_dims, dtype, device, requires_grad)
        if rots.shape != trans.shape[:-1] or rots.device != trans.device:
            raise ValueError("Rots and trans incompatible")
        self._rots = rots
        self._trans = trans.to(dtype=torch.float32)

    @staticmethod
    def identity(shape, dtype=None, device=None, requires_grad=True, fmt="quat") -> "Rigid":
        return Rigid(Rotation.identity(shape, dtype, device, requires_grad, fmt=fmt), identity_trans(shape, dtype, device, requires_grad))

    def __getitem__(self, index: Any) -> "Rigid":
        if type(index) != tuple:
            index = (index,)
        return Rigid(self._rots[index], self._trans[index + (slice(None),)])

    def __mul__(self, right: torch.Tensor) -> "Rigid":
        return Rigid(self._rots * right, self._trans * right[..., None])

    __rmul__ = __mul__

    @property
    def shape(self):
        return self._trans.shape[:-1]

    @property
    def device(self):
        return self._trans.device

    @property
    def dtype(self):
        return self._trans.dtype

    def get_rots(self) -> Rotation:
        return self._rots

    def get_trans(self) -> torch.Tensor:
        return self._trans

    def compose_q_update_vec(self, q_update_vec: torch.Tensor) -> "Rigid":
        """Backbone update: the first three numbers rotate, the last three translate (in the local frame)."""
        q_vec, t_vec = q_update_vec[..., :3], q_update_vec[..., 3:]
        new_rots = self._rots.compose_q_update_vec(q_vec)
        return Rigid(new_rots, self._trans + self._rots.apply(t_vec))

    def compose(self, r: "Rigid") -> "Rigid":
        return Rigid(self._rots.compose_r(r._rots), self._rots.apply(r._trans) + self._trans)

    def apply(self, pts: torch.Tensor) -> torch.Tensor:
        return self._rots.apply(pts) + self._trans

    def invert_apply(self, pts: torch.Tensor) -> torch.Tensor:
        return self._rots.invert_apply(pts - self._trans)

    def invert(self) -> "Rigid":
        rot_inv = self._rots.invert()
        return Rigid(rot_inv, -1 * rot_inv.apply(self._trans))

    def map_tensor_fn(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "Rigid":
        new_trans = torch.stack(list(map(fn, torch.unbind(self._trans, dim=-1))), dim=-1)
        return Rigid(self._rots.map_tensor_fn(fn), new_trans)

    def to_tensor_4x4(self) -> torch.Tensor:
        tensor = self._trans.new_zeros((*self.shape, 4, 4))
        tensor[..., :3, :3] = self._rots.get_rot_mats()
        tensor[..., :3, 3] = self._trans
        tensor[..., 3, 3] = 1
        return tensor

    @staticmethod
    def from_tensor_4x4(t: torch.Tensor) -> "Rigid":
        if t.shape[-2:] != (4, 4):
            raise ValueError("Incorrectly shaped input tensor")
        return Rigid(Rotation(rot_mats=t[..., :3, :3]), t[..., :3, 3])

    def to_tensor_7(self) -> torch.Tensor:
        tensor = self._trans.new_zeros((*self.shape, 7))
        tensor[..., :4] = self._rots.get_quats()
        tensor[..., 4:] = self._trans
        return tensor

    @staticmethod
    def from_tensor_7(t: torch.Tensor, normalize_quats: bool = False) -> "Rigid":
        if t.shape[-1] != 7:
            raise ValueError("Incorrectly shaped input tensor")
        return Rigid(Rotation(quats=t[..., :4], normalize_quats=normalize_quats), t[..., 4:])

    @staticmethod
    def from_3_points(p_neg_x_axis: torch.Tensor, origin: torch.Tensor, p_xy_plane: torch.Tensor, eps: float = 1e-8) -> "Rigid":
        """Gram-Schmidt frame from three points (Algorithm 21): x axis from ``p_neg_x_axis`` to ``origin``."""
        e0 = origin - p_neg_x_axis
        e1 = p_xy_plane - origin
        e0 = e0 / torch.sqrt(torch.sum(e0 ** 2, dim=-1, keepdim=True) + eps)
        e1 = e1 - e0 * torch.sum(e0 * e1, dim=-1, keepdim=True)
        e1 = e1 / torch.sqrt(torch.sum(e1 ** 2, dim=-1, keepdim=True) + eps)
        e2 = torch.cross(e0, e1, dim=-1)
        rots = torch.stack([e0, e1, e2], dim=-1)
        return Rigid(Rotation(rot_mats=rots), origin)

    def unsqueeze(self, dim: int) -> "Rigid":
        if dim >= len(self.shape):
            raise ValueError("Invalid dimension")
        return Rigid(self._rots.unsqueeze(dim), self._trans.unsqueeze(dim if dim >= 0 else dim - 1))

    @staticmethod
    def cat(ts: Sequence["Rigid"], dim: int) -> "Rigid":
        rots = Rotation.cat([t._rots for t in ts], dim)
        trans = torch.cat([t._trans for t in ts], dim=dim if dim >= 0 else dim - 1)
        return Rigid(rots, trans)

    def apply_rot_fn(self, fn: Callable[[Rotation], Rotation]) -> "Rigid":
        return Rigid(fn(self._rots), self._trans)

    def apply_trans_fn(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "Rigid":
        return Rigid(self._rots, fn(self._trans))

    def scale_translation(self, trans_scale_factor: float) -> "Rigid":
        return self.apply_trans_fn(lambda t: t * trans_scale_factor)

    def stop_rot_gradient(self) -> "Rigid":
        return self.apply_rot_fn(lambda r: r.detach())

    @staticmethod
    def make_transform_from_reference(n_xyz, ca_xyz, c_xyz, eps=1e-20) -> "Rigid":
        """Backbone frame from N, CA, C coordinates with CA at the origin and C on the x axis side (Algorithm 21,
        the rotation-by-rotation construction used for template / ground-truth frames)."""
        translation = -1 * ca_xyz
        n_xyz = n_xyz + translation
        c_xyz = c_xyz + translation
        c_x, c_y, c_z = [c_xyz[..., i] for i in range(3)]
        norm = torch.sqrt(eps + c_x ** 2 + c_y ** 2)
        sin_c1, cos_c1 = -c_y / norm, c_x / norm
        c1_rots = sin_c1.new_zeros((*sin_c1.shape, 3, 3))
        c1_rots[..., 0, 0], c1_rots[..., 0, 1] = cos_c1, -1 * sin_c1
        c1_rots[..., 1, 0], c1_rots[..., 1, 1] = sin_c1, cos_c1
        c1_rots[..., 2, 2] = 1
        norm = torch.sqrt(eps + c_x ** 2 + c_y ** 2 + c_z ** 2)
        sin_c2, cos_c2 = c_z / norm, torch.sqrt(c_x ** 2 + c_y ** 2) / norm
        c2_rots = sin_c2.new_zeros((*sin_c2.shape, 3, 3))
        c2_rots[..., 0, 0], c2_rots[..., 0, 2] = cos_c2, sin_c2
        c2_rots[..., 1, 1] = 1
        c2_rots[..., 2, 0], c2_rots[..., 2, 2] = -1 * sin_c2, cos_c2
        c_rots = rot_matmul(c2_rots, c1_rots)
        n_xyz = rot_vec_mul(c_rots, n_xyz)
        _, n_y, n_z = [n_xyz[..., i] for i in range(3)]
        norm = torch.sqrt(eps + n_y ** 2 + n_z ** 2)
        sin_n, cos_n = -n_z / norm, n_y / norm
        n_rots = sin_c2.new_zeros((*sin_c2.shape, 3, 3))
        n_rots[..., 0, 0] = 1
        n_rots[..., 1, 1], n_rots[..., 1, 2] = cos_n, -1 * sin_n
        n_rots[..., 2, 1], n_rots[..., 2, 2] = sin_n, cos_n
        rots = rot_matmul(n_rots, c_rots).transpose(-1, -2)
        return Rigid(Rotation(rot_mats=rots), -1 * translation)

    def cuda(self) -> "Rigid":
        return Rigid(self._rots.cuda(), self._trans.cuda())

    def to(self, device=None, dtype=None) -> "Rigid":
        return Rigid(self._rots.to(device=device, dtype=dtype), self._trans.to(device=device, dtype=dtype))
