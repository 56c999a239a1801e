"""Struct-of-arrays geometry used by the multimer code paths: ``Vec3Array``, ``Rot3Array``, ``Rigid3Array``.

Every component is its own tensor (x, y, z / xx..zz), so that products are written out term by term and stay in the
precision of their inputs instead of going through ``matmul`` (which may pick reduced precision).  Same role as
fastfold/utils/geometry/{vector,rotation_matrix,rigid_matrix_vector,quat_rigid}.py.
"""
import dataclasses
from typing import Tuple

import torch


@dataclasses.dataclass(frozen=True)
class Vec3Array:
    x: torch.Tensor
    y: torch.Tensor
    z: torch.Tensor

    def __add__(self, o):
        return Vec3Array(self.x + o.x, self.y + o.y, self.z + o.z)

    def __sub__(self, o):
        return Vec3Array(self.x - o.x, self.y - o.y, self.z - o.z)

    def __mul__(self, s):
        return Vec3Array(self.x * s, self.y * s, self.z * s)

    __rmul__ = __mul__

    def __truediv__(self, s):
        return Vec3Array(self.x / s, self.y / s, self.z / s)

    def __neg__(self):
        return Vec3Array(-self.x, -self.y, -self.z)

    def __getitem__(self, idx):
        return Vec3Array(self.x[idx], self.y[idx], self.z[idx])

    def __iter__(self):
        return iter((self.x, self.y, self.z))

    @property
    def shape(self):
        return self.x.shape

    def map_tensor_fn(self, fn):
        return Vec3Array(fn(self.x), fn(self.y), fn(self.z))

    def cross(self, o):
        return Vec3Array(self.y * o.z - self.z * o.y, self.z * o.x - self.x * o.z, self.x * o.y - self.y * o.x)

    def dot(self, o):
        return self.x * o.x + self.y * o.y + self.z * o.z

    def norm2(self):
        return self.dot(self)

    def norm(self, epsilon: float = 1e-6):
        return torch.sqrt(torch.clamp(self.norm2(), min=epsilon ** 2))

    def normalized(self, epsilon: float = 1e-6):
        return self / self.norm(epsilon)

    def to_tensor(self):
        return torch.stack([self.x, self.y, self.z], dim=-1)

    def clone(self):
        return self.map_tensor_fn(torch.clone)

    def reshape(self, new_shape):
        return self.map_tensor_fn(lambda t: t.reshape(new_shape))

    def sum(self, dim: int):
        return self.map_tensor_fn(lambda t: t.sum(dim=dim))

    def unsqueeze(self, dim: int):
        return self.map_tensor_fn(lambda t: t.unsqueeze(dim))

    @classmethod
    def from_array(cls, t):
        return cls(*torch.unbind(t, dim=-1))

    @classmethod
    def zeros(cls, shape, device="cpu", dtype=torch.float32):
        z = torch.zeros(shape, dtype=dtype, device=device)
        return cls(z, z.clone(), z.clone())

    @classmethod
    def cat(cls, vecs, dim: int):
        return cls(torch.cat([v.x for v in vecs], dim=dim), torch.cat([v.y for v in vecs], dim=dim), torch.cat([v.z for v in vecs], dim=dim))


def dot(vector1: Vec3Array, vector2: Vec3Array):
    return vector1.dot(vector2)


def cross(vector1: Vec3Array, vector2: Vec3Array) -> Vec3Array:
    return vector1.cross(vector2)


def norm(vector: Vec3Array, epsilon: float = 1e-6):
    return vector.norm(epsilon)


def normalized(vector: Vec3Array, epsilon: float = 1e-6) -> Vec3Array:
    return vector.normalized(epsilon)


def get_field_names(cls):
    """Names of the tensor components of one of the struct-of-arrays classes, in declaration order."""
    return [f.name for f in dataclasses.fields(cls)]


def square_euclidean_distance(a: Vec3Array, b: Vec3Array, epsilon: float = 1e-6):
    d = a - b
    return torch.clamp(d.norm2(), min=epsilon)


def euclidean_distance(a: Vec3Array, b: Vec3Array, epsilon: float = 1e-6):
    return torch.sqrt(square_euclidean_distance(a, b, epsilon ** 2))


def dihedral_angle(a: Vec3Array, b: Vec3Array, c: Vec3Array, d: Vec3Array):
    v1, v2, v3 = a - b, b - c, d - c
    c1, c2 = v1.cross(v2), v3.cross(v2)
    c3 = c2.cross(c1)
    return torch.atan2(c3.dot(v2), v2.norm() * c1.dot(c2))


@dataclasses.dataclass(frozen=True)
class Rot3Array:
    xx: torch.Tensor
    xy: torch.Tensor
    xz: torch.Tensor
    yx: torch.Tensor
    yy: torch.Tensor
    yz: torch.Tensor
    zx: torch.Tensor
    zy: torch.Tensor
    zz: torch.Tensor

    def __getitem__(self, idx):
        return Rot3Array(*(getattr(self, f.name)[idx] for f in dataclasses.fields(self)))

    @property
    def shape(self):
        return self.xx.shape

    def inverse(self):
        return Rot3Array(self.xx, self.yx, self.zx, self.xy, self.yy, self.zy, self.xz, self.yz, self.zz)

    def apply_to_point(self, p: Vec3Array) -> Vec3Array:
        return Vec3Array(self.xx * p.x + self.xy * p.y + self.xz * p.z, self.yx * p.x + self.yy * p.y + self.yz * p.z,
                         self.zx * p.x + self.zy * p.y + self.zz * p.z)

    def apply_inverse_to_point(self, p: Vec3Array) -> Vec3Array:
        return self.inverse().apply_to_point(p)

    def __matmul__(self, o):
        c0 = self.apply_to_point(Vec3Array(o.xx, o.yx, o.zx))
        c1 = self.apply_to_point(Vec3Array(o.xy, o.yy, o.zy))
        c2 = self.apply_to_point(Vec3Array(o.xz, o.yz, o.zz))
        return Rot3Array(c0.x, c1.x, c2.x, c0.y, c1.y, c2.y, c0.z, c1.z, c2.z)

    def to_tensor(self):
        return torch.stack([torch.stack([self.xx, self.xy, self.xz], -1), torch.stack([self.yx, self.yy, self.yz], -1),
                            torch.stack([self.zx, self.zy, self.zz], -1)], dim=-2)

    def map_tensor_fn(self, fn):
        return Rot3Array(*(fn(getattr(self, f.name)) for f in dataclasses.fields(self)))

    def unsqueeze(self, dim: int):
        return self.map_tensor_fn(lambda t: t.unsqueeze(dim))

    def reshape(self, new_shape):
        return self.map_tensor_fn(lambda t: t.reshape(new_shape))

    def stop_gradient(self):
        return self.map_tensor_fn(lambda t: t.detach())

    @classmethod
    def cat(cls, rots, dim: int):
        return cls(*(torch.cat([getattr(r, f.name) for r in rots], dim=dim) for f in dataclasses.fields(cls)))

    @classmethod
    def from_array(cls, t):
        r = [torch.unbind(row, dim=-1) for row in torch.unbind(t, dim=-2)]
        return cls(r[0][0], r[0][1], r[0][2], r[1][0], r[1][1], r[1][2], r[2][0], r[2][1], r[2][2])

    @classmethod
    def identity(cls, shape, device="cpu", dtype=torch.float32):
        o, z = torch.ones(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device)
        return cls(o, z, z, z, o, z, z, z, o)

    @classmethod
    def from_two_vectors(cls, e0: Vec3Array, e1: Vec3Array):
        """Rotation whose x axis is ``e0`` and whose xy plane contains ``e1`` (Gram-Schmidt)."""
        e0 = e0.normalized()
        e1 = (e1 - e0 * e1.dot(e0)).normalized()
        e2 = e0.cross(e1)
        return cls(e0.x, e1.x, e2.x, e0.y, e1.y, e2.y, e0.z, e1.z, e2.z)

    @classmethod
    def from_quaternion(cls, w, x, y, z, normalize=True, eps=1e-6, epsilon=None):
        eps = eps if epsilon is None else epsilon
        if normalize:
            inv = torch.rsqrt(torch.clamp(w * w + x * x + y * y + z * z, min=eps))
            w, x, y, z = w * inv, x * inv, y * inv, z * inv
        return cls(1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y), 2 * (x * y + w * z), 1 - 2 * (x * x + z * z),
                   2 * (y * z - w * x), 2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y))


@dataclasses.dataclass(frozen=True)
class Rigid3Array:
    rotation: Rot3Array
    translation: Vec3Array

    def __getitem__(self, idx):
        return Rigid3Array(self.rotation[idx], self.translation[idx])

    @property
    def shape(self):
        return self.rotation.shape

    def __matmul__(self, o):
        return Rigid3Array(self.rotation @ o.rotation, self.apply_to_point(o.translation))

    def inverse(self):
        inv = self.rotation.inverse()
        return Rigid3Array(inv, -inv.apply_to_point(self.translation))

    def apply_to_point(self, p: Vec3Array) -> Vec3Array:
        return self.rotation.apply_to_point(p) + self.translation

    def apply_inverse_to_point(self, p: Vec3Array) -> Vec3Array:
        return self.rotation.apply_inverse_to_point(p - self.translation)

    def scale_translation(self, factor):
        return Rigid3Array(self.rotation, self.translation * factor)

    def map_tensor_fn(self, fn):
        return Rigid3Array(self.rotation.map_tensor_fn(fn), self.translation.map_tensor_fn(fn))

    def apply(self, point: torch.Tensor) -> Vec3Array:
        """``apply_to_point`` for a plain ``[..., 3]`` tensor."""
        return self.apply_to_point(Vec3Array.from_array(point))

    def compose_rotation(self, other_rotation: Rot3Array):
        return Rigid3Array(self.rotation @ other_rotation, self.translation)

    def compose(self, other_rigid):
        return self @ other_rigid

    def unsqueeze(self, dim: int):
        return self.map_tensor_fn(lambda t: t.unsqueeze(dim))

    def reshape(self, new_shape):
        return self.map_tensor_fn(lambda t: t.reshape(new_shape))

    def stop_rot_gradient(self):
        return Rigid3Array(self.rotation.stop_gradient(), self.translation)

    @property
    def dtype(self):
        return self.rotation.xx.dtype

    @property
    def device(self):
        return self.rotation.xx.device

    def to_tensor(self) -> torch.Tensor:
        """``[..., 3, 4]``: the rotation matrix with the translation as the fourth column."""
        return torch.cat([self.rotation.to_tensor(), self.translation.to_tensor()[..., None]], dim=-1)

    @classmethod
    def from_array(cls, array):
        """Inverse of ``to_tensor``."""
        return cls(Rot3Array.from_array(array[..., :3]), Vec3Array.from_array(array[..., 3]))

    @classmethod
    def from_array4x4(cls, array):
        return cls.from_tensor_4x4(array)

    @classmethod
    def cat(cls, rigids, dim: int):
        return cls(Rot3Array.cat([r.rotation for r in rigids], dim), Vec3Array.cat([r.translation for r in rigids], dim))

    def to_tensor_4x4(self):
        rot = self.rotation.to_tensor()
        top = torch.cat([rot, self.translation.to_tensor()[..., None]], dim=-1)
        bottom = torch.zeros_like(top[..., :1, :])
        bottom[..., 0, 3] = 1
        return torch.cat([top, bottom], dim=-2)

    @classmethod
    def from_tensor_4x4(cls, t):
        return cls(Rot3Array.from_array(t[..., :3, :3]), Vec3Array.from_array(t[..., :3, 3]))

    @classmethod
    def identity(cls, shape, device="cpu", dtype=torch.float32):
        return cls(Rot3Array.identity(shape, device, dtype), Vec3Array.zeros(shape, device, dtype))


class QuatRigid(torch.nn.Module):
    """Rigid update predicted as the imaginary part of a quaternion (real part 1) and a translation - the multimer
    structure module's backbone update (fastfold/utils/geometry/quat_rigid.py)."""

    def __init__(self, c_hidden, full_quat=False):
        super().__init__()
        self.full_quat = full_quat
        self.linear = torch.nn.Linear(c_hidden, 7 if full_quat else 6)
        torch.nn.init.zeros_(self.linear.weight)
        torch.nn.init.zeros_(self.linear.bias)

    def forward(self, activations) -> Rigid3Array:
        out = torch.unbind(self.linear(activations.float()), dim=-1)
        if self.full_quat:
            qw, qx, qy, qz = out[:4]
        else:
            qx, qy, qz = out[:3]
            qw = torch.ones_like(qx)
        return Rigid3Array(Rot3Array.from_quaternion(qw, qx, qy, qz, normalize=True), Vec3Array(*out[-3:]))


# ---------------------------------------------------------------------------
# assertions for tests (fastfold/utils/geometry/test_utils.py)
# ---------------------------------------------------------------------------
def _np(t):
    return t.detach().cpu().numpy() if torch.is_tensor(t) else t


def assert_rotation_matrix_equal(matrix1: Rot3Array, matrix2: Rot3Array):
    import numpy as np
    for f in dataclasses.fields(Rot3Array):
        np.testing.assert_array_equal(_np(getattr(matrix1, f.name)), _np(getattr(matrix2, f.name)))


def assert_rotation_matrix_close(mat1: Rot3Array, mat2: Rot3Array, atol=1e-6):
    import numpy as np
    np.testing.assert_allclose(_np(mat1.to_tensor()), _np(mat2.to_tensor()), atol=atol)


def assert_array_equal_to_rotation_matrix(array, matrix: Rot3Array):
    import numpy as np
    np.testing.assert_array_equal(_np(matrix.to_tensor()), _np(array))


def assert_array_close_to_rotation_matrix(array, matrix: Rot3Array, atol=1e-6):
    import numpy as np
    np.testing.assert_allclose(_np(matrix.to_tensor()), _np(array), atol=atol)


def assert_vectors_equal(vec1: Vec3Array, vec2: Vec3Array):
    import numpy as np
    for a, b in zip(vec1, vec2):
        np.testing.assert_array_equal(_np(a), _np(b))


def assert_vectors_close(vec1: Vec3Array, vec2: Vec3Array, atol=1e-6):
    import numpy as np
    for a, b in zip(vec1, vec2):
        np.testing.assert_allclose(_np(a), _np(b), atol=atol)


def assert_array_close_to_vector(array, vec: Vec3Array, atol=1e-6):
    import numpy as np
    np.testing.assert_allclose(_np(vec.to_tensor()), _np(array), atol=atol)


def assert_array_equal_to_vector(array, vec: Vec3Array):
    import numpy as np
    np.testing.assert_array_equal(_np(vec.to_tensor()), _np(array))


def assert_rigid_equal_to_rigid(rigid1: Rigid3Array, rigid2: Rigid3Array):
    assert_rot_trans_equal_to_rigid(rigid1.rotation, rigid1.translation, rigid2)


def assert_rigid_close_to_rigid(rigid1: Rigid3Array, rigid2: Rigid3Array, atol=1e-6):
    assert_rot_trans_close_to_rigid(rigid1.rotation, rigid1.translation, rigid2, atol)


def assert_rot_trans_equal_to_rigid(rot: Rot3Array, trans: Vec3Array, rigid: Rigid3Array):
    assert_rotation_matrix_equal(rot, rigid.rotation)
    assert_vectors_equal(trans, rigid.translation)


def assert_rot_trans_close_to_rigid(rot: Rot3Array, trans: Vec3Array, rigid: Rigid3Array, atol=1e-6):
    assert_rotation_matrix_close(rot, rigid.rotation, atol)
    assert_vectors_close(trans, rigid.translation, atol)

