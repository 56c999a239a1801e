"""Invariant point attention core (csrc/ipa.cu): logits, online softmax and the three weighted sums in one kernel.

``ipa_core`` takes the projected queries / keys / values, the global-frame points, the pair tensor and the bias
projection, and returns ``o [rows, H, C]``, ``o_pt [rows, H, Pv, 3]`` (global frame) and ``o_pair [rows, H, c_z]`` in
fp32.  ``ipa_core_ref`` is the same mathematics in plain PyTorch (the oracle of the GPU test and the CPU path).
Replaces lines 383-505 of the reference's fastfold/model/nn/structure_module.py between the projections and the
output projection.
"""
import ctypes
import math

import torch

from . import _lib

_declared = False


def _fn():
    global _declared
    lib = _lib.get()
    if not _declared:
        P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.ffb_ipa_fwd.argtypes = [P] * 14 + [I] * 8 + [F, F, F, P]
        lib.ffb_ipa_fwd.restype = I
        _declared = True
    return lib.ffb_ipa_fwd


def supported(q, q_pts, v_pts, z):
    return (z.is_cuda and z.dtype == torch.bfloat16 and q.dim() == 3 and q.shape[1] == 12 and q.shape[2] == 16 and q_pts.shape[-2] == 4
            and v_pts.shape[-2] == 8 and z.dim() == 3 and z.shape[-1] == 128 and z.is_contiguous() and not torch.is_grad_enabled())


def ipa_core_ref(q, k, v, q_pts, k_pts, v_pts, z, wb, bb, gamma, mask, w_c, w_b, inf, row0=0):
    """fp32 reference; ``z [rows, N, c_z]`` holds query rows ``row0 .. row0 + rows``."""
    rows = z.shape[0]
    qf, kf, vf = q.float()[row0:row0 + rows], k.float(), v.float()
    zf = z.float()
    a = w_c * torch.einsum("ihc,jhc->hij", qf, kf)
    a = a + w_b * (torch.einsum("ijc,hc->hij", zf, wb.float()) + bb.float()[:, None, None])
    d2 = ((q_pts.float()[row0:row0 + rows, None] - k_pts.float()[None]) ** 2).sum(-1).sum(-1)        # [i, j, h]
    a = a - 0.5 * gamma.float()[:, None, None] * d2.permute(2, 0, 1)
    a = a + inf * (mask.float()[row0:row0 + rows, None] * mask.float()[None, :] - 1.0)[None]
    a = torch.softmax(a, dim=-1)
    o = torch.einsum("hij,jhc->ihc", a, vf)
    o_pt = torch.einsum("hij,jhpx->ihpx", a, v_pts.float())
    o_pair = torch.einsum("hij,ijc->ihc", a, zf)
    return o, o_pt, o_pair


def ipa_core(q, k, v, q_pts, k_pts, v_pts, z, wb, bb, gamma, mask, w_c, w_b, inf, row0=0):
    """``q, k, v [N, H, C]``; ``*_pts [N, H, P, 3]`` (global frame); ``z [rows, N, c_z]`` bf16 = query rows
    ``row0 ..``; ``wb [H, c_z]``, ``bb [H]``: pair-bias projection; ``gamma [H]``: point weights; ``mask [N]``."""
    if not supported(q, q_pts, v_pts, z):
        return ipa_core_ref(q, k, v, q_pts, k_pts, v_pts, z, wb, bb, gamma, mask, w_c, w_b, inf, row0)
    f32 = lambda t: t.float().contiguous()
    q, k, v, q_pts, k_pts, v_pts, wb, bb, gamma, mask = (f32(t) for t in (q, k, v, q_pts, k_pts, v_pts, wb, bb, gamma, mask))
    N, H, C = q.shape
    rows = z.shape[0]
    o = torch.empty(rows, H, C, device=z.device, dtype=torch.float32)
    o_pt = torch.empty(rows, H, v_pts.shape[-2], 3, device=z.device, dtype=torch.float32)
    o_pair = torch.empty(rows, H, z.shape[-1], device=z.device, dtype=torch.float32)
    rc = _fn()(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(q_pts), _lib.ptr(k_pts), _lib.ptr(v_pts), _lib.ptr(z), _lib.ptr(wb), _lib.ptr(bb),
               _lib.ptr(gamma), _lib.ptr(mask), _lib.ptr(o), _lib.ptr(o_pt), _lib.ptr(o_pair), N, H, C, q_pts.shape[-2], v_pts.shape[-2],
               z.shape[-1], row0, rows, float(w_c), float(w_b), float(inf), _lib.stream_ptr())
    _lib.check(rc, "ffb_ipa_fwd(N=%d, rows=%d)" % (N, rows))
    return o, o_pt, o_pair
