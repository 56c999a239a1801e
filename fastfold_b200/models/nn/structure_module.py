"""Structure module: invariant point attention, backbone update, side-chain torsions (Algorithms 20-24).

OpenFold-layout module names (``ipa.linear_q``, ``ipa.head_weights``, ``bb_update.linear``,
``angle_resnet.layers.N.linear_1`` ...), so AlphaFold parameter archives import directly.  Eight iterations share
one set of weights; rigid-frame maths runs in fp32.  Same role as fastfold/model/nn/structure_module.py
(IPA :196-506, StructureModule :590-967, AngleResnet :72-157).
"""
import math

import torch
import torch.nn as nn

from ...common import residue_constants as rc
from ...utils.feats import frames_and_literature_positions_to_atom14_pos, torsion_angles_to_frames
from ...utils.rigid_utils import Rigid, Rotation
from ...utils.tensor_utils import dict_multimap, flatten_final_dims, permute_final_dims
from .primitives import LayerNorm, Linear, ipa_point_weights_init_


class AngleResnetBlock(nn.Module):
    def __init__(self, c_hidden):
        super().__init__()
        self.linear_1 = Linear(c_hidden, c_hidden, init="relu")
        self.linear_2 = Linear(c_hidden, c_hidden, init="final")
        self.relu = nn.ReLU()

    def forward(self, a):
        return a + self.linear_2(self.relu(self.linear_1(self.relu(a))))


class AngleResnet(nn.Module):
    """Algorithm 20, lines 11-14: torsion angles (as unnormalised and normalised sin/cos pairs) from the single rep."""

    def __init__(self, c_in, c_hidden, no_blocks, no_angles, epsilon):
        super().__init__()
        self.c_in, self.c_hidden, self.no_blocks, self.no_angles, self.eps = c_in, c_hidden, no_blocks, no_angles, epsilon
        self.linear_in = Linear(c_in, c_hidden)
        self.linear_initial = Linear(c_in, c_hidden)
        self.layers = nn.ModuleList([AngleResnetBlock(c_hidden) for _ in range(no_blocks)])
        self.linear_out = Linear(c_hidden, no_angles * 2)
        self.relu = nn.ReLU()

    def forward(self, s, s_initial):
        s = self.linear_in(self.relu(s)) + self.linear_initial(self.relu(s_initial))
        for layer in self.layers:
            s = layer(s)
        s = self.linear_out(self.relu(s))
        s = s.view(s.shape[:-1] + (-1, 2))
        unnormalized = s
        norm = torch.sqrt(torch.clamp(torch.sum(s ** 2, dim=-1, keepdim=True), min=self.eps))
        return unnormalized, s / norm


class PointProjection(nn.Module):
    """Multimer parameterisation of the point projections: one linear layer whose output is laid out
    ``[head][x | y | z][point]`` (fastfold/model/nn/structure_module.py:160-193); returns global-frame points
    ``[*, N, H, P, 3]``."""

    def __init__(self, c_hidden, num_points, no_heads, return_local_points=False):
        super().__init__()
        self.no_heads, self.num_points, self.return_local_points = no_heads, num_points, return_local_points
        self.linear = Linear(c_hidden, no_heads * 3 * num_points)

    def forward(self, activations, rigids):
        p = self.linear(activations)
        p = p.reshape(*p.shape[:-1], self.no_heads, 3, self.num_points).transpose(-1, -2)       # [*, N, H, P, 3]
        g = rigids[..., None, None].apply(p)
        return (g, p) if self.return_local_points else g


class InvariantPointAttention(nn.Module):
    """Algorithm 22.  Attention logits = scalar q.k + pair bias - weighted squared distances between query / key points
    expressed in the global frame; outputs = attended scalars, attended points (back in the local frame, plus their
    norms) and attended pair rows."""

    def __init__(self, c_s, c_z, c_hidden, no_heads, no_qk_points, no_v_points, inf=1e5, eps=1e-8, is_multimer=False):
        super().__init__()
        self.c_s, self.c_z, self.c_hidden, self.no_heads = c_s, c_z, c_hidden, no_heads
        self.no_qk_points, self.no_v_points, self.inf, self.eps = no_qk_points, no_v_points, inf, eps
        self.is_multimer = is_multimer
        hc = c_hidden * no_heads
        if is_multimer:
            # separate, bias-free q / k / v projections and one point projection per role (multimer checkpoint layout)
            self.linear_q = Linear(c_s, hc, bias=False)
            self.linear_k = Linear(c_s, hc, bias=False)
            self.linear_v = Linear(c_s, hc, bias=False)
            self.linear_q_points = PointProjection(c_s, no_qk_points, no_heads)
            self.linear_k_points = PointProjection(c_s, no_qk_points, no_heads)
            self.linear_v_points = PointProjection(c_s, no_v_points, no_heads)
        else:
            self.linear_q = Linear(c_s, hc)
            self.linear_kv = Linear(c_s, 2 * hc)
            self.linear_q_points = Linear(c_s, no_heads * no_qk_points * 3)
            self.linear_kv_points = Linear(c_s, no_heads * (no_qk_points + no_v_points) * 3)
        self.linear_b = Linear(c_z, no_heads)
        self.head_weights = nn.Parameter(torch.zeros((no_heads)))
        ipa_point_weights_init_(self.head_weights)
        concat_out_dim = no_heads * (c_z + c_hidden + no_v_points * 4)
        self.linear_out = Linear(concat_out_dim, c_s, init="final")
        self.softmax = nn.Softmax(dim=-1)
        self.softplus = nn.Softplus()

    def forward(self, s, z, r, mask):
        H = self.no_heads
        q = self.linear_q(s)
        q = q.view(q.shape[:-1] + (H, -1))
        if self.is_multimer:
            k = self.linear_k(s)
            v = self.linear_v(s)
            k = k.view(k.shape[:-1] + (H, -1))
            v = v.view(v.shape[:-1] + (H, -1))
            q_pts = self.linear_q_points(s, r)
            k_pts = self.linear_k_points(s, r)
            v_pts = self.linear_v_points(s, r)
        else:
            kv = self.linear_kv(s)
            kv = kv.view(kv.shape[:-1] + (H, -1))
            k, v = torch.split(kv, self.c_hidden, dim=-1)
            q_pts = self.linear_q_points(s)
            q_pts = torch.stack(torch.split(q_pts, q_pts.shape[-1] // 3, dim=-1), dim=-1)
            q_pts = r[..., None].apply(q_pts)
            q_pts = q_pts.view(q_pts.shape[:-2] + (H, self.no_qk_points, 3))
            kv_pts = self.linear_kv_points(s)
            kv_pts = torch.stack(torch.split(kv_pts, kv_pts.shape[-1] // 3, dim=-1), dim=-1)
            kv_pts = r[..., None].apply(kv_pts)
            kv_pts = kv_pts.view(kv_pts.shape[:-2] + (H, -1, 3))
            k_pts, v_pts = torch.split(kv_pts, [self.no_qk_points, self.no_v_points], dim=-2)
        head_w = self.softplus(self.head_weights) * math.sqrt(1.0 / (3 * (self.no_qk_points * 9.0 / 2)))
        from ...ops import ipa as ipa_op
        if s.dim() == 2 and z.shape[-3] != s.shape[-2]:
            # Row-parallel attention over the DAP group: this rank holds rows [row0, row0 + n_local) of the pair tensor,
            # which is all that queries row0 .. need (bias b[i, j] and o_pair[i] = sum_j a[i, j] z[i, j] use row i only).
            # Projections of s are replicated (tiny); the per-query outputs are all-gathered (N x 2016 floats).
            from ...parallel import comm, core
            assert not torch.is_grad_enabled(), "row-parallel invariant point attention is an inference path"
            row0 = core.get_dap_rank() * z.shape[-3]
            o, o_pt, o_pair = ipa_op.ipa_core(q, k, v, q_pts, k_pts, v_pts, z.contiguous(), self.linear_b.weight, self.linear_b.bias, head_w, mask,
                                              math.sqrt(1.0 / (3 * self.c_hidden)), math.sqrt(1.0 / 3), self.inf, row0=row0)
            o, o_pt, o_pair = (comm._gather(t.contiguous(), dim=0) for t in (o, o_pt, o_pair))
            o = flatten_final_dims(o, 2)
            o_pt = r[..., None, None].invert_apply(o_pt)
            o_pt_norm = flatten_final_dims(torch.sqrt(torch.sum(o_pt ** 2, dim=-1) + self.eps), 2)
            o_pt = o_pt.reshape(*o_pt.shape[:-3], -1, 3)
            o_pair = flatten_final_dims(o_pair, 2)
            cat = torch.cat((o, *torch.unbind(o_pt, dim=-1), o_pt_norm, o_pair), dim=-1).to(dtype=z.dtype)
            return self.linear_out(cat)
        if s.dim() == 2 and ipa_op.supported(q, q_pts, v_pts, z):
            # inference on the GPU: logits, softmax and the three weighted sums in one kernel; the pair row is read once
            # and neither the [H, N, N] attention tensor nor the [N, N, H, P, 3] point differences are materialised
            o, o_pt, o_pair = ipa_op.ipa_core(q, k, v, q_pts, k_pts, v_pts, z, self.linear_b.weight, self.linear_b.bias, head_w, mask,
                                              math.sqrt(1.0 / (3 * self.c_hidden)), math.sqrt(1.0 / 3), self.inf)
            o = flatten_final_dims(o, 2)
            o_pt = r[..., None, None].invert_apply(o_pt)
            o_pt_norm = flatten_final_dims(torch.sqrt(torch.sum(o_pt ** 2, dim=-1) + self.eps), 2)
            o_pt = o_pt.reshape(*o_pt.shape[:-3], -1, 3)
            o_pair = flatten_final_dims(o_pair, 2)
            cat = torch.cat((o, *torch.unbind(o_pt, dim=-1), o_pt_norm, o_pair), dim=-1).to(dtype=z.dtype)
            return self.linear_out(cat)
        b = self.linear_b(z)
        a = torch.matmul(permute_final_dims(q.float(), (1, 0, 2)), permute_final_dims(k.float(), (1, 2, 0)))
        a = a * math.sqrt(1.0 / (3 * self.c_hidden))
        a = a + math.sqrt(1.0 / 3) * permute_final_dims(b.float(), (2, 0, 1))
        pt_att = q_pts.unsqueeze(-4) - k_pts.unsqueeze(-5)
        pt_att = torch.sum(pt_att ** 2, dim=-1)
        head_weights = self.softplus(self.head_weights).view(*((1,) * len(pt_att.shape[:-2]) + (-1, 1)))
        head_weights = head_weights * math.sqrt(1.0 / (3 * (self.no_qk_points * 9.0 / 2)))
        pt_att = torch.sum(pt_att * head_weights, dim=-1) * (-0.5)
        square_mask = self.inf * (mask.unsqueeze(-1) * mask.unsqueeze(-2) - 1)
        a = a + permute_final_dims(pt_att, (2, 0, 1)) + square_mask.unsqueeze(-3)
        a = self.softmax(a)
        o = torch.matmul(a, v.transpose(-2, -3).to(dtype=a.dtype)).transpose(-2, -3)
        o = flatten_final_dims(o, 2)
        o_pt = torch.sum(a[..., None, :, :, None] * permute_final_dims(v_pts, (1, 3, 0, 2))[..., None, :, :], dim=-2)
        o_pt = permute_final_dims(o_pt, (2, 0, 3, 1))
        o_pt = r[..., None, None].invert_apply(o_pt)
        o_pt_norm = flatten_final_dims(torch.sqrt(torch.sum(o_pt ** 2, dim=-1) + self.eps), 2)
        o_pt = o_pt.reshape(*o_pt.shape[:-3], -1, 3)
        o_pair = torch.matmul(a.transpose(-2, -3), z.to(dtype=a.dtype))
        o_pair = flatten_final_dims(o_pair, 2)
        cat = torch.cat((o, *torch.unbind(o_pt, dim=-1), o_pt_norm, o_pair), dim=-1).to(dtype=z.dtype)
        return self.linear_out(cat)


class BackboneUpdate(nn.Module):
    """Algorithm 23: a 6-vector (quaternion imaginary part + translation) per residue."""

    def __init__(self, c_s):
        super().__init__()
        self.linear = Linear(c_s, 6, init="final")

    def forward(self, s):
        return self.linear(s)


class StructureModuleTransitionLayer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.linear_1 = Linear(c, c, init="relu")
        self.linear_2 = Linear(c, c, init="relu")
        self.linear_3 = Linear(c, c, init="final")
        self.relu = nn.ReLU()

    def forward(self, s):
        return s + self.linear_3(self.relu(self.linear_2(self.relu(self.linear_1(s)))))


class StructureModuleTransition(nn.Module):
    def __init__(self, c, num_layers, dropout_rate):
        super().__init__()
        self.layers = nn.ModuleList([StructureModuleTransitionLayer(c) for _ in range(num_layers)])
        self.dropout = nn.Dropout(dropout_rate)
        self.layer_norm = LayerNorm(c)

    def forward(self, s):
        for layer in self.layers:
            s = layer(s)
        return self.layer_norm(self.dropout(s))


class StructureModule(nn.Module):
    def __init__(self, c_s, c_z, c_ipa, c_resnet, no_heads_ipa, no_qk_points, no_v_points, dropout_rate, no_blocks, no_transition_layers,
                 no_resnet_blocks, no_angles, trans_scale_factor, epsilon, inf, is_multimer=False, **kwargs):
        super().__init__()
        self.is_multimer = is_multimer
        self.c_s, self.c_z, self.no_blocks, self.trans_scale_factor, self.epsilon, self.inf = c_s, c_z, no_blocks, trans_scale_factor, epsilon, inf
        self.default_frames = None
        self.group_idx = None
        self.atom_mask = None
        self.lit_positions = None
        self.layer_norm_s = LayerNorm(c_s)
        self.layer_norm_z = LayerNorm(c_z)
        self.linear_in = Linear(c_s, c_s)
        self.ipa = InvariantPointAttention(c_s, c_z, c_ipa, no_heads_ipa, no_qk_points, no_v_points, inf=inf, eps=epsilon, is_multimer=is_multimer)
        self.ipa_dropout = nn.Dropout(dropout_rate)
        self.layer_norm_ipa = LayerNorm(c_s)
        self.transition = StructureModuleTransition(c_s, no_transition_layers, dropout_rate)
        self.bb_update = BackboneUpdate(c_s)
        self.angle_resnet = AngleResnet(c_s, c_resnet, no_resnet_blocks, no_angles, epsilon)

    def forward(self, s, z, aatype, mask=None):
        """``s [*, N, C_s]``, ``z [*, N, N, C_z]``, ``aatype [*, N]`` -> dict of per-iteration outputs stacked on dim 0."""
        if mask is None:
            mask = s.new_ones(s.shape[:-1])
        s = self.layer_norm_s(s)
        z = self.layer_norm_z(z)
        s_initial = s
        s = self.linear_in(s)
        rigids = Rigid.identity(s.shape[:-1], s.dtype, s.device, self.training, fmt="quat")
        outputs = []
        for i in range(self.no_blocks):
            s = s + self.ipa(s, z, rigids, mask)
            s = self.ipa_dropout(s)
            s = self.layer_norm_ipa(s)
            s = self.transition(s)
            rigids = rigids.compose_q_update_vec(self.bb_update(s))
            # side chains are placed with rotation matrices; gradients keep flowing through the quaternion path above
            backb_to_global = Rigid(Rotation(rot_mats=rigids.get_rots().get_rot_mats(), quats=None), rigids.get_trans())
            backb_to_global = backb_to_global.scale_translation(self.trans_scale_factor)
            unnormalized_angles, angles = self.angle_resnet(s, s_initial)
            all_frames_to_global = self.torsion_angles_to_frames(backb_to_global, angles, aatype)
            pred_xyz = self.frames_and_literature_positions_to_atom14_pos(all_frames_to_global, aatype)
            scaled_rigids = rigids.scale_translation(self.trans_scale_factor)
            outputs.append({"frames": scaled_rigids.to_tensor_7(), "sidechain_frames": all_frames_to_global.to_tensor_4x4(),
                            "unnormalized_angles": unnormalized_angles, "angles": angles, "positions": pred_xyz})
            if i < (self.no_blocks - 1):
                rigids = rigids.stop_rot_gradient()
        outputs = dict_multimap(torch.stack, outputs)
        outputs["single"] = s
        return outputs

    def _init_residue_constants(self, float_dtype, device):
        if self.default_frames is None or self.default_frames.device != device:
            self.default_frames = torch.tensor(rc.restype_rigid_group_default_frame, dtype=float_dtype, device=device, requires_grad=False)
            self.group_idx = torch.tensor(rc.restype_atom14_to_rigid_group, device=device, requires_grad=False)
            self.atom_mask = torch.tensor(rc.restype_atom14_mask, dtype=float_dtype, device=device, requires_grad=False)
            self.lit_positions = torch.tensor(rc.restype_atom14_rigid_group_positions, dtype=float_dtype, device=device, requires_grad=False)

    def torsion_angles_to_frames(self, r, alpha, f):
        self._init_residue_constants(torch.float32, alpha.device)
        return torsion_angles_to_frames(r, alpha.float(), f, self.default_frames)

    def frames_and_literature_positions_to_atom14_pos(self, r, f):
        self._init_residue_constants(torch.float32, r.get_rots().device)
        return frames_and_literature_positions_to_atom14_pos(r, f, self.default_frames, self.group_idx, self.atom_mask, self.lit_positions)
