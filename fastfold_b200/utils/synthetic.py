"""Synthetic AlphaFold feature dictionaries of a named shape (no databases, no alignments).

The distributions follow the benchmark specification: ``target_feat`` one-hot over 22 classes with uniform residue
types, ``residue_index`` 0..N-1, ``msa_feat`` 49 channels = residue one-hot over 23 + has_deletion ~ Bernoulli(0.1)
+ deletion_value ~ U[0,1] + a 23-channel profile drawn from Dirichlet(1) + deletion_mean, extra-MSA features of the
same kind, and (optionally) random template features.  Every tensor gets the recycling dimension last, as the
real feature pipeline produces it.  The reference's counterpart draws ``msa_feat ~ U[0,1)`` (demo.py:36-84).
"""
import numpy as np
import torch

from ..common import residue_constants as rc


def random_features(n_res, n_seq, n_extra, n_templ=0, n_recycle=3, seed=0, device="cpu", supervised=False, chains=None):
    """``chains``: list of chain lengths summing to ``n_res`` -> multimer features (``asym_id`` / ``entity_id`` / ``sym_id``,
    per-chain ``residue_index``, 21-class ``target_feat``); chains of equal length count as copies of one entity."""
    g = torch.Generator().manual_seed(seed)
    R = n_recycle + 1
    aatype = torch.randint(0, 20, (n_res,), generator=g)
    msa = torch.randint(0, 21, (n_seq, n_res), generator=g)
    msa[0] = aatype
    has_del = (torch.rand(n_seq, n_res, generator=g) < 0.1).float()
    del_val = torch.rand(n_seq, n_res, generator=g)
    profile = torch.distributions.Dirichlet(torch.ones(23)).sample((n_res,))
    del_mean = torch.rand(n_res, generator=g)
    msa_feat = torch.cat([torch.nn.functional.one_hot(msa, 23).float(), has_del[..., None], (del_val * has_del)[..., None],
                          profile[None].expand(n_seq, -1, -1), del_mean[None, :, None].expand(n_seq, -1, -1)], dim=-1)
    target_feat = torch.nn.functional.one_hot(aatype + 1, 22).float()
    extra_msa = torch.randint(0, 21, (n_extra, n_res), generator=g)
    feats = {
        "aatype": aatype, "residue_index": torch.arange(n_res), "seq_length": torch.tensor(n_res), "target_feat": target_feat,
        "msa_feat": msa_feat, "seq_mask": torch.ones(n_res), "msa_mask": torch.ones(n_seq, n_res), "msa_row_mask": torch.ones(n_seq),
        "extra_msa": extra_msa, "extra_msa_mask": torch.ones(n_extra, n_res), "extra_msa_row_mask": torch.ones(n_extra),
        "extra_has_deletion": (torch.rand(n_extra, n_res, generator=g) < 0.1).float(),
        "extra_deletion_value": torch.rand(n_extra, n_res, generator=g),
        "bert_mask": (torch.rand(n_seq, n_res, generator=g) < 0.15).float(), "true_msa": msa,
        "atom14_atom_exists": torch.tensor(rc.restype_atom14_mask)[aatype], "atom37_atom_exists": torch.tensor(rc.restype_atom37_mask)[aatype],
        "residx_atom14_to_atom37": torch.tensor(rc.restype_atom14_to_atom37).long()[aatype],
        "residx_atom37_to_atom14": torch.tensor(rc.restype_atom37_to_atom14).long()[aatype],
    }
    if n_templ > 0:
        feats.update({
            "template_aatype": torch.randint(0, 20, (n_templ, n_res), generator=g),
            "template_all_atom_positions": torch.randn(n_templ, n_res, 37, 3, generator=g) * 5,
            "template_all_atom_mask": torch.ones(n_templ, n_res, 37),
            "template_pseudo_beta": torch.randn(n_templ, n_res, 3, generator=g) * 5,
            "template_pseudo_beta_mask": torch.ones(n_templ, n_res),
            "template_mask": torch.ones(n_templ),
            "template_torsion_angles_sin_cos": torch.randn(n_templ, n_res, 7, 2, generator=g),
            "template_alt_torsion_angles_sin_cos": torch.randn(n_templ, n_res, 7, 2, generator=g),
            "template_torsion_angles_mask": torch.ones(n_templ, n_res, 7),
            "template_sum_probs": torch.rand(n_templ, 1, generator=g),
        })
    if chains is not None:
        assert sum(chains) == n_res
        asym, entity, sym, ridx = [], [], [], []
        seen = {}
        for c, L in enumerate(chains):
            e = seen.setdefault(L, len(seen) + 1)
            copies = sum(1 for x in chains[:c] if x == L)
            asym += [c + 1] * L
            entity += [e] * L
            sym += [copies + 1] * L
            ridx += list(range(L))
        feats.update({"asym_id": torch.tensor(asym), "entity_id": torch.tensor(entity), "sym_id": torch.tensor(sym),
                      "residue_index": torch.tensor(ridx), "target_feat": torch.nn.functional.one_hot(aatype, 21).float()})
    if supervised:
        feats.update(random_ground_truth(aatype, g))
    out = {}
    for k, v in feats.items():
        out[k] = v.unsqueeze(-1).expand(*v.shape, R).contiguous().to(device)
    return out


def random_ground_truth(aatype, g):
    """A random-walk backbone with idealised side chains: enough structure for every loss term to be finite."""
    from .feats import frames_and_literature_positions_to_atom14_pos, torsion_angles_to_frames
    from .rigid_utils import Rigid, Rotation
    from ..data import data_transforms as dt
    n = aatype.shape[0]
    steps = torch.randn(n, 3, generator=g)
    ca = torch.cumsum(3.8 * steps / steps.norm(dim=-1, keepdim=True), dim=0)
    quats = torch.randn(n, 4, generator=g)
    bb = Rigid(Rotation(quats=quats, normalize_quats=True), ca)
    ang = torch.randn(n, 7, 2, generator=g)
    ang = ang / ang.norm(dim=-1, keepdim=True)
    frames = torsion_angles_to_frames(bb, ang, aatype, torch.tensor(rc.restype_rigid_group_default_frame, dtype=torch.float32))
    pos14 = frames_and_literature_positions_to_atom14_pos(frames, aatype, torch.tensor(rc.restype_rigid_group_default_frame, dtype=torch.float32),
                                                          torch.tensor(rc.restype_atom14_to_rigid_group), torch.tensor(rc.restype_atom14_mask),
                                                          torch.tensor(rc.restype_atom14_rigid_group_positions, dtype=torch.float32))
    idx37 = torch.tensor(rc.restype_atom37_to_atom14).long()[aatype]
    mask37 = torch.tensor(rc.restype_atom37_mask)[aatype]
    pos37 = torch.gather(pos14, 1, idx37[..., None].expand(-1, -1, 3)) * mask37[..., None]
    p = {"aatype": aatype, "all_atom_positions": pos37, "all_atom_mask": mask37}
    p = dt.make_atom14_masks(p)
    p = dt.make_atom14_positions(p)
    p = dt.atom37_to_frames(p)
    p = dt.atom37_to_torsion_angles("")(p)
    p = dt.make_pseudo_beta("")(p)
    p = dt.get_backbone_frames(p)
    p = dt.get_chi_angles(p)
    p["resolution"] = torch.tensor(1.0)
    p["use_clamped_fape"] = torch.tensor(1.0)
    p["is_distillation"] = torch.tensor(0.0)
    p.pop("aatype")
    return p
