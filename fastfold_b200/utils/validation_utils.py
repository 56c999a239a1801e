"""Validation metrics logged during training: lDDT-CA, dRMSD-CA and, after superposition, RMSD / GDT-TS / GDT-HA.

Same role as fastfold/utils/validation_utils.py:75-127 and superimposition.py.
"""
import torch

from ..common import residue_constants as rc


def drmsd(structure_1, structure_2, mask=None):
    def prep(s):
        d = s[..., :, None, :] - s[..., None, :, :]
        return torch.sqrt(torch.sum(d ** 2, dim=-1))
    d1, d2 = prep(structure_1), prep(structure_2)
    sq = (d1 - d2) ** 2
    if mask is not None:
        sq = sq * (mask[..., None] * mask[..., None, :])
    n = d1.shape[-1] if mask is None else torch.sum(mask, dim=-1)
    sq = torch.sum(sq, dim=(-1, -2))
    return torch.sqrt(sq * (1 / (n * (n - 1))) if mask is None else sq / (n * (n - 1)).clamp(min=1))


def superimpose(reference, coords, mask):
    """Kabsch superposition of ``coords`` onto ``reference`` over masked points -> (superimposed coords, rmsd)."""
    m = mask[..., None]
    n = mask.sum(-1, keepdim=True).clamp(min=1)[..., None]
    rc_, cc = (reference * m).sum(-2, keepdim=True) / n, (coords * m).sum(-2, keepdim=True) / n
    a, b = (reference - rc_) * m, (coords - cc) * m
    h = b.transpose(-1, -2) @ a
    u, _, vt = torch.linalg.svd(h.float())
    d = torch.sign(torch.linalg.det(u @ vt))
    dm = torch.diag_embed(torch.stack([torch.ones_like(d), torch.ones_like(d), d], dim=-1))
    rot = u @ dm @ vt
    sup = (coords - cc) @ rot.to(coords.dtype) + rc_
    rmsd = torch.sqrt((((sup - reference) ** 2).sum(-1) * mask).sum(-1) / mask.sum(-1).clamp(min=1))
    return sup, rmsd


def gdt(p1, p2, mask, cutoffs):
    n = torch.sum(mask, dim=-1).clamp(min=1)
    d = torch.sqrt(torch.sum((p1 - p2) ** 2, dim=-1))
    scores = [torch.sum((d <= c) * mask, dim=-1) / n for c in cutoffs]
    return sum(scores) / len(scores)


def gdt_ts(p1, p2, mask):
    return gdt(p1, p2, mask, [1.0, 2.0, 4.0, 8.0])


def gdt_ha(p1, p2, mask):
    return gdt(p1, p2, mask, [0.5, 1.0, 2.0, 4.0])


def validation_metrics(outputs, batch, superimposition_metrics=False):
    from ..models.hub.loss import lddt_ca
    metrics = {}
    gt, pred, mask = batch["all_atom_positions"].float(), outputs["final_atom_positions"].float(), batch["all_atom_mask"].float()
    metrics["lddt_ca"] = torch.mean(lddt_ca(pred, gt, mask, eps=1e-10, per_residue=False))
    ca = rc.atom_order["CA"]
    gt_ca, pred_ca, mask_ca = gt[..., ca, :], pred[..., ca, :], mask[..., ca]
    metrics["drmsd_ca"] = torch.mean(drmsd(pred_ca, gt_ca, mask=mask_ca))
    if superimposition_metrics:
        sup, rmsd = superimpose(gt_ca, pred_ca, mask_ca)
        metrics["alignment_rmsd"] = torch.mean(rmsd)
        metrics["gdt_ts"] = torch.mean(gdt_ts(sup, gt_ca, mask_ca))
        metrics["gdt_ha"] = torch.mean(gdt_ha(sup, gt_ca, mask_ca))
    return metrics


def drmsd_np(structure_1, structure_2, mask=None):
    """``drmsd`` on numpy inputs (returns a tensor, like the reference's helper of that name)."""
    return drmsd(torch.as_tensor(structure_1), torch.as_tensor(structure_2), None if mask is None else torch.as_tensor(mask))


def compute_validation_metrics(batch, outputs, superimposition_metrics=False):
    """The reference's argument order (``batch`` first) for ``validation_metrics``."""
    return validation_metrics(outputs, batch, superimposition_metrics=superimposition_metrics)

