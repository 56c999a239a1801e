"""Auxiliary heads: pLDDT, distogram, masked-MSA, experimentally-resolved, TM / PAE (cf. fastfold/model/nn/heads.py)."""
import torch
import torch.nn as nn

from .primitives import LayerNorm, Linear


def compute_plddt(logits):
    num_bins = logits.shape[-1]
    bin_width = 1.0 / num_bins
    bounds = torch.arange(start=0.5 * bin_width, end=1.0, step=bin_width, device=logits.device)
    probs = torch.nn.functional.softmax(logits, dim=-1)
    return torch.sum(probs * bounds.view(*((1,) * len(probs.shape[:-1])), *bounds.shape), dim=-1) * 100


def _calculate_bin_centers(boundaries):
    step = boundaries[1] - boundaries[0]
    centers = boundaries + step / 2
    return torch.cat([centers, (centers[-1] + step).unsqueeze(-1)], dim=0)


def compute_predicted_aligned_error(logits, max_bin=31, no_bins=64, **kwargs):
    boundaries = torch.linspace(0, max_bin, steps=(no_bins - 1), device=logits.device)
    probs = torch.nn.functional.softmax(logits, dim=-1)
    centers = _calculate_bin_centers(boundaries)
    return {"aligned_confidence_probs": probs, "predicted_aligned_error": torch.sum(probs * centers, dim=-1),
            "max_predicted_aligned_error": centers[-1]}


def compute_tm(logits, residue_weights=None, max_bin=31, no_bins=64, eps=1e-8, **kwargs):
    if residue_weights is None:
        residue_weights = logits.new_ones(logits.shape[-2])
    boundaries = torch.linspace(0, max_bin, steps=(no_bins - 1), device=logits.device)
    centers = _calculate_bin_centers(boundaries)
    n = logits.shape[-2]
    clipped_n = max(n, 19)
    d0 = 1.24 * (clipped_n - 15) ** (1.0 / 3) - 1.8
    probs = torch.nn.functional.softmax(logits, dim=-1)
    tm_per_bin = 1.0 / (1 + (centers ** 2) / (d0 ** 2))
    predicted_tm_term = torch.sum(probs * tm_per_bin, dim=-1)
    normed = residue_weights / (eps + residue_weights.sum())
    per_alignment = torch.sum(predicted_tm_term * normed, dim=-1)
    weighted = per_alignment * residue_weights
    argmax = (weighted == torch.max(weighted)).nonzero()[0]
    return per_alignment[tuple(argmax)]


class PerResidueLDDTCaPredictor(nn.Module):
    def __init__(self, no_bins, c_in, c_hidden):
        super().__init__()
        self.layer_norm = LayerNorm(c_in)
        self.linear_1 = Linear(c_in, c_hidden, init="relu")
        self.linear_2 = Linear(c_hidden, c_hidden, init="relu")
        self.linear_3 = Linear(c_hidden, no_bins, init="final")
        self.relu = nn.ReLU()

    def forward(self, s):
        s = self.relu(self.linear_1(self.layer_norm(s)))
        return self.linear_3(self.relu(self.linear_2(s)))


class DistogramHead(nn.Module):
    def __init__(self, c_z, no_bins, **kwargs):
        super().__init__()
        self.linear = Linear(c_z, no_bins, init="final")

    def forward(self, z):
        logits = self.linear(z)
        if z.shape[-3] != z.shape[-2]:
            # row shard [N/P, N, c] under DAP: the transposed term logits[j, i] for the local rows i is the column shard
            # of the logits, obtained with one axis switch
            from ...parallel import comm
            cols = comm.row_to_col(logits.unsqueeze(0)).squeeze(0)            # [N, N/P, bins]
            return logits + cols.transpose(-2, -3)
        return logits + logits.transpose(-2, -3)


class TMScoreHead(nn.Module):
    def __init__(self, c_z, no_bins, **kwargs):
        super().__init__()
        self.linear = Linear(c_z, no_bins, init="final")

    def forward(self, z):
        return self.linear(z)


class MaskedMSAHead(nn.Module):
    def __init__(self, c_m, c_out, **kwargs):
        super().__init__()
        self.linear = Linear(c_m, c_out, init="final")

    def forward(self, m):
        return self.linear(m)


class ExperimentallyResolvedHead(nn.Module):
    def __init__(self, c_s, c_out, **kwargs):
        super().__init__()
        self.linear = Linear(c_s, c_out, init="final")

    def forward(self, s):
        return self.linear(s)


class AuxiliaryHeads(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.plddt = PerResidueLDDTCaPredictor(**config["lddt"])
        self.distogram = DistogramHead(**config["distogram"])
        self.masked_msa = MaskedMSAHead(**config["masked_msa"])
        self.experimentally_resolved = ExperimentallyResolvedHead(**config["experimentally_resolved"])
        if config.tm.enabled:
            self.tm = TMScoreHead(**config.tm)
        self.config = config

    def forward(self, outputs):
        aux = {}
        lddt_logits = self.plddt(outputs["sm"]["single"])
        aux["lddt_logits"] = lddt_logits
        aux["plddt"] = compute_plddt(lddt_logits)
        aux["distogram_logits"] = self.distogram(outputs["pair"])
        aux["masked_msa_logits"] = self.masked_msa(outputs["msa"])
        aux["experimentally_resolved_logits"] = self.experimentally_resolved(outputs["single"])
        if self.config.tm.enabled:
            tm_logits = self.tm(outputs["pair"])
            aux["tm_logits"] = tm_logits
            aux["predicted_tm_score"] = compute_tm(tm_logits, **self.config.tm)
            aux.update(compute_predicted_aligned_error(tm_logits, **self.config.tm))
        return aux
