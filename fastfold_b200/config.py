"""Model / data / loss configuration with named presets.

``model_config(name, train=False, low_prec=False)`` returns the configuration tree of a preset
(``initial_training``, ``finetuning``, ``model_1`` .. ``model_5`` and their ``_ptm`` variants, ``multimer``), as a
``ConfigDict``: a nested dict with attribute access.  Values shared by many sub-trees (channel widths, ``eps``,
``chunk_size``, ``blocks_per_ckpt``) are ``Ref`` cells: assigning through any alias, or ``config.set_shared(name,
value)``, updates every place that refers to it.  No third-party config library is involved (the reference builds
the same tree on ``ml_collections``: fastfold/config.py:30-125 presets, :128-533 tree, :535-606 multimer).
"""
import copy
from collections.abc import Mapping, MutableMapping


class Ref:
    """A shared mutable cell; ``ConfigDict`` reads through it transparently."""
    __slots__ = ("value", "name")

    def __init__(self, value, name=None):
        self.value = value
        self.name = name

    def __repr__(self):
        return "Ref(%r)" % (self.value,)


class ConfigDict(MutableMapping):
    """Nested mapping with attribute access, transparent ``Ref`` cells and ``ml_collections``-like helpers.

    (Deliberately not a ``dict`` subclass: ``**cfg`` on a dict subclass bypasses ``__getitem__`` and would hand out
    the ``Ref`` cells themselves.)"""

    def __init__(self, init=None):
        object.__setattr__(self, "_d", {})
        for k, v in (init or {}).items():
            self._d[k] = ConfigDict(v) if isinstance(v, Mapping) and not isinstance(v, ConfigDict) else v

    def __getitem__(self, k):
        v = self._d[k]
        return v.value if isinstance(v, Ref) else v

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k)

    def __setitem__(self, k, v):
        cur = self._d.get(k)
        if isinstance(cur, Ref) and not isinstance(v, Ref):
            cur.value = v
        else:
            self._d[k] = ConfigDict(v) if isinstance(v, Mapping) and not isinstance(v, ConfigDict) else v

    def __setattr__(self, k, v):
        self[k] = v

    def __delitem__(self, k):
        del self._d[k]

    def __iter__(self):
        return iter(self._d)

    def __len__(self):
        return len(self._d)

    def __contains__(self, k):
        return k in self._d

    def __repr__(self):
        return "ConfigDict(%r)" % (self.to_dict(),)

    def raw(self, k):
        """The stored object (a ``Ref`` for shared values)."""
        return self._d[k]

    def to_dict(self):
        return {k: (v.to_dict() if isinstance(v, ConfigDict) else v) for k, v in self.items()}

    def update_from(self, other):
        for k, v in other.items():
            if isinstance(v, Mapping) and isinstance(self.get(k), ConfigDict):
                self[k].update_from(v)
            else:
                self[k] = v

    def unlocked(self):
        return _Null()

    def __deepcopy__(self, memo):
        out = ConfigDict()
        for k, v in self._d.items():
            out._d[k] = copy.deepcopy(v, memo)
        return out

    def __getstate__(self):
        return self._d

    def __setstate__(self, d):
        object.__setattr__(self, "_d", d)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def set_inf(c, inf):
    for k in list(c.keys()):
        if k == "_shared":
            continue
        v = c[k]
        if isinstance(v, ConfigDict):
            set_inf(v, inf)
        elif k == "inf":
            c[k] = inf


NUM_RES = "num residues placeholder"
NUM_MSA_SEQ = "msa placeholder"
NUM_EXTRA_SEQ = "extra msa placeholder"
NUM_TEMPLATES = "num templates placeholder"


def _base_config():
    c_z, c_m, c_t, c_e, c_s = (Ref(128, "c_z"), Ref(256, "c_m"), Ref(64, "c_t"), Ref(64, "c_e"), Ref(384, "c_s"))
    blocks_per_ckpt = Ref(None, "blocks_per_ckpt")
    chunk_size = Ref(None, "chunk_size")
    max_extra_msa = Ref(1024, "max_extra_msa")        # one value for every mode, also reachable as data.common.max_extra_msa
    aux_distogram_bins = Ref(64, "aux_distogram_bins")
    tm_enabled = Ref(False, "tm_enabled")
    eps = Ref(1e-8, "eps")
    templates_enabled = Ref(True, "templates_enabled")
    embed_template_torsion_angles = Ref(True, "embed_template_torsion_angles")
    shared = {"c_z": c_z, "c_m": c_m, "c_t": c_t, "c_e": c_e, "c_s": c_s, "blocks_per_ckpt": blocks_per_ckpt, "chunk_size": chunk_size,
              "aux_distogram_bins": aux_distogram_bins, "tm_enabled": tm_enabled, "eps": eps, "templates_enabled": templates_enabled,
              "embed_template_torsion_angles": embed_template_torsion_angles, "max_extra_msa": max_extra_msa}
    feat = {
        "aatype": [NUM_RES], "all_atom_mask": [NUM_RES, None], "all_atom_positions": [NUM_RES, None, None],
        "alt_chi_angles": [NUM_RES, None], "atom14_alt_gt_exists": [NUM_RES, None], "atom14_alt_gt_positions": [NUM_RES, None, None],
        "atom14_atom_exists": [NUM_RES, None], "atom14_atom_is_ambiguous": [NUM_RES, None], "atom14_gt_exists": [NUM_RES, None],
        "atom14_gt_positions": [NUM_RES, None, None], "atom37_atom_exists": [NUM_RES, None], "backbone_rigid_mask": [NUM_RES],
        "backbone_rigid_tensor": [NUM_RES, None, None], "bert_mask": [NUM_MSA_SEQ, NUM_RES], "chi_angles_sin_cos": [NUM_RES, None, None],
        "chi_mask": [NUM_RES, None], "extra_deletion_value": [NUM_EXTRA_SEQ, NUM_RES], "extra_has_deletion": [NUM_EXTRA_SEQ, NUM_RES],
        "extra_msa": [NUM_EXTRA_SEQ, NUM_RES], "extra_msa_mask": [NUM_EXTRA_SEQ, NUM_RES], "extra_msa_row_mask": [NUM_EXTRA_SEQ],
        "is_distillation": [], "msa_feat": [NUM_MSA_SEQ, NUM_RES, None], "msa_mask": [NUM_MSA_SEQ, NUM_RES], "msa_row_mask": [NUM_MSA_SEQ],
        "no_recycling_iters": [], "pseudo_beta": [NUM_RES, None], "pseudo_beta_mask": [NUM_RES], "residue_index": [NUM_RES],
        "residx_atom14_to_atom37": [NUM_RES, None], "residx_atom37_to_atom14": [NUM_RES, None], "resolution": [],
        "rigidgroups_alt_gt_frames": [NUM_RES, None, None, None], "rigidgroups_group_exists": [NUM_RES, None],
        "rigidgroups_group_is_ambiguous": [NUM_RES, None], "rigidgroups_gt_exists": [NUM_RES, None],
        "rigidgroups_gt_frames": [NUM_RES, None, None, None], "seq_length": [], "seq_mask": [NUM_RES], "target_feat": [NUM_RES, None],
        "template_aatype": [NUM_TEMPLATES, NUM_RES], "template_all_atom_mask": [NUM_TEMPLATES, NUM_RES, None],
        "template_all_atom_positions": [NUM_TEMPLATES, NUM_RES, None, None], "template_alt_torsion_angles_sin_cos": [NUM_TEMPLATES, NUM_RES, None, None],
        "template_backbone_rigid_mask": [NUM_TEMPLATES, NUM_RES], "template_backbone_rigid_tensor": [NUM_TEMPLATES, NUM_RES, None, None],
        "template_mask": [NUM_TEMPLATES], "template_pseudo_beta": [NUM_TEMPLATES, NUM_RES, None], "template_pseudo_beta_mask": [NUM_TEMPLATES, NUM_RES],
        "template_sum_probs": [NUM_TEMPLATES, None], "template_torsion_angles_mask": [NUM_TEMPLATES, NUM_RES, None],
        "template_torsion_angles_sin_cos": [NUM_TEMPLATES, NUM_RES, None, None], "true_msa": [NUM_MSA_SEQ, NUM_RES], "use_clamped_fape": [],
    }
    mode_common = {"fixed_size": True, "subsample_templates": False, "masked_msa_replace_fraction": 0.15, "max_msa_clusters": 128,
                   "max_extra_msa": max_extra_msa, "max_template_hits": 4, "max_templates": 4, "crop": False, "crop_size": None, "supervised": False,
                   "uniform_recycling": False}
    cfg = {
        "data": {
            "common": {
                "feat": feat,
                "masked_msa": {"profile_prob": 0.1, "same_prob": 0.1, "uniform_prob": 0.1},
                "max_extra_msa": max_extra_msa, "max_recycling_iters": 3, "msa_cluster_features": True, "reduce_msa_clusters_by_max_templates": False, "resample_msa_in_recycling": True,
                "template_features": ["template_all_atom_positions", "template_sum_probs", "template_aatype", "template_all_atom_mask"],
                "unsupervised_features": ["aatype", "residue_index", "msa", "num_alignments", "seq_length", "between_segment_residues", "deletion_matrix",
                                          "no_recycling_iters"],
                "use_templates": templates_enabled, "use_template_torsion_angles": embed_template_torsion_angles,
            },
            "supervised": {"clamp_prob": 0.9, "supervised_features": ["all_atom_mask", "all_atom_positions", "resolution", "use_clamped_fape",
                                                                      "is_distillation"]},
            "predict": dict(mode_common, masked_msa_replace_fraction=0.15),
            "eval": dict(mode_common, subsample_templates=False, supervised=True),
            "train": dict(mode_common, subsample_templates=True, crop=True, crop_size=256, supervised=True, clamp_prob=0.9,
                          max_distillation_msa_clusters=1000, uniform_recycling=True, distillation_prob=0.75, shuffle_top_k_prefiltered=20),
            "data_module": {"use_small_bfd": False, "data_loaders": {"batch_size": 1, "num_workers": 16}},
        },
        "globals": {"blocks_per_ckpt": blocks_per_ckpt, "chunk_size": chunk_size, "c_z": c_z, "c_m": c_m, "c_t": c_t, "c_e": c_e, "c_s": c_s,
                    "eps": eps, "inplace": False, "is_multimer": False, "shard_pair": False},
        "model": {
            "_mask_trans": False,
            "input_embedder": {"tf_dim": 22, "msa_dim": 49, "c_z": c_z, "c_m": c_m, "relpos_k": 32},
            "recycling_embedder": {"c_z": c_z, "c_m": c_m, "min_bin": 3.25, "max_bin": 20.75, "no_bins": 15, "inf": 1e8},
            "template": {
                "distogram": {"min_bin": 3.25, "max_bin": 50.75, "no_bins": 39},
                "template_angle_embedder": {"c_in": 57, "c_out": c_m},
                "template_pair_embedder": {"c_in": 88, "c_out": c_t},
                "template_pair_stack": {"c_t": c_t, "c_hidden_tri_att": 16, "c_hidden_tri_mul": 64, "no_blocks": 2, "no_heads": 4,
                                        "pair_transition_n": 2, "dropout_rate": 0.25, "blocks_per_ckpt": blocks_per_ckpt, "inf": 1e9},
                "template_pointwise_attention": {"c_t": c_t, "c_z": c_z, "c_hidden": 16, "no_heads": 4, "inf": 1e5},
                "inf": 1e5, "eps": eps, "enabled": templates_enabled, "embed_angles": embed_template_torsion_angles, "use_unit_vector": False,
            },
            "extra_msa": {
                "extra_msa_embedder": {"c_in": 25, "c_out": c_e},
                "extra_msa_stack": {"c_m": c_e, "c_z": c_z, "c_hidden_msa_att": 8, "c_hidden_opm": 32, "c_hidden_mul": 128, "c_hidden_pair_att": 32,
                                    "no_heads_msa": 8, "no_heads_pair": 4, "no_blocks": 4, "transition_n": 4, "msa_dropout": 0.15, "pair_dropout": 0.25,
                                    "clear_cache_between_blocks": True, "inf": 1e9, "eps": eps, "ckpt": True},
                "enabled": True,
            },
            "evoformer_stack": {"c_m": c_m, "c_z": c_z, "c_hidden_msa_att": 32, "c_hidden_opm": 32, "c_hidden_mul": 128, "c_hidden_pair_att": 32,
                                "c_s": c_s, "no_heads_msa": 8, "no_heads_pair": 4, "no_blocks": 48, "transition_n": 4, "msa_dropout": 0.15,
                                "pair_dropout": 0.25, "blocks_per_ckpt": blocks_per_ckpt, "clear_cache_between_blocks": False, "inf": 1e9, "eps": eps},
            "structure_module": {"c_s": c_s, "c_z": c_z, "c_ipa": 16, "c_resnet": 128, "no_heads_ipa": 12, "no_qk_points": 4, "no_v_points": 8,
                                 "dropout_rate": 0.1, "no_blocks": 8, "no_transition_layers": 1, "no_resnet_blocks": 2, "no_angles": 7,
                                 "trans_scale_factor": 10, "epsilon": eps, "inf": 1e5},
            "heads": {
                "lddt": {"no_bins": 50, "c_in": c_s, "c_hidden": 128},
                "distogram": {"c_z": c_z, "no_bins": aux_distogram_bins},
                "tm": {"c_z": c_z, "no_bins": aux_distogram_bins, "enabled": tm_enabled},
                "masked_msa": {"c_m": c_m, "c_out": 23},
                "experimentally_resolved": {"c_s": c_s, "c_out": 37},
            },
        },
        "relax": {"max_iterations": 0, "tolerance": 2.39, "stiffness": 10.0, "max_outer_iterations": 20, "exclude_residues": []},
        "loss": {
            "distogram": {"min_bin": 2.3125, "max_bin": 21.6875, "no_bins": 64, "eps": eps, "weight": 0.3},
            "experimentally_resolved": {"eps": eps, "min_resolution": 0.1, "max_resolution": 3.0, "weight": 0.0},
            "fape": {"backbone": {"clamp_distance": 10.0, "loss_unit_distance": 10.0, "weight": 0.5},
                     "sidechain": {"clamp_distance": 10.0, "length_scale": 10.0, "weight": 0.5}, "eps": 1e-4, "weight": 1.0},
            "lddt": {"min_resolution": 0.1, "max_resolution": 3.0, "cutoff": 15.0, "no_bins": 50, "eps": eps, "weight": 0.01},
            "masked_msa": {"eps": eps, "weight": 2.0},
            "supervised_chi": {"chi_weight": 0.5, "angle_norm_weight": 0.01, "eps": eps, "weight": 1.0},
            "violation": {"violation_tolerance_factor": 12.0, "clash_overlap_tolerance": 1.5, "eps": eps, "weight": 0.0},
            "tm": {"max_bin": 31, "no_bins": 64, "min_resolution": 0.1, "max_resolution": 3.0, "eps": eps, "weight": 0.0, "enabled": tm_enabled},
            "eps": eps,
        },
        "ema": {"decay": 0.999},
    }
    c = ConfigDict(cfg)
    c._d["_shared"] = shared
    return c


def set_shared(config, name, value):
    """Sets one of the shared values (``c_m``, ``c_z``, ``c_t``, ``c_e``, ``c_s``, ``eps``, ``chunk_size``,
    ``blocks_per_ckpt``, ``templates_enabled``, ``tm_enabled`` ...) everywhere it is referenced."""
    config._d["_shared"][name].value = value


def _multimer_overrides(c):
    c.globals.is_multimer = True
    c.data.predict.max_msa_clusters = 252
    c.data.common.unsupervised_features = list(c.data.common.unsupervised_features) + ["msa_mask", "seq_mask", "asym_id", "entity_id", "sym_id"]
    c.model.input_embedder.update_from({"tf_dim": 21, "max_relative_idx": 32, "use_chain_relative": True, "max_relative_chain": 2})
    c.model.template.update_from({"template_single_embedder": {"c_in": 34, "c_m": c.globals.c_m},
                                  "template_pair_embedder": {"c_z": c.globals.c_z, "c_out": 64, "c_dgram": 39, "c_aatype": 22},
                                  "c_t": c.globals.c_t, "c_z": c.globals.c_z})
    c.model.template.template_pair_stack.tri_mul_first = True
    c.model.heads.masked_msa.c_out = 22
    c.model.structure_module.trans_scale_factor = 20
    c.loss.update_from({"chain_center_of_mass": {"clamp_distance": -4.0, "weight": 0.05, "eps": 1e-8, "enabled": False}})
    set_shared(c, "tm_enabled", True)
    c.loss.tm.weight = 0.1


def model_config(name, train=False, low_prec=False):
    c = _base_config()
    if name == "initial_training":
        pass
    elif name == "finetuning":
        c.data.train.max_extra_msa = 5120
        c.data.train.crop_size = 384
        c.data.train.max_msa_clusters = 512
        c.loss.violation.weight = 1.0
        c.loss.experimentally_resolved.weight = 0.01
    elif name in ("model_1", "model_2", "model_1_ptm", "model_2_ptm"):
        c.data.train.max_extra_msa = 5120 if name.startswith("model_1") else 1024
        c.data.predict.max_extra_msa = 5120 if name.startswith("model_1") else 1024
        c.data.common.reduce_max_clusters_by_max_templates = True
        c.data.common.use_templates = True
        c.data.common.use_template_torsion_angles = True
        c.model.template.enabled = True
    elif name in ("model_3", "model_4", "model_5", "model_3_ptm", "model_4_ptm", "model_5_ptm"):
        big = name.startswith(("model_3", "model_4"))
        c.data.train.max_extra_msa = 5120 if big else 1024
        c.data.predict.max_extra_msa = 5120 if big else 1024
        set_shared(c, "templates_enabled", False)
        set_shared(c, "embed_template_torsion_angles", False)
    elif name.startswith("multimer") or "multimer" in name:
        _multimer_overrides(c)
    else:
        raise ValueError("Invalid model name: %s" % name)
    if name.endswith("_ptm"):
        set_shared(c, "tm_enabled", True)
        c.loss.tm.weight = 0.1
    if train:
        set_shared(c, "blocks_per_ckpt", 1)
        set_shared(c, "chunk_size", None)
    if low_prec:
        set_shared(c, "eps", 1e-4)
        set_inf(c, 1e4)
    return c
