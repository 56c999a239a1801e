"""From a raw (numpy) example to model features: selection of the configured feature names, conversion to tensors
and the tensor pipeline of ``input_pipeline`` / ``data_transforms_multimer``.

Same entry points as fastfold/data/feature_pipeline.py:31-129: ``np_to_tensor_dict``, ``make_data_config``,
``np_example_to_features`` and the ``FeaturePipeline`` class that ``inference.py`` and the training datasets use.
"""
import copy

import numpy as np
import torch

from . import input_pipeline
from .data_pipeline import FeaturePipeline, np_to_tensor_dict          # noqa: F401  (they live beside the raw-feature pipeline)


def make_data_config(config, mode, num_res):
    """Copy of the data configuration with the crop size of ``mode`` resolved (``None`` -> the example's length) and
    the list of raw feature names that mode consumes."""
    cfg = copy.deepcopy(config)
    mode_cfg = cfg[mode]
    if mode_cfg.crop_size is None:
        mode_cfg.crop_size = num_res
    names = list(cfg.common.unsupervised_features)
    if cfg.common.use_templates:
        names += list(cfg.common.template_features)
    if mode_cfg.supervised:
        names += list(cfg.supervised.supervised_features)
    return cfg, names


def np_example_to_features(np_example, config, mode, seed=None):
    np_example = dict(np_example)
    num_res = int(np.asarray(np_example["seq_length"]).reshape(-1)[0])
    cfg, names = make_data_config(config, mode, num_res)
    if "template_all_atom_masks" in np_example:          # raw template features carry the AlphaFold spelling
        np_example["template_all_atom_mask"] = np_example.pop("template_all_atom_masks")
    if "deletion_matrix_int" in np_example:
        np_example["deletion_matrix"] = np.asarray(np_example.pop("deletion_matrix_int")).astype(np.float32)
    tensors = np_to_tensor_dict(np_example, names)
    with torch.no_grad():
        features = input_pipeline.process_tensors_from_config(tensors, cfg.common, cfg[mode], seed=seed)
    return {k: v for k, v in features.items()}
