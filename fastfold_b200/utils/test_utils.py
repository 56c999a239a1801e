"""Fixtures for tests and examples: deterministic seeding and the locations of optional external test data.

``set_seed`` as fastfold/utils/test_utils.py:25-32.  The data paths are read from the environment (the reference
hard-codes cluster paths): ``FASTFOLD_PARAM_PATH`` (an AlphaFold ``params_model_*.npz``), ``FASTFOLD_DATA_PATH`` (a pickled
inference batch) and ``FASTFOLD_TRAIN_DATA_PATH`` (a pickled training batch); a missing variable yields ``None`` and the
tests that need the file skip themselves.
"""
import os
import random

import numpy as np
import torch


def get_param_path():
    return os.environ.get("FASTFOLD_PARAM_PATH")


def get_data_path():
    return os.environ.get("FASTFOLD_DATA_PATH")


def get_train_data_path():
    return os.environ.get("FASTFOLD_TRAIN_DATA_PATH")


def set_seed(seed):
    random.seed(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
