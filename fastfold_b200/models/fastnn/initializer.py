"""AlphaFold-style Glorot-uniform initialiser (fan computed over the last two dims, JAX convention).

Same role as fastfold/model/fastnn/initializer.py:7-29.
"""
import math

import torch.nn as nn


def glorot_uniform_af(x, gain=1.0):
    fan_in, fan_out = x.shape[-2:]
    if x.dim() > 2:
        rf = 1
        for s in x.shape[:-2]:
            rf *= s
        fan_in *= rf
        fan_out *= rf
    std = gain * math.sqrt(2.0 / float(fan_in + fan_out))
    bound = math.sqrt(3.0) * std
    nn.init.uniform_(x, -bound, bound)
    return x
