"""Dropout with a mask shared along given dims (Algorithm 6 row-/column-wise dropout); cf. fastfold/model/nn/dropout.py."""
from functools import partialmethod

import torch
import torch.nn as nn


class Dropout(nn.Module):
    def __init__(self, r, batch_dim):
        super().__init__()
        self.r = r
        self.batch_dim = [batch_dim] if isinstance(batch_dim, int) else batch_dim
        self.dropout = nn.Dropout(self.r)

    def forward(self, x):
        shape = list(x.shape)
        for bd in self.batch_dim:
            shape[bd] = 1
        return x * self.dropout(x.new_ones(shape))


class DropoutRowwise(Dropout):
    __init__ = partialmethod(Dropout.__init__, batch_dim=-3)


class DropoutColumnwise(Dropout):
    __init__ = partialmethod(Dropout.__init__, batch_dim=-2)
