"""Irrep-wise dropout (interface of SS_Conv_lib/ss_conv/dropout.py): one Bernoulli mask per
field copy, shared by its 2l+1 components; identity in eval mode."""
import torch
import torch.nn as nn


class Dropout(nn.Module):
    def __init__(self, Rs, p=0.5):
        super().__init__()
        self.Rs = [(m, 2 * l + 1) for m, l in Rs]
        self.p = p

    def __repr__(self):
        return "{} (p={})".format(self.__class__.__name__, self.p)

    def forward(self, input):
        if not self.training:
            return input
        x = input.features
        n = x.size(0)
        masks = []
        for m, d in self.Rs:
            if self.p == 1:        # drop everything / keep everything without dividing by zero
                keep = x.new_zeros(n, m, 1)
            elif self.p == 0:
                keep = x.new_ones(n, m, 1)
            else:
                keep = x.new_empty(n, m, 1).bernoulli_(1 - self.p) / (1 - self.p)
            masks.append(keep.expand(n, m, d).reshape(n, m * d))
        input.features = x * torch.cat(masks, dim=1)
        return input
