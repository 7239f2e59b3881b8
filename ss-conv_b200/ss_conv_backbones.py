"""Plain sparse steerable backbones (interface of Common_utils/ss_conv_backbones.py:16-176): stacks
of SS_Conv blocks in four modules; the last block of a module is followed by an average pool
(kernel 3, stride 2) that halves the grid.  All blocks of a module share one indice_key, so the
rulebook of the module's first (submanifold) block serves all of them - including the last block,
which is declared non-submanifold but finds the cached rulebook under its key, exactly as in the
reference (SS_Conv_lib/ss_conv/sp_ops/conv.py:124-136).

On this library a module queues without a host round trip (row counts stay on the device), so a
whole backbone can be recorded into one CUDA graph (ss_conv.graph.GraphedChain)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ss_conv.pool import AvgPool
from ss_conv_modules import SS_Conv


class _basic_backbone(nn.Module):
    def __init__(self, irreps, strided_layers, kernel_size=3, dropout_p=0.015, use_bn=True, pool_type='avg'):
        super().__init__()
        module_index = 0
        modules = [[] for _ in range(len(strided_layers) + 1)]
        for i in range(len(irreps) - 1):
            subm = (i + 1) not in strided_layers
            modules[module_index].append(
                SS_Conv(irreps[i], irreps[i + 1], kernel_size, padding=kernel_size // 2, stride=1, subm=subm,
                        activation=(F.relu, torch.sigmoid), dropout_p=dropout_p, indice_key='key_' + str(module_index),
                        use_bn=use_bn, activation_checkpoint=False))
            if (i + 1) in strided_layers:
                assert pool_type == 'avg'
                modules[module_index].append(AvgPool(kernel_size, stride=2, padding=kernel_size // 2))
                module_index += 1
        self.module1 = nn.Sequential(*modules[0])
        self.module2 = nn.Sequential(*modules[1])
        self.module3 = nn.Sequential(*modules[2])
        self.module4 = nn.Sequential(*modules[3])

    def forward(self, inputs):
        feats1 = self.module1(inputs)
        feats2 = self.module2(feats1)
        feats3 = self.module3(feats2)
        feats4 = self.module4(feats3)
        return feats1, feats2, feats3, feats4


def _w(m):
    """Multiplicity m for every order l = 0..3."""
    return (m, m, m, m)


class Plain12(_basic_backbone):
    """12 blocks, widths 16-32-64-128-256 channels, pools after blocks 2, 6, 10
    (Common_utils/ss_conv_backbones.py:66-93)."""

    def __init__(self, irrep_in=(4,), dropout_p=0.015, use_bn=True, pool_type='avg'):
        irreps = [irrep_in, _w(1), _w(2)] + [_w(2)] * 3 + [_w(4)] + [_w(4)] * 3 + [_w(8)] + [_w(8), _w(16)]
        super().__init__(irreps, [2, 6, 10], dropout_p=dropout_p, use_bn=use_bn, pool_type=pool_type)


class Plain24Lite(_basic_backbone):
    """24 blocks at half the width of Plain24 (Common_utils/ss_conv_backbones.py:96-134)."""

    def __init__(self, irrep_in=(4,), dropout_p=0.015, use_bn=True, pool_type='avg'):
        irreps = [irrep_in] + [_w(2)] * 3 + [_w(4)] * 12 + [_w(8)] * 9
        super().__init__(irreps, [6, 12, 18], dropout_p=dropout_p, use_bn=use_bn, pool_type=pool_type)


class Plain24(_basic_backbone):
    """24 blocks: (4,4,4,4) x 3, (8,8,8,8) x 12, (16,16,16,16) x 9; pools after blocks 6, 12, 18
    (Common_utils/ss_conv_backbones.py:137-176)."""

    def __init__(self, irrep_in=(4,), dropout_p=0.015, use_bn=True, pool_type='avg'):
        irreps = [irrep_in] + [_w(4)] * 3 + [_w(8)] * 12 + [_w(16)] * 9
        super().__init__(irreps, [6, 12, 18], dropout_p=dropout_p, use_bn=use_bn, pool_type=pool_type)
