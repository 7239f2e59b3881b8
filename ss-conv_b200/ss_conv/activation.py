"""Gated non-linearity (interface of SS_Conv_lib/ss_conv/activation.py:16-160)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _ext
from ss_conv.utils.utils import Rs2dim

_RELU = (F.relu, torch.relu, torch.nn.functional.relu)
_SIGMOID = (torch.sigmoid, F.sigmoid)


def _act_code(fn):
    """0 identity, 1 relu, 2 sigmoid, None = not fusable."""
    if fn is None:
        return 0
    if any(fn is r for r in _RELU) or isinstance(fn, nn.ReLU):
        return 1
    if any(fn is s for s in _SIGMOID) or isinstance(fn, nn.Sigmoid):
        return 2
    return None


class _GateFn(torch.autograd.Function):
    """The fused gated activation (relu / sigmoid / identity, no biases) with the library's
    kernels in both directions."""

    @staticmethod
    def forward(ctx, x, module, s_code, g_code):
        x = x.contiguous()
        C = Rs2dim(module.Rs)
        table = module._gate_table(x.device)
        ctx.save_for_backward(x)
        ctx.module, ctx.codes, ctx.c_out = module, (s_code, g_code), C
        return _ext.bn_gate_forward(x, None, None, table, C, C, s_code, g_code, None, None)

    @staticmethod
    def backward(ctx, gy):
        (x,) = ctx.saved_tensors
        m = ctx.module
        start, length = m._field_ranges(x.device)
        return _ext.gate_backward(x, gy, ctx.c_out, m._gate_table(x.device), start, length, *ctx.codes), None, None, None


class ScalarActivation(nn.Module):
    """Holds the optional bias added before an activation of scalar channels."""

    def __init__(self, enable, bias=True, inplace=False):
        super().__init__()
        self.inplace = inplace
        self.enable = []
        for d, act in enable:
            if d == 0:
                continue
            if self.enable and self.enable[-1][1] is act:
                self.enable[-1] = (self.enable[-1][0] + d, act)
            else:
                self.enable.append((d, act))
        nbias = sum(d for d, act in self.enable if act is not None)
        self.bias = torch.nn.Parameter(torch.zeros(nbias)) if bias and nbias > 0 else None

    def forward(self, input):
        out = input if self.inplace else torch.empty_like(input)
        b1 = b2 = 0
        for d, act in self.enable:
            x = input[:, b1:b1 + d]
            if act is not None:
                if self.bias is not None:
                    x = x + self.bias[b2:b2 + d].view(1, d)
                    b2 += d
                x = act(x)
            if not self.inplace or act is not None:
                out[:, b1:b1 + d] = x
            b1 += d
        assert b1 == input.size(1)
        return out


class Activation(nn.Module):
    """Input channels [Rs channels | one gate scalar per l>0 field]; output: Rs channels.
    Scalars (first Rs entry, l=0) go through the scalar activation, every l>0 field is
    multiplied by the gate activation of its gate scalar.  relu / sigmoid / identity are fused
    in one CUDA pass; any other callable falls back to the composite of torch ops on the GPU."""

    def __init__(self, Rs, activation=(None, None), bias=True, checkpoint=True):
        super().__init__()
        self.Rs = Rs
        self.multiplicities = [m for m, _ in Rs]
        self.orders = [l for _, l in Rs]
        self.checkpoint = checkpoint
        scalar_activation, gate_activation = activation if type(activation) is tuple else (activation, activation)
        self._scalar_fn, self._gate_fn = scalar_activation, gate_activation
        if scalar_activation is not None and self.multiplicities[0] > 0 and self.orders[0] == 0:
            self.scalar_act = ScalarActivation([(self.multiplicities[0], scalar_activation)], bias=bias)
        else:
            self.scalar_act = None
        n_non_scalar = sum(self.multiplicities[1:])
        if gate_activation is not None and n_non_scalar > 0:
            self.gate_act = ScalarActivation([(n_non_scalar, gate_activation)], bias=bias)
        else:
            self.gate_act = None
        self._table = None

    def _gate_table(self, device):
        """Per output channel: -2 copy, -1 scalar activation, g >= 0 gate index."""
        if self._table is None or self._table[0] != device:
            tab, g = [], 0
            for m, l in self.Rs:
                d = 2 * l + 1
                if l == 0:
                    tab += [-1 if self.scalar_act is not None else -2] * (m * d)
                else:
                    for _ in range(m):
                        tab += [g if self.gate_act is not None else -2] * d
                        g += 1
            self._table = (device, torch.tensor(tab, dtype=torch.int32, device=device))
        return self._table[1]

    def _field_ranges(self, device):
        """Per gate scalar: first channel and length of the field it multiplies."""
        if getattr(self, "_ranges", None) is None or self._ranges[0] != device:
            start, length, ch = [], [], 0
            for m, l in self.Rs:
                d = 2 * l + 1
                for _ in range(m):
                    if l > 0:
                        start.append(ch)
                        length.append(d)
                    ch += d
            self._ranges = (device, torch.tensor(start or [0], dtype=torch.int32, device=device),
                            torch.tensor(length or [0], dtype=torch.int32, device=device))
        return self._ranges[1], self._ranges[2]

    def fusable(self):
        return _act_code(self._scalar_fn if self.scalar_act is not None else None) is not None and \
            _act_code(self._gate_fn if self.gate_act is not None else None) is not None

    def forward(self, input):
        if self.scalar_act is None and self.gate_act is None:
            return input
        aff = input._take_affine()                    # a batch norm's scale / shift still to be applied
        x = input.raw()[0]                            # row-wise: fine on a pending row count
        input.features = self._gate(x) if aff is None else self._gate(x, aff[0], aff[1])
        if input.pending():
            input._rows.post.append(self._gate)
        return input

    def _gate(self, y, scale=None, shift=None):
        C = Rs2dim(self.Rs)
        recording = torch.is_grad_enabled() and (y.requires_grad or
                                                 (self.training and any(p.requires_grad for p in self.parameters())))
        if self.fusable() and y.is_cuda and not recording:
            s_code = _act_code(self._scalar_fn) if self.scalar_act is not None else 0
            g_code = _act_code(self._gate_fn) if self.gate_act is not None else 0
            s_bias = None
            if self.scalar_act is not None and self.scalar_act.bias is not None:
                s_bias = torch.zeros(C, dtype=torch.float32, device=y.device)
                s_bias[:self.multiplicities[0]] = self.scalar_act.bias.detach()
            g_bias = self.gate_act.bias.detach() if (self.gate_act is not None and self.gate_act.bias is not None) else None
            return _ext.bn_gate_forward(y, scale, shift, self._gate_table(y.device), C, C, s_code, g_code, s_bias,
                                        g_bias, storage=_ext.get_feature_storage())
        no_bias = (self.scalar_act is None or self.scalar_act.bias is None) and \
            (self.gate_act is None or self.gate_act.bias is None)
        if self.fusable() and y.is_cuda and y.dtype == torch.float32 and no_bias and scale is None and y.shape[0] > 0:
            s_code = _act_code(self._scalar_fn) if self.scalar_act is not None else 0
            g_code = _act_code(self._gate_fn) if self.gate_act is not None else 0
            return _GateFn.apply(y, self, s_code, g_code)     # recording: the library's kernels forward and backward
        return self._gate_composite(y if scale is None else y * scale + shift)

    def _gate_composite(self, y):
        N, C = y.size(0), Rs2dim(self.Rs)
        g = self.gate_act(y[:, C:]) if self.gate_act is not None else None
        z = y.new_empty((N, C))
        by = bg = 0
        for m, l in self.Rs:
            if m == 0:
                continue
            d = 2 * l + 1
            f = y[:, by:by + m * d]
            if l == 0:
                f = self.scalar_act(f) if self.scalar_act is not None else f
            elif g is not None:
                f = (f.reshape(N, m, d) * g[:, bg:bg + m].reshape(N, m, 1)).reshape(N, m * d)
                bg += m
            z[:, by:by + m * d] = f
            by += m * d
        return z
