"""Irrep-wise batch normalisation (interface of SS_Conv_lib/ss_conv/batchnorm.py:13-136)."""
import torch
import torch.nn as nn

from . import _ext


def _channel_tables(Rs):
    """Per channel: index of its field (one per irrep copy) and of its scalar slot (-1 for l>0)."""
    field, scalar = [], []
    f = s = 0
    for m, l in Rs:
        d = 2 * l + 1
        for _ in range(m):
            field += [f] * d
            scalar += [s if d == 1 else -1] * d
            f += 1
            if d == 1:
                s += 1
    return field, scalar


class _BatchNormFn(torch.autograd.Function):
    """y = (x - mean) * weight / sqrt(var + eps) + bias with the library's kernels in both directions.
    Training mode: mean / var are the batch statistics (ssc_bn_stats) and the gradient flows through
    them; eval mode: the running buffers, constants."""

    @staticmethod
    def forward(ctx, x, weight, bias, module, training):
        x = x.contiguous()
        field, scalar = module._device_tables(x.device)
        n_field, n_scalar = module.running_var.numel(), module.running_mean.numel()
        if training:
            mean, var = _ext.bn_stats(x, field, scalar, n_field, n_scalar)
            with torch.no_grad():
                module.running_mean.mul_(1 - module.momentum).add_(module.momentum * mean)
                module.running_var.mul_(1 - module.momentum).add_(module.momentum * var)
        else:
            mean, var = module.running_mean.clone(), module.running_var.clone()
        w = None if weight is None else weight.detach().contiguous()
        b = None if (bias is None or n_scalar == 0) else bias.detach().contiguous()
        scale, shift = _ext.bn_fold(mean if n_scalar > 0 else None, var, w, b, field, scalar, module.eps)
        y = _ext.bn_gate_forward(x, scale, shift, None, x.size(1), 0, 0, 0, None, None)
        ctx.save_for_backward(x, mean, var, w if w is not None else x.new_empty(0))
        ctx.tables, ctx.sizes, ctx.eps, ctx.training_mode = (field, scalar), (n_field, n_scalar), module.eps, bool(training)
        ctx.has_w, ctx.has_b = weight is not None, bias is not None
        return y

    @staticmethod
    def backward(ctx, gy):
        x, mean, var, w = ctx.saved_tensors
        field, scalar = ctx.tables
        n_field, n_scalar = ctx.sizes
        gx, d_w, d_b = _ext.bn_backward(x, gy, field, scalar, n_field, n_scalar, mean, var, w if ctx.has_w else None,
                                        ctx.eps, ctx.training_mode)
        return gx, (d_w if ctx.has_w else None), (d_b if ctx.has_b else None), None, None


class BatchNorm(nn.Module):
    """Scalars (l=0) are centred and scaled; fields with l>0 are only scaled by the running mean
    of their squared norm, which keeps the layer equivariant.  Same parameters and buffers as
    the reference (`running_mean` [n_scalar], `running_var` [n_fields], `weight`, `bias`).

    Eval mode is one fused CUDA pass y = x*scale + shift with the statistics folded into
    per-channel constants.  Training mode computes batch statistics on the GPU (two
    reductions, added in a fixed order), updates the running buffers and applies the same pass.
    While autograd records, the same kernels run inside an autograd Function whose backward is the
    library's batch-norm gradient (through the batch statistics in training mode); only an
    unsupported `reduce` option or a CPU tensor takes the composite of torch ops."""

    def __init__(self, Rs, eps=1e-5, momentum=0.1, affine=True, reduce='mean'):
        super().__init__()
        self.Rs = Rs
        self.eps = eps
        self.momentum = momentum
        self.affine = affine
        self.reduce = reduce
        num_scalar = sum(m for m, l in Rs if l == 0)
        num_features = sum(m for m, l in Rs)
        self.register_buffer('running_mean', torch.zeros(num_scalar))
        self.register_buffer('running_var', torch.ones(num_features))
        if affine:
            self.weight = nn.Parameter(torch.ones(num_features))
            self.bias = nn.Parameter(torch.zeros(num_scalar))
        else:
            self.register_parameter('weight', None)
            self.register_parameter('bias', None)
        self._tables = None

    def __repr__(self):
        return "{} (Rs={}, eps={}, momentum={})".format(self.__class__.__name__, self.Rs, self.eps, self.momentum)

    def _device_tables(self, device):
        if self._tables is None or self._tables[0] != device:
            field, scalar = _channel_tables(self.Rs)
            self._tables = (device, torch.tensor(field, dtype=torch.int32, device=device),
                            torch.tensor(scalar, dtype=torch.int32, device=device))
        return self._tables[1], self._tables[2]

    def folded_affine(self, device, mean=None, var=None):
        """(scale, shift) per channel for the given statistics (default: running buffers)."""
        field, scalar = self._device_tables(device)
        running = mean is None and var is None
        mean = self.running_mean if mean is None else mean
        var = self.running_var if var is None else var
        w = self.weight.detach() if self.affine else None
        b = self.bias.detach() if self.affine else None
        # the fold of the running buffers is kept until one of its inputs changes (in-place updates bump
        # a tensor's version, moves and reloads change its address): an eval-mode network folds once
        key = None
        if running:
            key = tuple((t.data_ptr(), t._version) for t in (mean, var, w, b) if t is not None) + (str(device), self.eps)
            kept = getattr(self, "_folded", None)
            if kept is not None and kept[0] == key:
                return kept[1]
        if mean.numel() == 0:
            mean = None
            b = None
        folded = _ext.bn_fold(mean, var, w, b, field, scalar, self.eps)
        if key is not None:
            self._folded = (key, folded)
        return folded

    def _differentiable(self, x):
        """The layer as a composite of torch ops, used while autograd is recording so that
        gradients reach the input, the affine parameters and (training mode) the batch
        statistics; same arithmetic as the fused path."""
        parts = []
        new_mean, new_var = [], []
        ix = irm = irv = 0
        for m, l in self.Rs:
            d = 2 * l + 1
            f = x[:, ix:ix + m * d].reshape(-1, m, d)
            if d == 1:
                if self.training:
                    mu = f.mean(0).reshape(m)
                    new_mean.append(mu.detach())
                else:
                    mu = self.running_mean[irm:irm + m]
                f = f - mu.reshape(1, m, 1)
            if self.training:
                norm = f.pow(2).sum(2).mean(0)
                new_var.append(norm.detach())
            else:
                norm = self.running_var[irv:irv + m]
            scale = (norm + self.eps).pow(-0.5)
            if self.affine:
                scale = scale * self.weight[irv:irv + m]
            f = f * scale.reshape(1, m, 1)
            if d == 1 and self.affine:
                f = f + self.bias[irm:irm + m].reshape(1, m, 1)
            parts.append(f.reshape(-1, m * d))
            if d == 1:
                irm += m
            irv += m
            ix += m * d
        if self.training:
            with torch.no_grad():
                if new_mean:
                    self.running_mean.mul_(1 - self.momentum).add_(self.momentum * torch.cat(new_mean))
                self.running_var.mul_(1 - self.momentum).add_(self.momentum * torch.cat(new_var))
        return torch.cat(parts, dim=1)

    def forward(self, input):
        # inference without no_grad() (nothing upstream asks for a gradient) keeps the fused kernels
        if torch.is_grad_enabled() and (input.raw()[0].requires_grad or
                                        (self.training and self.affine and self.weight.requires_grad)):
            if self.training and self.reduce != 'mean':
                raise ValueError("Invalid reduce option {}".format(self.reduce))
            feats = input.features
            if feats.is_cuda and feats.dtype == torch.float32 and feats.shape[0] > 0:
                input.features = _BatchNormFn.apply(feats, self.weight if self.affine else None,
                                                    self.bias if self.affine else None, self, self.training)
            else:
                input.features = self._differentiable(feats)
            return input
        # eval mode works row by row, so it can run on a tensor whose row count is still pending
        x = input.features if self.training else input.raw()[0]
        field, scalar = self._device_tables(x.device)
        if field.numel() != x.size(1):
            raise AssertionError("`ix` should have reached features.size(1) ({}), but it ended at {}".format(
                x.size(1), field.numel()))
        if self.training:
            if self.reduce != 'mean':
                raise ValueError("Invalid reduce option {}".format(self.reduce))
            mean, var = _ext.bn_stats(x, field, scalar, self.running_var.numel(), self.running_mean.numel())
            scale, shift = self.folded_affine(x.device, mean, var)
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(self.momentum * mean)
                self.running_var.mul_(1 - self.momentum).add_(self.momentum * var)
        else:
            scale, shift = self.folded_affine(x.device)

        def apply(f):
            return _ext.bn_gate_forward(f, scale, shift, None, f.size(1), 0, 0, 0, None, None)

        if self.training:
            input.features = apply(x)
        else:
            input._affine = (scale, shift)   # applied by the next reader, fused into a gated Activation if that is next
        if input.pending():
            input._rows.post.append(apply)
        return input
