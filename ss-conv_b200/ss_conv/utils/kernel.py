"""Steerable kernel basis and its per-forward materialisation.

Interface of SS_Conv_lib/ss_conv/utils/kernel.py: `SE3Kernel(Rs_in, Rs_out, size, radial_window,
dyn_iso, verbose)` owns one flat parameter `weight` and one fp32 buffer `kernel_{i}_{j}` of
shape [n_basis, 2l_out+1, 2l_in+1, k, k, k] (or None) per (output irrep i, input irrep j), so
state dicts are interchangeable (kernel.py:251-255).  The basis is built once in float64 on
the host (kernel.py:30-92, 144-171, 240-249).  The contraction of the learned weights with the
basis (kernel.py:267-299) runs on the GPU as a single CUDA kernel writing the convolution
filters directly in the [K, Cin, Cout] layout the sparse convolution consumes.
"""
import math

import torch

from . import SO3
from .. import _ext

_SH_CUBE = {}


def _sample_sh_cube(size, J):
    """Spherical harmonics of order J at the k^3 kernel taps, [2J+1, k, k, k] float64."""
    key = (size, J)
    if key not in _SH_CUBE:
        rng = torch.linspace(-((size - 1) / 2), (size - 1) / 2, steps=size, dtype=torch.float64)
        xyz = torch.stack(torch.meshgrid(rng, rng, rng, indexing="ij"), dim=-1)
        _SH_CUBE[key] = SO3.spherical_harmonics_xyz(J, xyz.view(-1, 3)).view(2 * J + 1, size, size, size)
    return _SH_CUBE[key]


def _check_quarter_turn(K, order_in, order_out):
    """rho_out(u) K(u^-1 x) rho_in(u^-1) == K(x) for the quarter turn about y (kernel.py:51-61)."""
    tmp = K.transpose(-3, -1).flip(-1)
    lhs = torch.einsum("ij,...jkxyz,kl->...ilxyz",
                       SO3.irr_repr(order_out, 0, math.pi / 2, 0, dtype=K.dtype), tmp,
                       SO3.irr_repr(order_in, 0, -math.pi / 2, 0, dtype=K.dtype))
    if not torch.allclose(lhs, K, atol=1e-9):
        raise AssertionError("kernel basis is not equivariant under the quarter turn")


def _sample_cube(size, order_in, order_out):
    """Angular solutions K_J for J = |l_in-l_out| .. l_in+l_out, radius field, and the Js."""
    rng = torch.linspace(-((size - 1) / 2), (size - 1) / 2, steps=size, dtype=torch.float64)
    orders = list(range(abs(order_in - order_out), order_in + order_out + 1))
    sols = []
    for J in orders:
        Y = _sample_sh_cube(size, J)
        Q = SO3.basis_transformation_Q_J(J, order_in, order_out)
        K = torch.einsum("mn,nxyz->mxyz", Q, Y).view(2 * order_out + 1, 2 * order_in + 1, size, size, size)
        _check_quarter_turn(K, order_in, order_out)
        sols.append(K)
    r = (rng.view(-1, 1, 1) ** 2 + rng.view(1, -1, 1) ** 2 + rng.view(1, 1, -1) ** 2).sqrt()
    return sols, r, orders


def gaussian_window(solutions, r_field, order_irreps, radii, J_max_list, sigma=.6):
    """Radial Gaussian shells; shell i keeps the angular orders J <= J_max_list[i]."""
    assert len(radii) == len(J_max_list)
    out = []
    for r, jmax in zip(radii, J_max_list):
        win = torch.exp(-.5 * ((r_field - r) / sigma) ** 2) / (math.sqrt(2 * math.pi) * sigma)
        out += [sol * win for sol, J in zip(solutions, order_irreps) if J <= jmax]
    return torch.stack(out, dim=0) if out else None


def gaussian_window_wrapper(solutions, r_field, order_irreps, mode='compromise', border_dist=0., sigma=.6):
    """Predefined shell radii / band limits ('conservative', 'compromise', 'sfcnn')."""
    table = {'conservative': [0, 2, 4, 6, 8, 10, 12, 14], 'compromise': [0, 3, 5, 7, 9, 11, 13, 15],
             'sfcnn': [0, 4, 6, 8, 10, 12, 14, 16]}
    assert mode in table
    size = r_field.size(0)
    n_radial = size // 2 + 1
    radii = torch.linspace(0, size // 2 - border_dist, steps=n_radial, dtype=torch.float64)
    return gaussian_window(solutions, r_field, order_irreps, radii, table[mode][:n_radial], sigma)


def sigmoid_window(solutions, r_field, order_irreps, sharpness=5):
    size = r_field.size(0)
    n_radial = size // 2 + 1
    radii = torch.linspace(0.5, size // 2 + 0.5, steps=n_radial, dtype=torch.float64)
    out = []
    for i, r in enumerate(radii):
        win = torch.sigmoid(sharpness * (r - r_field))
        jmax = 2 * i + 1 if i > 0 else 0
        out += [sol * win for sol, J in zip(solutions, order_irreps) if J <= jmax]
    return torch.stack(out, dim=0) if out else None


def cube_basis_kernels(size, order_in, order_out, radial_window):
    """[n_basis, 2l_out+1, 2l_in+1, k, k, k] float64 basis or None."""
    basis = radial_window(*_sample_cube(size, order_in, order_out))
    if basis is not None:
        _check_quarter_turn(basis, order_in, order_out)
    return basis


def _orthogonal_(tensor, gain=1):
    rows, cols = tensor.size(0), tensor[0].numel()
    flat = tensor.new_empty(rows, cols).normal_(0, 1)
    for i in range(0, rows, cols):
        q, r = torch.linalg.qr(flat[i:i + cols].t())
        q = (q * torch.diag(r, 0).sign()).t()
        with torch.no_grad():
            tensor[i:i + cols].view_as(q).copy_(q)
    with torch.no_grad():
        tensor.mul_(gain)
    return tensor


class _Materialize(torch.autograd.Function):
    """filters = M(weight) by the CUDA kernel; the backward applies M^T with torch ops."""

    @staticmethod
    def forward(ctx, weight, kernel):
        ctx.kernel = kernel
        return kernel._materialize(weight)

    @staticmethod
    def backward(ctx, g):
        return ctx.kernel._weight_grad(g.contiguous()), None


class SE3Kernel(torch.nn.Module):
    def __init__(self, Rs_in, Rs_out, size, radial_window=gaussian_window_wrapper, dyn_iso=False, verbose=False):
        super().__init__()
        self.size = size
        self.Rs_out = [(m, l) for m, l in Rs_out if m >= 1]
        self.Rs_in = [(m, l) for m, l in Rs_in if m >= 1]
        self.multiplicities_out = [m for m, _ in self.Rs_out]
        self.multiplicities_in = [m for m, _ in self.Rs_in]
        self.dims_out = [2 * l + 1 for _, l in self.Rs_out]
        self.dims_in = [2 * l + 1 for _, l in self.Rs_in]
        self.n_out = sum(m * d for m, d in zip(self.multiplicities_out, self.dims_out))
        self.n_in = sum(m * d for m, d in zip(self.multiplicities_in, self.dims_in))

        weights = []
        for i, (m_out, l_out) in enumerate(self.Rs_out):
            for j, (m_in, l_in) in enumerate(self.Rs_in):
                basis = cube_basis_kernels(size, l_in, l_out, radial_window)
                name = "kernel_{}_{}".format(i, j)
                if basis is None:
                    self.register_buffer(name, None)
                    continue
                basis = basis.clone()
                if dyn_iso:
                    w = torch.zeros(m_out, m_in, basis.size(0))
                    if abs(l_out - l_in) == min(abs(l_out - l) for _, l in self.Rs_in):
                        _orthogonal_(w[:, :, 0])
                    weights.append(w.flatten())
                    basis /= basis.flatten(2).norm(dim=2).mean(1).view(-1, 1, 1, 1, 1, 1)
                else:
                    weights.append(torch.randn(m_out * m_in * basis.size(0)))
                    basis /= basis.flatten(1).norm(dim=1).view(-1, 1, 1, 1, 1, 1)
                    basis *= ((2 * l_out + 1) / (len(basis) * sum(self.multiplicities_in))) ** 0.5
                if verbose:
                    print("{} -> {} : {} basis elements".format(l_in, l_out, len(basis)))
                self.register_buffer(name, basis.type(torch.get_default_dtype()))
        self.weight = torch.nn.Parameter(torch.cat(weights))
        self._packed = None  # (device, blob, block_table, out_field, in_field)

    def __repr__(self):
        return "{} ({} -> {}, size={})".format(self.__class__.__name__, self.Rs_in, self.Rs_out, self.size)

    # ------------------------------------------------------------------ device-side tables
    def _tables(self, device):
        """Basis blob + index tables for the materialisation kernel, cached per device."""
        if self._packed is not None and self._packed[0] == device:
            return self._packed[1:]
        K = self.size ** 3
        blobs, table, boff, woff = [], [], 0, 0
        for i, (m_out, _) in enumerate(self.Rs_out):
            for j, (m_in, _) in enumerate(self.Rs_in):
                b = getattr(self, "kernel_{}_{}".format(i, j))
                if b is None:
                    table += [-1, 0, 0, m_in, self.dims_out[i], self.dims_in[j]]
                    continue
                nb = b.size(0)
                table += [boff, woff, nb, m_in, self.dims_out[i], self.dims_in[j]]
                blobs.append(b.detach().to(torch.float32).reshape(-1))
                boff += b.numel()
                woff += m_out * m_in * nb
        assert boff == sum(x.numel() for x in blobs) and K * 0 == 0
        out_field = [(i, u, a) for i, m in enumerate(self.multiplicities_out) for u in range(m)
                     for a in range(self.dims_out[i])]
        in_field = [(j, v, c) for j, m in enumerate(self.multiplicities_in) for v in range(m)
                    for c in range(self.dims_in[j])]
        blob = (torch.cat(blobs) if blobs else torch.zeros(1)).to(device)
        packed = (device, blob, torch.tensor(table, dtype=torch.int32, device=device),
                  torch.tensor(out_field, dtype=torch.int32, device=device).reshape(-1),
                  torch.tensor(in_field, dtype=torch.int32, device=device).reshape(-1))
        self._packed = packed
        return packed[1:]

    def _apply(self, fn, *args, **kwargs):
        self._packed = None
        return super()._apply(fn, *args, **kwargs)

    def filters(self, weight=None):
        """Convolution filters [k, k, k, Cin, Cout] (contiguous, fp32) on the weight's device.
        Differentiable with respect to the weights when autograd is recording."""
        weight = self.weight if weight is None else weight
        if torch.is_grad_enabled() and weight.requires_grad:
            return _Materialize.apply(weight, self)
        return self._materialize(weight)

    def _materialize(self, weight):
        blob, table, out_field, in_field = self._tables(weight.device)
        K = self.size ** 3
        flt = _ext.materialize(weight.detach().contiguous(), blob, table, len(self.Rs_in), out_field, in_field,
                               self.n_out, self.n_in, K)
        return flt.view(self.size, self.size, self.size, self.n_in, self.n_out)

    def _weight_grad(self, g):
        """Adjoint of the (linear) materialisation: g [k,k,k,Cin,Cout] -> gradient of the flat
        weight vector, block by block (weights of block (i,j) are laid out [m_out, m_in, n_basis])."""
        k = self.size
        grads = []
        out_off = 0
        for i, (m_out, _) in enumerate(self.Rs_out):
            do = self.dims_out[i]
            in_off = 0
            for j, (m_in, _) in enumerate(self.Rs_in):
                di = self.dims_in[j]
                b = getattr(self, "kernel_{}_{}".format(i, j))
                if b is not None:
                    blk = g[:, :, :, in_off:in_off + m_in * di, out_off:out_off + m_out * do]
                    blk = blk.reshape(k, k, k, m_in, di, m_out, do)
                    grads.append(torch.einsum("xyzvcua,bacxyz->uvb", blk, b.to(g.dtype)).reshape(-1))
                in_off += m_in * di
            out_off += m_out * do
        return torch.cat(grads) if grads else g.new_zeros(0)

    def combination(self, weight):
        """[Cout, Cin, k, k, k] kernel (a permuted view of `filters`)."""
        return self.filters(weight).permute(4, 3, 0, 1, 2)

    def forward(self):
        return self.combination(self.weight)
