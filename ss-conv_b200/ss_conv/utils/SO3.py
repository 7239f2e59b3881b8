"""SO(3) helpers for the steerable basis: ZYZ rotations, real spherical harmonics,
real Wigner-D matrices and the Clebsch-Gordan-like change of basis Q_J.

Mirrors the interface of the reference module SS_Conv_lib/ss_conv/utils/SO3.py
(rot :41-45, x_to_alpha_beta :48-57, irr_repr :66-76, spherical_harmonics :79-106,
spherical_harmonics_xyz :109-129, kron :204-207, basis_transformation_Q_J :239-274) but does
not depend on the third-party `lie_learn` package the reference imports there: the
spherical harmonics are evaluated from the associated-Legendre recurrence and the Wigner-D
matrix of a rotation R is obtained as the unique matrix with Y(R x) = D(R) Y(x) (solved on a
fixed set of sample directions in float64).  Everything here is one-time float64 set-up on
the host; the per-forward arithmetic lives in the CUDA library.
"""
import math

import numpy as np
import torch


def rot_z(gamma):
    c, s = math.cos(float(gamma)), math.sin(float(gamma))
    return torch.tensor([[c, -s, 0.0], [s, c, 0.0], [0.0, 0.0, 1.0]], dtype=torch.float64)


def rot_y(beta):
    c, s = math.cos(float(beta)), math.sin(float(beta))
    return torch.tensor([[c, 0.0, s], [0.0, 1.0, 0.0], [-s, 0.0, c]], dtype=torch.float64)


def rot(alpha, beta, gamma):
    """ZYZ Euler rotation matrix (float64)."""
    return rot_z(alpha) @ rot_y(beta) @ rot_z(gamma)


def x_to_alpha_beta(x):
    """Direction (x, y, z) -> (alpha, beta) with beta the polar angle."""
    x = torch.as_tensor(x, dtype=torch.float64)
    x = x / torch.norm(x, 2, -1, keepdim=True)
    return torch.atan2(x[..., 1], x[..., 0]), torch.acos(x[..., 2].clamp(-1.0, 1.0))


def _assoc_legendre(l, c):
    """P_l^m(c) for m = 0..l WITHOUT the Condon-Shortley phase; c is a float64 ndarray."""
    s = np.sqrt(np.maximum(0.0, 1.0 - c * c))
    out = []
    pmm = np.ones_like(c)
    for m in range(l + 1):
        if m > 0:
            pmm = pmm * (2 * m - 1) * s
        if m == l:
            out.append(pmm)
            continue
        p_prev, p_cur = pmm, c * (2 * m + 1) * pmm
        for ll in range(m + 2, l + 1):
            p_prev, p_cur = p_cur, ((2 * ll - 1) * c * p_cur - (ll + m - 1) * p_prev) / (ll - m)
        out.append(p_cur)
    return out


def _real_sh(l, alpha, beta):
    """Real orthonormal spherical harmonics of degree l at azimuth alpha, polar angle beta.
    Rows m = -l..l: sqrt(2) N P_l^|m|(cos beta) sin(|m| alpha) for m<0, N P_l^0 for m=0,
    sqrt(2) N P_l^m cos(m alpha) for m>0 (no Condon-Shortley phase), so degree 1 is
    proportional to (y, z, x).  This is the convention in which the real Wigner-D matrices
    factor as Z(alpha) J Z(beta) J Z(gamma) with the J matrices the reference ships for its
    own feature rotations (Common_utils/rotation_utils.py:333-370)."""
    alpha = np.asarray(alpha, dtype=np.float64)
    beta = np.asarray(beta, dtype=np.float64)
    P = _assoc_legendre(l, np.cos(beta))
    rows = [None] * (2 * l + 1)
    for m in range(0, l + 1):
        norm = math.sqrt((2 * l + 1) / (4 * math.pi) * math.factorial(l - m) / math.factorial(l + m))
        if m == 0:
            rows[l] = norm * P[0]
        else:
            rows[l + m] = math.sqrt(2.0) * norm * P[m] * np.cos(m * alpha)
            rows[l - m] = math.sqrt(2.0) * norm * P[m] * np.sin(m * alpha)
    return np.stack(rows, axis=0)


def spherical_harmonics(order, alpha, beta, dtype=None):
    """[sum(2J+1), A] real spherical harmonics for `order` (int or list of ints)."""
    orders = order if isinstance(order, list) else [order]
    a = torch.as_tensor(alpha, dtype=torch.float64).numpy()
    b = torch.as_tensor(beta, dtype=torch.float64).numpy()
    Y = np.concatenate([_real_sh(J, a, b) for J in orders], axis=0)
    return torch.tensor(Y, dtype=torch.get_default_dtype() if dtype is None else dtype)


def spherical_harmonics_xyz(order, xyz):
    """Real spherical harmonics at directions xyz [..., 3] (float64); at the origin the l=0
    component keeps its constant value and every l>0 component is zero (SO3.py:124-127)."""
    orders = order if isinstance(order, list) else [order]
    xyz = torch.as_tensor(xyz, dtype=torch.float64)
    r = torch.norm(xyz, 2, -1)
    safe = torch.where(r.unsqueeze(-1) > 0, xyz, torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64).expand_as(xyz))
    alpha, beta = x_to_alpha_beta(safe)
    out = spherical_harmonics(orders, alpha, beta, dtype=torch.float64)
    if bool((r == 0).any()):
        val = torch.cat([spherical_harmonics(0, 0.0, 0.0, dtype=torch.float64).reshape(1) if J == 0
                         else torch.zeros(2 * J + 1, dtype=torch.float64) for J in orders])
        out[..., r == 0] = val.view(-1, *([1] * (out.dim() - 1))).expand_as(out)[..., r == 0]
    return out


_SAMPLE_CACHE = {}


def _sample_dirs(l):
    if l not in _SAMPLE_CACHE:
        rng = np.random.RandomState(1234 + l)
        v = rng.randn(6 * (2 * l + 1) + 8, 3)
        v /= np.linalg.norm(v, axis=1, keepdims=True)
        a = np.arctan2(v[:, 1], v[:, 0])
        b = np.arccos(np.clip(v[:, 2], -1, 1))
        _SAMPLE_CACHE[l] = (v, np.linalg.pinv(_real_sh(l, a, b)))
    return _SAMPLE_CACHE[l]


def irr_repr(order, alpha, beta, gamma, dtype=None):
    """Real Wigner-D matrix of rot(alpha, beta, gamma) in the basis of `spherical_harmonics`:
    the matrix D with Y(R x) = D Y(x) for all x."""
    v, pinvY = _sample_dirs(order)
    R = rot(alpha, beta, gamma).numpy()
    w = v @ R.T
    a = np.arctan2(w[:, 1], w[:, 0])
    b = np.arccos(np.clip(w[:, 2], -1, 1))
    D = _real_sh(order, a, b) @ pinvY
    return torch.tensor(D, dtype=torch.get_default_dtype() if dtype is None else dtype)


def irr_repr_of_matrix(order, R):
    """Real Wigner-D matrix of the proper rotation R (3x3) in the basis of `spherical_harmonics`:
    Y(R x) = D Y(x), obtained by projection on sample directions (no Euler angles needed)."""
    v, pinvY = _sample_dirs(order)
    w = v @ np.asarray(R, dtype=np.float64).T
    a = np.arctan2(w[:, 1], w[:, 0])
    b = np.arccos(np.clip(w[:, 2], -1, 1))
    return _real_sh(order, a, b) @ pinvY


# Axis relabelling between the frame the feature-steering code describes rotations in (polar axis
# y; Common_utils/rotation_utils.py:334-372 builds D from Y-X-Y angles) and the frame of
# `spherical_harmonics` here (polar axis z): D_steer(R) = irr_repr_of_matrix(S R S^T).
_STEER_AXES = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0], [0.0, 1.0, 0.0]])


def D_from_matrix(R, l, frame="reference"):
    """Representation matrices D^l [..., 2l+1, 2l+1] of rotation matrices R [..., 3, 3], the
    function of the same name in the reference (Common_utils/rotation_utils.py:424-447): an
    improper R is first multiplied by -1 (its parity factor is 1 there).
    frame="reference" reproduces that function (rotations described in a frame whose polar axis
    is y); frame="kernel" is the representation in the frame of the filter basis
    (`spherical_harmonics`, polar axis z, axes = voxel axes), the one under which the steerable
    convolution of this package commutes with rotations of the voxel grid."""
    Rn = np.asarray(R.detach().cpu().double() if torch.is_tensor(R) else R, dtype=np.float64)
    flat = Rn.reshape(-1, 3, 3)
    out = np.empty((flat.shape[0], 2 * l + 1, 2 * l + 1), dtype=np.float64)
    for i, Ri in enumerate(flat):
        Ri = Ri * np.sign(np.linalg.det(Ri))
        out[i] = irr_repr_of_matrix(l, Ri if frame == "kernel" else _STEER_AXES @ Ri @ _STEER_AXES.T)
    out = out.reshape(Rn.shape[:-2] + (2 * l + 1, 2 * l + 1))
    if torch.is_tensor(R):
        return torch.as_tensor(out, dtype=R.dtype, device=R.device)
    return out


def kron(x, y):
    return torch.einsum("ij,kl->ikjl", x, y).reshape(x.size(0) * y.size(0), x.size(1) * y.size(1))


_Q_ANGLES = [
    [4.41301023, 5.56684102, 4.59384642],
    [4.93325116, 6.12697327, 4.14574096],
    [0.53878964, 4.09050444, 5.36539036],
    [2.16017393, 3.48835314, 5.55174441],
    [2.52385107, 0.2908958, 3.90040975],
]
_Q_CACHE = {}


def basis_transformation_Q_J(J, order_in, order_out):
    """[(2*order_out+1)*(2*order_in+1), 2J+1] float64 matrix Q with
    (D_out (x) D_in) Q = Q D_J for every rotation: the one-dimensional common null space of
    the Sylvester operators of five fixed rotations (the reference's angles, SO3.py:254-260).
    The overall sign of the null vector is fixed by making its largest-magnitude entry
    positive, so that repeated construction is reproducible."""
    key = (J, order_in, order_out)
    if key in _Q_CACHE:
        return _Q_CACHE[key].clone()
    f64 = torch.float64

    def r_tensor(a, b, c):
        return kron(irr_repr(order_out, a, b, c, f64), irr_repr(order_in, a, b, c, f64))

    blocks = []
    for a, b, c in _Q_ANGLES:
        Rt = r_tensor(a, b, c)
        RJ = irr_repr(J, a, b, c, f64)
        blocks.append(kron(Rt, torch.eye(RJ.size(0), dtype=f64)) - kron(torch.eye(Rt.size(0), dtype=f64), RJ.t()))
    A = torch.cat(blocks, dim=0)
    _u, s, vh = torch.linalg.svd(A, full_matrices=True)
    svals = torch.zeros(A.size(1), dtype=f64)
    svals[: s.numel()] = s
    null = vh[svals < 1e-8]
    if null.size(0) != 1:
        raise RuntimeError("expected a one-dimensional intertwiner space, got %d" % null.size(0))
    q = null[0]
    q = q * torch.sign(q[torch.argmax(q.abs())])
    Q = q.view((2 * order_out + 1) * (2 * order_in + 1), 2 * J + 1)
    g = torch.Generator().manual_seed(7)
    for a, b, c in torch.rand(4, 3, generator=g, dtype=f64):
        lhs = r_tensor(a.item(), b.item(), c.item()) @ Q
        rhs = Q @ irr_repr(J, a.item(), b.item(), c.item(), f64)
        if not torch.allclose(lhs, rhs, atol=1e-9):
            raise RuntimeError("Q_J does not intertwine the representations")
    _Q_CACHE[key] = Q
    return Q.clone()
