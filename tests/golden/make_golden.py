"""Generate the golden fixtures under tests/golden/ by RUNNING THE REFERENCE ITSELF.

Runs only where the reference checkout and its compiled extension exist (the development
container): the reference's Python package (SS_Conv_lib/ss_conv) is imported from its own
location with `ss_conv._ext` bound to the extension built by oracle/build_ref.py, on CPU
tensors, so every array written here is an output of the reference's code
(C++ rulebook / gather-GEMM-scatter / max-pool functors, Python SE3Kernel, BatchNorm,
Activation).

The reference imports the third-party package `lie_learn` (not installed, not pinned) for
real Wigner-D matrices and spherical harmonics.  A stand-in built from the reference's own
J matrices (Common_utils/new_constants.pt, formula of Common_utils/rotation_utils.py:314-370)
is installed under that module name; Y_J(x) is taken as sqrt((2J+1)/4pi) * D^J(alpha,beta,0)[:,J].
Basis fixtures are therefore pinned to that stand-in, not to a genuine lie_learn build.

Usage: python tests/golden/make_golden.py [path of the reference checkout]
"""
import importlib
import math
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def install_reference(ref_root):
    from ref_loader import load_ref_ext
    ext = load_ref_ext()
    if ext is None:
        raise SystemExit("build the reference extension first: python oracle/build_ref.py")
    np.float = float  # aliases removed in numpy 2, used by the reference's voxelize.py
    np.int = int
    Jd = [j.double().numpy() for j in torch.load(os.path.join(ref_root, "Common_utils", "new_constants.pt"))]

    def z_rot(angle, l):
        M = np.zeros((2 * l + 1, 2 * l + 1))
        inds = np.arange(2 * l + 1)
        freq = np.arange(l, -l - 1, -1)
        M[inds, inds[::-1]] = np.sin(freq * angle)
        M[inds, inds] = np.cos(freq * angle)
        return M

    def wigner_D_matrix(l, alpha, beta, gamma, **kw):
        return z_rot(float(alpha), l) @ Jd[l] @ z_rot(float(beta), l) @ Jd[l] @ z_rot(float(gamma), l)

    def sh(Js, Ms, theta, phi, **kw):
        # the reference calls sh(J, M, pi - beta, alpha) (SO3.py:104)
        Js, Ms = np.asarray(Js), np.asarray(Ms)
        beta = math.pi - np.asarray(theta, dtype=np.float64)
        alpha = np.asarray(phi, dtype=np.float64)
        shape = np.broadcast(Js, Ms, beta, alpha).shape
        out = np.zeros(shape)
        Jb, Mb = np.broadcast_to(Js, shape), np.broadcast_to(Ms, shape)
        bb, ab = np.broadcast_to(beta, shape), np.broadcast_to(alpha, shape)
        for ix in np.ndindex(*shape):
            J, M = int(Jb[ix]), int(Mb[ix])
            D = wigner_D_matrix(J, ab[ix], bb[ix], 0.0)
            out[ix] = math.sqrt((2 * J + 1) / (4 * math.pi)) * D[M + J, J]
        return out

    for name in ["lie_learn", "lie_learn.representations", "lie_learn.representations.SO3",
                 "lie_learn.representations.SO3.wigner_d", "lie_learn.representations.SO3.spherical_harmonics"]:
        sys.modules[name] = types.ModuleType(name)
    sys.modules["lie_learn.representations.SO3.wigner_d"].wigner_D_matrix = wigner_D_matrix
    sys.modules["lie_learn.representations.SO3.spherical_harmonics"].sh = sh

    pkg = types.ModuleType("ss_conv")
    pkg.__path__ = [os.path.join(ref_root, "SS_Conv_lib", "ss_conv")]
    sys.modules["ss_conv"] = pkg
    sys.modules["ss_conv._ext"] = ext
    pkg._ext = ext
    return ext


def surface_indices(rng, batch, V, n_pts):
    """Voxelised ellipsoid-surface points (the shape family of the benchmark inputs)."""
    rows = []
    for b in range(batch):
        axes = rng.uniform(0.3, 0.5, 3)
        A = np.linalg.qr(rng.randn(3, 3))[0]
        d = rng.randn(n_pts, 3)
        d /= np.linalg.norm(d, axis=1, keepdims=True)
        p = (d * axes) @ A.T
        p = np.clip(p, -0.499, 0.499)
        v = np.floor((p + 0.5) * V).astype(np.int64)
        v = np.unique(v, axis=0)
        rows.append(np.concatenate([np.full((v.shape[0], 1), b), v], 1))
    return np.concatenate(rows).astype(np.int32)


def main():
    if len(sys.argv) > 1:
        ref_root = sys.argv[1]
    else:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "oracle"))
        from ref_loader import reference_root
        ref_root = reference_root()
    ext = install_reference(ref_root)
    os.chdir(tempfile.mkdtemp())  # the reference writes its basis cache under ./cache
    convolution = importlib.import_module("ss_conv.convolution")
    batchnorm = importlib.import_module("ss_conv.batchnorm")
    activation = importlib.import_module("ss_conv.activation")
    pool = importlib.import_module("ss_conv.pool")
    tensor = importlib.import_module("ss_conv.sp_ops.tensor")
    kernel = importlib.import_module("ss_conv.utils.kernel")
    SO3 = importlib.import_module("ss_conv.utils.SO3")
    rng = np.random.RandomState(20240607)
    out = {}

    # ---- rulebooks from the reference's C++ CPU functor (geometry.h:140-288)
    cases = [(3, 1, 1, 1, 0), (3, 2, 1, 1, 0), (2, 2, 0, 1, 0), (3, 1, 0, 2, 0), (3, 1, 1, 1, 1), (5, 1, 2, 1, 1),
             (3, 3, 2, 1, 0), (3, 1, 1, 2, 1)]
    ind = surface_indices(rng, 2, 12, 160)
    out["rb_indices"] = ind
    out["rb_cases"] = np.array(cases, dtype=np.int32)
    for ci, (k, s, p, d, subm) in enumerate(cases):
        V = 12
        osz = [V] * 3 if subm else [(V + 2 * p - d * (k - 1) - 1) // s + 1] * 3
        r = ext.get_indice_pairs_3d(torch.from_numpy(ind), 2, osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [d] * 3,
                                    [0] * 3, subm, 0)
        out["rb%d_outids" % ci] = r[0].numpy().copy()
        out["rb%d_pairs" % ci] = r[1].numpy().copy()
        out["rb%d_num" % ci] = r[2].numpy().copy()

    # ---- transposed rulebooks (getIndicePairsDeConv, geometry.h:191-239)
    tcases = [(3, 2, 1, 1), (2, 2, 0, 0), (3, 1, 1, 0)]          # (k, stride, pad, output_padding)
    tind = surface_indices(rng, 2, 8, 90)
    out["rbt_indices"] = tind
    out["rbt_cases"] = np.array(tcases, dtype=np.int32)
    for ci, (k, s, p, op) in enumerate(tcases):
        osz = [(8 - 1) * s - 2 * p + k + op] * 3
        r = ext.get_indice_pairs_3d(torch.from_numpy(tind), 2, osz, [8] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3,
                                    [op] * 3, 0, 1)
        out["rbt%d_outids" % ci] = r[0].numpy().copy()
        out["rbt%d_pairs" % ci] = r[1].numpy().copy()
        out["rbt%d_num" % ci] = r[2].numpy().copy()

    # ---- one steerable layer through the reference's Python API on CPU tensors
    torch.manual_seed(7)
    Rs_in = [(2, 0), (2, 1), (1, 2)]
    Rs_out = [(2, 0), (1, 1), (1, 2), (2, 0)]      # trailing (2,0) = gate scalars
    for tag, kw in (("conv", dict(kernel_size=3, stride=1, padding=1)), ("strided", dict(kernel_size=3, stride=2, padding=1)),
                    ("subm", dict(kernel_size=3, subm=True, padding=1))):
        conv = convolution.Convolution(Rs_in, Rs_out, **kw).eval()
        ind_l = surface_indices(rng, 2, 10, 120)
        feats = rng.randn(ind_l.shape[0], conv.in_channels).astype(np.float32)
        x = tensor.SparseTensor(torch.from_numpy(feats), torch.from_numpy(ind_l), [10, 10, 10], 2)
        with torch.no_grad():
            y = conv(x)
        out[tag + "_indices"] = ind_l
        out[tag + "_features"] = feats
        out[tag + "_weight"] = conv.kernel.weight.detach().numpy().copy()
        out[tag + "_filters"] = conv.weight.detach().contiguous().numpy().copy()   # [k,k,k,Cin,Cout]
        out[tag + "_out_features"] = y.features.numpy().copy()
        out[tag + "_out_indices"] = y.indices.numpy().copy()
        if tag == "conv":
            for i in range(len(conv.kernel.Rs_out)):
                for j in range(len(conv.kernel.Rs_in)):
                    b = getattr(conv.kernel, "kernel_%d_%d" % (i, j))
                    out["basis_%d_%d" % (i, j)] = np.zeros(0, np.float32) if b is None else b.numpy().copy()
            # BatchNorm (eval + train) and gated activation on the layer output
            Rs_act = Rs_out[:-1]
            bn = batchnorm.BatchNorm(Rs_out, momentum=0.1)
            with torch.no_grad():
                bn.running_mean.copy_(torch.from_numpy(rng.randn(bn.running_mean.numel()).astype(np.float32) * 0.1))
                bn.running_var.copy_(torch.from_numpy(rng.uniform(0.5, 2.0, bn.running_var.numel()).astype(np.float32)))
                bn.weight.copy_(torch.from_numpy(rng.uniform(0.5, 1.5, bn.weight.numel()).astype(np.float32)))
                bn.bias.copy_(torch.from_numpy(rng.randn(bn.bias.numel()).astype(np.float32) * 0.1))
            for name in ("running_mean", "running_var", "weight", "bias"):
                out["bn_" + name] = getattr(bn, name).detach().numpy().copy()
            yt = tensor.SparseTensor(y.features.clone(), y.indices, y.spatial_shape, 2)
            bn.eval()
            with torch.no_grad():
                out["bn_eval_out"] = bn(yt).features.numpy().copy()
            yt = tensor.SparseTensor(y.features.clone(), y.indices, y.spatial_shape, 2)
            bn.train()
            with torch.no_grad():
                out["bn_train_out"] = bn(yt).features.numpy().copy()
            out["bn_train_running_mean"] = bn.running_mean.numpy().copy()
            out["bn_train_running_var"] = bn.running_var.numpy().copy()
            act = activation.Activation(Rs_act, (torch.relu, torch.sigmoid), bias=True, checkpoint=False)
            with torch.no_grad():
                act.scalar_act.bias.copy_(torch.from_numpy(rng.randn(act.scalar_act.bias.numel()).astype(np.float32) * 0.2))
                act.gate_act.bias.copy_(torch.from_numpy(rng.randn(act.gate_act.bias.numel()).astype(np.float32) * 0.2))
            out["act_scalar_bias"] = act.scalar_act.bias.detach().numpy().copy()
            out["act_gate_bias"] = act.gate_act.bias.detach().numpy().copy()
            yt = tensor.SparseTensor(torch.from_numpy(out["bn_eval_out"]).clone(), y.indices, y.spatial_shape, 2)
            with torch.no_grad():
                out["act_out"] = act(yt).features.numpy().copy()
            # sparse max pool (C++ CPU functor) on the layer output
            mp = pool.MaxPool(2, stride=2)
            yt = tensor.SparseTensor(y.features.clone(), y.indices, y.spatial_shape, 2)
            with torch.no_grad():
                z = mp(yt)
            out["maxpool_out_features"] = z.features.numpy().copy()
            out["maxpool_out_indices"] = z.indices.numpy().copy()

    # ---- backward of the C++ CPU path: indiceConvBackward (indice_conv.h:344-426) and
    #      indiceMaxPoolBackward (indice_maxpool.h:94-127) on a strided and a submanifold rulebook
    brng = np.random.RandomState(4711)
    bind = surface_indices(brng, 2, 10, 150)
    out["bw_indices"] = bind
    for tag, (k, s, p, subm) in (("bw_strided", (3, 2, 1, 0)), ("bw_subm", (3, 1, 1, 1))):
        V, ci, co = 10, 6, 5
        osz = [V] * 3 if subm else [(V + 2 * p - (k - 1) - 1) // s + 1] * 3
        o, pr, nm = ext.get_indice_pairs_3d(torch.from_numpy(bind), 2, osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3,
                                            [1] * 3, [0] * 3, subm, 0)
        feats = brng.randn(bind.shape[0], ci).astype(np.float32)
        W = (brng.randn(k, k, k, ci, co) / np.sqrt(ci * k ** 3)).astype(np.float32)
        dout = brng.randn(o.shape[0], co).astype(np.float32)
        din, dW = ext.indice_conv_backward_fp32(torch.from_numpy(feats), torch.from_numpy(W), torch.from_numpy(dout),
                                                pr, nm, 0, subm)
        out[tag + "_geom"] = np.array([k, s, p, subm], dtype=np.int32)
        out[tag + "_features"], out[tag + "_filters"], out[tag + "_dout"] = feats, W, dout
        out[tag + "_din"], out[tag + "_dfilters"] = din.numpy().copy(), dW.numpy().copy()
        out[tag + "_outids"], out[tag + "_pairs"], out[tag + "_num"] = o.numpy().copy(), pr.numpy().copy(), nm.numpy().copy()
        if not subm:
            pf = np.maximum(feats, 0).round(1)          # ties between inputs and a zero floor are exercised
            y = ext.indice_maxpool_fp32(torch.from_numpy(pf), pr, nm, o.shape[0])
            dy = brng.randn(o.shape[0], ci).astype(np.float32)
            dp = ext.indice_maxpool_backward_fp32(torch.from_numpy(pf), y, torch.from_numpy(dy), pr, nm)
            out["bw_pool_features"], out["bw_pool_out"], out["bw_pool_dout"] = pf, y.numpy().copy(), dy
            out["bw_pool_din"] = dp.numpy().copy()

    # ---- feature steering (Common_utils/ss_conv_modules.py:173-224, rotation_utils.py:424-447): the
    #      per-point change of frame of points and irrep features, and the D matrices it uses
    sys.path.insert(0, os.path.join(ref_root, "Common_utils"))
    modules = importlib.import_module("ss_conv_modules")
    rot_utils = importlib.import_module("rotation_utils")
    frng = np.random.RandomState(99)
    Bf, Nf, irrep = 3, 40, (2, 2, 1, 1)
    q = frng.randn(Bf, 4)
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    Rf = rot_utils.quaternion_to_matrix(torch.from_numpy(q)).float()
    tf = torch.from_numpy(frng.randn(Bf, 3).astype(np.float32) * 0.1)
    sf = torch.from_numpy(frng.uniform(0.8, 1.2, Bf).astype(np.float32))
    idf = torch.from_numpy(np.sort(frng.randint(0, Bf, Nf)).astype(np.int64))
    pf = torch.from_numpy(frng.randn(Nf, 3).astype(np.float32) * 0.3)
    Cf = sum(m * (2 * l + 1) for l, m in enumerate(irrep))
    ff = torch.from_numpy(frng.randn(Nf, Cf).astype(np.float32))
    holder = type("H", (), {"irrep": irrep})()
    out["fsm_R"], out["fsm_t"], out["fsm_s"] = Rf.numpy(), tf.numpy(), sf.numpy()
    out["fsm_ids"], out["fsm_points"], out["fsm_feats"] = idf.numpy().astype(np.int32), pf.numpy(), ff.numpy()
    out["fsm_irrep"] = np.array(irrep, dtype=np.int32)
    out["fsm_new_points"] = modules.Feature_Steering_Module._transform_points(holder, pf, Rf[idf], tf[idf], sf[idf]).numpy()
    out["fsm_new_points_noscale"] = modules.Feature_Steering_Module._transform_points(holder, pf, Rf[idf], tf[idf]).squeeze(1).numpy()
    out["fsm_new_feats"] = modules.Feature_Steering_Module._transform_feats(holder, ff, Rf[idf]).numpy()
    for l in range(len(irrep)):
        out["fsm_D%d" % l] = rot_utils.D_from_matrix(Rf.double(), l).numpy()

    # ---- Wigner-D / Q_J values the basis is built from (stand-in convention)
    out["irr_repr_l2"] = SO3.irr_repr(2, 0.3, 1.1, -2.0, dtype=torch.float64).numpy()
    out["Q_J_1_1_1"] = kernel.basis_transformation_Q_J(1, 1, 1).numpy() if hasattr(kernel, "basis_transformation_Q_J") \
        else SO3.basis_transformation_Q_J(1, 1, 1).numpy()
    out["meta_Rs_in"] = np.array(Rs_in, dtype=np.int32)
    out["meta_Rs_out"] = np.array(Rs_out, dtype=np.int32)
    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, "%.1f KB" % (os.path.getsize(path) / 1024), len(out), "arrays")


if __name__ == "__main__":
    main()
