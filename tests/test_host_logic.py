"""CPU-side checks: the C-ABI library loads and exports every declared symbol, the ctypes
table covers the header, steerable-basis construction, sharding arithmetic."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ssconv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ssc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from ss_conv import _ext
    assert os.path.exists(_ext.LIB_PATH), "build the library: python ss-conv_b200/build.py"
    h = ctypes.CDLL(_ext.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 29
    for n in names:
        assert hasattr(h, n), n
    assert sorted(_ext.SIGNATURES) == names
    assert _ext.lib().ssc_version() >= 100
    assert _ext.lib().ssc_has_tcgen05() == 1


def test_argument_errors_without_gpu():
    """Size queries and argument validation run on the host only."""
    from ss_conv import _ext
    L = _ext.lib()
    I3 = ctypes.c_int * 3
    assert L.ssc_rulebook_scratch_bytes(1000, 2, I3(16, 16, 16), I3(16, 16, 16), 27) > 1000 * 2 * 8
    assert L.ssc_conv_packed_bytes(27, 64, 76, _ext.PREC_TF32) == 27 * 2 * 80 * 128
    assert L.ssc_conv_packed_bytes(27, 64, 600, _ext.PREC_TF32) == 0
    rc = L.ssc_maxpool_fwd(None, 0, None, 27, 5, None, None, None)
    assert rc == 1 and b"bad sizes" in L.ssc_last_error()
    with pytest.raises(RuntimeError):
        _ext.indice_maxpool_fp32(torch.zeros(4, 4), torch.zeros(1, 2, 4, dtype=torch.int32),
                                 torch.zeros(1, dtype=torch.int32), 4)
    with pytest.raises(NotImplementedError):
        _ext.indice_field_maxpool_fp32()


def test_output_size_and_shards():
    from ss_conv.sp_ops.ops import get_conv_output_size, get_deconv_output_size
    from ss_conv.parallel import shard_range
    assert get_conv_output_size([64] * 3, [3] * 3, [2] * 3, [1] * 3, [1] * 3) == [32] * 3
    assert get_conv_output_size([32] * 3, [2] * 3, [2] * 3, [0] * 3, [1] * 3) == [16] * 3
    assert get_deconv_output_size([16] * 3, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [1] * 3) == [32] * 3
    for n, w in ((256, 8), (10, 4), (3, 8), (0, 2)):
        r = [shard_range(n, k, w) for k in range(w)]
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        sizes = [b - a for a, b in r]
        assert max(sizes) - min(sizes) <= 1


def test_wigner_and_intertwiner_against_reference_values(golden):
    from ss_conv.utils import SO3
    D = SO3.irr_repr(2, 0.3, 1.1, -2.0, dtype=torch.float64).numpy()
    assert np.abs(D - golden["irr_repr_l2"]).max() < 1e-12
    Q = SO3.basis_transformation_Q_J(1, 1, 1).numpy()
    R = golden["Q_J_1_1_1"]
    assert min(np.abs(Q - R).max(), np.abs(Q + R).max()) < 1e-10      # null vector: sign is free
    # representation property and SH compatibility, the reference's own self-checks (SO3.py:340-378)
    for l in range(4):
        a = SO3.irr_repr(l, 0.2, 0.5, 0.9, torch.float64)
        b = SO3.irr_repr(l, 1.2, 0.3, 2.1, torch.float64)
        Rm = SO3.rot(0.2, 0.5, 0.9) @ SO3.rot(1.2, 0.3, 2.1)
        x = torch.randn(5, 3, dtype=torch.float64)
        Y = SO3.spherical_harmonics_xyz(l, x)
        Yr = SO3.spherical_harmonics_xyz(l, x @ Rm.T)
        assert torch.allclose(Yr, a @ b @ Y, atol=1e-10)


def test_basis_buffers_match_reference(golden):
    """Same shapes, norms and (up to the free sign of each basis element) same values as the
    basis the reference builds with its in-tree Wigner-D stand-in."""
    from ss_conv.utils.kernel import SE3Kernel
    Rs_in = [tuple(int(v) for v in r) for r in golden["meta_Rs_in"]]
    Rs_out = [tuple(int(v) for v in r) for r in golden["meta_Rs_out"]]
    torch.manual_seed(0)
    k = SE3Kernel(Rs_in, Rs_out, 3)
    assert k.weight.numel() == golden["conv_weight"].size
    for i in range(len(Rs_out)):
        for j in range(len(Rs_in)):
            ref = golden["basis_%d_%d" % (i, j)]
            mine = getattr(k, "kernel_%d_%d" % (i, j))
            if ref.size == 0:
                assert mine is None
                continue
            mine = mine.numpy()
            assert mine.shape == ref.shape
            for b in range(ref.shape[0]):
                err = min(np.abs(mine[b] - ref[b]).max(), np.abs(mine[b] + ref[b]).max())
                assert err < 1e-6, (i, j, b, err)


def test_synthetic_inputs_are_seeded_per_sample():
    from ss_conv.utils import synthetic as S
    a = S.surface_voxels([3, 4], 32, 4096, base_seed=100)
    b = S.surface_voxels([4], 32, 4096, base_seed=100)
    assert np.array_equal(a[a[:, 0] == 1][:, 1:], b[:, 1:])
    assert a[:, 1:].min() >= 0 and a[:, 1:].max() < 32
    p, f, ids = S.object_points([0, 1], 1024)
    assert p.shape == (2048, 3) and np.abs(p).max() < 0.5 and f.min() >= 0 and f.max() <= 1


def test_packed_filter_sizes_follow_the_operand_layout():
    """ssc_conv_packed_bytes is pure host arithmetic.  TF32: one 128-byte operand row holds 32 input
    channels, or the neighbours at 8 / 4 / 2 kernel offsets when the rows pad to 4 / 8 / 16 channels;
    16-bit: 64 channels per row, never grouped."""
    from ss_conv import _ext
    L = _ext.lib()
    n_pad = 48                                        # 38 output channels padded to a multiple of 16
    full = lambda K, slabs: K * slabs * n_pad * 128   # noqa: E731
    assert L.ssc_conv_packed_bytes(27, 32, 38, _ext.PREC_TF32) == full(27, 1)
    assert L.ssc_conv_packed_bytes(27, 64, 38, _ext.PREC_TF32) == full(27, 2)
    assert L.ssc_conv_packed_bytes(27, 20, 38, _ext.PREC_TF32) == full(27, 1)        # pads to 20: not grouped
    assert L.ssc_conv_packed_bytes(27, 3, 38, _ext.PREC_TF32) == full(4, 1)          # 8 offsets per row
    assert L.ssc_conv_packed_bytes(27, 8, 38, _ext.PREC_TF32) == full(7, 1)          # 4 offsets per row
    assert L.ssc_conv_packed_bytes(27, 16, 38, _ext.PREC_TF32) == full(14, 1)        # 2 offsets per row
    assert L.ssc_conv_packed_bytes(27, 3, 38, _ext.PREC_BF16) == full(27, 1)
    assert L.ssc_conv_packed_bytes(27, 100, 38, _ext.PREC_F16) == full(27, 2)
    assert L.ssc_conv_pairs_supported(16, 256, _ext.PREC_TF32) == 0                  # grouped filters: not for the pair-list kernel
