"""Native-op module of the B200 build: the names the reference exports from its pybind11
extension `ss_conv._ext` (SS_Conv_lib/src/ss_conv_ops_api.cpp:15-55), implemented as thin
ctypes calls into the C-ABI CUDA library libssconv_b200.so (include/ssconv_b200.h).

PyTorch is used only to allocate device memory and to supply the current CUDA stream.  There
is no CPU path: every function raises if the library is missing or a tensor is not on a CUDA
device.  The forward and backward entry points of the 3-D path are implemented (fp32, and the half
variants of convolution and pools); only the functions the reference's own Python never reaches
(indice_field_maxpool_*, voxelize_idx, point_recover_*) and the 2-D rulebooks raise NotImplementedError.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SSCONV_B200_LIB selects another build of the same library (e.g. a debug build)
LIB_PATH = os.environ.get("SSCONV_B200_LIB", os.path.join(_HERE, "libssconv_b200.so"))

PREC_FP32, PREC_TF32, PREC_F16, PREC_BF16 = 0, 1, 2, 3
_PREC_OF = {"tf32": PREC_TF32, "fp16": PREC_F16, "bf16": PREC_BF16}
_precision = os.environ.get("SSCONV_PRECISION", "auto")

c_int, c_size_t, c_void_p, c_float = ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_float
_I3 = ctypes.c_int * 3
_F3 = ctypes.c_float * 3

# name -> (restype, argtypes); kept in one table so tests can check it against the header
SIGNATURES = {
    "ssc_version": (c_int, []),
    "ssc_last_error": (ctypes.c_char_p, []),
    "ssc_has_tcgen05": (c_int, []),
    "ssc_kernel_launches": (ctypes.c_ulonglong, []),
    "ssc_rulebook_scratch_bytes": (c_size_t, [c_int, c_int, _I3, _I3, c_int]),
    "ssc_rulebook_subm": (c_int, [c_void_p, c_int, c_int, _I3, _I3, _I3, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_size_t, c_void_p]),
    "ssc_rulebook_subm_static": (c_int, [c_void_p, c_int, c_int, _I3, _I3, _I3, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p]),
    "ssc_rulebook_subm_ahead": (c_int, [c_void_p, c_int, c_int, _I3, _I3, _I3, c_void_p, c_void_p, c_void_p, c_size_t,
                                        c_void_p, c_void_p]),
    "ssc_rulebook_conv_count": (c_int, [c_void_p, c_int, c_int, _I3, _I3, _I3, _I3, _I3, _I3, c_int, c_void_p,
                                        c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "ssc_rulebook_conv_fill": (c_int, [c_void_p, c_int, c_int, _I3, _I3, _I3, _I3, _I3, _I3, c_int, c_int, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_pairs_to_nbr": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ssc_pairs_from_nbr_scratch_bytes": (c_size_t, [c_int, c_int]),
    "ssc_pairs_from_nbr": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_materialize": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_void_p, c_void_p]),
    "ssc_conv_packed_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "ssc_conv_pack_filters": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ssc_conv_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "ssc_conv_fwd": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                             c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "ssc_conv_pairs_list_bytes": (c_size_t, [c_int, c_int]),
    "ssc_conv_pairs_supported": (c_int, [c_int, c_int, c_int]),
    "ssc_conv_pairs_build": (c_int, [c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "ssc_conv_fwd_pairs": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_size_t, c_int, c_int,
                                   c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_nbr_transpose": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ssc_nbr_row_order_scratch_bytes": (c_size_t, [c_int, c_int]),
    "ssc_nbr_row_order": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_nbr_row_order_planes_scratch_bytes": (c_size_t, [_I3, c_int]),
    "ssc_nbr_row_order_planes": (c_int, [c_void_p, _I3, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "ssc_conv_stage": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "ssc_conv_fwd_ordered": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    "ssc_conv_wgrad_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "ssc_conv_wgrad": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_size_t, c_void_p]),
    "ssc_maxpool_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "ssc_avgpool_bwd": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "ssc_global_avgpool_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ssc_global_maxpool_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ssc_voxelize_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ssc_three_interpolate_bwd": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ssc_steer_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                              c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "ssc_p2v_stats": (c_int, [c_void_p, c_void_p, c_int, _I3, _F3, c_void_p, c_void_p]),
    "ssc_maxpool_fwd": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "ssc_avgpool_fwd": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ssc_summary_rf": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "ssc_global_avgpool_fwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "ssc_global_maxpool_fwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "ssc_batch_offsets": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "ssc_voxel2point_map": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "ssc_voxelize_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "ssc_p2v_scratch_bytes": (c_size_t, [c_int, c_int, _I3]),
    "ssc_p2v_count": (c_int, [c_void_p, c_void_p, c_int, c_int, _I3, _F3, c_void_p, c_void_p, c_void_p, c_size_t,
                              c_void_p]),
    "ssc_p2v_fill": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, _I3, _F3, c_int, c_int, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_three_nn_scratch_bytes": (c_size_t, [c_int]),
    "ssc_three_nn": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_three_interpolate_fwd": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ssc_bn_fold": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p,
                            c_void_p, c_void_p]),
    "ssc_bn_gate_fwd": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_void_p, c_void_p, c_void_p, c_void_p]),
    "ssc_bn_gate_fwd16": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ssc_bn_scratch_bytes": (c_size_t, [c_int, c_int]),
    "ssc_bn_stats": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                             c_size_t, c_void_p]),
    "ssc_bn_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                           c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "ssc_gate_bwd": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_void_p, c_void_p]),
    "ssc_scatter_add_rate": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
}

_lib_handle = None


def lib():
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib_handle
    if _lib_handle is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("libssconv_b200.so is missing: run `python ss-conv_b200/build.py` "
                               "(there is no CPU or PyTorch fallback)")
        h = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)
            fn.restype = res
            fn.argtypes = args
        _lib_handle = h
    return _lib_handle


def kernel_launches():
    """CUDA kernels launched by the library in this process so far."""
    return int(lib().ssc_kernel_launches())


def set_precision(mode):
    """'fp32' (exact CUDA-core path), 'tf32' (tcgen05 tensor cores), 'fp16' (tcgen05 with
    fp16 operands: the same 11-bit significand as TF32 but fp16's range, half the gathered
    bytes and half the tensor-core instructions; opt-in only), 'bf16' (tcgen05 with bfloat16
    operands: fp32's range, 8 significant bits, the same halved traffic; opt-in only) or 'auto'
    (tf32 when the layer has at least 16 input channels)."""
    global _precision
    if mode not in ("fp32", "tf32", "fp16", "bf16", "auto"):
        raise ValueError("precision must be 'fp32', 'tf32', 'fp16', 'bf16' or 'auto'")
    _precision = mode


def get_precision():
    return _precision


# Feature storage between layers: None (fp32, the reference's format) or 'fp16' / 'bf16': a gated
# Activation then writes its result in that 16-bit type (when the channel count is a multiple of 8)
# and the next convolution gathers those rows as its operands - no staging pass, half the bytes
# between the layers.  The convolution's operand precision follows the stored type.
_storage = None
_DTYPE_OF = {"fp16": torch.float16, "bf16": torch.bfloat16}
_PREC_OF_DTYPE = {torch.float16: "fp16", torch.bfloat16: "bf16"}


def set_feature_storage(mode):
    global _storage
    if mode not in (None, "fp16", "bf16"):
        raise ValueError("feature storage must be None, 'fp16' or 'bf16'")
    _storage = mode


def get_feature_storage():
    return _storage


def _check(rc):
    if rc != 0:
        msg = lib().ssc_last_error().decode()
        if rc == 1:
            raise ValueError("ssconv_b200: " + msg)
        raise RuntimeError("ssconv_b200 (code %d): %s" % (rc, msg))


def _p(t, dtype=None):
    """Device pointer of a contiguous CUDA tensor (None -> NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("ssconv_b200 runs on CUDA tensors only (got a %s tensor)" % t.device.type)
    if dtype is not None and t.dtype != dtype:
        raise TypeError("expected dtype %s, got %s" % (dtype, t.dtype))
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    return t.data_ptr()  # ctypes turns the int into a void* (NULL must be passed as None)


def _stream():
    """Raw handle of torch's current stream on the current device (None = the default stream);
    the C-level getters cost a fraction of a microsecond, torch.cuda.current_stream() ~15."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()) or None


_i3_cache = {}


def _i3(v):
    """ctypes int[3] for a geometry triple (cached: the same few triples recur every call)."""
    key = (int(v[0]), int(v[1]), int(v[2]))
    arr = _i3_cache.get(key)
    if arr is None:
        arr = _i3_cache[key] = _I3(*key)
    return arr


_status = {}
_scratch_cache = {}


def status_word(device):
    """Per-device int32 that kernels OR error bits into (read it with check_status())."""
    key = torch.device(device).index
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device=None):
    """Synchronising read of the device status word; raises on a recorded kernel problem."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    s = status_word(device)
    v = int(s.item())
    if v != 0:
        s.zero_()
        raise RuntimeError("ssconv_b200 kernel status 0x%x (%s)" % (v, _STATUS_TEXT))


_STATUS_TEXT = ("1: coordinate out of range, 2: hash full, 16: a bounded wait inside a tensor-core kernel ran out "
                "(its output is incomplete)")


def raise_on_status(value, device):
    """Turn a non-zero status word that was read back into an error (and clear it on the device)."""
    if value:
        status_word(device).zero_()
        raise RuntimeError("ssconv_b200 kernel status 0x%x (%s)" % (int(value), _STATUS_TEXT))


def read_count(n_dev):
    """Host value of a device row count.  The per-device status word rides along in the same
    read-back, so a kernel that gave up (bounded wait, full hash, bad coordinate) surfaces here,
    where the host waits for the device anyway, instead of handing out partial results."""
    st = status_word(n_dev.device)
    n, bad = torch.cat([n_dev.reshape(1), st]).tolist()
    raise_on_status(bad, n_dev.device)
    return int(n)


# =============================================================================== rulebook
def build_rulebook(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding, dilation, subm, transpose,
                   want_pairs=True):
    """(outids, nbr[K,n_out], pairs[K,2,n_in] or None, indice_num[K]) for one layer."""
    L = lib()
    if indices.dtype != torch.int32:
        raise TypeError("indices must be int32")
    indices = indices.contiguous()
    dev = indices.device
    n_in = indices.shape[0]
    K = int(ksize[0]) * int(ksize[1]) * int(ksize[2])
    grid = spatial_shape if subm else out_shape
    for shp in (spatial_shape, grid):
        if int(batch_size) * int(shp[0]) * int(shp[1]) * int(shp[2]) >= 2 ** 31 - 1:
            raise ValueError("ssconv_b200: batch*volume does not fit the int32 flat index")
    if K > 256:
        raise ValueError("ssconv_b200: kernel volume %d > 256" % K)
    skey = (n_in, int(batch_size), tuple(spatial_shape), tuple(grid), K)
    sbytes = _scratch_cache.get(skey)
    if sbytes is None:
        if len(_scratch_cache) > 4096:
            _scratch_cache.clear()
        sbytes = _scratch_cache[skey] = max(int(L.ssc_rulebook_scratch_bytes(n_in, int(batch_size), _i3(spatial_shape),
                                                                             _i3(grid), K)), 256)
    scratch = torch.empty(sbytes, dtype=torch.uint8, device=dev)
    small = torch.empty(K + 1, dtype=torch.int32, device=dev)   # [indice_num (K) | n_out]
    num = small[:K]
    pairs = torch.empty((K, 2, n_in), dtype=torch.int32, device=dev) if want_pairs else None
    st = status_word(dev)
    if subm:
        nbr = torch.empty((K, n_in), dtype=torch.int32, device=dev)
        _check(L.ssc_rulebook_subm(_p(indices), n_in, int(batch_size), _i3(spatial_shape), _i3(ksize), _i3(dilation),
                                   _p(nbr), _p(pairs), _p(num), _p(st), _p(scratch), scratch.numel(), _stream()))
        return indices, nbr, pairs, num
    n_out_dev = small[K:]
    geo = (_i3(spatial_shape), _i3(out_shape), _i3(ksize), _i3(stride), _i3(padding), _i3(dilation), int(transpose))
    _check(L.ssc_rulebook_conv_count(_p(indices), n_in, int(batch_size), *geo, _p(n_out_dev), _p(st), _p(scratch),
                                     scratch.numel(), None, _stream()))
    n_out = read_count(n_out_dev)  # the one host sync of a regular rulebook (the status word comes with it)
    outids = torch.empty((n_out, 4), dtype=torch.int32, device=dev)
    nbr = torch.empty((K, n_out), dtype=torch.int32, device=dev)
    _check(L.ssc_rulebook_conv_fill(_p(indices), n_in, int(batch_size), *geo, n_out, _p(outids), _p(nbr), _p(pairs),
                                    _p(num), _p(st), _p(scratch), scratch.numel(), None, _stream()))
    _note_ratio(_geometry_key(spatial_shape, ksize, stride, padding, dilation, transpose), n_in, n_out)
    return outids, nbr, pairs, num


# ------------------------------------------------------------------ rulebooks that run ahead
# The number of active outputs of a regular (strided) rulebook is only known on the device after
# its counting phase.  Waiting for it on the host stalls the GPU twice per layer (the wait itself,
# then the launches that follow).  A layer can instead size the second phase and its own kernel
# by a CAPACITY guessed from the output/input ratio this geometry produced before, queue
# everything, and read the count back once at the end; the count is then checked against the
# capacity and, if it did not fit, the layer is redone the slow way.  The layers chain this: a
# tensor with a pending count can feed the next layer (sp_ops/tensor.py), so the host reads counts
# back only where somebody looks at a result.  SSCONV_AHEAD=0 turns it off.
AHEAD = os.environ.get("SSCONV_AHEAD", "1") != "0"
AHEAD_MARGIN = 1.10
_ratio_hint = {}


def _geometry_key(spatial_shape, ksize, stride, padding, dilation, transpose):
    return (tuple(spatial_shape), tuple(ksize), tuple(stride), tuple(padding), tuple(dilation), bool(transpose))


def _note_ratio(key, n_in, n_out):
    if n_in > 0:
        r = float(n_out) / float(n_in)
        if r > _ratio_hint.get(key, 0.0):
            if len(_ratio_hint) > 4096:
                _ratio_hint.clear()
            _ratio_hint[key] = r


def get_indice_pairs_ahead(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding, dilation, transpose,
                           n_in_dev=None):
    """Regular rulebook whose output count stays on the device: returns [outids_cap [cap,4],
    LazyPairs (pending, capacity cap), indice_num] or None when no capacity can be guessed yet
    (first call for this geometry) or the feature is off.  The caller runs its kernel with
    n_out = pairs.capacity and reads the count back later (pairs.resolve()).  n_in_dev: device
    word with the exact number of input rows when `indices` itself is only filled up to a count
    that has not been read back yet (its length is then a capacity)."""
    if not AHEAD:
        return None
    key = _geometry_key(spatial_shape, ksize, stride, padding, dilation, transpose)
    ratio = _ratio_hint.get(key)
    if ratio is None:
        return None
    L = lib()
    if indices.dtype != torch.int32:
        raise TypeError("indices must be int32")
    indices = indices.contiguous()
    dev = indices.device
    n_in = indices.shape[0]
    K = int(ksize[0]) * int(ksize[1]) * int(ksize[2])
    cells = int(batch_size) * int(out_shape[0]) * int(out_shape[1]) * int(out_shape[2])
    if K > 256 or n_in == 0 or cells >= 2 ** 31 - 1:
        return None
    bound = min(n_in * K, cells)
    cap = min(bound, int(n_in * ratio * AHEAD_MARGIN) + 1024)
    skey = (n_in, int(batch_size), tuple(spatial_shape), tuple(out_shape), K)
    sbytes = _scratch_cache.get(skey)
    if sbytes is None:
        if len(_scratch_cache) > 4096:
            _scratch_cache.clear()
        sbytes = _scratch_cache[skey] = max(int(L.ssc_rulebook_scratch_bytes(n_in, int(batch_size), _i3(spatial_shape),
                                                                             _i3(out_shape), K)), 256)
    scratch = torch.empty(sbytes, dtype=torch.uint8, device=dev)
    n_out_dev = torch.empty(1, dtype=torch.int32, device=dev)
    st = status_word(dev)
    geo = (_i3(spatial_shape), _i3(out_shape), _i3(ksize), _i3(stride), _i3(padding), _i3(dilation), int(transpose))
    _check(L.ssc_rulebook_conv_count(_p(indices), n_in, int(batch_size), *geo, _p(n_out_dev), _p(st), _p(scratch),
                                     sbytes, _p(n_in_dev), _stream()))
    outids = torch.empty((cap, 4), dtype=torch.int32, device=dev)
    nbr = torch.empty((K, cap), dtype=torch.int32, device=dev)
    # the per-offset pair counts (indice_num) are not needed by the kernels that consume the table:
    # they are computed only if somebody turns the handle into reference-format pair lists
    _check(L.ssc_rulebook_conv_fill(_p(indices), n_in, int(batch_size), *geo, cap, _p(outids), _p(nbr), None, None,
                                    _p(st), _p(scratch), sbytes, _p(n_out_dev), _stream()))
    return [outids, LazyPairs(nbr, n_in, n_out_dev=n_out_dev, ratio_key=None if n_in_dev is not None else key), None]


def get_indice_pairs_subm_ahead(indices_cap, batch_size, spatial_shape, ksize, dilation, n_in_dev):
    """Submanifold rulebook on rows whose count is still on the device (indices_cap [cap, 4], the
    first n_in_dev[0] rows meaningful): LazyPairs over the table [K, cap], pending on the same device
    word.  Never waits for the device."""
    L = lib()
    indices_cap = indices_cap.contiguous()
    dev = indices_cap.device
    cap = indices_cap.shape[0]
    K = int(ksize[0]) * int(ksize[1]) * int(ksize[2])
    if K > 256:
        raise ValueError("ssconv_b200: kernel volume %d > 256" % K)
    if int(batch_size) * int(spatial_shape[0]) * int(spatial_shape[1]) * int(spatial_shape[2]) >= 2 ** 31 - 1:
        raise ValueError("ssconv_b200: batch*volume does not fit the int32 flat index")
    skey = (cap, int(batch_size), tuple(spatial_shape), tuple(spatial_shape), K)
    sbytes = _scratch_cache.get(skey)
    if sbytes is None:
        sbytes = _scratch_cache[skey] = max(int(L.ssc_rulebook_scratch_bytes(cap, int(batch_size), _i3(spatial_shape),
                                                                             _i3(spatial_shape), K)), 256)
    scratch = torch.empty(sbytes, dtype=torch.uint8, device=dev)
    nbr = torch.empty((K, cap), dtype=torch.int32, device=dev)
    _check(L.ssc_rulebook_subm_ahead(_p(indices_cap, torch.int32), cap, int(batch_size), _i3(spatial_shape), _i3(ksize),
                                     _i3(dilation), _p(nbr), _p(status_word(dev)), _p(scratch), sbytes, _p(n_in_dev),
                                     _stream()))
    return LazyPairs(nbr, cap, n_out_dev=n_in_dev)


def get_indice_pairs_3d(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding, dilation,
                        out_padding, subm, transpose):
    """[outids, indicePairs [K,2,N], indiceNum [K]] as getIndicePair<3> returns them
    (SS_Conv_lib/src/conv/indice_conv.h:21-131).  The neighbour table the CUDA kernels use is
    attached to the returned pair tensor as `_ssc_nbr`."""
    outids, nbr, pairs, num = build_rulebook(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding,
                                             dilation, bool(subm), bool(transpose))
    pairs._ssc_nbr = nbr
    return [outids, pairs, num]


def get_indice_pairs_lazy(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding, dilation, subm,
                          transpose):
    """Same as get_indice_pairs_3d but the pair lists are a LazyPairs (no pair-list kernels run
    unless somebody looks at them).  Used by the layers of this package."""
    outids, nbr, _, num = build_rulebook(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding,
                                         dilation, bool(subm), bool(transpose), want_pairs=False)
    return [outids, LazyPairs(nbr, indices.shape[0]), num]


def get_indice_pairs_grid_3d(indices, grid, batch_size, out_shape, spatial_shape, ksize, stride, padding, dilation,
                             out_padding, subm, transpose):
    """Pre-allocated-grid variant (indice_conv.h:133-244): the grid is not needed here."""
    return get_indice_pairs_3d(indices, batch_size, out_shape, spatial_shape, ksize, stride, padding, dilation,
                               out_padding, subm, transpose)


def _no_2d(*a, **k):
    raise NotImplementedError("2-D rulebooks are not part of the steerable (3-D) path")


get_indice_pairs_2d = _no_2d
get_indice_pairs_grid_2d = _no_2d


class LazyPairs(object):
    """Stand-in for the reference-format pair tensor [K, 2, n_in] of a rulebook that so far only
    exists as a neighbour table.  The CUDA kernels never need the pair lists, so the layers of
    this package build rulebooks without them; anything that does ask for tensor behaviour
    (indexing, .cpu(), arithmetic ...) gets the real tensor, built on first use by
    ssc_pairs_from_nbr."""

    def __init__(self, nbr, n_in, n_out_dev=None, ratio_key=None):
        self._nbr_cap = nbr                  # [K, capacity]; capacity == n_out unless built ahead
        self.capacity = int(nbr.shape[1])
        self._n_out_dev = n_out_dev          # device count of a rulebook built ahead, until resolved
        self._n_out = None if n_out_dev is not None else self.capacity
        self._ratio_key = ratio_key
        self._n_in = int(n_in)
        self._tensor = None
        self.shape = torch.Size((nbr.shape[0], 2, self._n_in))
        self.device = nbr.device
        self.dtype = torch.int32

    def pending(self):
        return self._n_out is None

    def resolve(self):
        """Reads the output count of a rulebook built ahead (one host sync).  Returns it, or None
        when it exceeded the capacity (everything computed from this handle is then invalid)."""
        if self._n_out is None:
            n = read_count(self._n_out_dev)
            if self._ratio_key is not None:
                _note_ratio(self._ratio_key, self._n_in, n)
            if n > self.capacity:
                return None
            self._n_out = n
            self._n_out_dev = None
        return self._n_out

    @property
    def _ssc_nbr(self):
        """The exact table [K, n_out], contiguous (compacted on first use if the capacity was larger)."""
        n = self.resolve()
        if n is None:
            raise RuntimeError("rulebook built ahead overflowed its capacity and was not rebuilt")
        if self.capacity != n:
            self._nbr_cap = self._nbr_cap[:, :n].contiguous()
            self.capacity = n
        return self._nbr_cap

    def to(self, *args, **kwargs):
        return self

    def materialize(self):
        if self._tensor is None:
            nbr = self._ssc_nbr
            K, n_out = nbr.shape
            pairs = torch.empty((K, 2, self._n_in), dtype=torch.int32, device=nbr.device)
            num = torch.empty(K, dtype=torch.int32, device=nbr.device)
            nbytes = int(lib().ssc_pairs_from_nbr_scratch_bytes(K, n_out))
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=nbr.device)
            _check(lib().ssc_pairs_from_nbr(_p(nbr), K, n_out, self._n_in, _p(pairs), _p(num), _p(scratch), nbytes,
                                            _stream()))
            pairs._ssc_nbr = nbr
            self._tensor = pairs
        return self._tensor

    def __getattr__(self, name):  # only reached for attributes this class does not define
        return getattr(self.materialize(), name)

    def __getitem__(self, item):
        return self.materialize()[item]

    def __len__(self):
        return self.shape[0]


def _table_for(pairs, num, n_out, inverse=False):
    """(nbr, n_out_dev): the table a kernel launch with bound n_out should use.  n_out_dev is the
    device row count when the rulebook was built ahead, is still pending, and n_out is its
    capacity; otherwise None and the table is exact."""
    if isinstance(pairs, LazyPairs) and not inverse and pairs.pending() and pairs.capacity == n_out:
        return pairs._nbr_cap, pairs._n_out_dev
    return neighbour_table(pairs, num, n_out, inverse), None


def neighbour_table(pairs, num, n_out, inverse=False):
    """nbr [K, n_out] for a reference-format rulebook (cached on the pair tensor when possible)."""
    if isinstance(pairs, LazyPairs):
        if not inverse and pairs._ssc_nbr.shape[1] == n_out:
            return pairs._ssc_nbr
        pairs = pairs.materialize()
    nbr = getattr(pairs, "_ssc_nbr", None)
    if nbr is not None and not inverse and nbr.shape[1] == n_out and nbr.device == pairs.device:
        return nbr
    cache = "_ssc_nbr_inv" if inverse else "_ssc_nbr"
    cached = getattr(pairs, cache, None)
    if cached is not None and cached.shape[1] == n_out:
        return cached
    pairs = pairs.contiguous()
    K, _, n_cols = pairs.shape
    nbr = torch.empty((K, n_out), dtype=torch.int32, device=pairs.device)
    _check(lib().ssc_pairs_to_nbr(_p(pairs, torch.int32), _p(num.to(pairs.device), torch.int32), K, n_cols, int(n_out),
                                  int(bool(inverse)), _p(nbr), _stream()))
    try:
        setattr(pairs, cache, nbr)
    except Exception:
        pass
    return nbr


# ============================================================== materialisation and conv
def materialize(weight, basis, block_table, n_blocks_in, out_field, in_field, c_out, c_in, K):
    flt = torch.empty((K, c_in, c_out), dtype=torch.float32, device=weight.device)
    _check(lib().ssc_materialize(_p(weight, torch.float32), _p(basis, torch.float32), _p(block_table, torch.int32),
                                 int(n_blocks_in), _p(out_field, torch.int32), _p(in_field, torch.int32), int(c_out),
                                 int(c_in), int(K), _p(flt), _stream()))
    return flt


def pack_filters(filters_kio, prec=PREC_TF32):
    """Tensor-core operand image (TF32 or fp16) of contiguous filters [K, Cin, Cout]."""
    K, c_in, c_out = filters_kio.shape
    nbytes = lib().ssc_conv_packed_bytes(K, c_in, c_out, prec)
    if nbytes == 0:
        raise ValueError("channel count not supported by the tensor-core path")
    packed = torch.empty(int(nbytes), dtype=torch.uint8, device=filters_kio.device)
    _check(lib().ssc_conv_pack_filters(_p(filters_kio, torch.float32), K, c_in, c_out, prec, _p(packed), _stream()))
    return packed


def _resolve_precision(c_in, c_out, precision=None):
    mode = precision or _precision
    if mode == "auto":
        mode = "tf32" if (c_in >= 16 and c_out <= 512) else "fp32"
    return mode


# Layers with fewer output rows do not stage a TF32-rounded copy of their input rows (the extra
# launch would cost more than it saves), so no staging buffer is allocated for them.
STAGING_MIN_ROWS = 8 * 128

# Which tensor-core kernel a convolution call takes: 'auto' (by shape, see _use_pairs), 'rows' (the
# output-stationary kernel: one CTA per 128 output rows, bitwise repeatable) or 'pairs' (the
# pair-list kernel: dense 128-pair tiles per kernel offset, reductions into the output rows).
_algo = os.environ.get("SSCONV_ALGO", "auto")


def set_algo(mode):
    global _algo
    if mode not in ("auto", "rows", "pairs"):
        raise ValueError("algo must be 'auto', 'rows' or 'pairs'")
    _algo = mode


def get_algo():
    return _algo


def _use_pairs(K, c_in, c_out, n_out, prec, algo=None):
    """The pair-list kernel pays when a row tile of the output-stationary kernel would be mostly
    absent rows AND the layer is wide enough for the tensor cores to be the limit: many kernel
    offsets (a 5^3 submanifold kernel at 10 % occupancy fills a tenth of its table) and at least
    128 x 128 channels.  Narrow 3^3 layers stay output-stationary (their bound is the gather)."""
    algo = algo or _algo
    if algo == "rows" or not lib().ssc_conv_pairs_supported(int(c_in), int(c_out), int(prec)):
        return False
    if algo == "pairs":
        return True
    return K >= 64 and c_in >= 128 and c_out >= 128 and n_out >= 8 * 128


def pair_lists(nbr):
    """Compacted per-offset (input row, output row) lists of a neighbour table, kept with the
    table (layers that share a rulebook share them)."""
    kept = getattr(nbr, "_ssc_pair_lists", None)
    if kept is not None:
        return kept
    K, n_out = nbr.shape
    nbytes = int(lib().ssc_conv_pairs_list_bytes(K, n_out))
    lists = torch.empty(nbytes, dtype=torch.uint8, device=nbr.device)
    _check(lib().ssc_conv_pairs_build(_p(nbr, torch.int32), K, n_out, _p(lists), nbytes, _stream()))
    if not torch.cuda.is_current_stream_capturing():
        try:
            nbr._ssc_pair_lists = lists
        except Exception:
            pass
    return lists


PRESTAGED = 0x100
TABLE_IN_ORDER = 0x200
# (features.data_ptr(), filters.data_ptr()) -> (prec, packed, scratch, nbytes) left by conv_prepare for the
# conv_forward call that follows on the same tensors
_prepared = {}
_side_streams = {}


def side_stream(device, which=0):
    """Side streams used while a CUDA graph is recorded, to give the graph parallel branches:
    0 - the part of a convolution call that does not need its rulebook (filter packing, staging);
    1 - the rulebook of a layer, which needs the indices of its input but not the features, so it
        can run next to the kernels that are still producing those features."""
    key = (torch.device(device).index, which)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device)
    return _side_streams[key]


def rulebook_next_to_features(rows, build):
    """build() queues a rulebook.  While a graph is recorded and the input's indices are known to be
    complete at an event (rows.indices_ready, left by the layer that made them), it is queued on side
    stream 1 behind that event only - not behind the feature kernels on the current stream - and the
    current stream joins afterwards.  Returns (build(), event after the rulebook or None)."""
    if not torch.cuda.is_current_stream_capturing():
        return build(), None
    dev = torch.cuda.current_device()
    cur = torch.cuda.current_stream(dev)
    ready = getattr(rows, "indices_ready", None) if rows is not None else None
    after = torch.cuda.Event()
    if ready is None:
        out = build()
        after.record(cur)
        return out, after
    rb = side_stream(dev, 1)
    rb.wait_event(ready)
    with torch.cuda.stream(rb):
        out = build()
        after.record(rb)
    cur.wait_stream(rb)
    return out, after


def conv_prepare(features, filters, precision=None):
    """Everything of a tensor-core convolution call that does not need the rulebook - the packed
    filter image and the staged (TF32- or fp16-rounded) copy of the feature rows - queued on the
    current stream (meant to be a side stream running next to the rulebook kernels).  The
    conv_forward call on the same two tensors picks the result up.  Returns False when the call
    would not use a staged image (exact fp32, small layers)."""
    flt = filters.reshape(-1, filters.shape[-2], filters.shape[-1])
    if not (flt.is_contiguous() and features.is_contiguous() and features.dtype == torch.float32):
        return False      # (16-bit features are their own staged image: nothing to prepare but the filters)
    K, c_in, c_out = flt.shape
    mode = _resolve_precision(c_in, c_out, precision)
    if mode not in _PREC_OF or (mode != "tf32" and c_out > 512):
        return False
    if mode == "tf32" and features.shape[0] < STAGING_MIN_ROWS:
        return False
    prec = _PREC_OF[mode]
    packed = pack_filters(flt, prec)
    nbytes = int(lib().ssc_conv_scratch_bytes(features.shape[0], c_in, c_out, prec))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=features.device)
    _check(lib().ssc_conv_stage(_p(features, torch.float32), features.shape[0], c_in, prec, _p(scratch), nbytes, _stream()))
    _prepared[(features.data_ptr(), flt.data_ptr())] = (prec, packed, scratch, nbytes)
    return True


def conv_forward(features, filters, nbr, n_out, precision=None, n_out_dev=None, row_order=None, algo=None,
                 table_in_order=False):
    """out [n_out, Cout] = sum over offsets of gathered rows times filters (one launch).
    n_out_dev: device word with the exact row count when n_out is only a capacity.
    row_order: permutation of the output rows from nbr_row_order (same result, fewer steps).
    table_in_order: nbr is the table with its columns already in that order (nbr_row_order_planes).
    algo: None (the module setting), 'rows' or 'pairs' (see set_algo)."""
    if filters.dim() != 3:
        filters = filters.reshape(-1, filters.shape[-2], filters.shape[-1])
    K, c_in, c_out = filters.shape
    if features.shape[1] != c_in:
        raise ValueError("features have %d channels, filters expect %d" % (features.shape[1], c_in))
    features = features.contiguous()
    if features.dtype in _PREC_OF_DTYPE:
        if c_in % 8 == 0 and c_out <= 512 and row_order is None:
            return _conv_forward_stored16(features, filters, nbr, n_out, n_out_dev, algo)
        features = features.float()
    out = torch.empty((n_out, c_out), dtype=torch.float32, device=features.device)
    mode = _resolve_precision(c_in, c_out, precision)
    st = status_word(features.device)
    if mode in ("fp16", "bf16") and c_out > 512:
        mode = "fp32"
    if (mode in _PREC_OF and n_out_dev is None and row_order is None and nbr.shape[1] == n_out
            and _use_pairs(K, c_in, c_out, n_out, _PREC_OF[mode], algo)):
        return _conv_forward_pairs(features, filters, nbr, n_out, _PREC_OF[mode], out, st)
    flag = TABLE_IN_ORDER if (table_in_order and row_order is not None) else 0
    if flag and mode not in _PREC_OF:
        raise ValueError("ssconv_b200: a table in row order needs a tensor-core precision")
    ready = None
    if _prepared:   # only the call that directly follows conv_prepare may use what it left
        ready = _prepared.pop((features.data_ptr(), filters.data_ptr()), None)
        _prepared.clear()
    if ready is not None and ready[0] == _PREC_OF.get(mode, -1):
        prec, packed, scratch, nbytes = ready
        _check(lib().ssc_conv_fwd_ordered(_p(features, torch.float32), features.shape[0], c_in, _p(packed), K, c_out,
                                          _p(nbr, torch.int32), int(n_out), prec | PRESTAGED | flag, _p(out), _p(st), _p(scratch),
                                          nbytes, _p(n_out_dev), _p(row_order), _stream()))
    elif mode in _PREC_OF:
        prec = _PREC_OF[mode]
        packed = _packed_filters(filters, prec)
        # the 16-bit kernels always gather from their staged image
        # (layers with up to 16 input channels have filters packed for several offsets per operand row,
        #  which the kernel feeds from the staged rows only)
        stage = prec != PREC_TF32 or n_out >= STAGING_MIN_ROWS or c_in <= 16
        nbytes = lib().ssc_conv_scratch_bytes(features.shape[0], c_in, c_out, prec) if stage else 0
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=features.device) if nbytes else None
        _check(lib().ssc_conv_fwd_ordered(_p(features, torch.float32), features.shape[0], c_in, _p(packed), K, c_out,
                                          _p(nbr, torch.int32), int(n_out), prec | flag, _p(out), _p(st), _p(scratch), nbytes,
                                          _p(n_out_dev), _p(row_order), _stream()))
    else:
        filters = filters.contiguous()
        _check(lib().ssc_conv_fwd(_p(features, torch.float32), features.shape[0], c_in, _p(filters, torch.float32), K,
                                  c_out, _p(nbr, torch.int32), int(n_out), PREC_FP32, _p(out), _p(st), None, 0,
                                  _p(n_out_dev), _stream()))
    return out


def _packed_filters(filters, prec):
    """Operand image of filters [K, Cin, Cout], kept with the tensor until it changes."""
    tag = (prec, filters._version)
    packed = getattr(filters, "_ssc_packed", None)
    if packed is None or getattr(filters, "_ssc_packed_version", None) != tag:
        packed = pack_filters(filters.contiguous(), prec)
        try:
            filters._ssc_packed = packed
            filters._ssc_packed_version = tag
        except Exception:
            pass
    return packed


def _conv_forward_stored16(features, filters, nbr, n_out, n_out_dev, algo):
    """Convolution on features stored as fp16 / bf16 rows [n_in, Cin] (Cin a multiple of 8): the rows
    ARE the staged operand image, so the call is the kernel alone."""
    K, c_in, c_out = filters.shape
    prec = _PREC_OF[_PREC_OF_DTYPE[features.dtype]]
    out = torch.empty((n_out, c_out), dtype=torch.float32, device=features.device)
    st = status_word(features.device)
    packed = _packed_filters(filters, prec)
    nbytes = features.numel() * 2
    if n_out_dev is None and nbr.shape[1] == n_out and _use_pairs(K, c_in, c_out, n_out, prec, algo):
        lists = pair_lists(nbr)
        _check(lib().ssc_conv_fwd_pairs(None, features.shape[0], c_in, _p(packed), K, c_out, _p(lists), lists.numel(),
                                        int(n_out), prec | PRESTAGED, _p(out), _p(st), _p(features), nbytes, _stream()))
        return out
    _check(lib().ssc_conv_fwd_ordered(None, features.shape[0], c_in, _p(packed), K, c_out, _p(nbr, torch.int32),
                                      int(n_out), prec | PRESTAGED, _p(out), _p(st), _p(features), nbytes, _p(n_out_dev),
                                      None, _stream()))
    return out


def _conv_forward_pairs(features, filters, nbr, n_out, prec, out, st):
    """The pair-list kernel: staging + (lists, once per table) + strips + one persistent launch."""
    K, c_in, c_out = filters.shape
    ready = None
    if _prepared:
        ready = _prepared.pop((features.data_ptr(), filters.data_ptr()), None)
        _prepared.clear()
    flag = 0
    if ready is not None and ready[0] == prec:
        _, packed, scratch, nbytes = ready
        flag = PRESTAGED
    else:
        packed = _packed_filters(filters, prec)
        nbytes = int(lib().ssc_conv_scratch_bytes(features.shape[0], c_in, c_out, prec))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=features.device)
    lists = pair_lists(nbr)
    _check(lib().ssc_conv_fwd_pairs(_p(features, torch.float32), features.shape[0], c_in, _p(packed), K, c_out, _p(lists),
                                    lists.numel(), int(n_out), prec | flag, _p(out), _p(st), _p(scratch), nbytes, _stream()))
    return out


def indice_conv_fp32(features, filters, indice_pairs, indice_num, num_act_out, inverse, subm):
    """Reference signature (SS_Conv_lib/src/ss_conv_ops.h:43-45); filters [k,k,k,Cin,Cout]
    (a permuted view is accepted).  The submanifold centre needs no special case."""
    if features.dtype != torch.float32 and features.dtype not in _PREC_OF_DTYPE:
        raise TypeError("indice_conv_fp32 expects float32 features (or features stored in fp16 / bf16 by this library)")
    c_in, c_out = filters.shape[-2], filters.shape[-1]
    cached = getattr(filters, "_ssc_flat", None)
    if cached is not None and cached[0] == filters._version:
        flt = cached[1]
    else:
        flt = filters.reshape(-1, c_in, c_out).contiguous()  # no copy when already contiguous
        try:
            filters._ssc_flat = (filters._version, flt)
        except Exception:
            pass
    nbr, n_out_dev = _table_for(indice_pairs, indice_num, int(num_act_out), bool(inverse))
    order = None
    if inverse and n_out_dev is None and int(num_act_out) >= ROW_ORDER_MIN_ROWS and nbr.shape[0] > 1:
        # an inverse convolution gathers through its partner's table with the roles exchanged: like the
        # input gradient, every output row uses only the offsets of its parity class
        order = nbr_row_order(nbr)
    return conv_forward(features, flt, nbr, int(num_act_out), n_out_dev=n_out_dev, row_order=order)


def _not_built(name):
    def f(*a, **k):
        raise NotImplementedError(name + " is not built: the reference's own Python never calls it "
                                  "(dead entry point of its extension)")
    f.__name__ = name
    return f


def input_major_table(nbr, n_in):
    """nbr_in [K, n_in]: for every (offset, input row) the output row it contributes to, or -1."""
    K, n_out = nbr.shape
    nbr_in = torch.empty((K, int(n_in)), dtype=torch.int32, device=nbr.device)
    _check(lib().ssc_nbr_transpose(_p(nbr, torch.int32), K, n_out, int(n_in), _p(nbr_in), _stream()))
    return nbr_in


# Tables with fewer rows are not worth the three launches of the ordering.
ROW_ORDER_MIN_ROWS = 64 * 128
def nbr_row_order_planes(nbr, ksize, n_rows_dev=None, with_table=False):
    """Permutation of the rows of a forward table nbr [K, n] (K = ksize[0] * ksize[1] * ksize[2]) that
    groups the rows by the kernel planes their neighbours lie in, groups that allow more offsets first
    (for conv_forward(row_order=...)); None for kernels it does not cover.  n_rows_dev: device word
    with the live row count when n is a capacity.  with_table: also return the table with its
    columns moved into that order (for conv_forward(..., table_in_order=True)).
    Opt-in: on a 64 -> 76 channel layer of 129 k surface rows the call drops from 0.154 to 0.129 ms
    (45 % fewer steps, the long tiles first) and the ordering takes 0.044 ms, so it pays from the
    third layer that shares a table on; the layers do not ask for it themselves."""
    K, n = nbr.shape
    ks = [int(v) for v in ksize]
    if len(ks) != 3 or ks[0] * ks[1] * ks[2] != K or n == 0:
        return None
    nbytes = int(lib().ssc_nbr_row_order_planes_scratch_bytes(_i3(ks), n))
    if nbytes == 0:
        return None
    order = torch.empty(n, dtype=torch.int32, device=nbr.device)
    moved = torch.empty_like(nbr) if with_table else None
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=nbr.device)
    _check(lib().ssc_nbr_row_order_planes(_p(nbr, torch.int32), _i3(ks), n, _p(order), _p(moved), _p(scratch), nbytes,
                                          _p(n_rows_dev), _stream()))
    return (order, moved) if with_table else order


def nbr_row_order(nbr):
    """Permutation of the rows of nbr [K, n] that groups rows by the first kernel offset they use
    (for conv_forward(row_order=...)); None where the library has no ordering for this table."""
    K, n = nbr.shape
    nbytes = int(lib().ssc_nbr_row_order_scratch_bytes(K, n))
    if nbytes == 0 or n == 0:
        return None
    order = torch.empty(n, dtype=torch.int32, device=nbr.device)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=nbr.device)
    _check(lib().ssc_nbr_row_order(_p(nbr, torch.int32), K, n, _p(order), _p(scratch), nbytes, _stream()))
    return order


def conv_wgrad(features, out_grad, nbr, precision=None):
    """d_filters [K, Cin, Cout] = sum over output rows of gathered input rows (outer) out_grad rows
    (tensor cores with TF32 operands or exact fp32, chosen like the forward pass)."""
    K, n_out = nbr.shape
    c_in, c_out = features.shape[1], out_grad.shape[1]
    # the filter gradient has no 16-bit form: 'fp16' / 'bf16' take the TF32 kernel
    mode = PREC_TF32 if _resolve_precision(c_in, c_out, precision) in _PREC_OF else PREC_FP32
    d_flt = torch.empty((K, c_in, c_out), dtype=torch.float32, device=features.device)
    nbytes = int(lib().ssc_conv_wgrad_scratch_bytes(K, c_in, c_out, n_out))
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=features.device)
    _check(lib().ssc_conv_wgrad(_p(features, torch.float32), c_in, _p(out_grad, torch.float32), c_out,
                                _p(nbr, torch.int32), K, n_out, mode, _p(d_flt), _p(status_word(features.device)),
                                _p(scratch), nbytes, _stream()))
    return d_flt


def conv_backward(features, flt, out_bp, nbr, nbr_in=None, order=None, precision=None):
    """(input gradient [n_in, Cin], filter gradient [K, Cin, Cout]) of out = conv(features, flt [K, Cin, Cout])
    over the table nbr [K, n_out].  nbr_in / order: the input-major table and its row order when the
    caller kept them with the rulebook (built here otherwise)."""
    n_in = features.shape[0]
    # the two gradients do not depend on each other: while a graph is recorded the filter gradient
    # goes to a side stream, so the graph runs it next to the input gradient
    forked = torch.cuda.is_current_stream_capturing()
    if forked:
        cur, side = torch.cuda.current_stream(features.device), side_stream(features.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            d_flt = conv_wgrad(features, out_bp, nbr, precision)
    if nbr_in is None:
        kept = getattr(nbr, "_ssc_in_major", None)     # layers that share a rulebook share these too
        if kept is not None and kept[0] == n_in:
            nbr_in, order = kept[1], kept[2]
        else:
            nbr_in = input_major_table(nbr, n_in)
            # rows of the input-major table use few of the offsets each (their parity class under a
            # stride): grouped tiles skip the rest
            order = nbr_row_order(nbr_in) if (n_in >= ROW_ORDER_MIN_ROWS and nbr_in.shape[0] > 1) else None
            if not forked:                             # tensors made while a graph is recorded belong to the graph
                try:
                    nbr._ssc_in_major = (n_in, nbr_in, order)
                except Exception:
                    pass
    d_in = conv_forward(out_bp, flt.transpose(1, 2).contiguous(), nbr_in, n_in, precision, row_order=order)
    if forked:
        cur.wait_stream(side)
    else:
        d_flt = conv_wgrad(features, out_bp, nbr, precision)
    return d_in, d_flt


def indice_conv_backward_fp32(features, filters, out_bp, indice_pairs, indice_num, inverse, subm):
    """Reference signature (SS_Conv_lib/src/ss_conv_ops.h:46-48): [input_grad, filters_grad].
    The input gradient is the forward gather-GEMM over the input-major table with the filters
    transposed; both gradients use the operand precision set for the forward pass.  The
    submanifold centre needs no special case."""
    if features.dtype != torch.float32:
        raise TypeError("indice_conv_backward_fp32 expects float32 features")
    features, out_bp = features.contiguous(), out_bp.contiguous()
    c_in, c_out = filters.shape[-2], filters.shape[-1]
    flt = filters.reshape(-1, c_in, c_out)
    n_in, n_out = features.shape[0], out_bp.shape[0]
    nbr = neighbour_table(indice_pairs, indice_num, n_out, bool(inverse))
    d_in, d_flt = conv_backward(features, flt, out_bp, nbr)
    return [d_in, d_flt.reshape(filters.shape)]


def indice_conv_half(features, filters, indice_pairs, indice_num, num_act_out, inverse, subm):
    """Reference signature (SS_Conv_lib/src/ss_conv_ops.h:49-51): half tensors in, half tensor out.
    The tensor cores take the fp16 operands as they are and accumulate in fp32 (the reference's
    cuBLAS half GEMM per kernel offset rounds every partial product sum to fp16); only the result
    is rounded to fp16."""
    if features.dtype != torch.half or filters.dtype != torch.half:
        raise TypeError("indice_conv_half expects float16 features and filters")
    c_in, c_out = filters.shape[-2], filters.shape[-1]
    flt = filters.reshape(-1, c_in, c_out).float()
    nbr, n_out_dev = _table_for(indice_pairs, indice_num, int(num_act_out), bool(inverse))
    out = conv_forward(features.float(), flt, nbr, int(num_act_out), precision="fp16", n_out_dev=n_out_dev)
    return out.half()


def indice_conv_backward_half(features, filters, out_bp, indice_pairs, indice_num, inverse, subm):
    """Reference signature (SS_Conv_lib/src/ss_conv_ops.h:52-54): [input_grad, filters_grad] in half.
    The input gradient runs on fp16 operands, the filter gradient on TF32 operands (the same
    significand, fp32 range), both with fp32 accumulation."""
    if features.dtype != torch.half or filters.dtype != torch.half:
        raise TypeError("indice_conv_backward_half expects float16 features and filters")
    c_in, c_out = filters.shape[-2], filters.shape[-1]
    flt = filters.reshape(-1, c_in, c_out).float()
    feats, grad = features.float().contiguous(), out_bp.float().contiguous()
    n_in, n_out = feats.shape[0], grad.shape[0]
    nbr = neighbour_table(indice_pairs, indice_num, n_out, bool(inverse))
    nbr_in = input_major_table(nbr, n_in)
    order = nbr_row_order(nbr_in) if (n_in >= ROW_ORDER_MIN_ROWS and nbr_in.shape[0] > 1) else None
    d_in = conv_forward(grad, flt.transpose(1, 2).contiguous(), nbr_in, n_in, precision="fp16", row_order=order)
    d_flt = conv_wgrad(feats, grad, nbr, precision="tf32")
    return [d_in.half(), d_flt.reshape(filters.shape).half()]


# ================================================================================== pools
def indice_maxpool_fp32(features, indice_pairs, indice_num, num_act):
    features = features.contiguous()
    nbr, n_out_dev = _table_for(indice_pairs, indice_num, int(num_act))
    out = torch.empty((int(num_act), features.shape[1]), dtype=torch.float32, device=features.device)
    _check(lib().ssc_maxpool_fwd(_p(features, torch.float32), features.shape[1], _p(nbr), nbr.shape[0], int(num_act),
                                 _p(out), _p(n_out_dev), _stream()))
    return out


def indice_avgpool_fp32(features, indice_pairs, indice_num, num_act, summaryrf):
    features = features.contiguous()
    nbr, n_out_dev = _table_for(indice_pairs, indice_num, int(num_act))
    out = torch.empty((int(num_act), features.shape[1]), dtype=torch.float32, device=features.device)
    rf = None if summaryrf is None else summaryrf.to(torch.int32).contiguous()
    _check(lib().ssc_avgpool_fwd(_p(features, torch.float32), features.shape[1], _p(nbr), nbr.shape[0], int(num_act),
                                 _p(rf), _p(out), _p(n_out_dev), _stream()))
    return out


def indiceSummaryRF(indice_pairs, indice_num, num_act):
    nbr = neighbour_table(indice_pairs, indice_num, int(num_act))
    rf = torch.empty(int(num_act), dtype=torch.int32, device=nbr.device)
    _check(lib().ssc_summary_rf(_p(nbr), nbr.shape[0], int(num_act), _p(rf), _stream()))
    return rf


def indice_maxpool_half(features, indice_pairs, indice_num, num_act):
    """(SS_Conv_lib/src/ss_conv_ops.h:58) half tensors in and out; the pool kernel works on the
    widened values (a maximum of fp16 values is exact), the result is narrowed again."""
    if features.dtype != torch.half:
        raise TypeError("indice_maxpool_half expects float16 features")
    return indice_maxpool_fp32(features.float(), indice_pairs, indice_num, num_act).half()


def indice_avgpool_half(features, indice_pairs, indice_num, num_act, summaryrf):
    """(SS_Conv_lib/src/ss_conv_ops.h:62) half tensors in and out, sums in fp32, one rounding at the end."""
    if features.dtype != torch.half:
        raise TypeError("indice_avgpool_half expects float16 features")
    return indice_avgpool_fp32(features.float(), indice_pairs, indice_num, num_act, summaryrf).half()
def indice_maxpool_backward_fp32(features, out_features, out_bp, indice_pairs, indice_num):
    """(SS_Conv_lib/src/ss_conv_ops.h:58-59) gradient to every input that equals its pooled value."""
    features, out_features, out_bp = features.contiguous(), out_features.contiguous(), out_bp.contiguous()
    nbr_in = input_major_table(neighbour_table(indice_pairs, indice_num, out_features.shape[0]), features.shape[0])
    d_in = torch.empty_like(features)
    _check(lib().ssc_maxpool_bwd(_p(features, torch.float32), _p(out_features, torch.float32), _p(out_bp, torch.float32),
                                 features.shape[1], _p(nbr_in), nbr_in.shape[0], features.shape[0], _p(d_in), _stream()))
    return d_in


def indice_avgpool_backward_fp32(features, out_features, out_bp, indice_pairs, indice_num, summaryrf):
    """(SS_Conv_lib/src/ss_conv_ops.h:62-63) d_in[i] = sum of out_bp[o] / summaryrf[o]."""
    features, out_bp = features.contiguous(), out_bp.contiguous()
    nbr_in = input_major_table(neighbour_table(indice_pairs, indice_num, out_bp.shape[0]), features.shape[0])
    rf = None if summaryrf is None else summaryrf.to(torch.int32).contiguous()
    d_in = torch.empty_like(features)
    _check(lib().ssc_avgpool_bwd(_p(out_bp, torch.float32), features.shape[1], _p(nbr_in), nbr_in.shape[0],
                                 features.shape[0], _p(rf), _p(d_in), _stream()))
    return d_in


def indice_maxpool_backward_half(features, out_features, out_bp, indice_pairs, indice_num):
    """(SS_Conv_lib/src/ss_conv_ops.h:59) half tensors in and out."""
    return indice_maxpool_backward_fp32(features.float(), out_features.float(), out_bp.float(), indice_pairs,
                                        indice_num).half()


def indice_avgpool_backward_half(features, out_features, out_bp, indice_pairs, indice_num, summaryrf):
    """(SS_Conv_lib/src/ss_conv_ops.h:63) half tensors in and out."""
    return indice_avgpool_backward_fp32(features.float(), out_features.float(), out_bp.float(), indice_pairs, indice_num,
                                        summaryrf).half()
indice_field_maxpool_fp32 = _not_built("indice_field_maxpool_fp32")
indice_field_maxpool_half = _not_built("indice_field_maxpool_half")


def global_avgpool_fp(feats, offsets, out, maxidx, n_proposal, c):
    _check(lib().ssc_global_avgpool_fwd(_p(feats, torch.float32), _p(offsets, torch.int32), int(n_proposal), int(c),
                                        _p(out, torch.float32), _stream()))


def global_maxpool_fp(feats, offsets, out, maxidx, n_proposal, c):
    _check(lib().ssc_global_maxpool_fwd(_p(feats, torch.float32), _p(offsets, torch.int32), int(n_proposal), int(c),
                                        _p(out, torch.float32), _p(maxidx, torch.int32), _stream()))


def global_avgpool_bp(d_feats, offsets, maxidx, d_out, n_proposal, c):
    """(SS_Conv_lib/src/pool/global_avgpool.h:25) writes d_feats [N, C] in place."""
    _check(lib().ssc_global_avgpool_bwd(_p(d_out, torch.float32), _p(offsets, torch.int32), int(n_proposal), int(c),
                                        d_feats.shape[0], _p(d_feats, torch.float32), _stream()))


def global_maxpool_bp(d_feats, offsets, maxidx, d_out, n_proposal, c):
    _check(lib().ssc_global_maxpool_bwd(_p(d_out, torch.float32), _p(maxidx, torch.int32), int(n_proposal), int(c),
                                        d_feats.shape[0], _p(d_feats, torch.float32), _stream()))


def batch_offsets(indices, batch_size, n_dev=None):
    """Row offsets [B+1] (int32, on device) of the samples of an indices tensor, no host sync.
    n_dev: device word with the exact row count when the tensor's length is only a capacity."""
    off = torch.empty(int(batch_size) + 1, dtype=torch.int32, device=indices.device)
    _check(lib().ssc_batch_offsets(_p(indices.contiguous(), torch.int32), indices.shape[0], int(batch_size), _p(off),
                                   _p(n_dev), _stream()))
    return off


# =========================================================================== voxelization
def voxel2point_map(inverse, ids, output_maps, n_point, max_active, mode):
    _check(lib().ssc_voxel2point_map(_p(inverse, torch.int32), _p(ids, torch.int32), _p(output_maps, torch.int32),
                                     int(n_point), output_maps.shape[0], int(max_active), int(mode), _stream()))


def voxelize_fp(feats, output_feats, map_rule, mode, n_voxel, max_active, c):
    _check(lib().ssc_voxelize_fwd(_p(feats, torch.float32), _p(output_feats, torch.float32), _p(map_rule, torch.int32),
                                  int(mode), int(n_voxel), int(max_active), int(c), _stream()))


def voxelize_bp(d_output_feats, d_feats, map_rule, mode, n_voxel, max_active, c):
    """(SS_Conv_lib/src/ss_conv_ops.h:71-72) writes d_feats [N, C] in place."""
    _check(lib().ssc_voxelize_bwd(_p(d_output_feats, torch.float32), _p(map_rule, torch.int32), int(mode), int(n_voxel),
                                  int(max_active), int(c), d_feats.shape[0], _p(d_feats, torch.float32), _stream()))

voxelize_idx = _not_built("voxelize_idx")
point_recover_fp = _not_built("point_recover_fp")
point_recover_bp = _not_built("point_recover_bp")


def steer(points, feats, ids, rot, trans, scale, dmats, chan):
    """(new_points [N,3], new_feats [N,C]) of the feature-steering change of frame (one launch)."""
    n, c = feats.shape
    new_points = torch.empty((n, 3), dtype=torch.float32, device=feats.device)
    new_feats = torch.empty((n, c), dtype=torch.float32, device=feats.device)
    _check(lib().ssc_steer_fwd(_p(points, torch.float32), _p(feats, torch.float32), _p(ids, torch.int32),
                               _p(rot, torch.float32), _p(trans, torch.float32), _p(scale), _p(dmats, torch.float32),
                               dmats.shape[1], _p(chan, torch.int32), n, c, rot.shape[0], _p(new_points), _p(new_feats),
                               _stream()))
    return new_points, new_feats


def p2v_stats(points, batch_ids, grid, unit):
    """[n outside the grid, n places where batch_ids decreases, n places where it changes, last id]
    of a point batch (one kernel, one read-back)."""
    stats = torch.empty(4, dtype=torch.int32, device=points.device)
    _check(lib().ssc_p2v_stats(_p(points, torch.float32), _p(batch_ids, torch.int32), points.shape[0], _i3(grid),
                               _F3(*[float(u) for u in unit]), _p(stats), _stream()))
    return stats.tolist()


def point2voxel(points, feats, batch_ids, batch_size, grid, unit, mode, ahead=False):
    """Fused voxelizer core: (voxel_indices [M,4] int32, inverse [N] int32, voxel_feats [M,C])
    for batch-sorted, in-range points (one host sync for M).  ahead=True skips that sync: the
    outputs then have N rows (a voxel count can never exceed the point count), of which the first
    M are meaningful, and a fourth value is returned, the device word holding M."""
    L = lib()
    dev = points.device
    points = points.contiguous().float()
    feats = feats.contiguous().float()
    batch_ids = batch_ids.contiguous().to(torch.int32)
    n = points.shape[0]
    sbytes = L.ssc_p2v_scratch_bytes(n, int(batch_size), _i3(grid))
    scratch = torch.empty(max(int(sbytes), 256), dtype=torch.uint8, device=dev)
    m_dev = torch.empty(1, dtype=torch.int32, device=dev)
    st = status_word(dev)
    unit3 = _F3(*[float(u) for u in unit])
    _check(L.ssc_p2v_count(_p(points), _p(batch_ids), n, int(batch_size), _i3(grid), unit3, _p(m_dev), _p(st),
                           _p(scratch), scratch.numel(), _stream()))
    m = n if ahead else read_count(m_dev)
    vox = torch.empty((m, 4), dtype=torch.int32, device=dev)
    inverse = torch.empty(n, dtype=torch.int32, device=dev)
    vfeat = torch.empty((m, feats.shape[1]), dtype=torch.float32, device=dev)
    _check(L.ssc_p2v_fill(_p(points), _p(batch_ids), _p(feats), n, feats.shape[1], int(batch_size), _i3(grid), unit3,
                          int(mode), m, _p(vox), _p(inverse), _p(vfeat), _p(scratch), scratch.numel(), _stream()))
    if ahead:
        return vox, inverse, vfeat, m_dev
    return vox, inverse, vfeat


def three_nn(n, m, unknown, known, dist2, idx):
    L = lib()
    sbytes = max(int(L.ssc_three_nn_scratch_bytes(int(m))), 256)
    scratch = torch.empty(sbytes, dtype=torch.uint8, device=unknown.device)
    _check(L.ssc_three_nn(int(n), int(m), _p(unknown, torch.float32), _p(known, torch.float32),
                          _p(dist2, torch.float32), _p(idx, torch.int32), _p(scratch), scratch.numel(), _stream()))


def three_interpolate_fp(c, m, n, points, idx, weight, out):
    _check(lib().ssc_three_interpolate_fwd(int(c), int(m), int(n), _p(points, torch.float32), _p(idx, torch.int32),
                                           _p(weight, torch.float32), _p(out, torch.float32), _stream()))


def three_interpolate_bp(c, n, m, grad_out, idx, weight, grad_points):
    """(SS_Conv_lib/src/voxelize/interpolate.h:23-25) writes grad_points [M, C] in place."""
    _check(lib().ssc_three_interpolate_bwd(int(c), int(n), int(m), _p(grad_out, torch.float32), _p(idx, torch.int32),
                                           _p(weight, torch.float32), _p(grad_points, torch.float32), _stream()))


# ================================================================ BatchNorm / activation
def bn_fold(running_mean, running_var, weight, bias, field_of_channel, scalar_of_channel, eps):
    c = field_of_channel.numel()
    scale = torch.empty(c, dtype=torch.float32, device=running_var.device)
    shift = torch.empty_like(scale)
    _check(lib().ssc_bn_fold(_p(running_mean), _p(running_var), _p(weight), _p(bias), _p(field_of_channel, torch.int32),
                             _p(scalar_of_channel, torch.int32), c, float(eps), _p(scale), _p(shift), _stream()))
    return scale, shift


def bn_gate_forward(x, scale, shift, gate_of_channel, c_out, c_gate_base, scalar_act, gate_act, scalar_bias,
                    gate_bias, storage=None):
    """storage 'fp16' / 'bf16': the result is written in that type (see set_feature_storage) when the
    shapes allow 16-byte rows; otherwise fp32."""
    x = x.contiguous()
    if (storage in _DTYPE_OF and int(c_out) % 8 == 0 and x.shape[1] % 4 == 0 and int(c_gate_base) % 4 == 0
            and x.shape[0] * int(c_out) // 4 < 2 ** 31):
        out = torch.empty((x.shape[0], int(c_out)), dtype=_DTYPE_OF[storage], device=x.device)
        _check(lib().ssc_bn_gate_fwd16(_p(x, torch.float32), x.shape[0], x.shape[1], _p(scale), _p(shift),
                                       _p(gate_of_channel), int(c_out), int(c_gate_base), int(scalar_act), int(gate_act),
                                       _p(scalar_bias), _p(gate_bias), _PREC_OF[storage], _p(out), _stream()))
        return out
    out = torch.empty((x.shape[0], int(c_out)), dtype=torch.float32, device=x.device)
    _check(lib().ssc_bn_gate_fwd(_p(x, torch.float32), x.shape[0], x.shape[1], _p(scale), _p(shift),
                                 _p(gate_of_channel), int(c_out), int(c_gate_base), int(scalar_act), int(gate_act),
                                 _p(scalar_bias), _p(gate_bias), _p(out), _stream()))
    return out


def bn_stats(x, field_of_channel, scalar_of_channel, n_field, n_scalar):
    x = x.contiguous()
    mean = torch.empty(max(n_scalar, 1), dtype=torch.float32, device=x.device)
    var = torch.empty(n_field + x.shape[1], dtype=torch.float32, device=x.device)
    nbytes = int(lib().ssc_bn_scratch_bytes(x.shape[0], x.shape[1]))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    _check(lib().ssc_bn_stats(_p(x, torch.float32), x.shape[0], x.shape[1], _p(field_of_channel, torch.int32),
                              _p(scalar_of_channel, torch.int32), int(n_field), int(n_scalar), _p(mean), _p(var),
                              _p(scratch), nbytes, _stream()))
    return mean[:n_scalar], var[:n_field]


def bn_backward(x, gy, field_of_channel, scalar_of_channel, n_field, n_scalar, mean, var, weight, eps, training):
    """(gx [n, c], d_weight [n_field], d_bias [n_scalar]) of y = (x - mean) * weight / sqrt(var + eps) + bias;
    training: mean / var are the batch statistics of x and the gradient flows through them."""
    x, gy = x.contiguous(), gy.contiguous()
    n, c = x.shape
    gx = torch.empty_like(x)
    d_w = torch.empty(n_field, dtype=torch.float32, device=x.device)
    d_b = torch.empty(max(n_scalar, 1), dtype=torch.float32, device=x.device)
    nbytes = int(lib().ssc_bn_scratch_bytes(n, c))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    mean_c = None if n_scalar == 0 else mean.contiguous()
    _check(lib().ssc_bn_bwd(_p(x, torch.float32), _p(gy, torch.float32), n, c, _p(field_of_channel, torch.int32),
                            _p(scalar_of_channel, torch.int32), int(n_field), int(n_scalar), _p(mean_c),
                            _p(var.contiguous()), _p(weight), float(eps), int(bool(training)), _p(gx), _p(d_w), _p(d_b),
                            _p(scratch), nbytes, _stream()))
    return gx, d_w, d_b[:n_scalar]


def gate_backward(x, gy, c_out, gate_of_channel, field_start, field_len, scalar_act, gate_act):
    """gx [n, c_total] of the gated activation (no biases) at input x, output gradient gy [n, c_out]."""
    x, gy = x.contiguous(), gy.contiguous()
    gx = torch.empty_like(x)
    _check(lib().ssc_gate_bwd(_p(x, torch.float32), _p(gy, torch.float32), x.shape[0], x.shape[1], int(c_out),
                              _p(gate_of_channel, torch.int32), _p(field_start), _p(field_len), int(scalar_act),
                              int(gate_act), _p(gx), _stream()))
    return gx


def scatter_add_rate(out, rows, steps, lanes_per_row=8, warps_per_sm=16):
    """Launches the library's reduction-only kernel (ssc_scatter_add_rate): 1.0 is added to
    out[rows[j], :] for steps * 32 * (warps of the grid) list positions.  Returns the bytes
    reduced; the caller times the launch.  out [n_rows, c] fp32 scratch with c % 32 == 0.
    lanes_per_row: 16-byte pieces per row and instruction (1, 2, 4, 8); warps_per_sm: issuing warps."""
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] % 32 == 0
    rows = rows.to(torch.int32).contiguous()
    nbytes = ctypes.c_ulonglong(0)
    _check(lib().ssc_scatter_add_rate(_p(out), int(out.shape[1]), _p(rows, torch.int32), int(rows.numel()), int(steps),
                                      int(lanes_per_row), int(warps_per_sm), ctypes.byref(nbytes), _stream()))
    return int(nbytes.value)
