/*
 * ssconv_b200 — C ABI of the B200 (sm_100a) sparse steerable convolution library.
 *
 * This header is the drop-in boundary for the native part of the reference project
 * (SS_Conv_lib/src, exported to Python as the pybind11 module `ss_conv._ext`,
 * SS_Conv_lib/src/ss_conv_ops_api.cpp:15-55).  Every entry point is `extern "C"`, takes plain
 * device pointers and sizes, launches on the CUDA stream passed as `stream`
 * (a cudaStream_t cast to void*; NULL = legacy default stream) and returns 0 on success or a
 * non-zero SSC_ERR_* code; ssc_last_error() then holds a human-readable message.  Nothing
 * here allocates device memory unless stated: results and scratch are caller-provided, so a
 * host language binding (ctypes, cgo, JNI ...) owns all allocation.  No entry point exits
 * the process or traps the GPU (the reference calls exit(-1) in
 * SS_Conv_lib/src/voxelize/interpolate_cuda_kernel.cu:71-75 and throws std::runtime_error
 * from SS_Conv_lib/src/utils/tensorview.h:70-101).
 *
 * Conventions shared by all entry points
 *   indices      int32 [N,4] rows (batch, x, y, z), row-major
 *   features     float32 [N,C] row-major
 *   K            kernel volume kx*ky*kz (<= 256, SS_Conv_lib/src/conv/indice_conv.h:44);
 *                kernel offset index kappa = (kx_i*ky + ky_i)*kz + kz_i
 *   nbr          int32 [K, n_out]: nbr[kappa*n_out + o] = input row feeding output row o at
 *                offset kappa, or -1.  This output-major "neighbour table" is the layout the
 *                CUDA kernels consume; the reference's indicePairs [K,2,N] (-1 padded) and
 *                indiceNum [K] are produced beside it for API compatibility.
 */
#ifndef SSCONV_B200_H_
#define SSCONV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSC_OK 0
#define SSC_ERR_INVALID 1   /* bad argument (shape, null pointer, unsupported size)          */
#define SSC_ERR_CUDA 2      /* a CUDA runtime call or launch failed                          */
#define SSC_ERR_SCRATCH 3   /* scratch buffer too small                                      */
#define SSC_ERR_DEVICE 4    /* a kernel reported a problem through its status word           */

/* Library identification.  No reference counterpart. */
int ssc_version(void);
/* Message of the last failing call on this host thread ("" if none).  Replaces the exception
 * text of TV_ASSERT_RT_ERR / TV_CHECK_CUDA_ERR (SS_Conv_lib/src/utils/tensorview.h:70-101). */
const char *ssc_last_error(void);
/* Number of CUDA kernels this library has launched in the calling process (memsets and copies
 * not counted).  No reference counterpart. */
unsigned long long ssc_kernel_launches(void);
/* 1 if the tcgen05 tensor-core kernels were compiled in (always for sm_100a builds). */
int ssc_has_tcgen05(void);

/* ------------------------------------------------------------------ rulebook generation
 * Replaces getIndicePair<3> (SS_Conv_lib/src/conv/indice_conv.h:21-131) and the kernels of
 * SS_Conv_lib/src/conv/indice_cuda_functor.cu:23-241.  Geometry follows getValidOutPos
 * (SS_Conv_lib/src/conv/geometry.h:18-80).  Output rows are numbered by ascending flat index
 * ((b*O0+x)*O1+y)*O2+z, the order the reference's GPU path produces
 * (indice_conv.h:120, indice_cuda_functor.cu:113-129).  Pairs inside one offset are listed by
 * ascending output row (the reference's order there is atomic-arbitrary).
 */

/* Bytes of scratch the rulebook entry points need for n_in active inputs, a batch of
 * `batch` samples, an input grid of in_shape and an output grid of out_shape (the same grid
 * twice for submanifold).  Input rows are found through a dense row map over the input grid when
 * that grid is at most 64 cells per active voxel (and 2^26 cells), else through a hash table;
 * SSC_RULEBOOK_TABLE=hash|dense overrides the choice. */
size_t ssc_rulebook_scratch_bytes(int n_in, int batch, const int in_shape[3], const int out_shape[3], int K);

/* Submanifold rulebook (stride 1, padding k/2 forced as in indice_conv.h:68-73; output rows
 * are the input rows, indice_conv.h:96).  Writes nbr [K,n_in]; pairs [K,2,n_in] and
 * indice_num [K] unless NULL.  status: device int32, set non-zero on a device-side problem
 * (coordinate out of range, hash overflow); may be NULL. */
int ssc_rulebook_subm(const int32_t *indices, int n_in, int batch, const int shape[3],
                      const int ksize[3], const int dilation[3], int32_t *nbr, int32_t *pairs,
                      int32_t *indice_num, int32_t *status, void *scratch, size_t scratch_bytes,
                      void *stream);

/* Submanifold rulebook for callers that must not allocate device memory (no counterpart in
 * the reference).  Who needs it: a plugin inside a host application that owns every byte of
 * device memory and lends none, a long-running service whose device pool is frozen after
 * start-up so that no request can fail or stall on an allocation, a component built without
 * any allocator.  Same results as ssc_rulebook_subm, but the hash table and the counters sit
 * in a fixed array inside the library (about 1.1 MB, held by every GPU that loads the library
 * until the process exits) instead of a caller buffer.  The entry point calls neither
 * cudaMalloc nor cudaFree nor any allocating library routine; inputs and outputs are still
 * the caller's.
 *   Limits   : n_in <= 65536 active voxels, kernel volume <= 256; larger requests are refused
 *              with SSC_ERR_INVALID and a message naming the limit.
 *   Set-up   : the first call on each device looks up the array's device address (once per
 *              device, with that device current).  Make that first call before any stream
 *              capture begins.
 *   Sharing  : all calls use the same array and it keeps what the last call left; each call
 *              clears what it needs cleared.  Two calls that overlap on one GPU (different
 *              streams or threads) race on it: run them one after the other. */
int ssc_rulebook_subm_static(const int32_t *indices, int n_in, int batch, const int shape[3],
                             const int ksize[3], const int dilation[3], int32_t *nbr,
                             int32_t *pairs, int32_t *indice_num, int32_t *status, void *stream);

/* The submanifold rulebook on rows whose count is still on the device: `indices` has n_cap rows of
 * which the first *n_in_dev are meaningful (the output of a layer that ran ahead of its row count,
 * see ssc_rulebook_conv_fill).  Writes the neighbour table [K, n_cap] for the meaningful rows only;
 * consumers pass the same device word as their n_out_dev.  No pair lists (they need the count on the
 * host).  Same geometry rules as ssc_rulebook_subm (SS_Conv_lib/src/conv/indice_conv.h:70-96). */
int ssc_rulebook_subm_ahead(const int32_t *indices, int n_cap, int batch, const int shape[3],
                            const int ksize[3], const int dilation[3], int32_t *nbr, int32_t *status,
                            void *scratch, size_t scratch_bytes, const int32_t *n_in_dev, void *stream);

/* Regular / strided (transpose = 0) or transposed (transpose = 1,
 * getValidOutPosTranspose geometry.h:82-138) rulebook, phase 1: build the input coordinate
 * hash, mark every reachable output cell and count them.  n_out_dev: device int32 that
 * receives the number of active outputs; the caller reads it back (one 4-byte copy, the
 * counterpart of the host sync inside torch::_unique, indice_conv.h:120) to size phase 2.
 * n_in_dev: NULL, or a device word with the exact number of input rows when n_in is only the
 * capacity of `indices` (the output of a layer whose own count has not been read back yet). */
int ssc_rulebook_conv_count(const int32_t *indices, int n_in, int batch, const int in_shape[3],
                            const int out_shape[3], const int ksize[3], const int stride[3],
                            const int padding[3], const int dilation[3], int transpose,
                            int32_t *n_out_dev, int32_t *status, void *scratch,
                            size_t scratch_bytes, const int32_t *n_in_dev, void *stream);

/* Phase 2 (same arguments and the SAME untouched scratch as phase 1): writes
 * out_indices [n_out,4], nbr [K,n_out], pairs [K,2,n_in] (may be NULL), indice_num [K].
 *
 * Running ahead of the count.  n_out_dev (may be NULL) is the device word phase 1 wrote.  When
 * it is given, n_out is only a CAPACITY chosen by the caller (>= the true count, <= the bound
 * min(n_in*K, batch*out cells)): it sizes the launches and is the row stride of nbr, the exact
 * count is read on the device, and table rows between the count and the capacity are -1.  A
 * caller can then queue phase 2 and the layer that consumes the table (ssc_conv_fwd and the
 * pools accept the same pair n_out / n_out_dev) without waiting for the 4-byte read-back of
 * phase 1, and check afterwards that the count did fit (if not, repeat with the exact count).
 * pairs must be NULL in that mode (indice_num is still produced).  No counterpart in the
 * reference. */
int ssc_rulebook_conv_fill(const int32_t *indices, int n_in, int batch, const int in_shape[3],
                           const int out_shape[3], const int ksize[3], const int stride[3],
                           const int padding[3], const int dilation[3], int transpose, int n_out,
                           int32_t *out_indices, int32_t *nbr, int32_t *pairs,
                           int32_t *indice_num, int32_t *status, void *scratch,
                           size_t scratch_bytes, const int32_t *n_out_dev, void *stream);

/* Neighbour table from a reference-format rulebook (indicePairs [K,2,n_cols], indiceNum [K]):
 * nbr[kappa][pairs[kappa][1-swap][i]] = pairs[kappa][swap][i].  swap = 1 is the "inverse"
 * convolution of indice_conv.h:301-311 (roles of the two pair rows exchanged). */
int ssc_pairs_to_nbr(const int32_t *pairs, const int32_t *indice_num, int K, int n_cols,
                     int n_out, int swap, int32_t *nbr, void *stream);

/* The reverse direction: reference-format pair lists (indicePairs [K,2,n_in], -1 padded, and
 * indiceNum [K], SS_Conv_lib/src/conv/indice_conv.h:49-53) from a neighbour table, pairs of an
 * offset in ascending output row.  Lets a caller build rulebooks without pair lists (the CUDA
 * kernels only need the table) and materialise them on demand. */
size_t ssc_pairs_from_nbr_scratch_bytes(int K, int n_out);
int ssc_pairs_from_nbr(const int32_t *nbr, int K, int n_out, int n_in, int32_t *pairs,
                       int32_t *indice_num, void *scratch, size_t scratch_bytes, void *stream);

/* --------------------------------------------------------- steerable kernel materialisation
 * Replaces SE3Kernel.combination (SS_Conv_lib/ss_conv/utils/kernel.py:267-299) followed by
 * permute(2,3,4,1,0) (SS_Conv_lib/ss_conv/convolution.py:56):
 *   filters[kappa][cin][cout] = sum_b weight[woff + (u*m_in+v)*nb + b] * basis[boff + ((b*d_out+a)*d_in+c)*K + kappa]
 * out_field/in_field map a channel to (block row/col, copy u/v, component a/c) packed as
 * int32 triples; block_table holds per (i,j) block {basis_offset or -1, weight_offset, nb,
 * m_in, d_out, d_in} as int32 sextuples, row-major over (i,j). */
int ssc_materialize(const float *weight, const float *basis, const int32_t *block_table,
                    int n_blocks_in, const int32_t *out_field, const int32_t *in_field, int c_out,
                    int c_in, int K, float *filters, void *stream);

/* Pack filters [K,Cin,Cout] fp32 into the tensor-core operand image used by ssc_conv_fwd
 * with precision SSC_PREC_TF32 (round-to-nearest TF32, K-major, 128-byte swizzled, padded) or
 * SSC_PREC_F16 (the same layout with fp16 elements, 64 input channels per 128-byte row).
 * ssc_conv_packed_bytes gives the size of `packed`.  TF32 layers whose input rows pad to 4, 8 or 16
 * channels (c_in = 1..8, 13..16) are packed with 8, 4 or 2 kernel offsets side by side in one
 * operand row; ssc_conv_fwd then needs its staging buffer (ssc_conv_scratch_bytes) whatever the
 * size of the layer, and the pair-list entry points do not take such layers. */
size_t ssc_conv_packed_bytes(int K, int c_in, int c_out, int precision);
int ssc_conv_pack_filters(const float *filters, int K, int c_in, int c_out, int precision,
                          void *packed, void *stream);

/* ------------------------------------------------------------ gather-GEMM-scatter (forward)
 * Replaces indiceConv<float> (SS_Conv_lib/src/conv/indice_conv.h:247-343) and the gather /
 * scatter kernels of SS_Conv_lib/src/conv/reordering_cuda_functor.cu:23-159:
 *   out[o,:] = sum_kappa features[nbr[kappa][o],:] * filters[kappa]   (fp32 accumulate)
 * as ONE launch, output-stationary (no scatter atomics, deterministic).
 * precision: SSC_PREC_FP32 = exact fp32 FMA on CUDA cores (filters = [K,Cin,Cout] fp32);
 *            SSC_PREC_TF32 = tcgen05 tensor cores, TF32 operands (filters = packed image);
 *            SSC_PREC_F16  = tcgen05 tensor cores, fp16 operands and fp32 accumulation (the
 *            reference's half-precision entry point indice_conv_half, SS_Conv_lib/src/ss_conv_ops.h:49-51): the same
 *            11-bit significand as TF32 within fp16's range (finite values beyond +-65504
 *            saturate, magnitudes below 6e-5 lose bits), half the gathered bytes and half the
 *            tensor-core instructions.  Needs `scratch` (the fp16 copy of the feature rows).
 *            SSC_PREC_BF16 = the same with bfloat16 operands (fp32's exponent range, 8 significant
 *            bits; max rel. error target 1e-2).  The reference has no bf16 entry point.
 * status: device int32 that receives a non-zero value if a bounded wait inside the kernel
 * ran out (may be NULL).
 * scratch: optional device buffer of ssc_conv_scratch_bytes() bytes, 16-byte aligned.  With it
 * the TF32 path of a large layer first writes a TF32-rounded copy of the feature rows there and
 * gathers from the copy (a row is gathered about K/2 times; rounding once instead of after every
 * gather feeds the tensor core the same operands, bit for bit); without it (NULL / too small)
 * the rows are rounded in shared memory after every gather.  The 16-bit precisions need it.
 * n_out_dev: NULL, or the device word holding the exact number of output rows when n_out is a
 * capacity (see ssc_rulebook_conv_fill); rows past the exact count are not written. */
#define SSC_PREC_FP32 0
#define SSC_PREC_TF32 1
#define SSC_PREC_F16 2
#define SSC_PREC_BF16 3
/* OR'ed into `precision` of ssc_conv_fwd / ssc_conv_fwd_ordered: `scratch` already holds the staged
 * copy of the feature rows, written by ssc_conv_stage (e.g. on another stream, next to the
 * rulebook kernels, which do not depend on the features); the call then skips its staging launch. */
#define SSC_CONV_PRESTAGED 0x100
int ssc_conv_stage(const float *features, int n_in, int c_in, int precision, void *scratch,
                   size_t scratch_bytes, void *stream);
size_t ssc_conv_scratch_bytes(int n_in, int c_in, int c_out, int precision);
int ssc_conv_fwd(const float *features, int n_in, int c_in, const void *filters, int K, int c_out,
                 const int32_t *nbr, int n_out, int precision, float *out, int32_t *status,
                 void *scratch, size_t scratch_bytes, const int32_t *n_out_dev, void *stream);

/* Pair-list form of the same convolution, for sparsely filled tables (wide submanifold layers):
 * per kernel offset the present (input row, output row) pairs are compacted into lists, every
 * 128 pairs form a dense tile [128, Cin] x filters[kappa] on the tensor cores, and the rows of the
 * product are added to their output rows - the reference's gather / GEMM / scatter-add per offset
 * (SS_Conv_lib/src/conv/indice_conv.h:290-338, reordering_cuda_functor.cu:161-273) as one persistent
 * launch with the filter matrix of an offset resident in shared memory.  The sums of an output row
 * arrive in no fixed order (fp32 reductions at L2): results repeat only up to rounding.
 *   ssc_conv_pairs_list_bytes : size of `lists` for a table [K, n_out] (256-byte aligned buffer)
 *   ssc_conv_pairs_supported  : 1 if the kernel covers (c_in, c_out, precision), else 0
 *   ssc_conv_pairs_build      : lists from the neighbour table (three small launches; reusable for
 *                               every layer that shares the table)
 *   ssc_conv_fwd_pairs        : staging (unless SSC_CONV_PRESTAGED) + clear + convolution;
 *                               precision SSC_PREC_TF32 / _F16 / _BF16, `filters` the packed image,
 *                               `scratch` the staging buffer of ssc_conv_scratch_bytes(). */
size_t ssc_conv_pairs_list_bytes(int K, int n_out);
int ssc_conv_pairs_supported(int c_in, int c_out, int precision);
int ssc_conv_pairs_build(const int32_t *nbr, int K, int n_out, void *lists, size_t list_bytes, void *stream);
int ssc_conv_fwd_pairs(const float *features, int n_in, int c_in, const void *filters, int K, int c_out,
                       void *lists, size_t list_bytes, int n_out, int precision, float *out,
                       int32_t *status, void *scratch, size_t scratch_bytes, void *stream);

/* ---------------------------------------------------------------------------- sparse pools
 * Replace indiceMaxPool / indiceAvgPool (SS_Conv_lib/src/pool/indice_maxpool.h:15-50,
 * SS_Conv_lib/src/pool/indice_avgpool.h:17-52) and their K-launch kernels.  Max: output starts
 * at zero (indice_maxpool.h:24) so the result is max(0, max_i x_i).  Avg: out = sum_i x_i /
 * summaryrf[o] accumulated in ascending offset order (indice_avgpool_cuda_functor.cu:43);
 * summaryrf NULL means "divide by K" (SS_Conv_lib/ss_conv/sp_ops/functional.py:171-176).
 * n_out_dev as in ssc_conv_fwd. */
int ssc_maxpool_fwd(const float *features, int c, const int32_t *nbr, int K, int n_out, float *out,
                    const int32_t *n_out_dev, void *stream);
int ssc_avgpool_fwd(const float *features, int c, const int32_t *nbr, int K, int n_out,
                    const int32_t *summaryrf, float *out, const int32_t *n_out_dev, void *stream);
/* Replaces indiceSummaryRF (SS_Conv_lib/src/pool/indiceSummaryRF.cu:21-63). */
int ssc_summary_rf(const int32_t *nbr, int K, int n_out, int32_t *rf, void *stream);

/* Replace global_avgpool_fp / global_maxpool_fp
 * (SS_Conv_lib/src/pool/global_avgpool_cuda_kernel.cu:16-42,
 *  SS_Conv_lib/src/pool/global_maxpool_cuda_kernel.cu:16-43): per-sample mean / max over the
 * row ranges offsets[s]..offsets[s+1]; out [B,C]; maxidx [B,C] (first arg-max row, -1 if empty). */
int ssc_global_avgpool_fwd(const float *feats, const int32_t *offsets, int n_samples, int c,
                           float *out, void *stream);
int ssc_global_maxpool_fwd(const float *feats, const int32_t *offsets, int n_samples, int c,
                           float *out, int32_t *maxidx, void *stream);
/* Row offsets [B+1] of a batch-sorted indices [N,4] tensor; replaces the B host syncs of
 * SparseTensor.get_offsets (SS_Conv_lib/ss_conv/sp_ops/tensor.py:59-65).  n_dev: NULL, or the
 * device word with the exact row count when n is a capacity. */
int ssc_batch_offsets(const int32_t *indices, int n, int batch, int32_t *offsets, const int32_t *n_dev,
                      void *stream);

/* ------------------------------------------------------------------------------- backward
 * Replace indiceConvBackward<float> (SS_Conv_lib/src/conv/indice_conv.h:344-426),
 * indiceMaxPoolBackward / indiceAvgPoolBackward (SS_Conv_lib/src/pool/indice_maxpool.h:94-127,
 * SS_Conv_lib/src/pool/indice_avgpool.h:54-90) and global_avgpool_bp / global_maxpool_bp
 * (SS_Conv_lib/src/pool/global_avgpool_cuda_kernel.cu:45-65,
 *  SS_Conv_lib/src/pool/global_maxpool_cuda_kernel.cu:46-61).
 *
 * ssc_nbr_transpose: input-major table nbr_in[kappa][i] = o from the output-major nbr[kappa][o] = i
 * (each (offset, input row) has at most one output row).  With it
 *   input gradient  = ssc_conv_fwd(out_grad, filters transposed to [K,Cout,Cin], nbr_in, n_in)
 * (the reference's gather -> mm(filters^T) -> scatter-add loop, :412-424), and the pool
 * gradients below need no atomics.
 * ssc_conv_wgrad: d_filters[kappa] = sum_o features[nbr[kappa][o]]^T . out_grad[o]  ([K,Cin,Cout],
 * the reference's mm(inputBuffer^T, outputBuffer), :411), bitwise repeatable; precision
 * SSC_PREC_FP32 = exact fp32 FMA, SSC_PREC_TF32 = tcgen05 with TF32 operands (both operands are
 * transposed into K-major shared-memory tiles on the fly; up to 256 input channels, else fp32).
 * ssc_maxpool_bwd: d_in[i,c] = sum over outputs o of i with out[o,c] == in[i,c] of out_grad[o,c]
 * (indice_maxpool_cpp_functor.cpp:78-84); ssc_avgpool_bwd: d_in[i] = sum_o out_grad[o] / rf[o]
 * (rf NULL: / K; indice_avgpool_cuda_functor.cu:195-205), both in ascending offset order. */
int ssc_nbr_transpose(const int32_t *nbr, int K, int n_out, int n_in, int32_t *nbr_in, void *stream);

/* Row order for ssc_conv_fwd_ordered.  order[0..n_rows) is a permutation of the rows of the table
 * nbr[K][n_rows] that puts rows with the same first used kernel offset next to each other
 * (ascending row number inside a group; rows without any neighbour last).  The convolution
 * kernel works on tiles of 128 rows of that order and skips the offsets no row of a tile uses:
 * on the input-major table of a strided convolution (the reference's input-gradient loop,
 * SS_Conv_lib/src/conv/indice_conv.h:412-424, and the forward pass of a transposed convolution)
 * a row uses only the offsets of its parity class, so grouped tiles skip 7/8 of the steps of a
 * 3^3 stride-2 kernel.  The result of the convolution does not depend on the order, bit for bit.
 * Kernel volumes up to 343. */
size_t ssc_nbr_row_order_scratch_bytes(int K, int n_rows);
int ssc_nbr_row_order(const int32_t *nbr, int K, int n_rows, int32_t *order, void *scratch,
                      size_t scratch_bytes, void *stream);
/* The same for the output-major table of a forward convolution with a small kernel (ksize[0] +
 * ksize[1] + ksize[2] <= 9, e.g. 3^3): rows are grouped by WHICH PLANES of the kernel hold one of
 * their neighbours (one bit per kx, ky and kz; offsets numbered (kx * ksize[1] + ky) * ksize[2] + kz
 * as in SS_Conv_lib/src/conv/geometry.h:56-65), groups with more possible offsets first, ascending
 * row number inside a group.  On surface-like inputs 128 consecutive output rows together use
 * every offset although each row uses a quarter of them; tiles of this order skip about 45 % of
 * the (tile, offset) steps of the reference's per-offset loop (indice_conv.h:290-338).
 * nbr_in_order (may be NULL): receives the table with its columns moved into that order (column j
 * = the column of row order[j]); pass it with SSC_CONV_TABLE_IN_ORDER so that the kernel reads
 * the table coalesced.  n_rows_dev (may be NULL): device word with the number of live rows when
 * n_rows is a capacity; the live rows then come first in the order.  No bit of the convolution's
 * result depends on the order. */
size_t ssc_nbr_row_order_planes_scratch_bytes(const int ksize[3], int n_rows);
int ssc_nbr_row_order_planes(const int32_t *nbr, const int ksize[3], int n_rows, int32_t *order,
                             int32_t *nbr_in_order, void *scratch, size_t scratch_bytes,
                             const int32_t *n_rows_dev, void *stream);
/* OR'ed into `precision` of ssc_conv_fwd_ordered: `nbr` is the table in the order of `row_order`
 * (nbr_in_order above), i.e. column j belongs to output row row_order[j]. */
#define SSC_CONV_TABLE_IN_ORDER 0x200
int ssc_conv_fwd_ordered(const float *features, int n_in, int c_in, const void *filters, int K, int c_out,
                         const int32_t *nbr, int n_out, int precision, float *out, int32_t *status,
                         void *scratch, size_t scratch_bytes, const int32_t *n_out_dev,
                         const int32_t *row_order, void *stream);
size_t ssc_conv_wgrad_scratch_bytes(int K, int c_in, int c_out, int n_out);
int ssc_conv_wgrad(const float *features, int c_in, const float *out_grad, int c_out, const int32_t *nbr,
                   int K, int n_out, int precision, float *d_filters, int32_t *status, void *scratch,
                   size_t scratch_bytes, void *stream);
int ssc_maxpool_bwd(const float *features, const float *out_features, const float *out_grad, int c,
                    const int32_t *nbr_in, int K, int n_in, float *d_in, void *stream);
int ssc_avgpool_bwd(const float *out_grad, int c, const int32_t *nbr_in, int K, int n_in,
                    const int32_t *summaryrf, float *d_in, void *stream);
/* d_feats [n_rows, C] is written completely (rows outside every sample range get zero). */
int ssc_global_avgpool_bwd(const float *d_out, const int32_t *offsets, int n_samples, int c, int n_rows,
                           float *d_feats, void *stream);
int ssc_global_maxpool_bwd(const float *d_out, const int32_t *maxidx, int n_samples, int c, int n_rows,
                           float *d_feats, void *stream);
/* Replace voxelize_bp (SS_Conv_lib/src/voxelize/voxelize_cuda_kernel.h:44-62: every point listed in
 * a voxel's rule row receives the voxel's gradient, divided by the count in mean mode 4) and
 * three_interpolate_grad (SS_Conv_lib/src/voxelize/interpolate_cuda_kernel.cu:123-165).  Both write
 * their whole output (zero where nothing arrives); the interpolation gradient uses float atomics
 * like the reference, so its low-order bits depend on the order of arrival. */
int ssc_voxelize_bwd(const float *d_out, const int32_t *rules, int mode, int n_voxel, int max_active, int c,
                     int n_point, float *d_feats, void *stream);
int ssc_three_interpolate_bwd(int c, int n, int m, const float *grad_out, const int32_t *idx,
                              const float *weight, float *grad_points, void *stream);

/* ---------------------------------------------------------------------------- voxelization
 * ssc_voxel2point_map replaces voxel2point_fp (SS_Conv_lib/src/voxelize/voxel2point_cuda_kernel.cu:16-42):
 * maps [M, max_active+1] pre-initialised by the caller as in
 * SS_Conv_lib/ss_conv/sp_ops/functional.py:344-351; modes 3/4 list point ids in ascending
 * order (the reference's order there is atomic-arbitrary). */
int ssc_voxel2point_map(const int32_t *inverse, const int32_t *ids, int32_t *maps, int n_point,
                        int n_voxel, int max_active, int mode, void *stream);
/* Replaces voxelize_fp (SS_Conv_lib/src/voxelize/voxelize_cuda_kernel.h:18-40). */
int ssc_voxelize_fwd(const float *feats, float *out, const int32_t *maps, int mode, int n_voxel,
                     int max_active, int c, void *stream);

/* Fused Point2Voxel core, replacing torch.unique + voxel2point_map + voxelize_fp
 * (SS_Conv_lib/ss_conv/sp_ops/voxelize.py:85-96).  Phase 1 bins batch-sorted in-range points
 * into voxels ((p + half)/unit truncated), marks occupied cells and counts them
 * (n_voxel_dev, max_count_dev: device int32).  Phase 2 writes voxel_indices [M,4] in
 * ascending (b,x,y,z) order, inverse [N], and the voxel features (mode 1 first / 2 last /
 * 3 sum / 4 mean over points in ascending point id). */
size_t ssc_p2v_scratch_bytes(int n_point, int batch, const int grid[3]);
/* Feature steering (Feature_Steering_Module._transform_points / _transform_feats,
 * Common_utils/ss_conv_modules.py:198-224): new_points[p] = (points[p] - trans[b]) . rot[b]
 * (divided by scale[b] + 1e-8 when scale is given), new_feats[p, block] = feats[p, block] . D_b for
 * every irrep block, b = ids[p].  rot [B,3,3], trans [B,3], scale [B] or NULL; dmats [B, d_stride]
 * holds the sample's D^l matrices (row-major, one per order l) back to back; chan [C,3] gives per
 * channel (first channel of its block, block width 2l+1, offset of D^l inside a dmats row). */
int ssc_steer_fwd(const float *points, const float *feats, const int32_t *ids, const float *rot,
                  const float *trans, const float *scale, const float *dmats, int d_stride,
                  const int32_t *chan, int n, int c, int n_sample, float *new_points, float *new_feats,
                  void *stream);

/* One pass over a point batch telling the host which path Point2Voxel can take
 * (SS_Conv_lib/ss_conv/sp_ops/voxelize.py:38-84 answers the same questions with two torch.unique
 * calls, a sort and three read-backs): stats_dev[0] = points outside the grid, [1] = places where
 * batch_ids decreases, [2] = places where it changes (distinct samples - 1 when sorted), [3] = the
 * last batch id. */
int ssc_p2v_stats(const float *points, const int32_t *batch_ids, int n_point, const int grid[3],
                  const float unit[3], int32_t *stats_dev, void *stream);
int ssc_p2v_count(const float *points, const int32_t *batch_ids, int n_point, int batch,
                  const int grid[3], const float unit[3], int32_t *n_voxel_dev, int32_t *status,
                  void *scratch, size_t scratch_bytes, void *stream);
int ssc_p2v_fill(const float *points, const int32_t *batch_ids, const float *feats, int n_point,
                 int c, int batch, const int grid[3], const float unit[3], int mode, int n_voxel,
                 int32_t *voxel_indices, int32_t *inverse, float *voxel_feats, void *scratch,
                 size_t scratch_bytes, void *stream);

/* three_nn / three_interpolate_fp replacements
 * (SS_Conv_lib/src/voxelize/interpolate_cuda_kernel.cu:8-55, 79-101): unknown [N,4] and
 * known [M,4] are (batch,x,y,z) float rows; dist2 [N,3] squared distances, idx [N,3].
 * Same neighbours and tie order as the reference's exhaustive scan.  scratch (device,
 * ssc_three_nn_scratch_bytes(m) bytes) holds the batch-id range of each 1024-row tile of
 * `known`, which lets a block skip tiles of other samples. */
size_t ssc_three_nn_scratch_bytes(int m);
int ssc_three_nn(int n, int m, const float *unknown, const float *known, float *dist2,
                 int32_t *idx, void *scratch, size_t scratch_bytes, void *stream);
int ssc_three_interpolate_fwd(int c, int m, int n, const float *points, const int32_t *idx,
                              const float *weight, float *out, void *stream);

/* ------------------------------------------------ irrep-wise BatchNorm + gated activation
 * Replace the torch op chains of BatchNorm.forward (SS_Conv_lib/ss_conv/batchnorm.py:49-136)
 * and Activation._gate (SS_Conv_lib/ss_conv/activation.py:55-100).
 * ssc_bn_fold: per-channel scale/shift of eval-mode BN from the running statistics:
 *   scale[ch] = weight[f]/sqrt(running_var[f]+eps); shift[ch] = bias[s]-running_mean[s]*scale
 *   for scalar fields, 0 otherwise.  field_of_channel / scalar_of_channel: int32 [C]
 *   (scalar_of_channel = -1 for l>0).  weight/bias may be NULL (affine=False). */
int ssc_bn_fold(const float *running_mean, const float *running_var, const float *weight,
                const float *bias, const int32_t *field_of_channel,
                const int32_t *scalar_of_channel, int c, float eps, float *scale, float *shift,
                void *stream);
/* y = act(x*scale+shift): x [N, c_in_total]; out [N, c_out].  scale/shift NULL = no affine.
 * gate_of_channel int32 [c_out]: -2 = copy, -1 = scalar activation (scalar_act, bias
 * scalar_bias[ch] if non-NULL), g>=0 = multiply by gate_act(x[:, c_gate_base+g] (+gate_bias[g])).
 * NULL gate_of_channel = affine only (c_out == c_in_total).  act codes: 0 identity, 1 relu,
 * 2 sigmoid. */
int ssc_bn_gate_fwd(const float *x, int n, int c_in_total, const float *scale, const float *shift,
                    const int32_t *gate_of_channel, int c_out, int c_gate_base, int scalar_act,
                    int gate_act, const float *scalar_bias, const float *gate_bias, float *out,
                    void *stream);
/* The same pass with a 16-bit result (precision SSC_PREC_F16 or SSC_PREC_BF16): out16 [n, c_out]
 * fp16 / bf16, c_out a multiple of 8.  The rows are then already the operand image of the next
 * convolution (ssc_conv_fwd with SSC_CONV_PRESTAGED and scratch = out16): no staging pass, half the
 * bytes between the layers.  No counterpart in the reference (its layers exchange fp32). */
int ssc_bn_gate_fwd16(const float *x, int n, int c_in_total, const float *scale, const float *shift,
                      const int32_t *gate_of_channel, int c_out, int c_gate_base, int scalar_act,
                      int gate_act, const float *scalar_bias, const float *gate_bias, int precision,
                      void *out16, void *stream);
/* Training-mode statistics (SS_Conv_lib/ss_conv/batchnorm.py:73-99): mean [n_scalar] of scalar
 * fields and var = batch mean of the squared field norm (about the batch mean for scalars); `var`
 * must have room for n_field + c floats: the first n_field are the result, the tail is scratch.
 * Partial sums are added in a fixed order (bitwise repeatable).  scratch: ssc_bn_scratch_bytes(n, c). */
size_t ssc_bn_scratch_bytes(int n, int c);
int ssc_bn_stats(const float *x, int n, int c, const int32_t *field_of_channel,
                 const int32_t *scalar_of_channel, int n_field, int n_scalar, float *mean,
                 float *var, void *scratch, size_t scratch_bytes, void *stream);

/* Backward of the batch norm (what autograd derives from SS_Conv_lib/ss_conv/batchnorm.py:49-136):
 * y = (x - mean) * w / sqrt(var + eps) (+ bias for scalars).  training != 0: mean / var are the batch
 * statistics of x (gradients flow through them); else they are constants (running buffers).
 * gx [n, c]; d_weight [n_field] and d_bias [n_scalar] may be NULL.  weight NULL = no affine part. */
int ssc_bn_bwd(const float *x, const float *gy, int n, int c, const int32_t *field_of_channel,
               const int32_t *scalar_of_channel, int n_field, int n_scalar, const float *mean,
               const float *var, const float *weight, float eps, int training, float *gx,
               float *d_weight, float *d_bias, void *scratch, size_t scratch_bytes, void *stream);

/* Backward of the gated activation without biases (SS_Conv_lib/ss_conv/activation.py:55-100):
 * x [n, c_total] = [c_out Rs channels | gate scalars] is the layer's input, gy [n, c_out] the gradient
 * of its output, gx [n, c_total].  gate_of_channel as in ssc_bn_gate_fwd; field_start / field_len
 * [c_total - c_out]: the channel range that gate j multiplies. */
int ssc_gate_bwd(const float *x, const float *gy, int n, int c_total, int c_out,
                 const int32_t *gate_of_channel, const int32_t *field_start, const int32_t *field_len,
                 int scalar_act, int gate_act, float *gx, void *stream);

/* Measurement support, no counterpart in the reference: issues nothing but fp32 scatter-add
 * reductions (red.global.add.v4.f32) of 1.0 into out[rows[j], :] for steps * 32 * (warps of the grid)
 * list positions j, wrapping round the list of n_idx row numbers.  lanes_per_row (1, 2, 4, 8) =
 * contiguous 16-byte pieces per row and instruction, warps_per_sm (1..16) = issuing warps; (8, 16)
 * measures the device's scatter-add rate, the ceiling of the pair-list convolution's reduction
 * traffic (4 P Cout bytes).  out [n_rows, row_floats] is caller scratch, row_floats a multiple of 32.
 * *bytes receives the bytes reduced; the caller times the launch. */
int ssc_scatter_add_rate(float *out, int row_floats, const int32_t *rows, int n_idx, int steps,
                         int lanes_per_row, int warps_per_sm, unsigned long long *bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SSCONV_B200_H_ */
