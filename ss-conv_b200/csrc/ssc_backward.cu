// Backward kernels of the sparse convolution and the pools.
//
// Input gradient of a convolution = the forward gather-GEMM with the roles exchanged: rows of
// outGrad gathered through the INPUT-major table nbr_in[kappa][i] = o (ssc_nbr_transpose) and
// multiplied by the transposed filters, so ssc_conv_fwd (tcgen05 or exact fp32) serves it and
// every input row is written once, without atomics.
//
// Filter gradient: dW[kappa] = sum over output rows o of x[nbr[kappa][o]]^T . dY[o].  The rows
// are split into ranges; a CTA owns one (offset, range, 64x64 tile of dW), streams 32-row
// chunks of both operands through shared memory (chunks without any neighbour are skipped) and
// writes its partial tile; a second kernel adds the partials in a fixed order, so the result is
// bitwise repeatable.
//
// Pool gradients walk the input-major table: one thread per (input row, 4 channels) adds its
// outputs' gradients in ascending offset order (the order of the reference's loop), no atomics.
#include "ssc_common.cuh"

namespace ssc {

__global__ void nbr_transpose_kernel(const int32_t *__restrict__ nbr, int n_out, int n_in, int32_t *__restrict__ nbr_in) {
  int o = blockIdx.x * blockDim.x + threadIdx.x;
  int kappa = blockIdx.y;
  if (o >= n_out) return;
  int i = __ldg(nbr + (size_t)kappa * n_out + o);
  if (i >= 0 && i < n_in) nbr_in[(size_t)kappa * n_in + i] = o;
}

constexpr int WG_T = 64;      // tile edge of dW handled by one CTA
constexpr int WG_ROWS = 32;   // output rows per shared-memory chunk

// grid (splits, K, tiles_ci * tiles_co), block 256 (16 x 16 threads, 4 x 4 results each).
__global__ void __launch_bounds__(256)
conv_wgrad_partial_kernel(const float *__restrict__ features, int c_in, const float *__restrict__ out_grad, int c_out,
                          const int32_t *__restrict__ nbr, int n_out, int rows_per_split, int tiles_co,
                          float *__restrict__ partial) {
  __shared__ float As[WG_ROWS][WG_T + 4];
  __shared__ float Bs[WG_ROWS][WG_T + 4];
  __shared__ int rows[WG_ROWS];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int split = blockIdx.x, kappa = blockIdx.y;
  const int ci0 = (blockIdx.z / tiles_co) * WG_T, co0 = (blockIdx.z % tiles_co) * WG_T;
  const int r_begin = split * rows_per_split;
  const int r_end = min(n_out, r_begin + rows_per_split);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int r0 = r_begin; r0 < r_end; r0 += WG_ROWS) {
    int src = -1;
    if (tid < WG_ROWS && r0 + tid < r_end) src = __ldg(nbr + (size_t)kappa * n_out + r0 + tid);
    const int any = __syncthreads_or(src >= 0);  // also: the previous chunk has been consumed
    if (!any) continue;
    if (tid < WG_ROWS) rows[tid] = src;
    __syncthreads();
    for (int e = tid; e < WG_ROWS * WG_T; e += 256) {
      const int r = e / WG_T, c = e - r * WG_T;
      const int s = rows[r];
      As[r][c] = (s >= 0 && ci0 + c < c_in) ? __ldg(features + (size_t)s * c_in + ci0 + c) : 0.f;
      Bs[r][c] = (s >= 0 && co0 + c < c_out) ? __ldg(out_grad + (size_t)(r0 + r) * c_out + co0 + c) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int r = 0; r < WG_ROWS; ++r) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[r][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[r][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
  float *dst = partial + ((size_t)split * gridDim.y + kappa) * (size_t)c_in * c_out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ci = ci0 + ty * 4 + i;
    if (ci >= c_in) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int co = co0 + tx * 4 + j;
      if (co < c_out) dst[(size_t)ci * c_out + co] = acc[i][j];
    }
  }
}

__global__ void wgrad_reduce_kernel(const float *__restrict__ partial, int splits, long long elems, float *__restrict__ out) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= elems) return;
  float s = 0.f;
  for (int p = 0; p < splits; ++p) s += partial[(size_t)p * elems + e];
  out[e] = s;
}

// MODE 0: max pool (gradient goes to every input equal to the pooled value), 1: avg pool.
template <int MODE>
__global__ void pool_bwd_kernel(const float *__restrict__ features, const float *__restrict__ out_features,
                                const float *__restrict__ out_grad, int c, const int32_t *__restrict__ nbr_in, int K,
                                int n_in, const int32_t *__restrict__ summaryrf, float *__restrict__ d_in) {
  const int cg = (c + 3) >> 2;
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n_in * cg) return;
  const int i = (int)(t / cg);
  const int c0 = (int)(t - (long long)i * cg) * 4;
  float x[4] = {0.f, 0.f, 0.f, 0.f}, acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (MODE == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (c0 + q < c) x[q] = __ldg(features + (size_t)i * c + c0 + q);
  }
  for (int kappa = 0; kappa < K; ++kappa) {
    const int o = __ldg(nbr_in + (size_t)kappa * n_in + i);
    if (o < 0) continue;
    float div = 1.f;
    if (MODE == 1) div = summaryrf ? (float)__ldg(summaryrf + o) : (float)K;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (c0 + q >= c) continue;
      const float g = __ldg(out_grad + (size_t)o * c + c0 + q);
      if (MODE == 0) {
        if (__ldg(out_features + (size_t)o * c + c0 + q) == x[q]) acc[q] += g;
      } else {
        acc[q] += g / div;
      }
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q)
    if (c0 + q < c) d_in[(size_t)i * c + c0 + q] = acc[q];
}

// grid (samples, channel groups of 32), block (32, 8)
__global__ void global_avgpool_bwd_kernel(const float *__restrict__ d_out, const int32_t *__restrict__ offsets, int c,
                                          float *__restrict__ d_feats) {
  const int s = blockIdx.x, ch = blockIdx.y * 32 + threadIdx.x;
  const int start = offsets[s], end = offsets[s + 1];
  if (ch >= c || end <= start) return;
  const float g = d_out[(size_t)s * c + ch] / (float)(end - start);
  for (int r = start + threadIdx.y; r < end; r += 8) d_feats[(size_t)r * c + ch] = g;
}

__global__ void global_maxpool_bwd_kernel(const float *__restrict__ d_out, const int32_t *__restrict__ maxidx, long long total,
                                          int c, long long n_rows, float *__restrict__ d_feats) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int row = maxidx[e];
  if (row >= 0 && row < n_rows) d_feats[(size_t)row * c + (e % c)] = d_out[e];  // one writer per (row, channel) of a sample
}

// One thread per (voxel, channel): hands the voxel's gradient to the points listed in its rule
// row [count, point ids...].  A point is listed by one voxel only, so plain stores suffice.
__global__ void voxelize_bwd_kernel(const float *__restrict__ d_out, const int32_t *__restrict__ rules, int n_voxel,
                                    int max_active, int c, int average, float *__restrict__ d_feats) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n_voxel * c) return;
  const int v = (int)(t / c), ch = (int)(t - (long long)v * c);
  const int32_t *r = rules + (size_t)v * (max_active + 1);
  int n_act = r[0];
  if (n_act > max_active) n_act = max_active;
  const float g = d_out[t] * ((average && n_act > 0) ? 1.f / (float)n_act : 1.f);
  for (int i = 1; i <= n_act; ++i) d_feats[(size_t)r[i] * c + ch] = g;
}

// One thread per (point, channel): adds weight * gradient to each of the point's three voxels.
__global__ void three_interpolate_bwd_kernel(int c, int n, const float *__restrict__ grad_out,
                                             const int32_t *__restrict__ idx, const float *__restrict__ weight,
                                             float *__restrict__ grad_points) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n * c) return;
  const int p = (int)(t / c), ch = (int)(t - (long long)p * c);
  const float g = grad_out[t];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int v = idx[p * 3 + j];
    if (v >= 0) atomicAdd(grad_points + (size_t)v * c + ch, g * weight[p * 3 + j]);
  }
}

}  // namespace ssc

using namespace ssc;

extern "C" int ssc_voxelize_bwd(const float *d_out, const int32_t *rules, int mode, int n_voxel, int max_active, int c,
                                int n_point, float *d_feats, void *stream) {
  SSC_REQUIRE(n_voxel >= 0 && max_active >= 0 && c > 0 && n_point >= 0, "voxelize_bwd: bad sizes");
  cudaStream_t st = as_stream(stream);
  if (n_point > 0) {
    SSC_REQUIRE(d_feats, "voxelize_bwd: null pointer");
    cudaMemsetAsync(d_feats, 0, (size_t)n_point * c * 4, st);
  }
  if (n_voxel == 0 || n_point == 0) return SSC_OK;
  SSC_REQUIRE(d_out && rules, "voxelize_bwd: null pointer");
  long long total = (long long)n_voxel * c;
  { voxelize_bwd_kernel<<<ceil_div(total, 256), 256, 0, st>>>(d_out, rules, n_voxel, max_active, c, mode == 4, d_feats); note_launches(1); }
  SSC_CHECK_LAUNCH("voxelize_bwd");
  return SSC_OK;
}

extern "C" int ssc_three_interpolate_bwd(int c, int n, int m, const float *grad_out, const int32_t *idx,
                                         const float *weight, float *grad_points, void *stream) {
  SSC_REQUIRE(c > 0 && n >= 0 && m >= 0, "three_interpolate_bwd: bad sizes");
  cudaStream_t st = as_stream(stream);
  if (m > 0) {
    SSC_REQUIRE(grad_points, "three_interpolate_bwd: null pointer");
    cudaMemsetAsync(grad_points, 0, (size_t)m * c * 4, st);
  }
  if (n == 0 || m == 0) return SSC_OK;
  SSC_REQUIRE(grad_out && idx && weight, "three_interpolate_bwd: null pointer");
  long long total = (long long)n * c;
  { three_interpolate_bwd_kernel<<<ceil_div(total, 256), 256, 0, st>>>(c, n, grad_out, idx, weight, grad_points); note_launches(1); }
  SSC_CHECK_LAUNCH("three_interpolate_bwd");
  return SSC_OK;
}

extern "C" int ssc_nbr_transpose(const int32_t *nbr, int K, int n_out, int n_in, int32_t *nbr_in, void *stream) {
  SSC_REQUIRE(K >= 1 && n_out >= 0 && n_in >= 0, "nbr_transpose: bad sizes");
  if (n_in == 0) return SSC_OK;
  SSC_REQUIRE(nbr_in && (n_out == 0 || nbr), "nbr_transpose: null pointer");
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(nbr_in, 0xFF, (size_t)K * n_in * 4, st);
  if (n_out > 0) {
    dim3 grid(ceil_div(n_out, 256), K);
    { nbr_transpose_kernel<<<grid, 256, 0, st>>>(nbr, n_out, n_in, nbr_in); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("nbr_transpose");
  return SSC_OK;
}

static int wgrad_splits(int K, int c_in, int c_out, int n_out) {
  const int tiles = ceil_div(c_in, WG_T) * ceil_div(c_out, WG_T);
  int splits = ceil_div(4 * 148, (long long)K * tiles);  // about four CTAs per SM in flight
  const int max_splits = ceil_div(n_out > 0 ? n_out : 1, 4 * WG_ROWS);
  if (splits > max_splits) splits = max_splits;
  if (splits > 256) splits = 256;
  if (splits < 1) splits = 1;
  return splits;
}

namespace ssc {
int conv_wgrad_tc(const float *features, int c_in, const float *out_grad, int c_out, const int32_t *nbr, int K, int n_out,
                  int max_splits, int *splits_used, float *partial, void *lists, int32_t *status, cudaStream_t st);
size_t conv_wgrad_tc_list_bytes(int K, int n_out);
}

// [partial tiles of the row ranges][pair lists of the tensor-core kernel]
static size_t wgrad_partial_bytes(int K, int c_in, int c_out, int n_out) {
  const size_t b = (size_t)wgrad_splits(K, c_in, c_out, n_out) * K * c_in * c_out * sizeof(float);
  return (b + 255) & ~(size_t)255;
}

extern "C" size_t ssc_conv_wgrad_scratch_bytes(int K, int c_in, int c_out, int n_out) {
  if (K < 1 || c_in < 1 || c_out < 1 || n_out < 0) return 0;
  return wgrad_partial_bytes(K, c_in, c_out, n_out) + conv_wgrad_tc_list_bytes(K, n_out);
}

extern "C" int ssc_conv_wgrad(const float *features, int c_in, const float *out_grad, int c_out, const int32_t *nbr, int K,
                              int n_out, int precision, float *d_filters, int32_t *status, void *scratch,
                              size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(K >= 1 && c_in >= 1 && c_out >= 1 && n_out >= 0 && d_filters, "conv_wgrad: bad arguments");
  cudaStream_t st = as_stream(stream);
  const long long elems = (long long)K * c_in * c_out;
  if (n_out == 0) {
    cudaMemsetAsync(d_filters, 0, (size_t)elems * 4, st);
    return SSC_OK;
  }
  SSC_REQUIRE(features && out_grad && nbr, "conv_wgrad: null pointer");
  const int splits = wgrad_splits(K, c_in, c_out, n_out);
  const size_t need = ssc_conv_wgrad_scratch_bytes(K, c_in, c_out, n_out);
  if (scratch == nullptr || scratch_bytes < need)
    return fail(SSC_ERR_SCRATCH, "conv_wgrad: scratch %zu < %zu bytes", scratch_bytes, need);
  int rows_per_split = ceil_div(n_out, splits);
  rows_per_split = ceil_div(rows_per_split, WG_ROWS) * WG_ROWS;
  int rc = -1, used = splits;
  if (precision == SSC_PREC_TF32)  // tensor cores where the shape allows, else the exact kernel below
    rc = conv_wgrad_tc(features, c_in, out_grad, c_out, nbr, K, n_out, splits, &used, (float *)scratch,
                       (uint8_t *)scratch + wgrad_partial_bytes(K, c_in, c_out, n_out), status, st);
  if (rc > 0) return rc;
  if (rc < 0) {
    const int tiles_co = ceil_div(c_out, WG_T);
    dim3 grid(splits, K, ceil_div(c_in, WG_T) * tiles_co);
    { conv_wgrad_partial_kernel<<<grid, 256, 0, st>>>(features, c_in, out_grad, c_out, nbr, n_out, rows_per_split, tiles_co,
                                                     (float *)scratch); note_launches(1); }
    SSC_CHECK_LAUNCH("conv_wgrad_partial");
    used = splits;
  }
  { wgrad_reduce_kernel<<<ceil_div(elems, 256), 256, 0, st>>>((const float *)scratch, used, elems, d_filters); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_wgrad_reduce");
  return SSC_OK;
}

template <int MODE>
static int launch_pool_bwd(const float *features, const float *out_features, const float *out_grad, int c,
                           const int32_t *nbr_in, int K, int n_in, const int32_t *rf, float *d_in, void *stream,
                           const char *name) {
  SSC_REQUIRE(c > 0 && K > 0 && n_in >= 0, "%s: bad sizes", name);
  if (n_in == 0) return SSC_OK;
  SSC_REQUIRE(out_grad && nbr_in && d_in && (MODE == 1 || (features && out_features)), "%s: null pointer", name);
  long long threads = (long long)n_in * ((c + 3) / 4);
  { pool_bwd_kernel<MODE><<<ceil_div(threads, 256), 256, 0, as_stream(stream)>>>(features, out_features, out_grad, c, nbr_in,
                                                                              K, n_in, rf, d_in); note_launches(1); }
  SSC_CHECK_LAUNCH(name);
  return SSC_OK;
}

extern "C" int ssc_maxpool_bwd(const float *features, const float *out_features, const float *out_grad, int c,
                               const int32_t *nbr_in, int K, int n_in, float *d_in, void *stream) {
  return launch_pool_bwd<0>(features, out_features, out_grad, c, nbr_in, K, n_in, nullptr, d_in, stream, "maxpool_bwd");
}

extern "C" int ssc_avgpool_bwd(const float *out_grad, int c, const int32_t *nbr_in, int K, int n_in,
                               const int32_t *summaryrf, float *d_in, void *stream) {
  return launch_pool_bwd<1>(nullptr, nullptr, out_grad, c, nbr_in, K, n_in, summaryrf, d_in, stream, "avgpool_bwd");
}

extern "C" int ssc_global_avgpool_bwd(const float *d_out, const int32_t *offsets, int n_samples, int c, int n_rows,
                                      float *d_feats, void *stream) {
  SSC_REQUIRE(n_samples >= 0 && c > 0 && n_rows >= 0, "global_avgpool_bwd: bad sizes");
  cudaStream_t st = as_stream(stream);
  if (n_rows > 0) cudaMemsetAsync(d_feats, 0, (size_t)n_rows * c * 4, st);  // rows outside every sample range
  if (n_samples == 0 || n_rows == 0) return SSC_OK;
  SSC_REQUIRE(d_out && offsets && d_feats, "global_avgpool_bwd: null pointer");
  dim3 grid(n_samples, ceil_div(c, 32)), block(32, 8);
  { global_avgpool_bwd_kernel<<<grid, block, 0, st>>>(d_out, offsets, c, d_feats); note_launches(1); }
  SSC_CHECK_LAUNCH("global_avgpool_bwd");
  return SSC_OK;
}

extern "C" int ssc_global_maxpool_bwd(const float *d_out, const int32_t *maxidx, int n_samples, int c, int n_rows,
                                      float *d_feats, void *stream) {
  SSC_REQUIRE(n_samples >= 0 && c > 0 && n_rows >= 0, "global_maxpool_bwd: bad sizes");
  cudaStream_t st = as_stream(stream);
  if (n_rows > 0) cudaMemsetAsync(d_feats, 0, (size_t)n_rows * c * 4, st);
  if (n_samples == 0 || n_rows == 0) return SSC_OK;
  SSC_REQUIRE(d_out && maxidx && d_feats, "global_maxpool_bwd: null pointer");
  long long total = (long long)n_samples * c;
  { global_maxpool_bwd_kernel<<<ceil_div(total, 256), 256, 0, st>>>(d_out, maxidx, total, c, n_rows, d_feats); note_launches(1); }
  SSC_CHECK_LAUNCH("global_maxpool_bwd");
  return SSC_OK;
}
