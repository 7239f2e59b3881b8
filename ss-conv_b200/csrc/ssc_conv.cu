// Steerable kernel materialisation and the exact-fp32 (CUDA core) output-stationary
// gather-GEMM kernel.  The tensor-core (tcgen05) variant lives in ssc_conv_tc.cu.
#include "ssc_conv_internal.cuh"

namespace ssc {

// filters[kappa][cin][cout] = sum_b w[u,v,b] * basis[b,a,c,kappa]; one thread per element,
// cout fastest so the (large) filter tensor is written coalesced; the basis blob is small
// and stays in L1/L2.
__global__ void materialize_kernel(const float *__restrict__ weight, const float *__restrict__ basis,
                                   const int32_t *__restrict__ block_table, int n_blocks_in,
                                   const int32_t *__restrict__ out_field, const int32_t *__restrict__ in_field,
                                   int c_out, int c_in, int K, float *__restrict__ filters) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)K * c_in * c_out;
  if (t >= total) return;
  int co = (int)(t % c_out);
  long long r = t / c_out;
  int ci = (int)(r % c_in);
  int kappa = (int)(r / c_in);
  int i = out_field[co * 3 + 0], u = out_field[co * 3 + 1], a = out_field[co * 3 + 2];
  int j = in_field[ci * 3 + 0], v = in_field[ci * 3 + 1], c = in_field[ci * 3 + 2];
  const int32_t *blk = block_table + (size_t)(i * n_blocks_in + j) * 6;
  int boff = blk[0];
  float acc = 0.f;
  if (boff >= 0) {
    int woff = blk[1], nb = blk[2], m_in = blk[3], d_out = blk[4], d_in = blk[5];
    const float *w = weight + woff + (size_t)(u * m_in + v) * nb;
    const float *bp = basis + boff + (size_t)(a * d_in + c) * K + kappa;
    size_t bstride = (size_t)d_out * d_in * K;
    for (int b = 0; b < nb; ++b) acc = fmaf(w[b], bp[b * bstride], acc);
  }
  filters[t] = acc;
}

// ---------------------------------------------------------------------------------------
// Exact fp32 path: tile of 64 output rows x 64 output channels per block, 256 threads with a
// 4x4 register tile each, reduction over (kernel offset, input channel) in chunks of 16.
// Offsets with no neighbour inside the tile are skipped.
constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
conv_fwd_fp32_kernel(const float *__restrict__ features, int c_in, const float *__restrict__ filters, int K,
                     int c_out, const int32_t *__restrict__ nbr, int n_out, float *__restrict__ out,
                     const int32_t *__restrict__ n_out_dev) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  __shared__ int rows[BM];
  int tid = threadIdx.x;
  int tx = tid & 15, ty = tid >> 4;
  int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int n_rows = live_rows(n_out, n_out_dev);
  if (m0 >= n_rows) return;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int kappa = 0; kappa < K; ++kappa) {
    int r = -1;
    if (tid < BM && m0 + tid < n_rows) r = nbr[(size_t)kappa * n_out + m0 + tid];
    __syncthreads();  // previous iteration finished reading rows/As/Bs
    if (tid < BM) rows[tid] = r;
    if (!__syncthreads_or(r >= 0)) continue;
    const float *wk = filters + (size_t)kappa * c_in * c_out;
    for (int kc = 0; kc < c_in; kc += BK) {
      {  // A tile: 64 rows x 16 channels, 4 consecutive channels per thread
        int m = tid >> 2, k4 = (tid & 3) * 4;
        int row = rows[m];
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (row >= 0) {
          const float *src = features + (size_t)row * c_in + kc + k4;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (kc + k4 + q < c_in) v[q] = __ldg(src + q);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) As[k4 + q][m] = v[q];
      }
      {  // B tile: 16 input channels x 64 output channels
        int k = tid >> 4, n4 = (tid & 15) * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (kc + k < c_in) {
          const float *src = wk + (size_t)(kc + k) * c_out + n0 + n4;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (n0 + n4 + q < c_out) v[q] = __ldg(src + q);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) Bs[k][n4 + q] = v[q];
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK; ++k) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty * 4 + i;
    if (m >= n_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n < c_out) out[(size_t)m * c_out + n] = acc[i][j];
    }
  }
}

}  // namespace ssc

using namespace ssc;

extern "C" int ssc_materialize(const float *weight, const float *basis, const int32_t *block_table,
                               int n_blocks_in, const int32_t *out_field, const int32_t *in_field, int c_out,
                               int c_in, int K, float *filters, void *stream) {
  SSC_REQUIRE(c_out > 0 && c_in > 0 && K > 0 && n_blocks_in > 0, "materialize: bad sizes");
  SSC_REQUIRE(weight && basis && block_table && out_field && in_field && filters, "materialize: null pointer");
  long long total = (long long)K * c_in * c_out;
  { materialize_kernel<<<ceil_div(total, 256), 256, 0, as_stream(stream)>>>(weight, basis, block_table, n_blocks_in,
                                                                         out_field, in_field, c_out, c_in, K, filters); note_launches(1); }
  SSC_CHECK_LAUNCH("materialize");
  return SSC_OK;
}

extern "C" size_t ssc_conv_scratch_bytes(int n_in, int c_in, int c_out, int precision) {
  if (n_in < 0 || c_in < 1 || c_out < 1) return 0;
  (void)c_out;
  if (precision == SSC_PREC_F16 || precision == SSC_PREC_BF16) return conv_f16_scratch_bytes(n_in, c_in);
  if (precision != SSC_PREC_TF32) return 0;
  return conv_tf32_scratch_bytes(n_in, c_in);
}

extern "C" int ssc_conv_stage(const float *features, int n_in, int c_in, int precision, void *scratch, size_t scratch_bytes,
                              void *stream) {
  SSC_REQUIRE(c_in > 0 && n_in >= 0 && (n_in == 0 || features) && scratch, "conv_stage: bad arguments");
  SSC_REQUIRE(precision == SSC_PREC_TF32 || precision == SSC_PREC_F16 || precision == SSC_PREC_BF16, "conv_stage: precision %d has no staged image", precision);
  SSC_REQUIRE(scratch_bytes + 16 >= ssc_conv_scratch_bytes(n_in, c_in, 1, precision) && ((uintptr_t)scratch & 15u) == 0,
              "conv_stage: scratch too small or not 16-byte aligned");
  return precision == SSC_PREC_TF32 ? stage_features(features, n_in, c_in, scratch, as_stream(stream))
                                    : stage_features_16(features, n_in, c_in, precision == SSC_PREC_BF16, scratch, as_stream(stream));
}

extern "C" int ssc_conv_fwd_ordered(const float *features, int n_in, int c_in, const void *filters, int K, int c_out,
                                    const int32_t *nbr, int n_out, int precision, float *out, int32_t *status,
                                    void *scratch, size_t scratch_bytes, const int32_t *n_out_dev,
                                    const int32_t *row_order, void *stream) {
  SSC_REQUIRE(c_in > 0 && c_out > 0 && K > 0 && n_in >= 0 && n_out >= 0, "conv_fwd: bad sizes");
  const bool prestaged = (precision & SSC_CONV_PRESTAGED) != 0;
  const bool table_in_order = (precision & SSC_CONV_TABLE_IN_ORDER) != 0;
  precision &= ~(SSC_CONV_PRESTAGED | SSC_CONV_TABLE_IN_ORDER);
  if (n_out == 0) return SSC_OK;
  SSC_REQUIRE(filters && nbr && out && (n_in == 0 || features || prestaged), "conv_fwd: null pointer");
  SSC_REQUIRE(!table_in_order || (row_order && precision != SSC_PREC_FP32),
              "conv_fwd: SSC_CONV_TABLE_IN_ORDER needs a row order and a tensor-core precision");
  cudaStream_t st = as_stream(stream);
  if (precision == SSC_PREC_FP32) {
    dim3 grid(ceil_div(n_out, BM), ceil_div(c_out, BN));
    { conv_fwd_fp32_kernel<<<grid, 256, 0, st>>>(features, c_in, (const float *)filters, K, c_out, nbr, n_out, out, n_out_dev); note_launches(1); }
    SSC_CHECK_LAUNCH("conv_fwd_fp32");
    return SSC_OK;
  }
  if (precision == SSC_PREC_TF32) return conv_fwd_tf32(features, n_in, c_in, filters, K, c_out, nbr, n_out, out, status, scratch, scratch_bytes, n_out_dev, row_order, prestaged, table_in_order, st);
  if (precision == SSC_PREC_F16 || precision == SSC_PREC_BF16)
    return conv_fwd_16(features, n_in, c_in, precision == SSC_PREC_BF16, filters, K, c_out, nbr, n_out, out, status, scratch, scratch_bytes, n_out_dev, row_order, prestaged, table_in_order, st);
  return fail(SSC_ERR_INVALID, "conv_fwd: unknown precision %d", precision);
}

extern "C" int ssc_conv_fwd(const float *features, int n_in, int c_in, const void *filters, int K, int c_out,
                            const int32_t *nbr, int n_out, int precision, float *out, int32_t *status,
                            void *scratch, size_t scratch_bytes, const int32_t *n_out_dev, void *stream) {
  return ssc_conv_fwd_ordered(features, n_in, c_in, filters, K, c_out, nbr, n_out, precision, out, status, scratch,
                              scratch_bytes, n_out_dev, nullptr, stream);
}
