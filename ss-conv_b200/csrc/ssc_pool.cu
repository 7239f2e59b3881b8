// Sparse max / avg pooling over the output-major neighbour table (one launch, each output
// row written once) and per-sample global pooling.  All HBM-bound.
#include "ssc_common.cuh"

namespace ssc {

// MODE 0 = max (output starts at 0), 1 = avg (sum of x / divisor in ascending offset order).
// One thread per (output row, 4 channels).
template <int MODE, bool VEC>
__global__ void pool_fwd_kernel(const float *__restrict__ features, int c, const int32_t *__restrict__ nbr, int K,
                                int n_out, const int32_t *__restrict__ summaryrf, float *__restrict__ out,
                                const int32_t *__restrict__ n_out_dev) {
  int cg = (c + 3) >> 2;
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)live_rows(n_out, n_out_dev) * cg) return;  // n_out stays the row stride of nbr
  int o = (int)(t / cg);
  int c0 = (int)(t - (long long)o * cg) * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float div = 1.f;
  if (MODE == 1) div = summaryrf ? (float)summaryrf[o] : (float)K;
  for (int kappa = 0; kappa < K; ++kappa) {
    int src = __ldg(nbr + (size_t)kappa * n_out + o);
    if (src < 0) continue;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const float *fp = features + (size_t)src * c + c0;
    if (VEC) {
      float4 f = __ldg((const float4 *)fp);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (c0 + q < c) v[q] = __ldg(fp + q);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (MODE == 0) acc[q] = v[q] > acc[q] ? v[q] : acc[q];
      else acc[q] = acc[q] + v[q] / div;
    }
  }
  float *op = out + (size_t)o * c + c0;
  if (VEC) {
    *(float4 *)op = make_float4(acc[0], acc[1], acc[2], acc[3]);
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (c0 + q < c) op[q] = acc[q];
  }
}

__global__ void summary_rf_kernel(const int32_t *__restrict__ nbr, int K, int n_out, int32_t *__restrict__ rf) {
  int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n_out) return;
  int cnt = 0;
  for (int kappa = 0; kappa < K; ++kappa) cnt += nbr[(size_t)kappa * n_out + o] >= 0;
  rf[o] = cnt;
}

// grid (samples, channel groups of 32), block (32, 8): the 8 row groups stride over the
// sample's rows, partial results are combined in shared memory.
template <bool MAX>
__global__ void global_pool_kernel(const float *__restrict__ feats, const int32_t *__restrict__ offsets, int c,
                                   float *__restrict__ out, int32_t *__restrict__ maxidx) {
  __shared__ float sv[8][33];
  __shared__ int si[8][33];
  int s = blockIdx.x;
  int ch = blockIdx.y * 32 + threadIdx.x;
  int start = offsets[s], end = offsets[s + 1];
  float acc = MAX ? -INFINITY : 0.f;
  int arg = -1;
  if (ch < c) {
    for (int r = start + threadIdx.y; r < end; r += 8) {
      float v = __ldg(feats + (size_t)r * c + ch);
      if (MAX) {
        if (v > acc) { acc = v; arg = r; }
      } else {
        acc += v;
      }
    }
  }
  sv[threadIdx.y][threadIdx.x] = acc;
  si[threadIdx.y][threadIdx.x] = arg;
  __syncthreads();
  if (threadIdx.y == 0 && ch < c) {
    for (int g = 1; g < 8; ++g) {
      float v = sv[g][threadIdx.x];
      int a = si[g][threadIdx.x];
      if (MAX) {
        if (a >= 0 && (v > acc || (v == acc && (arg < 0 || a < arg)))) { acc = v; arg = a; }
      } else {
        acc += v;
      }
    }
    if (MAX) {
      out[(size_t)s * c + ch] = acc;
      if (maxidx) maxidx[(size_t)s * c + ch] = arg;
    } else {
      out[(size_t)s * c + ch] = acc / (float)(end - start);
    }
  }
}

// offsets[b+1] = number of rows with batch id <= b: histogram, then an in-place scan by one warp.
__global__ void batch_count_kernel(const int4 *__restrict__ indices, int n, int batch, int32_t *offsets,
                                   const int32_t *__restrict__ n_dev) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= live_rows(n, n_dev)) return;
  int b = indices[i].x;
  if ((unsigned)b < (unsigned)batch) atomicAdd(offsets + b + 1, 1);
}

__global__ void batch_scan_kernel(int32_t *offsets, int batch) {
  int lane = threadIdx.x;
  int running = 0;
  for (int base = 1; base <= batch; base += 32) {
    int i = base + lane;
    int v = i <= batch ? offsets[i] : 0;
    int incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (i <= batch) offsets[i] = running + incl;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
}

}  // namespace ssc

using namespace ssc;

template <int MODE>
static int launch_pool(const float *features, int c, const int32_t *nbr, int K, int n_out, const int32_t *rf,
                       float *out, const int32_t *n_out_dev, void *stream, const char *name) {
  SSC_REQUIRE(c > 0 && K > 0 && n_out >= 0, "%s: bad sizes", name);
  if (n_out == 0) return SSC_OK;
  SSC_REQUIRE(features && nbr && out, "%s: null pointer", name);
  long long threads = (long long)n_out * ((c + 3) / 4);
  bool vec = (c % 4 == 0) && (((uintptr_t)features | (uintptr_t)out) % 16 == 0);
  if (vec)
    { pool_fwd_kernel<MODE, true><<<ceil_div(threads, 256), 256, 0, as_stream(stream)>>>(features, c, nbr, K, n_out, rf, out, n_out_dev); note_launches(1); }
  else
    { pool_fwd_kernel<MODE, false><<<ceil_div(threads, 256), 256, 0, as_stream(stream)>>>(features, c, nbr, K, n_out, rf, out, n_out_dev); note_launches(1); }
  SSC_CHECK_LAUNCH(name);
  return SSC_OK;
}

extern "C" int ssc_maxpool_fwd(const float *features, int c, const int32_t *nbr, int K, int n_out, float *out,
                               const int32_t *n_out_dev, void *stream) {
  return launch_pool<0>(features, c, nbr, K, n_out, nullptr, out, n_out_dev, stream, "maxpool_fwd");
}

extern "C" int ssc_avgpool_fwd(const float *features, int c, const int32_t *nbr, int K, int n_out,
                               const int32_t *summaryrf, float *out, const int32_t *n_out_dev, void *stream) {
  return launch_pool<1>(features, c, nbr, K, n_out, summaryrf, out, n_out_dev, stream, "avgpool_fwd");
}

extern "C" int ssc_summary_rf(const int32_t *nbr, int K, int n_out, int32_t *rf, void *stream) {
  SSC_REQUIRE(K > 0 && n_out >= 0, "summary_rf: bad sizes");
  if (n_out == 0) return SSC_OK;
  SSC_REQUIRE(nbr && rf, "summary_rf: null pointer");
  { summary_rf_kernel<<<ceil_div(n_out, 256), 256, 0, as_stream(stream)>>>(nbr, K, n_out, rf); note_launches(1); }
  SSC_CHECK_LAUNCH("summary_rf");
  return SSC_OK;
}

extern "C" int ssc_global_avgpool_fwd(const float *feats, const int32_t *offsets, int n_samples, int c, float *out,
                                      void *stream) {
  SSC_REQUIRE(n_samples >= 0 && c > 0, "global_avgpool: bad sizes");
  if (n_samples == 0) return SSC_OK;
  SSC_REQUIRE(offsets && out, "global_avgpool: null pointer");
  dim3 grid(n_samples, ceil_div(c, 32)), block(32, 8);
  { global_pool_kernel<false><<<grid, block, 0, as_stream(stream)>>>(feats, offsets, c, out, nullptr); note_launches(1); }
  SSC_CHECK_LAUNCH("global_avgpool");
  return SSC_OK;
}

extern "C" int ssc_global_maxpool_fwd(const float *feats, const int32_t *offsets, int n_samples, int c, float *out,
                                      int32_t *maxidx, void *stream) {
  SSC_REQUIRE(n_samples >= 0 && c > 0, "global_maxpool: bad sizes");
  if (n_samples == 0) return SSC_OK;
  SSC_REQUIRE(offsets && out, "global_maxpool: null pointer");
  dim3 grid(n_samples, ceil_div(c, 32)), block(32, 8);
  { global_pool_kernel<true><<<grid, block, 0, as_stream(stream)>>>(feats, offsets, c, out, maxidx); note_launches(1); }
  SSC_CHECK_LAUNCH("global_maxpool");
  return SSC_OK;
}

extern "C" int ssc_batch_offsets(const int32_t *indices, int n, int batch, int32_t *offsets, const int32_t *n_dev,
                                 void *stream) {
  SSC_REQUIRE(n >= 0 && batch >= 1 && offsets, "batch_offsets: bad arguments");
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(offsets, 0, (size_t)(batch + 1) * 4, st);
  if (n > 0) { batch_count_kernel<<<ceil_div(n, 256), 256, 0, st>>>((const int4 *)indices, n, batch, offsets, n_dev); note_launches(1); }
  { batch_scan_kernel<<<1, 32, 0, st>>>(offsets, batch); note_launches(1); }
  SSC_CHECK_LAUNCH("batch_offsets");
  return SSC_OK;
}
