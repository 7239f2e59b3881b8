// Staged operand images of the feature rows for the tensor-core convolution kernels.
//
// A feature row is gathered once per neighbour (about K/2 times for a 3^3 kernel), so the rounding
// to the operand precision is done once per call, up front, into a caller-supplied buffer:
//   TF32 : [n_in, c_pad] fp32 words rounded to nearest TF32, c_pad = c_in rounded up to 4
//   fp16 / bf16 : [n_in, c_pad] 16-bit values, c_pad = c_in rounded up to 8 (16-byte rows)
// Padding channels are zero.  A layer that already holds its features in the 16-bit form (written
// by ssc_bn_gate_fwd16, or uploaded that way) hands them to the convolution as the staged image.
#include "ssc_conv_internal.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

__global__ void stage_features_kernel(const float4 *__restrict__ in, long long n_vec, long long total_vec,
                                      uint4 *__restrict__ out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; i < total_vec; i += step) {
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (i < n_vec) {
      float4 v = __ldg(in + i);
      o = make_uint4(to_tf32(v.x), to_tf32(v.y), to_tf32(v.z), to_tf32(v.w));
    }
    out[i] = o;
  }
}

// Channel counts that are not a multiple of four: rows padded with zeros to c_pad floats.
__global__ void stage_features_padded_kernel(const float *__restrict__ in, long long n_rows, int c_in, int c_pad,
                                             long long total, uint32_t *__restrict__ out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const long long r = i / c_pad;
    const int c = (int)(i - r * c_pad);
    out[i] = (r < n_rows && c < c_in) ? to_tf32(__ldg(in + r * c_in + c)) : 0u;
  }
}

// The same for up to 1024 channels with a block shaped (groups of four channels, rows): one 16-byte
// store per thread and no integer division (the kernel above spends most of its time in a 64-bit
// division per element).
__global__ void __launch_bounds__(256)
stage_features_padded_rows_kernel(const float *__restrict__ in, int n_rows, int c_in, uint4 *__restrict__ out) {
  const int row = blockIdx.x * blockDim.y + threadIdx.y, c0 = threadIdx.x * 4;
  if (row >= n_rows) return;
  const float *src = in + (size_t)row * c_in + c0;
  uint32_t v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) v[q] = c0 + q < c_in ? to_tf32(__ldg(src + q)) : 0u;
  out[(size_t)row * blockDim.x + threadIdx.x] = make_uint4(v[0], v[1], v[2], v[3]);
}

size_t conv_tf32_scratch_bytes(int n_in, int c_in) {
  return align_up((size_t)n_in * (size_t)((c_in + 3) & ~3) * sizeof(float), 16) + 16;
}

int stage_features(const float *features, int n_in, int c_in, void *staged, cudaStream_t st) {
  const int c_pad = (c_in + 3) & ~3;
  const int max_blocks = sm_count() * 16;
  if (n_in == 0) return SSC_OK;
  if (c_pad == c_in && ((uintptr_t)features & 15u) == 0) {
    const long long n_vec = (long long)n_in * c_in / 4, total_vec = n_vec;
    int blocks = ceil_div(total_vec, 256 * 4);
    if (blocks > max_blocks) blocks = max_blocks;
    { stage_features_kernel<<<blocks, 256, 0, st>>>((const float4 *)features, n_vec, total_vec, (uint4 *)staged); note_launches(1); }
  } else if (c_pad <= 1024) {
    const int groups = c_pad >> 2, rows = 256 / groups;
    { stage_features_padded_rows_kernel<<<ceil_div(n_in, rows), dim3(groups, rows), 0, st>>>(features, n_in, c_in, (uint4 *)staged); note_launches(1); }
  } else {
    const long long total = (long long)n_in * c_pad;
    int blocks = ceil_div(total, 256 * 4);
    if (blocks > max_blocks) blocks = max_blocks;
    { stage_features_padded_kernel<<<blocks, 256, 0, st>>>(features, n_in, c_in, c_pad, total, (uint32_t *)staged); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("stage_features");
  return SSC_OK;
}

// 16-bit images: one thread per pair of channels; BF16 selects bfloat16 (fp32's exponent range,
// 8 significant bits) instead of fp16 (11 significant bits, finite values beyond +-65504 saturate).
template <bool BF16>
__global__ void stage_features_16_kernel(const float *__restrict__ in, long long n_rows, int c_in, int c_pad,
                                         long long total_pairs, uint32_t *__restrict__ out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  const int pairs = c_pad >> 1;
  for (; i < total_pairs; i += step) {
    const long long r = i / pairs;
    const int c = (int)(i - r * pairs) * 2;
    float a = 0.f, b = 0.f;
    if (r < n_rows) {
      if (c < c_in) a = __ldg(in + r * c_in + c);
      if (c + 1 < c_in) b = __ldg(in + r * c_in + c + 1);
    }
    out[i] = BF16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
  }
}

size_t conv_f16_scratch_bytes(int n_in, int c_in) { return (size_t)n_in * (size_t)f16_row_words(c_in) * 4 + 16; }

int stage_features_16(const float *features, int n_in, int c_in, bool bf16, void *staged, cudaStream_t st) {
  if (n_in == 0) return SSC_OK;
  const int words = f16_row_words(c_in);
  const long long total_pairs = (long long)n_in * words;
  int blocks = ceil_div(total_pairs, 256 * 4);
  const int max_blocks = sm_count() * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  if (bf16) { stage_features_16_kernel<true><<<blocks, 256, 0, st>>>(features, n_in, c_in, words * 2, total_pairs, (uint32_t *)staged); note_launches(1); }
  else { stage_features_16_kernel<false><<<blocks, 256, 0, st>>>(features, n_in, c_in, words * 2, total_pairs, (uint32_t *)staged); note_launches(1); }
  SSC_CHECK_LAUNCH("stage_features_16");
  return SSC_OK;
}

}  // namespace ssc
