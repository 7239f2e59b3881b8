// Irrep-wise BatchNorm (eval: folded per-channel affine; train: statistics) and the gated
// activation, as single elementwise passes.  HBM-bound.
#include "ssc_common.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

__global__ void bn_fold_kernel(const float *running_mean, const float *running_var, const float *weight,
                               const float *bias, const int32_t *field_of_channel, const int32_t *scalar_of_channel,
                               int c, float eps, float *scale, float *shift) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  int f = field_of_channel[ch], s = scalar_of_channel[ch];
  float sc = 1.0f / sqrtf(running_var[f] + eps);
  if (weight) sc *= weight[f];
  float sh = 0.f;
  if (s >= 0) {
    sh = -running_mean[s] * sc;
    if (bias) sh += bias[s];
  }
  scale[ch] = sc;
  shift[ch] = sh;
}

__device__ __forceinline__ float apply_act(float v, int kind) {
  if (kind == 1) return v > 0.f ? v : 0.f;
  if (kind == 2) return 1.0f / (1.0f + expf(-v));
  return v;
}

// One thread per output element (any channel counts / alignment).
__global__ void bn_gate_kernel(const float *__restrict__ x, long long total, int c_in_total,
                               const float *__restrict__ scale, const float *__restrict__ shift,
                               const int32_t *__restrict__ gate_of_channel, int c_out, int c_gate_base,
                               int scalar_act, int gate_act, const float *__restrict__ scalar_bias,
                               const float *__restrict__ gate_bias, float *__restrict__ out) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  long long row = t / c_out;
  int ch = (int)(t - row * c_out);
  const float *xr = x + row * c_in_total;
  float v = xr[ch];
  if (scale) v = fmaf(v, scale[ch], shift[ch]);
  if (gate_of_channel) {
    int g = gate_of_channel[ch];
    if (g == -1) {
      if (scalar_bias) v += scalar_bias[ch];
      v = apply_act(v, scalar_act);
    } else if (g >= 0) {
      float gv = xr[c_gate_base + g];
      if (scale) gv = fmaf(gv, scale[c_gate_base + g], shift[c_gate_base + g]);
      if (gate_bias) gv += gate_bias[g];
      v *= apply_act(gv, gate_act);
    }
  }
  out[t] = v;
}

// Four consecutive output channels per thread (16-byte loads and stores, 32-bit index arithmetic):
// channel counts that are multiples of four, 16-byte aligned rows.  Same arithmetic per element
// as the scalar kernel.  groups = c_out / 4; total = rows * groups < 2^31.
__global__ void __launch_bounds__(256)
bn_gate_vec4_kernel(const float *__restrict__ x, uint32_t total, uint32_t groups, int c_in_total,
                    const float *__restrict__ scale, const float *__restrict__ shift,
                    const int32_t *__restrict__ gate_of_channel, int c_gate_base, int scalar_act, int gate_act,
                    const float *__restrict__ scalar_bias, const float *__restrict__ gate_bias, float *__restrict__ out) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const uint32_t row = t / groups, g4 = t - row * groups;
  const int ch0 = (int)g4 * 4;
  const float *xr = x + (size_t)row * c_in_total;
  const float4 xv = __ldg((const float4 *)(xr + ch0));
  float v[4] = {xv.x, xv.y, xv.z, xv.w};
  if (scale) {
    const float4 sc = __ldg((const float4 *)(scale + ch0)), sh = __ldg((const float4 *)(shift + ch0));
    v[0] = fmaf(v[0], sc.x, sh.x);
    v[1] = fmaf(v[1], sc.y, sh.y);
    v[2] = fmaf(v[2], sc.z, sh.z);
    v[3] = fmaf(v[3], sc.w, sh.w);
  }
  if (gate_of_channel) {
    const int4 gi = __ldg((const int4 *)(gate_of_channel + ch0));
    const int g[4] = {gi.x, gi.y, gi.z, gi.w};
    int last_g = -2;
    float last_a = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (g[q] == -1) {
        if (scalar_bias) v[q] += scalar_bias[ch0 + q];
        v[q] = apply_act(v[q], scalar_act);
      } else if (g[q] >= 0) {
        if (g[q] != last_g) {   // the channels of a field share their gate
          float gv = __ldg(xr + c_gate_base + g[q]);
          if (scale) gv = fmaf(gv, scale[c_gate_base + g[q]], shift[c_gate_base + g[q]]);
          if (gate_bias) gv += gate_bias[g[q]];
          last_a = apply_act(gv, gate_act);
          last_g = g[q];
        }
        v[q] *= last_a;
      }
    }
  }
  *(float4 *)(out + (size_t)t * 4) = make_float4(v[0], v[1], v[2], v[3]);
}

// The same with a 16-bit result (OUT = 1 fp16, 2 bf16): the features leave the layer in the operand
// precision of the next convolution, which then gathers them as they are (no staging pass).
// Four consecutive output channels per thread:
// channel counts that are multiples of four, 16-byte aligned rows.  Same arithmetic per element
// as the scalar kernel.  groups = c_out / 4; total = rows * groups < 2^31.
template <int OUT>
__global__ void __launch_bounds__(256)
bn_gate_vec4_out16_kernel(const float *__restrict__ x, uint32_t total, uint32_t groups, int c_in_total,
                    const float *__restrict__ scale, const float *__restrict__ shift,
                    const int32_t *__restrict__ gate_of_channel, int c_gate_base, int scalar_act, int gate_act,
                    const float *__restrict__ scalar_bias, const float *__restrict__ gate_bias, uint2 *__restrict__ out) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const uint32_t row = t / groups, g4 = t - row * groups;
  const int ch0 = (int)g4 * 4;
  const float *xr = x + (size_t)row * c_in_total;
  const float4 xv = __ldg((const float4 *)(xr + ch0));
  float v[4] = {xv.x, xv.y, xv.z, xv.w};
  if (scale) {
    const float4 sc = __ldg((const float4 *)(scale + ch0)), sh = __ldg((const float4 *)(shift + ch0));
    v[0] = fmaf(v[0], sc.x, sh.x);
    v[1] = fmaf(v[1], sc.y, sh.y);
    v[2] = fmaf(v[2], sc.z, sh.z);
    v[3] = fmaf(v[3], sc.w, sh.w);
  }
  if (gate_of_channel) {
    const int4 gi = __ldg((const int4 *)(gate_of_channel + ch0));
    const int g[4] = {gi.x, gi.y, gi.z, gi.w};
    int last_g = -2;
    float last_a = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (g[q] == -1) {
        if (scalar_bias) v[q] += scalar_bias[ch0 + q];
        v[q] = apply_act(v[q], scalar_act);
      } else if (g[q] >= 0) {
        if (g[q] != last_g) {   // the channels of a field share their gate
          float gv = __ldg(xr + c_gate_base + g[q]);
          if (scale) gv = fmaf(gv, scale[c_gate_base + g[q]], shift[c_gate_base + g[q]]);
          if (gate_bias) gv += gate_bias[g[q]];
          last_a = apply_act(gv, gate_act);
          last_g = g[q];
        }
        v[q] *= last_a;
      }
    }
  }
  out[t] = OUT == 2 ? make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]))
                    : make_uint2(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]));
}

// Column sums with one block per 32-channel group: block (32, 8), rows strided by 8*gridDim.y.
// pass 0: sum of x per channel; pass 1: sum of (x - mean_ch)^2 per channel (mean_ch = 0 for
// non-scalar channels), accumulated per field.
__global__ void bn_colsum_kernel(const float *__restrict__ x, int n, int c, const float *__restrict__ chan_mean,
                                 float *__restrict__ acc, const int32_t *__restrict__ bucket_of_channel) {
  __shared__ float sm[8][33];
  int ch = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (ch < c) {
    float mu = chan_mean ? chan_mean[ch] : 0.f;
    for (int r = blockIdx.y * 8 + threadIdx.y; r < n; r += 8 * gridDim.y) {
      float v = x[(size_t)r * c + ch] - mu;
      s += chan_mean ? v * v : v;
    }
  }
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && ch < c) {
    for (int g = 1; g < 8; ++g) s += sm[g][threadIdx.x];
    int b = bucket_of_channel[ch];
    if (b >= 0) atomicAdd(acc + b, s);
  }
}

// chan_mean[ch] = batch mean of a scalar channel (0 for l>0 channels), from the channel sums.
__global__ void bn_chan_mean_kernel(const float *sum_scalar, int n, const int32_t *scalar_of_channel, int c,
                                    float *chan_mean) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= c) return;
  int s = scalar_of_channel[i];
  chan_mean[i] = s >= 0 ? sum_scalar[s] / (float)n : 0.f;
}

__global__ void bn_finish_var_kernel(float *var, int n_field, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_field) var[i] = var[i] / (float)n;
}

}  // namespace ssc

using namespace ssc;

extern "C" int ssc_bn_fold(const float *running_mean, const float *running_var, const float *weight,
                           const float *bias, const int32_t *field_of_channel, const int32_t *scalar_of_channel,
                           int c, float eps, float *scale, float *shift, void *stream) {
  SSC_REQUIRE(c >= 1 && running_var && field_of_channel && scalar_of_channel && scale && shift, "bn_fold: bad arguments");
  { bn_fold_kernel<<<ceil_div(c, 128), 128, 0, as_stream(stream)>>>(running_mean, running_var, weight, bias,
                                                                 field_of_channel, scalar_of_channel, c, eps, scale, shift); note_launches(1); }
  SSC_CHECK_LAUNCH("bn_fold");
  return SSC_OK;
}

extern "C" int ssc_bn_gate_fwd(const float *x, int n, int c_in_total, const float *scale, const float *shift,
                               const int32_t *gate_of_channel, int c_out, int c_gate_base, int scalar_act,
                               int gate_act, const float *scalar_bias, const float *gate_bias, float *out,
                               void *stream) {
  SSC_REQUIRE(n >= 0 && c_in_total >= 1 && c_out >= 1 && c_out <= c_in_total, "bn_gate_fwd: bad sizes");
  SSC_REQUIRE((scale == nullptr) == (shift == nullptr), "bn_gate_fwd: scale and shift go together");
  if (n == 0) return SSC_OK;
  SSC_REQUIRE(x && out, "bn_gate_fwd: null pointer");
  long long total = (long long)n * c_out;
  const bool vec = (c_out & 3) == 0 && (c_in_total & 3) == 0 && (c_gate_base & 3) == 0 && total / 4 < (1ll << 31) &&
                   (((uintptr_t)x | (uintptr_t)out | (uintptr_t)scale | (uintptr_t)shift | (uintptr_t)gate_of_channel) & 15u) == 0;
  if (vec) {
    const uint32_t groups = (uint32_t)(c_out >> 2), total4 = (uint32_t)(total >> 2);
    { bn_gate_vec4_kernel<<<ceil_div(total4, 256), 256, 0, as_stream(stream)>>>(x, total4, groups, c_in_total, scale, shift,
                                                                            gate_of_channel, c_gate_base, scalar_act, gate_act,
                                                                            scalar_bias, gate_bias, out); note_launches(1); }
    SSC_CHECK_LAUNCH("bn_gate_fwd");
    return SSC_OK;
  }
  { bn_gate_kernel<<<ceil_div(total, 256), 256, 0, as_stream(stream)>>>(x, total, c_in_total, scale, shift, gate_of_channel,
                                                                     c_out, c_gate_base, scalar_act, gate_act,
                                                                     scalar_bias, gate_bias, out); note_launches(1); }
  SSC_CHECK_LAUNCH("bn_gate_fwd");
  return SSC_OK;
}

extern "C" int ssc_bn_gate_fwd16(const float *x, int n, int c_in_total, const float *scale, const float *shift,
                                 const int32_t *gate_of_channel, int c_out, int c_gate_base, int scalar_act,
                                 int gate_act, const float *scalar_bias, const float *gate_bias, int precision,
                                 void *out16, void *stream) {
  SSC_REQUIRE(n >= 0 && c_in_total >= 1 && c_out >= 1 && c_out <= c_in_total, "bn_gate_fwd16: bad sizes");
  SSC_REQUIRE(precision == SSC_PREC_F16 || precision == SSC_PREC_BF16, "bn_gate_fwd16: precision must be SSC_PREC_F16 or SSC_PREC_BF16");
  SSC_REQUIRE((scale == nullptr) == (shift == nullptr), "bn_gate_fwd16: scale and shift go together");
  SSC_REQUIRE((c_out & 7) == 0 && (c_in_total & 3) == 0 && (c_gate_base & 3) == 0,
              "bn_gate_fwd16: needs c_out a multiple of 8 (16-byte rows) and c_in_total, c_gate_base multiples of 4");
  if (n == 0) return SSC_OK;
  SSC_REQUIRE(x && out16, "bn_gate_fwd16: null pointer");
  SSC_REQUIRE((((uintptr_t)x | (uintptr_t)out16 | (uintptr_t)scale | (uintptr_t)shift | (uintptr_t)gate_of_channel) & 15u) == 0,
              "bn_gate_fwd16: pointers must be 16-byte aligned");
  const long long total = (long long)n * c_out;
  SSC_REQUIRE(total / 4 < (1ll << 31), "bn_gate_fwd16: tensor too large");
  const uint32_t groups = (uint32_t)(c_out >> 2), total4 = (uint32_t)(total >> 2);
  if (precision == SSC_PREC_BF16) {
    { bn_gate_vec4_out16_kernel<2><<<ceil_div(total4, 256), 256, 0, as_stream(stream)>>>(x, total4, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act, scalar_bias, gate_bias, (uint2 *)out16); note_launches(1); }
  } else {
    { bn_gate_vec4_out16_kernel<1><<<ceil_div(total4, 256), 256, 0, as_stream(stream)>>>(x, total4, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act, scalar_bias, gate_bias, (uint2 *)out16); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("bn_gate_fwd16");
  return SSC_OK;
}

// mean/var double as accumulators; chan_mean lives in the first c floats after var's
// n_field entries is NOT assumed: the caller passes var with room for n_field + c floats.
extern "C" int ssc_bn_stats(const float *x, int n, int c, const int32_t *field_of_channel,
                            const int32_t *scalar_of_channel, int n_field, int n_scalar, float *mean, float *var,
                            void *stream) {
  SSC_REQUIRE(n >= 1 && c >= 1 && n_field >= 1 && n_scalar >= 0, "bn_stats: bad sizes");
  SSC_REQUIRE(x && field_of_channel && scalar_of_channel && mean && var, "bn_stats: null pointer");
  cudaStream_t st = as_stream(stream);
  float *chan_mean = var + n_field;  // scratch tail, c floats
  cudaMemsetAsync(mean, 0, (size_t)(n_scalar > 0 ? n_scalar : 1) * 4, st);
  cudaMemsetAsync(var, 0, (size_t)n_field * 4, st);
  dim3 block(32, 8);
  int row_blocks = ceil_div(n, 8 * 64);
  if (row_blocks > 64) row_blocks = 64;
  dim3 grid(ceil_div(c, 32), row_blocks);
  { bn_colsum_kernel<<<grid, block, 0, st>>>(x, n, c, nullptr, mean, scalar_of_channel); note_launches(1); }
  { bn_chan_mean_kernel<<<ceil_div(c, 128), 128, 0, st>>>(mean, n, scalar_of_channel, c, chan_mean); note_launches(1); }
  if (n_scalar > 0) { bn_finish_var_kernel<<<ceil_div(n_scalar, 128), 128, 0, st>>>(mean, n_scalar, n); note_launches(1); }
  { bn_colsum_kernel<<<grid, block, 0, st>>>(x, n, c, chan_mean, var, field_of_channel); note_launches(1); }
  { bn_finish_var_kernel<<<ceil_div(n_field, 128), 128, 0, st>>>(var, n_field, n); note_launches(1); }
  SSC_CHECK_LAUNCH("bn_stats");
  return SSC_OK;
}
