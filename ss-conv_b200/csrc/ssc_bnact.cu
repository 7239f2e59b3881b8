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
  if (kind == 2) return __frcp_rn(1.0f + expf(-v));   // the correctly rounded reciprocal: the bits of 1.0f / (...)
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

// The gated pass with every gate evaluated ONCE per row: a block owns R = 256 / groups whole rows,
// first fills gate_s[r][g] = act(BN(x[row, c_gate_base + g]) + bias) for its rows (one value per
// thread), then every thread finishes four consecutive channels of one row and takes its gates
// from shared memory.  The per-element arithmetic is that of the kernels above (same bits); what
// changes is the instruction count: a thread of the kernels above evaluates up to four
// sigmoids (expf + IEEE division each, every path taken by some lane of the warp), which made
// the pass instruction-bound at half the memory rate.  OUT = 0 fp32, 1 fp16, 2 bf16 result.
template <int OUT, int VEC>
__global__ void __launch_bounds__(256)
bn_gate_rows_kernel(const float *__restrict__ x, uint32_t n_rows, uint32_t groups, int c_in_total,
                    const float *__restrict__ scale, const float *__restrict__ shift,
                    const int32_t *__restrict__ gate_of_channel, int c_gate_base, int n_gates, int scalar_act,
                    int gate_act, const float *__restrict__ scalar_bias, const float *__restrict__ gate_bias,
                    void *__restrict__ out) {
  extern __shared__ float gate_s[];                    // [R][n_gates]
  // block = (groups, R): threadIdx.x is the group of VEC channels, threadIdx.y the row of the block
  // (no integer division anywhere in the kernel).  VEC = 4 / 2 / 1 for channel counts that are
  // multiples of four / even / odd (rows 16- / 8- / 4-byte aligned).
  const uint32_t R = blockDim.y, r = threadIdx.y, gq = threadIdx.x, row = blockIdx.x * R + r;
  const bool active = row < n_rows;
  const int ch0 = (int)gq * VEC;
  // this thread's channels: the load goes out before the gate phase, so that both phases'
  // memory latencies overlap
  float v[VEC];
#pragma unroll
  for (int q = 0; q < VEC; ++q) v[q] = 0.f;
  if (active) {
    const float *xp = x + (size_t)row * c_in_total + ch0;
    if (VEC == 4) {
      const float4 t = __ldg((const float4 *)xp);
      v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
    } else if (VEC == 2) {
      const float2 t = __ldg((const float2 *)xp);
      v[0] = t.x; v[1 % VEC] = t.y;
    } else {
      v[0] = __ldg(xp);
    }
    float *my_gates_w = gate_s + r * (uint32_t)n_gates;
    for (uint32_t g = gq; g < (uint32_t)n_gates; g += groups) {
      float gv = __ldg(x + (size_t)row * c_in_total + c_gate_base + g);
      if (scale) gv = fmaf(gv, scale[c_gate_base + g], shift[c_gate_base + g]);
      if (gate_bias) gv += gate_bias[g];
      my_gates_w[g] = apply_act(gv, gate_act);
    }
  }
  __syncthreads();
  if (!active) return;
  const float *my_gates = gate_s + r * (uint32_t)n_gates;
  float sc[VEC], sh[VEC];
  int gi[VEC];
  if (VEC == 4) {   // 16-byte aligned tables (checked by the caller)
    const int4 t = __ldg((const int4 *)(gate_of_channel + ch0));
    gi[0] = t.x; gi[1 % VEC] = t.y; gi[2 % VEC] = t.z; gi[3 % VEC] = t.w;
    if (scale) {
      const float4 a = __ldg((const float4 *)(scale + ch0)), b = __ldg((const float4 *)(shift + ch0));
      sc[0] = a.x; sc[1 % VEC] = a.y; sc[2 % VEC] = a.z; sc[3 % VEC] = a.w;
      sh[0] = b.x; sh[1 % VEC] = b.y; sh[2 % VEC] = b.z; sh[3 % VEC] = b.w;
    }
  } else {
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
      gi[q] = __ldg(gate_of_channel + ch0 + q);
      if (scale) { sc[q] = __ldg(scale + ch0 + q); sh[q] = __ldg(shift + ch0 + q); }
    }
  }
#pragma unroll
  for (int q = 0; q < VEC; ++q) {
    if (scale) v[q] = fmaf(v[q], sc[q], sh[q]);
    const int g = gi[q];
    if (g == -1) {
      if (scalar_bias) v[q] += scalar_bias[ch0 + q];
      v[q] = apply_act(v[q], scalar_act);
    } else if (g >= 0) {
      v[q] *= my_gates[g];
    }
  }
  const size_t t = (size_t)row * groups + gq;
  if (OUT == 0) {
    if (VEC == 4) ((float4 *)out)[t] = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
    else if (VEC == 2) ((float2 *)out)[t] = make_float2(v[0], v[1 % VEC]);
    else ((float *)out)[t] = v[0];
  } else if (OUT == 2) {
    ((uint2 *)out)[t] = make_uint2(pack_bf16x2(v[0], v[1 % VEC]), pack_bf16x2(v[2 % VEC], v[3 % VEC]));
  } else {
    ((uint2 *)out)[t] = make_uint2(pack_f16x2(v[0], v[1 % VEC]), pack_f16x2(v[2 % VEC], v[3 % VEC]));
  }
}

// Launch of the row-block kernel when it applies (gated pass, at most 256 channel groups per row).
template <int OUT, int VEC>
static bool launch_bn_gate_rows(const float *x, int n, uint32_t groups, int c_in_total, const float *scale, const float *shift,
                                const int32_t *gate_of_channel, int c_gate_base, int scalar_act, int gate_act,
                                const float *scalar_bias, const float *gate_bias, void *out, cudaStream_t st) {
  const int n_gates = c_in_total - c_gate_base;
  if (gate_of_channel == nullptr || n_gates < 1 || groups < 1 || groups > 256) return false;
  const uint32_t R = 256u / groups;
  const size_t smem = (size_t)R * n_gates * sizeof(float);
  if (smem > 48 * 1024) return false;
  { bn_gate_rows_kernel<OUT, VEC><<<ceil_div(n, (int)R), dim3(groups, R), smem, st>>>(x, (uint32_t)n, groups, c_in_total, scale, shift,
                                                                          gate_of_channel, c_gate_base, n_gates, scalar_act, gate_act,
                                                                          scalar_bias, gate_bias, out); note_launches(1); }
  return true;
}

// Column sums, deterministic: block (32, 8) owns 32 channels and every gridDim.y-th group of 8
// rows and writes its partial sums to part[blockIdx.y][channel]; colsum_finish adds the partials
// of a bucket's channels in a fixed order (ascending channel, ascending row block), so the batch
// statistics repeat bit for bit.  MODE 0: sum of x; 1: sum of (x - mean_ch)^2; 2: TWO sums for the
// backward pass, of gy (part) and of gy * (x - mean_ch) (part2).
template <int MODE>
__global__ void bn_colsum_kernel(const float *__restrict__ x, const float *__restrict__ gy, int n, int c,
                                 const float *__restrict__ chan_mean, float *__restrict__ part,
                                 float *__restrict__ part2) {
  __shared__ float sm[8][33], sm2[8][33];
  const int ch = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f, s2 = 0.f;
  if (ch < c) {
    const float mu = (MODE != 0 && chan_mean) ? chan_mean[ch] : 0.f;
    for (int r = blockIdx.y * 8 + threadIdx.y; r < n; r += 8 * gridDim.y) {
      const float v = x[(size_t)r * c + ch] - mu;
      if (MODE == 0) s += v;
      else if (MODE == 1) s += v * v;
      else {
        const float g = gy[(size_t)r * c + ch];
        s += g;
        s2 += g * v;
      }
    }
  }
  sm[threadIdx.y][threadIdx.x] = s;
  if (MODE == 2) sm2[threadIdx.y][threadIdx.x] = s2;
  __syncthreads();
  if (threadIdx.y == 0 && ch < c) {
    for (int g = 1; g < 8; ++g) s += sm[g][threadIdx.x];
    part[(size_t)blockIdx.y * c + ch] = s;
    if (MODE == 2) {
      for (int g = 1; g < 8; ++g) s2 += sm2[g][threadIdx.x];
      part2[(size_t)blockIdx.y * c + ch] = s2;
    }
  }
}

// acc[b] = sum over the channels ch with bucket_of_channel[ch] == b (consecutive channels) and over
// the row blocks of part[rb][ch]; one thread per bucket, fixed order.
__global__ void colsum_finish_kernel(const float *__restrict__ part, int row_blocks, int c,
                                     const int32_t *__restrict__ bucket_of_channel, int n_bucket, float *__restrict__ acc) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_bucket) return;
  float s = 0.f;
  for (int ch = 0; ch < c; ++ch) {
    if (bucket_of_channel[ch] != b) continue;
    for (int rb = 0; rb < row_blocks; ++rb) s += part[(size_t)rb * c + ch];
  }
  acc[b] = s;
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

// ------------------------------------------------------------------ backward of the batch norm
// y = (x - mu) * r * w (+ b), r = (v + eps)^-1/2, v = mean over rows of the squared field norm.
// With A_f = sum over rows and components of gy * (x - mu) and G_s = sum over rows of gy:
//   d_w[f] = r A_f,  d_b[s] = G_s,
//   training:  gx = r w gy - (w r^3 A_f / N) (x - mu) - [scalars] (r w G_s / N)
//   eval:      gx = r w gy
// Per channel: ks = r w, ka = w r^3 A / N (0 in eval mode), kg = r w G / N (scalars in training mode).
__global__ void bn_bwd_coef_kernel(const float *__restrict__ A, const float *__restrict__ G, const float *__restrict__ var,
                                   const float *__restrict__ weight, const int32_t *__restrict__ field_of_channel,
                                   const int32_t *__restrict__ scalar_of_channel, int c, int n_field, int n, float eps,
                                   int training, float *__restrict__ ks, float *__restrict__ ka, float *__restrict__ kg,
                                   float *__restrict__ d_weight, float *__restrict__ d_bias, int n_scalar) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < c) {
    const int f = field_of_channel[i], s = scalar_of_channel[i];
    const float r = 1.0f / sqrtf(var[f] + eps), w = weight ? weight[f] : 1.f;
    ks[i] = r * w;
    ka[i] = training ? w * r * r * r * A[f] / (float)n : 0.f;
    kg[i] = (training && s >= 0) ? r * w * G[s] / (float)n : 0.f;
  }
  if (i < n_field && d_weight) d_weight[i] = A[i] / sqrtf(var[i] + eps);
  if (i < n_scalar && d_bias) d_bias[i] = G[i];
}

__global__ void bn_bwd_apply_kernel(const float *__restrict__ x, const float *__restrict__ gy, long long total, int c,
                                    const float *__restrict__ chan_mean, const float *__restrict__ ks,
                                    const float *__restrict__ ka, const float *__restrict__ kg, float *__restrict__ gx) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int ch = (int)(t % c);
  gx[t] = ks[ch] * gy[t] - ka[ch] * (x[t] - chan_mean[ch]) - kg[ch];
}

// ------------------------------------------------------------- backward of the gated activation
// x [n, c_total] = [Rs channels | gate scalars], gy [n, c_out] -> gx [n, c_total].
//   copy channel: gx = gy; scalar channel: gx = gy * act'(x); gated channel: gx = gy * act(gate);
//   gate scalar j: gx = act'(x_gate) * sum over the channels ch of its field of gy[ch] * x[ch].
__device__ __forceinline__ float act_grad(float v, int kind) {
  if (kind == 1) return v > 0.f ? 1.f : 0.f;
  if (kind == 2) {
    const float sg = 1.0f / (1.0f + expf(-v));
    return sg * (1.f - sg);
  }
  return 1.f;
}

__global__ void gate_bwd_kernel(const float *__restrict__ x, const float *__restrict__ gy, long long total, int c_total,
                                int c_out, const int32_t *__restrict__ gate_of_channel,
                                const int32_t *__restrict__ field_start, const int32_t *__restrict__ field_len,
                                int scalar_act, int gate_act, float *__restrict__ gx) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const long long row = t / c_total;
  const int ch = (int)(t - row * c_total);
  const float *xr = x + row * c_total;
  const float *gr = gy + row * c_out;
  float v;
  if (ch < c_out) {
    const int g = gate_of_channel[ch];
    if (g == -1) v = gr[ch] * act_grad(xr[ch], scalar_act);
    else if (g >= 0) v = gr[ch] * apply_act(xr[c_out + g], gate_act);
    else v = gr[ch];
  } else {
    const int j = ch - c_out, s0 = field_start[j], len = field_len[j];
    float acc = 0.f;
    for (int q = 0; q < len; ++q) acc += gr[s0 + q] * xr[s0 + q];
    v = acc * act_grad(xr[ch], gate_act);
  }
  gx[t] = v;
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
    if (launch_bn_gate_rows<0, 4>(x, n, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act,
                                  scalar_bias, gate_bias, out, as_stream(stream))) {
      SSC_CHECK_LAUNCH("bn_gate_fwd");
      return SSC_OK;
    }
    { bn_gate_vec4_kernel<<<ceil_div(total4, 256), 256, 0, as_stream(stream)>>>(x, total4, groups, c_in_total, scale, shift,
                                                                            gate_of_channel, c_gate_base, scalar_act, gate_act,
                                                                            scalar_bias, gate_bias, out); note_launches(1); }
    SSC_CHECK_LAUNCH("bn_gate_fwd");
    return SSC_OK;
  }
  // channel counts that are not multiples of four: two channels per thread when everything is even,
  // else one (the row-block kernel still evaluates every gate once per row)
  const bool even = (c_out & 1) == 0 && (c_in_total & 1) == 0 && (((uintptr_t)x | (uintptr_t)out) & 7u) == 0;
  if (even ? launch_bn_gate_rows<0, 2>(x, n, (uint32_t)(c_out >> 1), c_in_total, scale, shift, gate_of_channel, c_gate_base,
                                       scalar_act, gate_act, scalar_bias, gate_bias, out, as_stream(stream))
           : launch_bn_gate_rows<0, 1>(x, n, (uint32_t)c_out, c_in_total, scale, shift, gate_of_channel, c_gate_base,
                                       scalar_act, gate_act, scalar_bias, gate_bias, out, as_stream(stream))) {
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
  if (precision == SSC_PREC_BF16
          ? launch_bn_gate_rows<2, 4>(x, n, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act,
                                   scalar_bias, gate_bias, out16, as_stream(stream))
          : launch_bn_gate_rows<1, 4>(x, n, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act,
                                   scalar_bias, gate_bias, out16, as_stream(stream))) {
    SSC_CHECK_LAUNCH("bn_gate_fwd16");
    return SSC_OK;
  }
  if (precision == SSC_PREC_BF16) {
    { bn_gate_vec4_out16_kernel<2><<<ceil_div(total4, 256), 256, 0, as_stream(stream)>>>(x, total4, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act, scalar_bias, gate_bias, (uint2 *)out16); note_launches(1); }
  } else {
    { bn_gate_vec4_out16_kernel<1><<<ceil_div(total4, 256), 256, 0, as_stream(stream)>>>(x, total4, groups, c_in_total, scale, shift, gate_of_channel, c_gate_base, scalar_act, gate_act, scalar_bias, gate_bias, (uint2 *)out16); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("bn_gate_fwd16");
  return SSC_OK;
}

// Row blocks of the column-sum kernels (each contributes one partial per channel).
static int bn_row_blocks(int n) {
  int rb = ceil_div(n, 8 * 64);
  return rb > 64 ? 64 : (rb < 1 ? 1 : rb);
}

extern "C" size_t ssc_bn_scratch_bytes(int n, int c) {
  if (n < 0 || c < 1) return 0;
  // two partial-sum planes [row_blocks, c], per-channel mean and three coefficient rows, two bucket rows
  return ((size_t)2 * bn_row_blocks(n) * c + (size_t)6 * c + 64) * sizeof(float);
}

// var must have room for n_field + c floats (the tail holds the per-channel means); scratch holds the
// partial sums: ssc_bn_scratch_bytes(n, c).
extern "C" int ssc_bn_stats(const float *x, int n, int c, const int32_t *field_of_channel,
                            const int32_t *scalar_of_channel, int n_field, int n_scalar, float *mean, float *var,
                            void *scratch, size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(n >= 1 && c >= 1 && n_field >= 1 && n_scalar >= 0, "bn_stats: bad sizes");
  SSC_REQUIRE(x && field_of_channel && scalar_of_channel && mean && var, "bn_stats: null pointer");
  SSC_REQUIRE(scratch && scratch_bytes >= ssc_bn_scratch_bytes(n, c), "bn_stats: scratch too small (ssc_bn_scratch_bytes)");
  cudaStream_t st = as_stream(stream);
  float *chan_mean = var + n_field;  // scratch tail, c floats
  float *part = (float *)scratch;
  const int rb = bn_row_blocks(n);
  dim3 block(32, 8), grid(ceil_div(c, 32), rb);
  { bn_colsum_kernel<0><<<grid, block, 0, st>>>(x, nullptr, n, c, nullptr, part, nullptr); note_launches(1); }
  if (n_scalar > 0) { colsum_finish_kernel<<<ceil_div(n_scalar, 64), 64, 0, st>>>(part, rb, c, scalar_of_channel, n_scalar, mean); note_launches(1); }
  { bn_chan_mean_kernel<<<ceil_div(c, 128), 128, 0, st>>>(mean, n, scalar_of_channel, c, chan_mean); note_launches(1); }
  if (n_scalar > 0) { bn_finish_var_kernel<<<ceil_div(n_scalar, 128), 128, 0, st>>>(mean, n_scalar, n); note_launches(1); }
  { bn_colsum_kernel<1><<<grid, block, 0, st>>>(x, nullptr, n, c, chan_mean, part, nullptr); note_launches(1); }
  { colsum_finish_kernel<<<ceil_div(n_field, 64), 64, 0, st>>>(part, rb, c, field_of_channel, n_field, var); note_launches(1); }
  { bn_finish_var_kernel<<<ceil_div(n_field, 128), 128, 0, st>>>(var, n_field, n); note_launches(1); }
  SSC_CHECK_LAUNCH("bn_stats");
  return SSC_OK;
}

extern "C" int ssc_bn_bwd(const float *x, const float *gy, int n, int c, const int32_t *field_of_channel,
                          const int32_t *scalar_of_channel, int n_field, int n_scalar, const float *mean,
                          const float *var, const float *weight, float eps, int training, float *gx,
                          float *d_weight, float *d_bias, void *scratch, size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(n >= 1 && c >= 1 && n_field >= 1 && n_scalar >= 0, "bn_bwd: bad sizes");
  SSC_REQUIRE(x && gy && field_of_channel && scalar_of_channel && var && gx && (n_scalar == 0 || mean), "bn_bwd: null pointer");
  SSC_REQUIRE(scratch && scratch_bytes >= ssc_bn_scratch_bytes(n, c), "bn_bwd: scratch too small (ssc_bn_scratch_bytes)");
  cudaStream_t st = as_stream(stream);
  const int rb = bn_row_blocks(n);
  float *part = (float *)scratch, *part2 = part + (size_t)rb * c;
  float *chan_mean = part2 + (size_t)rb * c, *ks = chan_mean + c, *ka = ks + c, *kg = ka + c;
  float *A = kg + c, *G = A + c;     // per field / per scalar (at most c entries each)
  { bn_chan_mean_kernel<<<ceil_div(c, 128), 128, 0, st>>>(mean, 1, scalar_of_channel, c, chan_mean); note_launches(1); }   // mean itself (n = 1)
  dim3 block(32, 8), grid(ceil_div(c, 32), rb);
  { bn_colsum_kernel<2><<<grid, block, 0, st>>>(x, gy, n, c, chan_mean, part, part2); note_launches(1); }
  if (n_scalar > 0) { colsum_finish_kernel<<<ceil_div(n_scalar, 64), 64, 0, st>>>(part, rb, c, scalar_of_channel, n_scalar, G); note_launches(1); }
  { colsum_finish_kernel<<<ceil_div(n_field, 64), 64, 0, st>>>(part2, rb, c, field_of_channel, n_field, A); note_launches(1); }
  const int m = c > n_field ? c : n_field;
  { bn_bwd_coef_kernel<<<ceil_div(m, 128), 128, 0, st>>>(A, G, var, weight, field_of_channel, scalar_of_channel, c, n_field, n, eps,
                                                     training, ks, ka, kg, d_weight, d_bias, n_scalar); note_launches(1); }
  const long long total = (long long)n * c;
  { bn_bwd_apply_kernel<<<ceil_div(total, 256), 256, 0, st>>>(x, gy, total, c, chan_mean, ks, ka, kg, gx); note_launches(1); }
  SSC_CHECK_LAUNCH("bn_bwd");
  return SSC_OK;
}

extern "C" int ssc_gate_bwd(const float *x, const float *gy, int n, int c_total, int c_out,
                            const int32_t *gate_of_channel, const int32_t *field_start, const int32_t *field_len,
                            int scalar_act, int gate_act, float *gx, void *stream) {
  SSC_REQUIRE(n >= 0 && c_total >= 1 && c_out >= 1 && c_out <= c_total, "gate_bwd: bad sizes");
  if (n == 0) return SSC_OK;
  SSC_REQUIRE(x && gy && gx && gate_of_channel && (c_total == c_out || (field_start && field_len)), "gate_bwd: null pointer");
  const long long total = (long long)n * c_total;
  { gate_bwd_kernel<<<ceil_div(total, 256), 256, 0, as_stream(stream)>>>(x, gy, total, c_total, c_out, gate_of_channel, field_start,
                                                                      field_len, scalar_act, gate_act, gx); note_launches(1); }
  SSC_CHECK_LAUNCH("gate_bwd");
  return SSC_OK;
}
