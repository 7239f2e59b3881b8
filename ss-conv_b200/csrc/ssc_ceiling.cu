// Measurement support: the rate at which this device takes fp32 scatter-add traffic.
//
// The pair-list convolution (ssc_conv_pairs.cu) adds every 128 x Cout accumulator tile to
// scattered output rows with red.global.add.v4.f32; those reductions are executed by the L2
// slices, whose rate -- not HBM, not the tensor pipe -- bounds that kernel.  This kernel issues
// nothing but such reductions, in the friendliest shape (eight neighbouring lanes add the 128
// contiguous bytes of one row; all warps of the grid walk the row list side by side, so the
// rows stay in L2), and the caller times it: bytes / time is the ceiling that the convolution's
// reduction traffic 4 P Cout can be compared with.
#include "ssc_common.cuh"

namespace ssc {

// LPR lanes share one row: an instruction adds LPR x 16 contiguous bytes to each of 32 / LPR rows.
template <int LPR>
__global__ void __launch_bounds__(256) scatter_add_rate_kernel(float *__restrict__ out, int row_floats,
                                                               const int32_t *__restrict__ rows, int n_idx, int steps) {
  const int lane = threadIdx.x & 31;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = (gridDim.x * blockDim.x) >> 5;
  constexpr int RPI = 32 / LPR;                         // rows per instruction
  const int sub = lane % LPR, grp = lane / LPR;
  for (int s = 0; s < steps; ++s) {
    // 32 list positions per warp and step
    const long long j0 = ((long long)s * n_warps + gwarp) * 32;
#pragma unroll
    for (int r0 = 0; r0 < 32; r0 += RPI) {
      const int row = __ldg(rows + (int)((j0 + r0 + grp) % n_idx));
      float *dst = out + (size_t)row * row_floats + sub * 4;
      for (int c = 0; c < row_floats; c += LPR * 4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %1, %1, %1};" ::"l"(dst + c), "f"(1.0f) : "memory");
    }
  }
}

}  // namespace ssc

using namespace ssc;

// Adds 1.0 to out[rows[j], :] for steps * (warps of the grid) * 32 list positions j (wrapping round
// the list); returns the bytes reduced through *bytes so that the caller can turn its own timing
// into a rate.  out [n_rows, row_floats] is scratch of the caller; every rows[j] < n_rows.
// lanes_per_row (1, 2, 4, 8): contiguous 16-byte pieces per row and instruction; warps_per_sm (1 .. 16):
// issuing warps.  (8, 16) measures the ceiling; the other settings show how the rate depends on the
// shape of a reduction instruction and on the number of warps that issue them.
extern "C" int ssc_scatter_add_rate(float *out, int row_floats, const int32_t *rows, int n_idx, int steps, int lanes_per_row,
                                    int warps_per_sm, unsigned long long *bytes, void *stream) {
  SSC_REQUIRE(out && rows && n_idx > 0 && steps > 0 && row_floats >= 32 && row_floats % 32 == 0 &&
                  ((uintptr_t)out & 15u) == 0,
              "scatter_add_rate: bad arguments (row_floats must be a multiple of 32, out 16-byte aligned)");
  SSC_REQUIRE((lanes_per_row == 1 || lanes_per_row == 2 || lanes_per_row == 4 || lanes_per_row == 8) && warps_per_sm >= 1 &&
                  warps_per_sm <= 16,
              "scatter_add_rate: lanes_per_row must be 1, 2, 4 or 8 and warps_per_sm 1..16");
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // one block per SM for up to 8 warps, two beyond
  const int blocks = warps_per_sm <= 8 ? sms : sms * 2, threads = (warps_per_sm <= 8 ? warps_per_sm : warps_per_sm / 2) * 32;
  cudaStream_t st = as_stream(stream);
  switch (lanes_per_row) {
    case 1: { scatter_add_rate_kernel<1><<<blocks, threads, 0, st>>>(out, row_floats, rows, n_idx, steps); note_launches(1); } break;
    case 2: { scatter_add_rate_kernel<2><<<blocks, threads, 0, st>>>(out, row_floats, rows, n_idx, steps); note_launches(1); } break;
    case 4: { scatter_add_rate_kernel<4><<<blocks, threads, 0, st>>>(out, row_floats, rows, n_idx, steps); note_launches(1); } break;
    default: { scatter_add_rate_kernel<8><<<blocks, threads, 0, st>>>(out, row_floats, rows, n_idx, steps); note_launches(1); } break;
  }
  SSC_CHECK_LAUNCH("scatter_add_rate");
  if (bytes) *bytes = (unsigned long long)blocks * (unsigned long long)(threads / 32) * 32ull * (unsigned long long)steps * (unsigned long long)row_floats * 4ull;
  return SSC_OK;
}
