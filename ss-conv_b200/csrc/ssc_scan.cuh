// Block-level scan helpers and the three-kernel exclusive scan used for ranking bitmap bits
// (popcount of each 32-bit word) and for CSR offsets (plain int32 counts).
#pragma once
#include "ssc_common.cuh"

namespace ssc {

__device__ __forceinline__ uint32_t block_reduce_sum(uint32_t v, uint32_t *smem) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  uint32_t r = 0;
  if (warp == 0) {
    r = lane < (blockDim.x >> 5) ? smem[lane] : 0;
    for (int o = 16; o > 0; o >>= 1) r += __shfl_down_sync(0xffffffffu, r, o);
  }
  return r;  // valid in thread 0
}

// Exclusive scan of one value per thread over a block of up to 1024 threads.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t *smem, uint32_t *total) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t incl = v;
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) smem[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < (blockDim.x >> 5) ? smem[lane] : 0;
    uint32_t wi = w;
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    smem[lane] = wi - w;           // exclusive warp offsets
    if (lane == 31) smem[32] = wi; // block total
  }
  __syncthreads();
  uint32_t res = smem[warp] + incl - v;
  if (total) *total = smem[32];
  __syncthreads();
  return res;
}

// 256 threads x 4 words per block.
template <bool POPC>
__global__ void popc_block_sums_kernel(const uint32_t *__restrict__ bitmap, long long n_words,
                                       uint32_t *block_sums) {
  __shared__ uint32_t smem[33];
  long long base = (long long)blockIdx.x * 1024 + threadIdx.x * 4;
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (base + i < n_words) s += POPC ? (uint32_t)__popc(bitmap[base + i]) : bitmap[base + i];
  uint32_t r = block_reduce_sum(s, smem);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = r;
}

// Single block: in-place exclusive scan of block_sums[0..n); writes the total to
// block_sums[n] and to the two int32 outputs.
static __global__ void scan_block_sums_kernel(uint32_t *block_sums, int n, int32_t *total_a, int32_t *total_b) {
  __shared__ uint32_t smem[33];
  uint32_t running = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    int i = base + threadIdx.x;
    uint32_t v = i < n ? block_sums[i] : 0;
    uint32_t tot;
    uint32_t ex = block_exclusive_scan(v, smem, &tot);
    if (i < n) block_sums[i] = running + ex;
    running += tot;
  }
  if (threadIdx.x == 0) {
    block_sums[n] = running;
    if (total_a) *total_a = (int32_t)running;
    if (total_b) *total_b = (int32_t)running;
  }
}

template <bool POPC>
__global__ void word_prefix_kernel(const uint32_t *__restrict__ bitmap, long long n_words,
                                   const uint32_t *__restrict__ block_sums, uint32_t *word_prefix) {
  __shared__ uint32_t smem[33];
  long long base = (long long)blockIdx.x * 1024 + threadIdx.x * 4;
  uint32_t c[4];
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    c[i] = (base + i < n_words) ? (POPC ? (uint32_t)__popc(bitmap[base + i]) : bitmap[base + i]) : 0;
    s += c[i];
  }
  uint32_t ex = block_exclusive_scan(s, smem, nullptr) + block_sums[blockIdx.x];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (base + i < n_words) word_prefix[base + i] = ex;
    ex += c[i];
  }
}


// Small inputs (up to kSingleScanMax values): the whole exclusive scan in ONE block of 1024
// threads, each thread owning a contiguous run of values — one launch instead of three when the
// three would each be pure launch latency.
constexpr long long kSingleScanMax = 1 << 13;
template <bool POPC>
__global__ void __launch_bounds__(1024)
single_block_scan_kernel(const uint32_t *values, int n, uint32_t *prefix, int32_t *total_a, int32_t *total_b) {
  // values and prefix may be the same array (in-place scan): every value is read before its slot is written
  __shared__ uint32_t smem[33];
  const int per = (n + 1023) / 1024;          // values per thread (<= 8)
  const int begin = threadIdx.x * per, end = min(n, begin + per);
  uint32_t s = 0;
  for (int i = begin; i < end; ++i) s += POPC ? (uint32_t)__popc(values[i]) : values[i];
  uint32_t tot;
  uint32_t run = block_exclusive_scan(s, smem, &tot);
  for (int i = begin; i < end; ++i) {
    const uint32_t v = POPC ? (uint32_t)__popc(values[i]) : values[i];
    prefix[i] = run;
    run += v;
  }
  if (threadIdx.x == 0) {
    if (total_a) *total_a = (int32_t)tot;
    if (total_b) *total_b = (int32_t)tot;
  }
}

// Exclusive scan of n values (popcounts of words if POPC, else the words themselves):
// prefix[i] = sum of values before i; the grand total goes to total_a / total_b (may be NULL).
// block_sums needs ceil(n/1024)+1 entries.
template <bool POPC>
static inline int exclusive_scan_u32(const uint32_t *values, long long n, uint32_t *prefix, uint32_t *block_sums,
                                     int32_t *total_a, int32_t *total_b, cudaStream_t st) {
  if (n >= 1 && n <= kSingleScanMax) {
    { single_block_scan_kernel<POPC><<<1, 1024, 0, st>>>(values, (int)n, prefix, total_a, total_b); note_launches(1); }
    cudaError_t e1 = cudaGetLastError();
    if (e1 != cudaSuccess) return fail(SSC_ERR_CUDA, "exclusive_scan: %s", cudaGetErrorString(e1));
    return 0;
  }
  int blocks = (int)((n + 1023) / 1024);
  if (blocks < 1) blocks = 1;
  { popc_block_sums_kernel<POPC><<<blocks, 256, 0, st>>>(values, n, block_sums); note_launches(1); }
  { scan_block_sums_kernel<<<1, 1024, 0, st>>>(block_sums, blocks, total_a, total_b); note_launches(1); }
  { word_prefix_kernel<POPC><<<blocks, 256, 0, st>>>(values, n, block_sums, prefix); note_launches(1); }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "exclusive_scan: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace ssc
