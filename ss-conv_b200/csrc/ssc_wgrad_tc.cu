// Filter gradient of the sparse convolution on the tensor cores (tcgen05, TF32 operands).
//
//   dW[kappa][ci][co] = sum over output rows o with a neighbour i = nbr[kappa][o]:  x[i][ci] * dy[o][co]
//
// The (output row, input row) pairs of every kernel offset are first compacted into lists (a
// bitmap of the neighbour table, a popcount scan, a scatter: ascending output row inside an
// offset, so the lists - and the sums below - are repeatable); rows without a neighbour, more
// than half of the table of a strided convolution, then cost nothing.
// One CTA owns one kernel offset, one range of that offset's pair list and one block of 128 output
// channels, and accumulates D[co][ci] (M = 128 rows = output channels, N = input channels) in
// tensor memory over chunks of 32 pairs (the K dimension of the MMA).  Both operands have to be K-major,
// i.e. transposed with respect to how the rows lie in memory, so the producer warps transpose on
// the way into shared memory: lane = row of the chunk; for every channel the 32 lanes store 32
// consecutive K elements of that channel's operand row (one conflict-free 128-byte store, in the
// 128-byte-swizzled layout), rounded to TF32; the lanes past the end of the list store zeros.  Operand
// rows of channels past c_out / c_in are zeroed once and never touched again.
//
// warps 0-3: producers (warp w prepares chunks w, w+4, ...), then the epilogue (each lane owns one
// output channel and writes its row of D into the partial tile, transposed back to [ci][co]);
// warp 4: tensor-memory allocation and the MMA-issuing thread.  The partial tiles of the row
// ranges are added by wgrad_reduce_kernel in a fixed order (bitwise repeatable).
// Every wait is bounded (status bit 16 on expiry).
#include "ssc_conv_internal.cuh"
#include "ssc_scan.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

constexpr int WT_M = 128;          // output channels per CTA
constexpr int WT_K = 32;           // output rows per chunk
constexpr int WT_STAGES = 4;
constexpr int WT_A_BYTES = WT_M * 128;
constexpr int WT_THREADS = 160;

// One warp per 32 output rows of one kernel offset: which of them have a neighbour.
__global__ void pair_bitmap_kernel(const int32_t *__restrict__ nbr, int K, int n_out, int words_per_row,
                                   uint32_t *__restrict__ bitmap) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (gw >= (long long)K * words_per_row) return;
  const int kappa = (int)(gw / words_per_row), r = (int)(gw % words_per_row) * 32 + (int)(threadIdx.x & 31);
  const bool have = r < n_out && __ldg(nbr + (size_t)kappa * n_out + r) >= 0;
  const unsigned m = __ballot_sync(0xffffffffu, have);
  if ((threadIdx.x & 31) == 0) bitmap[gw] = m;
}
// prefix[w] = number of pairs before word w (over all offsets): the lists of the offsets follow one
// another in pair_out / pair_in, starts[kappa] is where the list of offset kappa begins.
__global__ void pair_scatter_kernel(const int32_t *__restrict__ nbr, int K, int n_out, int words_per_row,
                                    const uint32_t *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                                    int32_t *__restrict__ pair_out, int32_t *__restrict__ pair_in, int32_t *__restrict__ starts) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (gw >= (long long)K * words_per_row) return;
  const int lane = threadIdx.x & 31;
  const int kappa = (int)(gw / words_per_row), w = (int)(gw % words_per_row), r = w * 32 + lane;
  const uint32_t m = bitmap[gw], base = prefix[gw];
  if (w == 0 && lane == 0) starts[kappa] = (int32_t)base;
  if ((m >> lane) & 1u) {
    const uint32_t pos = base + (uint32_t)__popc(m & ((1u << lane) - 1u));
    pair_out[pos] = r;
    pair_in[pos] = __ldg(nbr + (size_t)kappa * n_out + r);
  }
}

__device__ __forceinline__ uint32_t wt_off(int row, int k) {  // byte offset of element (row, k) of a K-major SW128 tile
  return (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u + ((((uint32_t)k >> 2) ^ (uint32_t)(row & 7)) << 4) +
         ((uint32_t)k & 3u) * 4u;
}

__global__ void __launch_bounds__(WT_THREADS)
conv_wgrad_tc_kernel(const float *__restrict__ features, int c_in, const float *__restrict__ out_grad, int c_out,
                     const int32_t *__restrict__ pair_out, const int32_t *__restrict__ pair_in,
                     const int32_t *__restrict__ starts, int n_pad, uint32_t tmem_cols, float *__restrict__ partial,
                     int32_t *status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int b_bytes = n_pad * 128;
  const int stage_bytes = WT_A_BYTES + b_bytes;
  uint8_t *ctrl = smem + (size_t)WT_STAGES * stage_bytes;
  uint64_t *full_bars = (uint64_t *)ctrl;                  // [WT_STAGES]
  uint64_t *empty_bars = full_bars + WT_STAGES;            // [WT_STAGES]
  uint64_t *done_bar = empty_bars + WT_STAGES;
  uint32_t *tmem_slot = (uint32_t *)(done_bar + 1);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kappa = blockIdx.y, co0 = blockIdx.z * WT_M;
  // this CTA's share of the offset's pair list: equal ranges of whole chunks
  const int list0 = starts[kappa], n_pairs = starts[kappa + 1] - list0;
  const int rows_per_split = (((n_pairs + (int)gridDim.x - 1) / (int)gridDim.x + WT_K - 1) / WT_K) * WT_K;
  const int r_begin = split * rows_per_split;
  const int r_end = min(n_pairs, r_begin + rows_per_split);
  const int n_chunks = r_end > r_begin ? (r_end - r_begin + WT_K - 1) / WT_K : 0;

  if (tid == 0) {
    for (int s = 0; s < WT_STAGES; ++s) {
      mbar_init(smem_u32(full_bars + s), 32);
      mbar_init(smem_u32(empty_bars + s), 1);
    }
    mbar_init(smem_u32(done_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    // operand rows of channels that do not exist stay zero for the whole kernel
    for (int s = 0; s < WT_STAGES; ++s) {
      uint4 *st = (uint4 *)(smem + (size_t)s * stage_bytes);
      for (int i = tid; i < stage_bytes / 16; i += 128) st[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);
  const int m_cnt = min(WT_M, c_out - co0);   // output channels of this CTA

  if (warp < 4) {
    // ====================================== producers ========================================
    // Chunk ch uses ring slot ch % WT_STAGES; with as many producer warps as slots, warp w always
    // works on slot w.
    uint32_t par = 0;
    const int slot = warp;
    uint8_t *a_tile = smem + (size_t)slot * stage_bytes;
    uint8_t *b_tile = a_tile + WT_A_BYTES;
    const bool vec = ((c_in | c_out) & 3) == 0 && (((uintptr_t)features | (uintptr_t)out_grad) & 15u) == 0;
    for (int ch = warp; ch < n_chunks; ch += 4) {
      const int j = r_begin + ch * WT_K + lane;   // position in the offset's pair list
      const int r = j < r_end ? __ldg(pair_out + list0 + j) : 0;
      const int src = j < r_end ? __ldg(pair_in + list0 + j) : -1;
      if (ch >= WT_STAGES) {
        if (!mbar_wait_warp(smem_u32(empty_bars + slot), par ^ 1u, abort_flag)) break;
        tc_fence_after();
      }
      const bool valid = src >= 0;
      // A operand: dy^T (tile row = output channel), B operand: x^T (tile row = input channel);
      // K index = this lane's row of the chunk
      const float *gy = out_grad + (size_t)(valid ? r : 0) * c_out + co0;
      const float *gx = features + (size_t)(valid ? src : 0) * c_in;
      if (vec) {
        // 32 channels at a time: eight independent 16-byte loads in flight, then 32 transposed stores
        auto transpose_in = [&](const float *g, int n_ch, uint8_t *tile) {
          for (int c0 = 0; c0 < n_ch; c0 += 32) {
            float4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
              v[q] = (valid && c0 + q * 4 < n_ch) ? __ldg((const float4 *)(g + c0 + q * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int c = c0 + q * 4;
              if (c < n_ch) {
                *(uint32_t *)(tile + wt_off(c + 0, lane)) = to_tf32(v[q].x);
                *(uint32_t *)(tile + wt_off(c + 1, lane)) = to_tf32(v[q].y);
                *(uint32_t *)(tile + wt_off(c + 2, lane)) = to_tf32(v[q].z);
                *(uint32_t *)(tile + wt_off(c + 3, lane)) = to_tf32(v[q].w);
              }
            }
          }
        };
        transpose_in(gy, m_cnt, a_tile);
        transpose_in(gx, c_in, b_tile);
      } else {
        for (int c = 0; c < m_cnt; ++c) *(uint32_t *)(a_tile + wt_off(c, lane)) = to_tf32(valid ? __ldg(gy + c) : 0.f);
        for (int c = 0; c < c_in; ++c) *(uint32_t *)(b_tile + wt_off(c, lane)) = to_tf32(valid ? __ldg(gx + c) : 0.f);
      }
      fence_async_smem();
      mbar_arrive(smem_u32(full_bars + slot));
      par ^= 1u;
    }
  } else if (lane == 0) {
    // ====================================== MMA issuer =======================================
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n_pad >> 3) << 17) | ((uint32_t)(WT_M >> 4) << 24);
    uint32_t par = 0;
    for (int ch = 0; ch < n_chunks; ++ch) {
      const uint32_t s = (uint32_t)(ch % WT_STAGES);
      if (!mbar_wait(smem_u32(full_bars + s), par, abort_flag)) break;
      tc_fence_after();
      const uint32_t a_lo = desc_lo(smem_base + s * (uint32_t)stage_bytes);
      const uint32_t b_lo = desc_lo(smem_base + s * (uint32_t)stage_bytes + WT_A_BYTES);
      mma_tf32_ss(tmem_base, a_lo, b_lo, idesc, ch > 0 ? 1u : 0u);
      mma_tf32_ss(tmem_base, a_lo + 2u, b_lo + 2u, idesc, 1u);
      mma_tf32_ss(tmem_base, a_lo + 4u, b_lo + 4u, idesc, 1u);
      mma_tf32_ss(tmem_base, a_lo + 6u, b_lo + 6u, idesc, 1u);
      mma_commit(smem_u32(empty_bars + s));
      if (s == WT_STAGES - 1) par ^= 1u;
    }
    mma_commit(smem_u32(done_bar));
  }

  // ====================================== epilogue ===========================================
  if (warp < 4) {
    __syncwarp();
    bool ok = !*abort_flag;
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_chunks > 0) ok = mbar_wait_warp(smem_u32(done_bar), 0u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const int co = co0 + warp * 32 + lane;
    float *dst = partial + ((size_t)split * gridDim.y + kappa) * (size_t)c_in * c_out;
    for (int c0 = 0; c0 < n_pad; c0 += 16) {
      uint32_t v[16];
      if (ok && n_chunks > 0) {
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) v[q] = 0u;
      }
      if (co < c_out) {
#pragma unroll
        for (int q = 0; q < 16; ++q)
          if (c0 + q < c_in) dst[(size_t)(c0 + q) * c_out + co] = __uint_as_float(v[q]);  // lanes = consecutive co: coalesced
      }
    }
  }
  // a wait gave up: what was issued still arrives on done_bar (committed on every path); let it retire
  if (warp == 4 && lane == 0 && *abort_flag && n_chunks > 0) mbar_wait_drain(smem_u32(done_bar), 0u);
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) atomicOr(status, 16);
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

size_t pair_lists_bytes(int K, int n_out) {
  const size_t wpr = (size_t)ceil_div(n_out > 0 ? n_out : 1, 32), words = (size_t)K * wpr;
  auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
  return 2 * al(words * 4) + al((words / 1024 + 2) * 4) + 2 * al((size_t)K * n_out * 4) + al((size_t)(K + 1) * 4);
}
size_t conv_wgrad_tc_list_bytes(int K, int n_out) { return pair_lists_bytes(K, n_out); }

namespace {
struct ListPlan {
  uint32_t *bitmap, *prefix, *block_sums;
  int32_t *pair_out, *pair_in, *starts;
  int wpr;
  long long words;
};
ListPlan plan_lists(void *lists, int K, int n_out) {
  ListPlan p;
  p.wpr = ceil_div(n_out > 0 ? n_out : 1, 32);
  p.words = (long long)K * p.wpr;
  auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
  uint8_t *sp = (uint8_t *)lists;
  p.bitmap = (uint32_t *)sp;
  sp += al((size_t)p.words * 4);
  p.prefix = (uint32_t *)sp;
  sp += al((size_t)p.words * 4);
  p.block_sums = (uint32_t *)sp;
  sp += al(((size_t)p.words / 1024 + 2) * 4);
  p.pair_out = (int32_t *)sp;
  sp += al((size_t)K * n_out * 4);
  p.pair_in = (int32_t *)sp;
  sp += al((size_t)K * n_out * 4);
  p.starts = (int32_t *)sp;
  return p;
}
}  // namespace

PairLists pair_lists_view(void *lists, int K, int n_out) {
  const ListPlan p = plan_lists(lists, K, n_out);
  return PairLists{p.pair_out, p.pair_in, p.starts};
}

// bitmap of the table, popcount scan, scatter: three small launches
int pair_lists_build(const int32_t *nbr, int K, int n_out, void *lists, PairLists *out, cudaStream_t st) {
  const ListPlan p = plan_lists(lists, K, n_out);
  { pair_bitmap_kernel<<<ceil_div(p.words * 32, 256), 256, 0, st>>>(nbr, K, n_out, p.wpr, p.bitmap); note_launches(1); }
  SSC_CHECK_LAUNCH("pair_bitmap");
  int rc = exclusive_scan_u32<true>(p.bitmap, p.words, p.prefix, p.block_sums, p.starts + K, nullptr, st);
  if (rc != 0) return rc;
  { pair_scatter_kernel<<<ceil_div(p.words * 32, 256), 256, 0, st>>>(nbr, K, n_out, p.wpr, p.bitmap, p.prefix, p.pair_out, p.pair_in, p.starts); note_launches(1); }
  SSC_CHECK_LAUNCH("pair_scatter");
  if (out) *out = PairLists{p.pair_out, p.pair_in, p.starts};
  return SSC_OK;
}

// returns -1 when the shape is not covered (the caller then uses the CUDA-core kernel)
int conv_wgrad_tc(const float *features, int c_in, const float *out_grad, int c_out, const int32_t *nbr, int K, int n_out,
                  int max_splits, int *splits_used, float *partial, void *lists, int32_t *status, cudaStream_t st) {
  const int n_pad = (c_in + 15) & ~15;
  if (n_pad > 256) return -1;
  // as many ranges per offset as fit one wave of two resident CTAs per SM (never more than the scratch holds)
  const int sms = sm_count();
  int splits = (2 * sms) / (K * ceil_div(c_out, WT_M));
  if (splits > max_splits) splits = max_splits;
  const int most = ceil_div(n_out, WT_K);   // a range is at least one chunk
  if (splits > most) splits = most;
  if (splits < 1) splits = 1;
  *splits_used = splits;
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < n_pad) tmem_cols <<= 1;
  const size_t smem = (size_t)WT_STAGES * (WT_A_BYTES + n_pad * 128) + 1024 + 256;
  if (smem > 227 * 1024) return -1;
  PairLists pl;
  int rc = pair_lists_build(nbr, K, n_out, lists, &pl, st);
  if (rc != SSC_OK) return rc;
  cudaError_t e = cudaFuncSetAttribute(conv_wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_wgrad(tf32): smem attribute: %s", cudaGetErrorString(e));
  dim3 grid(splits, K, ceil_div(c_out, WT_M));
  { conv_wgrad_tc_kernel<<<grid, WT_THREADS, smem, st>>>(features, c_in, out_grad, c_out, pl.pair_out, pl.pair_in, pl.starts, n_pad,
                                                      tmem_cols, partial, status); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_wgrad_tc");
  return SSC_OK;
}

}  // namespace ssc
