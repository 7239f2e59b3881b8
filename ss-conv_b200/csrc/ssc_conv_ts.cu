// Output-stationary gather-GEMM with the gathered operand in TENSOR MEMORY (tcgen05, sm_100a).
//
// Same contract as the shared-memory-operand kernel of ssc_conv_tc.cu (one CTA = 128 output
// rows, accumulators resident in TMEM over all kernel offsets, every output row written once),
// but the A operand never touches shared memory:
//   * four producer warps, thread <-> output row <-> TMEM lane.  For each step (kernel offset
//     with a neighbour in the tile) x (32-channel slab) a thread whose row has a neighbour
//     loads that feature row's 128-byte slab into registers (several steps ahead, in rotating
//     register sets), rounds it fp32 -> TF32 (round to nearest) and writes it with
//     tcgen05.st into one of a few 32-column A slots of tensor memory; rows without a
//     neighbour write zeros with the same instruction.  No swizzle, no shared-memory round
//     trip, no proxy fence.
//   * the filter slabs (pre-packed TF32 operand images) stream through a small shared-memory
//     ring, one bulk asynchronous copy per step, issued by a loader thread.
//   * tcgen05.mma reads A from tensor memory and B from shared memory.  When two accumulator
//     sets fit, even and odd steps accumulate into different sets, each issued by its own
//     thread (issuing is the serial bottleneck); the epilogue adds the sets.
//   * the tile's slice of the neighbour table is staged in shared memory once, so the row
//     loads of a step depend on no other global load.
// Every mbarrier wait is bounded (see ssc_conv_tc.cu).
#include "ssc_common.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

constexpr int TS_M = 128;
constexpr int TS_SLAB = 32;
constexpr int TS_THREADS = 224;  // 4 producer warps, 2 MMA warps, filter-loader warp
constexpr int TS_NBUF = 3;       // register sets of row slabs in flight per producer thread
constexpr int TS_MAX_B_STAGES = 8;

struct TsParams {
  int k_slabs, n_pad, n_tiles, tile_n, b_bytes;
  int n_acc;      // accumulator sets (1 or 2)
  int a_slots;    // 32-column A slots in tensor memory
  int a_col0;     // first column of the A slots
  int tmem_cols;  // allocation (power of two)
  int b_stages;
  int nbr_smem;   // bytes of the neighbour-table slice kept in shared memory (0: read it from global)
};

static bool ts_params(int c_in, int c_out, int K, TsParams &p) {
  p.k_slabs = (c_in + TS_SLAB - 1) / TS_SLAB;
  int n16 = (c_out + 15) / 16 * 16;
  p.n_tiles = (n16 + 255) / 256;
  p.tile_n = ((n16 + p.n_tiles - 1) / p.n_tiles + 15) / 16 * 16;
  p.n_pad = p.n_tiles * p.tile_n;
  if (p.n_pad > 384) return false;  // needs room for A slots beside the accumulators
  p.b_bytes = p.n_pad * 128;
  if (2 * p.n_pad + 3 * TS_SLAB <= 256) {
    p.n_acc = 2;
    p.tmem_cols = 256;
  } else {
    p.n_acc = 1;
    p.tmem_cols = p.n_pad + 2 * TS_SLAB <= 256 ? 256 : 512;
  }
  p.a_col0 = p.n_acc * p.n_pad;
  p.a_slots = (p.tmem_cols - p.a_col0) / TS_SLAB;
  if (p.a_slots > 8) p.a_slots = 8;
  int ctas = 512 / p.tmem_cols;
  p.nbr_smem = K <= 128 ? K * TS_M * 4 : 0;
  int budget = (227 * 1024) / ctas - 1024 - 2048 - p.nbr_smem;
  p.b_stages = budget / p.b_bytes;
  if (p.b_stages > TS_MAX_B_STAGES) p.b_stages = TS_MAX_B_STAGES;
  return p.a_slots >= 2 && p.b_stages >= 2;
}

__device__ __forceinline__ void mma_tf32_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      :
      : "r"(tmem_c), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

// Eight consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t *r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(TS_THREADS, 2)
conv_fwd_tf32_ts_kernel(const float *__restrict__ features, int c_in, const uint4 *__restrict__ packed, int K,
                        int c_out, const int32_t *__restrict__ nbr, int n_out, float *__restrict__ out,
                        int32_t *status, TsParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *ctrl = smem + (size_t)p.b_stages * p.b_bytes;
  uint64_t *fulla_bars = (uint64_t *)ctrl;                  // [8] A slot written by all 128 producer threads
  uint64_t *emptya_bars = (uint64_t *)(ctrl + 64);          // [8] MMAs reading the A slot retired
  uint64_t *fullb_bars = (uint64_t *)(ctrl + 128);          // [8] filter slab landed
  uint64_t *emptyb_bars = (uint64_t *)(ctrl + 192);         // [8] MMAs reading the filter slab retired
  uint64_t *done_bar = (uint64_t *)(ctrl + 256);
  uint32_t *tmem_slot = (uint32_t *)(ctrl + 264);
  volatile int *abort_flag = (volatile int *)(ctrl + 268);
  int *n_act_s = (int *)(ctrl + 272);
  uint8_t *act_flag = ctrl + 512;                           // [256]
  uint8_t *act_list = ctrl + 768;                           // [256]
  int32_t *nbr_s = (int32_t *)(ctrl + 1024);                // [K][128] when it fits
  const bool nbr_in_smem = p.nbr_smem > 0;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * TS_M;
  const int SA = p.a_slots, SB = p.b_stages;

  if (tid == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(smem_u32(fulla_bars + s), 128);
      mbar_init(smem_u32(emptya_bars + s), 1);
      mbar_init(smem_u32(fullb_bars + s), 1);
      mbar_init(smem_u32(emptyb_bars + s), 1);
    }
    mbar_init(smem_u32(done_bar), (uint32_t)p.n_acc);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else if (warp < 4) {
    // which kernel offsets touch this tile (and stage the tile's slice of the neighbour table):
    // four offsets per pass so that 16 loads are in flight per lane before the first ballot
    for (int k0 = warp * 4; k0 < K; k0 += 16) {
      int v[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          int r = m0 + q * 32 + lane;
          v[i][q] = (k0 + i < K && r < n_out) ? __ldg(nbr + (size_t)(k0 + i) * n_out + r) : -1;
        }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (k0 + i < K) {
          if (nbr_in_smem) {
#pragma unroll
            for (int q = 0; q < 4; ++q) nbr_s[(k0 + i) * TS_M + q * 32 + lane] = v[i][q];
          }
          bool any = (v[i][0] >= 0) | (v[i][1] >= 0) | (v[i][2] >= 0) | (v[i][3] >= 0);
          unsigned b = __ballot_sync(0xffffffffu, any);
          if (lane == 0) act_flag[k0 + i] = b != 0;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {
    int n = 0;
    for (int kappa = 0; kappa < K; ++kappa)
      if (act_flag[kappa]) act_list[n++] = (uint8_t)kappa;
    *n_act_s = n;
  }
  __syncthreads();
  const uint32_t tmem_base = *tmem_slot;
  const int n_act = *n_act_s;
  const int n_iter = n_act * p.k_slabs;

  if (warp < 4) {
    // ============================ producers: thread <-> output row <-> TMEM lane =============
    const int m = m0 + tid;
    const bool row_valid = m < n_out;
    const bool vec_ok = (c_in & 3) == 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)p.a_col0;
    float4 buf[TS_NBUF][8];
    bool has[TS_NBUF];

    auto fetch = [&](int j, float4 *dst, bool &present) {
      const int act = j / p.k_slabs, slab = j - act * p.k_slabs;
      const int kap = act_list[act];
      const int src = nbr_in_smem ? nbr_s[kap * TS_M + tid] : (row_valid ? __ldg(nbr + (size_t)kap * n_out + m) : -1);
      const int ch0 = slab * TS_SLAB;
      present = src >= 0;
      if (present) {
        const float *fp = features + (size_t)src * c_in + ch0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int ch = ch0 + c * 4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (vec_ok) {
            if (ch < c_in) v = __ldg((const float4 *)(fp + c * 4));
          } else {
            if (ch + 0 < c_in) v.x = __ldg(fp + c * 4 + 0);
            if (ch + 1 < c_in) v.y = __ldg(fp + c * 4 + 1);
            if (ch + 2 < c_in) v.z = __ldg(fp + c * 4 + 2);
            if (ch + 3 < c_in) v.w = __ldg(fp + c * 4 + 3);
          }
          dst[c] = v;
        }
      }
    };
    auto publish = [&](int j, const float4 *src_regs, bool present) -> bool {
      const int sa = j % SA, use = j / SA;
      if (use > 0) {
        if (!mbar_wait_warp(smem_u32(emptya_bars + sa), (uint32_t)((use - 1) & 1), abort_flag)) return false;
        tc_fence_after();
      }
      const uint32_t taddr = lane_addr + (uint32_t)(sa * TS_SLAB);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t r[8];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float4 v = present ? src_regs[g * 2 + e] : make_float4(0.f, 0.f, 0.f, 0.f);
          r[e * 4 + 0] = to_tf32(v.x);
          r[e * 4 + 1] = to_tf32(v.y);
          r[e * 4 + 2] = to_tf32(v.z);
          r[e * 4 + 3] = to_tf32(v.w);
        }
        tmem_st8(taddr + (uint32_t)(g * 8), r);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      mbar_arrive(smem_u32(fulla_bars + sa));
      return true;
    };

#pragma unroll
    for (int b = 0; b < TS_NBUF; ++b) {
      has[b] = false;
      if (b < n_iter) fetch(b, buf[b], has[b]);
    }
    bool alive = true;
    for (int j0 = 0; j0 < n_iter && alive; j0 += TS_NBUF) {
#pragma unroll
      for (int b = 0; b < TS_NBUF; ++b) {
        const int j = j0 + b;
        if (j < n_iter && alive) {
          alive = publish(j, buf[b], has[b]);
          alive = __all_sync(0xffffffffu, alive);  // tcgen05.st is warp-collective
          has[b] = false;
          if (alive && j + TS_NBUF < n_iter) fetch(j + TS_NBUF, buf[b], has[b]);
        }
      }
    }

    // ============================ epilogue =================================================
    bool ok = alive && !*abort_flag;
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_iter > 0) ok = mbar_wait_warp(smem_u32(done_bar), 0u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const int n_cols = (c_out + 15) & ~15;
    const bool two = p.n_acc == 2 && n_iter > 1;
    for (int c0 = 0; c0 < n_cols && c0 < p.n_pad; c0 += 16) {
      uint32_t r[16];
      if (ok && n_iter > 0) {
        uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
        tmem_ld16(taddr, r);
        if (two) {
          uint32_t r2[16];
          tmem_ld16(taddr + (uint32_t)p.n_pad, r2);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int q = 0; q < 16; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) + __uint_as_float(r2[q]));
        } else {
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) r[q] = 0u;
      }
      if (row_valid) {
        float *op = out + (size_t)m * c_out + c0;
        if ((c_out & 3) == 0) {
#pragma unroll
          for (int q = 0; q < 16; q += 4)
            if (c0 + q < c_out)
              *(float4 *)(op + q) = make_float4(__uint_as_float(r[q]), __uint_as_float(r[q + 1]),
                                                __uint_as_float(r[q + 2]), __uint_as_float(r[q + 3]));
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q)
            if (c0 + q < c_out) op[q] = __uint_as_float(r[q]);
        }
      }
    }
  } else if ((warp == 4 || warp == 5) && lane == 0 && (warp - 4) < p.n_acc) {
    // ============================ MMA issuers ===============================================
    // Issuing one tcgen05.mma occupies its thread for a couple of hundred cycles, so with two
    // accumulator sets two threads issue: thread e takes the steps t = e, e+2, ... and
    // accumulates them into set e (different A slots, filter slabs and TMEM columns, hence no
    // ordering between the two is needed).
    const int e = warp - 4, stride = p.n_acc;
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.tile_n >> 3) << 17) | ((uint32_t)(TS_M >> 4) << 24);
    const uint32_t b_lo0 = desc_lo(smem_u32(smem)), b_step = (uint32_t)p.b_bytes >> 4, n_step = (uint32_t)(p.tile_n * 128) >> 4;
    const uint32_t fulla0 = smem_u32(fulla_bars), fullb0 = smem_u32(fullb_bars);
    const uint32_t emptya0 = smem_u32(emptya_bars), emptyb0 = smem_u32(emptyb_bars);
    const uint32_t d0 = tmem_base + (uint32_t)(e * p.n_pad);
    const uint32_t a_base = tmem_base + (uint32_t)p.a_col0;
    for (int t = e; t < n_iter; t += stride) {
      const uint32_t sa = (uint32_t)(t % SA), sb = (uint32_t)(t % SB);
      if (!mbar_wait(fulla0 + sa * 8u, (uint32_t)((t / SA) & 1), abort_flag)) break;
      if (!mbar_wait(fullb0 + sb * 8u, (uint32_t)((t / SB) & 1), abort_flag)) break;
      tc_fence_after();
      const uint32_t a_col = a_base + sa * TS_SLAB, b_lo = b_lo0 + sb * b_step;
      const uint32_t fresh = t < stride ? 0u : 1u;  // the first step into an accumulator set overwrites it
      for (int nt = 0; nt < p.n_tiles; ++nt) {
        const uint32_t dn = d0 + (uint32_t)(nt * p.tile_n), bn = b_lo + (uint32_t)nt * n_step;
        mma_tf32_ts_lo(dn, a_col, bn, idesc, fresh);
        mma_tf32_ts_lo(dn, a_col + 8u, bn + 2u, idesc, 1u);
        mma_tf32_ts_lo(dn, a_col + 16u, bn + 4u, idesc, 1u);
        mma_tf32_ts_lo(dn, a_col + 24u, bn + 6u, idesc, 1u);
      }
      mma_commit(emptya0 + sa * 8u);
      mma_commit(emptyb0 + sb * 8u);
    }
    mma_commit(smem_u32(done_bar));
  } else if (warp == 6 && lane == 0) {
    // ============================ filter-slab loader ========================================
    const uint32_t smem_base = smem_u32(smem);
    for (int j = 0; j < n_iter; ++j) {
      const int sb = j % SB, use = j / SB;
      if (use > 0 && !mbar_wait(smem_u32(emptyb_bars + sb), (uint32_t)((use - 1) & 1), abort_flag)) break;
      const int act = j / p.k_slabs, slab = j - act * p.k_slabs;
      const uint4 *bsrc = packed + ((size_t)act_list[act] * p.k_slabs + slab) * (size_t)(p.n_pad * 8);
      const uint32_t bar = smem_u32(fullb_bars + sb);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)p.b_bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_base + (uint32_t)sb * (uint32_t)p.b_bytes),
                   "l"(bsrc), "r"((uint32_t)p.b_bytes), "r"(bar)
                   : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) atomicOr(status, 16);
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

// Returns SSC_OK, or -1 when the shape is not covered by this variant (caller falls back to
// the shared-memory-operand kernel).
int conv_fwd_tf32_ts(const float *features, int n_in, int c_in, const void *packed, int K, int c_out,
                     const int32_t *nbr, int n_out, float *out, int32_t *status, cudaStream_t st) {
  TsParams p;
  if (!ts_params(c_in, c_out, K, p)) return -1;
  size_t smem = (size_t)p.b_stages * p.b_bytes + 1024 + 1024 + p.nbr_smem;
  cudaError_t e = cudaFuncSetAttribute(conv_fwd_tf32_ts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd(tf32, tmem operand): smem attribute: %s", cudaGetErrorString(e));
  int grid = ceil_div(n_out, TS_M);
  { conv_fwd_tf32_ts_kernel<<<grid, TS_THREADS, smem, st>>>(features, c_in, (const uint4 *)packed, K, c_out, nbr, n_out,
                                                           out, status, p); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_tf32_ts");
  return SSC_OK;
}

}  // namespace ssc
