// Persistent gather-GEMM, one CTA per SM, several row tiles per pass sharing every filter slab.
//
// The one-tile-per-CTA kernel (ssc_conv_tc.cu) fetches each filter slab once per 128-row tile and
// keeps only two operand slots per CTA.  Here a CTA owns a contiguous run of row tiles and works
// through it in passes of T tiles whose accumulators sit side by side in one half of tensor
// memory; inside a pass the loop order is  kernel offset > 32-channel slab > tile,  so a filter
// slab is fetched once per pass, and all the shared memory that the co-resident CTAs of the other
// kernel spend on copies of the filter slab becomes gathered-operand slots (a ring of up to 12).
//
//   producer warps   : a stage = (offset, slab, tile); stages are numbered in loop order and dealt
//                      round-robin to the warps.  A warp claims ring slot (stage % slots), looks up
//                      the 128 neighbour rows (lane = row, prefetched one stage ahead), writes the
//                      stage's tag and row mask, pulls the present rows of the staged TF32 image
//                      with cp.async.cg straight into the swizzled operand layout and arrives on
//                      the slot's barrier.
//   1 filter warp    : walks the (offset, slab) groups of the pass in the same order and keeps a
//                      small ring of filter slabs filled with bulk copies.
//   T MMA threads    : one per tile of the pass (a single issuing thread is the serial bottleneck
//                      of such a pipeline: each barrier round trip and each tcgen05 instruction
//                      costs it some hundred cycles).  Thread t walks the groups in order, takes
//                      the stage of tile t in each, switches rows without a neighbour off with the
//                      disable-output-lane mask, and its commits release operand and filter slots.
//   4 epilogue warps : drain the finished half of tensor memory while the next pass runs in the
//                      other half, clear it and hand it back.
//
// Needs the staged (TF32-rounded) feature image.  Every wait is bounded; on expiry the waiting
// thread raises the CTA's abort flag, every role leaves its loop at its next wait, the kernel
// releases its tensor memory and reports through `status`.
#include <stdlib.h>

#include "ssc_common.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

bool tc_operand_layout(int c_in, int c_out, int *k_slabs, int *n_pad, int *tile_n, int *n_tiles);

constexpr int WD_M = 128;
constexpr int WD_A_BYTES = WD_M * 128;
constexpr int WD_MAX_A = 12;
constexpr int WD_MAX_B = 4;
constexpr int WD_MAX_T = 4;
constexpr int WD_MAX_PROD = 12;                    // producer warps (one stage in flight each)
constexpr int WD_MAX_THREADS = (4 + WD_MAX_PROD + WD_MAX_T + 1) * 32;  // warps: 4 epilogue, the producers, T x MMA, filters
constexpr int WD_MAX_K = 512;                      // kernel volume the per-pass activity table holds
constexpr int WD_CTRL_BYTES = 2048;                // barriers, tags, masks, two activity tables
constexpr uint32_t WD_TMEM_COLS = 512;

struct WideParams {
  int k_slabs, n_pad, b_bytes;
  int a_slots, b_slots, n_prod;
  int sps;       // 32-channel slabs per stage (1 or 2): one barrier round trip of an MMA thread covers them all
  int k_groups;  // ceil(k_slabs / sps)
  int slot_bytes;  // sps * WD_A_BYTES
  int T;        // tiles per pass
};

__device__ __forceinline__ void wd_cp16(uint32_t dst, const void *src, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__global__ void __launch_bounds__(WD_MAX_THREADS, 1)
conv_fwd_tf32_wide_kernel(const float *__restrict__ staged, int c_in, const uint4 *__restrict__ packed, int K, int c_out,
                          const int32_t *__restrict__ nbr, int n_out, float *__restrict__ out, int32_t *status,
                          WideParams p, const int32_t *__restrict__ n_out_dev) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *b_ring = smem + (size_t)p.a_slots * p.slot_bytes;
  uint8_t *ctrl = b_ring + (size_t)p.b_slots * p.sps * p.b_bytes;
  uint64_t *full_a = (uint64_t *)ctrl;                 // [WD_MAX_A]
  uint64_t *empty_a = full_a + WD_MAX_A;               // [WD_MAX_A]
  uint64_t *full_b = empty_a + WD_MAX_A;               // [WD_MAX_B]
  uint64_t *empty_b = full_b + WD_MAX_B;               // [WD_MAX_B]
  uint64_t *acc_full = empty_b + WD_MAX_B;             // [2]
  uint64_t *acc_empty = acc_full + 2;                  // [2]
  uint64_t *act_ready = acc_empty + 2;                 // activity table of the pass written
  uint64_t *act_free = act_ready + 1;                  // ... and no longer read
  uint32_t *masks = (uint32_t *)(ctrl + 320);          // [WD_MAX_A][4] rows WITHOUT a neighbour (16-byte aligned)
  uint32_t *slot_seq = masks + WD_MAX_A * 4;           // [WD_MAX_A] number of the stage that the slot holds
  uint32_t *tmem_slot = slot_seq + WD_MAX_A;
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  uint8_t *act = (uint8_t *)(tmem_slot + 2);           // [WD_MAX_K] per offset: which tiles of the pass it touches

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rows = live_rows(n_out, n_out_dev);
  const int total_tiles = (n_rows + WD_M - 1) / WD_M;
  const int base = total_tiles / (int)gridDim.x, extra = total_tiles % (int)gridDim.x;
  const int my_tiles = base + ((int)blockIdx.x < extra ? 1 : 0);
  const int first_tile = (int)blockIdx.x * base + min((int)blockIdx.x, extra);
  const int n_pass = (my_tiles + p.T - 1) / p.T;
  if (my_tiles == 0) return;

  if (tid == 0) {
    for (int s = 0; s < p.a_slots; ++s) {
      mbar_init(smem_u32(full_a + s), 32 * p.sps);  // one warp per slab of the stage
      mbar_init(smem_u32(empty_a + s), 1);
    }
    for (int s = 0; s < p.b_slots; ++s) {
      mbar_init(smem_u32(full_b + s), 1);
      mbar_init(smem_u32(empty_b + s), p.T);  // every MMA thread passes every group
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(smem_u32(acc_full + h), p.T);
      mbar_init(smem_u32(acc_empty + h), 4);
    }
    mbar_init(smem_u32(act_ready), p.n_prod);
    mbar_init(smem_u32(act_free), p.n_prod + 1 + p.T);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4 + p.n_prod) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(WD_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t b_base = smem_u32(b_ring);
  const int acc_cols = p.T * p.n_pad;  // columns of one half in use

  if (warp < 4) {
    // ====================================== epilogue ========================================
    // both halves start as zero: every MMA accumulates under a row mask
    for (int h = 0; h < 2; ++h)
      for (int c0 = 0; c0 < acc_cols; c0 += 16) {
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(h * 256 + c0);
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr),
                     "r"(0u)
                     : "memory");
      }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(smem_u32(acc_empty + 0));
      mbar_arrive(smem_u32(acc_empty + 1));
    }
    const int n_cols = (c_out + 15) & ~15;
    for (int pass = 0; pass < n_pass; ++pass) {
      const uint32_t half = (uint32_t)(pass & 1), use = (uint32_t)(pass >> 1);
      if (!mbar_wait_warp_backoff(smem_u32(acc_full + half), use & 1u, abort_flag, 400)) break;
      tc_fence_after();
      const int t_cnt = min(p.T, my_tiles - pass * p.T);
      for (int t = 0; t < p.T; ++t) {
        const int m = (first_tile + pass * p.T + t) * WD_M + warp * 32 + lane;
        for (int c0 = 0; c0 < n_cols; c0 += 16) {
          const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + half * 256u + (uint32_t)(t * p.n_pad + c0);
          if (t < t_cnt) {
            uint32_t r[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (m < n_rows) {
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
            // clear what was read so that the half can be accumulated into again
            asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr),
                         "r"(0u)
                         : "memory");
          }
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_empty + half));
    }
  } else if (warp < 4 + p.n_prod) {
    // ====================================== producers =======================================
    const int pw = warp - 4;
    const int slot_id = pw % p.a_slots, part = pw / p.a_slots;  // this warp fills slab `part` of the stages in slot `slot_id`
    uint32_t base_seq = 0;  // number of the pass's first stage: identical in every producer warp
    // which offsets touch which tiles of a pass (this warp's share of the offsets)
    auto scan_pass = [&](int pass) {
      const int t_cnt = min(p.T, my_tiles - pass * p.T);
      const int row0 = (first_tile + pass * p.T) * WD_M;
      uint8_t *dst = act + (pass & 1) * WD_MAX_K;
      for (int kappa = pw; kappa < K; kappa += p.n_prod) {
        const int32_t *src = nbr + (size_t)kappa * n_out;
        uint32_t m = 0;
        int v[WD_MAX_T];  // every load of the offset in flight before the first is looked at
#pragma unroll
        for (int t = 0; t < WD_MAX_T; ++t) {
          v[t] = -1;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int r = row0 + t * WD_M + q * 32 + lane;
            v[t] &= (t < t_cnt && r < n_rows) ? __ldg(src + r) : -1;
          }
        }
#pragma unroll
        for (int t = 0; t < WD_MAX_T; ++t)  // a row has a neighbour when its index has no sign bit
          if (__ballot_sync(0xffffffffu, v[t] >= 0)) m |= 1u << t;
        if (lane == 0) dst[kappa] = (uint8_t)m;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(act_ready));
    };
    scan_pass(0);
    for (int pass = 0; pass < n_pass; ++pass) {
      const int row0 = (first_tile + pass * p.T) * WD_M;
      const uint8_t *act_p = act + (pass & 1) * WD_MAX_K;
      if (!mbar_wait_warp_backoff(smem_u32(act_ready), (uint32_t)pass & 1u, abort_flag, 100)) break;
      // stages of the pass: offset-major, then slab, then tile
      int total = 0;
      for (int k0 = lane; k0 < K; k0 += 32) total += __popc(act_p[k0]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
      total *= p.k_groups;
      // this warp takes the stages whose number is slot_id modulo the slot count
      int kappa = 0, cnt = (K > 0 ? __popc(act_p[0]) : 0) * p.k_groups;
      int pos = (slot_id + p.a_slots - (int)(base_seq % (uint32_t)p.a_slots)) % p.a_slots;  // within offset `kappa`
      int local = pos;                                                             // within the pass
      struct Stage {
        int kappa, slab, t, valid;
        uint32_t seq;
      };
      auto locate = [&](Stage &st) {  // the stage at (kappa, pos), skipping offsets that are used up
        while (kappa < K && pos >= cnt) {
          pos -= cnt;
          ++kappa;
          cnt = kappa < K ? __popc(act_p[kappa]) * p.k_groups : 0;
        }
        st.valid = kappa < K;
        if (!st.valid) return;
        const uint32_t m = act_p[kappa];
        const int pc = __popc(m);
        const int slab = pos / pc, j = pos - slab * pc;
        st.kappa = kappa;
        st.slab = slab;
        st.t = __fns(m, 0, j + 1);  // j-th set bit
        st.seq = base_seq + (uint32_t)local;
      };
      int idx_cur[4], idx_nxt[4];
      auto load_idx = [&](const Stage &st, int *dst) {
        const int32_t *src = nbr + (size_t)st.kappa * n_out;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int r = row0 + st.t * WD_M + q * 32 + lane;
          dst[q] = r < n_rows ? __ldg(src + r) : -1;
        }
      };
      Stage cur, nxt;
      bool live = true;
      locate(nxt);
      if (nxt.valid) load_idx(nxt, idx_nxt);
      while (nxt.valid) {
        cur = nxt;
#pragma unroll
        for (int q = 0; q < 4; ++q) idx_cur[q] = idx_nxt[q];
        pos += p.a_slots;
        local += p.a_slots;
        locate(nxt);
        if (nxt.valid) load_idx(nxt, idx_nxt);
        // ---- produce stage `cur`
        const uint32_t slot = (uint32_t)slot_id, a_use = cur.seq / (uint32_t)p.a_slots;
        if (!mbar_wait_warp_backoff(smem_u32(empty_a + slot), (a_use & 1u) ^ 1u, abort_flag, 64)) { live = false; break; }
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const unsigned have = __ballot_sync(0xffffffffu, idx_cur[q] >= 0);
          if (lane == 0 && part == 0) masks[slot * 4 + q] = ~have;
        }
        if (lane == 0 && part == 0) slot_seq[slot] = cur.seq;
        const int ch0 = (cur.slab * p.sps + part) * 32;  // cur.slab counts slab groups
        const uint32_t sw = (uint32_t)(lane & 7);
        bool any = false;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (idx_cur[q] >= 0 && ch0 < c_in) {
            const float *fp = staged + (size_t)idx_cur[q] * c_in + ch0;
            const uint32_t a_row = smem_base + slot * (uint32_t)p.slot_bytes + (uint32_t)part * (uint32_t)WD_A_BYTES +
                                   (uint32_t)(q * 4 + (lane >> 3)) * 1024u + sw * 128u;
#pragma unroll
            for (int c = 0; c < 8; ++c) {  // chunks past the last channel are zero-filled
              const bool ok = ch0 + c * 4 < c_in;
              wd_cp16(a_row + ((c ^ sw) << 4), ok ? (const void *)(fp + c * 4) : (const void *)staged, ok ? 16u : 0u);
            }
            any = true;
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (any) fence_async_smem();
        mbar_arrive(smem_u32(full_a + slot));
      }
      if (!live) break;
      base_seq += (uint32_t)total;
      // The table of the next pass goes where that of the previous one was.  Wait for that phase
      // BEFORE arriving for this one: once this warp has arrived the barrier can move on two
      // phases, and a parity wait cannot tell a phase from the one two before it.
      if (pass >= 1 && !mbar_wait_warp_backoff(smem_u32(act_free), (uint32_t)(pass - 1) & 1u, abort_flag, 100)) break;
      if (lane == 0) mbar_arrive(smem_u32(act_free));  // done with this pass's table
      if (pass + 1 < n_pass) scan_pass(pass + 1);
    }
  } else if (warp < 4 + p.n_prod + p.T) {
   if (lane == 0) {
    // ====================================== MMA issuers =====================================
    // One thread per warp, on its own: every dependent instruction of this loop (a barrier poll, a
    // shared-memory read, a shuffle) adds its latency to each stage, so nothing here is warp-wide.
    const int t = warp - (4 + p.n_prod);  // the tile of each pass that this thread accumulates
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.n_pad >> 3) << 17) | ((uint32_t)(WD_M >> 4) << 24);
    const uint32_t below = (1u << t) - 1u;
    uint32_t base_seq = 0, bslot = 0, b_par = 0;
    bool live = true;
    for (int pass = 0; pass < n_pass && live; ++pass) {
      const uint32_t half = (uint32_t)(pass & 1), use = (uint32_t)(pass >> 1);
      const uint8_t *act_p = act + (pass & 1) * WD_MAX_K;
      if (!mbar_wait(smem_u32(act_ready), (uint32_t)pass & 1u, abort_flag)) break;
      // the half must have been drained and cleared (every phase is waited for, used or not)
      if (!mbar_wait(smem_u32(acc_empty + half), use & 1u, abort_flag)) break;
      tc_fence_after();
      const uint32_t d = tmem_base + half * 256u + (uint32_t)t * (uint32_t)p.n_pad;
      bool began = false;
      uint32_t off_seq = base_seq;  // number of the first stage of the current offset
      for (int kappa = 0; kappa < K && live; ++kappa) {
        const uint32_t m = act_p[kappa];
        if (m == 0) continue;
        const uint32_t pc = (uint32_t)__popc(m), rank = (uint32_t)__popc(m & below);
        const bool mine = (m >> t) & 1u;
        for (int kg = 0; kg < p.k_groups; ++kg) {
          // every group's filter phase is waited for, used or not: a parity wait cannot tell a
          // phase from the one two before it
          if (!mbar_wait(smem_u32(full_b + bslot), b_par, abort_flag)) { live = false; break; }
          if (mine) {
            const uint32_t seq = off_seq + (uint32_t)kg * pc + rank;
            const uint32_t slot = seq % (uint32_t)p.a_slots, a_use = seq / (uint32_t)p.a_slots;
            // The slot's word names the stage it holds: the threads run up to a few groups apart, and
            // a parity wait alone could take the slot's previous turn, not yet filled, for this one.
            bool have = false;
            for (uint32_t i = 0; i < kSpinLimit && !have; ++i) {
              have = mbar_try_wait(smem_u32(full_a + slot), a_use & 1u) && *(volatile uint32_t *)(slot_seq + slot) == seq;
              if (!have && (i & 1023u) == 1023u && *abort_flag) break;
            }
            if (!have) { *abort_flag = 1; live = false; break; }
            tc_fence_after();
            const uint4 off = *(const uint4 *)(masks + slot * 4u);
            const int n_sub = min(p.sps, p.k_slabs - kg * p.sps);
            for (int ss = 0; ss < n_sub; ++ss) {
              const uint32_t a_lo = desc_lo(smem_base + slot * (uint32_t)p.slot_bytes + (uint32_t)ss * (uint32_t)WD_A_BYTES);
              const uint32_t b_lo = desc_lo(b_base + bslot * (uint32_t)(p.sps * p.b_bytes) + (uint32_t)ss * (uint32_t)p.b_bytes);
              mma_tf32_ss_masked(d, a_lo, b_lo, idesc, off);
              mma_tf32_ss_masked(d, a_lo + 2u, b_lo + 2u, idesc, off);
              mma_tf32_ss_masked(d, a_lo + 4u, b_lo + 4u, idesc, off);
              mma_tf32_ss_masked(d, a_lo + 6u, b_lo + 6u, idesc, off);
            }
            began = true;
            mma_commit(smem_u32(empty_a + slot));
            mma_commit(smem_u32(empty_b + bslot));
          } else {
            mbar_arrive(smem_u32(empty_b + bslot));
          }
          if (++bslot == (uint32_t)p.b_slots) { bslot = 0; b_par ^= 1u; }
        }
        off_seq += pc * (uint32_t)p.k_groups;
      }
      if (!live) break;
      base_seq = off_seq;
      if (began) mma_commit(smem_u32(acc_full + half));
      else mbar_arrive(smem_u32(acc_full + half));
      mbar_arrive(smem_u32(act_free));
    }
   }
  } else {
    // ====================================== filter slabs ====================================
    uint32_t grp = 0;
    bool live = true;
    for (int pass = 0; pass < n_pass && live; ++pass) {
      if (!mbar_wait_warp_backoff(smem_u32(act_ready), (uint32_t)pass & 1u, abort_flag, 100)) break;
      const uint8_t *act_p = act + (pass & 1) * WD_MAX_K;
      for (int kappa = 0; kappa < K && live; ++kappa) {
        if (act_p[kappa] == 0) continue;
        for (int kg = 0; kg < p.k_groups; ++kg, ++grp) {
          const uint32_t bslot = grp % (uint32_t)p.b_slots, b_use = grp / (uint32_t)p.b_slots;
          if (!mbar_wait_warp_backoff(smem_u32(empty_b + bslot), (b_use & 1u) ^ 1u, abort_flag, 200)) { live = false; break; }
          if (lane == 0) {
            const int slab0 = kg * p.sps, n_sub = min(p.sps, p.k_slabs - slab0);
            const uint4 *bsrc = packed + ((size_t)kappa * p.k_slabs + slab0) * (size_t)(p.n_pad * 8);
            const uint32_t bar = smem_u32(full_b + bslot), nbytes = (uint32_t)(n_sub * p.b_bytes);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(nbytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             b_base + bslot * (uint32_t)(p.sps * p.b_bytes)),
                         "l"(bsrc), "r"(nbytes), "r"(bar)
                         : "memory");
          }
        }
      }
      if (lane == 0) mbar_arrive(smem_u32(act_free));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) atomicOr(status, 16);
  if (warp == 4 + p.n_prod) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(WD_TMEM_COLS) : "memory");
  }
}

// returns -1 when this variant does not apply (the caller then uses the one-tile-per-CTA kernel)
int conv_fwd_tf32_wide(const float *staged, int c_pad, int c_in, const void *packed, int K, int c_out, const int32_t *nbr,
                       int n_out, float *out, int32_t *status, const int32_t *n_out_dev, cudaStream_t st) {
  WideParams p;
  int tile_n, n_tiles;
  if (!tc_operand_layout(c_in, c_out, &p.k_slabs, &p.n_pad, &tile_n, &n_tiles)) return -1;
  if (n_tiles != 1 || p.n_pad > 256 || K > WD_MAX_K) return -1;
  p.b_bytes = p.n_pad * 128;
  p.T = 256 / p.n_pad;
  if (p.T > WD_MAX_T) p.T = WD_MAX_T;
  p.sps = p.k_slabs >= 2 ? 2 : 1;
  const char *sps_env = getenv("SSC_WIDE_SPS");
  if (sps_env != nullptr && atoi(sps_env) == 1) p.sps = 1;
  p.k_groups = (p.k_slabs + p.sps - 1) / p.sps;
  p.slot_bytes = p.sps * WD_A_BYTES;
  const int group_bytes = p.sps * p.b_bytes;
  p.b_slots = group_bytes <= 12 * 1024 ? 3 : 2;
  const int budget = 227 * 1024 - 1024 - WD_CTRL_BYTES - p.b_slots * group_bytes;
  p.a_slots = budget / p.slot_bytes;
  if (p.a_slots > WD_MAX_PROD / p.sps) p.a_slots = WD_MAX_PROD / p.sps;  // one producer warp per slab of every slot
  if (p.a_slots < 2) return -1;
  p.n_prod = p.a_slots * p.sps;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t smem = (size_t)p.a_slots * p.slot_bytes + (size_t)p.b_slots * group_bytes + WD_CTRL_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(conv_fwd_tf32_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd(tf32, wide): smem attribute: %s", cudaGetErrorString(e));
  const int total_tiles = ceil_div(n_out, WD_M);
  const int grid = total_tiles < sms ? total_tiles : sms;
  { conv_fwd_tf32_wide_kernel<<<grid, (4 + p.n_prod + p.T + 1) * 32, smem, st>>>(staged, c_pad, (const uint4 *)packed, K, c_out, nbr, n_out, out,
                                                           status, p, n_out_dev); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_tf32_wide");
  return SSC_OK;
}

}  // namespace ssc
