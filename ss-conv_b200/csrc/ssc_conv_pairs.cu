// Pair-list gather-GEMM-scatter on the 5th-generation tensor cores (tcgen05, sm_100a): the forward
// convolution for layers whose neighbour table is sparsely filled (wide submanifold layers: a
// 5^3 kernel at 10 % occupancy has 12 of its 125 offsets present per output row, so an
// output-stationary tile would spend 90 % of every MMA on absent rows).
//
//   for every kernel offset kappa, for every 128 pairs (i, o) of its compacted pair list:
//       D[128, Cout] = X[i, :] * W[kappa]          (dense M tile, all rows live)
//       out[o, :]   += D                           (one output row occurs once per offset)
//
// which is what the reference does with a gather, a cuBLAS GEMM and a scatter-add per offset
// (SS_Conv_lib/src/conv/indice_conv.h:290-338), here as ONE persistent launch:
//
//   * The work is cut into strips.  A strip belongs to one kernel offset (times one range of
//     output channels when the filter matrix of an offset does not fit shared memory whole) and is
//     every c-th 128-pair tile of that offset's list.  A CTA keeps the filter matrix of its strip
//     RESIDENT in shared memory (one bulk copy per 32/64-channel slab, once per strip), so the
//     only operand traffic per tile is the gathered rows.  All strips walk their lists from the
//     first row to the last at the same pace, so at any time the CTAs of the grid read and update
//     the same window of rows: the gathers and the reductions hit L2.
//   * warps 0 .. S-1: producers.  Warp w owns ring slot w: two lanes per row (each 32-byte sector
//     is asked for once), 16-byte cp.async copies of the row's 128-byte slab from the staged operand
//     image (TF32-rounded fp32, fp16 or bf16) into the K-major 128-byte-swizzled operand layout,
//     then one arrival per lane on the slot's "full" mbarrier.
//   * warp S: tensor-memory allocation and the MMA-issuing thread: tcgen05.mma M=128, N<=256,
//     accumulating over the slabs of a tile in one of TWO accumulator buffers, tcgen05.commit to
//     the slot's "empty" barrier and, after the last slab, to the buffer's "accumulator full"
//     barrier.
//   * warps S+1 .. S+8: epilogue, two per quarter of the tensor-memory lanes (they take the
//     32-column blocks in turn).  tcgen05.ld (lane = pair), a transposition through shared memory,
//     16 rows at a time, so that eight neighbouring lanes hold the 128 contiguous bytes of one
//     output row, then red.global.add.v4.f32: the reductions reach L2 as whole 128-byte lines.
//     The epilogue of tile t runs under the MMAs of tile t+1.
//
// The output must be zero before the launch (the host wrapper clears it).  The sums of an output
// row arrive in no fixed order, so results are reproducible only up to fp32 rounding of a sum of
// about K/2 terms; the output-stationary kernel (ssc_conv_tc.cu) is the bitwise-repeatable one.
// Every wait is bounded; on expiry status bit 16 is set, tensor memory is freed, the kernel returns.
#include "ssc_conv_internal.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

constexpr int PL_M = 128;                 // pairs per tile
constexpr int PL_A_BYTES = PL_M * 128;    // one gathered slab
constexpr int PL_MAX_STAGES = 6;
constexpr int PL_EPI_WARPS = 8;
constexpr int PL_STG_ROW = 144;           // bytes per row of the epilogue's transpose block (128 + 16 pad)
constexpr int PL_STG_BYTES = PL_EPI_WARPS * 16 * PL_STG_ROW;
constexpr int PL_CTRL_BYTES = 1024;
constexpr int PL_MAX_CTAS = 320;

struct PlParams {
  int k_slabs;      // 128-byte slabs per operand row
  int slab_words;   // 4-byte words of a staged row that are real data (the rest of the last slab is zero-filled)
  int row_words;    // row stride of the staged image in 4-byte words
  int n_pad;        // rows of one slab of the packed filter image
  int n_split;      // ranges of output channels (each a strip of its own)
  int n_cta;        // output channels per CTA = n_pad / n_split: multiple of 16, <= 256
  int acc_cols;     // tensor-memory columns of one accumulator buffer (power of two >= n_cta, >= 32)
  int stages;       // ring slots = producer warps
  int w_bytes;      // k_slabs * n_cta * 128: the resident filter matrix
  int threads;
  int ctas_per_sm;
  uint32_t idesc;
  int f16;          // kind::f16 (fp16 / bf16 operands) instead of kind::tf32
};

// Strip table of one (pair lists, grid) combination.
//   strips[s] = {virtual offset kv = kappa * n_split + half, first tile, tile stride, number of tiles}
//   owner[s]  = the CTA that runs strip s (a CTA runs its strips in ascending s)
//   hdr       = {number of strips, K, n_split, n_ctas}: the table is kept with the pair lists and only
//               built when the header does not match (another grid or channel split)
// L = the grid's fair share of all tiles.  An offset with T <= L tiles is one strip; up to 1.5 L it
// is a main strip of L tiles plus a tail; beyond that it is cut into round(T / L) interleaved strips
// (tiles r, r + c, ...: the centre offset of a submanifold layer).  Strips then go to the CTAs
// greedily, main strips first, each to the CTA with the least work so far: every CTA starts with a
// strip that walks its offset's list from the first row (all CTAs sweep the rows together, which keeps
// gathers and reductions in L2) and the tails fill the CTAs whose offsets were short.
__global__ void pl_strips_kernel(const int32_t *__restrict__ starts, int K, int n_split, int n_ctas,
                                 int32_t *__restrict__ hdr, int4 *__restrict__ strips, int32_t *__restrict__ owner) {
  __shared__ int tiles[256];
  __shared__ int first[257];
  __shared__ int load_s[PL_MAX_CTAS];
  __shared__ long long L_s;
  const int tid = threadIdx.x;
  if (hdr[0] > 0 && hdr[1] == K && hdr[2] == n_split && hdr[3] == n_ctas) return;   // built before for this grid
  int T = 0;
  if (tid < K) {
    const int n = starts[tid + 1] - starts[tid];
    T = n > 0 ? (n + PL_M - 1) / PL_M : 0;
  }
  tiles[tid] = T;
  __syncthreads();
  if (tid == 0) {
    long long tot = 0;
    for (int k = 0; k < K; ++k) tot += tiles[k];
    tot *= n_split;
    const long long L = (tot + n_ctas - 1) / n_ctas;
    L_s = L < 1 ? 1 : L;
  }
  __syncthreads();
  const int L = (int)L_s;
  int mains = 0, tail = 0;
  if (T > 0) {
    if (T > L + L / 2) mains = (T + L / 2) / L;
    else { mains = 1; tail = T > L ? 1 : 0; }
  }
  __syncthreads();
  tiles[tid] = (mains + tail) * n_split;
  __syncthreads();
  if (tid == 0) {
    int s = 0;
    for (int k = 0; k < K; ++k) {
      first[k] = s;
      s += tiles[k];
    }
    first[256] = s;
  }
  __syncthreads();
  const int n_strips = first[256];
  if (tid < K && T > 0) {
    int s = first[tid];
    for (int h = 0; h < n_split; ++h) {
      const int kv = tid * n_split + h;
      if (mains > 1) {
        for (int r = 0; r < mains; ++r) { strips[s] = make_int4(kv, r, mains, (T - r + mains - 1) / mains); owner[s++] = -1; }
      } else {
        strips[s] = make_int4(kv, 0, 1, T < L ? T : L);
        owner[s++] = -1;
        if (tail) { strips[s] = make_int4(kv, L, 1, T - L); owner[s++] = -2; }
      }
    }
  }
  __syncthreads();
  if (tid < 32) {   // one warp: greedy assignment, main strips (-1) first, then tails (-2)
    for (int b = tid; b < n_ctas; b += 32) load_s[b] = 0;
    __syncwarp();
    for (int pass = -1; pass >= -2; --pass) {
      for (int s = 0; s < n_strips; ++s) {
        if (owner[s] != pass) continue;            // warp-uniform
        int best = 0x7fffffff, arg = 0x7fffffff;
        for (int b = tid; b < n_ctas; b += 32) {
          const int v = load_s[b];
          if (v < best) { best = v; arg = b; }     // ascending b: the lowest index wins ties
        }
        for (int o = 16; o > 0; o >>= 1) {
          const int ob = __shfl_xor_sync(0xffffffffu, best, o), oa = __shfl_xor_sync(0xffffffffu, arg, o);
          if (ob < best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (tid == 0) {
          owner[s] = arg;
          load_s[arg] = best + strips[s].w;
        }
        __syncwarp();
      }
    }
    if (tid == 0) {
      hdr[1] = K;
      hdr[2] = n_split;
      hdr[3] = n_ctas;
      __threadfence();
      hdr[0] = n_strips;
    }
  }
}

template <bool F16>
__global__ void __launch_bounds__((PL_MAX_STAGES + 1 + PL_EPI_WARPS) * 32, 1)
conv_fwd_pairs_kernel(const float *__restrict__ staged, const uint4 *__restrict__ packed, int c_out,
                      const int32_t *__restrict__ pair_out, const int32_t *__restrict__ pair_in,
                      const int32_t *__restrict__ starts, const int4 *__restrict__ strips,
                      const int32_t *__restrict__ owner, const int32_t *__restrict__ n_strips_dev,
                      float *__restrict__ out, int32_t *status, PlParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *w_smem = smem;                                       // resident filters, [k_slabs][n_cta][128 B]
  uint8_t *a_smem = smem + p.w_bytes;                           // [stages][16 KB]
  uint8_t *stg = a_smem + (size_t)p.stages * PL_A_BYTES;        // epilogue transpose blocks
  uint8_t *ctrl = stg + PL_STG_BYTES;
  uint64_t *full_bars = (uint64_t *)ctrl;                       // [stages] gathered slab landed
  uint64_t *empty_bars = full_bars + PL_MAX_STAGES;             // [stages] its MMAs retired
  uint64_t *accf_bars = empty_bars + PL_MAX_STAGES;             // [2] accumulator buffer complete
  uint64_t *acce_bars = accf_bars + 2;                          // [2] accumulator buffer read out
  uint64_t *wfull_bar = acce_bars + 2;                          // filters of the strip landed
  uint64_t *wfree_bar = wfull_bar + 1;                          // every MMA of the strip retired
  uint64_t *final_bar = wfree_bar + 1;
  uint32_t *tmem_slot = (uint32_t *)(final_bar + 1);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;
  const int mma_warp = S;
  const int n_strips = *n_strips_dev;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(full_bars + s), 32);
      mbar_init(smem_u32(empty_bars + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(accf_bars + b), 1);
      mbar_init(smem_u32(acce_bars + b), PL_EPI_WARPS);
    }
    mbar_init(smem_u32(wfull_bar), 1);
    mbar_init(smem_u32(wfree_bar), 1);
    mbar_init(smem_u32(final_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == mma_warp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)(2 * p.acc_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t a_base = smem_u32(a_smem), w_base = smem_u32(w_smem);

  // Every role walks the same strips and keeps the same counters: g = ring steps so far (slot
  // g % S, use g / S), tcount = tiles so far (buffer tcount % 2), scount = strips so far.
  if (warp < S) {
    // ==================================== producers =============================================
    // Two lanes per row: lanes 2j and 2j+1 copy neighbouring 16-byte chunks, i.e. one whole 32-byte
    // sector per pair of lanes and instruction (one lane per row would ask for every sector twice,
    // once per half).  Pass p of a step covers rows 16 p .. 16 p + 15; a lane copies four chunks
    // (2 cc + its parity, cc = 0..3) of its row in each of the eight passes.
    const int lrow = lane >> 1, lpar = lane & 1;
    const uint32_t sw = (uint32_t)(lrow & 7);             // row & 7 (16 p keeps the low three bits)
    const uint32_t row_off0 = (uint32_t)(lrow >> 3) * 1024u + sw * 128u;   // + p * 2048
    const uint32_t slot_addr = a_base + (uint32_t)warp * PL_A_BYTES;
    long long g = 0;
    int scount = 0, w_issued = 0;
    bool alive = true;
    for (int si = 0; si < n_strips && alive; ++si) {
      if (__ldg(owner + si) != (int)blockIdx.x) continue;
      const int4 sd = __ldg(strips + si);
      const int kappa = sd.x / p.n_split, half = sd.x - kappa * p.n_split;
      const int list0 = __ldg(starts + kappa), n_pairs = __ldg(starts + kappa + 1) - list0;
      const int n_tiles = sd.w;
      if (warp == 0 && lane == 0) {
        // the strip's filter matrix: one bulk copy per slab, after the MMAs of the last strip retired
        bool ok = true;
        if (scount > 0) ok = mbar_wait_backoff(smem_u32(wfree_bar), (uint32_t)(scount - 1) & 1u, abort_flag, 128);
        if (ok) {
          const uint32_t bar = smem_u32(wfull_bar), slab_bytes = (uint32_t)p.n_cta * 128u;
          mbar_expect_tx(bar, (uint32_t)p.w_bytes);
          for (int s = 0; s < p.k_slabs; ++s) {
            const uint4 *src = packed + ((size_t)kappa * p.k_slabs + s) * (size_t)(p.n_pad * 8) + (size_t)half * (size_t)(p.n_cta * 8);
            bulk_g2s(w_base + (uint32_t)s * slab_bytes, src, slab_bytes, bar);
          }
          ++w_issued;
        }
      }
      const long long n_steps = (long long)n_tiles * p.k_slabs;
      // input rows of step q (the same for every slab of a tile)
      auto load_rows = [&](long long q, int *dst) {
        const int ti = (int)(q / p.k_slabs);
        const int row0 = (sd.y + ti * sd.z) * PL_M;       // position of the tile in the offset's list
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int j = row0 + r * 16 + lrow;
          dst[r] = j < n_pairs ? __ldg(pair_in + list0 + j) : -1;
        }
      };
      // first step of this strip that falls on this warp's slot
      long long q = ((long long)warp - g % S + S) % S;
      int src[8], nxt[8];
      if (q < n_steps) load_rows(q, nxt);
      for (; q < n_steps; q += S) {
        const int ti = (int)(q / p.k_slabs), slab = (int)(q - (long long)ti * p.k_slabs);
#pragma unroll
        for (int r = 0; r < 8; ++r) src[r] = nxt[r];
        if (q + S < n_steps) load_rows(q + S, nxt);       // in flight while this step waits and copies
        const long long use = (g + q) / S;
        if (use > 0) {
          if (!mbar_wait_warp_backoff(smem_u32(empty_bars + warp), (uint32_t)(use - 1) & 1u, abort_flag, 32)) { alive = false; break; }
          tc_fence_after();
        }
        const int w0 = slab * 32;                          // first 4-byte word of the slab
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (src[r] >= 0) {
            const float *fp = staged + (size_t)src[r] * p.row_words + w0;
            const uint32_t a_row = slot_addr + row_off0 + (uint32_t)r * 2048u;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {   // chunks past the last real word are zero-filled
              const int c = 2 * cc + lpar;
              const bool ok = w0 + c * 4 < p.slab_words;
              cp_async16_cg(a_row + (((uint32_t)c ^ sw) << 4), ok ? (const void *)(fp + c * 4) : (const void *)staged, ok ? 16u : 0u);
            }
          }
        }
        cp_async_commit();
        cp_async_wait_all();
        fence_async_smem();
        mbar_arrive(smem_u32(full_bars + warp));
      }
      g += n_steps;
      ++scount;
    }
    // a wait gave up while a filter copy may still be in flight: let it land before the CTA exits
    if (warp == 0 && lane == 0 && *abort_flag && w_issued > 0) mbar_wait_drain(smem_u32(wfull_bar), (uint32_t)(w_issued - 1) & 1u);
  } else if (warp == mma_warp) {
    // ==================================== MMA issuer ============================================
    if (lane == 0) {
      long long g = 0;
      int tcount = 0, scount = 0;
      bool alive = true;
      for (int si = 0; si < n_strips && alive; ++si) {
        if (__ldg(owner + si) != (int)blockIdx.x) continue;
        const int4 sd = __ldg(strips + si);
        const int n_tiles = sd.w;
        if (!mbar_wait_backoff(smem_u32(wfull_bar), (uint32_t)scount & 1u, abort_flag, 64)) break;
        tc_fence_after();
        for (int ti = 0; ti < n_tiles && alive; ++ti, ++tcount) {
          const int buf = tcount & 1;
          if (tcount >= 2) {
            if (!mbar_wait_backoff(smem_u32(acce_bars + buf), (uint32_t)((tcount >> 1) - 1) & 1u, abort_flag, 64)) { alive = false; break; }
            tc_fence_after();
          }
          const uint32_t d = tmem_base + (uint32_t)(buf * p.acc_cols);
          for (int s = 0; s < p.k_slabs; ++s, ++g) {
            const uint32_t slot = (uint32_t)(g % S), par = (uint32_t)(g / S) & 1u;
            if (!mbar_wait_backoff(smem_u32(full_bars + slot), par, abort_flag, 32)) { alive = false; break; }
            tc_fence_after();
            const uint32_t a_lo = desc_lo(a_base + slot * PL_A_BYTES);
            const uint32_t b_lo = desc_lo(w_base + (uint32_t)s * (uint32_t)p.n_cta * 128u);
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk) {
              if (F16) mma_f16_ss(d, a_lo + 2u * kk, b_lo + 2u * kk, p.idesc, (s | (int)kk) != 0 ? 1u : 0u);
              else mma_tf32_ss(d, a_lo + 2u * kk, b_lo + 2u * kk, p.idesc, (s | (int)kk) != 0 ? 1u : 0u);
            }
            mma_commit(smem_u32(empty_bars + slot));
          }
          if (alive) mma_commit(smem_u32(accf_bars + buf));
        }
        if (alive) mma_commit(smem_u32(wfree_bar));
        ++scount;
      }
      // everything issued above (on any path) retires before the CTA hands its tensor memory back
      mma_commit(smem_u32(final_bar));
      mbar_wait_drain(smem_u32(final_bar), 0u);
    }
  } else {
    // ==================================== epilogue ==============================================
    // Two warps per quarter of the tensor-memory lanes; they take the 32-column blocks of the
    // accumulator in turn.  The load of a warp's next block is in flight while it transposes and
    // reduces the current one.
    const int ew = warp - mma_warp - 1;                    // 0 .. 7
    const int quarter = warp & 3;                          // the 32 tensor-memory lanes this warp may read
    const int part = ew >> 2;                              // blocks part, part + 2, ...
    uint8_t *blk = stg + (size_t)ew * 16 * PL_STG_ROW;
    const bool vec_ok = (c_out & 3) == 0 && ((uintptr_t)out & 15u) == 0;
    const int sub = lane & 7, grp = lane >> 3;             // 16-byte piece of a row, row of a pass
    int tcount = 0;
    bool alive = true;
    for (int si = 0; si < n_strips && alive; ++si) {
      if (__ldg(owner + si) != (int)blockIdx.x) continue;
      const int4 sd = __ldg(strips + si);
      const int kappa = sd.x / p.n_split, half = sd.x - kappa * p.n_split;
      const int list0 = __ldg(starts + kappa), n_pairs = __ldg(starts + kappa + 1) - list0;
      const int n_tiles = sd.w;
      const int col0 = half * p.n_cta;
      const int cols = min(p.n_cta, c_out - col0);
      const int n_blocks = cols > 0 ? (cols + 31) >> 5 : 0;       // 32-column blocks with real columns
      // output row of this lane's pair, fetched one tile ahead
      auto out_row_of = [&](int ti) {
        const int j = (sd.y + ti * sd.z) * PL_M + quarter * 32 + lane;
        return (ti < n_tiles && j < n_pairs) ? __ldg(pair_out + list0 + j) : -1;
      };
      int next_out = out_row_of(0);
      for (int ti = 0; ti < n_tiles; ++ti, ++tcount) {
        const int buf = tcount & 1;
        const int my_out = next_out;
        next_out = out_row_of(ti + 1);
        if (!mbar_wait_warp(smem_u32(accf_bars + buf), (uint32_t)(tcount >> 1) & 1u, abort_flag)) { alive = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.acc_cols);
        // one load = this lane's row of a 32 x 32 block (two x16 loads in flight together)
        auto tld = [&](uint32_t(&v)[32], int blk_i) {
          const uint32_t ta = taddr + (uint32_t)(blk_i * 32);
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
              : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
              : "r"(ta)
              : "memory");
          if (blk_i * 32 + 16 < p.n_cta) {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                : "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                  "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(ta + 16u)
                : "memory");
          }
        };
        // The 32 columns of 16 lanes' rows go to shared memory, then four rows per pass come back with
        // eight neighbouring lanes holding the 128 contiguous bytes of one output row: the
        // reductions reach L2 as whole 128-byte lines (the L2 slices take ~20 % more bytes per
        // second in that shape than in 64-byte pieces).
        auto reduce_block = [&](const uint32_t(&v)[32], int blk_i) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if ((lane >> 4) == h) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *(uint4 *)(blk + (lane & 15) * PL_STG_ROW + q * 16) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
            __syncwarp();
            const int c_local = blk_i * 32 + sub * 4;       // column within the strip's range
            const int cc = col0 + c_local;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int row = 4 * i + grp;
              const int orow = __shfl_sync(0xffffffffu, my_out, 16 * h + row);
              const float4 x = *(const float4 *)(blk + row * PL_STG_ROW + sub * 16);
              if (orow >= 0 && c_local < cols) {
                float *dst = out + (size_t)orow * c_out + cc;
                if (vec_ok) {
                  red_add_v4(dst, x);
                } else {
                  atomicAdd(dst, x.x);
                  if (cc + 1 < c_out) atomicAdd(dst + 1, x.y);
                  if (cc + 2 < c_out) atomicAdd(dst + 2, x.z);
                  if (cc + 3 < c_out) atomicAdd(dst + 3, x.w);
                }
              }
            }
            __syncwarp();
          }
        };
        uint32_t va[32], vb[32];
        if (part < n_blocks) tld(va, part);
        for (int b = part; b < n_blocks; b += 4) {
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (b + 2 < n_blocks) tld(vb, b + 2);
          reduce_block(va, b);
          if (b + 2 < n_blocks) {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (b + 4 < n_blocks) tld(va, b + 4);
            reduce_block(vb, b + 2);
          }
        }
        // this warp has read its share of the buffer: the MMA thread may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(acce_bars + buf));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) atomicOr(status, 16);
  if (warp == mma_warp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * p.acc_cols))
                 : "memory");
  }
}

static size_t pl_smem_bytes(const PlParams &p) {
  return (size_t)p.w_bytes + (size_t)p.stages * PL_A_BYTES + PL_STG_BYTES + PL_CTRL_BYTES + 1024 /*alignment slack*/;
}

// Shapes the kernel covers: the filter matrix of one offset (or one range of its output channels)
// resident in shared memory next to at least three ring slots.
static bool pl_params(int c_in, int c_out, int precision, PlParams &p) {
  const bool is16 = precision == SSC_PREC_F16 || precision == SSC_PREC_BF16;
  if (!is16 && tf32_offsets_per_row(c_in) > 1) return false;   // those filters are packed several offsets per row
  const int words = is16 ? f16_row_words(c_in) : c_in;
  int tile_n, n_tiles;
  if (!tc_operand_layout(words, c_out, &p.k_slabs, &p.n_pad, &tile_n, &n_tiles)) return false;
  p.f16 = is16 ? 1 : 0;
  p.slab_words = is16 ? words : c_in;
  p.row_words = is16 ? words : ((c_in + 3) & ~3);
  const size_t budget = 227 * 1024 - PL_STG_BYTES - PL_CTRL_BYTES - 1024;
  p.n_split = 0;
  for (int ns = 1; ns <= 8; ++ns) {
    if (p.n_pad % (16 * ns) != 0) continue;
    const int n_cta = p.n_pad / ns;
    if (n_cta > 256) continue;
    const size_t w = (size_t)p.k_slabs * n_cta * 128;
    if (w + 3 * (size_t)PL_A_BYTES > budget) continue;
    p.n_split = ns;
    p.n_cta = n_cta;
    p.w_bytes = (int)w;
    break;
  }
  if (p.n_split == 0 || p.n_cta < 16) return false;
  p.acc_cols = 32;
  while (p.acc_cols < p.n_cta) p.acc_cols <<= 1;
  p.ctas_per_sm = 1;      // 13 to 15 warps with ~100 registers each: one persistent CTA per SM
  const size_t b = budget;
  p.stages = (int)((b - p.w_bytes) / PL_A_BYTES);
  if (p.stages > PL_MAX_STAGES) p.stages = PL_MAX_STAGES;
  if (p.stages < 3) return false;
  p.threads = (p.stages + 1 + PL_EPI_WARPS) * 32;
  const uint32_t fmt = is16 ? (precision == SSC_PREC_BF16 ? 1u : 0u) : 2u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.n_cta >> 3) << 17) | ((uint32_t)(PL_M >> 4) << 24);
  return true;
}

bool conv_pairs_supported(int c_in, int c_out, int precision) {
  PlParams p;
  return pl_params(c_in, c_out, precision, p);
}

static size_t max_strips(int K) { return (size_t)PL_MAX_CTAS + 16 * (size_t)K + 16; }   // mains + tails of K * n_split (<= 8) virtual offsets

size_t conv_pairs_strip_bytes(int K) { return 256 + max_strips(K) * (sizeof(int4) + sizeof(int32_t)); }

// `staged`: the operand image of the feature rows (ssc_conv_stage); `strip_mem`: conv_pairs_strip_bytes(K) bytes.
int conv_fwd_pairs(const void *staged, int c_in, const void *packed, int K, int c_out, int precision,
                   const PairLists &pl, int n_out, float *out, int32_t *status, void *strip_mem, cudaStream_t st) {
  PlParams p;
  if (K > 256 || !pl_params(c_in, c_out, precision, p))
    return fail(SSC_ERR_INVALID, "conv_fwd_pairs: shape (c_in %d, c_out %d, kernel volume %d) not covered by the pair-list kernel", c_in, c_out, K);
  int n_ctas = sm_count() * p.ctas_per_sm;
  if (n_ctas > PL_MAX_CTAS) n_ctas = PL_MAX_CTAS;
  int32_t *hdr = (int32_t *)strip_mem;
  int4 *strips = (int4 *)((uint8_t *)strip_mem + 256);
  int32_t *owner = (int32_t *)(strips + max_strips(K));
  cudaError_t e = cudaMemsetAsync(out, 0, (size_t)n_out * c_out * sizeof(float), st);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd_pairs: clearing the output: %s", cudaGetErrorString(e));
  { pl_strips_kernel<<<1, 256, 0, st>>>(pl.starts, K, p.n_split, n_ctas, hdr, strips, owner); note_launches(1); }
  SSC_CHECK_LAUNCH("pl_strips");
  const size_t smem = pl_smem_bytes(p);
  auto kernel = p.f16 ? conv_fwd_pairs_kernel<true> : conv_fwd_pairs_kernel<false>;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd_pairs: smem attribute: %s", cudaGetErrorString(e));
  { kernel<<<n_ctas, p.threads, smem, st>>>((const float *)staged, (const uint4 *)packed, c_out, pl.pair_out, pl.pair_in, pl.starts,
                                          strips, owner, hdr, out, status, p); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_pairs");
  return SSC_OK;
}

}  // namespace ssc

using namespace ssc;

extern "C" size_t ssc_conv_pairs_list_bytes(int K, int n_out) {
  if (K < 1 || K > 256 || n_out < 0) return 0;
  return align_up(pair_lists_bytes(K, n_out), 256) + conv_pairs_strip_bytes(K);
}

extern "C" int ssc_conv_pairs_supported(int c_in, int c_out, int precision) {
  return (c_in >= 1 && c_out >= 1 && conv_pairs_supported(c_in, c_out, precision)) ? 1 : 0;
}

extern "C" int ssc_conv_pairs_build(const int32_t *nbr, int K, int n_out, void *lists, size_t list_bytes, void *stream) {
  SSC_REQUIRE(K >= 1 && K <= 256 && n_out >= 1 && nbr && lists, "conv_pairs_build: bad arguments");
  SSC_REQUIRE(list_bytes >= ssc_conv_pairs_list_bytes(K, n_out) && ((uintptr_t)lists & 255u) == 0,
              "conv_pairs_build: list buffer too small or not 256-byte aligned");
  // the strip table kept behind the lists belongs to the old lists: forget it
  void *strip_mem = (uint8_t *)lists + align_up(pair_lists_bytes(K, n_out), 256);
  cudaError_t e = cudaMemsetAsync(strip_mem, 0, 256, as_stream(stream));
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_pairs_build: %s", cudaGetErrorString(e));
  return pair_lists_build(nbr, K, n_out, lists, nullptr, as_stream(stream));
}

extern "C" int ssc_conv_fwd_pairs(const float *features, int n_in, int c_in, const void *packed, int K, int c_out,
                                  void *lists, size_t list_bytes, int n_out, int precision, float *out, int32_t *status,
                                  void *scratch, size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(c_in > 0 && c_out > 0 && K > 0 && K <= 256 && n_in >= 0 && n_out >= 0, "conv_fwd_pairs: bad sizes");
  const bool prestaged = (precision & SSC_CONV_PRESTAGED) != 0;
  precision &= ~SSC_CONV_PRESTAGED;
  if (n_out == 0) return SSC_OK;
  SSC_REQUIRE(packed && lists && out && scratch && (n_in == 0 || features || prestaged), "conv_fwd_pairs: null pointer");
  SSC_REQUIRE(precision == SSC_PREC_TF32 || precision == SSC_PREC_F16 || precision == SSC_PREC_BF16,
              "conv_fwd_pairs: precision %d has no tensor-core form", precision);
  SSC_REQUIRE(list_bytes >= ssc_conv_pairs_list_bytes(K, n_out) && ((uintptr_t)lists & 255u) == 0,
              "conv_fwd_pairs: list buffer too small or not 256-byte aligned");
  SSC_REQUIRE(scratch_bytes + 16 >= ssc_conv_scratch_bytes(n_in, c_in, c_out, precision) && ((uintptr_t)scratch & 15u) == 0,
              "conv_fwd_pairs: staging buffer too small or not 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  if (!prestaged) {
    int rc = precision == SSC_PREC_TF32 ? stage_features(features, n_in, c_in, scratch, st)
                                        : stage_features_16(features, n_in, c_in, precision == SSC_PREC_BF16, scratch, st);
    if (rc != SSC_OK) return rc;
  }
  const PairLists pl = pair_lists_view(lists, K, n_out);
  void *strip_mem = (uint8_t *)lists + align_up(pair_lists_bytes(K, n_out), 256);
  return conv_fwd_pairs(scratch, c_in, packed, K, c_out, precision, pl, n_out, out, status, strip_mem, st);
}
