// Output-stationary gather-GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// One CTA owns 128 consecutive output rows and runs a warp-specialised pipeline over the
// steps (kernel offset with a neighbour in the tile) x (32-channel slab of the input).  The
// operand ring has one slot per producer warp:
//   * producer warp w owns ring slot w and prepares the steps w, w+S, w+2S, ...: each lane
//     looks up the neighbour rows of its four output rows and pulls the 128-byte slab of every
//     present feature row with cp.async straight into the K-major 128-byte-swizzled operand
//     layout; rows without a neighbour stay zero (a slot row is cleared again only if it held
//     data before).  When its copies have landed the lane rounds its rows fp32 -> TF32 (round
//     to nearest) in place and arrives on the slot's "A full" mbarrier.  Lane 0 also brings in
//     the pre-packed filter slab (already TF32, already in operand layout) with one bulk
//     asynchronous copy that completes on the "B full" mbarrier.  The global-memory latency
//     of a step is paid inside one warp while the other warps work on the neighbouring steps.
//   * one MMA warp: a single thread waits for both barriers of a slot, issues tcgen05.mma
//     (M=128, N<=256, K=8 per instruction) accumulating in tensor memory (fp32), and commits
//     the group to the slot's "empty" mbarrier, which lets the owner refill the slot.
// There is no CTA-wide barrier inside the loop.  Accumulators stay in TMEM across all
// offsets; four warps then read them with tcgen05.ld and write each output row exactly once
// (no scatter atomics, deterministic order).
//
// Every wait on an mbarrier is bounded: on expiry the thread records an error in `status`
// through a shared flag, every other wait then gives up too, and the kernel frees its tensor
// memory and returns.
#include "ssc_conv_internal.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

constexpr int TC_M = 128;
constexpr int TC_SLAB = 32;            // tf32 elements per 128-byte operand row
constexpr int TC_MAX_STAGES = 8;       // producer warps = ring slots
constexpr int TC_EPI_WARPS = 4;        // warps 0..3 also run the epilogue (one TMEM lane quarter each)
constexpr int TC_A_BYTES = TC_M * 128;
constexpr int TC_CTRL_BYTES = 1024;

struct TcParams {
  int k_slabs;    // ceil(c_in / 32)
  int n_pad;      // padded output channels (n_tiles * tile_n)
  int n_tiles;    // MMA instructions along N per k-step
  int tile_n;     // N of one MMA, multiple of 16, <= 256
  int tmem_cols;  // power of two >= max(32, n_pad)
  int stages;     // operand ring depth = number of producer warps (>= 4)
  int threads;    // (max(n_prod, 4) + 1) * 32
  int n_prod;     // producer warps: a multiple of the slots (several warps share a slot's rows)
  int b_bytes;    // n_pad * 128
  int sps;        // 32-channel slabs per ring slot (a step covers sps slabs of one kernel offset)
  int k_groups;   // ceil(k_slabs / sps) = steps per kernel offset
  int nt_cta;     // N tiles handled by one CTA: n_tiles, or 1 when the N tiles are spread over gridDim.y
  int n_cta;      // nt_cta * tile_n: accumulator columns / filter-slab rows per CTA
  int fmt16;      // 16-bit operands: 0 = fp16, 1 = bf16 (operand format field of the instruction descriptor)
  int last_kk;    // MMA k-steps (32 bytes of K each) that hold real channels in the LAST slab: 1..4
  int opk;        // kernel offsets per 128-byte operand row: 1, or 32 / c_pad for TF32 layers with c_pad = 4, 8, 16
  int nbr_by_pos; // 1: the table's columns are already in the order of `order` (column j <-> output row order[j])
                  // channels (a first layer with 3 input channels packs 8 offsets into one step)
};

// Shared-memory plan: [stages x (A 16 KB + B)] [control 1 KB].
static bool tc_params(int c_in, int c_out, TcParams &p, bool split_n = false, bool one_cta_per_sm = false, int opk = 1) {
  p.k_slabs = (c_in + TC_SLAB - 1) / TC_SLAB;
  p.last_kk = (c_in - (p.k_slabs - 1) * TC_SLAB + 7) / 8;     // c_in counts 4-byte words of an operand row
  p.opk = opk;
  p.nbr_by_pos = 0;
  if (opk > 1) {     // grouped offsets: one full slab per group of offsets
    p.k_slabs = 1;
    p.last_kk = 4;
  }
  int n16 = (c_out + 15) / 16 * 16;
  p.n_tiles = (n16 + 255) / 256;
  p.tile_n = ((n16 + p.n_tiles - 1) / p.n_tiles + 15) / 16 * 16;
  p.n_pad = p.n_tiles * p.tile_n;
  if (p.n_pad > 512) return false;
  // A layer with few row tiles and more than one N tile gets one CTA per (row tile, N tile): more
  // CTAs in flight, each with a smaller accumulator and filter slab (the rows are gathered twice).
  p.nt_cta = (split_n && p.n_tiles > 1) ? 1 : p.n_tiles;
  p.n_cta = p.nt_cta * p.tile_n;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.n_cta) p.tmem_cols <<= 1;
  p.b_bytes = p.n_cta * 128;
  // One 32-channel slab per step: two slabs per step halve the per-step bookkeeping but also the
  // resident CTAs, and measured slower (0.21 vs 0.18 ms on the 64 -> 76 channel layer).
  p.sps = 1;
  p.fmt16 = 0;
  p.k_groups = (p.k_slabs + p.sps - 1) / p.sps;
  int stage = p.sps * (TC_A_BYTES + p.b_bytes);
  int fixed = TC_CTRL_BYTES + 1024;
  // Resident CTAs hide each other's per-step latencies, so take as many per SM as tensor
  // memory (512 columns) and shared memory (two ring slots each at least) allow, up to four.
  // A launch with no more CTAs than SMs has nobody to share an SM with: all of the shared memory
  // goes into ring slots (a deeper pipeline is what a lone CTA has against the latency of a step).
  int ctas = 512 / p.tmem_cols;
  if (ctas > 4) ctas = 4;
  if (one_cta_per_sm) ctas = 1;
  while (ctas > 1 && ((227 * 1024) / ctas - 1024 - fixed) / stage < 2) --ctas;
  p.stages = ((227 * 1024) / ctas - 1024 - fixed) / stage;
  if (p.stages > TC_MAX_STAGES) p.stages = TC_MAX_STAGES;
  if (p.stages < 2) return false;
  // producer warps: one per slot with four or more slots, else the slots' rows are split over four warps
  p.n_prod = p.stages < TC_EPI_WARPS ? (TC_EPI_WARPS / p.stages) * p.stages : p.stages;
  p.threads = ((p.n_prod > TC_EPI_WARPS ? p.n_prod : TC_EPI_WARPS) + 1) * 32;
  return true;
}

// Geometry of the packed filter image, for the other kernels that consume it.
bool tc_operand_layout(int c_in, int c_out, int *k_slabs, int *n_pad, int *tile_n, int *n_tiles) {
  TcParams p;
  if (!tc_params(c_in, c_out, p)) return false;
  *k_slabs = p.k_slabs;
  *n_pad = p.n_pad;
  *tile_n = p.tile_n;
  *n_tiles = p.n_tiles;
  return true;
}

// Filter packing: filters [K, c_in, c_out] fp32 -> [K][k_slabs][n_pad rows][32 tf32] in the
// swizzled operand layout (row = output channel, 16-byte chunk index XOR (row & 7)).
__global__ void pack_filters_tf32_kernel(const float *__restrict__ filters, int K, int c_in, int c_out, TcParams p,
                                         uint4 *__restrict__ packed) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)K * p.k_slabs * p.n_pad * 8;
  if (t >= total) return;
  int chunk = (int)(t & 7);
  long long r = t >> 3;
  int n = (int)(r % p.n_pad);
  r /= p.n_pad;
  int slab = (int)(r % p.k_slabs);
  int kappa = (int)(r / p.k_slabs);
  uint32_t v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    int ci = slab * TC_SLAB + chunk * 4 + q;
    float f = (ci < c_in && n < c_out) ? filters[((size_t)kappa * c_in + ci) * c_out + n] : 0.f;
    v[q] = to_tf32(f);
  }
  size_t block = ((size_t)kappa * p.k_slabs + slab) * (size_t)(p.n_pad * 8);
  size_t off = (size_t)(n >> 3) * 64 + (size_t)(n & 7) * 8 + (size_t)(chunk ^ (n & 7));
  packed[block + off] = make_uint4(v[0], v[1], v[2], v[3]);
}

// The grouped form for few input channels (c_pad = 4, 8, 16; opk = 32 / c_pad offsets per operand row):
// [ceil(K / opk)][n_pad rows][32 tf32], word (o' * c_pad + c) of a row = W[g * opk + o', c, n].
__global__ void pack_filters_tf32_grouped_kernel(const float *__restrict__ filters, int K, int c_in, int c_out, int c_pad,
                                                 int opk, int n_groups, int n_pad, uint4 *__restrict__ packed) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)n_groups * n_pad * 8;
  if (t >= total) return;
  const int chunk = (int)(t & 7);
  long long r = t >> 3;
  const int n = (int)(r % n_pad), g = (int)(r / n_pad);
  uint32_t v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int w = chunk * 4 + q, o = w / c_pad, ci = w - o * c_pad, kappa = g * opk + o;
    const float f = (o < opk && kappa < K && ci < c_in && n < c_out) ? filters[((size_t)kappa * c_in + ci) * c_out + n] : 0.f;
    v[q] = to_tf32(f);
  }
  const size_t block = (size_t)g * (size_t)(n_pad * 8);
  const size_t off = (size_t)(n >> 3) * 64 + (size_t)(n & 7) * 8 + (size_t)(chunk ^ (n & 7));
  packed[block + off] = make_uint4(v[0], v[1], v[2], v[3]);
}

// Warps 0 .. n_prod-1 are producers (warp w <-> ring slot w; with fewer than four slots the
// spare warps only help in the prologue and epilogue), the last warp issues the MMAs.
// F16: the staged image and the filter slabs hold fp16 (64 channels per 128-byte row); the
// gather is the same byte-for-byte, `c_in` is then the row length in 4-byte units.
template <bool STAGED, bool F16 = false, bool GROUPED = false>
__global__ void __launch_bounds__((TC_MAX_STAGES + 1) * 32)
conv_fwd_tf32_kernel(const float *__restrict__ features, int c_in, const uint4 *__restrict__ packed, int K,
                     int c_out, const int32_t *__restrict__ nbr, int n_out, float *__restrict__ out,
                     int32_t *status, TcParams p, const int32_t *__restrict__ n_out_dev,
                     const int32_t *__restrict__ order) {
  // `order` (may be NULL): the rows of tile t are order[128 t .. 128 t + 127] instead of the same
  // consecutive numbers; rows that use the same kernel offsets, put next to each other, make a
  // tile skip the offsets none of them uses.
  // n_out is the row stride of nbr and the launch bound; the exact row count may still be on the
  // device (a rulebook sized optimistically): CTAs past it have nothing to do.
  const int n_rows = live_rows(n_out, n_out_dev);
  if ((int)blockIdx.x * TC_M >= n_rows) return;
  extern __shared__ uint8_t smem_raw[];
  // operand stages need 1024-byte alignment for the 128-byte swizzle
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = p.sps * (TC_A_BYTES + p.b_bytes);   // [sps x gathered slab][sps x filter slab]
  uint8_t *ctrl = smem + (size_t)p.stages * stage_bytes;
  uint64_t *empty_bars = (uint64_t *)ctrl;                 // [stages] slot free (its MMAs retired)
  uint64_t *fulla_bars = (uint64_t *)(ctrl + 64);          // [stages] gathered rows ready
  uint64_t *done_bar = (uint64_t *)(ctrl + 192);           // all MMAs of the tile retired
  uint32_t *tmem_slot = (uint32_t *)(ctrl + 200);
  volatile int *abort_flag = (volatile int *)(ctrl + 204);
  int *n_act_s = (int *)(ctrl + 208);
  uint8_t *act_flag = ctrl + 256;                          // [256]
  uint8_t *act_list = ctrl + 512;                          // [256]
  uint32_t *slot_masks = (uint32_t *)(ctrl + 768);         // [stages][4] rows of the step WITHOUT a neighbour

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_warps = blockDim.x >> 5;
  const int mma_warp = n_warps - 1;
  const int m0 = blockIdx.x * TC_M;
  const int nt0 = (int)blockIdx.y * p.nt_cta;   // first N tile of this CTA
  const int S = p.stages;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(empty_bars + s), 1);
      // one barrier per slot for both operands: every producer lane arrives for its gathered rows,
      // and the lane that starts the filter copy arrives once more with the copy's byte count
      // (the issuing thread then pays one barrier round trip per step, not two)
      mbar_init(smem_u32(fulla_bars + s), 32u * (uint32_t)(p.n_prod / S) + 1u);
    }
    mbar_init(smem_u32(done_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == mma_warp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else if (!GROUPED) {   // (grouped offsets: every group is a step, absent neighbours are zero-filled pieces)
    // which kernel offsets touch this tile: four offsets per pass so that 16 loads are in
    // flight per lane before the first ballot
    int scan_rows[4];  // this lane's four rows of the tile (-1 past the end)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = m0 + q * 32 + lane;
      scan_rows[q] = r < n_rows ? ((order && !p.nbr_by_pos) ? __ldg(order + r) : r) : -1;
    }
    for (int k0 = warp * 4; k0 < K; k0 += mma_warp * 4) {
      int v[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int r = scan_rows[q];
          v[i][q] = (k0 + i < K && r >= 0) ? __ldg(nbr + (size_t)(k0 + i) * n_out + r) : -1;
        }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        bool any = (v[i][0] >= 0) | (v[i][1] >= 0) | (v[i][2] >= 0) | (v[i][3] >= 0);
        unsigned b = __ballot_sync(0xffffffffu, any);
        if (lane == 0 && k0 + i < K) act_flag[k0 + i] = b != 0;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < TC_EPI_WARPS) {
    // Clear the accumulators.  Every MMA below accumulates, and rows without a neighbour at a
    // step are switched off through the MMA's disable-output-lane mask, so the gathered operand
    // never has to hold zero rows (stale rows of an earlier step are simply not written back).
    for (int c0 = 0; c0 < p.n_cta; c0 += 16) {
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr),
          "r"(0u)
          : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    int n = 0;
    if (GROUPED) {   // steps are groups of opk offsets, all of them
      for (int g = 0; g * p.opk < K; ++g) act_list[n++] = (uint8_t)g;
    } else {
      for (int kappa = 0; kappa < K; ++kappa)
        if (act_flag[kappa]) act_list[n++] = (uint8_t)kappa;
    }
    *n_act_s = n;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n_act = *n_act_s;
  const int n_iter = n_act * p.k_groups;
  const uint32_t smem_base = smem_u32(smem);

  const int n_prod = p.n_prod;  // producer warps (2 slots -> 4 warps)
  if (warp < n_prod) {
    // ====================== producer warp ====================================================
    // With S >= 4 ring slots, warp w owns slot w and prepares all 128 rows of the steps
    // w, w+S, ...; with fewer slots several warps share a slot and split its rows.
    const int slot = warp % S;
    const int share = n_prod / S;              // warps per slot
    const int part = warp / S;                 // which share of the rows this warp prepares
    const int q_per = 4 / share;               // 32-row groups per warp (share is 1, 2 or 4)
    const int q0 = part * q_per;
    const bool vec_ok = (c_in & 3) == 0;
    const uint32_t slot_addr = smem_base + (uint32_t)slot * (uint32_t)stage_bytes;
    uint8_t *slot_ptr = smem + (size_t)slot * stage_bytes;
    (void)slot_ptr;
    const uint32_t sw = (uint32_t)(lane & 7);
    // row q*32+lane of the slot: 8-row group (q*4 + lane/8), row-in-group lane%8
    uint32_t row_off[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) row_off[q] = (uint32_t)(q * 4 + (lane >> 3)) * 1024u + sw * 128u;
    uint32_t par = 0;          // parity of the slot's current use
    int src[4], nxt[4];
    int my_rows[4];            // this lane's four rows of the tile (-1 past the end)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = m0 + q * 32 + lane;
      my_rows[q] = r < n_rows ? ((order && !p.nbr_by_pos) ? __ldg(order + r) : r) : -1;
    }
    auto load_rows = [&](int j, int *dst) {
      const int kap = act_list[j / p.k_groups];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        dst[q] = (q >= q0 && q < q0 + q_per && my_rows[q] >= 0) ? __ldg(nbr + (size_t)kap * n_out + my_rows[q]) : -1;
    };
    if (GROUPED) {
      // Grouped offsets (TF32, staged rows of c_in = 4, 8 or 16 floats): the 128-byte operand row of a
      // step holds the rows' neighbours at opk consecutive offsets side by side; a missing neighbour is
      // a zero-filled piece, so no row is ever switched off.  The filter slab of the group is packed to match.
      const int cpc = c_in >> 2;                   // 16-byte chunks per offset
      // (the loops over the 32-row groups are kept rolled: this path runs four steps per CTA, and as
      //  straight-line code it spent most of its time waiting for instruction fetches)
      for (int j = slot; j < n_iter; j += S) {
        const int group = act_list[j];
        if (j >= S) {
          if (!mbar_wait_warp(smem_u32(empty_bars + slot), par ^ 1u, abort_flag)) break;
          tc_fence_after();
        }
        if (part == 0 && lane == 0) {
          const uint4 *bsrc = packed + (size_t)group * (size_t)(p.n_pad * 8) + (size_t)nt0 * (size_t)(p.tile_n * 8);
          const uint32_t bar = smem_u32(fulla_bars + slot), nbytes = (uint32_t)p.b_bytes;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(nbytes) : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           slot_addr + (uint32_t)TC_A_BYTES),
                       "l"(bsrc), "r"(nbytes), "r"(bar)
                       : "memory");
        }
#pragma unroll 1
        for (int q = q0; q < q0 + q_per; ++q) {
          const int row = m0 + q * 32 + lane;
          const int my_row = row < n_rows ? ((order && !p.nbr_by_pos) ? __ldg(order + row) : row) : -1;
          int idx[8];
#pragma unroll
          for (int o = 0; o < 8; ++o) {
            const int kap = group * p.opk + o;
            idx[o] = (o < p.opk && kap < K && my_row >= 0) ? __ldg(nbr + (size_t)kap * n_out + my_row) : -1;
          }
          if (lane == 0) slot_masks[slot * 4 + q] = 0u;          // every row takes part
          const uint32_t a_row = slot_addr + (uint32_t)(q * 4 + (lane >> 3)) * 1024u + sw * 128u;
#pragma unroll
          for (int o = 0; o < 8; ++o) {
            if (o >= p.opk) break;
            const int src_row = idx[o];
            const float *fp = features + (size_t)(src_row >= 0 ? src_row : 0) * c_in;
#pragma unroll 1
            for (int cc = 0; cc < cpc; ++cc) {
              const uint32_t chunk = (uint32_t)(o * cpc + cc);
              cp_async16_cg(a_row + ((chunk ^ sw) << 4), fp + cc * 4, src_row >= 0 ? 16u : 0u);
            }
          }
        }
        cp_async_commit();
        cp_async_wait(0);
        fence_async_smem();
        mbar_arrive(smem_u32(fulla_bars + slot));
        par ^= 1u;
      }
    } else {
    if (slot < n_iter) load_rows(slot, nxt);
    for (int j = slot; j < n_iter; j += S) {
      const int act = j / p.k_groups, slab0 = (j - act * p.k_groups) * p.sps;
      const int n_sub = min(p.sps, p.k_slabs - slab0);   // slabs of this step
      const int kappa = act_list[act];
#pragma unroll
      for (int q = 0; q < 4; ++q) src[q] = nxt[q];
      if (j + S < n_iter) load_rows(j + S, nxt);  // neighbour rows of this warp's next step
      if (j >= S) {
        if (!mbar_wait_warp(smem_u32(empty_bars + slot), par ^ 1u, abort_flag)) break;
        tc_fence_after();
      }
      if (part == 0 && lane == 0) {  // the pre-packed filter slab of this step: one bulk copy
        const uint4 *bsrc = packed + ((size_t)kappa * p.k_slabs + slab0) * (size_t)(p.n_pad * 8) +
                            (size_t)nt0 * (size_t)(p.tile_n * 8);
        const uint32_t bar = smem_u32(fulla_bars + slot), nbytes = (uint32_t)(n_sub * p.b_bytes);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(nbytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         slot_addr + (uint32_t)(p.sps * TC_A_BYTES)),
                     "l"(bsrc), "r"(nbytes), "r"(bar)
                     : "memory");
      }
      uint32_t present = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // rows of this step that the MMA must leave alone
        const unsigned have = __ballot_sync(0xffffffffu, src[q] >= 0);
        if (lane == 0 && q >= q0 && q < q0 + q_per) slot_masks[slot * 4 + q] = ~have;
      }
      for (int ss = 0; ss < n_sub; ++ss) {
      const int ch0 = (slab0 + ss) * TC_SLAB;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (src[q] >= 0 && ch0 < c_in) {
          const float *fp = features + (size_t)src[q] * c_in + ch0;
          const uint32_t a_row = slot_addr + (uint32_t)(ss * TC_A_BYTES) + row_off[q];
          if (vec_ok) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {  // chunks past the last channel are zero-filled
              bool ok = ch0 + c * 4 < c_in;
              if (STAGED) cp_async16_cg(a_row + ((c ^ sw) << 4), ok ? (const void *)(fp + c * 4) : (const void *)features, ok ? 16u : 0u);
              else cp_async16(a_row + ((c ^ sw) << 4), ok ? (const void *)(fp + c * 4) : (const void *)features, ok ? 16u : 0u);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 8; ++c)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                bool ok = ch0 + c * 4 + e < c_in;
                cp_async4(a_row + ((c ^ sw) << 4) + 4u * e, ok ? (const void *)(fp + c * 4 + e) : (const void *)features,
                          ok ? 4u : 0u);
              }
          }
          present |= 1u << q;
        }
      }
      }
      cp_async_commit();
      cp_async_wait(0);
      // copies landed: round the gathered rows to TF32 in place
      for (int ss = 0; ss < (STAGED ? 0 : n_sub); ++ss)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (!STAGED && (present & (1u << q))) {
          uint8_t *row = slot_ptr + (size_t)ss * TC_A_BYTES + row_off[q];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 *ptr = (uint4 *)(row + ((c ^ sw) << 4));
            uint4 v = *ptr;
            v.x = to_tf32(__uint_as_float(v.x));
            v.y = to_tf32(__uint_as_float(v.y));
            v.z = to_tf32(__uint_as_float(v.z));
            v.w = to_tf32(__uint_as_float(v.w));
            *ptr = v;
          }
        }
      }
      if (present) fence_async_smem();  // make this lane's rows visible to the tensor core
      mbar_arrive(smem_u32(fulla_bars + slot));
      par ^= 1u;
    }
    }   // one offset per step
  } else if (warp == mma_warp && lane == 0) {
    // ================================ MMA issuer ============================================
    // The issuing thread is the serial bottleneck of the pipeline, so its loop is kept to a
    // handful of instructions: slot index, parity and descriptor halves are running values.
    // fp32 accumulator; operand formats: kind::tf32 2 = TF32; kind::f16 0 = fp16, 1 = bf16
    const uint32_t fmt = F16 ? (uint32_t)p.fmt16 : 2u;
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.tile_n >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
    const uint32_t a_lo0 = desc_lo(smem_base), slot_step = (uint32_t)stage_bytes >> 4, n_step = (uint32_t)(p.tile_n * 128) >> 4;
    const uint32_t fulla0 = smem_u32(fulla_bars), empty0 = smem_u32(empty_bars);
    uint32_t s = 0, par = 0, a_lo = a_lo0;
    int grp = 0;  // which slab group of its kernel offset the current step is
    for (int it = 0; it < n_iter; ++it) {
      if (!mbar_wait(fulla0 + s * 8u, par, abort_flag)) break;
      tc_fence_after();
      const uint4 off = *(const uint4 *)(slot_masks + s * 4u);  // rows to leave untouched
      const int n_sub = min(p.sps, p.k_slabs - grp * p.sps);
      for (int ss = 0; ss < n_sub; ++ss) {
        const uint32_t an = a_lo + (uint32_t)ss * (TC_A_BYTES >> 4);
        // k-steps of this slab that hold real channels (the rest of the last slab is zero on both
        // sides: a 3-channel first layer needs one MMA per step, not four)
        const int n_kk = grp * p.sps + ss == p.k_slabs - 1 ? p.last_kk : 4;
        for (int nt = 0; nt < p.nt_cta; ++nt) {
          const uint32_t dn = tmem_base + (uint32_t)(nt * p.tile_n);
          const uint32_t bn = a_lo + (uint32_t)(p.sps * TC_A_BYTES >> 4) + (uint32_t)ss * ((uint32_t)p.b_bytes >> 4) + (uint32_t)nt * n_step;
          if (n_kk == 4) {   // the common case, straight-line
            if (F16) {
              mma_f16_ss_masked(dn, an, bn, idesc, off);
              mma_f16_ss_masked(dn, an + 2u, bn + 2u, idesc, off);
              mma_f16_ss_masked(dn, an + 4u, bn + 4u, idesc, off);
              mma_f16_ss_masked(dn, an + 6u, bn + 6u, idesc, off);
            } else {
              mma_tf32_ss_masked(dn, an, bn, idesc, off);
              mma_tf32_ss_masked(dn, an + 2u, bn + 2u, idesc, off);
              mma_tf32_ss_masked(dn, an + 4u, bn + 4u, idesc, off);
              mma_tf32_ss_masked(dn, an + 6u, bn + 6u, idesc, off);
            }
          } else {
            for (int kk = 0; kk < n_kk; ++kk) {
              if (F16) mma_f16_ss_masked(dn, an + 2u * (uint32_t)kk, bn + 2u * (uint32_t)kk, idesc, off);
              else mma_tf32_ss_masked(dn, an + 2u * (uint32_t)kk, bn + 2u * (uint32_t)kk, idesc, off);
            }
          }
        }
      }
      if (++grp == p.k_groups) grp = 0;
      mma_commit(empty0 + s * 8u);
      a_lo += slot_step;
      if (++s == (uint32_t)S) { s = 0; par ^= 1u; a_lo = a_lo0; }
    }
    mma_commit(smem_u32(done_bar));  // arrives once everything issued above has retired
  }

  // ================================ epilogue: TMEM -> registers -> global ====================
  if (warp < TC_EPI_WARPS) {
    __syncwarp();
    bool ok = !*abort_flag;
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_iter > 0) ok = mbar_wait_warp(smem_u32(done_bar), 0u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
    tc_fence_after();
    const int m_tile = m0 + warp * 32 + lane;
    const int m = m_tile < n_rows ? (order ? __ldg(order + m_tile) : m_tile) : n_rows;
    const int col0 = nt0 * p.tile_n;   // first output channel of this CTA
    for (int c0 = 0; c0 < p.n_cta && col0 + c0 < c_out; c0 += 16) {
      uint32_t r[16];
      if (ok && n_iter > 0) {
        uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) r[q] = 0u;
      }
      if (m < n_rows) {
        float *op = out + (size_t)m * c_out + col0 + c0;
        if ((c_out & 3) == 0) {
#pragma unroll
          for (int q = 0; q < 16; q += 4)
            if (col0 + c0 + q < c_out)
              *(float4 *)(op + q) = make_float4(__uint_as_float(r[q]), __uint_as_float(r[q + 1]),
                                                __uint_as_float(r[q + 2]), __uint_as_float(r[q + 3]));
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q)
            if (col0 + c0 + q < c_out) op[q] = __uint_as_float(r[q]);
        }
      }
    }
  }
  // a wait gave up: the instructions already issued still arrive on done_bar (committed above on
  // every path); let them retire before the accumulators are handed back
  if (warp == mma_warp && lane == 0 && *abort_flag && n_iter > 0) mbar_wait_drain(smem_u32(done_bar), 0u);
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) atomicOr(status, 16);
  if (warp == mma_warp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

static size_t tc_smem_bytes(const TcParams &p) {
  return (size_t)p.stages * p.sps * (TC_A_BYTES + p.b_bytes) + 1024 /*alignment slack*/ + TC_CTRL_BYTES;
}

// 16-bit operands: filters [K, c_in, c_out] fp32 -> [K][k_slabs][n_pad rows][64 fp16 or bf16], same
// swizzle (a 16-byte chunk holds 8 input channels).
template <bool BF16>
__global__ void pack_filters_16_kernel(const float *__restrict__ filters, int K, int c_in, int c_out, TcParams p,
                                        uint4 *__restrict__ packed) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)K * p.k_slabs * p.n_pad * 8;
  if (t >= total) return;
  int chunk = (int)(t & 7);
  long long r = t >> 3;
  int n = (int)(r % p.n_pad);
  r /= p.n_pad;
  int slab = (int)(r % p.k_slabs);
  int kappa = (int)(r / p.k_slabs);
  uint32_t v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float f[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int ci = slab * 64 + chunk * 8 + q * 2 + h;
      f[h] = (ci < c_in && n < c_out) ? filters[((size_t)kappa * c_in + ci) * c_out + n] : 0.f;
    }
    v[q] = BF16 ? pack_bf16x2(f[0], f[1]) : pack_f16x2(f[0], f[1]);
  }
  size_t block = ((size_t)kappa * p.k_slabs + slab) * (size_t)(p.n_pad * 8);
  size_t off = (size_t)(n >> 3) * 64 + (size_t)(n & 7) * 8 + (size_t)(chunk ^ (n & 7));
  packed[block + off] = make_uint4(v[0], v[1], v[2], v[3]);
}

int conv_fwd_16(const float *features, int n_in, int c_in, bool bf16, const void *packed, int K, int c_out,
                const int32_t *nbr, int n_out, float *out, int32_t *status, void *scratch, size_t scratch_bytes,
                const int32_t *n_out_dev, const int32_t *order, bool prestaged, bool table_in_order, cudaStream_t st) {
  if (K > 256) return fail(SSC_ERR_INVALID, "conv_fwd(16-bit): kernel volume %d > 256", K);
  const int words = f16_row_words(c_in);
  if (scratch == nullptr || scratch_bytes + 16 < conv_f16_scratch_bytes(n_in, c_in) || ((uintptr_t)scratch & 15u) != 0)
    return fail(SSC_ERR_INVALID, "conv_fwd(16-bit): needs the staging buffer of ssc_conv_scratch_bytes (16-byte aligned)");
  int grid = ceil_div(n_out, TC_M);
  const int sms = sm_count();
  TcParams p;
  if (!tc_params(words, c_out, p, grid < 2 * sms))
    return fail(SSC_ERR_INVALID, "conv_fwd(16-bit): c_out %d / kernel volume %d not supported", c_out, K);
  if (grid * (p.n_tiles / p.nt_cta) <= sms) tc_params(words, c_out, p, grid < 2 * sms, true);
  p.fmt16 = bf16 ? 1 : 0;
  p.nbr_by_pos = (table_in_order && order) ? 1 : 0;
  if (!prestaged) {
    int rc = stage_features_16(features, n_in, c_in, bf16, scratch, st);
    if (rc != SSC_OK) return rc;
  }
  const size_t smem = tc_smem_bytes(p);
  auto kernel = conv_fwd_tf32_kernel<true, true>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd(16-bit): smem attribute: %s", cudaGetErrorString(e));
  const dim3 grid2(grid, p.n_tiles / p.nt_cta);
  { kernel<<<grid2, p.threads, smem, st>>>((const float *)scratch, words, (const uint4 *)packed, K, c_out, nbr, n_out, out, status, p, n_out_dev, order); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_16");
  return SSC_OK;
}

// Smallest problem (in 128-row tiles) for which the extra staging launch pays for itself.
constexpr int kStagingMinTiles = 8;

int conv_fwd_tf32(const float *features, int n_in, int c_in, const void *packed, int K, int c_out,
                  const int32_t *nbr, int n_out, float *out, int32_t *status, void *scratch, size_t scratch_bytes,
                  const int32_t *n_out_dev, const int32_t *order, bool prestaged, bool table_in_order, cudaStream_t st) {
  TcParams p;
  if (K > 256) return fail(SSC_ERR_INVALID, "conv_fwd(tf32): kernel volume %d > 256", K);
  int grid = ceil_div(n_out, TC_M);
  const bool split_n = grid < 2 * sm_count();   // few row tiles: spread the N tiles over CTAs too
  const int opk = tf32_offsets_per_row(c_in);
  if (!tc_params(c_in, c_out, p, split_n, false, opk)) return fail(SSC_ERR_INVALID, "conv_fwd(tf32): c_out %d / kernel volume %d not supported", c_out, K);
  if (grid * (p.n_tiles / p.nt_cta) <= sm_count()) tc_params(c_in, c_out, p, split_n, true, opk);
  p.nbr_by_pos = (table_in_order && order) ? 1 : 0;
  size_t smem = tc_smem_bytes(p);
  // With a staging buffer the feature rows are rounded to TF32 once, up front, instead of after
  // every gather (a row is gathered about K/2 times).
  const int c_pad = (c_in + 3) & ~3;  // row stride of the staged image (zero-padded channels)
  const size_t stage_need = conv_tf32_scratch_bytes(n_in, c_in);
  const bool fits = scratch != nullptr && scratch_bytes + 16 >= stage_need && ((uintptr_t)scratch & 15u) == 0;
  if (prestaged && !fits) return fail(SSC_ERR_INVALID, "conv_fwd(tf32): SSC_CONV_PRESTAGED without the staged image in scratch");
  // layers with few input channels have their filters packed for several offsets per operand row,
  // which the kernel can only feed from the staged (padded) rows
  if (opk > 1 && !fits) return fail(SSC_ERR_SCRATCH, "conv_fwd(tf32): a layer with %d input channels needs the staging buffer (ssc_conv_scratch_bytes)", c_in);
  const bool staged = fits && (prestaged || grid >= kStagingMinTiles || opk > 1);
  if (staged && !prestaged) {
    int rc = stage_features(features, n_in, c_in, scratch, st);
    if (rc != SSC_OK) return rc;
  }
  auto kernel = opk > 1 ? conv_fwd_tf32_kernel<true, false, true> : staged ? conv_fwd_tf32_kernel<true> : conv_fwd_tf32_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd(tf32): smem attribute: %s", cudaGetErrorString(e));
  const dim3 grid2(grid, p.n_tiles / p.nt_cta);
  { kernel<<<grid2, p.threads, smem, st>>>(staged ? (const float *)scratch : features, staged ? c_pad : c_in, (const uint4 *)packed, K, c_out,
                                        nbr, n_out, out, status, p, n_out_dev, order); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_tf32");
  return SSC_OK;
}

}  // namespace ssc

using namespace ssc;

static bool is16(int precision) { return precision == SSC_PREC_F16 || precision == SSC_PREC_BF16; }

extern "C" size_t ssc_conv_packed_bytes(int K, int c_in, int c_out, int precision) {
  if ((precision != SSC_PREC_TF32 && !is16(precision)) || K < 1 || c_in < 1 || c_out < 1) return 0;
  TcParams p;
  if (!tc_params(is16(precision) ? f16_row_words(c_in) : c_in, c_out, p)) return 0;
  if (!is16(precision) && tf32_offsets_per_row(c_in) > 1)
    return (size_t)ceil_div(K, tf32_offsets_per_row(c_in)) * p.n_pad * 128;
  return (size_t)K * p.k_slabs * p.n_pad * 128;
}

extern "C" int ssc_conv_pack_filters(const float *filters, int K, int c_in, int c_out, int precision, void *packed,
                                     void *stream) {
  SSC_REQUIRE(precision == SSC_PREC_TF32 || is16(precision), "conv_pack_filters: only SSC_PREC_TF32, SSC_PREC_F16 and SSC_PREC_BF16 have a packed form");
  SSC_REQUIRE(filters && packed && K >= 1 && c_in >= 1 && c_out >= 1, "conv_pack_filters: bad arguments");
  TcParams p;
  SSC_REQUIRE(tc_params(is16(precision) ? f16_row_words(c_in) : c_in, c_out, p), "conv_pack_filters: c_out %d not supported (max 512)", c_out);
  if (precision == SSC_PREC_TF32 && tf32_offsets_per_row(c_in) > 1) {
    const int opk = tf32_offsets_per_row(c_in), n_groups = ceil_div(K, opk);
    const long long total_g = (long long)n_groups * p.n_pad * 8;
    { pack_filters_tf32_grouped_kernel<<<ceil_div(total_g, 256), 256, 0, as_stream(stream)>>>(filters, K, c_in, c_out, (c_in + 3) & ~3, opk,
                                                                                         n_groups, p.n_pad, (uint4 *)packed); note_launches(1); }
    SSC_CHECK_LAUNCH("pack_filters");
    return SSC_OK;
  }
  long long total = (long long)K * p.k_slabs * p.n_pad * 8;
  const int blocks = ceil_div(total, 256);
  if (precision == SSC_PREC_F16) { pack_filters_16_kernel<false><<<blocks, 256, 0, as_stream(stream)>>>(filters, K, c_in, c_out, p, (uint4 *)packed); note_launches(1); }
  else if (precision == SSC_PREC_BF16) { pack_filters_16_kernel<true><<<blocks, 256, 0, as_stream(stream)>>>(filters, K, c_in, c_out, p, (uint4 *)packed); note_launches(1); }
  else { pack_filters_tf32_kernel<<<blocks, 256, 0, as_stream(stream)>>>(filters, K, c_in, c_out, p, (uint4 *)packed); note_launches(1); }
  SSC_CHECK_LAUNCH("pack_filters");
  return SSC_OK;
}
