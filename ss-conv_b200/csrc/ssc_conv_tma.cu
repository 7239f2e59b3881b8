// Persistent gather-GEMM: TMA row gather (cp.async.bulk.tensor ... tile::gather4) feeding
// tcgen05.mma, one CTA per SM.
//
// The 128-row output tiles are dealt to the CTAs in contiguous runs; a CTA works through its
// run in passes of T tiles whose accumulators sit side by side in one half of tensor memory
// (T = 256 / padded output channels).  Inside a pass the loop order is
//     kernel offset  >  32-channel slab  >  tile,
// so a filter slab is fetched once per pass and reused by every tile of the pass, and the two
// halves of tensor memory alternate between passes: while the four epilogue warps drain pass p,
// the producer and the MMA thread already work on pass p+1.
//
//   producer warp : reads the neighbour rows of the pass (lane l owns rows 4l..4l+3 of every
//                   tile), skips offsets without any neighbour, and for every (offset, slab,
//                   tile) arms one ring slot: each lane issues ONE gather4 that drops four
//                   128-byte row slabs into the K-major 128-byte-swizzled operand layout.
//                   Rows without a neighbour use an out-of-range row index, which the copy
//                   engine zero-fills.  No thread touches the gathered data: the copy engine
//                   writes shared memory, the tensor core reads it.
//   MMA thread    : consumes ring slots in order; a slot's tag says which accumulator it feeds
//                   and whether it opens / closes the use of a filter slot.
//   epilogue warps: tcgen05.ld the accumulators of a finished pass and store each output row
//                   once; then hand the half back.
//
// The gathered operand must already be TF32-representable: stage_features_kernel makes a
// round-to-nearest copy of the feature rows (plus the zero row) once per call, so that a row
// gathered ~K/2 times is rounded once.
//
// Measured on B200 (64 -> 76 channels, 3^3 offsets, 130 k output rows): the copy engine retires
// one gather4 (4 x 128 bytes) about every 58 cycles per SM, which makes this kernel ~2.4x slower
// than gathering with the load-store units (ssc_conv_tc.cu); it is kept as an option
// (SSC_TC_VARIANT=gather4) for wider rows and as the reference point for that measurement.
//
// Every wait is bounded; on expiry the waiting thread raises the CTA's abort flag, every other
// role leaves its loop at its next wait, the kernel releases its tensor memory and reports
// through `status`.
#include <cuda.h>
#include <stdlib.h>

#include "ssc_common.cuh"
#include "ssc_tc_ptx.cuh"

namespace ssc {

bool tc_operand_layout(int c_in, int c_out, int *k_slabs, int *n_pad, int *tile_n, int *n_tiles);

constexpr int G4_M = 128;
constexpr int G4_A_BYTES = G4_M * 128;
constexpr int G4_MAX_A = 12;            // gathered-operand ring slots
constexpr int G4_MAX_B = 4;             // filter-slab ring slots
constexpr int G4_MAX_T = 4;             // tiles per pass
constexpr int G4_CTRL_BYTES = 1024;
constexpr int G4_THREADS = 192;         // warps 0-3 epilogue, warp 4 producer, warp 5 MMA + TMEM
constexpr uint32_t G4_TMEM_COLS = 512;

// slot tag written by the producer, read by the MMA thread
constexpr uint32_t TAG_TILE_MASK = 0x7u;
constexpr uint32_t TAG_OPEN_B = 1u << 3;    // first tile of a (offset, slab): wait for the filter slab
constexpr uint32_t TAG_CLOSE_B = 1u << 4;   // last tile of a (offset, slab): release the filter slot
constexpr uint32_t TAG_END_PASS = 1u << 5;  // no data: the pass is complete
constexpr uint32_t TAG_END_ALL = 1u << 6;   // no data: nothing follows

struct G4Params {
  int k_slabs, n_pad, b_bytes;
  int a_slots, b_slots;
  int T;              // tiles per pass
  int halves;         // 2: passes alternate between TMEM columns [0,256) and [256,512)
  int zero_row;       // row index of the all-zero row in the staged feature image
};

__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int r0, int r1, int r2,
                                            int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// features [n_in, c] fp32 -> staged [n_in + 1, c]: round-to-nearest TF32 copy, last row zero.
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

__global__ void __launch_bounds__(G4_THREADS, 1)
conv_fwd_tf32_gather4_kernel(const __grid_constant__ CUtensorMap feat_map, const uint4 *__restrict__ packed, int K,
                             int c_out, const int32_t *__restrict__ nbr, int n_out, float *__restrict__ out,
                             int32_t *status, G4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *b_ring = smem + (size_t)p.a_slots * G4_A_BYTES;
  uint8_t *ctrl = b_ring + (size_t)p.b_slots * p.b_bytes;
  uint64_t *full_a = (uint64_t *)ctrl;                       // [G4_MAX_A]
  uint64_t *empty_a = full_a + G4_MAX_A;                     // [G4_MAX_A]
  uint64_t *full_b = empty_a + G4_MAX_A;                     // [G4_MAX_B]
  uint64_t *empty_b = full_b + G4_MAX_B;                     // [G4_MAX_B]
  uint64_t *acc_full = empty_b + G4_MAX_B;                   // [2] MMAs of a pass retired
  uint64_t *acc_info = acc_full + 2;                         // [2] started[] of the pass is written
  uint64_t *acc_empty = acc_info + 2;                        // [2] epilogue has drained the half
  uint32_t *tags = (uint32_t *)(acc_empty + 2);              // [G4_MAX_A]
  uint32_t *started = tags + G4_MAX_A;                       // [2] tiles of the pass that received an MMA
  uint32_t *tmem_slot = started + 2;
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total_tiles = (n_out + G4_M - 1) / G4_M;
  // contiguous run of tiles for this CTA: the first `extra` CTAs take one tile more
  const int base = total_tiles / (int)gridDim.x, extra = total_tiles % (int)gridDim.x;
  const int my_tiles = base + ((int)blockIdx.x < extra ? 1 : 0);
  const int first_tile = (int)blockIdx.x * base + min((int)blockIdx.x, extra);
  const int n_pass = (my_tiles + p.T - 1) / p.T;

  if (tid == 0) {
    for (int s = 0; s < p.a_slots; ++s) {
      mbar_init(smem_u32(full_a + s), 1);
      mbar_init(smem_u32(empty_a + s), 1);
    }
    for (int s = 0; s < p.b_slots; ++s) {
      mbar_init(smem_u32(full_b + s), 1);
      mbar_init(smem_u32(empty_b + s), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(smem_u32(acc_full + h), 1);
      mbar_init(smem_u32(acc_info + h), 1);
      mbar_init(smem_u32(acc_empty + h), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(G4_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t b_base = smem_u32(b_ring);

  if (warp == 4) {
    // ====================================== producer ========================================
    uint32_t sa = 0, pha = 0, sb = 0, phb = 0;
    bool live = true;
    // Claim the next operand slot: wait until its previous MMAs have retired.
    auto claim_a = [&]() -> bool { return mbar_wait_warp(smem_u32(empty_a + sa), pha ^ 1u, abort_flag); };
    auto next_a = [&]() {
      if (++sa == (uint32_t)p.a_slots) { sa = 0; pha ^= 1u; }
    };
    for (int pass = 0; pass < n_pass && live; ++pass) {
      const int t_cnt = min(p.T, my_tiles - pass * p.T);
      const int row0 = (first_tile + pass * p.T) * G4_M + lane * 4;
      int cur[G4_MAX_T][4], nxt[G4_MAX_T][4];
      auto load_rows = [&](int kappa, int(*dst)[4]) {
        const int32_t *src = nbr + (size_t)kappa * n_out;
#pragma unroll
        for (int t = 0; t < G4_MAX_T; ++t)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int r = row0 + t * G4_M + q;
            dst[t][q] = (t < t_cnt && r < n_out) ? __ldg(src + r) : -1;
          }
      };
      load_rows(0, nxt);
      for (int kappa = 0; kappa < K && live; ++kappa) {
#pragma unroll
        for (int t = 0; t < G4_MAX_T; ++t)
#pragma unroll
          for (int q = 0; q < 4; ++q) cur[t][q] = nxt[t][q];
        if (kappa + 1 < K) load_rows(kappa + 1, nxt);
        uint32_t mask = 0;
#pragma unroll
        for (int t = 0; t < G4_MAX_T; ++t) {
          const bool any = (cur[t][0] & cur[t][1] & cur[t][2] & cur[t][3]) >= 0;  // some index non-negative
          if (__ballot_sync(0xffffffffu, any)) mask |= 1u << t;
        }
        if (mask == 0) continue;
        const int last_t = 31 - __clz(mask), first_t = __ffs(mask) - 1;
        for (int slab = 0; slab < p.k_slabs && live; ++slab) {
          // filter slab of (kappa, slab) into the next filter slot
          if (!mbar_wait_warp(smem_u32(empty_b + sb), phb ^ 1u, abort_flag)) { live = false; break; }
          if (lane == 0) {
            const uint4 *bsrc = packed + ((size_t)kappa * p.k_slabs + slab) * (size_t)(p.n_pad * 8);
            const uint32_t bar = smem_u32(full_b + sb);
            mbar_expect_tx(bar, (uint32_t)p.b_bytes);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             b_base + sb * (uint32_t)p.b_bytes),
                         "l"(bsrc), "r"((uint32_t)p.b_bytes), "r"(bar)
                         : "memory");
          }
          if (++sb == (uint32_t)p.b_slots) { sb = 0; phb ^= 1u; }
#pragma unroll
          for (int t = 0; t < G4_MAX_T; ++t) {
            if (!(mask & (1u << t)) || !live) continue;
            if (!claim_a()) { live = false; continue; }
            const uint32_t bar = smem_u32(full_a + sa);
            if (lane == 0) {
              tags[sa] = (uint32_t)t | (t == first_t ? TAG_OPEN_B : 0u) | (t == last_t ? TAG_CLOSE_B : 0u);
              mbar_expect_tx(bar, (uint32_t)G4_A_BYTES);
            }
            int r[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) r[q] = cur[t][q] < 0 ? p.zero_row : cur[t][q];
            tma_gather4(smem_base + sa * (uint32_t)G4_A_BYTES + (uint32_t)lane * 512u, &feat_map, bar, slab * 32, r[0], r[1],
                        r[2], r[3]);
            next_a();
          }
        }
      }
      if (live) {  // tell the MMA thread that the pass is complete
        if (!claim_a()) { live = false; break; }
        if (lane == 0) {
          tags[sa] = TAG_END_PASS | (pass + 1 == n_pass ? TAG_END_ALL : 0u);
          mbar_arrive(smem_u32(full_a + sa));
        }
        next_a();
      }
    }
  } else if (warp == 5 && lane == 0) {
    // ====================================== MMA issuer ======================================
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.n_pad >> 3) << 17) | ((uint32_t)(G4_M >> 4) << 24);
    uint32_t sa = 0, pha = 0, sb = 0, phb = 0;
    uint32_t began = 0;      // tiles of the current pass that already hold a partial sum
    int pass = 0;
    bool acc_ready = false;  // the current half has been handed back by the epilogue
    while (pass < n_pass) {
      if (!mbar_wait(smem_u32(full_a + sa), pha, abort_flag)) break;
      const uint32_t tag = tags[sa];
      const uint32_t half = p.halves == 2 ? (uint32_t)(pass & 1) : 0u;
      const uint32_t use = (uint32_t)(p.halves == 2 ? pass >> 1 : pass);  // how often this half was used before
      if (tag & TAG_END_PASS) {
        started[half] = began;
        mbar_arrive(smem_u32(acc_info + half));
        if (began) mma_commit(smem_u32(acc_full + half));
        else mbar_arrive(smem_u32(acc_full + half));
        mbar_arrive(smem_u32(empty_a + sa));
        began = 0;
        acc_ready = false;
        ++pass;
      } else {
        if (!acc_ready) {  // first MMA of the pass: the half must have been drained
          if (!mbar_wait(smem_u32(acc_empty + half), (use & 1u) ^ 1u, abort_flag)) break;
          acc_ready = true;
        }
        if (tag & TAG_OPEN_B) {
          if (!mbar_wait(smem_u32(full_b + sb), phb, abort_flag)) break;
        }
        tc_fence_after();
        const uint32_t t = tag & TAG_TILE_MASK;
        const uint32_t d = tmem_base + half * 256u + t * (uint32_t)p.n_pad;
        const uint32_t a_lo = desc_lo(smem_base + sa * (uint32_t)G4_A_BYTES);
        const uint32_t b_lo = desc_lo(b_base + sb * (uint32_t)p.b_bytes);
        mma_tf32_ss(d, a_lo, b_lo, idesc, (began >> t) & 1u);
        mma_tf32_ss(d, a_lo + 2u, b_lo + 2u, idesc, 1u);
        mma_tf32_ss(d, a_lo + 4u, b_lo + 4u, idesc, 1u);
        mma_tf32_ss(d, a_lo + 6u, b_lo + 6u, idesc, 1u);
        began |= 1u << t;
        mma_commit(smem_u32(empty_a + sa));
        if (tag & TAG_CLOSE_B) {
          mma_commit(smem_u32(empty_b + sb));
          if (++sb == (uint32_t)p.b_slots) { sb = 0; phb ^= 1u; }
        }
      }
      if (++sa == (uint32_t)p.a_slots) { sa = 0; pha ^= 1u; }
    }
  } else if (warp < 4) {
    // ====================================== epilogue ========================================
    const int n_cols = (c_out + 15) & ~15;
    for (int pass = 0; pass < n_pass; ++pass) {
      const uint32_t half = p.halves == 2 ? (uint32_t)(pass & 1) : 0u;
      const uint32_t use = (uint32_t)(p.halves == 2 ? pass >> 1 : pass);
      bool ok = mbar_wait_warp(smem_u32(acc_info + half), use & 1u, abort_flag);
      ok = ok && mbar_wait_warp(smem_u32(acc_full + half), use & 1u, abort_flag);
      if (!ok) break;  // uniform across the warp
      tc_fence_after();
      const uint32_t began = started[half];
      const int t_cnt = min(p.T, my_tiles - pass * p.T);
      for (int t = 0; t < t_cnt; ++t) {
        const int m = (first_tile + pass * p.T + t) * G4_M + warp * 32 + lane;
        const bool have = (began >> t) & 1u;
        for (int c0 = 0; c0 < n_cols; c0 += 16) {
          uint32_t r[16];
          if (have) {
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + half * 256u + (uint32_t)(t * p.n_pad + c0);
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
          if (m < n_out) {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_empty + half));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) atomicOr(status, 16);
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(G4_TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return (EncodeTiledFn)sym;
  }();
  return fn;
}

static int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1) return 148;
    return v;
  }();
  return n;
}

static bool g4_params(int c_in, int c_out, G4Params &p) {
  int tile_n, n_tiles;
  if (!tc_operand_layout(c_in, c_out, &p.k_slabs, &p.n_pad, &tile_n, &n_tiles)) return false;
  if (n_tiles != 1 || p.n_pad > 256 || (c_in & 3) != 0) return false;
  p.b_bytes = p.n_pad * 128;
  p.halves = 2;
  p.T = 256 / p.n_pad;
  if (p.T > G4_MAX_T) p.T = G4_MAX_T;
  p.b_slots = p.b_bytes <= 16 * 1024 ? 3 : 2;
  const int budget = 227 * 1024 - 1024 - G4_CTRL_BYTES - p.b_slots * p.b_bytes;
  p.a_slots = budget / G4_A_BYTES;
  if (p.a_slots > G4_MAX_A) p.a_slots = G4_MAX_A;
  return p.a_slots >= 2;
}

// Same for channel counts that are not a multiple of four: rows padded with zeros to c_pad floats.
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

// staged = TF32-rounded copy of features [n_in, c_in] plus one all-zero row; the row stride is
// c_in rounded up to a multiple of four floats (16-byte copies in the convolution kernel).
int stage_features(const float *features, int n_in, int c_in, void *staged, cudaStream_t st) {
  const int c_pad = (c_in + 3) & ~3;
  if (c_pad == c_in && ((uintptr_t)features & 15u) == 0) {
    const long long n_vec = (long long)n_in * c_in / 4, total_vec = ((long long)n_in + 1) * c_in / 4;
    int blocks = ceil_div(total_vec, 256 * 4);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    { stage_features_kernel<<<blocks, 256, 0, st>>>((const float4 *)features, n_vec, total_vec, (uint4 *)staged); note_launches(1); }
  } else {
    const long long total = ((long long)n_in + 1) * c_pad;
    int blocks = ceil_div(total, 256 * 4);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    { stage_features_padded_kernel<<<blocks, 256, 0, st>>>(features, n_in, c_in, c_pad, total, (uint32_t *)staged); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("stage_features");
  return SSC_OK;
}

size_t conv_gather4_scratch_bytes(int n_in, int c_in, int c_out) {
  (void)c_out;
  return ((size_t)n_in + 1) * (size_t)((c_in + 3) & ~3) * sizeof(float);
}

// returns -1 when this variant does not apply (the caller then uses another kernel)
int conv_fwd_tf32_gather4(const float *features, int n_in, int c_in, const void *packed, int K, int c_out,
                          const int32_t *nbr, int n_out, float *out, int32_t *status, void *scratch,
                          size_t scratch_bytes, cudaStream_t st) {
  G4Params p;
  if (!g4_params(c_in, c_out, p)) return -1;   // (requires c_in % 4 == 0, so the staged row stride is c_in)
  const size_t need = ((size_t)n_in + 1) * (size_t)c_in * sizeof(float);
  if (scratch == nullptr || scratch_bytes < need || ((uintptr_t)scratch & 127u) != 0) return -1;
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return -1;

  if (((uintptr_t)features & 15u) != 0) return -1;
  int rc = stage_features(features, n_in, c_in, scratch, st);
  if (rc != SSC_OK) return rc;

  CUtensorMap map;
  // The map covers the n_in real rows only: index n_in (used for "no neighbour") is out of
  // bounds, so the copy engine fills zeros without touching memory.  The staged image still holds
  // a zero row there, which keeps the result right on a device that would fetch it instead.
  const cuuint64_t dims[2] = {(cuuint64_t)c_in, (cuuint64_t)(n_in > 0 ? n_in : 1)};
  const cuuint64_t strides[1] = {(cuuint64_t)c_in * sizeof(float)};
  const cuuint32_t box[2] = {32u, 1u};  // gather4 takes one row per index
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, scratch, dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(SSC_ERR_CUDA, "conv_fwd(tf32): tensor map encode failed (%d)", (int)cr);
  p.zero_row = n_in;

  const size_t smem = (size_t)p.a_slots * G4_A_BYTES + (size_t)p.b_slots * p.b_bytes + G4_CTRL_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(conv_fwd_tf32_gather4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd(tf32): smem attribute: %s", cudaGetErrorString(e));
  const int total_tiles = ceil_div(n_out, G4_M);
  const int grid = total_tiles < sm_count() ? total_tiles : sm_count();
  { conv_fwd_tf32_gather4_kernel<<<grid, G4_THREADS, smem, st>>>(map, (const uint4 *)packed, K, c_out, nbr, n_out, out,
                                                               status, p); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_tf32_gather4");
  return SSC_OK;
}

}  // namespace ssc
