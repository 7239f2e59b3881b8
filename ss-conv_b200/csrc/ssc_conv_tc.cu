// Output-stationary gather-GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// One CTA owns 128 consecutive output rows.  Its slice of the neighbour table (K x 128 row
// indices) is staged in shared memory once.  For every kernel offset that has at least one
// neighbour inside the tile, and every 32-channel slab of the input channels, the CTA
//   * gathers the present neighbour rows with cp.async (16-byte chunks) straight into the
//     K-major 128-byte-swizzled operand layout, several stages ahead of use (chunks of absent
//     rows stay zero and are only rewritten when they held data before), then rounds its own
//     chunks fp32 -> TF32 (round to nearest) in place,
//   * brings in the matching pre-packed filter slab (already TF32, already in operand layout)
//     with one bulk asynchronous copy that signals an mbarrier,
//   * lets one thread issue tcgen05.mma (M=128, N<=256, K=8 per instruction) accumulating in
//     tensor memory (fp32), and commits the group to an mbarrier that frees the stage.
// Accumulators stay in TMEM across all offsets; the epilogue reads them with tcgen05.ld and
// writes each output row exactly once (no scatter atomics, deterministic order).
//
// Every wait on an mbarrier is bounded: on expiry the kernel records an error in `status`,
// stops issuing work, frees its tensor memory and returns.
#include <stdlib.h>

#include "ssc_common.cuh"

namespace ssc {

constexpr int TC_M = 128;
constexpr int TC_SLAB = 32;          // tf32 elements per 128-byte operand row
constexpr int TC_THREADS = 256;
constexpr int TC_A_BYTES = TC_M * 128;
constexpr int TC_CTRL_BYTES = 1024;
constexpr uint32_t kSpinLimit = 1u << 22;

struct TcParams {
  int k_slabs;    // ceil(c_in / 32)
  int n_pad;      // padded output channels (n_tiles * tile_n)
  int n_tiles;    // MMA instructions along N per k-step
  int tile_n;     // N of one MMA, multiple of 16, <= 256
  int tmem_cols;  // power of two >= max(32, n_pad)
  int stages;     // operand ring depth
  int lookahead;  // stages of loads in flight ahead of the MMA
  int b_bytes;    // n_pad * 128
  int nbr_bytes;  // K * 128 * 4
};

// Shared-memory plan: [stages x (A 16 KB + B)] [control 1 KB] [neighbour slice K x 512 B].
// Two CTAs per SM are preferred (their barrier stalls overlap) when that leaves >= 3 stages.
static bool tc_params(int c_in, int c_out, int K, TcParams &p) {
  p.k_slabs = (c_in + TC_SLAB - 1) / TC_SLAB;
  int n16 = (c_out + 15) / 16 * 16;
  p.n_tiles = (n16 + 255) / 256;
  p.tile_n = ((n16 + p.n_tiles - 1) / p.n_tiles + 15) / 16 * 16;
  p.n_pad = p.n_tiles * p.tile_n;
  if (p.n_pad > 512) return false;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.n_pad) p.tmem_cols <<= 1;
  p.b_bytes = p.n_pad * 128;
  p.nbr_bytes = K * TC_M * 4;
  int stage = TC_A_BYTES + p.b_bytes;
  int fixed = TC_CTRL_BYTES + p.nbr_bytes + 1024;
  int two = (112 * 1024 - fixed) / stage;   // per-CTA budget when two CTAs share an SM
  int one = (226 * 1024 - fixed) / stage;
  int ctas = (p.tmem_cols <= 256 && two >= 3) ? 2 : 1;
  if (const char *e = getenv("SSC_TC_CTAS_PER_SM")) {
    int v = atoi(e);
    if (v == 1 || (v == 2 && p.tmem_cols <= 256 && two >= 2)) ctas = v;
  }
  p.stages = ctas == 2 ? two : one;
  if (p.stages > 8) p.stages = 8;
  if (const char *e = getenv("SSC_TC_STAGES")) {
    int v = atoi(e);
    if (v >= 2 && v <= p.stages) p.stages = v;
  }
  if (p.stages < 2) return false;
  p.lookahead = p.stages - 2;
  return true;
}

// ------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart, descriptor version 1 (sm_100)
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
  d |= (uint64_t)1 << 46;                 // version
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      :
      : "r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Wait until at most n of this thread's most recent copy groups are still in flight.
__device__ __forceinline__ void cp_async_wait(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
  }
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

__global__ void __launch_bounds__(TC_THREADS, 2)
conv_fwd_tf32_kernel(const float *__restrict__ features, int c_in, const uint4 *__restrict__ packed, int K,
                     int c_out, const int32_t *__restrict__ nbr, int n_out, float *__restrict__ out,
                     int32_t *status, TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  // operand stages need 1024-byte alignment for the 128-byte swizzle
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = TC_A_BYTES + p.b_bytes;
  uint8_t *ctrl = smem + (size_t)p.stages * stage_bytes;
  uint64_t *bars = (uint64_t *)ctrl;                       // [stages] slot free (MMAs retired)
  uint64_t *full_bars = (uint64_t *)(ctrl + 640);          // [stages] filter slab landed
  uint32_t *tmem_slot = (uint32_t *)(ctrl + 64);
  // abort flags are double-buffered by iteration parity so that every thread takes the same
  // decision after the per-iteration barrier
  volatile int *abort_flag = (volatile int *)(ctrl + 72);  // [2]
  int *n_act_s = (int *)(ctrl + 80);
  uint8_t *act_flag = ctrl + 128;                          // [256]
  uint8_t *act_list = ctrl + 128 + 256;                    // [256]
  int32_t *nbr_s = (int32_t *)(ctrl + TC_CTRL_BYTES);      // [K][128]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * TC_M;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(bars + s), 1);
      mbar_init(smem_u32(full_bars + s), 1);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // stage this tile's slice of the neighbour table and find the offsets that touch it
  for (int kappa = warp; kappa < K; kappa += TC_THREADS / 32) {
    bool any = false;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int r = q * 32 + lane;
      int v = (m0 + r < n_out) ? __ldg(nbr + (size_t)kappa * n_out + m0 + r) : -1;
      nbr_s[kappa * TC_M + r] = v;
      any |= v >= 0;
    }
    unsigned b = __ballot_sync(0xffffffffu, any);
    if (lane == 0) act_flag[kappa] = b != 0;
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
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.tile_n >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);

  const int g_row = tid >> 3;   // 0..31: row inside a 32-row pass
  const int g_chunk = tid & 7;  // 16-byte chunk inside the 128-byte slab row
  const bool vec_ok = (c_in & 3) == 0;
  const uint32_t smem_base = smem_u32(smem);
  const int S = p.stages, L = p.lookahead;
  // byte offset of this thread's chunk inside an A stage for pass 0 (add pass * 4096)
  const uint32_t a_off0 = (uint32_t)(g_row >> 3) * 1024u + (uint32_t)(g_row & 7) * 128u +
                          (uint32_t)((g_chunk ^ (g_row & 7)) << 4);
  // Every A chunk starts as zero; bit (slot*4 + pass) of `dirty` says that this thread's chunk
  // of that slot currently holds gathered data, so absent rows cost nothing unless the chunk
  // has to be cleared again.
  uint32_t dirty = 0;
  for (int sl = 0; sl < S; ++sl)
#pragma unroll
    for (int pass = 0; pass < 4; ++pass)
      *(uint4 *)(smem + (size_t)sl * stage_bytes + a_off0 + pass * 4096) = make_uint4(0u, 0u, 0u, 0u);

  // producer cursor: pipeline step `nxt`, its ring slot, (offset, slab) and slot-use parity
  int nxt = 0, slot_n = 0, par_n = 0, act_n = 0, slab_n = 0;

  auto issue_loads = [&]() {
    const int kappa = act_list[act_n];
    const uint32_t a_addr = smem_base + (uint32_t)slot_n * (uint32_t)stage_bytes;
    const int ch = slab_n * TC_SLAB + g_chunk * 4;
    const int32_t *rows = nbr_s + kappa * TC_M;
    const bool in_range = ch < c_in;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int src = rows[pass * 32 + g_row];
      const uint32_t bit = 1u << (slot_n * 4 + pass);
      const uint32_t dst = a_addr + a_off0 + (uint32_t)pass * 4096u;
      if (src >= 0 && in_range) {
        const float *fp = features + (size_t)src * c_in + ch;
        if (vec_ok) {
          cp_async16(dst, fp, 16u);
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            bool ok = ch + q < c_in;
            cp_async4(dst + 4u * q, ok ? (const void *)(fp + q) : (const void *)features, ok ? 4u : 0u);
          }
        }
        dirty |= bit;
      } else if (dirty & bit) {
        *(uint4 *)(smem + (size_t)slot_n * stage_bytes + a_off0 + pass * 4096) = make_uint4(0u, 0u, 0u, 0u);
        dirty &= ~bit;
      }
    }
    if (tid == 32) {  // one thread moves the whole pre-packed filter slab with a bulk copy
      const uint4 *bsrc = packed + ((size_t)kappa * p.k_slabs + slab_n) * (size_t)(p.n_pad * 8);
      const uint32_t bar = smem_u32(full_bars + slot_n);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)p.b_bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       a_addr + TC_A_BYTES),
                   "l"(bsrc), "r"((uint32_t)p.b_bytes), "r"(bar)
                   : "memory");
    }
    ++nxt;
    if (++slab_n == p.k_slabs) { slab_n = 0; ++act_n; }
    if (++slot_n == S) { slot_n = 0; par_n ^= 1; }
  };

  for (int j = 0; j < L; ++j) {
    if (nxt < n_iter) issue_loads();
    cp_async_commit();
  }

  int s = 0, par = 0;  // consumer cursor: ring slot of step `it` and its use parity
  int it = 0;
  for (; it < n_iter; ++it) {
    // 1. keep L steps of loads in flight: refill the slot whose MMAs have retired
    if (nxt < n_iter) {
      if (nxt >= S) {
        if (!mbar_wait(smem_u32(bars + slot_n), (uint32_t)(par_n ^ 1))) abort_flag[it & 1] = 1;
        tc_fence_after();
      }
      issue_loads();
    }
    cp_async_commit();
    // 2. this thread's copies for step `it` have landed: round its gathered chunks to TF32
    cp_async_wait(L);
    {
      uint8_t *a_s = smem + (size_t)s * stage_bytes;
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        if (dirty & (1u << (s * 4 + pass))) {
          uint4 *ptr = (uint4 *)(a_s + a_off0 + pass * 4096);
          uint4 v = *ptr;
          v.x = to_tf32(__uint_as_float(v.x));
          v.y = to_tf32(__uint_as_float(v.y));
          v.z = to_tf32(__uint_as_float(v.z));
          v.w = to_tf32(__uint_as_float(v.w));
          *ptr = v;
        }
      }
    }
    fence_async_smem();
    __syncthreads();
    if (abort_flag[it & 1]) break;
    // 3. one thread feeds the tensor core once the filter slab has landed too
    if (tid == 0) {
      if (!mbar_wait(smem_u32(full_bars + s), (uint32_t)par)) {
        abort_flag[(it + 1) & 1] = 1;
      } else {
        tc_fence_after();
        uint32_t a_addr = smem_base + (uint32_t)s * (uint32_t)stage_bytes, b_addr = a_addr + TC_A_BYTES;
        for (int nt = 0; nt < p.n_tiles; ++nt) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            uint64_t da = make_desc(a_addr + ks * 32);
            uint64_t db = make_desc(b_addr + nt * p.tile_n * 128 + ks * 32);
            mma_tf32(tmem_base + nt * p.tile_n, da, db, idesc, (it > 0 || ks > 0) ? 1u : 0u);
          }
        }
      }
      mma_commit(smem_u32(bars + s));
    }
    if (++s == S) { s = 0; par ^= 1; }
  }
  cp_async_wait(0);

  bool ok = !(abort_flag[0] | abort_flag[1]);
  if (!ok && tid == 32) {  // gave up early: let the filter copies still in flight land (bounded)
    for (int t = it; t < nxt; ++t) mbar_wait(smem_u32(full_bars + (t % S)), (uint32_t)((t / S) & 1));
  }
  if (ok && n_iter > 0) {
    int last = n_iter - 1;
    if (!mbar_wait(smem_u32(bars + (last % p.stages)), (uint32_t)((last / p.stages) & 1))) {
      abort_flag[0] = 1;
    }
  }
  tc_fence_after();
  __syncthreads();
  ok = !(abort_flag[0] | abort_flag[1]);
  if (!ok && tid == 0 && status) atomicOr(status, 16);

  // epilogue: warp w reads TMEM lanes 32*(w&3).., column groups alternate between warp halves
  {
    int q = warp & 3, half = warp >> 2;
    int m = m0 + q * 32 + lane;
    for (int c0 = half * 16; c0 < p.n_pad && c0 < ((c_out + 15) & ~15); c0 += 32) {
      uint32_t r[16];
      if (ok && n_iter > 0) {
        uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0u;
      }
      if (m < n_out) {
        float *op = out + (size_t)m * c_out + c0;
        if ((c_out & 3) == 0) {
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            if (c0 + j < c_out)
              *(float4 *)(op + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < c_out) op[j] = __uint_as_float(r[j]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

static size_t tc_smem_bytes(const TcParams &p) {
  return (size_t)p.stages * (TC_A_BYTES + p.b_bytes) + 1024 /*alignment slack*/ + TC_CTRL_BYTES + p.nbr_bytes;
}

int conv_fwd_tf32(const float *features, int n_in, int c_in, const void *packed, int K, int c_out,
                  const int32_t *nbr, int n_out, float *out, int32_t *status, cudaStream_t st) {
  TcParams p;
  if (K > 256) return fail(SSC_ERR_INVALID, "conv_fwd(tf32): kernel volume %d > 256", K);
  if (!tc_params(c_in, c_out, K, p)) return fail(SSC_ERR_INVALID, "conv_fwd(tf32): c_out %d / kernel volume %d not supported", c_out, K);
  size_t smem = tc_smem_bytes(p);
  cudaError_t e = cudaFuncSetAttribute(conv_fwd_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "conv_fwd(tf32): smem attribute: %s", cudaGetErrorString(e));
  int grid = ceil_div(n_out, TC_M);
  { conv_fwd_tf32_kernel<<<grid, TC_THREADS, smem, st>>>(features, c_in, (const uint4 *)packed, K, c_out, nbr, n_out,
                                                      out, status, p); note_launches(1); }
  SSC_CHECK_LAUNCH("conv_fwd_tf32");
  return SSC_OK;
}

}  // namespace ssc

using namespace ssc;

extern "C" size_t ssc_conv_packed_bytes(int K, int c_in, int c_out, int precision) {
  if (precision != SSC_PREC_TF32 || K < 1 || c_in < 1 || c_out < 1) return 0;
  TcParams p;
  if (!tc_params(c_in, c_out, 1, p)) return 0;
  return (size_t)K * p.k_slabs * p.b_bytes;
}

extern "C" int ssc_conv_pack_filters(const float *filters, int K, int c_in, int c_out, int precision, void *packed,
                                     void *stream) {
  SSC_REQUIRE(precision == SSC_PREC_TF32, "conv_pack_filters: only SSC_PREC_TF32 has a packed form");
  SSC_REQUIRE(filters && packed && K >= 1 && c_in >= 1 && c_out >= 1, "conv_pack_filters: bad arguments");
  TcParams p;
  SSC_REQUIRE(tc_params(c_in, c_out, 1, p), "conv_pack_filters: c_out %d not supported (max 512)", c_out);
  long long total = (long long)K * p.k_slabs * p.n_pad * 8;
  { pack_filters_tf32_kernel<<<ceil_div(total, 256), 256, 0, as_stream(stream)>>>(filters, K, c_in, c_out, p, (uint4 *)packed); note_launches(1); }
  SSC_CHECK_LAUNCH("pack_filters_tf32");
  return SSC_OK;
}
