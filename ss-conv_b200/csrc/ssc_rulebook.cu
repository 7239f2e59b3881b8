// Rulebook (indice-pair) generation on a GPU coordinate hash.
//
// Pipeline (regular / strided / transposed convolution and pooling):
//   1. hash_insert      : input coordinates -> open-addressing table (4-slot buckets)
//   2. mark_outputs     : every (input, kernel offset) sets the bit of the output cell it reaches
//   3. popcount scan    : rank of every set bit = output row (ascending flat index)
//   4. decode_outputs   : bit -> (b,x,y,z) row of out_indices
//   5. lookup_neighbours: for each (output, offset) probe the hash warp-cooperatively, write
//                         the output-major neighbour table nbr[K][n_out], count per chunk
//   6. scan_chunks + fill_pairs: compact per-offset pair lists [K,2,n_in] (-1 padded), counts
// Submanifold convolution skips 2-4 (outputs are the inputs).
// Everything is integer work bound by HBM/L2 traffic; no tensor cores involved.
#include "ssc_common.cuh"
#include "ssc_scan.cuh"

namespace ssc {

constexpr int kChunk = 1024;  // outputs per block in lookup / fill

// Input coordinates are looked up either in a dense row map over the input grid (one int32 per
// cell: a lookup is a single load) or, when the grid is large compared with the number of active
// voxels, in the bucketed hash table.  Both live in the same scratch region.
constexpr long long kDenseMaxCells = 1ll << 26;     // 256 MiB of row map at most
constexpr long long kDenseCellsPerRow = 64;         // clearing the map must stay cheap per active voxel

struct RulebookScratch {
  unsigned long long *table;
  int32_t *row_map;      // non-null: dense map in use instead of the hash table
  long long in_cells;
  uint32_t n_buckets;
  uint32_t *bitmap;
  uint32_t *word_prefix;
  uint32_t *block_sums;
  int32_t *chunk_counts;
  int32_t *misc;  // [0] n_out, [1] status
  long long n_words;
  int n_scan_blocks;
  long long out_cap;
  int n_chunks_cap;
  size_t total;
};

static bool use_dense_map(int n_in, long long in_cells) {
  const char *e = getenv("SSC_RULEBOOK_TABLE");
  const int forced = e == nullptr ? 0 : (strcmp(e, "hash") == 0 ? 1 : (strcmp(e, "dense") == 0 ? 2 : 0));
  if (forced == 1) return false;
  if (in_cells > kDenseMaxCells) return false;
  return forced == 2 || in_cells <= kDenseCellsPerRow * (long long)(n_in > 0 ? n_in : 1);
}

static RulebookScratch carve(void *base, int n_in, int batch, const int in_shape[3], const int out_shape[3], int K) {
  RulebookScratch s;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void *p = base ? (char *)base + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  long long vol = (long long)out_shape[0] * out_shape[1] * out_shape[2];
  long long cells = vol * batch;
  s.n_buckets = hash_buckets_for(n_in);
  s.in_cells = (long long)in_shape[0] * in_shape[1] * in_shape[2] * batch;
  if (use_dense_map(n_in, s.in_cells)) {
    s.row_map = (int32_t *)take((size_t)s.in_cells * 4);
    s.table = nullptr;
  } else {
    s.row_map = nullptr;
    s.table = (unsigned long long *)take((size_t)s.n_buckets * kBucketSlots * 8);
  }
  s.n_words = (cells + 31) / 32;
  s.bitmap = (uint32_t *)take((size_t)s.n_words * 4);
  s.word_prefix = (uint32_t *)take((size_t)s.n_words * 4);
  s.n_scan_blocks = (int)((s.n_words + 1023) / 1024);
  s.block_sums = (uint32_t *)take(((size_t)s.n_scan_blocks + 1) * 4);
  long long cap = (long long)n_in * K;
  if (cells < cap) cap = cells;
  if (cap < n_in) cap = n_in;
  s.out_cap = cap;
  s.n_chunks_cap = (int)((cap + kChunk - 1) / kChunk) + 1;
  s.chunk_counts = (int32_t *)take((size_t)s.n_chunks_cap * K * 4);
  s.misc = (int32_t *)take(256);
  s.total = off;
  return s;
}

// ------------------------------------------------------------------------------- kernels
__device__ __forceinline__ bool in_range3(int x, int y, int z, const int *shape) {
  return (unsigned)x < (unsigned)shape[0] && (unsigned)y < (unsigned)shape[1] &&
         (unsigned)z < (unsigned)shape[2];
}

__global__ void hash_insert_kernel(const int4 *__restrict__ indices, int n, int batch,
                                   Geometry g, unsigned long long *table, uint32_t mask,
                                   int32_t *status, const int32_t *__restrict__ n_dev) {
  int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= live_rows(n, n_dev)) return;
  int4 c = indices[j];
  if ((unsigned)c.x >= (unsigned)batch || !in_range3(c.y, c.z, c.w, g.in_shape)) {
    atomicOr(status, 1);
    return;
  }
  uint32_t key = (uint32_t)(((c.x * g.in_shape[0] + c.y) * g.in_shape[1] + c.z) * g.in_shape[2] + c.w);
  unsigned long long packed = ((unsigned long long)key << 32) | (uint32_t)j;
  uint32_t b = hash_mix(key) & mask;
  for (uint32_t probe = 0; probe <= mask; ++probe) {
    for (int s = 0; s < kBucketSlots; ++s) {
      unsigned long long *slot = table + (size_t)b * kBucketSlots + s;
      unsigned long long old = atomicCAS(slot, kEmptySlot, packed);
      if (old == kEmptySlot) return;
      if ((uint32_t)(old >> 32) == key) {  // duplicate coordinate: the largest row wins
        atomicMax(slot, packed);
        return;
      }
    }
    b = (b + 1) & mask;
  }
  atomicOr(status, 2);  // table full (cannot happen at load factor <= 0.5)
}

// Dense alternative to hash_insert_kernel: row_map[flat input cell] = row (largest row wins on
// duplicate coordinates, as in the hash table).
__global__ void map_insert_kernel(const int4 *__restrict__ indices, int n, int batch, Geometry g,
                                  int32_t *__restrict__ row_map, int32_t *status, const int32_t *__restrict__ n_dev) {
  int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= live_rows(n, n_dev)) return;
  int4 c = indices[j];
  if ((unsigned)c.x >= (unsigned)batch || !in_range3(c.y, c.z, c.w, g.in_shape)) {
    atomicOr(status, 1);
    return;
  }
  const long long cell = ((long long)(c.x * g.in_shape[0] + c.y) * g.in_shape[1] + c.z) * g.in_shape[2] + c.w;
  atomicMax(row_map + cell, j);
}

// One thread per input row: mark every output cell the row reaches.  Bits that fall into the
// same bitmap word (consecutive z) are merged before the atomic.
// Output coordinates an input coordinate reaches along one dimension form an arithmetic
// progression; this clips it to [0, limit) and returns its first element and length.
struct Reach {
  int first, step, n;
};
__device__ __forceinline__ Reach clip_progression(int lo, int step, int count, int limit) {
  Reach r;
  r.step = step;
  const int i_min = lo < 0 ? (-lo + step - 1) / step : 0;
  const int last = lo + (count - 1) * step;
  int i_max = count - 1;
  if (last > limit - 1) i_max = (limit - 1 - lo) >= 0 ? (limit - 1 - lo) / step : -1;
  r.first = lo + i_min * step;
  r.n = i_max - i_min + 1;
  return r;
}

// Needs, per dimension, stride == 1 or dilation == 1 (or the transposed geometry): then the reached
// outputs need no test of every kernel index and at most two divisions per dimension.
__device__ __forceinline__ Reach reach_of(const Geometry &g, int d, int in) {
  if (g.transpose)  // o = in*stride - pad + k*dil
    return clip_progression(in * g.stride[d] - g.padding[d], g.dilation[d], g.ksize[d], g.out_shape[d]);
  if (g.dilation[d] == 1) {  // o*stride = in + pad - k, k in [0, ksize): a contiguous range of o
    const int hi_num = in + g.padding[d], lo_num = hi_num - g.ksize[d] + 1;
    const int o_lo = lo_num <= 0 ? 0 : (lo_num + g.stride[d] - 1) / g.stride[d];
    const int o_hi = hi_num / g.stride[d];
    return clip_progression(o_lo, 1, o_hi - o_lo + 1, g.out_shape[d]);
  }
  // stride == 1: o = in + pad - k*dil
  return clip_progression(in + g.padding[d] - (g.ksize[d] - 1) * g.dilation[d], g.dilation[d], g.ksize[d], g.out_shape[d]);
}

// bitmap word |= bits, skipping the atomic when the bits are already there: on coarse grids most
// inputs of a sample reach the same few output cells and their atomics would queue up on one
// word (bits are only ever set while this runs, so a stale read costs at most a redundant atomic).
__device__ __forceinline__ void set_bits(uint32_t *word, uint32_t bits, bool look_first) {
  if (!look_first || (__ldcg(word) & bits) != bits) atomicOr(word, bits);
}

// A block ORs its rows' bits into a shared-memory image of the bitmap words between the first and
// the last cell its rows reach, then sends one atomic per non-zero word: rows that arrive in grid
// order (the order every rulebook and the voxelizer produce) reach a narrow range of words, many
// rows the same ones - on coarse grids all rows of a sample share a handful of words, whose atomics
// would otherwise queue up.  A block whose rows span more words than the image holds (rows in
// arbitrary order) marks them directly.
constexpr int kCoarseVolume = 4096;      // cells per sample up to which a direct atomic first looks at the word
constexpr int kMarkImageWords = 1024;
__global__ void __launch_bounds__(128)
mark_outputs_kernel(const int4 *__restrict__ indices, int n, int batch, Geometry g, uint32_t *bitmap,
                    const int32_t *__restrict__ n_dev) {
  __shared__ uint32_t image[kMarkImageWords];
  __shared__ unsigned cell_min, cell_max;
  __shared__ int any_row;
  const int live = live_rows(n, n_dev);
  if ((int)(blockIdx.x * blockDim.x) >= live) return;            // the whole block
  for (int i = threadIdx.x; i < kMarkImageWords; i += blockDim.x) image[i] = 0u;
  if (threadIdx.x == 0) { cell_min = 0xFFFFFFFFu; cell_max = 0u; any_row = 0; }
  __syncthreads();
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  int4 c = make_int4(0, 0, 0, 0);
  Reach rx = {0, 1, 0}, ry = {0, 1, 0}, rz = {0, 1, 0};
  bool ok = false;
  if (j < live) {
    c = indices[j];
    if ((unsigned)c.x < (unsigned)batch && in_range3(c.y, c.z, c.w, g.in_shape)) {
      rx = reach_of(g, 0, c.y); ry = reach_of(g, 1, c.z); rz = reach_of(g, 2, c.w);
      ok = rx.n > 0 && ry.n > 0 && rz.n > 0;
    }
  }
  const int base_b = c.x * g.out_shape[0];
  unsigned lo = 0xFFFFFFFFu, hi = 0u;                            // first and last cell this row reaches
  if (ok) {
    lo = (unsigned)((base_b + rx.first) * g.out_shape[1] + ry.first) * (unsigned)g.out_shape[2] + (unsigned)rz.first;
    hi = (unsigned)((base_b + rx.first + (rx.n - 1) * rx.step) * g.out_shape[1] + ry.first + (ry.n - 1) * ry.step) *
             (unsigned)g.out_shape[2] + (unsigned)(rz.first + (rz.n - 1) * rz.step);
  }
  const unsigned w_lo = __reduce_min_sync(0xFFFFFFFFu, lo), w_hi = __reduce_max_sync(0xFFFFFFFFu, hi);
  const bool w_any = __any_sync(0xFFFFFFFFu, ok);
  if ((threadIdx.x & 31) == 0 && w_any) { atomicMin(&cell_min, w_lo); atomicMax(&cell_max, w_hi); any_row = 1; }
  __syncthreads();
  if (!any_row) return;                                          // no row of the block reaches an output
  const uint32_t word_lo = cell_min >> 5, word_hi = cell_max >> 5;
  const bool staged = word_hi - word_lo < (uint32_t)kMarkImageWords;
  const bool look_first = g.out_shape[0] * g.out_shape[1] * g.out_shape[2] <= kCoarseVolume;
  if (ok) {
    for (int ix = 0, x = rx.first; ix < rx.n; ++ix, x += rx.step)
      for (int iy = 0, y = ry.first; iy < ry.n; ++iy, y += ry.step) {
        const uint32_t row = (uint32_t)((base_b + x) * g.out_shape[1] + y) * (uint32_t)g.out_shape[2];
        uint32_t word = 0xFFFFFFFFu, bits = 0u;
        for (int iz = 0, z = rz.first; iz < rz.n; ++iz, z += rz.step) {  // ascending z: bits of one word are merged
          const uint32_t flat = row + (uint32_t)z;
          if ((flat >> 5) != word) {
            if (bits) {
              if (staged) atomicOr(&image[word - word_lo], bits);
              else set_bits(bitmap + word, bits, look_first);
            }
            word = flat >> 5;
            bits = 0u;
          }
          bits |= 1u << (flat & 31);
        }
        if (bits) {
          if (staged) atomicOr(&image[word - word_lo], bits);
          else set_bits(bitmap + word, bits, look_first);
        }
      }
  }
  if (!staged) return;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i <= word_hi - word_lo; i += blockDim.x) {
    const uint32_t bits = image[i];
    if (bits) set_bits(bitmap + word_lo + i, bits, look_first);
  }
}

// General fallback (stride and dilation both above one in some dimension): one thread per (input row, kernel offset).
__global__ void mark_outputs_generic_kernel(const int4 *__restrict__ indices, int n, int batch, Geometry g,
                                            uint32_t *bitmap, const int32_t *__restrict__ n_dev) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)live_rows(n, n_dev) * g.K) return;
  int j = (int)(t / g.K);
  int kappa = (int)(t - (long long)j * g.K);
  int4 c = indices[j];
  if ((unsigned)c.x >= (unsigned)batch || !in_range3(c.y, c.z, c.w, g.in_shape)) return;
  int kk[3] = {kappa / (g.ksize[1] * g.ksize[2]), (kappa / g.ksize[2]) % g.ksize[1], kappa % g.ksize[2]};
  int in[3] = {c.y, c.z, c.w};
  int o[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    if (g.transpose) {
      o[d] = in[d] * g.stride[d] - g.padding[d] + kk[d] * g.dilation[d];
    } else {
      int num = in[d] + g.padding[d] - kk[d] * g.dilation[d];
      if (num < 0 || num % g.stride[d] != 0) return;
      o[d] = num / g.stride[d];
    }
    if ((unsigned)o[d] >= (unsigned)g.out_shape[d]) return;
  }
  uint32_t flat = (uint32_t)(((c.x * g.out_shape[0] + o[0]) * g.out_shape[1] + o[1]) * g.out_shape[2] + o[2]);
  atomicOr(bitmap + (flat >> 5), 1u << (flat & 31));
}

// One lane per bitmap bit (a warp per word), for small or densely set bitmaps: every set bit is written
// by a thread of its own (the per-word kernel below would write up to 32 rows one after the other).
__global__ void decode_outputs_bits_kernel(const uint32_t *__restrict__ bitmap,
                                           const uint32_t *__restrict__ word_prefix, long long n_words,
                                           Geometry g, int n_out, int4 *out_indices) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long w = t >> 5;
  if (w >= n_words) return;
  const int bit = (int)(t & 31);
  const uint32_t bits = __ldg(bitmap + w);
  if (!((bits >> bit) & 1u)) return;
  const uint32_t rank = __ldg(word_prefix + w) + (uint32_t)__popc(bits & ((1u << bit) - 1u));
  if ((int)rank >= n_out) return;
  const int vol = g.out_shape[0] * g.out_shape[1] * g.out_shape[2];
  const int yz = g.out_shape[1] * g.out_shape[2];
  const uint32_t flat = (uint32_t)(w * 32 + bit);
  const int b = flat / vol;
  int r = flat - b * vol;
  const int x = r / yz;
  r -= x * yz;
  const int y = r / g.out_shape[2];
  const int z = r - y * g.out_shape[2];
  out_indices[rank] = make_int4(b, x, y, z);
}

__global__ void decode_outputs_kernel(const uint32_t *__restrict__ bitmap,
                                      const uint32_t *__restrict__ word_prefix, long long n_words,
                                      Geometry g, int n_out, int4 *out_indices) {
  // one thread per bitmap word (32 cells): most words of a sparse grid are empty and leave at once;
  // the set bits of a word get consecutive ranks from the word's prefix.  The coordinates of the
  // word's first cell are decoded once (three integer divisions); a set bit is that cell plus its
  // bit number, carried over z, y and x.
  const long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  uint32_t bits = __ldg(bitmap + w);
  if (bits == 0u) return;
  uint32_t rank = __ldg(word_prefix + w);
  const int X = g.out_shape[0], Y = g.out_shape[1], Z = g.out_shape[2];
  const int vol = X * Y * Z, yz = Y * Z;
  const uint32_t flat0 = (uint32_t)(w * 32);
  const int b0 = flat0 / vol;
  int r = flat0 - b0 * vol;
  const int x0 = r / yz;
  r -= x0 * yz;
  const int y0 = r / Z, z0 = r - (r / Z) * Z;
  while (bits != 0u && (int)rank < n_out) {
    const int bit = __ffs((int)bits) - 1;
    bits &= bits - 1u;
    int b = b0, x = x0, y = y0, z = z0 + bit;
    while (z >= Z) { z -= Z; ++y; }
    while (y >= Y) { y -= Y; ++x; }
    while (x >= X) { x -= X; ++b; }
    out_indices[rank++] = make_int4(b, x, y, z);
  }
}

// Small bitmaps (coarse grids are densely set and have few words) take the per-bit kernel, large ones
// (fine grids: mostly empty words) the per-word kernel.
constexpr long long kDecodePerBitMaxWords = 32768;
static void launch_decode(const uint32_t *bitmap, const uint32_t *word_prefix, long long n_words, const Geometry &g, int n_out,
                          int4 *out_indices, cudaStream_t st) {
  if (n_words <= kDecodePerBitMaxWords) {
    { decode_outputs_bits_kernel<<<ceil_div(n_words * 32, 256), 256, 0, st>>>(bitmap, word_prefix, n_words, g, n_out, out_indices); note_launches(1); }
  } else {
    { decode_outputs_kernel<<<ceil_div(n_words, 256), 256, 0, st>>>(bitmap, word_prefix, n_words, g, n_out, out_indices); note_launches(1); }
  }
}

// Dense-map lookup: one thread per output row walks all kernel offsets, so the row's coordinates
// are decoded once; every offset costs a few integer operations, one load from the row map and
// one coalesced store.
// Block = kChunk rows; counts per (offset, chunk) are only produced when chunk_counts is given.
__global__ void __launch_bounds__(256)
lookup_dense_kernel(const int4 *__restrict__ out_indices, int n_out, int batch, Geometry g,
                    const int32_t *__restrict__ row_map, int32_t *__restrict__ nbr,
                    int32_t *__restrict__ chunk_counts, int n_chunks, const int32_t *__restrict__ n_out_dev) {
  extern __shared__ int32_t cnt[];  // [K] when counting
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_rows = live_rows(n_out, n_out_dev);
  const bool counting = chunk_counts != nullptr;
  if (counting) {
    for (int k = threadIdx.x; k < g.K; k += blockDim.x) cnt[k] = 0;
    __syncthreads();
  }
  int base = -1;
  int oc[3] = {0, 0, 0};
  if (o < n_rows) {
    const int4 c = out_indices[o];
    oc[0] = c.y; oc[1] = c.z; oc[2] = c.w;
    if ((unsigned)c.x < (unsigned)batch) base = c.x;
  }
  // input coordinate along dimension d for kernel index k, or -1
  auto coord = [&](int d, int k) -> int {
    int v;
    if (g.transpose) {
      const int num = oc[d] + g.padding[d] - k * g.dilation[d];
      v = (num >= 0 && num % g.stride[d] == 0) ? num / g.stride[d] : -1;
    } else {
      v = oc[d] * g.stride[d] - g.padding[d] + k * g.dilation[d];
    }
    return (unsigned)v < (unsigned)g.in_shape[d] ? v : -1;
  };
  // gridDim.y = kernel extent along x: a block walks the offsets of one kx (more threads in flight)
  int kappa = (int)blockIdx.y * g.ksize[1] * g.ksize[2];
  {
    const int kx = (int)blockIdx.y;
    const int x = coord(0, kx);
    for (int ky = 0; ky < g.ksize[1]; ++ky) {
      const int y = coord(1, ky);
      const long long plane = ((long long)(base * g.in_shape[0] + x) * g.in_shape[1] + y) * g.in_shape[2];
      for (int kz = 0; kz < g.ksize[2]; ++kz, ++kappa) {
        const int z = coord(2, kz);
        int found = -1;
        if (base >= 0 && (x | y | z) >= 0) found = __ldg(row_map + plane + z);
        if (o < n_out) nbr[(size_t)kappa * n_out + o] = found;
        if (counting) {
          const unsigned hits = __ballot_sync(0xffffffffu, found >= 0);
          if ((threadIdx.x & 31) == 0 && hits) atomicAdd(cnt + kappa, __popc(hits));
        }
      }
    }
  }
  if (counting) {
    __syncthreads();
    // chunk = kChunk rows = (kChunk / blockDim.x) consecutive blocks: add this block's share
    const int chunk = (int)(((long long)blockIdx.x * blockDim.x) / kChunk);
    for (int k = threadIdx.x; k < g.K; k += blockDim.x)
      if (cnt[k]) atomicAdd(chunk_counts + (size_t)k * n_chunks + chunk, cnt[k]);
  }
}

// grid (chunks, K), block kChunk threads: thread <-> output row; the hash is probed by
// groups of 4 lanes, each group reading one 32-byte bucket per probe.
__global__ void __launch_bounds__(kChunk)
lookup_neighbours_kernel(const int4 *__restrict__ out_indices, int n_out, int batch, Geometry g,
                         const unsigned long long *__restrict__ table, uint32_t mask,
                         int32_t *__restrict__ nbr, int32_t *__restrict__ chunk_counts, int n_chunks,
                         const int32_t *__restrict__ n_out_dev) {
  const unsigned full = 0xffffffffu;
  int kappa = blockIdx.y;
  int o = blockIdx.x * kChunk + threadIdx.x;
  uint32_t key = 0xFFFFFFFFu;
  const int n_rows = live_rows(n_out, n_out_dev);  // rows past it (up to the capacity n_out) get -1
  if (o < n_rows) {
    int4 c = out_indices[o];
    int kk[3] = {kappa / (g.ksize[1] * g.ksize[2]), (kappa / g.ksize[2]) % g.ksize[1], kappa % g.ksize[2]};
    int oc[3] = {c.y, c.z, c.w};
    int in[3];
    bool ok = (unsigned)c.x < (unsigned)batch;
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      if (g.transpose) {
        int num = oc[d] + g.padding[d] - kk[d] * g.dilation[d];
        ok = ok && num >= 0 && (num % g.stride[d] == 0);
        in[d] = num / g.stride[d];
      } else {
        in[d] = oc[d] * g.stride[d] - g.padding[d] + kk[d] * g.dilation[d];
      }
      ok = ok && (unsigned)in[d] < (unsigned)g.in_shape[d];
    }
    if (ok) key = (uint32_t)(((c.x * g.in_shape[0] + in[0]) * g.in_shape[1] + in[1]) * g.in_shape[2] + in[2]);
  }
  unsigned lane = threadIdx.x & 31u, sub = lane & 3u, gbase = lane & ~3u;
  unsigned gmask = 0xFu << gbase;
  // Round i serves the query of lane gbase+i; the four first probes are issued together so
  // that their memory latencies overlap.
  uint32_t qkey[4], bucket[4];
  unsigned long long slot[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    qkey[i] = __shfl_sync(full, key, gbase + i);
    bucket[i] = hash_mix(qkey[i]) & mask;
    slot[i] = qkey[i] != 0xFFFFFFFFu ? table[(size_t)bucket[i] * kBucketSlots + sub] : kEmptySlot;
  }
  int result = -1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    bool empty = slot[i] == kEmptySlot;
    bool hit = !empty && (uint32_t)(slot[i] >> 32) == qkey[i];
    unsigned hits = (__ballot_sync(full, hit) >> gbase) & 0xFu;
    unsigned empties = (__ballot_sync(full, empty) >> gbase) & 0xFu;
    uint32_t val = __shfl_sync(full, (uint32_t)slot[i], gbase + (hits ? __ffs(hits) - 1 : 0));
    int found = hits ? (int)val : -1;
    if (!hits && !empties) {  // full bucket without the key: keep probing (rare, group-uniform)
      uint32_t b = (bucket[i] + 1) & mask;
      for (uint32_t probe = 1; probe <= mask; ++probe) {
        unsigned long long sl = table[(size_t)b * kBucketSlots + sub];
        bool e2 = sl == kEmptySlot;
        bool h2 = !e2 && (uint32_t)(sl >> 32) == qkey[i];
        unsigned hs = __ballot_sync(gmask, h2);
        unsigned es = __ballot_sync(gmask, e2);
        if (hs) {
          found = (int)__shfl_sync(gmask, (uint32_t)sl, __ffs(hs) - 1);
          break;
        }
        if (es) break;
        b = (b + 1) & mask;
      }
    }
    if (sub == (unsigned)i) result = found;
  }
  if (o < n_out) nbr[(size_t)kappa * n_out + o] = result;
  int cnt = __syncthreads_count(o < n_out && result >= 0);
  if (threadIdx.x == 0) chunk_counts[(size_t)kappa * n_chunks + blockIdx.x] = cnt;
}

// One block per kernel offset: exclusive scan of its chunk counts, total -> indice_num.
__global__ void scan_chunks_kernel(int32_t *chunk_counts, int n_chunks, int32_t *indice_num) {
  __shared__ uint32_t smem[33];
  int32_t *row = chunk_counts + (size_t)blockIdx.x * n_chunks;
  uint32_t running = 0;
  for (int base = 0; base < n_chunks; base += blockDim.x) {
    int i = base + threadIdx.x;
    uint32_t v = i < n_chunks ? (uint32_t)row[i] : 0;
    uint32_t tot;
    uint32_t ex = block_exclusive_scan(v, smem, &tot);
    if (i < n_chunks) row[i] = (int32_t)(running + ex);
    running += tot;
  }
  if (threadIdx.x == 0) indice_num[blockIdx.x] = (int32_t)running;
}

// grid (max(chunks over n_out, chunks over n_in), K), block kChunk.
__global__ void __launch_bounds__(kChunk)
fill_pairs_kernel(const int32_t *__restrict__ nbr, int n_out, int n_in,
                  const int32_t *__restrict__ chunk_offsets, int n_chunks,
                  const int32_t *__restrict__ indice_num, int32_t *__restrict__ pairs) {
  __shared__ uint32_t smem[33];
  int kappa = blockIdx.y;
  int o = blockIdx.x * kChunk + threadIdx.x;
  int32_t *row_in = pairs + (size_t)kappa * 2 * n_in;
  int32_t *row_out = row_in + n_in;
  int v = -1;
  if (o < n_out) v = nbr[(size_t)kappa * n_out + o];
  uint32_t ex = block_exclusive_scan(v >= 0 ? 1u : 0u, smem, nullptr);
  if (v >= 0) {
    int pos = chunk_offsets[(size_t)kappa * n_chunks + blockIdx.x] + (int)ex;
    if (pos < n_in) {
      row_in[pos] = v;
      row_out[pos] = o;
    }
  }
  if (o < n_in && o >= indice_num[kappa]) {
    row_in[o] = -1;
    row_out[o] = -1;
  }
}

__global__ void pairs_to_nbr_kernel(const int32_t *__restrict__ pairs,
                                    const int32_t *__restrict__ indice_num, int n_cols, int n_out,
                                    int swap, int32_t *__restrict__ nbr) {
  int kappa = blockIdx.y;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_cols || i >= indice_num[kappa]) return;
  const int32_t *row = pairs + (size_t)kappa * 2 * n_cols;
  int src = row[(swap ? n_cols : 0) + i];
  int dst = row[(swap ? 0 : n_cols) + i];
  if ((unsigned)dst < (unsigned)n_out) nbr[(size_t)kappa * n_out + dst] = src;
}

// Per-chunk count of present neighbours (the counting half of lookup_neighbours, for tables
// that already exist).
__global__ void __launch_bounds__(kChunk)
count_chunks_kernel(const int32_t *__restrict__ nbr, int n_out, int32_t *__restrict__ chunk_counts, int n_chunks) {
  int kappa = blockIdx.y;
  int o = blockIdx.x * kChunk + threadIdx.x;
  int cnt = __syncthreads_count(o < n_out && nbr[(size_t)kappa * n_out + o] >= 0);
  if (threadIdx.x == 0) chunk_counts[(size_t)kappa * n_chunks + blockIdx.x] = cnt;
}

// ------------------------------------------------------------------------- host drivers
static int fill_geometry(Geometry &g, const int in_shape[3], const int out_shape[3], const int ksize[3],
                         const int stride[3], const int padding[3], const int dilation[3], int transpose) {
  g.K = 1;
  for (int d = 0; d < 3; ++d) {
    g.in_shape[d] = in_shape[d];
    g.out_shape[d] = out_shape[d];
    g.ksize[d] = ksize[d];
    g.stride[d] = stride[d];
    g.padding[d] = padding[d];
    g.dilation[d] = dilation[d];
    if (ksize[d] < 1 || stride[d] < 1 || dilation[d] < 1 || in_shape[d] < 1 || out_shape[d] < 1) return -1;
    g.K *= ksize[d];
  }
  g.transpose = transpose;
  return 0;
}

static int check_volume(int batch, const int shape[3], const char *what) {
  long long cells = (long long)batch * shape[0] * shape[1] * shape[2];
  if (batch < 1 || cells >= 2147483647ll)
    return fail(SSC_ERR_INVALID, "%s: batch*volume = %lld does not fit the int32 flat index", what, cells);
  return 0;
}

static int build_hash(const int32_t *indices, int n_in, int batch, const Geometry &g, RulebookScratch &s,
                      int32_t *status, cudaStream_t st, const int32_t *n_in_dev = nullptr) {
  cudaMemsetAsync(s.misc, 0, 256, st);
  if (s.row_map != nullptr) {
    cudaMemsetAsync(s.row_map, 0xFF, (size_t)s.in_cells * 4, st);
    if (n_in > 0) {
      { map_insert_kernel<<<ceil_div(n_in, 256), 256, 0, st>>>((const int4 *)indices, n_in, batch, g, s.row_map,
                                                            status ? status : s.misc + 1, n_in_dev); note_launches(1); }
    }
    SSC_CHECK_LAUNCH("map_insert");
    return 0;
  }
  cudaMemsetAsync(s.table, 0xFF, (size_t)s.n_buckets * kBucketSlots * 8, st);
  if (n_in > 0) {
    { hash_insert_kernel<<<ceil_div(n_in, 256), 256, 0, st>>>((const int4 *)indices, n_in, batch, g, s.table,
                                                           s.n_buckets - 1, status ? status : s.misc + 1, n_in_dev); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("hash_insert");
  return 0;
}

static int lookup_and_compact(const int32_t *out_indices, int n_out, int n_in, int batch, const Geometry &g,
                              RulebookScratch &s, int32_t *nbr, int32_t *pairs, int32_t *indice_num,
                              cudaStream_t st, const int32_t *n_out_dev = nullptr) {
  int K = g.K;
  int n_chunks = ceil_div(n_out > 0 ? n_out : 1, kChunk);
  if (n_chunks > s.n_chunks_cap) return fail(SSC_ERR_SCRATCH, "rulebook: n_out exceeds the scratch capacity");
  if (s.row_map != nullptr) {
    int32_t *counts = indice_num != nullptr ? s.chunk_counts : nullptr;
    if (counts) cudaMemsetAsync(counts, 0, (size_t)n_chunks * K * 4, st);
    const dim3 lgrid(ceil_div(n_out > 0 ? n_out : 1, 256), g.ksize[0]);
    { lookup_dense_kernel<<<lgrid, 256, K * sizeof(int32_t), st>>>(
          (const int4 *)out_indices, n_out, batch, g, s.row_map, nbr, counts, n_chunks, n_out_dev); note_launches(1); }
  } else {
    dim3 grid(n_chunks, K);
    { lookup_neighbours_kernel<<<grid, kChunk, 0, st>>>((const int4 *)out_indices, n_out, batch, g, s.table,
                                                     s.n_buckets - 1, nbr, s.chunk_counts, n_chunks, n_out_dev); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("lookup_neighbours");
  if (indice_num == nullptr) return 0;
  { scan_chunks_kernel<<<K, 256, 0, st>>>(s.chunk_counts, n_chunks, indice_num); note_launches(1); }
  SSC_CHECK_LAUNCH("scan_chunks");
  if (pairs != nullptr && n_in > 0) {
    int n_chunks_in = ceil_div(n_in, kChunk);
    dim3 grid2(n_chunks > n_chunks_in ? n_chunks : n_chunks_in, K);
    { fill_pairs_kernel<<<grid2, kChunk, 0, st>>>(nbr, n_out, n_in, s.chunk_counts, n_chunks, indice_num, pairs); note_launches(1); }
    SSC_CHECK_LAUNCH("fill_pairs");
  }
  return 0;
}

// Rows (b,x,y,z) of every set bit of a cell bitmap over a [batch, shape] grid, in ascending
// flat-index order (shared with the voxelizer).
int bitmap_decode(const uint32_t *bitmap, const uint32_t *word_prefix, long long n_words, const int shape[3],
                  int n_out, int32_t *out_indices, cudaStream_t st) {
  Geometry g;
  memset(&g, 0, sizeof(g));
  for (int d = 0; d < 3; ++d) g.out_shape[d] = shape[d];
  launch_decode(bitmap, word_prefix, n_words, g, n_out, (int4 *)out_indices, st);
  SSC_CHECK_LAUNCH("bitmap_decode");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Submanifold rulebook for callers that cannot allocate device memory.
//
// Some hosts of this library may never call cudaMalloc: a plugin loaded into an application
// that owns all device memory and hands out none, a service whose device pool is fixed at
// start-up so that an allocation can neither fail nor stall the device later on, a sandboxed
// component with no allocator at all.  For them the hash table and the per-chunk counters
// live in the array below, which every GPU that loads this library keeps until the process
// exits.  Its size fixes the limits: at most kStaticMaxRows active voxels and a kernel
// volume of at most 256.
constexpr int kStaticMaxRows = 65536;
constexpr size_t kStaticTableBytes = (size_t)(2 * kStaticMaxRows / kBucketSlots) * kBucketSlots * 8;  // 1 MiB
constexpr size_t kStaticChunkBytes = (size_t)(kStaticMaxRows / kChunk + 2) * 256 * 4;                 // 66 KiB
constexpr size_t kStaticScratchBytes = kStaticTableBytes + kStaticChunkBytes + 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch, looked up once per device (host code cannot use the
// symbol itself as a pointer).
static int static_scratch_address(unsigned char **out) {
  constexpr int kMaxDevices = 64;
  static unsigned char *address[kMaxDevices] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SSC_ERR_CUDA, "rulebook_subm_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(SSC_ERR_INVALID, "rulebook_subm_static: device index %d not supported", dev);
  unsigned char *p = __atomic_load_n(&address[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(SSC_ERR_CUDA, "rulebook_subm_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    __atomic_store_n(&address[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return 0;
}

}  // namespace ssc

using namespace ssc;

extern "C" int ssc_rulebook_subm_static(const int32_t *indices, int n_in, int batch, const int shape[3],
                                        const int ksize[3], const int dilation[3], int32_t *nbr, int32_t *pairs,
                                        int32_t *indice_num, int32_t *status, void *stream) {
  SSC_REQUIRE(n_in >= 0 && shape && ksize && dilation, "rulebook_subm_static: bad arguments");
  if (n_in > kStaticMaxRows)
    return fail(SSC_ERR_INVALID, "rulebook_subm_static: %d active voxels exceed the built-in scratch (max %d); "
                                 "use ssc_rulebook_subm with caller scratch", n_in, kStaticMaxRows);
  SSC_REQUIRE(n_in == 0 || (indices && nbr), "rulebook_subm_static: null pointer");
  int one[3] = {1, 1, 1};
  int pad[3] = {ksize[0] / 2, ksize[1] / 2, ksize[2] / 2};
  Geometry g;
  SSC_REQUIRE(fill_geometry(g, shape, shape, ksize, one, pad, dilation, 0) == 0, "rulebook_subm_static: bad geometry");
  SSC_REQUIRE(g.K <= 256, "rulebook_subm_static: kernel volume %d > 256", g.K);
  if (int e = check_volume(batch, shape, "rulebook_subm_static")) return e;
  unsigned char *base = nullptr;
  if (int e = static_scratch_address(&base)) return e;
  // Lay the pieces the submanifold path touches over the static array.  Everything a call
  // reads is (re)initialised by that call: the table and the status words are cleared in
  // build_hash, the chunk counters are fully rewritten by the lookup kernel.
  RulebookScratch s;
  memset(&s, 0, sizeof(s));
  s.n_buckets = hash_buckets_for(n_in);
  s.table = (unsigned long long *)base;
  s.chunk_counts = (int32_t *)(base + kStaticTableBytes);
  s.misc = (int32_t *)(base + kStaticTableBytes + kStaticChunkBytes);
  s.out_cap = n_in;
  s.n_chunks_cap = kStaticMaxRows / kChunk + 2;
  if ((size_t)s.n_buckets * kBucketSlots * 8 > kStaticTableBytes)
    return fail(SSC_ERR_INVALID, "rulebook_subm_static: hash table does not fit the built-in scratch");
  cudaStream_t st = as_stream(stream);
  if (int e = build_hash(indices, n_in, batch, g, s, status, st)) return e;
  if (int e = lookup_and_compact(indices, n_in, n_in, batch, g, s, nbr, pairs, indice_num, st)) return e;
  SSC_CHECK_LAUNCH("rulebook_subm_static");
  return SSC_OK;
}

namespace ssc {
}  // namespace ssc

using namespace ssc;

extern "C" size_t ssc_rulebook_scratch_bytes(int n_in, int batch, const int in_shape[3], const int out_shape[3], int K) {
  if (n_in < 0 || batch < 1 || K < 1 || !in_shape || !out_shape) return 0;
  return carve(nullptr, n_in, batch, in_shape, out_shape, K).total;
}

extern "C" int ssc_rulebook_subm(const int32_t *indices, int n_in, int batch, const int shape[3],
                                 const int ksize[3], const int dilation[3], int32_t *nbr, int32_t *pairs,
                                 int32_t *indice_num, int32_t *status, void *scratch, size_t scratch_bytes,
                                 void *stream) {
  SSC_REQUIRE(n_in >= 0 && shape && ksize && dilation, "rulebook_subm: bad arguments");
  SSC_REQUIRE(n_in == 0 || (indices && nbr), "rulebook_subm: null pointer");
  int one[3] = {1, 1, 1};
  int pad[3] = {ksize[0] / 2, ksize[1] / 2, ksize[2] / 2};
  Geometry g;
  SSC_REQUIRE(fill_geometry(g, shape, shape, ksize, one, pad, dilation, 0) == 0, "rulebook_subm: bad geometry");
  SSC_REQUIRE(g.K <= 256, "rulebook_subm: kernel volume %d > 256", g.K);
  if (int e = check_volume(batch, shape, "rulebook_subm")) return e;
  RulebookScratch s = carve(scratch, n_in, batch, shape, shape, g.K);
  if (scratch == nullptr || scratch_bytes < s.total)
    return fail(SSC_ERR_SCRATCH, "rulebook_subm: scratch %zu < %zu bytes", scratch_bytes, s.total);
  cudaStream_t st = as_stream(stream);
  if (int e = build_hash(indices, n_in, batch, g, s, status, st)) return e;
  if (int e = lookup_and_compact(indices, n_in, n_in, batch, g, s, nbr, pairs, indice_num, st)) return e;
  SSC_CHECK_LAUNCH("rulebook_subm");
  return SSC_OK;
}

extern "C" int ssc_rulebook_subm_ahead(const int32_t *indices, int n_cap, int batch, const int shape[3],
                                       const int ksize[3], const int dilation[3], int32_t *nbr, int32_t *status,
                                       void *scratch, size_t scratch_bytes, const int32_t *n_in_dev, void *stream) {
  SSC_REQUIRE(n_cap >= 0 && shape && ksize && dilation && n_in_dev, "rulebook_subm_ahead: bad arguments");
  SSC_REQUIRE(n_cap == 0 || (indices && nbr), "rulebook_subm_ahead: null pointer");
  int one[3] = {1, 1, 1};
  int pad[3] = {ksize[0] / 2, ksize[1] / 2, ksize[2] / 2};
  Geometry g;
  SSC_REQUIRE(fill_geometry(g, shape, shape, ksize, one, pad, dilation, 0) == 0, "rulebook_subm_ahead: bad geometry");
  SSC_REQUIRE(g.K <= 256, "rulebook_subm_ahead: kernel volume %d > 256", g.K);
  if (int e = check_volume(batch, shape, "rulebook_subm_ahead")) return e;
  RulebookScratch s = carve(scratch, n_cap, batch, shape, shape, g.K);
  if (scratch == nullptr || scratch_bytes < s.total)
    return fail(SSC_ERR_SCRATCH, "rulebook_subm_ahead: scratch %zu < %zu bytes", scratch_bytes, s.total);
  cudaStream_t st = as_stream(stream);
  if (int e = build_hash(indices, n_cap, batch, g, s, status, st, n_in_dev)) return e;
  if (int e = lookup_and_compact(indices, n_cap, n_cap, batch, g, s, nbr, nullptr, nullptr, st, n_in_dev)) return e;
  SSC_CHECK_LAUNCH("rulebook_subm_ahead");
  return SSC_OK;
}

extern "C" int ssc_rulebook_conv_count(const int32_t *indices, int n_in, int batch, const int in_shape[3],
                                       const int out_shape[3], const int ksize[3], const int stride[3],
                                       const int padding[3], const int dilation[3], int transpose,
                                       int32_t *n_out_dev, int32_t *status, void *scratch,
                                       size_t scratch_bytes, const int32_t *n_in_dev, void *stream) {
  SSC_REQUIRE(n_in >= 0 && in_shape && out_shape && ksize && stride && padding && dilation && n_out_dev,
              "rulebook_conv_count: bad arguments");
  Geometry g;
  SSC_REQUIRE(fill_geometry(g, in_shape, out_shape, ksize, stride, padding, dilation, transpose) == 0,
              "rulebook_conv_count: bad geometry");
  SSC_REQUIRE(g.K <= 256, "rulebook_conv_count: kernel volume %d > 256", g.K);
  if (int e = check_volume(batch, in_shape, "rulebook_conv_count(in)")) return e;
  if (int e = check_volume(batch, out_shape, "rulebook_conv_count(out)")) return e;
  RulebookScratch s = carve(scratch, n_in, batch, in_shape, out_shape, g.K);
  if (scratch == nullptr || scratch_bytes < s.total)
    return fail(SSC_ERR_SCRATCH, "rulebook_conv_count: scratch %zu < %zu bytes", scratch_bytes, s.total);
  cudaStream_t st = as_stream(stream);
  if (int e = build_hash(indices, n_in, batch, g, s, status, st, n_in_dev)) return e;
  cudaMemsetAsync(s.bitmap, 0, (size_t)s.n_words * 4, st);
  if (n_in > 0) {
    bool simple = true;
    for (int d = 0; d < 3; ++d) simple = simple && (g.transpose || g.stride[d] == 1 || g.dilation[d] == 1);
    if (simple) {
      { mark_outputs_kernel<<<ceil_div(n_in, 128), 128, 0, st>>>((const int4 *)indices, n_in, batch, g, s.bitmap, n_in_dev); note_launches(1); }
    } else {
      { mark_outputs_generic_kernel<<<ceil_div((long long)n_in * g.K, 256), 256, 0, st>>>((const int4 *)indices, n_in, batch, g, s.bitmap, n_in_dev); note_launches(1); }
    }
    SSC_CHECK_LAUNCH("mark_outputs");
  }
  if (int e = exclusive_scan_u32<true>(s.bitmap, s.n_words, s.word_prefix, s.block_sums, s.misc, n_out_dev, st)) return e;
  SSC_CHECK_LAUNCH("rulebook_conv_count");
  return SSC_OK;
}

extern "C" int ssc_rulebook_conv_fill(const int32_t *indices, int n_in, int batch, const int in_shape[3],
                                      const int out_shape[3], const int ksize[3], const int stride[3],
                                      const int padding[3], const int dilation[3], int transpose, int n_out,
                                      int32_t *out_indices, int32_t *nbr, int32_t *pairs, int32_t *indice_num,
                                      int32_t *status, void *scratch, size_t scratch_bytes,
                                      const int32_t *n_out_dev, void *stream) {
  SSC_REQUIRE(n_in >= 0 && n_out >= 0 && in_shape && out_shape && ksize && stride && padding && dilation,
              "rulebook_conv_fill: bad arguments");
  SSC_REQUIRE(n_out_dev == nullptr || pairs == nullptr,
              "rulebook_conv_fill: pair lists need the exact output count on the host");
  SSC_REQUIRE(n_out == 0 || (out_indices && nbr), "rulebook_conv_fill: null pointer");
  Geometry g;
  SSC_REQUIRE(fill_geometry(g, in_shape, out_shape, ksize, stride, padding, dilation, transpose) == 0,
              "rulebook_conv_fill: bad geometry");
  SSC_REQUIRE(g.K <= 256, "rulebook_conv_fill: kernel volume %d > 256", g.K);
  RulebookScratch s = carve(scratch, n_in, batch, in_shape, out_shape, g.K);
  if (scratch == nullptr || scratch_bytes < s.total)
    return fail(SSC_ERR_SCRATCH, "rulebook_conv_fill: scratch %zu < %zu bytes", scratch_bytes, s.total);
  SSC_REQUIRE((long long)n_out <= s.out_cap, "rulebook_conv_fill: n_out %d exceeds the possible maximum", n_out);
  cudaStream_t st = as_stream(stream);
  if (n_out > 0) {
    launch_decode(s.bitmap, s.word_prefix, s.n_words, g, n_out, (int4 *)out_indices, st);
    SSC_CHECK_LAUNCH("decode_outputs");
  }
  if (int e = lookup_and_compact(out_indices, n_out, n_in, batch, g, s, nbr, pairs, indice_num, st, n_out_dev)) return e;
  SSC_CHECK_LAUNCH("rulebook_conv_fill");
  return SSC_OK;
}

extern "C" int ssc_pairs_to_nbr(const int32_t *pairs, const int32_t *indice_num, int K, int n_cols, int n_out,
                                int swap, int32_t *nbr, void *stream) {
  SSC_REQUIRE(K >= 1 && n_cols >= 0 && n_out >= 0, "pairs_to_nbr: bad sizes");
  if (n_out == 0) return SSC_OK;
  SSC_REQUIRE(nbr && indice_num && (n_cols == 0 || pairs), "pairs_to_nbr: null pointer");
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(nbr, 0xFF, (size_t)K * n_out * 4, st);
  if (n_cols > 0) {
    dim3 grid(ceil_div(n_cols, 256), K);
    { pairs_to_nbr_kernel<<<grid, 256, 0, st>>>(pairs, indice_num, n_cols, n_out, swap, nbr); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("pairs_to_nbr");
  return SSC_OK;
}

extern "C" size_t ssc_pairs_from_nbr_scratch_bytes(int K, int n_out) {
  if (K < 1 || n_out < 0) return 0;
  return (size_t)K * (size_t)ceil_div(n_out > 0 ? n_out : 1, kChunk) * 4 + 256;
}

extern "C" int ssc_pairs_from_nbr(const int32_t *nbr, int K, int n_out, int n_in, int32_t *pairs, int32_t *indice_num,
                                  void *scratch, size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(K >= 1 && K <= 256 && n_out >= 0 && n_in >= 0, "pairs_from_nbr: bad sizes");
  SSC_REQUIRE(indice_num && (n_in == 0 || pairs) && (n_out == 0 || nbr), "pairs_from_nbr: null pointer");
  if (scratch == nullptr || scratch_bytes < ssc_pairs_from_nbr_scratch_bytes(K, n_out))
    return fail(SSC_ERR_SCRATCH, "pairs_from_nbr: scratch too small");
  cudaStream_t st = as_stream(stream);
  int n_chunks = ceil_div(n_out > 0 ? n_out : 1, kChunk);
  int32_t *chunk_counts = (int32_t *)scratch;
  dim3 grid(n_chunks, K);
  { count_chunks_kernel<<<grid, kChunk, 0, st>>>(nbr, n_out, chunk_counts, n_chunks); note_launches(1); }
  { scan_chunks_kernel<<<K, 256, 0, st>>>(chunk_counts, n_chunks, indice_num); note_launches(1); }
  if (n_in > 0) {
    int n_chunks_in = ceil_div(n_in, kChunk);
    dim3 grid2(n_chunks > n_chunks_in ? n_chunks : n_chunks_in, K);
    { fill_pairs_kernel<<<grid2, kChunk, 0, st>>>(nbr, n_out, n_in, chunk_counts, n_chunks, indice_num, pairs); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("pairs_from_nbr");
  return SSC_OK;
}
