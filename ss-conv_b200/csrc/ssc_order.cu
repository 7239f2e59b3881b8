// Row order for the gather-GEMM: rows that use the same kernel offsets next to each other.
//
// The convolution kernel works on tiles of 128 rows and skips, per tile, every kernel offset that
// none of the tile's rows uses.  In the input-major table of a strided convolution (the table
// the input gradient runs on, and the forward table of a transposed convolution) the offsets a
// row uses depend on the parity of its coordinates: a row sees 1/8 of the 27 offsets of a 3^3
// stride-2 kernel, but 128 consecutive rows see all of them, so nearly every (tile, offset) step
// runs with 7/8 of its rows switched off.  Grouping the rows by the first offset they use (which
// names the parity class) makes the tiles uniform: a tile then skips the other classes' offsets.
//
// A counting sort in three launches, stable (ascending row number inside a group), so the
// order - and with it everything computed through it - is repeatable:
//   1. key per row (first offset with a neighbour, K if none) + histogram per block of 1024 rows,
//   2. exclusive scan of the histograms laid out group-major,
//   3. scatter: position = scanned base of (group, block) + rank of the row inside its block.
#include "ssc_common.cuh"
#include "ssc_scan.cuh"

namespace ssc {

constexpr int ORD_BLOCK = 1024;
constexpr int ORD_MAX_K = 343;   // 7^3: the scatter kernel keeps 32 x (K + 1) counters in shared memory

__global__ void __launch_bounds__(ORD_BLOCK)
row_key_hist_kernel(const int32_t *__restrict__ nbr, int K, int n_rows, uint16_t *__restrict__ keys,
                    uint32_t *__restrict__ hist, int n_blocks) {
  extern __shared__ uint32_t hist_s[];  // [K + 1]
  const int B = K + 1;
  for (int b = threadIdx.x; b < B; b += ORD_BLOCK) hist_s[b] = 0u;
  __syncthreads();
  const int row = blockIdx.x * ORD_BLOCK + threadIdx.x;
  if (row < n_rows) {
    int key = K;
    for (int kappa = 0; kappa < K; ++kappa)
      if (__ldg(nbr + (size_t)kappa * n_rows + row) >= 0) {
        key = kappa;
        break;
      }
    keys[row] = (uint16_t)key;
    atomicAdd(&hist_s[key], 1u);  // a count: the order of the additions does not matter
  }
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += ORD_BLOCK) hist[(size_t)b * n_blocks + blockIdx.x] = hist_s[b];
}

__global__ void __launch_bounds__(ORD_BLOCK)
row_scatter_kernel(const uint16_t *__restrict__ keys, int B, int n_rows, const uint32_t *__restrict__ base, int n_blocks,
                   int32_t *__restrict__ order, const int32_t *__restrict__ nbr = nullptr, int K = 0,
                   int32_t *__restrict__ nbr_in_order = nullptr) {
  extern __shared__ uint32_t cnt[];  // [warps of the block][B] rows of each group in each warp
  for (int i = threadIdx.x; i < (int)(blockDim.x >> 5) * B; i += blockDim.x) cnt[i] = 0u;
  __syncthreads();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int key = row < n_rows ? (int)keys[row] : -1;
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  if (key >= 0 && rank == 0) cnt[warp * B + key] = (uint32_t)__popc(peers);
  __syncthreads();
  if (key >= 0) {
    uint32_t before = 0;
    for (int w = 0; w < warp; ++w) before += cnt[w * B + key];
    const uint32_t pos = base[(size_t)key * n_blocks + blockIdx.x] + before + (uint32_t)rank;
    order[pos] = row;
    if (nbr_in_order != nullptr)   // the table's column of this row moves to the row's position
      for (int kappa = 0; kappa < K; ++kappa)
        nbr_in_order[(size_t)kappa * n_rows + pos] = __ldg(nbr + (size_t)kappa * n_rows + row);
  }
}

// Key for the forward table of a convolution with a small kernel (kx + ky + kz <= 9 bits): which
// planes of the kernel hold a neighbour of the row - bit kx says "some offset (kx, *, *) is used",
// then the same for ky and kz.  A tile whose rows agree on those planes skips every offset outside
// their product; on surface-like inputs (a row uses 6 of 27 offsets, 128 consecutive rows together
// use all 27) grouping by this key nearly halves the (tile, offset) steps.  Rows at and beyond the
// device-side row count get the last bucket, so the first n_live entries of the order are the
// live rows.  Buckets are numbered by the number of offsets a key allows (the product of its set
// bits per axis), most first: a tile's index then falls with its step count, and the grid's tail
// is made of the short tiles.
constexpr int PLANE_BLOCK = 512;        // rows per block (16 warps x 513 counters fit the default shared memory)
constexpr int PLANE_MAX_BITS = 9;
// bucket_of[key] = rank of the key by (offsets it allows, descending; key, ascending): one block, once per call
__global__ void __launch_bounds__(PLANE_BLOCK)
plane_bucket_table_kernel(int kx, int ky, int kz, uint16_t *__restrict__ bucket_of) {
  __shared__ uint8_t weight_s[1 << PLANE_MAX_BITS];
  const int n_keys = 1 << (kx + ky + kz);
  for (int key = threadIdx.x; key < n_keys; key += PLANE_BLOCK)
    weight_s[key] = (uint8_t)(__popc(key & ((1 << kx) - 1)) * __popc((key >> kx) & ((1 << ky) - 1)) * __popc(key >> (kx + ky)));
  __syncthreads();
  for (int key = threadIdx.x; key < n_keys; key += PLANE_BLOCK) {
    const int w = weight_s[key];
    int before = 0;
    for (int other = 0; other < n_keys; ++other) {
      const int wo = weight_s[other];
      before += (wo > w) | ((wo == w) & (other < key));
    }
    bucket_of[key] = (uint16_t)before;
  }
}

__global__ void __launch_bounds__(PLANE_BLOCK)
row_plane_key_hist_kernel(const int32_t *__restrict__ nbr, int kx, int ky, int kz, int n_rows,
                          const int32_t *__restrict__ n_rows_dev, const uint16_t *__restrict__ bucket_table,
                          uint16_t *__restrict__ keys, uint32_t *__restrict__ hist, int n_blocks) {
  extern __shared__ uint32_t hist_s[];  // [B] counters, then [B - 1] bucket of every key
  const int bits = kx + ky + kz, B = (1 << bits) + 1;
  uint32_t *bucket_of = hist_s + B;
  for (int b = threadIdx.x; b < B; b += PLANE_BLOCK) hist_s[b] = 0u;
  for (int key = threadIdx.x; key < B - 1; key += PLANE_BLOCK) bucket_of[key] = bucket_table[key];
  __syncthreads();
  const int row = blockIdx.x * PLANE_BLOCK + threadIdx.x;
  if (row < n_rows) {
    int key = B - 1;
    if (row < live_rows(n_rows, n_rows_dev)) {
      key = 0;
      int kappa = 0;
      for (int x = 0; x < kx; ++x)
        for (int y = 0; y < ky; ++y)
          for (int z = 0; z < kz; ++z, ++kappa)
            if (__ldg(nbr + (size_t)kappa * n_rows + row) >= 0) key |= (1 << x) | (1 << (kx + y)) | (1 << (kx + ky + z));
      key = (int)bucket_of[key];
    }
    keys[row] = (uint16_t)key;
    atomicAdd(&hist_s[key], 1u);  // a count: the order of the additions does not matter
  }
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += PLANE_BLOCK) hist[(size_t)b * n_blocks + blockIdx.x] = hist_s[b];
}

}  // namespace ssc

using namespace ssc;

static size_t order_align(size_t x) { return (x + 255) & ~(size_t)255; }

extern "C" size_t ssc_nbr_row_order_scratch_bytes(int K, int n_rows) {
  if (K < 1 || K > ORD_MAX_K || n_rows < 0) return 0;
  const size_t n_blocks = (size_t)ceil_div(n_rows > 0 ? n_rows : 1, ORD_BLOCK);
  const size_t cells = (size_t)(K + 1) * n_blocks;
  return order_align((size_t)n_rows * 2) + 2 * order_align(cells * 4) + order_align((cells / 1024 + 2) * 4);
}

extern "C" int ssc_nbr_row_order(const int32_t *nbr, int K, int n_rows, int32_t *order, void *scratch, size_t scratch_bytes,
                                 void *stream) {
  SSC_REQUIRE(K >= 1 && K <= ORD_MAX_K && n_rows >= 0, "nbr_row_order: kernel volume %d not in 1..%d or bad row count", K, ORD_MAX_K);
  if (n_rows == 0) return SSC_OK;
  SSC_REQUIRE(nbr && order && scratch, "nbr_row_order: null pointer");
  SSC_REQUIRE(scratch_bytes >= ssc_nbr_row_order_scratch_bytes(K, n_rows), "nbr_row_order: scratch too small");
  cudaStream_t st = as_stream(stream);
  const int n_blocks = ceil_div(n_rows, ORD_BLOCK);
  const size_t cells = (size_t)(K + 1) * n_blocks;
  uint8_t *sp = (uint8_t *)scratch;
  uint16_t *keys = (uint16_t *)sp;
  sp += order_align((size_t)n_rows * 2);
  uint32_t *hist = (uint32_t *)sp;
  sp += order_align(cells * 4);
  uint32_t *base = (uint32_t *)sp;
  sp += order_align(cells * 4);
  uint32_t *block_sums = (uint32_t *)sp;
  { row_key_hist_kernel<<<n_blocks, ORD_BLOCK, (K + 1) * 4, st>>>(nbr, K, n_rows, keys, hist, n_blocks); note_launches(1); }
  SSC_CHECK_LAUNCH("row_key_hist");
  int rc = exclusive_scan_u32<false>(hist, (long long)cells, base, block_sums, nullptr, nullptr, st);
  if (rc != 0) return rc;
  { row_scatter_kernel<<<n_blocks, ORD_BLOCK, 32 * (K + 1) * 4, st>>>(keys, K + 1, n_rows, base, n_blocks, order); note_launches(1); }
  SSC_CHECK_LAUNCH("row_scatter");
  return SSC_OK;
}

extern "C" size_t ssc_nbr_row_order_planes_scratch_bytes(const int ksize[3], int n_rows) {
  if (!ksize || n_rows < 0 || ksize[0] < 1 || ksize[1] < 1 || ksize[2] < 1 || ksize[0] + ksize[1] + ksize[2] > PLANE_MAX_BITS) return 0;
  const size_t n_blocks = (size_t)ceil_div(n_rows > 0 ? n_rows : 1, PLANE_BLOCK);
  const size_t cells = (size_t)((1 << (ksize[0] + ksize[1] + ksize[2])) + 1) * n_blocks;
  return order_align((size_t)n_rows * 2) + 2 * order_align(cells * 4) + order_align((cells / 1024 + 2) * 4) +
         order_align((size_t)2 << PLANE_MAX_BITS);
}

extern "C" int ssc_nbr_row_order_planes(const int32_t *nbr, const int ksize[3], int n_rows, int32_t *order,
                                        int32_t *nbr_in_order, void *scratch, size_t scratch_bytes,
                                        const int32_t *n_rows_dev, void *stream) {
  SSC_REQUIRE(ksize && n_rows >= 0 && ksize[0] >= 1 && ksize[1] >= 1 && ksize[2] >= 1 &&
                  ksize[0] + ksize[1] + ksize[2] <= PLANE_MAX_BITS,
              "nbr_row_order_planes: kernel sizes must add up to at most %d", PLANE_MAX_BITS);
  if (n_rows == 0) return SSC_OK;
  SSC_REQUIRE(nbr && order && scratch, "nbr_row_order_planes: null pointer");
  SSC_REQUIRE(scratch_bytes >= ssc_nbr_row_order_planes_scratch_bytes(ksize, n_rows), "nbr_row_order_planes: scratch too small");
  cudaStream_t st = as_stream(stream);
  const int B = (1 << (ksize[0] + ksize[1] + ksize[2])) + 1;
  const int n_blocks = ceil_div(n_rows, PLANE_BLOCK);
  const size_t cells = (size_t)B * n_blocks;
  uint8_t *sp = (uint8_t *)scratch;
  uint16_t *keys = (uint16_t *)sp;
  sp += order_align((size_t)n_rows * 2);
  uint32_t *hist = (uint32_t *)sp;
  sp += order_align(cells * 4);
  uint32_t *base = (uint32_t *)sp;
  sp += order_align(cells * 4);
  uint32_t *block_sums = (uint32_t *)sp;
  sp += order_align((cells / 1024 + 2) * 4);
  uint16_t *bucket_table = (uint16_t *)sp;
  { plane_bucket_table_kernel<<<1, PLANE_BLOCK, 0, st>>>(ksize[0], ksize[1], ksize[2], bucket_table); note_launches(1); }
  { row_plane_key_hist_kernel<<<n_blocks, PLANE_BLOCK, (2 * B - 1) * 4, st>>>(nbr, ksize[0], ksize[1], ksize[2], n_rows, n_rows_dev, bucket_table, keys, hist, n_blocks); note_launches(1); }
  SSC_CHECK_LAUNCH("row_plane_key_hist");
  int rc = exclusive_scan_u32<false>(hist, (long long)cells, base, block_sums, nullptr, nullptr, st);
  if (rc != 0) return rc;
  { row_scatter_kernel<<<n_blocks, PLANE_BLOCK, (PLANE_BLOCK / 32) * B * 4, st>>>(keys, B, n_rows, base, n_blocks, order, nbr,
                                                                                    ksize[0] * ksize[1] * ksize[2], nbr_in_order); note_launches(1); }
  SSC_CHECK_LAUNCH("row_scatter");
  return SSC_OK;
}
