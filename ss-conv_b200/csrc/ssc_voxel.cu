// Voxelization (Point2Voxel), point<-voxel interpolation (Voxel2Point) helpers.  HBM-bound.
#include "ssc_common.cuh"
#include "ssc_scan.cuh"

namespace ssc {

// ------------------------------------------------------------ voxel2point_map / voxelize
__global__ void v2p_map_kernel(const int32_t *__restrict__ inverse, const int32_t *__restrict__ ids, int32_t *maps,
                               int n_point, int n_voxel, int max_active, int mode) {
  int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_point) return;
  int v = inverse[p];
  if ((unsigned)v >= (unsigned)n_voxel) return;
  int id = ids[p];
  int32_t *row = maps + (size_t)v * (max_active + 1);
  if (mode == 1) {
    atomicMin(row + 1, id);
    row[0] = 1;
  } else if (mode == 2) {
    atomicMax(row + 1, id);
    row[0] = 1;
  } else {
    int slot = atomicAdd(row, 1);
    if (slot < max_active) row[slot + 1] = id;
  }
}

// Modes 3/4: order every row's ids ascending so that later sums are reproducible.
__global__ void v2p_sort_rows_kernel(int32_t *maps, int n_voxel, int max_active) {
  int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= n_voxel) return;
  int32_t *row = maps + (size_t)v * (max_active + 1);
  int n = row[0];
  if (n > max_active) n = max_active;
  for (int i = 2; i <= n; ++i) {
    int key = row[i], j = i - 1;
    while (j >= 1 && row[j] > key) {
      row[j + 1] = row[j];
      --j;
    }
    row[j + 1] = key;
  }
}

__global__ void voxelize_fwd_kernel(const float *__restrict__ feats, float *__restrict__ out,
                                    const int32_t *__restrict__ maps, int average, int n_voxel, int max_active, int c) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n_voxel * c) return;
  int v = (int)(t / c), ch = (int)(t - (long long)v * c);
  const int32_t *row = maps + (size_t)v * (max_active + 1);
  int n = row[0];
  float mult = (average && n > 0) ? __fdiv_rn(1.f, (float)n) : 1.f;
  float acc = 0.f;
  for (int i = 1; i <= n; ++i) acc = __fadd_rn(acc, __fmul_rn(mult, __ldg(feats + (size_t)row[i] * c + ch)));
  out[t] = acc;
}

// ----------------------------------------------------------------- fused Point2Voxel core
struct P2VScratch {
  uint32_t *bitmap, *word_prefix, *block_sums;
  uint32_t *count;   // [n_point + 1] per-voxel point count, then exclusive start offsets
  uint32_t *cursor;  // [n_point] arrival rank of every point in its voxel (modes 3/4) or selected point per voxel (modes 1/2)
  int32_t *order;    // [n_point] point ids grouped by voxel
  uint32_t *block_sums2;
  int32_t *misc;
  long long n_words;
  size_t total;
};

static P2VScratch carve_p2v(void *base, int n_point, int batch, const int grid[3]) {
  P2VScratch s;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void *p = base ? (char *)base + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  long long cells = (long long)batch * grid[0] * grid[1] * grid[2];
  s.n_words = (cells + 31) / 32;
  s.bitmap = (uint32_t *)take((size_t)s.n_words * 4);
  s.word_prefix = (uint32_t *)take((size_t)s.n_words * 4);
  s.block_sums = (uint32_t *)take(((size_t)((s.n_words + 1023) / 1024) + 2) * 4);
  s.count = (uint32_t *)take(((size_t)n_point + 2) * 4);
  s.cursor = (uint32_t *)take(((size_t)n_point + 2) * 4);
  s.order = (int32_t *)take(((size_t)n_point + 2) * 4);
  s.block_sums2 = (uint32_t *)take(((size_t)((n_point + 1023) / 1024) + 2) * 4);
  s.misc = (int32_t *)take(256);
  s.total = off;
  return s;
}

struct VoxelGrid {
  int grid[3];
  float unit[3];
  float half[3];
};

// Cell of a point: int((p + half) / unit), fp32 arithmetic, truncation toward zero, exactly
// the element-wise torch expression it replaces.  Returns false when the cell lies outside
// the grid (such a point is dropped).
__device__ __forceinline__ bool point_cell(const float *p, int b, int batch, const VoxelGrid &g, uint32_t &flat) {
  int c[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    c[d] = (int)__fdiv_rn(__fadd_rn(p[d], g.half[d]), g.unit[d]);
    if ((unsigned)c[d] >= (unsigned)g.grid[d]) return false;
  }
  if ((unsigned)b >= (unsigned)batch) return false;
  flat = (uint32_t)(((b * g.grid[0] + c[0]) * g.grid[1] + c[1]) * g.grid[2] + c[2]);
  return true;
}

__global__ void p2v_mark_kernel(const float *__restrict__ points, const int32_t *__restrict__ batch_ids, int n,
                                int batch, VoxelGrid g, uint32_t *bitmap, int32_t *status) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float p[3] = {points[i * 3 + 0], points[i * 3 + 1], points[i * 3 + 2]};
  uint32_t flat;
  if (!point_cell(p, batch_ids[i], batch, g, flat)) {
    atomicOr(status, 1);
    return;
  }
  atomicOr(bitmap + (flat >> 5), 1u << (flat & 31));
}

// What the host needs to know about a point batch before voxelizing it, in one pass:
// stats[0] points outside the grid (|p| > half extent or cell index out of range),
// stats[1] positions where the batch id decreases, stats[2] positions where it changes,
// stats[3] the last batch id.
__global__ void p2v_stats_kernel(const float *__restrict__ points, const int32_t *__restrict__ batch_ids, int n,
                                 VoxelGrid g, int32_t *stats) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool out = false, down = false, change = false;
  if (i < n) {
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const float p = points[i * 3 + d];
      const int c = (int)__fdiv_rn(__fadd_rn(p, g.half[d]), g.unit[d]);
      out = out || fabsf(p) > g.half[d] || (unsigned)c >= (unsigned)g.grid[d];
    }
    if (i > 0) {
      const int a = batch_ids[i - 1], b = batch_ids[i];
      down = b < a;
      change = b != a;
    }
    if (i == n - 1) stats[3] = batch_ids[i];
  }
  const int n_out = __syncthreads_count(out), n_down = __syncthreads_count(down), n_change = __syncthreads_count(change);
  if (threadIdx.x == 0) {
    if (n_out) atomicAdd(stats + 0, n_out);
    if (n_down) atomicAdd(stats + 1, n_down);
    if (n_change) atomicAdd(stats + 2, n_change);
  }
}

__global__ void p2v_inverse_kernel(const float *__restrict__ points, const int32_t *__restrict__ batch_ids, int n,
                                   int batch, VoxelGrid g, const uint32_t *__restrict__ bitmap,
                                   const uint32_t *__restrict__ word_prefix, int mode, int32_t *inverse,
                                   uint32_t *count, uint32_t *select) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float p[3] = {points[i * 3 + 0], points[i * 3 + 1], points[i * 3 + 2]};
  uint32_t flat;
  if (!point_cell(p, batch_ids[i], batch, g, flat)) {
    inverse[i] = -1;
    return;
  }
  uint32_t w = flat >> 5, bit = flat & 31;
  int v = (int)(word_prefix[w] + __popc(bitmap[w] & ((1u << bit) - 1u)));
  inverse[i] = v;
  if (mode == 1) atomicMin(select + v, (uint32_t)i);
  else if (mode == 2) atomicMax(select + v, (uint32_t)i);
  else select[i] = atomicAdd(count + v, 1u);   // modes 3 / 4: arrival rank of the point in its voxel (select is per point then)
}

// order[start of the point's voxel + its arrival rank] = point: the rank was taken when the points were
// counted, so this pass needs no atomics (the lists are put into point order by the pass after it).
__global__ void p2v_scatter_kernel(const int32_t *__restrict__ inverse, int n, const uint32_t *__restrict__ start,
                                   const uint32_t *__restrict__ rank, int32_t *order) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int v = inverse[i];
  if (v < 0) return;
  order[__ldg(start + v) + __ldg(rank + i)] = i;
}

__global__ void p2v_sort_segments_kernel(const uint32_t *__restrict__ start, int n_voxel, int32_t *order) {
  int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= n_voxel) return;
  int a = (int)start[v], b = (int)start[v + 1];
  for (int i = a + 1; i < b; ++i) {
    int key = order[i], j = i - 1;
    while (j >= a && order[j] > key) {
      order[j + 1] = order[j];
      --j;
    }
    order[j + 1] = key;
  }
}

__global__ void p2v_reduce_kernel(const float *__restrict__ feats, int c, const uint32_t *__restrict__ start,
                                  const int32_t *__restrict__ order, int n_voxel, int average, float *__restrict__ out) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n_voxel * c) return;
  int v = (int)(t / c), ch = (int)(t - (long long)v * c);
  int a = (int)start[v], b = (int)start[v + 1];
  int n = b - a;
  float mult = (average && n > 0) ? __fdiv_rn(1.f, (float)n) : 1.f;
  float acc = 0.f;
  for (int i = a; i < b; ++i) acc = __fadd_rn(acc, __fmul_rn(mult, __ldg(feats + (size_t)order[i] * c + ch)));
  out[t] = acc;
}

// The same sums with one thread per voxel and the channels (at most 8: xyz, colour, a few scalars)
// in registers: the point list is read once per voxel instead of once per channel, no 64-bit
// division.  Per (voxel, channel) the additions happen in the same order as above: same bits.
template <int CMAX>
__global__ void __launch_bounds__(256)
p2v_reduce_small_kernel(const float *__restrict__ feats, int c, const uint32_t *__restrict__ start,
                        const int32_t *__restrict__ order, int n_voxel, int average, float *__restrict__ out) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= n_voxel) return;
  const int a = (int)start[v], b = (int)start[v + 1];
  const int n = b - a;
  const float mult = (average && n > 0) ? __fdiv_rn(1.f, (float)n) : 1.f;
  float acc[CMAX];
#pragma unroll
  for (int ch = 0; ch < CMAX; ++ch) acc[ch] = 0.f;
  for (int i = a; i < b; ++i) {
    const float *fp = feats + (size_t)__ldg(order + i) * c;
#pragma unroll
    for (int ch = 0; ch < CMAX; ++ch)
      if (ch < c) acc[ch] = __fadd_rn(acc[ch], __fmul_rn(mult, __ldg(fp + ch)));
  }
  float *op = out + (size_t)v * c;
#pragma unroll
  for (int ch = 0; ch < CMAX; ++ch)
    if (ch < c) op[ch] = acc[ch];
}

__global__ void p2v_select_kernel(const float *__restrict__ feats, int c, const uint32_t *__restrict__ select,
                                  int n_voxel, int n_point, float *__restrict__ out) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n_voxel * c) return;
  int v = (int)(t / c), ch = (int)(t - (long long)v * c);
  uint32_t p = select[v];
  out[t] = p < (uint32_t)n_point ? __ldg(feats + (size_t)p * c + ch) : 0.f;
}

static void fill_grid(VoxelGrid &g, const int grid[3], const float unit[3]) {
  for (int d = 0; d < 3; ++d) {
    g.grid[d] = grid[d];
    g.unit[d] = unit[d];
    float total = (float)grid[d] * unit[d];
    g.half[d] = 0.5f * total;
  }
}

// ----------------------------------------------------------------------- three_nn
constexpr int NN_TILE = 1024;

__global__ void nn_tile_range_kernel(const float4 *__restrict__ known, int m, float2 *ranges) {
  __shared__ float smin[8], smax[8];
  int tile = blockIdx.x;
  float lo = INFINITY, hi = -INFINITY;
  for (int i = threadIdx.x; i < NN_TILE; i += blockDim.x) {
    int k = tile * NN_TILE + i;
    if (k < m) {
      float b = known[k].x;
      lo = fminf(lo, b);
      hi = fmaxf(hi, b);
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_down_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_down_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0) {
    smin[threadIdx.x >> 5] = lo;
    smax[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) {
      lo = fminf(lo, smin[w]);
      hi = fmaxf(hi, smax[w]);
    }
    ranges[tile] = make_float2(lo, hi);
  }
}

// 256 queries per block; known points stream through shared memory in tiles of 1024, tiles
// whose batch-id range cannot match any query of the block are skipped.  Scan order and
// comparisons equal the exhaustive reference loop (ascending k, strict <).
__global__ void __launch_bounds__(256)
three_nn_kernel(int n, int m, const float4 *__restrict__ unknown, const float4 *__restrict__ known,
                const float2 *__restrict__ ranges, float *__restrict__ dist2, int32_t *__restrict__ idx) {
  __shared__ float4 tile[NN_TILE];
  __shared__ float qmin_s[8], qmax_s[8];
  int q = blockIdx.x * 256 + threadIdx.x;
  float4 u = q < n ? unknown[q] : make_float4(NAN, 0.f, 0.f, 0.f);
  float lo = q < n ? u.x : INFINITY, hi = q < n ? u.x : -INFINITY;
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_down_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_down_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0) {
    qmin_s[threadIdx.x >> 5] = lo;
    qmax_s[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  float qmin = qmin_s[0], qmax = qmax_s[0];
  for (int w = 1; w < 8; ++w) {
    qmin = fminf(qmin, qmin_s[w]);
    qmax = fmaxf(qmax, qmax_s[w]);
  }
  float best1 = INFINITY, best2 = INFINITY, best3 = INFINITY;
  int i1 = 0, i2 = 0, i3 = 0;
  int n_tiles = (m + NN_TILE - 1) / NN_TILE;
  for (int t = 0; t < n_tiles; ++t) {
    float2 r = ranges[t];
    if (r.y < qmin || r.x > qmax) continue;  // block-uniform
    __syncthreads();
    int base = t * NN_TILE;
    for (int i = threadIdx.x; i < NN_TILE; i += 256) tile[i] = base + i < m ? known[base + i] : make_float4(NAN, 0.f, 0.f, 0.f);
    __syncthreads();
    int cnt = min(NN_TILE, m - base);
    if (q < n && !(r.y < u.x || r.x > u.x)) {
      for (int i = 0; i < cnt; ++i) {
        float4 k = tile[i];
        if (k.x != u.x) continue;
        float dx = __fsub_rn(u.y, k.y), dy = __fsub_rn(u.z, k.z), dz = __fsub_rn(u.w, k.w);
        // the contraction nvcc applies to the reference's dx*dx + dy*dy + dz*dz
        // (interpolate_cuda_kernel.cu:39), checked bit for bit against the reference's own kernel
        float d = __fmaf_rn(dz, dz, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
        if (d < best1) {
          best3 = best2; i3 = i2;
          best2 = best1; i2 = i1;
          best1 = d; i1 = base + i;
        } else if (d < best2) {
          best3 = best2; i3 = i2;
          best2 = d; i2 = base + i;
        } else if (d < best3) {
          best3 = d; i3 = base + i;
        }
      }
    }
  }
  if (q < n) {
    dist2[q * 3 + 0] = best1; dist2[q * 3 + 1] = best2; dist2[q * 3 + 2] = best3;
    idx[q * 3 + 0] = i1; idx[q * 3 + 1] = i2; idx[q * 3 + 2] = i3;
  }
}

__global__ void three_interpolate_kernel(int c, int n, const float *__restrict__ points,
                                         const int32_t *__restrict__ idx, const float *__restrict__ weight,
                                         float *__restrict__ out) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (long long)n * c) return;
  int p = (int)(t / c), ch = (int)(t - (long long)p * c);
  float w0 = weight[p * 3 + 0], w1 = weight[p * 3 + 1], w2 = weight[p * 3 + 2];
  int i0 = idx[p * 3 + 0], i1 = idx[p * 3 + 1], i2 = idx[p * 3 + 2];
  // w0*p0 + w1*p1 + w2*p2 as nvcc contracts it in the reference (interpolate_cuda_kernel.cu:100),
  // checked bit for bit against the reference's own kernel
  float b = __fmul_rn(w1, __ldg(points + (size_t)i1 * c + ch));
  float a = __fmaf_rn(w0, __ldg(points + (size_t)i0 * c + ch), b);
  out[t] = __fmaf_rn(w2, __ldg(points + (size_t)i2 * c + ch), a);
}

// Four channels per thread (16-byte gathers and stores, 32-bit index arithmetic) for channel
// counts that are multiples of four; the same arithmetic per element.
__global__ void __launch_bounds__(256)
three_interpolate_vec4_kernel(uint32_t groups, uint32_t total, const float4 *__restrict__ points,
                              const int32_t *__restrict__ idx, const float *__restrict__ weight, float4 *__restrict__ out) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const uint32_t p = t / groups, g = t - p * groups;
  const float w0 = __ldg(weight + p * 3 + 0), w1 = __ldg(weight + p * 3 + 1), w2 = __ldg(weight + p * 3 + 2);
  const int i0 = __ldg(idx + p * 3 + 0), i1 = __ldg(idx + p * 3 + 1), i2 = __ldg(idx + p * 3 + 2);
  const float4 p0 = __ldg(points + (size_t)i0 * groups + g);
  const float4 p1 = __ldg(points + (size_t)i1 * groups + g);
  const float4 p2 = __ldg(points + (size_t)i2 * groups + g);
  float4 r;
  r.x = __fmaf_rn(w2, p2.x, __fmaf_rn(w0, p0.x, __fmul_rn(w1, p1.x)));
  r.y = __fmaf_rn(w2, p2.y, __fmaf_rn(w0, p0.y, __fmul_rn(w1, p1.y)));
  r.z = __fmaf_rn(w2, p2.z, __fmaf_rn(w0, p0.z, __fmul_rn(w1, p1.z)));
  r.w = __fmaf_rn(w2, p2.w, __fmaf_rn(w0, p0.w, __fmul_rn(w1, p1.w)));
  out[t] = r;
}

}  // namespace ssc

using namespace ssc;

extern "C" int ssc_voxel2point_map(const int32_t *inverse, const int32_t *ids, int32_t *maps, int n_point,
                                   int n_voxel, int max_active, int mode, void *stream) {
  SSC_REQUIRE(mode >= 1 && mode <= 4, "voxel2point_map: mode %d not in 1..4", mode);
  SSC_REQUIRE(n_point >= 0 && n_voxel >= 0 && max_active >= 1, "voxel2point_map: bad sizes");
  if (n_point == 0 || n_voxel == 0) return SSC_OK;
  SSC_REQUIRE(inverse && ids && maps, "voxel2point_map: null pointer");
  cudaStream_t st = as_stream(stream);
  { v2p_map_kernel<<<ceil_div(n_point, 256), 256, 0, st>>>(inverse, ids, maps, n_point, n_voxel, max_active, mode); note_launches(1); }
  if (mode >= 3) { v2p_sort_rows_kernel<<<ceil_div(n_voxel, 128), 128, 0, st>>>(maps, n_voxel, max_active); note_launches(1); }
  SSC_CHECK_LAUNCH("voxel2point_map");
  return SSC_OK;
}

extern "C" int ssc_voxelize_fwd(const float *feats, float *out, const int32_t *maps, int mode, int n_voxel,
                                int max_active, int c, void *stream) {
  SSC_REQUIRE(n_voxel >= 0 && max_active >= 1 && c >= 1, "voxelize_fwd: bad sizes");
  if (n_voxel == 0) return SSC_OK;
  SSC_REQUIRE(feats && out && maps, "voxelize_fwd: null pointer");
  long long threads = (long long)n_voxel * c;
  { voxelize_fwd_kernel<<<ceil_div(threads, 256), 256, 0, as_stream(stream)>>>(feats, out, maps, mode == 4, n_voxel,
                                                                            max_active, c); note_launches(1); }
  SSC_CHECK_LAUNCH("voxelize_fwd");
  return SSC_OK;
}

extern "C" size_t ssc_p2v_scratch_bytes(int n_point, int batch, const int grid[3]) {
  if (n_point < 0 || batch < 1 || !grid) return 0;
  return carve_p2v(nullptr, n_point, batch, grid).total;
}

// Feature steering: every point is moved into the frame of its sample, new_p = (p - t_b) . R_b
// (/ (s_b + 1e-8)), and every irrep block of its feature row is multiplied from the right by the
// sample's representation matrix D^l_b.  One thread per (point, output channel or coordinate).
__global__ void steer_kernel(const float *__restrict__ points, const float *__restrict__ feats,
                             const int32_t *__restrict__ ids, const float *__restrict__ rot, const float *__restrict__ trans,
                             const float *__restrict__ scale, const float *__restrict__ dmats, int d_stride,
                             const int32_t *__restrict__ chan, int n, int c, int n_sample, float *__restrict__ new_points,
                             float *__restrict__ new_feats) {
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int width = c + 3;
  if (t >= (long long)n * width) return;
  const int p = (int)(t / width), k = (int)(t - (long long)p * width);
  const int b = ids[p];
  if ((unsigned)b >= (unsigned)n_sample) {  // foreign batch id: leave a defined value
    if (k < c) new_feats[(size_t)p * c + k] = 0.f;
    else new_points[(size_t)p * 3 + (k - c)] = 0.f;
    return;
  }
  if (k >= c) {
    const int j = k - c;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 3; ++i) acc += (points[(size_t)p * 3 + i] - trans[b * 3 + i]) * rot[b * 9 + i * 3 + j];
    if (scale) acc = acc / (scale[b] + 1e-8f);
    new_points[(size_t)p * 3 + j] = acc;
    return;
  }
  const int start = chan[k * 3 + 0], d = chan[k * 3 + 1], off = chan[k * 3 + 2];
  const int j = k - start;
  const float *D = dmats + (size_t)b * d_stride + off;
  float acc = 0.f;
  for (int i = 0; i < d; ++i) acc += feats[(size_t)p * c + start + i] * D[i * d + j];
  new_feats[(size_t)p * c + k] = acc;
}

extern "C" int ssc_steer_fwd(const float *points, const float *feats, const int32_t *ids, const float *rot,
                             const float *trans, const float *scale, const float *dmats, int d_stride,
                             const int32_t *chan, int n, int c, int n_sample, float *new_points, float *new_feats,
                             void *stream) {
  SSC_REQUIRE(n >= 0 && c >= 1 && n_sample >= 1 && d_stride >= 1, "steer_fwd: bad sizes");
  if (n == 0) return SSC_OK;
  SSC_REQUIRE(points && feats && ids && rot && trans && dmats && chan && new_points && new_feats, "steer_fwd: null pointer");
  long long total = (long long)n * (c + 3);
  { steer_kernel<<<ceil_div(total, 256), 256, 0, as_stream(stream)>>>(points, feats, ids, rot, trans, scale, dmats, d_stride,
                                                                    chan, n, c, n_sample, new_points, new_feats); note_launches(1); }
  SSC_CHECK_LAUNCH("steer_fwd");
  return SSC_OK;
}

extern "C" int ssc_p2v_stats(const float *points, const int32_t *batch_ids, int n_point, const int grid[3],
                             const float unit[3], int32_t *stats_dev, void *stream) {
  SSC_REQUIRE(n_point >= 0 && grid && unit && stats_dev, "p2v_stats: bad arguments");
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(stats_dev, 0, 4 * sizeof(int32_t), st);
  if (n_point == 0) return SSC_OK;
  SSC_REQUIRE(points && batch_ids, "p2v_stats: null pointer");
  VoxelGrid g;
  fill_grid(g, grid, unit);
  { p2v_stats_kernel<<<ceil_div(n_point, 256), 256, 0, st>>>(points, batch_ids, n_point, g, stats_dev); note_launches(1); }
  SSC_CHECK_LAUNCH("p2v_stats");
  return SSC_OK;
}

extern "C" int ssc_p2v_count(const float *points, const int32_t *batch_ids, int n_point, int batch, const int grid[3],
                             const float unit[3], int32_t *n_voxel_dev, int32_t *status, void *scratch,
                             size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(n_point >= 0 && batch >= 1 && grid && unit && n_voxel_dev, "p2v_count: bad arguments");
  long long cells = (long long)batch * grid[0] * grid[1] * grid[2];
  SSC_REQUIRE(cells > 0 && cells < 2147483647ll, "p2v_count: batch*volume does not fit the int32 flat index");
  P2VScratch s = carve_p2v(scratch, n_point, batch, grid);
  if (!scratch || scratch_bytes < s.total) return fail(SSC_ERR_SCRATCH, "p2v_count: scratch %zu < %zu bytes", scratch_bytes, s.total);
  cudaStream_t st = as_stream(stream);
  VoxelGrid g;
  fill_grid(g, grid, unit);
  cudaMemsetAsync(s.bitmap, 0, (size_t)s.n_words * 4, st);
  cudaMemsetAsync(s.misc, 0, 256, st);
  if (n_point > 0) { p2v_mark_kernel<<<ceil_div(n_point, 256), 256, 0, st>>>(points, batch_ids, n_point, batch, g, s.bitmap, status ? status : s.misc + 1); note_launches(1); }
  SSC_CHECK_LAUNCH("p2v_mark");
  if (int e = exclusive_scan_u32<true>(s.bitmap, s.n_words, s.word_prefix, s.block_sums, s.misc, n_voxel_dev, st)) return e;
  SSC_CHECK_LAUNCH("p2v_count");
  return SSC_OK;
}

extern "C" int ssc_p2v_fill(const float *points, const int32_t *batch_ids, const float *feats, int n_point, int c,
                            int batch, const int grid[3], const float unit[3], int mode, int n_voxel,
                            int32_t *voxel_indices, int32_t *inverse, float *voxel_feats, void *scratch,
                            size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(mode >= 1 && mode <= 4, "p2v_fill: mode %d not in 1..4", mode);
  SSC_REQUIRE(n_point >= 0 && n_voxel >= 0 && n_voxel <= n_point && c >= 1 && grid && unit, "p2v_fill: bad arguments");
  if (n_voxel == 0) return SSC_OK;
  SSC_REQUIRE(points && batch_ids && feats && voxel_indices && inverse && voxel_feats, "p2v_fill: null pointer");
  P2VScratch s = carve_p2v(scratch, n_point, batch, grid);
  if (!scratch || scratch_bytes < s.total) return fail(SSC_ERR_SCRATCH, "p2v_fill: scratch %zu < %zu bytes", scratch_bytes, s.total);
  cudaStream_t st = as_stream(stream);
  VoxelGrid g;
  fill_grid(g, grid, unit);
  if (int e = bitmap_decode(s.bitmap, s.word_prefix, s.n_words, grid, n_voxel, voxel_indices, st)) return e;
  if (mode >= 3) cudaMemsetAsync(s.count, 0, ((size_t)n_voxel + 1) * 4, st);
  else cudaMemsetAsync(s.cursor, mode == 1 ? 0xFF : 0x00, (size_t)n_voxel * 4, st);
  { p2v_inverse_kernel<<<ceil_div(n_point, 256), 256, 0, st>>>(points, batch_ids, n_point, batch, g, s.bitmap, s.word_prefix,
                                                            mode, inverse, s.count, s.cursor); note_launches(1); }
  SSC_CHECK_LAUNCH("p2v_inverse");
  long long threads = (long long)n_voxel * c;
  if (mode >= 3) {
    // counts -> exclusive start offsets (in place), cursor = copy
    if (int e = exclusive_scan_u32<false>(s.count, (long long)n_voxel + 1, s.count, s.block_sums2, nullptr, nullptr, st)) return e;
    { p2v_scatter_kernel<<<ceil_div(n_point, 256), 256, 0, st>>>(inverse, n_point, s.count, s.cursor, s.order); note_launches(1); }
    { p2v_sort_segments_kernel<<<ceil_div(n_voxel, 128), 128, 0, st>>>(s.count, n_voxel, s.order); note_launches(1); }
    if (c <= 4) {
      { p2v_reduce_small_kernel<4><<<ceil_div(n_voxel, 256), 256, 0, st>>>(feats, c, s.count, s.order, n_voxel, mode == 4, voxel_feats); note_launches(1); }
    } else if (c <= 8) {
      { p2v_reduce_small_kernel<8><<<ceil_div(n_voxel, 256), 256, 0, st>>>(feats, c, s.count, s.order, n_voxel, mode == 4, voxel_feats); note_launches(1); }
    } else {
      { p2v_reduce_kernel<<<ceil_div(threads, 256), 256, 0, st>>>(feats, c, s.count, s.order, n_voxel, mode == 4, voxel_feats); note_launches(1); }
    }
  } else {
    { p2v_select_kernel<<<ceil_div(threads, 256), 256, 0, st>>>(feats, c, s.cursor, n_voxel, n_point, voxel_feats); note_launches(1); }
  }
  SSC_CHECK_LAUNCH("p2v_fill");
  return SSC_OK;
}

extern "C" size_t ssc_three_nn_scratch_bytes(int m) {
  return (size_t)ceil_div(m > 0 ? m : 1, NN_TILE) * sizeof(float2);
}

extern "C" int ssc_three_nn(int n, int m, const float *unknown, const float *known, float *dist2, int32_t *idx,
                            void *scratch, size_t scratch_bytes, void *stream) {
  SSC_REQUIRE(n >= 0 && m >= 0, "three_nn: bad sizes");
  if (n == 0) return SSC_OK;
  SSC_REQUIRE(unknown && dist2 && idx && (m == 0 || known), "three_nn: null pointer");
  cudaStream_t st = as_stream(stream);
  int n_tiles = ceil_div(m > 0 ? m : 1, NN_TILE);
  if (!scratch || scratch_bytes < (size_t)n_tiles * sizeof(float2))
    return fail(SSC_ERR_SCRATCH, "three_nn: scratch %zu < %zu bytes", scratch_bytes, (size_t)n_tiles * sizeof(float2));
  float2 *ranges = (float2 *)scratch;
  { nn_tile_range_kernel<<<n_tiles, 256, 0, st>>>((const float4 *)known, m, ranges); note_launches(1); }
  { three_nn_kernel<<<ceil_div(n, 256), 256, 0, st>>>(n, m, (const float4 *)unknown, (const float4 *)known, ranges, dist2, idx); note_launches(1); }
  SSC_CHECK_LAUNCH("three_nn");
  return SSC_OK;
}

extern "C" int ssc_three_interpolate_fwd(int c, int m, int n, const float *points, const int32_t *idx,
                                         const float *weight, float *out, void *stream) {
  SSC_REQUIRE(c >= 1 && n >= 0 && m >= 0, "three_interpolate: bad sizes");
  if (n == 0) return SSC_OK;
  SSC_REQUIRE(points && idx && weight && out, "three_interpolate: null pointer");
  long long threads = (long long)n * c;
  if ((c & 3) == 0 && threads / 4 < (1ll << 31) && (((uintptr_t)points | (uintptr_t)out) & 15u) == 0) {
    const uint32_t groups = (uint32_t)(c >> 2), total = (uint32_t)(threads >> 2);
    { three_interpolate_vec4_kernel<<<ceil_div(total, 256), 256, 0, as_stream(stream)>>>(groups, total, (const float4 *)points, idx, weight, (float4 *)out); note_launches(1); }
    SSC_CHECK_LAUNCH("three_interpolate");
    return SSC_OK;
  }
  { three_interpolate_kernel<<<ceil_div(threads, 256), 256, 0, as_stream(stream)>>>(c, n, points, idx, weight, out); note_launches(1); }
  SSC_CHECK_LAUNCH("three_interpolate");
  return SSC_OK;
}
