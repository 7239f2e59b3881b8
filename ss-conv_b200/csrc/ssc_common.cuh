// Shared host/device helpers for the ssconv_b200 library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/ssconv_b200.h"

namespace ssc {

// Per-thread error message behind ssc_last_error().
char *error_buffer();
int fail(int code, const char *fmt, ...);

// Kernel-launch bookkeeping behind ssc_kernel_launches().
void note_launches(int n);

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

#define SSC_CHECK_LAUNCH(name)                                                     \
  do {                                                                             \
    cudaError_t e__ = cudaGetLastError();                                          \
    if (e__ != cudaSuccess)                                                        \
      return ssc::fail(SSC_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e__));     \
  } while (0)

#define SSC_REQUIRE(cond, ...)                                                     \
  do {                                                                             \
    if (!(cond)) return ssc::fail(SSC_ERR_INVALID, __VA_ARGS__);                   \
  } while (0)

// Number of valid rows of a launch whose row count may still be on the device: `cap` is the
// host-side bound (and the row stride of the tables), `n_dev` (may be null) the exact count.
__device__ __forceinline__ int live_rows(int cap, const int32_t *n_dev) {
  if (n_dev == nullptr) return cap;
  const int v = *n_dev;
  return v < 0 ? 0 : (v < cap ? v : cap);
}

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// 3-D geometry of one rulebook request, passed by value to kernels.
struct Geometry {
  int in_shape[3];
  int out_shape[3];
  int ksize[3];
  int stride[3];
  int padding[3];
  int dilation[3];
  int K;
  int transpose;
};

// ----------------------------------------------------------------------------------
// Coordinate hash: open addressing over 4-slot buckets (one 32-byte sector per probe).
// A slot packs (key << 32 | row); the all-ones word marks an empty slot.
// ----------------------------------------------------------------------------------
constexpr unsigned long long kEmptySlot = 0xFFFFFFFFFFFFFFFFull;
constexpr int kBucketSlots = 4;

__host__ __device__ inline uint32_t hash_mix(uint32_t k) {
  k ^= k >> 16;
  k *= 0x85ebca6bu;
  k ^= k >> 13;
  k *= 0xc2b2ae35u;
  k ^= k >> 16;
  return k;
}

inline uint32_t hash_buckets_for(int n) {
  // load factor <= 0.5 over 4-slot buckets, power of two, at least 64 buckets
  uint32_t want = (uint32_t)((2ll * (n > 0 ? n : 1) + kBucketSlots - 1) / kBucketSlots);
  uint32_t b = 64;
  while (b < want) b <<= 1;
  return b;
}

int bitmap_decode(const uint32_t *bitmap, const uint32_t *word_prefix, long long n_words, const int shape[3],
                  int n_out, int32_t *out_indices, cudaStream_t st);

}  // namespace ssc
