// Declarations shared by the convolution sources (ssc_conv*.cu, ssc_wgrad_tc.cu).
#pragma once
#include "ssc_common.cuh"

namespace ssc {

int sm_count();

// staged operand images (ssc_conv_stage.cu)
size_t conv_tf32_scratch_bytes(int n_in, int c_in);
size_t conv_f16_scratch_bytes(int n_in, int c_in);
int stage_features(const float *features, int n_in, int c_in, void *staged, cudaStream_t st);
int stage_features_16(const float *features, int n_in, int c_in, bool bf16, void *staged, cudaStream_t st);

// Width of a 16-bit (fp16 / bf16) operand row in 4-byte units; rows are padded to 16 bytes.  The
// kernels gather such a row like an fp32 image of that many channels.
inline int f16_row_words(int c_in) { return ((c_in + 7) & ~7) / 2; }

// TF32 layers with few input channels: kernel offsets that share one 128-byte operand row (rows of
// the staged image are c_pad = 4, 8 or 16 floats): 8, 4, 2; else 1.  Decides the packed filter layout.
inline int tf32_offsets_per_row(int c_in) {
  const int c_pad = (c_in + 3) & ~3;
  return (c_pad == 4 || c_pad == 8 || c_pad == 16) ? 32 / c_pad : 1;
}

// geometry of the packed filter image [K][k_slabs][n_pad][128 bytes] (ssc_conv_tc.cu)
bool tc_operand_layout(int c_in_words, int c_out, int *k_slabs, int *n_pad, int *tile_n, int *n_tiles);

// output-stationary tensor-core kernels (ssc_conv_tc.cu)
int conv_fwd_tf32(const float *features, int n_in, int c_in, const void *packed, int K, int c_out,
                  const int32_t *nbr, int n_out, float *out, int32_t *status, void *scratch, size_t scratch_bytes,
                  const int32_t *n_out_dev, const int32_t *order, bool prestaged, bool table_in_order, cudaStream_t st);
int conv_fwd_16(const float *features, int n_in, int c_in, bool bf16, const void *packed, int K, int c_out,
                const int32_t *nbr, int n_out, float *out, int32_t *status, void *scratch, size_t scratch_bytes,
                const int32_t *n_out_dev, const int32_t *order, bool prestaged, bool table_in_order, cudaStream_t st);

// compacted per-offset pair lists of a neighbour table (ssc_wgrad_tc.cu): the lists of the kernel
// offsets follow one another in pair_out / pair_in (ascending output row inside an offset),
// starts[kappa] .. starts[kappa + 1] is the range of offset kappa, starts[K] the number of pairs.
struct PairLists {
  int32_t *pair_out;
  int32_t *pair_in;
  int32_t *starts;   // [K + 1]
};
size_t pair_lists_bytes(int K, int n_out);
int pair_lists_build(const int32_t *nbr, int K, int n_out, void *lists, PairLists *out, cudaStream_t st);
PairLists pair_lists_view(void *lists, int K, int n_out);

}  // namespace ssc
