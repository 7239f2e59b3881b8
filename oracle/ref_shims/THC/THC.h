// Stand-in for the THC umbrella header that PyTorch removed in 2.x.
// The reference sources only need the current-stream accessor from it
// (SS_Conv_lib/src/voxelize/interpolation.cpp:20,36,51); no arithmetic lives here.
#pragma once
#include <ATen/cuda/CUDAContext.h>
struct THCState;
static inline cudaStream_t THCState_getCurrentStream(THCState *) {
  return at::cuda::getCurrentCUDAStream();
}
