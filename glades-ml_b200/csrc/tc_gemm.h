// Interface between the C-ABI layer and the tensor-core (TMA + tcgen05, 3xTF32) batched path.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "glades_b200.h"

namespace glb {

struct TcState;

// True when every matrix product of a `rows`-row window of this network fits the tensor-core
// kernel's tiles (and, unless forced, is large enough to be worth it).
bool tc_shapes_ok(const gl_net_desc& d, int rows, bool forced);
TcState* tc_create(const gl_net_desc& d, float* dW, float* dBias, cudaStream_t s);
void tc_destroy(TcState* t);
// The fp32 master weights were overwritten from outside: the split operand copies are stale.
void tc_weights_changed(TcState* t);
// A_{l+1} = squash(A_l W_l^T + b_l) for l = 0..H; fp32 activations land in dA[1..H+1].
cudaError_t tc_forward(TcState* t, const float* X, int rows, float* const* dA, int64_t* launches);
// Given the output delta dD[H+1]: D_l for l = H..1 and the flat gradient dG (already scaled by lr).
cudaError_t tc_backward(TcState* t, const float* X, int rows, float* const* dA, float* const* dD, float* const* dC,
                        float* dG, int64_t* launches);
// Re-derive the split / transposed operand copies from the updated fp32 weights.
cudaError_t tc_after_update(TcState* t, int64_t* launches);

}  // namespace glb
