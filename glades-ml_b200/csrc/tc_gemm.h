// Tensor-core matrix product of batched mode: TMA-fed tcgen05.mma (kind::tf32) with the operands
// split into a high and a low TF32 part ("3xTF32"), fp32 accumulation in tensor memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "internal.h"

namespace glb {

// Tile constraints of the kernel: M % 128 == 0, N % 128 == 0, K % 16 == 0, every operand either
// K-contiguous or M/N-contiguous with 16-byte aligned rows, no per-k scale vector.
bool tc_gemm_supported(const GemmArgs& g);

// C = epilogue(A * B^T) with A ~ A + A_lo and B ~ B + B_lo, where X_lo = X - trunc_tf32(X) (see
// launch_split_lo).  Three tensor-core products per k-step: A*B_lo, A_lo*B, A*B; the tensor core
// reads only the upper 19 bits of each fp32 operand word, so passing X itself supplies trunc_tf32(X).
// err_flag: device int, set non-zero if a bounded wait inside the kernel ran out.
cudaError_t launch_gemm_tc(const GemmArgs& g, const float* A_lo, const float* B_lo, int* err_flag, cudaStream_t s);

// Launch counts per tile variant since the library was loaded: [0] 128-wide tiles, [1] 256-wide tiles,
// [2] launches whose persistent CTAs walked more than one tile each, [3] data-parallel (peer-store) launches,
// [4] launches that split their last wave of tiles along k.
void tc_variant_counts(long long out5[5]);

// Tensor map (128 bytes, 64-byte aligned storage) over a row-major [rows][cols] fp32 matrix with 32 x 32
// boxes, as the epilogue's bulk stores use it; for the per-owner bands of a data-parallel gradient.
bool tc_make_store_map(void* out128, const float* base, long long rows, long long cols, long long ld);

// General 2-D map over a row-major [rows][cols] fp32 matrix (row pitch ld floats, a multiple of 4; base
// 16-byte aligned): boxes of box_rows x box_cols, 128-byte swizzle (box_cols must then be 32) or none.
bool tc_make_map2d(void* out128, const float* base, long long rows, long long cols, long long ld, int box_cols, int box_rows,
                   int swizzle128);

// lo[i] = tf32_round(src[i] - trunc_tf32(src[i])); with rowscale: first dst_scaled[i] = src[i] *
// rowscale[i / ld] is formed (and stored), and lo is taken from that.
cudaError_t launch_split_lo(const float* src, float* lo, long long count, cudaStream_t s);
// dst = src and (lo != NULL) lo = low TF32 parts of src; count a multiple of 4, pointers 16-byte aligned
cudaError_t launch_copy_split_lo(const float* src, float* dst, float* lo, long long count, cudaStream_t s);
cudaError_t launch_scale_split_lo(const float* src, const float* rowscale, int ld, float* dst_scaled, float* lo,
                                  long long count, cudaStream_t s);

}  // namespace glb
