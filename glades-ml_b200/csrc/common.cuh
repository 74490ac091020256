// Shared device helpers of the glades feed-forward kernels (sm_100a only).
//
// Two families of scalar functions:
//   *_x  "exact order": every fp32 add / mul / div is an explicit round-to-nearest intrinsic, so
//        the compiler can neither contract a*b+c into an FMA nor reassociate, and transcendental
//        functions are evaluated in double and rounded once (correctly rounded except in ~2^-28 of
//        the cases).  Reference mode uses these; together with the reference's loop order they
//        make the kernels reproduce the reference's x86-64 SSE arithmetic bit for bit wherever
//        the host libm is correctly rounded.
//   plain batched-mode versions: ordinary fp32 with FMA and CUDA's fp32 libm.
//
// Activations and costs follow GMath::squash (GMath/gmath.cpp:22-101), GMath::activationErrDer
// (:182-245), GMath::outputNodeCost (:288-321) and GMath::costErrDer (:323-353) of the reference.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "glades_b200.h"

#define GL_OUTLIER 0.046f  // GMath::OUTLIER, GMath/gmath.h:35: ReLU / leaky threshold

namespace glb {

// ---- exact-order scalar functions (reference mode) ---------------------------------------
__device__ __forceinline__ float exp_x(float v) { return (float)exp((double)v); }
__device__ __forceinline__ float tanh_x(float v) { return (float)tanh((double)v); }
__device__ __forceinline__ float log_x(float v) { return (float)log((double)v); }

__device__ __forceinline__ float sigmoid_x(float z)
{
	return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_x(-z)));
}

__device__ inline float squash_x(float z, int act, float p)
{
	switch (act)
	{
	case GL_ACT_TANH: return tanh_x(z);
	case GL_ACT_TANHP:
		if (z > __fsub_rn(1.0f, p)) return 1.0f;
		if (z < __fsub_rn(p, 1.0f)) return -1.0f;
		return tanh_x(z);
	case GL_ACT_SIGMOID: return sigmoid_x(z);
	case GL_ACT_SIGMOIDP:
		if (z < p) return 0.01f;
		if (z > __fsub_rn(1.0f, p)) return 0.99f;
		return sigmoid_x(z);
	case GL_ACT_RELU: return z < GL_OUTLIER ? 0.0f : z;
	case GL_ACT_LEAKY: return z < GL_OUTLIER ? __fmul_rn(p, z) : z;
	case GL_ACT_LINEAR: return __fmul_rn(p, z);
	case GL_ACT_STEP: return z < p ? 0.0f : 1.0f;
	}
	return 0.0f;
}

// Derivative from the node's OUTPUT value a (the reference never keeps the pre-activation).
__device__ inline float act_der_x(float a, int act, float p)
{
	switch (act)
	{
	case GL_ACT_TANH:
	case GL_ACT_TANHP: return __fsub_rn(1.0f, __fmul_rn(a, a));
	case GL_ACT_SIGMOID:
	case GL_ACT_SIGMOIDP: return __fmul_rn(a, __fsub_rn(1.0f, a));
	case GL_ACT_RELU: return a > 0.0f ? 1.0f : 0.0f;
	case GL_ACT_LEAKY: return a > 0.0f ? 1.0f : (p < 0.0f ? p : -p);
	case GL_ACT_LINEAR: return p;
	case GL_ACT_STEP: return 0.0f;
	}
	return 1.0f;
}

__device__ inline float cost_x(float e, float p, float n, int fx)
{
	switch (fx)
	{
	case GL_OUT_REGRESSION:
	{
		float t = __fsub_rn(e, p);
		return __fdiv_rn(__fmul_rn(t, t), n);
	}
	case GL_OUT_CLASSIFICATION:
	{
		float a = __fmul_rn(e, log_x(p));
		float b = __fmul_rn(__fsub_rn(1.0f, e), log_x(__fsub_rn(1.0f, p)));
		return __fdiv_rn(-__fadd_rn(a, b), n);
	}
	case GL_OUT_KL: return __fdiv_rn(log_x(__fdiv_rn(e, p)), n);
	}
	return 0.0f;
}

__device__ inline float cost_der_x(float e, float p, int fx)
{
	switch (fx)
	{
	case GL_OUT_REGRESSION: return __fmul_rn(2.0f, __fsub_rn(p, e));
	case GL_OUT_CLASSIFICATION: return __fdiv_rn(__fsub_rn(p, e), __fmul_rn(__fsub_rn(1.0f, p), p));
	case GL_OUT_KL: return -__fdiv_rn(e, p);
	}
	return 1.0f;
}

// |p - e| accuracy of one output node, network.cpp:540-547 with GMath::PercentError.
__device__ __forceinline__ float node_accuracy_x(float e, float p)
{
	float pe = __fsub_rn(p, e);
	if (pe < 0.0f) pe = -pe;
	if (pe > 1.0f) pe = 1.0f;
	float acc = __fmul_rn(__fsub_rn(1.0f, pe), 100.0f);
	return acc < 0.0f ? 0.0f : acc;
}

// ---- batched-mode scalar functions ---------------------------------------------------------
__device__ __forceinline__ float squash_b(float z, int act, float p)
{
	switch (act)
	{
	case GL_ACT_TANH: return tanhf(z);
	case GL_ACT_TANHP:
		if (z > 1.0f - p) return 1.0f;
		if (z < p - 1.0f) return -1.0f;
		return tanhf(z);
	case GL_ACT_SIGMOID: return 1.0f / (1.0f + expf(-z));
	case GL_ACT_SIGMOIDP:
		if (z < p) return 0.01f;
		if (z > 1.0f - p) return 0.99f;
		return 1.0f / (1.0f + expf(-z));
	case GL_ACT_RELU: return z < GL_OUTLIER ? 0.0f : z;
	case GL_ACT_LEAKY: return z < GL_OUTLIER ? p * z : z;
	case GL_ACT_LINEAR: return p * z;
	case GL_ACT_STEP: return z < p ? 0.0f : 1.0f;
	case GL_ACT_SOFTMAX: return z;  // the row-wise normalisation is a separate pass
	}
	return 0.0f;
}

__device__ __forceinline__ float act_der_b(float a, int act, float p)
{
	switch (act)
	{
	case GL_ACT_TANH:
	case GL_ACT_TANHP: return 1.0f - a * a;
	case GL_ACT_SIGMOID:
	case GL_ACT_SIGMOIDP: return a * (1.0f - a);
	case GL_ACT_RELU: return a > 0.0f ? 1.0f : 0.0f;
	case GL_ACT_LEAKY: return a > 0.0f ? 1.0f : (p < 0.0f ? p : -p);
	case GL_ACT_LINEAR: return p;
	case GL_ACT_STEP: return 0.0f;
	}
	return 1.0f;
}

// Low TF32 part of an fp32 value for the 3xTF32 tensor-core products: v - trunc_tf32(v), rounded to
// TF32 (the tensor core itself reads trunc_tf32(v) from the unmodified fp32 word).
__device__ __forceinline__ float tf32_lo(float v)
{
	const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
	uint32_t t;
	asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v - hi));
	return __uint_as_float(t);
}

// ---- asynchronous global -> shared copies (cp.async); destinations are 32-bit shared-window addresses ----
__device__ __forceinline__ void cp_async4(uint32_t dst, const float* src, bool valid)
{
	const int bytes = valid ? 4 : 0;  // 0: nothing is read, the destination is zero-filled
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// 16 bytes, of which the first `floats` (0..4) values are read and the rest zero-filled; both addresses 16-byte aligned
__device__ __forceinline__ void cp_async16(uint32_t dst, const float* src, int floats)
{
	const int bytes = floats <= 0 ? 0 : (floats >= 4 ? 16 : floats * 4);
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}
__device__ __forceinline__ double warp_sum_d(double v)
{
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
	return v;
}

}  // namespace glb
