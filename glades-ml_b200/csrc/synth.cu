// Counter-based synthetic inputs: Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random
// numbers: as easy as 1, 2, 3", SC'11).  key = (seed lo, seed hi), counter = (index lo, index hi,
// stream, 0); element i takes word 0 of block i, so any element can be regenerated on its own, on
// the CPU or the GPU.  dist 0: U = (u32 >> 8) * 2^-24 (exact in fp32).  dist 1: N(0,1) by
// Box-Muller in double on the uniforms of elements 2*(i/2) and 2*(i/2)+1.
// out = offset + scale * value, with the product and the sum rounded separately so that the CPU
// and the GPU agree bit for bit on the uniform stream.
#include "common.cuh"
#include "internal.h"

namespace glb {

__device__ __forceinline__ unsigned philox_u32(unsigned long long seed, unsigned stream_id, unsigned long long index)
{
	unsigned c0 = (unsigned)index, c1 = (unsigned)(index >> 32), c2 = stream_id, c3 = 0u;
	unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
#pragma unroll
	for (int r = 0; r < 10; ++r)
	{
		const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
		const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
		const unsigned n0 = hi1 ^ c1 ^ k0;
		const unsigned n2 = hi0 ^ c3 ^ k1;
		c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
		k0 += 0x9E3779B9u;
		k1 += 0xBB67AE85u;
	}
	return c0;
}

// out[j] = element (first + j) of the stream, j < n; `first` must be even for dist 1 (pairs of elements
// share one Box-Muller draw).
__global__ void __launch_bounds__(256) synth_fill_kernel(float* out, long long n, long long first, unsigned long long seed,
                                                          unsigned stream_id, int dist, float scale, float offset)
{
	const long long stride = (long long)gridDim.x * blockDim.x;
	for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride)
	{
		const long long i = first + j;
		float v;
		if (dist == 0)
			v = __fmul_rn((float)(philox_u32(seed, stream_id, (unsigned long long)i) >> 8), 1.0f / 16777216.0f);
		else
		{
			const unsigned long long b = (unsigned long long)i & ~1ull;
			const float u1 = __fmul_rn(__fadd_rn((float)(philox_u32(seed, stream_id, b) >> 8), 0.5f), 1.0f / 16777216.0f);
			const float u2 = __fmul_rn((float)(philox_u32(seed, stream_id, b + 1) >> 8), 1.0f / 16777216.0f);
			const double rad = sqrt(-2.0 * log((double)u1));
			const double ang = 6.283185307179586 * (double)u2;
			v = (float)(rad * ((i & 1) ? sin(ang) : cos(ang)));
		}
		out[j] = __fadd_rn(offset, __fmul_rn(scale, v));
	}
}

cudaError_t launch_synth_fill(float* out, long long n, long long first, unsigned long long seed, unsigned stream_id, int dist,
                              float scale, float offset, cudaStream_t s)
{
	if (first < 0 || (dist == 1 && (first & 1))) return cudaErrorInvalidValue;
	long long blocks = (n + 255) / 256;
	if (blocks > 148 * 16) blocks = 148 * 16;
	if (blocks < 1) blocks = 1;
	synth_fill_kernel<<<(unsigned)blocks, 256, 0, s>>>(out, n, first, seed, stream_id, dist, scale, offset);
	return cudaGetLastError();
}

__global__ void __launch_bounds__(256) onehot_fill_kernel(float* y, const int* labels, long long rows, int n, float on, float off)
{
	const long long total = rows * n;
	const long long stride = (long long)gridDim.x * blockDim.x;
	for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
	{
		const long long r = i / n;
		y[i] = ((int)(i - r * n) == labels[r]) ? on : off;
	}
}

cudaError_t launch_onehot_fill(float* y, const int* labels, long long rows, int n, float on, float off, cudaStream_t s)
{
	long long blocks = (rows * n + 255) / 256;
	if (blocks > 148 * 16) blocks = 148 * 16;
	if (blocks < 1) blocks = 1;
	onehot_fill_kernel<<<(unsigned)blocks, 256, 0, s>>>(y, labels, rows, n, on, off);
	return cudaGetLastError();
}

}  // namespace glb
