// Data-parallel gradient exchange over peer memory (one process per GPU, NVLink): the replacement of
// the per-layer all-reduce of the minibatch gradient.
//
// Every weight layer's gradient matrix [n_out][n_in] is cut into row bands, band o owned by rank o.
//   1. reduce-scatter by push: each rank writes its contribution to band o straight into slot
//      [source rank] of rank o's exchange arena -- from the tensor-core product's epilogue (bulk tensor
//      stores through per-owner tensor maps), or with dp_push_bands_kernel for products that ran on the
//      FFMA kernel -- then raises a per-layer flag in every rank's arena (dp_signal_kernel);
//   2. the owner waits for the flags of all sources (dp_wait_kernel, bounded), sums the slots in rank
//      order, applies the update to its band of the weights and writes the new weights into EVERY
//      rank's staging vector (dp_reduce_update_kernel; a rank copies a layer from staging into its
//      weights once its own readers of the old weights are done), then raises a "weights of layer l
//      from owner o" flag everywhere;
//   3. the scalar bias sums and the loss / accuracy sums travel as one 80-byte record per rank
//      (dp_small_push_kernel), summed in rank order by dp_finish_kernel on every rank.
// Sums are taken in rank order, so every replica ends a window with bit-identical weights, run to
// run.  Flags are window counters that only grow; nothing is ever reset.  Every wait is bounded: when
// it runs out the kernel records a code in the handle's status word and returns.
#include "common.cuh"
#include "internal.h"

namespace glb {
namespace {

constexpr long long DP_WAIT_CYCLES = 20000000000ll;  // about 10 s: a peer may be busy on the host for a while

__device__ __forceinline__ void st_flag(unsigned* p, unsigned v) { *reinterpret_cast<volatile unsigned*>(p) = v; }
__device__ __forceinline__ unsigned ld_flag(const unsigned* p) { return *reinterpret_cast<const volatile unsigned*>(p); }

// Thread r < world publishes everything this stream wrote before (local and peer stores of earlier
// kernels) and then sets word `word` of rank r's flag area to `value`.
__global__ void dp_signal_kernel(DpPeers flags, int world, int word, unsigned value)
{
	const int r = threadIdx.x;
	if (r >= world) return;
	__threadfence_system();
	st_flag(reinterpret_cast<unsigned*>(flags.p[r]) + word, value);
}

// Thread t waits until its flag word has reached `value`.  Words: groups x per_group starting at w0
// with a stride of DP_MAX_WORLD words per group, then `extra_n` consecutive words from extra0.
__global__ void dp_wait_kernel(const unsigned* flags, int w0, int groups, int per_group, int extra0, int extra_n,
                               unsigned value, int* status, int code, long long max_cycles)
{
	const int t = threadIdx.x;
	int word = -1;
	if (t < groups * per_group) word = w0 + (t / per_group) * DP_MAX_WORLD + t % per_group;
	else if (t < groups * per_group + extra_n) word = extra0 + (t - groups * per_group);
	// once any wait of this handle has run out, no later one spins again: the exchange is broken and the
	// host reports it at its next status read
	if (word >= 0 && *reinterpret_cast<volatile int*>(status) == 0)
	{
		const long long t0 = clock64();
		while ((int)(ld_flag(flags + word) - value) < 0)
		{
			if (*reinterpret_cast<volatile int*>(status) != 0) break;
			if (clock64() - t0 > max_cycles)
			{
				atomicCAS(status, 0, code);
				break;
			}
			__nanosleep(100);
		}
	}
	__threadfence_system();
}

__global__ void dp_hello_write_kernel(DpPeers slot_heads, DpPeers flags, int world, int self)
{
	const int r = threadIdx.x;
	if (r >= world) return;
	float* dst = reinterpret_cast<float*>(slot_heads.p[r]);
	for (int k = 0; k < 16; ++k) dst[k] = (float)((self + 1) * 1000 + k);
	__threadfence_system();
	st_flag(reinterpret_cast<unsigned*>(flags.p[r]) + DP_WORD_HELLO + self, 1u);
}

__global__ void dp_hello_check_kernel(const float* slots, long long slot_stride, int world, int* status, int code)
{
	const int src = threadIdx.x >> 4, k = threadIdx.x & 15;
	if (src >= world) return;
	const float v = *reinterpret_cast<const volatile float*>(slots + (long long)src * slot_stride + k);
	if (v != (float)((src + 1) * 1000 + k)) atomicCAS(status, 0, code);
}

// Rows [o * band, ...) of the local gradient matrix G [n_out][n_in] -> slot of this rank at owner o.
__global__ void __launch_bounds__(256) dp_push_bands_kernel(const float* __restrict__ G, int n_out, int n_in, int band, DpPeers slot)
{
	const long long total = (long long)n_out * n_in;
	const long long stride = (long long)gridDim.x * blockDim.x;
	const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	if ((n_in & 3) == 0 && (reinterpret_cast<uintptr_t>(G) & 15) == 0)
	{
		const int n4 = n_in >> 2;
		for (long long i = i0; i < (total >> 2); i += stride)
		{
			const int row = (int)(i / n4);
			const int c4 = (int)(i - (long long)row * n4);
			const int o = row / band;
			reinterpret_cast<float4*>(slot.p[o])[(long long)(row - o * band) * n4 + c4] = reinterpret_cast<const float4*>(G)[i];
		}
	}
	else
	{
		for (long long i = i0; i < total; i += stride)
		{
			const int row = (int)(i / n_in);
			const int o = row / band;
			reinterpret_cast<float*>(slot.p[o])[(long long)(row - o * band) * n_in + (i - (long long)row * n_in)] = G[i];
		}
	}
}

// Owner side: g = sum over sources (rank order) of part[src * src_stride + i]; w = w_own[wbase + i] - g * inv_mb,
// written at [wbase + i] of every rank's destination vector W.p[r] (the staging vectors: a rank's own weights stay
// untouched until it commits the layer).  Non-finite results raise word `bad_word` in every rank's flags.
__global__ void __launch_bounds__(256) dp_reduce_update_kernel(const float* __restrict__ part, long long src_stride, int world,
                                                                long long count, float inv_mb, long long wbase,
                                                                const float* __restrict__ w_own, DpPeers W, DpPeers flags,
                                                                int bad_word)
{
	const long long stride = (long long)gridDim.x * blockDim.x;
	const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	const float* Wown = w_own + wbase;
	int bad = 0;
	if (((count | wbase | src_stride) & 3) == 0)
	{
		// two independent 16-byte chains per thread and iteration: the kernel runs on few CTAs beside the
		// backward products, so its bandwidth comes from loads in flight per thread
		const long long n4 = count >> 2;
		for (long long i = i0; i < n4; i += 2 * stride)
		{
			const long long j = i + stride;
			const bool two = j < n4;
			float4 g = reinterpret_cast<const float4*>(part)[i];
			float4 g2 = two ? reinterpret_cast<const float4*>(part)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
			for (int s = 1; s < world; ++s)
			{
				const float4* ps = reinterpret_cast<const float4*>(part + (long long)s * src_stride);
				const float4 h = ps[i];
				const float4 h2 = two ? ps[j] : make_float4(0.f, 0.f, 0.f, 0.f);
				g.x += h.x; g.y += h.y; g.z += h.z; g.w += h.w;
				g2.x += h2.x; g2.y += h2.y; g2.z += h2.z; g2.w += h2.w;
			}
			float4 w = reinterpret_cast<const float4*>(Wown)[i];
			w.x -= g.x * inv_mb; w.y -= g.y * inv_mb; w.z -= g.z * inv_mb; w.w -= g.w * inv_mb;
			if (!(isfinite(w.x) && isfinite(w.y) && isfinite(w.z) && isfinite(w.w))) bad = 1;
			for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(reinterpret_cast<float*>(W.p[r]) + wbase)[i] = w;
			if (two)
			{
				float4 w2 = reinterpret_cast<const float4*>(Wown)[j];
				w2.x -= g2.x * inv_mb; w2.y -= g2.y * inv_mb; w2.z -= g2.z * inv_mb; w2.w -= g2.w * inv_mb;
				if (!(isfinite(w2.x) && isfinite(w2.y) && isfinite(w2.z) && isfinite(w2.w))) bad = 1;
				for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(reinterpret_cast<float*>(W.p[r]) + wbase)[j] = w2;
			}
		}
	}
	else
	{
		for (long long i = i0; i < count; i += stride)
		{
			float g = part[i];
			for (int s = 1; s < world; ++s) g += part[(long long)s * src_stride + i];
			const float w = Wown[i] - g * inv_mb;
			if (!isfinite(w)) bad = 1;
			for (int r = 0; r < world; ++r) (reinterpret_cast<float*>(W.p[r]) + wbase)[i] = w;
		}
	}
	if (bad)
		for (int r = 0; r < world; ++r) st_flag(reinterpret_cast<unsigned*>(flags.p[r]) + bad_word, 1u);
}

// Thread r < world writes this rank's record (bias sums, loss sums) into rank r's arena, then the flag.
__global__ void dp_small_push_kernel(const float* gb, const double* sums2, DpPeers flags, int world, int self, int parity,
                                     unsigned value)
{
	const int r = threadIdx.x;
	if (r >= world) return;
	char* rec = reinterpret_cast<char*>(flags.p[r]) + DP_SMALL_OFFSET + (size_t)(parity * DP_MAX_WORLD + self) * DP_SMALL_BYTES;
	float* f = reinterpret_cast<float*>(rec);
	for (int l = 0; l < GL_MAX_WEIGHT_LAYERS; ++l) f[l] = gb[l];
	double* d = reinterpret_cast<double*>(rec + GL_MAX_WEIGHT_LAYERS * sizeof(float));
	d[0] = sums2[0];
	d[1] = sums2[1];
	__threadfence_system();
	st_flag(reinterpret_cast<unsigned*>(flags.p[r]) + DP_WORD_SFLAG + self, value);
}

// Every rank: sums the records in rank order, applies the bias update, leaves the global sums.
__global__ void dp_finish_kernel(const char* arena, int world, int parity, float* gb_out, double* sums2_out, float* bias,
                                 const float* bscale, int H, int* status_flags)
{
	const int t = threadIdx.x;
	const char* recs = arena + DP_SMALL_OFFSET + (size_t)parity * DP_MAX_WORLD * DP_SMALL_BYTES;
	if (t < GL_MAX_WEIGHT_LAYERS)
	{
		float s = 0.0f;
		for (int r = 0; r < world; ++r) s += reinterpret_cast<const float*>(recs + (size_t)r * DP_SMALL_BYTES)[t];
		gb_out[t] = s;
		if (t >= 1 && t <= H)
		{
			const float b = bias[t] - s * bscale[t];
			if (!isfinite(b)) atomicOr(status_flags, 1);
			bias[t] = b;
		}
	}
	else if (t < GL_MAX_WEIGHT_LAYERS + 2)
	{
		const int k = t - GL_MAX_WEIGHT_LAYERS;
		double s = 0.0;
		for (int r = 0; r < world; ++r)
			s += reinterpret_cast<const double*>(recs + (size_t)r * DP_SMALL_BYTES + GL_MAX_WEIGHT_LAYERS * sizeof(float))[k];
		sums2_out[k] = s;
	}
	else if (t >= 32 && t < 32 + world)
	{
		if (ld_flag(reinterpret_cast<const unsigned*>(arena) + DP_WORD_BAD + (t - 32))) atomicOr(status_flags, 1);
	}
}

}  // namespace

cudaError_t launch_dp_signal(const DpPeers& flags, int world, int word, unsigned value, cudaStream_t s)
{
	dp_signal_kernel<<<1, 32, 0, s>>>(flags, world, word, value);
	return cudaGetLastError();
}

cudaError_t launch_dp_hello_write(const DpPeers& slot_heads, const DpPeers& flags, int world, int self, cudaStream_t s)
{
	dp_hello_write_kernel<<<1, 32, 0, s>>>(slot_heads, flags, world, self);
	return cudaGetLastError();
}

cudaError_t launch_dp_hello_check(const float* slots, long long slot_stride, int world, int* status, int code, cudaStream_t s)
{
	dp_hello_check_kernel<<<1, 16 * DP_MAX_WORLD, 0, s>>>(slots, slot_stride, world, status, code);
	return cudaGetLastError();
}

cudaError_t launch_dp_wait(const void* arena, int w0, int groups, int per_group, int extra0, int extra_n, unsigned value,
                           int* status, int code, cudaStream_t s, long long max_cycles)
{
	const int need = groups * per_group + extra_n;
	if (need < 1 || need > 1024) return cudaErrorInvalidValue;
	dp_wait_kernel<<<1, ((need + 31) / 32) * 32, 0, s>>>(reinterpret_cast<const unsigned*>(arena), w0, groups, per_group, extra0,
	                                                    extra_n, value, status, code, max_cycles > 0 ? max_cycles : DP_WAIT_CYCLES);
	return cudaGetLastError();
}

cudaError_t launch_dp_push_bands(const float* G, int n_out, int n_in, int band, const DpPeers& slot, cudaStream_t s)
{
	const long long total = (long long)n_out * n_in;
	long long blocks = (total / 4 + 255) / 256;
	if (blocks > 148 * 4) blocks = 148 * 4;
	if (blocks < 1) blocks = 1;
	dp_push_bands_kernel<<<(unsigned)blocks, 256, 0, s>>>(G, n_out, n_in, band, slot);
	return cudaGetLastError();
}

cudaError_t launch_dp_reduce_update(const float* part, long long src_stride, int world, long long count, float inv_mb,
                                    long long wbase, const float* w_own, const DpPeers& W, int self, const DpPeers& flags, int blocks,
                                    cudaStream_t s)
{
	if (count < 1) return cudaSuccess;
	long long need = (count / 4 + 255) / 256;
	if (need < 1) need = 1;
	if (need > blocks) need = blocks;
	dp_reduce_update_kernel<<<(unsigned)need, 256, 0, s>>>(part, src_stride, world, count, inv_mb, wbase, w_own, W, flags,
	                                                       DP_WORD_BAD + self);
	return cudaGetLastError();
}

cudaError_t launch_dp_small_push(const float* gb, const double* sums2, const DpPeers& flags, int world, int self, int parity,
                                 unsigned value, cudaStream_t s)
{
	dp_small_push_kernel<<<1, 32, 0, s>>>(gb, sums2, flags, world, self, parity, value);
	return cudaGetLastError();
}

cudaError_t launch_dp_finish(const void* arena, int world, int parity, float* gb_out, double* sums2_out, float* bias,
                             const float* bscale, int H, int* status_flags, cudaStream_t s)
{
	dp_finish_kernel<<<1, 64, 0, s>>>(reinterpret_cast<const char*>(arena), world, parity, gb_out, sums2_out, bias, bscale, H,
	                                  status_flags);
	return cudaGetLastError();
}

}  // namespace glb
