// Batched-mode kernels that are not the tensor-core GEMM: the exact-fp32 FFMA tile GEMM with the
// fused layer epilogues, the output-layer head (delta + metrics + confusion counts, optional
// softmax), the scalar-bias reduction, the weight-decay column term and the fused update.
//
// One window step of batched mode is, per weight layer l (reference arithmetic of
// Networks/network.cpp:457-668 with aligned windows, frozen weights and a plain error sum):
//   forward   A_{l+1} = squash(A_l W_l^T + b_l)                       (EPI_FORWARD)
//   head      D_{H+1} = cost'(Y, A_{H+1})  or  softmax(Z) - Y;  metrics; confusion counts
//   errprop   D_l     = (D_{l+1} W_l) * act'(A_l)                     (EPI_ERRPROP)
//   gradient  G_l     = lr_l * D_{l+1}^T diag(c) A_l + decay          (EPI_GRAD)
//   update    W -= G / mb ;  b_l -= scale_l * lr_l * sum(D_{l+1})
#include "common.cuh"
#include "internal.h"

namespace glb {

// ---------------------------------------------------------------------------------------------
// FFMA tile GEMM, generic strides: C[m][n] = sum_k A(m,k) * B(n,k).  64x64 tile, 16-deep k-step,
// 256 threads, 4x4 outputs per thread, operands staged k-major in shared memory.
constexpr int FB_M = 64, FB_N = 64, FB_K = 16, FB_T = 256;

template <int EPI>
__global__ void __launch_bounds__(FB_T) gemm_ffma_kernel(const GemmArgs g)
{
	__shared__ __align__(16) float As[FB_K][FB_M + 4];
	__shared__ __align__(16) float Bs[FB_K][FB_N + 4];
	const int tid = threadIdx.x;
	const int tx = tid % 16, ty = tid / 16;
	const int m0 = blockIdx.y * FB_M, n0 = blockIdx.x * FB_N;
	const bool a_kcontig = (g.a_sk == 1), b_kcontig = (g.b_sk == 1);

	float acc[4][4];
#pragma unroll
	for (int i = 0; i < 4; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
	const float bias = (EPI == EPI_FORWARD && g.bias_ptr) ? *g.bias_ptr : 0.0f;

	for (int k0 = 0; k0 < g.K; k0 += FB_K)
	{
#pragma unroll
		for (int j = 0; j < (FB_M * FB_K) / FB_T; ++j)
		{
			const int idx = tid + j * FB_T;
			int m, k;
			if (a_kcontig) { k = idx % FB_K; m = idx / FB_K; }
			else { m = idx % FB_M; k = idx / FB_M; }
			const int gm = m0 + m, gk = k0 + k;
			float v = 0.0f;
			if (gm < g.M && gk < g.K)
			{
				v = g.A[(long long)gm * g.a_sm + (long long)gk * g.a_sk];
				if (g.kscale) v *= g.kscale[gk];
			}
			As[k][m] = v;
		}
#pragma unroll
		for (int j = 0; j < (FB_N * FB_K) / FB_T; ++j)
		{
			const int idx = tid + j * FB_T;
			int nn, k;
			if (b_kcontig) { k = idx % FB_K; nn = idx / FB_K; }
			else { nn = idx % FB_N; k = idx / FB_N; }
			const int gn = n0 + nn, gk = k0 + k;
			float v = 0.0f;
			if (gn < g.N && gk < g.K) v = g.B[(long long)gn * g.b_sn + (long long)gk * g.b_sk];
			Bs[k][nn] = v;
		}
		__syncthreads();
#pragma unroll
		for (int k = 0; k < FB_K; ++k)
		{
			const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
			const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
			const float a4[4] = {av.x, av.y, av.z, av.w};
			const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
			for (int i = 0; i < 4; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
		}
		__syncthreads();
	}

#pragma unroll
	for (int i = 0; i < 4; ++i)
	{
		const int gm = m0 + ty * 4 + i;
		if (gm >= g.M) continue;
#pragma unroll
		for (int j = 0; j < 4; ++j)
		{
			const int gn = n0 + tx * 4 + j;
			if (gn >= g.N) continue;
			float v = acc[i][j];
			if (EPI == EPI_FORWARD) v = squash_b(v + bias, g.act, g.par);
			else if (EPI == EPI_ERRPROP) v = v * act_der_b(g.aux[(long long)gm * g.ld_aux + gn], g.act, g.par);
			else if (EPI == EPI_GRAD) v = g.alpha * v + (g.colterm ? g.colterm[gn] : 0.0f);
			g.C[(long long)gm * g.ldc + gn] = v;
		}
	}
}

// ---------------------------------------------------------------------------------------------
// Skinny products (N <= 16 output nodes, e.g. a 10-class or single-node output layer): the whole B
// operand sits in shared memory, one warp per row of A, lanes stride over k with 16-byte loads, the
// N partial sums are combined by warp shuffles.  Bound by reading A once from HBM.
constexpr int SK_NMAX = 16;

// NN = the layer's width as a compile-time constant: the accumulators are registers and the inner loops carry
// no per-column predicates (the first version's 16-way predicated body stalled on instruction fetch).
template <int EPI, int NN>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const GemmArgs g)
{
	extern __shared__ __align__(16) float sW[];  // [N][K]
	const int K = g.K;
	constexpr int N = NN;
	for (int e = threadIdx.x; e < N * K; e += blockDim.x) sW[e] = g.B[(long long)(e / K) * g.b_sn + (e % K)];
	__syncthreads();
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
	const float bias = (EPI == EPI_FORWARD && g.bias_ptr) ? *g.bias_ptr : 0.0f;
	const int K4 = K >> 2;
	// a warp takes SK_ROWS consecutive rows at a time: every weight chunk read from shared memory serves
	// all of them, and the rows' independent 16-byte loads keep HBM busy
	constexpr int SK_ROWS = 4;
	const long long groups = (g.M + SK_ROWS - 1) / SK_ROWS;
	for (long long gi = (long long)blockIdx.x * wpb + warp; gi < groups; gi += (long long)gridDim.x * wpb)
	{
		const long long m0 = gi * SK_ROWS;
		const float4* arow[SK_ROWS];
#pragma unroll
		for (int r = 0; r < SK_ROWS; ++r)
		{
			const long long m = (m0 + r < g.M) ? m0 + r : g.M - 1;  // the tail repeats the last row (not stored)
			arow[r] = reinterpret_cast<const float4*>(g.A + m * g.a_sm);
		}
		float acc[SK_ROWS][NN];
#pragma unroll
		for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
			for (int n = 0; n < NN; ++n) acc[r][n] = 0.0f;
		// Two 16-byte chunks per row and lane, rotated: while one set of four loads is consumed the other set is in
		// flight, so the warp always has loads outstanding.  (Measured the same 2.7 TB/s as loading both sets and
		// then computing on both: with 16 warps per SM the kernel is bound by the latency of the bytes it can keep
		// in flight -- 123 registers, 80 KB of weights in shared memory per block -- not by instruction issue.)
		auto consume = [&](const float4 (&v)[SK_ROWS], int kq) {
#pragma unroll
			for (int n = 0; n < NN; ++n)
				if (n < N)
				{
					const float4 w = reinterpret_cast<const float4*>(sW + n * K)[kq];
#pragma unroll
					for (int r = 0; r < SK_ROWS; ++r)
						acc[r][n] = fmaf(v[r].x, w.x, fmaf(v[r].y, w.y, fmaf(v[r].z, w.z, fmaf(v[r].w, w.w, acc[r][n]))));
				}
		};
		float4 a[SK_ROWS], b[SK_ROWS];
		if (lane < K4)
		{
#pragma unroll
			for (int r = 0; r < SK_ROWS; ++r) a[r] = arow[r][lane];
		}
		for (int k4 = lane; k4 < K4; k4 += 64)
		{
			const int k4b = k4 + 32, k4n = k4 + 64;
			const bool two = k4b < K4;
			if (two)
			{
#pragma unroll
				for (int r = 0; r < SK_ROWS; ++r) b[r] = arow[r][k4b];
			}
			consume(a, k4);
			if (k4n < K4)
			{
#pragma unroll
				for (int r = 0; r < SK_ROWS; ++r) a[r] = arow[r][k4n];
			}
			if (two) consume(b, k4b);
		}
#pragma unroll
		for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
			for (int n = 0; n < NN; ++n)
				if (n < N) acc[r][n] = warp_sum(acc[r][n]);
		if (lane == 0)
		{
#pragma unroll
			for (int r = 0; r < SK_ROWS; ++r)
			{
				if (m0 + r >= g.M) break;
#pragma unroll
				for (int n = 0; n < NN; ++n)
					if (n < N)
					{
						float v = acc[r][n];
						if (EPI == EPI_FORWARD) v = squash_b(v + bias, g.act, g.par);
						g.C[(m0 + r) * g.ldc + n] = v;
					}
			}
		}
	}
}

static bool skinny_ok(const GemmArgs& g)
{
	return (g.epi == EPI_FORWARD || g.epi == EPI_NONE) && g.N <= SK_NMAX && g.a_sk == 1 && g.b_sk == 1 && !g.kscale &&
	       g.K % 4 == 0 && g.a_sm % 4 == 0 && (((uintptr_t)g.A) & 15) == 0 && (size_t)g.N * g.K * 4 <= 160 * 1024 && g.M >= 64;
}

cudaError_t launch_gemm_ffma(const GemmArgs& g, cudaStream_t s)
{
	if (skinny_ok(g))
	{
		const size_t bytes = (size_t)g.N * g.K * sizeof(float);
		long long blocks = (g.M + 31) / 32;  // 8 warps x 4 rows per CTA pass
		if (blocks > 148 * 4) blocks = 148 * 4;
		if (blocks < 1) blocks = 1;
		cudaError_t e = cudaErrorInvalidValue;
#define GL_SKINNY_CASE(NV)                                                                                                       \
	case NV:                                                                                                                     \
		if (g.epi == EPI_FORWARD)                                                                                                \
		{                                                                                                                        \
			e = cudaFuncSetAttribute(gemm_skinny_kernel<EPI_FORWARD, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); \
			if (e == cudaSuccess) gemm_skinny_kernel<EPI_FORWARD, NV><<<(unsigned)blocks, 256, bytes, s>>>(g);                    \
		}                                                                                                                        \
		else                                                                                                                     \
		{                                                                                                                        \
			e = cudaFuncSetAttribute(gemm_skinny_kernel<EPI_NONE, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);  \
			if (e == cudaSuccess) gemm_skinny_kernel<EPI_NONE, NV><<<(unsigned)blocks, 256, bytes, s>>>(g);                       \
		}                                                                                                                        \
		break;
		switch (g.N)
		{
			GL_SKINNY_CASE(1) GL_SKINNY_CASE(2) GL_SKINNY_CASE(3) GL_SKINNY_CASE(4) GL_SKINNY_CASE(5) GL_SKINNY_CASE(6)
			GL_SKINNY_CASE(7) GL_SKINNY_CASE(8) GL_SKINNY_CASE(9) GL_SKINNY_CASE(10) GL_SKINNY_CASE(11) GL_SKINNY_CASE(12)
			GL_SKINNY_CASE(13) GL_SKINNY_CASE(14) GL_SKINNY_CASE(15) GL_SKINNY_CASE(16)
		default: break;
		}
#undef GL_SKINNY_CASE
		if (e != cudaSuccess) return e;
		return cudaGetLastError();
	}
	dim3 grid((g.N + FB_N - 1) / FB_N, (g.M + FB_M - 1) / FB_M);
	switch (g.epi)
	{
	case EPI_FORWARD: gemm_ffma_kernel<EPI_FORWARD><<<grid, FB_T, 0, s>>>(g); break;
	case EPI_ERRPROP: gemm_ffma_kernel<EPI_ERRPROP><<<grid, FB_T, 0, s>>>(g); break;
	case EPI_GRAD: gemm_ffma_kernel<EPI_GRAD><<<grid, FB_T, 0, s>>>(g); break;
	default: gemm_ffma_kernel<EPI_NONE><<<grid, FB_T, 0, s>>>(g); break;
	}
	return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Output-layer head: one warp per row.  Metrics follow network.cpp:519-547 (cost / (rows*n_out),
// |p-e| accuracy) and CMatrix::addResult (GMath/cmatrix.cpp:57-98: strict > from 0, first maximum
// wins); the output delta is the bare cost derivative (network.cpp:599-612: the output activation's
// derivative is dropped), or p - y behind the softmax extension.
__global__ void __launch_bounds__(256) head_kernel(const HeadArgs h)
{
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	const int wpb = blockDim.x >> 5;
	double cost_acc = 0.0, acc_acc = 0.0;
	for (long long r = (long long)blockIdx.x * wpb + warp; r < h.rows; r += (long long)gridDim.x * wpb)
	{
		float* p = h.P + r * h.n;
		const float* y = h.Y + r * h.n;
		float mx = -INFINITY, inv_den = 1.0f;
		if (h.softmax)
		{
			// (unrolled: the row's loads are independent, and one warp per row leaves few warps to hide their latency)
#pragma unroll 8
			for (int o = lane; o < h.n; o += 32) mx = fmaxf(mx, p[o]);
			mx = warp_max(mx);
			float den = 0.0f;
#pragma unroll 8
			for (int o = lane; o < h.n; o += 32) den += expf(p[o] - mx);
			den = warp_sum(den);
			inv_den = 1.0f / den;
		}
		// running first-maximum argmax of expected and predicted (value, index) per lane
		float be = 0.0f, bp = 0.0f;
		int ie = -1, ip = -1;
#pragma unroll 4
		for (int o = lane; o < h.n; o += 32)
		{
			float pv = p[o];
			const float e = y[o];
			float cost;
			if (h.softmax)
			{
				pv = expf(pv - mx) * inv_den;
				p[o] = pv;
				cost = (e != 0.0f) ? -(e * logf(pv)) / h.data_size : 0.0f;
				if (h.D) h.D[r * h.n + o] = pv - e;
				if (h.D_lo) h.D_lo[r * h.n + o] = tf32_lo(pv - e);
			}
			else
			{
				if (h.out_type == GL_OUT_REGRESSION) { const float t = e - pv; cost = t * t / h.data_size; }
				else if (h.out_type == GL_OUT_CLASSIFICATION)
					cost = -((e * logf(pv)) + ((1.0f - e) * logf(1.0f - pv))) / h.data_size;
				else cost = logf(e / pv) / h.data_size;
				if (h.D)
				{
					float d;
					if (h.out_type == GL_OUT_REGRESSION) d = 2.0f * (pv - e);
					else if (h.out_type == GL_OUT_CLASSIFICATION) d = (pv - e) / ((1.0f - pv) * pv);
					else d = -(e / pv);
					h.D[r * h.n + o] = d;
					if (h.D_lo) h.D_lo[r * h.n + o] = tf32_lo(d);
				}
			}
			cost_acc += (double)cost;
			float pe = fabsf(pv - e);
			pe = fminf(pe, 1.0f);
			acc_acc += (double)fmaxf((1.0f - pe) * 100.0f, 0.0f);
			if (e > be) { be = e; ie = o; }
			if (pv > bp) { bp = pv; ip = o; }
		}
		// warp argmax: larger value wins, ties go to the smaller index (first maximum wins)
#pragma unroll
		for (int off = 16; off > 0; off >>= 1)
		{
			const float oe = __shfl_xor_sync(0xffffffffu, be, off);
			const int oie = __shfl_xor_sync(0xffffffffu, ie, off);
			if (oie >= 0 && (ie < 0 || oe > be || (oe == be && oie < ie))) { be = oe; ie = oie; }
			const float op = __shfl_xor_sync(0xffffffffu, bp, off);
			const int oip = __shfl_xor_sync(0xffffffffu, ip, off);
			if (oip >= 0 && (ip < 0 || op > bp || (op == bp && oip < ip))) { bp = op; ip = oip; }
		}
		if (lane == 0)
		{
			if (h.argmax) h.argmax[r] = ip;
			if (h.confusion && h.out_type != GL_OUT_REGRESSION && ie >= 0 && ip >= 0)
				atomicAdd(&h.confusion[ie * h.n + ip], 1);
		}
	}
	cost_acc = warp_sum_d(cost_acc);
	acc_acc = warp_sum_d(acc_acc);
	__shared__ double s_c[8], s_a[8];
	if (lane == 0) { s_c[warp] = cost_acc; s_a[warp] = acc_acc; }
	__syncthreads();
	if (threadIdx.x == 0 && h.sums2)
	{
		double c = 0.0, a = 0.0;
		for (int w = 0; w < wpb; ++w) { c += s_c[w]; a += s_a[w]; }
		atomicAdd(&h.sums2[0], c);
		atomicAdd(&h.sums2[1], a);
	}
}

cudaError_t launch_head(const HeadArgs& h, cudaStream_t s)
{
	const int wpb = 8;
	long long blocks = (h.rows + wpb - 1) / wpb;
	if (blocks > 148 * 8) blocks = 148 * 8;
	if (blocks < 1) blocks = 1;
	head_kernel<<<(unsigned)blocks, wpb * 32, 0, s>>>(h);
	return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// *out += alpha * sum(D[0..count)), reproducibly: every block sums a fixed set of elements in double and leaves its
// partial in `part`; the block that arrives last (a ticket counter) adds the partials in a fixed order and is the only
// one to touch *out.  (A float atomic per block would make the scalar bias depend on the order the blocks finish in.)
// part: gridDim.x doubles; ticket: one word, zero before the launch and zero again after it.
__global__ void __launch_bounds__(256) sum_scaled_kernel(const float* __restrict__ D, long long count, float alpha, float* out,
                                                         double* part, unsigned* ticket)
{
	double acc = 0.0;
	const long long stride = (long long)gridDim.x * blockDim.x;
	const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	if ((reinterpret_cast<uintptr_t>(D) & 15) == 0)
	{
		const long long n4 = count >> 2;
		const float4* D4 = reinterpret_cast<const float4*>(D);
#pragma unroll 4
		for (long long i = i0; i < n4; i += stride)
		{
			const float4 v = D4[i];
			acc += ((double)v.x + (double)v.y) + ((double)v.z + (double)v.w);
		}
		for (long long i = (n4 << 2) + i0; i < count; i += stride) acc += (double)D[i];
	}
	else
		for (long long i = i0; i < count; i += stride) acc += (double)D[i];
	acc = warp_sum_d(acc);
	__shared__ double sw[8];
	__shared__ bool last;
	if ((threadIdx.x & 31) == 0) sw[threadIdx.x >> 5] = acc;
	__syncthreads();
	if (threadIdx.x == 0)
	{
		double t = 0.0;
		for (int w = 0; w < 8; ++w) t += sw[w];
		part[blockIdx.x] = t;
		__threadfence();
		last = atomicAdd(ticket, 1u) == gridDim.x - 1;
	}
	__syncthreads();
	if (last && threadIdx.x < 32)
	{
		__threadfence();
		double t = 0.0;
		for (unsigned b = threadIdx.x; b < gridDim.x; b += 32) t += __ldcg(part + b);
		t = warp_sum_d(t);
		if (threadIdx.x == 0)
		{
			*out += (float)(t * (double)alpha);
			*ticket = 0u;
		}
	}
}

cudaError_t launch_sum_scaled(const float* D, long long count, float alpha, float* out, double* part, unsigned* ticket, cudaStream_t s)
{
	long long blocks = (count + 256 * 16 - 1) / (256 * 16);
	if (blocks > SUM_SCALED_MAX_BLOCKS) blocks = SUM_SCALED_MAX_BLOCKS;
	if (blocks < 1) blocks = 1;
	sum_scaled_kernel<<<(unsigned)blocks, 256, 0, s>>>(D, count, alpha, out, part, ticket);
	return cudaGetLastError();
}

// colterm[i] = lr * sum_j c_j * (wd1*|A[j][i]| + wd2*A[j][i])   (decay terms of Node::getDelta,
// State/node.cpp:284-289: they use the INPUT activation, not the weight)
__global__ void decay_colterm_kernel(const float* A, int rows, int n, const float* c, float lr, float wd1, float wd2,
                                     float* colterm)
{
	const int i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	double s = 0.0;
	for (int j = 0; j < rows; ++j)
	{
		const float a = A[(long long)j * n + i];
		const float cj = c ? c[j] : 1.0f;
		s += (double)cj * ((double)wd1 * fabs((double)a) + (double)wd2 * (double)a);
	}
	colterm[i] = (float)((double)lr * s);
}

cudaError_t launch_decay_colterm(const float* A, int rows, int n, const float* c, float lr, float wd1, float wd2,
                                 float* colterm, cudaStream_t s)
{
	decay_colterm_kernel<<<(n + 127) / 128, 128, 0, s>>>(A, rows, n, c, lr, wd1, wd2, colterm);
	return cudaGetLastError();
}

// W -= G * inv_mb (Node::applyDeltas, State/node.cpp:294-307: the window sum is always divided by
// the minibatch size); scalar biases; non-finite flag.
__global__ void __launch_bounds__(256) update_kernel(float* W, float* W_lo, const float* G, long long count, float inv_mb,
                                                      float* bias, const float* gb, const float* bscale, int H, int* flags)
{
	int bad = 0;
	const long long stride = (long long)gridDim.x * blockDim.x;
	const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	const long long n4 = count / 4;
	float4* W4 = reinterpret_cast<float4*>(W);
	const float4* G4 = reinterpret_cast<const float4*>(G);
	for (long long i = i0; i < n4; i += stride)
	{
		float4 w = W4[i];
		const float4 g = G4[i];
		w.x -= g.x * inv_mb; w.y -= g.y * inv_mb; w.z -= g.z * inv_mb; w.w -= g.w * inv_mb;
		if (!(isfinite(w.x) && isfinite(w.y) && isfinite(w.z) && isfinite(w.w))) bad = 1;
		W4[i] = w;
		if (W_lo) reinterpret_cast<float4*>(W_lo)[i] = make_float4(tf32_lo(w.x), tf32_lo(w.y), tf32_lo(w.z), tf32_lo(w.w));
	}
	for (long long i = n4 * 4 + i0; i < count; i += stride)
	{
		const float w = W[i] - G[i] * inv_mb;
		if (!isfinite(w)) bad = 1;
		W[i] = w;
		if (W_lo) W_lo[i] = tf32_lo(w);
	}
	if (blockIdx.x == 0 && threadIdx.x >= 1 && threadIdx.x <= H)
	{
		const float b = bias[threadIdx.x] - gb[threadIdx.x] * bscale[threadIdx.x];
		if (!isfinite(b)) bad = 1;
		bias[threadIdx.x] = b;
	}
	if (bad) atomicOr(flags, 1);
}

cudaError_t launch_update(float* W, float* W_lo, const float* G, long long count, float inv_mb, float* bias, const float* gb,
                          const float* bscale, int H, int* flags, cudaStream_t s)
{
	long long blocks = (count / 4 + 255) / 256;
	if (blocks > 148 * 8) blocks = 148 * 8;
	if (blocks < 1) blocks = 1;
	update_kernel<<<(unsigned)blocks, 256, 0, s>>>(W, W_lo, G, count, inv_mb, bias, gb, bscale, H, flags);
	return cudaGetLastError();
}

}  // namespace glb
