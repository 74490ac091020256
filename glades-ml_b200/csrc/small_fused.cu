// Batched mode for small networks: one persistent CTA trains n_epochs * windows in a single launch
// with ALL weights resident in shared memory.
//
// Per window (aligned, `mb` rows, weights frozen inside it):
//   phase 1  one warp per sample: forward (lane = output node, inputs broadcast from shared memory,
//            weight rows padded to an odd pitch so the 32 lanes hit 32 banks), optional softmax and the
//            output delta with warp-shuffle reductions for the row's cost / accuracy / argmax, then
//            the deltas of the hidden layers (lane = input node, plain error sum);
//   phase 2  one thread per weight: G = sum_j c_j * (lr*d_jo*a_ji + decay terms) over the window's
//            samples in row order (deterministic), W -= G / len; one warp per hidden layer sums its
//            scalar-bias delta; one thread adds the per-sample metric values in row order.
// Two block-wide barriers per window, no global-memory traffic except the window's input rows.
// Arithmetic = the batched mode of batched.cu (reference loop Networks/network.cpp:457-668 with
// aligned windows, frozen weights and a plain error sum); c_j is the closed form of the reference's
// intra-window momentum history (State/node.cpp:278-292).
#include "common.cuh"
#include "internal.h"

namespace glb {

__device__ __forceinline__ int sf_pitch(int ni) { return (ni & 1) ? ni : ni + 1; }

__global__ void __launch_bounds__(1024, 1) small_fused_kernel(const __grid_constant__ SmallFusedArgs a)
{
	extern __shared__ __align__(16) float sm[];
	const NetView& n = a.net;
	const int H = n.H;
	const int T = blockDim.x, t = threadIdx.x;
	const int lane = t & 31, warp = t >> 5, nwarps = T >> 5;
	const int n_out = n.sizes[H + 1];
	const int mb = n.mb;

	int node_off[GL_MAX_WEIGHT_LAYERS + 2];
	int tot = 0;
	for (int l = 0; l <= H + 1; ++l)
	{
		node_off[l] = tot;
		tot += n.sizes[l];
	}
	// shared memory: padded weights | activations [mb][tot] | deltas [mb][tot] | momentum weights
	// [H+1][mb] | biases | per-sample cost, accuracy, argmax pair
	float* Wp[GL_MAX_WEIGHT_LAYERS];
	float* cur = sm;
	for (int l = 0; l <= H; ++l)
	{
		Wp[l] = cur;
		cur += n.sizes[l + 1] * sf_pitch(n.sizes[l]);
	}
	float* A = cur;
	cur += (size_t)mb * tot;
	float* D = cur;
	cur += (size_t)mb * tot;
	float* cw = cur;
	cur += (H + 1) * mb;
	float* sbias = cur;
	cur += GL_MAX_WEIGHT_LAYERS;
	float* scost = cur;
	cur += mb;
	float* sacc = cur;
	cur += mb;
	int* sarg = reinterpret_cast<int*>(cur);  // [mb][2]

	for (int l = 0; l <= H; ++l)
	{
		const int ni = n.sizes[l], no = n.sizes[l + 1], ld = sf_pitch(ni);
		for (int e = t; e < ni * no; e += T) Wp[l][(e / ni) * ld + (e % ni)] = n.W[l][e];
	}
	if (t < GL_MAX_WEIGHT_LAYERS) sbias[t] = n.bias[t];
	__syncthreads();

	const float data_size = (float)(a.rows * (long long)n_out);
	const bool classify = n.out_type != GL_OUT_REGRESSION;
	const bool softmax = n.act[H] == GL_ACT_SOFTMAX;
	int cur_len = -1;

	for (int ep = 0; ep < a.n_epochs; ++ep)
	{
		const bool last_epoch = ep == a.n_epochs - 1;
		double ecost = 0.0, eacc = 0.0;  // thread 0 only
		if (classify)
			for (int e = t; e < n_out * n_out; e += T) a.confusion[e] = 0;
		for (long long r0 = 0; r0 < a.rows; r0 += mb)
		{
			const int len = (int)((a.rows - r0) < mb ? (a.rows - r0) : mb);
			if (len != cur_len)
			{
				// c_j = sum_{t=0}^{len-1-j} m^t
				for (int e = t; e < (H + 1) * len; e += T)
				{
					const int l = e / len, j = e - l * len;
					const double m = (double)n.mom[l];
					double s = 0.0, pw = 1.0;
					for (int q = 0; q < len - j; ++q)
					{
						s += pw;
						pw *= m;
						if (pw < 1e-30) break;
					}
					cw[l * mb + j] = (m == 0.0) ? 1.0f : (float)s;
				}
				cur_len = len;
			}
			// ---------------- phase 1: one warp per sample
			for (int j = warp; j < len; j += nwarps)
			{
				float* aj = A + (size_t)j * tot;
				float* dj = D + (size_t)j * tot;
				const float* xr = a.X + (r0 + j) * n.sizes[0];
				for (int i = lane; i < n.sizes[0]; i += 32) aj[i] = xr[i];
				__syncwarp();
				for (int l = 0; l <= H; ++l)
				{
					const int ni = n.sizes[l], no = n.sizes[l + 1], ld = sf_pitch(ni);
					const float* in = aj + node_off[l];
					float* out = aj + node_off[l + 1];
					const float b = (l >= 1) ? sbias[l] : 0.0f;
					for (int o = lane; o < no; o += 32)
					{
						const float* w = Wp[l] + o * ld;
						float z = 0.0f;
						for (int i = 0; i < ni; ++i) z = fmaf(w[i], in[i], z);
						out[o] = squash_b(z + b, n.act[l], n.par[l]);
					}
					__syncwarp();
				}
				// head: optional softmax, output delta, metrics of this row
				float* p = aj + node_off[H + 1];
				float* dout = dj + node_off[H + 1];
				const float* y = a.Y + (r0 + j) * n_out;
				float mx = -INFINITY, inv_den = 1.0f;
				if (softmax)
				{
					for (int o = lane; o < n_out; o += 32) mx = fmaxf(mx, p[o]);
					mx = warp_max(mx);
					float den = 0.0f;
					for (int o = lane; o < n_out; o += 32) den += expf(p[o] - mx);
					inv_den = 1.0f / warp_sum(den);
				}
				float c_acc = 0.0f, a_acc = 0.0f, be = 0.0f, bp = 0.0f;
				int ie = -1, ip = -1;
				for (int o = lane; o < n_out; o += 32)
				{
					float pv = p[o];
					const float e = y[o];
					float cost, d;
					if (softmax)
					{
						pv = expf(pv - mx) * inv_den;
						p[o] = pv;
						cost = (e != 0.0f) ? -(e * logf(pv)) / data_size : 0.0f;
						d = pv - e;
					}
					else if (n.out_type == GL_OUT_REGRESSION)
					{
						const float tt = e - pv;
						cost = tt * tt / data_size;
						d = 2.0f * (pv - e);
					}
					else if (n.out_type == GL_OUT_CLASSIFICATION)
					{
						cost = -((e * logf(pv)) + ((1.0f - e) * logf(1.0f - pv))) / data_size;
						d = (pv - e) / ((1.0f - pv) * pv);
					}
					else
					{
						cost = logf(e / pv) / data_size;
						d = -(e / pv);
					}
					dout[o] = d;
					c_acc += cost;
					a_acc += fmaxf((1.0f - fminf(fabsf(pv - e), 1.0f)) * 100.0f, 0.0f);
					if (e > be) { be = e; ie = o; }
					if (pv > bp) { bp = pv; ip = o; }
				}
				c_acc = warp_sum(c_acc);
				a_acc = warp_sum(a_acc);
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
					scost[j] = c_acc;
					sacc[j] = a_acc;
					sarg[2 * j] = ie;
					sarg[2 * j + 1] = ip;
				}
				if (a.last_out && last_epoch && r0 + j == a.rows - 1)
					for (int o = lane; o < n_out; o += 32) a.last_out[o] = p[o];
				__syncwarp();
				// deltas of the hidden layers: D_l = (D_{l+1} W_l) * act'(A_l)
				for (int L = H + 1; L >= 2; --L)
				{
					const int l = L - 1;
					const int ni = n.sizes[l], no = n.sizes[L], ld = sf_pitch(ni);
					const float* dup = dj + node_off[L];
					for (int i = lane; i < ni; i += 32)
					{
						float s = 0.0f;
						for (int o = 0; o < no; ++o) s = fmaf(dup[o], Wp[l][o * ld + i], s);
						dj[node_off[l] + i] = s * act_der_b(aj[node_off[l] + i], n.act[l - 1], 0.01f);
					}
					__syncwarp();
				}
			}
			__syncthreads();
			// ---------------- phase 2: gradient + update, one thread per weight
			const float inv_len = 1.0f / (float)len;
			for (int l = 0; l <= H; ++l)
			{
				const int ni = n.sizes[l], no = n.sizes[l + 1], ld = sf_pitch(ni);
				const float lr = n.lr[l], w1 = n.wd1[l] * lr, w2 = n.wd2[l] * lr;
				const float* c = cw + l * mb;
				for (int e = t; e < ni * no; e += T)
				{
					const int o = e / ni, i = e - o * ni;
					float g = 0.0f;
					for (int j = 0; j < len; ++j)
					{
						const float av = A[(size_t)j * tot + node_off[l] + i];
						const float dv = D[(size_t)j * tot + node_off[l + 1] + o];
						g = fmaf(c[j], fmaf(lr * dv, av, fmaf(w1, fabsf(av), w2 * av)), g);
					}
					Wp[l][o * ld + i] -= g * inv_len;
				}
			}
			if (warp >= 1 && warp <= H)
			{
				// scalar bias of hidden layer `warp`: lr * sum of the deltas of the layer above
				const int l = warp, no = n.sizes[l + 1];
				double s = 0.0;
				for (int e = lane; e < len * no; e += 32) s += (double)D[(size_t)(e / no) * tot + node_off[l + 1] + (e % no)];
				s = warp_sum_d(s) * (double)n.lr[l];
				if (lane == 0)
					sbias[l] -= (a.bias_rule == GL_BIAS_REFERENCE) ? (float)(s * (double)n.sizes[l]) : (float)(s / (double)len);
			}
			if (t == 0)
			{
				for (int j = 0; j < len; ++j)
				{
					ecost += (double)scost[j];
					eacc += (double)sacc[j];
					if (classify && sarg[2 * j] >= 0 && sarg[2 * j + 1] >= 0) a.confusion[sarg[2 * j] * n_out + sarg[2 * j + 1]] += 1;
				}
			}
			__syncthreads();
		}
		if (t == 0)
		{
			a.epoch_sums[2 * ep] = ecost;
			a.epoch_sums[2 * ep + 1] = eacc;
		}
	}
	// write the weights back and look for non-finite values
	int bad = 0;
	for (int l = 0; l <= H; ++l)
	{
		const int ni = n.sizes[l], no = n.sizes[l + 1], ld = sf_pitch(ni);
		for (int e = t; e < ni * no; e += T)
		{
			const float w = Wp[l][(e / ni) * ld + (e % ni)];
			n.W[l][e] = w;
			if (!isfinite(w)) bad = 1;
		}
	}
	if (t >= 1 && t <= H)
	{
		n.bias[t] = sbias[t];
		if (!isfinite(sbias[t])) bad = 1;
	}
	if (bad) atomicOr(a.flags, 1);
}

size_t small_fused_smem_bytes(const NetView& n)
{
	size_t f = 0;
	int tot = 0;
	for (int l = 0; l <= n.H + 1; ++l) tot += n.sizes[l];
	for (int l = 0; l <= n.H; ++l) f += (size_t)n.sizes[l + 1] * ((n.sizes[l] & 1) ? n.sizes[l] : n.sizes[l] + 1);
	f += 2 * (size_t)n.mb * tot + (size_t)(n.H + 1) * n.mb + GL_MAX_WEIGHT_LAYERS + 4 * (size_t)n.mb;
	return f * sizeof(float);
}

cudaError_t launch_small_fused(const SmallFusedArgs& a, cudaStream_t s)
{
	const size_t bytes = small_fused_smem_bytes(a.net);
	cudaError_t e = cudaFuncSetAttribute(small_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
	if (e != cudaSuccess) return e;
	int warps = a.net.mb < 32 ? a.net.mb : 32;
	if (warps < a.net.H + 1) warps = a.net.H + 1;  // phase 2 uses one warp per hidden layer
	if (warps < 4) warps = 4;
	if (warps > 32) warps = 32;
	small_fused_kernel<<<1, warps * 32, bytes, s>>>(a);
	return cudaGetLastError();
}

}  // namespace glb
