// Batched mode for mid-size networks (weights of a few hundred KB: too large for one SM's shared
// memory, far too small to fill the GPU one layer product at a time): ONE cooperative launch trains
// n_epochs * windows, every SM working on every window, with two grid-wide barriers per window.
//
// Per window (aligned, `mb` rows, weights frozen inside it):
//   phase 1  a CTA takes groups of GF_ROWS samples through the whole network: per layer a
//            [256 outputs] x [32 inputs] weight tile is staged in shared memory (coalesced loads from L2,
//            the weights change every window) and thread = output node accumulates the group's
//            GF_ROWS pre-activations in registers; head (optional softmax, output delta, cost /
//            accuracy / argmax, one warp per sample); then the hidden deltas the same way with
//            thread = input node over [32 outputs] x [256 inputs] tiles.  Activations and deltas of
//            the group go to a window-sized scratch in global memory (it stays in L2).
//   phase 2  the weights are cut into 16 x 32 tiles, one per CTA at a time: thread = 2 weights sums
//            c_j * (lr * d_jo * a_ji + decay terms) over the window's samples in row order
//            (deterministic) from 64-row shared-memory tiles and applies W -= G / len in place; CTA 0
//            adds the CTAs' partial sums (cost, accuracy, scalar-bias deltas) in CTA order.
// Arithmetic = the batched mode of batched.cu / small_fused.cu (reference loop
// Networks/network.cpp:457-668 with aligned windows, frozen weights and a plain error sum); c_j is
// the closed form of the reference's intra-window momentum history (State/node.cpp:278-292).
#include <cooperative_groups.h>

#include "common.cuh"
#include "internal.h"

namespace cg = cooperative_groups;

namespace glb {
namespace {

constexpr int GF_THREADS = 256;
constexpr int GF_ROWS = 8;      // samples a CTA carries through the network together
constexpr int GF_WT = 256 * 33;  // floats of the weight-tile buffer ([256][33] forward, [32][256] backward)
constexpr int GF_TO = 16, GF_TI = 32, GF_TJ = 64;  // phase 2: weight tile 16 outputs x 32 inputs, 64 rows per step
constexpr int GF_PART = 2 + GL_MAX_WEIGHT_LAYERS;  // doubles per CTA: cost, accuracy, bias-delta sums per layer

__global__ void __launch_bounds__(GF_THREADS, 1) grid_fused_kernel(const __grid_constant__ GridFusedArgs a)
{
	extern __shared__ __align__(16) float sm[];
	cg::grid_group grid = cg::this_grid();
	const NetView& n = a.net;
	const int H = n.H;
	const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
	const int n_out = n.sizes[H + 1];
	const int mb = n.mb;

	int node_off[GL_MAX_WEIGHT_LAYERS + 2];
	int tot = 0;
	for (int l = 0; l <= H + 1; ++l)
	{
		node_off[l] = tot;
		tot += n.sizes[l];
	}
	// shared memory: activations [tot][GF_ROWS] | deltas [tot][GF_ROWS] | weight tile | momentum table
	// [H+1][mb+1] | phase-2 tiles | per-row metric scratch
	float* As = sm;
	float* Ds = As + (size_t)tot * GF_ROWS;
	float* Wt = Ds + (size_t)tot * GF_ROWS;
	float* ck = Wt + GF_WT;
	float* Dt = ck + (((size_t)(H + 1) * (mb + 1) + 3) & ~(size_t)3);  // [GF_TJ][GF_TO]
	float* At = Dt + GF_TJ * GF_TO;               // [GF_TJ][GF_TI]
	float* Ct = At + GF_TJ * GF_TI;               // [GF_TJ]
	float* rowm = Ct + GF_TJ;                     // [GF_ROWS][2]: cost, accuracy of the group's rows
	__shared__ double s_part[GF_PART];

	// ck[l][k] = sum_{q<k} m_l^q: the weight of a sample with k samples of its window still to come (itself included)
	for (int e = t; e < (H + 1) * (mb + 1); e += GF_THREADS)
	{
		const int l = e / (mb + 1), k = e - l * (mb + 1);
		const double m = (double)n.mom[l];
		double s = 0.0, pw = 1.0;
		for (int q = 0; q < k; ++q)
		{
			s += pw;
			pw *= m;
			if (pw < 1e-30) break;
		}
		ck[e] = (m == 0.0) ? (k > 0 ? 1.0f : 0.0f) : (float)s;
	}
	__syncthreads();

	const bool classify = n.out_type != GL_OUT_REGRESSION;
	const bool softmax = n.act[H] == GL_ACT_SOFTMAX;
	const float data_size = a.data_size;

	// phase-2 tile list: layer l has ceil(no/16) * ceil(ni/32) tiles
	int tile_off[GL_MAX_WEIGHT_LAYERS + 1];
	int tiles = 0;
	for (int l = 0; l <= H; ++l)
	{
		tile_off[l] = tiles;
		tiles += ((n.sizes[l + 1] + GF_TO - 1) / GF_TO) * ((n.sizes[l] + GF_TI - 1) / GF_TI);
	}
	tile_off[H + 1] = tiles;

	int bad = 0;
	for (int ep = 0; ep < a.n_epochs; ++ep)
	{
		const bool last_epoch = ep == a.n_epochs - 1;
		double ecost = 0.0, eacc = 0.0;  // CTA 0, thread 0
		for (long long r0 = 0; r0 < a.rows; r0 += mb)
		{
			const int len = (int)((a.rows - r0) < mb ? (a.rows - r0) : mb);
			const int groups = (len + GF_ROWS - 1) / GF_ROWS;
			if (t < GF_PART) s_part[t] = 0.0;
			// ================= phase 1: forward, head, deltas, GF_ROWS samples at a time
			for (int gidx = blockIdx.x; gidx < groups; gidx += gridDim.x)
			{
				const int j0 = gidx * GF_ROWS;
				const int valid = (len - j0) < GF_ROWS ? (len - j0) : GF_ROWS;
				__syncthreads();
				// inputs of the group, transposed to [node][row]
				for (int e = t; e < n.sizes[0] * GF_ROWS; e += GF_THREADS)
				{
					const int r = e / n.sizes[0], i = e - r * n.sizes[0];
					As[i * GF_ROWS + r] = (r < valid) ? a.X[(r0 + j0 + r) * n.sizes[0] + i] : 0.0f;
				}
				for (int l = 0; l <= H; ++l)
				{
					const int ni = n.sizes[l], no = n.sizes[l + 1];
					const float* W = n.W[l];
					const float* in = As + (size_t)node_off[l] * GF_ROWS;
					float* out = As + (size_t)node_off[l + 1] * GF_ROWS;
					const float b = (l >= 1) ? __ldcg(n.bias + l) : 0.0f;
					const int act = n.act[l];
					const float par = n.par[l];
					for (int o0 = 0; o0 < no; o0 += GF_THREADS)
					{
						float acc[GF_ROWS];
#pragma unroll
						for (int r = 0; r < GF_ROWS; ++r) acc[r] = 0.0f;
						for (int i0 = 0; i0 < ni; i0 += 32)
						{
							__syncthreads();  // the tile's previous contents (and `in`) are settled
							for (int e = t; e < GF_THREADS * 32; e += GF_THREADS)
							{
								const int oo = e >> 5, ii = e & 31;
								const int o = o0 + oo, i = i0 + ii;
								Wt[oo * 33 + ii] = (o < no && i < ni) ? __ldcg(W + (size_t)o * ni + i) : 0.0f;
							}
							__syncthreads();
							const int lim = (ni - i0) < 32 ? (ni - i0) : 32;
							const float* wrow = Wt + t * 33;
							for (int ii = 0; ii < lim; ++ii)
							{
								const float w = wrow[ii];
								const float4 a0 = *reinterpret_cast<const float4*>(in + (size_t)(i0 + ii) * GF_ROWS);
								const float4 a1 = *reinterpret_cast<const float4*>(in + (size_t)(i0 + ii) * GF_ROWS + 4);
								acc[0] = fmaf(w, a0.x, acc[0]); acc[1] = fmaf(w, a0.y, acc[1]);
								acc[2] = fmaf(w, a0.z, acc[2]); acc[3] = fmaf(w, a0.w, acc[3]);
								acc[4] = fmaf(w, a1.x, acc[4]); acc[5] = fmaf(w, a1.y, acc[5]);
								acc[6] = fmaf(w, a1.z, acc[6]); acc[7] = fmaf(w, a1.w, acc[7]);
							}
						}
						const int o = o0 + t;
						if (o < no)
						{
#pragma unroll
							for (int r = 0; r < GF_ROWS; ++r) out[(size_t)o * GF_ROWS + r] = squash_b(acc[r] + b, act, par);
						}
					}
				}
				__syncthreads();
				// ---- head: warp = sample of the group
				if (warp < GF_ROWS)
				{
					const int r = warp;
					float* p = As + (size_t)node_off[H + 1] * GF_ROWS + r;   // stride GF_ROWS
					float* dout = Ds + (size_t)node_off[H + 1] * GF_ROWS + r;
					float c_acc = 0.0f, a_acc = 0.0f, be = 0.0f, bp = 0.0f;
					int ie = -1, ip = -1;
					if (r < valid)
					{
						const float* y = a.Y + (r0 + j0 + r) * n_out;
						float mx = -INFINITY, inv_den = 1.0f;
						if (softmax)
						{
							for (int o = lane; o < n_out; o += 32) mx = fmaxf(mx, p[(size_t)o * GF_ROWS]);
							mx = warp_max(mx);
							float den = 0.0f;
							for (int o = lane; o < n_out; o += 32) den += expf(p[(size_t)o * GF_ROWS] - mx);
							inv_den = 1.0f / warp_sum(den);
						}
						for (int o = lane; o < n_out; o += 32)
						{
							float pv = p[(size_t)o * GF_ROWS];
							const float e = y[o];
							float cost, d;
							if (softmax)
							{
								pv = expf(pv - mx) * inv_den;
								p[(size_t)o * GF_ROWS] = pv;
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
							dout[(size_t)o * GF_ROWS] = d;
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
						if (lane == 0 && classify && last_epoch && ie >= 0 && ip >= 0) atomicAdd(a.confusion + ie * n_out + ip, 1);
						if (a.last_out && last_epoch && r0 + j0 + r == a.rows - 1)
							for (int o = lane; o < n_out; o += 32) a.last_out[o] = p[(size_t)o * GF_ROWS];
					}
					else
					{
						for (int o = lane; o < n_out; o += 32) dout[(size_t)o * GF_ROWS] = 0.0f;
					}
					if (lane == 0)
					{
						rowm[2 * r] = c_acc;
						rowm[2 * r + 1] = a_acc;
					}
				}
				__syncthreads();
				// ---- hidden deltas: D_l = (D_{l+1} W_l) * act'(A_l), thread = input node
				for (int L = H + 1; L >= 2; --L)
				{
					const int l = L - 1;
					const int ni = n.sizes[l], no = n.sizes[L];
					const float* W = n.W[l];
					const float* dup = Ds + (size_t)node_off[L] * GF_ROWS;
					const int act = n.act[l - 1];
					for (int i0 = 0; i0 < ni; i0 += GF_THREADS)
					{
						float acc[GF_ROWS];
#pragma unroll
						for (int r = 0; r < GF_ROWS; ++r) acc[r] = 0.0f;
						for (int o0 = 0; o0 < no; o0 += 32)
						{
							__syncthreads();
							for (int e = t; e < 32 * GF_THREADS; e += GF_THREADS)
							{
								const int oo = e >> 8, ii = e & 255;
								const int o = o0 + oo, i = i0 + ii;
								Wt[oo * GF_THREADS + ii] = (o < no && i < ni) ? __ldcg(W + (size_t)o * ni + i) : 0.0f;
							}
							__syncthreads();
							const int lim = (no - o0) < 32 ? (no - o0) : 32;
							for (int oo = 0; oo < lim; ++oo)
							{
								const float w = Wt[oo * GF_THREADS + t];
								const float4 d0 = *reinterpret_cast<const float4*>(dup + (size_t)(o0 + oo) * GF_ROWS);
								const float4 d1 = *reinterpret_cast<const float4*>(dup + (size_t)(o0 + oo) * GF_ROWS + 4);
								acc[0] = fmaf(w, d0.x, acc[0]); acc[1] = fmaf(w, d0.y, acc[1]);
								acc[2] = fmaf(w, d0.z, acc[2]); acc[3] = fmaf(w, d0.w, acc[3]);
								acc[4] = fmaf(w, d1.x, acc[4]); acc[5] = fmaf(w, d1.y, acc[5]);
								acc[6] = fmaf(w, d1.z, acc[6]); acc[7] = fmaf(w, d1.w, acc[7]);
							}
						}
						const int i = i0 + t;
						if (i < ni)
						{
#pragma unroll
							for (int r = 0; r < GF_ROWS; ++r)
							{
								const float av = As[(size_t)(node_off[l] + i) * GF_ROWS + r];
								Ds[(size_t)(node_off[l] + i) * GF_ROWS + r] = (r < valid) ? acc[r] * act_der_b(av, act, 0.01f) : 0.0f;
							}
						}
					}
					__syncthreads();
				}
				// ---- the group's activations and deltas to the window scratch ([row][node]); partial sums
				for (int r = 0; r < valid; ++r)
				{
					float* ga = a.actbuf + (size_t)(j0 + r) * tot;
					float* gd = a.delbuf + (size_t)(j0 + r) * tot;
					for (int e = t; e < tot; e += GF_THREADS)
					{
						ga[e] = As[(size_t)e * GF_ROWS + r];
						if (e >= n.sizes[0]) gd[e] = Ds[(size_t)e * GF_ROWS + r];
					}
				}
				if (warp >= 1 && warp <= H)
				{
					// scalar-bias delta of hidden layer `warp`: sum of the deltas of the layer above, this group's rows
					const int l = warp, no = n.sizes[l + 1];
					double s = 0.0;
					for (int e = lane; e < no * GF_ROWS; e += 32) s += (double)Ds[(size_t)node_off[l + 1] * GF_ROWS + e];
					s = warp_sum_d(s);
					if (lane == 0) s_part[2 + l] += s;
				}
				if (t == 0)
				{
					for (int r = 0; r < valid; ++r)
					{
						s_part[0] += (double)rowm[2 * r];
						s_part[1] += (double)rowm[2 * r + 1];
					}
				}
			}
			__syncthreads();
			if (t < GF_PART) a.part[(size_t)blockIdx.x * GF_PART + t] = s_part[t];
			grid.sync();

			// ================= phase 2: gradient + update per weight tile; CTA 0 also the scalars
			const float inv_len = 1.0f / (float)len;
			for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x)
			{
				int l = 0;
				while (tile >= tile_off[l + 1]) ++l;
				const int ni = n.sizes[l], no = n.sizes[l + 1];
				const int tiles_i = (ni + GF_TI - 1) / GF_TI;
				const int tl = tile - tile_off[l];
				const int o0 = (tl / tiles_i) * GF_TO, i0 = (tl % tiles_i) * GF_TI;
				const float lr = n.lr[l], w1 = n.wd1[l] * lr, w2 = n.wd2[l] * lr;
				const float* ckl = ck + (size_t)l * (mb + 1);
				const int oo = t >> 4, i2 = (t & 15) * 2;  // this thread's output row and its two input columns
				float g0 = 0.0f, g1 = 0.0f;
				for (int jb = 0; jb < len; jb += GF_TJ)
				{
					const int jn = (len - jb) < GF_TJ ? (len - jb) : GF_TJ;
					__syncthreads();
					for (int e = t; e < GF_TJ * GF_TO; e += GF_THREADS)
					{
						const int jj = e / GF_TO, x = e - jj * GF_TO;
						Dt[e] = (jj < jn && o0 + x < no) ? __ldcg(a.delbuf + (size_t)(jb + jj) * tot + node_off[l + 1] + o0 + x) : 0.0f;
					}
					for (int e = t; e < GF_TJ * GF_TI; e += GF_THREADS)
					{
						const int jj = e / GF_TI, x = e - jj * GF_TI;
						At[e] = (jj < jn && i0 + x < ni) ? __ldcg(a.actbuf + (size_t)(jb + jj) * tot + node_off[l] + i0 + x) : 0.0f;
					}
					if (t < GF_TJ) Ct[t] = (t < jn) ? ckl[len - (jb + t)] : 0.0f;
					__syncthreads();
					for (int jj = 0; jj < jn; ++jj)
					{
						const float c = Ct[jj];
						const float dv = lr * Dt[jj * GF_TO + oo];
						const float2 av = *reinterpret_cast<const float2*>(At + jj * GF_TI + i2);
						g0 = fmaf(c, fmaf(dv, av.x, fmaf(w1, fabsf(av.x), w2 * av.x)), g0);
						g1 = fmaf(c, fmaf(dv, av.y, fmaf(w1, fabsf(av.y), w2 * av.y)), g1);
					}
				}
				const int o = o0 + oo;
				if (o < no)
				{
					float* wp = n.W[l] + (size_t)o * ni + i0 + i2;
					if (i0 + i2 < ni)
					{
						const float w = __ldcg(wp) - g0 * inv_len;
						if (!isfinite(w)) bad = 1;
						wp[0] = w;
					}
					if (i0 + i2 + 1 < ni)
					{
						const float w = __ldcg(wp + 1) - g1 * inv_len;
						if (!isfinite(w)) bad = 1;
						wp[1] = w;
					}
				}
			}
			if (blockIdx.x == 0)
			{
				if (warp >= 1 && warp <= H)
				{
					const int l = warp;
					double s = 0.0;
					for (int b = lane; b < (int)gridDim.x; b += 32) s += __ldcg(a.part + (size_t)b * GF_PART + 2 + l);
					s = warp_sum_d(s) * (double)n.lr[l];
					if (lane == 0)
					{
						const float nb = __ldcg(n.bias + l) -
						                 ((a.bias_rule == GL_BIAS_REFERENCE) ? (float)(s * (double)n.sizes[l]) : (float)(s / (double)len));
						if (!isfinite(nb)) bad = 1;
						n.bias[l] = nb;
					}
				}
				if (t == 0)
				{
					for (int b = 0; b < (int)gridDim.x; ++b)
					{
						ecost += __ldcg(a.part + (size_t)b * GF_PART);
						eacc += __ldcg(a.part + (size_t)b * GF_PART + 1);
					}
				}
			}
			grid.sync();
		}
		if (blockIdx.x == 0 && t == 0)
		{
			a.epoch_sums[2 * ep] = ecost;
			a.epoch_sums[2 * ep + 1] = eacc;
		}
	}
	if (bad) atomicOr(a.flags, 1);
}

}  // namespace

size_t grid_fused_smem_bytes(const NetView& n)
{
	int tot = 0;
	for (int l = 0; l <= n.H + 1; ++l) tot += n.sizes[l];
	size_t f = 2 * (size_t)tot * GF_ROWS + GF_WT + (((size_t)(n.H + 1) * (n.mb + 1) + 3) & ~(size_t)3) + GF_TJ * GF_TO + GF_TJ * GF_TI + GF_TJ + 2 * GF_ROWS;
	return f * sizeof(float) + 64;
}

int grid_fused_total_nodes(const NetView& n)
{
	int tot = 0;
	for (int l = 0; l <= n.H + 1; ++l) tot += n.sizes[l];
	return tot;
}

cudaError_t launch_grid_fused(const GridFusedArgs& a, int* grid_out, cudaStream_t s)
{
	const size_t bytes = grid_fused_smem_bytes(a.net);
	cudaError_t e = cudaFuncSetAttribute(grid_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
	if (e != cudaSuccess) return e;
	int dev = 0, sms = 0, per_sm = 0;
	cudaGetDevice(&dev);
	e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
	if (e != cudaSuccess) return e;
	e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, grid_fused_kernel, GF_THREADS, bytes);
	if (e != cudaSuccess) return e;
	if (per_sm < 1) return cudaErrorInvalidConfiguration;
	int grid = sms;  // one CTA per SM; a.part is sized for grid_fused_max_grid() CTAs
	if (grid > a.part_ctas) grid = a.part_ctas;
	if (grid_out) *grid_out = grid;
	GridFusedArgs copy = a;
	void* params[] = {&copy};
	return cudaLaunchCooperativeKernel((void*)grid_fused_kernel, dim3((unsigned)grid), dim3(GF_THREADS), params, bytes, s);
}

}  // namespace glb
