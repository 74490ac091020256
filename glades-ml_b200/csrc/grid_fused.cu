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

#include "tc_device.cuh"

namespace cg = cooperative_groups;

namespace glb {
using namespace tc;
namespace {

constexpr int GF_THREADS = 256;
constexpr int GF_ROWS = 8;      // samples a CTA carries through the network together
constexpr int GF_WT = 256 * 33;  // floats of the weight-tile buffer ([256][33] forward, [32][256] backward)
constexpr int GF_TO = 16, GF_TJ = 64;  // phase 2: weight tile 16 outputs x 32 inputs, 64 rows per stage
constexpr int GF_NS = 3;                // stages of the weight-tile ring (bulk tensor copies, 32 KB each)
constexpr int GF_STAGE = 32768;
constexpr int GF_SEQ_MAX = 512;         // weight tiles one sample group walks through, at most, on the ring path
static_assert(GF_WT * 4 <= GF_NS * GF_STAGE, "the register-path tile buffer lives inside the ring");
constexpr int GF_PART = 2 + GL_MAX_WEIGHT_LAYERS;  // doubles per CTA: cost, accuracy, bias-delta sums per layer

// ---- phase 2, asynchronous fill ------------------------------------------------------------------
// One 16 x 32 tile of layer l's weights.  The window's deltas and activations reach shared memory through a ring
// of GF_P2_STAGES 64-row stages filled by 4-byte cp.async copies (zero-filled outside the window or the layer):
// three stages are in flight while one is consumed, so a step no longer waits one L2 round trip (the former
// global -> registers -> shared memory fill with one step of prefetch did: 16 steps x 1.2 us per tile).
// Lane = 4 outputs x 4 inputs (four output groups x eight input groups: 16 multiply-adds per two 16-byte loads),
// warp w takes rows 8w..8w+7 of every stage; the eight warps' partial sums are added in warp order and the update
// is applied in place.  Deterministic; the sum is no longer one chain in row order.
constexpr int GF_P2_TI = 32;
constexpr int GF_P2_STAGES = 6;   // tile path: five stages in flight while one is consumed
constexpr int GF_P2N_STAGES = 4;  // narrow-layer path (its stages are larger)
constexpr int GF_P2_STAGE_FLOATS = GF_TJ * GF_TO + GF_TJ * GF_P2_TI + GF_TJ;          // deltas, activations, momentum weights
constexpr int GF_P2_FLOATS = GF_P2_STAGES * GF_P2_STAGE_FLOATS + 8 * GF_TO * GF_P2_TI;  // + the warps' partial sums
static_assert(GF_P2_FLOATS * 4 <= GF_NS * GF_STAGE, "the phase-2 stages live inside the weight-tile ring");
static_assert((GF_P2_STAGE_FLOATS * 4) % 16 == 0, "stages keep the 16-byte alignment of the vector loads");

__device__ __forceinline__ void gf_grad_tile_async(const GridFusedArgs& a, int l, int o0, int i0, int len, int pitch, int off_in,
                                                   int off_out, float* stages, const float* ckl, float inv_len, int& bad)
{
	const NetView& n = a.net;
	const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
	const int ni = n.sizes[l], no = n.sizes[l + 1];
	const float lr = n.lr[l], w1 = n.wd1[l] * lr, w2 = n.wd2[l] * lr;
	const bool decay = w1 != 0.0f || w2 != 0.0f;
	const int og = lane >> 3, ig = lane & 7;
	float* red = stages + GF_P2_STAGES * GF_P2_STAGE_FLOATS;
	const uint32_t st_addr = smem_u32(stages);
	float g[4][4];
#pragma unroll
	for (int x = 0; x < 4; ++x)
#pragma unroll
		for (int y = 0; y < 4; ++y) g[x][y] = 0.0f;
	const int steps = (len + GF_TJ - 1) / GF_TJ;
	// one 16-byte copy of deltas and two of activations per thread and stage (the scratch rows and the layers'
	// first columns are 16-byte aligned), one 4-byte copy of a momentum weight for the first 64 threads
	const int d_jj = t >> 2, d_x = (t & 3) << 2;
	auto issue = [&](int s) {
		if (s < steps)
		{
			const int jb = s * GF_TJ;
			const int jn = (len - jb) < GF_TJ ? (len - jb) : GF_TJ;
			const uint32_t base = st_addr + (uint32_t)((s % GF_P2_STAGES) * GF_P2_STAGE_FLOATS * 4);
			{
				const int left = (d_jj < jn) ? no - (o0 + d_x) : 0;
				cp_async16(base + (uint32_t)t * 16, left > 0 ? a.delbuf + (size_t)(jb + d_jj) * pitch + off_out + o0 + d_x : a.delbuf, left);
			}
#pragma unroll
			for (int k = 0; k < 2; ++k)
			{
				const int e = t + k * GF_THREADS, jj = e >> 3, x = (e & 7) << 2;
				const int left = (jj < jn) ? ni - (i0 + x) : 0;
				cp_async16(base + (uint32_t)(GF_TJ * GF_TO * 4) + (uint32_t)e * 16,
				           left > 0 ? a.actbuf + (size_t)(jb + jj) * pitch + off_in + i0 + x : a.actbuf, left);
			}
			if (t < GF_TJ)
			{
				const bool ok = t < jn;
				cp_async4(base + (uint32_t)(GF_TJ * GF_TO + GF_TJ * GF_P2_TI + t) * 4, ok ? ckl + (len - (jb + t)) : ckl, ok);
			}
		}
		cp_async_commit();  // one group per step, empty ones included: the wait counts groups
	};
	__syncthreads();  // the previous work item no longer reads the stages
#pragma unroll
	for (int s = 0; s < GF_P2_STAGES - 1; ++s) issue(s);
	for (int s = 0; s < steps; ++s)
	{
		cp_async_wait<GF_P2_STAGES - 2>();  // this thread's copies of stage s have landed
		__syncthreads();                    // everybody's have; and stage s - 1 is no longer read
		issue(s + GF_P2_STAGES - 1);        // refills the stage consumed in the previous step
		const float* Dt = stages + (s % GF_P2_STAGES) * GF_P2_STAGE_FLOATS;
		const float* At = Dt + GF_TJ * GF_TO;
		const float* Ct = At + GF_TJ * GF_P2_TI;
#pragma unroll 4
		for (int q = 0; q < 8; ++q)
		{
			const int jj = warp * 8 + q;  // rows beyond the window hold zeros
			const float4 dv = *reinterpret_cast<const float4*>(Dt + jj * GF_TO + og * 4);
			const float4 av = *reinterpret_cast<const float4*>(At + jj * GF_P2_TI + ig * 4);
			const float c = Ct[jj];
			const float d4[4] = {dv.x, dv.y, dv.z, dv.w};
			const float a4[4] = {av.x, av.y, av.z, av.w};
			if (!decay)
			{
				// c_j * lr * d_jo first (rounded as the staged fill used to round it), then one multiply-add per weight
#pragma unroll
				for (int x = 0; x < 4; ++x)
				{
					const float dx = d4[x] * lr * c;
#pragma unroll
					for (int y = 0; y < 4; ++y) g[x][y] = fmaf(dx, a4[y], g[x][y]);
				}
			}
			else
			{
				float dec[4];
#pragma unroll
				for (int y = 0; y < 4; ++y) dec[y] = fmaf(w1, fabsf(a4[y]), w2 * a4[y]);
#pragma unroll
				for (int x = 0; x < 4; ++x)
#pragma unroll
					for (int y = 0; y < 4; ++y) g[x][y] = fmaf(c, fmaf(lr * d4[x], a4[y], dec[y]), g[x][y]);
			}
		}
	}
	cp_async_wait<0>();
	// the warps' partial sums: red[warp][output 0..15][input 0..31] (not part of the stages)
#pragma unroll
	for (int x = 0; x < 4; ++x)
		*reinterpret_cast<float4*>(red + warp * (GF_TO * GF_P2_TI) + (og * 4 + x) * GF_P2_TI + ig * 4) = make_float4(g[x][0], g[x][1], g[x][2], g[x][3]);
	__syncthreads();
#pragma unroll
	for (int k = 0; k < GF_TO * GF_P2_TI / GF_THREADS; ++k)
	{
		const int e = t + k * GF_THREADS;
		const int o = o0 + e / GF_P2_TI, i = i0 + (e & (GF_P2_TI - 1));
		float sum = red[e];
#pragma unroll
		for (int w = 1; w < 8; ++w) sum += red[w * (GF_TO * GF_P2_TI) + e];
		if (o < no && i < ni)
		{
			float* wp = n.W[l] + (size_t)o * ni + i;
			const float wv = __ldcg(wp) - sum * inv_len;
			if (!isfinite(wv)) bad = 1;
			*wp = wv;
		}
	}
}


// Phase 2 for a layer with at most GF_NARROW output nodes (the usual regression head): one work item per GF_NCOLS
// input columns, the same ring of 64-row stages (activations [64][64], deltas [64][4], momentum weights [64]);
// thread = one column and the rows 16p..16p+15 of every stage (p = thread / 64); the four parts are added in fixed
// order through shared memory.
constexpr int GF_NARROW = 4;
constexpr int GF_NCOLS = 64;
constexpr int GF_P2N_STAGE_FLOATS = GF_TJ * GF_NCOLS + GF_TJ * GF_NARROW + GF_TJ;
constexpr int GF_P2N_FLOATS = GF_P2N_STAGES * GF_P2N_STAGE_FLOATS + GF_THREADS * GF_NARROW;
static_assert(GF_P2N_FLOATS * 4 <= GF_NS * GF_STAGE, "the narrow-layer stages live inside the weight-tile ring");
constexpr int GF_P2_MAX_FLOATS = GF_P2N_FLOATS > GF_P2_FLOATS ? GF_P2N_FLOATS : GF_P2_FLOATS;
__device__ __forceinline__ void gf_grad_narrow(const GridFusedArgs& a, int l, int i0, int len, int pitch, int off_in, int off_out,
                                               const float* ckl, float inv_len, float* stages, int& bad)
{
	const NetView& n = a.net;
	const int t = threadIdx.x;
	const int ni = n.sizes[l], no = n.sizes[l + 1];
	const int col = t & (GF_NCOLS - 1), part = t / GF_NCOLS;  // 4 parts
	const int i = i0 + col;
	const float lr = n.lr[l], w1 = n.wd1[l] * lr, w2 = n.wd2[l] * lr;
	float* red = stages + GF_P2N_STAGES * GF_P2N_STAGE_FLOATS;
	const uint32_t st_addr = smem_u32(stages);
	float g[GF_NARROW];
#pragma unroll
	for (int o = 0; o < GF_NARROW; ++o) g[o] = 0.0f;
	const int steps = (len + GF_TJ - 1) / GF_TJ;
	auto issue = [&](int s) {
		if (s < steps)
		{
			const int jb = s * GF_TJ;
			const int jn = (len - jb) < GF_TJ ? (len - jb) : GF_TJ;
			const uint32_t base = st_addr + (uint32_t)((s % GF_P2N_STAGES) * GF_P2N_STAGE_FLOATS * 4);
#pragma unroll
			for (int k = 0; k < 4; ++k)
			{
				const int e = t + k * GF_THREADS, jj = e >> 4, x = (e & 15) << 2;
				const int left = (jj < jn) ? ni - (i0 + x) : 0;
				cp_async16(base + (uint32_t)e * 16, left > 0 ? a.actbuf + (size_t)(jb + jj) * pitch + off_in + i0 + x : a.actbuf, left);
			}
			if (t < GF_TJ)
			{
				const int left = (t < jn) ? no : 0;
				cp_async16(base + (uint32_t)(GF_TJ * GF_NCOLS * 4) + (uint32_t)t * 16, left > 0 ? a.delbuf + (size_t)(jb + t) * pitch + off_out : a.delbuf,
				           left);
			}
			else if (t < 2 * GF_TJ)
			{
				const int r = t - GF_TJ;
				const bool ok = r < jn;
				cp_async4(base + (uint32_t)(GF_TJ * GF_NCOLS + GF_TJ * GF_NARROW + r) * 4, ok ? ckl + (len - (jb + r)) : ckl, ok);
			}
		}
		cp_async_commit();
	};
	__syncthreads();  // the previous work item no longer reads the stages
#pragma unroll
	for (int s = 0; s < GF_P2N_STAGES - 1; ++s) issue(s);
	for (int s = 0; s < steps; ++s)
	{
		cp_async_wait<GF_P2N_STAGES - 2>();
		__syncthreads();
		issue(s + GF_P2N_STAGES - 1);
		const float* At = stages + (s % GF_P2N_STAGES) * GF_P2N_STAGE_FLOATS;
		const float* Dt = At + GF_TJ * GF_NCOLS;
		const float* Ct = Dt + GF_TJ * GF_NARROW;
#pragma unroll 4
		for (int q = 0; q < GF_TJ / 4; ++q)
		{
			const int jj = part * (GF_TJ / 4) + q;  // rows beyond the window hold zeros (c = 0)
			const float av = At[jj * GF_NCOLS + col];
			const float4 dv = *reinterpret_cast<const float4*>(Dt + jj * GF_NARROW);
			const float c = Ct[jj];
			const float dec = fmaf(w1, fabsf(av), w2 * av);
			const float d4[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
			for (int o = 0; o < GF_NARROW; ++o) g[o] = fmaf(c, fmaf(lr * d4[o], av, dec), g[o]);
		}
	}
	cp_async_wait<0>();
#pragma unroll
	for (int o = 0; o < GF_NARROW; ++o) red[(part * GF_NCOLS + col) * GF_NARROW + o] = g[o];
	__syncthreads();
	if (part == 0 && i < ni)
	{
#pragma unroll
		for (int o = 0; o < GF_NARROW; ++o)
			if (o < no)
			{
				float sum = red[col * GF_NARROW + o];
				for (int p2 = 1; p2 < GF_THREADS / GF_NCOLS; ++p2) sum += red[(p2 * GF_NCOLS + col) * GF_NARROW + o];
				float* wp = n.W[l] + (size_t)o * ni + i;
				const float w = __ldcg(wp) - sum * inv_len;
				if (!isfinite(w)) bad = 1;
				*wp = w;
			}
	}
}

// The window scratch: one row per sample, layer l's nodes from column soff[l] on; every layer starts at a multiple
// of 4 columns and the pitch is one too, so that rows and layers are 16-byte aligned for the copies of phase 2.
__host__ __device__ inline int gf_scratch_layout(const NetView& n, int* soff)
{
	int c = 0;
	for (int l = 0; l <= n.H + 1; ++l)
	{
		soff[l] = c;
		c += (n.sizes[l] + 3) & ~3;
	}
	return c;
}

// USE_TMA: the weight tiles arrive through the ring of bulk tensor copies (a.tma != NULL), else through registers.
// Two instantiations rather than a run-time flag: each carries one tile path only, which halves the body the
// instruction cache has to hold (instruction fetch showed among the kernel's stalls).
template <bool USE_TMA>
__global__ void __launch_bounds__(GF_THREADS, 1) grid_fused_kernel(const __grid_constant__ GridFusedArgs a)
{
	extern __shared__ __align__(16) float sm[];
	cg::grid_group grid = cg::this_grid();
	const NetView& n = a.net;
	const int H = n.H;
	const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
	const int n_out = n.sizes[H + 1];
	const int mb = n.mb;

	// layer l's nodes start at node_off[l], a multiple of 4, in shared memory and in the window scratch alike
	// (tot = the scratch's pitch); the few padding nodes are carried along and never read as values
	int node_off[GL_MAX_WEIGHT_LAYERS + 2];
	const int tot = gf_scratch_layout(n, node_off);
	// shared memory: activations [tot][GF_ROWS] | deltas [tot][GF_ROWS] | per-row metric scratch | tile list |
	// weight-tile ring (phase 2 reuses it for its stages)
	float* As = sm;
	float* Ds = As + (size_t)tot * GF_ROWS;
	float* rowm = Ds + (size_t)tot * GF_ROWS;  // [GF_ROWS][2]: cost, accuracy of the group's rows
	int* seq = reinterpret_cast<int*>(rowm + 2 * GF_ROWS);  // [GF_SEQ_MAX][3]: tensor map, x, y of a group's weight tiles
	// weight tiles: a ring of GF_NS stages filled by bulk tensor copies (1024-byte aligned for the
	// 128-byte swizzle), or -- where the weights' layout does not allow tensor maps -- one tile buffer
	// filled through registers
	// A narrow output layer (at most GF_NARROW nodes: the usual regression head) does not go through weight tiles --
	// a [256 outputs] x [32 inputs] tile would carry one useful row and leave 255 threads idle for n_in / 32
	// steps.  Its few weight rows are copied to shared memory once per window (wn); the forward product splits the
	// inputs over the threads and adds the partial sums in a fixed order, the hidden deltas read wn directly.
	const bool narrow_head = n.sizes[H + 1] <= GF_NARROW && H >= 1;
	float* wn = reinterpret_cast<float*>(seq + 3 * GF_SEQ_MAX);          // [n_out][n_H]
	float* nred = wn + (narrow_head ? ((n.sizes[H + 1] * n.sizes[H] + 3) & ~3) : 0);  // [8 warps][GF_ROWS][GF_NARROW]
	uint8_t* ring_gen;
	{
		uint8_t* after = reinterpret_cast<uint8_t*>(nred + (narrow_head ? 8 * GF_ROWS * GF_NARROW : 0));
		const uint32_t au = smem_u32(after);
		ring_gen = after + (((au + 1023u) & ~1023u) - au);
	}
	const uint32_t ring = smem_u32(ring_gen);
	float* Wt = reinterpret_cast<float*>(ring_gen);
	__shared__ double s_part[GF_PART];
	__shared__ uint64_t gf_bars[GF_NS];
	__shared__ int gf_abort;
	constexpr bool use_tma = USE_TMA;
	const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(a.tma);
	int nsteps = 0;  // weight tiles per sample group
	if (use_tma)
	{
		if (t == 0)
		{
			for (int sidx = 0; sidx < GF_NS; ++sidx) mbar_init(smem_u32(&gf_bars[sidx]), 1);
			gf_abort = 0;
			asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
		}
		// the tile order of one group: forward layer by layer (output chunk, then input tile), then the
		// hidden deltas from the top (input chunk, then output tile)
		for (int l = 0; l <= H - (narrow_head ? 1 : 0); ++l)
			for (int o0 = 0; o0 < n.sizes[l + 1]; o0 += GF_THREADS)
				for (int i0 = 0; i0 < n.sizes[l]; i0 += 32, ++nsteps)
					if (t == 0) { seq[3 * nsteps] = 2 * l; seq[3 * nsteps + 1] = i0; seq[3 * nsteps + 2] = o0; }
		for (int L = H + 1 - (narrow_head ? 1 : 0); L >= 2; --L)
			for (int i0 = 0; i0 < n.sizes[L - 1]; i0 += GF_THREADS)
				for (int o0 = 0; o0 < n.sizes[L]; o0 += 32, ++nsteps)
					if (t == 0) { seq[3 * nsteps] = 2 * (L - 1) + 1; seq[3 * nsteps + 1] = i0; seq[3 * nsteps + 2] = o0; }
	}
	// optional phase timing (diagnostics): CTA 0, thread 0 adds up the nanoseconds of
	// [phase 1, barrier, phase 2, barrier] in a.timing[0..3]
	const bool timed = a.timing != nullptr && blockIdx.x == 0 && t == 0;
	unsigned long long tm[16] = {}, t_a = 0, t_b = 0, t_c = 0, t_d = 0;
	// tm[9..14]: inside phase 1 -- waits for weight tiles, the barriers that release them, forward, head, deltas, tail
	auto now = []() {
		unsigned long long v;
		asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
		return v;
	};

	unsigned cs = 0;                         // ring steps consumed so far (every thread)
	unsigned ps = 0, p_base = 0, p_end = 0;  // thread 0: steps issued, first and end step of the current window
	bool dead = false;                       // a bounded wait ran out: stop waiting, finish the launch
	auto issue = [&]() {
		const int* e = seq + 3 * ((ps - p_base) % (unsigned)nsteps);
		const uint32_t bar = smem_u32(&gf_bars[ps % GF_NS]);
		mbar_expect_tx(bar, GF_STAGE);
		tma_load_2d(ring + (ps % GF_NS) * GF_STAGE, maps + e[0], bar, e[1], e[2]);
		++ps;
	};
	auto acquire = [&]() -> const float* {
		const unsigned sidx = cs % GF_NS;
		unsigned long long t0 = 0;
		if (timed) t0 = now();
		if (!dead && !mbar_wait(smem_u32(&gf_bars[sidx]), (cs / GF_NS) & 1u, &gf_abort, a.flags + 1, 30)) dead = true;
		if (timed) tm[9] += now() - t0;
		return reinterpret_cast<const float*>(ring_gen + sidx * GF_STAGE);
	};
	auto release = [&]() {
		unsigned long long t0 = 0;
		if (timed) t0 = now();
		__syncthreads();  // every thread is done with the stage
		if (timed) tm[10] += now() - t0;
		++cs;
		if (t == 0 && ps < p_end) issue();
	};

	// a.ck[l][k] = sum_{q<k} m_l^q: the weight of a sample with k samples of its window still to come (itself
	// included); made once on the host, [H+1][mb+1], read by phase 2 straight from global memory

	const bool classify = n.out_type != GL_OUT_REGRESSION;
	const bool softmax = n.act[H] == GL_ACT_SOFTMAX;
	const float data_size = a.data_size;

	// phase-2 tile list: layer l has ceil(no/16) * ceil(ni/32) tiles
	const int tile_i = GF_P2_TI;
	int tile_off[GL_MAX_WEIGHT_LAYERS + 1];
	int tiles = 0;
	for (int l = 0; l <= H; ++l)
	{
		tile_off[l] = tiles;
		tiles += (n.sizes[l + 1] <= GF_NARROW) ? (n.sizes[l] + GF_NCOLS - 1) / GF_NCOLS
		                                       : ((n.sizes[l + 1] + GF_TO - 1) / GF_TO) * ((n.sizes[l] + tile_i - 1) / tile_i);
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
			if (use_tma && t == 0)
			{
				// this window's tiles: nsteps per group of this CTA; never run ahead into the next window,
				// whose weights do not exist yet
				const int mine = (groups > (int)blockIdx.x) ? (groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
				p_base = ps;
				p_end = ps + (unsigned)(mine * nsteps);
				for (int k = 0; k < GF_NS && ps < p_end; ++k) issue();
			}
			if (narrow_head)
				for (int e = t; e < n.sizes[H + 1] * n.sizes[H]; e += GF_THREADS) wn[e] = __ldcg(n.W[H] + e);  // visible after the group's first barrier
			if (timed) t_a = now();
			// ================= phase 1: forward, head, deltas, GF_ROWS samples at a time
			for (int gidx = blockIdx.x; gidx < groups; gidx += gridDim.x)
			{
				const int j0 = gidx * GF_ROWS;
				const int valid = (len - j0) < GF_ROWS ? (len - j0) : GF_ROWS;
				if (timed) t_c = now();
				__syncthreads();
				// inputs of the group, transposed to [node][row]
				for (int e = t; e < n.sizes[0] * GF_ROWS; e += GF_THREADS)
				{
					const int r = e / n.sizes[0], i = e - r * n.sizes[0];
					As[i * GF_ROWS + r] = (r < valid) ? a.X[(r0 + j0 + r) * n.sizes[0] + i] : 0.0f;
				}
				if (use_tma) __syncthreads();
				for (int l = 0; l <= H; ++l)
				{
					const int ni = n.sizes[l], no = n.sizes[l + 1];
					const float* W = n.W[l];
					const float* in = As + (size_t)node_off[l] * GF_ROWS;
					float* out = As + (size_t)node_off[l + 1] * GF_ROWS;
					const float b = (l >= 1) ? __ldcg(n.bias + l) : 0.0f;
					const int act = n.act[l];
					const float par = n.par[l];
					if (narrow_head && l == H)
					{
						// thread = (row r, input class q): inputs i = q, q + 32, ...; the four classes of a warp are added
						// by shuffles, the eight warps' sums through shared memory in warp order
						const int r = t & 7, q = t >> 3;
						if (!use_tma) __syncthreads();  // the register path ends a layer without a barrier: the inputs must be complete
						float s4[GF_NARROW];
#pragma unroll
						for (int o = 0; o < GF_NARROW; ++o) s4[o] = 0.0f;
						for (int i = q; i < ni; i += 32)
						{
							const float av = in[(size_t)i * GF_ROWS + r];
#pragma unroll
							for (int o = 0; o < GF_NARROW; ++o)
								if (o < no) s4[o] = fmaf(wn[o * ni + i], av, s4[o]);
						}
#pragma unroll
						for (int o = 0; o < GF_NARROW; ++o)
						{
							s4[o] += __shfl_xor_sync(0xffffffffu, s4[o], 8);
							s4[o] += __shfl_xor_sync(0xffffffffu, s4[o], 16);
						}
						if (lane < GF_ROWS)
						{
#pragma unroll
							for (int o = 0; o < GF_NARROW; ++o) nred[(warp * GF_ROWS + lane) * GF_NARROW + o] = s4[o];
						}
						__syncthreads();
						if (t < GF_ROWS * no)
						{
							const int rr = t % GF_ROWS, o = t / GF_ROWS;
							float z = nred[rr * GF_NARROW + o];
							for (int w = 1; w < 8; ++w) z += nred[(w * GF_ROWS + rr) * GF_NARROW + o];
							out[(size_t)o * GF_ROWS + rr] = squash_b(z + b, act, par);
						}
						__syncthreads();
						continue;
					}
					for (int o0 = 0; o0 < no; o0 += GF_THREADS)
					{
						float acc[GF_ROWS];
#pragma unroll
						for (int r = 0; r < GF_ROWS; ++r) acc[r] = 0.0f;
						if (use_tma)
						{
							const bool computes = o0 + t < no;
							for (int i0 = 0; i0 < ni; i0 += 32)
							{
								// tile rows = output nodes o0.., 32 inputs each, 16-byte chunks XOR-swizzled by the row
								const float* stg = acquire();
								unsigned long long tq = 0;
								if (timed) tq = now();
								if (computes)
								{
									const float* inb = in + (size_t)i0 * GF_ROWS;
									const float* wrow = stg + t * 32;
									const int sw = t & 7;
									auto stepw = [&](int ii, float w) {
										const float4 a0 = *reinterpret_cast<const float4*>(inb + ii * GF_ROWS);
										const float4 a1 = *reinterpret_cast<const float4*>(inb + ii * GF_ROWS + 4);
										acc[0] = fmaf(w, a0.x, acc[0]); acc[1] = fmaf(w, a0.y, acc[1]);
										acc[2] = fmaf(w, a0.z, acc[2]); acc[3] = fmaf(w, a0.w, acc[3]);
										acc[4] = fmaf(w, a1.x, acc[4]); acc[5] = fmaf(w, a1.y, acc[5]);
										acc[6] = fmaf(w, a1.z, acc[6]); acc[7] = fmaf(w, a1.w, acc[7]);
									};
									if (ni - i0 >= 32)
									{
										// the activations of four inputs (eight 16-byte broadcast loads) are fetched before the
										// 32 multiply-adds that use them, and the loop is unrolled so that the next group's loads
										// issue under the current group's arithmetic: with two warps per scheduler the step is
										// bound by shared-memory latency, not by issue slots
#pragma unroll 4
										for (int c = 0; c < 8; ++c)
										{
											const float4 w4 = *reinterpret_cast<const float4*>(wrow + ((c ^ sw) << 2));
											const float* ib = inb + 4 * c * GF_ROWS;
											float4 x[8];
#pragma unroll
											for (int q = 0; q < 8; ++q) x[q] = *reinterpret_cast<const float4*>(ib + 4 * q);
											const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
											for (int q = 0; q < 4; ++q)
											{
												acc[0] = fmaf(wv[q], x[2 * q].x, acc[0]); acc[1] = fmaf(wv[q], x[2 * q].y, acc[1]);
												acc[2] = fmaf(wv[q], x[2 * q].z, acc[2]); acc[3] = fmaf(wv[q], x[2 * q].w, acc[3]);
												acc[4] = fmaf(wv[q], x[2 * q + 1].x, acc[4]); acc[5] = fmaf(wv[q], x[2 * q + 1].y, acc[5]);
												acc[6] = fmaf(wv[q], x[2 * q + 1].z, acc[6]); acc[7] = fmaf(wv[q], x[2 * q + 1].w, acc[7]);
											}
										}
									}
									else
										for (int ii = 0; ii < ni - i0; ++ii) stepw(ii, wrow[(((ii >> 2) ^ sw) << 2) + (ii & 3)]);
								}
								if (timed) { tm[15] += now() - tq; tm[8] += 1; }
								release();
							}
						}
						else
						{
							// weight tiles travel global -> registers -> shared memory, the next tile's loads in flight
							// while the current one is consumed
							float pre[32];
							// this thread's part of a tile: column `lane`, rows warp, warp + 8, ... (kmax of them exist)
							const float* wsrc = W + (size_t)(o0 + warp) * ni + lane;
							const size_t wstep = (size_t)8 * ni;
							const int kmax = (no - o0 - warp + 7) >> 3;  // may be <= 0 or > 32
							const bool computes = o0 + t < no;
							{
								const float* q = wsrc;
								const bool col = lane < ni;
	#pragma unroll
								for (int k = 0; k < 32; ++k, q += wstep) pre[k] = (col && k < kmax) ? __ldcg(q) : 0.0f;
							}
							for (int i0 = 0; i0 < ni; i0 += 32)
							{
								__syncthreads();  // the tile's previous contents (and `in`) are settled
	#pragma unroll
								for (int k = 0; k < 32; ++k) Wt[(warp + 8 * k) * 33 + lane] = pre[k];
								__syncthreads();
								if (i0 + 32 < ni)
								{
									const float* q = wsrc + i0 + 32;
									const bool col = i0 + 32 + lane < ni;
	#pragma unroll
									for (int k = 0; k < 32; ++k, q += wstep) pre[k] = (col && k < kmax) ? __ldcg(q) : 0.0f;
								}
								const int lim = (ni - i0) < 32 ? (ni - i0) : 32;
								const float* wrow = Wt + t * 33;
								const float* inb = in + (size_t)i0 * GF_ROWS;
								auto step = [&](int ii) {
									const float w = wrow[ii];
									const float4 a0 = *reinterpret_cast<const float4*>(inb + ii * GF_ROWS);
									const float4 a1 = *reinterpret_cast<const float4*>(inb + ii * GF_ROWS + 4);
									acc[0] = fmaf(w, a0.x, acc[0]); acc[1] = fmaf(w, a0.y, acc[1]);
									acc[2] = fmaf(w, a0.z, acc[2]); acc[3] = fmaf(w, a0.w, acc[3]);
									acc[4] = fmaf(w, a1.x, acc[4]); acc[5] = fmaf(w, a1.y, acc[5]);
									acc[6] = fmaf(w, a1.z, acc[6]); acc[7] = fmaf(w, a1.w, acc[7]);
								};
								if (!computes)
								{
									// no output node for this thread in this pass: it only helps moving tiles
								}
								else if (lim == 32)
								{
									// full tile: a fixed trip count lets the shared-memory loads of several steps overlap
	#pragma unroll 4
									for (int ii = 0; ii < 32; ++ii) step(ii);
								}
								else
									for (int ii = 0; ii < lim; ++ii) step(ii);
							}
						}
						const int o = o0 + t;
						if (o < no)
						{
#pragma unroll
							for (int r = 0; r < GF_ROWS; ++r) out[(size_t)o * GF_ROWS + r] = squash_b(acc[r] + b, act, par);
						}
						if (use_tma) __syncthreads();  // the next tile step reads these outputs without another barrier
					}
				}
				__syncthreads();
				if (timed) { t_d = now(); tm[11] += t_d - t_c; t_c = t_d; }
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
				if (timed) { t_d = now(); tm[12] += t_d - t_c; t_c = t_d; }
				// ---- hidden deltas: D_l = (D_{l+1} W_l) * act'(A_l), thread = input node
				for (int L = H + 1; L >= 2; --L)
				{
					const int l = L - 1;
					const int ni = n.sizes[l], no = n.sizes[L];
					const float* W = n.W[l];
					const float* dup = Ds + (size_t)node_off[L] * GF_ROWS;
					const int act = n.act[l - 1];
					if (narrow_head && L == H + 1)
					{
						// D_H = (D_out W_H) * act'(A_H) from the shared copy of the head's weights: thread = input node
						for (int i = t; i < ni; i += GF_THREADS)
						{
							float acc[GF_ROWS];
#pragma unroll
							for (int r = 0; r < GF_ROWS; ++r) acc[r] = 0.0f;
							for (int o = 0; o < no; ++o)
							{
								const float w = wn[o * ni + i];
								const float4 d0 = *reinterpret_cast<const float4*>(dup + o * GF_ROWS);
								const float4 d1 = *reinterpret_cast<const float4*>(dup + o * GF_ROWS + 4);
								acc[0] = fmaf(w, d0.x, acc[0]); acc[1] = fmaf(w, d0.y, acc[1]);
								acc[2] = fmaf(w, d0.z, acc[2]); acc[3] = fmaf(w, d0.w, acc[3]);
								acc[4] = fmaf(w, d1.x, acc[4]); acc[5] = fmaf(w, d1.y, acc[5]);
								acc[6] = fmaf(w, d1.z, acc[6]); acc[7] = fmaf(w, d1.w, acc[7]);
							}
#pragma unroll
							for (int r = 0; r < GF_ROWS; ++r)
							{
								const float av = As[(size_t)(node_off[l] + i) * GF_ROWS + r];
								Ds[(size_t)(node_off[l] + i) * GF_ROWS + r] = (r < valid) ? acc[r] * act_der_b(av, act, 0.01f) : 0.0f;
							}
						}
						__syncthreads();
						continue;
					}
					for (int i0 = 0; i0 < ni; i0 += GF_THREADS)
					{
						float acc[GF_ROWS];
#pragma unroll
						for (int r = 0; r < GF_ROWS; ++r) acc[r] = 0.0f;
						if (use_tma)
						{
							const bool computes = i0 + t < ni;
							for (int o0 = 0; o0 < no; o0 += 32)
							{
								// tile rows = 32 output nodes o0.., columns = input nodes i0.. (plain layout)
								const float* stg = acquire();
								if (computes)
								{
									const int lim = (no - o0) < 32 ? (no - o0) : 32;
									const float* dub = dup + (size_t)o0 * GF_ROWS;
									auto step = [&](int oo) {
										const float w = stg[oo * GF_THREADS + t];
										const float4 d0 = *reinterpret_cast<const float4*>(dub + oo * GF_ROWS);
										const float4 d1 = *reinterpret_cast<const float4*>(dub + oo * GF_ROWS + 4);
										acc[0] = fmaf(w, d0.x, acc[0]); acc[1] = fmaf(w, d0.y, acc[1]);
										acc[2] = fmaf(w, d0.z, acc[2]); acc[3] = fmaf(w, d0.w, acc[3]);
										acc[4] = fmaf(w, d1.x, acc[4]); acc[5] = fmaf(w, d1.y, acc[5]);
										acc[6] = fmaf(w, d1.z, acc[6]); acc[7] = fmaf(w, d1.w, acc[7]);
									};
									if (lim == 32)
									{
										// loads of eight rows of the tile first, then their 64 multiply-adds (see the forward loop)
#pragma unroll 2
										for (int ob = 0; ob < 32; ob += 8)
										{
											float wv[8];
											float4 d[16];
#pragma unroll
											for (int q = 0; q < 8; ++q) wv[q] = stg[(ob + q) * GF_THREADS + t];
#pragma unroll
											for (int q = 0; q < 16; ++q) d[q] = *reinterpret_cast<const float4*>(dub + ob * GF_ROWS + 4 * q);
#pragma unroll
											for (int q = 0; q < 8; ++q)
											{
												acc[0] = fmaf(wv[q], d[2 * q].x, acc[0]); acc[1] = fmaf(wv[q], d[2 * q].y, acc[1]);
												acc[2] = fmaf(wv[q], d[2 * q].z, acc[2]); acc[3] = fmaf(wv[q], d[2 * q].w, acc[3]);
												acc[4] = fmaf(wv[q], d[2 * q + 1].x, acc[4]); acc[5] = fmaf(wv[q], d[2 * q + 1].y, acc[5]);
												acc[6] = fmaf(wv[q], d[2 * q + 1].z, acc[6]); acc[7] = fmaf(wv[q], d[2 * q + 1].w, acc[7]);
											}
										}
									}
									else
										for (int oo = 0; oo < lim; ++oo) step(oo);
								}
								release();
							}
						}
						else
						{
							float pre[32];
							const bool computes = i0 + t < ni;  // also: this thread's column of the tiles exists
							const float* wsrc = W + i0 + t;     // row o of the tile: wsrc + o * ni
							{
								const float* q = wsrc;
	#pragma unroll
								for (int k = 0; k < 32; ++k, q += ni) pre[k] = (computes && k < no) ? __ldcg(q) : 0.0f;
							}
							for (int o0 = 0; o0 < no; o0 += 32)
							{
								__syncthreads();
	#pragma unroll
								for (int k = 0; k < 32; ++k) Wt[k * GF_THREADS + t] = pre[k];
								__syncthreads();
								if (o0 + 32 < no)
								{
									const float* q = wsrc + (size_t)(o0 + 32) * ni;
									const int left = no - (o0 + 32);
	#pragma unroll
									for (int k = 0; k < 32; ++k, q += ni) pre[k] = (computes && k < left) ? __ldcg(q) : 0.0f;
								}
								const int lim = (no - o0) < 32 ? (no - o0) : 32;
								const float* dub = dup + (size_t)o0 * GF_ROWS;
								auto step = [&](int oo) {
									const float w = Wt[oo * GF_THREADS + t];
									const float4 d0 = *reinterpret_cast<const float4*>(dub + oo * GF_ROWS);
									const float4 d1 = *reinterpret_cast<const float4*>(dub + oo * GF_ROWS + 4);
									acc[0] = fmaf(w, d0.x, acc[0]); acc[1] = fmaf(w, d0.y, acc[1]);
									acc[2] = fmaf(w, d0.z, acc[2]); acc[3] = fmaf(w, d0.w, acc[3]);
									acc[4] = fmaf(w, d1.x, acc[4]); acc[5] = fmaf(w, d1.y, acc[5]);
									acc[6] = fmaf(w, d1.z, acc[6]); acc[7] = fmaf(w, d1.w, acc[7]);
								};
								if (!computes)
								{
								}
								else if (lim == 32)
								{
	#pragma unroll 4
									for (int oo = 0; oo < 32; ++oo) step(oo);
								}
								else
									for (int oo = 0; oo < lim; ++oo) step(oo);
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
				if (timed) { t_d = now(); tm[13] += t_d - t_c; t_c = t_d; }
				// ---- the group's activations and deltas to the window scratch ([row][node]); partial sums
				for (int r = 0; r < valid; ++r)
				{
					float* ga = a.actbuf + (size_t)(j0 + r) * tot;
					float* gd = a.delbuf + (size_t)(j0 + r) * tot;
					for (int e = t; e < tot; e += GF_THREADS)
					{
						ga[e] = As[(size_t)e * GF_ROWS + r];
						if (e >= node_off[1]) gd[e] = Ds[(size_t)e * GF_ROWS + r];
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
			if (timed) { t_b = now(); tm[0] += t_b - t_a; if (t_c) tm[14] += t_b - t_c; }
			grid.sync();
			if (timed) { t_a = now(); tm[1] += t_a - t_b; }

			// ================= phase 2: gradient + update per weight tile; CTA 0 also the scalars
			const float inv_len = 1.0f / (float)len;
			for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x)
			{
				int l = 0;
				while (tile >= tile_off[l + 1]) ++l;
				const int tiles_i = (n.sizes[l] + tile_i - 1) / tile_i;
				const int tl = tile - tile_off[l];
				const int o0 = (tl / tiles_i) * GF_TO, i0 = (tl % tiles_i) * tile_i;
				// the weight-tile ring is idle in this phase (every tile of the window has been consumed, the next
				// window's are issued after the grid barrier): it holds the stages of the asynchronous fill
				if (n.sizes[l + 1] <= GF_NARROW)
					gf_grad_narrow(a, l, tl * GF_NCOLS, len, tot, node_off[l], node_off[l + 1], a.ck + (size_t)l * (mb + 1), inv_len, Wt, bad);
				else
					gf_grad_tile_async(a, l, o0, i0, len, tot, node_off[l], node_off[l + 1], Wt, a.ck + (size_t)l * (mb + 1), inv_len, bad);
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
				if (warp == 0)
				{
					// the CTAs' cost / accuracy partials: lanes stride over the CTAs, then a fixed shuffle tree
					double c = 0.0, q = 0.0;
					for (int b = lane; b < (int)gridDim.x; b += 32)
					{
						c += __ldcg(a.part + (size_t)b * GF_PART);
						q += __ldcg(a.part + (size_t)b * GF_PART + 1);
					}
					c = warp_sum_d(c);
					q = warp_sum_d(q);
					if (lane == 0)
					{
						ecost += c;
						eacc += q;
					}
				}
			}
			if (timed) { t_b = now(); tm[2] += t_b - t_a; }
			grid.sync();
			if (timed) { t_a = now(); tm[3] += t_a - t_b; }
		}
		if (blockIdx.x == 0 && t == 0)
		{
			a.epoch_sums[2 * ep] = ecost;
			a.epoch_sums[2 * ep + 1] = eacc;
		}
	}
	if (timed)
		for (int k = 0; k < 16; ++k) a.timing[k] += tm[k];
	if (bad) atomicOr(a.flags, 1);
}

// =================================================================================================
// Cluster variant of the whole-window kernel.
//
// grid_fused_kernel's phase 1 is bound by how fast ONE SM gets the network's weights delivered: every CTA
// streams all of them per sample group.  Here a thread-block cluster of CF_CS CTAs carries CF_R rows through the
// network together and every CTA owns 1/CF_CS of each layer's NODES: it keeps the weight rows of its nodes
// (forward) and the weight columns of its nodes (hidden deltas) in shared memory for the whole window -- read
// from L2 once per window instead of once per sample group -- computes its nodes' activations for the
// CF_R rows and stores them into the activation buffers of all CF_CS CTAs over distributed shared memory
// (st.shared::cluster: plain stores), one cluster barrier per layer.  The head runs on every CTA's own
// copy (side effects from cluster rank 0 only).  Activations and deltas go to the same window scratch as in
// grid_fused_kernel, and phase 2 sums the window's rows per weight tile -- here with a 4 x 4 register tile per
// lane and the 64 rows of a step dealt over the eight warps, whose partial sums are added in warp order.
// Everything is deterministic.  All barriers are executed unconditionally by every thread of every CTA.
constexpr int CF_CS = 8;   // CTAs per cluster (the portable maximum)
constexpr int CF_R = 32;   // rows a cluster carries through the network together

struct CfPlan
{
	int tot;                                  // nodes of the network
	int node_off[GL_MAX_WEIGHT_LAYERS + 2];   // first node of layer j
	int sl[GL_MAX_WEIGHT_LAYERS + 2];         // nodes of layer j one CTA owns (a multiple of 4)
	int d_off[GL_MAX_WEIGHT_LAYERS + 2];      // first row of layer j's deltas in the delta buffer (j >= 1)
	int d_rows;                               // rows of the delta buffer (each layer rounded up to 4 nodes)
	int wf[GL_MAX_WEIGHT_LAYERS + 1];         // float offset of the forward slice of weight layer l
	int wb[GL_MAX_WEIGHT_LAYERS + 1];         // float offset of the delta slice of node layer j (1..H)
	int rowm;                                 // float offset of the per-row metric scratch
	int soff[GL_MAX_WEIGHT_LAYERS + 2];       // the window scratch: first column of layer j
	int pitch;                                // and its pitch
	int floats;                               // dynamic shared memory, floats
};

__host__ __device__ inline void cf_plan(const NetView& n, CfPlan& p)
{
	const int H = n.H;
	int tot = 0;
	for (int j = 0; j <= H + 1; ++j)
	{
		p.node_off[j] = tot;
		tot += n.sizes[j];
		p.sl[j] = (((n.sizes[j] + CF_CS - 1) / CF_CS) + 3) & ~3;
	}
	p.tot = tot;
	int dr = 0;
	p.d_off[0] = 0;
	for (int j = 1; j <= H + 1; ++j)
	{
		p.d_off[j] = dr;
		dr += (n.sizes[j] + 3) & ~3;
	}
	p.d_rows = dr;
	int f = (tot + dr) * CF_R;
	for (int l = 0; l <= H; ++l)
	{
		p.wf[l] = f;
		f += p.sl[l + 1] * (n.sizes[l] + 4);
	}
	p.wb[0] = 0;
	for (int j = 1; j <= H; ++j)
	{
		p.wb[j] = f;
		f += p.sl[j] * (((n.sizes[j + 1] + 3) & ~3) + 4);
	}
	p.rowm = f;
	f += 2 * CF_R;
	p.pitch = gf_scratch_layout(n, p.soff);
	p.floats = f > GF_P2_MAX_FLOATS ? f : GF_P2_MAX_FLOATS;  // the phase-2 stages alias the phase-1 buffers
}

__device__ __forceinline__ uint32_t cl_rank()
{
	uint32_t r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}
// every thread of every CTA of the cluster; orders shared::cluster stores before it against loads after it
__device__ __forceinline__ void cl_sync()
{
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cl_map(uint32_t local_addr, uint32_t rank)
{
	uint32_t r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
	return r;
}
__device__ __forceinline__ void cl_store4(uint32_t cluster_addr, float x, float y, float z, float w)
{
	asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

// s[q] = sum_k InT[k][4 * sq + q] * Wsl[n][k] (q = 0..3) for the CTA's `cnt` nodes n; InT is [K][CF_R], Wsl is
// [cnt][K + 4], K a multiple of 4.  Thread = one node and four rows (eight row quads x 32 nodes per pass); where
// the CTA owns at most 8 nodes a warp takes one node and its four lane groups a quarter of k each, added in
// lane-group order.  epi(n, sq, s0, s1, s2, s3) runs once per node and row quad.
template <typename Epi>
__device__ __forceinline__ void cf_product(const float* InT, int K, const float* Wsl, int cnt, Epi epi)
{
	const int t = threadIdx.x, sq = t & 7;
	const int ws = K + 4;
	const float* in = InT + 4 * sq;
	auto dot = [&](const float* w, int k0, int k1, float& a0, float& a1, float& a2, float& a3) {
#pragma unroll 2
		for (int k = k0; k < k1; k += 4)
		{
			const float4 wv = *reinterpret_cast<const float4*>(w + k);
			const float4 x0 = *reinterpret_cast<const float4*>(in + (size_t)(k + 0) * CF_R);
			const float4 x1 = *reinterpret_cast<const float4*>(in + (size_t)(k + 1) * CF_R);
			const float4 x2 = *reinterpret_cast<const float4*>(in + (size_t)(k + 2) * CF_R);
			const float4 x3 = *reinterpret_cast<const float4*>(in + (size_t)(k + 3) * CF_R);
			a0 = fmaf(wv.x, x0.x, a0); a1 = fmaf(wv.x, x0.y, a1); a2 = fmaf(wv.x, x0.z, a2); a3 = fmaf(wv.x, x0.w, a3);
			a0 = fmaf(wv.y, x1.x, a0); a1 = fmaf(wv.y, x1.y, a1); a2 = fmaf(wv.y, x1.z, a2); a3 = fmaf(wv.y, x1.w, a3);
			a0 = fmaf(wv.z, x2.x, a0); a1 = fmaf(wv.z, x2.y, a1); a2 = fmaf(wv.z, x2.z, a2); a3 = fmaf(wv.z, x2.w, a3);
			a0 = fmaf(wv.w, x3.x, a0); a1 = fmaf(wv.w, x3.y, a1); a2 = fmaf(wv.w, x3.z, a2); a3 = fmaf(wv.w, x3.w, a3);
		}
	};
	if (cnt <= 8)
	{
		const int n = t >> 5, kc = (t >> 3) & 3;
		const int chunk = (((K + 3) / 4) + 3) & ~3;
		float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
		if (n < cnt)
		{
			const int k0 = kc * chunk, k1 = (k0 + chunk) < K ? (k0 + chunk) : K;
			dot(Wsl + (size_t)n * ws, k0, k1, a0, a1, a2, a3);
		}
		// whole warps take part in the shuffles (n is uniform in a warp)
#pragma unroll
		for (int off = 8; off <= 16; off <<= 1)
		{
			a0 += __shfl_xor_sync(0xffffffffu, a0, off);
			a1 += __shfl_xor_sync(0xffffffffu, a1, off);
			a2 += __shfl_xor_sync(0xffffffffu, a2, off);
			a3 += __shfl_xor_sync(0xffffffffu, a3, off);
		}
		if (n < cnt && kc == 0) epi(n, sq, a0, a1, a2, a3);
		return;
	}
	for (int nb = 0; nb < cnt; nb += 32)
	{
		const int n = nb + (t >> 3);
		if (n < cnt)
		{
			float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
			dot(Wsl + (size_t)n * ws, 0, K, a0, a1, a2, a3);
			epi(n, sq, a0, a1, a2, a3);
		}
	}
}

__global__ void __launch_bounds__(GF_THREADS, 1) cluster_fused_kernel(const __grid_constant__ GridFusedArgs a)
{
	extern __shared__ __align__(16) float sm[];
	cg::grid_group grid = cg::this_grid();
	const NetView& n = a.net;
	const int H = n.H;
	const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
	const int n_out = n.sizes[H + 1];
	const int mb = n.mb;
	const int crank = (int)cl_rank();
	const int cid = (int)blockIdx.x / CF_CS, nclusters = (int)gridDim.x / CF_CS;
	__shared__ CfPlan P;
	__shared__ double s_part[GF_PART];
	if (t == 0) cf_plan(n, P);
	__syncthreads();
	const int tot = P.tot;
	const int pitch = P.pitch;
	float* AT = sm;                          // [tot][CF_R] activations, node-major
	float* DT = sm + (size_t)tot * CF_R;     // [d_rows][CF_R] deltas of node layers 1..H+1
	float* rowm = sm + P.rowm;               // [CF_R][2]: cost, accuracy of the pass's rows
	// the phase-2 stages alias the phase-1 region (the phases are separated by grid barriers)
	const uint32_t at_addr = smem_u32(AT), dt_addr = smem_u32(DT);

	const bool classify = n.out_type != GL_OUT_REGRESSION;
	const bool softmax = n.act[H] == GL_ACT_SOFTMAX;
	const float data_size = a.data_size;

	// phase-2 work items: layer l has ceil(no/16) * ceil(ni/32) tiles, or ceil(ni/64) column groups where no <= 4
	int tile_off[GL_MAX_WEIGHT_LAYERS + 2];
	int tiles = 0;
	for (int l = 0; l <= H; ++l)
	{
		tile_off[l] = tiles;
		tiles += (n.sizes[l + 1] <= GF_NARROW) ? (n.sizes[l] + GF_NCOLS - 1) / GF_NCOLS
		                                       : ((n.sizes[l + 1] + GF_TO - 1) / GF_TO) * ((n.sizes[l] + GF_P2_TI - 1) / GF_P2_TI);
	}
	tile_off[H + 1] = tiles;

	const bool timed = a.timing != nullptr && blockIdx.x == 0 && t == 0;
	unsigned long long tm[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0}, t_a = 0, t_b = 0, t_c = 0, t_d = 0;
	auto now = []() {
		unsigned long long v;
		asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
		return v;
	};

	cl_sync();  // every CTA of the cluster is running before the first store into its shared memory
	int bad = 0;
	for (int ep = 0; ep < a.n_epochs; ++ep)
	{
		const bool last_epoch = ep == a.n_epochs - 1;
		double ecost = 0.0, eacc = 0.0;  // CTA 0, thread 0
		for (long long r0 = 0; r0 < a.rows; r0 += mb)
		{
			const int len = (int)((a.rows - r0) < mb ? (a.rows - r0) : mb);
			const int passes = (len + CF_R - 1) / CF_R;
			if (t < GF_PART) s_part[t] = 0.0;
			if (timed) t_a = now();
			// ---- this window's weights of the CTA's nodes: rows of W_l (forward), columns of W_j (hidden deltas)
			for (int l = 0; l <= H; ++l)
			{
				const int K = n.sizes[l], nb0 = crank * P.sl[l + 1];
				int cnt = n.sizes[l + 1] - nb0;
				cnt = cnt < 0 ? 0 : (cnt > P.sl[l + 1] ? P.sl[l + 1] : cnt);
				const float* src = n.W[l] + (size_t)nb0 * K;
				float* dst = sm + P.wf[l];
				const int kq = K >> 2;
				for (int e = t; e < cnt * kq; e += GF_THREADS)
				{
					const int r = e / kq, k = (e - r * kq) << 2;
					*reinterpret_cast<float4*>(dst + (size_t)r * (K + 4) + k) = __ldcg(reinterpret_cast<const float4*>(src + (size_t)r * K + k));
				}
			}
			for (int j = 1; j <= H; ++j)
			{
				const int ni = n.sizes[j], no = n.sizes[j + 1], K4 = (no + 3) & ~3, i0 = crank * P.sl[j];
				int cnt = ni - i0;
				cnt = cnt < 0 ? 0 : (cnt > P.sl[j] ? P.sl[j] : cnt);
				const float* src = n.W[j] + i0;
				float* dst = sm + P.wb[j];
				for (int e = t; e < cnt * K4; e += GF_THREADS)
				{
					const int o = e / cnt, i = e - o * cnt;
					dst[(size_t)i * (K4 + 4) + o] = (o < no) ? __ldcg(src + (size_t)o * ni + i) : 0.0f;
				}
			}
			__syncthreads();
			if (timed) { t_c = now(); tm[4] += t_c - t_a; }
			// ================= phase 1: forward, head, deltas, CF_R rows per cluster pass
			for (int pass = cid; pass < passes; pass += nclusters)
			{
				const int j0 = pass * CF_R;
				const int valid = (len - j0) < CF_R ? (len - j0) : CF_R;
				{
					// inputs of the pass, transposed to [node][row]; every CTA reads them itself
					const int n0 = n.sizes[0], kq = n0 >> 2;
					for (int e = t; e < CF_R * kq; e += GF_THREADS)
					{
						const int r = e / kq, i = (e - r * kq) << 2;
						float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
						if (r < valid) v = *reinterpret_cast<const float4*>(a.X + (size_t)(r0 + j0 + r) * n0 + i);
						AT[(i + 0) * CF_R + r] = v.x;
						AT[(i + 1) * CF_R + r] = v.y;
						AT[(i + 2) * CF_R + r] = v.z;
						AT[(i + 3) * CF_R + r] = v.w;
					}
				}
				__syncthreads();
				for (int l = 0; l <= H; ++l)
				{
					const int nb0 = crank * P.sl[l + 1];
					int cnt = n.sizes[l + 1] - nb0;
					cnt = cnt < 0 ? 0 : (cnt > P.sl[l + 1] ? P.sl[l + 1] : cnt);
					const float b = (l >= 1) ? __ldcg(n.bias + l) : 0.0f;
					const int act = n.act[l];
					const float par = n.par[l];
					const int out_node = P.node_off[l + 1] + nb0, out_col = P.soff[l + 1] + nb0;
					const bool hidden = l < H;
					cf_product(AT + (size_t)P.node_off[l] * CF_R, n.sizes[l], sm + P.wf[l], cnt,
					           [&](int nn, int sq, float s0, float s1, float s2, float s3) {
						           const float v0 = squash_b(s0 + b, act, par), v1 = squash_b(s1 + b, act, par);
						           const float v2 = squash_b(s2 + b, act, par), v3 = squash_b(s3 + b, act, par);
						           const uint32_t local = at_addr + (uint32_t)(((out_node + nn) * CF_R + 4 * sq) * 4);
#pragma unroll
						           for (int dst = 0; dst < CF_CS; ++dst) cl_store4(cl_map(local, (uint32_t)dst), v0, v1, v2, v3);
						           if (hidden)
						           {
							           float* ga = a.actbuf + (size_t)(j0 + 4 * sq) * pitch + out_col + nn;
							           if (4 * sq + 0 < valid) ga[0] = v0;
							           if (4 * sq + 1 < valid) ga[(size_t)pitch] = v1;
							           if (4 * sq + 2 < valid) ga[(size_t)2 * pitch] = v2;
							           if (4 * sq + 3 < valid) ga[(size_t)3 * pitch] = v3;
						           }
					           });
					cl_sync();  // the layer's activations have landed in every CTA of the cluster
				}
				if (timed) { t_d = now(); tm[5] += t_d - t_c; t_c = t_d; }
				// ---- head on this CTA's copy: warp = four rows of the pass; side effects from cluster rank 0 only
				for (int rr = 0; rr < CF_R / 8; ++rr)
				{
					const int r = warp * (CF_R / 8) + rr;
					float* p = AT + (size_t)P.node_off[H + 1] * CF_R + r;  // stride CF_R
					float* dout = DT + (size_t)P.d_off[H + 1] * CF_R + r;
					float c_acc = 0.0f, a_acc = 0.0f, be = 0.0f, bp = 0.0f;
					int ie = -1, ip = -1;
					if (r < valid)
					{
						const float* y = a.Y + (r0 + j0 + r) * n_out;
						float mx = -INFINITY, inv_den = 1.0f;
						if (softmax)
						{
							for (int o = lane; o < n_out; o += 32) mx = fmaxf(mx, p[(size_t)o * CF_R]);
							mx = warp_max(mx);
							float den = 0.0f;
							for (int o = lane; o < n_out; o += 32) den += expf(p[(size_t)o * CF_R] - mx);
							inv_den = 1.0f / warp_sum(den);
						}
						for (int o = lane; o < n_out; o += 32)
						{
							float pv = p[(size_t)o * CF_R];
							const float e = y[o];
							float cost, d;
							if (softmax)
							{
								pv = expf(pv - mx) * inv_den;
								p[(size_t)o * CF_R] = pv;
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
							dout[(size_t)o * CF_R] = d;
							if (crank == 0)
							{
								a.actbuf[(size_t)(j0 + r) * pitch + P.soff[H + 1] + o] = pv;
								a.delbuf[(size_t)(j0 + r) * pitch + P.soff[H + 1] + o] = d;
							}
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
						if (crank == 0)
						{
							if (lane == 0 && classify && last_epoch && ie >= 0 && ip >= 0) atomicAdd(a.confusion + ie * n_out + ip, 1);
							if (a.last_out && last_epoch && r0 + j0 + r == a.rows - 1)
								for (int o = lane; o < n_out; o += 32) a.last_out[o] = p[(size_t)o * CF_R];
						}
					}
					else
					{
						for (int o = lane; o < n_out; o += 32) dout[(size_t)o * CF_R] = 0.0f;
					}
					// rows of the delta buffer beyond the layer's nodes (rounded up to 4) take part in the next product as zeros
					for (int o = n_out + lane; o < ((n_out + 3) & ~3); o += 32) dout[(size_t)o * CF_R] = 0.0f;
					if (lane == 0)
					{
						rowm[2 * r] = c_acc;
						rowm[2 * r + 1] = a_acc;
					}
				}
				__syncthreads();
				if (timed) { t_d = now(); tm[6] += t_d - t_c; t_c = t_d; }
				// ---- hidden deltas of the CTA's nodes: D_j = (D_{j+1} W_j) * act'(A_j)
				for (int j = H; j >= 1; --j)
				{
					const int i0 = crank * P.sl[j];
					int cnt = n.sizes[j] - i0;
					cnt = cnt < 0 ? 0 : (cnt > P.sl[j] ? P.sl[j] : cnt);
					const int act = n.act[j - 1];
					const int node = P.node_off[j] + i0, drow = P.d_off[j] + i0, dcol = P.soff[j] + i0;
					const bool gather = j >= 2;
					cf_product(DT + (size_t)P.d_off[j + 1] * CF_R, (n.sizes[j + 1] + 3) & ~3, sm + P.wb[j], cnt,
					           [&](int nn, int sq, float s0, float s1, float s2, float s3) {
						           const float4 av = *reinterpret_cast<const float4*>(AT + (size_t)(node + nn) * CF_R + 4 * sq);
						           const float d0 = (4 * sq + 0 < valid) ? s0 * act_der_b(av.x, act, 0.01f) : 0.0f;
						           const float d1 = (4 * sq + 1 < valid) ? s1 * act_der_b(av.y, act, 0.01f) : 0.0f;
						           const float d2 = (4 * sq + 2 < valid) ? s2 * act_der_b(av.z, act, 0.01f) : 0.0f;
						           const float d3 = (4 * sq + 3 < valid) ? s3 * act_der_b(av.w, act, 0.01f) : 0.0f;
						           if (gather)
						           {
							           const uint32_t local = dt_addr + (uint32_t)(((drow + nn) * CF_R + 4 * sq) * 4);
#pragma unroll
							           for (int dst = 0; dst < CF_CS; ++dst) cl_store4(cl_map(local, (uint32_t)dst), d0, d1, d2, d3);
						           }
						           float* gd = a.delbuf + (size_t)(j0 + 4 * sq) * pitch + dcol + nn;
						           if (4 * sq + 0 < valid) gd[0] = d0;
						           if (4 * sq + 1 < valid) gd[(size_t)pitch] = d1;
						           if (4 * sq + 2 < valid) gd[(size_t)2 * pitch] = d2;
						           if (4 * sq + 3 < valid) gd[(size_t)3 * pitch] = d3;
					           });
					if (gather) cl_sync();
				}
				if (timed) { t_d = now(); tm[7] += t_d - t_c; t_c = t_d; }
				// the inputs of the pass belong to the window scratch too (phase 2 of layer 0 reads them)
				{
					const int n0 = n.sizes[0];
					for (int e = t + crank * GF_THREADS; e < valid * n0; e += GF_THREADS * CF_CS)
					{
						const int r = e / n0, i = e - r * n0;
						a.actbuf[(size_t)(j0 + r) * pitch + i] = AT[(size_t)i * CF_R + r];
					}
				}
				if (crank == 0)
				{
					if (warp >= 1 && warp <= H)
					{
						// scalar-bias delta of hidden layer `warp`: sum of the deltas of the layer above, this pass's rows
						const int l = warp, no = n.sizes[l + 1];
						double s = 0.0;
						for (int e = lane; e < no * CF_R; e += 32) s += (double)DT[(size_t)P.d_off[l + 1] * CF_R + e];
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
				cl_sync();  // nobody of the cluster reads this pass's buffers any more: the next pass may overwrite them
				if (timed) { t_d = now(); tm[8] += t_d - t_c; t_c = t_d; }
			}
			__syncthreads();
			if (t < GF_PART) a.part[(size_t)blockIdx.x * GF_PART + t] = s_part[t];
			if (timed) { t_b = now(); tm[0] += t_b - t_a; }
			grid.sync();
			if (timed) { t_a = now(); tm[1] += t_a - t_b; }

			// ================= phase 2: gradient + update per weight tile; CTA 0 also the scalars
			const float inv_len = 1.0f / (float)len;
			for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x)
			{
				int l = 0;
				while (tile >= tile_off[l + 1]) ++l;
				const int tiles_i = (n.sizes[l] + GF_P2_TI - 1) / GF_P2_TI;
				const int tl = tile - tile_off[l];
				const float* ckl = a.ck + (size_t)l * (mb + 1);
				if (n.sizes[l + 1] <= GF_NARROW)
					gf_grad_narrow(a, l, tl * GF_NCOLS, len, pitch, P.soff[l], P.soff[l + 1], ckl, inv_len, sm, bad);
				else
					gf_grad_tile_async(a, l, (tl / tiles_i) * GF_TO, (tl % tiles_i) * GF_P2_TI, len, pitch, P.soff[l], P.soff[l + 1], sm,
					                   ckl, inv_len, bad);
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
				if (warp == 0)
				{
					double c = 0.0, q = 0.0;
					for (int b = lane; b < (int)gridDim.x; b += 32)
					{
						c += __ldcg(a.part + (size_t)b * GF_PART);
						q += __ldcg(a.part + (size_t)b * GF_PART + 1);
					}
					c = warp_sum_d(c);
					q = warp_sum_d(q);
					if (lane == 0)
					{
						ecost += c;
						eacc += q;
					}
				}
			}
			if (timed) { t_b = now(); tm[2] += t_b - t_a; }
			grid.sync();
			if (timed) { t_a = now(); tm[3] += t_a - t_b; }
		}
		if (blockIdx.x == 0 && t == 0)
		{
			a.epoch_sums[2 * ep] = ecost;
			a.epoch_sums[2 * ep + 1] = eacc;
		}
	}
	if (timed)
		for (int k = 0; k < 9; ++k) a.timing[k] += tm[k];
	if (bad) atomicOr(a.flags, 1);
}

}  // namespace

size_t grid_fused_smem_bytes(const NetView& n)
{
	int off[GL_MAX_WEIGHT_LAYERS + 2];
	const int tot = gf_scratch_layout(n, off);
	size_t f = 2 * (size_t)tot * GF_ROWS + 2 * GF_ROWS + 3 * GF_SEQ_MAX;
	if (n.sizes[n.H + 1] <= GF_NARROW && n.H >= 1)  // the narrow head's weights and the partial sums of its forward product
		f += (((size_t)n.sizes[n.H + 1] * n.sizes[n.H] + 3) & ~(size_t)3) + 8 * GF_ROWS * GF_NARROW;
	// + alignment slack + the ring (its first stage doubles as the register-path tile buffer, GF_WT floats)
	return f * sizeof(float) + 1024 + (size_t)GF_NS * GF_STAGE + 64;
}

int grid_fused_scratch_pitch(const NetView& n)
{
	int soff[GL_MAX_WEIGHT_LAYERS + 2];
	return gf_scratch_layout(n, soff);
}

int grid_fused_total_nodes(const NetView& n)
{
	int tot = 0;
	for (int l = 0; l <= n.H + 1; ++l) tot += n.sizes[l];
	return tot;
}

int grid_fused_group_tiles(const NetView& n)
{
	const int skip = (n.sizes[n.H + 1] <= GF_NARROW && n.H >= 1) ? 1 : 0;  // a narrow head goes without tiles
	int steps = 0;
	for (int l = 0; l <= n.H - skip; ++l) steps += ((n.sizes[l + 1] + GF_THREADS - 1) / GF_THREADS) * ((n.sizes[l] + 31) / 32);
	for (int L = n.H + 1 - skip; L >= 2; --L) steps += ((n.sizes[L - 1] + GF_THREADS - 1) / GF_THREADS) * ((n.sizes[L] + 31) / 32);
	return steps;
}

cudaError_t launch_grid_fused(const GridFusedArgs& a, cudaStream_t s)
{
	const size_t bytes = grid_fused_smem_bytes(a.net);
	{
		// the attribute belongs to the current device: set it per launch (a cheap call) rather than cache it per process
		cudaError_t e = a.tma ? cudaFuncSetAttribute(grid_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes)
		                      : cudaFuncSetAttribute(grid_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
		if (e != cudaSuccess) return e;
	}
	if (a.part_ctas < 1) return cudaErrorInvalidValue;
	GridFusedArgs copy = a;
	void* params[] = {&copy};
	// one CTA per SM (the shared-memory footprint allows no more), all co-resident as the grid barrier needs
	void* fn = a.tma ? (void*)grid_fused_kernel<true> : (void*)grid_fused_kernel<false>;
	return cudaLaunchCooperativeKernel(fn, dim3((unsigned)a.part_ctas), dim3(GF_THREADS), params, bytes, s);
}

// ---- cluster variant: host side ------------------------------------------------------------------
size_t cluster_fused_smem_bytes(const NetView& n)
{
	CfPlan p;
	cf_plan(n, p);
	return (size_t)p.floats * sizeof(float);
}

// The variant wants every layer that is read as an input (0..H) to be a multiple of 4 nodes (16-byte rows for
// the vector loads), at least one hidden layer, and its buffers inside one SM's shared memory.
bool cluster_fused_fits(const NetView& n)
{
	if (n.H < 1) return false;
	for (int l = 0; l <= n.H; ++l)
		if (n.sizes[l] % 4 != 0) return false;
	return cluster_fused_smem_bytes(n) <= (size_t)226 * 1024;
}

static cudaError_t cluster_fused_config(const NetView& n, cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attrs, unsigned grid, cudaStream_t s)
{
	const size_t bytes = cluster_fused_smem_bytes(n);
	cudaError_t e = cudaFuncSetAttribute(cluster_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
	if (e != cudaSuccess) return e;
	memset(&cfg, 0, sizeof cfg);
	cfg.gridDim = dim3(grid);
	cfg.blockDim = dim3(GF_THREADS);
	cfg.dynamicSmemBytes = bytes;
	cfg.stream = s;
	attrs[0].id = cudaLaunchAttributeClusterDimension;
	attrs[0].val.clusterDim.x = CF_CS;
	attrs[0].val.clusterDim.y = 1;
	attrs[0].val.clusterDim.z = 1;
	attrs[1].id = cudaLaunchAttributeCooperative;
	attrs[1].val.cooperative = 1;
	cfg.attrs = attrs;
	cfg.numAttrs = 2;
	return cudaSuccess;
}

// CTAs of the largest co-resident grid of whole clusters on the current device (0: the variant cannot run here)
int cluster_fused_max_ctas(const NetView& n)
{
	cudaLaunchConfig_t cfg;
	cudaLaunchAttribute attrs[2];
	if (cluster_fused_config(n, cfg, attrs, CF_CS, 0) != cudaSuccess)
	{
		cudaGetLastError();
		return 0;
	}
	cfg.numAttrs = 1;  // the occupancy query takes the cluster shape; co-residency is what it reports
	int clusters = 0;
	if (cudaOccupancyMaxActiveClusters(&clusters, cluster_fused_kernel, &cfg) != cudaSuccess)
	{
		cudaGetLastError();
		return 0;
	}
	return clusters * CF_CS;
}

cudaError_t launch_cluster_fused(const GridFusedArgs& a, cudaStream_t s)
{
	if (a.part_ctas < CF_CS || a.part_ctas % CF_CS != 0) return cudaErrorInvalidValue;
	cudaLaunchConfig_t cfg;
	cudaLaunchAttribute attrs[2];
	cudaError_t e = cluster_fused_config(a.net, cfg, attrs, (unsigned)a.part_ctas, s);
	if (e != cudaSuccess) return e;
	return cudaLaunchKernelEx(&cfg, cluster_fused_kernel, a);
}

}  // namespace glb
