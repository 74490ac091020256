// Device-side building blocks shared by the tensor-core layer-product kernels (one-CTA and CTA-pair
// variants): mbarrier waits with a bound, TMA tile loads, shared-memory matrix descriptors, the
// tcgen05 MMA / commit / tensor-memory load wrappers, and the epilogue's staged bulk-store sink.
#pragma once
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tc_gemm.h"

namespace glb {
namespace tc {

constexpr int TC_BM = 128;
constexpr int TC_CHUNK_K = 128;  // k held by one tensor-memory accumulator before it is drained
constexpr long long TC_WAIT_CYCLES = 2000000000ll;  // about a second

struct TcParams
{
	float* C;
	float* C_lo;
	long long ldc;
	int K;
	int a_mn, b_mn;  // 1: operand is M/N-contiguous (MN-major), 0: K-contiguous (K-major)
	int epi;
	const float* bias_ptr;
	int act;
	float par;
	const float* aux;
	long long ld_aux;
	float alpha;
	const float* colterm;
	int* err_flag;
	unsigned* relu_mask_out;
	const unsigned* relu_mask_in;
	int mask_ld;           // words per row of the ReLU masks (= N / 32)
	int debug;             // experiments only: bit 0 skips the global stores of the epilogue
	int tiles_m, tiles_n;  // the CTAs walk the tiles_m * tiles_n output tiles persistently
	// Split of the last, partial wave of tiles along k ("stream-K", see TcWork): the first sk_full_tiles tiles
	// are whole-tile work items; the k-blocks of the remaining tiles are dealt out evenly over the CTAs.
	// sk_work == NULL: every tile is a whole-tile item.
	float* sk_work;        // [grid][128 x BN] fp32: a CTA's partial tile, if it has one
	unsigned* sk_flags;    // [grid][8]: launch number, per epilogue warp, once that warp's part of the partial is stored
	unsigned sk_epoch;     // this launch's number (flags only ever grow)
	int sk_full_tiles;
};

// The work items of one CTA, the same sequence for the producer, the MMA lane and the epilogue warps.
// First the whole tiles t = cta, cta + grid, ... below sk_full_tiles.  Then the CTA's share of the remaining
// tiles' k-blocks: with R tiles of KB k-blocks left, CTA c owns the units [c * R * KB / grid, (c + 1) * R * KB / grid)
// of the sequence (tile 0 k-block 0, tile 0 k-block 1, ..., tile R - 1 k-block KB - 1) -- at most the tail of one tile
// (a PARTIAL: its accumulators go to the CTA's workspace slot), whole tiles, and the head of one more tile (the
// tile's FINISHER: it adds the partials of the CTAs that hold the rest of the tile, in CTA order, and runs the
// epilogue).  A CTA computes its partial first and finishes a tile last, so a finisher rarely waits.  The split
// depends only on the shape and the grid, and the partials are added in a fixed order: results are reproducible.
struct TcWork
{
	// (ints: the launch only splits when grid * units fits 31 bits)
	int grid, KB, full, units;
	int u, u1;  // units of the split region still to do: [u, u1)
	int t;      // next whole tile of the first phase
	__device__ TcWork(int cta, int grid_, int KB_, int total, int full_)
	    : grid(grid_), KB(KB_), full(full_), units((total - full_) * KB_), t(cta)
	{
		u = share_begin(cta);
		u1 = share_begin(cta + 1);
	}
	// tile, k-block range [kb0, kb1) of the next item; false when the CTA is done
	__device__ bool next(int& tile, int& kb0, int& kb1)
	{
		if (t < full)
		{
			tile = t;
			kb0 = 0;
			kb1 = KB;
			t += grid;
			return true;
		}
		if (u >= u1) return false;
		const int tr = u / KB;
		tile = full + tr;
		kb0 = u - tr * KB;
		kb1 = min(KB, kb0 + (u1 - u));
		u += kb1 - kb0;
		return true;
	}
	// first unit of CTA j's share
	__device__ int share_begin(int j) const { return (int)(((unsigned)j * (unsigned)units) / (unsigned)grid); }
};

// Data-parallel weight gradient: rows [o * band_rows, (o + 1) * band_rows) of C belong to rank o and
// are stored straight into that rank's memory (maps[o] / bases[o] describe the band as a
// [band_rows][N] matrix there) instead of into C.
struct TcPeer
{
	const CUtensorMap* maps;  // device array, one map per owner
	float* const* bases;      // device array, one base pointer per owner
	int band_rows;
	int self;                 // this rank: its CTAs walk the owners' bands starting with owner self + 1
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.b32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok)
	    : "r"(bar), "r"(parity)
	    : "memory");
	return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already gave up.
__device__ __noinline__ static bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err_flag, int code)
{
	if (mbar_try(bar, parity)) return true;
	const long long t0 = clock64();
	for (;;)
	{
		if (mbar_try(bar, parity)) return true;
		if (*abort_flag) return false;
		if (clock64() - t0 > TC_WAIT_CYCLES)
		{
			*abort_flag = 1;
			atomicExch(err_flag, code);
			return false;
		}
	}
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1)
{
	asm volatile(
	    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
	    "l"(map), "r"(bar), "r"(c0), "r"(c1)
	    : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2)
{
	asm volatile(
	    "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
	    "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
	    : "memory");
}

// Shared-memory matrix descriptor (descriptor version 1).  layout_type 2 = 128-byte swizzle of
// 16-byte chunks (K-major tiles); layout_type 1 = 128-byte swizzle of 32-byte chunks, the only
// swizzle the tensor core accepts for 32-bit operands stored M/N-contiguous.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type)
{
	uint64_t d = 0;
	d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
	d |= (uint64_t)(lbo_bytes >> 4) << 16;
	d |= (uint64_t)(sbo_bytes >> 4) << 32;
	d |= 1ull << 46;
	d |= (uint64_t)layout_type << 61;
	return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "setp.ne.b32 p, %4, 0;\n\t"
	    "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
	    "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
	    : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
	asm volatile(
	    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
	    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
	    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
	    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
	      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
	      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
	      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
	    : "r"(taddr)
	    : "memory");
}


// Where one epilogue warp's 32 x 128 block of C goes.  Normal path: 32-column pieces are written
// into the warp's 4 KB staging area in the 128-byte-swizzled order of the tensor map and leave as
// one bulk tensor store each, so global memory sees whole 128-byte rows instead of 32 scattered
// 16-byte pieces per instruction, and the warp does not wait for the stores.  direct = the plain
// per-thread float4 stores (comparison runs only).
struct RowSink
{
	float* crow;    // direct path: this thread's row of C, and of the low-part matrix (or NULL)
	float* lorow;
	uint32_t stage; // shared-memory address of the warp's staging area
	const CUtensorMap* mapC;
	const CUtensorMap* mapClo;  // or NULL
	int col0, row0;  // first column of the warp's block, first row of the warp's 32 rows
	int lane;
	bool direct;
	int nbuf;        // staging areas of this warp (1 or 2), 4 KB apart
	int* turn;       // running count of pieces, to alternate between the areas
};

// Start of a 32-column piece: pick the staging area and make sure no earlier store still reads it.
__device__ __forceinline__ uint32_t sink_begin(const RowSink& k)
{
	const uint32_t area = k.stage + (uint32_t)((*k.turn) % k.nbuf) * 4096u;
	++*k.turn;
	if (k.lane == 0)
	{
		if (k.nbuf == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
		else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
	}
	__syncwarp();
	return area;
}
// Four consecutive values of this thread's row, 16-byte chunk v of the piece, in the swizzled order.
__device__ __forceinline__ void sink_put(const RowSink& k, uint32_t area, int v, float o0, float o1, float o2, float o3)
{
	asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(area + (uint32_t)k.lane * 128u + (uint32_t)((v ^ (k.lane & 7)) << 4)),
	             "f"(o0), "f"(o1), "f"(o2), "f"(o3)
	             : "memory");
}
// End of the piece: hand the 32 x 32 block to the copy engine.
__device__ __forceinline__ void sink_end(const RowSink& k, uint32_t area, const CUtensorMap* map, int piece)
{
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
	__syncwarp();
	if (k.lane == 0)
	{
		asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(area),
		             "r"(k.col0 + piece * 32), "r"(k.row0)
		             : "memory");
		asm volatile("cp.async.bulk.commit_group;" ::: "memory");
	}
}

// One thread's 128 accumulators -> its row of C (and optionally the low TF32 parts), through the
// element-wise function f(value, column).  Fully unrolled so that acc[] stays in registers.
template <class F>
__device__ __forceinline__ void store_row(const float (&acc)[128], const RowSink& k, F f)
{
	if (k.direct)
	{
#pragma unroll
		for (int v = 0; v < 32; ++v)
		{
			const float o0 = f(acc[v * 4 + 0], v * 4 + 0), o1 = f(acc[v * 4 + 1], v * 4 + 1);
			const float o2 = f(acc[v * 4 + 2], v * 4 + 2), o3 = f(acc[v * 4 + 3], v * 4 + 3);
			*reinterpret_cast<float4*>(k.crow + v * 4) = make_float4(o0, o1, o2, o3);
			if (k.lorow)
				*reinterpret_cast<float4*>(k.lorow + v * 4) = make_float4(tf32_lo(o0), tf32_lo(o1), tf32_lo(o2), tf32_lo(o3));
		}
		return;
	}
#pragma unroll
	for (int piece = 0; piece < 4; ++piece)
	{
		uint32_t area = sink_begin(k);
#pragma unroll
		for (int v = 0; v < 8; ++v)
		{
			const int c = piece * 32 + v * 4;
			sink_put(k, area, v, f(acc[c], c), f(acc[c + 1], c + 1), f(acc[c + 2], c + 2), f(acc[c + 3], c + 3));
		}
		sink_end(k, area, k.mapC, piece);
		if (k.mapClo)
		{
			area = sink_begin(k);
#pragma unroll
			for (int v = 0; v < 8; ++v)
			{
				const int c = piece * 32 + v * 4;
				sink_put(k, area, v, tf32_lo(f(acc[c], c)), tf32_lo(f(acc[c + 1], c + 1)), tf32_lo(f(acc[c + 2], c + 2)),
				         tf32_lo(f(acc[c + 3], c + 3)));
			}
			sink_end(k, area, k.mapClo, piece);
		}
	}
}

// The fused layer epilogue of one thread's row: bias + activation (forward), times the activation
// derivative (error propagation), times the learning rate (+ decay column term) for the weight
// gradient, or a plain copy.
__device__ __forceinline__ void apply_epilogue(const float (&acc)[128], const RowSink& out, const TcParams& p, int row, int col0)
{
	// The element-wise part is chosen ONCE per tile: the store loop is fully unrolled (the
	// accumulators must stay in registers), so a per-element switch over the activation ids would
	// replicate the transcendental code 128 times and thrash the instruction cache.
	if (p.epi == EPI_FORWARD)
	{
		const float bias = p.bias_ptr ? *p.bias_ptr : 0.0f;
		const float par = p.par;
		switch (p.act)
		{
		case GL_ACT_RELU:
			if (p.relu_mask_out)
			{
				// one bit per output: what the error propagation needs of this layer's activations
				unsigned wds[4] = {0u, 0u, 0u, 0u};
#pragma unroll
				for (int c = 0; c < 128; ++c)
					if (!(acc[c] + bias < GL_OUTLIER)) wds[c >> 5] |= 1u << (c & 31);
				*reinterpret_cast<uint4*>(p.relu_mask_out + (long long)row * p.mask_ld + (col0 >> 5)) =
				    make_uint4(wds[0], wds[1], wds[2], wds[3]);
			}
			store_row(acc, out, [=](float z, int) { z += bias; return z < GL_OUTLIER ? 0.0f : z; });
			break;
		case GL_ACT_LEAKY:
			store_row(acc, out, [=](float z, int) { z += bias; return z < GL_OUTLIER ? par * z : z; });
			break;
		case GL_ACT_LINEAR:
			store_row(acc, out, [=](float z, int) { return par * (z + bias); });
			break;
		case GL_ACT_SOFTMAX:
			store_row(acc, out, [=](float z, int) { return z + bias; });
			break;
		case GL_ACT_TANH:
			store_row(acc, out, [=](float z, int) { return tanhf(z + bias); });
			break;
		case GL_ACT_SIGMOID:
			store_row(acc, out, [=](float z, int) { return 1.0f / (1.0f + expf(-(z + bias))); });
			break;
		default:
		{
			const int act = p.act;
			store_row(acc, out, [=](float z, int) { return squash_b(z + bias, act, par); });
			break;
		}
		}
	}
	else if (p.epi == EPI_ERRPROP && p.act == GL_ACT_RELU && p.relu_mask_in)
	{
		const uint4 mk = *reinterpret_cast<const uint4*>(p.relu_mask_in + (long long)row * p.mask_ld + (col0 >> 5));
		const unsigned wds[4] = {mk.x, mk.y, mk.z, mk.w};
		store_row(acc, out, [=](float e, int c) { return ((wds[c >> 5] >> (c & 31)) & 1u) ? e : 0.0f; });
	}
	else if (p.epi == EPI_ERRPROP)
	{
		const float* auxrow = p.aux + (long long)row * p.ld_aux + col0;
		const float par = p.par;
		switch (p.act)
		{
		case GL_ACT_RELU:
			store_row(acc, out, [=](float e, int c) { return auxrow[c] > 0.0f ? e : 0.0f; });
			break;
		case GL_ACT_TANH:
		case GL_ACT_TANHP:
			store_row(acc, out, [=](float e, int c) { const float a = auxrow[c]; return e * (1.0f - a * a); });
			break;
		case GL_ACT_SIGMOID:
		case GL_ACT_SIGMOIDP:
			store_row(acc, out, [=](float e, int c) { const float a = auxrow[c]; return e * (a * (1.0f - a)); });
			break;
		default:
		{
			const int act = p.act;
			store_row(acc, out, [=](float e, int c) { return e * act_der_b(auxrow[c], act, par); });
			break;
		}
		}
	}
	else if (p.epi == EPI_GRAD)
	{
		const float alpha = p.alpha;
		if (p.colterm)
		{
			const float* ct = p.colterm + col0;
			store_row(acc, out, [=](float g, int c) { return alpha * g + ct[c]; });
		}
		else
			store_row(acc, out, [=](float g, int) { return alpha * g; });
	}
	else
		store_row(acc, out, [](float v, int) { return v; });
}

// k-block depth of the one-CTA tile variant in use (16 default, GLADES_TC_BK=32 for comparison runs)
int tc_bk();
// CTA-pair variant (gemm_tcgen05_pair.cu): maps = {A, A_lo, B, B_lo, C, C_lo}, A and B boxes 128 rows
bool tc_pair_supported(const GemmArgs& g);
cudaError_t launch_gemm_tc_pair(const CUtensorMap maps[6], const TcParams& p, int M, int N, int sm_reserve, cudaStream_t s);

}  // namespace tc
}  // namespace glb
