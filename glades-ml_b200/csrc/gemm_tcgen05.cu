// Batched-mode matrix product on the 5th-generation tensor cores (sm_100a): TMA-fed tcgen05.mma
// kind::tf32 with an fp32 accumulator in tensor memory, made fp32-faithful by the 3xTF32 split
//     A*B  ~=  A_hi*B_lo + A_lo*B_hi + A_hi*B_hi,      X_hi = trunc_tf32(X),  X_lo = tf32(X - X_hi).
// The tensor core reads only the upper 19 bits of an fp32 operand word, so the unmodified fp32
// matrix serves as X_hi and only the X_lo matrices are materialised (launch_split_lo).
//
// One CTA computes one 128 x BN tile of C (BN = 256 or 128):
//   warp 0, one lane   TMA producer: per 32-deep k-block, four tiled bulk copies (A, A_lo, B, B_lo)
//                      into a 128-byte-swizzled shared-memory stage, completion on an mbarrier;
//   warp 1             allocates 2*BN tensor-memory columns (two accumulators); one lane issues 3
//                      MMAs per 8-deep k-step (12 per stage) and commits the stage's "empty" barrier;
//   warps 2..          epilogue, one warp per (32-lane quarter, 128-column half): drains every
//                      finished 128-deep chunk of the accumulation into fp32 registers, then applies
//                      the fused layer epilogue (bias + activation, or times activation derivative,
//                      or times learning rate) and writes 16-byte global stores.
// Both operand layouts of the layer products are consumed as they lie in memory: K-contiguous
// rows (forward: activations and weights) through K-major descriptors, and M/N-contiguous rows
// (error propagation reads W_l as [k][n]; the weight gradient reads deltas and activations as
// [batch][node]) through MN-major descriptors, so no transposed copies exist.
// Every wait on an mbarrier is bounded: when it runs out the kernel raises *err_flag, leaves its
// loops, waits (bounded) for the copies it still has in flight, frees its tensor memory and returns.
#include <atomic>

#include "tc_device.cuh"

namespace glb {
using namespace tc;
namespace {

// launches per tile variant since the library was loaded (diagnostics for the tests: which instantiation
// a shape ran on): [0] 128-wide tiles, [1] 256-wide tiles, [2] launches whose CTAs walked more than one
// tile each, [3] launches of the data-parallel variant that stores into the owners' memory, [4] launches
// that split their last wave of tiles along k
std::atomic<long long> g_variant_counts[5];

// BK = fp32 elements per k-block: 32 (128-byte rows, 128-byte swizzle) or 16 (64-byte rows, 64-byte
// swizzle).  The shallower block with twice the stages keeps more bytes in flight for the same
// shared memory, which is what bounds this kernel (operand bytes per flop are 4x those of a bf16 GEMM).
template <int BN, int BK, int STAGES, int SBUF = 1>
struct TcSmem
{
	static constexpr int A_BYTES = TC_BM * BK * 4;
	static constexpr int B_BYTES = BN * BK * 4;
	static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
	static constexpr int TILES_BYTES = STAGES * STAGE_BYTES;
	static constexpr int EPI_WARPS = 4 * (BN / 128);  // one warp per (lane quarter, 128-column half)
	static constexpr int STAGING_BYTES = EPI_WARPS * 4096 * SBUF;  // per epilogue warp: SBUF areas of 32 rows x 32 columns of C
	static constexpr int TOTAL = TILES_BYTES + STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
	static constexpr int THREADS = 64 + 32 * EPI_WARPS;
};

// The tensor core adds into its fp32 accumulator with truncation, not round-to-nearest: a chain of n
// accumulations drifts by up to n * 2^-24 of the running sum, always towards zero (measured: -8e-5
// relative at K = 4096 on all-positive operands).  So the accumulator in tensor memory only ever
// holds TC_CHUNK_K = 128 k (48 accumulations); the epilogue warps drain each finished
// chunk into fp32 registers with round-to-nearest adds while the MMA warp fills the other of two
// tensor-memory accumulators.

// PEER: the data-parallel weight-gradient variant, whose epilogue (learning rate, decay term) stores
// each tile into the memory of the rank that owns its row band; a separate instantiation so that the
// register allocation of the plain kernel stays as it was tuned.
template <int BN, int BK, int STAGES, int SBUF, bool PEER>
__global__ void __launch_bounds__(TcSmem<BN, BK, STAGES, SBUF>::THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapAlo,
                   const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapBlo,
                   const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapClo, const TcParams p,
                   const TcPeer peer)
{
	using S = TcSmem<BN, BK, STAGES, SBUF>;
	constexpr int TC_BK = BK;
	constexpr int TC_CHUNK_KB = TC_CHUNK_K / BK;
	extern __shared__ uint8_t smem_raw[];
	// the swizzled tiles need a 1024-byte aligned base
	const uint32_t raw = smem_u32(smem_raw);
	const uint32_t base = (raw + 1023u) & ~1023u;
	uint8_t* gen_base = smem_raw + (base - raw);
	const uint32_t staging0 = base + S::TILES_BYTES;  // 1024-byte aligned, as the swizzled stores need
	uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + S::TILES_BYTES + S::STAGING_BYTES);
	const uint32_t bar0 = base + S::TILES_BYTES + S::STAGING_BYTES;
	// barrier slots: full[s] = s, empty[s] = STAGES + s, acc_full[b] = 2*STAGES + b, acc_empty[b] = 2*STAGES + 2 + b
	constexpr int NBARS = 2 * STAGES + 4;
	const uint32_t bar_acc_full = bar0 + 8 * (2 * STAGES);
	const uint32_t bar_acc_empty = bar0 + 8 * (2 * STAGES + 2);
	uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
	volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

	const int warp = threadIdx.x >> 5;
	const int lane = threadIdx.x & 31;
	const int KB = p.K / TC_BK;
	// Persistent CTAs: tile t of this CTA is blockIdx.x + i * gridDim.x.  Tiles are numbered m-fastest
	// inside bands of TC_BAND m-tiles, so that the CTAs running at one time share a band of A rows
	// and a few B column blocks in L2.  All three roles walk the same sequence; the stage and
	// accumulator barriers simply keep counting across tiles, which lets the producer and the MMA lane
	// run ahead into the next tile while the epilogue warps still store the previous one.
	const int total_tiles = p.tiles_m * p.tiles_n;
	constexpr int TC_BAND = 16;
	auto tile_origin = [&](int t, int& m0, int& n0) {
		if (PEER)
		{
			// Data-parallel weight gradient: the tiles are walked owner band by owner band, m-fastest inside a
			// band, and every rank starts with the band of the rank after it.  At any moment the ranks of the
			// group therefore store into different owners, so no owner's NVLink ingress carries more than one
			// sender's stream (all ranks walking the bands in the same order would aim all their stores at the same
			// owner at once).  This rank's own band comes last: its stores are local.
			const int band_mt = peer.band_rows / TC_BM;
			const int nbands = (p.tiles_m + band_mt - 1) / band_mt;
			int left = t;
			for (int s = 0; s < nbands; ++s)
			{
				const int band = (peer.self + 1 + s) % nbands;
				const int mt_in = min(band_mt, p.tiles_m - band * band_mt);
				const int cnt = mt_in * p.tiles_n;
				if (left < cnt)
				{
					m0 = (band * band_mt + left % mt_in) * TC_BM;
					n0 = (left / mt_in) * BN;
					return;
				}
				left -= cnt;
			}
			m0 = 0;  // not reached: t < tiles_m * tiles_n
			n0 = 0;
			return;
		}
		const int band_tiles = TC_BAND * p.tiles_n;
		const int band = t / band_tiles;
		const int in_band = t - band * band_tiles;
		const int band_m = min(TC_BAND, p.tiles_m - band * TC_BAND);
		const int mt = band * TC_BAND + in_band % band_m;
		const int nt = in_band / band_m;
		m0 = mt * TC_BM;
		n0 = nt * BN;
	};

	if (threadIdx.x == 0)
	{
		for (int s = 0; s < STAGES; ++s)
		{
			mbar_init(bar0 + 8 * s, 1);
			mbar_init(bar0 + 8 * (STAGES + s), 1);
		}
		for (int b = 0; b < 2; ++b)
		{
			mbar_init(bar_acc_full + 8 * b, 1);
			mbar_init(bar_acc_empty + 8 * b, S::EPI_WARPS);
		}
		*abort_flag = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 1)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
		             "r"(2 * BN)
		             : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = *tmem_slot;

	if (warp == 0 && lane == 0)
	{
		// ------------------------------------------------ TMA producer
		int issued = 0;
		int it = 0;  // k-blocks issued so far, over all work items
		bool ok = true;
		TcWork work(blockIdx.x, gridDim.x, KB, total_tiles, p.sk_work ? p.sk_full_tiles : total_tiles);
		int t, kb0, kb1;
		while (ok && work.next(t, kb0, kb1))
		{
		int m0, n0;
		tile_origin(t, m0, n0);
		for (int kb = kb0; kb < kb1; ++kb, ++it)
		{
			const int s = it % STAGES;
			const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
			if (!mbar_wait(bar0 + 8 * (STAGES + s), ph ^ 1u, abort_flag, p.err_flag, 1))
			{
				ok = false;
				break;
			}
			const uint32_t full = bar0 + 8 * s;
			mbar_expect_tx(full, S::STAGE_BYTES);
			const uint32_t sa = base + s * S::STAGE_BYTES;
			const uint32_t sal = sa + S::A_BYTES;
			const uint32_t sb = sal + S::A_BYTES;
			const uint32_t sbl = sb + S::B_BYTES;
			const int k0 = kb * TC_BK;
			if (p.a_mn)
			{
				tma_load_3d(sa, &mapA, full, 0, k0, m0 / 32);
				tma_load_3d(sal, &mapAlo, full, 0, k0, m0 / 32);
			}
			else
			{
				tma_load_2d(sa, &mapA, full, k0, m0);
				tma_load_2d(sal, &mapAlo, full, k0, m0);
			}
			if (p.b_mn)
			{
				tma_load_3d(sb, &mapB, full, 0, k0, n0 / 32);
				tma_load_3d(sbl, &mapBlo, full, 0, k0, n0 / 32);
			}
			else
			{
				tma_load_2d(sb, &mapB, full, k0, n0);
				tma_load_2d(sbl, &mapBlo, full, k0, n0);
			}
			issued = it + 1;
		}
		}
		if (*abort_flag)
		{
			// give copies that are still in flight a bounded time to land before the CTA ends
			const int lo = issued > STAGES ? issued - STAGES : 0;
			for (int kb = lo; kb < issued; ++kb)
			{
				const long long t0 = clock64();
				while (!mbar_try(bar0 + 8 * (kb % STAGES), (uint32_t)(kb / STAGES) & 1u) && clock64() - t0 < TC_WAIT_CYCLES) {}
			}
		}
	}
	else if (warp == 1 && lane == 0)
	{
		// ------------------------------------------------ MMA issuer
		const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
		                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
		// K-major: rows of 128 bytes, 8-row groups 1024 bytes apart; a k-step is 32 bytes along the row.
		// MN-major: 32-element (128-byte) runs, one k per 128-byte row, swizzle atoms of 4 k-rows
		// (512 bytes apart), so a k-step of 8 is 1024 bytes; the next 32-element chunk of M/N lies a
		// whole 32x32 box (4096 bytes) further.
		// With 16-deep blocks the K-major rows are 64 bytes (64-byte swizzle, layout type 4, 8-row groups
		// 512 bytes apart) and an MN-major 32-element chunk is a 32x16 box (2048 bytes).
		constexpr uint32_t K_SBO = (BK == 32) ? 1024u : 512u, K_LT = (BK == 32) ? 2u : 4u, MN_LBO = 128u * BK;
		const uint32_t a_lbo = p.a_mn ? MN_LBO : 0u, a_sbo = p.a_mn ? 512u : K_SBO, a_kstep = p.a_mn ? 1024u : 32u;
		const uint32_t b_lbo = p.b_mn ? MN_LBO : 0u, b_sbo = p.b_mn ? 512u : K_SBO, b_kstep = p.b_mn ? 1024u : 32u;
		const uint32_t a_lt = p.a_mn ? 1u : K_LT, b_lt = p.b_mn ? 1u : K_LT;
		bool ok = true;
		int it = 0;  // k-blocks consumed so far, over all work items
		int gc = 0;  // accumulator chunks started so far, over all work items
		TcWork work(blockIdx.x, gridDim.x, KB, total_tiles, p.sk_work ? p.sk_full_tiles : total_tiles);
		int t, kb0, kb1;
		while (ok && work.next(t, kb0, kb1))
		for (int kb = kb0; kb < kb1 && ok; ++kb, ++it)
		{
			const int s = it % STAGES;
			const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
			const int kin = (kb - kb0) % TC_CHUNK_KB;  // chunks count from the item's first k-block
			const int chunk = gc;
			const int buf = chunk & 1;
			const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
			if (kin == 0)
			{
				// this accumulator must have been drained by the epilogue (two chunks ago)
				const uint32_t use = (uint32_t)(chunk >> 1);
				if (!mbar_wait(bar_acc_empty + 8 * buf, (use & 1u) ^ 1u, abort_flag, p.err_flag, 4))
				{
					ok = false;
					break;
				}
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			}
			if (!mbar_wait(bar0 + 8 * s, ph, abort_flag, p.err_flag, 2))
			{
				ok = false;
				break;
			}
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			const uint32_t sa = base + s * S::STAGE_BYTES;
			const uint32_t sal = sa + S::A_BYTES;
			const uint32_t sb = sal + S::A_BYTES;
			const uint32_t sbl = sb + S::B_BYTES;
#pragma unroll
			for (int j = 0; j < TC_BK / 8; ++j)
			{
				const uint64_t dA = make_smem_desc(sa + j * a_kstep, a_lbo, a_sbo, a_lt);
				const uint64_t dAl = make_smem_desc(sal + j * a_kstep, a_lbo, a_sbo, a_lt);
				const uint64_t dB = make_smem_desc(sb + j * b_kstep, b_lbo, b_sbo, b_lt);
				const uint64_t dBl = make_smem_desc(sbl + j * b_kstep, b_lbo, b_sbo, b_lt);
				umma_tf32(tmem_d, dA, dBl, idesc, (kin | j) != 0 ? 1u : 0u);
				umma_tf32(tmem_d, dAl, dB, idesc, 1u);
				umma_tf32(tmem_d, dA, dB, idesc, 1u);
			}
			umma_commit(bar0 + 8 * (STAGES + s));  // frees the stage once these MMAs have read it
			if (kin == TC_CHUNK_KB - 1 || kb == kb1 - 1)
			{
				umma_commit(bar_acc_full + 8 * buf);  // chunk complete
				++gc;
			}
		}
	}
	else if (warp >= 2)
	{
		// ------------------------------------------------ epilogue: drain chunks, then the layer epilogue
		const int q = warp & 3;          // the tensor-memory lane quarter this warp may read
		const int half = (warp - 2) >> 2;  // which 128 columns of the tile
		bool ok = true;
		int piece_turn = 0;
		int gc = 0;  // accumulator chunks drained so far, over all work items
		TcWork work(blockIdx.x, gridDim.x, KB, total_tiles, p.sk_work ? p.sk_full_tiles : total_tiles);
		int t, kb0, kb1;
		while (ok && work.next(t, kb0, kb1))
		{
		int m0, n0;
		tile_origin(t, m0, n0);
		const int nchunk = (kb1 - kb0 + TC_CHUNK_KB - 1) / TC_CHUNK_KB;
		float acc[128];
#pragma unroll
		for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
		for (int c_in = 0; c_in < nchunk && ok; ++c_in, ++gc)
		{
			const int buf = gc & 1;
			const uint32_t use = (uint32_t)(gc >> 1);
			if (!mbar_wait(bar_acc_full + 8 * buf, use & 1u, abort_flag, p.err_flag, 3))
			{
				ok = false;
				break;
			}
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * 128);
#pragma unroll
			for (int c = 0; c < 4; ++c)
			{
				uint32_t r[32];
				tmem_ld32(taddr + (uint32_t)(c * 32), r);
				asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
				for (int e = 0; e < 32; ++e) acc[c * 32 + e] += __uint_as_float(r[e]);
			}
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
			__syncwarp();
			if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty + 8 * buf) : "memory");
		}
		if (ok && kb0 != 0)
		{
			// a partial: the tile's finisher (an earlier CTA) adds it.  Layout of this warp's 32 x 128 block in the
			// CTA's workspace slot: 32 pieces of 512 bytes, piece v = columns 4v..4v+3 of the 32 rows (one float4
			// per lane), so every store instruction of the warp writes 512 contiguous bytes.
			float4* ws = reinterpret_cast<float4*>(p.sk_work + (size_t)blockIdx.x * (TC_BM * BN) + (size_t)(warp - 2) * 4096);
#pragma unroll
			for (int v = 0; v < 32; ++v) ws[v * 32 + lane] = make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
			__threadfence();
			__syncwarp();
			if (lane == 0)
				asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + (size_t)blockIdx.x * 8 + (warp - 2)), "r"(p.sk_epoch) : "memory");
			continue;
		}
		if (ok && kb1 != KB)
		{
			// the tile's finisher: the rest of the tile's k-blocks were computed by the next CTAs as their first
			// items; add their partials in CTA order
			const int tile_end = (t - work.full + 1) * KB;
			for (int j = blockIdx.x + 1; j < (int)gridDim.x && work.share_begin(j) < tile_end && ok; ++j)
			{
				if (work.share_begin(j + 1) <= work.share_begin(j)) continue;  // an empty share
				const unsigned* flag = p.sk_flags + (size_t)j * 8 + (warp - 2);
				unsigned seen;
				const long long t0 = clock64();
				for (;;)
				{
					asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
					if (seen == p.sk_epoch) break;
					if (*abort_flag || clock64() - t0 > TC_WAIT_CYCLES)
					{
						*abort_flag = 1;
						atomicExch(p.err_flag, 5);
						ok = false;
						break;
					}
				}
				if (!ok) break;
				const float4* ws = reinterpret_cast<const float4*>(p.sk_work + (size_t)j * (TC_BM * BN) + (size_t)(warp - 2) * 4096);
#pragma unroll
				for (int v = 0; v < 32; ++v)
				{
					const float4 w4 = __ldcg(ws + v * 32 + lane);
					acc[4 * v] += w4.x;
					acc[4 * v + 1] += w4.y;
					acc[4 * v + 2] += w4.z;
					acc[4 * v + 3] += w4.w;
				}
			}
		}
		if (ok && !(p.debug & 1))
		{
			const int row = m0 + q * 32 + lane;
			const int col0 = n0 + half * 128;
			RowSink out;
			out.crow = p.C + (long long)row * p.ldc + col0;
			out.lorow = p.C_lo ? p.C_lo + (long long)row * p.ldc + col0 : nullptr;
			out.stage = staging0 + (uint32_t)(warp - 2) * (4096u * SBUF);
			out.nbuf = SBUF;
			out.turn = &piece_turn;
			out.mapC = &mapC;
			out.mapClo = p.C_lo ? &mapClo : nullptr;
			out.col0 = col0;
			out.row0 = m0 + q * 32;
			out.lane = lane;
			out.direct = (p.debug & 2) != 0;
			if (PEER)
			{
				// the tile's rows lie inside one owner's band (bands are whole tiles): store them there
				const int owner = m0 / peer.band_rows;
				out.mapC = peer.maps + owner;
				out.row0 = m0 - owner * peer.band_rows + q * 32;
				if (out.direct) out.crow = peer.bases[owner] + (long long)(out.row0 + lane) * p.ldc + col0;
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
				apply_epilogue(acc, out, p, row, col0);
		}
		}
		// every bulk store of this warp must have completed before the CTA may exit
		if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 1)
	{
		asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
	}
}

// ---- host side: tensor maps ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
	static EncodeTiledFn fn = nullptr;
	if (!fn)
	{
		void* p = nullptr;
		cudaDriverEntryPointQueryResult qr;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
		    qr == cudaDriverEntryPointSuccess)
			fn = (EncodeTiledFn)p;
	}
	return fn;
}

// Operand X(r, k), r in [0, R): mn == 0: X[r*ld + k] (K-contiguous), box = 32 k x box_r rows;
// mn == 1: X[k*ld + r] (row-contiguous in r), viewed as [r/32][k][r%32], box = 32 x 32 k x box_r/32.
bool make_map(CUtensorMap* m, const float* ptr, int mn, long long R, long long K, long long ld, int box_r, int bk)
{
	EncodeTiledFn fn = encode_fn();
	if (!fn) return false;
	CUresult r;
	if (!mn)
	{
		cuuint64_t dim[2] = {(cuuint64_t)K, (cuuint64_t)R};
		cuuint64_t str[1] = {(cuuint64_t)ld * 4};
		cuuint32_t box[2] = {(cuuint32_t)bk, (cuuint32_t)box_r};
		cuuint32_t es[2] = {1, 1};
		r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)ptr, dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
		       bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
		       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	}
	else
	{
		cuuint64_t dim[3] = {32, (cuuint64_t)K, (cuuint64_t)(R / 32)};
		cuuint64_t str[2] = {(cuuint64_t)ld * 4, 128};
		cuuint32_t box[3] = {32, (cuuint32_t)bk, (cuuint32_t)(box_r / 32)};
		cuuint32_t es[3] = {1, 1, 1};
		r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)ptr, dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
		       CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	}
	return r == CUDA_SUCCESS;
}

template <int BN, int BK, int STAGES, int SBUF, bool PEER = false>
cudaError_t launch_cfg(const CUtensorMap& mA, const CUtensorMap& mAl, const CUtensorMap& mB, const CUtensorMap& mBl,
                       const CUtensorMap& mC, const CUtensorMap& mCl, const TcParams& p, int M, int N, int sm_reserve,
                       cudaStream_t s, const TcPeer& peer = TcPeer(), const TcSplitK* sk = nullptr)
{
	using S = TcSmem<BN, BK, STAGES, SBUF>;
	// the shared-memory opt-in and the SM count belong to a device, not to the process
	constexpr int kMaxDev = 64;
	static bool attr_set[kMaxDev] = {};
	static int sm_counts[kMaxDev] = {};
	int dev = 0;
	if (cudaError_t e = cudaGetDevice(&dev)) return e;
	const int slot = (dev >= 0 && dev < kMaxDev) ? dev : -1;
	if (slot < 0 || !attr_set[slot])
	{
		cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, BK, STAGES, SBUF, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
		if (e != cudaSuccess) return e;
		if (slot >= 0) attr_set[slot] = true;
	}
	TcParams q = p;
	q.tiles_m = M / TC_BM;
	q.tiles_n = N / BN;
	int sm_count = slot >= 0 ? sm_counts[slot] : 0;
	if (!sm_count)
	{
		if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count < 1) sm_count = 148;
		if (slot >= 0) sm_counts[slot] = sm_count;
	}
	const int total = q.tiles_m * q.tiles_n;
	int avail = sm_count - sm_reserve;
	if (avail < 1) avail = 1;
	int grid = total < avail ? total : avail;
	// Split the last, partial wave of tiles along k over all CTAs where that wave would leave a quarter or more of
	// the SMs idle (32 tiles of a narrow layer; 68 tiles after three whole waves) and the caller gave a workspace.
	// Not below that: CTAs that share a tile's operands then sit at different k offsets, the operands stop being
	// fetched once and shared through L2, and 128 tiles on 148 SMs measured 17-30 % slower split than whole.
	// The data-parallel variant (epilogue stores into peers' memory) is never split: with the SMs it leaves to the
	// exchange its tile counts are whole waves, and the combination has no parity test.
	q.sk_full_tiles = total;
	const int KB = p.K / BK;
	if (q.sk_work && sk && KB >= 8 && !PEER)
	{
		const int g2 = avail;
		const int full = (total / g2) * g2;
		const int rem = total - full;
		if (rem > 0 && (g2 - rem) * 100 >= g2 * sk->min_idle_pct && (long long)rem * KB >= 4ll * g2 && (size_t)g2 <= sk->slots &&
		    (long long)(g2 + 1) * rem * KB < (1ll << 31))
		{
			grid = g2;
			q.sk_full_tiles = full;
			q.sk_epoch = ++*sk->epoch;
		}
	}
	if (q.sk_full_tiles == total) q.sk_work = nullptr;
	g_variant_counts[BN == 256 ? 1 : 0].fetch_add(1, std::memory_order_relaxed);
	if (total > grid) g_variant_counts[2].fetch_add(1, std::memory_order_relaxed);
	if (PEER) g_variant_counts[3].fetch_add(1, std::memory_order_relaxed);
	if (q.sk_work) g_variant_counts[4].fetch_add(1, std::memory_order_relaxed);
	gemm_tc_kernel<BN, BK, STAGES, SBUF, PEER><<<grid, S::THREADS, S::TOTAL, s>>>(mA, mAl, mB, mBl, mC, mCl, q, peer);
	return cudaGetLastError();
}

__global__ void __launch_bounds__(256) split_lo_kernel(const float4* __restrict__ src, float4* __restrict__ lo, long long n4)
{
	const long long stride = (long long)gridDim.x * blockDim.x;
	for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
	{
		const float4 a = src[i];
		const float v[4] = {a.x, a.y, a.z, a.w};
		const float o[4] = {tf32_lo(v[0]), tf32_lo(v[1]), tf32_lo(v[2]), tf32_lo(v[3])};
		lo[i] = make_float4(o[0], o[1], o[2], o[3]);
	}
}

// dst = src and lo = the low TF32 parts of src, in one pass (lo may be NULL)
__global__ void __launch_bounds__(256) copy_split_lo_kernel(const float4* __restrict__ src, float4* __restrict__ dst, float4* __restrict__ lo,
                                                             long long n4)
{
	const long long stride = (long long)gridDim.x * blockDim.x;
	for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
	{
		const float4 a = __ldcg(src + i);
		dst[i] = a;
		if (lo) lo[i] = make_float4(tf32_lo(a.x), tf32_lo(a.y), tf32_lo(a.z), tf32_lo(a.w));
	}
}

__global__ void __launch_bounds__(256) scale_split_lo_kernel(const float* __restrict__ src, const float* __restrict__ rowscale,
                                                              int ld, float* __restrict__ dst, float* __restrict__ lo,
                                                              long long n)
{
	const long long stride = (long long)gridDim.x * blockDim.x;
	for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
	{
		const float v = src[i] * rowscale[i / ld];
		dst[i] = v;
		lo[i] = tf32_lo(v);
	}
}

}  // namespace

int tc_splitk_min_idle_pct()
{
	const char* e = getenv("GLADES_TC_SPLITK_IDLE");
	const int v = e ? atoi(e) : 25;
	return v < 1 ? 1 : (v > 100 ? 100 : v);
}
void tc_variant_counts(long long out5[5])
{
	for (int i = 0; i < 5; ++i) out5[i] = g_variant_counts[i].load(std::memory_order_relaxed);
}

bool tc_make_store_map(void* out128, const float* base, long long rows, long long cols, long long ld)
{
	return make_map(reinterpret_cast<CUtensorMap*>(out128), base, 0, rows, cols, ld, 32, 32);
}

bool tc_make_map2d(void* out128, const float* base, long long rows, long long cols, long long ld, int box_cols, int box_rows,
                   int swizzle128)
{
	EncodeTiledFn fn = encode_fn();
	if (!fn) return false;
	cuuint64_t dim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
	cuuint64_t str[1] = {(cuuint64_t)ld * 4};
	cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
	cuuint32_t es[2] = {1, 1};
	return fn(reinterpret_cast<CUtensorMap*>(out128), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dim, str, box, es,
	          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
	          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// k-block depth of the tile variant in use: 16 (default) or 32 (GLADES_TC_BK=32, kept for comparison)
int tc::tc_bk()
{
	static int bk_choice = 0;
	if (!bk_choice)
	{
		const char* e = getenv("GLADES_TC_BK");
		bk_choice = (e && atoi(e) == 32) ? 32 : 16;
	}
	return bk_choice;
}

bool tc_gemm_supported(const GemmArgs& g)
{
	const int TC_KALIGN = tc_bk();
	if (g.M < TC_BM || g.N < 128 || g.K < TC_KALIGN) return false;
	if (g.M % TC_BM || g.N % 128 || g.K % TC_KALIGN) return false;
	if (g.kscale) return false;
	const bool a_k = (g.a_sk == 1), a_mn = (g.a_sm == 1);
	const bool b_k = (g.b_sk == 1), b_mn = (g.b_sn == 1);
	if (!(a_k || a_mn) || !(b_k || b_mn)) return false;
	const long long lda = a_k ? g.a_sm : g.a_sk, ldb = b_k ? g.b_sn : g.b_sk;
	if (lda % 4 || ldb % 4 || g.ldc % 4) return false;
	if (((uintptr_t)g.A | (uintptr_t)g.B | (uintptr_t)g.C) & 15) return false;
	if (g.epi == EPI_ERRPROP && (!g.aux || (g.ld_aux % 4) || ((uintptr_t)g.aux & 15))) return false;
	return encode_fn() != nullptr;
}

cudaError_t launch_gemm_tc(const GemmArgs& g, const float* A_lo, const float* B_lo, int* err_flag, cudaStream_t s)
{
	if (!tc_gemm_supported(g) || !A_lo || !B_lo) return cudaErrorInvalidValue;
	// a K-contiguous operand with a single row (ld == 1 on both strides) is read as K-major
	const int a_mn = (g.a_sk == 1) ? 0 : 1;
	const int b_mn = (g.b_sk == 1) ? 0 : 1;
	const long long lda = a_mn ? g.a_sk : g.a_sm, ldb = b_mn ? g.b_sk : g.b_sn;
	// 256-wide tiles unless they would leave more than half of the SMs without a tile
	const bool pair = !g.peer_maps && tc_pair_supported(g);
	const long long wide_tiles = (long long)(g.M / TC_BM) * (g.N / 256);
	// (with a split-k workspace a few wide tiles still fill the GPU: their k-blocks are dealt out over all CTAs)
	const bool can_split = g.sk && g.sk->work && g.K / tc_bk() >= 8;
	const int BN = (g.N % 256 == 0 && (pair || wide_tiles >= 74 || (can_split && wide_tiles >= 16))) ? 256 : 128;
	// tile variant: 16-deep k-blocks with twice the stages by default; GLADES_TC_BK=32 selects the
	// 32-deep blocks (kept for comparison runs)
	const int bk = tc_bk();
	const int box_b = pair ? 128 : BN;  // a CTA of a pair loads half of the 256-wide B tile
	CUtensorMap mA, mAl, mB, mBl;
	if (!make_map(&mA, g.A, a_mn, g.M, g.K, lda, TC_BM, bk) || !make_map(&mAl, A_lo, a_mn, g.M, g.K, lda, TC_BM, bk) ||
	    !make_map(&mB, g.B, b_mn, g.N, g.K, ldb, box_b, bk) || !make_map(&mBl, B_lo, b_mn, g.N, g.K, ldb, box_b, bk))
		return cudaErrorInvalidValue;
	// C (and its low-part matrix) as [M][N] row-major with 32 x 32 boxes for the epilogue's bulk stores
	CUtensorMap mC, mCl;
	if (!make_map(&mC, g.C, 0, g.M, g.N, g.ldc, 32, 32)) return cudaErrorInvalidValue;
	mCl = mC;
	if (g.C_lo && !make_map(&mCl, g.C_lo, 0, g.M, g.N, g.ldc, 32, 32)) return cudaErrorInvalidValue;
	TcParams p;
	p.C = g.C;
	p.C_lo = g.C_lo;
	p.ldc = g.ldc;
	p.K = g.K;
	p.a_mn = a_mn;
	p.b_mn = b_mn;
	p.epi = g.epi;
	p.bias_ptr = g.bias_ptr;
	p.act = g.act;
	p.par = g.par;
	p.aux = g.aux;
	p.ld_aux = g.ld_aux;
	p.alpha = g.alpha;
	p.colterm = g.colterm;
	p.relu_mask_out = g.relu_mask_out;
	p.relu_mask_in = g.relu_mask_in;
	p.mask_ld = g.N / 32;
	p.err_flag = err_flag;
	p.sk_work = can_split ? g.sk->work : nullptr;
	p.sk_flags = can_split ? g.sk->flags : nullptr;
	p.sk_epoch = 0;
	p.sk_full_tiles = 0;
	const TcSplitK* sk = can_split ? g.sk : nullptr;
	TcPeer peer;
	peer.maps = reinterpret_cast<const CUtensorMap*>(g.peer_maps);
	peer.bases = g.peer_bases;
	peer.band_rows = g.band_rows;
	peer.self = g.peer_self;
	if (g.peer_maps && (g.band_rows < TC_BM || g.band_rows % TC_BM || g.C_lo)) return cudaErrorInvalidValue;
	{
		static int dbg = -1;
		if (dbg < 0)
		{
			const char* e = getenv("GLADES_TC_DEBUG");
			dbg = e ? atoi(e) : 0;
		}
		p.debug = dbg;
	}
	if (pair)
	{
		const CUtensorMap maps[6] = {mA, mAl, mB, mBl, mC, mCl};
		return launch_gemm_tc_pair(maps, p, g.M, g.N, g.sm_reserve, s);
	}
	if (g.peer_maps)
	{
		if (g.epi != EPI_GRAD) return cudaErrorInvalidValue;
		if (BN == 256) return launch_cfg<256, 16, 4, 1, true>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s, peer, sk);
		return launch_cfg<128, 16, 6, 2, true>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s, peer, sk);
	}
	if (bk == 32)
	{
		if (BN == 256) return launch_cfg<256, 32, 2, 1>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s);
		return launch_cfg<128, 32, 3, 1>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s);
	}
	if (BN == 256)
	{
		// GLADES_TC_STAGES=3: one pipeline stage fewer, two staging areas per epilogue warp
		static int st = 0;
		if (!st)
		{
			const char* e = getenv("GLADES_TC_STAGES");
			st = (e && atoi(e) == 3) ? 3 : 4;
		}
		if (st == 3) return launch_cfg<256, 16, 3, 2>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s);
		return launch_cfg<256, 16, 4, 1>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s, TcPeer(), sk);
	}
	return launch_cfg<128, 16, 6, 2>(mA, mAl, mB, mBl, mC, mCl, p, g.M, g.N, g.sm_reserve, s, TcPeer(), sk);
}

cudaError_t launch_split_lo(const float* src, float* lo, long long count, cudaStream_t s)
{
	if (count % 4 || (((uintptr_t)src | (uintptr_t)lo) & 15)) return cudaErrorInvalidValue;
	const long long n4 = count / 4;
	long long blocks = (n4 + 255) / 256;
	if (blocks > 148 * 8) blocks = 148 * 8;
	if (blocks < 1) blocks = 1;
	split_lo_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(lo), n4);
	return cudaGetLastError();
}

cudaError_t launch_copy_split_lo(const float* src, float* dst, float* lo, long long count, cudaStream_t s)
{
	if (count < 1) return cudaSuccess;
	if ((count & 3) || (((uintptr_t)src | (uintptr_t)dst | (uintptr_t)lo) & 15)) return cudaErrorInvalidValue;
	const long long n4 = count >> 2;
	long long blocks = (n4 + 255) / 256;
	if (blocks > 148 * 4) blocks = 148 * 4;
	copy_split_lo_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst),
	                                                     reinterpret_cast<float4*>(lo), n4);
	return cudaGetLastError();
}

cudaError_t launch_scale_split_lo(const float* src, const float* rowscale, int ld, float* dst_scaled, float* lo,
                                  long long count, cudaStream_t s)
{
	long long blocks = (count + 255) / 256;
	if (blocks > 148 * 8) blocks = 148 * 8;
	if (blocks < 1) blocks = 1;
	scale_split_lo_kernel<<<(unsigned)blocks, 256, 0, s>>>(src, rowscale, ld, dst_scaled, lo, count);
	return cudaGetLastError();
}

}  // namespace glb
