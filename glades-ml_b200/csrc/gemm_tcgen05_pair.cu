// CTA-pair variant of the tensor-core layer product: two CTAs of a cluster (two SMs) compute one
// 256 x 256 tile of C with tcgen05.mma.cta_group::2.
//
// Why: the one-CTA kernel is bound by the operand bytes it can keep in flight (3xTF32 on fp32 operands
// moves 4x the bytes per flop of a bf16 product).  In a pair each CTA holds its own 128 rows of A and
// only HALF of the B tile (128 of the 256 columns' rows); the tensor cores of both SMs read both
// halves.  Per 16-deep k-block a CTA therefore loads 32 KB instead of 48 KB for the same work per SM,
// and six pipeline stages fit where four did.
//
// Roles per CTA (320 threads):  warp 0 lane 0  TMA producer for this CTA's A rows and B half; the
// copies of BOTH CTAs complete on the LEADER's (cluster rank 0) "full" barrier, which expects the
// bytes of both.  warp 1: both CTAs allocate tensor memory together; only the leader's lane 0 issues
// the MMAs and commits, signalling the "empty" and "accumulator full" barriers of both CTAs.  warps
// 2..9: epilogue as in the one-CTA kernel (each CTA drains its own 128 x 256 accumulator chunks into
// fp32 registers and stores its rows through the staged bulk-store sink); "accumulator drained" is
// signalled on the leader's barrier by the epilogue warps of both CTAs.
// Loads are plain per-CTA tile copies.  Every wait is bounded, as in the one-CTA kernel.
#include <stdio.h>

#include "tc_device.cuh"

namespace glb {
using namespace tc;
namespace {

constexpr int P_BN = 256;   // tile columns
constexpr int P_BK = 16;    // k-block depth (64-byte K-major rows)
constexpr int P_STAGES = 6;
constexpr int P_HALF = 128;  // rows of A, and rows of the B half, per CTA
constexpr int P_A_BYTES = P_HALF * P_BK * 4;                 // 8 KB per part
constexpr int P_STAGE_BYTES = 4 * P_A_BYTES;                 // A, A_lo, B half, B_lo half = 32 KB
constexpr int P_TILES_BYTES = P_STAGES * P_STAGE_BYTES;      // 192 KB
constexpr int P_EPI_WARPS = 8;
constexpr int P_STAGING_BYTES = P_EPI_WARPS * 4096;
constexpr int P_THREADS = 64 + 32 * P_EPI_WARPS;
constexpr int P_TOTAL = P_TILES_BYTES + P_STAGING_BYTES + 1024 + 256;
constexpr int P_CHUNK_KB = TC_CHUNK_K / P_BK;

__device__ __forceinline__ uint32_t cluster_rank()
{
	uint32_t r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank)
{
	uint32_t r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
	return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_pair_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1)
{
	asm volatile(
	    "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
	    "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
	    : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2)
{
	asm volatile(
	    "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
	    "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
	    : "memory");
}
__device__ __forceinline__ void umma_pair_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "setp.ne.b32 p, %4, 0;\n\t"
	    "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}" ::"r"(tmem_d),
	    "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0)
	    : "memory");
}
// arrive on a barrier of either CTA of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_pair_commit(uint32_t bar_cluster)
{
	asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster)
{
	asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
    gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapAlo,
                        const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapBlo,
                        const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapClo, const TcParams p)
{
	extern __shared__ uint8_t smem_raw[];
	const uint32_t raw = smem_u32(smem_raw);
	const uint32_t base = (raw + 1023u) & ~1023u;
	uint8_t* gen_base = smem_raw + (base - raw);
	const uint32_t staging0 = base + P_TILES_BYTES;
	uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + P_TILES_BYTES + P_STAGING_BYTES);
	const uint32_t bar0 = base + P_TILES_BYTES + P_STAGING_BYTES;
	// barrier slots: full[s] = s, empty[s] = STAGES + s, acc_full[b] = 2*STAGES + b, acc_empty[b] = 2*STAGES + 2 + b
	constexpr int NBARS = 2 * P_STAGES + 4;
	const uint32_t bar_acc_full = bar0 + 8 * (2 * P_STAGES);
	const uint32_t bar_acc_empty = bar0 + 8 * (2 * P_STAGES + 2);
	uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
	volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

	const int warp = threadIdx.x >> 5;
	const int lane = threadIdx.x & 31;
	const uint32_t rank = cluster_rank();
	const bool leader = rank == 0;
	const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
	const int KB = p.K / P_BK;
	const int NCHUNK = (KB + P_CHUNK_KB - 1) / P_CHUNK_KB;
	const int total_tiles = p.tiles_m * p.tiles_n;  // 256 x 256 tiles
	constexpr int BAND = 8;
	auto tile_origin = [&](int t, int& m0, int& n0) {
		const int band_tiles = BAND * p.tiles_n;
		const int band = t / band_tiles;
		const int in_band = t - band * band_tiles;
		const int band_m = min(BAND, p.tiles_m - band * BAND);
		m0 = (band * BAND + in_band % band_m) * 256;
		n0 = (in_band / band_m) * P_BN;
	};

	if (threadIdx.x == 0)
	{
		for (int s = 0; s < P_STAGES; ++s)
		{
			mbar_init(bar0 + 8 * s, 1);
			mbar_init(bar0 + 8 * (P_STAGES + s), 1);
		}
		for (int b = 0; b < 2; ++b)
		{
			mbar_init(bar_acc_full + 8 * b, 1);
			mbar_init(bar_acc_empty + 8 * b, 2 * P_EPI_WARPS);  // the epilogue warps of both CTAs
		}
		*abort_flag = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 1)
	{
		asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * P_BN)
		             : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	cluster_sync_all();  // both CTAs' barriers exist before either touches the other's
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = *tmem_slot;

	if (warp == 0 && lane == 0)
	{
		// ------------------------------------------------ TMA producer (both CTAs)
		int it = 0;
		bool ok = true;
		for (int t = pair; t < total_tiles && ok; t += npairs)
		{
			int m0, n0;
			tile_origin(t, m0, n0);
			const int am0 = m0 + (int)rank * P_HALF;  // this CTA's rows of A
			const int bn0 = n0 + (int)rank * P_HALF;  // this CTA's half of the B tile
			for (int kb = 0; kb < KB; ++kb, ++it)
			{
				const int s = it % P_STAGES;
				const uint32_t ph = (uint32_t)(it / P_STAGES) & 1u;
				if (!mbar_wait(bar0 + 8 * (P_STAGES + s), ph ^ 1u, abort_flag, p.err_flag, 1))
				{
					ok = false;
					break;
				}
				const uint32_t full_local = bar0 + 8 * s;
				if (leader) mbar_expect_tx(full_local, 2 * P_STAGE_BYTES);  // the copies of both CTAs
				const uint32_t full = map_to_rank(full_local, 0);
				const uint32_t sa = base + s * P_STAGE_BYTES;
				const uint32_t sal = sa + P_A_BYTES;
				const uint32_t sb = sal + P_A_BYTES;
				const uint32_t sbl = sb + P_A_BYTES;
				const int k0 = kb * P_BK;
				if (p.a_mn)
				{
					tma_pair_load_3d(sa, &mapA, full, 0, k0, am0 / 32);
					tma_pair_load_3d(sal, &mapAlo, full, 0, k0, am0 / 32);
				}
				else
				{
					tma_pair_load_2d(sa, &mapA, full, k0, am0);
					tma_pair_load_2d(sal, &mapAlo, full, k0, am0);
				}
				if (p.b_mn)
				{
					tma_pair_load_3d(sb, &mapB, full, 0, k0, bn0 / 32);
					tma_pair_load_3d(sbl, &mapBlo, full, 0, k0, bn0 / 32);
				}
				else
				{
					tma_pair_load_2d(sb, &mapB, full, k0, bn0);
					tma_pair_load_2d(sbl, &mapBlo, full, k0, bn0);
				}
			}
		}
	}
	else if (warp == 1 && lane == 0 && leader)
	{
		// ------------------------------------------------ MMA issuer (leader CTA only)
		const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
		                       ((uint32_t)(P_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
		constexpr uint32_t K_SBO = 512u, K_LT = 4u, MN_LBO = 128u * P_BK;
		const uint32_t a_lbo = p.a_mn ? MN_LBO : 0u, a_sbo = p.a_mn ? 512u : K_SBO, a_kstep = p.a_mn ? 1024u : 32u;
		const uint32_t b_lbo = p.b_mn ? MN_LBO : 0u, b_sbo = p.b_mn ? 512u : K_SBO, b_kstep = p.b_mn ? 1024u : 32u;
		const uint32_t a_lt = p.a_mn ? 1u : K_LT, b_lt = p.b_mn ? 1u : K_LT;
		bool ok = true;
		int it = 0, gc = 0;
		for (int t = pair; t < total_tiles && ok; t += npairs)
			for (int kb = 0; kb < KB && ok; ++kb, ++it)
			{
				const int s = it % P_STAGES;
				const uint32_t ph = (uint32_t)(it / P_STAGES) & 1u;
				const int kin = kb % P_CHUNK_KB;
				if (kin == 0 && kb != 0) ++gc;
				const int buf = gc & 1;
				const uint32_t tmem_d = tmem_base + (uint32_t)(buf * P_BN);
				if (kin == 0)
				{
					const uint32_t use = (uint32_t)(gc >> 1);
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
				const uint32_t sa = base + s * P_STAGE_BYTES;
				const uint32_t sal = sa + P_A_BYTES;
				const uint32_t sb = sal + P_A_BYTES;
				const uint32_t sbl = sb + P_A_BYTES;
#pragma unroll
				for (int j = 0; j < P_BK / 8; ++j)
				{
					const uint64_t dA = make_smem_desc(sa + j * a_kstep, a_lbo, a_sbo, a_lt);
					const uint64_t dAl = make_smem_desc(sal + j * a_kstep, a_lbo, a_sbo, a_lt);
					const uint64_t dB = make_smem_desc(sb + j * b_kstep, b_lbo, b_sbo, b_lt);
					const uint64_t dBl = make_smem_desc(sbl + j * b_kstep, b_lbo, b_sbo, b_lt);
					umma_pair_tf32(tmem_d, dA, dBl, idesc, (kin | j) != 0 ? 1u : 0u);
					umma_pair_tf32(tmem_d, dAl, dB, idesc, 1u);
					umma_pair_tf32(tmem_d, dA, dB, idesc, 1u);
				}
				// the stage is free in BOTH CTAs once these MMAs have read it
				const uint32_t empty_local = bar0 + 8 * (P_STAGES + s);
				umma_pair_commit(map_to_rank(empty_local, 0));
				umma_pair_commit(map_to_rank(empty_local, 1));
				if (kin == P_CHUNK_KB - 1 || kb == KB - 1)
				{
					umma_pair_commit(map_to_rank(bar_acc_full + 8 * buf, 0));
					umma_pair_commit(map_to_rank(bar_acc_full + 8 * buf, 1));
				}
				if (kb == KB - 1) ++gc;
			}
	}
	else if (warp >= 2)
	{
		// ------------------------------------------------ epilogue (both CTAs, own 128 rows)
		const int q = warp & 3;
		const int half = (warp - 2) >> 2;
		bool ok = true;
		int piece_turn = 0;
		int gc = 0;
		for (int t = pair; t < total_tiles && ok; t += npairs)
		{
			int m0, n0;
			tile_origin(t, m0, n0);
			m0 += (int)rank * P_HALF;
			float acc[128];
#pragma unroll
			for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
			for (int c_in = 0; c_in < NCHUNK && ok; ++c_in, ++gc)
			{
				const int buf = gc & 1;
				const uint32_t use = (uint32_t)(gc >> 1);
				if (!mbar_wait(bar_acc_full + 8 * buf, use & 1u, abort_flag, p.err_flag, 3))
				{
					ok = false;
					break;
				}
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * P_BN + half * 128);
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
				if (lane == 0) mbar_arrive_cluster(map_to_rank(bar_acc_empty + 8 * buf, 0));
			}
			if (ok && !(p.debug & 1))
			{
				const int row = m0 + q * 32 + lane;
				const int col0 = n0 + half * 128;
				RowSink out;
				out.crow = p.C + (long long)row * p.ldc + col0;
				out.lorow = p.C_lo ? p.C_lo + (long long)row * p.ldc + col0 : nullptr;
				out.stage = staging0 + (uint32_t)(warp - 2) * 4096u;
				out.mapC = &mapC;
				out.mapClo = p.C_lo ? &mapClo : nullptr;
				out.col0 = col0;
				out.row0 = m0 + q * 32;
				out.lane = lane;
				out.direct = (p.debug & 2) != 0;
				out.nbuf = 1;
				out.turn = &piece_turn;
				apply_epilogue(acc, out, p, row, col0);
			}
		}
		if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
	if (warp == 1)
	{
		asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * P_BN) : "memory");
	}
}

}  // namespace

bool tc::tc_pair_supported(const GemmArgs& g)
{
	static int enabled = -1;
	if (enabled < 0)
	{
		// Off unless GLADES_TC_PAIR=1: on the wide-MLP step the pair kernel measured 5 % slower than the
		// one-CTA kernel (212 vs 222 TFLOP/s sustained under the power cap; it runs at a higher clock but
		// does less per clock), so it is kept as a tested variant, not the default.
		const char* e = getenv("GLADES_TC_PAIR");
		enabled = (e && atoi(e) == 1) ? 1 : 0;
	}
	return enabled && tc_bk() == 16 && g.M % 256 == 0 && g.N % 256 == 0;
}

cudaError_t tc::launch_gemm_tc_pair(const CUtensorMap maps[6], const TcParams& p, int M, int N, int sm_reserve, cudaStream_t s)
{
	// per launch: the opt-in and the SM count belong to the current device, not to the process
	if (cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_TOTAL)) return e;
	TcParams q = p;
	q.tiles_m = M / 256;
	q.tiles_n = N / P_BN;
	int sm_count = 0, dev = 0;
	if (cudaError_t e = cudaGetDevice(&dev)) return e;
	if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count < 2) sm_count = 148;
	int pairs = (sm_count - sm_reserve) / 2;
	if (pairs < 1) pairs = 1;
	const int total = q.tiles_m * q.tiles_n;
	if (pairs > total) pairs = total;
	gemm_tc_pair_kernel<<<2 * pairs, P_THREADS, P_TOTAL, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], q);
	cudaError_t le = cudaGetLastError();
	if (le != cudaSuccess && getenv("GLADES_TC_DEBUG"))
	{
		cudaFuncAttributes fa;
		cudaFuncGetAttributes(&fa, gemm_tc_pair_kernel);
		fprintf(stderr, "[pair] launch failed: %s; regs %d maxThreads %d static smem %zu maxDyn %d local %zu; grid %d threads %d dyn %d\n",
		        cudaGetErrorString(le), fa.numRegs, fa.maxThreadsPerBlock, fa.sharedSizeBytes, fa.maxDynamicSharedSizeBytes,
		        fa.localSizeBytes, 2 * pairs, P_THREADS, P_TOTAL);
	}
	return le;
}

}  // namespace glb
