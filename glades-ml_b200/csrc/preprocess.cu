// Input standardisation on the device: the step in front of the training loop,
// NumberInput::standardizeInputTable (DataObjects/NumberInput.cpp:43-285) with the one-hot vectors of
// OHE::operator[] (GMath/OHE.cpp:159-198), on a raw table that already lies in HBM as a row-major
// [rows][cols] fp32 matrix (a categorical column holds each cell's category index, in order of first
// appearance -- the strings themselves stay on the host).
//
// Pass 1, column statistics.  Minimum and maximum do not depend on the order of the rows, so they are
// reduced in parallel: the grid's threads stride over the row-major cells with coalesced reads (the stride
// is a multiple of the column count, so a thread stays on one column and keeps its extrema in registers)
// and merge with atomics on an order-preserving integer image of the floats.  The reference starts the running minimum and maximum from the first cell
// only for raw column 0 and from 0.0 for every other column (NumberInput.cpp:105-109): columns other than
// 0 therefore start their reduction at 0.  The mean and the standard deviation (z-score mode only) are
// sequential fp32 sums in row order in the reference (:118-121,236-249), so they run as one thread per
// column walking the rows -- coalesced across the columns of a warp -- to stay bit-identical.
// Pass 2, transform.  One thread per (row, raw column): scale with separately rounded fp32 operations
// in the reference's order, ((x - min) / range) * 0.98 + 0.01 (any categorical column in the table) or
// (x - min) / range, or (x - mean) / stdev, and write the cell -- or the 0.99 / 0.01 one-hot group of a
// categorical cell -- at its place in the input matrix X or the expected matrix Y.
// HBM traffic: rows * cols * 4 bytes read twice, rows * (nx + ny) * 4 bytes written once.
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace glb {
namespace {

__device__ __forceinline__ int float_order(float f)
{
	// monotone map float -> int (so that integer atomicMin / atomicMax order floats)
	const int i = __float_as_int(f);
	return i >= 0 ? i : i ^ 0x7FFFFFFF;
}
__device__ __forceinline__ float order_float(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7FFFFFFF); }

// stats: [cols][4] = min image, max image (ints, pre-set by the host to the images of the start values),
// mean, stdev.  Thread t of the grid handles column t % cols of every (grid size / cols)-th row: the grid size
// is a multiple of cols, so a thread stays on one column (extrema in registers, no division in the loop) while
// consecutive threads read consecutive addresses.  A block merges its threads' extrema in shared memory and
// issues one global atomic per column it touched.
__global__ void __launch_bounds__(256) minmax_kernel(const float* __restrict__ raw, long long rows, int cols, int* stats)
{
	extern __shared__ int sext[];  // [2][cols]: images of the block's minimum and maximum per column
	for (int c = threadIdx.x; c < cols; c += blockDim.x)
	{
		sext[c] = 0x7FFFFFFF;
		sext[cols + c] = (int)0x80000000;
	}
	__syncthreads();
	const long long total = rows * (long long)cols;
	const long long stride = (long long)gridDim.x * blockDim.x;
	const long long start = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	const int c = (int)(start % cols);
	float mn = __int_as_float(0x7F800000), mx = __int_as_float(0xFF800000);
	bool any = false;
	// four independent loads in flight per thread: the pass is a pure stream, bandwidth comes from bytes in flight
	long long i = start;
	for (; i + 3 * stride < total; i += 4 * stride)
	{
		const float v0 = raw[i], v1 = raw[i + stride], v2 = raw[i + 2 * stride], v3 = raw[i + 3 * stride];
		mn = fminf(fminf(mn, v0), fminf(v1, fminf(v2, v3)));
		mx = fmaxf(fmaxf(mx, v0), fmaxf(v1, fmaxf(v2, v3)));
		any = true;
	}
	for (; i < total; i += stride)
	{
		const float v = raw[i];
		mn = fminf(mn, v);
		mx = fmaxf(mx, v);
		any = true;
	}
	if (any)
	{
		atomicMin(sext + c, float_order(mn));
		atomicMax(sext + cols + c, float_order(mx));
	}
	__syncthreads();
	for (int k = threadIdx.x; k < cols; k += blockDim.x)
	{
		if (sext[k] != 0x7FFFFFFF) atomicMin(stats + 4 * k, sext[k]);
		if (sext[cols + k] != (int)0x80000000) atomicMax(stats + 4 * k + 1, sext[cols + k]);
	}
}

__global__ void __launch_bounds__(128) mean_stdev_kernel(const float* __restrict__ raw, long long rows, int cols,
                                                          const int* __restrict__ kind, float* stats)
{
	const int c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c >= cols || kind[c] != 0) return;
	// sequential fp32 sums in row order, as the reference accumulates them
	float mean = 0.0f;
	for (long long r = 0; r < rows; ++r) mean = __fadd_rn(mean, raw[r * cols + c]);
	mean = __fdiv_rn(mean, (float)(unsigned int)rows);
	float sd = 0.0f;
	for (long long r = 0; r < rows; ++r)
	{
		const float d = __fsub_rn(raw[r * cols + c], mean);
		sd = __fadd_rn(sd, __fmul_rn(d, d));
	}
	sd = __fsqrt_rn(__fdiv_rn(sd, (float)((unsigned int)rows - 1u)));
	stats[4 * c + 2] = mean;
	stats[4 * c + 3] = sd;
}

struct ColumnPlan
{
	int kind;     // 0 numeric, 1 categorical
	int classes;  // categorical: one-hot width
	int dst;      // 0: X, 1: Y
	int at;       // first destination column
};

// The same geometry as minmax_kernel: a thread stays on one raw column, so its plan record and scale factors
// are loaded once; the row advances by (grid size / cols) per iteration.
__global__ void __launch_bounds__(256) transform_kernel(const float* __restrict__ raw, long long rows, int cols,
                                                         const ColumnPlan* __restrict__ plan, const int* __restrict__ stats,
                                                         int flag, int classification, float* __restrict__ X, int ldx,
                                                         float* __restrict__ Y, int ldy)
{
	const long long total = rows * (long long)cols;
	const long long stride = (long long)gridDim.x * blockDim.x;
	const long long start = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	if (start >= total) return;
	const int c = (int)(start % cols);
	long long r = start / cols;
	const long long rstep = stride / cols;
	const ColumnPlan p = plan[c];
	float* const base = p.dst ? Y : X;
	const long long ld = p.dst ? ldy : ldx;
	const float mn = order_float(stats[4 * c]), mx = order_float(stats[4 * c + 1]);
	const float range = __fsub_rn(mx, mn);
	const float mean = __int_as_float(stats[4 * c + 2]), sd = __int_as_float(stats[4 * c + 3]);
	auto put = [&](long long row, float v) {
		float* dst = base + row * ld + p.at;
		if (p.kind == 1)
		{
			const int id = (int)v;
			for (int k = 0; k < p.classes; ++k) dst[k] = (k == id) ? 0.99f : 0.01f;
			return;
		}
		if (flag == 0)
		{
			if (range != 0.0f)
			{
				v = __fdiv_rn(__fsub_rn(v, mn), range);
				if (classification) v = __fadd_rn(__fmul_rn(v, 0.98f), 0.01f);
			}
		}
		else
			v = __fdiv_rn(__fsub_rn(v, mean), sd);
		*dst = v;
	};
	// four independent loads in flight per thread before the first is consumed
	long long i = start;
	for (; i + 3 * stride < total; i += 4 * stride, r += 4 * rstep)
	{
		const float v0 = raw[i], v1 = raw[i + stride], v2 = raw[i + 2 * stride], v3 = raw[i + 3 * stride];
		put(r, v0);
		put(r + rstep, v1);
		put(r + 2 * rstep, v2);
		put(r + 3 * rstep, v3);
	}
	for (; i < total; i += stride, r += rstep) put(r, raw[i]);
}

}  // namespace

// blocks of 256 threads for a pass over rows * cols cells: about eight cells per thread, at most per_sm blocks per
// SM, and a multiple of cols, so that the grid size is a multiple of cols (a thread then stays on one column)
static unsigned column_pass_blocks(long long total, int cols, int per_sm)
{
	long long blocks = (total / 8 + 255) / 256;
	const long long cap = 148ll * per_sm;
	if (blocks > cap) blocks = cap;
	if (blocks < 1) blocks = 1;
	blocks = ((blocks + cols - 1) / cols) * cols;
	return (unsigned)blocks;
}

cudaError_t launch_column_minmax(const float* raw, long long rows, int cols, int* d_stats, cudaStream_t s)
{
	const long long total = rows * (long long)cols;
	if (total < 1) return cudaSuccess;
	if (cols > 6000) return cudaErrorInvalidValue;  // the block's extrema live in shared memory
	// every block ends with two atomics per column on the same 2 * cols words: fewer, longer blocks
	minmax_kernel<<<column_pass_blocks(total, cols, 6), 256, (size_t)2 * cols * sizeof(int), s>>>(raw, rows, cols, d_stats);
	return cudaGetLastError();
}

cudaError_t launch_column_mean_stdev(const float* raw, long long rows, int cols, const int* d_kind, float* d_stats, cudaStream_t s)
{
	mean_stdev_kernel<<<(cols + 127) / 128, 128, 0, s>>>(raw, rows, cols, d_kind, d_stats);
	return cudaGetLastError();
}

cudaError_t launch_column_transform(const float* raw, long long rows, int cols, const void* d_plan, const int* d_stats, int flag,
                                    int classification, float* X, int ldx, float* Y, int ldy, cudaStream_t s)
{
	const long long total = rows * (long long)cols;
	if (total < 1) return cudaSuccess;
	transform_kernel<<<column_pass_blocks(total, cols, 16), 256, 0, s>>>(raw, rows, cols, static_cast<const ColumnPlan*>(d_plan), d_stats, flag,
	                                                  classification, X, ldx, Y, ldy);
	return cudaGetLastError();
}

int float_order_host(float f)
{
	int i;
	memcpy(&i, &f, sizeof i);
	return i >= 0 ? i : i ^ 0x7FFFFFFF;
}
float order_float_host(int i)
{
	i = i >= 0 ? i : i ^ 0x7FFFFFFF;
	float f;
	memcpy(&f, &i, sizeof f);
	return f;
}

}  // namespace glb
