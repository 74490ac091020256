// gl_matmul_static: the tensor-core layer product for callers that must not allocate.
//
// Some hosts of this library cannot let it call cudaMalloc: a process that has handed all of the
// GPU's memory to its own arena up front (a library-side cudaMalloc would then simply fail), and a
// caller that drives the GPU from a loop which must never stall (cudaMalloc and cudaFree are
// device-wide synchronisation points, so one call from here would serialise every stream of the
// process, e.g. a training loop that streams snapshots to a viewer on a second stream).  The regular
// gl_matmul entry point allocates its scratch (the low TF32 parts of both operands and a status
// word) on every call.  This variant keeps that scratch in a fixed array that is part of the loaded
// library image instead, so it calls no allocating routine at all.
//
// The price: the array occupies GL_STATIC_SCRATCH_BYTES (16 MiB + 256 B) on every GPU that loads the
// library, until the process exits; operands are limited to GL_STATIC_MAX_OPERAND_FLOATS floats
// each; and every call shares the one array, so two calls whose GPU work overlaps (different
// streams, threads or processes sharing a context) race on it -- callers serialise them.  The array
// keeps the previous call's contents; the status word is cleared at the start of every call and the
// low-part regions are rewritten for exactly the extents this call's product reads.
//
// The array's name is only a host-side stand-in in host code; the device address is fetched once
// per device with cudaGetSymbolAddress (with that device current) and handed to the kernels.  The same
// set-up creates one private non-blocking stream per device: every piece of GPU work of this entry
// point runs on it, so a call neither waits for nor holds up the caller's other streams (the legacy
// default stream would serialise with all of them).  The set-up happens inside the first call on a
// device, so make that first call outside any stream capture.  The call leaves the caller's current
// device as it found it.
#include <mutex>

#include <stdio.h>
#include <string.h>

#include "internal.h"
#include "tc_gemm.h"

#define GL_STATIC_MAX_OPERAND_FLOATS (2ll * 1024 * 1024)
#define GL_STATIC_HEADER_FLOATS 64  // 256 bytes: status word, padding to keep the operands 256-byte aligned
#define GL_STATIC_SCRATCH_FLOATS (GL_STATIC_HEADER_FLOATS + 2 * GL_STATIC_MAX_OPERAND_FLOATS)

static __device__ __align__(256) float g_static_scratch[GL_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
cudaStream_t g_stream[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local char g_static_err[256];

// Once per device, with that device current: the device address of the static array and the private
// stream this entry point works on.
cudaError_t scratch_for_current_device(int device, float** out, cudaStream_t* stream)
{
	std::lock_guard<std::mutex> lock(g_setup_mutex);
	if (!g_scratch_addr[device])
	{
		float* p = nullptr;
		cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
		if (e != cudaSuccess) return e;
		cudaStream_t st = nullptr;
		e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
		if (e != cudaSuccess) return e;
		g_stream[device] = st;
		g_scratch_addr[device] = p;
	}
	*out = g_scratch_addr[device];
	*stream = g_stream[device];
	return cudaSuccess;
}

// Puts the caller's current device back when the entry point returns, whichever way it returns.
struct DeviceRestore
{
	int prev = -1;
	DeviceRestore() { if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; cudaGetLastError(); } }
	~DeviceRestore() { if (prev >= 0) cudaSetDevice(prev); }
};
}  // namespace

extern "C" const char* gl_matmul_static_error(void) { return g_static_err; }

extern "C" int gl_matmul_static(const float* d_a, int64_t a_sm, int64_t a_sk, const float* d_b, int64_t b_sn, int64_t b_sk,
                                float* d_c, int64_t ldc, int32_t m, int32_t n, int32_t k, int32_t device)
{
	using namespace glb;
	g_static_err[0] = 0;
	if (!d_a || !d_b || !d_c || m < 1 || n < 1 || k < 1 || device < 0 || device >= kMaxDevices)
	{
		snprintf(g_static_err, sizeof g_static_err, "gl_matmul_static: bad argument");
		return GL_ERR_INVALID;
	}
	{
		int major = 0;
		if (gl_device_count() < 1 || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major != 10)
		{
			cudaGetLastError();
			snprintf(g_static_err, sizeof g_static_err, "gl_matmul_static: device %d is not an sm_100 device (there is no CPU path)", device);
			return GL_ERR_NO_DEVICE;
		}
	}
	GemmArgs g;
	memset(&g, 0, sizeof g);
	g.A = d_a; g.a_sm = a_sm; g.a_sk = a_sk;
	g.B = d_b; g.b_sn = b_sn; g.b_sk = b_sk;
	g.C = d_c; g.ldc = ldc;
	g.M = m; g.N = n; g.K = k;
	g.epi = EPI_NONE;
	if (!tc_gemm_supported(g))
	{
		snprintf(g_static_err, sizeof g_static_err,
		         "gl_matmul_static: %dx%dx%d with these strides does not fit the tensor-core tiles "
		         "(M %% 128, N %% 128, K %% 16, operands contiguous in k or in m/n, 16-byte aligned)", m, n, k);
		return GL_ERR_INVALID;
	}
	// extents of the two operands as the product reads them
	const long long ca = (a_sk == 1) ? (long long)(m - 1) * a_sm + k : (long long)(k - 1) * a_sk + m;
	const long long cb = (b_sk == 1) ? (long long)(n - 1) * b_sn + k : (long long)(k - 1) * b_sk + n;
	if (ca > GL_STATIC_MAX_OPERAND_FLOATS || cb > GL_STATIC_MAX_OPERAND_FLOATS)
	{
		snprintf(g_static_err, sizeof g_static_err,
		         "gl_matmul_static: operands of %lld and %lld floats exceed the static scratch limit of %lld floats "
		         "each; use gl_matmul (which allocates) for larger products", ca, cb, (long long)GL_STATIC_MAX_OPERAND_FLOATS);
		return GL_ERR_TOO_LARGE;
	}
	DeviceRestore restore;
	cudaError_t e = cudaSetDevice(device);
	float* scratch = nullptr;
	cudaStream_t st = nullptr;
	if (e == cudaSuccess) e = scratch_for_current_device(device, &scratch, &st);
	if (e != cudaSuccess)
	{
		snprintf(g_static_err, sizeof g_static_err, "gl_matmul_static: set-up failed: %s", cudaGetErrorString(e));
		return GL_ERR_CUDA;
	}
	int* flag = reinterpret_cast<int*>(scratch);
	float* a_lo = scratch + GL_STATIC_HEADER_FLOATS;
	float* b_lo = a_lo + GL_STATIC_MAX_OPERAND_FLOATS;
	// the status word must start at zero; the low parts are fully rewritten below
	// (all on the private stream: the product reads the caller's operands, so the caller's own work
	// that produces them must have finished before this call, as with gl_matmul)
	e = cudaMemsetAsync(flag, 0, GL_STATIC_HEADER_FLOATS * sizeof(float), st);
	if (e == cudaSuccess) e = launch_split_lo(d_a, a_lo, ca, st);
	if (e == cudaSuccess) e = launch_split_lo(d_b, b_lo, cb, st);
	if (e == cudaSuccess) e = launch_gemm_tc(g, a_lo, b_lo, flag, st);
	int hflag = 0;
	if (e == cudaSuccess) e = cudaMemcpyAsync(&hflag, flag, sizeof hflag, cudaMemcpyDeviceToHost, st);
	if (e == cudaSuccess) e = cudaStreamSynchronize(st);
	if (e != cudaSuccess)
	{
		snprintf(g_static_err, sizeof g_static_err, "gl_matmul_static: %s", cudaGetErrorString(e));
		return GL_ERR_CUDA;
	}
	if (hflag)
	{
		snprintf(g_static_err, sizeof g_static_err, "gl_matmul_static: a bounded wait inside the kernel ran out (role %d)", hflag);
		return GL_ERR_TIMEOUT;
	}
	return GL_OK;
}
