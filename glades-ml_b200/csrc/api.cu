// extern "C" layer of the B200-native glades feed-forward path (declared in include/glades_b200.h).
// It owns the device memory of one network, packs rows and weights into contiguous row-major
// device matrices, and drives the kernels of ref_mode.cu (reference arithmetic), small_fused.cu /
// grid_fused.cu / batched.cu / gemm_tcgen05.cu (batched arithmetic: whole-network, whole-window and
// per-layer engines), dp_push.cu (data-parallel exchange over peer memory) and synth.cu.  There is no
// CPU compute path: every compute entry point fails with GL_ERR_NO_DEVICE when no sm_100 device is
// present.
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>
#include <vector>

#include "internal.h"
#include "tc_gemm.h"

using namespace glb;

// ------------------------------------------------------------------------------------------------
static thread_local std::string g_err;

static int fail(int code, const char* fmt, ...)
{
	char buf[512];
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(buf, sizeof buf, fmt, ap);
	va_end(ap);
	g_err = buf;
	return code;
}

#define CU(call)                                                                                     \
	do                                                                                               \
	{                                                                                                \
		cudaError_t e__ = (call);                                                                    \
		if (e__ != cudaSuccess)                                                                      \
			return fail(GL_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
	} while (0)

extern "C" const char* gl_last_error(void) { return g_err.c_str(); }

extern "C" int gl_device_count(void)
{
	int n = 0;
	if (cudaGetDeviceCount(&n) != cudaSuccess)
	{
		cudaGetLastError();
		return 0;
	}
	int ok = 0;
	for (int i = 0; i < n; ++i)
	{
		int major = 0;
		if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++ok;
	}
	return ok;
}

// ---- NCCL, bound at run time so that single-GPU users need no NCCL at all ----------------------
namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
struct NcclApi
{
	void* so = nullptr;
	int (*GetUniqueId)(nccl_uid*) = nullptr;
	int (*CommInitRank)(nccl_comm*, int, nccl_uid, int) = nullptr;
	int (*CommDestroy)(nccl_comm) = nullptr;
	int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
	int (*AllGather)(const void*, void*, size_t, int, nccl_comm, cudaStream_t) = nullptr;
	int (*GroupStart)() = nullptr;
	int (*GroupEnd)() = nullptr;
	const char* (*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;
enum { NCCL_INT8 = 0, NCCL_INT32 = 2, NCCL_FLOAT32 = 7, NCCL_FLOAT64 = 8, NCCL_SUM = 0 };

int nccl_load()
{
	if (g_nccl.so) return 0;
	const char* names[] = {"libnccl.so.2", "libnccl.so"};
	void* so = nullptr;
	for (const char* nm : names)
	{
		so = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
		if (so) break;
	}
	if (!so) return fail(GL_ERR_COMM, "cannot load libnccl.so.2: %s", dlerror());
	g_nccl.GetUniqueId = (int (*)(nccl_uid*))dlsym(so, "ncclGetUniqueId");
	g_nccl.CommInitRank = (int (*)(nccl_comm*, int, nccl_uid, int))dlsym(so, "ncclCommInitRank");
	g_nccl.CommDestroy = (int (*)(nccl_comm))dlsym(so, "ncclCommDestroy");
	g_nccl.AllReduce =
	    (int (*)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t))dlsym(so, "ncclAllReduce");
	g_nccl.AllGather = (int (*)(const void*, void*, size_t, int, nccl_comm, cudaStream_t))dlsym(so, "ncclAllGather");
	g_nccl.GroupStart = (int (*)())dlsym(so, "ncclGroupStart");
	g_nccl.GroupEnd = (int (*)())dlsym(so, "ncclGroupEnd");
	g_nccl.GetErrorString = (const char* (*)(int))dlsym(so, "ncclGetErrorString");
	if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.GroupStart || !g_nccl.GroupEnd)
		return fail(GL_ERR_COMM, "libnccl lacks a required symbol");
	g_nccl.so = so;
	return 0;
}
}  // namespace

#define NC(call)                                                                                 \
	do                                                                                           \
	{                                                                                            \
		int r__ = (call);                                                                        \
		if (r__ != 0)                                                                            \
			return fail(GL_ERR_COMM, "%s failed: %s", #call,                                     \
			            g_nccl.GetErrorString ? g_nccl.GetErrorString(r__) : "nccl error");     \
	} while (0)

// ------------------------------------------------------------------------------------------------
struct gl_net
{
	gl_net_desc d;
	int H = 0;
	int64_t nw = 0;
	int64_t woff[GL_MAX_WEIGHT_LAYERS + 1];
	int n_out = 0;
	int total_nodes = 0;
	int softmax = 0;
	cudaStream_t stream = nullptr;
	cudaEvent_t ev0 = nullptr, ev1 = nullptr;

	float* dW = nullptr;      // flat weights
	float* dBias = nullptr;   // [GL_MAX_WEIGHT_LAYERS]
	float* dG = nullptr;      // flat gradient | per-layer bias sums (GL_MAX_WEIGHT_LAYERS floats)
	float* dBscale = nullptr; // [GL_MAX_WEIGHT_LAYERS]
	int* dFlags = nullptr;
	double* dSums = nullptr;  // [2] cost, accuracy (batched)
	double* winSums = nullptr; // the sums the current window step accumulates into (dSums or a pipeline slot)
	// two-deep pipeline of host-buffer windows (gl_train_window_host_submit / _result)
	struct Slot
	{
		float* dX = nullptr;
		float* dY = nullptr;
		int64_t cap = 0;
		double* dSums = nullptr;
		double* hSums = nullptr;  // pinned: cost, accuracy, then the status words
		int* hArg = nullptr;      // pinned: predicted classes of an inference batch (gl_forward_host_submit)
		int64_t argCap = 0;
		bool infer = false, hasY = false;
		cudaEvent_t copied = nullptr, done = nullptr, t0 = nullptr;
		int rows = 0, globalRows = 0;
		int64_t launches = 0;
		bool pending = false;
	} slot[2];
	cudaStream_t copyStream = nullptr;
	uint64_t submitted = 0, collected = 0;
	float* dSumsF = nullptr;  // reference mode: [n_epochs][2]
	int sumsFCap = 0;
	int* dConf = nullptr;     // [n_out][n_out]
	float* dLastOut = nullptr; // [n_out]: predictions of the last row the last call processed
	// reference mode
	float* dHist = nullptr;
	int* dHistLen = nullptr;
	float* dScratch = nullptr;
	// asynchronous snapshot for live views (gl_snapshot_submit / _collect): weights | layer-indexed biases |
	// pre-activations of the last row, copied device-to-device beside the compute stream, then to pinned memory
	float* dPreact = nullptr;   // [total nodes - n_0]
	float* dSnap = nullptr;
	float* hSnap = nullptr;
	cudaStream_t snapStream = nullptr;
	cudaEvent_t evSnapSrc = nullptr, evSnapCopied = nullptr, evSnapReady = nullptr;
	bool snapPending = false;
	// reference mode with dropout: per-edge history lengths and last deltas, the error accumulators that
	// survive a row, and one epoch's node flags (drawn on the host with rand(), in the reference's order)
	bool dropout = false;
	int maskStride = 0;
	int* dHlen = nullptr;
	float* dHlast = nullptr;
	float* dErrState = nullptr;
	unsigned char* dMasks = nullptr;
	int64_t maskCapRows = 0;
	std::vector<unsigned char> hMasks;
	std::vector<unsigned char> dropFlags;  // the flags of the current row, carried over where a layer draws nothing
	// data
	const float* dX = nullptr;
	const float* dY = nullptr;
	float* ownX = nullptr;
	float* ownY = nullptr;
	int64_t rows = 0;
	// batched work buffers
	int64_t capRows = 0;
	float* dA[GL_MAX_WEIGHT_LAYERS + 2] = {};
	float* dD[GL_MAX_WEIGHT_LAYERS + 2] = {};
	float* dC[GL_MAX_WEIGHT_LAYERS] = {};  // momentum weights per layer (NULL when momentum is 0)
	float* dColterm = nullptr;
	double* dSumPart = nullptr;      // scratch of the reproducible bias sums (launch_sum_scaled)
	unsigned* dSumTicket = nullptr;
	int cRows = -1, cGlobal = -1, cFirst = -1;
	int* dArgmax = nullptr;
	// host-window staging
	float* dXwin = nullptr;
	float* dYwin = nullptr;
	int64_t winCap = 0;
	float* hPinned = nullptr;
	size_t pinnedBytes = 0;
	// low TF32 parts of the tensor-core operands (X_lo = X - trunc_tf32(X)), made on demand
	float* dXlo = nullptr;
	float* dWlo = nullptr;
	float* dAlo[GL_MAX_WEIGHT_LAYERS + 2] = {};
	float* dDlo[GL_MAX_WEIGHT_LAYERS + 2] = {};
	unsigned* dMask[GL_MAX_WEIGHT_LAYERS + 2] = {};  // ReLU layers: (activation > 0) bits, [rows][n_l/32]
	bool maskValid[GL_MAX_WEIGHT_LAYERS + 2] = {};
	float* dDc = nullptr;     // momentum-weighted copy of one delta matrix and its low part
	float* dDclo = nullptr;
	bool loX = false, loW = false, loDc = false;
	bool loA[GL_MAX_WEIGHT_LAYERS + 2] = {};
	bool loD[GL_MAX_WEIGHT_LAYERS + 2] = {};
	int64_t tcLaunches = 0;
	int64_t lastWindowLaunches = 0;
	// workspace for splitting a partial wave of tiles along k (all tensor-core products of the compute stream)
	TcSplitK sk = {nullptr, nullptr, nullptr, 0, 0};
	unsigned skEpoch = 0;
	// optional per-launch timing of the layer products (gl_profile_enable)
	bool profile = false;
	std::vector<cudaEvent_t> profEv;   // pairs
	std::vector<double> profFlops;
	std::vector<int> profIsTc;
	std::vector<int> profShape;  // M, N, K, epilogue per recorded launch
	size_t profUsed = 0;
	cudaEvent_t tim0 = nullptr, tim1 = nullptr;

	// whole-window cooperative kernel for mid-size networks (grid_fused.cu)
	float* gfAct = nullptr;
	float* gfDel = nullptr;
	double* gfPart = nullptr;
	float* gfCk = nullptr;   // momentum table for windows of gfCkMb rows
	void* gfMaps = nullptr;  // device array of the weight tensor maps (NULL: the register path)
	bool gfMapsTried = false;
	unsigned long long* gfTiming = nullptr;  // GLADES_GF_TIMING=1: phase nanoseconds, printed when the handle goes
	int gfRows = 0, gfCtas = 0, gfCkMb = 0;
	int gfOk = -1;  // -1 not decided yet
	int gfClusterCtas = -1;  // CTAs of the cluster variant's grid; 0: the variant does not apply; -1 not decided yet

	int epochs = 0;
	volatile int stop = 0;
	int64_t launches = 0;
	// data parallel
	int rank = 0, world = 1;
	nccl_comm comm = nullptr;
	int globalRows = 0, firstPos = 0;
	int bscaleRows = -1;
	// gradient all-reduce overlapped with the rest of the backward pass
	cudaStream_t commStream = nullptr;
	// peer-memory exchange: layer l's exchange runs on its own stream (round robin over DP_COMM_STREAMS) so
	// that a small layer's update does not queue behind a large one's; evLayer[l] fires when every owner's band
	// of layer l's new weights (and their low TF32 parts) has landed here.  The next use of W_l waits for it --
	// normally the next window's forward product of that layer, so the tail of the exchange overlaps the next
	// window instead of ending this one.
	enum { DP_COMM_STREAMS = 4 };
	cudaStream_t layerStream[DP_COMM_STREAMS] = {};
	cudaEvent_t evLayer[GL_MAX_WEIGHT_LAYERS] = {};
	bool layerPending[GL_MAX_WEIGHT_LAYERS] = {};
	cudaEvent_t evGrad[GL_MAX_WEIGHT_LAYERS + 1] = {};
	cudaEvent_t evRead[GL_MAX_WEIGHT_LAYERS] = {};  // the window's last product that reads the OLD W_l has finished
	size_t dpStageOff = 0;  // byte offset of the weight staging vector inside every rank's arena
	int dpStoreMode = 0;    // how a gradient's bands reach their owners: 0 from the product's epilogue, 1 copy kernel, 2 copy engines
	cudaEvent_t evComm = nullptr;
	int dpOverlap = 1;
	int dpReserveSms = 20;  // upper bound; a product keeps fewer free where that saves it a wave of tiles
	// gradient exchange over peer memory (dp_push.cu); dpPush == false: the NCCL all-reduce path
	bool dpPush = false;
	unsigned dpStep = 0;                 // window counter, the value the flags are raised to
	void* dpRec = nullptr;               // set-up scratch: gathered handles / agreement words (allocated before the communicator)
	char* dpArena = nullptr;             // this rank's arena: flag area, then one gradient slot per source rank
	void* dpPeerArena[DP_MAX_WORLD] = {}; // every rank's arena as mapped here (own entry = dpArena)
	void* dpPeerW[DP_MAX_WORLD] = {};     // every rank's weight vector as mapped here (own entry = dW)
	int dpBand[GL_MAX_WEIGHT_LAYERS] = {};        // rows of layer l's gradient per owner (a multiple of 128)
	int64_t dpSlotOff[GL_MAX_WEIGHT_LAYERS + 1] = {};  // float offset of layer l inside a slot; [H+1] = slot size
	void* dpMaps = nullptr;              // device: [layer][owner] tensor maps of the owners' bands (this rank's slot)
	float** dpBases = nullptr;           // device: [layer][owner] base pointers of the same
	float* hostBases[GL_MAX_WEIGHT_LAYERS][DP_MAX_WORLD] = {};
	int dpPushBlocks = 296;              // CTAs of an owner's update kernel while the backward pass still runs (8 GPUs: 32 -> 6.05 M, 128 -> 6.33 M, 296 -> 6.55 M, 592 -> 6.40 M samples/s)
};

static NetView make_view(const gl_net* n)
{
	NetView v;
	memset(&v, 0, sizeof v);
	v.H = n->H;
	for (int l = 0; l <= n->H + 1; ++l) v.sizes[l] = n->d.sizes[l];
	for (int l = 0; l <= n->H; ++l)
	{
		v.lr[l] = n->d.lr[l];
		v.mom[l] = n->d.momentum[l];
		v.wd1[l] = n->d.wd1[l];
		v.wd2[l] = n->d.wd2[l];
		v.act[l] = n->d.activation[l];
		v.par[l] = n->d.act_param[l];
		v.W[l] = n->dW + n->woff[l];
	}
	v.out_type = n->d.output_type;
	v.mb = n->d.batch_size;
	v.bias = n->dBias;
	return v;
}

static int use_device(const gl_net* n)
{
	CU(cudaSetDevice(n->d.device));
	return 0;
}

// Peer-memory exchange: makes the compute stream wait until layer l's new weights have landed (no-op when
// nothing is outstanding).
static int dp_wait_layer(gl_net* n, int l)
{
	if (n->layerPending[l])
	{
		CU(cudaStreamWaitEvent(n->stream, n->evLayer[l], 0));
		n->layerPending[l] = false;
	}
	return 0;
}
// The same for every layer: before anything but the next window's own products reads or replaces the weights.
static int dp_join(gl_net* n)
{
	for (int l = 0; l <= n->H; ++l)
		if (int r = dp_wait_layer(n, l)) return r;
	return 0;
}

static bool grid_fused_fits(const gl_net* n);

extern "C" int gl_create(const gl_net_desc* d, gl_net** out)
{
	if (!d || !out) return fail(GL_ERR_INVALID, "gl_create: null argument");
	*out = nullptr;
	const int H = d->n_layers - 2;
	if (H < 1 || H + 1 > GL_MAX_WEIGHT_LAYERS) return fail(GL_ERR_INVALID, "gl_create: n_layers %d out of range", d->n_layers);
	for (int l = 0; l <= H + 1; ++l)
		if (d->sizes[l] < 1) return fail(GL_ERR_INVALID, "gl_create: layer %d has size %d", l, d->sizes[l]);
	if (d->batch_size < 1) return fail(GL_ERR_INVALID, "gl_create: batch_size must be >= 1");
	if (d->mode != GL_MODE_REFERENCE && d->mode != GL_MODE_BATCHED) return fail(GL_ERR_INVALID, "gl_create: bad mode");
	for (int l = 0; l <= H; ++l)
	{
		if (d->p_dropout[l] != 0.0f && d->mode != GL_MODE_REFERENCE)
			return fail(GL_ERR_INVALID, "gl_create: dropout runs in reference mode only (p_dropout[%d] = %g)", l, (double)d->p_dropout[l]);
		if (!(d->p_dropout[l] >= 0.0f)) return fail(GL_ERR_INVALID, "gl_create: p_dropout[%d] is negative or not a number", l);
		const int a = d->activation[l];
		if (a < 0 || a > GL_ACT_SOFTMAX) return fail(GL_ERR_INVALID, "gl_create: bad activation id %d", a);
		if (a == GL_ACT_SOFTMAX && (l != H || d->mode != GL_MODE_BATCHED))
			return fail(GL_ERR_INVALID, "gl_create: softmax is only legal on the last layer of a batched-mode net");
	}
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device: this library has no CPU path");
	int major = 0;
	if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d->device) != cudaSuccess || major != 10)
		return fail(GL_ERR_NO_DEVICE, "device %d is not an sm_100 device", d->device);

	gl_net* n = new gl_net();
	n->d = *d;
	n->H = H;
	n->n_out = d->sizes[H + 1];
	n->softmax = d->activation[H] == GL_ACT_SOFTMAX;
	n->woff[0] = 0;
	for (int l = 0; l <= H; ++l) n->woff[l + 1] = n->woff[l] + (int64_t)d->sizes[l] * d->sizes[l + 1];
	n->nw = n->woff[H + 1];
	for (int l = 0; l <= H + 1; ++l) n->total_nodes += d->sizes[l];
	n->globalRows = 0;

	CU(cudaSetDevice(d->device));
	CU(cudaStreamCreateWithFlags(&n->stream, cudaStreamNonBlocking));
	CU(cudaEventCreate(&n->ev0));
	CU(cudaEventCreate(&n->ev1));
	CU(cudaMalloc(&n->dW, (n->nw + 4) * sizeof(float)));
	CU(cudaMemset(n->dW, 0, (n->nw + 4) * sizeof(float)));
	CU(cudaMalloc(&n->dBias, GL_MAX_WEIGHT_LAYERS * sizeof(float)));
	CU(cudaMemset(n->dBias, 0, GL_MAX_WEIGHT_LAYERS * sizeof(float)));
	CU(cudaMalloc(&n->dBscale, GL_MAX_WEIGHT_LAYERS * sizeof(float)));
	CU(cudaMalloc(&n->dFlags, 4 * sizeof(int)));
	CU(cudaMemset(n->dFlags, 0, 4 * sizeof(int)));
	CU(cudaMalloc(&n->dSums, 2 * sizeof(double)));
	CU(cudaMemset(n->dSums, 0, 2 * sizeof(double)));
	CU(cudaMalloc(&n->dLastOut, (size_t)n->n_out * sizeof(float)));
	CU(cudaMemset(n->dLastOut, 0, (size_t)n->n_out * sizeof(float)));
	CU(cudaMalloc(&n->dConf, (size_t)n->n_out * n->n_out * sizeof(int)));
	CU(cudaMemset(n->dConf, 0, (size_t)n->n_out * n->n_out * sizeof(int)));
	CU(cudaMalloc(&n->dPreact, (size_t)(n->total_nodes - d->sizes[0]) * sizeof(float)));
	CU(cudaMemset(n->dPreact, 0, (size_t)(n->total_nodes - d->sizes[0]) * sizeof(float)));
	if (d->mode == GL_MODE_REFERENCE)
	{
		CU(cudaMalloc(&n->dHist, (size_t)n->nw * d->batch_size * sizeof(float)));
		CU(cudaMemset(n->dHist, 0, (size_t)n->nw * d->batch_size * sizeof(float)));
		CU(cudaMalloc(&n->dHistLen, sizeof(int)));
		CU(cudaMemset(n->dHistLen, 0, sizeof(int)));
		for (int l = 0; l <= H; ++l)
		{
			if (d->p_dropout[l] != 0.0f) n->dropout = true;
			n->maskStride += d->sizes[l];
		}
		if (n->dropout)
		{
			CU(cudaMalloc(&n->dHlen, (size_t)n->nw * sizeof(int)));
			CU(cudaMemset(n->dHlen, 0, (size_t)n->nw * sizeof(int)));
			CU(cudaMalloc(&n->dHlast, (size_t)n->nw * sizeof(float)));
			CU(cudaMemset(n->dHlast, 0, (size_t)n->nw * sizeof(float)));
			CU(cudaMalloc(&n->dErrState, (size_t)n->total_nodes * sizeof(float)));
			CU(cudaMemset(n->dErrState, 0, (size_t)n->total_nodes * sizeof(float)));
			n->dropFlags.assign((size_t)n->maskStride, 0);
		}
	}
	else
	{
		CU(cudaMalloc(&n->dG, (n->nw + GL_MAX_WEIGHT_LAYERS + 4) * sizeof(float)));
		CU(cudaMemset(n->dG, 0, (n->nw + GL_MAX_WEIGHT_LAYERS + 4) * sizeof(float)));
		int maxn = 1;
		for (int l = 0; l <= H + 1; ++l) maxn = d->sizes[l] > maxn ? d->sizes[l] : maxn;
		CU(cudaMalloc(&n->dColterm, maxn * sizeof(float)));
		CU(cudaMalloc(&n->dSumPart, SUM_SCALED_MAX_BLOCKS * sizeof(double)));
		CU(cudaMalloc(&n->dSumTicket, sizeof(unsigned)));
		CU(cudaMemset(n->dSumTicket, 0, sizeof(unsigned)));
	}
	if (d->gemm < GL_GEMM_AUTO || d->gemm > GL_GEMM_GRID_FUSED || (d->gemm == GL_GEMM_GRID_FUSED && !grid_fused_fits(n)))
	{
		const bool range = d->gemm < GL_GEMM_AUTO || d->gemm > GL_GEMM_GRID_FUSED;
		gl_destroy(n);
		return fail(GL_ERR_INVALID, range ? "gl_create: bad engine id"
		                                  : "gl_create: the network does not fit the whole-window cooperative kernel (batched mode, "
		                                    "<= 7 hidden layers, layers <= 1024 wide, <= 512 Ki weights)");
	}
	*out = n;
	return GL_OK;
}

static void free_work(gl_net* n)
{
	for (int l = 0; l <= GL_MAX_WEIGHT_LAYERS + 1; ++l)
	{
		if (n->dA[l]) cudaFree(n->dA[l]);
		if (n->dD[l]) cudaFree(n->dD[l]);
		n->dA[l] = n->dD[l] = nullptr;
	}
	for (int l = 0; l < GL_MAX_WEIGHT_LAYERS; ++l)
	{
		if (n->dC[l]) cudaFree(n->dC[l]);
		n->dC[l] = nullptr;
	}
	for (int l = 0; l <= GL_MAX_WEIGHT_LAYERS + 1; ++l)
	{
		if (n->dAlo[l]) cudaFree(n->dAlo[l]);
		if (n->dDlo[l]) cudaFree(n->dDlo[l]);
		n->dAlo[l] = n->dDlo[l] = nullptr;
		if (n->dMask[l]) cudaFree(n->dMask[l]);
		n->dMask[l] = nullptr;
	}
	if (n->dXlo) cudaFree(n->dXlo);
	if (n->dDc) cudaFree(n->dDc);
	if (n->dDclo) cudaFree(n->dDclo);
	n->dXlo = n->dDc = n->dDclo = nullptr;
	if (n->dArgmax) cudaFree(n->dArgmax);
	n->dArgmax = nullptr;
	n->capRows = 0;
	n->cRows = -1;
}

static void dp_push_release(gl_net* n);
static void dp_barrier(gl_net* n)
{
	if (!n->comm || !n->dFlags) return;
	if (g_nccl.AllReduce(n->dFlags + 2, n->dFlags + 2, 1, NCCL_INT32, NCCL_SUM, n->comm, n->stream) == 0) cudaStreamSynchronize(n->stream);
}

extern "C" int gl_destroy(gl_net* n)
{
	if (!n) return GL_OK;
	cudaSetDevice(n->d.device);
	if (n->stream) cudaStreamSynchronize(n->stream);
	if (n->commStream) cudaStreamSynchronize(n->commStream);
	for (int i = 0; i < gl_net::DP_COMM_STREAMS; ++i)
		if (n->layerStream[i]) cudaStreamSynchronize(n->layerStream[i]);
	if (n->dpArena)
	{
		// peers may still be writing into this rank's memory, and this rank maps theirs: meet once
		// before unmapping and once before the memory goes away
		dp_barrier(n);
		dp_push_release(n);
		dp_barrier(n);
	}
	if (n->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(n->comm);
	if (n->commStream) cudaStreamDestroy(n->commStream);
	for (int i = 0; i < gl_net::DP_COMM_STREAMS; ++i)
		if (n->layerStream[i]) cudaStreamDestroy(n->layerStream[i]);
	for (int l = 0; l < GL_MAX_WEIGHT_LAYERS; ++l) if (n->evLayer[l]) cudaEventDestroy(n->evLayer[l]);
	for (int l = 0; l <= GL_MAX_WEIGHT_LAYERS; ++l) if (n->evGrad[l]) cudaEventDestroy(n->evGrad[l]);
	for (int l = 0; l < GL_MAX_WEIGHT_LAYERS; ++l) if (n->evRead[l]) cudaEventDestroy(n->evRead[l]);
	if (n->evComm) cudaEventDestroy(n->evComm);
	free_work(n);
	cudaFree(n->dHlen); cudaFree(n->dHlast); cudaFree(n->dErrState); cudaFree(n->dMasks);
	if (n->snapStream) cudaStreamSynchronize(n->snapStream);
	cudaFree(n->dPreact); cudaFree(n->dSnap);
	if (n->hSnap) cudaFreeHost(n->hSnap);
	if (n->evSnapSrc) cudaEventDestroy(n->evSnapSrc);
	if (n->evSnapCopied) cudaEventDestroy(n->evSnapCopied);
	if (n->evSnapReady) cudaEventDestroy(n->evSnapReady);
	if (n->snapStream) cudaStreamDestroy(n->snapStream);
	cudaFree(n->dpRec);
	cudaFree(n->sk.work); cudaFree(n->sk.flags);
	cudaFree(n->dWlo);
	cudaFree(n->dW); cudaFree(n->dBias); cudaFree(n->dG); cudaFree(n->dBscale); cudaFree(n->dFlags);
	cudaFree(n->dSums); cudaFree(n->dSumsF); cudaFree(n->dConf); cudaFree(n->dHist); cudaFree(n->dHistLen);
	cudaFree(n->dLastOut);
	cudaFree(n->dScratch); cudaFree(n->ownX); cudaFree(n->ownY); cudaFree(n->dColterm); cudaFree(n->dSumPart); cudaFree(n->dSumTicket);
	cudaFree(n->dXwin); cudaFree(n->dYwin);
	if (n->gfTiming)
	{
		unsigned long long tm[16] = {};
		if (cudaMemcpy(tm, n->gfTiming, sizeof tm, cudaMemcpyDeviceToHost) == cudaSuccess)
		{
			fprintf(stderr, "[grid-fused] CTA 0: phase 1 %.3f ms, barrier %.3f ms, phase 2 %.3f ms, barrier %.3f ms\n", tm[0] * 1e-6,
			        tm[1] * 1e-6, tm[2] * 1e-6, tm[3] * 1e-6);
			if (tm[11])
				fprintf(stderr, "[grid-fused] inside phase 1: forward %.3f ms, head %.3f ms, deltas %.3f ms, tail %.3f ms; of which waits for weight tiles %.3f ms, barriers releasing them %.3f ms; thread 0's arithmetic in %llu forward tile steps %.3f ms\n",
				        tm[11] * 1e-6, tm[12] * 1e-6, tm[13] * 1e-6, tm[14] * 1e-6, tm[9] * 1e-6, tm[10] * 1e-6, tm[8], tm[15] * 1e-6);
			if (tm[4])
				fprintf(stderr, "[grid-fused] cluster variant, inside phase 1: weights %.3f ms, forward %.3f ms, head %.3f ms, deltas %.3f ms, pass end %.3f ms\n",
				        tm[4] * 1e-6, tm[5] * 1e-6, tm[6] * 1e-6, tm[7] * 1e-6, tm[8] * 1e-6);
		}
		cudaFree(n->gfTiming);
	}
	cudaFree(n->gfAct); cudaFree(n->gfDel); cudaFree(n->gfPart); cudaFree(n->gfCk); cudaFree(n->gfMaps);
	for (int i = 0; i < 2; ++i)
	{
		cudaFree(n->slot[i].dX); cudaFree(n->slot[i].dY); cudaFree(n->slot[i].dSums);
		if (n->slot[i].hSums) cudaFreeHost(n->slot[i].hSums);
		if (n->slot[i].hArg) cudaFreeHost(n->slot[i].hArg);
		n->slot[i].hArg = nullptr;
		n->slot[i].argCap = 0;
		if (n->slot[i].copied) cudaEventDestroy(n->slot[i].copied);
		if (n->slot[i].done) cudaEventDestroy(n->slot[i].done);
		if (n->slot[i].t0) cudaEventDestroy(n->slot[i].t0);
	}
	if (n->copyStream) cudaStreamDestroy(n->copyStream);
	if (n->hPinned) cudaFreeHost(n->hPinned);
	for (cudaEvent_t e : n->profEv) cudaEventDestroy(e);
	if (n->tim0) cudaEventDestroy(n->tim0);
	if (n->tim1) cudaEventDestroy(n->tim1);
	if (n->ev0) cudaEventDestroy(n->ev0);
	if (n->ev1) cudaEventDestroy(n->ev1);
	if (n->stream) cudaStreamDestroy(n->stream);
	delete n;
	return GL_OK;
}

extern "C" int64_t gl_weight_count(const gl_net* n) { return n ? n->nw : 0; }
extern "C" int gl_get_epochs(const gl_net* n) { return n ? n->epochs : 0; }
extern "C" void gl_stop(gl_net* n) { if (n) n->stop = 1; }

static int ensure_pinned(gl_net* n, size_t bytes)
{
	if (n->pinnedBytes >= bytes) return 0;
	for (int i = 0; i < 2; ++i)
	{
		cudaFree(n->slot[i].dX); cudaFree(n->slot[i].dY); cudaFree(n->slot[i].dSums);
		if (n->slot[i].hSums) cudaFreeHost(n->slot[i].hSums);
		if (n->slot[i].hArg) cudaFreeHost(n->slot[i].hArg);
		n->slot[i].hArg = nullptr;
		n->slot[i].argCap = 0;
		if (n->slot[i].copied) cudaEventDestroy(n->slot[i].copied);
		if (n->slot[i].done) cudaEventDestroy(n->slot[i].done);
		if (n->slot[i].t0) cudaEventDestroy(n->slot[i].t0);
	}
	if (n->copyStream) cudaStreamDestroy(n->copyStream);
	if (n->hPinned) cudaFreeHost(n->hPinned);
	n->hPinned = nullptr;
	n->pinnedBytes = 0;
	CU(cudaMallocHost(&n->hPinned, bytes));
	n->pinnedBytes = bytes;
	return 0;
}

// Host -> device through the pinned staging buffer, in chunks.
static int upload(gl_net* n, float* dst, const float* src, size_t count)
{
	const size_t chunk = (size_t)16 << 20;  // floats per chunk (64 MB)
	if (int r = ensure_pinned(n, (count < chunk ? count : chunk) * sizeof(float))) return r;
	for (size_t off = 0; off < count; off += chunk)
	{
		const size_t c = count - off < chunk ? count - off : chunk;
		memcpy(n->hPinned, src + off, c * sizeof(float));
		CU(cudaMemcpyAsync(dst + off, n->hPinned, c * sizeof(float), cudaMemcpyHostToDevice, n->stream));
		CU(cudaStreamSynchronize(n->stream));
	}
	return 0;
}

extern "C" int gl_set_weights(gl_net* n, const float* w, const float* bias)
{
	if (!n || !w) return fail(GL_ERR_INVALID, "gl_set_weights: null argument");
	if (int r = use_device(n)) return r;
	if (int r = dp_join(n)) return r;
	if (int r = upload(n, n->dW, w, (size_t)n->nw)) return r;
	float b[GL_MAX_WEIGHT_LAYERS] = {0};
	for (int l = 1; l <= n->H; ++l) b[l] = bias ? bias[l - 1] : 0.0f;
	CU(cudaMemcpyAsync(n->dBias, b, sizeof b, cudaMemcpyHostToDevice, n->stream));
	if (n->dHist)
	{
		CU(cudaMemsetAsync(n->dHist, 0, (size_t)n->nw * n->d.batch_size * sizeof(float), n->stream));
		CU(cudaMemsetAsync(n->dHistLen, 0, sizeof(int), n->stream));
	}
	if (n->dropout)
	{
		CU(cudaMemsetAsync(n->dHlen, 0, (size_t)n->nw * sizeof(int), n->stream));
		CU(cudaMemsetAsync(n->dHlast, 0, (size_t)n->nw * sizeof(float), n->stream));
		CU(cudaMemsetAsync(n->dErrState, 0, (size_t)n->total_nodes * sizeof(float), n->stream));
	}
	CU(cudaMemsetAsync(n->dFlags, 0, 4 * sizeof(int), n->stream));
	if (n->dpArena)  // the owners' sticky "non-finite weight" words belong to the old weights
		CU(cudaMemsetAsync(n->dpArena + DP_WORD_BAD * sizeof(unsigned), 0, DP_MAX_WORLD * sizeof(unsigned), n->stream));
	CU(cudaStreamSynchronize(n->stream));
	n->loW = false;
	return GL_OK;
}

extern "C" int gl_get_weights(gl_net* n, float* w, float* bias)
{
	if (!n || !w) return fail(GL_ERR_INVALID, "gl_get_weights: null argument");
	if (int r = use_device(n)) return r;
	if (int r = dp_join(n)) return r;
	CU(cudaStreamSynchronize(n->stream));
	CU(cudaMemcpy(w, n->dW, (size_t)n->nw * sizeof(float), cudaMemcpyDeviceToHost));
	if (bias)
	{
		float b[GL_MAX_WEIGHT_LAYERS];
		CU(cudaMemcpy(b, n->dBias, sizeof b, cudaMemcpyDeviceToHost));
		for (int l = 1; l <= n->H; ++l) bias[l - 1] = b[l];
	}
	return GL_OK;
}


// ---- checkpoint: weights, scalar biases, epoch counter and (reference mode) the pending deltas ----
namespace {
struct StateHeader
{
	char magic[8];  // "GLB200S1"
	int32_t n_layers;
	int32_t sizes[GL_MAX_WEIGHT_LAYERS + 1];
	int32_t mode;
	int32_t batch_size;
	int32_t epochs;
	int32_t hist_len;   // pending deltas per edge (reference mode), 0 otherwise
	int64_t nw;
	int64_t hist_floats;  // floats of pending-delta history that follow the biases
};
}  // namespace

extern "C" int gl_save_state(gl_net* n, const char* path)
{
	if (!n || !path) return fail(GL_ERR_INVALID, "gl_save_state: bad argument");
	if (int r = use_device(n)) return r;
	if (int r = dp_join(n)) return r;
	CU(cudaStreamSynchronize(n->stream));
	StateHeader h;
	memset(&h, 0, sizeof h);
	memcpy(h.magic, "GLB200S1", 8);
	h.n_layers = n->d.n_layers;
	for (int l = 0; l <= n->H + 1; ++l) h.sizes[l] = n->d.sizes[l];
	h.mode = n->d.mode;
	h.batch_size = n->d.batch_size;
	h.epochs = n->epochs;
	h.nw = n->nw;
	if (n->dHist)
	{
		CU(cudaMemcpy(&h.hist_len, n->dHistLen, sizeof(int), cudaMemcpyDeviceToHost));
		h.hist_floats = n->nw * (int64_t)n->d.batch_size;
	}
	std::vector<float> buf((size_t)n->nw + GL_MAX_WEIGHT_LAYERS + (size_t)h.hist_floats);
	CU(cudaMemcpy(buf.data(), n->dW, (size_t)n->nw * sizeof(float), cudaMemcpyDeviceToHost));
	CU(cudaMemcpy(buf.data() + n->nw, n->dBias, GL_MAX_WEIGHT_LAYERS * sizeof(float), cudaMemcpyDeviceToHost));
	if (h.hist_floats)
		CU(cudaMemcpy(buf.data() + n->nw + GL_MAX_WEIGHT_LAYERS, n->dHist, (size_t)h.hist_floats * sizeof(float),
		              cudaMemcpyDeviceToHost));
	// a network with dropout also carries every edge's own history length and last delta, and the error
	// accumulators that survive a row: format "S2", the three arrays appended
	std::vector<float> extra;
	if (n->dropout)
	{
		memcpy(h.magic, "GLB200S2", 8);
		extra.resize((size_t)2 * n->nw + (size_t)n->total_nodes);
		CU(cudaMemcpy(extra.data(), n->dHlen, (size_t)n->nw * sizeof(int), cudaMemcpyDeviceToHost));
		CU(cudaMemcpy(extra.data() + n->nw, n->dHlast, (size_t)n->nw * sizeof(float), cudaMemcpyDeviceToHost));
		CU(cudaMemcpy(extra.data() + 2 * n->nw, n->dErrState, (size_t)n->total_nodes * sizeof(float), cudaMemcpyDeviceToHost));
	}
	FILE* f = fopen(path, "wb");
	if (!f) return fail(GL_ERR_INVALID, "gl_save_state: cannot open %s for writing", path);
	const bool ok = fwrite(&h, sizeof h, 1, f) == 1 && fwrite(buf.data(), sizeof(float), buf.size(), f) == buf.size() &&
	                (extra.empty() || fwrite(extra.data(), sizeof(float), extra.size(), f) == extra.size());
	if (fclose(f) != 0 || !ok) return fail(GL_ERR_INVALID, "gl_save_state: short write to %s", path);
	return GL_OK;
}

extern "C" int gl_load_state(gl_net* n, const char* path)
{
	if (!n || !path) return fail(GL_ERR_INVALID, "gl_load_state: bad argument");
	if (int r = use_device(n)) return r;
	FILE* f = fopen(path, "rb");
	if (!f) return fail(GL_ERR_INVALID, "gl_load_state: cannot open %s", path);
	StateHeader h;
	if (fread(&h, sizeof h, 1, f) != 1 || (memcmp(h.magic, "GLB200S1", 8) != 0 && memcmp(h.magic, "GLB200S2", 8) != 0))
	{
		fclose(f);
		return fail(GL_ERR_INVALID, "gl_load_state: %s is not a state file", path);
	}
	const bool with_dropout = memcmp(h.magic, "GLB200S2", 8) == 0;
	if (with_dropout != n->dropout)
	{
		fclose(f);
		return fail(GL_ERR_INVALID, "gl_load_state: %s was written by a network %s dropout, this one is %s", path,
		            with_dropout ? "with" : "without", n->dropout ? "with" : "without");
	}
	bool same = h.n_layers == n->d.n_layers && h.nw == n->nw && h.mode == n->d.mode && h.batch_size == n->d.batch_size;
	for (int l = 0; same && l <= n->H + 1; ++l) same = h.sizes[l] == n->d.sizes[l];
	const int64_t want_hist = n->dHist ? n->nw * (int64_t)n->d.batch_size : 0;
	if (!same || h.hist_floats != want_hist || h.hist_len < 0 || h.hist_len > n->d.batch_size)
	{
		fclose(f);
		return fail(GL_ERR_INVALID, "gl_load_state: %s was written by a network of another shape, mode or minibatch size", path);
	}
	std::vector<float> buf((size_t)n->nw + GL_MAX_WEIGHT_LAYERS + (size_t)h.hist_floats);
	std::vector<float> extra(with_dropout ? (size_t)2 * n->nw + (size_t)n->total_nodes : 0);
	const bool ok = fread(buf.data(), sizeof(float), buf.size(), f) == buf.size() &&
	                (extra.empty() || fread(extra.data(), sizeof(float), extra.size(), f) == extra.size());
	fclose(f);
	if (!ok) return fail(GL_ERR_INVALID, "gl_load_state: %s is truncated", path);
	// the stored biases are indexed by layer (entry 0 unused); gl_set_weights takes them from hidden layer 1 on.
	// It also clears the history and the status words.
	if (int r = gl_set_weights(n, buf.data(), buf.data() + n->nw + 1)) return r;
	if (h.hist_floats)
	{
		CU(cudaMemcpy(n->dHist, buf.data() + n->nw + GL_MAX_WEIGHT_LAYERS, (size_t)h.hist_floats * sizeof(float),
		              cudaMemcpyHostToDevice));
		CU(cudaMemcpy(n->dHistLen, &h.hist_len, sizeof(int), cudaMemcpyHostToDevice));
	}
	if (with_dropout)
	{
		CU(cudaMemcpy(n->dHlen, extra.data(), (size_t)n->nw * sizeof(int), cudaMemcpyHostToDevice));
		CU(cudaMemcpy(n->dHlast, extra.data() + n->nw, (size_t)n->nw * sizeof(float), cudaMemcpyHostToDevice));
		CU(cudaMemcpy(n->dErrState, extra.data() + 2 * n->nw, (size_t)n->total_nodes * sizeof(float), cudaMemcpyHostToDevice));
	}
	n->epochs = h.epochs;
	return GL_OK;
}

extern "C" int gl_set_data(gl_net* n, const float* x, const float* y, int64_t rows)
{
	if (!n || !x || !y || rows < 1) return fail(GL_ERR_INVALID, "gl_set_data: bad argument");
	if (int r = use_device(n)) return r;
	cudaFree(n->ownX);
	cudaFree(n->ownY);
	n->ownX = n->ownY = nullptr;
	const size_t cx = (size_t)rows * n->d.sizes[0], cy = (size_t)rows * n->n_out;
	CU(cudaMalloc(&n->ownX, cx * sizeof(float)));
	CU(cudaMalloc(&n->ownY, cy * sizeof(float)));
	if (int r = upload(n, n->ownX, x, cx)) return r;
	if (int r = upload(n, n->ownY, y, cy)) return r;
	n->dX = n->ownX;
	n->dY = n->ownY;
	n->rows = rows;
	return GL_OK;
}

extern "C" int gl_set_data_device(gl_net* n, const float* dx, const float* dy, int64_t rows)
{
	if (!n || !dx || rows < 1) return fail(GL_ERR_INVALID, "gl_set_data_device: bad argument");
	n->dX = dx;
	n->dY = dy;
	n->rows = rows;
	return GL_OK;
}

// ---- confusion-matrix figures, CMatrix::updateResultParams + getters (GMath/cmatrix.cpp:100-266)
static void class_metrics(const int* cm, int c, gl_metrics* m)
{
	float acc = 0, prec = 0, rec = 0, spec = 0, f1 = 0;
	for (int k = 0; k < c; ++k)
	{
		long long tp = cm[k * c + k], tn = 0, fp = 0, fn = 0;
		for (int j = 0; j < c; ++j)
			if (j != k)
			{
				tn += cm[j * c + j];
				fp += cm[j * c + k];
				fn += cm[k * c + j];
			}
		const float truth = (float)(int)(tp + tn), untruth = (float)(int)(fp + fn);
		acc += truth / (truth + untruth);
		const float p = ((float)(int)tp) / ((float)(int)(tp + fp));
		const float r = ((float)(int)tp) / ((float)(int)(tp + fn));
		prec += p;
		rec += r;
		spec += ((float)(int)tn) / ((float)(int)(tn + fp));
		f1 += (2.0f * r * p) / (r + p);
	}
	m->class_accuracy = (acc / (float)c) * 100.0f;
	m->class_precision = (prec / (float)c) * 100.0f;
	m->class_recall = (rec / (float)c) * 100.0f;
	m->class_specificity = (spec / (float)c) * 100.0f;
	m->class_f1 = (f1 / (float)c) * 100.0f;
}

static int finish_metrics(gl_net* n, gl_metrics* out, float tot_err, float tot_acc_raw, int64_t rows, float ms,
                          int64_t launches, bool with_class)
{
	if (!out) return 0;
	memset(out, 0, sizeof *out);
	out->total_error = tot_err;
	out->total_accuracy = tot_acc_raw / (((float)rows) * ((float)n->n_out));  // network.cpp:194-195
	out->epochs = n->epochs;
	out->rows = rows;
	out->device_ms = ms;
	out->kernel_launches = launches;
	int flags[4];
	CU(cudaMemcpy(flags, n->dFlags, sizeof flags, cudaMemcpyDeviceToHost));
	out->nonfinite = flags[0] & 1;
	if (with_class && n->d.output_type != GL_OUT_REGRESSION && n->n_out <= 4096)
	{
		std::vector<int> cm((size_t)n->n_out * n->n_out);
		CU(cudaMemcpy(cm.data(), n->dConf, cm.size() * sizeof(int), cudaMemcpyDeviceToHost));
		class_metrics(cm.data(), n->n_out, out);
	}
	return 0;
}

// ------------------------------------------------------------------------------------------------
// reference mode

// Layer::generateDropout (State/layer.cpp:102-134) for one layer of one row: the rate is the integer
// percentage int(p * 100.0f); a rate < 0 or >= 100 draws nothing and leaves the flags as they are;
// otherwise one rand() per node, dropped when rand() % 100 + 1 <= rate, the whole layer drawn again
// while every node came out dropped.
static void draw_layer_flags(unsigned char* flag, int size, float p)
{
	const int rate = (int)(p * 100.0f);
	if (rate < 0 || rate >= 100) return;
	bool all;
	do
	{
		all = true;
		for (int i = 0; i < size; ++i)
		{
			const int dart = (rand() % 100) + 1;
			if (dart <= rate) flag[i] = 1;
			else
			{
				flag[i] = 0;
				all = false;
			}
		}
	} while (all);
}

// LayerBuilder::scrambleDropout (State/LayerBuilder.cpp:497-523) for `rows` consecutive rows: per row the
// input layer first, then the hidden layers in order -- the C library's rand() is consumed exactly as the
// reference consumes it, so after the same srand() the same nodes drop.  Leaves the flags on the device.
static int draw_and_upload_masks(gl_net* n, int64_t rows)
{
	const size_t stride = (size_t)n->maskStride;
	n->hMasks.resize((size_t)rows * stride);
	for (int64_t r = 0; r < rows; ++r)
	{
		int off = 0;
		for (int j = 0; j <= n->H; ++j)
		{
			draw_layer_flags(n->dropFlags.data() + off, n->d.sizes[j], n->d.p_dropout[j]);
			off += n->d.sizes[j];
		}
		memcpy(n->hMasks.data() + (size_t)r * stride, n->dropFlags.data(), stride);
	}
	if (n->maskCapRows < rows)
	{
		cudaFree(n->dMasks);
		n->dMasks = nullptr;
		n->maskCapRows = 0;
		CU(cudaMalloc(&n->dMasks, (size_t)rows * stride));
		n->maskCapRows = rows;
	}
	CU(cudaMemcpyAsync(n->dMasks, n->hMasks.data(), (size_t)rows * stride, cudaMemcpyHostToDevice, n->stream));
	CU(cudaStreamSynchronize(n->stream));  // hMasks is pageable and reused by the next epoch
	return 0;
}

static void fill_dropout_args(gl_net* n, RefTrainArgs& a)
{
	a.masks = n->dMasks;
	a.mask_stride = n->maskStride;
	for (int l = 0; l <= n->H; ++l)
	{
		a.hlen[l] = n->dHlen + n->woff[l];
		a.hlast[l] = n->dHlast + n->woff[l];
	}
	a.err_state = n->dErrState;
}

static int ref_train(gl_net* n, int n_epochs, gl_metrics* out)
{
	if (n->sumsFCap < n_epochs)
	{
		cudaFree(n->dSumsF);
		n->dSumsF = nullptr;
		CU(cudaMalloc(&n->dSumsF, (size_t)2 * n_epochs * sizeof(float)));
		n->sumsFCap = n_epochs;
	}
	RefTrainArgs a;
	memset(&a, 0, sizeof a);
	a.net = make_view(n);
	for (int l = 0; l <= n->H; ++l) a.hist[l] = n->dHist + n->woff[l] * n->d.batch_size;
	a.hist_len = n->dHistLen;
	a.X = n->dX;
	a.Y = n->dY;
	a.rows = n->rows;
	a.n_epochs = n_epochs;
	a.epoch_sums = n->dSumsF;
	a.confusion = n->dConf;
	a.outputs = nullptr;
	a.last_out = n->dLastOut;
	a.flags = n->dFlags;
	a.preact_out = n->dPreact;
	a.weights_in_smem = ref_train_smem_bytes(a.net, true) <= (size_t)227 * 1024;
	if (!a.weights_in_smem && ref_train_smem_bytes(a.net, false) > (size_t)227 * 1024)
		return fail(GL_ERR_TOO_LARGE, "reference mode: %d nodes do not fit the per-sample shared-memory vectors", n->total_nodes);
	float ms = 0;
	int launches = 1;
	if (n->dropout)
	{
		// one launch per epoch: each epoch's node flags are drawn (rand(), the reference's order) before it
		if (ref_train_dropout_smem_bytes(a.net) > (size_t)227 * 1024)
			return fail(GL_ERR_TOO_LARGE, "reference mode with dropout: %d nodes do not fit the per-sample shared-memory vectors", n->total_nodes);
		a.train = 1;
		launches = 0;
		for (int ep = 0; ep < n_epochs && !n->stop; ++ep)
		{
			if (int r = draw_and_upload_masks(n, n->rows)) return r;
			fill_dropout_args(n, a);
			a.epoch_sums = n->dSumsF;
			CU(cudaEventRecord(n->ev0, n->stream));
			CU(launch_ref_train(a, n->stream));
			CU(cudaEventRecord(n->ev1, n->stream));
			CU(cudaStreamSynchronize(n->stream));
			float t = 0;
			CU(cudaEventElapsedTime(&t, n->ev0, n->ev1));
			ms += t;
			++launches;
			n->epochs += 1;
		}
		n->launches += launches;
		float sums[2];
		CU(cudaMemcpy(sums, n->dSumsF, sizeof sums, cudaMemcpyDeviceToHost));
		return finish_metrics(n, out, sums[0], sums[1], n->rows, ms, launches, true);
	}
	CU(cudaEventRecord(n->ev0, n->stream));
	CU(launch_ref_train(a, n->stream));
	CU(cudaEventRecord(n->ev1, n->stream));
	CU(cudaStreamSynchronize(n->stream));
	n->launches += 1;
	n->epochs += n_epochs;
	CU(cudaEventElapsedTime(&ms, n->ev0, n->ev1));
	float sums[2];
	CU(cudaMemcpy(sums, n->dSumsF + 2 * (n_epochs - 1), sizeof sums, cudaMemcpyDeviceToHost));
	return finish_metrics(n, out, sums[0], sums[1], n->rows, ms, 1, true);
}

static int ensure_work(gl_net* n, int64_t rows)
{
	if (rows <= n->capRows) return 0;
	free_work(n);
	for (int l = 1; l <= n->H + 1; ++l)
	{
		CU(cudaMalloc(&n->dA[l], (size_t)rows * n->d.sizes[l] * sizeof(float)));
		if (n->d.mode == GL_MODE_BATCHED) CU(cudaMalloc(&n->dD[l], (size_t)rows * n->d.sizes[l] * sizeof(float)));
	}
	CU(cudaMalloc(&n->dArgmax, (size_t)rows * sizeof(int)));
	if (n->d.mode == GL_MODE_BATCHED && n->d.gemm != GL_GEMM_FFMA)
	{
		int maxn = 1;
		for (int l = 0; l <= n->H + 1; ++l) maxn = n->d.sizes[l] > maxn ? n->d.sizes[l] : maxn;
		CU(cudaMalloc(&n->dXlo, (size_t)rows * n->d.sizes[0] * sizeof(float)));
		for (int l = 1; l <= n->H + 1; ++l)
		{
			CU(cudaMalloc(&n->dAlo[l], (size_t)rows * n->d.sizes[l] * sizeof(float)));
			CU(cudaMalloc(&n->dDlo[l], (size_t)rows * n->d.sizes[l] * sizeof(float)));
			if (l <= n->H && n->d.sizes[l] % 128 == 0 && n->d.activation[l - 1] == GL_ACT_RELU)
				CU(cudaMalloc(&n->dMask[l], (size_t)rows * (n->d.sizes[l] / 32) * sizeof(unsigned)));
		}
		CU(cudaMalloc(&n->dDc, (size_t)rows * maxn * sizeof(float)));
		CU(cudaMalloc(&n->dDclo, (size_t)rows * maxn * sizeof(float)));
		if (!n->dWlo) CU(cudaMalloc(&n->dWlo, (size_t)(n->nw + 4) * sizeof(float)));
		if (!n->sk.work && !(getenv("GLADES_TC_SPLITK") && atoi(getenv("GLADES_TC_SPLITK")) == 0))
		{
			int sms = 0;
			CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, n->d.device));
			CU(cudaMalloc(&n->sk.work, (size_t)sms * 128 * 256 * sizeof(float)));
			CU(cudaMalloc(&n->sk.flags, (size_t)sms * 8 * sizeof(unsigned)));
			CU(cudaMemset(n->sk.flags, 0, (size_t)sms * 8 * sizeof(unsigned)));
			n->sk.epoch = &n->skEpoch;
			n->sk.slots = (size_t)sms;
			n->sk.min_idle_pct = tc_splitk_min_idle_pct();
		}
	}
	n->capRows = rows;
	return 0;
}

// ------------------------------------------------------------------------------------------------
// batched mode
static int set_momentum_weights(gl_net* n, int rows, int global_rows, int first_pos)
{
	if (n->cRows == rows && n->cGlobal == global_rows && n->cFirst == first_pos) return 0;
	std::vector<float> c(rows);
	for (int l = 0; l <= n->H; ++l)
	{
		const double m = (double)n->d.momentum[l];
		if (m == 0.0)
		{
			if (n->dC[l]) cudaFree(n->dC[l]);
			n->dC[l] = nullptr;
			continue;
		}
		// c_j = sum_{t=0}^{global_rows-1-pos} m^t: the closed form of the reference's intra-window
		// momentum history (State/node.cpp:278-292), which restarts at every apply.
		for (int j = 0; j < rows; ++j)
		{
			const int terms = global_rows - (first_pos + j);
			double s = 0.0, pw = 1.0;
			for (int t = 0; t < terms; ++t) { s += pw; pw *= m; if (pw < 1e-30) break; }
			c[j] = (float)s;
		}
		if (n->dC[l]) cudaFree(n->dC[l]);
		CU(cudaMalloc(&n->dC[l], (size_t)n->capRows * sizeof(float)));
		CU(cudaMemcpyAsync(n->dC[l], c.data(), rows * sizeof(float), cudaMemcpyHostToDevice, n->stream));
		CU(cudaStreamSynchronize(n->stream));
	}
	n->cRows = rows;
	n->cGlobal = global_rows;
	n->cFirst = first_pos;
	return 0;
}

// One operand of a layer product: the fp32 matrix it is a slice of, the buffer for that matrix's low
// TF32 part with the flag that says whether it is current, and the slice of the low part to use.
struct Operand
{
	const float* src_all;
	float* lo_all;
	bool* valid;
	long long count_all;
	const float* lo_use;
};

// Runs one layer product on the tensor-core kernel when its shape fits (and the network allows it),
// else on the exact-fp32 FFMA kernel.
static int run_gemm(gl_net* n, GemmArgs g, Operand a, Operand b, int64_t* launches, bool* used_tc = nullptr)
{
	bool tc = false;
	if (n->d.gemm != GL_GEMM_FFMA && a.lo_all && b.lo_all)
	{
		GemmArgs probe = g;
		probe.kscale = nullptr;  // a per-k scale is folded into a scaled operand copy below
		tc = tc_gemm_supported(probe) &&
		     (n->d.gemm == GL_GEMM_TCGEN05 || (long long)g.M * g.N * g.K >= (1ll << 24));
	}
	if (used_tc) *used_tc = tc;
	if (!tc)
	{
		g.C_lo = nullptr;
		g.peer_maps = nullptr;  // the FFMA kernel writes the local C; the caller forwards it
	}
	cudaEvent_t pe0 = nullptr, pe1 = nullptr;
	if (n->profile)
	{
		if (n->profUsed + 2 > n->profEv.size())
		{
			cudaEvent_t a, b;
			CU(cudaEventCreate(&a));
			CU(cudaEventCreate(&b));
			n->profEv.push_back(a);
			n->profEv.push_back(b);
		}
		pe0 = n->profEv[n->profUsed];
		pe1 = n->profEv[n->profUsed + 1];
		n->profUsed += 2;
		n->profFlops.push_back(2.0 * (double)g.M * (double)g.N * (double)g.K);
		n->profIsTc.push_back(tc ? 1 : 0);
		n->profShape.push_back(g.M); n->profShape.push_back(g.N); n->profShape.push_back(g.K); n->profShape.push_back(g.epi);
	}
	if (!tc)
	{
		if (pe0) CU(cudaEventRecord(pe0, n->stream));
		CU(launch_gemm_ffma(g, n->stream));
		if (pe1) CU(cudaEventRecord(pe1, n->stream));
		++*launches;
		return 0;
	}
	if (g.kscale)
	{
		// momentum weights: A(m,k) * c_k becomes a scaled copy of the delta matrix (rows = k)
		CU(launch_scale_split_lo(g.A, g.kscale, (int)g.a_sk, n->dDc, n->dDclo, (long long)g.M * g.K, n->stream));
		++*launches;
		g.A = n->dDc;
		a.lo_use = n->dDclo;
		g.kscale = nullptr;
	}
	else if (!*a.valid)
	{
		CU(launch_split_lo(a.src_all, a.lo_all, a.count_all, n->stream));
		++*launches;
		*a.valid = true;
	}
	if (!*b.valid)
	{
		CU(launch_split_lo(b.src_all, b.lo_all, b.count_all, n->stream));
		++*launches;
		*b.valid = true;
	}
	g.sk = n->sk.work ? &n->sk : nullptr;
	if (pe0) CU(cudaEventRecord(pe0, n->stream));
	CU(launch_gemm_tc(g, a.lo_use, b.lo_use, n->dFlags + 1, n->stream));
	if (pe1) CU(cudaEventRecord(pe1, n->stream));
	++*launches;
	++n->tcLaunches;
	return 0;
}

// Writing the low TF32 part of a product's output from the tensor-core epilogue saves a split pass but
// doubles the epilogue's store burst, which measured slower on the wide-MLP step (185.9 vs 197
// TFLOP/s); it stays off unless GLADES_TC_FUSE_LO=1.  The head and update kernels always fuse theirs.
static bool fuse_lo_in_epilogue()
{
	static int v = -1;
	if (v < 0)
	{
		const char* e = getenv("GLADES_TC_FUSE_LO");
		v = (e && atoi(e) == 1) ? 1 : 0;
	}
	return v == 1;
}

// all weight layers share one flat low-part buffer and one flag: it is refreshed as a whole
static Operand op_w(gl_net* n, int l)
{
	Operand o = {n->dW, n->dWlo, &n->loW, ((n->nw + 3) / 4) * 4, n->dWlo ? n->dWlo + n->woff[l] : nullptr};
	return o;
}
static Operand op_act(gl_net* n, int l, const float* X, int rows)
{
	if (l == 0)
	{
		Operand o = {X, n->dXlo, &n->loX, (long long)rows * n->d.sizes[0], n->dXlo};
		return o;
	}
	Operand o = {n->dA[l], n->dAlo[l], &n->loA[l], (long long)rows * n->d.sizes[l], n->dAlo[l]};
	return o;
}
static Operand op_delta(gl_net* n, int L, int rows)
{
	Operand o = {n->dD[L], n->dDlo[L], &n->loD[L], (long long)rows * n->d.sizes[L], n->dDlo[L]};
	return o;
}

// SMs a data-parallel product leaves free for the exchange kernels that run beside it: as many as
// dpReserveSms, but never so many that the product's tiles need another wave.
static int dp_reserve_for(const gl_net* n, int M, int N)
{
	if (!(n->world > 1 && n->dpOverlap) || n->dpReserveSms <= 0) return 0;
	static int sms = 0;
	if (!sms)
	{
		if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, n->d.device) != cudaSuccess || sms < 1) sms = 148;
	}
	const long long wide = (long long)(M / 128) * (N / 256);
	const long long tiles = (N % 256 == 0 && wide >= 74) ? wide : (long long)(M / 128) * (N / 128);
	if (tiles < 1) return n->dpReserveSms;
	const int floor_r = n->dpReserveSms < 8 ? n->dpReserveSms : 8;
	const long long waves = (tiles + (sms - floor_r) - 1) / (sms - floor_r);
	int r = n->dpReserveSms;
	while (r > floor_r && (tiles + (sms - r) - 1) / (sms - r) > waves) --r;
	return r;
}

// Forward of `rows` rows starting at device pointer X; activations land in dA[1..H+1].
static int batched_forward(gl_net* n, const float* X, int rows, int64_t* launches)
{
	const float* in = X;
	n->loX = false;
	for (int l = 0; l <= n->H; ++l)
	{
		if (int r = dp_wait_layer(n, l)) return r;
		GemmArgs g;
		memset(&g, 0, sizeof g);
		g.A = in;
		g.B = n->dW + n->woff[l];
		g.C = n->dA[l + 1];
		g.M = rows;
		g.N = n->d.sizes[l + 1];
		g.K = n->d.sizes[l];
		g.a_sm = g.K; g.a_sk = 1;
		g.b_sn = g.K; g.b_sk = 1;
		g.ldc = g.N;
		g.epi = EPI_FORWARD;
		g.bias_ptr = (l >= 1) ? n->dBias + l : nullptr;
		g.act = n->d.activation[l];
		g.par = n->d.act_param[l];
		// the tensor-core epilogue also writes the low TF32 part of its output, so the next layer's
		// products need no separate split pass (not for the last layer: the head rewrites it)
		g.C_lo = (l < n->H && fuse_lo_in_epilogue()) ? n->dAlo[l + 1] : nullptr;
		g.relu_mask_out = (l < n->H) ? n->dMask[l + 1] : nullptr;
		g.sm_reserve = dp_reserve_for(n, g.M, g.N);  // the previous window's exchange may still be finishing beside it
		bool tc = false;
		if (int r = run_gemm(n, g, op_act(n, l, X, rows), op_w(n, l), launches, &tc)) return r;
		n->loA[l + 1] = tc && g.C_lo != nullptr;
		n->maskValid[l + 1] = tc && g.relu_mask_out != nullptr;
		in = n->dA[l + 1];
	}
	return 0;
}

// GLADES_DP_TRACE=1 (diagnostics): time stamps of one window's phases on both streams, printed per window.
struct DpTrace
{
	bool on = false;
	std::vector<cudaEvent_t> ev;
	std::vector<std::string> name;
	void mark(const char* what, int l, cudaStream_t s)
	{
		if (!on) return;
		cudaEvent_t e;
		cudaEventCreate(&e);
		cudaEventRecord(e, s);
		ev.push_back(e);
		name.push_back(std::string(what) + (l >= 0 ? std::to_string(l) : std::string()));
	}
	void dump(int rank, cudaStream_t a, cudaStream_t b, cudaStream_t* more, int n_more)
	{
		if (!on) return;
		cudaStreamSynchronize(a);
		if (b) cudaStreamSynchronize(b);
		for (int i = 0; i < n_more; ++i)
			if (more[i]) cudaStreamSynchronize(more[i]);
		for (size_t i = 1; i < ev.size(); ++i)
		{
			float ms = 0;
			cudaEventElapsedTime(&ms, ev[0], ev[i]);
			fprintf(stderr, "[dp-trace r%d] %-18s %8.3f ms\n", rank, name[i].c_str(), ms);
		}
		for (cudaEvent_t e : ev) cudaEventDestroy(e);
		ev.clear();
		name.clear();
	}
};


// Metrics of a finished window step (when the caller wants them): waits for the stream.
static int window_result(gl_net* n, gl_metrics* out, const double* sums2, int global_rows, int64_t launches)
{
	if (out)
	{
		CU(cudaStreamSynchronize(n->stream));
		float ms = 0;
		CU(cudaEventElapsedTime(&ms, n->ev0, n->ev1));
		double sums[2];
		CU(cudaMemcpy(sums, sums2, sizeof sums, cudaMemcpyDeviceToHost));
		memset(out, 0, sizeof *out);
		out->total_error = (float)sums[0];
		out->total_accuracy = (float)(sums[1] / ((double)global_rows * (double)n->n_out));
		out->epochs = n->epochs;
		out->rows = global_rows;
		out->device_ms = ms;
		out->kernel_launches = launches;
		int flags[4];
		CU(cudaMemcpy(flags, n->dFlags, sizeof flags, cudaMemcpyDeviceToHost));
		out->nonfinite = flags[0] & 1;
		if (flags[1])
			return fail(GL_ERR_TIMEOUT, "a bounded wait on the device ran out (code %d: 1-4 tensor-core pipeline, 20+ gradient exchange)", flags[1]);
	}
	return GL_OK;
}

// ---- whole-window cooperative kernel for mid-size networks ----------------------------------------
// Fits: batched mode on one GPU, at most 7 hidden layers, layers at most 1024 wide, at most 512 Ki
// weights (beyond that the per-layer tensor-core products win), shared memory within the SM's limit.
static bool grid_fused_fits(const gl_net* n)
{
	if (n->d.mode != GL_MODE_BATCHED || n->H > 7 || n->nw > (1 << 19)) return false;
	for (int l = 0; l <= n->H + 1; ++l)
		if (n->d.sizes[l] > 1024) return false;
	const NetView v = make_view(n);
	return grid_fused_smem_bytes(v) <= (size_t)220 * 1024;
}
static bool grid_fused_ok(gl_net* n)
{
	if (n->world > 1) return false;
	if (n->gfOk < 0)
	{
		const char* e = getenv("GLADES_GRID_FUSED");
		const bool allowed = n->d.gemm == GL_GEMM_GRID_FUSED || (n->d.gemm == GL_GEMM_AUTO && !(e && atoi(e) == 0));
		n->gfOk = (allowed && grid_fused_fits(n)) ? 1 : 0;
	}
	return n->gfOk == 1;
}

// Runs `n_epochs` passes over `rows` rows (windows of `mb`) in one cooperative launch; sums of the
// last epoch land in sums_out[0..1] on the device.
static int grid_fused_launch(gl_net* n, const float* X, const float* Y, int64_t rows, int mb, int n_epochs, int64_t metric_rows,
                             double* epoch_sums)
{
	const NetView base = make_view(n);
	const int tot = grid_fused_scratch_pitch(base);
	if (n->gfRows < mb)
	{
		cudaFree(n->gfAct);
		cudaFree(n->gfDel);
		n->gfAct = n->gfDel = nullptr;
		n->gfRows = 0;
		CU(cudaMalloc(&n->gfAct, (size_t)mb * tot * sizeof(float)));
		CU(cudaMalloc(&n->gfDel, (size_t)mb * tot * sizeof(float)));
		n->gfRows = mb;
	}
	if (!n->gfPart)
	{
		int sms = 0;
		CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, n->d.device));
		n->gfCtas = sms;
		CU(cudaMalloc(&n->gfPart, (size_t)sms * (2 + GL_MAX_WEIGHT_LAYERS) * sizeof(double)));
	}
	if (n->gfClusterCtas < 0)
	{
		// the cluster variant only on request (GLADES_GF_CLUSTER=1; it measured slower than the plain kernel), where the
		// network allows it and the device can hold whole clusters
		const char* e = getenv("GLADES_GF_CLUSTER");
		int ctas = 0;
		if (e && atoi(e) == 1 && cluster_fused_fits(base))
		{
			bool aligned = true;
			for (int l = 0; l <= n->H; ++l) aligned = aligned && n->woff[l] % 4 == 0;
			if (aligned) ctas = cluster_fused_max_ctas(base);
			if (ctas > n->gfCtas) ctas = (n->gfCtas / 8) * 8;
		}
		n->gfClusterCtas = ctas >= 16 ? ctas : 0;
	}
	if (!n->gfMapsTried)
	{
		// weight tiles by bulk tensor copies where every layer's rows are multiples of 16 bytes
		n->gfMapsTried = true;
		const char* e = getenv("GLADES_GF_TMA");
		bool ok = !(e && atoi(e) == 0) && grid_fused_group_tiles(base) <= 512;
		for (int l = 0; ok && l <= n->H; ++l) ok = n->d.sizes[l] % 4 == 0 && n->woff[l] % 4 == 0;
		if (ok)
		{
			std::vector<unsigned char> raw((size_t)2 * (n->H + 1) * 128 + 64);
			unsigned char* maps = raw.data() + ((64 - ((uintptr_t)raw.data() & 63)) & 63);
			for (int l = 0; ok && l <= n->H; ++l)
			{
				const int ni = n->d.sizes[l], no = n->d.sizes[l + 1];
				ok = tc_make_map2d(maps + (size_t)(2 * l) * 128, n->dW + n->woff[l], no, ni, ni, 32, 256, 1) &&
				     tc_make_map2d(maps + (size_t)(2 * l + 1) * 128, n->dW + n->woff[l], no, ni, ni, 256, 32, 0);
			}
			if (ok)
			{
				CU(cudaMalloc(&n->gfMaps, (size_t)2 * (n->H + 1) * 128));
				CU(cudaMemcpy(n->gfMaps, maps, (size_t)2 * (n->H + 1) * 128, cudaMemcpyHostToDevice));
			}
		}
	}
	if (n->gfCkMb != mb)
	{
		// ck[l][k] = sum_{q<k} m_l^q, summed like the per-sample momentum history builds it up
		std::vector<float> ck((size_t)(n->H + 1) * (mb + 1));
		for (int l = 0; l <= n->H; ++l)
		{
			const double m = (double)n->d.momentum[l];
			double sum = 0.0, pw = 1.0;
			for (int k = 0; k <= mb; ++k)
			{
				ck[(size_t)l * (mb + 1) + k] = (m == 0.0) ? (k > 0 ? 1.0f : 0.0f) : (float)sum;
				sum += pw;
				pw *= m;
			}
		}
		cudaFree(n->gfCk);
		n->gfCk = nullptr;
		n->gfCkMb = 0;
		CU(cudaMalloc(&n->gfCk, ck.size() * sizeof(float)));
		CU(cudaMemcpyAsync(n->gfCk, ck.data(), ck.size() * sizeof(float), cudaMemcpyHostToDevice, n->stream));
		CU(cudaStreamSynchronize(n->stream));
		n->gfCkMb = mb;
	}
	GridFusedArgs a;
	memset(&a, 0, sizeof a);
	a.net = base;
	a.net.mb = mb;
	a.X = X;
	a.Y = Y;
	a.rows = rows;
	a.n_epochs = n_epochs;
	a.bias_rule = n->d.bias_rule;
	a.data_size = (float)(metric_rows * (int64_t)n->n_out);
	a.actbuf = n->gfAct;
	a.delbuf = n->gfDel;
	a.part = n->gfPart;
	a.part_ctas = n->gfCtas;
	a.ck = n->gfCk;
	a.tma = n->gfMaps;
	a.epoch_sums = epoch_sums;
	a.confusion = n->dConf;
	a.last_out = n->dLastOut;
	a.flags = n->dFlags;
	static int want_timing = -1;
	if (want_timing < 0) want_timing = getenv("GLADES_GF_TIMING") ? 1 : 0;
	if (want_timing && !n->gfTiming)
	{
		CU(cudaMalloc(&n->gfTiming, 16 * sizeof(unsigned long long)));
		CU(cudaMemset(n->gfTiming, 0, 16 * sizeof(unsigned long long)));
	}
	a.timing = n->gfTiming;
	const bool cluster = n->gfClusterCtas > 0 && (((uintptr_t)X | (uintptr_t)Y) & 15) == 0;
	if (cluster) a.part_ctas = n->gfClusterCtas;
	cudaError_t e = cluster ? launch_cluster_fused(a, n->stream) : launch_grid_fused(a, n->stream);
	if (e != cudaSuccess)
		return fail(GL_ERR_CUDA, "whole-window cooperative kernel%s: %s", cluster ? " (cluster variant)" : "", cudaGetErrorString(e));
	n->loW = false;
	return GL_OK;
}

static int batched_window(gl_net* n, const float* X, const float* Y, int rows, int64_t metric_rows, gl_metrics* out)
{
	DpTrace tr;
	{
		static int t = -1;
		if (t < 0) t = getenv("GLADES_DP_TRACE") ? 1 : 0;
		tr.on = t == 1 && n->world > 1;
	}
	const int global_rows = (n->world > 1 && n->globalRows > 0) ? n->globalRows : rows;
	double* const sums2 = n->winSums ? n->winSums : n->dSums;
	int64_t launches = 0;
	if (grid_fused_ok(n))
	{
		// mid-size network on one GPU: the whole window in one cooperative launch
		CU(cudaEventRecord(n->ev0, n->stream));
		if (int r = grid_fused_launch(n, X, Y, rows, rows, 1, metric_rows, sums2)) return r;
		CU(cudaEventRecord(n->ev1, n->stream));
		launches = 1;
		n->launches += launches;
		n->lastWindowLaunches = launches;
		return window_result(n, out, sums2, global_rows, launches);
	}
	if (int r = ensure_work(n, rows)) return r;
	const int first_pos = (n->world > 1) ? n->firstPos : 0;
	if (int r = set_momentum_weights(n, rows, global_rows, first_pos)) return r;
	const bool push = n->world > 1 && n->dpPush;
	bool lo_all = true;  // peer-memory exchange: every layer's low weight parts were refreshed beside the backward pass
	const unsigned stepv = push ? ++n->dpStep : 0u;
	DpPeers peerFlags, peerStage;
	for (int r = 0; r < DP_MAX_WORLD; ++r)
	{
		peerFlags.p[r] = n->dpPeerArena[r];
		peerStage.p[r] = n->dpPeerArena[r] ? static_cast<char*>(n->dpPeerArena[r]) + n->dpStageOff : nullptr;
	}
	CU(cudaEventRecord(n->ev0, n->stream));
	tr.mark("start", -1, n->stream);
	CU(cudaMemsetAsync(sums2, 0, 2 * sizeof(double), n->stream));
	CU(cudaMemsetAsync(n->dG + n->nw, 0, GL_MAX_WEIGHT_LAYERS * sizeof(float), n->stream));
	if (int r = batched_forward(n, X, rows, &launches)) return r;
	tr.mark("forward done", -1, n->stream);

	HeadArgs h;
	memset(&h, 0, sizeof h);
	h.P = n->dA[n->H + 1];
	h.Y = Y;
	h.D = n->dD[n->H + 1];
	h.D_lo = n->dDlo[n->H + 1];
	h.rows = rows;
	h.n = n->n_out;
	h.out_type = n->d.output_type;
	h.softmax = n->softmax;
	h.data_size = (float)(metric_rows * (int64_t)n->n_out);
	h.sums2 = sums2;
	h.confusion = (n->d.output_type != GL_OUT_REGRESSION) ? n->dConf : nullptr;
	CU(launch_head(h, n->stream));
	++launches;
	n->loD[n->H + 1] = n->dDlo[n->H + 1] != nullptr;
	n->loA[n->H + 1] = false;  // the softmax head rewrote the last activations in place
	CU(cudaMemcpyAsync(n->dLastOut, n->dA[n->H + 1] + (size_t)(rows - 1) * n->n_out, (size_t)n->n_out * sizeof(float),
	                   cudaMemcpyDeviceToDevice, n->stream));

	// ---- backward pass: two kinds of product per layer, as lambdas so that the order can depend on the exchange
	// D_{L-1} = (D_L W_{L-1}) * act'(A_{L-1}): the one product of the backward pass that reads W_{L-1}
	auto errprop = [&](int L) -> int {
		const int l = L - 1;
		const int ni = n->d.sizes[l], no = n->d.sizes[L];
		GemmArgs g;
		memset(&g, 0, sizeof g);
		g.A = n->dD[L]; g.a_sm = no; g.a_sk = 1;
		g.B = n->dW + n->woff[l]; g.b_sn = 1; g.b_sk = ni;
		g.C = n->dD[l]; g.ldc = ni;
		g.M = rows; g.N = ni; g.K = no;
		g.epi = EPI_ERRPROP;
		g.aux = n->dA[l]; g.ld_aux = ni;
		g.act = n->d.activation[l - 1];
		g.par = 0.01f;  // the reference passes a fixed 0.01, network.cpp:618
		g.C_lo = fuse_lo_in_epilogue() ? n->dDlo[l] : nullptr;
		g.relu_mask_in = n->maskValid[l] ? n->dMask[l] : nullptr;
		g.sm_reserve = dp_reserve_for(n, g.M, g.N);
		bool tc = false;
		if (int r = run_gemm(n, g, op_delta(n, L, rows), op_w(n, l), &launches, &tc)) return r;
		n->loD[l] = tc && g.C_lo != nullptr;
		if (push) CU(cudaEventRecord(n->evRead[l], n->stream));  // the old W_l is not read again in this window
		return 0;
	};
	// G_l = D_{l+1}^T A_l (times learning rate, plus decay terms); under data parallelism followed by the first half
	// of the layer's exchange.  `last`: no product follows, the owner's update may take the whole GPU.
	auto gradient = [&](int l, bool last) -> int {
		const int L = l + 1;
		const int ni = n->d.sizes[l], no = n->d.sizes[L];
		const float* Al = (l == 0) ? X : n->dA[l];
		const Operand opD = op_delta(n, L, rows);
		const float* colterm = nullptr;
		bool fused_store = false;
		if (n->d.wd1[l] != 0.0f || n->d.wd2[l] != 0.0f)
		{
			CU(launch_decay_colterm(Al, rows, ni, n->dC[l], n->d.lr[l], n->d.wd1[l], n->d.wd2[l], n->dColterm, n->stream));
			++launches;
			colterm = n->dColterm;
		}
		{
			GemmArgs g;
			memset(&g, 0, sizeof g);
			g.A = n->dD[L]; g.a_sm = 1; g.a_sk = no;
			g.B = Al; g.b_sn = 1; g.b_sk = ni;
			g.C = n->dG + n->woff[l]; g.ldc = ni;
			g.M = no; g.N = ni; g.K = rows;
			g.kscale = n->dC[l];
			g.epi = EPI_GRAD;
			g.alpha = n->d.lr[l];
			g.colterm = colterm;
			g.sm_reserve = dp_reserve_for(n, no, ni);
			if (push && n->dpStoreMode == 0)
			{
				// the tensor-core epilogue stores every row band straight into its owner's memory
				g.peer_maps = static_cast<const char*>(n->dpMaps) + (size_t)l * DP_MAX_WORLD * 128;
				g.peer_bases = n->dpBases + (size_t)l * DP_MAX_WORLD;
				g.band_rows = n->dpBand[l];
				g.peer_self = n->rank;
			}
			bool gtc = false;
			if (int r = run_gemm(n, g, opD, op_act(n, l, X, rows), &launches, &gtc)) return r;
			fused_store = push && n->dpStoreMode == 0;
			if (fused_store && !gtc)
			{
				DpPeers slot;
				for (int o = 0; o < DP_MAX_WORLD; ++o) slot.p[o] = n->hostBases[l][o];
				CU(launch_dp_push_bands(n->dG + n->woff[l], no, ni, n->dpBand[l], slot, n->stream));
				++launches;
			}
		}
		if (l >= 1)
		{
			CU(launch_sum_scaled(n->dD[L], (int64_t)rows * no, n->d.lr[l], n->dG + n->nw + l, n->dSumPart, n->dSumTicket, n->stream));
			++launches;
		}
		if (push)
		{
			// this rank's contributions to layer l have been stored at their owners: tell them, and let the
			// layer's exchange stream do this rank's own band (sum the sources in rank order, update, write the
			// new weights into every replica's STAGING vector) while the compute stream goes on
			cudaStream_t cs = n->layerStream[l % gl_net::DP_COMM_STREAMS];
			if (fused_store)
			{
				CU(launch_dp_signal(peerFlags, n->world, DP_WORD_GFLAG + l * DP_MAX_WORLD + n->rank, stepv, n->stream));
				tr.mark("grad stored L", l, n->stream);
				CU(cudaEventRecord(n->evGrad[l], n->stream));
				CU(cudaStreamWaitEvent(cs, n->evGrad[l], 0));
			}
			else
			{
				// the product wrote the gradient locally; its bands travel to their owners on the layer's exchange
				// stream, beside the next products: by a copy kernel (mode 1) or by the copy engines (mode 2)
				CU(cudaEventRecord(n->evGrad[l], n->stream));
				CU(cudaStreamWaitEvent(cs, n->evGrad[l], 0));
				if (n->dpStoreMode == 1)
				{
					DpPeers slot;
					for (int o = 0; o < DP_MAX_WORLD; ++o) slot.p[o] = n->hostBases[l][o];
					CU(launch_dp_push_bands(n->dG + n->woff[l], no, ni, n->dpBand[l], slot, cs));
					++launches;
				}
				else
				{
					const int band = n->dpBand[l];
					for (int k = 0; k < n->world; ++k)
					{
						const int o = (n->rank + 1 + k) % n->world;  // every rank starts with another owner
						int rows_o = no - o * band;
						rows_o = rows_o < 0 ? 0 : (rows_o > band ? band : rows_o);
						if (rows_o > 0)
							CU(cudaMemcpyAsync(n->hostBases[l][o], n->dG + n->woff[l] + (size_t)o * band * ni, (size_t)rows_o * ni * sizeof(float),
							                   cudaMemcpyDeviceToDevice, cs));
					}
				}
				CU(launch_dp_signal(peerFlags, n->world, DP_WORD_GFLAG + l * DP_MAX_WORLD + n->rank, stepv, cs));
				tr.mark("grad stored L", l, cs);
			}
			CU(launch_dp_wait(n->dpArena, DP_WORD_GFLAG + l * DP_MAX_WORLD, 1, n->world, 0, 0, stepv, n->dFlags + 1, 20 + l, cs));
			tr.mark("owner has all L", l, cs);
			const int band = n->dpBand[l];
			int own_rows = no - n->rank * band;
			own_rows = own_rows < 0 ? 0 : (own_rows > band ? band : own_rows);
			const float* part = reinterpret_cast<const float*>(n->dpArena + DP_FLAG_BYTES) + n->dpSlotOff[l];
			CU(launch_dp_reduce_update(part, n->dpSlotOff[n->H + 1], n->world, (long long)own_rows * ni, 1.0f / (float)global_rows,
			                           n->woff[l] + (long long)n->rank * band * ni, n->dW, peerStage, n->rank, peerFlags,
			                           last ? 148 * 4 : n->dpPushBlocks, cs));
			CU(launch_dp_signal(peerFlags, n->world, DP_WORD_WFLAG + l * DP_MAX_WORLD + n->rank, stepv, cs));
			tr.mark("band updated L", l, cs);
			launches += 4;
		}
		else if (n->world > 1 && n->dpOverlap)
		{
			// this layer's gradient is complete: reduce it on the communication stream while the compute
			// stream goes on with the other gradients
			CU(cudaEventRecord(n->evGrad[l], n->stream));
			CU(cudaStreamWaitEvent(n->commStream, n->evGrad[l], 0));
			NC(g_nccl.AllReduce(n->dG + n->woff[l], n->dG + n->woff[l], (size_t)(n->woff[l + 1] - n->woff[l]), NCCL_FLOAT32,
			                    NCCL_SUM, n->comm, n->commStream));
		}
		return 0;
	};
	if (push)
	{
		// Exchange over peer memory: the owners write a layer's new weights into staging vectors, so nothing that
		// this window still reads is overwritten and every gradient can be taken as early as its delta exists --
		// hidden layers from the top (each preceded by the error propagation that makes its delta), the output
		// layer's gradient last: its weights are the last ones the next window's forward pass needs, so its
		// exchange has the longest stretch to hide under.  The largest exchanges thus start early and run under the
		// rest of the backward pass instead of piling up on NVLink behind the last product.
		for (int l = n->H - 1; l >= 0; --l)
		{
			if (int r = errprop(l + 2)) return r;
			if (int r = gradient(l, false)) return r;
		}
		tr.mark("deltas done", -1, n->stream);
		if (int r = gradient(n->H, true)) return r;
		// second half of every layer's exchange, queued now that this window's readers of the old weights are all
		// on the compute stream: once every owner's band of layer l has landed in this rank's staging vector and
		// the product that read the old W_l has finished, copy the layer into the weights (splitting off the low
		// TF32 parts on the way); evLayer[l] then releases the next product that reads W_l
		const float* stage = reinterpret_cast<const float*>(n->dpArena + n->dpStageOff);
		for (int k = 0; k <= n->H; ++k)
		{
			const int l = (k < n->H) ? n->H - 1 - k : n->H;  // the order the exchanges were started in
			cudaStream_t cs = n->layerStream[l % gl_net::DP_COMM_STREAMS];
			CU(launch_dp_wait(n->dpArena, DP_WORD_WFLAG + l * DP_MAX_WORLD, 1, n->world, 0, 0, stepv, n->dFlags + 1, 40 + l, cs));
			if (l >= 1) CU(cudaStreamWaitEvent(cs, n->evRead[l], 0));
			const int64_t cnt = n->woff[l + 1] - n->woff[l];
			if (n->dWlo && cnt % 4 == 0 && n->woff[l] % 4 == 0)
				CU(launch_copy_split_lo(stage + n->woff[l], n->dW + n->woff[l], n->dWlo + n->woff[l], cnt, cs));
			else
			{
				CU(cudaMemcpyAsync(n->dW + n->woff[l], stage + n->woff[l], (size_t)cnt * sizeof(float), cudaMemcpyDeviceToDevice, cs));
				lo_all = false;
			}
			tr.mark("layer complete L", l, cs);
			CU(cudaEventRecord(n->evLayer[l], cs));
			n->layerPending[l] = true;
			launches += 2;
		}
	}
	else
	{
		// Error propagation first, down the whole chain: D_{H+1} -> D_H -> ... -> D_1, then the weight gradients,
		// largest layer first (with the NCCL exchange each one starts its layer's all-reduce, and the largest one
		// gets the remaining products to hide under; the weights change only after all of them, in launch_update)
		for (int L = n->H + 1; L >= 2; --L)
			if (int r = errprop(L)) return r;
		tr.mark("deltas done", -1, n->stream);
		int order[GL_MAX_WEIGHT_LAYERS];
		for (int l = 0; l <= n->H; ++l) order[l] = l;
		for (int i = 1; i <= n->H; ++i)
			for (int j = i; j > 0 && (n->woff[order[j] + 1] - n->woff[order[j]]) > (n->woff[order[j - 1] + 1] - n->woff[order[j - 1]]); --j)
			{
				const int t = order[j];
				order[j] = order[j - 1];
				order[j - 1] = t;
			}
		for (int oi = 0; oi <= n->H; ++oi)
			if (int r = gradient(order[oi], oi == n->H)) return r;
	}
	if (n->world > 1 && !push)
	{
		if (n->dpOverlap)
		{
			CU(cudaEventRecord(n->evGrad[GL_MAX_WEIGHT_LAYERS], n->stream));
			CU(cudaStreamWaitEvent(n->commStream, n->evGrad[GL_MAX_WEIGHT_LAYERS], 0));
			NC(g_nccl.GroupStart());
			NC(g_nccl.AllReduce(n->dG + n->nw, n->dG + n->nw, (size_t)GL_MAX_WEIGHT_LAYERS, NCCL_FLOAT32, NCCL_SUM, n->comm, n->commStream));
			NC(g_nccl.AllReduce(sums2, sums2, 2, NCCL_FLOAT64, NCCL_SUM, n->comm, n->commStream));
			NC(g_nccl.GroupEnd());
			CU(cudaEventRecord(n->evComm, n->commStream));
			CU(cudaStreamWaitEvent(n->stream, n->evComm, 0));
		}
		else
		{
			NC(g_nccl.GroupStart());
			NC(g_nccl.AllReduce(n->dG, n->dG, (size_t)(n->nw + GL_MAX_WEIGHT_LAYERS), NCCL_FLOAT32, NCCL_SUM, n->comm, n->stream));
			NC(g_nccl.AllReduce(sums2, sums2, 2, NCCL_FLOAT64, NCCL_SUM, n->comm, n->stream));
			NC(g_nccl.GroupEnd());
		}
	}
	if (n->bscaleRows != global_rows)
	{
		float bscale[GL_MAX_WEIGHT_LAYERS] = {0};
		for (int l = 1; l <= n->H; ++l)
			bscale[l] = (n->d.bias_rule == GL_BIAS_REFERENCE) ? (float)n->d.sizes[l] : 1.0f / (float)global_rows;
		CU(cudaMemcpyAsync(n->dBscale, bscale, sizeof bscale, cudaMemcpyHostToDevice, n->stream));
		CU(cudaStreamSynchronize(n->stream));
		n->bscaleRows = global_rows;
	}
	if (push)
	{
		// bias and loss sums of this rank to everyone; then wait until every owner's band of every layer
		// and every rank's record have landed here, and finish the window locally
		CU(launch_dp_small_push(n->dG + n->nw, sums2, peerFlags, n->world, n->rank, (int)(stepv & 1u), stepv, n->stream));
		tr.mark("backward done", -1, n->stream);
		CU(launch_dp_wait(n->dpArena, 0, 0, 0, DP_WORD_SFLAG, n->world, stepv, n->dFlags + 1, 60, n->stream));
		// (the layers' new weights are NOT awaited here: the next product that reads W_l waits for evLayer[l],
		// so the end of the exchange runs under the next window's forward pass; see dp_wait_layer / dp_join)
		CU(launch_dp_finish(n->dpArena, n->world, (int)(stepv & 1u), n->dG + n->nw, sums2, n->dBias, n->dBscale, n->H, n->dFlags,
		                    n->stream));
		tr.mark("window done", -1, n->stream);
		launches += 3;
		n->loW = lo_all && n->dWlo != nullptr;
		// a network with a layer whose low parts cannot be split per layer refreshes them as a whole before its
		// next tensor-core product, which reads every layer's weights: all layers must have landed by then
		if (!lo_all)
			if (int r = dp_join(n)) return r;
	}
	else
	{
		CU(launch_update(n->dW, n->dWlo, n->dG, n->nw, 1.0f / (float)global_rows, n->dBias, n->dG + n->nw, n->dBscale, n->H,
		                 n->dFlags, n->stream));
		++launches;
		n->loW = n->dWlo != nullptr;
	}
	CU(cudaEventRecord(n->ev1, n->stream));
	tr.dump(n->rank, n->stream, n->commStream, n->layerStream, gl_net::DP_COMM_STREAMS);
	n->launches += launches;
	n->lastWindowLaunches = launches;
	return window_result(n, out, sums2, global_rows, launches);
}

extern "C" int gl_train_window(gl_net* n, int64_t first_row, int32_t rows, gl_metrics* out)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_train_window: null handle");
	if (n->d.mode != GL_MODE_BATCHED) return fail(GL_ERR_STATE, "gl_train_window needs a batched-mode network");
	if (!n->dX || !n->dY) return fail(GL_ERR_STATE, "gl_train_window: no data (inputs and expected rows) set");
	if (first_row < 0 || rows < 1 || first_row + rows > n->rows) return fail(GL_ERR_INVALID, "gl_train_window: row range");
	if (int r = use_device(n)) return r;
	// the cost divisor of a single window call is that window's global row count
	const int64_t win_rows = (n->world > 1 && n->globalRows > 0) ? n->globalRows : rows;
	return batched_window(n, n->dX + first_row * n->d.sizes[0], n->dY + first_row * n->n_out, rows, win_rows, out);
}

static int ensure_window_staging(gl_net* n, int64_t rows)
{
	if (rows <= n->winCap) return 0;
	cudaFree(n->dXwin);
	cudaFree(n->dYwin);
	n->dXwin = n->dYwin = nullptr;
	CU(cudaMalloc(&n->dXwin, (size_t)rows * n->d.sizes[0] * sizeof(float)));
	CU(cudaMalloc(&n->dYwin, (size_t)rows * n->n_out * sizeof(float)));
	n->winCap = rows;
	return 0;
}

extern "C" int gl_train_window_host(gl_net* n, const float* x, const float* y, int32_t rows, gl_metrics* out)
{
	if (!n || !x || !y || rows < 1) return fail(GL_ERR_INVALID, "gl_train_window_host: bad argument");
	if (n->d.mode != GL_MODE_BATCHED) return fail(GL_ERR_STATE, "gl_train_window_host needs a batched-mode network");
	if (int r = use_device(n)) return r;
	if (int r = ensure_window_staging(n, rows)) return r;
	// the caller's buffers are read directly by the copy engine (fast when they are pinned)
	CU(cudaMemcpyAsync(n->dXwin, x, (size_t)rows * n->d.sizes[0] * sizeof(float), cudaMemcpyHostToDevice, n->stream));
	CU(cudaMemcpyAsync(n->dYwin, y, (size_t)rows * n->n_out * sizeof(float), cudaMemcpyHostToDevice, n->stream));
	const int64_t win_rows = (n->world > 1 && n->globalRows > 0) ? n->globalRows : rows;
	return batched_window(n, n->dXwin, n->dYwin, rows, win_rows, out);
}

// ---- pipelined host-buffer windows ------------------------------------------------------------------
// submit() queues the copy of the window's rows on a copy stream and the step on the compute stream and
// returns at once; result() waits for the oldest submitted window.  Two windows may be in flight, so the
// copy of window i+1 overlaps the compute of window i.
static int slot_prepare(gl_net* n, gl_net::Slot& sl, int64_t rows)
{
	if (!sl.copied)
	{
		CU(cudaEventCreateWithFlags(&sl.copied, cudaEventDisableTiming));
		CU(cudaEventCreate(&sl.done));
		CU(cudaEventCreate(&sl.t0));
		CU(cudaMalloc(&sl.dSums, 2 * sizeof(double)));
		CU(cudaMallocHost(&sl.hSums, 4 * sizeof(double)));
	}
	if (rows > sl.cap)
	{
		cudaFree(sl.dX);
		cudaFree(sl.dY);
		sl.dX = sl.dY = nullptr;
		CU(cudaMalloc(&sl.dX, (size_t)rows * n->d.sizes[0] * sizeof(float)));
		CU(cudaMalloc(&sl.dY, (size_t)rows * n->n_out * sizeof(float)));
		sl.cap = rows;
	}
	return 0;
}

extern "C" int gl_train_window_host_submit(gl_net* n, const float* x, const float* y, int32_t rows)
{
	if (!n || !x || !y || rows < 1) return fail(GL_ERR_INVALID, "gl_train_window_host_submit: bad argument");
	if (n->d.mode != GL_MODE_BATCHED) return fail(GL_ERR_STATE, "gl_train_window_host_submit needs a batched-mode network");
	if (n->submitted - n->collected >= 2) return fail(GL_ERR_STATE, "two windows are already in flight: collect a result first");
	if (int r = use_device(n)) return r;
	if (!n->copyStream) CU(cudaStreamCreateWithFlags(&n->copyStream, cudaStreamNonBlocking));
	gl_net::Slot& sl = n->slot[n->submitted & 1];
	const bool used_before = sl.copied != nullptr;
	if (int r = slot_prepare(n, sl, rows)) return r;
	// the slot's buffers are free once the step that last read them has finished
	if (used_before) CU(cudaStreamWaitEvent(n->copyStream, sl.done, 0));
	CU(cudaMemcpyAsync(sl.dX, x, (size_t)rows * n->d.sizes[0] * sizeof(float), cudaMemcpyHostToDevice, n->copyStream));
	CU(cudaMemcpyAsync(sl.dY, y, (size_t)rows * n->n_out * sizeof(float), cudaMemcpyHostToDevice, n->copyStream));
	CU(cudaEventRecord(sl.copied, n->copyStream));
	CU(cudaStreamWaitEvent(n->stream, sl.copied, 0));
	CU(cudaEventRecord(sl.t0, n->stream));
	const int64_t win_rows = (n->world > 1 && n->globalRows > 0) ? n->globalRows : rows;
	n->winSums = sl.dSums;
	const int st = batched_window(n, sl.dX, sl.dY, rows, win_rows, nullptr);
	n->winSums = nullptr;
	if (st != GL_OK) return st;
	CU(cudaMemcpyAsync(sl.hSums, sl.dSums, 2 * sizeof(double), cudaMemcpyDeviceToHost, n->stream));
	CU(cudaMemcpyAsync(sl.hSums + 2, n->dFlags, 4 * sizeof(int), cudaMemcpyDeviceToHost, n->stream));
	CU(cudaEventRecord(sl.done, n->stream));
	sl.rows = rows;
	sl.globalRows = (int)win_rows;
	sl.launches = n->lastWindowLaunches;
	sl.pending = true;
	sl.infer = false;
	++n->submitted;
	return GL_OK;
}

extern "C" int gl_train_window_host_result(gl_net* n, gl_metrics* out)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_train_window_host_result: null handle");
	if (n->submitted == n->collected) return fail(GL_ERR_STATE, "no window in flight");
	if (int r = use_device(n)) return r;
	gl_net::Slot& sl = n->slot[n->collected & 1];
	if (sl.infer) return fail(GL_ERR_STATE, "the oldest call in flight is an inference batch: collect it with gl_forward_host_result");
	CU(cudaEventSynchronize(sl.done));
	sl.pending = false;
	++n->collected;
	int flags[4];
	memcpy(flags, sl.hSums + 2, sizeof flags);
	if (out)
	{
		float ms = 0;
		CU(cudaEventElapsedTime(&ms, sl.t0, sl.done));
		memset(out, 0, sizeof *out);
		out->total_error = (float)sl.hSums[0];
		out->total_accuracy = (float)(sl.hSums[1] / ((double)sl.globalRows * (double)n->n_out));
		out->epochs = n->epochs;
		out->rows = sl.globalRows;
		out->device_ms = ms;
		out->kernel_launches = sl.launches;
		out->nonfinite = flags[0] & 1;
	}
	if (flags[1]) return fail(GL_ERR_TIMEOUT, "a bounded wait on the device ran out (code %d: 1-4 tensor-core pipeline, 20+ gradient exchange)", flags[1]);
	return GL_OK;
}

// Batched mode, small network: every weight fits in shared memory, so whole epochs run in one launch
// of the fused kernel (GLADES_SMALL_FUSED=0 keeps the per-layer kernels instead).
static bool small_fused_ok(const gl_net* n)
{
	if (n->world > 1 || n->d.gemm == GL_GEMM_TCGEN05 || n->d.gemm == GL_GEMM_GRID_FUSED) return false;
	static int enabled = -1;
	if (enabled < 0)
	{
		const char* e = getenv("GLADES_SMALL_FUSED");
		enabled = (e && atoi(e) == 0) ? 0 : 1;
	}
	if (!enabled) return false;
	const NetView v = make_view(n);
	return small_fused_smem_bytes(v) <= (size_t)200 * 1024;
}

static int small_fused_train(gl_net* n, int n_epochs, gl_metrics* out)
{
	double* dEpoch = nullptr;
	CU(cudaMalloc(&dEpoch, (size_t)2 * n_epochs * sizeof(double)));
	SmallFusedArgs a;
	memset(&a, 0, sizeof a);
	a.net = make_view(n);
	a.X = n->dX;
	a.Y = n->dY;
	a.rows = n->rows;
	a.n_epochs = n_epochs;
	a.bias_rule = n->d.bias_rule;
	a.epoch_sums = dEpoch;
	a.confusion = n->dConf;
	a.last_out = n->dLastOut;
	a.flags = n->dFlags;
	CU(cudaEventRecord(n->ev0, n->stream));
	cudaError_t e = launch_small_fused(a, n->stream);
	if (e == cudaSuccess) e = cudaEventRecord(n->ev1, n->stream);
	if (e == cudaSuccess) e = cudaStreamSynchronize(n->stream);
	double sums[2] = {0, 0};
	if (e == cudaSuccess) e = cudaMemcpy(sums, dEpoch + 2 * (n_epochs - 1), sizeof sums, cudaMemcpyDeviceToHost);
	cudaFree(dEpoch);
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "fused small-network kernel: %s", cudaGetErrorString(e));
	n->launches += 1;
	n->epochs += n_epochs;
	n->loW = false;
	float ms = 0;
	CU(cudaEventElapsedTime(&ms, n->ev0, n->ev1));
	return finish_metrics(n, out, (float)sums[0], (float)sums[1], n->rows, ms, 1, true);
}

// All epochs and windows of a mid-size network in one cooperative launch.
static int grid_fused_train(gl_net* n, int n_epochs, gl_metrics* out)
{
	double* dEpoch = nullptr;
	CU(cudaMalloc(&dEpoch, (size_t)2 * n_epochs * sizeof(double)));
	CU(cudaMemsetAsync(n->dConf, 0, (size_t)n->n_out * n->n_out * sizeof(int), n->stream));
	CU(cudaEventRecord(n->ev0, n->stream));
	int r = grid_fused_launch(n, n->dX, n->dY, n->rows, n->d.batch_size, n_epochs, n->rows, dEpoch);
	cudaError_t e = cudaSuccess;
	if (r == GL_OK) e = cudaEventRecord(n->ev1, n->stream);
	if (r == GL_OK && e == cudaSuccess) e = cudaStreamSynchronize(n->stream);
	double sums[2] = {0, 0};
	if (r == GL_OK && e == cudaSuccess) e = cudaMemcpy(sums, dEpoch + 2 * (n_epochs - 1), sizeof sums, cudaMemcpyDeviceToHost);
	cudaFree(dEpoch);
	if (r != GL_OK) return r;
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "whole-window cooperative kernel: %s", cudaGetErrorString(e));
	n->launches += 1;
	n->epochs += n_epochs;
	float ms = 0;
	CU(cudaEventElapsedTime(&ms, n->ev0, n->ev1));
	return finish_metrics(n, out, (float)sums[0], (float)sums[1], n->rows, ms, 1, true);
}

extern "C" int gl_train_epochs(gl_net* n, int32_t n_epochs, gl_metrics* out)
{
	if (!n || n_epochs < 1) return fail(GL_ERR_INVALID, "gl_train_epochs: bad argument");
	if (!n->dX || !n->dY) return fail(GL_ERR_STATE, "gl_train_epochs: no data (inputs and expected rows) set");
	if (int r = use_device(n)) return r;
	n->stop = 0;
	if (n->d.mode == GL_MODE_REFERENCE) return ref_train(n, n_epochs, out);
	if (small_fused_ok(n)) return small_fused_train(n, n_epochs, out);
	if (grid_fused_ok(n)) return grid_fused_train(n, n_epochs, out);
	// batched mode: aligned windows of batch_size rows; epoch figures are sums over the windows
	const int mb = n->d.batch_size;
	gl_metrics last;
	memset(&last, 0, sizeof last);
	for (int ep = 0; ep < n_epochs && !n->stop; ++ep)
	{
		double cost = 0.0, acc = 0.0, ms = 0.0;
		int64_t launches = 0;
		int nonfinite = 0;
		CU(cudaMemsetAsync(n->dConf, 0, (size_t)n->n_out * n->n_out * sizeof(int), n->stream));
		for (int64_t r0 = 0; r0 < n->rows; r0 += mb)
		{
			const int cnt = (int)((n->rows - r0) < mb ? (n->rows - r0) : mb);
			gl_metrics m;
			if (int r = batched_window(n, n->dX + r0 * n->d.sizes[0], n->dY + r0 * n->n_out, cnt, n->rows, &m)) return r;
			cost += (double)m.total_error;
			acc += (double)m.total_accuracy * (double)m.rows * (double)n->n_out;
			ms += m.device_ms;
			launches += m.kernel_launches;
			nonfinite |= m.nonfinite;
		}
		n->epochs += 1;
		if (int r = finish_metrics(n, &last, (float)cost, (float)acc, n->rows, (float)ms, launches, true)) return r;
		last.nonfinite = nonfinite;
	}
	if (out) *out = last;
	return GL_OK;
}

// ------------------------------------------------------------------------------------------------
// Reference mode with dropout: the test pass draws node flags per row too (SGDHelper calls scrambleDropout
// whatever the run type, network.cpp:408-411).  One launch of the sample-loop kernel without its backward
// half; outputs and activations come back through temporary device buffers.
static int ref_forward_dropout(gl_net* n, const float* X, const float* Y, int64_t rows, int64_t metric_rows, float* outputs,
                               int32_t* argmax, float* acts_last, gl_metrics* out)
{
	if (int r = draw_and_upload_masks(n, rows)) return r;
	if (n->sumsFCap < 1)
	{
		CU(cudaMalloc(&n->dSumsF, 2 * sizeof(float)));
		n->sumsFCap = 1;
	}
	RefTrainArgs a;
	memset(&a, 0, sizeof a);
	a.net = make_view(n);
	if (ref_train_dropout_smem_bytes(a.net) > (size_t)227 * 1024)
		return fail(GL_ERR_TOO_LARGE, "reference mode with dropout: %d nodes do not fit the per-sample shared-memory vectors", n->total_nodes);
	for (int l = 0; l <= n->H; ++l) a.hist[l] = n->dHist + n->woff[l] * n->d.batch_size;
	a.hist_len = n->dHistLen;
	a.X = X;
	a.Y = Y;
	a.rows = rows;
	a.data_rows = metric_rows;
	a.n_epochs = 1;
	a.epoch_sums = n->dSumsF;
	a.confusion = n->dConf;
	a.last_out = n->dLastOut;
	a.flags = n->dFlags;
	a.train = 0;
	a.preact_out = n->dPreact;
	fill_dropout_args(n, a);
	float* dOut = nullptr;
	float* dActs = nullptr;
	const bool want_out = outputs || argmax;
	if (want_out) CU(cudaMalloc(&dOut, (size_t)rows * n->n_out * sizeof(float)));
	cudaError_t e = cudaSuccess;
	if (acts_last) e = cudaMalloc(&dActs, (size_t)(n->total_nodes - n->d.sizes[0]) * sizeof(float));
	a.outputs = dOut;
	a.acts_out = dActs;
	if (e == cudaSuccess) e = cudaEventRecord(n->ev0, n->stream);
	if (e == cudaSuccess) e = launch_ref_train(a, n->stream);
	if (e == cudaSuccess) e = cudaEventRecord(n->ev1, n->stream);
	if (e == cudaSuccess) e = cudaStreamSynchronize(n->stream);
	std::vector<float> hOut;
	if (e == cudaSuccess && want_out)
	{
		hOut.resize((size_t)rows * n->n_out);
		e = cudaMemcpy(hOut.data(), dOut, hOut.size() * sizeof(float), cudaMemcpyDeviceToHost);
	}
	if (e == cudaSuccess && acts_last)
		e = cudaMemcpy(acts_last, dActs, (size_t)(n->total_nodes - n->d.sizes[0]) * sizeof(float), cudaMemcpyDeviceToHost);
	cudaFree(dOut);
	cudaFree(dActs);
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "reference-mode forward with dropout: %s", cudaGetErrorString(e));
	n->launches += 1;
	if (outputs) memcpy(outputs, hOut.data(), hOut.size() * sizeof(float));
	if (argmax)
		for (int64_t r = 0; r < rows; ++r)
		{
			// GMath::naiveVectorDecomp (GMath/gmath.cpp:435-455): strict > from 0, first maximum wins, -1 for none
			float mx = 0.0f;
			int idx = -1;
			for (int o = 0; o < n->n_out; ++o)
				if (hOut[(size_t)r * n->n_out + o] > mx)
				{
					mx = hOut[(size_t)r * n->n_out + o];
					idx = o;
				}
			argmax[r] = idx;
		}
	if (out)
	{
		float ms = 0;
		CU(cudaEventElapsedTime(&ms, n->ev0, n->ev1));
		float sums[2] = {0, 0};
		if (Y) CU(cudaMemcpy(sums, n->dSumsF, sizeof sums, cudaMemcpyDeviceToHost));
		return finish_metrics(n, out, sums[0], sums[1], rows, ms, 1, Y != nullptr);
	}
	return GL_OK;
}

static int forward_rows(gl_net* n, const float* X, const float* Y, int64_t rows, int64_t metric_rows, float* outputs,
                        int32_t* argmax, gl_metrics* out)
{
	if (n->d.mode == GL_MODE_REFERENCE && n->dropout)
		return ref_forward_dropout(n, X, Y, rows, metric_rows, outputs, argmax, nullptr, out);
	const int64_t chunk_max = (n->d.mode == GL_MODE_REFERENCE) ? 65536 : (rows < 65536 ? rows : 65536);
	if (int r = ensure_work(n, chunk_max < rows ? chunk_max : rows)) return r;
	int64_t launches = 0;
	CU(cudaEventRecord(n->ev0, n->stream));
	CU(cudaMemsetAsync(n->dSums, 0, 2 * sizeof(double), n->stream));
	CU(cudaMemsetAsync(n->dConf, 0, (size_t)n->n_out * n->n_out * sizeof(int), n->stream));
	float* dSumsRef = nullptr;
	if (n->d.mode == GL_MODE_REFERENCE)
	{
		if (n->sumsFCap < 1)
		{
			CU(cudaMalloc(&n->dSumsF, 2 * sizeof(float)));
			n->sumsFCap = 1;
		}
		dSumsRef = n->dSumsF;
		CU(cudaMemsetAsync(dSumsRef, 0, 2 * sizeof(float), n->stream));
	}
	const NetView v = make_view(n);
	for (int64_t r0 = 0; r0 < rows; r0 += n->capRows)
	{
		const int cnt = (int)((rows - r0) < n->capRows ? (rows - r0) : n->capRows);
		const float* Xc = X + r0 * n->d.sizes[0];
		const float* Yc = Y ? Y + r0 * n->n_out : nullptr;
		if (n->d.mode == GL_MODE_REFERENCE)
		{
			CU(launch_ref_forward(v, Xc, cnt, n->dA, n->stream));
			launches += n->H + 1;
			if (Yc && out)
			{
				CU(launch_ref_metrics(v, n->dA[n->H + 1], Yc, cnt, metric_rows, dSumsRef, n->dConf, n->stream));
				++launches;
			}
		}
		else
		{
			if (int r = batched_forward(n, Xc, cnt, &launches)) return r;
		}
		if (n->d.mode == GL_MODE_BATCHED || argmax)
		{
			// batched head: softmax normalisation, argmax, and (with targets) the metric sums
			HeadArgs h;
			memset(&h, 0, sizeof h);
			h.P = n->dA[n->H + 1];
			h.Y = Yc ? Yc : n->dA[n->H + 1];
			h.rows = cnt;
			h.n = n->n_out;
			h.out_type = n->d.output_type;
			h.softmax = n->softmax;
			h.data_size = (float)(metric_rows * (int64_t)n->n_out);
			h.sums2 = (Yc && n->d.mode == GL_MODE_BATCHED) ? n->dSums : nullptr;
			h.confusion = (Yc && n->d.mode == GL_MODE_BATCHED && n->d.output_type != GL_OUT_REGRESSION) ? n->dConf : nullptr;
			h.argmax = n->dArgmax;
			CU(launch_head(h, n->stream));
			++launches;
		}
		if (r0 + cnt == rows)
			CU(cudaMemcpyAsync(n->dLastOut, n->dA[n->H + 1] + (size_t)(cnt - 1) * n->n_out, (size_t)n->n_out * sizeof(float),
			                   cudaMemcpyDeviceToDevice, n->stream));
		if (outputs)
			CU(cudaMemcpyAsync(outputs + r0 * n->n_out, n->dA[n->H + 1], (size_t)cnt * n->n_out * sizeof(float),
			                   cudaMemcpyDeviceToHost, n->stream));
		if (argmax)
			CU(cudaMemcpyAsync(argmax + r0, n->dArgmax, (size_t)cnt * sizeof(int), cudaMemcpyDeviceToHost, n->stream));
		if (outputs || argmax) CU(cudaStreamSynchronize(n->stream));  // the work buffers are reused by the next chunk
	}
	CU(cudaEventRecord(n->ev1, n->stream));
	CU(cudaStreamSynchronize(n->stream));
	n->launches += launches;
	if (out)
	{
		float ms = 0;
		CU(cudaEventElapsedTime(&ms, n->ev0, n->ev1));
		float te = 0, ta = 0;
		if (Y)
		{
			if (n->d.mode == GL_MODE_REFERENCE)
			{
				float s[2];
				CU(cudaMemcpy(s, dSumsRef, sizeof s, cudaMemcpyDeviceToHost));
				te = s[0];
				ta = s[1];
			}
			else
			{
				double s[2];
				CU(cudaMemcpy(s, n->dSums, sizeof s, cudaMemcpyDeviceToHost));
				te = (float)s[0];
				ta = (float)s[1];
			}
		}
		return finish_metrics(n, out, te, ta, rows, ms, launches, Y != nullptr);
	}
	return GL_OK;
}

extern "C" int gl_forward(gl_net* n, int64_t first_row, int64_t rows, float* outputs, int32_t* argmax, gl_metrics* out)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_forward: null handle");
	if (!n->dX) return fail(GL_ERR_STATE, "gl_forward: no data set");
	if (first_row < 0 || rows < 1 || first_row + rows > n->rows) return fail(GL_ERR_INVALID, "gl_forward: row range");
	if (int r = use_device(n)) return r;
	return forward_rows(n, n->dX + first_row * n->d.sizes[0], n->dY ? n->dY + first_row * n->n_out : nullptr, rows,
	                    n->rows, outputs, argmax, out);
}

extern "C" int gl_forward_host(gl_net* n, const float* x, const float* y, int64_t rows, float* outputs, int32_t* argmax,
                               gl_metrics* out)
{
	if (!n || !x || rows < 1) return fail(GL_ERR_INVALID, "gl_forward_host: bad argument");
	if (int r = use_device(n)) return r;
	if (int r = ensure_window_staging(n, rows)) return r;
	CU(cudaMemcpyAsync(n->dXwin, x, (size_t)rows * n->d.sizes[0] * sizeof(float), cudaMemcpyHostToDevice, n->stream));
	if (y) CU(cudaMemcpyAsync(n->dYwin, y, (size_t)rows * n->n_out * sizeof(float), cudaMemcpyHostToDevice, n->stream));
	return forward_rows(n, n->dXwin, y ? n->dYwin : nullptr, rows, rows, outputs, argmax, out);
}

// ---- inference from host buffers, two batches in flight -------------------------------------------
extern "C" int gl_forward_host_submit(gl_net* n, const float* x, const float* y, int32_t rows)
{
	if (!n || !x || rows < 1) return fail(GL_ERR_INVALID, "gl_forward_host_submit: bad argument");
	if (n->d.mode != GL_MODE_BATCHED) return fail(GL_ERR_STATE, "gl_forward_host_submit needs a batched-mode network");
	if (rows > 65536) return fail(GL_ERR_INVALID, "gl_forward_host_submit: at most 65536 rows per batch");
	if (n->submitted - n->collected >= 2) return fail(GL_ERR_STATE, "two batches are already in flight: collect a result first");
	if (int r = use_device(n)) return r;
	if (int r = ensure_work(n, rows)) return r;
	if (!n->copyStream) CU(cudaStreamCreateWithFlags(&n->copyStream, cudaStreamNonBlocking));
	gl_net::Slot& sl = n->slot[n->submitted & 1];
	const bool used_before = sl.copied != nullptr;
	if (int r = slot_prepare(n, sl, rows)) return r;
	if (rows > sl.argCap)
	{
		if (sl.hArg) cudaFreeHost(sl.hArg);
		sl.hArg = nullptr;
		sl.argCap = 0;
		CU(cudaMallocHost(&sl.hArg, (size_t)rows * sizeof(int)));
		sl.argCap = rows;
	}
	if (used_before) CU(cudaStreamWaitEvent(n->copyStream, sl.done, 0));
	CU(cudaMemcpyAsync(sl.dX, x, (size_t)rows * n->d.sizes[0] * sizeof(float), cudaMemcpyHostToDevice, n->copyStream));
	if (y) CU(cudaMemcpyAsync(sl.dY, y, (size_t)rows * n->n_out * sizeof(float), cudaMemcpyHostToDevice, n->copyStream));
	CU(cudaEventRecord(sl.copied, n->copyStream));
	CU(cudaStreamWaitEvent(n->stream, sl.copied, 0));
	CU(cudaEventRecord(sl.t0, n->stream));
	CU(cudaMemsetAsync(sl.dSums, 0, 2 * sizeof(double), n->stream));
	int64_t launches = 0;
	if (int r = batched_forward(n, sl.dX, rows, &launches)) return r;
	HeadArgs h;
	memset(&h, 0, sizeof h);
	h.P = n->dA[n->H + 1];
	h.Y = y ? sl.dY : n->dA[n->H + 1];
	h.rows = rows;
	h.n = n->n_out;
	h.out_type = n->d.output_type;
	h.softmax = n->softmax;
	h.data_size = (float)((int64_t)rows * (int64_t)n->n_out);
	h.sums2 = y ? sl.dSums : nullptr;
	h.argmax = n->dArgmax;
	CU(launch_head(h, n->stream));
	++launches;
	CU(cudaMemcpyAsync(n->dLastOut, n->dA[n->H + 1] + (size_t)(rows - 1) * n->n_out, (size_t)n->n_out * sizeof(float),
	                   cudaMemcpyDeviceToDevice, n->stream));
	CU(cudaMemcpyAsync(sl.hArg, n->dArgmax, (size_t)rows * sizeof(int), cudaMemcpyDeviceToHost, n->stream));
	CU(cudaMemcpyAsync(sl.hSums, sl.dSums, 2 * sizeof(double), cudaMemcpyDeviceToHost, n->stream));
	CU(cudaMemcpyAsync(sl.hSums + 2, n->dFlags, 4 * sizeof(int), cudaMemcpyDeviceToHost, n->stream));
	CU(cudaEventRecord(sl.done, n->stream));
	n->launches += launches;
	sl.rows = rows;
	sl.globalRows = rows;
	sl.launches = launches;
	sl.pending = true;
	sl.infer = true;
	sl.hasY = y != nullptr;
	++n->submitted;
	return GL_OK;
}

extern "C" int gl_forward_host_result(gl_net* n, int32_t* argmax, gl_metrics* out)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_forward_host_result: null handle");
	if (n->submitted == n->collected) return fail(GL_ERR_STATE, "no batch in flight");
	if (int r = use_device(n)) return r;
	gl_net::Slot& sl = n->slot[n->collected & 1];
	if (!sl.infer) return fail(GL_ERR_STATE, "the oldest call in flight is a training window: collect it with gl_train_window_host_result");
	CU(cudaEventSynchronize(sl.done));
	sl.pending = false;
	sl.infer = false;
	++n->collected;
	int flags[4];
	memcpy(flags, sl.hSums + 2, sizeof flags);
	if (argmax) memcpy(argmax, sl.hArg, (size_t)sl.rows * sizeof(int));
	if (out)
	{
		float ms = 0;
		CU(cudaEventElapsedTime(&ms, sl.t0, sl.done));
		memset(out, 0, sizeof *out);
		if (sl.hasY)
		{
			out->total_error = (float)sl.hSums[0];
			out->total_accuracy = (float)(sl.hSums[1] / ((double)sl.rows * (double)n->n_out));
		}
		out->epochs = n->epochs;
		out->rows = sl.rows;
		out->device_ms = ms;
		out->kernel_launches = sl.launches;
		out->nonfinite = flags[0] & 1;
	}
	if (flags[1])
		return fail(GL_ERR_TIMEOUT, "a bounded wait on the device ran out (code %d: 1-4 tensor-core pipeline, 20+ gradient exchange)", flags[1]);
	return GL_OK;
}

extern "C" int gl_get_activations(gl_net* n, int64_t row, float* out)
{
	if (!n || !out) return fail(GL_ERR_INVALID, "gl_get_activations: null argument");
	if (!n->dX || row < 0 || row >= n->rows) return fail(GL_ERR_STATE, "gl_get_activations: no such row");
	if (int r = use_device(n)) return r;
	if (n->d.mode == GL_MODE_REFERENCE && n->dropout)  // draws this row's node flags like any forward of the reference
		return ref_forward_dropout(n, n->dX + row * n->d.sizes[0], nullptr, 1, 1, nullptr, nullptr, out, nullptr);
	if (int r = ensure_work(n, 1)) return r;
	int64_t launches = 0;
	const float* X = n->dX + row * n->d.sizes[0];
	if (n->d.mode == GL_MODE_REFERENCE)
	{
		const NetView v = make_view(n);
		CU(launch_ref_forward(v, X, 1, n->dA, n->stream));
		launches = n->H + 1;
	}
	else
	{
		if (int r = batched_forward(n, X, 1, &launches)) return r;
		if (n->softmax)
		{
			HeadArgs h;
			memset(&h, 0, sizeof h);
			h.P = n->dA[n->H + 1];
			h.Y = n->dA[n->H + 1];
			h.rows = 1;
			h.n = n->n_out;
			h.out_type = n->d.output_type;
			h.softmax = 1;
			h.data_size = 1.0f;
			CU(launch_head(h, n->stream));
			++launches;
		}
	}
	n->launches += launches;
	size_t k = 0;
	for (int l = 1; l <= n->H + 1; ++l)
	{
		CU(cudaMemcpyAsync(out + k, n->dA[l], n->d.sizes[l] * sizeof(float), cudaMemcpyDeviceToHost, n->stream));
		k += n->d.sizes[l];
	}
	CU(cudaStreamSynchronize(n->stream));
	return GL_OK;
}

extern "C" int gl_get_pending_delta(gl_net* n, int32_t k, float* out)
{
	if (!n || !out) return fail(GL_ERR_INVALID, "gl_get_pending_delta: null argument");
	if (n->d.mode != GL_MODE_REFERENCE) return fail(GL_ERR_STATE, "pending deltas exist in reference mode only");
	if (int r = use_device(n)) return r;
	if (n->dropout)
	{
		// every edge has its own history length
		memset(out, 0, (size_t)n->nw * sizeof(float));
		if (k < 0 || k >= n->d.batch_size) return GL_OK;
		std::vector<int> len((size_t)n->nw);
		std::vector<float> slice((size_t)n->nw);
		CU(cudaMemcpy(len.data(), n->dHlen, len.size() * sizeof(int), cudaMemcpyDeviceToHost));
		for (int l = 0; l <= n->H; ++l)
		{
			const int64_t cnt = n->woff[l + 1] - n->woff[l];
			CU(cudaMemcpy(slice.data() + n->woff[l], n->dHist + n->woff[l] * n->d.batch_size + (int64_t)k * cnt, cnt * sizeof(float),
			              cudaMemcpyDeviceToHost));
		}
		for (int64_t e = 0; e < n->nw; ++e)
			if (k < len[(size_t)e]) out[e] = slice[(size_t)e];
		return GL_OK;
	}
	int len = 0;
	CU(cudaMemcpy(&len, n->dHistLen, sizeof len, cudaMemcpyDeviceToHost));
	if (k < 0 || k >= len || k >= n->d.batch_size)
	{
		memset(out, 0, (size_t)n->nw * sizeof(float));
		return GL_OK;
	}
	for (int l = 0; l <= n->H; ++l)
	{
		const int64_t cnt = n->woff[l + 1] - n->woff[l];
		CU(cudaMemcpy(out + n->woff[l], n->dHist + n->woff[l] * n->d.batch_size + (int64_t)k * cnt, cnt * sizeof(float),
		              cudaMemcpyDeviceToHost));
	}
	return GL_OK;
}

extern "C" int gl_get_last_outputs(gl_net* n, float* out)
{
	if (!n || !out) return fail(GL_ERR_INVALID, "gl_get_last_outputs: null argument");
	if (int r = use_device(n)) return r;
	CU(cudaStreamSynchronize(n->stream));
	CU(cudaMemcpy(out, n->dLastOut, (size_t)n->n_out * sizeof(float), cudaMemcpyDeviceToHost));
	return GL_OK;
}

extern "C" int gl_get_confusion(gl_net* n, int32_t* out)
{
	if (!n || !out) return fail(GL_ERR_INVALID, "gl_get_confusion: null argument");
	if (int r = use_device(n)) return r;
	CU(cudaStreamSynchronize(n->stream));
	CU(cudaMemcpy(out, n->dConf, (size_t)n->n_out * n->n_out * sizeof(int), cudaMemcpyDeviceToHost));
	return GL_OK;
}

// ------------------------------------------------------------------------------------------------
extern "C" void gl_shard_range(int64_t rows, int32_t rank, int32_t world, int64_t* first, int64_t* count)
{
	if (world < 1) world = 1;
	const int64_t base = rows / world, rem = rows % world;
	const int64_t f = (int64_t)rank * base + (rank < rem ? rank : rem);
	if (first) *first = f;
	if (count) *count = base + (rank < rem ? 1 : 0);
}


// Unmaps the peers' memory and frees this rank's exchange buffers (no collective inside).
static void dp_push_release(gl_net* n)
{
	for (int r = 0; r < DP_MAX_WORLD; ++r)
	{
		if (r != n->rank)
		{
			if (n->dpPeerArena[r]) cudaIpcCloseMemHandle(n->dpPeerArena[r]);
			if (n->dpPeerW[r]) cudaIpcCloseMemHandle(n->dpPeerW[r]);
		}
		n->dpPeerArena[r] = nullptr;
		n->dpPeerW[r] = nullptr;
	}
	cudaFree(n->dpMaps);
	cudaFree(n->dpBases);
	cudaFree(n->dpArena);
	n->dpMaps = nullptr;
	n->dpBases = nullptr;
	n->dpArena = nullptr;
	n->dpPush = false;
	cudaGetLastError();
}

// Sets up the gradient exchange over peer memory: bands, the exchange arena, the inter-process
// mappings of every rank's arena and weight vector, the per-owner tensor maps.  Collective: every
// rank of the communicator calls it.  On failure the handle stays on the NCCL path.
//
// The function contains four collectives (gather of the handles, two agreements, the handshake's
// agreement).  A rank must never leave between them while its peers wait inside the next one, so a
// local failure (allocation, handle export, mapping, copy) is only recorded; it travels to the next
// agreement, after which all ranks release and return together.  The gather buffer n->dpRec was
// allocated by gl_dp_init before the communicator existed.
namespace {
struct DpRec { cudaIpcMemHandle_t arena, w; };
}
static int dp_push_setup(gl_net* n)
{
	const int W = n->world;
	if (W > DP_MAX_WORLD) return fail(GL_ERR_INVALID, "the peer-memory exchange handles at most %d ranks", DP_MAX_WORLD);
	if (!g_nccl.AllGather) return fail(GL_ERR_COMM, "libnccl lacks ncclAllGather");
	int64_t off = 0;
	for (int l = 0; l <= n->H; ++l)
	{
		const int no = n->d.sizes[l + 1], ni = n->d.sizes[l];
		const int per = (no + W - 1) / W;
		n->dpBand[l] = ((per + 127) / 128) * 128;
		n->dpSlotOff[l] = off;
		const int64_t cap = (int64_t)(n->dpBand[l] < no ? n->dpBand[l] : no) * ni;
		off += ((cap + 3) / 4) * 4;
	}
	n->dpSlotOff[n->H + 1] = off;
	// behind the gradient slots: a staging vector for the new weights (the owners write a layer's updated bands there;
	// every rank copies them into its weights once its own last reader of the old ones has finished)
	n->dpStageOff = ((DP_FLAG_BYTES + (size_t)W * (size_t)off * sizeof(float)) + 255) & ~(size_t)255;
	const size_t bytes = n->dpStageOff + ((size_t)n->nw + 4) * sizeof(float);
	int failed = 0;
	char why[160] = "";
	auto local = [&](cudaError_t e, const char* what) {
		if (e == cudaSuccess || failed) return;
		failed = 1;
		snprintf(why, sizeof why, "%s: %s", what, cudaGetErrorString(e));
		cudaGetLastError();
	};
	DpRec* dRec = static_cast<DpRec*>(n->dpRec);
	DpRec mine;
	memset(&mine, 0, sizeof mine);
	local(cudaMalloc(&n->dpArena, bytes), "exchange arena");
	if (!failed) local(cudaMemset(n->dpArena, 0, bytes), "clearing the exchange arena");
	if (!failed) local(cudaIpcGetMemHandle(&mine.arena, n->dpArena), "exporting the exchange arena");
	if (!failed) local(cudaIpcGetMemHandle(&mine.w, n->dW), "exporting the weights");
	local(cudaMemcpy(dRec + W, &mine, sizeof mine, cudaMemcpyHostToDevice), "staging the handles");
	NC(g_nccl.AllGather(dRec + W, dRec, sizeof(DpRec), NCCL_INT8, n->comm, n->stream));
	local(cudaStreamSynchronize(n->stream), "gathering the handles");
	std::vector<DpRec> all((size_t)W);
	local(cudaMemcpy(all.data(), dRec, sizeof(DpRec) * (size_t)W, cudaMemcpyDeviceToHost), "reading the handles");
	for (int r = 0; r < W && !failed; ++r)
	{
		if (r == n->rank)
		{
			n->dpPeerArena[r] = n->dpArena;
			n->dpPeerW[r] = n->dW;
			continue;
		}
		local(cudaIpcOpenMemHandle(&n->dpPeerArena[r], all[(size_t)r].arena, cudaIpcMemLazyEnablePeerAccess), "mapping a peer's arena");
		if (!failed) local(cudaIpcOpenMemHandle(&n->dpPeerW[r], all[(size_t)r].w, cudaIpcMemLazyEnablePeerAccess), "mapping a peer's weights");
	}
	// per layer and owner: where this rank's contribution to the owner's band goes
	const size_t nmaps = (size_t)GL_MAX_WEIGHT_LAYERS * DP_MAX_WORLD;
	if (!failed)
	{
		std::vector<unsigned char> raw(nmaps * 128 + 64);
		unsigned char* maps = raw.data() + ((64 - ((uintptr_t)raw.data() & 63)) & 63);
		std::vector<float*> bases(nmaps, nullptr);
		for (int l = 0; l <= n->H; ++l)
		{
			const int no = n->d.sizes[l + 1], ni = n->d.sizes[l];
			for (int o = 0; o < W; ++o)
			{
				int rows = no - o * n->dpBand[l];
				rows = rows < 0 ? 0 : (rows > n->dpBand[l] ? n->dpBand[l] : rows);
				float* base = reinterpret_cast<float*>(static_cast<char*>(n->dpPeerArena[o]) + DP_FLAG_BYTES) +
				              (int64_t)n->rank * off + n->dpSlotOff[l];
				bases[(size_t)l * DP_MAX_WORLD + o] = base;
				n->hostBases[l][o] = base;
				if (rows >= 128 && rows % 128 == 0 && ni % 128 == 0)
					tc_make_store_map(maps + ((size_t)l * DP_MAX_WORLD + o) * 128, base, rows, ni, ni);
			}
		}
		local(cudaMalloc(&n->dpMaps, nmaps * 128), "tensor maps of the owners' bands");
		if (!failed) local(cudaMalloc(&n->dpBases, nmaps * sizeof(float*)), "base pointers of the owners' bands");
		if (!failed) local(cudaMemcpy(n->dpMaps, maps, nmaps * 128, cudaMemcpyHostToDevice), "uploading the tensor maps");
		if (!failed) local(cudaMemcpy(n->dpBases, bases.data(), nmaps * sizeof(float*), cudaMemcpyHostToDevice), "uploading the base pointers");
	}
	// Every rank must take the same path: agree on the outcome.  This all-reduce is also the point after
	// which every rank has zeroed and mapped everything, so nobody writes into a peer before it.
	int* dAgree = reinterpret_cast<int*>(dRec);
	int total_failed = failed;
	{
		cudaError_t e = cudaMemcpy(dAgree, &failed, sizeof failed, cudaMemcpyHostToDevice);
		if (e != cudaSuccess && !failed)
		{
			// this rank cannot even report: it still joins the collective (with whatever the word holds) and fails locally
			local(e, "staging the agreement word");
		}
		NC(g_nccl.AllReduce(dAgree, dAgree, 1, NCCL_INT32, NCCL_SUM, n->comm, n->stream));
		local(cudaStreamSynchronize(n->stream), "agreeing on the mappings");
		if (cudaMemcpy(&total_failed, dAgree, sizeof total_failed, cudaMemcpyDeviceToHost) != cudaSuccess) total_failed = 1;
		if (failed && !total_failed) total_failed = 1;
	}
	if (total_failed)
	{
		dp_push_release(n);
		return fail(GL_ERR_COMM, "the ranks cannot set up the exchange over each other's device memory (%d rank(s) failed; this rank: %s); "
		                         "staying on the NCCL all-reduce", total_failed, failed ? why : "ok");
	}
	// Handshake over the mapped memory itself: every rank stores a pattern into its slot at every owner and
	// raises a flag there; every rank then waits (a few seconds at most) for all flags and checks all
	// patterns.  Only if that works on EVERY rank does the handle use the exchange over peer memory.
	{
		DpPeers heads, fl;
		for (int r = 0; r < DP_MAX_WORLD; ++r)
		{
			fl.p[r] = n->dpPeerArena[r];
			heads.p[r] = (r < W) ? static_cast<void*>(reinterpret_cast<float*>(static_cast<char*>(n->dpPeerArena[r]) + DP_FLAG_BYTES) +
			                                          (int64_t)n->rank * off)
			                     : nullptr;
		}
		int* dStatus = dAgree + 1;
		int zero = 0, status = 0;
		local(cudaMemcpy(dStatus, &zero, sizeof zero, cudaMemcpyHostToDevice), "clearing the handshake status");
		if (!failed) local(launch_dp_hello_write(heads, fl, W, n->rank, n->stream), "handshake store");
		if (!failed) local(launch_dp_wait(n->dpArena, 0, 0, 0, DP_WORD_HELLO, W, 1u, dStatus, 1, n->stream, 8000000000ll), "handshake wait");
		if (!failed) local(launch_dp_hello_check(reinterpret_cast<const float*>(n->dpArena + DP_FLAG_BYTES), off, W, dStatus, 2, n->stream), "handshake check");
		local(cudaStreamSynchronize(n->stream), "handshake");
		if (!failed) local(cudaMemcpy(&status, dStatus, sizeof status, cudaMemcpyDeviceToHost), "reading the handshake status");
		int bad = (failed || status != 0) ? 1 : 0;
		total_failed = bad;
		cudaMemcpy(dAgree, &bad, sizeof bad, cudaMemcpyHostToDevice);
		NC(g_nccl.AllReduce(dAgree, dAgree, 1, NCCL_INT32, NCCL_SUM, n->comm, n->stream));
		local(cudaStreamSynchronize(n->stream), "agreeing on the handshake");
		if (cudaMemcpy(&total_failed, dAgree, sizeof total_failed, cudaMemcpyDeviceToHost) != cudaSuccess) total_failed = 1;
		if (bad && !total_failed) total_failed = 1;
		if (total_failed)
		{
			dp_push_release(n);
			return fail(GL_ERR_COMM, "the handshake over peer memory failed on %d rank(s) (this rank: %s); staying on the NCCL all-reduce",
			            total_failed, failed ? why : (status == 0 ? "ok" : (status == 1 ? "a flag did not arrive" : "a pattern did not arrive")));
		}
	}
	n->dpPush = true;
	n->dpStep = 0;
	return GL_OK;
}

extern "C" int gl_dp_unique_id(void* id128)
{
	if (!id128) return fail(GL_ERR_INVALID, "gl_dp_unique_id: null argument");
	if (int r = nccl_load()) return r;
	nccl_uid id;
	NC(g_nccl.GetUniqueId(&id));
	memcpy(id128, &id, sizeof id);
	return GL_OK;
}

extern "C" int gl_dp_init(gl_net* n, int32_t rank, int32_t world, const void* id128)
{
	if (!n || !id128 || world < 1 || rank < 0 || rank >= world) return fail(GL_ERR_INVALID, "gl_dp_init: bad argument");
	if (n->d.mode != GL_MODE_BATCHED) return fail(GL_ERR_STATE, "data parallelism needs a batched-mode network");
	if (int r = use_device(n)) return r;
	n->rank = rank;
	n->world = world;
	if (world == 1) return GL_OK;
	if (int r = nccl_load()) return r;
	nccl_uid id;
	memcpy(&id, id128, sizeof id);
	// scratch of the collective set-up below: allocated before any collective, so that a failure here
	// cannot strand the peers inside one
	if (!n->dpRec) CU(cudaMalloc(&n->dpRec, (size_t)(DP_MAX_WORLD + 1) * 2 * sizeof(cudaIpcMemHandle_t) + 64));
	NC(g_nccl.CommInitRank(&n->comm, world, id, rank));
	{
		// the exchange work is short and sits on the critical path: let its CTAs go first
		int lo = 0, hi = 0;
		CU(cudaDeviceGetStreamPriorityRange(&lo, &hi));
		CU(cudaStreamCreateWithPriority(&n->commStream, cudaStreamNonBlocking, hi));
	}
	for (int l = 0; l <= GL_MAX_WEIGHT_LAYERS; ++l) CU(cudaEventCreateWithFlags(&n->evGrad[l], cudaEventDisableTiming));
	{
		int lo = 0, hi = 0;
		CU(cudaDeviceGetStreamPriorityRange(&lo, &hi));
		for (int i = 0; i < gl_net::DP_COMM_STREAMS; ++i) CU(cudaStreamCreateWithPriority(&n->layerStream[i], cudaStreamNonBlocking, hi));
		for (int l = 0; l < GL_MAX_WEIGHT_LAYERS; ++l) CU(cudaEventCreateWithFlags(&n->evLayer[l], cudaEventDisableTiming));
		for (int l = 0; l < GL_MAX_WEIGHT_LAYERS; ++l) CU(cudaEventCreateWithFlags(&n->evRead[l], cudaEventDisableTiming));
	}
	CU(cudaEventCreateWithFlags(&n->evComm, cudaEventDisableTiming));
	if (const char* e = getenv("GLADES_DP_OVERLAP")) n->dpOverlap = atoi(e) != 0;
	if (const char* e = getenv("GLADES_DP_RESERVE_SMS")) n->dpReserveSms = atoi(e);
	if (const char* e = getenv("GLADES_DP_PUSH_BLOCKS")) n->dpPushBlocks = atoi(e) > 0 ? atoi(e) : 296;
	if (const char* e = getenv("GLADES_DP_STORE")) n->dpStoreMode = (atoi(e) >= 0 && atoi(e) <= 2) ? atoi(e) : 0;
	// GLADES_DP_PUSH=0: the NCCL all-reduce path; =1: the exchange over peer memory or an error;
	// unset: the exchange over peer memory when the ranks can map each other's memory, else NCCL
	const char* e = getenv("GLADES_DP_PUSH");
	const int want = e ? atoi(e) : -1;
	if (want != 0)
	{
		const int r = dp_push_setup(n);
		if (r != GL_OK && want == 1) return r;
	}
	return GL_OK;
}

extern "C" int gl_dp_mode(const gl_net* n) { return (n && n->world > 1) ? (n->dpPush ? 2 : 1) : 0; }

extern "C" int gl_dp_set_window(gl_net* n, int32_t global_rows, int32_t first_global_pos)
{
	if (!n || global_rows < 1 || first_global_pos < 0) return fail(GL_ERR_INVALID, "gl_dp_set_window: bad argument");
	n->globalRows = global_rows;
	n->firstPos = first_global_pos;
	return GL_OK;
}

// ---- timing helpers: CUDA events on the handle's own stream ---------------------------------------
extern "C" int gl_timer_start(gl_net* n)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_timer_start: null handle");
	if (int r = use_device(n)) return r;
	if (!n->tim0)
	{
		CU(cudaEventCreate(&n->tim0));
		CU(cudaEventCreate(&n->tim1));
	}
	CU(cudaEventRecord(n->tim0, n->stream));
	return GL_OK;
}
extern "C" int gl_timer_stop(gl_net* n, double* ms)
{
	if (!n || !ms || !n->tim0) return fail(GL_ERR_INVALID, "gl_timer_stop: bad argument");
	if (int r = use_device(n)) return r;
	if (int r = dp_join(n)) return r;  // the timed work includes the end of the last window's gradient exchange
	CU(cudaEventRecord(n->tim1, n->stream));
	CU(cudaEventSynchronize(n->tim1));
	float f = 0;
	CU(cudaEventElapsedTime(&f, n->tim0, n->tim1));
	*ms = f;
	return GL_OK;
}
extern "C" int gl_profile_enable(gl_net* n, int32_t on)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_profile_enable: null handle");
	n->profile = on != 0;
	n->profUsed = 0;
	n->profFlops.clear();
	n->profIsTc.clear();
	n->profShape.clear();
	return GL_OK;
}
// Sums the recorded layer-product launches since gl_profile_enable: out[0] launches, out[1] total ms,
// out[2] total flop (2*M*N*K each), for the tensor-core kernel; out[3..5] the same for the FFMA kernel.
extern "C" int gl_profile_read(gl_net* n, double* out6)
{
	if (!n || !out6) return fail(GL_ERR_INVALID, "gl_profile_read: bad argument");
	if (int r = use_device(n)) return r;
	CU(cudaStreamSynchronize(n->stream));
	for (int i = 0; i < 6; ++i) out6[i] = 0.0;
	for (size_t i = 0; i < n->profFlops.size(); ++i)
	{
		float f = 0;
		CU(cudaEventElapsedTime(&f, n->profEv[2 * i], n->profEv[2 * i + 1]));
		const int o = n->profIsTc[i] ? 0 : 3;
		out6[o] += 1.0;
		out6[o + 1] += f;
		out6[o + 2] += n->profFlops[i];
		if (getenv("GLADES_PROFILE_DUMP"))
			fprintf(stderr, "[profile] %s M=%d N=%d K=%d epi=%d %.4f ms %.1f TFLOP/s\n", n->profIsTc[i] ? "tc" : "ffma",
			        n->profShape[4 * i], n->profShape[4 * i + 1], n->profShape[4 * i + 2], n->profShape[4 * i + 3], f,
			        n->profFlops[i] / (f * 1e-3) / 1e12);
	}
	return GL_OK;
}

extern "C" int64_t gl_tensor_core_launches(const gl_net* n) { return n ? n->tcLaunches : 0; }
extern "C" void gl_tc_variant_counts(int64_t* out5)
{
	if (!out5) return;
	long long c[5];
	tc_variant_counts(c);
	for (int i = 0; i < 5; ++i) out5[i] = c[i];
}
extern "C" int64_t gl_kernel_launches(const gl_net* n) { return n ? n->launches : 0; }
extern "C" int32_t gl_window_cluster_ctas(const gl_net* n) { return n ? n->gfClusterCtas : -1; }

extern "C" int gl_sync(gl_net* n)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_sync: null handle");
	if (int r = use_device(n)) return r;
	if (int r = dp_join(n)) return r;
	CU(cudaStreamSynchronize(n->stream));
	int flags[4];
	CU(cudaMemcpy(flags, n->dFlags, sizeof flags, cudaMemcpyDeviceToHost));
	if (flags[1]) return fail(GL_ERR_TIMEOUT, "a bounded wait on the device ran out (code %d: 1-4 tensor-core pipeline, 20+ gradient exchange)", flags[1]);
	return GL_OK;
}

// ---- asynchronous snapshot for live views -------------------------------------------------------------
// What the reference's GUI callbacks read after an epoch (Networks/network.cpp:258-357): every weight
// (LayerBuilder::getWeights, State/LayerBuilder.cpp:390-410), and the pre-activations of the last row
// (network.cpp:510-514).  submit() queues, behind the work already on the compute stream, a device-to-device
// copy into a snapshot buffer on a side stream -- the compute stream only waits for that short copy, then
// goes on training -- and the copy of the snapshot into pinned host memory after it.  collect() hands the
// oldest submitted snapshot out.  One snapshot may be in flight.
static size_t snap_floats(const gl_net* n) { return (size_t)n->nw + GL_MAX_WEIGHT_LAYERS + (size_t)(n->total_nodes - n->d.sizes[0]); }

extern "C" int gl_snapshot_submit(gl_net* n)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_snapshot_submit: null handle");
	if (n->snapPending) return fail(GL_ERR_STATE, "a snapshot is already in flight: collect it first");
	if (int r = use_device(n)) return r;
	if (int r = dp_join(n)) return r;
	if (!n->snapStream)
	{
		CU(cudaStreamCreateWithFlags(&n->snapStream, cudaStreamNonBlocking));
		CU(cudaEventCreateWithFlags(&n->evSnapSrc, cudaEventDisableTiming));
		CU(cudaEventCreateWithFlags(&n->evSnapCopied, cudaEventDisableTiming));
		CU(cudaEventCreateWithFlags(&n->evSnapReady, cudaEventDisableTiming));
		CU(cudaMalloc(&n->dSnap, snap_floats(n) * sizeof(float)));
		CU(cudaMallocHost(&n->hSnap, snap_floats(n) * sizeof(float)));
	}
	if (n->d.mode == GL_MODE_BATCHED && n->dX && n->rows > 0)
	{
		// batched mode keeps no pre-activations: they are evaluated for the last resident row, in the exact
		// summation order, under the weights as they stand now
		if (int r = ensure_work(n, 1)) return r;
		const NetView v = make_view(n);
		CU(launch_ref_forward(v, n->dX + (n->rows - 1) * n->d.sizes[0], 1, n->dA, n->stream, n->dPreact));
		n->launches += n->H + 1;
	}
	const size_t np = (size_t)(n->total_nodes - n->d.sizes[0]);
	CU(cudaEventRecord(n->evSnapSrc, n->stream));
	CU(cudaStreamWaitEvent(n->snapStream, n->evSnapSrc, 0));
	CU(cudaMemcpyAsync(n->dSnap, n->dW, (size_t)n->nw * sizeof(float), cudaMemcpyDeviceToDevice, n->snapStream));
	CU(cudaMemcpyAsync(n->dSnap + n->nw, n->dBias, GL_MAX_WEIGHT_LAYERS * sizeof(float), cudaMemcpyDeviceToDevice, n->snapStream));
	CU(cudaMemcpyAsync(n->dSnap + n->nw + GL_MAX_WEIGHT_LAYERS, n->dPreact, np * sizeof(float), cudaMemcpyDeviceToDevice, n->snapStream));
	CU(cudaEventRecord(n->evSnapCopied, n->snapStream));
	CU(cudaStreamWaitEvent(n->stream, n->evSnapCopied, 0));  // later training may overwrite the weights only after the copy
	CU(cudaMemcpyAsync(n->hSnap, n->dSnap, snap_floats(n) * sizeof(float), cudaMemcpyDeviceToHost, n->snapStream));
	CU(cudaEventRecord(n->evSnapReady, n->snapStream));
	n->snapPending = true;
	return GL_OK;
}

// Returns GL_OK and fills w (flat weights), bias (H floats, hidden layers 1..H) and preact (pre-activations
// of layers 1..H+1 of the last row, concatenated) -- each may be NULL -- or 1 when wait == 0 and the snapshot
// has not reached host memory yet.
extern "C" int gl_snapshot_collect(gl_net* n, float* w, float* bias, float* preact, int32_t wait)
{
	if (!n) return fail(GL_ERR_INVALID, "gl_snapshot_collect: null handle");
	if (!n->snapPending) return fail(GL_ERR_STATE, "no snapshot in flight");
	if (int r = use_device(n)) return r;
	if (!wait)
	{
		const cudaError_t q = cudaEventQuery(n->evSnapReady);
		if (q == cudaErrorNotReady) return 1;
		if (q != cudaSuccess) return fail(GL_ERR_CUDA, "gl_snapshot_collect: %s", cudaGetErrorString(q));
	}
	else
		CU(cudaEventSynchronize(n->evSnapReady));
	n->snapPending = false;
	if (w) memcpy(w, n->hSnap, (size_t)n->nw * sizeof(float));
	if (bias)
		for (int l = 1; l <= n->H; ++l) bias[l - 1] = n->hSnap[n->nw + l];
	if (preact) memcpy(preact, n->hSnap + n->nw + GL_MAX_WEIGHT_LAYERS, (size_t)(n->total_nodes - n->d.sizes[0]) * sizeof(float));
	return GL_OK;
}

// Self-test of the bounded device waits: queues the exchange's wait kernel on a flag word that nothing
// ever raises, with a limit of `max_cycles` SM clock cycles.  The wait gives up when the limit runs out
// and records code 99 in the handle's status word; the next status read (gl_sync, a window's metrics)
// then reports GL_ERR_TIMEOUT, later waits of the handle return at once (the condition is sticky), and
// gl_set_weights clears it.  *waited_ms receives the device time the wait took.
extern "C" int gl_selftest_bounded_wait(gl_net* n, int64_t max_cycles, double* waited_ms)
{
	if (!n || max_cycles < 1 || max_cycles > 4000000000ll)
		return fail(GL_ERR_INVALID, "gl_selftest_bounded_wait: the limit must be between 1 and 4e9 cycles (about 2 s)");
	if (int r = use_device(n)) return r;
	unsigned* words = nullptr;
	CU(cudaMalloc(&words, 256));
	cudaError_t e = cudaMemsetAsync(words, 0, 256, n->stream);
	if (e == cudaSuccess) e = cudaEventRecord(n->ev0, n->stream);
	if (e == cudaSuccess) e = launch_dp_wait(words, 0, 0, 0, 0, 1, 1u, n->dFlags + 1, 99, n->stream, max_cycles);
	if (e == cudaSuccess) e = cudaEventRecord(n->ev1, n->stream);
	if (e == cudaSuccess) e = cudaStreamSynchronize(n->stream);
	float ms = 0;
	if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, n->ev0, n->ev1);
	cudaFree(words);
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "gl_selftest_bounded_wait: %s", cudaGetErrorString(e));
	if (waited_ms) *waited_ms = ms;
	n->launches += 1;
	return GL_OK;
}

// Diagnostic matrix product on device buffers: C[m][n] = sum_k A(m,k) * B(n,k) with
// A(m,k) = dA[m*a_sm + k*a_sk], B(n,k) = dB[n*b_sn + k*b_sk].
extern "C" int gl_matmul(const float* dA, int64_t a_sm, int64_t a_sk, const float* dB, int64_t b_sn, int64_t b_sk, float* dC,
                         int64_t ldc, int32_t M, int32_t N, int32_t K, int32_t engine, int32_t device)
{
	if (!dA || !dB || !dC || M < 1 || N < 1 || K < 1) return fail(GL_ERR_INVALID, "gl_matmul: bad argument");
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device");
	CU(cudaSetDevice(device));
	GemmArgs g;
	memset(&g, 0, sizeof g);
	g.A = dA; g.a_sm = a_sm; g.a_sk = a_sk;
	g.B = dB; g.b_sn = b_sn; g.b_sk = b_sk;
	g.C = dC; g.ldc = ldc;
	g.M = M; g.N = N; g.K = K;
	g.epi = EPI_NONE;
	if (engine == GL_GEMM_FFMA)
	{
		CU(launch_gemm_ffma(g, 0));
		CU(cudaDeviceSynchronize());
		return GL_OK;
	}
	if (!tc_gemm_supported(g)) return fail(GL_ERR_INVALID, "gl_matmul: shape or strides do not fit the tensor-core tiles");
	// extents of the two operand allocations, from their strides
	const long long ca = (a_sk == 1) ? (long long)(M - 1) * a_sm + K : (long long)(K - 1) * a_sk + M;
	const long long cb = (b_sk == 1) ? (long long)(N - 1) * b_sn + K : (long long)(K - 1) * b_sk + N;
	float *alo = nullptr, *blo = nullptr;
	int* flag = nullptr;
	CU(cudaMalloc(&alo, (size_t)(ca + 4) * sizeof(float)));
	CU(cudaMalloc(&blo, (size_t)(cb + 4) * sizeof(float)));
	CU(cudaMalloc(&flag, sizeof(int)));
	CU(cudaMemset(flag, 0, sizeof(int)));
	// a workspace of its own for the split of a partial wave of tiles along k (GLADES_TC_SPLITK=0: none)
	TcSplitK sk = {nullptr, nullptr, nullptr, 0};
	unsigned epoch = 0;
	if (!(getenv("GLADES_TC_SPLITK") && atoi(getenv("GLADES_TC_SPLITK")) == 0))
	{
		int sms = 0;
		CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
		CU(cudaMalloc(&sk.work, (size_t)sms * 128 * 256 * sizeof(float)));
		CU(cudaMalloc(&sk.flags, (size_t)sms * 8 * sizeof(unsigned)));
		CU(cudaMemset(sk.flags, 0, (size_t)sms * 8 * sizeof(unsigned)));
		sk.epoch = &epoch;
		sk.slots = (size_t)sms;
		sk.min_idle_pct = tc_splitk_min_idle_pct();
		g.sk = &sk;
	}
	cudaError_t e = launch_split_lo(dA, alo, (ca / 4) * 4, 0);
	if (e == cudaSuccess) e = launch_split_lo(dB, blo, (cb / 4) * 4, 0);
	if (e == cudaSuccess) e = launch_gemm_tc(g, alo, blo, flag, 0);
	if (e == cudaSuccess) e = cudaDeviceSynchronize();
	int hflag = 0;
	if (e == cudaSuccess) e = cudaMemcpy(&hflag, flag, sizeof hflag, cudaMemcpyDeviceToHost);
	cudaFree(alo); cudaFree(blo); cudaFree(flag); cudaFree(sk.work); cudaFree(sk.flags);
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "gl_matmul: %s", cudaGetErrorString(e));
	if (hflag) return fail(GL_ERR_TIMEOUT, "gl_matmul: a bounded wait inside the tensor-core kernel ran out (role %d)", hflag);
	return GL_OK;
}

// ------------------------------------------------------------------------------------------------
extern "C" int gl_synth_fill(float* d_out, int64_t count, uint64_t seed, uint32_t stream_id, int32_t dist, float scale,
                             float offset, int32_t device)
{
	if (!d_out || count < 0) return fail(GL_ERR_INVALID, "gl_synth_fill: bad argument");
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device");
	CU(cudaSetDevice(device));
	CU(launch_synth_fill(d_out, count, 0, seed, stream_id, dist, scale, offset, 0));
	CU(cudaDeviceSynchronize());
	return GL_OK;
}

extern "C" int gl_synth_fill_at(float* d_out, int64_t count, int64_t first_index, uint64_t seed, uint32_t stream_id, int32_t dist,
                                float scale, float offset, int32_t device)
{
	if (!d_out || count < 0 || first_index < 0) return fail(GL_ERR_INVALID, "gl_synth_fill_at: bad argument");
	if (dist == 1 && (first_index & 1)) return fail(GL_ERR_INVALID, "gl_synth_fill_at: normal draws come in pairs, first_index must be even");
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device");
	CU(cudaSetDevice(device));
	CU(launch_synth_fill(d_out, count, first_index, seed, stream_id, dist, scale, offset, 0));
	CU(cudaDeviceSynchronize());
	return GL_OK;
}

extern "C" int gl_onehot_fill(float* d_y, const int32_t* labels, int64_t rows, int32_t n, float on, float off, int32_t device)
{
	if (!d_y || !labels || rows < 1 || n < 1) return fail(GL_ERR_INVALID, "gl_onehot_fill: bad argument");
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device");
	CU(cudaSetDevice(device));
	int* dl = nullptr;
	CU(cudaMalloc(&dl, (size_t)rows * sizeof(int)));
	CU(cudaMemcpy(dl, labels, (size_t)rows * sizeof(int), cudaMemcpyHostToDevice));
	cudaError_t e = launch_onehot_fill(d_y, dl, rows, n, on, off, 0);
	if (e == cudaSuccess) e = cudaDeviceSynchronize();
	cudaFree(dl);
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "gl_onehot_fill: %s", cudaGetErrorString(e));
	return GL_OK;
}

// ---- input standardisation ---------------------------------------------------------------------
// Per-device scratch of gl_standardize_table (column statistics, kinds, plan: 36 bytes per column), kept between
// calls: a call then costs two kernels and one small read-back, not three allocations.  One call at a time per
// device (the mutex); the buffers grow with the widest table seen and live until the process ends.
namespace {
struct StdScratch
{
	int* stats = nullptr;
	int* kind = nullptr;
	void* plan = nullptr;
	int* host = nullptr;  // pinned staging: [cols][4] statistics, [cols][4] plan, [cols] kinds
	int cap = 0;
};
StdScratch g_stdScratch[64];
std::mutex g_stdMutex[64];
}  // namespace

extern "C" int gl_standardize_table(const float* d_raw, int64_t rows, int32_t cols, const int32_t* kind, const int32_t* classes,
                                    const int32_t* to_output, int32_t flag, float* d_x, int32_t* nx, float* d_y, int32_t* ny,
                                    float* stats_out, int32_t device)
{
	if (!d_raw || rows < 1 || cols < 1 || !kind || !classes || !to_output || !nx || !ny || (flag != 0 && flag != 1))
		return fail(GL_ERR_INVALID, "gl_standardize_table: bad argument");
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device: this library has no CPU path");
	CU(cudaSetDevice(device));
	int classification = 0;
	for (int c = 0; c < cols; ++c)
	{
		if (kind[c] != 0 && kind[c] != 1) return fail(GL_ERR_INVALID, "gl_standardize_table: kind[%d] must be 0 or 1", c);
		if (kind[c] == 1)
		{
			if (classes[c] < 1) return fail(GL_ERR_INVALID, "gl_standardize_table: categorical column %d has no classes", c);
			classification = 1;
		}
	}
	// pass 1: extrema.  Raw column 0 starts from its own first cell (a neutral start gives the same extrema),
	// every other column from 0.0 (NumberInput.cpp:105-109).
	std::vector<int> st((size_t)cols * 4, 0);
	for (int c = 0; c < cols; ++c)
	{
		st[4 * (size_t)c] = (c == 0) ? 0x7FFFFFFF : float_order_host(0.0f);
		st[4 * (size_t)c + 1] = (c == 0) ? (int)0x80000000 : float_order_host(0.0f);
	}
	if (device < 0 || device >= 64) return fail(GL_ERR_INVALID, "gl_standardize_table: device ordinal out of range");
	std::lock_guard<std::mutex> lock(g_stdMutex[device]);
	StdScratch& sc = g_stdScratch[device];
	if (sc.cap < cols)
	{
		cudaFree(sc.stats);
		cudaFree(sc.kind);
		cudaFree(sc.plan);
		cudaFreeHost(sc.host);
		sc = StdScratch();
		CU(cudaMalloc(&sc.stats, (size_t)cols * 4 * sizeof(int)));
		CU(cudaMalloc(&sc.kind, (size_t)cols * sizeof(int)));
		CU(cudaMalloc(&sc.plan, (size_t)cols * 4 * sizeof(int)));
		CU(cudaMallocHost(&sc.host, (size_t)cols * 9 * sizeof(int)));
		sc.cap = cols;
	}
	int* dStats = sc.stats;
	int* dKind = sc.kind;
	void* dPlan = sc.plan;
	// the small records travel through pinned staging as asynchronous copies on the stream of the kernels: one
	// wait for the extrema (the layout depends on them), one at the end
	int* hStats = sc.host;
	int* hPlan = sc.host + (size_t)cols * 4;
	int* hKind = sc.host + (size_t)cols * 8;
	memcpy(hStats, st.data(), st.size() * sizeof(int));
	cudaError_t e = cudaMemcpyAsync(dStats, hStats, st.size() * sizeof(int), cudaMemcpyHostToDevice, 0);
	if (e == cudaSuccess) e = launch_column_minmax(d_raw, rows, cols, dStats, 0);
	if (e == cudaSuccess && flag == 1)
	{
		memcpy(hKind, kind, (size_t)cols * sizeof(int));
		e = cudaMemcpyAsync(dKind, hKind, (size_t)cols * sizeof(int), cudaMemcpyHostToDevice, 0);
		if (e == cudaSuccess) e = launch_column_mean_stdev(d_raw, rows, cols, dKind, reinterpret_cast<float*>(dStats), 0);
	}
	if (e == cudaSuccess) e = cudaMemcpyAsync(hStats, dStats, st.size() * sizeof(int), cudaMemcpyDeviceToHost, 0);
	if (e == cudaSuccess) e = cudaStreamSynchronize(0);
	if (e == cudaSuccess) memcpy(st.data(), hStats, st.size() * sizeof(int));
	// the layout: columns keep their raw order inside each destination; a numeric column whose range is 0 is
	// copied unscaled and lands in the input matrix whatever its output mark (NumberInput.cpp:166-171)
	int* plan = hPlan;
	int cx = 0, cy = 0;
	if (e == cudaSuccess)
		for (int c = 0; c < cols; ++c)
		{
			int dst = to_output[c] ? 1 : 0;
			int width = 1;
			if (kind[c] == 1) width = classes[c];
			else if (flag == 0 && order_float_host(st[4 * (size_t)c + 1]) - order_float_host(st[4 * (size_t)c]) == 0.0f) dst = 0;
			plan[4 * (size_t)c] = kind[c];
			plan[4 * (size_t)c + 1] = classes[c];
			plan[4 * (size_t)c + 2] = dst;
			plan[4 * (size_t)c + 3] = dst ? cy : cx;
			(dst ? cy : cx) += width;
		}
	int status = GL_OK;
	if (e == cudaSuccess && (d_x || d_y))
	{
		if (*nx != cx || *ny != cy || (cx > 0 && !d_x) || (cy > 0 && !d_y))
			status = fail(GL_ERR_INVALID, "gl_standardize_table: the table standardises to %d input and %d expected columns, the caller gave %d and %d",
			              cx, cy, *nx, *ny);
		else
		{
			e = cudaMemcpyAsync(dPlan, plan, (size_t)cols * 4 * sizeof(int), cudaMemcpyHostToDevice, 0);
			if (e == cudaSuccess) e = launch_column_transform(d_raw, rows, cols, dPlan, dStats, flag, classification, d_x, cx, d_y, cy, 0);
			if (e == cudaSuccess) e = cudaStreamSynchronize(0);
		}
	}
	if (e != cudaSuccess) return fail(GL_ERR_CUDA, "gl_standardize_table: %s", cudaGetErrorString(e));
	if (status != GL_OK) return status;
	*nx = cx;
	*ny = cy;
	if (stats_out)
		for (int c = 0; c < cols; ++c)
		{
			stats_out[4 * (size_t)c] = order_float_host(st[4 * (size_t)c]);
			stats_out[4 * (size_t)c + 1] = order_float_host(st[4 * (size_t)c + 1]);
			memcpy(&stats_out[4 * (size_t)c + 2], &st[4 * (size_t)c + 2], 2 * sizeof(float));
		}
	return GL_OK;
}

extern "C" int gl_device_alloc(void** p, int64_t bytes, int32_t device)
{
	if (!p || bytes < 0) return fail(GL_ERR_INVALID, "gl_device_alloc: bad argument");
	if (gl_device_count() < 1) return fail(GL_ERR_NO_DEVICE, "no sm_100 CUDA device");
	CU(cudaSetDevice(device));
	CU(cudaMalloc(p, (size_t)bytes));
	return GL_OK;
}
extern "C" int gl_device_mem_info(int32_t device, int64_t* free_bytes, int64_t* total_bytes)
{
	CU(cudaSetDevice(device));
	size_t f = 0, t = 0;
	CU(cudaMemGetInfo(&f, &t));
	if (free_bytes) *free_bytes = (int64_t)f;
	if (total_bytes) *total_bytes = (int64_t)t;
	return GL_OK;
}
extern "C" int gl_device_free(void* p, int32_t device)
{
	CU(cudaSetDevice(device));
	CU(cudaFree(p));
	return GL_OK;
}
extern "C" int gl_memcpy_h2d(void* d, const void* h, int64_t bytes, int32_t device)
{
	CU(cudaSetDevice(device));
	CU(cudaMemcpy(d, h, (size_t)bytes, cudaMemcpyHostToDevice));
	return GL_OK;
}
extern "C" int gl_memcpy_d2h(void* h, const void* d, int64_t bytes, int32_t device)
{
	CU(cudaSetDevice(device));
	CU(cudaMemcpy(h, d, (size_t)bytes, cudaMemcpyDeviceToHost));
	return GL_OK;
}
extern "C" int gl_host_alloc_pinned(void** p, int64_t bytes)
{
	if (!p || bytes < 0) return fail(GL_ERR_INVALID, "gl_host_alloc_pinned: bad argument");
	CU(cudaMallocHost(p, (size_t)bytes));
	return GL_OK;
}
extern "C" int gl_host_free_pinned(void* p)
{
	CU(cudaFreeHost(p));
	return GL_OK;
}
