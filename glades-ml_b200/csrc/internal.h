// Internal declarations shared by the C-ABI layer (api.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "glades_b200.h"

namespace glb {

// Device-side view of one network, passed by value to the kernels.
struct NetView
{
	int H;                                   // hidden layers; weight layers are 0..H
	int sizes[GL_MAX_WEIGHT_LAYERS + 1];
	float lr[GL_MAX_WEIGHT_LAYERS], mom[GL_MAX_WEIGHT_LAYERS], wd1[GL_MAX_WEIGHT_LAYERS], wd2[GL_MAX_WEIGHT_LAYERS];
	int act[GL_MAX_WEIGHT_LAYERS];
	float par[GL_MAX_WEIGHT_LAYERS];
	int out_type;
	int mb;
	float* W[GL_MAX_WEIGHT_LAYERS];          // W_l [n_{l+1}][n_l], slices of one flat allocation
	float* bias;                             // [GL_MAX_WEIGHT_LAYERS], entry l used for l = 1..H
};

// ---- reference mode (ref_mode.cu) ----------------------------------------------------------
struct RefTrainArgs
{
	NetView net;
	float* hist[GL_MAX_WEIGHT_LAYERS];  // pending deltas [mb][n_{l+1}*n_l]
	int* hist_len;                      // device scalar
	const float* X;
	const float* Y;
	long long rows;
	int n_epochs;
	float* scratch;                     // 3 * total_nodes floats: activations, error accumulators, d / base
	float* epoch_sums;                  // [n_epochs][2]: raw cost sum, raw accuracy sum
	int* confusion;                     // [n_out][n_out], counts of the LAST epoch
	float* outputs;                     // optional [rows][n_out], predictions of the last epoch
	float* last_out;                    // [n_out]: predictions of the last row of the last epoch
	int* flags;                         // [0] non-finite weight seen after the call
	int weights_in_smem;                // stage W and hist in shared memory for the whole launch
	// dropout (masks != NULL selects the dropout kernel: one epoch per launch, n_epochs is ignored)
	const unsigned char* masks;         // [rows][mask_stride]: 1 = node dropped; node layers 0..H side by side
	int mask_stride;                    // n_0 + ... + n_H
	int train;                          // 0: forward + metrics only (the test pass drops nodes too)
	int* hlen[GL_MAX_WEIGHT_LAYERS];    // per edge: deltas pushed since its last apply
	float* hlast[GL_MAX_WEIGHT_LAYERS]; // per edge: the last pushed delta
	float* err_state;                   // [total nodes]: error accumulators carried from launch to launch
	long long data_rows;                // rows of the data set for the cost divisor (0: `rows`)
	float* acts_out;                    // optional: activations of layers 1..H+1 of the LAST row, concatenated
	float* preact_out;                  // optional: pre-activations (sum + bias, before the activation function) of
	                                    // layers 1..H+1 for the LAST row of the LAST epoch, concatenated: what the
	                                    // reference collects for its live view (network.cpp:510-514)
};
size_t ref_train_smem_bytes(const NetView& n, bool weights_in_smem);
size_t ref_train_dropout_smem_bytes(const NetView& n);
cudaError_t launch_ref_train(const RefTrainArgs& a, cudaStream_t s);

// Exact-order forward of rows [first, first+rows): one thread per (row, output node), k ascending.
// acts: per-layer activation buffers [rows][n_l] for l = 1..H+1 (device).
// zout (optional): pre-activations of layers 1..H+1 of row 0 of the call, concatenated
cudaError_t launch_ref_forward(const NetView& n, const float* X, long long rows, float* const* acts, cudaStream_t s,
                               float* zout = nullptr);
// Sequential (row-major) metric accumulation over predictions P [rows][n_out] against Y.
cudaError_t launch_ref_metrics(const NetView& n, const float* P, const float* Y, long long rows, long long data_rows,
                               float* sums2, int* confusion, cudaStream_t s);

// ---- batched mode (batched.cu) ---------------------------------------------------------------
enum { EPI_NONE = 0, EPI_FORWARD = 1, EPI_ERRPROP = 2, EPI_GRAD = 3 };
// Workspace of the tensor-core kernel's split of a partial wave of tiles along k: one 128 x 256 fp32 partial
// tile and eight flag words per CTA, and the host-side launch counter the flags are compared with.  One
// workspace serves the launches of ONE stream (consecutive launches reuse it; the flags only ever grow).
struct TcSplitK
{
	float* work;       // device, slots * 128 * 256 floats
	unsigned* flags;   // device, slots * 8 words, zero-initialised
	unsigned* epoch;   // host counter
	size_t slots;      // CTAs the workspace has room for
	int min_idle_pct;  // split only where the last wave would leave at least this share of the SMs idle
};
// the share of idle SMs from which a last wave is split (GLADES_TC_SPLITK_IDLE, percent; default 25)
int tc_splitk_min_idle_pct();
struct GemmArgs
{
	// C[M][N] (ldc) = sum_k A(m,k) * B(n,k);  A(m,k) = A[m*a_sm + k*a_sk], B(n,k) = B[n*b_sn + k*b_sk]
	const float* A;
	const float* B;
	float* C;
	float* C_lo;           // tensor-core kernel only: also write the low TF32 part of C here (same layout), or NULL
	int M, N, K;
	long long a_sm, a_sk, b_sn, b_sk, ldc;
	const float* kscale;   // optional per-k factor (momentum weights c_j), applied to A(m,k)
	int epi;
	// EPI_FORWARD: C = squash(acc + bias, act, par).  EPI_ERRPROP: C = acc * act'(aux[m][n]).
	// EPI_GRAD: C = alpha * acc + colterm[n]
	const float* bias_ptr;  // device scalar added before the activation, or NULL
	int act;
	float par;
	const float* aux;
	long long ld_aux;
	float alpha;
	const float* colterm;
	// tensor-core kernel, ReLU layers: the forward epilogue can record (output > 0) as one bit per element
	// ([M][N/32] words) and the error-propagation epilogue can read that instead of the fp32 activations
	unsigned* relu_mask_out;
	const unsigned* relu_mask_in;
	int sm_reserve;        // tensor-core kernel: leave this many SMs without a CTA (for a concurrent collective)
	// tensor-core kernel, data-parallel weight gradient: row band o of C goes to rank o's memory through
	// peer_maps[o] (device array of 128-byte tensor maps) / peer_bases[o]; NULL = everything to C
	const void* peer_maps;
	float* const* peer_bases;
	int band_rows;
	int peer_self;         // this rank (the walk over the owners' bands starts with the rank after it)
	const TcSplitK* sk;    // tensor-core kernel: workspace for splitting a partial wave of tiles along k, or NULL
};
cudaError_t launch_gemm_ffma(const GemmArgs& g, cudaStream_t s);

struct HeadArgs
{
	// Output layer: predictions P [rows][n] (for softmax: logits in, probabilities out), targets Y,
	// writes D = delta of the output layer and accumulates metrics.
	float* P;
	const float* Y;
	float* D;          // may be NULL (inference)
	float* D_lo;       // optional: low TF32 part of D for the tensor-core products
	int rows, n;
	int out_type;
	int softmax;
	float data_size;   // rows_of_epoch * n_out, the cost divisor
	double* sums2;     // [0] cost sum, [1] accuracy sum (atomic)
	int* confusion;    // [n][n] or NULL
	int* argmax;       // optional [rows]
};
cudaError_t launch_head(const HeadArgs& h, cudaStream_t s);

// sum over all elements of D [rows*n] times alpha, atomically added to *out
// *out += alpha * sum(D), reproducibly; part: SUM_SCALED_MAX_BLOCKS doubles of scratch, ticket: one zeroed word (both owned
// by the caller and used by one launch at a time)
constexpr int SUM_SCALED_MAX_BLOCKS = 148 * 8;
cudaError_t launch_sum_scaled(const float* D, long long count, float alpha, float* out, double* part, unsigned* ticket, cudaStream_t s);
// colterm[i] = lr * sum_j c_j * (wd1*|A[j][i]| + wd2*A[j][i])
cudaError_t launch_decay_colterm(const float* A, int rows, int n, const float* c, float lr, float wd1, float wd2,
                                 float* colterm, cudaStream_t s);
// W -= G * inv_mb for the flat weight vector; biases b_l -= gb_l * bscale_l; sets flags[0] on non-finite
// W_lo (optional): the low TF32 part of the updated weights, for the tensor-core products
cudaError_t launch_update(float* W, float* W_lo, const float* G, long long count, float inv_mb, float* bias, const float* gb,
                          const float* bscale, int H, int* flags, cudaStream_t s);

// ---- batched mode, whole small network in shared memory (small_fused.cu) -------------------------
struct SmallFusedArgs
{
	NetView net;
	const float* X;
	const float* Y;
	long long rows;
	int n_epochs;
	int bias_rule;
	double* epoch_sums;  // [n_epochs][2]: cost sum, accuracy sum
	int* confusion;      // [n_out][n_out], counts of the last epoch
	float* last_out;     // [n_out]
	int* flags;
};
size_t small_fused_smem_bytes(const NetView& n);
cudaError_t launch_small_fused(const SmallFusedArgs& a, cudaStream_t s);

// ---- batched mode, mid-size network, one cooperative launch over all SMs (grid_fused.cu) ----------
struct GridFusedArgs
{
	NetView net;         // net.mb = rows per window
	const float* X;
	const float* Y;
	long long rows;      // rows this launch walks through, in windows of net.mb, n_epochs times
	int n_epochs;
	int bias_rule;
	float data_size;     // the cost divisor: rows of the epoch * n_out
	float* actbuf;       // [net.mb][grid_fused_scratch_pitch] scratch: the window's activations
	float* delbuf;       // [net.mb][grid_fused_scratch_pitch] scratch: the window's deltas
	double* part;        // [part_ctas][2 + GL_MAX_WEIGHT_LAYERS] per-CTA partial sums of a window
	int part_ctas;       // = the grid of the launch (one CTA per SM)
	const float* ck;     // [H+1][net.mb+1]: ck[l][k] = sum_{q<k} momentum_l^q
	double* epoch_sums;  // [n_epochs][2]: cost sum, accuracy sum
	int* confusion;      // [n_out][n_out]: the last epoch's counts are ADDED (the caller clears)
	float* last_out;     // [n_out] or NULL
	int* flags;
	// Device array of 128-byte tensor maps, two per weight layer -- [2l]: W_l as [n_out][n_in] with boxes of
	// 256 rows x 32 columns, 128-byte swizzle (forward tiles); [2l+1]: boxes of 32 rows x 256 columns, plain
	// (hidden-delta tiles) -- or NULL: the weights' layout allows no tensor maps (rows not multiples of 16
	// bytes) and the tiles travel through registers instead.
	const void* tma;
	unsigned long long* timing;  // optional diagnostics: ns spent in [phase 1, barrier, phase 2, barrier] by CTA 0
};
size_t grid_fused_smem_bytes(const NetView& n);
int grid_fused_total_nodes(const NetView& n);
// floats per row of the window scratch (every layer padded to a multiple of 4 columns)
int grid_fused_scratch_pitch(const NetView& n);
// weight tiles one sample group walks through (the ring path needs <= 512)
int grid_fused_group_tiles(const NetView& n);
cudaError_t launch_grid_fused(const GridFusedArgs& a, cudaStream_t s);
// cluster variant (thread-block clusters of 8 CTAs share a group of rows, every CTA owning an eighth of each
// layer's nodes with their weights resident in shared memory): same arguments, part_ctas = a multiple of 8 that
// cluster_fused_max_ctas allows; tma is not used
bool cluster_fused_fits(const NetView& n);
size_t cluster_fused_smem_bytes(const NetView& n);
int cluster_fused_max_ctas(const NetView& n);
cudaError_t launch_cluster_fused(const GridFusedArgs& a, cudaStream_t s);

// ---- data-parallel gradient exchange over peer memory (dp_push.cu) ---------------------------------
// Every rank owns an exchange arena that all ranks map: a flag area of DP_FLAG_BYTES (32-bit window
// counters written by peers, then the small per-rank records) followed by one gradient slot per
// source rank.  Word indices inside the flag area:
//   DP_WORD_GFLAG + l * DP_MAX_WORLD + src    src's contribution to layer l has landed here
//   DP_WORD_WFLAG + l * DP_MAX_WORLD + owner  owner's band of the new layer-l weights has landed here
//   DP_WORD_SFLAG + src                       src's bias / loss record has landed here
//   DP_WORD_BAD + owner                       owner saw a non-finite weight (sticky)
//   DP_WORD_HELLO + src                       set-up handshake: src's test pattern has landed in its slot here
enum
{
	DP_MAX_WORLD = 8,
	DP_WORD_GFLAG = 0,
	DP_WORD_WFLAG = GL_MAX_WEIGHT_LAYERS * DP_MAX_WORLD,
	DP_WORD_SFLAG = 2 * GL_MAX_WEIGHT_LAYERS * DP_MAX_WORLD,
	DP_WORD_BAD = DP_WORD_SFLAG + DP_MAX_WORLD,
	DP_WORD_HELLO = DP_WORD_BAD + DP_MAX_WORLD,  // + src: set-up handshake (src's test pattern has landed here)
	DP_SMALL_OFFSET = 2048,  // bytes: records [parity 2][rank DP_MAX_WORLD][DP_SMALL_BYTES]
	DP_SMALL_BYTES = 128,    // GL_MAX_WEIGHT_LAYERS floats (bias sums) + 2 doubles (cost, accuracy sums)
	DP_FLAG_BYTES = 4096
};
struct DpPeers { void* p[DP_MAX_WORLD]; };  // one pointer per rank (this rank's own entry is a local pointer)

cudaError_t launch_dp_signal(const DpPeers& flags, int world, int word, unsigned value, cudaStream_t s);
// max_cycles <= 0: the default bound (about 10 s)
cudaError_t launch_dp_wait(const void* arena, int w0, int groups, int per_group, int extra0, int extra_n, unsigned value,
                           int* status, int code, cudaStream_t s, long long max_cycles = 0);
// Set-up handshake.  hello_write: thread r < world stores the pattern (self + 1) * 1000 + k, k < 16, at the head of
// this rank's slot in rank r's arena, then raises DP_WORD_HELLO + self there.  hello_check (after a wait on
// those words): every source's pattern must be in its slot here, else *status = code.
cudaError_t launch_dp_hello_write(const DpPeers& slot_heads, const DpPeers& flags, int world, int self, cudaStream_t s);
cudaError_t launch_dp_hello_check(const float* slots, long long slot_stride, int world, int* status, int code, cudaStream_t s);
cudaError_t launch_dp_push_bands(const float* G, int n_out, int n_in, int band, const DpPeers& slot, cudaStream_t s);
// w_own: this rank's weight vector (read); W.p[r]: rank r's destination vector (the staging vector inside its arena)
cudaError_t launch_dp_reduce_update(const float* part, long long src_stride, int world, long long count, float inv_mb,
                                    long long wbase, const float* w_own, const DpPeers& W, int self, const DpPeers& flags, int blocks,
                                    cudaStream_t s);
cudaError_t launch_dp_small_push(const float* gb, const double* sums2, const DpPeers& flags, int world, int self, int parity,
                                 unsigned value, cudaStream_t s);
cudaError_t launch_dp_finish(const void* arena, int world, int parity, float* gb_out, double* sums2_out, float* bias,
                             const float* bscale, int H, int* status_flags, cudaStream_t s);

// ---- input standardisation (preprocess.cu) -------------------------------------------------------
// d_stats: device [cols][4] words per column: order image of the minimum, of the maximum (ints), then the
// mean and the standard deviation (floats).  The caller presets the two images to the column's start values.
cudaError_t launch_column_minmax(const float* raw, long long rows, int cols, int* d_stats, cudaStream_t s);
cudaError_t launch_column_mean_stdev(const float* raw, long long rows, int cols, const int* d_kind, float* d_stats, cudaStream_t s);
// d_plan: device array of `cols` records {kind, classes, destination matrix (0 X, 1 Y), first destination column}
cudaError_t launch_column_transform(const float* raw, long long rows, int cols, const void* d_plan, const int* d_stats, int flag,
                                    int classification, float* X, int ldx, float* Y, int ldy, cudaStream_t s);
int float_order_host(float f);    // the order-preserving integer image used for the min / max atomics
float order_float_host(int i);

// ---- synthetic inputs (synth.cu) ---------------------------------------------------------------
// out[j] = element (first + j) of stream `stream_id`; `first` must be even for dist 1
cudaError_t launch_synth_fill(float* out, long long n, long long first, unsigned long long seed, unsigned stream_id, int dist,
                              float scale, float offset, cudaStream_t s);

// y[r][c] = (c == labels[r]) ? on : off  (expected rows in the reference's one-hot convention)
cudaError_t launch_onehot_fill(float* y, const int* labels, long long rows, int n, float on, float off, cudaStream_t s);

}  // namespace glb
