/*
 * glades_b200.h -- C ABI of the B200-native deep feed-forward train/infer path.
 *
 * The reference library (Gattic/glades-ml) has no FFI: its feed-forward path is the C++ member
 * function NNetwork::run (Backend/Machine Learning/Networks/network.cpp:114-397) and the
 * per-node / per-edge heap objects below it (State/LayerBuilder.cpp, State/node.cpp,
 * State/edge.cpp, GMath/gmath.cpp, GMath/cmatrix.cpp).  This header is the boundary a maintainer
 * binds instead: plain pointers and sizes, no C++ or torch types.  Each entry point names the
 * reference code it replaces.  All entry points return 0 on success or a negative gl_status;
 * gl_last_error() gives the text of the last failure on the calling thread.
 *
 * Layout conventions (all fp32, row-major):
 *   layers 0..H+1 (0 = input, H+1 = output), n_l nodes each;
 *   W_l is [n_{l+1}][n_l] (node-major, edge-minor, the order of LayerBuilder::getWeights,
 *   State/LayerBuilder.cpp:390-410); the flat weight vector is W_0 | W_1 | ... | W_H;
 *   one scalar bias per hidden layer l = 1..H (State/layer.h:35), used when computing layer l+1;
 *   X is [rows][n_0], Y (expected) is [rows][n_{H+1}].
 *
 * The library needs a CUDA device of compute capability 10.0 (B200); there is no CPU path.
 */
#ifndef GLADES_B200_H
#define GLADES_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GL_MAX_WEIGHT_LAYERS 16

/* activation ids: GMath::TANH..STEP, GMath/gmath.h:43-50; GL_ACT_SOFTMAX is an extension that
 * the reference does not have (it is only legal on the last layer of a batched-mode network). */
enum { GL_ACT_TANH = 0, GL_ACT_TANHP = 1, GL_ACT_SIGMOID = 2, GL_ACT_SIGMOIDP = 3, GL_ACT_LINEAR = 4,
       GL_ACT_RELU = 5, GL_ACT_LEAKY = 6, GL_ACT_STEP = 7, GL_ACT_SOFTMAX = 8 };
/* cost ids: GMath::REGRESSION / CLASSIFICATION / KL, GMath/gmath.h:38-40 */
enum { GL_OUT_REGRESSION = 0, GL_OUT_CLASSIFICATION = 1, GL_OUT_KL = 2 };

/* Arithmetic mode.
 * GL_MODE_REFERENCE reproduces NNetwork::SGDHelper exactly, sample after sample: the online scalar
 * bias update (network.cpp:653-656), the doubling error accumulation (network.cpp:660-662 with
 * State/node.cpp:173-176), the {0},{1..mb},{mb+1..2mb} apply rows (network.cpp:646-651) and the
 * intra-window momentum history (node.cpp:278-307).  It is sequential by construction.
 * GL_MODE_BATCHED is the data-parallel mode: aligned windows of batch_size rows, weights and
 * biases frozen inside a window, plain error sum, bias delta summed per window, optional
 * softmax + cross-entropy head.  It is the only mode that shards over GPUs. */
enum { GL_MODE_REFERENCE = 0, GL_MODE_BATCHED = 1 };

/* Batched-mode scalar-bias step: GL_BIAS_MEAN b_l -= lr_l*sum(D)/mb; GL_BIAS_REFERENCE keeps the
 * reference's magnitude b_l -= n_l*lr_l*sum(D) (the update runs once per (input, output) pair
 * per sample, network.cpp:585-587,653-656). */
enum { GL_BIAS_MEAN = 0, GL_BIAS_REFERENCE = 1 };

/* Engine of batched mode.  GL_GEMM_AUTO picks by size: whole-network fused kernels for small and
 * mid-size networks on one GPU (all weights in one SM's shared memory; or one cooperative launch
 * over all SMs per window), else one matrix product per layer and pass, on the tensor cores where
 * the shape fits and is large enough.  GL_GEMM_FFMA forces the per-layer products on the exact-fp32
 * FFMA tile kernel; GL_GEMM_TCGEN05 forces them on the TMA + tcgen05 3xTF32 kernel wherever the
 * shape fits its tiles, however small; GL_GEMM_GRID_FUSED forces the cooperative whole-window kernel
 * (gl_create fails if the network does not fit it). */
enum { GL_GEMM_AUTO = 0, GL_GEMM_FFMA = 1, GL_GEMM_TCGEN05 = 2, GL_GEMM_GRID_FUSED = 3 };

typedef enum gl_status {
	GL_OK = 0,
	GL_ERR_INVALID = -1,    /* bad argument / descriptor */
	GL_ERR_CUDA = -2,       /* a CUDA call failed; text in gl_last_error() */
	GL_ERR_NO_DEVICE = -3,  /* no sm_100 device: there is no CPU fallback */
	GL_ERR_STATE = -4,      /* call order (no data, no weights, wrong mode) */
	GL_ERR_NONFINITE = -5,  /* reserved: weights went inf/NaN (reported in gl_metrics, not fatal) */
	GL_ERR_TIMEOUT = -6,    /* a bounded device-side wait ran out */
	GL_ERR_COMM = -7,       /* NCCL failure */
	GL_ERR_TOO_LARGE = -8   /* size beyond a stated maximum */
} gl_status;

/* Hyper-parameters of one network, as NNInfo hands them to the loop.  Index l of the per-layer
 * arrays is NNInfo's index l (Structure/nninfo.cpp:240-373): l = 0 the InputLayerInfo, l >= 1
 * hidden layer l-1; entry l governs W_l and the activation that produces layer l+1
 * (network.cpp:505-506,635-638).  The caller resolves NNInfo's quirks when filling it, e.g.
 * getWeightDecay2(0) returning weightDecay1 (nninfo.cpp:305-306). */
typedef struct gl_net_desc {
	int32_t n_layers;                          /* node layers incl. input and output = H + 2 */
	int32_t sizes[GL_MAX_WEIGHT_LAYERS + 1];   /* n_0 .. n_{H+1} */
	float lr[GL_MAX_WEIGHT_LAYERS];
	float momentum[GL_MAX_WEIGHT_LAYERS];
	float wd1[GL_MAX_WEIGHT_LAYERS];
	float wd2[GL_MAX_WEIGHT_LAYERS];
	float p_dropout[GL_MAX_WEIGHT_LAYERS];     /* dropout probability of NODE layer j = 0..H (0 = input), as the loop
	                                            * uses it: [0] = NNInfo::getPInput(), [j] = getPDropout(j-1), whose
	                                            * index 0 is again the input layer's value (nninfo.cpp:140-146,
	                                            * 321-333).  Reference mode only; see gl_train_epochs. */
	int32_t activation[GL_MAX_WEIGHT_LAYERS];
	float act_param[GL_MAX_WEIGHT_LAYERS];
	int32_t output_type;                       /* GL_OUT_* (NNInfo::getOutputType) */
	int32_t batch_size;                        /* NNInfo::getBatchSize, nninfo.cpp:154-160 */
	int32_t mode;                              /* GL_MODE_* */
	int32_t bias_rule;                         /* GL_BIAS_*, batched mode only */
	int32_t gemm;                              /* GL_GEMM_* */
	int32_t device;                            /* CUDA device ordinal */
} gl_net_desc;

/* Per-epoch (or per-call) statistics: the members NNetwork::run leaves behind
 * (network.cpp:179-224): overallTotalError, overallTotalAccuracy (already divided by
 * rows*n_out) and the five confusion-matrix figures in percent. */
typedef struct gl_metrics {
	float total_error;
	float total_accuracy;
	float class_accuracy;
	float class_precision;
	float class_recall;
	float class_specificity;
	float class_f1;
	int32_t epochs;          /* epochs completed by this handle so far */
	int32_t nonfinite;       /* 1 if a weight or bias is inf/NaN after the call */
	int64_t rows;            /* rows the figures cover (all ranks) */
	double device_ms;        /* device time of the call, CUDA events on the library's stream */
	int64_t kernel_launches; /* kernels of this library launched by the call */
} gl_metrics;

typedef struct gl_net gl_net;

const char* gl_last_error(void);
/* Number of usable sm_100 devices (0 when there is none or no driver). */
int gl_device_count(void);

/* Replaces LayerBuilder::build (State/LayerBuilder.cpp:54-98) minus the weight draw: allocates
 * the per-layer device matrices.  Weights start at 0 until gl_set_weights. */
int gl_create(const gl_net_desc* desc, gl_net** out);
/* Replaces LayerBuilder::clean / NNetwork::~NNetwork. */
int gl_destroy(gl_net* net);

/* Replaces Node::setEdgeWeight / Layer::setBiasWeight (State/node.cpp:142-148,
 * State/layer.cpp:70-73) for the whole network.  bias has H entries (hidden layers 1..H) and
 * may be NULL (= zeros).  Also clears pending deltas and error accumulators. */
int gl_set_weights(gl_net* net, const float* w_flat, const float* bias);
/* Replaces LayerBuilder::getWeights (State/LayerBuilder.cpp:390-410) + Layer::getBiasWeight. */
int gl_get_weights(gl_net* net, float* w_flat, float* bias);
/* Total number of weights, sum of n_{l+1}*n_l. */
int64_t gl_weight_count(const gl_net* net);

/* Checkpoint and true resume: writes / reads one binary file holding the shapes, the flat weights,
 * the scalar biases, the epoch counter and -- reference mode -- every edge's pending deltas of the
 * open minibatch window, so that a loaded network continues exactly where the saved one stood.
 * gl_load_state refuses a file written by a network of another shape, mode or minibatch size.
 * The reference saves only the NNInfo skeleton; its weight persistence is commented out
 * (Networks/network.cpp:701-722, State/LayerBuilder.cpp:659-709). */
int gl_save_state(gl_net* net, const char* path);
int gl_load_state(gl_net* net, const char* path);

/* Replaces LayerBuilder::buildInputLayers (State/LayerBuilder.cpp:101-189) and the
 * DataInput::getTrainRow / getTrainExpectedRow reads of the loop (network.cpp:523,605): the rows
 * are packed once.  Host pointers are copied (through pinned staging) before the call returns. */
int gl_set_data(gl_net* net, const float* x, const float* y, int64_t rows);
/* Same, for rows that already live in device memory; the buffers are borrowed, not copied, and
 * must outlive the handle's use of them.  d_y may be NULL for forward-only use without metrics. */
int gl_set_data_device(gl_net* net, const float* d_x, const float* d_y, int64_t rows);

/* The host-buffer window step as a two-deep pipeline: submit() queues the copy of the rows (x and y must
 * stay valid, and should be pinned, until the matching result() returns) and the step, and returns at
 * once; result() waits for the oldest submitted window and reports its figures.  At most two windows are
 * in flight, so the copy of one overlaps the compute of the other.  No counterpart in the reference. */
int gl_train_window_host_submit(gl_net* net, const float* x, const float* y, int32_t rows);
int gl_train_window_host_result(gl_net* net, gl_metrics* out);
/* Batched mode, inference from host buffers with two batches in flight (the test() pass of
 * NNetwork::run, network.cpp:109-112,428, fed batch by batch): submit copies `rows` (<= 65536) rows
 * in on a copy stream while the previous batch still computes and queues the forward pass; result
 * waits for the OLDEST batch and hands out its predicted classes (argmax, `rows` ints, may be NULL)
 * and -- when expected rows were given -- its cost / accuracy sums over that batch.  Confusion counts
 * are not kept on this path.  Shares its two slots with gl_train_window_host_submit. */
int gl_forward_host_submit(gl_net* net, const float* x, const float* y, int32_t rows);
int gl_forward_host_result(gl_net* net, int32_t* argmax, gl_metrics* out);

/* Replaces n iterations of the epoch loop of NNetwork::run with RUN_TRAIN
 * (network.cpp:173-256): every row through SGDHelper (forward, metrics, confusion counts,
 * backward, update).  out (may be NULL) receives the last epoch's figures.
 * Dropout (reference mode, any p_dropout != 0; replaces LayerBuilder::scrambleDropout and
 * Layer::generateDropout, State/LayerBuilder.cpp:497-523, State/layer.cpp:102-134, and the skip rules
 * of network.cpp:480-488,620-657): before every epoch -- and before every gl_forward /
 * gl_get_activations, the reference drops nodes in its test pass too -- the library draws the node
 * flags of all rows on the host with the C library's rand(), one call per node in the reference's
 * order (per row: input layer, then hidden layers; integer-percent threshold rand() % 100 + 1 <=
 * int(p * 100); a layer that came out all dropped is drawn again; int(p * 100) >= 100 draws nothing).
 * After the same srand() the same nodes drop as in the reference. */
int gl_train_epochs(gl_net* net, int32_t n_epochs, gl_metrics* out);
/* Batched mode: one window step (forward, backward, update) over rows
 * [first_row, first_row+rows) of the resident data.  Under data parallelism each rank passes its
 * own shard of the global window and the gradient is all-reduced before the update.  The cost in
 * `out` is divided by (rows of the global window * n_out); gl_train_epochs divides by the data set's rows
 * as the reference does. */
int gl_train_window(gl_net* net, int64_t first_row, int32_t rows, gl_metrics* out);
/* Batched mode: the same step with the window's rows in host memory (copied in by the call). */
int gl_train_window_host(gl_net* net, const float* x, const float* y, int32_t rows, gl_metrics* out);

/* Replaces NNetwork::run with RUN_TEST (network.cpp:109-112,428): forward only over rows
 * [first_row, first_row+rows) of the resident data.  outputs ([rows][n_out], host) and argmax
 * ([rows], host; -1 when no output exceeds 0, GMath::naiveVectorDecomp gmath.cpp:435-455) may
 * each be NULL.  Metrics and confusion counts are accumulated exactly as the train pass does. */
int gl_forward(gl_net* net, int64_t first_row, int64_t rows, float* outputs, int32_t* argmax, gl_metrics* out);
/* Forward over rows in host memory (copied in by the call), results to host memory. */
int gl_forward_host(gl_net* net, const float* x, const float* y, int64_t rows, float* outputs, int32_t* argmax,
                    gl_metrics* out);

/* Activations of every non-input layer for one resident row, concatenated n_1 | ... | n_{H+1}
 * (what Node::getWeight holds after ForwardPass, network.cpp:517). */
int gl_get_activations(gl_net* net, int64_t row, float* out);
/* Reference mode: the k-th pending delta of every edge (Edge::prevDelta[k], State/edge.cpp:54-60;
 * 0 where the history is shorter), flat like the weights. */
int gl_get_pending_delta(gl_net* net, int32_t k, float* out);
/* Predictions of the last row the last train / forward call processed, n_out floats: the
 * `predicted` half of NNetwork::getResults() (network.cpp:529-530; during training these are the
 * outputs computed before that row's own update). */
int gl_get_last_outputs(gl_net* net, float* out);
/* Confusion counts of the last epoch / forward call, [expected][predicted], n_out*n_out ints
 * (CMatrix::addResult, GMath/cmatrix.cpp:57-98). */
int gl_get_confusion(gl_net* net, int32_t* out);
/* Epoch counter, NNetwork::getEpochs. */
int gl_get_epochs(const gl_net* net);

/* Waits for the handle's queued device work (gl_train_window with out == NULL returns before the
 * device has finished) and reports a tensor-core kernel whose bounded wait ran out. */
int gl_sync(gl_net* net);
/* Self-test of the failure path of the bounded device waits: queues the gradient exchange's wait
 * kernel on a flag that nothing raises, limited to max_cycles SM cycles (<= 4e9).  The wait gives
 * up, returns and leaves code 99 in the handle's status word: the next gl_sync reports
 * GL_ERR_TIMEOUT, later waits of the handle return at once, gl_set_weights clears the condition.
 * The context stays usable throughout.  waited_ms (may be NULL): device time of the wait.
 * No counterpart in the reference. */
int gl_selftest_bounded_wait(gl_net* net, int64_t max_cycles, double* waited_ms);
/* Diagnostics: kernels launched by this handle so far, and how many of them were tensor-core
 * (tcgen05) products.  No counterpart in the reference. */
int64_t gl_kernel_launches(const gl_net* net);
int64_t gl_tensor_core_launches(const gl_net* net);
/* Diagnostics: CTAs of the whole-window kernel's thread-block-cluster variant on this handle: > 0 once a window has
 * run on it, 0 where the variant is not in use (it is opt-in: GLADES_GF_CLUSTER=1; network shape; device), -1 before
 * the first whole-window launch decided.  No counterpart in the reference. */
int32_t gl_window_cluster_ctas(const gl_net* net);
/* Diagnostics: tensor-core product launches of this process per tile variant -- out5[0] 128-wide
 * tiles, [1] 256-wide tiles, [2] launches whose persistent CTAs walked more than one tile each,
 * [3] launches of the data-parallel variant whose epilogue stores into the owning rank's memory,
 * [4] launches that split their last, partial wave of tiles along k over all CTAs.
 * Lets a test assert which instantiation a shape ran on.  No counterpart in the reference. */
void gl_tc_variant_counts(int64_t* out5);
/* Diagnostic matrix product on device buffers, C[m][n] = sum_k A(m,k)*B(n,k) with
 * A(m,k) = d_a[m*a_sm + k*a_sk] and B(n,k) = d_b[n*b_sn + k*b_sk]; engine GL_GEMM_FFMA or
 * GL_GEMM_TCGEN05 (M % 128 == 0, N % 128 == 0, K % 16 == 0, each operand contiguous in k or in
 * m/n).  It exposes the layer-product kernels of the path for numerical tests; the reference has
 * no matrix product (it walks edges, network.cpp:461-508). */
int gl_matmul(const float* d_a, int64_t a_sm, int64_t a_sk, const float* d_b, int64_t b_sn, int64_t b_sk, float* d_c,
              int64_t ldc, int32_t m, int32_t n, int32_t k, int32_t engine, int32_t device);

/* The same tensor-core product for callers that cannot allocate device memory: hosts that gave the
 * whole GPU to their own arena, or loops that must not hit cudaMalloc/cudaFree's device-wide
 * synchronisation.  It has no counterpart in the reference.  Its scratch (the operands' low TF32
 * parts and a status word) is a fixed 16 MiB + 256 B array inside the library image, held by every
 * GPU that loads the library; the call allocates nothing.  Limits: tensor-core engine only (shape
 * rules of gl_matmul), each operand at most 2 Mi floats as addressed by its strides (else
 * GL_ERR_TOO_LARGE).  All calls share the array: do not let two calls overlap on the GPU.  The first
 * call on a device looks the array's address up and creates the private non-blocking stream that all
 * of this entry point's GPU work runs on; make that first call outside any stream capture.  Because
 * the stream is private and non-blocking, a call neither waits for nor stalls the caller's other
 * streams -- so the operands must be complete (their producers synchronised) before the call.  The
 * call returns after the product has finished and leaves the caller's current device unchanged.
 * gl_matmul_static_error() gives the text of this entry point's last failure on the calling thread. */
int gl_matmul_static(const float* d_a, int64_t a_sm, int64_t a_sk, const float* d_b, int64_t b_sn, int64_t b_sk,
                     float* d_c, int64_t ldc, int32_t m, int32_t n, int32_t k, int32_t device);
const char* gl_matmul_static_error(void);

/* Asynchronous snapshot for live views: replaces what the reference's GUI callbacks read after an
 * epoch (Networks/network.cpp:258-357) -- every weight (LayerBuilder::getWeights,
 * State/LayerBuilder.cpp:390-410) and the pre-activations of the epoch's last row (network.cpp:510-514;
 * reference mode records them during the pass, batched mode evaluates them for the last resident row
 * under the current weights).  submit queues, behind the work already queued on the handle, a
 * device-to-device copy on a side stream (training waits only for that copy) followed by the copy into
 * pinned host memory; it returns at once.  collect hands the snapshot out: w flat weights, bias H floats,
 * preact the pre-activations of layers 1..H+1 concatenated (each may be NULL); with wait == 0 it
 * returns 1 instead of blocking while the copy is still under way.  One snapshot may be in flight. */
int gl_snapshot_submit(gl_net* net);
int gl_snapshot_collect(gl_net* net, float* w, float* bias, float* preact, int32_t wait);

/* Replaces NNetwork::stop (network.cpp:99-102): async-signal-safe; the flag is looked at between
 * epochs of gl_train_epochs. */
void gl_stop(gl_net* net);

/* ---- data parallelism (batched mode) --------------------------------------------------- */
/* Contiguous shard of `rows` for `rank` of `world` (remainder rows go to the lowest ranks). */
void gl_shard_range(int64_t rows, int32_t rank, int32_t world, int64_t* first, int64_t* count);
/* Fills 128 bytes with an NCCL unique id (rank 0 calls it and hands the bytes to the others). */
int gl_dp_unique_id(void* id128);
/* Joins this handle to a data-parallel group (collective: every rank calls it); gradients, bias
 * sums and metric sums of every gl_train_window call are then summed over the group before the
 * update.  With up to 8 ranks on GPUs that can map each other's memory the exchange runs over peer
 * memory: the weight-gradient products store their row bands into the owning rank, which sums the
 * sources in rank order, updates its band and writes the new weights into every replica.  Else
 * (or with GLADES_DP_PUSH=0) it is one NCCL all-reduce per layer.  gl_destroy of such a handle is
 * collective too.  The reference has no counterpart: its training loop is single-process
 * (network.cpp:258-378). */
int gl_dp_init(gl_net* net, int32_t rank, int32_t world, const void* id128);
/* 0: not data parallel, 1: NCCL all-reduce per layer, 2: exchange over peer memory. */
int gl_dp_mode(const gl_net* net);
/* Position of this rank's shard inside the global window (used for the momentum weights) and
 * the global window length. */
int gl_dp_set_window(gl_net* net, int32_t global_rows, int32_t first_global_pos);

/* ---- synthetic inputs (counter-based, identical on CPU and GPU) ------------------------- */
/* Philox4x32-10 stream: element i of stream `stream` under `seed`.  dist 0: U[0,1) with 24 bits;
 * dist 1: N(0,1) by Box-Muller on elements (2i, 2i+1); out = offset + scale*value.
 * d_out is a device pointer. */
int gl_synth_fill(float* d_out, int64_t n, uint64_t seed, uint32_t stream, int32_t dist, float scale, float offset,
                  int32_t device);

/* The same stream from element `first_index` on: d_out[j] = element first_index + j.  Ranks that fill
 * their own row ranges of one global table use it so that the table does not depend on how many
 * ranks there are.  first_index must be even for dist 1 (two elements share one Box-Muller draw). */
int gl_synth_fill_at(float* d_out, int64_t n, int64_t first_index, uint64_t seed, uint32_t stream, int32_t dist,
                     float scale, float offset, int32_t device);

/* Expected rows from class labels, on the device: d_y[r][c] = (c == labels[r]) ? on : off
 * (the reference's one-hot encoder writes 0.99 / 0.01, GMath/OHE.cpp:159-198).  labels is a host
 * array. */
int gl_onehot_fill(float* d_y, const int32_t* labels, int64_t rows, int32_t n, float on, float off, int32_t device);

/* ---- input standardisation -------------------------------------------------------------- */
/* Replaces the arithmetic of NumberInput::standardizeInputTable (DataObjects/NumberInput.cpp:43-285)
 * and the one-hot vectors of OHE::operator[] (GMath/OHE.cpp:159-198) for a raw table that lies in
 * device memory as a row-major [rows][cols] fp32 matrix.  Column c is numeric (kind[c] = 0) or
 * categorical (kind[c] = 1: each cell holds its category's index in order of first appearance, the
 * order OHE::addString builds; classes[c] categories, expanded to that many 0.99 / 0.01 columns);
 * to_output[c] = 1 sends it to the expected-rows matrix d_y, else to the input matrix d_x; columns
 * keep their raw order inside each matrix.  flag: 0 min-max, 1 z-score (GMath/gmath.h:53-54).
 * Kept from the reference: the running minimum / maximum start from 0.0 for every raw column but the
 * first (NumberInput.cpp:105-109); numeric columns scale to [0.01, 0.99] when the table has any
 * categorical column, else to [0, 1] (:196-214); a min-max column with range 0 is copied unscaled into
 * the INPUT matrix whatever its output mark (:166-171); mean and deviation are sequential fp32 sums.
 * Because of the range-0 rule the widths depend on the data: call once with d_x = d_y = NULL to get
 * *nx and *ny, allocate [rows][*nx] and [rows][*ny], and call again with those widths.
 * stats_out (host, may be NULL): [cols][4] = minimum, maximum, mean, deviation (the last two in z-score
 * mode only).  Results are bit-identical to the reference's. */
int gl_standardize_table(const float* d_raw, int64_t rows, int32_t cols, const int32_t* kind, const int32_t* classes,
                         const int32_t* to_output, int32_t flag, float* d_x, int32_t* nx, float* d_y, int32_t* ny,
                         float* stats_out, int32_t device);

/* ---- measurement helpers (no counterpart in the reference) ------------------------------ */
/* CUDA events on the handle's own stream around whatever is queued between the two calls. */
int gl_timer_start(gl_net* net);
int gl_timer_stop(gl_net* net, double* ms);
/* Per-launch event timing of the layer products.  gl_profile_read fills out6 with
 * {launches, total ms, total flop (2*M*N*K each)} for the tensor-core kernel, then for the FFMA
 * kernel, since gl_profile_enable(net, 1). */
int gl_profile_enable(gl_net* net, int32_t on);
int gl_profile_read(gl_net* net, double* out6);

/* ---- raw device helpers for callers that keep data resident ---------------------------- */
int gl_device_alloc(void** d_ptr, int64_t bytes, int32_t device);
int gl_device_free(void* d_ptr, int32_t device);
/* Free and total device memory in bytes (cudaMemGetInfo). */
int gl_device_mem_info(int32_t device, int64_t* free_bytes, int64_t* total_bytes);
int gl_memcpy_h2d(void* d_dst, const void* h_src, int64_t bytes, int32_t device);
int gl_memcpy_d2h(void* h_dst, const void* d_src, int64_t bytes, int32_t device);
int gl_host_alloc_pinned(void** h_ptr, int64_t bytes);
int gl_host_free_pinned(void* h_ptr);

#ifdef __cplusplus
}
#endif
#endif /* GLADES_B200_H */
