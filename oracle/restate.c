/*
 * TEST INFRASTRUCTURE ONLY -- the checker, never the thing shipped or measured as the product.
 * Only tests/, the smoke check and the CPU-baseline leg of bench.py may load this library.
 *
 * CPU restatement, on dense row-major matrices, of the reference's deep feed-forward path:
 *   NNetwork::run / SGDHelper / ForwardPass / BackPropagation   Networks/network.cpp:114-668
 *   Node::getActivation / getDelta / applyDeltas                State/node.cpp:82-93,278-307
 *   Edge history                                                State/edge.cpp:54-60,87-107
 *   GMath::squash / activationErrDer / costs / naiveVectorDecomp GMath/gmath.cpp:22-101,182-353,435-455
 *   CMatrix::addResult / updateResultParams / getters           GMath/cmatrix.cpp:57-266
 *
 * Reference mode (rs_epoch, rs_train_row, rs_forward_row) keeps the reference's operation order
 * in fp32 -- product rounded, then sum rounded, i ascending; glibc expf/tanhf/logf -- and is
 * checked bit-for-bit against the compiled reference (oracle/_ref) by tests/test_oracle_pin.py.
 * Batched mode (rs_window_*) is the same arithmetic with the documented switches flipped
 * (aligned windows, frozen weights, plain error sum, summed bias delta, optional softmax head);
 * its sums are accumulated in double so that a comparison against it measures only the rounding
 * of the kernel under test.
 *
 * Build: gcc -std=c11 -O2 -ffp-contract=off -fopenmp (see Makefile); no FMA contraction.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "glades_b200.h"

#define OUTLIER 0.046f /* GMath/gmath.h:35 */

typedef struct rs_net {
	gl_net_desc d;
	int H;             /* hidden layers */
	int64_t rows;
	const float* x;    /* borrowed */
	const float* y;
	float* w[GL_MAX_WEIGHT_LAYERS];     /* W_l [n_{l+1}][n_l] */
	float bias[GL_MAX_WEIGHT_LAYERS];   /* bias[l], l = 1..H (index 0 unused) */
	float* hist[GL_MAX_WEIGHT_LAYERS];  /* pending deltas [mb][n_{l+1}*n_l] */
	int hist_len;
	float* act[GL_MAX_WEIGHT_LAYERS + 1]; /* a_l, l = 0..H+1 (one row) */
	float* err[GL_MAX_WEIGHT_LAYERS + 1]; /* E_l accumulators */
	int32_t* cm;       /* confusion [n_out][n_out] */
	float tot_err, tot_acc;
	int epochs;
	int math_mode;     /* 0 glibc single precision (reference); 1 double then round (kernel) */
	/* dropout (reference mode, any p_dropout != 0): the current row's flags per non-output node layer,
	 * and per-edge histories of their own length (a dropped pair pushes nothing) */
	int dropout_on;
	unsigned char* drop[GL_MAX_WEIGHT_LAYERS + 1]; /* drop[l][i] = 1: node i of layer l is dropped, l = 0..H */
	int32_t* hlen[GL_MAX_WEIGHT_LAYERS];           /* entries pushed on edge e since its last clear */
	float* hlast[GL_MAX_WEIGHT_LAYERS];            /* the last pushed entry (the momentum term reads it) */
} rs_net;

/* accessors for fastport.c (the timed CPU baseline), which works on the same network object */
const gl_net_desc* rs_desc(const rs_net* n) { return &n->d; }
float* rs_weights(rs_net* n, int l) { return n->w[l]; }
float* rs_biases(rs_net* n) { return n->bias; }
const float* rs_x(const rs_net* n) { return n->x; }
const float* rs_y(const rs_net* n) { return n->y; }

static int g_math_mode = 0;
void rs_set_math_mode(int m) { g_math_mode = m; }

/* Threads of the OpenMP loops below.  A launcher may export OMP_NUM_THREADS=1 for its children (torchrun
 * does); a caller that wants all cores says so here.  rs_get_threads reports what the loops will use. */
#ifdef _OPENMP
#include <omp.h>
void rs_set_threads(int t) { if (t >= 1) omp_set_num_threads(t); }
int rs_get_threads(void) { return omp_get_max_threads(); }
#else
void rs_set_threads(int t) { (void)t; }
int rs_get_threads(void) { return 1; }
#endif

static float f_exp(float v) { return g_math_mode ? (float)exp((double)v) : expf(v); }
static float f_tanh(float v) { return g_math_mode ? (float)tanh((double)v) : tanhf(v); }
static float f_log(float v) { return g_math_mode ? (float)log((double)v) : logf(v); }

/* GMath::squash, gmath.cpp:22-101 */
float rs_squash(float z, int act, float p)
{
	switch (act)
	{
	case GL_ACT_TANH: return f_tanh(z);
	case GL_ACT_TANHP:
		if (z > 1.0f - p) return 1.0f;
		if (z < p - 1.0f) return -1.0f;
		return f_tanh(z);
	case GL_ACT_SIGMOID: return 1.0f / (1.0f + f_exp(-z));
	case GL_ACT_SIGMOIDP:
		if (z < p) return 0.01f;
		if (z > 1.0f - p) return 0.99f;
		return 1.0f / (1.0f + f_exp(-z));
	case GL_ACT_RELU: return z < OUTLIER ? 0.0f : z;
	case GL_ACT_LEAKY: return z < OUTLIER ? p * z : z;
	case GL_ACT_LINEAR: return p * z;
	case GL_ACT_STEP: return z < p ? 0.0f : 1.0f;
	}
	return 0.0f;
}

/* GMath::activationErrDer, gmath.cpp:182-245 (argument is the node's OUTPUT value) */
float rs_act_der(float a, int act, float p)
{
	switch (act)
	{
	case GL_ACT_TANH:
	case GL_ACT_TANHP: return 1.0f - (a * a);
	case GL_ACT_SIGMOID:
	case GL_ACT_SIGMOIDP: return a * (1.0f - a);
	case GL_ACT_RELU: return a > 0.0f ? 1.0f : 0.0f;
	case GL_ACT_LEAKY: return a > 0.0f ? 1.0f : (p < 0 ? p : -p);
	case GL_ACT_LINEAR: return p;
	case GL_ACT_STEP: return 0.0f;
	}
	return 1.0f;
}

/* GMath::outputNodeCost, gmath.cpp:288-321 */
float rs_cost(float e, float p, float n, int fx)
{
	float c = 0.0f;
	switch (fx)
	{
	case GL_OUT_REGRESSION: { float t = e - p; c = t * t; c /= n; break; }
	case GL_OUT_CLASSIFICATION: c = -((e * f_log(p)) + ((1.0f - e) * f_log(1.0f - p))); c /= n; break;
	case GL_OUT_KL: c = f_log(e / p); c /= n; break;
	}
	return c;
}

/* GMath::costErrDer, gmath.cpp:323-353 */
float rs_cost_der(float e, float p, int fx)
{
	switch (fx)
	{
	case GL_OUT_REGRESSION: return 2.0f * (p - e);
	case GL_OUT_CLASSIFICATION: return (p - e) / ((1.0f - p) * p);
	case GL_OUT_KL: return -(e / p);
	}
	return 1.0f;
}

/* GMath::naiveVectorDecomp, gmath.cpp:435-455: strict > starting from 0, first maximum wins,
 * -1 when nothing exceeds 0. */
static int rs_argmax(const float* v, int n, int stride)
{
	float mx = 0.0f;
	int idx = -1;
	for (int i = 0; i < n; ++i)
		if (v[(size_t)i * stride] > mx)
		{
			mx = v[(size_t)i * stride];
			idx = i;
		}
	return idx;
}

static size_t wcount(const rs_net* n, int l) { return (size_t)n->d.sizes[l + 1] * n->d.sizes[l]; }

rs_net* rs_create(const gl_net_desc* d, const float* x, const float* y, int64_t rows)
{
	rs_net* n = (rs_net*)calloc(1, sizeof *n);
	n->d = *d;
	n->H = d->n_layers - 2;
	n->rows = rows;
	n->x = x;
	n->y = y;
	int mb = d->batch_size > 0 ? d->batch_size : 1;
	for (int l = 0; l <= n->H; ++l)
	{
		n->w[l] = (float*)calloc(wcount(n, l), sizeof(float));
		if (d->mode == GL_MODE_REFERENCE)
			n->hist[l] = (float*)calloc(wcount(n, l) * mb, sizeof(float));
	}
	for (int l = 0; l <= n->H + 1; ++l)
	{
		n->act[l] = (float*)calloc(d->sizes[l], sizeof(float));
		n->err[l] = (float*)calloc(d->sizes[l], sizeof(float));
	}
	int no = d->sizes[n->H + 1];
	n->cm = (int32_t*)calloc((size_t)no * no, sizeof(int32_t));
	for (int l = 0; l <= n->H; ++l)
		if (d->p_dropout[l] != 0.0f) n->dropout_on = 1;
	if (n->dropout_on && d->mode == GL_MODE_REFERENCE)
		for (int l = 0; l <= n->H; ++l)
		{
			n->drop[l] = (unsigned char*)calloc(d->sizes[l], 1);
			n->hlen[l] = (int32_t*)calloc(wcount(n, l), sizeof(int32_t));
			n->hlast[l] = (float*)calloc(wcount(n, l), sizeof(float));
		}
	return n;
}

void rs_destroy(rs_net* n)
{
	if (!n) return;
	for (int l = 0; l <= n->H; ++l) { free(n->w[l]); free(n->hist[l]); free(n->drop[l]); free(n->hlen[l]); free(n->hlast[l]); }
	for (int l = 0; l <= n->H + 1; ++l) { free(n->act[l]); free(n->err[l]); }
	free(n->cm);
	free(n);
}

void rs_set_data(rs_net* n, const float* x, const float* y, int64_t rows) { n->x = x; n->y = y; n->rows = rows; }

void rs_set_weights(rs_net* n, const float* w, const float* bias)
{
	size_t k = 0;
	for (int l = 0; l <= n->H; ++l)
	{
		memcpy(n->w[l], w + k, wcount(n, l) * sizeof(float));
		k += wcount(n, l);
		if (l >= 1) n->bias[l] = bias ? bias[l - 1] : 0.0f;
	}
	n->hist_len = 0;
	for (int l = 0; l <= n->H + 1; ++l) memset(n->err[l], 0, n->d.sizes[l] * sizeof(float));
	for (int l = 0; l <= n->H; ++l)
		if (n->hlen[l])
		{
			memset(n->hlen[l], 0, wcount(n, l) * sizeof(int32_t));
			memset(n->hlast[l], 0, wcount(n, l) * sizeof(float));
		}
}

void rs_get_weights(const rs_net* n, float* w, float* bias)
{
	size_t k = 0;
	for (int l = 0; l <= n->H; ++l)
	{
		memcpy(w + k, n->w[l], wcount(n, l) * sizeof(float));
		k += wcount(n, l);
		if (l >= 1 && bias) bias[l - 1] = n->bias[l];
	}
}

void rs_get_pending_delta(const rs_net* n, int k, float* out)
{
	size_t j = 0;
	for (int l = 0; l <= n->H; ++l)
	{
		size_t c = wcount(n, l);
		for (size_t e = 0; e < c; ++e)
		{
			const int len = n->hlen[l] ? n->hlen[l][e] : n->hist_len;
			out[j++] = (k < len && k < n->d.batch_size) ? n->hist[l][(size_t)k * c + e] : 0.0f;
		}
	}
}

/* ForwardPass for one row, network.cpp:457-575 (metrics excluded). */
static void forward_row(rs_net* n, int64_t r)
{
	const gl_net_desc* d = &n->d;
	memcpy(n->act[0], n->x + (size_t)r * d->sizes[0], d->sizes[0] * sizeof(float));
	for (int l = 0; l <= n->H; ++l)
	{
		const int ni = d->sizes[l], no = d->sizes[l + 1];
		const float* W = n->w[l];
		const float* a = n->act[l];
		for (int o = 0; o < no; ++o)
		{
			float z = 0.0f;
			for (int i = 0; i < ni; ++i)
			{
				float prod = W[(size_t)o * ni + i] * a[i]; /* Edge::activation, a float member */
				z = z + prod;                               /* Node::getActivation, node.cpp:82-93 */
			}
			if (l >= 1) z = z + n->bias[l];               /* network.cpp:501-502 */
			n->act[l + 1][o] = rs_squash(z, d->activation[l], d->act_param[l]);
		}
	}
}

/* Output-layer metrics of one row, network.cpp:519-547, and CMatrix::addResult. */
static void metrics_row(rs_net* n, int64_t r)
{
	const gl_net_desc* d = &n->d;
	const int no = d->sizes[n->H + 1];
	const float* p = n->act[n->H + 1];
	const float* e = n->y + (size_t)r * no;
	const float dataSize = (float)(n->rows * no);
	for (int o = 0; o < no; ++o)
	{
		float cost = rs_cost(e[o], p[o], dataSize, d->output_type);
		n->tot_err += cost;
		float pe = p[o] - e[o];
		if (pe < 0.0f) pe = -pe;
		if (pe > 1.0f) pe = 1.0f;
		float acc = (1.0f - pe) * 100.0f;
		if (acc < 0.0f) acc = 0.0f;
		n->tot_acc += acc;
	}
	if (d->output_type != GL_OUT_REGRESSION)
	{
		int ie = rs_argmax(e, no, 1), ip = rs_argmax(p, no, 1);
		if (ie >= 0 && ip >= 0) n->cm[ie * no + ip] += 1;
	}
}

/* BackPropagation for one row, network.cpp:577-668: layer from the top, input node OUTER,
 * output node INNER. */
static void backward_row(rs_net* n, int64_t r)
{
	const gl_net_desc* d = &n->d;
	const int mb = d->batch_size;
	const int apply = (r % mb) == 0;                     /* network.cpp:647 */
	const float* e = n->y + (size_t)r * d->sizes[n->H + 1];
	const int k = n->hist_len;                           /* slot this row's deltas go to */
	for (int L = n->H + 1; L >= 1; --L)
	{
		const int l = L - 1;
		const int ni = d->sizes[l], no = d->sizes[L];
		float* W = n->w[l];
		float* hist = n->hist[l];
		const size_t cnt = (size_t)ni * no;
		const float lr = d->lr[l], m = d->momentum[l], wd1 = d->wd1[l], wd2 = d->wd2[l];
		float* EL = n->err[L];
		float* El = n->err[l];
		for (int i = 0; i < ni; ++i)
		{
			const float ai = n->act[l][i];
			for (int o = 0; o < no; ++o)
			{
				float der = 1.0f;
				if (L == n->H + 1)
				{
					/* clearErrDer + adjustErrDer: 0 + cost' */
					EL[o] = 0.0f + rs_cost_der(e[o], n->act[L][o], d->output_type);
				}
				else
					der = rs_act_der(n->act[L][o], d->activation[l], 0.01f); /* network.cpp:618 */
				float dd = EL[o] * der;
				if (i == ni - 1) EL[o] = 0.0f;
				float base = lr * dd;
				/* Node::getDelta, node.cpp:278-292 */
				size_t eidx = (size_t)o * ni + i;
				float last = (k > 0) ? hist[(size_t)(k - 1) * cnt + eidx] : 0.0f;
				float absa = ai < 0.0f ? -ai : ai;
				float delta = (((base * ai) + (m * last)) + (wd1 * lr * absa)) + (wd2 * lr * ai);
				hist[(size_t)k * cnt + eidx] = delta;
				if (apply)
				{
					/* Node::applyDeltas, node.cpp:294-307 */
					float s = 0.0f;
					for (int t = 0; t < mb; ++t)
						s += (t <= k) ? hist[(size_t)t * cnt + eidx] : 0.0f;
					s /= (float)mb;
					W[eidx] = W[eidx] - s;
				}
				if (l >= 1) n->bias[l] = n->bias[l] - base;      /* network.cpp:654-656 */
				if (l >= 1)
				{
					float t = El[i] + (dd * W[eidx]);              /* network.cpp:660-661 */
					El[i] += t;                                    /* Node::adjustErrDer */
				}
			}
		}
	}
	n->hist_len = apply ? 0 : k + 1;
}


/* ------------------------------------------------------------------------------------------
 * Dropout (reference mode).  LayerBuilder::scrambleDropout (State/LayerBuilder.cpp:497-523) runs
 * before EVERY row, in training and in testing (network.cpp:408-411): Layer::generateDropout
 * (State/layer.cpp:102-134) for the row's input layer with NNInfo::getPInput(), then for hidden
 * layer i with NNInfo::getPDropout(i) -- whose index 0 is the INPUT layer's value (nninfo.cpp:321-333),
 * so the first hidden layer drops with the input layer's probability and the last hidden layer's own
 * value is never read.  The descriptor carries the resolved values: p_dropout[j] is what the loop uses
 * for node layer j (0 = input, 1..H hidden).
 * The rate is an integer percentage, int(p * 100.0f); a rate < 0 or >= 100 draws nothing and leaves the
 * flags alone (all clear); otherwise one rand() per node, dart = rand() % 100 + 1, dropped when
 * dart <= rate, the whole layer redrawn while every node dropped.
 * ------------------------------------------------------------------------------------------ */
static void draw_layer_dropout(unsigned char* flag, int size, float p)
{
	int rate = (int)(p * 100.0f);
	if (rate < 0 || rate >= 100) return;
	int all;
	do
	{
		all = 1;
		for (int i = 0; i < size; ++i)
		{
			int dart = (rand() % 100) + 1;
			if (dart <= rate) flag[i] = 1;
			else { flag[i] = 0; all = 0; }
		}
	} while (all);
}

static void draw_row_dropout(rs_net* n)
{
	for (int j = 0; j <= n->H; ++j) draw_layer_dropout(n->drop[j], n->d.sizes[j], n->d.p_dropout[j]);
}

/* ForwardPass with dropped nodes (network.cpp:476-508): an edge is activated only when both of its
 * nodes are kept; the node's sum runs over its activated edges in i order (node.cpp:82-93); a dropped
 * node therefore gets squash(0 + bias). */
static void forward_row_dropout(rs_net* n, int64_t r)
{
	const gl_net_desc* d = &n->d;
	memcpy(n->act[0], n->x + (size_t)r * d->sizes[0], d->sizes[0] * sizeof(float));
	for (int l = 0; l <= n->H; ++l)
	{
		const int ni = d->sizes[l], no = d->sizes[l + 1];
		const float* W = n->w[l];
		const float* a = n->act[l];
		const unsigned char* din = n->drop[l];
		const unsigned char* dout = (l + 1 <= n->H) ? n->drop[l + 1] : NULL;
		for (int o = 0; o < no; ++o)
		{
			float z = 0.0f;
			if (!(dout && dout[o]))
				for (int i = 0; i < ni; ++i)
				{
					if (din[i]) continue;
					float prod = W[(size_t)o * ni + i] * a[i];
					z = z + prod;
				}
			if (l >= 1) z = z + n->bias[l];
			n->act[l + 1][o] = rs_squash(z, d->activation[l], d->act_param[l]);
		}
	}
}

/* BackPropagation with dropped nodes (network.cpp:577-668).  For a dropped pair the node delta is the
 * raw accumulator (no derivative factor), nothing is pushed, applied or subtracted from the bias, and
 * the accumulator is not cleared -- but the pair still feeds the input node's accumulator
 * (network.cpp:659-662).  The clear happens on the pair with i == n_in - 1 only when that pair is kept
 * (network.cpp:630-632), so accumulators of hidden nodes can survive into the next row.  Each edge's
 * history has its own length (Edge::prevDelta): Node::applyDeltas sums its first mb entries
 * (node.cpp:299-301) and the clear empties it, whatever its length. */
static void backward_row_dropout(rs_net* n, int64_t r)
{
	const gl_net_desc* d = &n->d;
	const int mb = d->batch_size;
	const int apply = (r % mb) == 0;
	const float* e = n->y + (size_t)r * d->sizes[n->H + 1];
	for (int L = n->H + 1; L >= 1; --L)
	{
		const int l = L - 1;
		const int ni = d->sizes[l], no = d->sizes[L];
		float* W = n->w[l];
		float* hist = n->hist[l];
		int32_t* hlen = n->hlen[l];
		float* hlast = n->hlast[l];
		const size_t cnt = (size_t)ni * no;
		const float lr = d->lr[l], m = d->momentum[l], wd1 = d->wd1[l], wd2 = d->wd2[l];
		float* EL = n->err[L];
		float* El = n->err[l];
		const unsigned char* din = n->drop[l];
		const unsigned char* dout = (L <= n->H) ? n->drop[L] : NULL;
		for (int i = 0; i < ni; ++i)
		{
			const float ai = n->act[l][i];
			for (int o = 0; o < no; ++o)
			{
				float der = 1.0f;
				if (L == n->H + 1)
					EL[o] = 0.0f + rs_cost_der(e[o], n->act[L][o], d->output_type);
				else
					der = rs_act_der(n->act[L][o], d->activation[l], 0.01f);
				const int dropped = din[i] || (dout && dout[o]);
				float dd = EL[o];
				size_t eidx = (size_t)o * ni + i;
				if (!dropped)
				{
					dd = dd * der;
					if (i == ni - 1) EL[o] = 0.0f;
					float base = lr * dd;
					float last = (hlen[eidx] > 0) ? hlast[eidx] : 0.0f;
					float absa = ai < 0.0f ? -ai : ai;
					float delta = (((base * ai) + (m * last)) + (wd1 * lr * absa)) + (wd2 * lr * ai);
					if (hlen[eidx] < mb) hist[(size_t)hlen[eidx] * cnt + eidx] = delta;
					hlast[eidx] = delta;
					hlen[eidx] += 1;
					if (apply)
					{
						float s = 0.0f;
						for (int t = 0; t < mb; ++t)
							s += (t < hlen[eidx]) ? hist[(size_t)t * cnt + eidx] : 0.0f;
						s /= (float)mb;
						W[eidx] = W[eidx] - s;
						hlen[eidx] = 0;
					}
					if (l >= 1) n->bias[l] = n->bias[l] - base;
				}
				if (l >= 1)
				{
					float t = El[i] + (dd * W[eidx]);
					El[i] += t;
				}
			}
		}
	}
}

static void finish_class_metrics(const rs_net* n, gl_metrics* m)
{
	/* CMatrix::updateResultParams + getters, cmatrix.cpp:100-266 */
	const int c = n->d.sizes[n->H + 1];
	float acc = 0, prec = 0, rec = 0, spec = 0, f1 = 0;
	for (int k = 0; k < c; ++k)
	{
		int tp = n->cm[k * c + k], tn = 0, fp = 0, fn = 0;
		for (int j = 0; j < c; ++j)
		{
			if (j != k) { tn += n->cm[j * c + j]; fp += n->cm[j * c + k]; fn += n->cm[k * c + j]; }
		}
		float truth = (float)(tp + tn), untruth = (float)(fp + fn);
		acc += truth / (truth + untruth);
		float p = ((float)tp) / ((float)(tp + fp));
		float r = ((float)tp) / ((float)(tp + fn));
		prec += p;
		rec += r;
		spec += ((float)tn) / ((float)(tn + fp));
		f1 += (2.0f * r * p) / (r + p);
	}
	m->class_accuracy = (acc / (float)c) * 100.0f;
	m->class_precision = (prec / (float)c) * 100.0f;
	m->class_recall = (rec / (float)c) * 100.0f;
	m->class_specificity = (spec / (float)c) * 100.0f;
	m->class_f1 = (f1 / (float)c) * 100.0f;
}

static void fill_metrics(const rs_net* n, gl_metrics* m)
{
	if (!m) return;
	memset(m, 0, sizeof *m);
	const int no = n->d.sizes[n->H + 1];
	m->total_error = n->tot_err;
	m->total_accuracy = n->tot_acc / (((float)n->rows) * ((float)no));  /* network.cpp:194-195 */
	m->epochs = n->epochs;
	m->rows = n->rows;
	if (n->d.output_type != GL_OUT_REGRESSION) finish_class_metrics(n, m);
	size_t k = 0;
	for (int l = 0; l <= n->H; ++l)
		for (size_t e = 0; e < wcount(n, l); ++e, ++k)
			if (!isfinite(n->w[l][e])) m->nonfinite = 1;
}

/* One epoch of NNetwork::run (network.cpp:179-195), reference mode.  run_type 0 train, 1 test. */
int rs_epoch(rs_net* n, int run_type, gl_metrics* m, int32_t* confusion, float* outputs)
{
	const int no = n->d.sizes[n->H + 1];
	n->tot_err = 0.0f;
	n->tot_acc = 0.0f;
	memset(n->cm, 0, (size_t)no * no * sizeof(int32_t));
	for (int64_t r = 0; r < n->rows; ++r)
	{
		if (n->dropout_on)
		{
			draw_row_dropout(n);
			forward_row_dropout(n, r);
		}
		else
			forward_row(n, r);
		metrics_row(n, r);
		if (outputs) memcpy(outputs + (size_t)r * no, n->act[n->H + 1], no * sizeof(float));
		if (run_type == 0)
		{
			if (n->dropout_on) backward_row_dropout(n, r);
			else backward_row(n, r);
		}
	}
	if (run_type == 0) n->epochs += 1;
	fill_metrics(n, m);
	if (confusion) memcpy(confusion, n->cm, (size_t)no * no * sizeof(int32_t));
	return 0;
}

int rs_forward_row(rs_net* n, int64_t row, float* acts)
{
	if (n->dropout_on)
	{
		draw_row_dropout(n);
		forward_row_dropout(n, row);
	}
	else
		forward_row(n, row);
	size_t k = 0;
	for (int l = 1; l <= n->H + 1; ++l)
	{
		memcpy(acts + k, n->act[l], n->d.sizes[l] * sizeof(float));
		k += n->d.sizes[l];
	}
	return 0;
}

int rs_train_row(rs_net* n, int64_t row)
{
	if (n->dropout_on)
	{
		draw_row_dropout(n);
		forward_row_dropout(n, row);
		backward_row_dropout(n, row);
		return 0;
	}
	forward_row(n, row);
	backward_row(n, row);
	return 0;
}

/* ------------------------------------------------------------------------------------------
 * Batched mode.  One window = rows [first, first+cnt) which sit at positions
 * [first_pos, first_pos+cnt) of a global window of global_rows rows.  rs_window_grad computes this
 * shard's contribution
 *     grad = [ G_0 | ... | G_H | bias sums (H) | cost sum | accuracy sum ]   (doubles)
 * and rs_window_apply applies a (summed) contribution.  With one shard, grad then apply is the
 * whole step.  Softmax head: activation GL_ACT_SOFTMAX on the last weight layer.
 * ------------------------------------------------------------------------------------------ */
int64_t rs_grad_len(const rs_net* n)
{
	int64_t k = 0;
	for (int l = 0; l <= n->H; ++l) k += (int64_t)wcount(n, l);
	return k + n->H + 2;
}

/* Forward of a block of rows in batched arithmetic (double accumulation, fp32 storage).
 * acts[l] : [cnt][n_l] for l = 0..H+1 (caller-allocated). */
static void forward_block(const rs_net* n, int64_t first, int cnt, float** acts)
{
	const gl_net_desc* d = &n->d;
	memcpy(acts[0], n->x + (size_t)first * d->sizes[0], (size_t)cnt * d->sizes[0] * sizeof(float));
	for (int l = 0; l <= n->H; ++l)
	{
		const int ni = d->sizes[l], no = d->sizes[l + 1];
		const float* W = n->w[l];
#pragma omp parallel for schedule(static)
		for (int j = 0; j < cnt; ++j)
		{
			const float* a = acts[l] + (size_t)j * ni;
			float* out = acts[l + 1] + (size_t)j * no;
			if (d->activation[l] == GL_ACT_SOFTMAX)
			{
				double* z = (double*)malloc(no * sizeof(double));
				double mx = -INFINITY;
				for (int o = 0; o < no; ++o)
				{
					double s = 0.0;
					for (int i = 0; i < ni; ++i) s += (double)W[(size_t)o * ni + i] * (double)a[i];
					if (l >= 1) s += (double)n->bias[l];
					z[o] = (double)(float)s;
					if (z[o] > mx) mx = z[o];
				}
				double den = 0.0;
				for (int o = 0; o < no; ++o) den += exp(z[o] - mx);
				for (int o = 0; o < no; ++o) out[o] = (float)(exp(z[o] - mx) / den);
				free(z);
			}
			else
				for (int o = 0; o < no; ++o)
				{
					double s = 0.0;
					for (int i = 0; i < ni; ++i) s += (double)W[(size_t)o * ni + i] * (double)a[i];
					if (l >= 1) s += (double)n->bias[l];
					out[o] = rs_squash((float)s, d->activation[l], d->act_param[l]);
				}
		}
	}
}

/* Batched forward for inference checks: outputs [cnt][n_out], argmax [cnt] (either may be NULL);
 * also the pre-activation-free per-layer activations of the LAST row into acts_last if given. */
int rs_forward_block(rs_net* n, int64_t first, int cnt, float* outputs, int32_t* argmax)
{
	float* acts[GL_MAX_WEIGHT_LAYERS + 1];
	for (int l = 0; l <= n->H + 1; ++l) acts[l] = (float*)malloc((size_t)cnt * n->d.sizes[l] * sizeof(float));
	forward_block(n, first, cnt, acts);
	const int no = n->d.sizes[n->H + 1];
	if (outputs) memcpy(outputs, acts[n->H + 1], (size_t)cnt * no * sizeof(float));
	if (argmax)
		for (int j = 0; j < cnt; ++j) argmax[j] = rs_argmax(acts[n->H + 1] + (size_t)j * no, no, 1);
	for (int l = 0; l <= n->H + 1; ++l) free(acts[l]);
	return 0;
}

int rs_window_grad(rs_net* n, int64_t first, int cnt, int global_rows, int first_pos, double* grad,
                   int32_t* confusion_add, int64_t metric_rows)
{
	const gl_net_desc* d = &n->d;
	const int H = n->H;
	const int no_out = d->sizes[H + 1];
	float* acts[GL_MAX_WEIGHT_LAYERS + 1];
	float* D[GL_MAX_WEIGHT_LAYERS + 1];
	for (int l = 0; l <= H + 1; ++l)
	{
		acts[l] = (float*)malloc((size_t)cnt * d->sizes[l] * sizeof(float));
		D[l] = (float*)calloc((size_t)cnt * d->sizes[l], sizeof(float));
	}
	forward_block(n, first, cnt, acts);
	memset(grad, 0, rs_grad_len(n) * sizeof(double));
	int64_t off[GL_MAX_WEIGHT_LAYERS + 1];
	off[0] = 0;
	for (int l = 0; l <= H; ++l) off[l + 1] = off[l] + (int64_t)wcount(n, l);
	double* gb = grad + off[H + 1];      /* H bias sums: gb[l-1] for l = 1..H */
	double* gm = gb + H;                  /* cost sum, accuracy sum */
	const int softmax = d->activation[H] == GL_ACT_SOFTMAX;
	const float dataSize = (float)(metric_rows * no_out);

	/* metrics + output delta */
	for (int j = 0; j < cnt; ++j)
	{
		const float* p = acts[H + 1] + (size_t)j * no_out;
		const float* e = n->y + (size_t)(first + j) * no_out;
		for (int o = 0; o < no_out; ++o)
		{
			float cost;
			if (softmax)
				cost = (e[o] != 0.0f) ? (-(e[o] * (float)log((double)p[o]))) / dataSize : 0.0f;
			else
				cost = rs_cost(e[o], p[o], dataSize, d->output_type);
			gm[0] += (double)cost;
			float pe = p[o] - e[o];
			if (pe < 0.0f) pe = -pe;
			if (pe > 1.0f) pe = 1.0f;
			float acc = (1.0f - pe) * 100.0f;
			if (acc < 0.0f) acc = 0.0f;
			gm[1] += (double)acc;
			D[H + 1][(size_t)j * no_out + o] = softmax ? (p[o] - e[o]) : rs_cost_der(e[o], p[o], d->output_type);
		}
		if (confusion_add && d->output_type != GL_OUT_REGRESSION)
		{
			int ie = rs_argmax(e, no_out, 1), ip = rs_argmax(p, no_out, 1);
			if (ie >= 0 && ip >= 0) confusion_add[ie * no_out + ip] += 1;
		}
	}
	/* layers from the top */
	for (int L = H + 1; L >= 1; --L)
	{
		const int l = L - 1;
		const int ni = d->sizes[l], no = d->sizes[L];
		const float lr = d->lr[l], wd1 = d->wd1[l], wd2 = d->wd2[l];
		const double m = (double)d->momentum[l];
		const float* W = n->w[l];
		/* momentum weights c_j = sum_{t=0}^{mb-1-pos} m^t, closed form of the reference's
		 * intra-window history (node.cpp:278-292) */
		double* c = (double*)malloc(cnt * sizeof(double));
		for (int j = 0; j < cnt; ++j)
		{
			int terms = global_rows - (first_pos + j);
			double s = 0.0, pw = 1.0;
			for (int t = 0; t < terms; ++t) { s += pw; pw *= m; }
			c[j] = s;
		}
		/* propagate the error first (plain sum), needed only for l >= 1 */
		if (l >= 1)
		{
#pragma omp parallel for schedule(static)
			for (int j = 0; j < cnt; ++j)
				for (int i = 0; i < ni; ++i)
				{
					double s = 0.0;
					for (int o = 0; o < no; ++o)
						s += (double)D[L][(size_t)j * no + o] * (double)W[(size_t)o * ni + i];
					/* D_l = E_l * act'(A_l), derivative of the activation that produced layer l */
					float der = rs_act_der(acts[l][(size_t)j * ni + i], d->activation[l - 1], 0.01f);
					D[l][(size_t)j * ni + i] = (float)s * der;
				}
		}
		/* weight gradient G_l = lr * D_L^T diag(c) A_l + decay terms */
		double* G = grad + off[l];
#pragma omp parallel for schedule(static)
		for (int o = 0; o < no; ++o)
			for (int i = 0; i < ni; ++i)
			{
				double s = 0.0;
				for (int j = 0; j < cnt; ++j)
				{
					double a = (double)acts[l][(size_t)j * ni + i];
					double g = (double)lr * (double)D[L][(size_t)j * no + o] * a +
					           (double)wd1 * (double)lr * fabs(a) + (double)wd2 * (double)lr * a;
					s += c[j] * g;
				}
				G[(size_t)o * ni + i] = s;
			}
		if (l >= 1)
		{
			double s = 0.0;
			for (int j = 0; j < cnt; ++j)
				for (int o = 0; o < no; ++o) s += (double)lr * (double)D[L][(size_t)j * no + o];
			gb[l - 1] = s;
		}
		free(c);
	}
	for (int l = 0; l <= H + 1; ++l) { free(acts[l]); free(D[l]); }
	return 0;
}

int rs_window_apply(rs_net* n, const double* grad, int global_rows)
{
	const int H = n->H;
	int64_t k = 0;
	for (int l = 0; l <= H; ++l)
	{
		size_t c = wcount(n, l);
		for (size_t e = 0; e < c; ++e, ++k)
			n->w[l][e] = n->w[l][e] - (float)(grad[k] / (double)global_rows);
	}
	for (int l = 1; l <= H; ++l)
	{
		double s = grad[k + l - 1];
		if (n->d.bias_rule == GL_BIAS_REFERENCE)
			n->bias[l] = n->bias[l] - (float)((double)n->d.sizes[l] * s);
		else
			n->bias[l] = n->bias[l] - (float)(s / (double)global_rows);
	}
	return 0;
}

/* ------------------------------------------------------------------------------------------
 * Counter-based synthetic inputs: Philox4x32-10 (Salmon et al., SC'11), key = (seed lo, seed hi),
 * counter = (index lo, index hi, stream, 0); element i uses word 0 of block i.
 * dist 0: U = (u32 >> 8) * 2^-24.  dist 1: N(0,1) by Box-Muller on the uniforms of elements
 * 2*(i/2) and 2*(i/2)+1 (cos for even i, sin for odd i), with U1 nudged away from 0.
 * ------------------------------------------------------------------------------------------ */
static inline void philox_round(uint32_t* c, uint32_t* k)
{
	const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
	const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
	uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0];
	uint32_t n1 = (uint32_t)p1;
	uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1];
	uint32_t n3 = (uint32_t)p0;
	c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
	k[0] += 0x9E3779B9u;
	k[1] += 0xBB67AE85u;
}

uint32_t rs_philox_u32(uint64_t seed, uint32_t stream, uint64_t index)
{
	uint32_t c[4] = { (uint32_t)index, (uint32_t)(index >> 32), stream, 0u };
	uint32_t k[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) };
	for (int r = 0; r < 10; ++r) philox_round(c, k);
	return c[0];
}

void rs_synth_fill(float* out, int64_t n, uint64_t seed, uint32_t stream, int dist, float scale, float offset)
{
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < n; ++i)
	{
		float v;
		if (dist == 0)
			v = (float)(rs_philox_u32(seed, stream, (uint64_t)i) >> 8) * (1.0f / 16777216.0f);
		else
		{
			uint64_t b = (uint64_t)i & ~(uint64_t)1;
			float u1 = ((float)(rs_philox_u32(seed, stream, b) >> 8) + 0.5f) * (1.0f / 16777216.0f);
			float u2 = (float)(rs_philox_u32(seed, stream, b + 1) >> 8) * (1.0f / 16777216.0f);
			double rad = sqrt(-2.0 * log((double)u1));
			double ang = 6.283185307179586 * (double)u2;
			v = (float)(rad * ((i & 1) ? sin(ang) : cos(ang)));
		}
		out[i] = offset + scale * v;
	}
}

/* ------------------------------------------------------------------------------------------
 * Input standardisation: NumberInput::standardizeInputTable (DataObjects/NumberInput.cpp:43-285) and
 * the one-hot vectors of OHE::operator[] (GMath/OHE.cpp:159-198), restated on a flat raw table.
 *   raw[r*cols + c]   the cell as a float; for a categorical column the category's index in order of
 *                     first appearance (the order OHE::addString builds, OHE.cpp:54-64)
 *   kind[c]           0 numeric, 1 categorical with classes[c] categories
 *   to_output[c]      1: the column goes to the expected-rows table
 *   flag              0 MINMAX, 1 ZSCORE (GMath/gmath.h:53-54)
 * Facts of the reference that are kept: the running minimum and maximum start from the first cell only
 * for raw column 0 and from 0.0 for every other column (NumberInput.cpp:105-109); a table with any
 * categorical column scales numeric columns to [0.01, 0.99], else to [0, 1] (:196-214); a column whose
 * (zero-including) range is 0 is copied unscaled and always lands in the INPUT table (:166-171); the mean
 * is a sequential fp32 sum divided once (:118-121), the deviation sqrt(sum((x-mean)^2) / (rows-1)).
 * Columns keep their raw order inside each output table.  x / y are row-major with nx / ny columns.
 * Returns 0, or -1 when the outputs' widths do not match the plan.
 * ------------------------------------------------------------------------------------------ */
int rs_standardize_table(const float* raw, int64_t rows, int cols, const int* kind, const int* classes,
                         const int* to_output, int flag, float* x, int nx, float* y, int ny)
{
	int classification = 0;
	for (int c = 0; c < cols; ++c)
		if (kind[c] == 1) classification = 1;
	int cx = 0, cy = 0;
	for (int c = 0; c < cols; ++c)
	{
		if (kind[c] == 1)
		{
			float* dst = to_output[c] ? y : x;
			const int ld = to_output[c] ? ny : nx;
			int* at = to_output[c] ? &cy : &cx;
			if (*at + classes[c] > ld) return -1;
			for (int k = 0; k < classes[c]; ++k)
				for (int64_t r = 0; r < rows; ++r)
					dst[(size_t)r * ld + *at + k] = ((int)raw[(size_t)r * cols + c] == k) ? 0.99f : 0.01f;
			*at += classes[c];
			continue;
		}
		float fMin = 0.0f, fMax = 0.0f, fMean = 0.0f;
		for (int64_t r = 0; r < rows; ++r)
		{
			const float cell = raw[(size_t)r * cols + c];
			if (r == 0 && c == 0) { fMin = cell; fMax = cell; }
			if (cell < fMin) fMin = cell;
			if (cell > fMax) fMax = cell;
			fMean += cell;
			if (r == rows - 1) fMean /= (float)(unsigned int)rows;
		}
		int out = to_output[c];
		float fStDev = 0.0f;
		const float xRange = fMax - fMin;
		if (flag == 0 && xRange == 0.0f) out = 0;  /* constant column: copied, to the input table */
		if (flag == 1)
		{
			for (int64_t r = 0; r < rows; ++r)
			{
				const float cell = raw[(size_t)r * cols + c];
				fStDev += ((cell - fMean) * (cell - fMean));
			}
			fStDev = sqrtf(fStDev / (float)((unsigned int)rows - 1u));
		}
		float* dst = out ? y : x;
		const int ld = out ? ny : nx;
		int* at = out ? &cy : &cx;
		if (*at + 1 > ld) return -1;
		for (int64_t r = 0; r < rows; ++r)
		{
			float cell = raw[(size_t)r * cols + c];
			if (flag == 0)
			{
				if (xRange != 0.0f)
					cell = classification ? ((((cell - fMin) / (xRange)) * 0.98f) + 0.01f) : ((cell - fMin) / (xRange));
			}
			else
				cell = ((cell - fMean) / fStDev);
			dst[(size_t)r * ld + *at] = cell;
		}
		*at += 1;
	}
	return (cx == nx && cy == ny) ? 0 : -1;
}
