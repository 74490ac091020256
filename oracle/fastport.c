/*
 * TEST INFRASTRUCTURE ONLY -- the timed CPU baseline of the benchmark's reference arm for the shapes on
 * which the reference's own compiled code cannot be timed (the wide network: one training row takes eleven
 * minutes there).  Never linked into, imported by or called from the product library, and not the checker
 * either: parity is checked against restate.c, which accumulates in double.
 *
 * What it is: the batched-mode window step of restate.c (rs_window_grad + rs_window_apply: forward, softmax
 * or per-node head, plain error sum, weight gradient with the intra-window momentum weights, update) with
 * the three layer products done as cache-blocked, register-tiled fp32 matrix products over all host cores --
 * a fair CPU figure for the same arithmetic (fp32 accumulation, as the GPU path has it), where restate.c's
 * loop nests are written for clarity.  Checked against restate.c by tests/test_oracle_pin.py.
 *
 * Build: part of librestate.so (see Makefile), -O3, function multi-versioning for AVX2 / AVX-512 hosts.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "glades_b200.h"

/* accessors of the restatement's network object (restate.c) */
typedef struct rs_net rs_net;
const gl_net_desc* rs_desc(const rs_net* n);
float* rs_weights(rs_net* n, int l);
float* rs_biases(rs_net* n);
const float* rs_x(const rs_net* n);
const float* rs_y(const rs_net* n);
float rs_squash(float z, int act, float p);
float rs_act_der(float a, int act, float p);
float rs_cost(float e, float p, float n, int fx);
float rs_cost_der(float e, float p, int fx);

#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define MULTIVERSION __attribute__((target_clones("default", "avx2,fma", "avx512f")))
#else
#define MULTIVERSION
#endif

enum { MR = 4, NR = 32, KC = 256, MC = 64 };
typedef float vf __attribute__((vector_size(64)));  /* 16 floats; split by the compiler where the host has narrower registers */

/* C[m][n] (ldc) (+)= sum_k A(m,k) * B(n,k), A(m,k) = A[m*a_sm + k*a_sk], B(n,k) = B[n*b_sn + k*b_sk].
 * Panels of A (MR rows) and B (NR columns) are packed k-major so that the inner loop streams both. */
MULTIVERSION
static void micro(int kc, const float* restrict Ap, const float* restrict Bp, float* restrict C, long ldc, int mr, int nr,
                  int accumulate)
{
	vf acc[MR][NR / 16];
	for (int r = 0; r < MR; ++r)
		for (int v = 0; v < NR / 16; ++v) acc[r][v] = (vf){0};
	for (int k = 0; k < kc; ++k)
	{
		const vf* b = (const vf*)(Bp + (size_t)k * NR);
		for (int r = 0; r < MR; ++r)
		{
			const float a = Ap[(size_t)k * MR + r];
			for (int v = 0; v < NR / 16; ++v) acc[r][v] += a * b[v];
		}
	}
	for (int r = 0; r < mr; ++r)
		for (int c = 0; c < nr; ++c)
		{
			const float s = acc[r][c / 16][c % 16];
			C[(size_t)r * ldc + c] = accumulate ? C[(size_t)r * ldc + c] + s : s;
		}
}

MULTIVERSION
static void sgemm(int M, int N, int K, const float* A, long a_sm, long a_sk, const float* B, long b_sn, long b_sk, float* C,
                  long ldc)
{
#pragma omp parallel
	{
		float* Ap = (float*)aligned_alloc(64, (size_t)MC * KC * sizeof(float));
		float* Bp = (float*)aligned_alloc(64, (size_t)NR * KC * sizeof(float));
		/* one (MC rows) x (NR columns) block of C per work item: each thread packs what it needs */
		const int mblocks = (M + MC - 1) / MC, nblocks = (N + NR - 1) / NR;
#pragma omp for schedule(static) collapse(2)
		for (int mb = 0; mb < mblocks; ++mb)
			for (int nb = 0; nb < nblocks; ++nb)
			{
				const int m0 = mb * MC, mc = (M - m0 < MC) ? M - m0 : MC;
				const int n0 = nb * NR, nr = (N - n0 < NR) ? N - n0 : NR;
				for (int k0 = 0; k0 < K; k0 += KC)
				{
					const int kc = (K - k0 < KC) ? K - k0 : KC;
					for (int k = 0; k < kc; ++k)
					{
						for (int c = 0; c < nr; ++c) Bp[(size_t)k * NR + c] = B[(size_t)(n0 + c) * b_sn + (size_t)(k0 + k) * b_sk];
						for (int c = nr; c < NR; ++c) Bp[(size_t)k * NR + c] = 0.0f;
					}
					for (int i0 = 0; i0 < mc; i0 += MR)
					{
						const int mr = (mc - i0 < MR) ? mc - i0 : MR;
						float* ap = Ap + (size_t)i0 * KC;
						for (int k = 0; k < kc; ++k)
						{
							for (int r = 0; r < mr; ++r) ap[(size_t)k * MR + r] = A[(size_t)(m0 + i0 + r) * a_sm + (size_t)(k0 + k) * a_sk];
							for (int r = mr; r < MR; ++r) ap[(size_t)k * MR + r] = 0.0f;
						}
						micro(kc, ap, Bp, C + (size_t)(m0 + i0) * ldc + n0, ldc, mr, nr, k0 > 0);
					}
				}
			}
		free(Ap);
		free(Bp);
	}
}

/* One batched-mode window step over rows [first, first + cnt): the arithmetic of rs_window_grad followed by
 * rs_window_apply (one shard, mean bias rule or the reference's), fp32 throughout.  Returns the window's cost
 * sum through *cost (may be NULL). */
int rs_window_step_fast(rs_net* n, int64_t first, int cnt, float* cost_out)
{
	const gl_net_desc* d = rs_desc(n);
	const int H = d->n_layers - 2;
	const int n_out = d->sizes[H + 1];
	float* act[GL_MAX_WEIGHT_LAYERS + 1];
	float* D[GL_MAX_WEIGHT_LAYERS + 1];
	for (int l = 0; l <= H + 1; ++l)
	{
		act[l] = (float*)malloc((size_t)cnt * d->sizes[l] * sizeof(float));
		D[l] = (float*)malloc((size_t)cnt * d->sizes[l] * sizeof(float));
	}
	memcpy(act[0], rs_x(n) + (size_t)first * d->sizes[0], (size_t)cnt * d->sizes[0] * sizeof(float));
	const float* bias = rs_biases(n);
	/* forward */
	for (int l = 0; l <= H; ++l)
	{
		const int ni = d->sizes[l], no = d->sizes[l + 1];
		sgemm(cnt, no, ni, act[l], ni, 1, rs_weights(n, l), ni, 1, act[l + 1], no);
		const float b = l >= 1 ? bias[l] : 0.0f;
		const int a = d->activation[l];
		const float par = d->act_param[l];
#pragma omp parallel for schedule(static)
		for (int j = 0; j < cnt; ++j)
		{
			float* z = act[l + 1] + (size_t)j * no;
			if (a == GL_ACT_SOFTMAX)
			{
				float mx = -INFINITY, den = 0.0f;
				for (int o = 0; o < no; ++o)
				{
					z[o] += b;
					if (z[o] > mx) mx = z[o];
				}
				for (int o = 0; o < no; ++o)
				{
					z[o] = expf(z[o] - mx);
					den += z[o];
				}
				for (int o = 0; o < no; ++o) z[o] /= den;
			}
			else
				for (int o = 0; o < no; ++o) z[o] = rs_squash(z[o] + b, a, par);
		}
	}
	/* head: cost and output delta */
	const int softmax = d->activation[H] == GL_ACT_SOFTMAX;
	const float dataSize = (float)((int64_t)cnt * n_out);
	double cost = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : cost)
	for (int j = 0; j < cnt; ++j)
	{
		const float* p = act[H + 1] + (size_t)j * n_out;
		const float* e = rs_y(n) + (size_t)(first + j) * n_out;
		float* dd = D[H + 1] + (size_t)j * n_out;
		for (int o = 0; o < n_out; ++o)
		{
			if (softmax)
			{
				if (e[o] != 0.0f) cost += (double)((-(e[o] * logf(p[o]))) / dataSize);
				dd[o] = p[o] - e[o];
			}
			else
			{
				cost += (double)rs_cost(e[o], p[o], dataSize, d->output_type);
				dd[o] = rs_cost_der(e[o], p[o], d->output_type);
			}
		}
	}
	/* backward and update, layer by layer from the top (weights are frozen inside the window: the deltas of
	 * all layers are formed before any weight changes) */
	for (int L = H + 1; L >= 2; --L)
	{
		const int l = L - 1, ni = d->sizes[l], no = d->sizes[L];
		sgemm(cnt, ni, no, D[L], no, 1, rs_weights(n, l), 1, ni, D[l], ni);
		const int a = d->activation[l - 1];
#pragma omp parallel for schedule(static)
		for (int j = 0; j < cnt; ++j)
			for (int i = 0; i < ni; ++i) D[l][(size_t)j * ni + i] *= rs_act_der(act[l][(size_t)j * ni + i], a, 0.01f);
	}
	float* G = NULL;
	size_t gcap = 0;
	for (int l = 0; l <= H; ++l)
	{
		const int L = l + 1, ni = d->sizes[l], no = d->sizes[L];
		const float lr = d->lr[l], m = d->momentum[l];
		/* momentum weights c_j = sum_{t < cnt - j} m^t scale the delta rows (the closed form of the reference's
		 * intra-window history) */
		float bsum = 0.0f;
		for (int j = 0; j < cnt; ++j)
		{
			float c = 0.0f, pw = 1.0f;
			for (int t = 0; t < cnt - j && (m != 0.0f || t == 0); ++t)
			{
				c += pw;
				pw *= m;
			}
			float* row = D[L] + (size_t)j * no;
			for (int o = 0; o < no; ++o)
			{
				bsum += lr * row[o];
				row[o] *= c;
			}
		}
		if ((size_t)no * ni > gcap)
		{
			free(G);
			gcap = (size_t)no * ni;
			G = (float*)malloc(gcap * sizeof(float));
		}
		sgemm(no, ni, cnt, D[L], 1, no, act[l], 1, ni, G, ni);
		float* W = rs_weights(n, l);
		const float inv = 1.0f / (float)cnt;
		float* colterm = NULL;
		if (d->wd1[l] != 0.0f || d->wd2[l] != 0.0f)
		{
			colterm = (float*)calloc(ni, sizeof(float));
			for (int j = 0; j < cnt; ++j)
			{
				float c = 0.0f, pw = 1.0f;
				for (int t = 0; t < cnt - j && (m != 0.0f || t == 0); ++t)
				{
					c += pw;
					pw *= m;
				}
				for (int i = 0; i < ni; ++i)
				{
					const float a = act[l][(size_t)j * ni + i];
					colterm[i] += c * (d->wd1[l] * lr * fabsf(a) + d->wd2[l] * lr * a);
				}
			}
		}
#pragma omp parallel for schedule(static)
		for (int o = 0; o < no; ++o)
			for (int i = 0; i < ni; ++i)
				W[(size_t)o * ni + i] -= (lr * G[(size_t)o * ni + i] + (colterm ? colterm[i] : 0.0f)) * inv;
		free(colterm);
		if (l >= 1)
		{
			float* bb = rs_biases(n);
			bb[l] -= (d->bias_rule == GL_BIAS_REFERENCE) ? (float)d->sizes[l] * bsum : bsum * inv;
		}
	}
	free(G);
	for (int l = 0; l <= H + 1; ++l)
	{
		free(act[l]);
		free(D[l]);
	}
	if (cost_out) *cost_out = (float)cost;
	return 0;
}
