// Reference-mode kernels: the reference's per-sample SGD, sample after sample, in its exact fp32
// operation order.
//
// ref_train_kernel is one persistent CTA that runs n_epochs * rows samples in a single launch.  A
// sample of NNetwork::SGDHelper (Networks/network.cpp:399-455) is restated on dense matrices:
//   forward   (network.cpp:457-575)  one thread per output node, k ascending, product rounded then
//             sum rounded (Node::getActivation, State/node.cpp:82-93), scalar layer bias added
//             after the sum, then GMath::squash;
//   metrics   (network.cpp:519-547)  one thread, row-major (row, output) order, because the
//             reference's epoch sums are sequential fp32 accumulations;
//   backward  (network.cpp:577-668)  per weight layer from the top: first the node deltas
//             d_o = E_o * act'(a_o); then one thread per INPUT node i walks o = 0..n-1 (the
//             reference's inner loop): pending delta (Node::getDelta, node.cpp:278-292), apply on
//             rows with r % mb == 0 (node.cpp:294-307), and the doubling error accumulation
//             E_i += E_i + d_o*W_oi with the already-updated weight (network.cpp:660-662); the
//             scalar bias recurrence b -= lr*d_o, executed n_in*n_out times per sample
//             (network.cpp:653-656), is a strictly sequential fp32 chain and runs on one thread
//             beside the column threads.
// Weights, pending deltas and all per-sample vectors live in shared memory when they fit
// (up to 227 KB); otherwise in global memory (L1-resident for one CTA).
#include "common.cuh"
#include "internal.h"

namespace glb {

__device__ __forceinline__ int argmax_ref(const float* v, int n)
{
	// GMath::naiveVectorDecomp (GMath/gmath.cpp:435-455): strict > from 0, first maximum wins.
	float mx = 0.0f;
	int idx = -1;
	for (int i = 0; i < n; ++i)
		if (v[i] > mx)
		{
			mx = v[i];
			idx = i;
		}
	return idx;
}

// the epoch's confusion counts stay in shared memory up to this many cells
constexpr int REF_CONF_SMEM = 1024;

__global__ void __launch_bounds__(1024, 1) ref_train_kernel(const __grid_constant__ RefTrainArgs a)
{
	extern __shared__ __align__(16) float smem[];
	const NetView& n = a.net;
	const int H = n.H;
	const int T = blockDim.x;
	const int t = threadIdx.x;
	const int n_out = n.sizes[H + 1];

	int total_nodes = 0;
	for (int l = 0; l <= H + 1; ++l) total_nodes += n.sizes[l];

	// per-sample vectors: activations | error accumulators | d | base
	float* act_base = smem;
	float* err_base = act_base + total_nodes;
	float* dvec = err_base + total_nodes;
	float* basev = dvec + total_nodes;
	float* sbias = basev + total_nodes;  // GL_MAX_WEIGHT_LAYERS floats
	float* mcost = sbias + GL_MAX_WEIGHT_LAYERS;  // per output node: cost and accuracy of this sample
	float* macc = mcost + n_out;
	// the next sample's input and target rows arrive by asynchronous copies while the current sample runs (the
	// sample loop is one dependent chain: a global load at its head would be paid in full every sample)
	float* xbuf = macc + n_out;               // [2][n_in]
	float* ybuf = xbuf + 2 * n.sizes[0];      // [2][n_out]
	// the confusion counts of the running epoch, where they fit (else straight in global memory)
	const bool conf_smem = n_out * n_out <= REF_CONF_SMEM;
	int* sconf = reinterpret_cast<int*>(ybuf + 2 * n_out);
	float* wcur = reinterpret_cast<float*>(sconf + (conf_smem ? n_out * n_out : 0));

	float* actp[GL_MAX_WEIGHT_LAYERS + 1];
	float* errp[GL_MAX_WEIGHT_LAYERS + 1];
	float* Wp[GL_MAX_WEIGHT_LAYERS];
	float* Hp[GL_MAX_WEIGHT_LAYERS];
	{
		int off = 0;
		for (int l = 0; l <= H + 1; ++l)
		{
			actp[l] = act_base + off;
			errp[l] = err_base + off;
			off += n.sizes[l];
		}
	}
	for (int l = 0; l <= H; ++l)
	{
		const int cnt = n.sizes[l] * n.sizes[l + 1];
		if (a.weights_in_smem)
		{
			Wp[l] = wcur;
			wcur += cnt;
			Hp[l] = wcur;
			wcur += (size_t)cnt * n.mb;
			for (int e = t; e < cnt; e += T) Wp[l][e] = n.W[l][e];
			for (int e = t; e < cnt * n.mb; e += T) Hp[l][e] = a.hist[l][e];
		}
		else
		{
			Wp[l] = n.W[l];
			Hp[l] = a.hist[l];
		}
	}
	for (int e = t; e < total_nodes; e += T) err_base[e] = 0.0f;
	if (t < GL_MAX_WEIGHT_LAYERS) sbias[t] = n.bias[t];
	__shared__ int s_hist_len;
	__shared__ float s_tot_err, s_tot_acc;
	if (t == 0) s_hist_len = *a.hist_len;
	__syncthreads();

	const float data_size = (float)(a.rows * (long long)n_out);
	const bool classify = n.out_type != GL_OUT_REGRESSION;
	int* const conf = conf_smem ? sconf : a.confusion;
	const uint32_t xb_addr = (uint32_t)__cvta_generic_to_shared(xbuf), yb_addr = (uint32_t)__cvta_generic_to_shared(ybuf);
	auto prefetch = [&](long long row, int buf) {
		for (int i = t; i < n.sizes[0]; i += T) cp_async4(xb_addr + (uint32_t)(buf * n.sizes[0] + i) * 4, a.X + row * n.sizes[0] + i, true);
		for (int o = t; o < n_out; o += T) cp_async4(yb_addr + (uint32_t)(buf * n_out + o) * 4, a.Y + row * n_out + o, true);
		cp_async_commit();
	};
	if (a.n_epochs > 0 && a.rows > 0) prefetch(0, 0);
	int buf = 0;

	for (int ep = 0; ep < a.n_epochs; ++ep)
	{
		const bool last_epoch = (ep == a.n_epochs - 1);
		if (t == 0)
		{
			s_tot_err = 0.0f;
			s_tot_acc = 0.0f;
		}
		if (classify)
			for (int e = t; e < n_out * n_out; e += T) conf[e] = 0;
		__syncthreads();

		for (long long r = 0; r < a.rows; ++r)
		{
			// ---------------- this sample's rows have landed; the next sample's start travelling
			cp_async_wait<0>();
			__syncthreads();
			actp[0] = xbuf + buf * n.sizes[0];
			const float* yr = ybuf + buf * n_out;
			{
				const long long nr = (r + 1 < a.rows) ? r + 1 : ((ep + 1 < a.n_epochs) ? 0 : -1);
				if (nr >= 0) prefetch(nr, buf ^ 1);  // that buffer was last read by the previous sample, whose end all threads have passed
			}
			buf ^= 1;
			// ---------------- forward
			for (int l = 0; l <= H; ++l)
			{
				const int ni = n.sizes[l], no = n.sizes[l + 1];
				const float* W = Wp[l];
				const float* ain = actp[l];
				for (int o = t; o < no; o += T)
				{
					float z = 0.0f;
					const float* wr = W + (size_t)o * ni;
					for (int i = 0; i < ni; ++i) z = __fadd_rn(z, __fmul_rn(wr[i], ain[i]));
					if (l >= 1) z = __fadd_rn(z, sbias[l]);
					actp[l + 1][o] = squash_x(z, n.act[l], n.par[l]);
					if (a.preact_out && last_epoch && r == a.rows - 1) a.preact_out[(actp[l + 1] - actp[1]) + o] = z;
				}
				__syncthreads();
			}
			// ---------------- metrics: sequential fp32 sums in (row, output) order
			// the per-node values are independent (computed in parallel); only their accumulation into the
			// epoch sums is order-sensitive and stays on one thread
			for (int o = t; o < n_out; o += T)
			{
				mcost[o] = cost_x(yr[o], actp[H + 1][o], data_size, n.out_type);
				macc[o] = node_accuracy_x(yr[o], actp[H + 1][o]);
			}
			__syncthreads();
			if (t == 0)
			{
				const float* p = actp[H + 1];
				float te = s_tot_err, ta = s_tot_acc;
				for (int o = 0; o < n_out; ++o)
				{
					te = __fadd_rn(te, mcost[o]);
					ta = __fadd_rn(ta, macc[o]);
				}
				s_tot_err = te;
				s_tot_acc = ta;
				if (classify)
				{
					int ie = argmax_ref(yr, n_out), ip = argmax_ref(p, n_out);
					if (ie >= 0 && ip >= 0) conf[ie * n_out + ip] += 1;
				}
			}
			if (a.outputs && last_epoch)
				for (int o = t; o < n_out; o += T) a.outputs[r * n_out + o] = actp[H + 1][o];
			if (a.last_out && last_epoch && r == a.rows - 1)
				for (int o = t; o < n_out; o += T) a.last_out[o] = actp[H + 1][o];

			// ---------------- backward
			const int k = s_hist_len;
			const bool apply = (r % n.mb) == 0;
			for (int L = H + 1; L >= 1; --L)
			{
				const int l = L - 1;
				const int ni = n.sizes[l], no = n.sizes[L];
				const float lr = n.lr[l], mom = n.mom[l];
				// node deltas of layer L
				for (int o = t; o < no; o += T)
				{
					float E, der = 1.0f;
					if (L == H + 1)
						E = __fadd_rn(0.0f, cost_der_x(yr[o], actp[L][o], n.out_type));
					else
					{
						E = errp[L][o];
						der = act_der_x(actp[L][o], n.act[l], 0.01f);  // parameter fixed by the caller, network.cpp:618
						errp[L][o] = 0.0f;
					}
					const float d = __fmul_rn(E, der);
					dvec[o] = d;
					basev[o] = __fmul_rn(lr, d);
				}
				__syncthreads();
				float* W = Wp[l];
				float* hist = Hp[l];
				const size_t cnt = (size_t)ni * no;
				const float wl1 = __fmul_rn(n.wd1[l], lr), wl2 = __fmul_rn(n.wd2[l], lr);
				const float fmb = (float)n.mb;
				for (int i = t; i < ni; i += T)
				{
					const float ai = actp[l][i];
					const float c3 = __fmul_rn(wl1, fabsf(ai));
					const float c4 = __fmul_rn(wl2, ai);
					float E = (l >= 1) ? errp[l][i] : 0.0f;
					for (int o = 0; o < no; ++o)
					{
						const size_t e = (size_t)o * ni + i;
						const float last = (k > 0) ? hist[(size_t)(k - 1) * cnt + e] : 0.0f;
						const float delta = __fadd_rn(
						    __fadd_rn(__fadd_rn(__fmul_rn(basev[o], ai), __fmul_rn(mom, last)), c3), c4);
						hist[(size_t)k * cnt + e] = delta;
						float w = W[e];
						if (apply)
						{
							float s = 0.0f;
							for (int q = 0; q < k; ++q) s = __fadd_rn(s, hist[(size_t)q * cnt + e]);
							s = __fadd_rn(s, delta);
							if (fmb != 1.0f) s = __fdiv_rn(s, fmb);  // x / 1 is x in IEEE arithmetic: the division is skipped, not changed
							w = __fsub_rn(w, s);
							W[e] = w;
						}
						if (l >= 1)
						{
							const float tt = __fadd_rn(E, __fmul_rn(dvec[o], w));
							E = __fadd_rn(E, tt);
						}
					}
					if (l >= 1) errp[l][i] = E;
				}
				// scalar bias recurrence of the input-side hidden layer: one sequential chain
				if (l >= 1 && t == T - 1)
				{
					float b = sbias[l];
					for (int i = 0; i < ni; ++i)
						for (int o = 0; o < no; ++o) b = __fsub_rn(b, basev[o]);
					sbias[l] = b;
				}
				__syncthreads();
			}
			if (t == 0) s_hist_len = apply ? 0 : k + 1;
			__syncthreads();
		}
		if (t == 0)
		{
			a.epoch_sums[2 * ep + 0] = s_tot_err;
			a.epoch_sums[2 * ep + 1] = s_tot_acc;
		}
		if (classify && conf_smem && last_epoch)
			for (int e = t; e < n_out * n_out; e += T) a.confusion[e] = sconf[e];
		__syncthreads();
	}

	// write back state and look for non-finite weights
	int bad = 0;
	for (int l = 0; l <= H; ++l)
	{
		const int cnt = n.sizes[l] * n.sizes[l + 1];
		if (a.weights_in_smem)
		{
			for (int e = t; e < cnt; e += T) n.W[l][e] = Wp[l][e];
			for (int e = t; e < cnt * n.mb; e += T) a.hist[l][e] = Hp[l][e];
		}
		for (int e = t; e < cnt; e += T)
			if (!isfinite(Wp[l][e])) bad = 1;
	}
	if (t < GL_MAX_WEIGHT_LAYERS)
	{
		n.bias[t] = sbias[t];
		if (t >= 1 && t <= H && !isfinite(sbias[t])) bad = 1;
	}
	if (t == 0) *a.hist_len = s_hist_len;
	if (bad) atomicOr(a.flags, 1);
}

// ---------------------------------------------------------------------------------------------
// The same sample loop with dropped nodes (LayerBuilder::scrambleDropout, State/LayerBuilder.cpp:497-523;
// the flags are drawn on the host in the reference's rand() order and arrive as one byte per node of
// every non-output layer, [rows][mask_stride]).  What changes (network.cpp:476-508,620-662):
//   forward   an edge counts only when both of its nodes are kept; the sum of a node runs over its kept
//             inputs in i order; a dropped node gets squash(0 + bias);
//   backward  a dropped pair uses the raw accumulator E_o as its delta (no derivative factor), pushes,
//             applies and subtracts nothing, but still feeds E_i += E_i + E_o * W_oi; E_o is cleared
//             only when the pair (n_in - 1, o) is kept, so hidden accumulators can survive a row (they
//             are carried from launch to launch in a.err_state);
//   history   every edge has its own history length (a dropped pair pushes nothing): hlen / hlast hold
//             the length and the last pushed delta per edge, hist its first mb entries; an apply sums
//             those first mb entries (Node::applyDeltas, node.cpp:299-301) and empties the history.
// One epoch per launch (the host draws each epoch's flags before it).  Weights, histories and flags stay
// in global memory (one CTA: they sit in L1/L2); the per-sample vectors are in shared memory.
__global__ void __launch_bounds__(1024, 1) ref_train_dropout_kernel(const __grid_constant__ RefTrainArgs a)
{
	extern __shared__ __align__(16) float smem[];
	const NetView& n = a.net;
	const int H = n.H;
	const int T = blockDim.x;
	const int t = threadIdx.x;
	const int n_out = n.sizes[H + 1];

	int total_nodes = 0;
	for (int l = 0; l <= H + 1; ++l) total_nodes += n.sizes[l];

	float* act_base = smem;
	float* err_base = act_base + total_nodes;
	float* dvec = err_base + total_nodes;    // E_o * act'(a_o): the delta of a kept pair
	float* basev = dvec + total_nodes;       // lr * delta
	float* rawv = basev + total_nodes;       // E_o itself: the delta of a dropped pair
	float* sbias = rawv + total_nodes;
	float* mcost = sbias + GL_MAX_WEIGHT_LAYERS;
	float* macc = mcost + n_out;

	float* actp[GL_MAX_WEIGHT_LAYERS + 1];
	float* errp[GL_MAX_WEIGHT_LAYERS + 1];
	int moff[GL_MAX_WEIGHT_LAYERS + 1];
	{
		int off = 0;
		for (int l = 0; l <= H + 1; ++l)
		{
			actp[l] = act_base + off;
			errp[l] = err_base + off;
			moff[l] = off;  // node layer l's flags start here inside a row of flags (l <= H)
			off += n.sizes[l];
		}
	}
	for (int e = t; e < total_nodes; e += T) err_base[e] = a.err_state[e];
	if (t < GL_MAX_WEIGHT_LAYERS) sbias[t] = n.bias[t];
	__shared__ float s_tot_err, s_tot_acc;
	if (t == 0)
	{
		s_tot_err = 0.0f;
		s_tot_acc = 0.0f;
	}
	const float data_size = (float)((a.data_rows > 0 ? a.data_rows : a.rows) * (long long)n_out);
	const bool classify = n.out_type != GL_OUT_REGRESSION;
	if (classify)
		for (int e = t; e < n_out * n_out; e += T) a.confusion[e] = 0;
	__syncthreads();

	for (long long r = 0; r < a.rows; ++r)
	{
		const unsigned char* mrow = a.masks + r * a.mask_stride;
		// ---------------- forward
		for (int i = t; i < n.sizes[0]; i += T) actp[0][i] = a.X[r * n.sizes[0] + i];
		__syncthreads();
		for (int l = 0; l <= H; ++l)
		{
			const int ni = n.sizes[l], no = n.sizes[l + 1];
			const float* W = n.W[l];
			const float* ain = actp[l];
			const unsigned char* din = mrow + moff[l];
			const unsigned char* dout = (l + 1 <= H) ? mrow + moff[l + 1] : nullptr;
			for (int o = t; o < no; o += T)
			{
				float z = 0.0f;
				if (!(dout && dout[o]))
				{
					const float* wr = W + (size_t)o * ni;
					for (int i = 0; i < ni; ++i)
						if (!din[i]) z = __fadd_rn(z, __fmul_rn(wr[i], ain[i]));
				}
				if (l >= 1) z = __fadd_rn(z, sbias[l]);
				actp[l + 1][o] = squash_x(z, n.act[l], n.par[l]);
				if (a.preact_out && r == a.rows - 1) a.preact_out[(actp[l + 1] - actp[1]) + o] = z;
			}
			__syncthreads();
		}
		// ---------------- metrics
		const float* yr = a.Y ? a.Y + r * n_out : nullptr;  // forward-only calls may come without expected rows
		if (yr)
			for (int o = t; o < n_out; o += T)
			{
				mcost[o] = cost_x(yr[o], actp[H + 1][o], data_size, n.out_type);
				macc[o] = node_accuracy_x(yr[o], actp[H + 1][o]);
			}
		__syncthreads();
		if (t == 0 && yr)
		{
			const float* p = actp[H + 1];
			float te = s_tot_err, ta = s_tot_acc;
			for (int o = 0; o < n_out; ++o)
			{
				te = __fadd_rn(te, mcost[o]);
				ta = __fadd_rn(ta, macc[o]);
			}
			s_tot_err = te;
			s_tot_acc = ta;
			if (classify)
			{
				int ie = argmax_ref(yr, n_out), ip = argmax_ref(p, n_out);
				if (ie >= 0 && ip >= 0) a.confusion[ie * n_out + ip] += 1;
			}
		}
		if (a.outputs)
			for (int o = t; o < n_out; o += T) a.outputs[r * n_out + o] = actp[H + 1][o];
		if (a.last_out && r == a.rows - 1)
			for (int o = t; o < n_out; o += T) a.last_out[o] = actp[H + 1][o];
		if (a.acts_out && r == a.rows - 1)
			for (int e = t; e < total_nodes - n.sizes[0]; e += T) a.acts_out[e] = act_base[n.sizes[0] + e];
		if (!a.train || !yr)
		{
			__syncthreads();
			continue;
		}

		// ---------------- backward
		const bool apply = (r % n.mb) == 0;
		for (int L = H + 1; L >= 1; --L)
		{
			const int l = L - 1;
			const int ni = n.sizes[l], no = n.sizes[L];
			const float lr = n.lr[l], mom = n.mom[l];
			const unsigned char* din = mrow + moff[l];
			const unsigned char* dout = (L <= H) ? mrow + moff[L] : nullptr;
			const bool last_in_kept = !din[ni - 1];
			for (int o = t; o < no; o += T)
			{
				float E, der = 1.0f;
				if (L == H + 1)
					E = __fadd_rn(0.0f, cost_der_x(yr[o], actp[L][o], n.out_type));
				else
				{
					E = errp[L][o];
					der = act_der_x(actp[L][o], n.act[l], 0.01f);
					// cleared by the pair (n_in - 1, o), and only when that pair is kept
					if (last_in_kept && !dout[o]) errp[L][o] = 0.0f;
				}
				const float d = __fmul_rn(E, der);
				rawv[o] = E;
				dvec[o] = d;
				basev[o] = __fmul_rn(lr, d);
			}
			__syncthreads();
			float* W = n.W[l];
			float* hist = a.hist[l];
			int* hlen = a.hlen[l];
			float* hlast = a.hlast[l];
			const size_t cnt = (size_t)ni * no;
			const float wl1 = __fmul_rn(n.wd1[l], lr), wl2 = __fmul_rn(n.wd2[l], lr);
			const float fmb = (float)n.mb;
			for (int i = t; i < ni; i += T)
			{
				const float ai = actp[l][i];
				const float c3 = __fmul_rn(wl1, fabsf(ai));
				const float c4 = __fmul_rn(wl2, ai);
				const bool in_dropped = din[i] != 0;
				float E = (l >= 1) ? errp[l][i] : 0.0f;
				for (int o = 0; o < no; ++o)
				{
					const size_t e = (size_t)o * ni + i;
					const bool dropped = in_dropped || (dout && dout[o]);
					float w = W[e];
					float dd = rawv[o];
					if (!dropped)
					{
						dd = dvec[o];
						int len = hlen[e];
						const float last = (len > 0) ? hlast[e] : 0.0f;
						const float delta = __fadd_rn(
						    __fadd_rn(__fadd_rn(__fmul_rn(basev[o], ai), __fmul_rn(mom, last)), c3), c4);
						if (len < n.mb) hist[(size_t)len * cnt + e] = delta;
						hlast[e] = delta;
						++len;
						if (apply)
						{
							float s = 0.0f;
							const int q_end = len < n.mb ? len : n.mb;
							for (int q = 0; q < q_end; ++q) s = __fadd_rn(s, hist[(size_t)q * cnt + e]);
							s = __fdiv_rn(s, fmb);
							w = __fsub_rn(w, s);
							W[e] = w;
							len = 0;
						}
						hlen[e] = len;
					}
					if (l >= 1)
					{
						const float tt = __fadd_rn(E, __fmul_rn(dd, w));
						E = __fadd_rn(E, tt);
					}
				}
				if (l >= 1) errp[l][i] = E;
			}
			// scalar bias recurrence over the kept pairs, i outer, o inner: one sequential chain
			if (l >= 1 && t == T - 1)
			{
				float b = sbias[l];
				for (int i = 0; i < ni; ++i)
				{
					if (din[i]) continue;
					for (int o = 0; o < no; ++o)
						if (!(dout && dout[o])) b = __fsub_rn(b, basev[o]);
				}
				sbias[l] = b;
			}
			__syncthreads();
		}
	}
	if (t == 0)
	{
		a.epoch_sums[0] = s_tot_err;
		a.epoch_sums[1] = s_tot_acc;
	}
	__syncthreads();
	for (int e = t; e < total_nodes; e += T) a.err_state[e] = err_base[e];
	int bad = 0;
	for (int l = 0; l <= H; ++l)
	{
		const int cnt = n.sizes[l] * n.sizes[l + 1];
		for (int e = t; e < cnt; e += T)
			if (!isfinite(n.W[l][e])) bad = 1;
	}
	if (t < GL_MAX_WEIGHT_LAYERS)
	{
		n.bias[t] = sbias[t];
		if (t >= 1 && t <= H && !isfinite(sbias[t])) bad = 1;
	}
	if (bad) atomicOr(a.flags, 1);
}

static int total_nodes_of(const NetView& n)
{
	int s = 0;
	for (int l = 0; l <= n.H + 1; ++l) s += n.sizes[l];
	return s;
}

size_t ref_train_smem_bytes(const NetView& n, bool weights_in_smem)
{
	const size_t n_out = (size_t)n.sizes[n.H + 1];
	size_t f = 4 * (size_t)total_nodes_of(n) + GL_MAX_WEIGHT_LAYERS + 2 * n_out;
	f += 2 * ((size_t)n.sizes[0] + n_out);                       // double-buffered input and target rows
	if (n_out * n_out <= (size_t)REF_CONF_SMEM) f += n_out * n_out;  // confusion counts
	if (weights_in_smem)
		for (int l = 0; l <= n.H; ++l) f += (size_t)n.sizes[l] * n.sizes[l + 1] * (1 + (size_t)n.mb);
	return f * sizeof(float);
}

size_t ref_train_dropout_smem_bytes(const NetView& n)
{
	return (5 * (size_t)total_nodes_of(n) + GL_MAX_WEIGHT_LAYERS + 2 * (size_t)n.sizes[n.H + 1]) * sizeof(float);
}

cudaError_t launch_ref_train(const RefTrainArgs& a, cudaStream_t s)
{
	int maxw = 1;
	for (int l = 0; l <= a.net.H + 1; ++l) maxw = a.net.sizes[l] > maxw ? a.net.sizes[l] : maxw;
	int T = ((maxw + 1 + 31) / 32) * 32;  // one spare thread for the bias chain
	if (T > 1024) T = 1024;
	if (a.masks)
	{
		const size_t bytes = ref_train_dropout_smem_bytes(a.net);
		cudaError_t e = cudaFuncSetAttribute(ref_train_dropout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
		if (e != cudaSuccess) return e;
		ref_train_dropout_kernel<<<1, T, bytes, s>>>(a);
		return cudaGetLastError();
	}
	const size_t bytes = ref_train_smem_bytes(a.net, a.weights_in_smem != 0);
	cudaError_t e = cudaFuncSetAttribute(ref_train_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
	if (e != cudaSuccess) return e;
	ref_train_kernel<<<1, T, bytes, s>>>(a);
	return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Exact-order forward for inference / read-back: rows are independent, so the grid runs over
// (row, output node); each thread still sums k ascending with separately rounded products.
struct FwdLayerArgs
{
	const float* in;   // [rows][ni]
	float* out;        // [rows][no]
	const float* W;
	const float* bias; // device array, entry l
	int ni, no, l, act;
	float par;
	long long rows;
	float* zout;       // optional: pre-activations of row 0, `no` floats
};

__global__ void ref_forward_layer_kernel(const FwdLayerArgs f)
{
	const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	const long long total = f.rows * f.no;
	if (idx >= total) return;
	const long long r = idx / f.no;
	const int o = (int)(idx - r * f.no);
	const float* x = f.in + r * f.ni;
	const float* w = f.W + (size_t)o * f.ni;
	float z = 0.0f;
	for (int i = 0; i < f.ni; ++i) z = __fadd_rn(z, __fmul_rn(w[i], x[i]));
	if (f.l >= 1) z = __fadd_rn(z, f.bias[f.l]);
	f.out[idx] = squash_x(z, f.act, f.par);
	if (f.zout && r == 0) f.zout[o] = z;
}

cudaError_t launch_ref_forward(const NetView& n, const float* X, long long rows, float* const* acts, cudaStream_t s, float* zout)
{
	const float* in = X;
	int zoff = 0;
	for (int l = 0; l <= n.H; ++l)
	{
		FwdLayerArgs f;
		f.in = in;
		f.out = acts[l + 1];
		f.W = n.W[l];
		f.bias = n.bias;
		f.ni = n.sizes[l];
		f.no = n.sizes[l + 1];
		f.l = l;
		f.act = n.act[l];
		f.par = n.par[l];
		f.rows = rows;
		f.zout = zout ? zout + zoff : nullptr;
		zoff += n.sizes[l + 1];
		const long long total = rows * f.no;
		const int T = 128;
		ref_forward_layer_kernel<<<(unsigned)((total + T - 1) / T), T, 0, s>>>(f);
		cudaError_t e = cudaGetLastError();
		if (e != cudaSuccess) return e;
		in = f.out;
	}
	return cudaSuccess;
}

// Sequential metric accumulation in the reference's (row, output) order -- one thread, because
// fp32 addition is not associative and the epoch figures are compared bit for bit.
__global__ void ref_metrics_kernel(NetView n, const float* P, const float* Y, long long rows, long long data_rows,
                                   float* sums2, int* confusion)
{
	if (threadIdx.x != 0 || blockIdx.x != 0) return;
	const int no = n.sizes[n.H + 1];
	const float data_size = (float)(data_rows * (long long)no);
	float te = sums2[0], ta = sums2[1];
	for (long long r = 0; r < rows; ++r)
	{
		const float* p = P + r * no;
		const float* y = Y + r * no;
		for (int o = 0; o < no; ++o)
		{
			te = __fadd_rn(te, cost_x(y[o], p[o], data_size, n.out_type));
			ta = __fadd_rn(ta, node_accuracy_x(y[o], p[o]));
		}
		if (n.out_type != GL_OUT_REGRESSION && confusion)
		{
			int ie = argmax_ref(y, no), ip = argmax_ref(p, no);
			if (ie >= 0 && ip >= 0) confusion[ie * no + ip] += 1;
		}
	}
	sums2[0] = te;
	sums2[1] = ta;
}

cudaError_t launch_ref_metrics(const NetView& n, const float* P, const float* Y, long long rows, long long data_rows,
                               float* sums2, int* confusion, cudaStream_t s)
{
	ref_metrics_kernel<<<1, 32, 0, s>>>(n, P, Y, rows, data_rows, sums2, confusion);
	return cudaGetLastError();
}

}  // namespace glb
