// TEST INFRASTRUCTURE ONLY -- the checker, never the thing shipped or measured as the product.
//
// Harness around the UNMODIFIED reference sources (compiled where they lie by ./Makefile into
// oracle/_ref/libglades_ref.so).  It is built with -fno-access-control so it can reach the
// private members of NNetwork / LayerBuilder: the reference has no API to inject weights, to read
// per-layer activations or to read the confusion counts after run() has cleaned them.
//
// What is the reference's own code here: NNetwork::train / test / run / SGDHelper / ForwardPass /
// BackPropagation (Networks/network.cpp), LayerBuilder / Layer / Node / Edge (State/), GMath and
// CMatrix (GMath/), NNInfo and the *LayerInfo classes (Structure/).  What is ours: this file, the
// shmea link shim and a DataInput subclass that serves rows from flat float arrays.
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#include <string>
#include <vector>

#include "Backend/Machine Learning/DataObjects/DataInput.h"
#include "Backend/Machine Learning/DataObjects/NumberInput.h"
#include "Backend/Machine Learning/GMath/OHE.h"
#include "Backend/Machine Learning/GMath/cmatrix.h"
#include "Backend/Machine Learning/GMath/gmath.h"
#include "Backend/Machine Learning/Networks/network.h"
#include "Backend/Machine Learning/State/LayerBuilder.h"
#include "Backend/Machine Learning/State/layer.h"
#include "Backend/Machine Learning/State/node.h"
#include "Backend/Machine Learning/Structure/hiddenlayerinfo.h"
#include "Backend/Machine Learning/Structure/inputlayerinfo.h"
#include "Backend/Machine Learning/Structure/nninfo.h"
#include "Backend/Machine Learning/Structure/outputlayerinfo.h"

#include "glades_b200.h"

// shim/shmea_shim.cpp
namespace shmea {
void shimRegisterTable(const char* name, const GTable& t);
struct ShimMessage
{
	std::string command, kind;
	std::vector<double> args, payload;
	int rows, cols;
};
void shimClearMessages();
size_t shimMessageCount();
const ShimMessage& shimMessage(size_t i);
}

namespace {

// Rows served from flat arrays through the reference's abstract DataInput interface
// (DataObjects/DataInput.h:26-50).
class ArrayInput : public glades::DataInput
{
public:
	const float* x;
	const float* y;
	unsigned int rows, nIn, nOut;
	std::vector<shmea::GList> xr, yr;

	ArrayInput(const float* nx, const float* ny, unsigned int r, unsigned int ni, unsigned int no)
		: x(nx), y(ny), rows(r), nIn(ni), nOut(no)
	{
		featureIsCategorical.assign(ni, false);
		xr.resize(r);
		yr.resize(r);
		for (unsigned int i = 0; i < r; ++i)
		{
			for (unsigned int c = 0; c < ni; ++c)
				xr[i].addFloat(x[(size_t)i * ni + c]);
			for (unsigned int c = 0; c < no; ++c)
				yr[i].addFloat(y[(size_t)i * no + c]);
		}
	}
	virtual void import(shmea::GString) {}
	virtual shmea::GList getTrainRow(unsigned int r) const { return xr[r]; }
	virtual shmea::GList getTrainExpectedRow(unsigned int r) const { return yr[r]; }
	virtual shmea::GList getTestRow(unsigned int r) const { return xr[r]; }
	virtual shmea::GList getTestExpectedRow(unsigned int r) const { return yr[r]; }
	virtual unsigned int getTrainSize() const { return rows; }
	virtual unsigned int getTestSize() const { return 0; }
	virtual unsigned int getFeatureCount() const { return nIn; }
	virtual int getType() const { return CSV; }
};

// The reference prints several lines per input row while building and the whole network after
// every run(); silence stdout around its calls.
struct Quiet
{
	int saved;
	Quiet()
	{
		fflush(stdout);
		saved = dup(1);
		FILE* f = fopen("/dev/null", "w");
		dup2(fileno(f), 1);
		fclose(f);
	}
	~Quiet()
	{
		fflush(stdout);
		dup2(saved, 1);
		close(saved);
	}
};

struct RefNet
{
	gl_net_desc desc;
	std::vector<float> x, y;
	glades::NNInfo* info;
	ArrayInput* di;
	glades::NNetwork* net;
	int epochsDone;
};

} // namespace

extern "C" {

void* ref_create(const gl_net_desc* d, const float* x, const float* y, int64_t rows)
{
	using namespace glades;
	const int H = d->n_layers - 2;
	if (H < 1 || rows <= 0)
		return NULL;
	// The descriptor holds EFFECTIVE values.  NNInfo::getWeightDecay2(0) returns the input layer's
	// weightDecay1 (Structure/nninfo.cpp:305-306), so the reference cannot express wd2[0] != wd1[0].
	if (d->wd2[0] != d->wd1[0])
		return NULL;
	// Dropout, effective values too: p_dropout[j] is the probability the loop uses for node layer j.  The
	// loop reads getPInput() for the input layer and getPDropout(i) for hidden layer i, and getPDropout(0)
	// is again the input layer's value (Structure/nninfo.cpp:140-146,321-333; network.cpp:408-411): the
	// reference cannot express p_dropout[1] != p_dropout[0], and hidden layer k's own value is what
	// governs hidden layer k+1.
	if (d->p_dropout[1] != d->p_dropout[0])
		return NULL;
	RefNet* r = new RefNet();
	r->desc = *d;
	r->x.assign(x, x + (size_t)rows * d->sizes[0]);
	r->y.assign(y, y + (size_t)rows * d->sizes[H + 1]);
	r->epochsDone = 0;

	InputLayerInfo* in = new InputLayerInfo(d->batch_size, d->lr[0], d->momentum[0], d->wd1[0], d->wd2[0],
	                                        d->p_dropout[0], d->activation[0], d->act_param[0]);
	std::vector<HiddenLayerInfo*> hidden;
	for (int l = 1; l <= H; ++l)
		hidden.push_back(new HiddenLayerInfo(d->sizes[l], d->lr[l], d->momentum[l], d->wd1[l], d->wd2[l],
		                                     l + 1 <= H ? d->p_dropout[l + 1] : 0.0f, d->activation[l], d->act_param[l]));
	OutputLayerInfo* out = new OutputLayerInfo(d->sizes[H + 1], d->output_type);
	r->info = new NNInfo("oracle", in, hidden, out);
	r->di = new ArrayInput(&r->x[0], &r->y[0], (unsigned int)rows, d->sizes[0], d->sizes[H + 1]);
	r->net = new NNetwork(r->info);
	{
		Quiet q;
		// What run() does on its first call (network.cpp:127-128).
		r->net->di = r->di;
		r->net->meat.build(r->info, r->di, r->net->netType);
	}
	// epochs != 0 keeps run() from rebuilding (and re-drawing random weights).
	r->net->epochs = 1;
	return r;
}

void ref_destroy(void* h)
{
	RefNet* r = (RefNet*)h;
	if (!r)
		return;
	delete r->net;
	delete r->info; // owns the layer infos
	delete r->di;
	delete r;
}

// Node::setEdgeWeight / Layer::setBiasWeight for every edge; also clears pending deltas.
int ref_set_weights(void* h, const float* w, const float* bias)
{
	RefNet* r = (RefNet*)h;
	const int H = r->desc.n_layers - 2;
	size_t k = 0;
	for (int l = 0; l <= H; ++l)
	{
		glades::Layer* L = r->net->meat.layers[l];
		for (unsigned int o = 0; o < L->size(); ++o)
		{
			glades::Node* n = L->getNode(o);
			// A node can own more (or fewer) edges than its layer has inputs: when the weight builder
			// restarts (State/LayerBuilder.cpp:212-221) it keeps the previous fan-in.  The dense view
			// has exactly n_l weights per node; surplus edges are never read by the loop.
			for (unsigned int i = 0; i < (unsigned int)r->desc.sizes[l]; ++i)
			{
				n->setEdgeWeight(i, w[k++]);
				n->clearPrevDeltas(i);
			}
			n->clearErrDer();
		}
		if (l < H)
			L->setBiasWeight(bias ? bias[l] : 0.0f);
	}
	return 0;
}

int ref_get_weights(void* h, float* w, float* bias)
{
	RefNet* r = (RefNet*)h;
	const int H = r->desc.n_layers - 2;
	size_t k = 0;
	for (int l = 0; l <= H; ++l)
	{
		glades::Layer* L = r->net->meat.layers[l];
		for (unsigned int o = 0; o < L->size(); ++o)
		{
			glades::Node* n = L->getNode(o);
			for (unsigned int i = 0; i < (unsigned int)r->desc.sizes[l]; ++i)
				w[k++] = n->getEdgeWeight(i);  // 0 for an edge the node does not own
		}
		if (l < H && bias)
			bias[l] = L->getBiasWeight();
	}
	return 0;
}

// k-th pending delta of every edge (0 where the history is shorter).
int ref_get_pending_delta(void* h, int k, float* out)
{
	RefNet* r = (RefNet*)h;
	const int H = r->desc.n_layers - 2;
	size_t j = 0;
	for (int l = 0; l <= H; ++l)
	{
		glades::Layer* L = r->net->meat.layers[l];
		for (unsigned int o = 0; o < L->size(); ++o)
		{
			glades::Node* n = L->getNode(o);
			for (unsigned int i = 0; i < (unsigned int)r->desc.sizes[l]; ++i)
			{
				std::vector<float> pd = n->getPrevDeltas(i);
				out[j++] = (k < (int)pd.size()) ? pd[k] : 0.0f;
			}
		}
	}
	return 0;
}

static void fillMetrics(RefNet* r, gl_metrics* m)
{
	if (!m)
		return;
	memset(m, 0, sizeof *m);
	m->total_error = r->net->overallTotalError;
	m->total_accuracy = r->net->overallTotalAccuracy;
	m->class_accuracy = r->net->overallClassAccuracy;
	m->class_precision = r->net->overallClassPrecision;
	m->class_recall = r->net->overallClassRecall;
	m->class_specificity = r->net->overallClassSpecificity;
	m->class_f1 = r->net->overallClassF1;
	m->epochs = r->epochsDone;
	m->rows = r->di->getTrainSize();
}

// n epochs through the PUBLIC path NNetwork::train(DataInput*) (network.cpp:104-107): the
// terminator stops the loop when epochs % (n+1) == 0, with epochs preset to 1.
int ref_train_public(void* h, int n, gl_metrics* m)
{
	RefNet* r = (RefNet*)h;
	if (n < 1)
		return -1;
	r->net->epochs = 1;
	r->net->terminator.setEpoch(n + 1);
	{
		Quiet q;
		r->net->train(r->di);
	}
	r->epochsDone += n;
	fillMetrics(r, m);
	return 0;
}

// One pass through the PUBLIC path NNetwork::test(DataInput*) (network.cpp:109-112).
int ref_test_public(void* h, gl_metrics* m)
{
	RefNet* r = (RefNet*)h;
	r->net->epochs = 1;
	{
		Quiet q;
		r->net->test(r->di);
	}
	fillMetrics(r, m);
	return 0;
}

// One epoch driven row by row through the reference's private SGDHelper, restating only the
// epoch bookkeeping of run() (network.cpp:179-195,218-224), so that the confusion counts can
// be read before run() would clean them.  run_type: 0 train, 1 test.  confusion (may be NULL)
// receives n_out*n_out ints, [expected][predicted].  outputs (may be NULL) receives the
// per-row predictions [rows][n_out] taken from `results` (network.cpp:529-530).
int ref_epoch(void* h, int run_type, gl_metrics* m, int32_t* confusion, float* outputs)
{
	using namespace glades;
	RefNet* r = (RefNet*)h;
	NNetwork* net = r->net;
	const int nOut = r->info->getOutputLayerSize();
	const bool cls = (r->info->getOutputType() == GMath::CLASSIFICATION) || (r->info->getOutputType() == GMath::KL);
	Quiet q;
	net->di = r->di;
	net->minibatchSize = r->info->getBatchSize();
	if (cls && net->confusionMatrix.matrix.numberOfRows() == 0)
		net->confusionMatrix.build(nOut);
	net->overallTotalError = 0.0f;
	net->overallTotalAccuracy = 0.0f;
	if (cls)
		net->confusionMatrix.reset();
	const unsigned int rows = net->meat.getInputLayersSize();
	for (unsigned int row = 0; row < rows; ++row)
	{
		net->SGDHelper(row, run_type);
		if (outputs)
			for (int o = 0; o < nOut; ++o)
				outputs[(size_t)row * nOut + o] = net->results.getFloat(2 * o + 1);
	}
	++net->epochs;
	net->overallTotalAccuracy /= ((float)rows) * ((float)nOut);
	if (cls)
	{
		net->confusionMatrix.updateResultParams();
		net->overallClassAccuracy = net->confusionMatrix.getOverallAccuracy() * 100.0f;
		net->overallClassPrecision = net->confusionMatrix.getOverallPrecision() * 100.0f;
		net->overallClassRecall = net->confusionMatrix.getOverallRecall() * 100.0f;
		net->overallClassSpecificity = net->confusionMatrix.getOverallSpecificity() * 100.0f;
		net->overallClassF1 = net->confusionMatrix.getOverallF1Score() * 100.0f;
		if (confusion)
			for (int a = 0; a < nOut; ++a)
				for (int b = 0; b < nOut; ++b)
					confusion[a * nOut + b] = net->confusionMatrix.matrix.getCell(a, b).getInt();
	}
	if (run_type == 0)
		r->epochsDone += 1;
	fillMetrics(r, m);
	return 0;
}

// Forward pass of one row (SGDHelper with RUN_TEST); activations of all non-input layers,
// concatenated n_1 | ... | n_{H+1}, as Node::getWeight holds them afterwards (network.cpp:517).
int ref_forward_row(void* h, int64_t row, float* acts)
{
	RefNet* r = (RefNet*)h;
	const int H = r->desc.n_layers - 2;
	{
		Quiet q;
		r->net->di = r->di;
		r->net->SGDHelper((unsigned int)row, glades::NNetwork::RUN_TEST);
	}
	size_t k = 0;
	for (int l = 0; l <= H; ++l)
	{
		glades::Layer* L = r->net->meat.layers[l];
		for (unsigned int o = 0; o < L->size(); ++o)
			acts[k++] = L->getNode(o)->getWeight();
	}
	return 0;
}

// One training row (SGDHelper with RUN_TRAIN) -- step-level parity and timing.
int ref_train_row(void* h, int64_t row)
{
	RefNet* r = (RefNet*)h;
	Quiet q;
	r->net->di = r->di;
	r->net->minibatchSize = r->info->getBatchSize();
	if (r->net->confusionMatrix.matrix.numberOfRows() == 0 &&
	    r->info->getOutputType() != glades::GMath::REGRESSION)
		r->net->confusionMatrix.build(r->info->getOutputLayerSize());
	r->net->SGDHelper((unsigned int)row, glades::NNetwork::RUN_TRAIN);
	return 0;
}

// NumberInput::standardizeInputTable (DataObjects/NumberInput.cpp:43-285) with GMath/OHE.cpp, the
// reference's own code, on a typed raw table built from flat arrays and handed over through the shim's
// table registry (the reference reads it with its "file" constructor).
//   col_type[c]    0: float cells, 1: string cells (category k is the string "s<k>", k = (int)value),
//                  2: int cells
//   col_output[c]  1: the column is marked as an output column of the raw table
// x_out / y_out receive trainTable / trainExpectedTable row-major; their column counts come back in
// nx / ny (call with x_out == NULL first to size the buffers).  Returns the row count of trainTable.
int64_t ref_number_input(const float* values, int64_t rows, int cols, const int* col_type, const int* col_output,
                         int standardize_flag, float* x_out, int* nx, float* y_out, int* ny)
{
	std::vector<shmea::GString> headers;
	for (int c = 0; c < cols; ++c)
	{
		char h[32];
		snprintf(h, sizeof h, "col%d", c);
		headers.push_back(shmea::GString(h));
	}
	shmea::GTable raw(',', headers);
	for (int64_t r = 0; r < rows; ++r)
	{
		shmea::GList row;
		for (int c = 0; c < cols; ++c)
		{
			const float v = values[(size_t)r * cols + c];
			if (col_type[c] == 1)
			{
				char sbuf[32];
				snprintf(sbuf, sizeof sbuf, "s%d", (int)v);
				row.addString(sbuf);
			}
			else if (col_type[c] == 2)
				row.addInt((int)v);
			else
				row.addFloat(v);
		}
		raw.addRow(row);
	}
	for (int c = 0; c < cols; ++c)
		if (col_output[c])
			raw.toggleOutput(c);
	shmea::shimRegisterTable("oracle-raw-table", raw);
	glades::NumberInput in;
	{
		Quiet q;
		in.standardizeInputTable(shmea::GString("oracle-raw-table"), standardize_flag);
	}
	const int cx = (int)in.trainTable.numberOfCols(), cy = (int)in.trainExpectedTable.numberOfCols();
	if (nx) *nx = cx;
	if (ny) *ny = cy;
	const int64_t outRows = in.trainTable.numberOfRows();
	if (x_out)
		for (int64_t r = 0; r < outRows; ++r)
			for (int c = 0; c < cx; ++c)
				x_out[(size_t)r * cx + c] = in.trainTable.getCell(r, c).getFloat();
	if (y_out)
		for (int64_t r = 0; r < (int64_t)in.trainExpectedTable.numberOfRows(); ++r)
			for (int c = 0; c < cy; ++c)
				y_out[(size_t)r * cy + c] = in.trainExpectedTable.getCell(r, c).getFloat();
	for (unsigned int c = 0; c < in.OHEMaps.size(); ++c)
		delete in.OHEMaps[c];
	return outRows;
}

// NNetwork::train() with a server and a connection attached: the reference then streams its GUI messages
// (Networks/network.cpp:258-357) through GNet::GServer::send, which the shim records.  The terminator is set
// to `epochs`; below 10 epochs every epoch sends (the 60 Hz throttle starts at epoch 10, network.cpp:264).
// The messages come back flattened into `out` (at most `cap` doubles; the needed count is returned):
//   per message: kind id (0 PROGRESSIVE, 1 ACTIVATIONS, 2 WEIGHTS, 3 ACC, 4 CONF, -1 other), number of
//   extra arguments, the arguments, payload rows, payload columns (0, 0 for a list), payload length, payload.
// A string cell of a payload (the ',' and ';' separators) is 1e9 + its character code.
int64_t ref_train_gui(void* h, int epochs, double* out, int64_t cap)
{
	RefNet* r = (RefNet*)h;
	shmea::shimClearMessages();
	{
		Quiet q;
		r->net->setServer((GNet::GServer*)0x10, (GNet::Connection*)0x10);
		r->net->terminator.setEpoch(r->net->epochs - 1 + epochs);  // run() starts from epochs = 1 (see ref_create)
		r->net->train(r->di);
		r->net->setServer(NULL, NULL);
	}
	static const char* kinds[] = {"PROGRESSIVE", "ACTIVATIONS", "WEIGHTS", "ACC", "CONF"};
	int64_t k = 0;
	for (size_t i = 0; i < shmea::shimMessageCount(); ++i)
	{
		const shmea::ShimMessage& m = shmea::shimMessage(i);
		double id = -1;
		for (int t = 0; t < 5; ++t)
			if (m.kind == kinds[t])
				id = t;
		std::vector<double> rec;
		rec.push_back(id);
		rec.push_back((double)m.args.size());
		rec.insert(rec.end(), m.args.begin(), m.args.end());
		rec.push_back(m.rows);
		rec.push_back(m.cols);
		rec.push_back((double)m.payload.size());
		rec.insert(rec.end(), m.payload.begin(), m.payload.end());
		for (size_t j = 0; j < rec.size(); ++j, ++k)
			if (out && k < cap)
				out[k] = rec[j];
	}
	return k;
}

// Scalar functions of GMath, for known-answer tables.
float ref_squash(float z, int act, float p) { return glades::GMath::squash(z, act, p); }
float ref_act_der(float a, int act, float p) { return glades::GMath::activationErrDer(a, act, p); }
float ref_cost(float e, float p, float n, int fx) { return glades::GMath::outputNodeCost(e, p, n, fx); }
float ref_cost_der(float e, float p, int fx) { return glades::GMath::costErrDer(e, p, fx); }

} // extern "C"
