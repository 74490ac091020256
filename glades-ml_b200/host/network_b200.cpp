// Host-side mirror of the reference's feed-forward interface over the C ABI (see glades_b200.hpp).
// NNetwork::run follows Networks/network.cpp:114-397: the same guards with silent returns, the same
// printf lines, build-once on the first call, per-epoch statistics, Terminator check, one pass for
// RUN_TEST.  The per-row work (SGDHelper) is one C-ABI call per epoch.
#include "glades_b200.hpp"

#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

namespace glades_b200 {

// ---------------------------------------------------------------------------------------------
ArrayInput::ArrayInput(const float* nx, const float* ny, unsigned int r, unsigned int ni, unsigned int no)
    : x(nx, nx + (size_t)r * ni), y(ny, ny + (size_t)r * no), rows(r), nIn(ni), nOut(no)
{
}
shmea::GList ArrayInput::getTrainRow(unsigned int r) const
{
	shmea::GList l;
	if (r < rows)
		for (unsigned int c = 0; c < nIn; ++c) l.addFloat(x[(size_t)r * nIn + c]);
	return l;
}
shmea::GList ArrayInput::getTrainExpectedRow(unsigned int r) const
{
	shmea::GList l;
	if (r < rows)
		for (unsigned int c = 0; c < nOut; ++c) l.addFloat(y[(size_t)r * nOut + c]);
	return l;
}

InputLayerInfo::InputLayerInfo(int newBatchSize, float lr, float mom, float wd1, float wd2, float pDrop, int act,
                               float actParam)
    : LayerInfo(0), batchSize(newBatchSize)
{
	learningRate = lr;
	momentumFactor = mom;
	weightDecay1 = wd1;
	weightDecay2 = wd2;
	pDropout = pDrop;
	activationType = act;
	activationParam = actParam;
}
HiddenLayerInfo::HiddenLayerInfo(int newSize, float lr, float mom, float wd1, float wd2, float pDrop, int act,
                                 float actParam)
    : LayerInfo(newSize)
{
	learningRate = lr;
	momentumFactor = mom;
	weightDecay1 = wd1;
	weightDecay2 = wd2;
	pDropout = pDrop;
	activationType = act;
	activationParam = actParam;
}

NNInfo::NNInfo(const std::string& newName, InputLayerInfo* in, const std::vector<HiddenLayerInfo*>& hidden,
               OutputLayerInfo* out)
    : name(newName), inputLayer(in), outputLayer(out), layers(hidden)
{
}
NNInfo::~NNInfo()
{
	for (size_t i = 0; i < layers.size(); ++i) delete layers[i];
	delete inputLayer;
	delete outputLayer;
}
int NNInfo::getOutputType() const { return outputLayer ? outputLayer->getOutputType() : OutputLayerInfo::REGRESSION; }
float NNInfo::getPInput() const { return inputLayer ? inputLayer->getPDropout() : 0.0f; }
int NNInfo::getBatchSize() const { return inputLayer ? inputLayer->getBatchSize() : 1; }
int NNInfo::getHiddenLayerSize(unsigned int i) const { return i < layers.size() && layers[i] ? (int)layers[i]->size() : 0; }
unsigned int NNInfo::getOutputLayerSize() const { return outputLayer ? outputLayer->size() : 0; }

// One accessor shape for all per-layer getters: index past the end -> the reference's default,
// index 0 -> the input layer's info, else hidden layer index-1 (nninfo.cpp:240-373).
#define GLB_GETTER(NAME, TYPE, DEFAULT, INPUT_EXPR, HIDDEN_EXPR) \
	TYPE NNInfo::NAME(unsigned int index) const                  \
	{                                                            \
		if (index > layers.size()) return DEFAULT;               \
		if (index == 0) return inputLayer->INPUT_EXPR;           \
		if (!layers[index - 1]) return DEFAULT;                  \
		return layers[index - 1]->HIDDEN_EXPR;                   \
	}
GLB_GETTER(getLearningRate, float, 0.01f, getLearningRate(), getLearningRate())
GLB_GETTER(getMomentumFactor, float, 0.0f, getMomentumFactor(), getMomentumFactor())
GLB_GETTER(getWeightDecay1, float, 0.0f, getWeightDecay1(), getWeightDecay1())
// index 0 hands back weightDecay1, as the reference does (nninfo.cpp:305-306)
GLB_GETTER(getWeightDecay2, float, 0.0f, getWeightDecay1(), getWeightDecay2())
GLB_GETTER(getPDropout, float, 1.0f, getPDropout(), getPDropout())
GLB_GETTER(getActivationType, int, 0, getActivationType(), getActivationType())
GLB_GETTER(getActivationParam, float, 0.0f, getActivationParam(), getActivationParam())
#undef GLB_GETTER

bool Terminator::triggered(int64_t cTimestamp, int64_t cEpoch, float cAccuracy) const
{
	if (timestamp > 0 && cTimestamp % timestamp == 0) return true;
	if (epoch > 0 && cEpoch % epoch == 0) return true;
	if (accuracy > 0.0f && cAccuracy >= accuracy) return true;
	return false;
}

bool packDescriptor(const NNInfo& info, unsigned int featureCount, int mode, gl_net_desc* d)
{
	memset(d, 0, sizeof *d);
	const int H = info.numHiddenLayers();
	if (H < 1 || H + 1 > GL_MAX_WEIGHT_LAYERS) return false;
	d->n_layers = H + 2;
	d->sizes[0] = (int)featureCount;
	for (int l = 1; l <= H; ++l) d->sizes[l] = info.getHiddenLayerSize(l - 1);
	d->sizes[H + 1] = (int)info.getOutputLayerSize();
	for (int l = 0; l <= H; ++l)
	{
		d->lr[l] = info.getLearningRate(l);
		d->momentum[l] = info.getMomentumFactor(l);
		d->wd1[l] = info.getWeightDecay1(l);
		d->wd2[l] = info.getWeightDecay2(l);
		d->activation[l] = info.getActivationType(l);
		d->act_param[l] = info.getActivationParam(l);
	}
	// SGDHelper hands scrambleDropout getPInput() and getPDropout(0..H-1) (network.cpp:405-411)
	d->p_dropout[0] = info.getPInput();
	for (int l = 1; l <= H; ++l) d->p_dropout[l] = info.getPDropout(l - 1);
	d->output_type = info.getOutputType();
	d->batch_size = info.getBatchSize();
	d->mode = mode;
	d->bias_rule = GL_BIAS_MEAN;
	d->gemm = GL_GEMM_AUTO;
	d->device = 0;
	return true;
}

// ---------------------------------------------------------------------------------------------
// Weight draw.  Inverse normal CDF: P. J. Acklam's rational approximation (the algorithm the
// reference cites at GMath/gmath.cpp:355-405), evaluated in double on float-typed inputs exactly as
// the reference's expression types make it: logf / sqrtf on the float argument, the rational
// functions in double.
static float normInvCdf(float x)
{
	static const double A[6] = {-39.69683028665376, 220.9460984245205, -275.9285104469687,
	                            138.3577518672690, -30.66479806614716, 2.506628277459239};
	static const double B[5] = {-54.47609879822406, 161.5858368580409, -155.6989798598866, 66.80131188771972,
	                            -13.280681552885721};
	static const double Cc[6] = {-0.007784894002430293, -0.3223964580411365, -2.400758277161838,
	                             -2.549732539343734, 4.374664141464968, 2.938163982698783};
	static const double D[4] = {0.007784695709041462, 0.3224671290700398, 2.445134137142996, 3.754408661907416};
	const float pLow = 0.02452f;
	const float pHigh = 1 - pLow;
	if (x < pLow || !(x < pHigh))
	{
		const bool lower = x < pLow;
		const double q = sqrtf(-2 * logf(lower ? x : 1 - x));
		double num = Cc[0], den = D[0];
		for (int i = 1; i < 6; ++i) num = num * q + Cc[i];
		for (int i = 1; i < 4; ++i) den = den * q + D[i];
		den = den * q + 1;
		return lower ? (float)(num / den) : (float)(-num / den);
	}
	const double q = x - 0.5;
	const double r = q * q;
	double num = A[0], den = B[0];
	for (int i = 1; i < 6; ++i) num = num * r + A[i];
	for (int i = 1; i < 5; ++i) den = den * r + B[i];
	den = den * r + 1;
	return (float)((num * q) / den);
}

static float normalPdf(float z)
{
	return (float)((1 / sqrt(6.2831853)) * expf(-(z * z) / 2));
}

static void drawNode(unsigned int fanIn, const float* zigg, int activationType, float* out)
{
	const float stdDev = (activationType != GMath::RELU) ? sqrtf(1 / (float)fanIn) : sqrtf(2 / (float)fanIn);
	for (unsigned int e = 0; e < fanIn; ++e)
	{
		float x = 0.0f;
		for (;;)
		{
			const int strip = rand() % 2048;
			x = rand() / (RAND_MAX / zigg[strip]);
			if (strip == 0) continue;  // the tail strip is never sampled
			if (x < zigg[strip + 1]) break;
			if (x > zigg[strip + 1])
			{
				const float u = rand() / RAND_MAX;  // integer division, as in the reference
				const float y = normalPdf(zigg[strip]) + u * (normalPdf(zigg[strip - 1] - normalPdf(zigg[strip])));
				if (y < normalPdf(x)) break;
			}
		}
		out[e] = x * stdDev;
	}
}

void drawInitialWeights(const NNInfo& info, unsigned int featureCount, std::vector<float>& w)
{
	// strip table of Layer::initWeights (layer.cpp:199-211), rebuilt per layer there, identical each time
	std::vector<float> zigg(2049);
	float cdf = 1.0;
	for (unsigned int i = 1; i < 2048; ++i)
	{
		cdf = cdf - (1 / ((float)2048 * 2));
		zigg[i] = normInvCdf(cdf);
	}
	zigg[0] = zigg[1];
	zigg[2048] = 0;

	const int H = info.numHiddenLayers();
	const int outputType = info.getOutputType();
	// LayerBuilder::buildHiddenLayers (LayerBuilder.cpp:192-234): the first layer whose activation is
	// SIGMOID / RELU / LEAKY (or any layer of a classification net) makes the builder throw away what
	// it has drawn and start again from layer 0 -- the discarded draws still consumed rand().
	// On that restart the builder does NOT reset its running fan-in, so the re-drawn first layer gets
	// as many edges per node as the layer before the restart point had nodes; the loop only ever
	// reads the first n_in of them (a missing edge reads as weight 0, State/node.cpp getEdgeWeight).
	std::vector<std::vector<float> > hidden;
	bool isPositive = false;
	int prev = (int)featureCount;
	for (int i = 0; i < H; ++i)
	{
		const int act = info.getActivationType(i);
		const int n = info.getHiddenLayerSize(i);
		if (!isPositive && (act == GMath::SIGMOID || act == GMath::RELU || act == GMath::LEAKY ||
		                    outputType == GMath::CLASSIFICATION))
		{
			isPositive = true;
			hidden.clear();
			i = -1;
			continue;
		}
		const int trueFanIn = (i == 0) ? (int)featureCount : info.getHiddenLayerSize(i - 1);
		std::vector<float> layer((size_t)n * trueFanIn, 0.0f);
		std::vector<float> drawn(prev);
		for (int o = 0; o < n; ++o)
		{
			drawNode(prev, &zigg[0], act, &drawn[0]);
			for (int e = 0; e < trueFanIn && e < prev; ++e) layer[(size_t)o * trueFanIn + e] = drawn[e];
		}
		hidden.push_back(layer);
		prev = n;
	}
	// LayerBuilder::buildOutputLayer (LayerBuilder.cpp:236-267) scales by the activation type of the
	// LAST index its loop visited, i.e. NNInfo index H-1.
	const int outAct = H > 0 ? info.getActivationType(H - 1) : 0;
	const int nOut = (int)info.getOutputLayerSize();
	std::vector<float> outLayer((size_t)nOut * prev);
	for (int o = 0; o < nOut; ++o) drawNode(prev, &zigg[0], outAct, &outLayer[(size_t)o * prev]);
	w.clear();
	for (size_t l = 0; l < hidden.size(); ++l) w.insert(w.end(), hidden[l].begin(), hidden[l].end());
	w.insert(w.end(), outLayer.begin(), outLayer.end());
}

// ---------------------------------------------------------------------------------------------
NNetwork::NNetwork()
    : di(NULL), skeleton(NULL), handle(NULL), running(false), epochs(0), overallTotalError(0.0f),
      overallTotalAccuracy(0.0f), overallClassAccuracy(0.0f), overallClassPrecision(0.0f), overallClassRecall(0.0f),
      overallClassSpecificity(0.0f), overallClassF1(0.0f), minibatchSize(1), mode(GL_MODE_REFERENCE), deviceOrdinal(0),
      quiet(false), haveInit(false), serverInstance(NULL), cConnection(NULL), firstRunActivation(false), ownsSkeleton(false)
{
	const char* m = getenv("GLADES_B200_MODE");
	if (m && strcmp(m, "batched") == 0) mode = GL_MODE_BATCHED;
}

NNetwork::NNetwork(NNInfo* newNNInfo)
    : di(NULL), skeleton(NULL), handle(NULL), running(false), epochs(0), overallTotalError(0.0f),
      overallTotalAccuracy(0.0f), overallClassAccuracy(0.0f), overallClassPrecision(0.0f), overallClassRecall(0.0f),
      overallClassSpecificity(0.0f), overallClassF1(0.0f), minibatchSize(1), mode(GL_MODE_REFERENCE), deviceOrdinal(0),
      quiet(false), haveInit(false), serverInstance(NULL), cConnection(NULL), firstRunActivation(false), ownsSkeleton(false)
{
	const char* m = getenv("GLADES_B200_MODE");
	if (m && strcmp(m, "batched") == 0) mode = GL_MODE_BATCHED;
	if (!newNNInfo) return;
	skeleton = newNNInfo;
	minibatchSize = skeleton->getBatchSize();
}

NNetwork::~NNetwork()
{
	if (handle) gl_destroy(handle);
	if (ownsSkeleton) delete skeleton;
}

int64_t NNetwork::getCurrentTimeMilliseconds() const
{
	struct timespec ts;
	clock_gettime(CLOCK_REALTIME, &ts);
	return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

void NNetwork::setServer(GNet::GServer* newServer, GNet::Connection* newConnection)
{
	serverInstance = newServer;
	cConnection = newConnection;
}

// NNetwork::load / save (network.cpp:701-722): the skeleton only.
bool NNetwork::load(const std::string& netName, const std::string& directory)
{
	NNInfo* info = NNInfo::load(netName, directory);
	if (!info) return false;
	if (ownsSkeleton) delete skeleton;
	skeleton = info;
	ownsSkeleton = true;
	minibatchSize = skeleton->getBatchSize();
	return true;
}

bool NNetwork::save(const std::string& directory) const
{
	if (!skeleton) return false;
	return skeleton->save(directory);
}

// ---- live view -------------------------------------------------------------------------------
// After an epoch whose frame is due, queueFrame() notes the epoch's figures and queues an asynchronous
// snapshot of the weights and the last row's pre-activations (gl_snapshot_submit: training only waits for a
// device-to-device copy).  The frame is sent when the snapshot has reached host memory -- at the next due
// frame or at the end of the run -- so the copy to the host runs under the following epochs.
void NNetwork::queueFrame()
{
	if (frame.pending) sendFrame();
	if (gl_snapshot_submit(handle) != GL_OK)
	{
		fprintf(stderr, "[NN] %s\n", gl_last_error());
		return;
	}
	frame.pending = true;
	frame.epochs = epochs;
	frame.error = overallTotalError;
	frame.accuracy = overallTotalAccuracy;
	frame.confusion = lastConfusion;
	// CMatrix::getOverallFalseAlarm / getOverallRecall (GMath/cmatrix.cpp:178-243), as fractions
	const int c = (int)skeleton->getOutputLayerSize();
	float fa = 0.0f, rec = 0.0f;
	if ((int)lastConfusion.size() == c * c)
		for (int k = 0; k < c; ++k)
		{
			int tp = lastConfusion[(size_t)k * c + k], tn = 0, fp = 0, fn = 0;
			for (int j = 0; j < c; ++j)
				if (j != k)
				{
					tn += lastConfusion[(size_t)j * c + j];
					fp += lastConfusion[(size_t)j * c + k];
					fn += lastConfusion[(size_t)k * c + j];
				}
			fa += ((float)fp) / ((float)(tn + fp));
			rec += ((float)tp) / ((float)(tp + fn));
		}
	frame.falseAlarm = fa / (float)c;
	frame.recall = rec / (float)c;
}

void NNetwork::sendFrame()
{
	if (!frame.pending) return;
	frame.pending = false;
	const int H = skeleton->numHiddenLayers();
	std::vector<int> sizes;
	sizes.push_back((int)di->getFeatureCount());
	for (int l = 0; l < H; ++l) sizes.push_back(skeleton->getHiddenLayerSize(l));
	sizes.push_back((int)skeleton->getOutputLayerSize());
	size_t nw = 0, nz = 0;
	for (int l = 0; l <= H; ++l)
	{
		nw += (size_t)sizes[l] * sizes[l + 1];
		nz += sizes[l + 1];
	}
	std::vector<float> w(nw), z(nz);
	if (gl_snapshot_collect(handle, &w[0], NULL, &z[0], 1) != GL_OK)
	{
		fprintf(stderr, "[NN] %s\n", gl_last_error());
		return;
	}
	if (!serverInstance || !cConnection) return;
	const bool classify = skeleton->getOutputType() == GMath::CLASSIFICATION || skeleton->getOutputType() == GMath::KL;
	if (frame.epochs > 0)
	{
		// the learning curve: (epochs - 1, error)
		shmea::GList wData, argData;
		wData.addInt(frame.epochs - 1);
		wData.addFloat(frame.error);
		argData.addString("PROGRESSIVE");
		shmea::ServiceData* cData = new shmea::ServiceData(cConnection, "GUI_Callback");
		cData->set(wData);
		cData->setArgList(argData);
		serverInstance->send(cData);
		// the layer sizes on the first frame of a run, then the last row's pre-activations, ',' after every layer
		argData.clear();
		argData.addString("ACTIVATIONS");
		cData = new shmea::ServiceData(cConnection, "GUI_Callback");
		shmea::GList act;
		if (!firstRunActivation)
		{
			firstRunActivation = true;
			for (size_t l = 0; l < sizes.size(); ++l) act.addInt(sizes[l]);
		}
		else
		{
			size_t k = 0;
			for (int l = 1; l <= H + 1; ++l)
			{
				for (int o = 0; o < sizes[l]; ++o) act.addFloat(z[k++]);
				act.addString(",");
			}
		}
		cData->set(act);
		cData->setArgList(argData);
		serverInstance->send(cData);
		// every weight, node by node (',' after a node's edges), layer by layer (';' after a layer)
		argData.clear();
		argData.addString("WEIGHTS");
		shmea::GList wl;
		size_t k = 0;
		for (int l = 0; l <= H; ++l)
		{
			for (int o = 0; o < sizes[l + 1]; ++o)
			{
				for (int i = 0; i < sizes[l]; ++i) wl.addFloat(w[k++]);
				wl.addString(",");
			}
			wl.addString(";");
		}
		cData = new shmea::ServiceData(cConnection, "GUI_Callback");
		cData->set(wl);
		cData->setArgList(argData);
		serverInstance->send(cData);
	}
	{
		shmea::GList argData, wData;
		argData.addString("ACC");
		wData.addInt(frame.epochs);
		wData.addFloat(frame.accuracy);
		shmea::ServiceData* cData = new shmea::ServiceData(cConnection, "GUI_Callback");
		cData->set(wData);
		cData->setArgList(argData);
		serverInstance->send(cData);
	}
	if (classify)
	{
		shmea::GList argData;
		argData.addString("CONF");
		argData.addFloat(frame.falseAlarm);
		argData.addFloat(frame.recall);
		shmea::ServiceData* cData = new shmea::ServiceData(cConnection, "GUI_Callback");
		const int c = (int)skeleton->getOutputLayerSize();
		cData->setTable(frame.confusion, c, c);
		cData->setArgList(argData);
		serverInstance->send(cData);
	}
}

void NNetwork::stop()
{
	running = false;
	if (handle) gl_stop(handle);
}

void NNetwork::train(DataInput* newDataInput) { run(newDataInput, RUN_TRAIN); }
void NNetwork::test(DataInput* newDataInput) { run(newDataInput, RUN_TEST); }

void NNetwork::setWeights(const std::vector<float>& w, const std::vector<float>& bias)
{
	initW = w;
	initB = bias;
	haveInit = true;
	if (handle && gl_set_weights(handle, &initW[0], initB.empty() ? NULL : &initB[0]) != GL_OK)
		fprintf(stderr, "[NN] %s\n", gl_last_error());
}

bool NNetwork::getWeights(std::vector<float>& w, std::vector<float>& bias) const
{
	if (!handle) return false;
	w.resize((size_t)gl_weight_count(handle));
	bias.resize(skeleton->numHiddenLayers());
	return gl_get_weights(handle, &w[0], bias.empty() ? NULL : &bias[0]) == GL_OK;
}

bool NNetwork::saveState(const std::string& path) const
{
	if (!handle) return false;
	if (gl_save_state(handle, path.c_str()) == GL_OK) return true;
	fprintf(stderr, "[NN] %s\n", gl_last_error());
	return false;
}

bool NNetwork::loadState(const std::string& path)
{
	if (!handle)
	{
		pendingState = path;  // applied by build()
		return true;
	}
	if (gl_load_state(handle, path.c_str()) != GL_OK)
	{
		fprintf(stderr, "[NN] %s\n", gl_last_error());
		return false;
	}
	epochs = gl_get_epochs(handle);
	return true;
}

// What meat.build() did on the first run (network.cpp:127-128): pack the rows and create the
// device network.  Every failure is the reference's silent return, plus one line on stderr.
bool NNetwork::build(DataInput* d)
{
	gl_net_desc desc;
	if (!packDescriptor(*skeleton, d->getFeatureCount(), mode, &desc))
	{
		fprintf(stderr, "[NN] %s: skeleton cannot be expressed on the device path\n", skeleton->getName().c_str());
		return false;
	}
	desc.device = deviceOrdinal;
	const unsigned int rows = d->getTrainSize(), nIn = d->getFeatureCount(), nOut = skeleton->getOutputLayerSize();
	// rows that already lie in device memory (a NumberInput standardised on the GPU) are used where they are
	const float *devX = NULL, *devY = NULL;
	int devOrdinal = 0;
	const bool onDevice = d->deviceRows(&devX, &devY, &devOrdinal) && devX && devY && devOrdinal == deviceOrdinal;
	std::vector<float> x, y;
	if (!onDevice)
	{
		x.resize((size_t)rows * nIn);
		y.resize((size_t)rows * nOut);
		for (unsigned int r = 0; r < rows; ++r)
		{
			// one row copy per row (the reference copies the whole row per cell, LayerBuilder.cpp:139)
			const shmea::GList xr = d->getTrainRow(r);
			const shmea::GList yr = d->getTrainExpectedRow(r);
			for (unsigned int c = 0; c < nIn; ++c) x[(size_t)r * nIn + c] = xr.getFloat(c);
			for (unsigned int c = 0; c < nOut; ++c) y[(size_t)r * nOut + c] = yr.getFloat(c);
		}
	}
	if (gl_create(&desc, &handle) != GL_OK)
	{
		fprintf(stderr, "[NN] %s\n", gl_last_error());
		handle = NULL;
		return false;
	}
	if (!haveInit)
	{
		drawInitialWeights(*skeleton, nIn, initW);
		initB.assign(skeleton->numHiddenLayers(), 0.0f);
		haveInit = true;
	}
	if ((int64_t)initW.size() != gl_weight_count(handle) ||
	    gl_set_weights(handle, &initW[0], initB.empty() ? NULL : &initB[0]) != GL_OK ||
	    (onDevice ? gl_set_data_device(handle, devX, devY, rows) : gl_set_data(handle, &x[0], &y[0], rows)) != GL_OK)
	{
		fprintf(stderr, "[NN] %s\n", (int64_t)initW.size() != gl_weight_count(handle) ? "weight vector has the wrong length" : gl_last_error());
		gl_destroy(handle);
		handle = NULL;
		return false;
	}
	if (!pendingState.empty())
	{
		const std::string path = pendingState;
		pendingState.clear();
		if (!loadState(path))
		{
			gl_destroy(handle);
			handle = NULL;
			return false;
		}
	}
	return true;
}

void NNetwork::run(DataInput* newDataInput, int runType)
{
	if (!skeleton) return;
	if (!newDataInput) return;
	di = newDataInput;
	if ((di->getTrainSize() <= 0) || (di->getFeatureCount() <= 0)) return;
	if (epochs == 0 && !handle)
	{
		if (!build(di)) return;
	}
	if (!handle) return;
	minibatchSize = skeleton->getBatchSize();
	const int outputType = skeleton->getOutputType();
	const bool classify = (outputType == GMath::CLASSIFICATION) || (outputType == GMath::KL);
	const unsigned int nOut = skeleton->getOutputLayerSize();
	const unsigned int rows = di->getTrainSize();

	if (!quiet)
	{
		if (runType == RUN_TRAIN) printf("[NN] Training...\n");
		else if (runType == RUN_TEST) printf("[NN] Testing...\n");
		if (runType == RUN_TRAIN)
		{
			if (outputType == GMath::REGRESSION) printf("[NN] Epochs\tAccuracy\n");
			if (classify) printf("[NN] Epochs\tAccuracy\tPrecision\tRecall\t\tSpecificity\tF1 Score\n");
		}
	}
	running = true;
	firstRunActivation = false;
	learningCurve.clear();  // resetGraphs(), network.cpp:168,761-768
	int64_t lastUpdateTime = 0;
	std::vector<float> lastOut(nOut);
	while (running)
	{
		gl_metrics m;
		int st;
		if (runType == RUN_TRAIN) st = gl_train_epochs(handle, 1, &m);
		else st = gl_forward(handle, 0, rows, NULL, NULL, &m);
		if (st != GL_OK)
		{
			fprintf(stderr, "[NN] %s\n", gl_last_error());
			break;
		}
		++epochs;  // the reference counts test passes too (network.cpp:193)
		overallTotalError = m.total_error;
		overallTotalAccuracy = m.total_accuracy;
		if (outputType == GMath::REGRESSION)
		{
			if (runType == RUN_TRAIN && !quiet)
			{
				printf("\33[2K[NN] %d\t%f%%\r", epochs, overallTotalAccuracy);
				fflush(stdout);
			}
		}
		else if (classify)
		{
			overallClassAccuracy = m.class_accuracy;
			overallClassPrecision = m.class_precision;
			overallClassRecall = m.class_recall;
			overallClassSpecificity = m.class_specificity;
			overallClassF1 = m.class_f1;
			lastConfusion.resize((size_t)nOut * nOut);
			gl_get_confusion(handle, &lastConfusion[0]);
			if (runType == RUN_TRAIN && !quiet)
			{
				printf(epochs < 100 ? "\33[2K[NN] %d\t\t%f%%\t%f%%\t%f%%\t%f%%\t%f%%\r"
				                    : "\33[2K[NN] %d\t%f%%\t%f%%\t%f%%\t%f%%\t%f%%\r",
				       epochs, overallClassAccuracy, overallClassPrecision, overallClassRecall, overallClassSpecificity,
				       overallClassF1);
				fflush(stdout);
			}
		}
		if (runType == RUN_TRAIN)
		{
			if (epochs > 0)
			{
				learningCurve.addInt(epochs - 1);
				learningCurve.addFloat(overallTotalError);
			}
			// the live view: every epoch below 10, then at most every 16 ms (network.cpp:262-264)
			const int64_t ms = getCurrentTimeMilliseconds();
			if (serverInstance && cConnection && (epochs < 10 || ms - lastUpdateTime > 16))
			{
				queueFrame();
				lastUpdateTime = ms;
			}
		}
		if (terminator.triggered(time(NULL), epochs, overallTotalAccuracy)) break;
		if (runType == RUN_TEST) break;
	}
	sendFrame();  // the frame still in flight, if any
	// `results` holds the last row's (expected, predicted) pairs, as after the reference's last
	// SGDHelper call (network.cpp:529-530)
	results.clear();
	if (handle && rows > 0 && gl_get_last_outputs(handle, &lastOut[0]) == GL_OK)
	{
		const shmea::GList yr = di->getTrainExpectedRow(rows - 1);
		for (unsigned int o = 0; o < nOut; ++o)
		{
			results.addFloat(yr.getFloat(o));
			results.addFloat(lastOut[o]);
		}
	}
	if (!quiet)
	{
		if (runType == RUN_TRAIN) printf("\n");
		else if (runType == RUN_TEST) printf("[NN] %s Accuracy: %f%%\n", skeleton->getName().c_str(), overallTotalAccuracy);
		printf("\n");
	}
	running = false;
}

// ---------------------------------------------------------------------------------------------
MetaNetwork::MetaNetwork(const std::string& newName) : name(newName), collectionType(ONE_TO_ONE) {}

MetaNetwork::MetaNetwork(NNInfo* networkInfo, int subnetCount) : collectionType(subnetCount > 1 ? ONE_TO_MANY : ONE_TO_ONE)
{
	if (networkInfo) name = networkInfo->getName();
	for (int i = 0; i < subnetCount; ++i) addSubnet(networkInfo);
}

MetaNetwork::~MetaNetwork()
{
	name = "";
	clearSubnets();  // like the reference, the collection does not delete its networks (metanetwork.cpp:78-82,147-150)
}

void MetaNetwork::addSubnet(NNInfo* networkInfo)
{
	if (!networkInfo) return;
	subnets.push_back(new NNetwork(networkInfo));
}

void MetaNetwork::addSubnet(NNetwork* cNetwork)
{
	if (!cNetwork) return;
	subnets.push_back(cNetwork);
}

NNetwork* MetaNetwork::getSubnet(unsigned int index) { return index < subnets.size() ? subnets[index] : NULL; }

std::string MetaNetwork::getSubnetName(unsigned int index) const
{
	return index < subnets.size() ? subnets[index]->getName() : std::string();
}

NNetwork* MetaNetwork::getSubnetByName(const std::string& newName) const
{
	for (size_t i = 0; i < subnets.size(); ++i)
		if (subnets[i]->getName() == newName) return subnets[i];
	return NULL;
}

namespace {
struct ReplicaJob
{
	std::vector<NNetwork*> nets;
	DataInput* di;
};
void* replicaThread(void* p)
{
	ReplicaJob* job = static_cast<ReplicaJob*>(p);
	for (size_t i = 0; i < job->nets.size(); ++i) job->nets[i]->train(job->di);
	return NULL;
}
}  // namespace

int MetaNetwork::trainReplicas(DataInput* newDataInput)
{
	if (!newDataInput || subnets.empty()) return 0;
	int gpus = gl_device_count();
	if (gpus < 1) gpus = 1;
	if (gpus > (int)subnets.size()) gpus = (int)subnets.size();
	// subnet i runs on GPU i % gpus; one host thread drives each GPU's networks one after the other (a
	// handle belongs to one host thread at a time, distinct handles may run from distinct threads)
	std::vector<ReplicaJob> jobs((size_t)gpus);
	for (size_t i = 0; i < subnets.size(); ++i)
	{
		subnets[i]->setDevice((int)(i % (size_t)gpus));
		jobs[i % (size_t)gpus].nets.push_back(subnets[i]);
		jobs[i % (size_t)gpus].di = newDataInput;
	}
	std::vector<pthread_t> threads((size_t)gpus);
	for (int g = 0; g < gpus; ++g) pthread_create(&threads[(size_t)g], NULL, replicaThread, &jobs[(size_t)g]);
	for (int g = 0; g < gpus; ++g) pthread_join(threads[(size_t)g], NULL);
	return gpus;
}

// glades::train / glades::test, main.cpp:82-243
static MetaNetwork* runAll(MetaNetwork* meta, DataInput* di, GNet::GServer* server, GNet::Connection* connection, bool training)
{
	const std::vector<NNetwork*> subnets = meta->getSubnets();
	for (size_t i = 0; i < subnets.size(); ++i)
	{
		if (server && connection) subnets[i]->setServer(server, connection);
		if (training) subnets[i]->train(di);
		else subnets[i]->test(di);
	}
	return meta;
}

MetaNetwork* train(NNInfo* networkInfo, DataInput* di, GNet::GServer* server, GNet::Connection* connection)
{
	if (!networkInfo) return NULL;
	MetaNetwork* meta = new MetaNetwork(networkInfo->getName());
	meta->addSubnet(networkInfo);
	return runAll(meta, di, server, connection, true);
}
MetaNetwork* train(NNetwork* cNetwork, DataInput* di, GNet::GServer* server, GNet::Connection* connection)
{
	if (!cNetwork) return NULL;
	MetaNetwork* meta = new MetaNetwork(cNetwork->getName());
	meta->addSubnet(cNetwork);
	return runAll(meta, di, server, connection, true);
}
MetaNetwork* train(MetaNetwork* meta, DataInput* di, GNet::GServer* server, GNet::Connection* connection)
{
	if (!meta) return NULL;
	return runAll(meta, di, server, connection, true);
}
MetaNetwork* test(NNInfo* networkInfo, DataInput* di, GNet::GServer* server, GNet::Connection* connection)
{
	if (!networkInfo) return NULL;
	MetaNetwork* meta = new MetaNetwork(networkInfo->getName());
	meta->addSubnet(networkInfo);
	return runAll(meta, di, server, connection, false);
}
MetaNetwork* test(NNetwork* cNetwork, DataInput* di, GNet::GServer* server, GNet::Connection* connection)
{
	if (!cNetwork) return NULL;
	MetaNetwork* meta = new MetaNetwork(cNetwork->getName());
	meta->addSubnet(cNetwork);
	return runAll(meta, di, server, connection, false);
}
MetaNetwork* test(MetaNetwork* meta, DataInput* di, GNet::GServer* server, GNet::Connection* connection)
{
	if (!meta) return NULL;
	return runAll(meta, di, server, connection, false);
}

}  // namespace glades_b200
