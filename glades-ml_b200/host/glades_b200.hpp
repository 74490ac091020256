// Host-side C++ mirror of the reference's interface for the deep feed-forward path, on top of the
// C ABI in glades_b200.h.  Same class and member names, argument meaning and error behaviour as the
// reference (Backend/Machine Learning): NNInfo and the *LayerInfo classes (Structure/nninfo.h:40-126,
// Structure/layerinfo.h:32-77), DataInput (DataObjects/DataInput.h:26-50), Terminator
// (State/Terminator.cpp:63-78) and NNetwork (Networks/network.h:59-141), so that code written
// against the reference compiles against this header with the namespace alone changed.
//
// The reference's containers come from the third-party shmea library, which is not part of this
// tree.  Define GLADES_B200_WITH_SHMEA and put the shmea headers on the include path to use the
// real shmea::GList; otherwise a minimal stand-in with the members this path touches is used.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "glades_b200.h"

#ifdef GLADES_B200_WITH_SHMEA
#include "Backend/Database/GList.h"
#else
namespace shmea {
// Stand-in for shmea::GList (include/Backend/Database/GList.h:32-104): a list of numeric cells.
class GList
{
	std::vector<float> items;

public:
	GList() {}
	void addFloat(float v) { items.push_back(v); }
	void addInt(int v) { items.push_back((float)v); }
	float getFloat(unsigned int i) const { return i < items.size() ? items[i] : 0.0f; }
	unsigned int size() const { return (unsigned int)items.size(); }
	bool empty() const { return items.empty(); }
	void clear() { items.clear(); }
};
}  // namespace shmea
#endif

namespace glades_b200 {

// GMath ids (GMath/gmath.h:38-50)
struct GMath
{
	static const int REGRESSION = 0, CLASSIFICATION = 1, KL = 2;
	static const int TANH = 0, TANHP = 1, SIGMOID = 2, SIGMOIDP = 3, LINEAR = 4, RELU = 5, LEAKY = 6, STEP = 7;
	static const int SOFTMAX = 8;  // extension, batched mode only
};

class DataInput
{
public:
	static const int CSV = 0, IMAGE = 1, TEXT = 2;
	virtual ~DataInput() {}
	virtual shmea::GList getTrainRow(unsigned int) const = 0;
	virtual shmea::GList getTrainExpectedRow(unsigned int) const = 0;
	virtual shmea::GList getTestRow(unsigned int) const = 0;
	virtual shmea::GList getTestExpectedRow(unsigned int) const = 0;
	virtual unsigned int getTrainSize() const = 0;
	virtual unsigned int getTestSize() const = 0;
	virtual unsigned int getFeatureCount() const = 0;
	virtual int getType() const = 0;
};

// Rows served from flat arrays (what NumberInput's standardised tables hold after import).
class ArrayInput : public DataInput
{
	std::vector<float> x, y;
	unsigned int rows, nIn, nOut;

public:
	ArrayInput(const float* nx, const float* ny, unsigned int r, unsigned int ni, unsigned int no);
	shmea::GList getTrainRow(unsigned int) const;
	shmea::GList getTrainExpectedRow(unsigned int) const;
	shmea::GList getTestRow(unsigned int r) const { return getTrainRow(r); }
	shmea::GList getTestExpectedRow(unsigned int r) const { return getTrainExpectedRow(r); }
	unsigned int getTrainSize() const { return rows; }
	unsigned int getTestSize() const { return 0; }
	unsigned int getFeatureCount() const { return nIn; }
	int getType() const { return CSV; }
};

class LayerInfo
{
protected:
	int lSize;
	float learningRate, momentumFactor, weightDecay1, weightDecay2, pDropout;
	int activationType;
	float activationParam;

public:
	LayerInfo(int s) : lSize(s), learningRate(0), momentumFactor(0), weightDecay1(0), weightDecay2(0), pDropout(0), activationType(0), activationParam(0) {}
	virtual ~LayerInfo() {}
	unsigned int size() const { return lSize; }
	float getLearningRate() const { return learningRate; }
	float getMomentumFactor() const { return momentumFactor; }
	float getWeightDecay1() const { return weightDecay1; }
	float getWeightDecay2() const { return weightDecay2; }
	float getPDropout() const { return pDropout; }
	int getActivationType() const { return activationType; }
	float getActivationParam() const { return activationParam; }
	void setLearningRate(float v) { learningRate = v; }
	void setMomentumFactor(float v) { momentumFactor = v; }
	void setActivationType(int v) { activationType = v; }
	void setActivationParam(float v) { activationParam = v; }
};

class InputLayerInfo : public LayerInfo
{
	int batchSize;

public:
	// argument order of Structure/inputlayerinfo.cpp:29-44
	InputLayerInfo(int newBatchSize, float lr, float mom, float wd1, float wd2, float pDrop, int act, float actParam);
	int getBatchSize() const { return batchSize; }
	void setBatchSize(int b) { batchSize = b; }
};

class HiddenLayerInfo : public LayerInfo
{
public:
	// argument order of Structure/hiddenlayerinfo.cpp:30-44
	HiddenLayerInfo(int newSize, float lr, float mom, float wd1, float wd2, float pDrop, int act, float actParam);
};

class OutputLayerInfo : public LayerInfo
{
	int outputType;

public:
	static const int REGRESSION = 0, CLASSIFICATION = 1;
	OutputLayerInfo(int newSize, int newOutputType) : LayerInfo(newSize), outputType(newOutputType) {}
	int getOutputType() const { return outputType; }
};

// Hyper-parameter skeleton; getters indexed as in Structure/nninfo.cpp:240-373 (index 0 = the input
// layer's info, index l >= 1 = hidden layer l-1), including their out-of-range defaults and the
// getWeightDecay2(0) quirk (it returns weightDecay1, nninfo.cpp:305-306).
class NNInfo
{
	std::string name;
	InputLayerInfo* inputLayer;
	OutputLayerInfo* outputLayer;
	std::vector<HiddenLayerInfo*> layers;

public:
	NNInfo(const std::string& newName, InputLayerInfo*, const std::vector<HiddenLayerInfo*>&, OutputLayerInfo*);
	~NNInfo();
	std::string getName() const { return name; }
	int getOutputType() const;
	float getPInput() const;
	int getBatchSize() const;
	int numHiddenLayers() const { return (int)layers.size(); }
	int getHiddenLayerSize(unsigned int) const;
	unsigned int getOutputLayerSize() const;
	float getLearningRate(unsigned int) const;
	float getMomentumFactor(unsigned int) const;
	float getWeightDecay1(unsigned int) const;
	float getWeightDecay2(unsigned int) const;
	float getPDropout(unsigned int) const;
	int getActivationType(unsigned int) const;
	float getActivationParam(unsigned int) const;
};

class Terminator
{
	int64_t timestamp, epoch;
	float accuracy;

public:
	Terminator() : timestamp(0), epoch(0), accuracy(0.0f) {}
	int64_t getTimestamp() const { return timestamp; }
	int64_t getEpoch() const { return epoch; }
	float getAccuracy() const { return accuracy; }
	void setTimestamp(int64_t v) { timestamp = v; }
	void setEpoch(int64_t v) { epoch = v; }
	void setAccuracy(float v) { accuracy = v; }
	bool triggered(int64_t cTimestamp, int64_t cEpoch, float cAccuracy) const;
};

// Fills the C-ABI descriptor from an NNInfo exactly as the reference's loop reads it.
// Returns false when the skeleton cannot be expressed (more than GL_MAX_WEIGHT_LAYERS layers).
bool packDescriptor(const NNInfo& info, unsigned int featureCount, int mode, gl_net_desc* out);

class NNetwork
{
	DataInput* di;
	NNInfo* skeleton;
	gl_net* handle;
	bool running;
	int epochs;
	float overallTotalError, overallTotalAccuracy;
	float overallClassAccuracy, overallClassPrecision, overallClassRecall, overallClassSpecificity, overallClassF1;
	int minibatchSize;
	int mode;
	bool quiet;
	std::vector<float> initW, initB;
	bool haveInit;
	shmea::GList results;
	std::vector<int32_t> lastConfusion;
	std::string pendingState;

	void run(DataInput*, int);
	bool build(DataInput*);

public:
	static const int TYPE_DFF = 0;
	static const int RUN_TRAIN = 0, RUN_TEST = 1;

	Terminator terminator;

	NNetwork(NNInfo*);
	virtual ~NNetwork();
	bool getRunning() const { return running; }
	int getEpochs() const { return epochs; }
	void stop();
	void train(DataInput*);
	void test(DataInput*);
	NNInfo* getNNInfo() { return skeleton; }
	float getAccuracy() const { return overallTotalAccuracy; }
	shmea::GList getResults() const { return results; }

	// ---- not in the reference: the reference can neither inject nor read weights as a whole ----
	// Arithmetic mode (GL_MODE_REFERENCE default; GL_MODE_BATCHED for data-parallel throughput).  Also
	// settable through the environment variable GLADES_B200_MODE=reference|batched.
	void setMode(int newMode) { mode = newMode; }
	void setQuiet(bool q) { quiet = q; }
	// Initial weights (flat W_0|...|W_H, row-major [n_{l+1}][n_l]) and hidden-layer scalar biases;
	// without them the first train()/test() draws weights like Layer::initWeights does.
	void setWeights(const std::vector<float>& w, const std::vector<float>& bias);
	bool getWeights(std::vector<float>& w, std::vector<float>& bias) const;
	// Checkpoint and true resume (weights, scalar biases, epoch counter, open-window pending deltas):
	// NNetwork::save()/load() of the reference persist only the skeleton (network.cpp:701-722).
	// loadState before the first train()/test() is applied when the device network is built.
	bool saveState(const std::string& path) const;
	bool loadState(const std::string& path);
	float getError() const { return overallTotalError; }
	float getClassAccuracy() const { return overallClassAccuracy; }
	float getClassF1() const { return overallClassF1; }
	const std::vector<int32_t>& getConfusion() const { return lastConfusion; }
};

// Weight draw of Layer::initWeights / Node::initWeights (State/layer.cpp:196-227,
// State/node.cpp:241-276): a 2048-strip Ziggurat half-normal driven by rand(), scaled by
// sqrt(1/n) (sqrt(2/n) for ReLU).  Fills flat weights in node-major order, consuming rand() in the
// reference's order.
void drawInitialWeights(const NNInfo& info, unsigned int featureCount, std::vector<float>& w);

// glades::train / glades::test (main.h:49-54) for one network: both return the network they ran.
NNetwork* train(NNetwork*, DataInput*);
NNetwork* test(NNetwork*, DataInput*);

}  // namespace glades_b200
