// Host-side C++ mirror of the reference's interface for the deep feed-forward path, on top of the
// C ABI in glades_b200.h.  Same class and member names, argument meaning and error behaviour as the
// reference (Backend/Machine Learning): NNInfo and the *LayerInfo classes (Structure/nninfo.h:40-126,
// Structure/layerinfo.h:32-77), DataInput (DataObjects/DataInput.h:26-50), Terminator
// (State/Terminator.cpp:63-78), NNetwork (Networks/network.h:59-141), MetaNetwork
// (Networks/metanetwork.h:35-73), OHE (GMath/OHE.h:33-72), NumberInput (DataObjects/NumberInput.h:30-88)
// and the glades::train / glades::test entry points (main.h:49-54), so that code written against the
// reference compiles against this header with the namespace changed.  Where the reference leans on types
// of third-party libraries that are not part of its tree (shmea containers, GNet server) small
// stand-ins with the members this path touches take their place; they are named where they appear.
//
// The reference's containers come from the third-party shmea library, which is not part of this
// tree.  Define GLADES_B200_WITH_SHMEA and put the shmea headers on the include path to use the
// real shmea::GList; otherwise a minimal stand-in with the members this path touches is used.
#pragma once
#include <stdint.h>

#include <map>
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
	std::map<unsigned int, std::string> strings;  // cells that hold text (the ',' and ';' separators of the live view)

public:
	GList() {}
	void addFloat(float v) { items.push_back(v); }
	void addInt(int v) { items.push_back((float)v); }
	void addString(const std::string& v)
	{
		strings[(unsigned int)items.size()] = v;
		items.push_back(0.0f);
	}
	float getFloat(unsigned int i) const { return i < items.size() ? items[i] : 0.0f; }
	bool isString(unsigned int i) const { return strings.find(i) != strings.end(); }
	std::string getString(unsigned int i) const
	{
		std::map<unsigned int, std::string>::const_iterator it = strings.find(i);
		return it == strings.end() ? std::string() : it->second;
	}
	unsigned int size() const { return (unsigned int)items.size(); }
	bool empty() const { return items.empty(); }
	void clear()
	{
		items.clear();
		strings.clear();
	}
};
}  // namespace shmea

// Stand-ins for the messaging types the live view goes through (include/Backend/Database/ServiceData.h,
// include/Backend/Networking/main.h:119): a message with a command, an argument list and a list or
// table payload, and a server whose send() takes ownership of the message.  A front end subclasses
// GServer (the real one queues the message for its writer thread).
namespace GNet {
class Connection
{
};
}  // namespace GNet
namespace shmea {
class ServiceData
{
	GNet::Connection* cConnection;
	std::string command;
	GList argList, repList;
	std::vector<int32_t> repTable;
	int tableRows, tableCols, type;

public:
	static const int TYPE_ACK = 0, TYPE_LIST = 1, TYPE_TABLE = 2;
	ServiceData(GNet::Connection* c, const std::string& cmd) : cConnection(c), command(cmd), tableRows(0), tableCols(0), type(TYPE_ACK) {}
	void set(const GList& l)
	{
		repList = l;
		type = TYPE_LIST;
	}
	void setTable(const std::vector<int32_t>& cells, int rows, int cols)
	{
		repTable = cells;
		tableRows = rows;
		tableCols = cols;
		type = TYPE_TABLE;
	}
	void setArgList(const GList& l) { argList = l; }
	GNet::Connection* getConnection() const { return cConnection; }
	std::string getCommand() const { return command; }
	int getType() const { return type; }
	const GList& getArgList() const { return argList; }
	const GList& getList() const { return repList; }
	const std::vector<int32_t>& getTableCells() const { return repTable; }
	int getTableRows() const { return tableRows; }
	int getTableCols() const { return tableCols; }
};
}  // namespace shmea
namespace GNet {
class GServer
{
public:
	virtual ~GServer() {}
	// takes ownership of the message
	virtual void send(shmea::ServiceData* data, bool = true, bool = false) = 0;
};
}  // namespace GNet
#endif

namespace glades_b200 {

// GMath ids (GMath/gmath.h:38-50)
struct GMath
{
	static const int MINMAX = 0, ZSCORE = 1;  // standardisation of input tables (GMath/gmath.h:53-54)
	static const int REGRESSION = 0, CLASSIFICATION = 1, KL = 2;
	static const int TANH = 0, TANHP = 1, SIGMOID = 2, SIGMOIDP = 3, LINEAR = 4, RELU = 5, LEAKY = 6, STEP = 7;
	static const int SOFTMAX = 8;  // extension, batched mode only
};

// One-hot maps of categorical columns (GMath/OHE.h:33-72, GMath/OHE.cpp): the category strings in
// order of first appearance, their counts, and the 0.99 / 0.01 vectors.
class OHE
{
	std::vector<std::string> OHEStrings;
	float fMin, fMax, fMean;

public:
	std::map<std::string, double> classCount;

	OHE() : fMin(0.0f), fMax(0.0f), fMean(0.0f) {}
	void addString(const std::string&);
	void setRange(float mn, float mx, float mean) { fMin = mn; fMax = mx; fMean = mean; }
	unsigned int size() const { return (unsigned int)OHEStrings.size(); }
	std::vector<std::string> getStrings() const { return OHEStrings; }
	bool contains(const std::string&) const;
	int indexAt(const std::string&) const;
	std::string classAt(unsigned int) const;
	float standardize(float) const;
	std::vector<float> operator[](const std::string&) const;   // 0.99 at the category's place, 0.01 elsewhere
	std::string operator[](const std::vector<float>&) const;   // the category of the largest entry (last one on ties)
};

class DataInput
{
public:
	static const int CSV = 0, IMAGE = 1, TEXT = 2;
	std::vector<OHE*> OHEMaps;
	std::vector<bool> featureIsCategorical;
	virtual ~DataInput() {}
	// Not in the reference: rows that already lie in device memory as row-major matrices (inputs
	// [rows][features], expected [rows][outputs]).  A network that finds them skips the row-by-row pack.
	virtual bool deviceRows(const float** d_x, const float** d_y, int* device) const
	{
		(void)d_x; (void)d_y; (void)device;
		return false;
	}
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

// Stand-in for the typed raw table the reference imports with shmea::GTable(file, ',', TYPE_FILE)
// (DataObjects/NumberInput.cpp:47): per column either numbers or strings, and the columns marked as outputs.
// shmea's file importer -- how it types the cells of a CSV file and which columns it marks as outputs -- is
// not part of the reference's tree; fromCSV states its own rule.
struct RawTable
{
	std::vector<std::string> headers;
	std::vector<bool> isString;                    // per column
	std::vector<bool> isOutput;                    // per column
	std::vector<std::vector<float> > numbers;      // [col][row], numeric columns
	std::vector<std::vector<std::string> > texts;  // [col][row], string columns
	unsigned int rows;

	RawTable() : rows(0) {}
	unsigned int numberOfCols() const { return (unsigned int)headers.size(); }
	void addNumberCol(const std::string& header, const std::vector<float>& cells, bool output = false);
	void addStringCol(const std::string& header, const std::vector<std::string>& cells, bool output = false);
	// Reads a comma-separated file with a header line.  A column is a string column when its first data
	// cell does not parse as a number (the reference decides by the first cell too, NumberInput.cpp:61-68);
	// the LAST `outputCols` columns are marked as outputs.
	static bool fromCSV(const std::string& path, RawTable& out, unsigned int outputCols = 1);
};

// NumberInput (DataObjects/NumberInput.h:30-88): imports a raw table, standardises it and serves the rows.
// The standardisation runs on the GPU (gl_standardize_table) and the standardised rows stay in device
// memory, where NNetwork picks them up without a host round trip; getTrainRow / getTrainExpectedRow read
// a host copy that is fetched on first use.
class NumberInput : public DataInput
{
	std::vector<float> x, y;       // host copies, row-major
	float* dX;
	float* dY;
	unsigned int rows, nIn, nOut;
	int device;
	mutable bool hostValid;
	std::string name;
	bool loaded;
	void release();
	void fetchHost() const;

public:
	NumberInput() : dX(NULL), dY(NULL), rows(0), nIn(0), nOut(0), device(0), hostValid(false), loaded(false) {}
	virtual ~NumberInput();
	void setDevice(int d) { device = d; }
	// import(file): RawTable::fromCSV (one output column, the last) + standardizeInputTable
	virtual void import(const std::string& fname);
	bool standardizeInputTable(const RawTable& raw, int standardizeFlag = GMath::MINMAX);
	shmea::GList getTrainRow(unsigned int) const;
	shmea::GList getTrainExpectedRow(unsigned int) const;
	shmea::GList getTestRow(unsigned int) const { return shmea::GList(); }
	shmea::GList getTestExpectedRow(unsigned int) const { return shmea::GList(); }
	unsigned int getTrainSize() const { return rows; }
	unsigned int getTestSize() const { return 0; }
	unsigned int getFeatureCount() const { return nIn; }
	unsigned int getOutputCount() const { return nOut; }
	int getType() const { return CSV; }
	bool deviceRows(const float** d_x, const float** d_y, int* dev) const;
	const std::vector<float>& hostInputs() const { fetchHost(); return x; }
	const std::vector<float>& hostExpected() const { fetchHost(); return y; }
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
	// NNInfo::save / load (Structure/nninfo.cpp:711-798): the skeleton as the reference's table -- header
	// line, one row for the input layer's info, one per hidden layer, one for the output layer, -1 in the
	// cells a row does not use (inputlayerinfo.cpp:70-89) -- written as comma-separated text to
	// <directory>/<name>.csv.  The reference stores the same table through shmea's SaveFolder
	// ("neuralnetworks"); `directory` stands in for that folder.
	bool save(const std::string& directory = "database/neuralnetworks") const;
	static NNInfo* load(const std::string& netName, const std::string& directory = "database/neuralnetworks");
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
	int deviceOrdinal;
	bool quiet;
	std::vector<float> initW, initB;
	bool haveInit;
	shmea::GList results;
	shmea::GList learningCurve;
	std::vector<int32_t> lastConfusion;
	std::string pendingState;
	GNet::GServer* serverInstance;
	GNet::Connection* cConnection;
	bool firstRunActivation;
	bool ownsSkeleton;
	// live view: one frame is in flight while training goes on (see sendFrame)
	struct Frame
	{
		bool pending;
		int epochs;
		float error, accuracy, falseAlarm, recall;
		std::vector<int32_t> confusion;
		Frame() : pending(false), epochs(0), error(0), accuracy(0), falseAlarm(0), recall(0) {}
	} frame;

	void run(DataInput*, int);
	bool build(DataInput*);
	void queueFrame();
	void sendFrame();

public:
	static const int TYPE_DFF = 0;
	static const int RUN_TRAIN = 0, RUN_TEST = 1;

	Terminator terminator;

	NNetwork();
	NNetwork(NNInfo*);
	virtual ~NNetwork();
	int64_t getCurrentTimeMilliseconds() const;
	bool getRunning() const { return running; }
	int getEpochs() const { return epochs; }
	void stop();
	void train(DataInput*);
	void test(DataInput*);
	NNInfo* getNNInfo() { return skeleton; }
	std::string getName() const { return skeleton ? skeleton->getName() : std::string(); }
	float getAccuracy() const { return overallTotalAccuracy; }
	shmea::GList getResults() const { return results; }
	// Database (network.cpp:701-722): only the skeleton is persisted, as in the reference; see
	// saveState / loadState below for the weights.
	bool load(const std::string& netName, const std::string& directory = "database/neuralnetworks");
	bool save(const std::string& directory = "database/neuralnetworks") const;
	// Live view (network.cpp:124, 258-357): with a server and a connection set, training sends the
	// GUI_Callback messages PROGRESSIVE, ACTIVATIONS, WEIGHTS, ACC and (classification) CONF after an epoch,
	// every epoch below 10 and at most every 16 ms after that.
	void setServer(GNet::GServer*, GNet::Connection*);
	// The reference declares the learning curve but never appends to it (network.h:93, network.cpp:766); here
	// it holds the points of the PROGRESSIVE stream of the last run: epoch - 1, error, epoch - 1, error, ...
	shmea::GList getLearningCurve() const { return learningCurve; }

	// ---- not in the reference: the reference can neither inject nor read weights as a whole ----
	// Arithmetic mode (GL_MODE_REFERENCE default; GL_MODE_BATCHED for data-parallel throughput).  Also
	// settable through the environment variable GLADES_B200_MODE=reference|batched.
	void setMode(int newMode) { mode = newMode; }
	void setQuiet(bool q) { quiet = q; }
	void setDevice(int d) { deviceOrdinal = d; }
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

// MetaNetwork (Networks/metanetwork.h:35-73): a named collection of networks, what glades::train and
// glades::test hand back.  Not in the reference: trainReplicas runs the subnets side by side, subnet i on
// GPU i % (number of GPUs), one host thread per GPU -- the use of a multi-GPU box for networks too small
// to shard (every replica is the whole, sequential training run).
class MetaNetwork
{
	static const int ONE_TO_ONE = 0, ONE_TO_MANY = 1;
	std::string name;
	int collectionType;
	std::vector<NNetwork*> subnets;

public:
	MetaNetwork(const std::string& newName);
	MetaNetwork(NNInfo*, int subnetCount = 1);
	virtual ~MetaNetwork();
	void clearSubnets() { subnets.clear(); }
	void setName(const std::string& n) { name = n; }
	void addSubnet(NNInfo*);
	void addSubnet(NNetwork*);
	std::string getName() const { return name; }
	int size() const { return (int)subnets.size(); }
	std::vector<NNetwork*> getSubnets() const { return subnets; }
	NNetwork* getSubnet(unsigned int);
	std::string getSubnetName(unsigned int) const;
	NNetwork* getSubnetByName(const std::string&) const;
	// every subnet trains on `di`; returns the number of GPUs used
	int trainReplicas(DataInput* di);
};

// glades::train / glades::test (main.h:49-54, main.cpp:82-243): NULL on a NULL first argument, else the
// MetaNetwork that holds what ran (a new one for the NNInfo* and NNetwork* forms, owned by the caller).
MetaNetwork* train(NNInfo*, DataInput*, GNet::GServer* = NULL, GNet::Connection* = NULL);
MetaNetwork* train(NNetwork*, DataInput*, GNet::GServer* = NULL, GNet::Connection* = NULL);
MetaNetwork* train(MetaNetwork*, DataInput*, GNet::GServer* = NULL, GNet::Connection* = NULL);
MetaNetwork* test(NNInfo*, DataInput*, GNet::GServer* = NULL, GNet::Connection* = NULL);
MetaNetwork* test(NNetwork*, DataInput*, GNet::GServer* = NULL, GNet::Connection* = NULL);
MetaNetwork* test(MetaNetwork*, DataInput*, GNet::GServer* = NULL, GNet::Connection* = NULL);

}  // namespace glades_b200
