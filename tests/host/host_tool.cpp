// Test driver for the C++ host mirror (glades-ml_b200/host): reads like the reference's own
// unit test (unit-tests/Backend/Machine Learning/nn-test.cpp:27-75: build the NNInfo, import the
// data, set the terminator, check the accuracy before training, call train) but takes its case from
// a file and writes what it ends with, so that the Python tests can compare it with the oracle.
//
//   host_tool unit                      host-only checks (no GPU needed); prints OK
//   host_tool init  <case> <out>        draws initial weights after srand(seed) and writes them
//   host_tool run   <case> <out>        trains / tests on the GPU through NNetwork and writes
//                                       weights, biases, metrics, results, confusion counts
//   host_tool gui   <case> <out>        trains with a recording server attached and writes the live-view
//                                       messages, flattened like the oracle harness flattens the reference's
//   host_tool replicas <case> <out> <k> trains k replicas through MetaNetwork::trainReplicas (one per GPU,
//                                       round robin) and writes every replica's weights
//   host_tool standardize <table> <out> standardises a typed raw table through NumberInput on the GPU and
//                                       writes the input and expected matrices
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "glades_b200.hpp"

using namespace glades_b200;

struct Case
{
	int nLayers;
	std::vector<int> sizes;
	std::vector<float> lr, mom, wd1, wd2, par;
	std::vector<int> act;
	int outType, batch, rows, epochs, runType, mode, haveWeights, seed;
	std::vector<float> x, y, w, b;
};

static bool rd(FILE* f, void* p, size_t n) { return fread(p, 1, n, f) == n; }

static bool loadCase(const char* path, Case& c)
{
	FILE* f = fopen(path, "rb");
	if (!f) return false;
	int hdr[9];
	if (!rd(f, hdr, sizeof hdr)) return false;
	c.nLayers = hdr[0]; c.outType = hdr[1]; c.batch = hdr[2]; c.rows = hdr[3]; c.epochs = hdr[4];
	c.runType = hdr[5]; c.mode = hdr[6]; c.haveWeights = hdr[7]; c.seed = hdr[8];
	const int L = c.nLayers - 1;
	c.sizes.resize(c.nLayers); c.act.resize(L);
	c.lr.resize(L); c.mom.resize(L); c.wd1.resize(L); c.wd2.resize(L); c.par.resize(L);
	bool ok = rd(f, &c.sizes[0], 4 * c.nLayers) && rd(f, &c.act[0], 4 * L) && rd(f, &c.lr[0], 4 * L) &&
	          rd(f, &c.mom[0], 4 * L) && rd(f, &c.wd1[0], 4 * L) && rd(f, &c.wd2[0], 4 * L) && rd(f, &c.par[0], 4 * L);
	size_t nw = 0;
	for (int l = 0; l < L; ++l) nw += (size_t)c.sizes[l] * c.sizes[l + 1];
	c.x.resize((size_t)c.rows * c.sizes[0]); c.y.resize((size_t)c.rows * c.sizes[L]);
	ok = ok && rd(f, &c.x[0], 4 * c.x.size()) && rd(f, &c.y[0], 4 * c.y.size());
	if (c.haveWeights)
	{
		c.w.resize(nw); c.b.resize(c.nLayers - 2);
		ok = ok && rd(f, &c.w[0], 4 * nw) && rd(f, &c.b[0], 4 * c.b.size());
	}
	fclose(f);
	return ok;
}

static NNInfo* makeInfo(const Case& c)
{
	// the same three steps as a caller of the reference: input-layer info, hidden infos, output info
	InputLayerInfo* in = new InputLayerInfo(c.batch, c.lr[0], c.mom[0], c.wd1[0], c.wd2[0], 0.0f, c.act[0], c.par[0]);
	std::vector<HiddenLayerInfo*> hidden;
	for (int l = 1; l <= c.nLayers - 2; ++l)
		hidden.push_back(new HiddenLayerInfo(c.sizes[l], c.lr[l], c.mom[l], c.wd1[l], c.wd2[l], 0.0f, c.act[l], c.par[l]));
	OutputLayerInfo* out = new OutputLayerInfo(c.sizes[c.nLayers - 1], c.outType);
	return new NNInfo("case", in, hidden, out);
}

// A server that records what the live view sends, flattened as the oracle harness flattens the reference's
// messages: kind id, number of extra arguments, the arguments, payload rows, payload columns, payload
// length, payload; a text cell is 1e9 + its first character's code.
struct RecordingServer : public GNet::GServer
{
	std::vector<double> log;
	static double cell(const shmea::GList& l, unsigned int i)
	{
		if (l.isString(i))
		{
			const std::string s = l.getString(i);
			return 1e9 + (double)(unsigned char)(s.empty() ? 0 : s[0]);
		}
		return (double)l.getFloat(i);
	}
	void send(shmea::ServiceData* d, bool, bool)
	{
		static const char* kinds[] = {"PROGRESSIVE", "ACTIVATIONS", "WEIGHTS", "ACC", "CONF"};
		const shmea::GList& args = d->getArgList();
		double id = -1;
		for (int t = 0; t < 5; ++t)
			if (args.size() > 0 && args.getString(0) == kinds[t]) id = t;
		log.push_back(id);
		log.push_back(args.size() > 0 ? (double)(args.size() - 1) : 0.0);
		for (unsigned int i = 1; i < args.size(); ++i) log.push_back(cell(args, i));
		if (d->getType() == shmea::ServiceData::TYPE_TABLE)
		{
			log.push_back(d->getTableRows());
			log.push_back(d->getTableCols());
			log.push_back((double)d->getTableCells().size());
			for (size_t i = 0; i < d->getTableCells().size(); ++i) log.push_back((double)d->getTableCells()[i]);
		}
		else
		{
			log.push_back(0);
			log.push_back(0);
			log.push_back((double)d->getList().size());
			for (unsigned int i = 0; i < d->getList().size(); ++i) log.push_back(cell(d->getList(), i));
		}
		delete d;
	}
};

#define CHECK(expr)                                                       \
	do                                                                    \
	{                                                                     \
		if (!(expr))                                                      \
		{                                                                 \
			printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #expr);    \
			return 1;                                                     \
		}                                                                 \
	} while (0)

static int unitChecks()
{
	// NNInfo getters: index 0 = input-layer info, index l = hidden l-1, defaults past the end
	InputLayerInfo* in = new InputLayerInfo(4, 0.1f, 0.9f, 0.001f, 0.5f, 0.0f, GMath::SIGMOID, 0.3f);
	std::vector<HiddenLayerInfo*> hidden;
	hidden.push_back(new HiddenLayerInfo(16, 0.2f, 0.8f, 0.002f, 0.004f, 0.0f, GMath::TANH, 0.7f));
	hidden.push_back(new HiddenLayerInfo(8, 0.3f, 0.7f, 0.003f, 0.006f, 0.0f, GMath::RELU, 0.9f));
	NNInfo info("unit", in, hidden, new OutputLayerInfo(3, OutputLayerInfo::CLASSIFICATION));
	CHECK(info.numHiddenLayers() == 2 && info.getBatchSize() == 4 && info.getOutputLayerSize() == 3);
	CHECK(info.getLearningRate(0) == 0.1f && info.getLearningRate(1) == 0.2f && info.getLearningRate(2) == 0.3f);
	CHECK(info.getLearningRate(3) == 0.01f);                  // past the end: the reference's default
	CHECK(info.getWeightDecay2(0) == 0.001f);                 // quirk: index 0 returns weightDecay1
	CHECK(info.getWeightDecay2(1) == 0.004f && info.getWeightDecay1(2) == 0.003f);
	CHECK(info.getPDropout(3) == 1.0f && info.getMomentumFactor(7) == 0.0f);
	CHECK(info.getActivationType(0) == GMath::SIGMOID && info.getActivationType(2) == GMath::RELU);
	CHECK(info.getActivationParam(1) == 0.7f && info.getOutputType() == GMath::CLASSIFICATION);
	gl_net_desc d;
	CHECK(packDescriptor(info, 5, GL_MODE_REFERENCE, &d));
	CHECK(d.n_layers == 4 && d.sizes[0] == 5 && d.sizes[1] == 16 && d.sizes[2] == 8 && d.sizes[3] == 3);
	CHECK(d.wd2[0] == 0.001f && d.wd2[2] == 0.006f && d.batch_size == 4 && d.output_type == GL_OUT_CLASSIFICATION);
	CHECK(d.activation[0] == GL_ACT_SIGMOID && d.activation[1] == GL_ACT_TANH && d.activation[2] == GL_ACT_RELU);
	// Terminator::triggered (Terminator.cpp:63-78): modulo on time and epoch, threshold on accuracy
	Terminator t;
	CHECK(!t.triggered(100, 7, 99.0f));
	t.setEpoch(5);
	CHECK(t.triggered(1, 10, 0.0f) && !t.triggered(1, 11, 0.0f));
	t.setEpoch(0);
	t.setAccuracy(95.0f);
	CHECK(t.triggered(1, 1, 95.0f) && !t.triggered(1, 1, 94.9f));
	t.setAccuracy(0.0f);
	t.setTimestamp(10);
	CHECK(t.triggered(20, 1, 0.0f) && !t.triggered(21, 1, 0.0f));
	// data interface
	const float x[6] = {1, 2, 3, 4, 5, 6}, y[2] = {0.5f, 0.25f};
	ArrayInput ai(x, y, 2, 3, 1);
	CHECK(ai.getTrainSize() == 2 && ai.getFeatureCount() == 3 && ai.getTrainRow(1).getFloat(2) == 6.0f);
	CHECK(ai.getTrainExpectedRow(1).getFloat(0) == 0.25f && ai.getTrainRow(5).size() == 0);
	// error behaviour: NULL arguments return silently / NULL like the reference (main.cpp:84-85)
	CHECK(train((NNetwork*)NULL, &ai) == NULL);
	NNetwork none(NULL);
	none.train(&ai);
	CHECK(none.getEpochs() == 0 && !none.getRunning());
	NNetwork net(&info);
	net.setQuiet(true);
	net.train(NULL);
	CHECK(net.getEpochs() == 0);
	// one-hot maps (GMath/OHE.cpp): categories in order of first appearance, 0.99 / 0.01 vectors, decoding
	OHE ohe;
	ohe.addString("b");
	ohe.addString("a");
	ohe.addString("b");
	CHECK(ohe.size() == 2 && ohe.indexAt("a") == 1 && ohe.indexAt("zzz") == -1 && ohe.classCount["b"] == 2.0);
	CHECK(ohe["a"][0] == 0.01f && ohe["a"][1] == 0.99f && ohe["zzz"][0] == 0.01f && ohe["zzz"][1] == 0.01f);
	std::vector<float> probe(2);
	probe[0] = 0.2f;
	probe[1] = 0.7f;
	CHECK(ohe[probe] == "a" && ohe.classAt(0) == "b" && ohe.classAt(9) == "");
	ohe.setRange(-1.0f, 3.0f, 0.0f);
	CHECK(ohe.standardize(3.0f) == 0.99f && ohe.standardize(-1.0f) == 0.01f);
	// the skeleton's table form (Structure/nninfo.cpp:711-798): save, load, same getters
	{
		char dir[] = "/tmp/glades_b200_unit_XXXXXX";
		CHECK(mkdtemp(dir) != NULL);
		CHECK(info.save(dir));
		NNInfo* back = NNInfo::load("unit", dir);
		CHECK(back != NULL && back->numHiddenLayers() == 2 && back->getBatchSize() == 4 && back->getOutputLayerSize() == 3);
		CHECK(back->getLearningRate(0) == 0.1f && back->getLearningRate(2) == 0.3f && back->getWeightDecay2(1) == 0.004f);
		CHECK(back->getActivationType(2) == GMath::RELU && back->getOutputType() == GMath::CLASSIFICATION);
		CHECK(back->getHiddenLayerSize(0) == 16 && back->getHiddenLayerSize(1) == 8 && back->getActivationParam(1) == 0.7f);
		CHECK(NNInfo::load("missing", dir) == NULL);
		NNetwork loaded;
		CHECK(loaded.load("unit", dir) && loaded.getName() == "unit" && loaded.getNNInfo()->numHiddenLayers() == 2);
		CHECK(!loaded.load("missing", dir));
		// a raw table from a comma-separated file: typing by the first cell, last column marked as output
		const std::string csv = std::string(dir) + "/t.csv";
		FILE* tf = fopen(csv.c_str(), "w");
		CHECK(tf != NULL);
		fprintf(tf, "len,colour,kind\n1.5,red,x\n2.5,blue,y\n-3,red,x\n");
		fclose(tf);
		RawTable rt;
		CHECK(RawTable::fromCSV(csv, rt, 1) && rt.rows == 3 && rt.numberOfCols() == 3);
		CHECK(!rt.isString[0] && rt.isString[1] && rt.isString[2] && !rt.isOutput[1] && rt.isOutput[2]);
		CHECK(rt.numbers[0][2] == -3.0f && rt.texts[1][1] == "blue");
		CHECK(!RawTable::fromCSV(std::string(dir) + "/none.csv", rt, 1));
		delete back;
	}
	// collections: NULL arguments, names, look-up (Networks/metanetwork.cpp)
	CHECK(train((NNInfo*)NULL, &ai) == NULL && test((MetaNetwork*)NULL, &ai) == NULL);
	MetaNetwork meta(&info, 3);
	CHECK(meta.size() == 3 && meta.getName() == "unit" && meta.getSubnetName(2) == "unit" && meta.getSubnet(3) == NULL);
	CHECK(meta.getSubnetByName("unit") == meta.getSubnet(0) && meta.getSubnetByName("other") == NULL);
	meta.addSubnet((NNetwork*)NULL);
	CHECK(meta.size() == 3);
	// shard arithmetic of the C ABI
	int64_t f = 0, c = 0;
	gl_shard_range(10, 0, 3, &f, &c);
	CHECK(f == 0 && c == 4);
	gl_shard_range(10, 2, 3, &f, &c);
	CHECK(f == 7 && c == 3);
	// without a GPU a training call returns silently with the epoch counter untouched
	if (gl_device_count() < 1)
	{
		const float xx[5] = {0, 0, 0, 0, 0}, yy[3] = {0.01f, 0.99f, 0.01f};
		ArrayInput one(xx, yy, 1, 5, 3);
		net.terminator.setEpoch(1);
		net.train(&one);
		CHECK(net.getEpochs() == 0 && net.getAccuracy() == 0.0f);
	}
	printf("OK\n");
	return 0;
}

// standardize: <table> = int32 rows, cols, flag; int32 type[cols] (0 number, 1 string: cell k is the text "s<k>");
// int32 output[cols]; float32 cells[rows][cols].  <out> = int32 rows, nx, ny; float32 X[rows][nx]; Y[rows][ny].
static int standardizeTable(const char* in, const char* outPath)
{
	FILE* f = fopen(in, "rb");
	if (!f) return 2;
	int hdr[3];
	if (!rd(f, hdr, sizeof hdr)) return 2;
	const int rows = hdr[0], cols = hdr[1], flag = hdr[2];
	std::vector<int> type(cols), output(cols);
	std::vector<float> cells((size_t)rows * cols);
	if (!rd(f, &type[0], 4 * cols) || !rd(f, &output[0], 4 * cols) || !rd(f, &cells[0], 4 * cells.size())) return 2;
	fclose(f);
	RawTable raw;
	for (int c = 0; c < cols; ++c)
	{
		char h[32];
		snprintf(h, sizeof h, "col%d", c);
		if (type[c] == 1)
		{
			std::vector<std::string> col(rows);
			for (int r = 0; r < rows; ++r)
			{
				char s[32];
				snprintf(s, sizeof s, "s%d", (int)cells[(size_t)r * cols + c]);
				col[r] = s;
			}
			raw.addStringCol(h, col, output[c] != 0);
		}
		else
		{
			std::vector<float> col(rows);
			for (int r = 0; r < rows; ++r) col[r] = cells[(size_t)r * cols + c];
			raw.addNumberCol(h, col, output[c] != 0);
		}
	}
	NumberInput ni;
	if (!ni.standardizeInputTable(raw, flag)) return 5;
	FILE* out = fopen(outPath, "wb");
	if (!out) return 2;
	const int dims[3] = {(int)ni.getTrainSize(), (int)ni.getFeatureCount(), (int)ni.getOutputCount()};
	fwrite(dims, 4, 3, out);
	// through the row getters, like a caller of the reference reads them
	for (int r = 0; r < dims[0]; ++r)
	{
		const shmea::GList row = ni.getTrainRow(r);
		for (int c = 0; c < dims[1]; ++c) { const float v = row.getFloat(c); fwrite(&v, 4, 1, out); }
	}
	for (int r = 0; r < dims[0]; ++r)
	{
		const shmea::GList row = ni.getTrainExpectedRow(r);
		for (int c = 0; c < dims[2]; ++c) { const float v = row.getFloat(c); fwrite(&v, 4, 1, out); }
	}
	fclose(out);
	return 0;
}

int main(int argc, char** argv)
{
	if (argc >= 2 && strcmp(argv[1], "unit") == 0) return unitChecks();
	if (argc < 4) return 2;
	if (strcmp(argv[1], "standardize") == 0) return standardizeTable(argv[2], argv[3]);
	Case c;
	if (!loadCase(argv[2], c)) { fprintf(stderr, "cannot read case %s\n", argv[2]); return 2; }
	NNInfo* info = makeInfo(c);
	FILE* out = fopen(argv[3], "wb");
	if (!out) return 2;
	if (strcmp(argv[1], "init") == 0)
	{
		srand((unsigned)c.seed);
		std::vector<float> w;
		drawInitialWeights(*info, c.sizes[0], w);
		fwrite(&w[0], 4, w.size(), out);
		fclose(out);
		return 0;
	}
	ArrayInput di(&c.x[0], &c.y[0], c.rows, c.sizes[0], c.sizes[c.nLayers - 1]);
	if (strcmp(argv[1], "replicas") == 0)
	{
		// k replicas of the same network, same injected weights, trained side by side; every replica must end
		// with the weights of a single run
		const int k = argc >= 5 ? atoi(argv[4]) : 2;
		MetaNetwork meta(info, k);
		for (int i = 0; i < k; ++i)
		{
			NNetwork* sub = meta.getSubnet(i);
			sub->setQuiet(true);
			sub->setMode(c.mode);
			sub->setWeights(c.w, c.b);
			sub->terminator.setEpoch(c.epochs);
		}
		const int gpus = meta.trainReplicas(&di);
		fwrite(&gpus, 4, 1, out);
		fwrite(&k, 4, 1, out);
		for (int i = 0; i < k; ++i)
		{
			std::vector<float> w, b;
			if (!meta.getSubnet(i)->getWeights(w, b)) { fclose(out); return 4; }
			const int e = meta.getSubnet(i)->getEpochs(), nw = (int)w.size();
			fwrite(&e, 4, 1, out);
			fwrite(&nw, 4, 1, out);
			fwrite(&w[0], 4, nw, out);
			delete meta.getSubnet(i);
		}
		fclose(out);
		delete info;
		return 0;
	}
	if (strcmp(argv[1], "gui") == 0)
	{
		RecordingServer server;
		GNet::Connection connection;
		NNetwork net(info);
		net.setQuiet(true);
		net.setMode(c.mode);
		net.setWeights(c.w, c.b);
		net.terminator.setEpoch(c.epochs);
		MetaNetwork* meta = train(&net, &di, &server, &connection);
		if (!meta || meta->size() != 1 || meta->getSubnet(0) != &net) return 6;
		delete meta;
		const shmea::GList curve = net.getLearningCurve();
		const int n = (int)server.log.size(), nc = (int)curve.size();
		fwrite(&n, 4, 1, out);
		if (n) fwrite(&server.log[0], 8, n, out);
		fwrite(&nc, 4, 1, out);
		for (int i = 0; i < nc; ++i) { const float v = curve.getFloat(i); fwrite(&v, 4, 1, out); }
		fclose(out);
		delete info;
		return 0;
	}
	NNetwork net(info);
	net.setQuiet(true);
	net.setMode(c.mode);
	if (c.haveWeights) net.setWeights(c.w, c.b);
	else srand((unsigned)c.seed);
	// like nn-test.cpp:69-75: terminator on the epoch count, accuracy below the bar before training
	net.terminator.setEpoch(c.epochs);
	if (net.getAccuracy() >= 95.0f) return 3;
	// glades::train / glades::test hand back a new collection that holds the network (main.cpp:112-134)
	MetaNetwork* ran = (c.runType == NNetwork::RUN_TRAIN) ? train(&net, &di) : test(&net, &di);
	if (!ran || ran->getSubnet(0) != &net) return 6;
	delete ran;
	std::vector<float> w, b;
	if (!net.getWeights(w, b)) { fclose(out); return 4; }
	const int epochs = net.getEpochs();
	float m[4] = {net.getError(), net.getAccuracy(), net.getClassAccuracy(), net.getClassF1()};
	const shmea::GList res = net.getResults();
	const int nres = (int)res.size();
	const int ncm = (int)net.getConfusion().size();
	fwrite(&epochs, 4, 1, out);
	fwrite(m, 4, 4, out);
	fwrite(&nres, 4, 1, out);
	for (int i = 0; i < nres; ++i) { float v = res.getFloat(i); fwrite(&v, 4, 1, out); }
	fwrite(&ncm, 4, 1, out);
	if (ncm) fwrite(&net.getConfusion()[0], 4, ncm, out);
	const int nw = (int)w.size(), nb = (int)b.size();
	fwrite(&nw, 4, 1, out);
	fwrite(&w[0], 4, nw, out);
	fwrite(&nb, 4, 1, out);
	if (nb) fwrite(&b[0], 4, nb, out);
	fclose(out);
	delete info;
	return 0;
}
