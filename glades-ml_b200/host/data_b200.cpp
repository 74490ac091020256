// Host-side mirror of the reference's data interface in front of the training loop: the one-hot maps
// (GMath/OHE.cpp), the typed raw table stand-in, NumberInput (DataObjects/NumberInput.cpp: import,
// standardizeInputTable, the row getters) and the skeleton's table form (Structure/nninfo.cpp:711-798).
// The standardisation itself runs on the GPU (gl_standardize_table); this file decides the column plan --
// which columns are categorical, the category indices in order of first appearance, which columns are
// outputs -- and keeps the standardised rows in device memory for the network.
#include "glades_b200.hpp"

#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>

namespace glades_b200 {

// ---------------------------------------------------------------------------------------------
// OHE (GMath/OHE.cpp:47-64,122-198,203-222,270-279)
void OHE::addString(const std::string& newString)
{
	if (!contains(newString))
	{
		OHEStrings.push_back(newString);
		classCount[newString] = 1;
	}
	else
		++classCount[newString];
}

bool OHE::contains(const std::string& s) const { return indexAt(s) >= 0; }

int OHE::indexAt(const std::string& needle) const
{
	for (size_t i = 0; i < OHEStrings.size(); ++i)
		if (OHEStrings[i] == needle) return (int)i;
	return -1;
}

std::string OHE::classAt(unsigned int cid) const { return cid < OHEStrings.size() ? OHEStrings[cid] : std::string(); }

float OHE::standardize(float val) const
{
	const float xRange = fMax - fMin;
	if (xRange == 0.0f) return 0.0f;
	return ((((val - fMin) / (xRange)) * 0.98f) + 0.01f);
}

std::vector<float> OHE::operator[](const std::string& needle) const
{
	std::vector<float> v(size(), 0.01f);
	const int at = indexAt(needle);
	if (at >= 0) v[(size_t)at] = 0.99f;
	return v;
}

std::string OHE::operator[](const std::vector<float>& needle) const
{
	// the largest entry, the last one on ties, starting from 0 (OHE.cpp:203-222)
	float max = 0.0f;
	int index = -1;
	for (size_t i = 0; i < needle.size(); ++i)
		if (needle[i] >= max)
		{
			max = needle[i];
			index = (int)i;
		}
	return (index >= 0 && (size_t)index < OHEStrings.size()) ? OHEStrings[(size_t)index] : std::string();
}

// ---------------------------------------------------------------------------------------------
void RawTable::addNumberCol(const std::string& header, const std::vector<float>& cells, bool output)
{
	headers.push_back(header);
	isString.push_back(false);
	isOutput.push_back(output);
	numbers.push_back(cells);
	texts.push_back(std::vector<std::string>());
	if (cells.size() > rows) rows = (unsigned int)cells.size();
}

void RawTable::addStringCol(const std::string& header, const std::vector<std::string>& cells, bool output)
{
	headers.push_back(header);
	isString.push_back(true);
	isOutput.push_back(output);
	numbers.push_back(std::vector<float>());
	texts.push_back(cells);
	if (cells.size() > rows) rows = (unsigned int)cells.size();
}

static void splitLine(const std::string& line, std::vector<std::string>& out)
{
	out.clear();
	size_t a = 0;
	for (;;)
	{
		const size_t b = line.find(',', a);
		std::string cell = line.substr(a, b == std::string::npos ? std::string::npos : b - a);
		while (!cell.empty() && (cell[cell.size() - 1] == '\r' || cell[cell.size() - 1] == ' ')) cell.erase(cell.size() - 1);
		while (!cell.empty() && cell[0] == ' ') cell.erase(0, 1);
		out.push_back(cell);
		if (b == std::string::npos) break;
		a = b + 1;
	}
}

static bool parseNumber(const std::string& s, float* v)
{
	if (s.empty()) return false;
	char* end = NULL;
	errno = 0;
	const double d = strtod(s.c_str(), &end);
	if (end == s.c_str() || *end != 0) return false;
	*v = (float)d;
	return true;
}

bool RawTable::fromCSV(const std::string& path, RawTable& out, unsigned int outputCols)
{
	FILE* f = fopen(path.c_str(), "r");
	if (!f) return false;
	out = RawTable();
	std::vector<std::vector<std::string> > cells;
	std::vector<std::string> row, head;
	char buf[1 << 16];
	bool first = true;
	while (fgets(buf, sizeof buf, f))
	{
		std::string line(buf);
		while (!line.empty() && (line[line.size() - 1] == '\n' || line[line.size() - 1] == '\r')) line.erase(line.size() - 1);
		if (line.empty()) continue;
		splitLine(line, row);
		if (first)
		{
			head = row;
			first = false;
			continue;
		}
		if (row.size() != head.size())
		{
			fclose(f);
			return false;
		}
		cells.push_back(row);
	}
	fclose(f);
	if (head.empty() || cells.empty()) return false;
	for (size_t c = 0; c < head.size(); ++c)
	{
		const bool output = c + outputCols >= head.size();
		float v = 0.0f;
		if (!parseNumber(cells[0][c], &v))
		{
			std::vector<std::string> col(cells.size());
			for (size_t r = 0; r < cells.size(); ++r) col[r] = cells[r][c];
			out.addStringCol(head[c], col, output);
		}
		else
		{
			std::vector<float> col(cells.size());
			for (size_t r = 0; r < cells.size(); ++r)
				if (!parseNumber(cells[r][c], &col[r])) return false;  // a string in a numeric column: the reference gives up too
			out.addNumberCol(head[c], col, output);
		}
	}
	return true;
}

// ---------------------------------------------------------------------------------------------
NumberInput::~NumberInput() { release(); }

void NumberInput::release()
{
	if (dX) gl_device_free(dX, device);
	if (dY) gl_device_free(dY, device);
	dX = dY = NULL;
	for (size_t c = 0; c < OHEMaps.size(); ++c) delete OHEMaps[c];
	OHEMaps.clear();
	featureIsCategorical.clear();
	x.clear();
	y.clear();
	rows = nIn = nOut = 0;
	hostValid = false;
}

void NumberInput::import(const std::string& fname)
{
	if (loaded) return;
	name = fname;
	RawTable raw;
	if (!RawTable::fromCSV(fname, raw, 1))
	{
		fprintf(stderr, "[NumberInput] cannot read %s\n", fname.c_str());
		return;
	}
	if (standardizeInputTable(raw)) loaded = true;
}

// standardizeInputTable, DataObjects/NumberInput.cpp:43-285.  Host side: the one-hot maps (strings in order
// of first appearance, NumberInput.cpp:55-71 with OHE::mapFeatureSpace), the raw matrix with category
// indices in the categorical columns, the per-column plan.  Device side: extrema, scaling and one-hot
// expansion into the input and expected matrices.  Every failure is the reference's silent return plus one
// line on stderr, and leaves the object empty.
bool NumberInput::standardizeInputTable(const RawTable& raw, int standardizeFlag)
{
	release();
	const unsigned int cols = raw.numberOfCols();
	if (raw.rows == 0 || cols == 0) return false;
	std::vector<float> flat((size_t)raw.rows * cols);
	std::vector<int32_t> kind(cols), classes(cols), toOutput(cols);
	for (unsigned int c = 0; c < cols; ++c)
	{
		OHE* cOHE = new OHE();
		featureIsCategorical.push_back(raw.isString[c]);
		toOutput[c] = raw.isOutput[c] ? 1 : 0;
		if (raw.isString[c])
		{
			if (raw.texts[c].size() != raw.rows)
			{
				delete cOHE;
				release();
				return false;
			}
			for (unsigned int r = 0; r < raw.rows; ++r)
			{
				cOHE->addString(raw.texts[c][r]);
				flat[(size_t)r * cols + c] = (float)cOHE->indexAt(raw.texts[c][r]);
			}
			kind[c] = 1;
			classes[c] = (int32_t)cOHE->size();
		}
		else
		{
			if (raw.numbers[c].size() != raw.rows)
			{
				delete cOHE;
				release();
				return false;
			}
			for (unsigned int r = 0; r < raw.rows; ++r) flat[(size_t)r * cols + c] = raw.numbers[c][r];
			kind[c] = 0;
			classes[c] = 0;
		}
		OHEMaps.push_back(cOHE);
	}
	void* dRaw = NULL;
	bool ok = gl_device_alloc(&dRaw, (int64_t)flat.size() * 4, device) == GL_OK &&
	          gl_memcpy_h2d(dRaw, &flat[0], (int64_t)flat.size() * 4, device) == GL_OK;
	int32_t nx = 0, ny = 0;
	std::vector<float> stats((size_t)cols * 4);
	ok = ok && gl_standardize_table(static_cast<const float*>(dRaw), raw.rows, (int32_t)cols, &kind[0], &classes[0], &toOutput[0],
	                                standardizeFlag, NULL, &nx, NULL, &ny, NULL, device) == GL_OK;
	if (ok && nx > 0) ok = gl_device_alloc(reinterpret_cast<void**>(&dX), (int64_t)raw.rows * nx * 4, device) == GL_OK;
	if (ok && ny > 0) ok = gl_device_alloc(reinterpret_cast<void**>(&dY), (int64_t)raw.rows * ny * 4, device) == GL_OK;
	ok = ok && gl_standardize_table(static_cast<const float*>(dRaw), raw.rows, (int32_t)cols, &kind[0], &classes[0], &toOutput[0],
	                                standardizeFlag, dX, &nx, dY, &ny, &stats[0], device) == GL_OK;
	if (dRaw) gl_device_free(dRaw, device);
	if (!ok)
	{
		fprintf(stderr, "[NumberInput] %s\n", gl_last_error());
		release();
		return false;
	}
	for (unsigned int c = 0; c < cols; ++c)
		if (!raw.isString[c]) OHEMaps[c]->setRange(stats[4 * (size_t)c], stats[4 * (size_t)c + 1], stats[4 * (size_t)c + 2]);
	rows = raw.rows;
	nIn = (unsigned int)nx;
	nOut = (unsigned int)ny;
	hostValid = false;
	return true;
}

void NumberInput::fetchHost() const
{
	if (hostValid) return;
	NumberInput* self = const_cast<NumberInput*>(this);
	self->x.assign((size_t)rows * nIn, 0.0f);
	self->y.assign((size_t)rows * nOut, 0.0f);
	if (dX && !x.empty()) gl_memcpy_d2h(&self->x[0], dX, (int64_t)x.size() * 4, device);
	if (dY && !y.empty()) gl_memcpy_d2h(&self->y[0], dY, (int64_t)y.size() * 4, device);
	hostValid = true;
}

shmea::GList NumberInput::getTrainRow(unsigned int r) const
{
	shmea::GList l;
	if (r >= rows) return l;
	fetchHost();
	for (unsigned int c = 0; c < nIn; ++c) l.addFloat(x[(size_t)r * nIn + c]);
	return l;
}

shmea::GList NumberInput::getTrainExpectedRow(unsigned int r) const
{
	shmea::GList l;
	if (r >= rows) return l;
	fetchHost();
	for (unsigned int c = 0; c < nOut; ++c) l.addFloat(y[(size_t)r * nOut + c]);
	return l;
}

bool NumberInput::deviceRows(const float** d_x, const float** d_y, int* dev) const
{
	if (!dX || !dY) return false;
	*d_x = dX;
	*d_y = dY;
	*dev = device;
	return true;
}

// ---------------------------------------------------------------------------------------------
// The skeleton as a table (Structure/nninfo.cpp:711-798; rows as inputlayerinfo.cpp:70-89,
// hiddenlayerinfo.cpp and outputlayerinfo.cpp build them): Size, batchSize, learningRate, momentumFactor,
// weightDecay1, weightDecay2, pDropout, activationType, activationParam, outputType; -1 where unused.
static bool makeDirs(const std::string& dir)
{
	std::string path;
	for (size_t i = 0; i <= dir.size(); ++i)
	{
		if (i == dir.size() || dir[i] == '/')
		{
			if (!path.empty() && mkdir(path.c_str(), 0777) != 0 && errno != EEXIST) return false;
		}
		if (i < dir.size()) path += dir[i];
	}
	return true;
}

bool NNInfo::save(const std::string& directory) const
{
	if (!inputLayer || !outputLayer || name.empty() || !makeDirs(directory)) return false;
	FILE* f = fopen((directory + "/" + name + ".csv").c_str(), "w");
	if (!f) return false;
	fprintf(f, "Size,batchSize,learningRate,momentumFactor,weightDecay1,weightDecay2,pDropout,activationType,activationParam,outputType\n");
	fprintf(f, "-1,%d,%f,%f,%f,%f,%f,%d,%f,-1\n", inputLayer->getBatchSize(), inputLayer->getLearningRate(),
	        inputLayer->getMomentumFactor(), inputLayer->getWeightDecay1(), inputLayer->getWeightDecay2(), inputLayer->getPDropout(),
	        inputLayer->getActivationType(), inputLayer->getActivationParam());
	for (size_t i = 0; i < layers.size(); ++i)
		fprintf(f, "%u,1,%f,%f,%f,%f,%f,%d,%f,-1\n", layers[i]->size(), layers[i]->getLearningRate(), layers[i]->getMomentumFactor(),
		        layers[i]->getWeightDecay1(), layers[i]->getWeightDecay2(), layers[i]->getPDropout(), layers[i]->getActivationType(),
		        layers[i]->getActivationParam());
	fprintf(f, "%u,1,-1.000000,-1.000000,-1.000000,-1.000000,-1.000000,-1,-1.000000,%d\n", outputLayer->size(), outputLayer->getOutputType());
	return fclose(f) == 0;
}

NNInfo* NNInfo::load(const std::string& netName, const std::string& directory)
{
	FILE* f = fopen((directory + "/" + netName + ".csv").c_str(), "r");
	if (!f) return NULL;
	std::vector<std::vector<float> > table;
	std::vector<std::string> row;
	char buf[4096];
	bool first = true;
	bool ok = true;
	while (fgets(buf, sizeof buf, f))
	{
		std::string line(buf);
		while (!line.empty() && (line[line.size() - 1] == '\n' || line[line.size() - 1] == '\r')) line.erase(line.size() - 1);
		if (line.empty()) continue;
		if (first)
		{
			first = false;
			continue;
		}
		splitLine(line, row);
		if (row.size() < 10)
		{
			ok = false;
			break;
		}
		std::vector<float> v(10);
		for (int c = 0; c < 10 && ok; ++c) ok = parseNumber(row[(size_t)c], &v[(size_t)c]);
		table.push_back(v);
	}
	fclose(f);
	// fromGTable (nninfo.cpp:732-785): at least an input row and an output row
	if (!ok || table.size() < 2) return NULL;
	const std::vector<float>& in = table[0];
	InputLayerInfo* inputInfo = new InputLayerInfo((int)in[1], in[2], in[3], in[4], in[5], in[6], (int)in[7], in[8]);
	std::vector<HiddenLayerInfo*> hidden;
	for (size_t i = 1; i + 1 < table.size(); ++i)
	{
		const std::vector<float>& h = table[i];
		hidden.push_back(new HiddenLayerInfo((int)h[0], h[2], h[3], h[4], h[5], h[6], (int)h[7], h[8]));
	}
	const std::vector<float>& out = table[table.size() - 1];
	return new NNInfo(netName, inputInfo, hidden, new OutputLayerInfo((int)out[0], (int)out[9]));
}

}  // namespace glades_b200
