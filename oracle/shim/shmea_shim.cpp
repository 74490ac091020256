// TEST INFRASTRUCTURE ONLY -- never linked into, imported by or called from the product library.
//
// Link shim for the un-vendored third-party `shmea` container library (GType / GString / GList /
// GTable), written from the declarations in the reference's header snapshot
// (include/Backend/Database/{GType,GString,GList,GTable}.h).  The reference's feed-forward path
// (Backend/Machine Learning/Networks/network.cpp and the State/, GMath/, Structure/ sources it
// calls) only needs these containers to carry floats and ints around; no arithmetic of the path
// lives in shmea.  The shim implements exactly the member functions the reference objects leave
// undefined, so that the reference sources can be compiled unmodified and driven by the harness
// in ../ref_harness.cpp.  Persistence and GUI-messaging symbols that the path never reaches are
// in trap_stubs.c.
//
// Every GType always owns an allocated block: the header's GPointer copy path mishandles a
// NULL-data pointer (include/Backend/Database/GPointer.h:50-56,63-85), so an empty value still
// gets a one-byte block.
#include "Backend/Database/GType.h"
#include "Backend/Database/GString.h"
#include "Backend/Database/GList.h"
#include "Backend/Database/GTable.h"
#include "Backend/Database/GObject.h"
#include "Backend/Database/ServiceData.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>

namespace shmea {

typedef GPointer<char, array_deleter<char> > Block;

static char* newBlock(const void* src, int64_t n)
{
	char* b = new char[n + 1];
	if (src && n > 0)
		memcpy(b, src, n);
	b[n] = 0;
	return b;
}

// ---------------------------------------------------------------- GType
GType::GType() : block(newBlock(NULL, 0)), blockSize(0), type(NULL_TYPE) {}
GType::GType(const GType& o) : block(o.block), blockSize(o.blockSize), type(o.type) {}
GType::GType(const bool& v) : block(newBlock(&v, sizeof(bool))), blockSize(sizeof(bool)), type(BOOLEAN_TYPE) {}
GType::GType(const char& v) : block(newBlock(&v, sizeof(char))), blockSize(sizeof(char)), type(CHAR_TYPE) {}
GType::GType(const short& v) : block(newBlock(&v, sizeof(short))), blockSize(sizeof(short)), type(SHORT_TYPE) {}
GType::GType(const int& v) : block(newBlock(&v, sizeof(int))), blockSize(sizeof(int)), type(INT_TYPE) {}
GType::GType(const int64_t& v) : block(newBlock(&v, sizeof(int64_t))), blockSize(sizeof(int64_t)), type(LONG_TYPE) {}
GType::GType(const float& v) : block(newBlock(&v, sizeof(float))), blockSize(sizeof(float)), type(FLOAT_TYPE) {}
GType::GType(const double& v) : block(newBlock(&v, sizeof(double))), blockSize(sizeof(double)), type(DOUBLE_TYPE) {}
GType::GType(const char* s) : block(newBlock(s, s ? strlen(s) : 0)), blockSize(s ? strlen(s) : 0), type(STRING_TYPE) {}
GType::GType(const char* s, unsigned int n) : block(newBlock(s, n)), blockSize(n), type(STRING_TYPE) {}
GType::GType(Type t, const void* p, int64_t n) : block(newBlock(p, n)), blockSize(n), type(t) {}
GType::~GType() {}

GType::Type GType::getType() const { return type; }
const char* GType::c_str() const { return block.get(); }
unsigned int GType::size() const { return blockSize; }

void GType::set(Type t, const void* p, int64_t n)
{
	block = Block(newBlock(p, n));
	blockSize = n;
	type = t;
}

// Numeric read-out: the value is converted from whatever type the cell holds.
static double asDouble(const GType& g)
{
	const char* b = g.c_str();
	switch (g.getType())
	{
	case GType::BOOLEAN_TYPE: { bool v; memcpy(&v, b, sizeof v); return v ? 1.0 : 0.0; }
	case GType::CHAR_TYPE: { char v; memcpy(&v, b, sizeof v); return v; }
	case GType::SHORT_TYPE: { short v; memcpy(&v, b, sizeof v); return v; }
	case GType::INT_TYPE: { int v; memcpy(&v, b, sizeof v); return v; }
	case GType::LONG_TYPE: { int64_t v; memcpy(&v, b, sizeof v); return (double)v; }
	case GType::FLOAT_TYPE: { float v; memcpy(&v, b, sizeof v); return v; }
	case GType::DOUBLE_TYPE: { double v; memcpy(&v, b, sizeof v); return v; }
	case GType::STRING_TYPE: return atof(b);
	default: return 0.0;
	}
}

// A float cell is returned bit-for-bit (no trip through double is needed, but it is exact anyway).
float GType::getFloat() const
{
	if (type == FLOAT_TYPE)
	{
		float v;
		memcpy(&v, block.get(), sizeof v);
		return v;
	}
	return (float)asDouble(*this);
}
double GType::getDouble() const { return asDouble(*this); }
int GType::getInt() const
{
	if (type == INT_TYPE)
	{
		int v;
		memcpy(&v, block.get(), sizeof v);
		return v;
	}
	return (int)asDouble(*this);
}
int64_t GType::getLong() const { return (int64_t)asDouble(*this); }
short GType::getShort() const { return (short)asDouble(*this); }
char GType::getChar() const { return (char)asDouble(*this); }
bool GType::getBoolean() const { return asDouble(*this) != 0.0; }

GType::operator const char*() const { return c_str(); }
GType::operator float() const { return getFloat(); }
GType::operator int() const { return getInt(); }

GType& GType::operator=(const GType& o)
{
	if (this != &o)
	{
		block = o.block;
		blockSize = o.blockSize;
		type = o.type;
	}
	return *this;
}

// ---------------------------------------------------------------- GString
GString::GString() : GType("") {}
GString::GString(const GString& o) : GType(o) {}
GString::GString(const char* s) : GType(s ? s : "") {}
GString::GString(const char& c) : GType(&c, 1u) {}
GString::GString(const GType& g) : GType("")
{
	if (g.getType() == STRING_TYPE)
	{
		set(STRING_TYPE, g.c_str(), g.size());
		return;
	}
	char buf[64];
	int n = 0;
	switch (g.getType())
	{
	case FLOAT_TYPE:
	case DOUBLE_TYPE: n = snprintf(buf, sizeof buf, "%f", g.getDouble()); break;
	case NULL_TYPE: n = 0; buf[0] = 0; break;
	default: n = snprintf(buf, sizeof buf, "%lld", (long long)g.getLong()); break;
	}
	set(STRING_TYPE, buf, n);
}
GString::~GString() {}

unsigned int GString::length() const { return blockSize; }
GString GString::intTOstring(int v)
{
	char buf[32];
	snprintf(buf, sizeof buf, "%d", v);
	return GString(buf);
}
GString GString::operator+=(const GString& o)
{
	std::string joined(block.get(), blockSize);
	joined.append(o.c_str(), o.length());
	set(STRING_TYPE, joined.data(), (int64_t)joined.size());
	return *this;
}
bool GString::operator==(const GString& o) const
{
	return blockSize == o.blockSize && memcmp(block.get(), o.block.get(), blockSize) == 0;
}
bool GString::operator!=(const char* s) const
{
	unsigned int n = s ? strlen(s) : 0;
	return !(blockSize == n && memcmp(block.get(), s, n) == 0);
}

// ---------------------------------------------------------------- GList
GList::GList() : xMin(0.0f), xMax(0.0f), xRange(0.0f) {}
GList::GList(const GList& o) : items(o.items), xMin(o.xMin), xMax(o.xMax), xRange(o.xRange) {}
GList::GList(int n, const GType& v) : items(n > 0 ? n : 0, v), xMin(0.0f), xMax(0.0f), xRange(0.0f) {}
GList::~GList() {}

void GList::addFloat(float v) { items.push_back(GType(v)); }
void GList::addInt(int v) { items.push_back(GType(v)); }
void GList::addLong(int64_t v) { items.push_back(GType(v)); }
void GList::addString(const char* s) { items.push_back(GType(s)); }
void GList::addString(const GString& s) { items.push_back(GType(s.c_str(), s.length())); }
void GList::addGType(const GType& v) { items.push_back(v); }
void GList::clear() { items.clear(); }
void GList::setGType(unsigned int i, const GType& v)
{
	if (i < items.size())
		items[i] = v;
}
float GList::getFloat(unsigned int i) const { return i < items.size() ? items[i].getFloat() : 0.0f; }
int GList::getInt(unsigned int i) const { return i < items.size() ? items[i].getInt() : 0; }
unsigned int GList::size() const { return items.size(); }
GType GList::operator[](unsigned int i) { return i < items.size() ? items[i] : GType(); }
const GType GList::operator[](unsigned int i) const { return i < items.size() ? items[i] : GType(); }
void GList::operator=(const GList& o)
{
	items = o.items;
	xMin = o.xMin;
	xMax = o.xMax;
	xRange = o.xRange;
}
void GList::print() const
{
	for (unsigned int i = 0; i < items.size(); ++i)
		printf("%s%f", i ? "," : "", items[i].getDouble());
	printf("\n");
}

// ---------------------------------------------------------------- GTable
GTable::GTable() : delimiter(','), xMin(0.0f), xMax(0.0f), xRange(0.0f) {}
GTable::GTable(char d) : delimiter(d), xMin(0.0f), xMax(0.0f), xRange(0.0f) {}
GTable::GTable(char d, const std::vector<GString>& h) : delimiter(d), header(h), xMin(0.0f), xMax(0.0f), xRange(0.0f) {}
GTable::GTable(const GTable& o)
	: delimiter(o.delimiter), header(o.header), cells(o.cells), xMin(o.xMin), xMax(o.xMax),
	  xRange(o.xRange), outputColumns(o.outputColumns)
{
}
GTable::~GTable() {}

// The reference reads its raw tables with GTable(file name, delimiter, TYPE_FILE)
// (DataObjects/NumberInput.cpp:47).  shmea's file importer -- how it types the cells of a CSV file and
// which column it marks as output -- is not part of the reference tree, so this shim does not imitate
// it: the harness registers an already typed table under a name, and the "file" constructor hands out
// a copy of the table registered under that name (an empty table for an unknown name).
static std::map<std::string, GTable>& tableRegistry()
{
	static std::map<std::string, GTable> reg;
	return reg;
}
void shimRegisterTable(const char* name, const GTable& t) { tableRegistry()[name] = t; }
GTable::GTable(const GString& fname, char d, int) : delimiter(d), xMin(0.0f), xMax(0.0f), xRange(0.0f)
{
	std::map<std::string, GTable>::const_iterator it = tableRegistry().find(std::string(fname.c_str(), fname.length()));
	if (it != tableRegistry().end())
		*this = it->second;
}
void GTable::operator=(const GTable& o)
{
	delimiter = o.delimiter;
	header = o.header;
	cells = o.cells;
	xMin = o.xMin;
	xMax = o.xMax;
	xRange = o.xRange;
	outputColumns = o.outputColumns;
}
// Appends a column: one cell per row (rows are created for the first column of an empty table).
void GTable::addCol(const GString& h, const GList& col, unsigned int)
{
	header.push_back(h);
	if (cells.size() < col.size())
		cells.resize(col.size());
	for (unsigned int r = 0; r < col.size(); ++r)
		cells[r].addGType(col[r]);
}
GList GTable::getRow(unsigned int r) const { return r < cells.size() ? cells[r] : GList(); }
GList GTable::getCol(unsigned int c) const
{
	GList out;
	for (unsigned int r = 0; r < cells.size(); ++r)
		out.addGType(cells[r][c]);
	return out;
}
bool GTable::isOutput(unsigned int c) const
{
	for (unsigned int i = 0; i < outputColumns.size(); ++i)
		if (outputColumns[i] == c)
			return true;
	return false;
}
void GTable::toggleOutput(unsigned int c)
{
	for (unsigned int i = 0; i < outputColumns.size(); ++i)
		if (outputColumns[i] == c)
		{
			outputColumns.erase(outputColumns.begin() + i);
			return;
		}
	outputColumns.push_back(c);
}

void GTable::addRow(const GList& r) { cells.push_back(r); }
void GTable::clear()
{
	header.clear();
	cells.clear();
	outputColumns.clear();
}
GType GTable::getCell(unsigned int r, unsigned int c) const
{
	if (r >= cells.size())
		return GType();
	return cells[r][c];
}
void GTable::setCell(unsigned int r, unsigned int c, const GType& v)
{
	if (r < cells.size())
		cells[r].setGType(c, v);
}
GString GTable::getHeader(unsigned int i) const { return i < header.size() ? header[i] : GString(); }
std::vector<GString> GTable::getHeaders() const { return header; }
void GTable::setHeaders(const std::vector<GString>& h) { header = h; }
unsigned int GTable::numberOfRows() const { return cells.size(); }
unsigned int GTable::numberOfCols() const
{
	if (!header.empty())
		return header.size();
	return cells.empty() ? 0 : cells[0].size();
}
const GList& GTable::operator[](unsigned int r) const
{
	static const GList empty;
	return r < cells.size() ? cells[r] : empty;
}
const GList& GTable::operator[](int r) const { return (*this)[(unsigned int)(r < 0 ? 0 : r)]; }
void GTable::print() const
{
	for (unsigned int r = 0; r < cells.size(); ++r)
		cells[r].print();
}

// ---------------------------------------------------------------- GObject / ServiceData (GUI messages)
GObject::GObject() {}
GObject::~GObject() {}

ServiceData::ServiceData(GNet::Connection* c, GString cmd)
	: cConnection(c), timesent(0), command(cmd), serviceNum(0), responseServiceNum(0), type(TYPE_ACK)
{
}
ServiceData::~ServiceData() {}
void ServiceData::set(const GList& l)
{
	repList = l;
	type = TYPE_LIST;
}
void ServiceData::set(const GTable& t)
{
	repTable = t;
	type = TYPE_TABLE;
}
void ServiceData::setArgList(const GList& l) { argList = l; }
GString ServiceData::getCommand() const { return command; }
int ServiceData::getType() const { return type; }
const GList& ServiceData::getArgList() const { return argList; }
const GList& ServiceData::getList() const { return repList; }
const GTable& ServiceData::getTable() const { return repTable; }

// What the reference hands to GNet::GServer::send (Networks/network.cpp:258-357), flattened: the argument
// list and the payload (a list, or a table row by row) as doubles; a string cell becomes its first
// character's code plus 1e9 (the payloads only carry the separators ',' and ';' and, in the argument
// list, the message kind, which is kept as text).
struct ShimMessage
{
	std::string command, kind;
	std::vector<double> args, payload;
	int rows, cols;
};
static std::vector<ShimMessage>& messageLog()
{
	static std::vector<ShimMessage> log;
	return log;
}
static double cellValue(const GType& g)
{
	if (g.getType() == GType::STRING_TYPE)
		return 1e9 + (double)(unsigned char)(g.size() ? g.c_str()[0] : 0);
	return g.getDouble();
}
void shimClearMessages() { messageLog().clear(); }
size_t shimMessageCount() { return messageLog().size(); }
const ShimMessage& shimMessage(size_t i) { return messageLog()[i]; }
void shimRecordMessage(const ServiceData* d, const GString& command, const GList& args, int type, const GList& list,
                       const GTable& table)
{
	ShimMessage m;
	m.command = std::string(command.c_str(), command.length());
	m.rows = m.cols = 0;
	for (unsigned int i = 0; i < args.size(); ++i)
	{
		const GType a = args[i];
		if (i == 0 && a.getType() == GType::STRING_TYPE)
			m.kind = std::string(a.c_str(), a.size());
		else
			m.args.push_back(cellValue(a));
	}
	if (type == ServiceData::TYPE_TABLE)
	{
		m.rows = (int)table.numberOfRows();
		m.cols = (int)table.numberOfCols();
		for (int r = 0; r < m.rows; ++r)
			for (int c = 0; c < m.cols; ++c)
				m.payload.push_back(cellValue(table.getCell(r, c)));
	}
	else
		for (unsigned int i = 0; i < list.size(); ++i)
			m.payload.push_back(cellValue(list[i]));
	messageLog().push_back(m);
	(void)d;
}

} // namespace shmea

// GNet::GServer::send(shmea::ServiceData*, bool, bool), defined by its mangled name because the class
// declaration drags in the whole networking layer (include/Backend/Networking/main.h:119).  The reference
// only needs a non-NULL server pointer to call it; `self` is never touched.
extern "C" void _ZN4GNet7GServer4sendEPN5shmea11ServiceDataEbb(void* self, shmea::ServiceData* d, bool, bool)
{
	(void)self;
	if (d)
		shmea::shimRecordMessage(d, d->getCommand(), d->getArgList(), d->getType(), d->getList(), d->getTable());
}
