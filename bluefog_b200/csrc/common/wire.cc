#include "wire.h"

#include <cstring>

namespace bfb {

const char* OpTypeName(OpType t) {
  switch (t) {
    case OpType::ALLREDUCE: return "ALLREDUCE";
    case OpType::ALLGATHER: return "ALLGATHER";
    case OpType::BROADCAST: return "BROADCAST";
    case OpType::NEIGHBOR_ALLREDUCE: return "NEIGHBOR_ALLREDUCE";
    case OpType::NEIGHBOR_ALLGATHER: return "NEIGHBOR_ALLGATHER";
    case OpType::WIN_CREATE: return "WIN_CREATE";
    case OpType::WIN_FREE: return "WIN_FREE";
    case OpType::WIN_PUT: return "WIN_PUT";
    case OpType::WIN_GET: return "WIN_GET";
    case OpType::WIN_ACCUMULATE: return "WIN_ACCUMULATE";
    case OpType::BARRIER: return "BARRIER";
    case OpType::PAIR_GOSSIP: return "PAIR_GOSSIP";
    case OpType::ERROR: return "ERROR";
  }
  return "UNKNOWN";
}

const char* DataTypeName(DataType t) {
  switch (t) {
    case DataType::UINT8: return "uint8";
    case DataType::INT8: return "int8";
    case DataType::UINT16: return "uint16";
    case DataType::INT16: return "int16";
    case DataType::INT32: return "int32";
    case DataType::INT64: return "int64";
    case DataType::FLOAT16: return "float16";
    case DataType::FLOAT32: return "float32";
    case DataType::FLOAT64: return "float64";
    case DataType::BOOL: return "bool";
    case DataType::BYTE: return "byte";
    case DataType::BFLOAT16: return "bfloat16";
  }
  return "unknown";
}

int DataTypeSize(DataType t) {
  switch (t) {
    case DataType::UINT8: case DataType::INT8: case DataType::BOOL: case DataType::BYTE: return 1;
    case DataType::UINT16: case DataType::INT16: case DataType::FLOAT16: case DataType::BFLOAT16: return 2;
    case DataType::INT32: case DataType::FLOAT32: return 4;
    case DataType::INT64: case DataType::FLOAT64: return 8;
  }
  return 1;
}

namespace {

class Writer {
 public:
  template <typename T>
  void Pod(T v) { out_.append(reinterpret_cast<const char*>(&v), sizeof(T)); }
  void Str(const std::string& s) {
    Pod<uint32_t>(static_cast<uint32_t>(s.size()));
    out_.append(s);
  }
  template <typename T>
  void Vec(const std::vector<T>& v) {
    Pod<uint32_t>(static_cast<uint32_t>(v.size()));
    if (!v.empty()) out_.append(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(T));
  }
  std::string Take() { return std::move(out_); }

 private:
  std::string out_;
};

class Reader {
 public:
  explicit Reader(const std::string& s) : p_(s.data()), end_(s.data() + s.size()) {}
  template <typename T>
  bool Pod(T* v) {
    if (static_cast<size_t>(end_ - p_) < sizeof(T)) return false;
    std::memcpy(v, p_, sizeof(T));
    p_ += sizeof(T);
    return true;
  }
  bool Str(std::string* s) {
    uint32_t n;
    if (!Pod(&n) || static_cast<size_t>(end_ - p_) < n) return false;
    s->assign(p_, n);
    p_ += n;
    return true;
  }
  template <typename T>
  bool Vec(std::vector<T>* v) {
    uint32_t n;
    if (!Pod(&n) || static_cast<size_t>(end_ - p_) < static_cast<size_t>(n) * sizeof(T)) return false;
    v->resize(n);
    if (n) std::memcpy(v->data(), p_, static_cast<size_t>(n) * sizeof(T));
    p_ += static_cast<size_t>(n) * sizeof(T);
    return true;
  }

 private:
  const char* p_;
  const char* end_;
};

constexpr uint32_t kRequestMagic = 0xB1F0A001u;
constexpr uint32_t kResponseMagic = 0xB1F0A002u;

}  // namespace

std::string RequestList::Serialize() const {
  Writer w;
  w.Pod<uint32_t>(kRequestMagic);
  w.Pod<uint8_t>(shutdown ? 1 : 0);
  w.Pod<uint32_t>(static_cast<uint32_t>(requests.size()));
  for (const auto& r : requests) {
    w.Pod<int32_t>(r.rank);
    w.Pod<int32_t>(static_cast<int32_t>(r.type));
    w.Pod<int32_t>(static_cast<int32_t>(r.dtype));
    w.Str(r.name);
    w.Pod<int32_t>(r.root_rank);
    w.Pod<int32_t>(r.device);
    w.Vec(r.shape);
    w.Pod<uint8_t>(r.is_hierarchical ? 1 : 0);
    w.Pod<uint64_t>(r.nbytes);
    w.Pod<uint64_t>(r.neighbor_sig);
  }
  return w.Take();
}

bool RequestList::Parse(const std::string& bytes, RequestList* out) {
  Reader r(bytes);
  uint32_t magic, n;
  uint8_t flag;
  if (!r.Pod(&magic) || magic != kRequestMagic || !r.Pod(&flag) || !r.Pod(&n)) return false;
  out->shutdown = flag != 0;
  out->requests.clear();
  out->requests.reserve(n);
  for (uint32_t i = 0; i < n; ++i) {
    Request q;
    int32_t type, dtype;
    uint8_t hier;
    if (!r.Pod(&q.rank) || !r.Pod(&type) || !r.Pod(&dtype) || !r.Str(&q.name) || !r.Pod(&q.root_rank) ||
        !r.Pod(&q.device) || !r.Vec(&q.shape) || !r.Pod(&hier) || !r.Pod(&q.nbytes) || !r.Pod(&q.neighbor_sig))
      return false;
    q.type = static_cast<OpType>(type);
    q.dtype = static_cast<DataType>(dtype);
    q.is_hierarchical = hier != 0;
    out->requests.push_back(std::move(q));
  }
  return true;
}

std::string ResponseList::Serialize() const {
  Writer w;
  w.Pod<uint32_t>(kResponseMagic);
  w.Pod<uint8_t>(shutdown ? 1 : 0);
  w.Pod<uint32_t>(static_cast<uint32_t>(responses.size()));
  for (const auto& p : responses) {
    w.Pod<int32_t>(static_cast<int32_t>(p.type));
    w.Pod<uint32_t>(static_cast<uint32_t>(p.names.size()));
    for (const auto& n : p.names) w.Str(n);
    w.Str(p.error_message);
    w.Vec(p.devices);
    w.Vec(p.first_dims);
  }
  return w.Take();
}

bool ResponseList::Parse(const std::string& bytes, ResponseList* out) {
  Reader r(bytes);
  uint32_t magic, n;
  uint8_t flag;
  if (!r.Pod(&magic) || magic != kResponseMagic || !r.Pod(&flag) || !r.Pod(&n)) return false;
  out->shutdown = flag != 0;
  out->responses.clear();
  for (uint32_t i = 0; i < n; ++i) {
    Response p;
    int32_t type;
    uint32_t nn;
    if (!r.Pod(&type) || !r.Pod(&nn)) return false;
    p.type = static_cast<OpType>(type);
    p.names.resize(nn);
    for (auto& s : p.names)
      if (!r.Str(&s)) return false;
    if (!r.Str(&p.error_message) || !r.Vec(&p.devices) || !r.Vec(&p.first_dims)) return false;
    out->responses.push_back(std::move(p));
  }
  return true;
}

}  // namespace bfb
