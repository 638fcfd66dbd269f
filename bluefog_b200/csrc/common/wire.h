// Negotiation messages exchanged between every rank and the coordinator (rank 0).
//
// Same information as the reference's Request/Response lists
// (bluefog/common/message.h:32-199, wire/message.fbs:21-122) but encoded with a small
// self-contained little-endian binary format instead of FlatBuffers, plus two fields the
// B200 runtime needs: the byte size of each tensor (fusion planning without shape
// products) and a signature of the per-rank neighbor lists and weights (so that only
// tensors that share one combine recipe on every rank are fused into one launch).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace bfb {

enum class OpType : int32_t {
  ALLREDUCE = 0,
  ALLGATHER = 1,
  BROADCAST = 2,
  NEIGHBOR_ALLREDUCE = 3,
  NEIGHBOR_ALLGATHER = 4,
  WIN_CREATE = 5,
  WIN_FREE = 6,
  WIN_PUT = 7,
  WIN_GET = 8,
  WIN_ACCUMULATE = 9,
  BARRIER = 10,
  PAIR_GOSSIP = 11,
  ERROR = 100,
};
const char* OpTypeName(OpType t);

// Element types understood by the runtime.  BFLOAT16 is new relative to the reference
// (bluefog/common/common.h:62-76 stops at FLOAT16).
enum class DataType : int32_t {
  UINT8 = 0, INT8 = 1, UINT16 = 2, INT16 = 3, INT32 = 4, INT64 = 5,
  FLOAT16 = 6, FLOAT32 = 7, FLOAT64 = 8, BOOL = 9, BYTE = 10, BFLOAT16 = 11,
};
const char* DataTypeName(DataType t);
int DataTypeSize(DataType t);

struct Request {
  int32_t rank = 0;
  OpType type = OpType::ALLREDUCE;
  DataType dtype = DataType::FLOAT32;
  std::string name;
  int32_t root_rank = -1;
  int32_t device = -1;  // -1 = host memory, otherwise CUDA device index
  std::vector<int64_t> shape;
  bool is_hierarchical = false;
  uint64_t nbytes = 0;
  uint64_t neighbor_sig = 0;
};

struct RequestList {
  std::vector<Request> requests;
  bool shutdown = false;
  std::string Serialize() const;
  static bool Parse(const std::string& bytes, RequestList* out);
};

struct Response {
  OpType type = OpType::ALLREDUCE;
  std::vector<std::string> names;  // more than one name = fused execution
  std::string error_message;
  std::vector<int32_t> devices;  // device of each rank for this response
  // ALLGATHER / NEIGHBOR_ALLGATHER: first-dimension size of every rank's tensor, names.size() x world.
  std::vector<int64_t> first_dims;
};

struct ResponseList {
  std::vector<Response> responses;
  bool shutdown = false;
  std::string Serialize() const;
  static bool Parse(const std::string& bytes, ResponseList* out);
};

}  // namespace bfb
