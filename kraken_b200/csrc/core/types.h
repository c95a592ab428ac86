// Shared enums, error codes and small PODs of the framework.
//
// The numeric values are part of the on-disk checkpoint format and of the
// Python API (they mirror kraken/common/info.h:13-72, kraken/t/element_type.h:23-37
// and kraken/common/error_code.h:7-33 of the reference), so they must not be
// renumbered.
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>

namespace kb {

enum class EmitterType : uint8_t { kDefault = 0, kDCT = 1 };

enum class TableType : uint8_t { kDense = 0, kSparse = 1 };

enum class OptimType : uint8_t { kAdagrad = 0, kAdam = 1, kRMSprop = 2, kSGD = 3 };

enum class InitializerType : uint8_t {
  kConstant = 0,
  kUniform = 1,
  kNormal = 2,
  kXavierUniform = 3,
  kXavierNormal = 4,
};

// Per-row / per-table optimizer state slots. Serialised as u32.
enum class StateType : uint32_t {
  kSteps = 0,
  kMomentumBuffer = 1,
  kStateSum = 2,
  kFirstMoment = 3,
  kSecondMoment = 4,
  kSecondMomentMax = 5,
  kSquareAverage = 6,
  kGAve = 7,
};

enum class DType : uint8_t {
  kUnknown = 0,
  kBool = 1,
  kUint8 = 2,
  kInt8 = 3,
  kUint16 = 4,
  kInt16 = 5,
  kUint32 = 6,
  kInt32 = 7,
  kUint64 = 8,
  kInt64 = 9,
  kFloat16 = 10,
  kFloat32 = 11,
  kFloat64 = 12,
};

enum class Layout : uint8_t { kStride = 0, kCoo = 1 };

inline size_t DTypeBytes(DType t) {
  switch (t) {
    case DType::kBool:
    case DType::kUint8:
    case DType::kInt8:
      return 1;
    case DType::kUint16:
    case DType::kInt16:
    case DType::kFloat16:
      return 2;
    case DType::kUint32:
    case DType::kInt32:
    case DType::kFloat32:
      return 4;
    case DType::kUint64:
    case DType::kInt64:
    case DType::kFloat64:
      return 8;
    default:
      return 0;
  }
}

inline const char* DTypeName(DType t) {
  static const char* names[] = {"UnKnown", "Bool",   "Uint8",  "Int8",    "Uint16",  "Int16",  "Uint32",
                                "Int32",   "Uint64", "Int64",  "Float16", "Float32", "Float64"};
  auto i = static_cast<uint8_t>(t);
  return i <= 12 ? names[i] : "UnKnown";
}

// Node status bit flags of a shard (a shard is "working" only when the word is exactly kWork).
struct NodeStatus {
  static constexpr uint32_t kInit = 1u << 0;
  static constexpr uint32_t kWork = 1u << 1;
  static constexpr uint32_t kProxy = 1u << 2;
  static constexpr uint32_t kTransfer = 1u << 3;
  static constexpr uint32_t kSave = 1u << 4;
  static constexpr uint32_t kLoad = 1u << 5;
};

// Error codes; device kernels write the same numbers into their status words.
namespace err {
constexpr int32_t kUnknown = -1;
constexpr int32_t kSuccess = 0;
constexpr int32_t kUnRegisterFunc = 1;
constexpr int32_t kSerializeRequest = 2;
constexpr int32_t kSerializeReply = 3;
constexpr int32_t kDeserializeRequest = 4;
constexpr int32_t kDeserializeReply = 5;
constexpr int32_t kSnappyUncompress = 6;
constexpr int32_t kNodeStatusInappropriate = 7;
constexpr int32_t kRouterVersion = 8;
constexpr int32_t kRouteWrongNode = 9;
constexpr int32_t kModelNotInitialized = 10;
constexpr int32_t kModelAlreadyInitialized = 11;
constexpr int32_t kTableNotExist = 12;
constexpr int32_t kTableTypeUnCompatible = 13;
constexpr int32_t kSparseDimensionUnCompatible = 14;
constexpr int32_t kSparseIdNotExist = 15;
constexpr int32_t kGradientUnCompatible = 16;
constexpr int32_t kTimeout = 17;
constexpr int32_t kInterfaceUnImplement = 18;
constexpr int32_t kDenseTableUnCompatible = 19;
constexpr int32_t kSparseTableUnCompatible = 20;
constexpr int32_t kTableFull = 21;       // device hash table has no free slot within the probe limit
constexpr int32_t kInboxOverflow = 22;   // a peer sent more unique ids than the inbox holds
constexpr int32_t kCheckpointIO = 23;
constexpr int32_t kBadArgument = 24;
constexpr int32_t kConnection = 25;     // the peer closed the connection or sent a broken frame

inline const char* Msg(int32_t c) {
  switch (c) {
    case kSuccess: return "success";
    case kUnRegisterFunc: return "unregistered function";
    case kSerializeRequest: return "serialize request error";
    case kSerializeReply: return "serialize reply error";
    case kDeserializeRequest: return "deserialize request error";
    case kDeserializeReply: return "deserialize reply error";
    case kSnappyUncompress: return "uncompress error";
    case kNodeStatusInappropriate: return "node status inappropriate";
    case kRouterVersion: return "router version mismatch";
    case kRouteWrongNode: return "routed to the wrong node";
    case kModelNotInitialized: return "model not initialized";
    case kModelAlreadyInitialized: return "model already initialized";
    case kTableNotExist: return "table does not exist";
    case kTableTypeUnCompatible: return "table type incompatible";
    case kSparseDimensionUnCompatible: return "sparse dimension incompatible";
    case kSparseIdNotExist: return "sparse id does not exist";
    case kGradientUnCompatible: return "gradient incompatible with value";
    case kTimeout: return "timeout";
    case kInterfaceUnImplement: return "interface not implemented";
    case kDenseTableUnCompatible: return "dense table incompatible";
    case kSparseTableUnCompatible: return "sparse table incompatible";
    case kTableFull: return "hash table full";
    case kInboxOverflow: return "peer inbox overflow";
    case kCheckpointIO: return "checkpoint I/O error";
    case kBadArgument: return "bad argument";
    case kConnection: return "connection lost";
    default: return "unknown error";
  }
}
}  // namespace err

struct KrakenError : public std::runtime_error {
  int32_t code;
  KrakenError(int32_t c, const std::string& what) : std::runtime_error(what), code(c) {}
};

#define KB_CHECK(cond, code, msg)                                                         \
  do {                                                                                    \
    if (!(cond)) {                                                                        \
      throw ::kb::KrakenError((code), std::string(__FILE__) + ":" + std::to_string(__LINE__) + \
                                          ": " + (msg));                                  \
    }                                                                                     \
  } while (0)

using Conf = std::map<std::string, std::string>;  // ordered: canonical on-disk order

}  // namespace kb
