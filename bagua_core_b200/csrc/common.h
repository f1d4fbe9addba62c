// Shared vocabulary of the native core: error type, logging, dtypes, reduction ops,
// environment knobs and CUDA / NCCL status checks that throw instead of exiting.
//
// Reference parity: the error kinds mirror `BaguaCoreError`
// (bagua-core-internal/src/lib.rs:41-61); dtype and reduction-op numbering mirror
// bagua-core-internal/src/datatypes/mod.rs:24-47.  Unlike the reference's
// CUDACHECK/NCCLCHECK (bagua-core-internal/cpp/include/bagua_utils.h:5-6), a failed
// call raises a C++ exception that the bindings turn into a Python RuntimeError, so a
// shared GPU context is never torn down by `exit()`.
#pragma once

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace bagua {

enum class ErrorKind : int {
  Bucket = 0,
  Tensor,
  MemPool,
  Backend,
  Communicator,
  Telemetry,
  Serialization,
  InternalChannel,
  HttpCommunication,
};

inline const char* error_kind_name(ErrorKind k) {
  switch (k) {
    case ErrorKind::Bucket: return "BucketError";
    case ErrorKind::Tensor: return "TensorError";
    case ErrorKind::MemPool: return "MemPoolError";
    case ErrorKind::Backend: return "BackendError";
    case ErrorKind::Communicator: return "CommunicatorError";
    case ErrorKind::Telemetry: return "TelemetryError";
    case ErrorKind::Serialization: return "SerializationSerdeJsonError";
    case ErrorKind::InternalChannel: return "InternalChannelError";
    case ErrorKind::HttpCommunication: return "HttpCommunicationError";
  }
  return "UnknownError";
}

class BaguaError : public std::runtime_error {
 public:
  BaguaError(ErrorKind kind, const std::string& msg)
      : std::runtime_error(std::string(error_kind_name(kind)) + ": " + msg), kind_(kind) {}
  ErrorKind kind() const { return kind_; }

 private:
  ErrorKind kind_;
};

// ---------------------------------------------------------------------------------
// Logging: LOG_LEVEL env (TRACE|DEBUG|INFO|WARN|ERROR, default WARN), to stderr.
// (reference: bagua-core-py/src/lib.rs:490-495)
// ---------------------------------------------------------------------------------
enum class LogLevel : int { Trace = 0, Debug = 1, Info = 2, Warn = 3, Error = 4, Off = 5 };

inline LogLevel parse_log_level(const char* s) {
  if (!s) return LogLevel::Warn;
  std::string v(s);
  for (auto& c : v) c = (char)toupper(c);
  if (v == "TRACE") return LogLevel::Trace;
  if (v == "DEBUG") return LogLevel::Debug;
  if (v == "INFO") return LogLevel::Info;
  if (v == "WARN" || v == "WARNING") return LogLevel::Warn;
  if (v == "ERROR") return LogLevel::Error;
  if (v == "OFF") return LogLevel::Off;
  return LogLevel::Warn;
}

inline std::atomic<int>& log_level_storage() {
  static std::atomic<int> lvl{(int)parse_log_level(std::getenv("LOG_LEVEL"))};
  return lvl;
}
inline bool log_enabled(LogLevel l) { return (int)l >= log_level_storage().load(std::memory_order_relaxed); }
inline void set_log_level(LogLevel l) { log_level_storage().store((int)l); }

void log_write(LogLevel l, const char* file, int line, const std::string& msg);

#define BAGUA_LOG(level, ...)                                                 \
  do {                                                                        \
    if (::bagua::log_enabled(::bagua::LogLevel::level)) {                     \
      std::ostringstream _oss;                                                \
      _oss << __VA_ARGS__;                                                    \
      ::bagua::log_write(::bagua::LogLevel::level, __FILE__, __LINE__, _oss.str()); \
    }                                                                         \
  } while (0)

// ---------------------------------------------------------------------------------
// dtypes / reduction ops
// ---------------------------------------------------------------------------------
enum class DType : uint8_t { F32 = 0, F16 = 1, U8 = 2, I64 = 3, U64 = 4, BF16 = 5 };

inline size_t dtype_bytes(DType d) {
  switch (d) {
    case DType::F32: return 4;
    case DType::F16: return 2;
    case DType::U8: return 1;
    case DType::I64: return 8;
    case DType::U64: return 8;
    case DType::BF16: return 2;
  }
  return 0;
}

inline const char* dtype_name(DType d) {
  switch (d) {
    case DType::F32: return "F32";
    case DType::F16: return "F16";
    case DType::U8: return "U8";
    case DType::I64: return "I64";
    case DType::U64: return "U64";
    case DType::BF16: return "BF16";
  }
  return "?";
}

// Numbering is part of the Python API (`op: u8` arguments).
enum class ReductionOp : uint8_t {
  SUM = 0, PROD = 1, MIN = 2, MAX = 3, LOR = 4, LAND = 5, LXOR = 6, BOR = 7, BAND = 8, BXOR = 9, AVG = 10
};

inline ReductionOp reduction_op_from_u8(int v) {
  if (v < 0 || v > 10) throw BaguaError(ErrorKind::Communicator, "unknown reduction op " + std::to_string(v));
  return (ReductionOp)v;
}

// ---------------------------------------------------------------------------------
// Environment knobs (all optional)
// ---------------------------------------------------------------------------------
inline long env_long(const char* name, long dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  long r = std::strtol(v, &end, 10);
  return end == v ? dflt : r;
}
inline double env_double(const char* name, double dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  double r = std::strtod(v, &end);
  return end == v ? dflt : r;
}
inline std::string env_str(const char* name, const std::string& dflt) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::string(v) : dflt;
}

inline uint64_t now_ms() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(
             std::chrono::system_clock::now().time_since_epoch())
      .count();
}
inline uint64_t now_us_steady() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Compact "%g" formatting for log and error messages (ostream's default would print
// 120000 as 120000 but 1e-07 style values less readably, and needs no locale lookup).
inline std::string fmt_double(double v) {
  char buf[48];
  std::snprintf(buf, sizeof(buf), "%g", v);
  return std::string(buf);
}

}  // namespace bagua

// ---------------------------------------------------------------------------------
// CUDA / NCCL checks (only meaningful in translation units that include the headers)
// ---------------------------------------------------------------------------------
#define BAGUA_CUDA_CHECK(expr)                                                              \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) {                                                                \
      throw ::bagua::BaguaError(::bagua::ErrorKind::Backend,                                \
                                std::string("CUDA call failed: ") + #expr + " -> " +        \
                                    cudaGetErrorString(_e) + " (" + __FILE__ + ":" +        \
                                    std::to_string(__LINE__) + ")");                        \
    }                                                                                       \
  } while (0)

#define BAGUA_NCCL_CHECK(expr)                                                              \
  do {                                                                                      \
    ncclResult_t _r = (expr);                                                               \
    if (_r != ncclSuccess && _r != ncclInProgress) {                                        \
      throw ::bagua::BaguaError(::bagua::ErrorKind::Communicator,                           \
                                std::string("NCCL call failed: ") + #expr + " -> " +        \
                                    ncclGetErrorString(_r) + " (" + __FILE__ + ":" +        \
                                    std::to_string(__LINE__) + ")");                        \
    }                                                                                       \
  } while (0)

#define BAGUA_CHECK(cond, kind, msg)                                              \
  do {                                                                            \
    if (!(cond)) {                                                                \
      std::ostringstream _oss;                                                    \
      _oss << msg;                                                                \
      throw ::bagua::BaguaError(::bagua::ErrorKind::kind, _oss.str());            \
    }                                                                             \
  } while (0)
