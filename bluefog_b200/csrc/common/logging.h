// Stream-style logger: BFLOG(INFO) << "text"; BFLOG(DEBUG, rank) << ...
// Levels TRACE..FATAL; filtered by BLUEFOG_LOG_LEVEL, timestamps hidden with
// BLUEFOG_LOG_HIDE_TIME (reference behaviour: bluefog/common/logging.cc:30-108).
// TRACE..INFO go to stdout, WARNING and above to stderr, FATAL aborts.
#pragma once
#include <cstdio>
#include <string>
#include <type_traits>

namespace bfb {

enum class LogLevel : int { TRACE = 0, DEBUG = 1, INFO = 2, WARNING = 3, ERROR = 4, FATAL = 5 };

LogLevel MinLogLevelFromEnv();
bool LogHideTimeFromEnv();
LogLevel ParseLogLevel(const char* text);

// Minimal string builder with stream syntax.  It formats numbers with snprintf instead of
// iostream facets, which keeps the runtime independent of the process-global C++ locale.
class StrBuilder {
 public:
  StrBuilder& operator<<(const char* v) { buf_ += (v ? v : "(null)"); return *this; }
  StrBuilder& operator<<(const std::string& v) { buf_ += v; return *this; }
  StrBuilder& operator<<(char v) { buf_ += v; return *this; }
  StrBuilder& operator<<(bool v) { buf_ += (v ? "true" : "false"); return *this; }
  template <typename T, typename std::enable_if<std::is_arithmetic<T>::value, int>::type = 0>
  StrBuilder& operator<<(T v) {
    char tmp[48];
    if (std::is_floating_point<T>::value) std::snprintf(tmp, sizeof(tmp), "%g", static_cast<double>(v));
    else if (std::is_signed<T>::value) std::snprintf(tmp, sizeof(tmp), "%lld", static_cast<long long>(v));
    else std::snprintf(tmp, sizeof(tmp), "%llu", static_cast<unsigned long long>(v));
    buf_ += tmp;
    return *this;
  }
  const std::string& str() const { return buf_; }

 private:
  std::string buf_;
};

class LogMessage : public StrBuilder {
 public:
  LogMessage(const char* file, int line, LogLevel level, int rank = -1);
  ~LogMessage();

 private:
  const char* file_;
  int line_;
  LogLevel level_;
  int rank_;
};

#define BFB_LOG_AT(level, ...) \
  if (static_cast<int>(::bfb::LogLevel::level) >= static_cast<int>(::bfb::MinLogLevelFromEnv())) \
  ::bfb::LogMessage(__FILE__, __LINE__, ::bfb::LogLevel::level, ##__VA_ARGS__)
#define BFLOG(level, ...) BFB_LOG_AT(level, ##__VA_ARGS__)

}  // namespace bfb
