#include "logging.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>
#include <strings.h>

namespace bfb {

LogLevel ParseLogLevel(const char* text) {
  if (text == nullptr) return LogLevel::WARNING;
  static const struct { const char* name; LogLevel level; } table[] = {
      {"trace", LogLevel::TRACE}, {"debug", LogLevel::DEBUG}, {"info", LogLevel::INFO},
      {"warning", LogLevel::WARNING}, {"warn", LogLevel::WARNING},
      {"error", LogLevel::ERROR}, {"fatal", LogLevel::FATAL}};
  for (const auto& e : table)
    if (strcasecmp(text, e.name) == 0) return e.level;
  return LogLevel::WARNING;
}

LogLevel MinLogLevelFromEnv() {
  static LogLevel level = ParseLogLevel(std::getenv("BLUEFOG_LOG_LEVEL"));
  return level;
}

bool LogHideTimeFromEnv() {
  static bool hide = [] {
    const char* v = std::getenv("BLUEFOG_LOG_HIDE_TIME");
    return v != nullptr && std::strtol(v, nullptr, 10) > 0;
  }();
  return hide;
}

LogMessage::LogMessage(const char* file, int line, LogLevel level, int rank)
    : file_(file), line_(line), level_(level), rank_(rank) {}

LogMessage::~LogMessage() {
  static std::mutex mu;
  static const char kLetters[] = "TDIWEF";
  const char* base = std::strrchr(file_, '/');
  base = base ? base + 1 : file_;
  FILE* out = static_cast<int>(level_) <= static_cast<int>(LogLevel::INFO) ? stdout : stderr;
  char stamp[64] = "";
  if (!LogHideTimeFromEnv()) {
    auto now = std::chrono::system_clock::now();
    std::time_t secs = std::chrono::system_clock::to_time_t(now);
    long micros = static_cast<long>(
        std::chrono::duration_cast<std::chrono::microseconds>(now.time_since_epoch()).count() % 1000000);
    struct tm tmv;
    localtime_r(&secs, &tmv);
    char buf[32];
    std::strftime(buf, sizeof(buf), "%Y-%m-%d %H:%M:%S", &tmv);
    std::snprintf(stamp, sizeof(stamp), "%s.%06ld: ", buf, micros);
  }
  {
    std::lock_guard<std::mutex> g(mu);
    if (rank_ >= 0)
      std::fprintf(out, "[%s%c %s:%d] [%d]: %s\n", stamp, kLetters[static_cast<int>(level_)], base, line_,
                   rank_, str().c_str());
    else
      std::fprintf(out, "[%s%c %s:%d] %s\n", stamp, kLetters[static_cast<int>(level_)], base, line_,
                   str().c_str());
    std::fflush(out);
  }
  if (level_ == LogLevel::FATAL) std::abort();
}

}  // namespace bfb
