// Leveled logging to stderr (or UCCL_DEBUG_FILE), level taken once from UCCL_DEBUG
// (NONE / ERROR / WARN / INFO / TRACE, default ERROR) -- same variable and levels as the
// reference's macro (src/misc/debug.h:18-50), plus a rank prefix and an optional file sink.
#pragma once
#include <stdarg.h>

namespace uccl {

enum LogLevel : int { LOG_NONE = 0, LOG_ERROR = 1, LOG_WARN = 2, LOG_INFO = 3, LOG_TRACE = 4 };

int logLevel();
void logSetRank(int rank);
void logPrint(int level, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 4, 5)));
// Prints the version banner once at INFO level.
void logBanner();

}  // namespace uccl

#define UCCL_LOG(LEVEL, ...)                                                       \
  do {                                                                             \
    if (::uccl::logLevel() >= ::uccl::LOG_##LEVEL)                                 \
      ::uccl::logPrint(::uccl::LOG_##LEVEL, __FILE__, __LINE__, __VA_ARGS__);      \
  } while (0)
