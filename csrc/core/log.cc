#include "log.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <unistd.h>

#include <atomic>
#include <mutex>

#include "uccl.h"

namespace uccl {

namespace {
std::atomic<int> g_level{-1};
std::atomic<int> g_rank{-1};
FILE* g_sink = nullptr;
std::mutex g_mu;

int parseLevel(const char* s) {
  if (!s || !*s) return LOG_ERROR;
  if (!strcasecmp(s, "NONE")) return LOG_NONE;
  if (!strcasecmp(s, "ERROR")) return LOG_ERROR;
  if (!strcasecmp(s, "WARN")) return LOG_WARN;
  if (!strcasecmp(s, "INFO")) return LOG_INFO;
  if (!strcasecmp(s, "TRACE")) return LOG_TRACE;
  return LOG_ERROR;
}
const char* levelName(int l) {
  switch (l) {
    case LOG_ERROR: return "ERROR";
    case LOG_WARN: return "WARN";
    case LOG_INFO: return "INFO";
    case LOG_TRACE: return "TRACE";
    default: return "NONE";
  }
}
}  // namespace

int logLevel() {
  int l = g_level.load(std::memory_order_relaxed);
  if (l >= 0) return l;
  std::lock_guard<std::mutex> lk(g_mu);
  l = g_level.load(std::memory_order_relaxed);
  if (l >= 0) return l;
  l = parseLevel(getenv("UCCL_DEBUG"));
  const char* f = getenv("UCCL_DEBUG_FILE");
  if (f && *f) {
    char path[512];
    snprintf(path, sizeof(path), "%s.%d", f, (int)getpid());
    g_sink = fopen(path, "a");
  }
  g_level.store(l, std::memory_order_relaxed);
  return l;
}

void logSetRank(int rank) { g_rank.store(rank, std::memory_order_relaxed); }

void logPrint(int level, const char* file, int line, const char* fmt, ...) {
  char msg[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  FILE* out = g_sink ? g_sink : stderr;
  std::lock_guard<std::mutex> lk(g_mu);
  int r = g_rank.load(std::memory_order_relaxed);
  if (r >= 0)
    fprintf(out, "[UCCL %s r%d] %s:%d %s\n", levelName(level), r, base, line, msg);
  else
    fprintf(out, "[UCCL %s] %s:%d %s\n", levelName(level), base, line, msg);
  fflush(out);
}

void logBanner() {
  static std::once_flag once;
  std::call_once(once, [] {
    UCCL_LOG(INFO, "unified collective library for sm_100a, version %d.%d.%d", UCCL_MAJOR, UCCL_MINOR,
             UCCL_PATCH);
  });
}

}  // namespace uccl
