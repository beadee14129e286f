// See log.h.
#include "log.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../api/oob.h"

namespace oob {
namespace {
std::atomic<int> g_level{-1};  // -1 = not read from the environment yet
std::atomic<oob_log_sink_t> g_sink{nullptr};
std::mutex g_write_mu;

int level_from_env() {
  const char* v = std::getenv("OOB_LOG_LEVEL");
  if (v == nullptr || *v == 0) return kLogWarn;
  if (!std::strcmp(v, "error") || !std::strcmp(v, "fatal") || !std::strcmp(v, "0")) return kLogError;
  if (!std::strcmp(v, "warn") || !std::strcmp(v, "warning") || !std::strcmp(v, "1")) return kLogWarn;
  if (!std::strcmp(v, "info") || !std::strcmp(v, "2")) return kLogInfo;
  if (!std::strcmp(v, "debug") || !std::strcmp(v, "trace") || !std::strcmp(v, "3")) return kLogDebug;
  return kLogWarn;
}
const char* const kNames[] = {"error", "warn", "info", "debug"};
}  // namespace

int log_level() {
  int l = g_level.load(std::memory_order_relaxed);
  if (l < 0) {
    l = level_from_env();
    g_level.store(l, std::memory_order_relaxed);
  }
  return l;
}

void log_write(int level, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (level < kLogError) level = kLogError;
  if (level > kLogDebug) level = kLogDebug;
  oob_log_sink_t sink = g_sink.load(std::memory_order_acquire);
  if (sink != nullptr) {
    sink(level, buf);
    return;
  }
  std::lock_guard<std::mutex> g(g_write_mu);
  std::fprintf(stderr, "[oob %s] %s\n", kNames[level], buf);
}
}  // namespace oob

extern "C" int oob_set_log_level(int level) {
  if (level < oob::kLogError || level > oob::kLogDebug) return OOB_ERR_INVALID;
  oob::g_level.store(level, std::memory_order_relaxed);
  return OOB_OK;
}

extern "C" int oob_get_log_level(void) { return oob::log_level(); }

extern "C" int oob_set_log_sink(oob_log_sink_t sink) {
  oob::g_sink.store(sink, std::memory_order_release);
  return OOB_OK;
}

extern "C" int oob_log_message(int level, const char* message) {
  if (message == nullptr) return OOB_ERR_INVALID;
  OOB_LOG(level, "%s", message);
  return OOB_OK;
}
