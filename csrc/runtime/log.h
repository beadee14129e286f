// Levelled logging of the native runtime.
//
// OOB_LOG_LEVEL = error | warn (default) | info | debug (or 0..3) selects what is written; records go to stderr as
// "[oob <level>] message" or to the sink installed with oob_set_log_sink (the Python package forwards them to its
// `logging` logger).  Every failing entry point also logs its error message at level info, so a log shows failures
// even when the caller drops the return code.
//
// Capability parity: the reference's OO_LOG / per-module verbosity (include/ooverlap/system/logging.h) and the
// peer-access diagnostics of src/comm/p2p_access.cu.
#pragma once
#include <cstdarg>

namespace oob {
enum LogLevel : int { kLogError = 0, kLogWarn = 1, kLogInfo = 2, kLogDebug = 3 };
int log_level();
void log_write(int level, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
}  // namespace oob

#define OOB_LOG(level, ...)                                             \
  do {                                                                  \
    if ((level) <= ::oob::log_level()) ::oob::log_write(level, __VA_ARGS__); \
  } while (0)
