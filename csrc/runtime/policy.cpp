// Size -> (algorithm, CTA budget) policy of the collectives.
//
// Capability parity: the reference's tuning policy
// (src/comm/tuning/tuning_policy.cpp:365-844): a JSON file named by an
// environment variable (here OOB_TUNING_POLICY, else ./oob_collective_policy.json),
// nearest measured point in log-ratio of the message size, environment caps on
// the CTA budget (OOB_MAX_CTAS), and a built-in default when no file exists.
// A point here also names the algorithm (one-shot / two-shot / NVLS), which
// the reference's planner derived from topology instead.
//
// File format:
//   {"points": [{"world": 8, "collective": "allreduce", "nvls": 1,
//                "bytes": 1048576, "algo": 2, "ctas": 16}, ...]}
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../api/oob.h"
#include "errors.h"
#include "log.h"

namespace oob {
namespace {

struct Point {
  int world, collective, nvls;
  double bytes;
  int algo, ctas;
};

std::mutex g_mu;
std::vector<Point> g_points;
bool g_loaded = false;

// ---- a JSON reader just big enough for the policy file ---------------------
struct Reader {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  std::string str() {
    ws();
    std::string s;
    if (p >= end || *p != '"') {
      ok = false;
      return s;
    }
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) ++p;
      s.push_back(*p++);
    }
    if (p < end) ++p; else ok = false;
    return s;
  }
  double num() {
    ws();
    char* e = nullptr;
    const double v = std::strtod(p, &e);
    if (e == p) ok = false;
    p = e;
    return v;
  }
  void skip_value() {
    ws();
    if (p >= end) {
      ok = false;
      return;
    }
    if (*p == '"') {
      str();
    } else if (*p == '{') {
      ++p;
      if (eat('}')) return;
      do {
        str();
        if (!eat(':')) ok = false;
        skip_value();
      } while (ok && eat(','));
      if (!eat('}')) ok = false;
    } else if (*p == '[') {
      ++p;
      if (eat(']')) return;
      do skip_value(); while (ok && eat(','));
      if (!eat(']')) ok = false;
    } else if (!std::strncmp(p, "true", 4)) {
      p += 4;
    } else if (!std::strncmp(p, "false", 5)) {
      p += 5;
    } else if (!std::strncmp(p, "null", 4)) {
      p += 4;
    } else {
      num();
    }
  }
};

int collective_id(const std::string& s) {
  if (s == "allreduce" || s == "all_reduce") return 0;
  if (s == "reduce_scatter" || s == "reducescatter") return 1;
  if (s == "all_gather" || s == "allgather") return 2;
  return -1;
}

bool parse_policy(const std::string& text, std::vector<Point>* out, std::string* err) {
  Reader r{text.data(), text.data() + text.size()};
  if (!r.eat('{')) {
    *err = "policy: expected an object";
    return false;
  }
  if (r.eat('}')) return true;
  do {
    const std::string key = r.str();
    if (!r.eat(':')) r.ok = false;
    if (key != "points") {
      r.skip_value();
      continue;
    }
    if (!r.eat('[')) {
      *err = "policy: \"points\" must be an array";
      return false;
    }
    if (r.eat(']')) continue;
    do {
      if (!r.eat('{')) {
        r.ok = false;
        break;
      }
      Point pt{0, -1, 0, 0.0, -1, 0};
      if (!r.eat('}')) {
        do {
          const std::string k = r.str();
          if (!r.eat(':')) r.ok = false;
          if (k == "collective") {
            pt.collective = collective_id(r.str());
          } else if (k == "world") {
            pt.world = static_cast<int>(r.num());
          } else if (k == "nvls") {
            pt.nvls = static_cast<int>(r.num());
          } else if (k == "bytes") {
            pt.bytes = r.num();
          } else if (k == "algo") {
            pt.algo = static_cast<int>(r.num());
          } else if (k == "ctas") {
            pt.ctas = static_cast<int>(r.num());
          } else {
            r.skip_value();
          }
        } while (r.ok && r.eat(','));
        if (!r.eat('}')) r.ok = false;
      }
      if (pt.world < 1 || pt.collective < 0 || pt.bytes <= 0 || pt.algo < 0 || pt.ctas < 1) {
        *err = "policy: a point is missing world / collective / bytes / algo / ctas";
        return false;
      }
      out->push_back(pt);
    } while (r.ok && r.eat(','));
    if (!r.eat(']')) r.ok = false;
  } while (r.ok && r.eat(','));
  if (!r.ok) {
    *err = "policy: malformed JSON";
    return false;
  }
  return true;
}

bool load_file(const char* path, std::string* err) {
  FILE* f = std::fopen(path, "rb");
  if (f == nullptr) {
    *err = std::string("policy: cannot open ") + path;
    return false;
  }
  std::string text;
  char buf[4096];
  size_t n;
  while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
  std::fclose(f);
  std::vector<Point> pts;
  if (!parse_policy(text, &pts, err)) return false;
  g_points.swap(pts);
  return true;
}

void ensure_loaded() {
  if (g_loaded) return;
  g_loaded = true;
  std::string err;
  const char* env = std::getenv("OOB_TUNING_POLICY");
  if (env != nullptr && *env) {
    load_file(env, &err);
    return;
  }
  FILE* f = std::fopen("oob_collective_policy.json", "rb");
  if (f != nullptr) {
    std::fclose(f);
    load_file("oob_collective_policy.json", &err);
  }
}

// Built-in choice when no measured point applies.
void builtin(int world, int collective, uint64_t bytes, int nvls, int* algo, int* ctas) {
  (void)world;
  int c;
  if (bytes <= (64u << 10)) c = 4;
  else if (bytes <= (512u << 10)) c = 8;
  else if (bytes <= (4u << 20)) c = 16;
  else if (bytes <= (64u << 20)) c = 32;
  else c = 48;
  *ctas = c;
  if (collective == 0) {
    if (bytes <= (256u << 10)) *algo = nvls ? OOB_AR_ONESHOT_NVLS : OOB_AR_ONESHOT_P2P;
    else *algo = nvls ? OOB_AR_TWOSHOT_NVLS : OOB_AR_TWOSHOT_P2P;
  } else if (collective == 1) {
    *algo = nvls ? OOB_RS_NVLS : OOB_RS_P2P;
  } else {
    *algo = nvls ? OOB_AG_PUSH_NVLS : OOB_AG_PUSH_P2P;
  }
}

}  // namespace
}  // namespace oob

extern "C" {

int oob_policy_load(const char* json_path) {
  using namespace oob;
  std::lock_guard<std::mutex> g(g_mu);
  g_loaded = true;
  if (json_path == nullptr || !*json_path) {
    g_points.clear();
    return OOB_OK;
  }
  std::string err;
  if (!load_file(json_path, &err)) return set_error(OOB_ERR_INVALID, err);
  OOB_LOG(kLogInfo, "tuning policy %s: %zu points", json_path, g_points.size());
  return OOB_OK;
}

int oob_policy_select(int world, int collective, uint64_t bytes, int nvls, int* algo, int* ctas) {
  using namespace oob;
  if (algo == nullptr || ctas == nullptr || collective < 0 || collective > 2)
    return set_error(OOB_ERR_INVALID, "bad argument");
  std::lock_guard<std::mutex> g(g_mu);
  ensure_loaded();
  const Point* best = nullptr;
  double best_d = 0;
  for (const Point& p : g_points) {
    if (p.world != world || p.collective != collective || (p.nvls != 0) != (nvls != 0)) continue;
    const double d = std::fabs(std::log(double(bytes > 0 ? bytes : 1) / p.bytes));
    if (best == nullptr || d < best_d) {
      best = &p;
      best_d = d;
    }
  }
  if (best != nullptr) {
    *algo = best->algo;
    *ctas = best->ctas;
  } else {
    builtin(world, collective, bytes, nvls, algo, ctas);
  }
  const char* cap = std::getenv("OOB_MAX_CTAS");
  if (cap != nullptr) {
    const int v = std::atoi(cap);
    if (v > 0 && *ctas > v) *ctas = v;
  }
  return OOB_OK;
}

}  // extern "C"
