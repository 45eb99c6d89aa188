// Per-family kernel timing with CUDA events recorded on the compute stream (see ProfScope in
// common.h).  Used by the benchmark's untimed profiling pass to report each kernel family's
// average launch duration next to its algorithmic bytes / flops.
#include "common.h"
#include <cstring>
#include <map>

namespace vb {
namespace {
struct Rec { int family; cudaEvent_t a, b; double units, dense; };
bool g_on = false;
std::vector<std::string>& g_names = *new std::vector<std::string>();
std::vector<Rec>& g_recs = *new std::vector<Rec>();
std::vector<cudaEvent_t>& g_pool = *new std::vector<cudaEvent_t>();
cudaEvent_t get_event() {
  if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
  cudaEvent_t e; cudaEventCreate(&e); return e;
}
int family_id(const char* f) {
  for (size_t i = 0; i < g_names.size(); ++i) if (g_names[i] == f) return (int)i;
  g_names.push_back(f); return (int)g_names.size() - 1;
}
}  // namespace

ProfScope::ProfScope(const char* family, double units, double dense_units) {
  if (!g_on || g_recs.size() > 200000) return;
  Rec r; r.family = family_id(family); r.a = get_event(); r.b = get_event(); r.units = units; r.dense = dense_units > 0.0 ? dense_units : units;
  cudaEventRecord(r.a, ctx().stream);
  g_recs.push_back(r); idx = (int)g_recs.size() - 1;
}
ProfScope::~ProfScope() { if (idx >= 0) cudaEventRecord(g_recs[idx].b, ctx().stream); }
}  // namespace vb

using namespace vb;
extern "C" {
int vb_profile_enable(int on) { g_on = on != 0; return VB_OK; }
int vb_profile_reset(void) {
  if (ctx().ready) cudaStreamSynchronize(ctx().stream);
  for (Rec& r : g_recs) { g_pool.push_back(r.a); g_pool.push_back(r.b); }
  g_recs.clear();
  return VB_OK;
}
int vb_profile_read(const char* family, double* total_ms, int64_t* launches, double* units, double* dense_units) {
  if (!ctx().ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  VB_CUDA(cudaStreamSynchronize(ctx().stream));
  double ms = 0, u = 0, du = 0; int64_t n = 0;
  for (Rec& r : g_recs) {
    if (g_names[r.family] != family) continue;
    float t = 0; VB_CUDA(cudaEventElapsedTime(&t, r.a, r.b));
    ms += t; u += r.units; du += r.dense; ++n;
  }
  if (total_ms) *total_ms = ms; if (launches) *launches = n; if (units) *units = u; if (dense_units) *dense_units = du;
  return VB_OK;
}
int vb_profile_families(char* buf, int buflen) {
  std::string s;
  for (size_t i = 0; i < g_names.size(); ++i) { if (i) s += ","; s += g_names[i]; }
  if ((int)s.size() + 1 > buflen) return set_error(VB_ERR_INVALID, "buffer too small");
  std::memcpy(buf, s.c_str(), s.size() + 1);
  return VB_OK;
}
}
