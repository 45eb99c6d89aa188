// Data-parallel gradient exchange over NCCL (NVLink 5 / NVSwitch), one process per GPU.
//
// New functionality: the reference is single-device (its CUDA backend opens device 0 only,
// crates/vearo-backend-cuda/src/lib.rs:20-24).  NCCL is loaded with dlopen at vb_dp_init so that
// the library has no link-time dependency on it.  Collectives run on a dedicated stream; each
// allreduce is ordered after the compute-stream work that produced its bucket through an event,
// and vb_dp_finish makes the compute stream wait for the last one — so buckets reduced early
// overlap the rest of the backward pass.  Failures never hang the host: completion is polled
// with a deadline and asynchronous NCCL errors abort the communicator.
#include "common.h"
#include <chrono>
#include <cstring>
#include <dlfcn.h>
#include <thread>
#include <unordered_map>

using namespace vb;

namespace {
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct Nccl {
  void* h = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  // optional (user-buffer registration): absent in old libraries, in which case gradients stay in ordinary memory
  int (*MemAlloc)(void**, size_t) = nullptr;
  int (*MemFree)(void*) = nullptr;
  int (*CommRegister)(ncclComm_t, void*, size_t, void**) = nullptr;
  int (*CommDeregister)(ncclComm_t, void*) = nullptr;
} g_nccl;
struct Registered { void* handle; size_t bytes; };
std::unordered_map<void*, Registered>& registered() { static auto* m = new std::unordered_map<void*, Registered>(); return *m; }
ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 1;

int load_nccl() {
  if (g_nccl.h) return VB_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) { g_nccl.h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (g_nccl.h) break; }
  if (!g_nccl.h) return set_error(VB_ERR_COMM, std::string("cannot load libnccl: ") + dlerror());
#define SYM(field, name) *(void**)(&g_nccl.field) = dlsym(g_nccl.h, name); if (!g_nccl.field) return set_error(VB_ERR_COMM, "libnccl lacks " name);
  SYM(GetUniqueId, "ncclGetUniqueId") SYM(CommInitRank, "ncclCommInitRank") SYM(AllReduce, "ncclAllReduce")
  SYM(CommDestroy, "ncclCommDestroy") SYM(CommAbort, "ncclCommAbort") SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
  *(void**)(&g_nccl.MemAlloc) = dlsym(g_nccl.h, "ncclMemAlloc"); *(void**)(&g_nccl.MemFree) = dlsym(g_nccl.h, "ncclMemFree");
  *(void**)(&g_nccl.CommRegister) = dlsym(g_nccl.h, "ncclCommRegister"); *(void**)(&g_nccl.CommDeregister) = dlsym(g_nccl.h, "ncclCommDeregister");
  return VB_OK;
}
// Releases a buffer made by vb_dp_alloc: nothing of either stream may still be using it.
void free_registered(void* p) {
  auto it = registered().find(p);
  if (it == registered().end()) return;
  cudaStreamSynchronize(ctx().comm_stream); cudaStreamSynchronize(ctx().stream);
  if (g_comm && g_nccl.CommDeregister && it->second.handle) g_nccl.CommDeregister(g_comm, it->second.handle);
  if (g_nccl.MemFree) g_nccl.MemFree(p);
  registered().erase(it);
}
bool registration_enabled() {
  static const bool on = [] { const char* e = getenv("VB200_DP_REGISTER"); return !(e && e[0] == '0'); }();
  return on;
}
int nccl_fail(const char* what, int rc) {
  return set_error(VB_ERR_COMM, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "nccl error"));
}
}  // namespace

extern "C" {

int vb_dp_unique_id(uint8_t id[128]) {
  VB_TRY(load_nccl());
  ncclUniqueId u;
  int rc = g_nccl.GetUniqueId(&u);
  if (rc != ncclSuccess) return nccl_fail("ncclGetUniqueId", rc);
  std::memcpy(id, u.internal, 128);
  return VB_OK;
}
int vb_dp_init(int rank, int world, const uint8_t id[128]) {
  if (!ctx().ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  VB_CHECK(world >= 1 && rank >= 0 && rank < world, "bad rank / world");
  g_rank = rank; g_world = world;
  if (world == 1) return VB_OK;
  VB_TRY(load_nccl());
  ncclUniqueId u; std::memcpy(u.internal, id, 128);
  int rc = g_nccl.CommInitRank(&g_comm, world, u, rank);
  if (rc != ncclSuccess) return nccl_fail("ncclCommInitRank", rc);
  return VB_OK;
}
// Memory for gradients that will be all-reduced in place.  With more than one rank it comes from the communication library's own
// allocator and is registered with the communicator, so that the NVLink-switch all-reduce can work on the buffer itself instead of
// staging it through its internal buffers; whenever that is not possible (one rank, an old library, a refusal) it is an ordinary slot.
int vb_dp_alloc(int64_t numel, int zero_fill, vb_slot* out) {
  if (!ctx().ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  VB_CHECK(numel >= 0 && out, "bad arguments");
  if (g_world > 1 && g_comm && numel > 0 && registration_enabled() && g_nccl.MemAlloc && g_nccl.MemFree && g_nccl.CommRegister) {
    void* p = nullptr;
    const size_t bytes = (size_t)numel * sizeof(float);
    if (g_nccl.MemAlloc(&p, bytes) == ncclSuccess && p) {
      void* handle = nullptr;
      if (g_nccl.CommRegister(g_comm, p, bytes, &handle) == ncclSuccess) {
        registered()[p] = Registered{handle, bytes};
        cudaError_t e = zero_fill ? cudaMemsetAsync(p, 0, bytes, ctx().stream) : cudaSuccess;
        if (e == cudaSuccess && slot_adopt_external((float*)p, numel, &free_registered, out) == VB_OK) return VB_OK;
        free_registered(p);
      } else g_nccl.MemFree(p);
    }
    cudaGetLastError();       // fall through to ordinary memory
  }
  return slot_alloc(numel, zero_fill != 0, out);
}
int vb_dp_is_registered(vb_slot slot, int* yes) {
  float* p; VB_TRY(slot_ptr(slot, &p));
  if (yes) *yes = registered().count((void*)p) ? 1 : 0;
  return VB_OK;
}
int vb_dp_world(int* rank, int* world) { if (rank) *rank = g_rank; if (world) *world = g_world; return VB_OK; }

int vb_dp_allreduce(vb_slot slot, int64_t offset, int64_t n) {
  float* p; i64 cap; VB_TRY(slot_ptr(slot, &p, &cap));
  VB_CHECK(offset >= 0 && n >= 0 && offset + n <= cap, "range exceeds the slot");
  if (g_world == 1 || n == 0) return VB_OK;
  if (!g_comm) return set_error(VB_ERR_COMM, "vb_dp_init has not been called");
  slot_touch(slot);                     // reduced in place: whatever was derived from the old contents (a lo plane) is void
  Ctx& c = ctx();
  VB_CUDA(cudaEventRecord(c.ev_compute, c.stream));
  VB_CUDA(cudaStreamWaitEvent(c.comm_stream, c.ev_compute, 0));
  int rc = g_nccl.AllReduce(p + offset, p + offset, (size_t)n, ncclFloat32, ncclSum, g_comm, c.comm_stream);
  if (rc != ncclSuccess) return nccl_fail("ncclAllReduce", rc);
  return VB_OK;
}
// Host-side wait for `ev` with a deadline, polling for asynchronous NCCL errors meanwhile.
static int wait_with_deadline(cudaEvent_t ev, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (true) {
    cudaError_t q = cudaEventQuery(ev);
    if (q == cudaSuccess) return VB_OK;
    if (q != cudaErrorNotReady) return set_error(VB_ERR_CUDA, cudaGetErrorString(q));
    int async_err = ncclSuccess;
    g_nccl.CommGetAsyncError(g_comm, &async_err);
    if (async_err != ncclSuccess && async_err != ncclInProgress) { g_nccl.CommAbort(g_comm); g_comm = nullptr; return nccl_fail("asynchronous NCCL error", async_err); }
    if (std::chrono::steady_clock::now() > deadline) { g_nccl.CommAbort(g_comm); g_comm = nullptr; return set_error(VB_ERR_COMM_TIMEOUT, "allreduce did not complete before the deadline"); }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}
// Deferred checks (vb_dp_finish with a negative deadline): the event of the step whose completion has not been looked at yet.
static cudaEvent_t g_ev_deferred[2] = {nullptr, nullptr};
static int g_deferred_at = 0, g_deferred_ms = 0;
static bool g_deferred_pending = false;
}  // extern "C"
namespace vb {
int dp_wait_pending() {
  if (!g_deferred_pending) return VB_OK;
  g_deferred_pending = false;
  if (!g_comm) return VB_OK;
  return wait_with_deadline(g_ev_deferred[g_deferred_at], g_deferred_ms);
}
}  // namespace vb
extern "C" {
int vb_dp_wait(void) { return dp_wait_pending(); }
int vb_dp_finish(int timeout_ms) {
  if (g_world == 1) return VB_OK;
  if (!g_comm) return set_error(VB_ERR_COMM, "vb_dp_init has not been called");
  Ctx& c = ctx();
  if (timeout_ms < 0) {
    // the previous step's collectives first (normally long complete: no waiting), then this step's are only enqueued
    VB_TRY(dp_wait_pending());
    if (!g_comm) return set_error(VB_ERR_COMM, "the communicator was aborted");
    const int at = g_deferred_at ^ 1;
    if (!g_ev_deferred[at]) VB_CUDA(cudaEventCreateWithFlags(&g_ev_deferred[at], cudaEventDisableTiming));
    VB_CUDA(cudaEventRecord(g_ev_deferred[at], c.comm_stream));
    VB_CUDA(cudaStreamWaitEvent(c.stream, g_ev_deferred[at], 0));
    g_deferred_at = at; g_deferred_ms = -timeout_ms; g_deferred_pending = true;
    return VB_OK;
  }
  VB_TRY(dp_wait_pending());
  if (!g_comm) return set_error(VB_ERR_COMM, "the communicator was aborted");
  VB_CUDA(cudaEventRecord(c.ev_comm, c.comm_stream));
  VB_CUDA(cudaStreamWaitEvent(c.stream, c.ev_comm, 0));
  if (timeout_ms > 0) return wait_with_deadline(c.ev_comm, timeout_ms);
  return VB_OK;
}
int vb_dp_shutdown(void) {
  g_deferred_pending = false;
  for (cudaEvent_t& e : g_ev_deferred) if (e) { cudaEventDestroy(e); e = nullptr; }
  if (g_comm) {
    cudaStreamSynchronize(ctx().comm_stream);
    for (auto& kv : registered()) if (g_nccl.CommDeregister && kv.second.handle) { g_nccl.CommDeregister(g_comm, kv.second.handle); kv.second.handle = nullptr; }
    g_nccl.CommDestroy(g_comm); g_comm = nullptr;
  }
  g_world = 1; g_rank = 0;
  return VB_OK;
}

}  // extern "C"
