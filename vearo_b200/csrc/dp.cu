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
} g_nccl;
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
  return VB_OK;
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
  if (g_comm) { cudaStreamSynchronize(ctx().comm_stream); g_nccl.CommDestroy(g_comm); g_comm = nullptr; }
  g_world = 1; g_rank = 0;
  return VB_OK;
}

}  // extern "C"
