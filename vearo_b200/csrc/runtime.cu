// Context, device-memory arena and the refcounted slot table.
//
// Replaces the device singleton, slot table, exact-size free list and hooks of the reference's
// CUDA backend (crates/vearo-backend-cuda/src/lib.rs:17-163).  Differences by design:
//   * the arena caches freed blocks by rounded size and hands them back without zero-filling
//     (the reference memsets every allocation, lib.rs:41-112); ops that need zeros ask for them;
//   * all work is ordered on one compute stream, so a freed block can be reused by the very next
//     launch without an event;
//   * errors are status codes, never panics.
#include "common.h"
#include <map>
#include <mutex>

namespace vb {

static Ctx g_ctx;
int64_t g_launcher_calls = 0;
Ctx& ctx() { return g_ctx; }

static thread_local std::string t_err;
int set_error(int status, const std::string& msg) { t_err = msg; return status; }

// ---- arena --------------------------------------------------------------------------------
struct Arena {
  std::multimap<size_t, void*> free_blocks;       // rounded size -> block
  std::map<void*, size_t> sizes;                  // every block ever cudaMalloc'ed -> rounded size
  size_t cached = 0, live = 0, peak = 0;
};
// Library-lifetime objects live on the heap and are never destroyed: tensors owned by other
// translation units may release slots during process exit, after static destructors would have run.
static Arena& g_arena = *new Arena();

static size_t round_size(size_t bytes) {
  if (bytes < 512) return 512;
  if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);
  return (bytes + (2u << 20) - 1) & ~size_t((2u << 20) - 1);       // 2 MiB granules above 1 MiB
}

static int arena_alloc(size_t bytes, void** p) {
  size_t r = round_size(bytes);
  auto it = g_arena.free_blocks.lower_bound(r);
  // accept a cached block up to 12.5 % larger than asked
  if (it != g_arena.free_blocks.end() && it->first <= r + r / 8) {
    *p = it->second;
    g_arena.cached -= it->first;
    g_arena.live += it->first;
    g_arena.free_blocks.erase(it);
  } else {
    cudaError_t e = cudaMalloc(p, r);
    if (e != cudaSuccess) {
      // give cached blocks back to the driver and retry once
      cudaGetLastError();
      cudaStreamSynchronize(g_ctx.stream);
      for (auto& kv : g_arena.free_blocks) { cudaFree(kv.second); g_arena.sizes.erase(kv.second); }
      g_arena.free_blocks.clear(); g_arena.cached = 0;
      e = cudaMalloc(p, r);
      if (e != cudaSuccess) { cudaGetLastError(); return set_error(VB_ERR_OOM, "device allocation of " + std::to_string(r) + " bytes failed"); }
    }
    g_arena.sizes[*p] = r;
    g_arena.live += r;
  }
  if (g_arena.live > g_arena.peak) g_arena.peak = g_arena.live;
  return VB_OK;
}
static void arena_free(void* p) {
  auto it = g_arena.sizes.find(p);
  if (it == g_arena.sizes.end()) return;
  g_arena.free_blocks.emplace(it->second, p);
  g_arena.cached += it->second;
  g_arena.live -= it->second;
}
int scratch_alloc(size_t bytes, void** p) { return arena_alloc(bytes ? bytes : 4, p); }
void scratch_free(void* p) { arena_free(p); }

// ---- slots --------------------------------------------------------------------------------
struct Slot { float* ptr = nullptr; i64 numel = 0; int refs = 0; uint64_t serial = 0; void (*ext_free)(void*) = nullptr; };     // ext_free: memory that is not the arena's
static uint64_t g_serial = 0;
static std::vector<Slot>& g_slots = *new std::vector<Slot>(1);       // slot 0 = none
static std::vector<vb_slot>& g_free_ids = *new std::vector<vb_slot>();
static i64 g_live_slots = 0;

int slot_alloc(i64 n, bool zero, vb_slot* out) {
  if (!g_ctx.ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  if (n < 0) return set_error(VB_ERR_INVALID, "negative numel");
  void* p = nullptr;
  VB_TRY(arena_alloc((size_t)(n > 0 ? n : 1) * sizeof(float), &p));
  if (zero && n > 0) VB_CUDA(cudaMemsetAsync(p, 0, (size_t)n * sizeof(float), g_ctx.stream));
  vb_slot id;
  if (!g_free_ids.empty()) { id = g_free_ids.back(); g_free_ids.pop_back(); }
  else { id = (vb_slot)g_slots.size(); g_slots.emplace_back(); }
  g_slots[id].ptr = (float*)p; g_slots[id].numel = n; g_slots[id].refs = 1; g_slots[id].serial = ++g_serial; g_slots[id].ext_free = nullptr;
  ++g_live_slots;
  *out = id;
  return VB_OK;
}
// A slot over memory obtained elsewhere (a buffer registered with the communication library): released through free_fn.
int slot_adopt_external(float* p, i64 n, void (*free_fn)(void*), vb_slot* out) {
  if (!g_ctx.ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  if (!p || n <= 0 || !free_fn) return set_error(VB_ERR_INVALID, "bad external buffer");
  vb_slot id;
  if (!g_free_ids.empty()) { id = g_free_ids.back(); g_free_ids.pop_back(); }
  else { id = (vb_slot)g_slots.size(); g_slots.emplace_back(); }
  g_slots[id].ptr = p; g_slots[id].numel = n; g_slots[id].refs = 1; g_slots[id].serial = ++g_serial; g_slots[id].ext_free = free_fn;
  ++g_live_slots;
  *out = id;
  return VB_OK;
}
static int slot_get(vb_slot s, Slot** out) {
  if (s == 0 || s >= g_slots.size() || g_slots[s].refs <= 0) return set_error(VB_ERR_INVALID, "bad or released slot " + std::to_string(s));
  *out = &g_slots[s];
  return VB_OK;
}
int slot_ptr(vb_slot s, float** p, i64* n) {
  Slot* sl; VB_TRY(slot_get(s, &sl));
  *p = sl->ptr; if (n) *n = sl->numel;
  return VB_OK;
}
uint64_t slot_serial(vb_slot s) { return (s == 0 || s >= g_slots.size()) ? 0 : g_slots[s].serial; }
void slot_touch(vb_slot s) { if (s != 0 && s < g_slots.size()) g_slots[s].serial = ++g_serial; }
int slot_retain(vb_slot s) { Slot* sl; VB_TRY(slot_get(s, &sl)); ++sl->refs; return VB_OK; }
int slot_release(vb_slot s, int* freed) {
  Slot* sl; VB_TRY(slot_get(s, &sl));
  if (freed) *freed = 0;
  if (--sl->refs == 0) {
    lo_plane_on_release(s);
    if (sl->ext_free) { sl->ext_free(sl->ptr); sl->ext_free = nullptr; } else arena_free(sl->ptr);
    sl->ptr = nullptr; sl->numel = 0;
    g_free_ids.push_back(s);
    --g_live_slots;
    if (freed) *freed = 1;
  }
  return VB_OK;
}

int tensor_ptr(const vb_tensor* t, float** p) {
  if (!t) return set_error(VB_ERR_INVALID, "null tensor");
  if (t->rank < 0 || t->rank > VB_MAX_RANK) return set_error(VB_ERR_INVALID, "rank out of range");
  float* base; i64 n;
  VB_TRY(slot_ptr(t->slot, &base, &n));
  // bounds of the view inside the slot
  i64 lo = t->offset, hi = t->offset;
  bool empty = false;
  for (int i = 0; i < t->rank; ++i) {
    if (t->dims[i] < 0) return set_error(VB_ERR_INVALID, "negative dim");
    if (t->dims[i] == 0) empty = true;
    else if (t->strides[i] >= 0) hi += (t->dims[i] - 1) * t->strides[i];
    else lo += (t->dims[i] - 1) * t->strides[i];
  }
  if (!empty && (lo < 0 || hi >= n)) return set_error(VB_ERR_INVALID, "view exceeds its slot");
  *p = base + t->offset;
  return VB_OK;
}

int new_output(vb_tensor* out, int rank, const i64* dims, bool zero) {
  if (!out) return set_error(VB_ERR_INVALID, "null output tensor");
  set_contiguous(*out, rank, dims);
  return slot_alloc(numel(*out), zero, &out->slot);
}

int contiguous_ptr(const vb_tensor* t, const float** p, Temp& hold) {
  float* base; VB_TRY(tensor_ptr(t, &base));
  if (is_contiguous(*t)) { *p = base; return VB_OK; }
  i64 n = numel(*t);
  VB_TRY(scratch_alloc((size_t)(n > 0 ? n : 1) * sizeof(float), &hold.p));
  Strided s{}; s.rank = t->rank;
  for (int i = 0; i < t->rank; ++i) { s.dims[i] = t->dims[i]; s.sa[i] = t->strides[i]; }
  if (n > 0) VB_TRY(launch_strided_copy(base, (float*)hold.p, n, s));
  *p = (const float*)hold.p;
  return VB_OK;
}

#ifdef VB200_BOUNDS_CHECK
std::vector<void (*)(int*)>& bc_setters() { static auto* v = new std::vector<void (*)(int*)>(); return *v; }
void bc_register(void (*setter)(int*)) { bc_setters().push_back(setter); }
#endif
}  // namespace vb

using namespace vb;

extern "C" {

const char* vb_last_error(void) { return t_err.c_str(); }

int vb_init(int device_ordinal) {
  if (g_ctx.ready) {
    if (g_ctx.device == device_ordinal) return VB_OK;
    return set_error(VB_ERR_INVALID, "already initialised on another device");
  }
  int count = 0;
  VB_CUDA(cudaGetDeviceCount(&count));
  if (device_ordinal < 0 || device_ordinal >= count) return set_error(VB_ERR_INVALID, "no such CUDA device");
  VB_CUDA(cudaSetDevice(device_ordinal));
  cudaDeviceProp prop;
  VB_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10) return set_error(VB_ERR_UNSUPPORTED, std::string("this library holds sm_100a code only; device is sm_") + std::to_string(prop.major) + std::to_string(prop.minor));
  g_ctx.device = device_ordinal;
  g_ctx.sm_count = prop.multiProcessorCount;
  VB_CUDA(cudaStreamCreateWithFlags(&g_ctx.stream, cudaStreamNonBlocking));
  VB_CUDA(cudaStreamCreateWithFlags(&g_ctx.comm_stream, cudaStreamNonBlocking));
  VB_CUDA(cudaEventCreateWithFlags(&g_ctx.ev_compute, cudaEventDisableTiming));
  VB_CUDA(cudaEventCreateWithFlags(&g_ctx.ev_comm, cudaEventDisableTiming));
  VB_CUDA(cudaMalloc(&g_ctx.d_err, sizeof(int)));
  VB_CUDA(cudaMemset(g_ctx.d_err, 0, sizeof(int)));
  VB_CUDA(cudaMalloc(&g_ctx.d_scalars, 64 * sizeof(float)));
  VB_CUDA(cudaMemset(g_ctx.d_scalars, 0, 64 * sizeof(float)));
  VB_CUDA(cudaMallocHost(&g_ctx.h_pinned, 64 * sizeof(float)));
#ifdef VB200_BOUNDS_CHECK
  for (void (*set)(int*) : bc_setters()) set(g_ctx.d_err);          // every translation unit learns where the error word is
  VB_CUDA(cudaGetLastError());
#endif
  g_ctx.ready = true;
  return VB_OK;
}

int vb_shutdown(void) {
  if (!g_ctx.ready) return VB_OK;
  cudaStreamSynchronize(g_ctx.stream);
  cudaStreamSynchronize(g_ctx.comm_stream);
  lo_planes_forget_all();
  for (auto& kv : g_arena.sizes) cudaFree(kv.first);
  g_arena.free_blocks.clear(); g_arena.sizes.clear(); g_arena.cached = g_arena.live = g_arena.peak = 0;
  g_slots.assign(1, Slot()); g_free_ids.clear(); g_live_slots = 0;
  cudaFree(g_ctx.d_err); cudaFree(g_ctx.d_scalars); cudaFreeHost(g_ctx.h_pinned);
  cudaEventDestroy(g_ctx.ev_compute); cudaEventDestroy(g_ctx.ev_comm);
  cudaStreamDestroy(g_ctx.stream); cudaStreamDestroy(g_ctx.comm_stream);
  g_ctx = Ctx();
  return VB_OK;
}

int vb_device_ordinal(int* ordinal) {
  if (!g_ctx.ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  *ordinal = g_ctx.device; return VB_OK;
}
int vb_sync(void) {
  if (!g_ctx.ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  VB_TRY(dp_wait_pending());      // a collective still unchecked gets its deadline here, not an unbounded wait below
  VB_CUDA(cudaStreamSynchronize(g_ctx.stream));
  return VB_OK;
}
int vb_stream(void** stream) {
  if (!g_ctx.ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  *stream = (void*)g_ctx.stream; return VB_OK;
}
int vb_check_errors(void) {
  if (!g_ctx.ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  int h = 0;
  VB_CUDA(cudaMemcpyAsync(&h, g_ctx.d_err, sizeof(int), cudaMemcpyDeviceToHost, g_ctx.stream));
  VB_CUDA(cudaStreamSynchronize(g_ctx.stream));
  if (h) {
    VB_CUDA(cudaMemsetAsync(g_ctx.d_err, 0, sizeof(int), g_ctx.stream));
    if (h & ERRBIT_WAIT_TIMEOUT) VB_TRY(gemm_tc_reset_state());
    std::string m;
    if (h & ERRBIT_NEG_ID) m += "Token ID / target class cannot be negative; ";
    if (h & ERRBIT_OOB_ID) m += "Token ID / target class out of bounds; ";
    if (h & ERRBIT_WAIT_TIMEOUT) m += "a device-side wait ran out; ";
    if (h & ERRBIT_BOUNDS) m += "a computed index left its tensor (bounds-check build); ";
    return set_error(VB_ERR_BAD_INDEX, m);
  }
  return VB_OK;
}

int vb_launch_count(int64_t* n) { *n = g_launcher_calls; return VB_OK; }
int vb_tc_launch_count(int64_t* n) { *n = g_tc_launches; return VB_OK; }
int vb_alloc(int64_t n, int zero_fill, vb_slot* out) { return slot_alloc(n, zero_fill != 0, out); }
int vb_retain(vb_slot s) { return slot_retain(s); }
int vb_release(vb_slot s, int* freed) { return slot_release(s, freed); }
int vb_ptr(vb_slot s, void** p) { float* f; VB_TRY(slot_ptr(s, &f)); *p = f; return VB_OK; }
int vb_slot_numel(vb_slot s, int64_t* n) { float* f; return slot_ptr(s, &f, n); }

int vb_write(vb_slot s, int64_t offset, const float* host, int64_t n) {
  float* p; i64 cap; VB_TRY(slot_ptr(s, &p, &cap));
  VB_CHECK(offset >= 0 && n >= 0 && offset + n <= cap, "range exceeds the slot");
  if (n) VB_CUDA(cudaMemcpyAsync(p + offset, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, g_ctx.stream));
  slot_touch(s);
  return VB_OK;
}
int vb_read(vb_slot s, int64_t offset, float* host, int64_t n) {
  float* p; i64 cap; VB_TRY(slot_ptr(s, &p, &cap));
  VB_CHECK(offset >= 0 && n >= 0 && offset + n <= cap, "range exceeds the slot");
  VB_TRY(dp_wait_pending());
  if (n) VB_CUDA(cudaMemcpyAsync(host, p + offset, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost, g_ctx.stream));
  VB_CUDA(cudaStreamSynchronize(g_ctx.stream));
  return VB_OK;
}
int vb_memory_stats(int64_t* live_slots, int64_t* live_bytes, int64_t* cached_bytes, int64_t* peak_bytes) {
  if (live_slots) *live_slots = g_live_slots;
  if (live_bytes) *live_bytes = (int64_t)g_arena.live;
  if (cached_bytes) *cached_bytes = (int64_t)g_arena.cached;
  if (peak_bytes) *peak_bytes = (int64_t)g_arena.peak;
  return VB_OK;
}
int vb_memory_reset_peak(void) { g_arena.peak = g_arena.live; return VB_OK; }

}  // extern "C"
