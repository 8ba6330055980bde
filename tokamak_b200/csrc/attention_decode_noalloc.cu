// Split-K paged decode attention for callers that cannot allocate device memory.
//
// No counterpart in WeichunK/tokamak.  See tokamak_b200_noalloc.h for who needs it
// and for the contract.  The scratch of the decode kernel (unnormalised partial
// outputs and their (maximum, normaliser) pairs, one set per key split, and the
// counters by which the last split to arrive is found) lives in the file-scope
// device arrays below; the kernel itself is the one behind
// tk_attention_decode, reached through that exported function with the array's
// device address as its scratch argument.
#include <mutex>

#include "common.cuh"
#include "tokamak_b200_noalloc.h"

// The existing entry point (attention_decode.cu); it launches one kernel and allocates nothing.
extern "C" int tk_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                   float* scratch, int* counters, const int* items, const int* positions,
                                   const int* tok_req, const int* req_slot, const int* block_table,
                                   int* err, int n_items, int n_reqs, int n_q_heads, int n_kv_heads,
                                   int head_dim, int page_size, int max_pages, int num_pages, int window,
                                   int n_splits, float scale, cudaStream_t stream);

namespace {

constexpr long long kScratchFloats = 1ll << 20;   // 4 MiB on every GPU that loads the library
constexpr int kCounters = 4096;                   // arrival counters, one per (token, kv head)
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime, not a device address:
// the address comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) float g_decode_scratch[kScratchFloats];
// Zero when the library is loaded; every call leaves the counters it used at zero again.
static __device__ __align__(256) int g_decode_counters[kCounters];

float* g_scratch_ptr[kMaxDevices] = {nullptr};
int* g_counter_ptr[kMaxDevices] = {nullptr};
std::mutex g_lookup_mutex;

// Device addresses of the arrays on the current device, looked up once per device.  The table
// is read and filled under a mutex, so host threads may make their first calls at the same time.
int scratch_for_current_device(float** out, int** counters) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return TK_NOALLOC_BAD_DEVICE;
  std::lock_guard<std::mutex> lock(g_lookup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_decode_scratch);
    if (e != cudaSuccess) return (int)e;
    int* cptr = nullptr;
    e = cudaGetSymbolAddress((void**)&cptr, g_decode_counters);
    if (e != cudaSuccess) return (int)e;
    g_counter_ptr[dev] = cptr;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  *counters = g_counter_ptr[dev];
  return 0;
}

}  // namespace

TK_API long long tk_attention_decode_noalloc_capacity_floats(void) { return kScratchFloats; }

TK_API const char* tk_noalloc_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case TK_NOALLOC_TOO_LARGE:
      return "the call needs more scratch than the library's static array holds "
             "(n_items * n_q_heads * n_splits * (head_dim + 2) floats; see "
             "tk_attention_decode_noalloc_capacity_floats): use fewer splits or fewer items per call";
    case TK_NOALLOC_BAD_DEVICE: return "the current device's index is beyond the library's table";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

TK_API int tk_attention_decode_noalloc(const void* q, void* out, const void* k_cache,
                                       const void* v_cache, const int* items, const int* positions,
                                       const int* tok_req, const int* req_slot, const int* block_table,
                                       int* err, int n_items, int n_reqs, int n_q_heads, int n_kv_heads,
                                       int head_dim, int page_size, int max_pages, int num_pages,
                                       int window, int n_splits, float scale, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (n_q_heads < 1 || head_dim < 1 || n_splits < 1) return (int)cudaErrorInvalidValue;
  // a call with one split stores its result itself and touches neither array
  const long long need = (long long)n_items * n_q_heads * n_splits * (head_dim + 2);
  if (n_splits > 1 && (need > kScratchFloats || (long long)n_items * n_kv_heads > kCounters))
    return TK_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  int* counters = nullptr;
  const int rc = scratch_for_current_device(&scratch, &counters);
  if (rc != 0) return rc;
  return tk_attention_decode(q, out, k_cache, v_cache, scratch, counters, items, positions, tok_req, req_slot,
                             block_table, err, n_items, n_reqs, n_q_heads, n_kv_heads, head_dim,
                             page_size, max_pages, num_pages, window, n_splits, scale, stream);
}
