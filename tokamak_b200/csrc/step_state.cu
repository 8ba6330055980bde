// Per-request state on the device and the kernels that open a step.
//
// Every request slot has one fixed-size record of kSlotWords 32-bit words:
//
//   0  num_computed   positions of the request that the cache holds
//   1  rng_counter    tokens sampled for the request so far = index of its next draw
//   2  seed (low)     3  seed (high)
//   4  temperature    (float bits)      5  top_k      6  top_p (float bits)
//   7  last_token     the token sampled last, -1 before the first
//
// The reference keeps the same facts on the host: a position derived from the sequence's
// length (src/tokamak/engine/llm.py:373-375) and one torch.Generator per request that outlives
// preemption (llm.py:178,441-445,464).  Here they live beside the block tables, so a step of
// single next tokens needs nothing from the host but the list of slots that take part, and that
// only when it changed: the record gives the token, its position and the sampling parameters,
// the sampling kernel writes the new token back and advances the counter.
//
// What the host changes between steps (records of newly admitted requests, block-table entries
// of new or returned pages) travels as one list of updates in a buffer at a fixed address:
//   words 0, 1: number of record writes R and of table writes T (cleared by the kernel that
//               applied them, so a step without changes uploads nothing)
//   then R x (slot + (mask << 16), 8 words): word j of the record is written where bit j of the
//   mask is set; then T x (index into the flat block tables, page id).
// Both kernels below apply the list first.  They run as ONE block, so that the order
// "updates, then the step's own reads and writes of the records" is a __syncthreads().
#include "common.cuh"
#include "timeline.cuh"

namespace tk {

constexpr int kSlotWords = 8;
constexpr int kRecComputed = 0, kRecCounter = 1, kRecLastToken = 7;
constexpr int kBeginThreads = 256;

struct UpdateList {
  int* ctl;              // [2 + 9 * max_rec + 2 * max_tab]
  int max_rec, max_tab;
  int* records;          // [max_slots, kSlotWords]
  int max_slots;
  int* tables;           // all groups' block tables, flat
  long long tables_len;
};

__device__ __forceinline__ void apply_updates(const UpdateList& u, int* err) {
  const int n_rec = min(u.ctl[0], u.max_rec);
  const int n_tab = min(u.ctl[1], u.max_tab);
  const int* rec = u.ctl + 2;
  const int* tab = rec + 9 * n_rec;
  for (int i = threadIdx.x; i < n_rec * kSlotWords; i += blockDim.x) {
    const int w = i / kSlotWords, j = i % kSlotWords;
    const int slot = rec[9 * w] & 0xFFFF, mask = (rec[9 * w] >> 16) & 0xFF;
    if (slot >= u.max_slots) { set_error(err, kErrRequest, -1, slot, u.max_slots); continue; }
    if ((mask >> j) & 1) u.records[(size_t)slot * kSlotWords + j] = rec[9 * w + 1 + j];
  }
  for (int i = threadIdx.x; i < n_tab; i += blockDim.x) {
    const long long at = (long long)(unsigned int)tab[2 * i];
    if (at >= u.tables_len) { set_error(err, kErrPage, -1, tab[2 * i], (int)u.tables_len); continue; }
    u.tables[at] = tab[2 * i + 1];
  }
  __syncthreads();
  if (threadIdx.x == 0) { u.ctl[0] = 0; u.ctl[1] = 0; }
}

// Opens a step that the host laid out: applies the updates; gives every request marked in
// `req_fed` the token its record holds (the one sampled last, which the host may not have read
// yet); notes in every record how far the cache reaches after this step.
__global__ void __launch_bounds__(kBeginThreads)
step_begin_kernel(UpdateList u, int* __restrict__ token_ids, const int* __restrict__ req_q_start,
                  const int* __restrict__ req_kv_len, const int* __restrict__ req_slot,
                  const int* __restrict__ req_fed, int n_reqs, int n_tokens, int* err) {
  pdl_trigger();
  pdl_wait();
  apply_updates(u, err);
  __syncthreads();
  for (int r = threadIdx.x; r < n_reqs; r += blockDim.x) {
    const int slot = req_slot[r];
    if (slot < 0 || slot >= u.max_slots) { set_error(err, kErrRequest, r, slot, u.max_slots); continue; }
    int* rec = u.records + (size_t)slot * kSlotWords;
    if (req_fed != nullptr && req_fed[r]) {
      const int t = req_q_start[r];
      const int tok = rec[kRecLastToken];
      if (tok < 0 || t < 0 || t >= n_tokens) set_error(err, kErrTokenId, r, tok, slot);
      else token_ids[t] = tok;
    }
    rec[kRecComputed] = req_kv_len[r];
  }
}

// Opens a step of single next tokens that is described by the records alone: request r of the
// step is the one in slot dec_slots[r]; its token is the one sampled last, its position the
// number of positions the cache holds, and the record moves on by one position.
__global__ void __launch_bounds__(kBeginThreads)
decode_begin_kernel(UpdateList u, const int* __restrict__ dec_slots, int n_reqs, int max_positions,
                    int* __restrict__ token_ids, int* __restrict__ positions, int* __restrict__ req_kv_len,
                    int* err) {
  pdl_trigger();
  if (threadIdx.x == 0) tl_mark(1, 0);
  pdl_wait();
  if (threadIdx.x == 0) tl_mark(1, 1);
  apply_updates(u, err);
  __syncthreads();
  for (int r = threadIdx.x; r < n_reqs; r += blockDim.x) {
    const int slot = dec_slots[r];
    int tok = 0, pos = 0;
    if (slot < 0 || slot >= u.max_slots) {
      set_error(err, kErrRequest, r, slot, u.max_slots);
    } else {
      int* rec = u.records + (size_t)slot * kSlotWords;
      tok = rec[kRecLastToken];
      pos = rec[kRecComputed];
      if (tok < 0) { set_error(err, kErrTokenId, r, tok, slot); tok = 0; }
      if (pos < 0 || pos >= max_positions) { set_error(err, kErrPosition, r, pos, max_positions); pos = 0; }
      else rec[kRecComputed] = pos + 1;
    }
    token_ids[r] = tok;
    positions[r] = pos;
    req_kv_len[r] = pos + 1;
  }
  if (threadIdx.x == 0) tl_mark(1, 4);
}

}  // namespace tk

TK_TIMELINE_SETTER(step_state)

TK_API int tk_slot_words() { return tk::kSlotWords; }

TK_API int tk_step_begin(int* ctl, int max_rec, int max_tab, int* records, int max_slots, int* tables,
                         long long tables_len, int* token_ids, const int* req_q_start, const int* req_kv_len,
                         const int* req_slot, const int* req_fed, int n_reqs, int n_tokens, int* err,
                         cudaStream_t stream) {
  tk::UpdateList u{ctl, max_rec, max_tab, records, max_slots, tables, tables_len};
  return (int)tk::launch(tk::step_begin_kernel, dim3(1), dim3(tk::kBeginThreads), 0, stream, u, token_ids,
                         req_q_start, req_kv_len, req_slot, req_fed, n_reqs, n_tokens, err);
}

TK_API int tk_decode_begin(int* ctl, int max_rec, int max_tab, int* records, int max_slots, int* tables,
                           long long tables_len, const int* dec_slots, int n_reqs, int max_positions,
                           int* token_ids, int* positions, int* req_kv_len, int* err, cudaStream_t stream) {
  if (n_reqs <= 0) return 0;
  tk::UpdateList u{ctl, max_rec, max_tab, records, max_slots, tables, tables_len};
  return (int)tk::launch(tk::decode_begin_kernel, dim3(1), dim3(tk::kBeginThreads), 0, stream, u, dec_slots,
                         n_reqs, max_positions, token_ids, positions, req_kv_len, err);
}
