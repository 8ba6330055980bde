// Per-head RMSNorm of q and k, NeoX rotary embedding, and the write of this
// step's keys and values into their cache pages, in one pass over the fused
// q|k|v projection output.
//
// Formulas: per-head norm over head_dim with one weight vector shared by all
// heads (src/tokamak/model/transformer.py:71-73, layers.py:28-33); angle =
// float(position) * inv_freq[j] and the half rotation out[i] = x[i]*c - x[i+d/2]*s,
// out[i+d/2] = x[i+d/2]*c + x[i]*s (src/tokamak/model/layers.py:56-58,61-89).
// Keys are stored after norm and rotation, values raw
// (src/tokamak/memory/paged_cache.py:72-81).  Everything is computed in float32
// and rounded once on store.
#include "common.cuh"

namespace tk {


struct RopeKvParams {
  const void* qkv;          // [n_tokens, row_stride] : q heads | k heads | v heads
  const float* qkv_parts;   // or float32 partial sums [n_parts, n_tokens, row_stride] to be added up
  int n_parts;
  void* q_out;              // [n_tokens, n_q_heads, head_dim]
  void* k_cache;            // [num_pages, n_kv_heads, page_size, head_dim]
  void* v_cache;
  const int* positions;     // [n_tokens]
  const int* tok_req;       // [n_tokens] row of the token's request in this step
  const int* req_slot;      // [n_reqs]   row of the request in block_table
  const int* block_table;   // [n_slots, max_pages]
  const float* q_norm_w;    // [head_dim] or null
  const float* k_norm_w;    // [head_dim] or null
  const float* inv_freq;    // [rotary_dim / 2] or null (no rotation)
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, head_dim, rotary_dim;
  int row_stride, page_size, max_pages, num_pages;
  int write_kv;             // 0: this layer reads another layer's cache; only q is produced
  float eps;
};

template <typename T>
__global__ void rope_kv_kernel(RopeKvParams p) {
  pdl_trigger();
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads_total = p.n_q_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)p.n_tokens * heads_total) return;
  const int t = (int)(item / heads_total);
  const int h = (int)(item - (long long)t * heads_total);
  const int d = p.head_dim;
  const int half = p.rotary_dim >> 1;

  // kind: 0 = q, 1 = k, 2 = v
  int kind, head;
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }

  const size_t src_off = (size_t)t * p.row_stride +
                         (size_t)(kind == 0 ? head
                                            : (kind == 1 ? p.n_q_heads + head
                                                         : p.n_q_heads + p.n_kv_heads + head)) * d;
  const T* src = (const T*)p.qkv + src_off;
  const float* parts = p.qkv_parts ? p.qkv_parts + src_off : nullptr;
  const size_t part_stride = (size_t)p.n_tokens * p.row_stride;
  // element e of this head's input: the tensor itself, or the sum of the partial products
  auto in = [&](int e) -> float {
    if (parts == nullptr) return to_f32<T>(src[e]);
    float acc = 0.0f;
    for (int s = 0; s < p.n_parts; ++s) acc += parts[(size_t)s * part_stride + e];
    return acc;
  };

  T* dst;
  if (kind == 0) {
    dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d;
  } else {
    const int pos = p.positions[t];
    const int r = p.tok_req[t];
    if (pos < 0) { if (lane == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
    if (r < 0 || r >= p.n_reqs) { if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    const int pidx = pos / p.page_size;
    if (pidx >= p.max_pages) { if (lane == 0) set_error(p.err, kErrPage, t, pidx, -1); return; }
    const int page = p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx];
    if (page < 0 || page >= p.num_pages) { if (lane == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
    T* base = (T*)(kind == 1 ? p.k_cache : p.v_cache);
    dst = base + (((size_t)page * p.n_kv_heads + head) * p.page_size + (pos % p.page_size)) * d;
  }

  if (kind == 2) {
    for (int e = lane; e < d; e += 32) dst[e] = from_f32<T>(in(e));
    return;
  }

  const float* w = (kind == 0) ? p.q_norm_w : p.k_norm_w;
  float rstd = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int e = lane; e < d; e += 32) { const float v = in(e); ss += v * v; }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)d + p.eps);
  }
  const float fpos = (float)p.positions[t];
  // rotated pairs (i, i + half) for i < half; elements beyond rotary_dim pass through
  for (int i = lane; i < half; i += 32) {
    float x1 = in(i) * rstd;
    float x2 = in(i + half) * rstd;
    if (w != nullptr) { x1 *= w[i]; x2 *= w[i + half]; }
    float c = 1.0f, s = 0.0f;
    if (p.inv_freq != nullptr) {
      const float ang = fpos * p.inv_freq[i];
      sincosf(ang, &s, &c);
    }
    dst[i] = from_f32<T>(x1 * c - x2 * s);
    dst[i + half] = from_f32<T>(x2 * c + x1 * s);
  }
  for (int e = 2 * half + lane; e < d; e += 32) {
    float x = in(e) * rstd;
    if (w != nullptr) x *= w[e];
    dst[e] = from_f32<T>(x);
  }
}

}  // namespace tk

TK_API int tk_rope_kv(const void* qkv, const float* qkv_parts, int n_parts, void* q_out, void* k_cache, void* v_cache,
                      const int* positions, const int* tok_req, const int* req_slot,
                      const int* block_table, const float* q_norm_w, const float* k_norm_w,
                      const float* inv_freq, int* err, int n_tokens, int n_reqs, int n_q_heads,
                      int n_kv_heads, int head_dim, int rotary_dim, int row_stride, int page_size,
                      int max_pages, int num_pages, int write_kv, float eps, int dtype,
                      cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim < 1 || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::RopeKvParams p;
  p.qkv = qkv; p.qkv_parts = qkv_parts; p.n_parts = n_parts; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.inv_freq = inv_freq; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim; p.rotary_dim = rotary_dim; p.row_stride = row_stride;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages;
  p.write_kv = write_kv; p.eps = eps;
  const int heads_total = n_q_heads + (write_kv ? 2 * n_kv_heads : 0);
  const int warps_per_block = 4;
  const long long items = (long long)n_tokens * heads_total;
  const long long blocks = (items + warps_per_block - 1) / warps_per_block;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::rope_kv_kernel<T>, dim3((unsigned)blocks), dim3(warps_per_block * 32), 0,
                                   stream, p));
  return (int)e;
}
