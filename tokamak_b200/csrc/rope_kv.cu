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
//
// The cosines and sines depend on the token's position only, so they are computed
// once per step into a float32 table [token, rotary_dim / 2] of (cos, sin) pairs
// (tk_rope_table) that every layer of the step reads.
#include "common.cuh"

namespace tk {

// table[t, j] = (cos, sin)(float(positions[t]) * inv_freq[j])
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int n_tokens, int half) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * half) return;
  const int t = idx / half, j = idx - t * half;
  const float ang = (float)positions[t] * inv_freq[j];
  float s, c;
  sincosf(ang, &s, &c);
  table[idx] = make_float2(c, s);
}

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
  const int* req_q_len;     // [n_reqs] tokens the request brings to this step, or null
  const int* req_kv_len;    // [n_reqs] positions of the request after this step, or null
  const float* q_norm_w;    // [head_dim] or null
  const float* k_norm_w;    // [head_dim] or null
  const float2* rope_table; // [n_tokens, rotary_dim / 2] (cos, sin) or null (no rotation)
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, head_dim, rotary_dim;
  int row_stride, page_size, max_pages, num_pages;
  int write_kv;             // 0: this layer reads another layer's cache; only q is produced
  int heads_per_warp;       // consecutive heads of one token that a warp works through
  float eps;
};

template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
  }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

// One thread block per (token, group of heads): each of its four warps works through
// heads_per_warp consecutive heads of the token, so that with many tokens the lookups of the
// token's position, request and page are shared by many heads, while with few tokens (decoding)
// every head still has a warp of its own.  head_dim and rotary_dim are multiples of 4, so every
// lane works on pairs of neighbouring elements with 4- and 8-byte accesses.
template <typename T>
__device__ __forceinline__ void rope_kv_head(const RopeKvParams& p, int t, int h, int lane, int d, int half);

template <typename T>
__global__ void rope_kv_kernel(RopeKvParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads_total = p.n_q_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const int t = blockIdx.x;
  const int h_begin = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * p.heads_per_warp;
  const int d = p.head_dim;
  const int half = p.rotary_dim >> 1;
  for (int h = h_begin; h < min(h_begin + p.heads_per_warp, heads_total); ++h) {
    rope_kv_head<T>(p, t, h, lane, d, half);
  }
}

template <typename T>
__device__ __forceinline__ void rope_kv_head(const RopeKvParams& p, int t, int h, int lane, int d, int half) {
  // kind: 0 = q, 1 = k, 2 = v
  int kind, head;
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }

  const size_t src_off = (size_t)t * p.row_stride + (size_t)h * d;   // heads lie in the order q | k | v
  const T* src = (const T*)p.qkv + src_off;
  const float* parts = p.qkv_parts ? p.qkv_parts + src_off : nullptr;
  const size_t part_stride = (size_t)p.n_tokens * p.row_stride;
  // elements e, e + 1 of this head's input: the tensor itself, or the sum of the partial products
  auto in2 = [&](int e) -> float2 {
    if (parts == nullptr) return Pair<T>::load(src + e);
    float2 acc = make_float2(0.0f, 0.0f);
    for (int s = 0; s < p.n_parts; ++s) {
      const float2 v = *reinterpret_cast<const float2*>(parts + (size_t)s * part_stride + e);
      acc.x += v.x; acc.y += v.y;
    }
    return acc;
  };

  T* dst;
  int zero_rows = 0;        // rows after this token's slot that are cleared (see below)
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
    // The request's last token of this step clears the rest of its page if the page was begun
    // in this step, so that a live page never holds stale values behind the last position:
    // kernels that load whole pages multiply them by probabilities that are exactly zero.
    if (p.req_kv_len != nullptr) {
      const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
      if (pos == kv_len - 1 && pos - pos % p.page_size >= kv_len - q_len) {
        zero_rows = p.page_size - 1 - pos % p.page_size;
      }
    }
  }
  for (int z = 1; z <= zero_rows; ++z) {
    for (int e = 2 * lane; e < d; e += 64) Pair<T>::store(dst + (size_t)z * d + e, 0.0f, 0.0f);
  }

  if (kind == 2) {
    for (int e = 2 * lane; e < d; e += 64) { const float2 v = in2(e); Pair<T>::store(dst + e, v.x, v.y); }
    return;
  }

  const float* w = (kind == 0) ? p.q_norm_w : p.k_norm_w;
  // The rotated pairs (i, i + half) are read once and kept in registers between the sum of
  // squares and the rotation (half <= 128: two pairs of neighbours per lane).
  constexpr int kMaxIter = 2;
  float2 x1[kMaxIter], x2[kMaxIter];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < kMaxIter; ++k) {
    const int i = 2 * lane + 64 * k;
    if (i < half) {
      x1[k] = in2(i); x2[k] = in2(i + half);
      ss += x1[k].x * x1[k].x + x1[k].y * x1[k].y + x2[k].x * x2[k].x + x2[k].y * x2[k].y;
    }
  }
  float rstd = 1.0f;
  if (w != nullptr) {
    for (int e = 2 * half + 2 * lane; e < d; e += 64) { const float2 v = in2(e); ss += v.x * v.x + v.y * v.y; }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)d + p.eps);
  }
  const float2* tab = p.rope_table ? p.rope_table + (size_t)t * half : nullptr;
#pragma unroll
  for (int k = 0; k < kMaxIter; ++k) {
    const int i = 2 * lane + 64 * k;
    if (i < half) {
      float2 a = x1[k], b = x2[k];
      a.x *= rstd; a.y *= rstd; b.x *= rstd; b.y *= rstd;
      if (w != nullptr) {
        const float2 w1 = *reinterpret_cast<const float2*>(w + i);
        const float2 w2 = *reinterpret_cast<const float2*>(w + i + half);
        a.x *= w1.x; a.y *= w1.y; b.x *= w2.x; b.y *= w2.y;
      }
      float4 cs = make_float4(1.0f, 0.0f, 1.0f, 0.0f);       // (cos, sin) of i and of i + 1
      if (tab != nullptr) cs = *reinterpret_cast<const float4*>(tab + i);
      Pair<T>::store(dst + i, a.x * cs.x - b.x * cs.y, a.y * cs.z - b.y * cs.w);
      Pair<T>::store(dst + i + half, b.x * cs.x + a.x * cs.y, b.y * cs.z + a.y * cs.w);
    }
  }
  for (int e = 2 * half + 2 * lane; e < d; e += 64) {
    float2 x = in2(e);
    x.x *= rstd; x.y *= rstd;
    if (w != nullptr) { x.x *= w[e]; x.y *= w[e + 1]; }
    Pair<T>::store(dst + e, x.x, x.y);
  }
}

}  // namespace tk

TK_API int tk_rope_table(const int* positions, const float* inv_freq, float* table, int n_tokens,
                         int rotary_dim, cudaStream_t stream) {
  if (n_tokens <= 0 || rotary_dim <= 0) return 0;
  if (rotary_dim & 1) return (int)cudaErrorInvalidValue;
  const int half = rotary_dim / 2;
  const int total = n_tokens * half;
  return (int)tk::launch(tk::rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, positions,
                         inv_freq, (float2*)table, n_tokens, half);
}

TK_API int tk_rope_kv(const void* qkv, const float* qkv_parts, int n_parts, void* q_out, void* k_cache,
                      void* v_cache, const int* positions, const int* tok_req, const int* req_slot,
                      const int* block_table, const int* req_q_len, const int* req_kv_len,
                      const float* q_norm_w, const float* k_norm_w,
                      const float* rope_table, int* err, int n_tokens, int n_reqs, int n_q_heads,
                      int n_kv_heads, int head_dim, int rotary_dim, int row_stride, int page_size,
                      int max_pages, int num_pages, int write_kv, float eps, int dtype,
                      cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  // pairs of neighbouring elements in both halves of the rotation: multiples of 4
  if (head_dim < 4 || head_dim % 4 != 0 || rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 4 != 0 ||
      rotary_dim > 256 || row_stride % 2 != 0) {
    return (int)cudaErrorInvalidValue;
  }
  tk::RopeKvParams p;
  p.qkv = qkv; p.qkv_parts = qkv_parts; p.n_parts = n_parts; p.q_out = q_out; p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.req_q_len = req_q_len; p.req_kv_len = req_kv_len;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.rope_table = (const float2*)rope_table; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim; p.rotary_dim = rotary_dim; p.row_stride = row_stride;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages;
  p.write_kv = write_kv; p.eps = eps;
  const int heads_total = n_q_heads + (write_kv ? 2 * n_kv_heads : 0);
  const int warps_per_block = 4;
  // many tokens: one block per token, every warp takes a quarter of the heads; few tokens: a warp per head
  p.heads_per_warp = n_tokens >= 256 ? (heads_total + warps_per_block - 1) / warps_per_block : 1;
  const int head_groups = (heads_total + warps_per_block * p.heads_per_warp - 1) / (warps_per_block * p.heads_per_warp);
  if (head_groups > 65535) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::rope_kv_kernel<T>, dim3((unsigned)n_tokens, (unsigned)head_groups),
                                   dim3(warps_per_block * 32), 0, stream, p));
  return (int)e;
}
