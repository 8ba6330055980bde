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

constexpr int kRopeIter = 2;     // pairs of neighbours per lane: rotary_dim / 2 <= 128
constexpr int kRopeUnroll = 4;   // heads in flight per warp

// One thread block per (token, group of heads): each of its four warps works through
// heads_per_warp consecutive heads of the token, four at a time so that their loads and
// reductions overlap.  With many tokens the lookups of the token's position, request and page
// and the loads of the rotation pairs and norm weights are shared by many heads, while with few
// tokens (decoding) every head still has a warp of its own.  head_dim and rotary_dim are
// multiples of 4, so every lane works on pairs of neighbouring elements with 4- and 8-byte
// accesses.
template <typename T>
__global__ void rope_kv_kernel(RopeKvParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads_total = p.n_q_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const int t = blockIdx.x;
  const int h_begin = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * p.heads_per_warp;
  const int h_end = min(h_begin + p.heads_per_warp, heads_total);
  if (h_begin >= h_end) return;
  const int d = p.head_dim;
  const int half = p.rotary_dim >> 1;

  // ---- what depends on the token and the lane only ---------------------------------------------
  float4 cs[kRopeIter];
  float2 wq1[kRopeIter], wq2[kRopeIter], wk1[kRopeIter], wk2[kRopeIter];
  const float2* tab = p.rope_table ? p.rope_table + (size_t)t * half : nullptr;
#pragma unroll
  for (int k = 0; k < kRopeIter; ++k) {
    const int i = 2 * lane + 64 * k;
    cs[k] = make_float4(1.0f, 0.0f, 1.0f, 0.0f);          // (cos, sin) of i and of i + 1
    wq1[k] = wq2[k] = wk1[k] = wk2[k] = make_float2(1.0f, 1.0f);
    if (i < half) {
      if (tab != nullptr) cs[k] = *reinterpret_cast<const float4*>(tab + i);
      if (p.q_norm_w != nullptr) {
        wq1[k] = *reinterpret_cast<const float2*>(p.q_norm_w + i);
        wq2[k] = *reinterpret_cast<const float2*>(p.q_norm_w + i + half);
      }
      if (p.k_norm_w != nullptr) {
        wk1[k] = *reinterpret_cast<const float2*>(p.k_norm_w + i);
        wk2[k] = *reinterpret_cast<const float2*>(p.k_norm_w + i + half);
      }
    }
  }

  // ---- where this token's keys and values go ---------------------------------------------------
  size_t cache_row = 0;        // row (of head 0) of the token's slot: ((page * Hkv + head) * page_size + slot)
  bool cache_ok = false;
  int zero_rows = 0;
  if (p.write_kv && h_end > p.n_q_heads) {
    const int pos = p.positions[t];
    const int r = p.tok_req[t];
    if (pos < 0) {
      if (lane == 0) set_error(p.err, kErrPosition, t, pos, 0);
    } else if (r < 0 || r >= p.n_reqs) {
      if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs);
    } else {
      const int pidx = pos / p.page_size;
      const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
      if (page < 0 || page >= p.num_pages) {
        if (lane == 0) set_error(p.err, kErrPage, t, pidx, page);
      } else {
        cache_ok = true;
        cache_row = (size_t)page * p.n_kv_heads * p.page_size + (pos % p.page_size);
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
    }
  }

  const size_t part_stride = (size_t)p.n_tokens * p.row_stride;
  for (int h0 = h_begin; h0 < h_end; h0 += kRopeUnroll) {
    float2 x1[kRopeUnroll][kRopeIter], x2[kRopeUnroll][kRopeIter];
    float ss[kRopeUnroll];
    // ---- loads of up to four heads ---------------------------------------------------------------
#pragma unroll
    for (int u = 0; u < kRopeUnroll; ++u) {
      const int h = h0 + u;
      ss[u] = 0.0f;
      if (h >= h_end) continue;
      const size_t src_off = (size_t)t * p.row_stride + (size_t)h * d;   // heads lie in the order q | k | v
      auto in2 = [&](int e) -> float2 {
        if (p.qkv_parts == nullptr) return Pair<T>::load((const T*)p.qkv + src_off + e);
        float2 acc = make_float2(0.0f, 0.0f);
        for (int s2 = 0; s2 < p.n_parts; ++s2) {
          const float2 v = *reinterpret_cast<const float2*>(p.qkv_parts + (size_t)s2 * part_stride + src_off + e);
          acc.x += v.x; acc.y += v.y;
        }
        return acc;
      };
#pragma unroll
      for (int k = 0; k < kRopeIter; ++k) {
        const int i = 2 * lane + 64 * k;
        x1[u][k] = x2[u][k] = make_float2(0.0f, 0.0f);
        if (i < half) {
          x1[u][k] = in2(i); x2[u][k] = in2(i + half);
          ss[u] += x1[u][k].x * x1[u][k].x + x1[u][k].y * x1[u][k].y + x2[u][k].x * x2[u][k].x +
                   x2[u][k].y * x2[u][k].y;
        }
      }
      for (int e = 2 * half + 2 * lane; e < d; e += 64) { const float2 v = in2(e); ss[u] += v.x * v.x + v.y * v.y; }
    }
#pragma unroll
    for (int u = 0; u < kRopeUnroll; ++u) ss[u] = warp_sum(ss[u]);

    // ---- norm, rotation, stores -------------------------------------------------------------------
#pragma unroll
    for (int u = 0; u < kRopeUnroll; ++u) {
      const int h = h0 + u;
      if (h >= h_end) continue;
      int kind, head;     // 0 = q, 1 = k, 2 = v
      if (h < p.n_q_heads) { kind = 0; head = h; }
      else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
      else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }
      T* dst;
      if (kind == 0) {
        dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d;
      } else {
        if (!cache_ok) continue;
        dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) + (cache_row + (size_t)head * p.page_size) * d;
        for (int z = 1; z <= zero_rows; ++z) {
          for (int e = 2 * lane; e < d; e += 64) Pair<T>::store(dst + (size_t)z * d + e, 0.0f, 0.0f);
        }
      }
      const bool normed = (kind == 0 && p.q_norm_w != nullptr) || (kind == 1 && p.k_norm_w != nullptr);
      const float rstd = normed ? rsqrtf(ss[u] / (float)d + p.eps) : 1.0f;
#pragma unroll
      for (int k = 0; k < kRopeIter; ++k) {
        const int i = 2 * lane + 64 * k;
        if (i >= half) continue;
        float2 a = x1[u][k], b = x2[u][k];
        if (kind == 2) {             // values are stored as they are
          Pair<T>::store(dst + i, a.x, a.y);
          Pair<T>::store(dst + i + half, b.x, b.y);
          continue;
        }
        const float2 w1 = (kind == 0) ? wq1[k] : wk1[k];
        const float2 w2 = (kind == 0) ? wq2[k] : wk2[k];
        a.x = a.x * rstd * w1.x; a.y = a.y * rstd * w1.y; b.x = b.x * rstd * w2.x; b.y = b.y * rstd * w2.y;
        const float4 c = cs[k];
        Pair<T>::store(dst + i, a.x * c.x - b.x * c.y, a.y * c.z - b.y * c.w);
        Pair<T>::store(dst + i + half, b.x * c.x + a.x * c.y, b.y * c.z + a.y * c.w);
      }
      // elements beyond the rotated part (rotary_dim < head_dim) pass through the norm only
      const size_t src_off = (size_t)t * p.row_stride + (size_t)h * d;
      for (int e = 2 * half + 2 * lane; e < d; e += 64) {
        float2 x;
        if (p.qkv_parts == nullptr) {
          x = Pair<T>::load((const T*)p.qkv + src_off + e);
        } else {
          x = make_float2(0.0f, 0.0f);
          for (int s2 = 0; s2 < p.n_parts; ++s2) {
            const float2 v = *reinterpret_cast<const float2*>(p.qkv_parts + (size_t)s2 * part_stride + src_off + e);
            x.x += v.x; x.y += v.y;
          }
        }
        if (kind != 2) {
          const float* w = (kind == 0) ? p.q_norm_w : p.k_norm_w;
          x.x *= rstd; x.y *= rstd;
          if (w != nullptr) { x.x *= w[e]; x.y *= w[e + 1]; }
        }
        Pair<T>::store(dst + e, x.x, x.y);
      }
    }
  }
}

// The same work for the common case (rotary_dim == head_dim, head_dim 16 * {1, 2, 4, 8, 16}) with
// 16-byte accesses: TPH = head_dim / 16 neighbouring threads share a head, each owning the chunk
// of 8 elements c and its rotation partner c + TPH, so a warp works on 32 / TPH heads at once and
// the per-head norm needs log2(TPH) shuffles.
template <typename T> struct Chunk8;
template <> struct Chunk8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Chunk8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

// (eight blocks of 128 threads to an SM, 64 registers: measured 7 % faster than the 72 registers and seven
// blocks that the compiler chooses by itself)
template <typename T, int TPH>
__global__ void __launch_bounds__(128, 8) rope_kv_chunk_kernel(RopeKvParams p) {
  pdl_trigger();
  pdl_wait();
  const int heads_total = p.n_q_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long item = gid / TPH;                // (token, head)
  const int c = (int)(gid - item * TPH);           // chunk of 8 elements inside the first half
  const bool active = item < (long long)p.n_tokens * heads_total;
  const int t = active ? (int)(item / heads_total) : 0;
  const int h = active ? (int)(item - (long long)t * heads_total) : 0;
  const int d = p.head_dim;
  const int half = d >> 1;

  float x1[8], x2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { x1[e] = 0.0f; x2[e] = 0.0f; }
  const size_t src_off = (size_t)t * p.row_stride + (size_t)h * d + 8 * c;
  if (active) {
    if (p.qkv_parts == nullptr) {
      Chunk8<T>::load((const T*)p.qkv + src_off, x1);
      Chunk8<T>::load((const T*)p.qkv + src_off + half, x2);
    } else {
      const size_t part_stride = (size_t)p.n_tokens * p.row_stride;
      for (int s2 = 0; s2 < p.n_parts; ++s2) {
        float a[8], b[8];
        Chunk8<float>::load(p.qkv_parts + (size_t)s2 * part_stride + src_off, a);
        Chunk8<float>::load(p.qkv_parts + (size_t)s2 * part_stride + src_off + half, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) { x1[e] += a[e]; x2[e] += b[e]; }
      }
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
#pragma unroll
  for (int o = TPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!active) return;

  int kind, head;     // 0 = q, 1 = k, 2 = v
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }

  T* dst;
  int zero_rows = 0;
  if (kind == 0) {
    dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d + 8 * c;
  } else {
    const int pos = p.positions[t];
    const int r = p.tok_req[t];
    if (pos < 0) { if (c == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
    if (r < 0 || r >= p.n_reqs) { if (c == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    const int pidx = pos / p.page_size;
    const int slot = pos - pidx * p.page_size;
    const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
    if (page < 0 || page >= p.num_pages) { if (c == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
    dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) +
          (((size_t)page * p.n_kv_heads + head) * p.page_size + slot) * d + 8 * c;
    if (p.req_kv_len != nullptr) {      // see rope_kv_kernel: the rest of a page begun in this step is cleared
      const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
      if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) zero_rows = p.page_size - 1 - slot;
    }
  }
  if (zero_rows > 0) {
    float zero[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) zero[e] = 0.0f;
    for (int z = 1; z <= zero_rows; ++z) {
      Chunk8<T>::store(dst + (size_t)z * d, zero);
      Chunk8<T>::store(dst + (size_t)z * d + half, zero);
    }
  }
  if (kind == 2) {
    Chunk8<T>::store(dst, x1);
    Chunk8<T>::store(dst + half, x2);
    return;
  }
  const float* w = (kind == 0) ? p.q_norm_w : p.k_norm_w;
  if (w != nullptr) {
    const float rstd = rsqrtf(ss / (float)d + p.eps);
    float w1[8], w2[8];
    Chunk8<float>::load(w + 8 * c, w1);
    Chunk8<float>::load(w + half + 8 * c, w2);
#pragma unroll
    for (int e = 0; e < 8; ++e) { x1[e] = x1[e] * rstd * w1[e]; x2[e] = x2[e] * rstd * w2[e]; }
  }
  float y1[8], y2[8];
  if (p.rope_table != nullptr) {
    const float4* tab = reinterpret_cast<const float4*>(p.rope_table + (size_t)t * half + 8 * c);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 cs = tab[e];           // (cos, sin) of elements 2e and 2e + 1 of the chunk
      y1[2 * e] = x1[2 * e] * cs.x - x2[2 * e] * cs.y;
      y2[2 * e] = x2[2 * e] * cs.x + x1[2 * e] * cs.y;
      y1[2 * e + 1] = x1[2 * e + 1] * cs.z - x2[2 * e + 1] * cs.w;
      y2[2 * e + 1] = x2[2 * e + 1] * cs.z + x1[2 * e + 1] * cs.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) { y1[e] = x1[e]; y2[e] = x2[e]; }
  }
  Chunk8<T>::store(dst, y1);
  Chunk8<T>::store(dst + half, y2);
}

template <typename T>
static cudaError_t launch_rope_chunk(const RopeKvParams& p, int tph, long long threads_total, cudaStream_t stream) {
  const unsigned blocks = (unsigned)((threads_total + 127) / 128);
  switch (tph) {
    case 1: return launch(rope_kv_chunk_kernel<T, 1>, dim3(blocks), dim3(128), 0, stream, p);
    case 2: return launch(rope_kv_chunk_kernel<T, 2>, dim3(blocks), dim3(128), 0, stream, p);
    case 4: return launch(rope_kv_chunk_kernel<T, 4>, dim3(blocks), dim3(128), 0, stream, p);
    case 8: return launch(rope_kv_chunk_kernel<T, 8>, dim3(blocks), dim3(128), 0, stream, p);
    default: return launch(rope_kv_chunk_kernel<T, 16>, dim3(blocks), dim3(128), 0, stream, p);
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
  const int tph = head_dim / 16;
  if (rotary_dim == head_dim && head_dim % 16 == 0 && (tph & (tph - 1)) == 0 && tph <= 16 &&
      row_stride % 8 == 0) {
    p.heads_per_warp = 0;
    const long long threads_total = (long long)n_tokens * heads_total * tph;
    cudaError_t e2 = cudaSuccess;
    TK_DISPATCH_DTYPE(dtype, T, e2 = tk::launch_rope_chunk<T>(p, tph, threads_total, stream));
    return (int)e2;
  }
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
