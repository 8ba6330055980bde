// Paged attention, general form: any mix of prompt portions and single decoded
// tokens, any head_dim up to 256, any group size, float32 or bfloat16 pages.
//
// One thread block per (token, query head).  The query at absolute position p
// sees keys [max(0, p - window + 1), p] of its own request (window <= 0: all),
// the causal rule of the reference for a chunk at start_pos > 0
// (src/tokamak/model/step_context.py:93-102) and its decode length mask
// (src/tokamak/kernels/paged_attention.py:97-123).  Scores are scaled by
// softmax_scale, the softmax is an online one with float32 running maximum,
// normaliser and accumulator (paged_attention.py:111-123,139-151).  This is the
// kernel of the float32 path and of every shape the tiled kernels refuse.
#include "common.cuh"

namespace tk {

constexpr int kPlainMaxPerLane = 8;  // head_dim <= 256
constexpr int kPlainWarps = 4;

struct AttnParams {
  const void* q;            // [n_tokens, n_q_heads, head_dim]
  void* out;                // [n_tokens, n_q_heads, head_dim]
  const void* k_cache;      // [num_pages, n_kv_heads, page_size, head_dim]
  const void* v_cache;
  const int* positions;     // [n_tokens]
  const int* tok_req;       // [n_tokens]
  const int* req_slot;      // [n_reqs]
  const int* block_table;   // [n_slots, max_pages]
  const int* items;         // [n_items] token indices to process, or null for all tokens
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, head_dim;
  int page_size, max_pages, num_pages, window;
  float scale;
};

template <typename T>
__global__ void attention_plain_kernel(AttnParams p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_m[kPlainWarps];
  __shared__ float s_l[kPlainWarps];
  __shared__ float s_acc[kPlainWarps][kPlainMaxPerLane * 32];

  const int t = p.items ? p.items[blockIdx.x] : blockIdx.x;
  const int hq = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int d = p.head_dim;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int hkv = hq / group;
  const int pos = p.positions[t];
  const int r = p.tok_req[t];
  if (pos < 0 || r < 0 || r >= p.n_reqs) {
    if (threadIdx.x == 0) set_error(p.err, pos < 0 ? kErrPosition : kErrRequest, t, pos, r);
    return;
  }
  const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;

  const T* qrow = (const T*)p.q + ((size_t)t * p.n_q_heads + hq) * d;
  float qreg[kPlainMaxPerLane];
  float acc[kPlainMaxPerLane];
#pragma unroll
  for (int i = 0; i < kPlainMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    qreg[i] = (e < d) ? to_f32<T>(qrow[e]) * p.scale : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;

  for (int j = lo + warp; j <= pos; j += kPlainWarps) {
    const int pidx = j / p.page_size;
    const int page = (pidx < p.max_pages) ? table[pidx] : -1;   // beyond the row: reported, not read
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) set_error(p.err, kErrPage, t, pidx, page);
      break;
    }
    const size_t off = (((size_t)page * p.n_kv_heads + hkv) * p.page_size + (j % p.page_size)) * d;
    const T* krow = (const T*)p.k_cache + off;
    const T* vrow = (const T*)p.v_cache + off;
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < kPlainMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < d) dot += qreg[i] * to_f32<T>(krow[e]);
    }
    dot = warp_sum(dot);
    const float m_new = fmaxf(m, dot);
    const float corr = expf(m - m_new);   // m = -inf on the first key: exp(-inf) = 0
    const float pj = expf(dot - m_new);
    l = l * corr + pj;
#pragma unroll
    for (int i = 0; i < kPlainMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < d) acc[i] = acc[i] * corr + pj * to_f32<T>(vrow[e]);
    }
    m = m_new;
  }

  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < kPlainMaxPerLane; ++i) s_acc[warp][i * 32 + lane] = acc[i];
  __syncthreads();

  if (warp == 0) {
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPlainWarps; ++w) m_all = fmaxf(m_all, s_m[w]);
    float l_all = 0.0f;
    float f[kPlainWarps];
#pragma unroll
    for (int w = 0; w < kPlainWarps; ++w) {
      f[w] = (s_m[w] == -INFINITY) ? 0.0f : expf(s_m[w] - m_all);
      l_all += s_l[w] * f[w];
    }
    const float inv = 1.0f / l_all;   // the query always sees its own key, so l_all > 0
    T* orow = (T*)p.out + ((size_t)t * p.n_q_heads + hq) * d;
#pragma unroll
    for (int i = 0; i < kPlainMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < d) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kPlainWarps; ++w) o += s_acc[w][e] * f[w];
        orow[e] = from_f32<T>(o * inv);
      }
    }
  }
}

}  // namespace tk

TK_API int tk_attention_plain(const void* q, void* out, const void* k_cache, const void* v_cache,
                              const int* positions, const int* tok_req, const int* req_slot,
                              const int* block_table, const int* items, int* err, int n_tokens, int n_reqs,
                              int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                              int max_pages, int num_pages, int window, float scale, int dtype,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim < 1 || head_dim > tk::kPlainMaxPerLane * 32 || n_kv_heads < 1 ||
      n_q_heads % n_kv_heads != 0 || n_q_heads > 65535) {
    return (int)cudaErrorInvalidValue;
  }
  tk::AttnParams p;
  p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.items = items; p.err = err; p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads;
  p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.page_size = page_size;
  p.max_pages = max_pages; p.num_pages = num_pages; p.window = window; p.scale = scale;
  dim3 grid(n_tokens, n_q_heads);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::attention_plain_kernel<T>, grid, dim3(tk::kPlainWarps * 32), 0, stream, p));
  return (int)e;
}
