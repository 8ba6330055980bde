// Paged flash attention for portions of prompts (bfloat16, head_dim 64 or 128).
//
// One thread block per (tile of 64 query tokens of one request, query head).  The
// tile's queries sit at absolute positions kv_len - q_len + i, so a portion that
// continues a request sees the pages earlier steps wrote plus its own keys, which
// this step wrote just before (the reference's chunk rule,
// src/tokamak/model/step_context.py:88-102).  Each of the four warps owns 16 query
// rows; tiles of 64 keys and values are gathered page by page into shared memory
// with cp.async, double-buffered, and shared by the warps.  Scores, running
// maximum, normaliser and output accumulator are float32; probabilities are rounded
// to bfloat16 only as the tensor-core operand of P*V.
//
// Keys outside the tile's visible range are zero-filled instead of loaded, so a
// partly written or given-back page cannot leak into the result.
#include "mma_utils.cuh"

namespace tk {

constexpr int kPfWarps = 4;
constexpr int kPfRows = kPfWarps * 16;   // query rows per block
constexpr int kPfKeys = 64;              // keys per tile
constexpr int kPfStages = 2;

struct PrefillParams {
  const __nv_bfloat16* q;        // [n_tokens, n_q_heads, D]
  __nv_bfloat16* out;            // [n_tokens, n_q_heads, D]
  const __nv_bfloat16* k_cache;  // [num_pages, n_kv_heads, page_size, D]
  const __nv_bfloat16* v_cache;
  const int* tiles;              // [n_tiles, 2]: request row, tile index within its tokens
  const int* req_q_start;        // [n_reqs] first token of the request in the flat batch
  const int* req_q_len;
  const int* req_kv_len;         // positions of the request after this step
  const int* req_slot;
  const int* block_table;
  int* err;
  int n_tiles, n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages, window;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kPfWarps * 32, 3)
attn_prefill_kernel(PrefillParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int CH = D / 8;
  constexpr int TILE_BYTES = kPfKeys * D * 2;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);

  // heads vary fastest: the tiles are listed with the most keys first, so the blocks start in
  // that order over all heads (the short ones fill the end), and the query heads that share a
  // kv head run at the same time and find its keys and values in L2
  const int head = blockIdx.x, tile_id = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int hkv = head / group;

  const int r = p.tiles[2 * tile_id];
  const int ti = p.tiles[2 * tile_id + 1];
  if (r < 0 || r >= p.n_reqs) {
    if (threadIdx.x == 0) set_error(p.err, kErrRequest, tile_id, r, p.n_reqs);
    return;
  }
  const int q_start = p.req_q_start[r], q_len = p.req_q_len[r], kv_len = p.req_kv_len[r];
  const int row0 = ti * kPfRows;                       // first row of the tile within the request's tokens
  const int rows_here = min(kPfRows, q_len - row0);
  if (rows_here <= 0 || kv_len < q_len) {
    if (threadIdx.x == 0) set_error(p.err, kErrPosition, tile_id, q_len, kv_len);
    return;
  }
  const int pos0 = kv_len - q_len + row0;              // absolute position of the tile's first row
  const int pos_last = pos0 + rows_here - 1;
  const int lo_tile = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;

  // this warp's rows: wr + g and wr + g + 8
  const int wr = warp * 16;
  const int rowA = wr + g, rowB = wr + g + 8;
  const bool hasA = rowA < rows_here, hasB = rowB < rows_here;
  const int posA = pos0 + rowA, posB = pos0 + rowB;
  const int loA = (p.window > 0 && posA - p.window + 1 > 0) ? posA - p.window + 1 : 0;
  const int loB = (p.window > 0 && posB - p.window + 1 > 0) ? posB - p.window + 1 : 0;

  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qA = p.q + ((size_t)(q_start + row0 + rowA) * p.n_q_heads + head) * D;
    const __nv_bfloat16* qB = p.q + ((size_t)(q_start + row0 + rowB) * p.n_q_heads + head) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c0 = ks * 16 + 2 * t4;
      qa[ks][0] = hasA ? *reinterpret_cast<const uint32_t*>(qA + c0) : 0u;
      qa[ks][1] = hasB ? *reinterpret_cast<const uint32_t*>(qB + c0) : 0u;
      qa[ks][2] = hasA ? *reinterpret_cast<const uint32_t*>(qA + c0 + 8) : 0u;
      qa[ks][3] = hasB ? *reinterpret_cast<const uint32_t*>(qB + c0 + 8) : 0u;
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};

  const int first_kt = lo_tile / kPfKeys;
  const int last_kt = pos_last / kPfKeys;
  const int n_kt = last_kt - first_kt + 1;

  auto issue_load = [&](int kt, int stage) {
    const uint32_t kdst = smem_base + stage * STAGE_BYTES;
    const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < (kPfKeys * CH) / (kPfWarps * 32); ++i) {
      const int idx = i * (kPfWarps * 32) + threadIdx.x;
      const int row = idx / CH, chunk = idx % CH;
      const int key = kt * kPfKeys + row;
      bool valid = key >= lo_tile && key <= pos_last;
      size_t src_row = 0;
      if (valid) {
        const int pidx = key / p.page_size;
        const int page = (pidx < p.max_pages) ? table[pidx] : -1;
        if (page < 0 || page >= p.num_pages) {
          set_error(p.err, kErrPage, tile_id, pidx, page);
          valid = false;
        } else {
          src_row = ((size_t)page * p.n_kv_heads + hkv) * p.page_size + (key % p.page_size);
        }
      }
      const int off = swizzled_offset(row, chunk, CH);
      cp_async16(kdst + off, p.k_cache + src_row * D + chunk * 8, valid);
      cp_async16(vdst + off, p.v_cache + src_row * D + chunk * 8, valid);
    }
  };

  issue_load(first_kt, 0);
  cp_async_commit();

  for (int it = 0; it < n_kt; ++it) {
    const int kt = first_kt + it;
    if (it + 1 < n_kt) issue_load(kt + 1, (it + 1) % kPfStages);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const uint32_t kbase = smem_base + (it % kPfStages) * STAGE_BYTES;
    const uint32_t vbase = kbase + TILE_BYTES;

    float s[kPfKeys / 8][4];
#pragma unroll
    for (int nt = 0; nt < kPfKeys / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < kPfKeys / 16; ++np) {
        const int row = np * 16 + ((lane >> 4) << 3) + (lane & 7);
        const int chunk = 2 * ks + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kbase + swizzled_offset(row, chunk, CH), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16_16816(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }

    float mx[2] = {-INFINITY, -INFINITY};
    // a tile that lies wholly below the diagonal and inside the window of all 16 rows of this
    // warp needs no mask
    const int key_first = kt * kPfKeys, key_last = key_first + kPfKeys - 1;
    const bool interior = (wr + 15 < rows_here) && key_last <= pos0 + wr &&
                          (p.window <= 0 || key_first >= pos0 + wr + 15 - p.window + 1);
    if (interior) {
#pragma unroll
      for (int nt = 0; nt < kPfKeys / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] *= p.scale_log2;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < kPfKeys / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_first + nt * 8 + 2 * t4 + (e & 1);
          const bool valid = (e < 2) ? (hasA && key <= posA && key >= loA)
                                     : (hasB && key <= posB && key >= loB);
          s[nt][e] = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = (m_new == -INFINITY) ? 0.0f : m_new;
      corr[h] = exp2f(m_run[h] - m_use[h]);
      m_run[h] = m_new;
    }
    float psum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < kPfKeys / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[nt][e] = exp2f(s[nt][e] - m_use[e >> 1]);
        psum[e >> 1] += s[nt][e];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + psum[h];
#pragma unroll
    for (int i2 = 0; i2 < D / 8; ++i2) {
      o[i2][0] *= corr[0]; o[i2][1] *= corr[0];
      o[i2][2] *= corr[1]; o[i2][3] *= corr[1];
    }

#pragma unroll
    for (int kk = 0; kk < kPfKeys / 16; ++kk) {
      const uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int c = 0; c < D / 8; c += 2) {
        const int row = kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
        const int chunk = c + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vbase + swizzled_offset(row, chunk, CH), b0, b1, b2, b3);
        mma_bf16_16816(o[c], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16_16816(o[c + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  const float invA = hasA ? 1.0f / l_run[0] : 0.0f;
  const float invB = hasB ? 1.0f / l_run[1] : 0.0f;
  __nv_bfloat16* oA = p.out + ((size_t)(q_start + row0 + rowA) * p.n_q_heads + head) * D;
  __nv_bfloat16* oB = p.out + ((size_t)(q_start + row0 + rowB) * p.n_q_heads + head) * D;
#pragma unroll
  for (int i2 = 0; i2 < D / 8; ++i2) {
    const int col = i2 * 8 + 2 * t4;
    if (hasA) *reinterpret_cast<uint32_t*>(oA + col) = pack_bf16(o[i2][0] * invA, o[i2][1] * invA);
    if (hasB) *reinterpret_cast<uint32_t*>(oB + col) = pack_bf16(o[i2][2] * invB, o[i2][3] * invB);
  }
}

template <int D>
static int launch_prefill(const PrefillParams& p, cudaStream_t stream) {
  constexpr int smem_bytes = kPfStages * 2 * kPfKeys * D * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (p.n_tiles > 65535) return (int)cudaErrorInvalidValue;
  dim3 grid(p.n_q_heads, p.n_tiles);
  return (int)launch(attn_prefill_kernel<D>, grid, dim3(kPfWarps * 32), smem_bytes, stream, p);
}

}  // namespace tk

TK_API int tk_attention_prefill(const void* q, void* out, const void* k_cache, const void* v_cache,
                                const int* tiles, const int* req_q_start, const int* req_q_len,
                                const int* req_kv_len, const int* req_slot, const int* block_table,
                                int* err, int n_tiles, int n_reqs, int n_q_heads, int n_kv_heads,
                                int head_dim, int page_size, int max_pages, int num_pages, int window,
                                float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || n_q_heads > 65535 ||
      (head_dim != 64 && head_dim != 128) || page_size < 1) {
    return (int)cudaErrorInvalidValue;
  }
  tk::PrefillParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.tiles = tiles; p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.req_kv_len = req_kv_len;
  p.req_slot = req_slot; p.block_table = block_table; p.err = err;
  p.n_tiles = n_tiles; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 128) return tk::launch_prefill<128>(p, stream);
  return tk::launch_prefill<64>(p, stream);
}
