// Split-K paged attention for single next tokens (bfloat16, head_dim 64 or 128).
//
// One thread block per (key split, kv head, decoded token).  The query heads that
// share the kv head form the rows of a 16-row tensor-core tile, so keys and values
// are read once for the whole group.  Each of the four warps walks its own 16-key
// tiles of the block's key range (one cache page, or a part of a larger page, per
// tile), copies them into shared memory with cp.async two tiles ahead of use, and
// keeps its own online-softmax state in registers: scores, running maximum,
// normaliser and output accumulator are float32
// (src/tokamak/kernels/paged_attention.py:111-123,139-151).  The warps are merged
// through shared memory.  A single split stores the output itself.  Several splits write
// unnormalised partial results with maximum and normaliser to scratch memory; the block
// that arrives last for a (token, kv head), counted with an atomic in scratch memory,
// merges them, writes the output and puts the counter back to zero.  (Merging two to eight
// splits inside a thread-block cluster over distributed shared memory instead was measured
// and is no faster: 2,108 tokens/s either way at batch 8.)
// The reference's kernel has no split and one program per (sequence, kv head)
// (paged_attention.py:19-20,202).
//
// Programmatic dependent launch: key and value tiles that lie wholly below the token's own
// position are requested before the wait on the preceding kernel (which writes the cache only
// at the new tokens' places); the queries and the tile of the new token come after it.
//
// Keys outside [max(0, pos - window + 1), pos] are never loaded: their rows are
// zero-filled, so stale or foreign data in a partly filled or given-back page
// cannot reach the result.
#include "mma_utils.cuh"
#include "timeline.cuh"

namespace tk {

constexpr int kDecWarps = 4;
constexpr int kDecTile = 16;      // keys per warp tile
constexpr int kDecStages = 3;
constexpr int kDecMaxSplits = 128;

struct DecodeParams {
  const __nv_bfloat16* q;       // [n_tokens, n_q_heads, D]
  const __nv_bfloat16* k_cache; // [num_pages, n_kv_heads, page_size, D]
  const __nv_bfloat16* v_cache;
  float* part_o;                // [n_items, n_q_heads, n_splits, D]
  float* part_ml;               // [n_items, n_q_heads, n_splits, 2]
  int* counters;                // [n_items, n_kv_heads] arrivals of the splits; zero before and after
  __nv_bfloat16* out;           // [n_tokens, n_q_heads, D]
  const int* items;             // [n_items] token index of each decoded token
  const int* positions;
  const int* tok_req;
  const int* req_slot;
  const int* block_table;
  int* err;
  int n_items, n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages, window, n_splits;
  float scale_log2;             // softmax scale * log2(e)
};

template <int D, int STAGES>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_split_kernel(DecodeParams p) {
  pdl_trigger();
  constexpr int CH = D / 8;                       // 16-byte chunks per row
  constexpr int TILE_BYTES = kDecTile * D * 2;    // one K or V tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];

  const int split = blockIdx.x, hkv = blockIdx.y, item = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int group = p.n_q_heads / p.n_kv_heads;

  const int tok = p.items[item];
  const int pos = p.positions[tok];
  const int r = p.tok_req[tok];
  bool bad = (pos < 0 || r < 0 || r >= p.n_reqs);
  if (bad && threadIdx.x == 0) set_error(p.err, pos < 0 ? kErrPosition : kErrRequest, tok, pos, r);
  const int* table = p.block_table + (size_t)(bad ? 0 : p.req_slot[r]) * p.max_pages;
  const int lo = (!bad && p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;

  // key tiles of this block
  const int first_tile = lo / kDecTile;
  const int last_tile = bad ? first_tile - 1 : pos / kDecTile;
  const int n_tiles = last_tile - first_tile + 1;
  const int per_split = (n_tiles + p.n_splits - 1) / p.n_splits;
  const int my_begin = first_tile + split * per_split;
  const int my_end = min(my_begin + per_split, last_tile + 1);

  unsigned char* my_smem = smem + warp * STAGES * STAGE_BYTES;
  const uint32_t my_smem_u32 = smem_u32(my_smem);

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};

  // ---- asynchronous load of one 16-key tile of K and V into a stage ------------------------
  auto issue_load = [&](int tile, int stage) {
    const int key0 = tile * kDecTile;
    const int pidx = key0 / p.page_size;
    int page = (pidx < p.max_pages) ? table[pidx] : -1;
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) set_error(p.err, kErrPage, tok, pidx, page);
      page = -1;
    }
    const size_t row0 = ((size_t)(page < 0 ? 0 : page) * p.n_kv_heads + hkv) * p.page_size +
                        (key0 % p.page_size);
    const __nv_bfloat16* ksrc = p.k_cache + row0 * D;
    const __nv_bfloat16* vsrc = p.v_cache + row0 * D;
    const uint32_t kdst = my_smem_u32 + stage * STAGE_BYTES;
    const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < (kDecTile * CH) / 32; ++i) {
      const int idx = i * 32 + lane;
      const int row = idx / CH, chunk = idx % CH;
      const int key = key0 + row;
      const bool valid = (page >= 0) && key >= lo && key <= pos;
      const int off = swizzled_offset(row, chunk, CH);
      cp_async16(kdst + off, ksrc + (size_t)row * D + chunk * 8, valid);
      cp_async16(vdst + off, vsrc + (size_t)row * D + chunk * 8, valid);
    }
  };

  // tiles of this warp: my_begin + warp, + kDecWarps, ...
  const int n_mine = (my_end - my_begin - warp + kDecWarps - 1) / kDecWarps;
  // Warm start.  The batch description and the block tables were written before the chain of
  // kernels of this step began, and the kernel before this one writes the cache only at the
  // new tokens' places, for this token at `pos`.  Tiles that end below `pos` are therefore
  // requested before the wait on that kernel; the tile that holds `pos`, and the queries, after.
  int warm = 0;
#pragma unroll
  for (; warm < STAGES - 1; ++warm) {
    const int tile = my_begin + warp + warm * kDecWarps;
    if (warm >= n_mine || tile >= last_tile) break;
    issue_load(tile, warm);
    cp_async_commit();
  }
  if (threadIdx.x == 0) tl_mark(2, 0);
  pdl_wait();
  if (threadIdx.x == 0) tl_mark(2, 1);
  // ---- query fragments: row g of the tile is query head hkv * group + g --------------------
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qbase = p.q + ((size_t)tok * p.n_q_heads + (size_t)hkv * group) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c0 = ks * 16 + 2 * t4;
      qa[ks][0] = (g < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g * D + c0) : 0u;
      qa[ks][2] = (g < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g * D + c0 + 8) : 0u;
      qa[ks][1] = (g + 8 < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)(g + 8) * D + c0) : 0u;
      qa[ks][3] = (g + 8 < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)(g + 8) * D + c0 + 8) : 0u;
    }
  }

  for (int s = warm; s < STAGES - 1; ++s) {
    if (s < n_mine) issue_load(my_begin + warp + s * kDecWarps, s);
    cp_async_commit();
  }

  for (int i = 0; i < n_mine; ++i) {
    const int tile = my_begin + warp + i * kDecWarps;
    {
      const int nxt = i + STAGES - 1;
      if (nxt < n_mine) issue_load(my_begin + warp + nxt * kDecWarps, nxt % STAGES);
      cp_async_commit();
    }
    cp_async_wait<STAGES - 1>();
    __syncwarp();

    const uint32_t kbase = my_smem_u32 + (i % STAGES) * STAGE_BYTES;
    const uint32_t vbase = kbase + TILE_BYTES;

    // scores of 16 rows x 16 keys
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int row = ((lane >> 4) << 3) + (lane & 7);
      const int chunk = 2 * ks + ((lane >> 3) & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(kbase + swizzled_offset(row, chunk, CH), b0, b1, b2, b3);
      mma_bf16_16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      mma_bf16_16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
    }

    // mask, running maximum, probabilities
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = tile * kDecTile + nt * 8 + 2 * t4 + (e & 1);
        const bool valid = key >= lo && key <= pos;
        s[nt][e] = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
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
    for (int nt = 0; nt < 2; ++nt) {
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

    // output += P * V
    const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]);
    const uint32_t pa1 = pack_bf16(s[0][2], s[0][3]);
    const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]);
    const uint32_t pa3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int c = 0; c < D / 8; c += 2) {
      const int row = (((lane >> 3) & 1) << 3) + (lane & 7);
      const int chunk = c + (lane >> 4);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vbase + swizzled_offset(row, chunk, CH), b0, b1, b2, b3);
      mma_bf16_16816(o[c], pa0, pa1, pa2, pa3, b0, b1);
      mma_bf16_16816(o[c + 1], pa0, pa1, pa2, pa3, b2, b3);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  if (threadIdx.x == 0) tl_mark(2, 2);

  // ---- merge the warps --------------------------------------------------------------------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();   // every warp is done with its stages; the memory is reused below
  float* so = reinterpret_cast<float*>(smem);                  // [warps][16][D]
  float* sml = so + kDecWarps * 16 * D;                        // [warps][16][2]
#pragma unroll
  for (int i2 = 0; i2 < D / 8; ++i2) {
    const int col = i2 * 8 + 2 * t4;
    float* row0 = so + ((size_t)warp * 16 + g) * D + col;
    float* row1 = so + ((size_t)warp * 16 + g + 8) * D + col;
    row0[0] = o[i2][0]; row0[1] = o[i2][1];
    row1[0] = o[i2][2]; row1[1] = o[i2][3];
  }
  if (t4 == 0) {
    sml[(warp * 16 + g) * 2 + 0] = m_run[0];     sml[(warp * 16 + g) * 2 + 1] = l_run[0];
    sml[(warp * 16 + g + 8) * 2 + 0] = m_run[1]; sml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < group * D; idx += kDecWarps * 32) {
    const int row = idx / D, col = idx % D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) m_all = fmaxf(m_all, sml[(w * 16 + row) * 2]);
    float acc = 0.0f, l_all = 0.0f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sml[(w * 16 + row) * 2];
      const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - m_all);
      acc += so[((size_t)w * 16 + row) * D + col] * f;
      l_all += sml[(w * 16 + row) * 2 + 1] * f;
    }
    if (p.n_splits == 1) {
      // the only block of this (token, kv head): its sums are the result
      const float inv = 1.0f / l_all;
      p.out[((size_t)tok * p.n_q_heads + (size_t)hkv * group + row) * D + col] = __float2bfloat16_rn(acc * inv);
    } else {
      const size_t pidx = ((size_t)item * p.n_q_heads + (size_t)hkv * group + row) * p.n_splits + split;
      p.part_o[pidx * D + col] = acc;
      if (col == 0) { p.part_ml[pidx * 2] = m_all; p.part_ml[pidx * 2 + 1] = l_all; }
    }
  }
  if (p.n_splits == 1) return;

  // ---- the last block of this (token, kv head) merges the splits ------------------------------
  __shared__ int s_last;
  __threadfence();                       // this block's partial result is visible before it is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(&p.counters[item * p.n_kv_heads + hkv], 1);
    s_last = (arrived == p.n_splits - 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) tl_mark(2, s_last ? 3 : 4);
  if (!s_last) return;
  __threadfence();                       // and the others' partial results before they are read
  // A thread adds up four neighbouring columns of one row over the splits, always in the order of
  // the splits, sixteen independent 16-byte loads at a time so that their latencies overlap; the
  // first sixteen are requested before the weights are worked out.
  constexpr int kMergeChunk = 16;
  constexpr int V4 = D / 4;
  const int n_vec = group * V4;
  auto load_chunk = [&](int idx, int s0, float4 (&v)[kMergeChunk]) {
    const int row = idx / V4, c4 = idx % V4;
    const size_t base = ((size_t)item * p.n_q_heads + (size_t)hkv * group + row) * p.n_splits;
    const float4* src = reinterpret_cast<const float4*>(p.part_o + base * D) + c4;
#pragma unroll
    for (int u = 0; u < kMergeChunk; ++u) {
      v[u] = (s0 + u < p.n_splits) ? __ldcg(src + (size_t)(s0 + u) * V4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  };
  float4 first[kMergeChunk];
  if ((int)threadIdx.x < n_vec) load_chunk(threadIdx.x, 0, first);
  // weights of the splits, row by row: f_s = 2^(m_s - m) / sum_s l_s 2^(m_s - m)
  float* sf = reinterpret_cast<float*>(smem);            // [group][n_splits]
  for (int row = warp; row < group; row += kDecWarps) {
    const size_t base = ((size_t)item * p.n_q_heads + (size_t)hkv * group + row) * p.n_splits;
    float m_loc[kDecMaxSplits / 32], l_loc[kDecMaxSplits / 32];
    float m_all = -INFINITY;
#pragma unroll
    for (int k = 0; k < kDecMaxSplits / 32; ++k) {
      const int s2 = k * 32 + lane;
      m_loc[k] = -INFINITY; l_loc[k] = 0.0f;
      if (s2 < p.n_splits) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(&p.part_ml[(base + s2) * 2]));
        m_loc[k] = ml.x; l_loc[k] = ml.y;
      }
      m_all = fmaxf(m_all, m_loc[k]);
    }
    m_all = warp_max(m_all);
    float l_all = 0.0f;
#pragma unroll
    for (int k = 0; k < kDecMaxSplits / 32; ++k) {
      m_loc[k] = (m_loc[k] == -INFINITY) ? 0.0f : exp2f(m_loc[k] - m_all);
      l_all += l_loc[k] * m_loc[k];
    }
    l_all = warp_sum(l_all);
    const float inv = 1.0f / l_all;
#pragma unroll
    for (int k = 0; k < kDecMaxSplits / 32; ++k) {
      const int s2 = k * 32 + lane;
      if (s2 < p.n_splits) sf[row * p.n_splits + s2] = m_loc[k] * inv;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_vec; idx += kDecWarps * 32) {
    const int row = idx / V4, c4 = idx % V4;
    const float* f = sf + row * p.n_splits;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s0 = 0; s0 < p.n_splits; s0 += kMergeChunk) {
      float4 v[kMergeChunk];
      if (s0 == 0 && idx == (int)threadIdx.x) {
#pragma unroll
        for (int u = 0; u < kMergeChunk; ++u) v[u] = first[u];
      } else {
        load_chunk(idx, s0, v);
      }
#pragma unroll
      for (int u = 0; u < kMergeChunk; ++u) {
        const float w = (s0 + u < p.n_splits) ? f[s0 + u] : 0.0f;
        acc.x += v[u].x * w; acc.y += v[u].y * w; acc.z += v[u].z * w; acc.w += v[u].w * w;
      }
    }
    uint2 packed;
    packed.x = pack_bf16(acc.x, acc.y);
    packed.y = pack_bf16(acc.z, acc.w);
    *reinterpret_cast<uint2*>(p.out + ((size_t)tok * p.n_q_heads + (size_t)hkv * group + row) * D + c4 * 4) = packed;
  }
  if (threadIdx.x == 0) { p.counters[item * p.n_kv_heads + hkv] = 0; tl_mark(2, 4); }
}

// ---- the same attention with the work dealt out evenly ---------------------------------------------
//
// The kernel above gives every (token, kv head) the same number of splits, so its blocks are as
// many as that product allows, not as many as the GPU holds: 512 blocks of equal length at batch
// 64 run as one and three quarter waves of 296, 256 blocks at batch 8 leave 40 SMs with half the
// work of the others.  Here the 16-key tiles of all (token, kv head) pairs form one sequence,
// pair after pair, and block b of G takes the tiles [T b / G, T (b + 1) / G): a run that ends
// one pair, covers whole pairs, and begins another.  A pair that lies wholly in one block is
// written out by it.  A part of a pair goes to one of the block's two scratch slots as an
// unnormalised sum with its maximum and normaliser; the blocks of a pair count their arrivals,
// and the last one merges the parts in the order of the blocks and puts the counter back to zero.
// The inner loop, the masking and the merge arithmetic are those of the kernel above.

constexpr int kDecBalMaxItems = 1024;
// The merging block keeps one weight per (query head of the group, block of the pair) in shared memory:
// 16 x 512 floats are 32 KB, less than the stages of either head size.
constexpr int kDecBalMaxBlocks = 512;

struct DecodeBalParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  float* parts;                 // [blocks][2][16 rows][D + 2]: unnormalised output, maximum, normaliser
  int* counters;                // [n_items, n_kv_heads]; zero before and after
  __nv_bfloat16* out;
  const int* items;
  const int* positions;
  const int* tok_req;
  const int* req_slot;
  const int* block_table;
  int* err;
  int n_items, n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages, window;
  float scale_log2;
};

// The block that holds tile t of the sequence of T tiles: the largest c with T c / G <= t.
__device__ __forceinline__ int bal_owner(long long T, int G, long long t) {
  return (int)(((t + 1) * G + T - 1) / T) - 1;
}

template <int D>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_balanced_kernel(DecodeBalParams p) {
  pdl_trigger();
  constexpr int CH = D / 8;
  constexpr int TILE_BYTES = kDecTile * D * 2;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int SLOT_FLOATS = 16 * (D + 2);
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_first[kDecBalMaxItems + 1];      // tiles of the items before item i (times kv heads: tiles of their pairs)
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int H = p.n_kv_heads;
  const int group = p.n_q_heads / H;
  const int b = blockIdx.x, G = gridDim.x;

  // ---- tiles of every item, and their running sum -------------------------------------------------
  if (threadIdx.x == 0) s_first[0] = 0;
  for (int i = threadIdx.x; i < p.n_items; i += kDecWarps * 32) {
    const int tok = p.items[i];
    const int pos = p.positions[tok];
    const int r = p.tok_req[tok];
    int tiles = 0;
    if (pos < 0 || r < 0 || r >= p.n_reqs) {
      set_error(p.err, pos < 0 ? kErrPosition : kErrRequest, tok, pos, r);
    } else {
      const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
      tiles = pos / kDecTile - lo / kDecTile + 1;
    }
    s_first[i + 1] = tiles;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < p.n_items; base += 32) {
      int v = (base + lane < p.n_items) ? s_first[base + lane + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (base + lane < p.n_items) s_first[base + lane + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  const long long T = (long long)s_first[p.n_items] * H;
  const long long t_begin = T * b / G, t_end = T * (b + 1) / G;
  if (t_begin >= t_end) return;

  // the item that holds tile t_begin: the largest i with s_first[i] * H <= t_begin
  int item = 0;
  {
    int lo_i = 0, hi_i = p.n_items - 1;
    while (lo_i < hi_i) {
      const int mid = (lo_i + hi_i + 1) >> 1;
      if ((long long)s_first[mid] * H <= t_begin) lo_i = mid; else hi_i = mid - 1;
    }
    item = lo_i;
  }

  unsigned char* my_smem = smem + warp * kDecStages * STAGE_BYTES;
  const uint32_t my_smem_u32 = smem_u32(my_smem);
  bool waited = false;
  long long t = t_begin;
  while (t < t_end) {
    const int tiles_item = s_first[item + 1] - s_first[item];
    const long long item_base = (long long)s_first[item] * H;
    if (tiles_item == 0 || t >= item_base + (long long)tiles_item * H) { ++item; continue; }
    const int hkv = (int)((t - item_base) / tiles_item);
    const long long pair_base = item_base + (long long)hkv * tiles_item;
    const int tile0 = (int)(t - pair_base);
    const long long room = t_end - pair_base;
    const int tile1 = room < tiles_item ? (int)room : tiles_item;
    const bool whole = (tile0 == 0 && tile1 == tiles_item);
    const int slot = (t == t_begin) ? 0 : 1;
    t = pair_base + tile1;

    const int tok = p.items[item];
    const int pos = p.positions[tok];
    const int r = p.tok_req[tok];
    const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int first_tile = lo / kDecTile;
    const int last_tile = pos / kDecTile;
    const int my_begin = first_tile + tile0;
    const int my_end = first_tile + tile1;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};

    auto issue_load = [&](int tile, int stage) {
      const int key0 = tile * kDecTile;
      const int pidx = key0 / p.page_size;
      int page = (pidx < p.max_pages) ? table[pidx] : -1;
      if (page < 0 || page >= p.num_pages) {
        if (lane == 0) set_error(p.err, kErrPage, tok, pidx, page);
        page = -1;
      }
      const size_t row0 = ((size_t)(page < 0 ? 0 : page) * p.n_kv_heads + hkv) * p.page_size +
                          (key0 % p.page_size);
      const __nv_bfloat16* ksrc = p.k_cache + row0 * D;
      const __nv_bfloat16* vsrc = p.v_cache + row0 * D;
      const uint32_t kdst = my_smem_u32 + stage * STAGE_BYTES;
      const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
      for (int i = 0; i < (kDecTile * CH) / 32; ++i) {
        const int idx = i * 32 + lane;
        const int row = idx / CH, chunk = idx % CH;
        const int key = key0 + row;
        const bool valid = (page >= 0) && key >= lo && key <= pos;
        const int off = swizzled_offset(row, chunk, CH);
        cp_async16(kdst + off, ksrc + (size_t)row * D + chunk * 8, valid);
        cp_async16(vdst + off, vsrc + (size_t)row * D + chunk * 8, valid);
      }
    };

    const int n_mine = (my_end - my_begin - warp + kDecWarps - 1) / kDecWarps;
    int warm = 0;
    if (!waited) {
      // tiles that end below the new token's place were written by earlier steps: they are
      // requested before the wait on the kernel that writes this step's keys and values
#pragma unroll
      for (; warm < kDecStages - 1; ++warm) {
        const int tile = my_begin + warp + warm * kDecWarps;
        if (warm >= n_mine || tile >= last_tile) break;
        issue_load(tile, warm);
        cp_async_commit();
      }
      pdl_wait();
      waited = true;
    }
    uint32_t qa[D / 16][4];
    {
      const __nv_bfloat16* qbase = p.q + ((size_t)tok * p.n_q_heads + (size_t)hkv * group) * D;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int c0 = ks * 16 + 2 * t4;
        qa[ks][0] = (g < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g * D + c0) : 0u;
        qa[ks][2] = (g < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g * D + c0 + 8) : 0u;
        qa[ks][1] = (g + 8 < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)(g + 8) * D + c0) : 0u;
        qa[ks][3] = (g + 8 < group) ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)(g + 8) * D + c0 + 8) : 0u;
      }
    }
    for (int s = warm; s < kDecStages - 1; ++s) {
      if (s < n_mine) issue_load(my_begin + warp + s * kDecWarps, s);
      cp_async_commit();
    }

    for (int i = 0; i < n_mine; ++i) {
      const int tile = my_begin + warp + i * kDecWarps;
      {
        const int nxt = i + kDecStages - 1;
        if (nxt < n_mine) issue_load(my_begin + warp + nxt * kDecWarps, nxt % kDecStages);
        cp_async_commit();
      }
      cp_async_wait<kDecStages - 1>();
      __syncwarp();
      const uint32_t kbase = my_smem_u32 + (i % kDecStages) * STAGE_BYTES;
      const uint32_t vbase = kbase + TILE_BYTES;
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int row = ((lane >> 4) << 3) + (lane & 7);
        const int chunk = 2 * ks + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kbase + swizzled_offset(row, chunk, CH), b0, b1, b2, b3);
        mma_bf16_16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16_16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = tile * kDecTile + nt * 8 + 2 * t4 + (e & 1);
          const bool valid = key >= lo && key <= pos;
          s[nt][e] = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
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
      for (int nt = 0; nt < 2; ++nt) {
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
      const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]);
      const uint32_t pa1 = pack_bf16(s[0][2], s[0][3]);
      const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]);
      const uint32_t pa3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int c = 0; c < D / 8; c += 2) {
        const int row = (((lane >> 3) & 1) << 3) + (lane & 7);
        const int chunk = c + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vbase + swizzled_offset(row, chunk, CH), b0, b1, b2, b3);
        mma_bf16_16816(o[c], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16_16816(o[c + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
      __syncwarp();
    }
    cp_async_wait<0>();

    // ---- merge the warps ------------------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();
    float* so = reinterpret_cast<float*>(smem);
    float* sml = so + kDecWarps * 16 * D;
#pragma unroll
    for (int i2 = 0; i2 < D / 8; ++i2) {
      const int col = i2 * 8 + 2 * t4;
      float* row0 = so + ((size_t)warp * 16 + g) * D + col;
      float* row1 = so + ((size_t)warp * 16 + g + 8) * D + col;
      row0[0] = o[i2][0]; row0[1] = o[i2][1];
      row1[0] = o[i2][2]; row1[1] = o[i2][3];
    }
    if (t4 == 0) {
      sml[(warp * 16 + g) * 2 + 0] = m_run[0];     sml[(warp * 16 + g) * 2 + 1] = l_run[0];
      sml[(warp * 16 + g + 8) * 2 + 0] = m_run[1]; sml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    float* part = p.parts + ((size_t)b * 2 + slot) * SLOT_FLOATS;
    for (int idx = threadIdx.x; idx < group * D; idx += kDecWarps * 32) {
      const int row = idx / D, col = idx % D;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) m_all = fmaxf(m_all, sml[(w * 16 + row) * 2]);
      float acc = 0.0f, l_all = 0.0f;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float mw = sml[(w * 16 + row) * 2];
        const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - m_all);
        acc += so[((size_t)w * 16 + row) * D + col] * f;
        l_all += sml[(w * 16 + row) * 2 + 1] * f;
      }
      if (whole) {
        p.out[((size_t)tok * p.n_q_heads + (size_t)hkv * group + row) * D + col] = __float2bfloat16_rn(acc / l_all);
      } else {
        part[row * D + col] = acc;
        if (col == 0) { part[16 * D + row * 2] = m_all; part[16 * D + row * 2 + 1] = l_all; }
      }
    }
    if (!whole) {
      // ---- count this part; the last block of the pair merges the parts ---------------------------
      const int c_first = bal_owner(T, G, pair_base);
      const int c_last = bal_owner(T, G, pair_base + tiles_item - 1);
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        int n_contrib = c_last - c_first + 1;
        if (T < G) {                      // fewer tiles than blocks: some blocks in between hold nothing
          n_contrib = 0;
          for (int c = c_first; c <= c_last; ++c) n_contrib += (T * (c + 1) / G > T * c / G) ? 1 : 0;
        }
        int* counter = p.counters + item * H + hkv;
        const int arrived = atomicAdd(counter, 1);
        s_last = (arrived == n_contrib - 1);
        if (s_last) *counter = 0;
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        // the slot of block c for this pair: its first segment if its run begins inside the pair
        auto part_of = [&](int c) -> const float* {
          const long long cb = T * c / G;
          return p.parts + ((size_t)c * 2 + (cb >= pair_base ? 0 : 1)) * SLOT_FLOATS;
        };
        const int n_c = c_last - c_first + 1;
        float* sf = reinterpret_cast<float*>(smem);          // [group][n_c] weights of the parts
        for (int row = warp; row < group; row += kDecWarps) {
          float m_all = -INFINITY;
          for (int c = lane; c < n_c; c += 32) {
            const bool has = T * (c_first + c + 1) / G > T * (c_first + c) / G;
            const float m = has ? __ldcg(part_of(c_first + c) + 16 * D + row * 2) : -INFINITY;
            sf[row * n_c + c] = m;
            m_all = fmaxf(m_all, m);
          }
          m_all = warp_max(m_all);
          float l_all = 0.0f;
          for (int c = lane; c < n_c; c += 32) {
            const float m = sf[row * n_c + c];
            const float f = (m == -INFINITY) ? 0.0f : exp2f(m - m_all);
            if (f != 0.0f) l_all += __ldcg(part_of(c_first + c) + 16 * D + row * 2 + 1) * f;
            sf[row * n_c + c] = f;
          }
          l_all = warp_sum(l_all);
          const float inv = 1.0f / l_all;
          __syncwarp();
          for (int c = lane; c < n_c; c += 32) sf[row * n_c + c] *= inv;
        }
        __syncthreads();
        constexpr int V4 = D / 4;
        constexpr int kChunk = 8;
        for (int idx = threadIdx.x; idx < group * V4; idx += kDecWarps * 32) {
          const int row = idx / V4, c4 = idx % V4;
          const float* f = sf + row * n_c;
          float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          for (int c0 = 0; c0 < n_c; c0 += kChunk) {
            float4 v[kChunk];
#pragma unroll
            for (int u = 0; u < kChunk; ++u) {
              const bool has = c0 + u < n_c && f[c0 + u] != 0.0f;
              v[u] = has ? __ldcg(reinterpret_cast<const float4*>(part_of(c_first + c0 + u) + row * D) + c4)
                         : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < kChunk; ++u) {
              const float w = (c0 + u < n_c) ? f[c0 + u] : 0.0f;
              acc.x += v[u].x * w; acc.y += v[u].y * w; acc.z += v[u].z * w; acc.w += v[u].w * w;
            }
          }
          uint2 packed;
          packed.x = pack_bf16(acc.x, acc.y);
          packed.y = pack_bf16(acc.z, acc.w);
          *reinterpret_cast<uint2*>(p.out + ((size_t)tok * p.n_q_heads + (size_t)hkv * group + row) * D + c4 * 4) = packed;
        }
      }
    }
    __syncthreads();          // the stages are loaded into again
  }
}

template <int D>
static int launch_decode_balanced(const DecodeBalParams& p, int blocks, cudaStream_t stream) {
  constexpr int smem_bytes = kDecWarps * kDecStages * 2 * kDecTile * D * 2;
  static_assert(16 * kDecBalMaxBlocks * 4 <= smem_bytes, "the weights of the parts do not fit the stages");
  static_assert(kDecWarps * 16 * D * 4 + kDecWarps * 16 * 2 * 4 <= smem_bytes, "merge area too small");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_balanced_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch(attn_decode_balanced_kernel<D>, dim3(blocks), dim3(kDecWarps * 32), smem_bytes, stream, p);
}

template <int D, int STAGES>
static int launch_decode_stages(const DecodeParams& p, cudaStream_t stream) {
  constexpr int smem_bytes = kDecWarps * STAGES * 2 * kDecTile * D * 2;
  static_assert(kDecWarps * 16 * D * 4 + kDecWarps * 16 * 2 * 4 <= smem_bytes, "merge area too small");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<D, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.n_splits, p.n_kv_heads, p.n_items);
  return (int)launch(attn_decode_split_kernel<D, STAGES>, grid, dim3(kDecWarps * 32), smem_bytes, stream, p);
}

// Three stages per warp (96 KB at head_dim 128: two blocks to an SM) where the grid fits two
// blocks to an SM anyway; two stages (64 KB, three blocks to an SM, by registers too) where it is
// larger: a block more per SM is then resident and has its first tiles on the way while the
// kernel before still runs.  Measured at Qwen3-8B sizes, context 4,096, whole decode steps: two
// stages with up to three blocks per SM +1.2 % at batch 8 and +1.5 % at batch 16 (6 and 3 splits);
// two stages for a grid of 256 blocks -1.1 % at batch 1 and -5 % at batch 32.
template <int D>
static int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  static int sm_count[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
  if (sms == 0) {
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) sm_count[dev] = sms;
  }
  const long long blocks = (long long)p.n_splits * p.n_kv_heads * p.n_items;
  if (blocks > 2LL * sms) return launch_decode_stages<D, 2>(p, stream);
  return launch_decode_stages<D, 3>(p, stream);
}

}  // namespace tk

TK_TIMELINE_SETTER(attention_decode)

// Floats of scratch that tk_attention_decode needs: partial outputs, then (max, sum) pairs.
// Beside them it needs n_items * n_kv_heads int counters that are zero before the call (the
// kernel leaves them at zero).
TK_API long long tk_attention_decode_scratch_floats(int n_items, int n_q_heads, int head_dim,
                                                    int n_splits) {
  return (long long)n_items * n_q_heads * n_splits * (head_dim + 2);
}

TK_API int tk_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                               float* scratch, int* counters, const int* items, const int* positions,
                               const int* tok_req, const int* req_slot, const int* block_table,
                               int* err, int n_items, int n_reqs, int n_q_heads, int n_kv_heads,
                               int head_dim, int page_size, int max_pages, int num_pages, int window,
                               int n_splits, float scale, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  const int group = n_kv_heads > 0 ? n_q_heads / n_kv_heads : 0;
  if (n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || group > 16 || page_size % 16 != 0 ||
      n_splits < 1 || n_splits > tk::kDecMaxSplits || n_items > 65535 || n_kv_heads > 65535 ||
      (head_dim != 64 && head_dim != 128)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::DecodeParams p;
  p.q = (const __nv_bfloat16*)q;
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
  p.part_o = scratch;
  p.part_ml = scratch + (size_t)n_items * n_q_heads * n_splits * head_dim;
  p.counters = counters; p.out = (__nv_bfloat16*)out;
  p.items = items; p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot;
  p.block_table = block_table; p.err = err;
  p.n_items = n_items; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.window = window;
  p.n_splits = n_splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 128) return tk::launch_decode<128>(p, stream);
  return tk::launch_decode<64>(p, stream);
}

// The same attention with the tiles of all (token, kv head) pairs dealt out evenly over `blocks`
// blocks (see attn_decode_balanced_kernel).  scratch holds blocks * 2 * 16 * (head_dim + 2) floats,
// counters n_items * n_kv_heads ints that are zero before the call and after it.
TK_API long long tk_attention_decode_balanced_scratch_floats(int blocks, int head_dim) {
  return (long long)blocks * 2 * 16 * (head_dim + 2);
}

TK_API int tk_attention_decode_balanced(const void* q, void* out, const void* k_cache, const void* v_cache,
                                        float* scratch, int* counters, const int* items, const int* positions,
                                        const int* tok_req, const int* req_slot, const int* block_table,
                                        int* err, int n_items, int n_reqs, int n_q_heads, int n_kv_heads,
                                        int head_dim, int page_size, int max_pages, int num_pages, int window,
                                        int blocks, float scale, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  const int group = n_kv_heads > 0 ? n_q_heads / n_kv_heads : 0;
  if (n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || group > 16 || page_size % 16 != 0 || blocks < 1 ||
      blocks > tk::kDecBalMaxBlocks || n_items > tk::kDecBalMaxItems || (head_dim != 64 && head_dim != 128)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::DecodeBalParams p;
  p.q = (const __nv_bfloat16*)q; p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.parts = scratch; p.counters = counters; p.out = (__nv_bfloat16*)out;
  p.items = items; p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot;
  p.block_table = block_table; p.err = err;
  p.n_items = n_items; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 128) return tk::launch_decode_balanced<128>(p, blocks, stream);
  return tk::launch_decode_balanced<64>(p, blocks, stream);
}
