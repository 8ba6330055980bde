// Paged flash attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head_dim 64 or 128).
//
// One thread block per (tile of 128 query tokens of one request, query head):
//   warp 0      TMA: the query tile once, then key and value tiles of 64 keys, page by page
//               (cp.async.bulk.tensor, 128-byte swizzle, no multicast), into a ring of stages;
//   warp 1      one thread issues tcgen05.mma: S = Q K^T (M 128, N 64) into one of two score
//               buffers in tensor memory, and O += P V (M 128, N head_dim) with V read straight
//               from its page layout as an MN-major operand;
//   warps 2..5  softmax: thread i owns query row i = tensor-memory lane i.  It reads its 64
//               scores with tcgen05.ld, masks (causal with offset kv_len - q_len, window),
//               keeps a reference maximum and the normaliser in float32, writes the
//               probabilities as bfloat16 into a swizzled shared tile for the second product,
//               and rescales the output accumulator in tensor memory only when the row maximum
//               has grown by more than 2^8 since the reference was set (the probabilities stay
//               below 2^8, exact enough in bfloat16; the result is the same softmax).
// The score buffers and the probability tiles are double-buffered, so the products of one key
// tile overlap the softmax of the next.
//
// Pages are loaded whole.  A page that lies outside the tile's visible keys is replaced by the
// page of the tile's last key (its probabilities are exactly zero), and the kernel that writes
// the cache zero-fills the unwritten rest of a request's last page, so no stale value can turn
// a zero probability into a NaN.  Every mbarrier wait is bounded and reports kErrWait.
#include "tcgen05_utils.cuh"

namespace tk {

constexpr int kAtBM = 128;
constexpr int kAtBN = 64;
constexpr int kAtStages = 3;
constexpr int kAtThreads = 192;
constexpr float kAtRescale = 8.0f;    // log2 units

struct AttnTcParams {
  __nv_bfloat16* out;            // [n_tokens, n_q_heads, D]
  const int* tiles;              // [n_tiles, 2]: request row, 128-token tile index within its tokens
  const int* req_q_start;
  const int* req_q_len;
  const int* req_kv_len;
  const int* req_slot;
  const int* block_table;
  int* err;
  int n_tiles, n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages, window;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kAtThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, AttnTcParams p) {
  constexpr int SUB = D / 64;                          // 64-column sub-tiles per row
  constexpr uint32_t Q_BYTES = kAtBM * D * 2;
  constexpr uint32_t KSUB_BYTES = kAtBN * 64 * 2;      // one sub-tile of a key or value tile
  constexpr uint32_t KV_BYTES = kAtBN * D * 2;         // one key tile (or one value tile)
  constexpr uint32_t STAGE_BYTES = 2 * KV_BYTES;
  constexpr uint32_t P_BYTES = kAtBM * kAtBN * 2;
  constexpr uint32_t TMEM_COLS = 256;                  // S0: 0..63, S1: 64..127, O: 128..128+D-1

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t raw = gt_smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t kv_smem = q_smem + Q_BYTES;
  const uint32_t p_smem = kv_smem + kAtStages * STAGE_BYTES;
  unsigned char* ctrl = smem + Q_BYTES + kAtStages * STAGE_BYTES + 2 * P_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* q_full = bars;                  // 1
  uint64_t* kv_full = bars + 1;             // kAtStages
  uint64_t* kv_empty = kv_full + kAtStages; // kAtStages
  uint64_t* s_full = kv_empty + kAtStages;  // 2
  uint64_t* s_empty = s_full + 2;           // 2
  uint64_t* p_full = s_empty + 2;           // 2
  uint64_t* p_empty = p_full + 2;           // 2
  uint64_t* o_full = p_empty + 2;           // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_id = blockIdx.x, head = blockIdx.y;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int hkv = head / group;

  pdl_trigger();
  if (threadIdx.x == 0) {
    mbar_init(gt_smem_u32(q_full), 1);
    for (int s = 0; s < kAtStages; ++s) {
      mbar_init(gt_smem_u32(&kv_full[s]), 1);
      mbar_init(gt_smem_u32(&kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(gt_smem_u32(&s_full[b]), 1);
      mbar_init(gt_smem_u32(&s_empty[b]), 4);
      mbar_init(gt_smem_u32(&p_full[b]), 4);
      mbar_init(gt_smem_u32(&p_empty[b]), 1);
    }
    mbar_init(gt_smem_u32(o_full), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(gt_smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();     // queries, cache pages and the step's tables come from earlier kernels and copies

  // ---- the tile's geometry (identical in every thread) -----------------------------------------
  const int r = p.tiles[2 * tile_id];
  const int ti = p.tiles[2 * tile_id + 1];
  bool geometry_ok = (r >= 0 && r < p.n_reqs);
  int q_start = 0, q_len = 0, kv_len = 0;
  if (geometry_ok) { q_start = p.req_q_start[r]; q_len = p.req_q_len[r]; kv_len = p.req_kv_len[r]; }
  const int row0 = ti * kAtBM;
  const int rows_here = min(kAtBM, q_len - row0);
  geometry_ok = geometry_ok && rows_here > 0 && kv_len >= q_len;
  if (!geometry_ok && threadIdx.x == 0) set_error(p.err, kErrRequest, tile_id, r, q_len);
  const int pos0 = kv_len - q_len + row0;
  const int pos_last = pos0 + rows_here - 1;
  const int lo_tile = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int first_kt = lo_tile / kAtBN;
  const int n_kt = geometry_ok ? (pos_last / kAtBN - first_kt + 1) : 0;

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------------
    if (lane == 0 && n_kt > 0) {
      const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;
      mbar_expect_tx(gt_smem_u32(q_full), Q_BYTES);
#pragma unroll
      for (int c = 0; c < SUB; ++c) {
        tma_load_3d(q_smem + c * (kAtBM * 128), &map_q, c * 64, head, q_start + row0, gt_smem_u32(q_full));
      }
      const int kpl = p.page_size < kAtBN ? p.page_size : kAtBN;     // keys per load
      for (int it = 0; it < n_kt; ++it) {
        const int s = it % kAtStages;
        const uint32_t round = (uint32_t)(it / kAtStages);
        if (round > 0 && !mbar_wait(gt_smem_u32(&kv_empty[s]), (round - 1) & 1u, abort_flag)) {
          set_error(p.err, kErrWait, 10, it, s);
          *abort_flag = 1;
          break;
        }
        const uint32_t full = gt_smem_u32(&kv_full[s]);
        mbar_expect_tx(full, STAGE_BYTES);
        const uint32_t kdst = kv_smem + s * STAGE_BYTES;
        const uint32_t vdst = kdst + KV_BYTES;
        const int kt = first_kt + it;
        for (int u = 0; u < kAtBN / kpl; ++u) {
          int key0 = kt * kAtBN + u * kpl;
          if (key0 + kpl - 1 < lo_tile || key0 > pos_last) key0 = (pos_last / kpl) * kpl;   // nothing visible here
          const int pidx = key0 / p.page_size;
          int page = (pidx < p.max_pages) ? table[pidx] : -1;
          if (page < 0 || page >= p.num_pages) {
            set_error(p.err, kErrPage, tile_id, pidx, page);
            page = 0;
          }
          const int row = (page * p.n_kv_heads + hkv) * p.page_size + (key0 % p.page_size);
#pragma unroll
          for (int c = 0; c < SUB; ++c) {
            tma_load_2d(kdst + c * KSUB_BYTES + u * kpl * 128, &map_k, c * 64, row, full);
            tma_load_2d(vdst + c * KSUB_BYTES + u * kpl * 128, &map_v, c * 64, row, full);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer --------------------------------------------------------------------------
    if (lane == 0 && n_kt > 0) {
      const uint32_t idesc_s = umma_idesc(kAtBN, false);
      const uint32_t idesc_o = umma_idesc(D, true);
      const uint32_t tmem_o = tmem_base + 128;
      bool ok = mbar_wait(gt_smem_u32(q_full), 0u, abort_flag);
      if (!ok) { set_error(p.err, kErrWait, 11, 0, 0); *abort_flag = 1; }
      for (int j = 0; j <= n_kt && ok; ++j) {
        if (j < n_kt) {
          const int s = j % kAtStages;
          ok = mbar_wait(gt_smem_u32(&kv_full[s]), (uint32_t)(j / kAtStages) & 1u, abort_flag);
          if (ok && j >= 2) ok = mbar_wait(gt_smem_u32(&s_empty[j & 1]), (uint32_t)((j >> 1) - 1) & 1u, abort_flag);
          if (!ok) { set_error(p.err, kErrWait, 12, j, s); *abort_flag = 1; break; }
          tc_fence_after();
          const uint32_t k_addr = kv_smem + s * STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t da = umma_desc_sw128(q_smem + (ks / 4) * (kAtBM * 128)) + (uint64_t)(2 * (ks % 4));
            const uint64_t db = umma_desc_sw128(k_addr + (ks / 4) * KSUB_BYTES) + (uint64_t)(2 * (ks % 4));
            umma_bf16(tmem_base + (uint32_t)(j & 1) * kAtBN, da, db, idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(gt_smem_u32(&s_full[j & 1]));
        }
        if (j >= 1) {
          const int jj = j - 1;
          const int s = jj % kAtStages;
          ok = mbar_wait(gt_smem_u32(&p_full[jj & 1]), (uint32_t)(jj >> 1) & 1u, abort_flag);
          if (!ok) { set_error(p.err, kErrWait, 13, jj, s); *abort_flag = 1; break; }
          tc_fence_after();
          const uint32_t v_addr = kv_smem + s * STAGE_BYTES + KV_BYTES;
          const uint32_t p_addr = p_smem + (uint32_t)(jj & 1) * P_BYTES;
#pragma unroll
          for (int kk = 0; kk < kAtBN / 16; ++kk) {
            const uint64_t da = umma_desc_sw128(p_addr) + (uint64_t)(2 * kk);
            const uint64_t db = umma_desc_sw128_mn(v_addr + kk * (16 * 128), KSUB_BYTES);
            umma_bf16(tmem_o, da, db, idesc_o, (jj > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(gt_smem_u32(&kv_empty[s]));
          umma_commit(gt_smem_u32(&p_empty[jj & 1]));
        }
      }
      if (ok) umma_commit(gt_smem_u32(o_full));
    }
  } else {
    // ---- softmax and epilogue: row = tensor-memory lane ---------------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool row_valid = row < rows_here;
    const int pos_r = pos0 + row;
    const int lo_r = (p.window > 0 && pos_r - p.window + 1 > 0) ? pos_r - p.window + 1 : 0;
    float m_ref = -INFINITY, l_sum = 0.0f;
    bool ok = true;

    for (int j = 0; j < n_kt && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&s_full[j & 1]), (uint32_t)(j >> 1) & 1u, abort_flag));
      if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 14, j, 0); *abort_flag = 1; } break; }
      tc_fence_after();
      uint32_t sraw[kAtBN];
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[32]);
        tmem_ld32(tmem_base + lane_addr + (uint32_t)(j & 1) * kAtBN, lo);
        tmem_ld32(tmem_base + lane_addr + (uint32_t)(j & 1) * kAtBN + 32, hi);
        tmem_wait_ld();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(gt_smem_u32(&s_empty[j & 1]));

      // Scores stay unscaled in sv; the softmax scale (> 0) is folded into the exponent below.
      // A tile wholly below this row's diagonal and inside its window needs no mask.
      const int key_first = (first_kt + j) * kAtBN;
      const bool interior = row_valid && key_first + kAtBN - 1 <= pos_r && key_first >= lo_r;
      float mx = -INFINITY;
      float sv[kAtBN];
      if (interior) {
#pragma unroll
        for (int c = 0; c < kAtBN; ++c) {
          sv[c] = __uint_as_float(sraw[c]);
          mx = fmaxf(mx, sv[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < kAtBN; ++c) {
          const int key = key_first + c;
          const bool valid = row_valid && key <= pos_r && key >= lo_r;
          sv[c] = valid ? __uint_as_float(sraw[c]) : -INFINITY;
          mx = fmaxf(mx, sv[c]);
        }
      }
      mx *= p.scale_log2;       // -inf stays -inf
      const float m_new = fmaxf(m_ref, mx);
      const bool need = m_new > m_ref + kAtRescale;     // also true when the first visible key arrives
      if (__any_sync(0xffffffffu, need)) {
        const float corr = need ? exp2f(m_ref - m_new) : 1.0f;
        if (need) { l_sum *= corr; m_ref = m_new; }
        if (j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&p_empty[(j - 1) & 1]),
                                                 (uint32_t)((j - 1) >> 1) & 1u, abort_flag));
          if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 15, j, 0); *abort_flag = 1; } break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_base + lane_addr + 128 + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st32(tmem_base + lane_addr + 128 + c * 32, o);
          }
          tmem_wait_st();
          tc_fence_before();
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
      float psum = 0.0f;
#pragma unroll
      for (int c = 0; c < kAtBN; ++c) {
        sv[c] = exp2f(fmaf(sv[c], p.scale_log2, -m_use));
        psum += sv[c];
      }
      l_sum += psum;

      if (j >= 2) {     // the probability tile is free once the second product of tile j - 2 is done
        ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&p_empty[j & 1]), (uint32_t)((j - 2) >> 1) & 1u,
                                               abort_flag));
        if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 16, j, 0); *abort_flag = 1; } break; }
      }
      unsigned char* prow = smem + Q_BYTES + kAtStages * STAGE_BYTES + (size_t)(j & 1) * P_BYTES +
                            (size_t)(row >> 3) * 1024 + (size_t)(row & 7) * 128;
#pragma unroll
      for (int ch = 0; ch < kAtBN / 8; ++ch) {
        uint4 v;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(sv[ch * 8 + 2 * e], sv[ch * 8 + 2 * e + 1]);
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = v;
      }
      fence_async_shared();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(gt_smem_u32(&p_full[j & 1]));
    }

    if (ok && n_kt > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(o_full), 0u, abort_flag));
      if (!ok && lane == 0) { set_error(p.err, kErrWait, 17, 0, 0); *abort_flag = 1; }
    }
    if (ok && n_kt > 0) {
      tc_fence_after();
      const float inv = (row_valid && l_sum > 0.0f) ? 1.0f / l_sum : 0.0f;
      __nv_bfloat16* orow = p.out + ((size_t)(q_start + row0 + row) * p.n_q_heads + head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_addr + 128 + c * 32, o);
        tmem_wait_ld();
        if (row_valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              h2[e] = __floats2bfloat162_rn(__uint_as_float(o[q4 * 8 + 2 * e]) * inv,
                                            __uint_as_float(o[q4 * 8 + 2 * e + 1]) * inv);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = v;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

template <int D>
static int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                             const AttnTcParams& p, cudaStream_t stream) {
  constexpr size_t smem_bytes = (size_t)kAtBM * D * 2 + (size_t)kAtStages * 2 * kAtBN * D * 2 +
                                2 * (size_t)kAtBM * kAtBN * 2 + 1024 /* alignment */ + 256 /* barriers */;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.n_tiles, p.n_q_heads);
  return (int)launch(attn_prefill_tc_kernel<D>, grid, dim3(kAtThreads), smem_bytes, stream, mq, mk, mv, p);
}

}  // namespace tk

// Whether tk_attention_prefill_tc takes a shape.
TK_API int tk_attention_prefill_tc_takes(int n_q_heads, int n_kv_heads, int head_dim, int page_size) {
  const bool pages_ok = page_size >= 8 && page_size % 8 == 0 && (64 % page_size == 0 || page_size % 64 == 0);
  return (head_dim == 64 || head_dim == 128) && n_kv_heads >= 1 && n_q_heads % n_kv_heads == 0 && pages_ok;
}

TK_API int tk_attention_prefill_tc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                   const int* tiles, const int* req_q_start, const int* req_q_len,
                                   const int* req_kv_len, const int* req_slot, const int* block_table,
                                   int* err, int n_tokens, int n_tiles, int n_reqs, int n_q_heads,
                                   int n_kv_heads, int head_dim, int page_size, int max_pages, int num_pages,
                                   int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!tk_attention_prefill_tc_takes(n_q_heads, n_kv_heads, head_dim, page_size) || n_q_heads > 65535) {
    return (int)cudaErrorInvalidValue;
  }
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)n_q_heads, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)n_q_heads * head_dim * 2};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)tk::kAtBM};
    int rc = tk::make_bf16_map(&mq, q, 3, dims, strides, box);
    if (rc != 0) return rc;
  }
  {
    const int kpl = page_size < tk::kAtBN ? page_size : tk::kAtBN;
    cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)num_pages * n_kv_heads * page_size};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)kpl};
    int rc = tk::make_bf16_map(&mk, k_cache, 2, dims, strides, box);
    if (rc != 0) return rc;
    rc = tk::make_bf16_map(&mv, v_cache, 2, dims, strides, box);
    if (rc != 0) return rc;
  }
  tk::AttnTcParams p;
  p.out = (__nv_bfloat16*)out; p.tiles = tiles; p.req_q_start = req_q_start; p.req_q_len = req_q_len;
  p.req_kv_len = req_kv_len; p.req_slot = req_slot; p.block_table = block_table; p.err = err;
  p.n_tiles = n_tiles; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 128) return tk::launch_prefill_tc<128>(mq, mk, mv, p, stream);
  return tk::launch_prefill_tc<64>(mq, mk, mv, p, stream);
}
