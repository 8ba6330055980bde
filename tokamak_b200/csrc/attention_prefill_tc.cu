// Paged flash attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head_dim 64 or 128).
//
// One thread block per (256 query tokens of one request, query head), handled as two query
// tiles of 128 rows that share every key and value tile:
//   warp 0       TMA: the query tiles once, then key and value tiles of 64 keys, page by page
//                (cp.async.bulk.tensor, 128-byte swizzle, every block for itself), into a ring of stages;
//                every lane looks one page up and issues one copy, so the look-ups of a stage
//                cost one memory latency, and the next stage's are under way while it waits;
//   warps 1, 10  one thread each issues tcgen05.mma for one query tile: S = Q K^T (M 128, N 64)
//                into one of the tile's two score buffers in tensor memory, and O += P V
//                (M 128, N head_dim) with P read from tensor memory and V straight from its page
//                layout as an MN-major operand (issuing is what a single thread is slow at,
//                hence one per tile);
//   warps 2..5   softmax of query tile 0, warps 6..9 of query tile 1: thread i owns query row
//                i = tensor-memory lane i.  It reads its 64 scores with tcgen05.ld, masks
//                (causal with offset kv_len - q_len, window), keeps a reference maximum and
//                the normaliser in float32, writes the probabilities as bfloat16 pairs over the
//                scores they came from (tcgen05.st), where the second product takes them as its
//                A operand straight from tensor memory, and rescales the output accumulator in
//                tensor memory only when the row maximum has grown by more than 2^8 since the
//                reference was set (the probabilities stay below 2^8, exact enough in bfloat16;
//                the result is the same softmax).
// Every query tile has two score buffers, so the tensor cores work for one tile, or on the next
// key tile, while the other tile's softmax runs; a buffer is written again only by a product that
// the same thread issues after the one that read the probabilities in it, and the tensor cores
// run a thread's products in order.  Two softmax warps share every scheduler.
//
// Pages are loaded whole.  A page that lies outside the block's visible keys is replaced by the
// page of the block's last key (its probabilities are exactly zero), and the kernel that writes
// the cache zero-fills the unwritten rest of a request's last page, so no stale value can turn
// a zero probability into a NaN.  Every mbarrier wait is bounded and reports kErrWait.
#include "tcgen05_utils.cuh"

namespace tk {

constexpr int kAtBM = 128;            // rows of one query tile
constexpr int kAtQT = 2;              // query tiles per block
constexpr int kAtBN = 64;             // keys per tile
constexpr int kAtStages = 3;
constexpr int kAtThreads = 64 + kAtQT * 128 + 32;   // TMA, MMA of tile 0, softmax warps, MMA of tile 1
constexpr int kAtMmaWarp1 = 2 + kAtQT * 4;           // the warp that issues for query tile 1
constexpr float kAtRescale = 8.0f;    // log2 units

struct AttnTcParams {
  __nv_bfloat16* out;            // [n_tokens, n_q_heads, D]
  const int* tiles;              // [n_tiles, 2]: request row, index of the 256-token tile within its tokens
  const int* req_q_start;
  const int* req_q_len;
  const int* req_kv_len;
  const int* req_slot;
  const int* block_table;
  int* err;
  int n_tiles, n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages, window;
  float scale_log2;
};

// Two float32 operations in one instruction (sm_100): the softmax warps are bound by the
// instructions they issue, so halving the multiply-adds and additions shows.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kAtThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, AttnTcParams p) {
  constexpr int SUB = D / 64;                          // 64-column sub-tiles per row
  constexpr uint32_t Q_BYTES = kAtBM * D * 2;          // one query tile
  constexpr uint32_t KSUB_BYTES = kAtBN * 64 * 2;      // one sub-tile of a key or value tile
  constexpr uint32_t KV_BYTES = kAtBN * D * 2;         // one key tile (or one value tile)
  constexpr uint32_t STAGE_BYTES = 2 * KV_BYTES;
  constexpr uint32_t TMEM_COLS = 512;   // per query tile t: scores at t*128 + {0, 64}; outputs at 256 + t*128
  constexpr uint32_t DATA_BYTES = kAtQT * Q_BYTES + kAtStages * STAGE_BYTES;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t raw = gt_smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t kv_smem = q_smem + kAtQT * Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DATA_BYTES);
  uint64_t* q_full = bars;                  // 1
  uint64_t* kv_full = bars + 1;             // kAtStages
  uint64_t* kv_empty = kv_full + kAtStages; // kAtStages
  uint64_t* tile_bars = kv_empty + kAtStages;   // per query tile: s_full[2] p_full[2] p_empty[2] o_full
  auto s_full = [&](int t, int b) { return gt_smem_u32(tile_bars + t * 7 + b); };
  auto p_full = [&](int t, int b) { return gt_smem_u32(tile_bars + t * 7 + 2 + b); };
  auto p_empty = [&](int t, int b) { return gt_smem_u32(tile_bars + t * 7 + 4 + b); };
  auto o_full = [&](int t) { return gt_smem_u32(tile_bars + t * 7 + 6); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tile_bars + kAtQT * 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads vary fastest: the tiles are listed with the most keys first, so the blocks start in
  // that order over all heads (the short ones fill the end), and the query heads that share a
  // kv head run at the same time and find its keys and values in L2
  const int head = blockIdx.x, tile_id = blockIdx.y;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int hkv = head / group;

  pdl_trigger();
  if (threadIdx.x == 0) {
    mbar_init(gt_smem_u32(q_full), 1);
    for (int s = 0; s < kAtStages; ++s) {
      mbar_init(gt_smem_u32(&kv_full[s]), 1);
      mbar_init(gt_smem_u32(&kv_empty[s]), kAtQT);      // one arrival per issuing warp
    }
    for (int t = 0; t < kAtQT; ++t) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(s_full(t, b), 1);
        mbar_init(p_full(t, b), 4);
        mbar_init(p_empty(t, b), 1);
      }
      mbar_init(o_full(t), 1);
    }
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

  // ---- geometry of the block and of its query tiles (identical in every thread) ----------------
  const int r = p.tiles[2 * tile_id];
  const int ti = p.tiles[2 * tile_id + 1];
  bool geometry_ok = (r >= 0 && r < p.n_reqs);
  int q_start = 0, q_len = 0, kv_len = 0;
  if (geometry_ok) { q_start = p.req_q_start[r]; q_len = p.req_q_len[r]; kv_len = p.req_kv_len[r]; }
  const int row0 = ti * (kAtQT * kAtBM);
  const int rows_block = min(kAtQT * kAtBM, q_len - row0);
  geometry_ok = geometry_ok && rows_block > 0 && kv_len >= q_len;
  if (!geometry_ok && threadIdx.x == 0) set_error(p.err, kErrRequest, tile_id, r, q_len);
  const int n_qt = !geometry_ok ? 0 : (rows_block > kAtBM ? 2 : 1);
  // query tile t: rows [t*128, t*128 + rows_t), positions pos0_t .., key tiles [first_t, last_t]
  int rows_t[kAtQT], pos0_t[kAtQT], first_t[kAtQT], last_t[kAtQT];
#pragma unroll
  for (int t = 0; t < kAtQT; ++t) {
    rows_t[t] = min(kAtBM, rows_block - t * kAtBM);
    pos0_t[t] = kv_len - q_len + row0 + t * kAtBM;
    const int lo = (p.window > 0 && pos0_t[t] - p.window + 1 > 0) ? pos0_t[t] - p.window + 1 : 0;
    first_t[t] = lo / kAtBN;
    last_t[t] = (pos0_t[t] + rows_t[t] - 1) / kAtBN;
  }
  const int lo_block = (p.window > 0 && pos0_t[0] - p.window + 1 > 0) ? pos0_t[0] - p.window + 1 : 0;
  const int pos_last = n_qt > 0 ? pos0_t[n_qt - 1] + rows_t[n_qt - 1] - 1 : 0;
  const int first_kt = first_t[0];
  const int n_kt = n_qt > 0 ? last_t[n_qt - 1] - first_kt + 1 : 0;

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------------
    if (n_kt > 0) {
      const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;
      if (lane == 0) {
        mbar_expect_tx(gt_smem_u32(q_full), (uint32_t)n_qt * Q_BYTES);
        for (int t = 0; t < n_qt; ++t) {
#pragma unroll
          for (int c = 0; c < SUB; ++c) {
            tma_load_3d(q_smem + t * Q_BYTES + c * (kAtBM * 128), &map_q, c * 64, head,
                        q_start + row0 + t * kAtBM, gt_smem_u32(q_full));
          }
        }
      }
      // a stage is (64 / kpl) page parts x SUB column halves x {key, value}: one copy per lane
      const int kpl = p.page_size < kAtBN ? p.page_size : kAtBN;     // keys per load
      const int n_loads = (kAtBN / kpl) * SUB * 2;                   // at most 32: page sizes from 8
      const bool loader = lane < n_loads;
      const int is_v = lane & 1, c = (lane >> 1) % SUB, u = lane / (2 * SUB);
      auto key0_of = [&](int it) {
        int key0 = (first_kt + it) * kAtBN + u * kpl;
        if (key0 + kpl - 1 < lo_block || key0 > pos_last) key0 = (pos_last / kpl) * kpl;   // nothing visible here
        return key0;
      };
      auto lookup = [&](int it) {
        const int pidx = key0_of(it) / p.page_size;
        return (loader && it < n_kt && pidx < p.max_pages) ? table[pidx] : -1;
      };
      int page = lookup(0);
      bool ok = true;
      for (int it = 0; it < n_kt; ++it) {
        const int s = it % kAtStages;
        const uint32_t round = (uint32_t)(it / kAtStages);
        const int page_next = lookup(it + 1);          // under way while this stage waits and is issued
        if (round > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&kv_empty[s]), (round - 1) & 1u, abort_flag));
          if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 10, it, s); *abort_flag = 1; } break; }
        }
        const uint32_t full = gt_smem_u32(&kv_full[s]);
        if (lane == 0) mbar_expect_tx(full, STAGE_BYTES);
        __syncwarp();
        if (loader) {
          const int key0 = key0_of(it);
          if (page < 0 || page >= p.num_pages) {
            set_error(p.err, kErrPage, tile_id, key0 / p.page_size, page);
            page = 0;
          }
          const int row = (page * p.n_kv_heads + hkv) * p.page_size + (key0 % p.page_size);
          const uint32_t dst = kv_smem + s * STAGE_BYTES + (is_v ? KV_BYTES : 0u) + c * KSUB_BYTES + u * kpl * 128;
          tma_load_2d(dst, is_v ? &map_v : &map_k, c * 64, row, full);
        }
        page = page_next;
      }
    }
  } else if (warp == 1 || warp == kAtMmaWarp1) {
    // ---- MMA issuer of query tile t ------------------------------------------------------------
    // Both issuers walk all key tiles of the block, so that each gives every stage back exactly
    // once; a tile outside the query tile's own range gets no products.
    const int t = warp == 1 ? 0 : 1;
    if (lane == 0 && n_kt > 0) {
      const uint32_t idesc_s = umma_idesc(kAtBN, false);
      const uint32_t idesc_o = umma_idesc(D, true);
      const bool mine = t < n_qt;
      // The descriptors are made once; a product adds what changes (16-byte units in the low bits):
      // issuing is a chain of dependent instructions in one thread, and every one of them counts.
      const uint64_t desc_q = umma_desc_sw128(q_smem + t * Q_BYTES);
      const uint64_t desc_k = umma_desc_sw128(kv_smem);
      const uint64_t desc_v = umma_desc_sw128_mn(kv_smem + KV_BYTES, KSUB_BYTES);
      const uint32_t tmem_o_t = tmem_base + (uint32_t)(256 + t * 128);
      bool ok = mbar_wait(gt_smem_u32(q_full), 0u, abort_flag);
      if (!ok) { set_error(p.err, kErrWait, 11, 0, t); *abort_flag = 1; }
      for (int j = 0; j <= n_kt && ok; ++j) {
        if (j < n_kt) {
          const int s = j % kAtStages;
          const int kt = first_kt + j;
          ok = mbar_wait(gt_smem_u32(&kv_full[s]), (uint32_t)(j / kAtStages) & 1u, abort_flag);
          if (!ok) { set_error(p.err, kErrWait, 12, j, s); *abort_flag = 1; break; }
          if (mine && kt >= first_t[t] && kt <= last_t[t]) {
            const uint64_t desc_ks = desc_k + (uint64_t)((uint32_t)s * (STAGE_BYTES >> 4));
            const int jt = kt - first_t[t], b = jt & 1;
            const uint32_t tmem_sb = tmem_base + (uint32_t)(t * 128 + b * kAtBN);
            // the score buffer also held the probabilities of key tile jt - 2: the second product
            // that read them was issued by this thread before, and the products run in order
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint64_t da = desc_q + (uint64_t)((ks / 4) * ((kAtBM * 128) >> 4) + 2 * (ks % 4));
              const uint64_t db = desc_ks + (uint64_t)((ks / 4) * (KSUB_BYTES >> 4) + 2 * (ks % 4));
              umma_bf16(tmem_sb, da, db, idesc_s, ks > 0 ? 1u : 0u);
            }
            umma_commit(s_full(t, b));
          }
        }
        if (j >= 1) {
          const int s = (j - 1) % kAtStages;
          const int kt = first_kt + j - 1;
          if (mine && kt >= first_t[t] && kt <= last_t[t]) {
            const uint64_t desc_vs = desc_v + (uint64_t)((uint32_t)s * (STAGE_BYTES >> 4));
            const int jt = kt - first_t[t], b = jt & 1;
            ok = mbar_wait(p_full(t, b), (uint32_t)(jt >> 1) & 1u, abort_flag);
            if (!ok) { set_error(p.err, kErrWait, 13, j, t); *abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t p_tmem = tmem_base + (uint32_t)(t * 128 + b * kAtBN);   // 16 keys = 8 columns
#pragma unroll
            for (int kk = 0; kk < kAtBN / 16; ++kk) {
              const uint64_t db = desc_vs + (uint64_t)(kk * ((16 * 128) >> 4));
              umma_bf16_ts(tmem_o_t, p_tmem + (uint32_t)(8 * kk), db, idesc_o, (jt > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(p_empty(t, b));
            if (kt == last_t[t]) umma_commit(o_full(t));
          }
          umma_commit(gt_smem_u32(&kv_empty[s]));    // this issuer is done with the stage
        }
      }
    }
  } else {
    // ---- softmax and epilogue of query tile t: row = tensor-memory lane ---------------------------
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_addr + (uint32_t)(t * 128);
    const uint32_t tmem_o = tmem_base + lane_addr + (uint32_t)(256 + t * 128);
    const bool active = t < n_qt;
    const int my_rows = active ? rows_t[t] : 0;
    const bool row_valid = row < my_rows;
    const int pos_r = pos0_t[t] + row;
    const int lo_r = (p.window > 0 && pos_r - p.window + 1 > 0) ? pos_r - p.window + 1 : 0;
    const int my_kt = active ? last_t[t] - first_t[t] + 1 : 0;
    float m_ref = -INFINITY, l_sum = 0.0f;
    bool ok = true;

    for (int j = 0; j < my_kt && ok; ++j) {
      const int b = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full(t, b), (uint32_t)(j >> 1) & 1u, abort_flag));
      if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 14, j, t); *abort_flag = 1; } break; }
      tc_fence_after();
      uint32_t sraw[kAtBN];
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[32]);
        tmem_ld32(tmem_s + (uint32_t)(b * kAtBN), lo);
        tmem_ld32(tmem_s + (uint32_t)(b * kAtBN) + 32, hi);
        tmem_wait_ld();
      }

      // Scores stay unscaled in sv; the softmax scale (> 0) is folded into the exponent below.
      // A tile wholly below this row's diagonal and inside its window needs no mask.
      const int key_first = (first_t[t] + j) * kAtBN;
      const bool interior = row_valid && key_first + kAtBN - 1 <= pos_r && key_first >= lo_r;
      float mx = -INFINITY;
      float sv[kAtBN];
      if (interior) {
#pragma unroll
        for (int c = 0; c < kAtBN; c += 2) {
          sv[c] = __uint_as_float(sraw[c]);
          sv[c + 1] = __uint_as_float(sraw[c + 1]);
          mx = max3(mx, sv[c], sv[c + 1]);
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
          ok = __all_sync(0xffffffffu, mbar_wait(p_empty(t, (j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u,
                                                 abort_flag));
          if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 15, j, t); *abort_flag = 1; } break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st32(tmem_o + c * 32, o);
          }
          tmem_wait_st();
          tc_fence_before();
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
      float2 psum = make_float2(0.0f, 0.0f);
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-m_use, -m_use);
#pragma unroll
      for (int c = 0; c < kAtBN; c += 2) {
        const float2 x = fma2(make_float2(sv[c], sv[c + 1]), scale2, shift2);
        sv[c] = ex2_approx(x.x);
        sv[c + 1] = ex2_approx(x.y);
        psum = add2(psum, make_float2(sv[c], sv[c + 1]));
      }
      l_sum += psum.x + psum.y;

      // the probabilities take the place of the scores they came from: bfloat16 pairs in the
      // first half of the score buffer, where the second product reads its A operand
      {
        uint32_t packed[kAtBN / 2];
#pragma unroll
        for (int c = 0; c < kAtBN / 2; ++c) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(sv[2 * c], sv[2 * c + 1]);
          packed[c] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        tmem_st32(tmem_s + (uint32_t)(b * kAtBN), packed);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(t, b));
    }

    if (ok && my_kt > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(o_full(t), 0u, abort_flag));
      if (!ok && lane == 0) { set_error(p.err, kErrWait, 17, 0, t); *abort_flag = 1; }
    }
    if (ok && my_kt > 0) {
      tc_fence_after();
      const float inv = (row_valid && l_sum > 0.0f) ? 1.0f / l_sum : 0.0f;
      __nv_bfloat16* orow = p.out + ((size_t)(q_start + row0 + t * kAtBM + row) * p.n_q_heads + head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + c * 32, o);
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
  constexpr size_t smem_bytes = (size_t)kAtQT * kAtBM * D * 2 + (size_t)kAtStages * 2 * kAtBN * D * 2 +
                                1024 /* alignment */ + 512 /* barriers */;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (p.n_tiles > 65535) return (int)cudaErrorInvalidValue;
  dim3 grid(p.n_q_heads, p.n_tiles);
  return (int)launch(attn_prefill_tc_kernel<D>, grid, dim3(kAtThreads), smem_bytes, stream, mq, mk, mv, p);
}

}  // namespace tk

// Query tokens that one block of tk_attention_prefill_tc covers (the tile list is cut by this).
TK_API int tk_attention_prefill_tc_rows(void) { return tk::kAtQT * tk::kAtBM; }

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
