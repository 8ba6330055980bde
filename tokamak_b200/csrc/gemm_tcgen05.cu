// bfloat16 matrix product for few tokens (decoding) on the 5th-generation tensor cores:
//   D[t, n] = sum_k X[t, k] * W[n, k]      (both operands K-major, float32 accumulation)
//
// The weight is the 128-row operand of the MMA and the tokens (at most 256, usually 1 to 64) its
// N side, so every byte of the weights is streamed exactly once.  One thread block per (128-row
// tile of W, token tile, K split).  Operand tiles of 64 k-elements travel global -> shared memory
// by TMA (cp.async.bulk.tensor, 128-byte swizzle, every block for itself) into a ring of stages
// guarded by mbarriers; one elected thread issues tcgen05.mma (M = 128, N = token tile, K = 16)
// with the accumulator in tensor memory; four epilogue warps read it with tcgen05.ld.
//
// The K range is split over blocks to fill the GPU.  The blocks of one output tile form a
// thread-block cluster: each stages its float32 partial accumulator in its own shared memory, and
// every block adds up its share of the token columns over distributed shared memory, always in
// the same order, and stores the float32 result [1, token, N_out] (no atomics).  Without the
// cluster every split stores its partial [split, token, N_out] and the consuming kernel adds
// them up.  The library's product takes the place of this kernel in the reference
// (src/tokamak/model/transformer.py:38-41).
//
// Every wait on an mbarrier is bounded; a wait that runs out records kErrWait, raises a
// block-wide abort flag and the block leaves through the common exit that frees its
// tensor memory.
#include "tcgen05_utils.cuh"
#include "timeline.cuh"

namespace tk {

constexpr int kGtBM = 128;        // rows of R per block = UMMA M
constexpr int kGtBK = 64;         // k-elements per stage = one 128-byte swizzle span of bf16
constexpr int kGtThreads = 192;   // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue
// Epilogue for a stacked gate/up weight whose rows alternate in blocks of
// 64 (64 gate rows, then the 64 up rows of the same outputs): a 128-row tile then holds both
// halves of 64 outputs, and the block that adds the splits up stores
// bf16(silu(gate) * up) as [token, rows / 2] instead of the float32 sums.
constexpr int kGtEpiSwiglu = 1;
// Epilogue for a product that ends a residual branch: the block that adds the
// splits up adds the sums to the float32 residual stream in place, stores
// bf16(residual * norm weight) for the product that follows the next RMSNorm, and the tile's
// share of every token's sum of squares.  The consumer of these (see colscale below) multiplies
// its own sums by rsqrt(mean square + eps): the norm between two products needs no kernel of its
// own (src/tokamak/model/layers.py:28-33, transformer.py:107-108; the 32-bit statistics are the
// same, the rounding to bfloat16 happens before instead of after the scaling by the statistic).
constexpr int kGtEpiResidualNorm = 2;
// Epilogue for the stacked q|k|v projection of heads of 128 elements, where a 128-row tile is one
// head of one token per column: the warp that adds the splits up holds the whole head, so it
// applies the per-head RMSNorm of q and k and the half rotation, stores q as bfloat16
// [token, head, 128] and writes k (normed and rotated) and v (as it is) into the token's place in
// its cache page.  Formulas and page addressing are those of the separate kernel in rope_kv.cu
// (src/tokamak/model/transformer.py:71-73, layers.py:56-89, memory/paged_cache.py:72-81).
constexpr int kGtEpiQkvRope = 3;
constexpr int kGtHeadDim = 128;   // the only head size of that epilogue

struct GemmQkvRope {
  __nv_bfloat16* q_out;     // [tokens, n_q_heads, 128]
  __nv_bfloat16* k_cache;   // [num_pages, n_kv_heads, page_size, 128]
  __nv_bfloat16* v_cache;
  const int* positions;     // [tokens]
  const int* tok_req;       // [tokens] row of the token's request in this step
  const int* req_slot;      // [n_reqs] row of the request in block_table
  const int* block_table;   // [n_slots, max_pages]
  const int* req_q_len;     // [n_reqs] tokens the request brings to this step, or null
  const int* req_kv_len;    // [n_reqs] positions of the request after this step, or null
  const float* q_norm_w;    // [128] or null
  const float* k_norm_w;    // [128] or null
  const float2* rope_table; // [tokens, 64] (cos, sin), or null: no rotation
  int n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages;
  float eps;
};

struct GemmTcParams {
  void* out;                // float [parts, cols_total, rows_total], or what the epilogue stores
  int* err;
  int rows_total;           // rows of R
  int cols_total;           // rows of C (columns of D)
  int k_total;
  int bn;                   // UMMA N: 16..256, multiple of 16
  int n_stages;
  int n_splits;
  int cluster_reduce;       // 0, or the cluster size: that many consecutive splits of a tile
                            // form a cluster and store their sum as one part (n_splits / cluster parts)
  int epilogue;             // 0 = float32 sums; 1 = gated activation, see kGtEpiSwiglu;
                            // 2 = residual sum and preparation of the next norm, see kGtEpiResidualNorm
  // every column (token) of the sums is multiplied by
  // rsqrt(sum_i colscale_parts[i, token] * colscale_inv_dim + colscale_eps) before it is stored
  const float* colscale_parts;
  int n_colscale_parts;
  float colscale_inv_dim, colscale_eps;
  // epilogue 2: the residual stream [tokens, rows] (float32, updated in place), the norm weight [rows],
  // the prepared activations [tokens, rows] and the sums of squares [row tiles, tokens]
  float* resid;
  const float* norm_w;
  __nv_bfloat16* xb_out;
  float* sumsq_out;
  GemmQkvRope qkv;          // epilogue 3
};

// Four blocks with rings of three stages fit an SM's shared memory; the register bound keeps it so
// (grids of up to four blocks per SM then run as one wave).
__global__ void __launch_bounds__(kGtThreads, 4)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_c,
                    GemmTcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the dynamic window is only guaranteed 16-byte aligned: round up to 1024 for the swizzle
  const uint32_t raw = gt_smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_r = blockIdx.x, tile_c = blockIdx.y, split = blockIdx.z;
  // residual epilogue: what the thread's first column needs from global memory, asked for while
  // the products still run (the sums are added to it some microseconds later)
  float4 pre_r = make_float4(0.0f, 0.0f, 0.0f, 0.0f), pre_w = pre_r;
  float4 pre_cs23 = pre_r;      // q|k|v epilogue: pre_w = norm weights, pre_r / pre_cs23 = (cos, sin) pairs
  float4 pre_r2 = pre_r;        // residual epilogue: the thread's second column (more than 32 tokens)
  int pre_c = -1;
  unsigned int tl_n = 0;        // time stamps of one thread of the blocks of row tile 1 (timeline builds only)
  const bool tl_me = warp == 2 && lane == 0 && blockIdx.x == 1 && blockIdx.y == 0;
  const uint32_t r_bytes = kGtBM * kGtBK * 2;
  const uint32_t c_bytes = (uint32_t)p.bn * kGtBK * 2;
  const uint32_t stage_bytes = r_bytes + ((c_bytes + 1023u) & ~1023u);

  // barriers and bookkeeping live behind the stages
  unsigned char* ctrl = smem + (size_t)p.n_stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + p.n_stages;
  uint64_t* accum_bar = empty_bar + p.n_stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int kb_total = (p.k_total + kGtBK - 1) / kGtBK;
  const int kb_per = (kb_total + p.n_splits - 1) / p.n_splits;
  const int kb_begin = split * kb_per;
  const int kb_end = min(kb_begin + kb_per, kb_total);
  const int n_kb = max(kb_end - kb_begin, 0);
  const uint32_t tmem_cols = p.bn < 32 ? 32u : (uint32_t)p.bn;   // bn is 16, 32, 64, 128 or 256

  // the sums pass through shared memory (and the cluster) whenever anything is done to them
  const bool staged = p.cluster_reduce > 1 || p.epilogue != 0 || p.colscale_parts != nullptr;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.n_stages; ++s) {
      mbar_init(gt_smem_u32(&full_bar[s]), 1);
      mbar_init(gt_smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(gt_smem_u32(accum_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // The first ring of stages: the weight tiles (which no kernel writes) are requested at once,
    // by the thread that made the barriers, before the block has tensor memory, has met at its
    // first barrier or has waited for the previous kernel: they stream in meanwhile.  The
    // activation tiles follow after that wait.
    const int first = min(n_kb, p.n_stages);
    for (int i = 0; i < first; ++i) {
      const uint32_t full = gt_smem_u32(&full_bar[i]);
      mbar_expect_tx(full, r_bytes + c_bytes);
      tma_load_2d(base + (uint32_t)i * stage_bytes, &map_r, (kb_begin + i) * kGtBK, tile_r * kGtBM, full);
    }
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(gt_smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------------
    if (lane == 0) {
      tl_mark(10 + p.epilogue, 0);
      const int first = min(n_kb, p.n_stages);       // their weight tiles are on the way already
      pdl_wait();
      tl_mark(10 + p.epilogue, 1);
      for (int i = 0; i < first; ++i) {
        const uint32_t full = gt_smem_u32(&full_bar[i]);
        const uint32_t dst = base + (uint32_t)i * stage_bytes;
        const int k0 = (kb_begin + i) * kGtBK;
        tma_load_2d(dst + r_bytes, &map_c, k0, tile_c * p.bn, full);
      }
      for (int i = first; i < n_kb; ++i) {
        const int s = i % p.n_stages;
        const uint32_t round = (uint32_t)(i / p.n_stages);
        if (!mbar_wait(gt_smem_u32(&empty_bar[s]), (round - 1) & 1u, abort_flag)) {
          set_error(p.err, kErrWait, 0, i, s);
          *abort_flag = 1;
          break;
        }
        const uint32_t full = gt_smem_u32(&full_bar[s]);
        const uint32_t dst = base + (uint32_t)s * stage_bytes;
        mbar_expect_tx(full, r_bytes + c_bytes);
        const int k0 = (kb_begin + i) * kGtBK;
        tma_load_2d(dst, &map_r, k0, tile_r * kGtBM, full);
        tma_load_2d(dst + r_bytes, &map_c, k0, tile_c * p.bn, full);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(p.bn);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % p.n_stages;
        const uint32_t round = (uint32_t)(i / p.n_stages);
        if (!mbar_wait(gt_smem_u32(&full_bar[s]), round & 1u, abort_flag)) {
          set_error(p.err, kErrWait, 1, i, s);
          *abort_flag = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_addr = base + (uint32_t)s * stage_bytes;
        const uint64_t desc_a = umma_desc_sw128(a_addr);
        const uint64_t desc_b = umma_desc_sw128(a_addr + r_bytes);
#pragma unroll
        for (int k = 0; k < kGtBK / 16; ++k) {
          // 16 k-elements = 32 bytes further inside the swizzle span: +2 in 16-byte units
          umma_bf16(tmem_base, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                    (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(gt_smem_u32(&empty_bar[s]));     // the stage may be refilled once these MMAs are done
      }
      if (ok) umma_commit(gt_smem_u32(accum_bar));  // the accumulator is complete
      tl_mark(10 + p.epilogue, 2);
    }
  } else {
    // ---- epilogue: warps 2..5, each owns the 32 accumulator lanes of its quarter --------------
    const int quarter = warp & 3;
    bool ok = true;
    pdl_wait();   // nothing is stored before the previous kernels are done with the output buffer
    if (p.epilogue == kGtEpiResidualNorm) {
      const int cs = p.cluster_reduce > 1 ? p.cluster_reduce : 1;
      const int t = (warp - 2) * 32 + lane;
      const int c = (p.cluster_reduce > 1 ? (int)cluster_ctarank() : 0) + cs * (t >> 5);
      const int row = tile_r * kGtBM + (t & 31) * 4;
      if (c < p.bn && tile_c * p.bn + c < p.cols_total && row < p.rows_total) {
        pre_c = c;
        pre_r = *reinterpret_cast<const float4*>(p.resid + (size_t)(tile_c * p.bn + c) * p.rows_total + row);
        pre_w = *reinterpret_cast<const float4*>(p.norm_w + row);
        const int c2 = c + 4 * cs;
        if (c2 < p.bn && tile_c * p.bn + c2 < p.cols_total) {
          pre_r2 = *reinterpret_cast<const float4*>(p.resid + (size_t)(tile_c * p.bn + c2) * p.rows_total + row);
        }
      }
    }
    if (p.epilogue == kGtEpiQkvRope) {
      const GemmQkvRope& e = p.qkv;
      const int cs = p.cluster_reduce > 1 ? p.cluster_reduce : 1;
      const int t = (warp - 2) * 32 + lane;
      const int c = (p.cluster_reduce > 1 ? (int)cluster_ctarank() : 0) + cs * (t >> 5);
      if (c < p.bn && tile_c * p.bn + c < p.cols_total) {
        pre_c = c;
        const int kind = tile_r < e.n_q_heads ? 0 : (tile_r < e.n_q_heads + e.n_kv_heads ? 1 : 2);
        const float* nw = kind == 0 ? e.q_norm_w : (kind == 1 ? e.k_norm_w : nullptr);
        if (nw != nullptr) pre_w = *reinterpret_cast<const float4*>(nw + (t & 31) * 4);
        if (kind != 2 && e.rope_table != nullptr) {
          const float4* cs4 = reinterpret_cast<const float4*>(e.rope_table + (size_t)(tile_c * p.bn + c) * (kGtHeadDim / 2) +
                                                               4 * (lane & 15));
          pre_r = cs4[0];
          pre_cs23 = cs4[1];
        }
      }
    }
    // the scale of this thread's column (token), while the products still run
    float my_scale = 1.0f;
    const int my_col = (warp - 2) * 32 + lane;
    if (p.colscale_parts != nullptr && my_col < p.bn && tile_c * p.bn + my_col < p.cols_total) {
      float ss = 0.0f;
      for (int i = 0; i < p.n_colscale_parts; ++i) {
        ss += p.colscale_parts[(size_t)i * p.cols_total + tile_c * p.bn + my_col];
      }
      my_scale = rsqrtf(ss * p.colscale_inv_dim + p.colscale_eps);
    }
    // the cache row of this thread's column (token), for the tiles that hold keys or values:
    // ((page * kv heads + 0) * page_size + slot), or -1; and how many rows behind it to clear
    long long my_cache_row = -1;
    int my_zero_rows = 0;
    if (p.epilogue == kGtEpiQkvRope && tile_r >= p.qkv.n_q_heads && my_col < p.bn &&
        tile_c * p.bn + my_col < p.cols_total) {
      const GemmQkvRope& e = p.qkv;
      const int t = tile_c * p.bn + my_col;
      const int pos = e.positions[t];
      const int r = e.tok_req[t];
      if (pos < 0) {
        set_error(p.err, kErrPosition, t, pos, 0);
      } else if (r < 0 || r >= e.n_reqs) {
        set_error(p.err, kErrRequest, t, r, e.n_reqs);
      } else {
        const int pidx = pos / e.page_size;
        const int page = (pidx < e.max_pages) ? e.block_table[(size_t)e.req_slot[r] * e.max_pages + pidx] : -1;
        if (page < 0 || page >= e.num_pages) {
          set_error(p.err, kErrPage, t, pidx, page);
        } else {
          my_cache_row = (long long)page * e.n_kv_heads * e.page_size + (pos % e.page_size);
          // the request's last token of this step clears the rest of a page begun in this step
          if (e.req_kv_len != nullptr) {
            const int kv_len = e.req_kv_len[r], q_len = e.req_q_len[r];
            if (pos == kv_len - 1 && pos - pos % e.page_size >= kv_len - q_len) {
              my_zero_rows = e.page_size - 1 - pos % e.page_size;
            }
          }
        }
      }
    }
    if (n_kb > 0) {
      ok = mbar_wait(gt_smem_u32(accum_bar), 0u, abort_flag);
      if (!ok && lane == 0) { set_error(p.err, kErrWait, 2, 0, 0); *abort_flag = 1; }
    }
    if (warp == 2 && lane == 0) tl_mark(10 + p.epilogue, 3);
    if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 20, (unsigned)split);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int row = tile_r * kGtBM + quarter * 32 + lane;      // row of R = lane of the accumulator
    if (staged && my_col < p.bn) {
      // behind the staging area, in the ring of stages that the products are done with
      reinterpret_cast<float*>(smem)[p.bn * kGtBM + my_col] = my_scale;
      if (p.epilogue == kGtEpiQkvRope) {
        unsigned char* behind = smem + (size_t)p.bn * kGtBM * 4 + (size_t)p.bn * 4;   // 8-byte aligned: bn is even
        reinterpret_cast<long long*>(behind)[my_col] = my_cache_row;
        reinterpret_cast<int*>(behind + (size_t)p.bn * 8)[my_col] = my_zero_rows;
      }
    }
    for (int c0 = 0; c0 < p.bn; c0 += 16) {
      uint32_t v[16];
      if (ok && n_kb > 0) {
        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = 0u;
      }
      if (staged) {
        // stage[column][row of the tile]: consecutive lanes write consecutive words
        float* stage = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int e = 0; e < 16; ++e) stage[(c0 + e) * kGtBM + quarter * 32 + lane] = __uint_as_float(v[e]);
        continue;
      }
      if (row >= p.rows_total) continue;
      float* part = reinterpret_cast<float*>(p.out) + (size_t)split * p.cols_total * p.rows_total;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int col = tile_c * p.bn + c0 + e;              // token
        if (col < p.cols_total) part[(size_t)col * p.rows_total + row] = __uint_as_float(v[e]);
      }
    }
  }

  if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 21, (unsigned)split);
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  if (!staged) __syncthreads();            // (the cluster barrier below holds every thread of the block too)
  if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 22, (unsigned)split);
  if (staged) {
    cluster_sync_all();                    // every block of the cluster has staged its partial
    if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 23, (unsigned)split);
    const int csize = p.cluster_reduce > 1 ? p.cluster_reduce : 1;
    const uint32_t my_rank = p.cluster_reduce > 1 ? cluster_ctarank() : 0u;
    const float* s_scale = reinterpret_cast<const float*>(smem) + p.bn * kGtBM;   // this block's own copy
    if (warp >= 2 && p.epilogue == kGtEpiSwiglu) {
      // thread -> four neighbouring outputs of the tile's 64 and one of eight column phases; gate
      // in tile rows j.., up in tile rows 64 + j..; the sum over the ranks runs in the same order
      // as without the activation, and the activation is the formula of the separate kernel
      const int t = (warp - 2) * 32 + lane;
      const int j4 = (t & 15) * 4, phase = t >> 4;
      const int inter = p.rows_total >> 1;
      const int oc = tile_r * 64 + j4;
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
      if (oc < inter) {                    // inter is a multiple of 64: all four outputs exist
        for (int c = (int)my_rank + csize * phase; c < p.bn; c += 8 * csize) {
          const int col = tile_c * p.bn + c;
          if (col >= p.cols_total) break;
          float4 g = cluster_sum_f32x4(base + (uint32_t)((c * kGtBM + j4) * 4), csize);
          float4 u = cluster_sum_f32x4(base + (uint32_t)((c * kGtBM + 64 + j4) * 4), csize);
          if (p.colscale_parts != nullptr) {
            const float sc = s_scale[c];
            g.x *= sc; g.y *= sc; g.z *= sc; g.w *= sc;
            u.x *= sc; u.y *= sc; u.z *= sc; u.w *= sc;
          }
          uint2 packed;
          *reinterpret_cast<__nv_bfloat162*>(&packed.x) =
              __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
          *reinterpret_cast<__nv_bfloat162*>(&packed.y) =
              __floats2bfloat162_rn(g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w);
          *reinterpret_cast<uint2*>(out + (size_t)col * inter + oc) = packed;
        }
      }
    } else if (warp >= 2) {
      // every block of the cluster adds up its share of the columns (tokens): column c belongs
      // to rank c mod cluster size; a warp takes one column at a time, its lanes four neighbouring
      // rows each; the order of the sum over the ranks is always the same
      const int t = (warp - 2) * 32 + lane;
      const int r4 = (t & 31) * 4, phase = t >> 5;
      const int row = tile_r * kGtBM + r4;
      const bool vec = (p.rows_total & 3) == 0;
      float* out = reinterpret_cast<float*>(p.out) +
                   (size_t)(split / csize) * p.cols_total * p.rows_total;
      // with the residual epilogue the rows are a multiple of 128: every lane has its four rows
      if (row < p.rows_total) {
        for (int c = (int)my_rank + csize * phase; c < p.bn; c += 4 * csize) {
          const int col = tile_c * p.bn + c;
          if (col >= p.cols_total) break;
          // the residual and the norm weight are on their way while the partials are added up
          float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f), w = r;
          if (p.epilogue == kGtEpiResidualNorm) {
            if (c == pre_c) {
              r = pre_r;
              w = pre_w;
            } else if (pre_c >= 0 && c == pre_c + 4 * csize) {
              r = pre_r2;
              w = pre_w;
            } else {
              r = *reinterpret_cast<const float4*>(p.resid + (size_t)col * p.rows_total + row);
              w = *reinterpret_cast<const float4*>(p.norm_w + row);
            }
          }
          float4 sum = cluster_sum_f32x4(base + (uint32_t)((c * kGtBM + r4) * 4), csize);
          if (p.colscale_parts != nullptr) {
            const float sc = s_scale[c];
            sum.x *= sc; sum.y *= sc; sum.z *= sc; sum.w *= sc;
          }
          if (p.epilogue == kGtEpiQkvRope) {
            // this warp holds head `tile_r` of token `col`: lane l the elements 4 l .. 4 l + 3
            const GemmQkvRope& e = p.qkv;
            const int kind = tile_r < e.n_q_heads ? 0 : (tile_r < e.n_q_heads + e.n_kv_heads ? 1 : 2);
            const float* nw = kind == 0 ? e.q_norm_w : (kind == 1 ? e.k_norm_w : nullptr);
            if (nw != nullptr) {
              const float4 w4 = c == pre_c ? pre_w : *reinterpret_cast<const float4*>(nw + r4);
              const float ss = warp_sum(sum.x * sum.x + sum.y * sum.y + sum.z * sum.z + sum.w * sum.w);
              const float rstd = rsqrtf(ss / (float)kGtHeadDim + e.eps);
              sum.x = sum.x * rstd * w4.x; sum.y = sum.y * rstd * w4.y;
              sum.z = sum.z * rstd * w4.z; sum.w = sum.w * rstd * w4.w;
            }
            if (kind != 2 && e.rope_table != nullptr) {
              // element i < 64 turns with element i + 64, which lane l ^ 16 holds
              const float4* cs = reinterpret_cast<const float4*>(e.rope_table + (size_t)col * (kGtHeadDim / 2) +
                                                                  4 * (lane & 15));
              const float4 cs01 = c == pre_c ? pre_r : cs[0];      // (cos, sin) of two elements each
              const float4 cs23 = c == pre_c ? pre_cs23 : cs[1];
              float4 other;
              other.x = __shfl_xor_sync(0xffffffffu, sum.x, 16); other.y = __shfl_xor_sync(0xffffffffu, sum.y, 16);
              other.z = __shfl_xor_sync(0xffffffffu, sum.z, 16); other.w = __shfl_xor_sync(0xffffffffu, sum.w, 16);
              if (lane < 16) {
                sum.x = sum.x * cs01.x - other.x * cs01.y; sum.y = sum.y * cs01.z - other.y * cs01.w;
                sum.z = sum.z * cs23.x - other.z * cs23.y; sum.w = sum.w * cs23.z - other.w * cs23.w;
              } else {
                sum.x = sum.x * cs01.x + other.x * cs01.y; sum.y = sum.y * cs01.z + other.y * cs01.w;
                sum.z = sum.z * cs23.x + other.z * cs23.y; sum.w = sum.w * cs23.z + other.w * cs23.w;
              }
            }
            uint2 packed;
            *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(sum.x, sum.y);
            *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(sum.z, sum.w);
            if (kind == 0) {
              *reinterpret_cast<uint2*>(e.q_out + ((size_t)col * e.n_q_heads + tile_r) * kGtHeadDim + r4) = packed;
            } else {
              const unsigned char* behind = smem + (size_t)p.bn * kGtBM * 4 + (size_t)p.bn * 4;
              const long long cache_row = reinterpret_cast<const long long*>(behind)[c];
              const int zero_rows = reinterpret_cast<const int*>(behind + (size_t)p.bn * 8)[c];
              if (cache_row >= 0) {
                const int head = tile_r - e.n_q_heads - (kind == 2 ? e.n_kv_heads : 0);
                __nv_bfloat16* dst = (kind == 1 ? e.k_cache : e.v_cache) +
                                     ((size_t)cache_row + (size_t)head * e.page_size) * kGtHeadDim + r4;
                *reinterpret_cast<uint2*>(dst) = packed;
                for (int z = 1; z <= zero_rows; ++z) {
                  *reinterpret_cast<uint2*>(dst + (size_t)z * kGtHeadDim) = make_uint2(0u, 0u);
                }
              }
            }
            continue;
          }
          if (p.epilogue == kGtEpiResidualNorm) {
            r.x += sum.x; r.y += sum.y; r.z += sum.z; r.w += sum.w;
            *reinterpret_cast<float4*>(p.resid + (size_t)col * p.rows_total + row) = r;
            uint2 packed;
            *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(r.x * w.x, r.y * w.y);
            *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(r.z * w.z, r.w * w.w);
            *reinterpret_cast<uint2*>(p.xb_out + (size_t)col * p.rows_total + row) = packed;
            const float ss = warp_sum(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w);
            if (lane == 0) p.sumsq_out[(size_t)tile_r * p.cols_total + col] = ss;
            continue;
          }
          float* dst = out + (size_t)col * p.rows_total + row;
          if (vec && row + 3 < p.rows_total) {
            *reinterpret_cast<float4*>(dst) = sum;
          } else {
            dst[0] = sum.x;
            if (row + 1 < p.rows_total) dst[1] = sum.y;
            if (row + 2 < p.rows_total) dst[2] = sum.z;
            if (row + 3 < p.rows_total) dst[3] = sum.w;
          }
        }
      }
    }
    if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 24, (unsigned)split);
    // "I read nobody's shared memory any more"; the wait for the others stands at the very end
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(tmem_cols)
                 : "memory");
    if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 26, (unsigned)split);
    if (lane == 0) tl_mark(10 + p.epilogue, 4);
  }
  if (staged) {
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");   // nobody reads this block's either
    if (tl_me) tl_own(8 + split, tl_n, 10 + p.epilogue, 25, (unsigned)split);
  }
}

// ---- host side ------------------------------------------------------------------------------

// Map of a row-major bf16 matrix [rows, k] (row stride ld elements) with boxes of box_rows x 64.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if (((uintptr_t)ptr & 15u) != 0 || (ld * 2) % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kGtBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Checks the sizes, makes the maps and launches; `p` comes with its epilogue's fields filled in.
static int launch_gemm(const void* r, const void* c, int rows, int cols, int k, long long ld_r, long long ld_c,
                       int bn, int n_splits, int max_stages, int cluster_reduce, GemmTcParams p,
                       cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (k <= 0 || k % 8 != 0 || (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) || n_splits < 1 ||
      (cluster_reduce > 1 && (cluster_reduce > 8 || n_splits % cluster_reduce != 0)) || cluster_reduce < 0) {
    return (int)cudaErrorInvalidValue;
  }
  const bool one_part = n_splits == (cluster_reduce > 1 ? cluster_reduce : 1);
  if (p.epilogue != 0 && (p.epilogue < kGtEpiSwiglu || p.epilogue > kGtEpiQkvRope || rows % 128 != 0 || !one_part)) {
    return (int)cudaErrorInvalidValue;
  }
  if (p.colscale_parts != nullptr && (p.n_colscale_parts < 1 || !one_part)) return (int)cudaErrorInvalidValue;
  CUtensorMap map_r, map_c;
  int rc = make_map(&map_r, r, rows, k, ld_r, kGtBM);
  if (rc != 0) return rc;
  rc = make_map(&map_c, c, cols, k, ld_c, bn);
  if (rc != 0) return rc;

  const unsigned r_bytes = kGtBM * kGtBK * 2;
  const unsigned c_bytes = ((unsigned)bn * kGtBK * 2 + 1023u) & ~1023u;
  const unsigned stage_bytes = r_bytes + c_bytes;
  const int kb_total = (k + kGtBK - 1) / kGtBK;
  const int kb_per = (kb_total + n_splits - 1) / n_splits;
  int n_stages = (int)((200u * 1024u) / stage_bytes);
  if (n_stages > 8) n_stages = 8;
  if (max_stages > 0 && n_stages > max_stages) n_stages = max_stages;
  if (n_stages > kb_per) n_stages = kb_per < 2 ? 2 : kb_per;
  const size_t smem_bytes = (size_t)n_stages * stage_bytes + 1024 /* alignment slack */ + 256 /* barriers */;

  static size_t configured = 0;
  if (smem_bytes > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(220 * 1024));
    if (e != cudaSuccess) return (int)e;
    configured = 220 * 1024;
  }
  p.rows_total = rows; p.cols_total = cols; p.k_total = k; p.bn = bn;
  p.n_stages = n_stages; p.n_splits = n_splits; p.cluster_reduce = cluster_reduce;
  dim3 grid((rows + kGtBM - 1) / kGtBM, (cols + bn - 1) / bn, n_splits);
  if (cluster_reduce > 1 || p.epilogue != 0 || p.colscale_parts != nullptr) {
    // the staging area [bn][128] floats, the column scales and (q|k|v epilogue) the cache rows
    // must fit into the ring of stages
    if ((size_t)bn * kGtBM * 4 + (size_t)bn * 16 > (size_t)n_stages * stage_bytes) return (int)cudaErrorInvalidValue;
    return (int)launch_cluster_z(gemm_tcgen05_kernel, grid, dim3(kGtThreads), smem_bytes, stream,
                                 (unsigned)(cluster_reduce > 1 ? cluster_reduce : 1), map_r, map_c, p);
  }
  return (int)launch(gemm_tcgen05_kernel, grid, dim3(kGtThreads), smem_bytes, stream, map_r, map_c, p);
}

}  // namespace tk

// D^T = (R * C^T)^T on tcgen05.  r: [rows, k] bf16 (the weight, row stride ld_r), c: [cols, k] bf16
// (the tokens, row stride ld_c).  out is float32 [parts, cols, rows] (partials, to be summed by the
// consumer); parts = n_splits, or n_splits / cluster_reduce when cluster_reduce > 1 (2..8, a divisor
// of n_splits): that many consecutive splits form a thread-block cluster and store their sum.
// epilogue = 1 (rows a multiple of 128 whose gate and up rows alternate in blocks of 64, all
// splits in one cluster): out is bfloat16 [cols, rows / 2] = silu(gate) * up.
// epilogue = 2 (rows a multiple of 128, all splits in one cluster): nothing goes to out; the
// sums are added to resid [cols, rows] (float32) in place, xb_out [cols, rows] receives
// bf16(resid * norm_w) and sumsq_out [rows / 128, cols] the tiles' sums of squares of resid.
// colscale_parts (or null): [n_colscale_parts, cols] float32; the sums of column c are
// multiplied by rsqrt(sum_i colscale_parts[i, c] * colscale_inv_dim + colscale_eps).
TK_TIMELINE_SETTER(gemm_tcgen05)

TK_API int tk_gemm_bf16_tcgen05(const void* r, const void* c, void* out, int* err, int rows, int cols, int k,
                                long long ld_r, long long ld_c, int bn, int n_splits,
                                int max_stages, int cluster_reduce, int epilogue,
                                const float* colscale_parts, int n_colscale_parts, float colscale_inv_dim,
                                float colscale_eps, float* resid, const float* norm_w, void* xb_out,
                                float* sumsq_out, cudaStream_t stream) {
  if (epilogue < 0 || epilogue > tk::kGtEpiResidualNorm) return (int)cudaErrorInvalidValue;
  if (epilogue == tk::kGtEpiResidualNorm &&
      (resid == nullptr || norm_w == nullptr || xb_out == nullptr || sumsq_out == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::GemmTcParams p = {};
  p.out = out; p.err = err; p.epilogue = epilogue;
  p.colscale_parts = colscale_parts; p.n_colscale_parts = n_colscale_parts; p.colscale_inv_dim = colscale_inv_dim;
  p.colscale_eps = colscale_eps; p.resid = resid; p.norm_w = norm_w; p.xb_out = (__nv_bfloat16*)xb_out; p.sumsq_out = sumsq_out;
  return tk::launch_gemm(r, c, rows, cols, k, ld_r, ld_c, bn, n_splits, max_stages, cluster_reduce, p, stream);
}

// The stacked q|k|v projection of heads of 128 elements with the per-head norms, the rotation and
// the cache write in its epilogue (see kGtEpiQkvRope): w is [(n_q_heads + 2 n_kv_heads) * 128, k],
// x is [tokens, k]; all n_splits blocks of a tile form one cluster.  q_out receives
// [tokens, n_q_heads, 128]; keys and values go to their pages as in tk_rope_kv.
TK_API int tk_gemm_qkv_rope(const void* w, const void* x, int* err, int tokens, int k, long long ld_w, long long ld_x,
                            int bn, int n_splits, int max_stages,
                            const float* colscale_parts, int n_colscale_parts, float colscale_inv_dim,
                            float colscale_eps,
                            void* q_out, void* k_cache, void* v_cache, const int* positions, const int* tok_req,
                            const int* req_slot, const int* block_table, const int* req_q_len,
                            const int* req_kv_len, const float* q_norm_w, const float* k_norm_w,
                            const void* rope_table, int n_reqs, int n_q_heads, int n_kv_heads, int page_size,
                            int max_pages, int num_pages, float eps, cudaStream_t stream) {
  if (n_q_heads < 1 || n_kv_heads < 1 || page_size < 1 || n_splits > 8 ||
      (req_kv_len != nullptr && req_q_len == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::GemmTcParams p = {};
  p.err = err; p.epilogue = tk::kGtEpiQkvRope;
  p.colscale_parts = colscale_parts; p.n_colscale_parts = n_colscale_parts; p.colscale_inv_dim = colscale_inv_dim;
  p.colscale_eps = colscale_eps;
  tk::GemmQkvRope& e = p.qkv;
  e.q_out = (__nv_bfloat16*)q_out; e.k_cache = (__nv_bfloat16*)k_cache; e.v_cache = (__nv_bfloat16*)v_cache;
  e.positions = positions; e.tok_req = tok_req; e.req_slot = req_slot; e.block_table = block_table;
  e.req_q_len = req_q_len; e.req_kv_len = req_kv_len; e.q_norm_w = q_norm_w; e.k_norm_w = k_norm_w;
  e.rope_table = (const float2*)rope_table;
  e.n_reqs = n_reqs; e.n_q_heads = n_q_heads; e.n_kv_heads = n_kv_heads; e.page_size = page_size;
  e.max_pages = max_pages; e.num_pages = num_pages; e.eps = eps;
  const int rows = (n_q_heads + 2 * n_kv_heads) * tk::kGtHeadDim;
  return tk::launch_gemm(w, x, rows, tokens, k, ld_w, ld_x, bn, n_splits, max_stages, n_splits > 1 ? n_splits : 0,
                         p, stream);
}
