// A chain of decode products in ONE persistent kernel:
//   D_p[t, n] = sum_k X_p[t, k] * W_p[n, k],   p = 0 .. P-1,   X_p made by the epilogue of D_(p-1)
// for few tokens (at most 64), bfloat16 operands, float32 accumulation on tcgen05.
//
// Why.  With one kernel per product a decode step pays, at every product, for what cannot overlap
// with anything: the blocks of a kernel all finish at about the same time, and while they add up
// their splits and store (about 4 us) no weight streams; the next kernel's blocks then wait to be
// released (1 to 2 us).  At the Qwen3-8B sizes that is a fifth of a layer's time.  Here one block
// per SM lives through all products of the chain (attention output -> o -> gate/up -> down ->
// q|k|v of the next layer).  Its TMA producer runs through the weights of the whole chain and is
// only ever stopped by a full ring, so while one product's sums are added up and stored, and
// while the blocks meet at the barrier between two products, the next product's weights are
// already on their way into shared memory.
//
// Work.  A product is n_tiles x kb_total units (128 weight rows x 64 k-elements); block b of nb
// takes the units [U b / nb, U (b + 1) / nb) in tile-major order: a contiguous run that ends
// one tile, covers whole tiles, and begins another (stream-K).  A block that holds a tile's whole
// k range applies the epilogue itself.  A part of a tile goes, as float32, to the block's scratch
// slot in global memory; the blocks of a tile count their arrivals, and the one that arrives last
// adds the parts up in the fixed order of the blocks (so the result does not depend on timing)
// and applies the epilogue.  The split of k never depends on the number of tokens.
//
// Roles in a block: warp 0 issues the TMA loads of the weights into a ring of stages, as early as
// the ring allows, whatever product they belong to; warp 6 copies the few rows of activations of
// every stage with cp.async (a second, small TMA load per stage was measured to cost a quarter
// of the streaming rate), and only once every block has finished the product that makes them;
// warp 1 issues tcgen05.mma into one of two accumulators in tensor memory; warps 2..5 drain an
// accumulator while the other one is being filled.  Between two products the blocks meet at a
// counter in global memory (release/acquire); all blocks are resident (one per SM, the grid is
// never larger than the GPU), so the barrier cannot deadlock, and every wait is bounded: one
// that runs out records kErrWait, raises the block's abort flag and the block leaves through the
// common exit that frees its tensor memory.
//
// The epilogues are those of gemm_tcgen05.cu (float32 sums; gated activation; residual sum with
// the next norm prepared; per-head norm, rotation and cache write of q|k|v), see there for the
// formulas and their places in the reference.
#include "tcgen05_utils.cuh"
#include "timeline.cuh"

namespace tk {

constexpr int kChBM = 128;          // weight rows per tile = UMMA M
constexpr int kChBK = 64;           // k-elements per stage
constexpr int kChIssuers = 1;       // threads that issue tcgen05.mma, one 16-wide k-slice of every stage each
// warp 0: TMA (weights), warp 1: MMA, warps 2..5: epilogue, warp 6: activations, warps 7..: further MMA issuers
constexpr int kChThreads = 224 + 32 * (kChIssuers - 1);
constexpr int kChMaxPhases = 6;
constexpr int kChMaxBN = 64;
constexpr int kChHeadDim = 128;
constexpr unsigned kChPollLimit = 1u << 22;

enum ChainEpilogue : int { kChPlain = 0, kChSwiglu = 1, kChResidualNorm = 2, kChQkvRope = 3 };

struct ChainQkv {
  __nv_bfloat16* q_out;     // [tokens, n_q_heads, 128]
  __nv_bfloat16* k_cache;   // [num_pages, n_kv_heads, page_size, 128]
  __nv_bfloat16* v_cache;
  const int* positions;
  const int* tok_req;
  const int* req_slot;
  const int* block_table;
  const int* req_q_len;     // or null
  const int* req_kv_len;    // or null
  const float* q_norm_w;    // [128] or null
  const float* k_norm_w;
  const float2* rope_table; // [tokens, 64] (cos, sin) or null
  int n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages;
  float eps;
};

struct ChainPhase {
  const __nv_bfloat16* x;           // [tokens, k] activations, row stride ld_x elements
  long long ld_x;
  int rows_total, k_total, n_tiles, kb_total, epilogue;
  void* out;                        // plain: float [tokens, rows]; gated: bf16 [tokens, rows / 2]
  const float* colscale_parts;      // [n_colscale_parts, tokens] or null (see gemm_tcgen05.cu)
  int n_colscale_parts;
  float colscale_inv_dim, colscale_eps;
  float* resid;                     // residual epilogue
  const float* norm_w;
  __nv_bfloat16* xb_out;
  float* sumsq_out;
  ChainQkv qkv;
};

struct ChainParams {
  int n_phases, bn, cols_total, n_stages, max_tiles;
  int* err;
  float* scratch;      // [blocks][2][bn * 128] parts of tiles
  int* counters;       // [kChMaxPhases][max_tiles] arrivals at a tile; zero before and after
  int* sync;           // [kChMaxPhases + 1] arrivals at the barrier after a product, and at the end; zero before and after
  ChainPhase phase[kChMaxPhases];
};

struct ChainMaps {
  CUtensorMap w[kChMaxPhases];
};

// The host makes sure that units x blocks stays below 2^31, so 32-bit arithmetic does.
__device__ __forceinline__ void chain_range(const ChainPhase& ph, int b, int nb, long long& u0, long long& u1) {
  const unsigned total = (unsigned)(ph.n_tiles * ph.kb_total);
  u0 = (long long)(total * (unsigned)b / (unsigned)nb);
  u1 = (long long)(total * (unsigned)(b + 1) / (unsigned)nb);
}

// The block that holds unit u: the largest b with U b / nb <= u.
__device__ __forceinline__ int chain_owner(const ChainPhase& ph, int nb, long long u) {
  const unsigned total = (unsigned)(ph.n_tiles * ph.kb_total);
  return (int)((((unsigned)u + 1u) * (unsigned)nb + total - 1u) / total) - 1;
}

// Walks the k-blocks of one block's share of every product, in order.
struct ChainCursor {
  int ph, tile, kb, kb_total;
  long long left;
  bool range_start;
  __device__ void seek(const ChainParams& p, int b, int nb) {
    while (ph < p.n_phases) {
      long long u0, u1;
      chain_range(p.phase[ph], b, nb, u0, u1);
      if (u1 > u0) {
        kb_total = p.phase[ph].kb_total;
        tile = (int)((unsigned)u0 / (unsigned)kb_total);
        kb = (int)((unsigned)u0 % (unsigned)kb_total);
        left = u1 - u0;
        range_start = true;
        return;
      }
      ++ph;
    }
  }
  __device__ bool done(const ChainParams& p) const { return ph >= p.n_phases; }
  __device__ bool seg_first() const { return range_start || kb == 0; }
  __device__ bool seg_last() const { return left == 1 || kb == kb_total - 1; }
  __device__ void next(const ChainParams& p, int b, int nb) {
    range_start = false;
    if (--left == 0) { ++ph; seek(p, b, nb); return; }
    if (++kb == kb_total) { kb = 0; ++tile; }
  }
};

__device__ __forceinline__ int ld_acquire_gpu(const int* ptr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* ptr, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;\n" ::"l"(ptr), "r"(v) : "memory");
}
// Orders accesses through the generic proxy (plain loads and stores) with those of the
// asynchronous proxy (TMA) to global memory.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;\n" ::: "memory");
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }
// Barrier of the 128 epilogue threads that also tells every one of them whether all of them
// passed `ok`: decisions to leave a loop are taken by all threads alike, or not at all.
__device__ __forceinline__ bool epi_all(bool ok) {
  uint32_t all;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n bar.red.and.pred q, 1, 128, p;\n selp.u32 %0, 1, 0, q;\n}\n"
      : "=r"(all) : "r"((uint32_t)(ok ? 1 : 0)) : "memory");
  return all != 0;
}

// Waits until every block has arrived at the barrier after product `ph`; false if the wait ran out.
__device__ __forceinline__ bool chain_wait_phase(const ChainParams& p, int ph, int nb, volatile int* abort_flag) {
  for (unsigned spin = 0; spin < kChPollLimit; ++spin) {
    if (ld_acquire_gpu(p.sync + ph) >= nb) return true;
    if (*abort_flag) return false;
    __nanosleep(40);
  }
  return false;
}

// Adds up the parts of tile `tile` in the order of the blocks that hold them and leaves the sums in
// `staging`.  Thread `et` of 128 owns NF4 float4 of the [column][row] tile; the parts of G blocks
// are requested together, so that their trips to the second-level cache overlap.
template <int NF4, int G>
__device__ __forceinline__ void chain_merge(float* staging, const float* scratch, size_t part_floats,
                                            const ChainPhase& P, int nb, int tile, int b_first, int b_last, int et) {
  float4 acc[NF4];
#pragma unroll
  for (int j = 0; j < NF4; ++j) acc[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  int cb = b_first;
  while (cb <= b_last) {
    const float4* src[G];
    int n = 0;
    while (n < G && cb <= b_last) {
      long long c0, c1;
      chain_range(P, cb, nb, c0, c1);
      if (c1 > c0) {
        const int cslot = ((int)((unsigned)c0 / (unsigned)P.kb_total) == tile) ? 0 : 1;
        src[n++] = reinterpret_cast<const float4*>(scratch + ((size_t)cb * 2 + cslot) * part_floats);
      }
      ++cb;
    }
    float4 x[G][NF4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (g < n) {
#pragma unroll
        for (int j = 0; j < NF4; ++j) x[g][j] = __ldcg(src[g] + et + 128 * j);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (g < n) {
#pragma unroll
        for (int j = 0; j < NF4; ++j) {
          acc[j].x += x[g][j].x; acc[j].y += x[g][j].y; acc[j].z += x[g][j].z; acc[j].w += x[g][j].w;
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NF4; ++j) reinterpret_cast<float4*>(staging)[et + 128 * j] = acc[j];
}

__global__ void __launch_bounds__(kChThreads, 1)
gemm_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t raw = gt_smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, nb = gridDim.x;
  const uint32_t r_bytes = kChBM * kChBK * 2;
  const uint32_t c_bytes = (uint32_t)p.bn * kChBK * 2;
  const uint32_t stage_bytes = r_bytes + ((c_bytes + 1023u) & ~1023u);
  const int S = p.n_stages;

  float* staging = reinterpret_cast<float*>(smem + (size_t)S * stage_bytes);         // [bn][128]
  float* s_scale = staging + p.bn * kChBM;                                          // [64]
  long long* s_cache_row = reinterpret_cast<long long*>(s_scale + kChMaxBN);        // [64]
  int* s_zero_rows = reinterpret_cast<int*>(s_cache_row + kChMaxBN);                // [64]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_zero_rows + kChMaxBN);
  uint64_t* empty_bar = full_bar + S;
  uint64_t* acc_full = empty_bar + S;       // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_last = abort_flag + 1;

  // A product of 16 to 64 columns does not fill the tensor pipe: products that add into the same
  // accumulator wait for one another, and one block per SM has no other block's products to
  // interleave with.  So the four 16-wide k-slices of a stage add into four accumulators of their
  // own, which the epilogue adds up (always as (0 + 1) + (2 + 3)); with two such sets, one being
  // drained while the other is filled, a block holds eight accumulators.
  const uint32_t acc_cols = p.bn < 32 ? 32u : (uint32_t)p.bn;      // columns of one accumulator
  const uint32_t tmem_cols = 8u * acc_cols;                        // 256 or 512: a power of two

  pdl_trigger();
  if (threadIdx.x < p.n_phases) {
    // the descriptors of all weights are brought in before the first load needs one
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&maps.w[threadIdx.x]) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      // a stage is full when the weights' bytes have landed (one arrival with the byte count)
      // and every lane of the activation warp has seen its copies complete
      mbar_init(gt_smem_u32(&full_bar[s]), 1 + 32);
      mbar_init(gt_smem_u32(&empty_bar[s]), kChIssuers);      // every issuer's products have read the stage
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(gt_smem_u32(&acc_full[a]), kChIssuers);
      mbar_init(gt_smem_u32(&acc_empty[a]), 4);      // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(gt_smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer: the weights of all products, as far ahead as the ring allows -------------
    // (Requesting the weights beyond the ring into the second-level cache while the ring is full
    // was measured and dropped: the burst delays the few loads and atomics by which the blocks
    // add up their parts and meet at the barrier, which are what the pause consists of.)
    if (lane == 0) {
      tl_mark(20, 0);
      ChainCursor wc;
      wc.ph = 0; wc.seek(p, b, nb);
      int w_s = 0;
      uint32_t w_round = 0;
      while (!wc.done(p)) {
        if (w_round > 0 && !mbar_wait(gt_smem_u32(&empty_bar[w_s]), (w_round - 1) & 1u, abort_flag)) {
          if (!*abort_flag) { set_error(p.err, kErrWait, 30, wc.ph, w_s); *abort_flag = 1; }
          break;
        }
        const uint32_t full = gt_smem_u32(&full_bar[w_s]);
        mbar_expect_tx(full, r_bytes);
        tma_load_2d(base + (uint32_t)w_s * stage_bytes, &maps.w[wc.ph], wc.kb * kChBK, wc.tile * kChBM, full);
        wc.next(p, b, nb);
        if (++w_s == S) { w_s = 0; ++w_round; }
      }
    }
  } else if (warp == 1 || warp >= 7) {
    // ---- MMA issuers ---------------------------------------------------------------------------------
    // A tcgen05.mma of 16 to 64 columns costs its issuing thread about 0.1 us whatever its size, and
    // the products of one thread run one after the other: four a stage from one thread is less than
    // the stream of weights needs.  So four threads (in four warps) issue one 16-wide k-slice of
    // every stage each, into an accumulator of their own; the epilogue adds the four up.
    const int issuer = warp == 1 ? 0 : warp - 6;
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(p.bn);
      ChainCursor c;
      c.ph = 0; c.seek(p, b, nb);
      int it = 0, s = 0;
      uint32_t round = 0;
      int seg = 0;
      bool ok = true;
#ifdef TK_TIMELINE
      unsigned long long t_wait = 0, t_begin = tl_now(), t_fence = 0, t_mma = 0, t_commit = 0;
#endif
      while (!c.done(p) && ok) {
        const int a = seg & 1;
        const bool first = c.seg_first();
        if (first && seg >= 2) {
          if (!mbar_wait(gt_smem_u32(&acc_empty[a]), (uint32_t)((seg >> 1) - 1) & 1u, abort_flag)) {
            set_error(p.err, kErrWait, 31, seg, a); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
        }
#ifdef TK_TIMELINE
        const unsigned long long t0 = tl_now();
#endif
        if (!mbar_wait(gt_smem_u32(&full_bar[s]), round & 1u, abort_flag)) {
          set_error(p.err, kErrWait, 32, it, s); *abort_flag = 1; ok = false; break;
        }
#ifdef TK_TIMELINE
        const unsigned long long t1 = tl_now();
        t_wait += t1 - t0;
#endif
        fence_async_shared();     // the activations were written by cp.async: the tensor core reads them through the other proxy
        tc_fence_after();
#ifdef TK_TIMELINE
        const unsigned long long t2 = tl_now();
        t_fence += t2 - t1;
#endif
        const uint32_t a_addr = base + (uint32_t)s * stage_bytes;
        const uint64_t desc_a = umma_desc_sw128(a_addr);
        const uint64_t desc_b = umma_desc_sw128(a_addr + r_bytes);
        const uint32_t d_addr = tmem_base + (uint32_t)(4 * a) * acc_cols;
#pragma unroll
        for (int k = issuer; k < kChBK / 16; k += kChIssuers) {
          umma_bf16(d_addr + (uint32_t)k * acc_cols, desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k), idesc,
                    first ? 0u : 1u);
        }
#ifdef TK_TIMELINE
        const unsigned long long t3 = tl_now();
        t_mma += t3 - t2;
#endif
        umma_commit(gt_smem_u32(&empty_bar[s]));
#ifdef TK_TIMELINE
        t_commit += tl_now() - t3;
#endif
        if (it == 0 && issuer == 0) tl_mark(20, 30);
        if (c.seg_last()) {
          umma_commit(gt_smem_u32(&acc_full[a]));
          ++seg;
        }
        if (c.left == 1 && issuer == 0) {
          tl_mark(20, 31 + c.ph);
#ifdef TK_TIMELINE
          tl_value(21, c.ph, (unsigned)t_wait);
          tl_value(22, c.ph, (unsigned)(tl_now() - t_begin));
          tl_value(23, c.ph, (unsigned)t_fence);
          tl_value(24, c.ph, (unsigned)t_mma);
          tl_value(25, c.ph, (unsigned)t_commit);
          t_wait = 0; t_begin = tl_now(); t_fence = 0; t_mma = 0; t_commit = 0;
#endif
        }
        c.next(p, b, nb);
        ++it;
        if (++s == S) { s = 0; ++round; }
      }
    }
  } else if (warp == 6) {
    // ---- activations: rows of X for every stage, copied with cp.async ------------------------------
    // rows that no token fills are zero in every stage, once and for all
    for (int st = 0; st < S; ++st) {
      uint4* xr = reinterpret_cast<uint4*>(smem + (size_t)st * stage_bytes + r_bytes);
      for (int i = lane; i < (int)(c_bytes / 16); i += 32) xr[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_async_shared();
    __syncwarp();
    ChainCursor c;
    c.ph = 0; c.seek(p, b, nb);
    int st = 0;
    uint32_t round = 0;
    int ready = 0;                  // the activations of products below `ready` exist
    bool ok = true;
    while (!c.done(p) && ok) {
      if (c.ph >= ready) {
        if (ready == 0) { pdl_wait(); if (lane == 0) tl_mark(20, 1); ready = 1; }
        if (c.ph >= ready) {
          int passed = 1;
          if (lane == 0) passed = chain_wait_phase(p, c.ph - 1, nb, abort_flag) ? 1 : 0;
          passed = __shfl_sync(0xffffffffu, passed, 0);
          if (!passed) {
            if (lane == 0 && !*abort_flag) { set_error(p.err, kErrWait, 35, c.ph, 0); *abort_flag = 1; }
            ok = false;
            break;
          }
          (void)ld_acquire_gpu(p.sync + c.ph - 1);     // every lane orders its own reads behind the barrier
          ready = c.ph + 1;
        }
      }
      if (round > 0) {
        ok = mbar_wait(gt_smem_u32(&empty_bar[st]), (round - 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0 && !*abort_flag) { set_error(p.err, kErrWait, 36, c.ph, st); *abort_flag = 1; }
          break;
        }
      }
      const ChainPhase& P = p.phase[c.ph];
      const uint32_t xdst = base + (uint32_t)st * stage_bytes + r_bytes;
      const int k0 = c.kb * kChBK;
      for (int idx = lane; idx < p.cols_total * 8; idx += 32) {
        const int row = idx >> 3, ch = idx & 7;
        const __nv_bfloat16* src = P.x + (size_t)row * P.ld_x + k0 + ch * 8;
        const uint32_t bytes = (k0 + ch * 8 < P.k_total) ? 16u : 0u;     // beyond k: zeros
        const uint32_t dst = xdst + (uint32_t)row * 128u + (uint32_t)((ch ^ (row & 7)) << 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(bytes ? src : P.x), "r"(bytes)
                     : "memory");
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(gt_smem_u32(&full_bar[st])) : "memory");
      c.next(p, b, nb);
      if (++st == S) { st = 0; ++round; }
    }
    if (ready == 0) pdl_wait();     // a block without work still orders itself behind the kernel before
    asm volatile("cp.async.wait_all;\n" ::: "memory");
  } else {
    // ---- epilogue: warps 2..5; warp w reads the accumulator lanes 32 (w mod 4) .. ---------------------
    const int quarter = warp & 3;
    const int et = (warp - 2) * 32 + lane;           // 0..127 within the epilogue group
    const int trow = quarter * 32 + lane;            // the tile row (accumulator lane) this thread drains
    bool ok = true;
    int seg = 0;
    pdl_wait();   // nothing is stored before the kernels before this one are done with the buffers
    for (int ph = 0; ph < p.n_phases && ok; ++ph) {
      const ChainPhase& P = p.phase[ph];
      if (ph > 0) {
        // the product before this one is complete everywhere: its outputs may be read, and what
        // it read may be overwritten
        if (et == 0) {
          if (!chain_wait_phase(p, ph - 1, nb, abort_flag)) {
            if (!*abort_flag) { set_error(p.err, kErrWait, 33, ph, 0); *abort_flag = 1; }
          }
        }
        if (!epi_all(*abort_flag == 0)) { ok = false; break; }
        (void)ld_acquire_gpu(p.sync + ph - 1);       // every thread orders its own reads behind the barrier
        if (et == 0) tl_mark(20, 50 + ph);
      }
      // what the epilogue needs per column (token): the owed norm scale, the token's cache row
      if (et < p.bn) {
        const int col = et;
        float scale = 1.0f;
        long long cache_row = -1;
        int zero_rows = 0;
        if (col < p.cols_total) {
          if (P.colscale_parts != nullptr) {
            float ss = 0.0f;
#pragma unroll 16
            for (int i = 0; i < P.n_colscale_parts; ++i) ss += __ldcg(P.colscale_parts + (size_t)i * p.cols_total + col);
            scale = rsqrtf(ss * P.colscale_inv_dim + P.colscale_eps);
          }
          if (P.epilogue == kChQkvRope) {
            const ChainQkv& e = P.qkv;
            const int pos = e.positions[col];
            const int r = e.tok_req[col];
            if (pos < 0) {
              set_error(p.err, kErrPosition, col, pos, 0);
            } else if (r < 0 || r >= e.n_reqs) {
              set_error(p.err, kErrRequest, col, r, e.n_reqs);
            } else {
              const int pidx = pos / e.page_size;
              const int page = (pidx < e.max_pages) ? e.block_table[(size_t)e.req_slot[r] * e.max_pages + pidx] : -1;
              if (page < 0 || page >= e.num_pages) {
                set_error(p.err, kErrPage, col, pidx, page);
              } else {
                cache_row = (long long)page * e.n_kv_heads * e.page_size + (pos % e.page_size);
                if (e.req_kv_len != nullptr) {
                  const int kv_len = e.req_kv_len[r], q_len = e.req_q_len[r];
                  if (pos == kv_len - 1 && pos - pos % e.page_size >= kv_len - q_len) {
                    zero_rows = e.page_size - 1 - pos % e.page_size;
                  }
                }
              }
            }
          }
        }
        s_scale[col] = scale;
        s_cache_row[col] = cache_row;
        s_zero_rows[col] = zero_rows;
      }
      epi_bar();

      long long u0, u1;
      chain_range(P, b, nb, u0, u1);
      long long u = u0;
      while (u < u1 && ok) {
        const int tile = (int)((unsigned)u / (unsigned)P.kb_total);
        const int kb0 = (int)((unsigned)u % (unsigned)P.kb_total);
        const long long room = (long long)P.kb_total - kb0;
        const int kb1 = kb0 + (int)((u1 - u) < room ? (u1 - u) : room);
        const bool whole = (kb0 == 0 && kb1 == P.kb_total);
        const int slot = (u == u0) ? 0 : 1;
        const int a = seg & 1;
        ok = mbar_wait(gt_smem_u32(&acc_full[a]), (uint32_t)(seg >> 1) & 1u, abort_flag);
        if (!ok && lane == 0 && !*abort_flag) { set_error(p.err, kErrWait, 34, seg, a); *abort_flag = 1; }
        ok = epi_all(ok);
        if (!ok) break;
        tc_fence_after();
        float* part = p.scratch + ((size_t)b * 2 + slot) * ((size_t)p.bn * kChBM);
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t v0[16], v1[16], v2[16], v3[16];
          const uint32_t at = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(4 * a) * acc_cols + (uint32_t)c0;
          tmem_ld16(at, v0);
          tmem_ld16(at + acc_cols, v1);
          tmem_ld16(at + 2u * acc_cols, v2);
          tmem_ld16(at + 3u * acc_cols, v3);
          tmem_wait_ld();
          float* dst = whole ? staging : part;
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            dst[(c0 + e) * kChBM + trow] = (__uint_as_float(v0[e]) + __uint_as_float(v1[e])) +
                                           (__uint_as_float(v2[e]) + __uint_as_float(v3[e]));
          }
        }
        // the accumulator may be filled again
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(gt_smem_u32(&acc_empty[a]));
        if (et == 0 && u + (kb1 - kb0) >= u1) tl_mark(20, 60 + ph);      // the last segment of the product is drained
        ++seg;
        u += kb1 - kb0;

        bool merge = whole;
        if (!whole) {
          // count this part; whoever arrives last at the tile adds the parts up
          __threadfence();
          epi_bar();
          const int b_first = chain_owner(P, nb, (long long)tile * P.kb_total);
          const int b_last = chain_owner(P, nb, (long long)(tile + 1) * P.kb_total - 1);
          if (et == 0) {
            int n_contrib = b_last - b_first + 1;        // every block in between holds a part, unless
            if (P.n_tiles * P.kb_total < nb) {           // there are fewer units than blocks
              n_contrib = 0;
              for (int c = b_first; c <= b_last; ++c) {
                long long c0, c1;
                chain_range(P, c, nb, c0, c1);
                n_contrib += (c1 > c0) ? 1 : 0;
              }
            }
            int* counter = p.counters + (size_t)ph * p.max_tiles + tile;
            const int arrived = atomicAdd(counter, 1);
            const int last = (arrived == n_contrib - 1);
            if (last) *counter = 0;
            *s_last = last;
          }
          epi_bar();
          merge = (*s_last != 0);
          if (merge) {
            __threadfence();
            const size_t part_floats = (size_t)p.bn * kChBM;
            if (p.bn == 16) chain_merge<4, 4>(staging, p.scratch, part_floats, P, nb, tile, b_first, b_last, et);
            else if (p.bn == 32) chain_merge<8, 2>(staging, p.scratch, part_floats, P, nb, tile, b_first, b_last, et);
            else chain_merge<16, 1>(staging, p.scratch, part_floats, P, nb, tile, b_first, b_last, et);
          }
        }
        epi_bar();                      // the tile's sums are complete in `staging`
        if (merge) {
          if (P.epilogue == kChSwiglu) {
            const int j4 = (et & 15) * 4, cphase = et >> 4;
            const int inter = P.rows_total >> 1;
            const int oc = tile * 64 + j4;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(P.out);
            if (oc < inter) {
              for (int c = cphase; c < p.bn; c += 8) {
                if (c >= p.cols_total) break;
                float4 g = *reinterpret_cast<const float4*>(staging + c * kChBM + j4);
                float4 uu = *reinterpret_cast<const float4*>(staging + c * kChBM + 64 + j4);
                const float sc = s_scale[c];
                g.x *= sc; g.y *= sc; g.z *= sc; g.w *= sc;
                uu.x *= sc; uu.y *= sc; uu.z *= sc; uu.w *= sc;
                uint2 packed;
                *reinterpret_cast<__nv_bfloat162*>(&packed.x) =
                    __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * uu.x, g.y / (1.0f + expf(-g.y)) * uu.y);
                *reinterpret_cast<__nv_bfloat162*>(&packed.y) =
                    __floats2bfloat162_rn(g.z / (1.0f + expf(-g.z)) * uu.z, g.w / (1.0f + expf(-g.w)) * uu.w);
                *reinterpret_cast<uint2*>(out + (size_t)c * inter + oc) = packed;
              }
            }
          } else {
            // a warp takes one column (token) at a time, its lanes four neighbouring rows each
            const int r4 = (et & 31) * 4, cphase = et >> 5;
            const int row = tile * kChBM + r4;
            if (row < P.rows_total) {
              for (int c = cphase; c < p.bn; c += 4) {
                if (c >= p.cols_total) break;
                float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f), w = r;
                if (P.epilogue == kChResidualNorm) {
                  r = *reinterpret_cast<const float4*>(P.resid + (size_t)c * P.rows_total + row);
                  w = *reinterpret_cast<const float4*>(P.norm_w + row);
                }
                float4 sum = *reinterpret_cast<const float4*>(staging + c * kChBM + r4);
                const float sc = s_scale[c];
                sum.x *= sc; sum.y *= sc; sum.z *= sc; sum.w *= sc;
                if (P.epilogue == kChQkvRope) {
                  // this warp holds head `tile` of token c: lane l the elements 4 l .. 4 l + 3
                  const ChainQkv& e = P.qkv;
                  const int kind = tile < e.n_q_heads ? 0 : (tile < e.n_q_heads + e.n_kv_heads ? 1 : 2);
                  const float* nw = kind == 0 ? e.q_norm_w : (kind == 1 ? e.k_norm_w : nullptr);
                  if (nw != nullptr) {
                    const float4 w4 = *reinterpret_cast<const float4*>(nw + r4);
                    const float ss = warp_sum(sum.x * sum.x + sum.y * sum.y + sum.z * sum.z + sum.w * sum.w);
                    const float rstd = rsqrtf(ss / (float)kChHeadDim + e.eps);
                    sum.x = sum.x * rstd * w4.x; sum.y = sum.y * rstd * w4.y;
                    sum.z = sum.z * rstd * w4.z; sum.w = sum.w * rstd * w4.w;
                  }
                  if (kind != 2 && e.rope_table != nullptr) {
                    // element i < 64 turns with element i + 64, which lane l ^ 16 holds
                    const float4* cs = reinterpret_cast<const float4*>(e.rope_table + (size_t)c * (kChHeadDim / 2) +
                                                                        4 * (lane & 15));
                    const float4 cs01 = cs[0], cs23 = cs[1];
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
                    *reinterpret_cast<uint2*>(e.q_out + ((size_t)c * e.n_q_heads + tile) * kChHeadDim + r4) = packed;
                  } else {
                    const long long cache_row = s_cache_row[c];
                    const int zero_rows = s_zero_rows[c];
                    if (cache_row >= 0) {
                      const int head = tile - e.n_q_heads - (kind == 2 ? e.n_kv_heads : 0);
                      __nv_bfloat16* dst = (kind == 1 ? e.k_cache : e.v_cache) +
                                           ((size_t)cache_row + (size_t)head * e.page_size) * kChHeadDim + r4;
                      *reinterpret_cast<uint2*>(dst) = packed;
                      for (int z = 1; z <= zero_rows; ++z) {
                        *reinterpret_cast<uint2*>(dst + (size_t)z * kChHeadDim) = make_uint2(0u, 0u);
                      }
                    }
                  }
                  continue;
                }
                if (P.epilogue == kChResidualNorm) {
                  r.x += sum.x; r.y += sum.y; r.z += sum.z; r.w += sum.w;
                  *reinterpret_cast<float4*>(P.resid + (size_t)c * P.rows_total + row) = r;
                  uint2 packed;
                  *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(r.x * w.x, r.y * w.y);
                  *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(r.z * w.z, r.w * w.w);
                  *reinterpret_cast<uint2*>(P.xb_out + (size_t)c * P.rows_total + row) = packed;
                  const float ss = warp_sum(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w);
                  if (lane == 0) P.sumsq_out[(size_t)tile * p.cols_total + c] = ss;
                  continue;
                }
                float* dst = reinterpret_cast<float*>(P.out) + (size_t)c * P.rows_total + row;
                if ((P.rows_total & 3) == 0 && row + 3 < P.rows_total) {
                  *reinterpret_cast<float4*>(dst) = sum;
                } else {
                  dst[0] = sum.x;
                  if (row + 1 < P.rows_total) dst[1] = sum.y;
                  if (row + 2 < P.rows_total) dst[2] = sum.z;
                  if (row + 3 < P.rows_total) dst[3] = sum.w;
                }
              }
            }
          }
        }
        epi_bar();                      // `staging` may be written again
      }
      // this block has finished product `ph`: its stores become visible, then it is counted
      if (et == 0) tl_mark(20, 70 + ph);
      __threadfence();
      fence_proxy_async_global();
      epi_bar();
      if (et == 0) {
        red_release_gpu_add(p.sync + ph, 1);
        tl_mark(20, 10 + ph);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(tmem_cols)
                 : "memory");
  }
  if (threadIdx.x == 0) {
    // the last block to leave puts the barrier counters back to zero: nobody polls them any more
    // (a block that aborted may have left some barrier short; then the error word says so and
    // the host clears the counters before the next launch)
    const int gone = atomicAdd(p.sync + kChMaxPhases, 1);
    if (gone == nb - 1) {
      for (int i = 0; i <= kChMaxPhases; ++i) p.sync[i] = 0;
      __threadfence();
    }
    tl_mark(20, 4);
  }
}

// ---- host side ------------------------------------------------------------------------------------

static int chain_make_map(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kChBK, (cuuint32_t)box_rows};
  return make_bf16_map(map, ptr, 2, dims, strides, box);
}

static int chain_blocks() {
  static int blocks = 0;
  if (blocks == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    blocks = sms;
  }
  return blocks;
}

}  // namespace tk

// One product of a chain, as the host describes it (plain C, filled by the caller).
struct TkChainPhaseArgs {
  const void* w;            // [rows, k] bf16, row stride ld_w
  const void* x;            // [tokens, k] bf16, row stride ld_x
  long long ld_w, ld_x;
  int rows, k, epilogue;    // epilogue as in tk_gemm_bf16_tcgen05, 3 = q|k|v (tk_gemm_qkv_rope)
  int n_colscale_parts;
  void* out;
  const float* colscale_parts;
  float colscale_inv_dim, colscale_eps;
  float* resid;
  const float* norm_w;
  void* xb_out;
  float* sumsq_out;
  void* q_out; void* k_cache; void* v_cache;
  const int* positions; const int* tok_req; const int* req_slot; const int* block_table;
  const int* req_q_len; const int* req_kv_len;
  const float* q_norm_w; const float* k_norm_w;
  const void* rope_table;
  int n_reqs, n_q_heads, n_kv_heads, page_size, max_pages, num_pages;
  float eps;
  int reserved;
};

TK_TIMELINE_SETTER(gemm_chain)

// Blocks of the chain kernel on the current device (one per SM) and what a launch needs beside
// its operands: scratch floats for the parts of tiles, and the number of int counters (tile
// arrivals for kChMaxPhases products of up to max_tiles tiles, then the barrier counters), which
// must be zero before the first launch; every launch leaves them at zero.
TK_API int tk_gemm_chain_blocks(void) { return tk::chain_blocks(); }
TK_API long long tk_gemm_chain_scratch_floats(int tokens) {
  int bn = 16;
  while (bn < tokens) bn *= 2;
  return (long long)tk::chain_blocks() * 2 * bn * tk::kChBM;
}
TK_API long long tk_gemm_chain_counter_ints(int max_tiles) {
  return (long long)tk::kChMaxPhases * max_tiles + tk::kChMaxPhases + 1;
}
TK_API int tk_gemm_chain_max_phases(void) { return tk::kChMaxPhases; }

// Runs the products phases[0 .. n_phases) as one kernel; the activations of every product after the
// first may be outputs of the products before it.  tokens <= 64.  counters is the int buffer of
// tk_gemm_chain_counter_ints(max_tiles).
TK_API int tk_gemm_chain(const TkChainPhaseArgs* phases, int n_phases, int tokens, int* err, float* scratch,
                         int* counters, int max_tiles, cudaStream_t stream) {
  using namespace tk;
  if (n_phases < 1 || n_phases > kChMaxPhases || tokens < 1 || tokens > kChMaxBN) return (int)cudaErrorInvalidValue;
  const int nb = chain_blocks();
  if (nb < 1) return (int)cudaErrorInvalidDevice;
  int bn = 16;
  while (bn < tokens) bn *= 2;
  ChainMaps maps;
  ChainParams p = {};
  p.n_phases = n_phases; p.bn = bn; p.cols_total = tokens; p.max_tiles = max_tiles;
  p.err = err; p.scratch = scratch; p.counters = counters; p.sync = counters + (size_t)kChMaxPhases * max_tiles;
  for (int i = 0; i < n_phases; ++i) {
    const TkChainPhaseArgs& a = phases[i];
    ChainPhase& ph = p.phase[i];
    if (a.rows <= 0 || a.k <= 0 || a.k % 8 != 0 || a.epilogue < kChPlain || a.epilogue > kChQkvRope) {
      return (int)cudaErrorInvalidValue;
    }
    if (((uintptr_t)a.x & 15u) != 0 || (a.ld_x * 2) % 16 != 0) return (int)cudaErrorInvalidValue;
    ph.x = (const __nv_bfloat16*)a.x; ph.ld_x = a.ld_x;
    ph.rows_total = a.rows; ph.k_total = a.k; ph.epilogue = a.epilogue;
    ph.n_tiles = (a.rows + kChBM - 1) / kChBM;
    ph.kb_total = (a.k + kChBK - 1) / kChBK;
    if (ph.n_tiles > max_tiles) return (int)cudaErrorInvalidValue;
    if ((long long)ph.n_tiles * ph.kb_total * (nb + 1) >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    if (a.epilogue != kChPlain && a.rows % kChBM != 0) return (int)cudaErrorInvalidValue;
    if (a.epilogue == kChResidualNorm &&
        (a.resid == nullptr || a.norm_w == nullptr || a.xb_out == nullptr || a.sumsq_out == nullptr)) {
      return (int)cudaErrorInvalidValue;
    }
    if ((a.epilogue == kChPlain || a.epilogue == kChSwiglu) && a.out == nullptr) return (int)cudaErrorInvalidValue;
    if (a.colscale_parts != nullptr && a.n_colscale_parts < 1) return (int)cudaErrorInvalidValue;
    ph.out = a.out;
    ph.colscale_parts = a.colscale_parts; ph.n_colscale_parts = a.n_colscale_parts;
    ph.colscale_inv_dim = a.colscale_inv_dim; ph.colscale_eps = a.colscale_eps;
    ph.resid = a.resid; ph.norm_w = a.norm_w; ph.xb_out = (__nv_bfloat16*)a.xb_out; ph.sumsq_out = a.sumsq_out;
    if (a.epilogue == kChQkvRope) {
      if (a.n_q_heads < 1 || a.n_kv_heads < 1 || a.page_size < 1 ||
          a.rows != (a.n_q_heads + 2 * a.n_kv_heads) * kChHeadDim || (a.req_kv_len != nullptr && a.req_q_len == nullptr)) {
        return (int)cudaErrorInvalidValue;
      }
      ChainQkv& e = ph.qkv;
      e.q_out = (__nv_bfloat16*)a.q_out; e.k_cache = (__nv_bfloat16*)a.k_cache; e.v_cache = (__nv_bfloat16*)a.v_cache;
      e.positions = a.positions; e.tok_req = a.tok_req; e.req_slot = a.req_slot; e.block_table = a.block_table;
      e.req_q_len = a.req_q_len; e.req_kv_len = a.req_kv_len; e.q_norm_w = a.q_norm_w; e.k_norm_w = a.k_norm_w;
      e.rope_table = (const float2*)a.rope_table;
      e.n_reqs = a.n_reqs; e.n_q_heads = a.n_q_heads; e.n_kv_heads = a.n_kv_heads; e.page_size = a.page_size;
      e.max_pages = a.max_pages; e.num_pages = a.num_pages; e.eps = a.eps;
    }
    int rc = chain_make_map(&maps.w[i], a.w, a.rows, a.k, a.ld_w, kChBM);
    if (rc != 0) return rc;
  }
  for (int i = n_phases; i < kChMaxPhases; ++i) maps.w[i] = maps.w[0];

  const unsigned r_bytes = kChBM * kChBK * 2;
  const unsigned c_bytes = ((unsigned)bn * kChBK * 2 + 1023u) & ~1023u;
  const unsigned stage_bytes = r_bytes + c_bytes;
  const size_t fixed = (size_t)bn * kChBM * 4 + kChMaxBN * 16 + 1024 /* alignment slack */ + 512 /* barriers */;
  const size_t limit = 227 * 1024;
  int n_stages = (int)((limit - fixed) / stage_bytes);
  if (n_stages > 12) n_stages = 12;
  if (n_stages < 2) return (int)cudaErrorInvalidValue;
  p.n_stages = n_stages;
  const size_t smem_bytes = (size_t)n_stages * stage_bytes + fixed;

  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_chain_kernel, kChThreads, limit);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;   // the blocks could not all be resident
    configured = true;
  }
  return (int)launch(gemm_chain_kernel, dim3(nb), dim3(kChThreads), smem_bytes, stream, maps, p);
}
