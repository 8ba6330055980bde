// Paged flash attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head_dim 64 or 128): a persistent kernel, one block per SM.
//
// Work is a list of items made by the host: (256 query tokens of one request, a range of
// 64-key tiles) for every query head.  The 256 tokens are two query tiles of 128 rows that share
// every key and value tile.  Items are listed longest first and dealt out by an atomic counter, so
// the SMs end together.  Where the list would leave SMs idle (one short portion against a long
// context) the host cuts the keys of a block of tokens into parts: each part leaves its
// unnormalised output, maximum and sum in scratch memory, and the part listed last adds them up.
//
//   warp 0       asks for the next item shortly before the current one is loaded, publishes its
//                geometry in shared memory, and loads with TMA (cp.async.bulk.tensor, 128-byte
//                swizzle, every block for itself): the query tiles into the buffers of the item's
//                parity (two sets, so the next item's queries arrive while this one runs), then
//                key tiles and value tiles, page by page, into two rings that run on across items
//                (a key tile is given back once its S is computed, a value tile after the second
//                product, so keys are requested a step earlier than values); every lane looks one
//                page up and issues one copy;
//   warps 1, 10  one thread each issues tcgen05.mma for one query tile: S = Q K^T (M 128, N 64)
//                into one of the tile's two score buffers in tensor memory, and O += P V
//                (M 128, N head_dim) with P read from tensor memory and V straight from its page
//                layout as an MN-major operand.  It is an event loop: S of the next key tile goes
//                out when its keys are there, the second product of the oldest pending key tile
//                when its probabilities are, across the end of an item too;
//   warps 2..5   softmax of query tile 0, warps 6..9 of query tile 1: thread i owns query row
//                i = tensor-memory lane i.  It reads its 64 scores with tcgen05.ld, masks
//                (causal with offset kv_len - q_len, window), keeps a reference maximum and
//                the normaliser in float32, writes the probabilities as bfloat16 pairs over the
//                scores they came from (tcgen05.st), where the second product takes them as its
//                A operand, and rescales the output accumulator in tensor memory only when the
//                row maximum has grown by more than 2^8 since the reference was set (the
//                probabilities stay below 2^8, exact enough in bfloat16; the result is the same
//                softmax).  At the end of an item it writes its rows out (or its part) and goes
//                on to the next item, whose first scores are waiting by then.
// Every query tile has two score buffers, so the tensor cores work for one tile, or on the next
// key tile, while the other tile's softmax runs; a buffer is written again only by a product that
// the same thread issues after the one that read the probabilities in it, and the tensor cores
// run a thread's products in order.  Two softmax warps share every scheduler.
//
// Pages are loaded whole.  A page that lies outside the item's visible keys is replaced by the
// page of its last visible key (its probabilities are exactly zero), and the kernel that writes
// the cache zero-fills the unwritten rest of a request's last page, so no stale value can turn
// a zero probability into a NaN.  Every wait is bounded and reports kErrWait; a block that gave
// up still leaves its loops, frees its tensor memory and counts itself out.
#include "tcgen05_utils.cuh"
#include "timeline.cuh"

namespace tk {

constexpr int kAtBM = 128;            // rows of one query tile
constexpr int kAtQT = 2;              // query tiles per item
constexpr int kAtBN = 64;             // keys per tile
constexpr int kAtStages = 3;          // stages of one key tile and its value tile
constexpr int kAtRec = 12;            // ints of an item record
constexpr int kAtThreads = 64 + kAtQT * 128 + 32;   // TMA, MMA of tile 0, softmax warps, MMA of tile 1
constexpr int kAtMmaWarp1 = 2 + kAtQT * 4;           // the warp that issues for query tile 1
constexpr int kAtMaxParts = 64;
constexpr float kAtRescale = 8.0f;    // log2 units

// An item record, as the host writes it (all int32):
//   0 tok0      first of the 256 tokens in q and out
//   1 rows      how many of the 256 exist
//   2 pos0      position of the first one in its request (kv_len - q_len + its index)
//   3 slot      the request's row of the block table
//   4 kt_begin  first 64-key tile of this part
//   5 kt_end    one past its last
//   6 part      index of the part
//   7 n_parts   parts that the tokens' keys were cut into (1: the rows are written out directly)
//   8 poff      parts of all cut token blocks listed before this one (scratch index)
//   9 split     index of this token block among the cut ones (counter index)
//  10 merger    1 for the part of a cut token block that is listed last: it adds the parts up
struct AttnTcParams {
  __nv_bfloat16* out;            // [n_tokens, n_q_heads, D]
  const int* records;            // [n_records, kAtRec], longest first
  const int* block_table;
  int* err;
  int* sched;                    // [2] zero between launches: next item, blocks done
  float* part_o;                 // [((poff + part) * n_q_heads + head) * 2 + tile][D / 4][128 rows] float4: unnormalised outputs
  float* part_ml;                // the same index: [2][128 rows] reference maximum (log2 units), then sum
  int* part_count;               // [(split * n_q_heads + head) * 2 + tile] zero between launches
  int n_records, n_q_heads, n_kv_heads, page_size, max_pages, num_pages, window;
  float scale_log2;
};

struct AttnItem {        // what a block's roles need of an item
  int tok0, rows, pos0, slot, kt_begin, kt_end, part, n_parts, poff, split, merger, head, valid, index;
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

// In builds with time stamps the softmax threads also sum, in registers, the clocks they spend in
// each part of a key tile; block 0's first row of each query tile reports the sums per item
// (kernel 32, phase = part, value = clocks; phase 8 = key tiles).  TL_AFTER(x) keeps the clock
// read behind the computation of x.
#ifdef TK_TIMELINE
#define TL_AFTER(x) asm volatile("" ::"r"(x) : "memory")
#define TLC_DECL long long tlc_last = clock64(); unsigned tlc_acc[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u}; unsigned tlc_n = 0u
#define TLC(i) { const long long tlc_now = clock64(); tlc_acc[i] += (unsigned)(tlc_now - tlc_last); tlc_last = tlc_now; }
#define TLC_TILE ++tlc_n
#define TLC_REPORT(on) { if (on) { for (int i_ = 0; i_ < 8; ++i_) tl_value(32, i_, tlc_acc[i_]); tl_value(32, 8, tlc_n); } \
    for (int i_ = 0; i_ < 8; ++i_) tlc_acc[i_] = 0u; tlc_n = 0u; }
#else
#define TL_AFTER(x)
#define TLC_DECL
#define TLC(i)
#define TLC_TILE
#define TLC_REPORT(on)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// One 32-byte store (the address a multiple of 32).
__device__ __forceinline__ void st_global_32B(void* ptr, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
               ::"l"(ptr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// All 128 threads of one softmax warpgroup (named barrier 1 + tile).
__device__ __forceinline__ void group_sync(int t) {
  asm volatile("bar.sync %0, 128;\n" ::"r"(1 + t) : "memory");
}

// The range of key tiles that query tile t visits within an item; empty when last < first.
struct TileRange { int rows, pos0, first, last; };
__device__ __forceinline__ TileRange tile_range(const AttnItem& it, int t, int window) {
  TileRange g;
  g.rows = min(kAtBM, it.rows - t * kAtBM);
  g.pos0 = it.pos0 + t * kAtBM;
  const int lo = (window > 0 && g.pos0 - window + 1 > 0) ? g.pos0 - window + 1 : 0;
  g.first = max(lo / kAtBN, it.kt_begin);
  g.last = g.rows > 0 ? min((g.pos0 + g.rows - 1) / kAtBN, it.kt_end - 1) : g.first - 1;
  return g;
}
// First key tile that the item loads at all (tile 0 has the lowest window edge).
__device__ __forceinline__ int item_first_kt(const AttnItem& it, int window) {
  const int lo = (window > 0 && it.pos0 - window + 1 > 0) ? it.pos0 - window + 1 : 0;
  return max(lo / kAtBN, it.kt_begin);
}

template <int D>
__global__ void __launch_bounds__(kAtThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, AttnTcParams p) {
  constexpr int SUB = D / 64;                          // 64-column sub-tiles per row
  constexpr uint32_t Q_BYTES = kAtBM * D * 2;          // one query tile
  constexpr uint32_t KSUB_BYTES = kAtBN * 64 * 2;      // one sub-tile of a key or value tile
  constexpr uint32_t KV_BYTES = kAtBN * D * 2;         // one key tile (or one value tile)
  constexpr uint32_t STAGE_BYTES = 2 * KV_BYTES;       // a key tile and its value tile
  constexpr uint32_t V_RING = kAtStages * KV_BYTES;    // the value tiles' ring lies behind the key tiles'
  constexpr uint32_t TMEM_COLS = 512;   // query tile t: scores at t*128 + {0, 64}, outputs at 256 + t*128
  constexpr uint32_t DATA_BYTES = 2 * kAtQT * Q_BYTES + kAtStages * STAGE_BYTES;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t raw = gt_smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);
  const uint32_t q_smem = base;                        // [item parity][query tile]
  const uint32_t kv_smem = q_smem + 2 * kAtQT * Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DATA_BYTES);
  // Key tiles and value tiles have rings of their own: a key tile is given back as soon as its
  // S is computed, a value tile only after the softmax and the second product, so the keys of the
  // tile after next can be on their way a whole step earlier than in a ring of (key, value) pairs.
  uint64_t* k_full = bars;                        // kAtStages each
  uint64_t* k_empty = k_full + kAtStages;
  uint64_t* v_full = k_empty + kAtStages;
  uint64_t* v_empty = v_full + kAtStages;
  uint64_t* work_full = v_empty + kAtStages;      // 2
  uint64_t* work_empty = work_full + 2;           // 2
  uint64_t* tile_bars = work_empty + 2;           // per query tile: q_full[2] q_empty[2] s_full[2] p_full[2] p_empty[2] o_full
  auto q_full = [&](int t, int par) { return gt_smem_u32(tile_bars + t * 11 + par); };
  auto q_empty = [&](int t, int par) { return gt_smem_u32(tile_bars + t * 11 + 2 + par); };
  auto s_full = [&](int t, int b) { return gt_smem_u32(tile_bars + t * 11 + 4 + b); };
  auto p_full = [&](int t, int b) { return gt_smem_u32(tile_bars + t * 11 + 6 + b); };
  auto p_empty = [&](int t, int b) { return gt_smem_u32(tile_bars + t * 11 + 8 + b); };
  auto o_full = [&](int t) { return gt_smem_u32(tile_bars + t * 11 + 10); };
  AttnItem* items = reinterpret_cast<AttnItem*>(tile_bars + kAtQT * 11);       // 2 slots
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(items + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;                           // per query tile: this part arrived last

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int n_items = p.n_records * p.n_q_heads;       // heads vary fastest: the query heads that share a
                                                       // kv head run at the same time and find its pages in L2
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAtStages; ++s) {
      mbar_init(gt_smem_u32(&k_full[s]), 1);
      mbar_init(gt_smem_u32(&k_empty[s]), kAtQT);       // one arrival per issuing warp
      mbar_init(gt_smem_u32(&v_full[s]), 1);
      mbar_init(gt_smem_u32(&v_empty[s]), kAtQT);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(gt_smem_u32(&work_full[s]), 1);
      mbar_init(gt_smem_u32(&work_empty[s]), kAtQT * 5);   // an issuing thread and four softmax warps per tile
    }
    for (int t = 0; t < kAtQT; ++t) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(q_full(t, b), 1);
        mbar_init(q_empty(t, b), 1);
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
  pdl_wait();     // queries, cache pages and the item list come from earlier kernels and copies

  if (warp == 0) {
    // ---- producer: items, query tiles, key and value tiles ------------------------------------
    // It runs ahead of the other roles: while the last stages of item n are loaded, item n + 1 is
    // published with its queries under way (the buffers of its parity are free since item n - 1),
    // so that no role finds the start of an item waiting for a chain of memory round trips.
    auto ask_index = [&]() { return lane == 0 ? atomicAdd(p.sched, 1) : 0; };          // lane 0 holds the answer
    auto ask_record = [&](int w) {
      return (w < n_items && lane < kAtRec) ? p.records[(size_t)(w / p.n_q_heads) * kAtRec + lane] : 0;
    };
    auto decode = [&](int w, int field) {
      AttnItem it;
      it.tok0 = __shfl_sync(0xffffffffu, field, 0);
      it.rows = __shfl_sync(0xffffffffu, field, 1);
      it.pos0 = __shfl_sync(0xffffffffu, field, 2);
      it.slot = __shfl_sync(0xffffffffu, field, 3);
      it.kt_begin = __shfl_sync(0xffffffffu, field, 4);
      it.kt_end = __shfl_sync(0xffffffffu, field, 5);
      it.part = __shfl_sync(0xffffffffu, field, 6);
      it.n_parts = __shfl_sync(0xffffffffu, field, 7);
      it.poff = __shfl_sync(0xffffffffu, field, 8);
      it.split = __shfl_sync(0xffffffffu, field, 9);
      it.merger = __shfl_sync(0xffffffffu, field, 10);
      it.head = w < n_items ? w % p.n_q_heads : 0;
      it.valid = w < n_items ? 1 : 0;
      it.index = w;
      if (it.valid && (it.rows <= 0 || it.rows > kAtQT * kAtBM || it.kt_begin < 0 || it.kt_end <= it.kt_begin ||
                       it.n_parts < 1 || it.n_parts > kAtMaxParts || it.part < 0 || it.part >= it.n_parts)) {
        if (lane == 0) set_error(p.err, kErrRequest, w / p.n_q_heads, it.rows, it.kt_end);
        it.valid = 0;
      }
      return it;
    };
    // item n goes into slot n & 1, free when every role has read item n - 2
    auto publish = [&](const AttnItem& it, int n) {
      const int s = n & 1;
      if (n >= 2 &&
          !__all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&work_empty[s]), (uint32_t)((n >> 1) - 1) & 1u, abort_flag))) {
        if (lane == 0) { set_error(p.err, kErrWait, 9, n, s); *abort_flag = 1; tl_value(31, 9, (unsigned)n); }
        return false;
      }
      if (lane == 0) {
        items[s] = it;
        mbar_arrive(gt_smem_u32(&work_full[s]));       // releases the slot's contents to the waiting roles
        tl_value(30, 1, (unsigned)it.index);
      }
      return true;
    };
    // the query tiles of item n go into the buffers of its parity, free since item n - 2
    auto load_queries = [&](const AttnItem& it, int n) {
      const int s = n & 1;
#pragma unroll
      for (int t = 0; t < kAtQT; ++t) {
        if (n >= 2 &&
            !__all_sync(0xffffffffu, mbar_wait(q_empty(t, s), (uint32_t)((n >> 1) - 1) & 1u, abort_flag))) {
          if (lane == 0) { set_error(p.err, kErrWait, 10, n, t); *abort_flag = 1; tl_value(31, 10, (unsigned)(n * 2 + t)); }
          return false;
        }
        if (lane == 0) {
          mbar_expect_tx(q_full(t, s), Q_BYTES);
#pragma unroll
          for (int cc = 0; cc < SUB; ++cc) {
            tma_load_3d(q_smem + (s * kAtQT + t) * Q_BYTES + cc * (kAtBM * 128), &map_q, cc * 64, it.head,
                        it.tok0 + t * kAtBM, q_full(t, s));
          }
        }
      }
      return true;
    };
    // a stage is (64 / kpl) page parts x SUB column halves x {key, value}: one copy per lane
    const int kpl = p.page_size < kAtBN ? p.page_size : kAtBN;     // keys per load
    const int n_loads = (kAtBN / kpl) * SUB * 2;                   // at most 32: page sizes from 8
    const bool loader = lane < n_loads;
    const int is_v = lane & 1, c = (lane >> 1) % SUB, u = lane / (2 * SUB);
    struct Walk { int first_kt, n_kt, lo_block, pos_last, hkv; const int* table; };
    auto walk_of = [&](const AttnItem& it) {
      Walk g;
      g.first_kt = item_first_kt(it, p.window);
      g.n_kt = it.valid ? max(0, it.kt_end - g.first_kt) : 0;
      g.lo_block = (p.window > 0 && it.pos0 - p.window + 1 > 0) ? it.pos0 - p.window + 1 : 0;
      g.pos_last = it.pos0 + it.rows - 1;
      g.hkv = it.head / group;
      g.table = p.block_table + (size_t)it.slot * p.max_pages;
      return g;
    };
    auto key0_of = [&](const Walk& g, int j) {
      int key0 = (g.first_kt + j) * kAtBN + u * kpl;
      if (key0 + kpl - 1 < g.lo_block || key0 > g.pos_last) key0 = (g.pos_last / kpl) * kpl;   // nothing visible here
      return key0;
    };
    auto lookup = [&](const Walk& g, int j) {
      const int pidx = key0_of(g, j) / p.page_size;
      return (loader && j < g.n_kt && pidx < p.max_pages) ? g.table[pidx] : -1;
    };

    int w_cur = ask_index();
    w_cur = __shfl_sync(0xffffffffu, w_cur, 0);
    AttnItem cur = decode(w_cur, ask_record(w_cur));
    bool ok = publish(cur, 0);
    if (ok && cur.valid) ok = load_queries(cur, 0);
    Walk walk = walk_of(cur);
    int page = lookup(walk, 0);
    int st = 0;                 // stage to fill next
    uint32_t sph = 0;           // its phase
    for (int n = 0; ok && cur.valid; ++n) {
      // The next item is asked for late, five stages before this one is loaded (the stages run a
      // few key tiles ahead of the products): early enough for its index, its record, its
      // queries and its first pages to arrive one after the other while the last stages go out,
      // late enough that an item is claimed only shortly before it starts, so the SMs end together.
      const int j_ask = max(0, walk.n_kt - 5);
      int w_nxt = 0, field_nxt = 0;
      AttnItem nxt = cur;
      Walk walk_nxt = walk;
      int page_nxt = -1;
      bool nxt_out = false;
      for (int j = 0; (j < walk.n_kt || !nxt_out) && ok; ++j) {
        if (j < walk.n_kt) {
          const int page_next = lookup(walk, j + 1);       // under way while this stage waits and is issued
          const int key0 = key0_of(walk, j);
          if (loader && (page < 0 || page >= p.num_pages)) {
            set_error(p.err, kErrPage, cur.index / p.n_q_heads, key0 / p.page_size, page);
            page = 0;
          }
          const int row = (page * p.n_kv_heads + walk.hkv) * p.page_size + (key0 % p.page_size);
          const uint32_t dst = kv_smem + st * KV_BYTES + c * KSUB_BYTES + u * kpl * 128;
          // the key tile, then the value tile: both issuers gave the buffer back (a fresh barrier
          // counts as given back once)
          ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&k_empty[st]), sph ^ 1u, abort_flag));
          if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 11, j, st); *abort_flag = 1; tl_value(31, 11, (unsigned)((n << 16) | (j << 4) | st)); } break; }
          if (lane == 0) mbar_expect_tx(gt_smem_u32(&k_full[st]), KV_BYTES);
          __syncwarp();
          if (loader && !is_v) tma_load_2d(dst, &map_k, c * 64, row, gt_smem_u32(&k_full[st]));
          ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&v_empty[st]), sph ^ 1u, abort_flag));
          if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 11, j, 8 + st); *abort_flag = 1; tl_value(31, 11, (unsigned)((n << 16) | (j << 4) | 8 | st)); } break; }
          if (lane == 0) mbar_expect_tx(gt_smem_u32(&v_full[st]), KV_BYTES);
          __syncwarp();
          if (loader && is_v) tma_load_2d(dst + V_RING, &map_v, c * 64, row, gt_smem_u32(&v_full[st]));
          if (++st == kAtStages) { st = 0; sph ^= 1u; }
          page = page_next;
        }
        if (j == j_ask) {
          w_nxt = ask_index();
        } else if (j == j_ask + 1) {
          w_nxt = __shfl_sync(0xffffffffu, w_nxt, 0);
          field_nxt = ask_record(w_nxt);
        } else if (j == j_ask + 2) {
          nxt = decode(w_nxt, field_nxt);
          ok = publish(nxt, n + 1);
          if (ok && nxt.valid) ok = load_queries(nxt, n + 1);
          walk_nxt = walk_of(nxt);
          page_nxt = lookup(walk_nxt, 0);
          nxt_out = true;
        }
      }
      cur = nxt;
      walk = walk_nxt;
      page = page_nxt;
    }
  } else if (warp == 1 || warp == kAtMmaWarp1) {
    // ---- MMA issuer of query tile t ------------------------------------------------------------
    // Both issuers walk all key tiles of every item, so that each gives every stage back exactly
    // once; a tile outside the query tile's own range gets no products.  The walk runs on across
    // items: S of a key tile is issued before the thread waits for the probabilities of the key
    // tile before, also when that one belongs to the item before.
    const int t = warp == 1 ? 0 : 1;
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(kAtBN, false);
      const uint32_t idesc_o = umma_idesc(D, true);
      // The descriptors are made once; a product adds what changes (16-byte units in the low bits):
      // issuing is a chain of dependent instructions in one thread, and every one of them counts.
      const uint64_t desc_q = umma_desc_sw128(q_smem + t * Q_BYTES);
      const uint64_t desc_k = umma_desc_sw128(kv_smem);
      const uint64_t desc_v = umma_desc_sw128_mn(kv_smem + V_RING, KSUB_BYTES);
      const uint32_t tmem_s_t = tmem_base + (uint32_t)(t * 128);
      const uint32_t tmem_o_t = tmem_base + (uint32_t)(256 + t * 128);
      int st = 0;                // stage of the key tile whose S comes next
      uint32_t sph = 0;
      uint32_t g_qk = 0, g_pv = 0;   // key tiles of this query tile whose S / whose O += P V has been issued
      unsigned int tl_n = 0;
      // the key tile whose S comes next: item n, tile j of its n_kt
      int n = -1, j = 0, n_kt = 0, first_kt = 0, par = 0;
      TileRange my = {0, 0, 0, -1};
      bool q_seen = false, q_given = true, ended = false;
      // up to two key tiles whose S has been issued (or that are not this tile's) and whose second
      // product and hand-back of the stage are still to come, oldest first
      // (packed: bit 0 this tile's, bit 1 its first, bit 2 its last key tile, bit 3 the phase, bits 4.. the stage)
      int pd0 = 0, pd1 = 0;
      int pd_head = 0, pd_size = 0;
      unsigned idle = 0;
      // An event loop, not a fixed order: the second product of the oldest pending key tile goes
      // out as soon as its probabilities are there, S of the next key tile as soon as its keys
      // are; neither waits for something the other could do meanwhile (the next item's first keys
      // arrive late, the last probabilities of an item must not wait for them).
      while (true) {
        bool progressed = false;
        if (pd_size > 0) {
          const int pd = pd_head ? pd1 : pd0;
          const bool pd_mine = pd & 1, pd_first = pd & 2, pd_last = pd & 4;
          const int pd_st = (pd >> 4) & 7;
          const uint32_t pd_ph = (uint32_t)(pd >> 3) & 1u;
          // the values have arrived (also where this tile does not read them: a buffer is given
          // back only after it was seen filled, or the barrier could get a phase ahead of the
          // producer's wait), and the probabilities are there
          if (mbar_test(gt_smem_u32(&v_full[pd_st]), pd_ph) &&
              (!pd_mine || mbar_test(p_full(t, g_pv & 1), (g_pv >> 1) & 1u))) {
            if (pd_mine) {
              const uint64_t desc_vs = desc_v + (uint64_t)((uint32_t)pd_st * (KV_BYTES >> 4));
              const int b = g_pv & 1;
              if (blockIdx.x == 0) tl_own(t, tl_n, 30, 84 + t, g_pv);
              tc_fence_after();
              const uint32_t p_tmem = tmem_s_t + (uint32_t)(b * kAtBN);      // 16 keys = 8 columns
#pragma unroll
              for (int kk = 0; kk < kAtBN / 16; ++kk) {
                const uint64_t db = desc_vs + (uint64_t)(kk * ((16 * 128) >> 4));
                umma_bf16_ts(tmem_o_t, p_tmem + (uint32_t)(8 * kk), db, idesc_o, (!pd_first || kk > 0) ? 1u : 0u);
              }
              umma_commit(p_empty(t, b));
              if (pd_last) umma_commit(o_full(t));
              ++g_pv;
              if (blockIdx.x == 0) tl_own(t, tl_n, 30, 86 + t, g_pv);
            }
            umma_commit(gt_smem_u32(&v_empty[pd_st]));     // this issuer is done with the value tile
            pd_head ^= 1;
            --pd_size;
            progressed = true;
          }
        }
        if (!ended && pd_size < 2) {
          if (j >= n_kt) {
            // The item is walked through: its queries are free after the products issued so far.
            // Only queries that have arrived are given back: an item without key tiles is walked
            // through at once, and a release that came before the producer had waited for the
            // release of the item two before would put the barrier a phase ahead of that wait.
            if (!q_given) {
              if (!q_seen) q_seen = mbar_test(q_full(t, par), (uint32_t)(n >> 1) & 1u);
              if (q_seen) { umma_commit(q_empty(t, par)); q_given = true; progressed = true; }
            }
            const int s = (n + 1) & 1;
            if (q_given && mbar_test(gt_smem_u32(&work_full[s]), (uint32_t)((n + 1) >> 1) & 1u)) {
              ++n;
              const AttnItem it = items[s];
              mbar_arrive(gt_smem_u32(&work_empty[s]));
              if (!it.valid) {
                ended = true;
              } else {
                my = tile_range(it, t, p.window);
                first_kt = item_first_kt(it, p.window);
                n_kt = max(0, it.kt_end - first_kt);
                j = 0;
                par = s;
                q_seen = false;
                q_given = false;
                tl_value(30, 60 + t, (unsigned)it.index);
              }
              progressed = true;
            }
          } else {
            const int kt = first_kt + j;
            const bool mine = kt >= my.first && kt <= my.last;
            // S of a key tile of this query tile goes into the buffer that held the probabilities
            // of the key tile two before: their second product must have been issued (the tensor
            // cores run this thread's products in order)
            bool can = mbar_test(gt_smem_u32(&k_full[st]), sph) && (!mine || g_qk - g_pv <= 1u);
            if (can && mine && !q_seen) {
              q_seen = mbar_test(q_full(t, par), (uint32_t)(n >> 1) & 1u);
              can = q_seen;
            }
            if (can) {
              if (mine) {
                const uint64_t desc_qs = desc_q + (uint64_t)((uint32_t)par * ((kAtQT * Q_BYTES) >> 4));
                const uint64_t desc_ks = desc_k + (uint64_t)((uint32_t)st * (KV_BYTES >> 4));
                const int b = g_qk & 1;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                  const uint64_t da = desc_qs + (uint64_t)((ks / 4) * ((kAtBM * 128) >> 4) + 2 * (ks % 4));
                  const uint64_t db = desc_ks + (uint64_t)((ks / 4) * (KSUB_BYTES >> 4) + 2 * (ks % 4));
                  umma_bf16(tmem_s_t + (uint32_t)(b * kAtBN), da, db, idesc_s, ks > 0 ? 1u : 0u);
                }
                umma_commit(s_full(t, b));
                ++g_qk;
                if (blockIdx.x == 0) tl_own(t, tl_n, 30, 82 + t, g_qk);
              }
              umma_commit(gt_smem_u32(&k_empty[st]));      // the key tile is free once S is computed
              const int pd_new = (mine ? 1 : 0) | (kt == my.first ? 2 : 0) | (kt == my.last ? 4 : 0) | ((int)sph << 3) | (st << 4);
              if (pd_head ^ (pd_size & 1)) pd1 = pd_new; else pd0 = pd_new;     // behind the pending one, if there is one
              ++pd_size;
              ++j;
              if (++st == kAtStages) { st = 0; sph ^= 1u; }
              progressed = true;
            }
          }
        }
        if (ended && pd_size == 0) break;
        if (progressed) {
          idle = 0;
        } else if (++idle >= kGtSpinLimit || ((idle & 1023u) == 1023u && *abort_flag)) {
          // what it was waiting for: tile, item, then pending key tiles | key tile of the item | products issued
          if (idle >= kGtSpinLimit) {
            set_error(p.err, kErrWait, 12 + 100 * t, n, (pd_size << 28) | ((j & 0xfff) << 16) | (int)(g_pv & 0xffffu));
            *abort_flag = 1;
          }
          tl_value(31, 12, (unsigned)((t << 31) | (n << 24) | (pd_size << 22) | ((j & 0xff) << 14) | ((n_kt & 0xff) << 6) | (ended ? 32 : 0) | (q_seen ? 16 : 0) | (st << 2)));
          break;
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
    uint32_t g = 0;              // key tiles of this query tile so far
    uint32_t n_out = 0;          // items in which this query tile had key tiles
    unsigned int tl_n = 0;
    bool ok = true;
    TLC_DECL;

    for (int n = 0; ok; ++n) {
      const int s = n & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&work_full[s]), (uint32_t)(n >> 1) & 1u, abort_flag));
      if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 17, n, t); *abort_flag = 1; tl_value(31, 17, (unsigned)(n * 2 + t)); } break; }
      const AttnItem it = items[s];
      __syncwarp();
      if (lane == 0) mbar_arrive(gt_smem_u32(&work_empty[s]));
      if (!it.valid) break;
      const TileRange my = tile_range(it, t, p.window);
      if (my.rows <= 0) continue;                       // the item has one query tile only
      const bool row_valid = row < my.rows;
      const int pos_r = my.pos0 + row;
      const int lo_r = (p.window > 0 && pos_r - p.window + 1 > 0) ? pos_r - p.window + 1 : 0;
      const int my_kt = my.last - my.first + 1;         // <= 0: a part without keys for this tile
      float m_ref = -INFINITY, l_sum = 0.0f;
      if (row == 0) tl_value(30, 10 + t, (unsigned)it.index);

      TLC(7);       // between items: the rows written out, the next item taken
      for (int j = 0; j < my_kt && ok; ++j, ++g) {
        const int b = g & 1;
        TLC(6);     // the loop itself
        ok = __all_sync(0xffffffffu, mbar_wait(s_full(t, b), (g >> 1) & 1u, abort_flag));
        if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 18, j, t); *abort_flag = 1; tl_value(31, 18, (unsigned)((n << 20) | (j << 8) | (my_kt << 1) | t)); } break; }
        tc_fence_after();
        TLC(0);     // waiting for S
        if (blockIdx.x == 0 && row == 0) tl_own(2 + t, tl_n, 30, 70 + t, g);
        uint32_t sraw[kAtBN];
        {
          uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[0]);
          uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[32]);
          tmem_ld32(tmem_s + (uint32_t)(b * kAtBN), lo);
          tmem_ld32(tmem_s + (uint32_t)(b * kAtBN) + 32, hi);
          tmem_wait_ld();
        }
        TL_AFTER(sraw[kAtBN - 1]);
        TLC(1);     // S loaded

        // Scores stay unscaled in sv; the softmax scale (> 0) is folded into the exponent below.
        // A tile wholly below this row's diagonal and inside its window needs no mask.
        const int key_first = (my.first + j) * kAtBN;
        // (decided per warp: a warp whose rows disagree would run both forms one after the other)
        const bool interior = __all_sync(0xffffffffu, row_valid && key_first + kAtBN - 1 <= pos_r && key_first >= lo_r);
        // (one chain each for the maximum and the sum below; two or four chains per thread were
        // measured 2 % slower: the instructions to join them cost more than the latency they hide)
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
        TL_AFTER(__float_as_uint(m_new));
        TLC(2);     // the maximum
        if (__any_sync(0xffffffffu, need)) {
          const float corr = need ? exp2f(m_ref - m_new) : 1.0f;
          if (need) { l_sum *= corr; m_ref = m_new; }
          if (j > 0) {
            // the product that added the key tile before to the output has to be done
            ok = __all_sync(0xffffffffu, mbar_wait(p_empty(t, (g - 1u) & 1u), ((g - 1u) >> 1) & 1u, abort_flag));
            if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 19, j, t); *abort_flag = 1; tl_value(31, 19, (unsigned)(n * 2 + t)); } break; }
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
          TL_AFTER(__float_as_uint(l_sum));
          TLC(3);   // exponentials, sum, conversion, store issued (and a rescaled output, when it happens)
          tmem_wait_st();
        }
        TLC(4);     // the store has arrived
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(t, b));
        TLC(5);     // fence and arrival
        TLC_TILE;
        if (blockIdx.x == 0 && row == 0) tl_own(2 + t, tl_n, 30, 74 + t, g);
      }
      TLC_REPORT(blockIdx.x == 0 && row == 0);
      if (!ok) break;
      if (row == 0) tl_value(30, 20 + t, (unsigned)it.index);

      if (my_kt > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(o_full(t), n_out & 1u, abort_flag));
        if (!ok) { if (lane == 0) { set_error(p.err, kErrWait, 20, n, t); *abort_flag = 1; tl_value(31, 20, (unsigned)(n * 2 + t)); } break; }
        ++n_out;
        tc_fence_after();
      }
      if (row == 0) tl_value(30, 30 + t, (unsigned)it.index);
      if (it.n_parts == 1) {
        if (my_kt > 0) {
          const float inv = (row_valid && l_sum > 0.0f) ? 1.0f / l_sum : 0.0f;
          __nv_bfloat16* orow = p.out + ((size_t)(it.tok0 + t * kAtBM + row) * p.n_q_heads + it.head) * D;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c * 32, o);
            tmem_wait_ld();
            if (row_valid) {
              // 32 bytes a store: a row is written by its own thread, so every store is a memory
              // transaction of its own, and half as many of them take half the time
#pragma unroll
              for (int q8 = 0; q8 < 2; ++q8) {
                uint32_t v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[q8 * 16 + 2 * e]) * inv,
                                                                  __uint_as_float(o[q8 * 16 + 2 * e + 1]) * inv);
                  v[e] = *reinterpret_cast<const uint32_t*>(&h2);
                }
                st_global_32B(orow + c * 32 + q8 * 16, v);
              }
            }
          }
        }
        if (row == 0) tl_value(30, 40 + t, (unsigned)it.index);
        continue;
      }

      // ---- one part of several --------------------------------------------------------------------
      // Every part but one leaves its unnormalised output, maximum and sum in scratch and counts
      // itself in; the part that the host lists last (`merger`) keeps its own in tensor memory,
      // waits until the others are counted and adds all up.  Items are handed out in list order,
      // so when the merger runs, every other part is running or done: the wait cannot starve.
      // Scratch of a (part, head, tile): float4 (c, row) at (c * 128 + row), so that the 32 rows of
      // a warp make one 512-byte access; maxima and sums as [2][128].
      const size_t slot0 = ((size_t)it.poff * p.n_q_heads + it.head) * kAtQT + t;   // part 0 of this tile
      const size_t slot_step = (size_t)p.n_q_heads * kAtQT;                          // from one part to the next
      auto part_rows = [&](int q) { return reinterpret_cast<float4*>(p.part_o) + (slot0 + q * slot_step) * (D / 4) * kAtBM + row; };
      auto part_m = [&](int q) { return p.part_ml + (slot0 + q * slot_step) * 2 * kAtBM + row; };
      int* count = p.part_count + ((size_t)it.split * p.n_q_heads + it.head) * kAtQT + t;
      const float l_own = (my_kt > 0 && row_valid) ? l_sum : 0.0f;
      if (!it.merger) {
        float4* po = part_rows(it.part);
        if (my_kt > 0) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              __stcg(po + (c * 8 + e) * kAtBM,
                     make_float4(__uint_as_float(o[4 * e]), __uint_as_float(o[4 * e + 1]), __uint_as_float(o[4 * e + 2]),
                                 __uint_as_float(o[4 * e + 3])));
            }
          }
        }
        __stcg(part_m(it.part), m_ref);
        __stcg(part_m(it.part) + kAtBM, l_own);
        group_sync(t);                  // the rows of all 128 threads are written
        if (row == 0) {
          __threadfence();              // and visible to the device before the count says so
          atomicAdd(count, 1);
          tl_value(30, 40 + t, (unsigned)it.index);
        }
        continue;
      }
      if (row == 0) {
        int seen = 0;
        unsigned spin = 0;
        for (; spin < kGtSpinLimit; ++spin) {
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(seen) : "l"(count) : "memory");
          if (seen >= it.n_parts - 1 || ((spin & 1023u) == 1023u && *abort_flag)) break;
          __nanosleep(64);
        }
        last_flag[t] = seen >= it.n_parts - 1;
        if (seen >= it.n_parts - 1) {
          *count = 0;                   // ready for the next launch
        } else {
          set_error(p.err, kErrWait, 21, it.index, seen);
          tl_value(31, 21, (unsigned)((n << 20) | (seen << 12) | (it.n_parts << 4) | t));
          *abort_flag = 1;
        }
        tl_value(30, 40 + t, (unsigned)it.index);
      }
      group_sync(t);
      ok = last_flag[t] != 0;
      group_sync(t);                    // the flag is read before another item writes it
      if (!ok) break;
      __threadfence();
      {
        // maxima and sums of the other parts, eight in flight at a time; this part's own are in registers
        float m_all = l_own > 0.0f ? m_ref : -INFINITY;
        for (int q0 = 0; q0 < it.n_parts; q0 += 8) {
          float m[8], l[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool on = q0 + i < it.n_parts && q0 + i != it.part;
            m[i] = on ? __ldcg(part_m(q0 + i)) : -INFINITY;
            l[i] = on ? __ldcg(part_m(q0 + i) + kAtBM) : 0.0f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) if (l[i] > 0.0f) m_all = fmaxf(m_all, m[i]);
        }
        float l_all = l_own > 0.0f ? l_own * exp2f(m_ref - m_all) : 0.0f;
        for (int q0 = 0; q0 < it.n_parts; q0 += 8) {
          float m[8], l[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool on = q0 + i < it.n_parts && q0 + i != it.part;
            m[i] = on ? __ldcg(part_m(q0 + i)) : -INFINITY;
            l[i] = on ? __ldcg(part_m(q0 + i) + kAtBM) : 0.0f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) if (l[i] > 0.0f) l_all += l[i] * exp2f(m[i] - m_all);
        }
        const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
        const float w_own = l_own > 0.0f ? exp2f(m_ref - m_all) * inv : 0.0f;
        __nv_bfloat16* orow = p.out + ((size_t)(it.tok0 + t * kAtBM + row) * p.n_q_heads + it.head) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          float acc[32];
          if (my_kt > 0) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) acc[e] = w_own > 0.0f ? __uint_as_float(o[e]) * w_own : 0.0f;
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) acc[e] = 0.0f;
          }
          for (int q0 = 0; q0 < it.n_parts; q0 += 2) {
            float4 v[2][8];
            float wgt[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const bool on = q0 + i < it.n_parts && q0 + i != it.part;
              const float m = on ? __ldcg(part_m(q0 + i)) : -INFINITY;
              const float l = on ? __ldcg(part_m(q0 + i) + kAtBM) : 0.0f;
              wgt[i] = l > 0.0f ? exp2f(m - m_all) * inv : 0.0f;
              const float4* po = part_rows(on ? q0 + i : it.part == 0 ? 1 : 0) + (size_t)c * 8 * kAtBM;
#pragma unroll
              for (int e = 0; e < 8; ++e) v[i][e] = __ldcg(po + e * kAtBM);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (wgt[i] > 0.0f) {         // a part without keys for this row holds no numbers
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  acc[4 * e] += v[i][e].x * wgt[i]; acc[4 * e + 1] += v[i][e].y * wgt[i];
                  acc[4 * e + 2] += v[i][e].z * wgt[i]; acc[4 * e + 3] += v[i][e].w * wgt[i];
                }
              }
            }
          }
          if (row_valid) {
#pragma unroll
            for (int q8 = 0; q8 < 2; ++q8) {
              uint32_t v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[q8 * 16 + 2 * e], acc[q8 * 16 + 2 * e + 1]);
                v[e] = *reinterpret_cast<const uint32_t*>(&h2);
              }
              st_global_32B(orow + c * 32 + q8 * 16, v);
            }
          }
        }
        if (row == 0) tl_value(30, 50 + t, (unsigned)it.index);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
  if (threadIdx.x == 0) {
    // the last block to leave puts the counters back for the next launch; every block asked for
    // its last item before it got here
    const int before = atomicAdd(p.sched + 1, 1);
    if (before == (int)gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

template <int D>
static int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                             const AttnTcParams& p, int blocks, cudaStream_t stream) {
  constexpr size_t smem_bytes = (size_t)2 * kAtQT * kAtBM * D * 2 + (size_t)kAtStages * 2 * kAtBN * D * 2 +
                                1024 /* alignment */ + 512 /* barriers, item slots */;
  static_assert(smem_bytes <= 232448, "shared memory of one block");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch(attn_prefill_tc_kernel<D>, dim3(blocks), dim3(kAtThreads), smem_bytes, stream, mq, mk, mv, p);
}

}  // namespace tk

TK_TIMELINE_SETTER(attention_prefill_tc)

// Query tokens of one item of tk_attention_prefill_tc, keys of one key tile, ints of an item
// record, and the most parts a block of tokens may be cut into.
TK_API int tk_attention_prefill_tc_rows(void) { return tk::kAtQT * tk::kAtBM; }
TK_API int tk_attention_prefill_tc_keys(void) { return tk::kAtBN; }
TK_API int tk_attention_prefill_tc_record_ints(void) { return tk::kAtRec; }
TK_API int tk_attention_prefill_tc_max_parts(void) { return tk::kAtMaxParts; }

// Whether tk_attention_prefill_tc takes a shape.
TK_API int tk_attention_prefill_tc_takes(int n_q_heads, int n_kv_heads, int head_dim, int page_size) {
  const bool pages_ok = page_size >= 8 && page_size % 8 == 0 &&
                        (tk::kAtBN % page_size == 0 || page_size % tk::kAtBN == 0);
  return (head_dim == 64 || head_dim == 128) && n_kv_heads >= 1 && n_q_heads % n_kv_heads == 0 && pages_ok;
}

// records: the item list (see AttnTcParams); sched: 2 ints, part_count: one int per (cut token
// block, head, query tile), both zero before the first launch (the kernel leaves them zero);
// part_o / part_ml: scratch for (parts of cut token blocks) x heads x 2 tiles x 128 rows x
// (head_dim | 2) floats, may be null when nothing is cut.  One launch at a time per set of
// counters and scratch.
TK_API int tk_attention_prefill_tc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                   const int* records, const int* block_table, int* err, int* sched,
                                   float* part_o, float* part_ml, int* part_count, int n_tokens, int n_records,
                                   int n_q_heads, int n_kv_heads, int head_dim, int page_size, int max_pages,
                                   int num_pages, int window, float scale, cudaStream_t stream) {
  if (n_records <= 0) return 0;
  if (!tk_attention_prefill_tc_takes(n_q_heads, n_kv_heads, head_dim, page_size) || n_q_heads > 65535 ||
      (long long)n_records * n_q_heads > 0x3fffffffLL) {
    return (int)cudaErrorInvalidValue;
  }
  static int sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidValue;
  if (sms[dev] == 0) {
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    sms[dev] = n;
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
  p.out = (__nv_bfloat16*)out; p.records = records; p.block_table = block_table; p.err = err; p.sched = sched;
  p.part_o = part_o; p.part_ml = part_ml; p.part_count = part_count;
  p.n_records = n_records; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const long long n_items = (long long)n_records * n_q_heads;
  const int blocks = (int)(n_items < sms[dev] ? n_items : sms[dev]);
  if (head_dim == 128) return tk::launch_prefill_tc<128>(mq, mk, mv, p, blocks, stream);
  return tk::launch_prefill_tc<64>(mq, mk, mv, p, blocks, stream);
}
