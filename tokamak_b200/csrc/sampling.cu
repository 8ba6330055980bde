// Token sampling over float32 logits, one cluster of thread blocks per row.
//
// Pipeline of the reference (src/tokamak/sampling/sampler.py:32-39,58-84):
// temperature 0 -> argmax; else logits / T -> top-k (keep values >= the k-th
// largest) -> top-p (in descending order, drop a token iff the probability mass
// before it already reached top_p) -> softmax -> one draw.  The draw here is an
// inverse-CDF lookup in vocabulary order with a Philox4x32-10 uniform keyed by
// the request's seed and counted by the index of the token being sampled, so a
// request's stream does not depend on batching or on preemption.  Tied values
// at a top-k or top-p threshold are all kept.
//
// Probability masses are accumulated as 64-bit fixed-point integers: integer
// sums do not depend on the order of the additions, so thresholds and draws are
// reproducible bit for bit.
#include "common.cuh"
#include "timeline.cuh"

namespace tk {

constexpr int kSampleThreads = 1024;
constexpr float kMassScale = 1099511627776.0f;  // 2^40

__device__ __forceinline__ unsigned int float_key(float v) {
  const unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__host__ __device__ inline void philox4x32_10(unsigned int c0, unsigned int c1, unsigned int c2,
                                              unsigned int c3, unsigned int k0, unsigned int k1,
                                              unsigned int* out) {
  const unsigned int M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = (unsigned long long)M0 * c0;
    const unsigned long long p1 = (unsigned long long)M1 * c2;
    const unsigned int hi0 = (unsigned int)(p0 >> 32), lo0 = (unsigned int)p0;
    const unsigned int hi1 = (unsigned int)(p1 >> 32), lo1 = (unsigned int)p1;
    const unsigned int n0 = hi1 ^ c1 ^ k0;
    const unsigned int n1 = lo1;
    const unsigned int n2 = hi0 ^ c3 ^ k1;
    const unsigned int n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct SampleParams {
  const float* logits;        // [n_rows, vocab], row stride = ld
  const float* temperature;   // [n_rows]
  const int* top_k;           // [n_rows], 0 = off
  const float* top_p;         // [n_rows], 1 = off
  const unsigned long long* seed;     // [n_rows]
  const unsigned int* counter;        // [n_rows] index of the token being sampled
  int* out_tokens;            // [n_rows]
  int vocab;
  long long ld;
  // With `records` the parameters of row r come from the state record of slot row_slot[r]
  // (layout in step_state.cu) instead of the arrays above, and the kernel writes the token
  // back into the record and advances its counter.
  int* records;
  const int* row_slot;
  int max_slots;
  int* err;
};

constexpr int kSlotWords = 8;

__device__ __forceinline__ unsigned long long warp_incl_scan_u64(unsigned long long v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  return v;
}

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kSampleCluster = 8;     // at most this many blocks share a row: a cluster, each with a slice of the vocabulary

__device__ __forceinline__ unsigned int ld_cluster_u32(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  unsigned int v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_cluster_u64(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];\n" : "=l"(v) : "r"(remote) : "memory");
  return v;
}

// One cluster of gridDim.x blocks (1, 2, 4 or 8: as many as keep all rows' blocks on the GPU at once) per
// row (blockIdx.y = row): every
// block works on its slice of the vocabulary, the blocks' histograms and sums meet in block 0 of the
// cluster over distributed shared memory, and what block 0 decides is read back the same way.  One
// block alone needed 15 us for every pass over a row of 151,936 logits, and a top-p threshold takes
// nine passes.  All blocks of a cluster take the same branches (they depend on the row only), so
// they meet at the same cluster barriers; the last barrier keeps every block's shared memory alive
// until nobody reads it any more.
__global__ void __launch_bounds__(kSampleThreads, 1) sample_kernel(SampleParams p) {
  pdl_trigger();
  if (threadIdx.x == 0) tl_mark(3, 0);
  pdl_wait();
  if (threadIdx.x == 0) tl_mark(3, 1);
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ unsigned int s_count[256];
  __shared__ unsigned long long s_mass[256];
  __shared__ unsigned long long s_warp_tot[32];
  __shared__ unsigned long long s_cta_tot;
  __shared__ unsigned int s_sel_key;
  __shared__ unsigned long long s_sel_rem;
  __shared__ int s_result;
  // Histograms of the first level, one per group of four warps: logits crowd into a few bins of the
  // top byte, and a thousand threads adding 64-bit masses to the same few words one after the other
  // took 0.5 ms per level (2 ms for a top-p threshold at a vocabulary of 151,936).  A mass (at most
  // 2^40) goes in as three pieces of 14, 14 and 12 bits with the hardware's own 32-bit additions; a
  // group adds at most vocab / 8 of them, fewer than 2^18 (the host checks the vocabulary).
  __shared__ unsigned int s_grp[kSampleThreads / 128][256][3];

  const int row = blockIdx.y;
  const uint32_t rank = cluster_ctarank();
  const int n_blocks = (int)gridDim.x;           // of this row's cluster
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int V = p.vocab;
  const float* lg = p.logits + (size_t)row * p.ld;
  int* rec = nullptr;
  if (p.records != nullptr) {
    const int slot = p.row_slot[row];
    if (slot < 0 || slot >= p.max_slots) {
      if (tid == 0 && rank == 0) { set_error(p.err, kErrRequest, row, slot, p.max_slots); p.out_tokens[row] = 0; }
      return;       // every block of the cluster, before any of them reads another's shared memory
    }
    rec = p.records + (size_t)slot * kSlotWords;
  }
  // everything that the record says is read now: the block that draws the token writes the record at the end
  const float T = rec ? __int_as_float(rec[4]) : p.temperature[row];
  const int k = rec ? rec[5] : p.top_k[row];
  const float top_p = rec ? __int_as_float(rec[6]) : p.top_p[row];
  const unsigned long long seed =
      rec ? ((unsigned long long)(unsigned int)rec[3] << 32) | (unsigned int)rec[2] : p.seed[row];
  const unsigned int counter = rec ? (unsigned int)rec[1] : p.counter[row];

  // this block's slice of the row: a multiple of 128 tokens, so that 16-byte loads stay aligned
  const int slice = ((V + n_blocks * 128 - 1) / (n_blocks * 128)) * 128;
  const int s_begin = min(V, (int)rank * slice);
  const int s_end = min(V, s_begin + slice);
  const int n_slice = s_end - s_begin;
  const float* ls = lg + s_begin;
  const bool vec = (reinterpret_cast<uintptr_t>(lg) & 15u) == 0;
  const int V4 = vec ? (n_slice >> 2) : 0;       // 16-byte loads of the slice
  // Every pass below walks the slice warp by warp with all 32 lanes in step (a lane beyond the end
  // brings nothing), 16 bytes a lane where the row starts on a 16-byte boundary.
  auto for_each = [&](auto&& body) {       // body(valid, index in the row, logit), called by all lanes of a warp together
    const float4* ls4 = reinterpret_cast<const float4*>(ls);
    for (int base = warp * 32; base < V4; base += kSampleThreads) {
      const int i4 = base + lane;
      const bool ok = i4 < V4;
      const float4 v = ok ? ls4[i4] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      body(ok, s_begin + 4 * i4, v.x);
      body(ok, s_begin + 4 * i4 + 1, v.y);
      body(ok, s_begin + 4 * i4 + 2, v.z);
      body(ok, s_begin + 4 * i4 + 3, v.w);
    }
    for (int base = V4 * 4 + warp * 32; base < n_slice; base += kSampleThreads) {
      const int i = base + lane;
      const bool ok = i < n_slice;
      body(ok, s_begin + i, ok ? ls[i] : 0.0f);
    }
  };

  // ---- pass 1: maximum and its lowest index ------------------------------------------
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for_each([&](bool ok, int i, float v) {
    if (ok && v > best) { best = v; best_i = i; }       // ascending i within a thread: the first maximum is kept
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane];
    best_i = s_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[0] = best; s_idx[0] = best_i; }
  }
  cluster_sync_all();                  // every block's maximum stands in its s_val[0], s_idx[0]
  best = -INFINITY;
  best_i = 0x7fffffff;
  for (uint32_t rk = 0; rk < (uint32_t)n_blocks; ++rk) {
    const float ov = __uint_as_float(ld_cluster_u32(&s_val[0], rk));
    const int oi = (int)ld_cluster_u32(&s_idx[0], rk);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  const float max_logit = best;
  const int arg_max = best_i;
  if (T == 0.0f) {
    if (tid == 0 && rank == 0) {
      p.out_tokens[row] = arg_max;
      if (rec) { rec[7] = arg_max; rec[1] += 1; }
      tl_mark(3, 4);
    }
    cluster_sync_all();                // nobody leaves while its maximum may still be read
    return;
  }
  const float zmax = max_logit / T;

  // ---- thresholds: radix descent over the order-preserving key of z = logit / T -------
  unsigned int thr_key = 0u;   // keep keys >= thr_key
  const bool use_k = (k > 0 && k < V);
  const bool use_p = (top_p < 1.0f);

  for (int phase = 0; phase < 2; ++phase) {
    if (phase == 0 && !use_k) continue;
    if (phase == 1 && !use_p) continue;
    unsigned int prefix = 0u, prefix_mask = 0u;
    unsigned long long remaining = 0ull;   // top-k: rank still to skip; top-p: mass target
    if (phase == 0) remaining = (unsigned long long)k;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      for (int b = tid; b < 256; b += kSampleThreads) { s_count[b] = 0u; s_mass[b] = 0ull; }
      if (level == 0) {
        unsigned int* flat = &s_grp[0][0][0];
        for (int i = tid; i < (kSampleThreads / 128) * 256 * 3; i += kSampleThreads) flat[i] = 0u;
      }
      __syncthreads();
      if (level == 0) {
        // every token of the slice takes part, in a few bins: into the histogram of the warp's group
        unsigned int (*mine)[3] = s_grp[warp >> 2];
        if (phase == 0) {
          for_each([&](bool ok, int, float logit) {
            const unsigned int key = float_key(logit / T);
            if (ok && key >= thr_key) atomicAdd(&mine[key >> 24][0], 1u);
          });
        } else {
          for_each([&](bool ok, int, float logit) {
            const float z = logit / T;
            const unsigned int key = float_key(z);
            if (ok && key >= thr_key) {
              const unsigned long long fx = __float2ull_rd(expf(z - zmax) * kMassScale);      // <= 2^40
              atomicAdd(&mine[key >> 24][0], (unsigned int)(fx & 0x3fffu));
              atomicAdd(&mine[key >> 24][1], (unsigned int)((fx >> 14) & 0x3fffu));
              atomicAdd(&mine[key >> 24][2], (unsigned int)(fx >> 28));
            }
          });
        }
        __syncthreads();
        if (tid < 256) {
          unsigned long long p0 = 0ull, p1 = 0ull, p2 = 0ull;
          for (int w = 0; w < kSampleThreads / 128; ++w) { p0 += s_grp[w][tid][0]; p1 += s_grp[w][tid][1]; p2 += s_grp[w][tid][2]; }
          s_count[tid] = (unsigned int)p0;
          s_mass[tid] = p0 + (p1 << 14) + (p2 << 28);
        }
      } else if (phase == 0) {
        // below the top byte the bins are many and the tokens in them few: they add for themselves
        for_each([&](bool ok, int, float logit) {
          const unsigned int key = float_key(logit / T);
          if (ok && key >= thr_key && (key & prefix_mask) == prefix) atomicAdd(&s_count[(key >> shift) & 0xffu], 1u);
        });
      } else {
        for_each([&](bool ok, int, float logit) {
          const float z = logit / T;
          const unsigned int key = float_key(z);
          if (ok && key >= thr_key && (key & prefix_mask) == prefix) {
            atomicAdd(&s_mass[(key >> shift) & 0xffu], __float2ull_rd(expf(z - zmax) * kMassScale));
          }
        });
      }
      cluster_sync_all();                // every block's histogram of its slice is complete
      if (rank == 0) {
        // block 0 adds the histograms up, bin by bin (a thread a bin), and decides
        unsigned int cnt = 0u;
        unsigned long long mass = 0ull;
        if (tid < 256) {
          for (uint32_t rk = 0; rk < (uint32_t)n_blocks; ++rk) {
            if (phase == 0) cnt += ld_cluster_u32(&s_count[tid], rk);
            else mass += ld_cluster_u64(&s_mass[tid], rk);
          }
          s_count[tid] = cnt;
          s_mass[tid] = mass;
        }
        __syncthreads();
        if (warp == 0) {
          // from the highest bin down: the first bin with anything in it whose count (mass), added to
          // what lies above it, reaches what remains.  Lane l holds the bins 255 - 8 l .. 248 - 8 l.
          unsigned long long w[8], mine = 0ull;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int b = 255 - (8 * lane + j);
            w[j] = (phase == 0) ? (unsigned long long)s_count[b] : s_mass[b];
            mine += w[j];
          }
          const unsigned long long all = warp_sum_u64(mine);
          if (phase == 1 && level == 0) {
            unsigned long long target = (unsigned long long)((double)top_p * (double)all);
            if (target > all) target = all;
            if (target == 0ull) target = 1ull;
            remaining = target;
          }
          unsigned long long cum = warp_incl_scan_u64(mine, lane) - mine;      // above this lane's bins
          int found = -1;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (found < 0) {
              if (w[j] > 0ull && cum + w[j] >= remaining) found = 255 - (8 * lane + j);
              else cum += w[j];
            }
          }
          const unsigned int hits = __ballot_sync(0xffffffffu, found >= 0);
          const int src = hits != 0u ? __ffs(hits) - 1 : 31;
          const int chosen = hits != 0u ? __shfl_sync(0xffffffffu, found, src) : 0;
          const unsigned long long above = __shfl_sync(0xffffffffu, cum, src);    // no hit: lane 31 has added all up
          if (lane == 0) {
            s_sel_key = (unsigned int)chosen;
            s_sel_rem = remaining - above;
          }
        }
      }
      cluster_sync_all();                // block 0 has decided; nobody clears a histogram before this
      prefix |= ld_cluster_u32(&s_sel_key, 0u) << shift;
      prefix_mask |= 0xffu << shift;
      remaining = ld_cluster_u64(&s_sel_rem, 0u);
    }
    if (prefix > thr_key) thr_key = prefix;
  }

  // ---- kept mass: every warp adds up one contiguous range of the block's slice -------------
  // (ranges of a multiple of 128 tokens, so that a lane's four tokens stay one 16-byte load)
  const int range = ((slice + 32 * 128 - 1) / (32 * 128)) * 128;
  const int r_begin = min(s_end, s_begin + warp * range);
  const int r_end = min(s_end, r_begin + range);
  auto mass_of = [&](float logit) -> unsigned long long {
    const float z = logit / T;
    return float_key(z) >= thr_key ? __float2ull_rd(expf(z - zmax) * kMassScale) : 0ull;
  };
  auto lane_masses = [&](int at, unsigned long long (&m)[4]) {      // tokens at .. at + 3 of this lane
    if (vec && at + 3 < r_end) {
      const float4 v = *reinterpret_cast<const float4*>(lg + at);
      m[0] = mass_of(v.x); m[1] = mass_of(v.y); m[2] = mass_of(v.z); m[3] = mass_of(v.w);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) m[j] = (at + j < r_end) ? mass_of(lg[at + j]) : 0ull;
    }
  };
  {
    unsigned long long local = 0ull;
    for (int at = r_begin + 4 * lane; at < r_end; at += 128) {
      unsigned long long m[4];
      lane_masses(at, m);
      local += m[0] + m[1] + m[2] + m[3];
    }
    local = warp_sum_u64(local);
    if (lane == 0) s_warp_tot[warp] = local;
    __syncthreads();
    if (tid == 0) {
      unsigned long long sum = 0ull;
      for (int w = 0; w < kSampleThreads / 32; ++w) sum += s_warp_tot[w];
      s_cta_tot = sum;
    }
  }
  cluster_sync_all();                    // every block's sum stands in its s_cta_tot
  unsigned long long total = 0ull, before = 0ull;       // of the row; of the slices before this block's
  for (uint32_t rk = 0; rk < (uint32_t)n_blocks; ++rk) {
    const unsigned long long t = ld_cluster_u64(&s_cta_tot, rk);
    if (rk < rank) before += t;
    total += t;
  }
  const unsigned long long mine_total = ld_cluster_u64(&s_cta_tot, rank);

  // ---- the draw: first index whose inclusive prefix exceeds u * total -------------------
  unsigned int rnd[4];
  philox4x32_10(counter, 0u, 0u, 0u, (unsigned int)seed, (unsigned int)(seed >> 32), rnd);
  // target = floor(rnd / 2^32 * total) < total
  const unsigned long long target = __umul64hi(total, (unsigned long long)rnd[0] << 32);
  // the block whose slice holds the target draws: its warp whose range holds it walks the range
  // again, 128 tokens at a time.  (Without any mass, which cannot be, block 0 gives the most likely token.)
  const bool owner = total > 0ull ? (before <= target && target < before + mine_total) : rank == 0u;
  if (owner) {
    if (tid == 0) s_result = arg_max;
    __syncthreads();
    for (int w = 0; w < warp; ++w) before += s_warp_tot[w];
    if (before <= target && target < before + s_warp_tot[warp]) {
      unsigned long long run = before;
      for (int at = r_begin + 4 * lane; at - 4 * lane < r_end; at += 128) {     // all lanes in step
        unsigned long long m[4];
        lane_masses(at, m);
        const unsigned long long mine = m[0] + m[1] + m[2] + m[3];
        const unsigned long long incl = warp_incl_scan_u64(mine, lane);
        const unsigned long long chunk = __shfl_sync(0xffffffffu, incl, 31);
        if (run + chunk > target) {
          unsigned long long at_me = run + incl - mine;          // mass before this lane's tokens
          if (at_me <= target && target < at_me + mine) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (target < at_me + m[j]) { s_result = at + j; break; }
              at_me += m[j];
            }
          }
          break;
        }
        run += chunk;
      }
    }
    __syncthreads();
    if (tid == 0) {
      p.out_tokens[row] = s_result;
      if (rec) { rec[7] = s_result; rec[1] += 1; }
      tl_mark(3, 4);
    }
  }
  cluster_sync_all();                    // nobody leaves while its sums may still be read
}

// As many blocks per row (a power of two, at most kSampleCluster) as keep all rows' blocks on the GPU at
// once (a block of 1,024 threads has an SM to itself); few blocks for a short row.
static int launch_sample(const SampleParams& p, int n_rows, cudaStream_t stream) {
  if (n_rows > 65535 || p.vocab > (1 << 21)) return (int)cudaErrorInvalidValue;    // (the pieces of the first histograms)
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
  int blocks = kSampleCluster;
  while (blocks > 1 && (n_rows * blocks > sms || p.vocab < blocks * 4096)) blocks >>= 1;
  return (int)launch_cluster(sample_kernel, dim3(blocks, n_rows), dim3(kSampleThreads), 0, stream, dim3(blocks, 1, 1), p);
}

}  // namespace tk

TK_TIMELINE_SETTER(sampling)

TK_API int tk_sample(const float* logits, long long ld, const float* temperature, const int* top_k,
                     const float* top_p, const unsigned long long* seed, const unsigned int* counter,
                     int* out_tokens, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab < 1) return (int)cudaErrorInvalidValue;
  tk::SampleParams p;
  p.logits = logits; p.temperature = temperature; p.top_k = top_k; p.top_p = top_p;
  p.seed = seed; p.counter = counter; p.out_tokens = out_tokens; p.vocab = vocab; p.ld = ld;
  p.records = nullptr; p.row_slot = nullptr; p.max_slots = 0; p.err = nullptr;
  return tk::launch_sample(p, n_rows, stream);
}

// The same with every row's parameters in the state record of its request's slot; the sampled
// token goes to out_tokens[row] and into the record, whose counter moves on by one.
TK_API int tk_sample_slots(const float* logits, long long ld, int* records, const int* row_slot, int max_slots,
                           int* out_tokens, int n_rows, int vocab, int* err, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab < 1 || records == nullptr || row_slot == nullptr) return (int)cudaErrorInvalidValue;
  tk::SampleParams p = {};
  p.logits = logits; p.out_tokens = out_tokens; p.vocab = vocab; p.ld = ld;
  p.records = records; p.row_slot = row_slot; p.max_slots = max_slots; p.err = err;
  return tk::launch_sample(p, n_rows, stream);
}

// Host copy of the generator, for callers that need the same uniform without a GPU.
TK_API void tk_philox_u32(unsigned long long seed, unsigned int counter, unsigned int* out4) {
  tk::philox4x32_10(counter, 0u, 0u, 0u, (unsigned int)seed, (unsigned int)(seed >> 32), out4);
}
