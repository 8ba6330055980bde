// Token sampling over float32 logits, one thread block per row.
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

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(SampleParams p) {
  pdl_trigger();
  if (threadIdx.x == 0) tl_mark(3, 0);
  pdl_wait();
  if (threadIdx.x == 0) tl_mark(3, 1);
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ unsigned int s_count[256];
  __shared__ unsigned long long s_mass[256];
  __shared__ unsigned long long s_warp_tot[32];
  __shared__ unsigned int s_sel_key;
  __shared__ unsigned long long s_sel_rem;
  __shared__ int s_result;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int V = p.vocab;
  const float* lg = p.logits + (size_t)row * p.ld;
  int* rec = nullptr;
  if (p.records != nullptr) {
    const int slot = p.row_slot[row];
    if (slot < 0 || slot >= p.max_slots) {
      if (tid == 0) { set_error(p.err, kErrRequest, row, slot, p.max_slots); p.out_tokens[row] = 0; }
      return;
    }
    rec = p.records + (size_t)slot * kSlotWords;
  }
  const float T = rec ? __int_as_float(rec[4]) : p.temperature[row];

  // ---- pass 1: maximum and its lowest index ------------------------------------------
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  // (16-byte loads, four of them in flight per thread, where the row starts on a 16-byte boundary:
  // one block reads the whole row, and with 4-byte loads one after the other a row of 151,936
  // logits took 14 us)
  const bool vec = (reinterpret_cast<uintptr_t>(lg) & 15u) == 0;
  const int V4 = vec ? (V >> 2) : 0;
  {
    const float4* lg4 = reinterpret_cast<const float4*>(lg);
    int i = tid;
    for (; i + 3 * kSampleThreads < V4; i += 4 * kSampleThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = lg4[i + u * kSampleThreads];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int at = (i + u * kSampleThreads) * 4;     // ascending within the thread: the first maximum is kept
        if (v[u].x > best) { best = v[u].x; best_i = at; }
        if (v[u].y > best) { best = v[u].y; best_i = at + 1; }
        if (v[u].z > best) { best = v[u].z; best_i = at + 2; }
        if (v[u].w > best) { best = v[u].w; best_i = at + 3; }
      }
    }
    for (; i < V4; i += kSampleThreads) {
      const float4 v = lg4[i];
      const int at = i * 4;
      if (v.x > best) { best = v.x; best_i = at; }
      if (v.y > best) { best = v.y; best_i = at + 1; }
      if (v.z > best) { best = v.z; best_i = at + 2; }
      if (v.w > best) { best = v.w; best_i = at + 3; }
    }
  }
  for (int i = V4 * 4 + tid; i < V; i += kSampleThreads) {
    const float v = lg[i];
    if (v > best) { best = v; best_i = i; }   // ascending i: the first maximum is kept
  }
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
  __syncthreads();
  const float max_logit = s_val[0];
  if (T == 0.0f) {
    if (tid == 0) {
      p.out_tokens[row] = s_idx[0];
      if (rec) { rec[7] = s_idx[0]; rec[1] += 1; }
      tl_mark(3, 4);
    }
    return;
  }
  const float zmax = max_logit / T;

  // ---- thresholds: radix descent over the order-preserving key of z = logit / T -------
  unsigned int thr_key = 0u;   // keep keys >= thr_key
  const int k = rec ? rec[5] : p.top_k[row];
  const float top_p = rec ? __int_as_float(rec[6]) : p.top_p[row];
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
      __syncthreads();
      for (int i = tid; i < V; i += kSampleThreads) {
        const float z = lg[i] / T;
        const unsigned int key = float_key(z);
        if (key < thr_key || (key & prefix_mask) != prefix) continue;
        const unsigned int b = (key >> shift) & 0xffu;
        if (phase == 0) {
          atomicAdd(&s_count[b], 1u);
        } else {
          const unsigned long long fx = __float2ull_rd(expf(z - zmax) * kMassScale);
          atomicAdd(&s_mass[b], fx);
        }
      }
      __syncthreads();
      if (tid == 0) {
        if (phase == 1 && level == 0) {
          unsigned long long total = 0ull;
          for (int b = 0; b < 256; ++b) total += s_mass[b];
          unsigned long long target = (unsigned long long)((double)top_p * (double)total);
          if (target > total) target = total;
          if (target == 0ull) target = 1ull;
          remaining = target;
        }
        unsigned long long cum = 0ull;
        int chosen = 0;
        for (int b = 255; b >= 0; --b) {
          const unsigned long long w = (phase == 0) ? (unsigned long long)s_count[b] : s_mass[b];
          if (cum + w >= remaining && w > 0ull) { chosen = b; break; }
          cum += w;
          if (b == 0) chosen = 0;
        }
        s_sel_key = (unsigned int)chosen;
        s_sel_rem = remaining - cum;
      }
      __syncthreads();
      prefix |= s_sel_key << shift;
      prefix_mask |= 0xffu << shift;
      remaining = s_sel_rem;
      __syncthreads();
    }
    if (prefix > thr_key) thr_key = prefix;
  }

  // ---- total kept mass ------------------------------------------------------------------
  unsigned long long local = 0ull;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float z = lg[i] / T;
    if (float_key(z) >= thr_key) local += __float2ull_rd(expf(z - zmax) * kMassScale);
  }
  {
    unsigned long long w = local;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    __syncthreads();
    if (lane == 0) s_warp_tot[warp] = w;
    __syncthreads();
  }
  unsigned long long total = 0ull;
  for (int w = 0; w < kSampleThreads / 32; ++w) total += s_warp_tot[w];

  // ---- the draw: first index whose inclusive prefix exceeds u * total -------------------
  unsigned int rnd[4];
  const unsigned long long seed =
      rec ? ((unsigned long long)(unsigned int)rec[3] << 32) | (unsigned int)rec[2] : p.seed[row];
  const unsigned int counter = rec ? (unsigned int)rec[1] : p.counter[row];
  philox4x32_10(counter, 0u, 0u, 0u, (unsigned int)seed, (unsigned int)(seed >> 32), rnd);
  // target = floor(rnd / 2^32 * total) < total
  const unsigned long long target = __umul64hi(total, (unsigned long long)rnd[0] << 32);

  if (tid == 0) s_result = best_i >= 0 ? s_idx[0] : 0;   // fallback: the most likely token
  __syncthreads();
  constexpr int kItems = 4;
  unsigned long long base = 0ull;
  bool done = false;
  for (int start = 0; start < V && !done; start += kSampleThreads * kItems) {
    unsigned long long item[kItems];
    unsigned long long mine = 0ull;
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      const int i = start + tid * kItems + j;
      unsigned long long fx = 0ull;
      if (i < V) {
        const float z = lg[i] / T;
        if (float_key(z) >= thr_key) fx = __float2ull_rd(expf(z - zmax) * kMassScale);
      }
      item[j] = fx;
      mine += fx;
    }
    const unsigned long long incl = warp_incl_scan_u64(mine, lane);
    __syncthreads();
    if (lane == 31) s_warp_tot[warp] = incl;
    __syncthreads();
    unsigned long long warp_base = 0ull, chunk_total = 0ull;
    for (int w = 0; w < kSampleThreads / 32; ++w) {
      const unsigned long long tw = s_warp_tot[w];
      if (w < warp) warp_base += tw;
      chunk_total += tw;
    }
    if (base + chunk_total > target) {
      unsigned long long run = base + warp_base + incl - mine;   // exclusive prefix of this thread
      if (run <= target && target < run + mine) {
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          if (target < run + item[j]) { s_result = start + tid * kItems + j; break; }
          run += item[j];
        }
      }
      done = true;
    }
    base += chunk_total;
  }
  __syncthreads();
  if (tid == 0) {
    p.out_tokens[row] = s_result;
    if (rec) { rec[7] = s_result; rec[1] += 1; }
    tl_mark(3, 4);
  }
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
  return (int)tk::launch(tk::sample_kernel, dim3(n_rows), dim3(tk::kSampleThreads), 0, stream, p);
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
  return (int)tk::launch(tk::sample_kernel, dim3(n_rows), dim3(tk::kSampleThreads), 0, stream, p);
}

// Host copy of the generator, for callers that need the same uniform without a GPU.
TK_API void tk_philox_u32(unsigned long long seed, unsigned int counter, unsigned int* out4) {
  tk::philox4x32_10(counter, 0u, 0u, 0u, (unsigned int)seed, (unsigned int)(seed >> 32), out4);
}
