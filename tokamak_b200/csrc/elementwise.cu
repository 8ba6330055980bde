// Embedding lookup, residual add + RMSNorm, and the SwiGLU gate.
//
// The residual stream is float32 in every engine dtype, so the residual sum is
// always a 32-bit sum; the normalised output is rounded once to the activation
// type.  RMSNorm statistics are 32-bit as in the reference
// (src/tokamak/model/layers.py:28-33).
#include "common.cuh"
#include "timeline.cuh"

namespace tk {

// resid[t, :] = float(table[ids[t], :])                 (src/tokamak/model/transformer.py:140)
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ resid, int hidden, int vocab, int* err) {
  pdl_trigger();
  if (threadIdx.x == 0) tl_mark(4, 0);
  pdl_wait();
  if (threadIdx.x == 0) tl_mark(4, 1);
  const int t = blockIdx.x;
  const int id = ids[t];
  float* out = resid + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) set_error(err, kErrTokenId, t, id, vocab);
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) out[h] = 0.0f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) out[h] = to_f32<T>(row[h]);
}

// x = resid[r] (+ delta[r]);  resid[r] = x (when written back);
// out[i] = weight * x * rsqrt(mean(x^2) + eps)
// rows == nullptr: r = i = blockIdx.x and the sum is written back to resid.
// rows != nullptr: r = rows[i]; resid is left untouched (used for the final norm
// over the positions whose logits are wanted).
template <typename TOut, typename TDelta>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TDelta* __restrict__ delta,
                                   const float* __restrict__ parts, int n_parts, size_t part_stride,
                                   const float* __restrict__ weight, TOut* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  const TDelta* d = delta ? delta + (size_t)r * hidden : nullptr;
  const float* ps = parts ? parts + (size_t)r * hidden : nullptr;
  const bool has_delta = (d != nullptr) || (ps != nullptr);
  const bool write_back = (rows == nullptr) && has_delta;
  auto branch = [&](int h) -> float {
    if (d) return to_f32<TDelta>(d[h]);
    float acc = 0.0f;
    for (int s = 0; s < n_parts; ++s) acc += ps[(size_t)s * part_stride + h];
    return acc;
  };
  float ss = 0.0f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float v = x[h];
    if (has_delta) v += branch(h);
    if (write_back) x[h] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  TOut* o = out + (size_t)i * hidden;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float v;
    if (write_back || !has_delta) {
      v = x[h];
    } else {
      v = x[h] + branch(h);
    }
    o[h] = from_f32<TOut>(v * rstd * weight[h]);
  }
}

// Same operation for widths that are a multiple of 8: every thread keeps its values in
// registers between the sum of squares and the scaling, so the row is read once, with
// 16- and 32-byte accesses.
template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <typename T, int ITERS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ parts, int n_parts, size_t part_stride,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  const T* d = delta ? delta + (size_t)r * hidden : nullptr;
  const float* ps = parts ? parts + (size_t)r * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr || ps != nullptr);
  float v[ITERS][8];
  float ss = 0.0f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int h = (it * blockDim.x + threadIdx.x) * 8;
    if (h < hidden) {
      Vec8<float>::load(x + h, v[it]);
      if (d) {
        float dv[8];
        Vec8<T>::load(d + h, dv);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[it][e] += dv[e];
      } else if (ps) {
        for (int s = 0; s < n_parts; ++s) {
          float dv[8];
          Vec8<float>::load(ps + (size_t)s * part_stride + h, dv);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[it][e] += dv[e];
        }
      }
      if (write_back) Vec8<float>::store(x + h, v[it]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[it][e] * v[it][e];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int h = (it * blockDim.x + threadIdx.x) * 8;
    if (h < hidden) {
      float w[8], y[8];
      Vec8<float>::load(weight + h, w);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[it][e] * rstd * w[e];
      Vec8<T>::store(o + h, y);
    }
  }
}

// out[t, j] = silu(gate[t, j]) * up[t, j]           (src/tokamak/model/layers.py:103)
// A row of gu holds gate and up alternating in blocks: `block` gate values, then the `block` up
// values of the same outputs (block = inter: all gate values, then all up values).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, const float* __restrict__ parts, int n_parts,
                              size_t part_stride, T* __restrict__ out, int inter, int block, size_t total) {
  pdl_trigger();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const size_t at = t * 2 * inter + (size_t)(j / block) * 2 * block + (j % block);
    float g, u;
    if (parts == nullptr) {
      g = to_f32<T>(gu[at]);
      u = to_f32<T>(gu[at + block]);
    } else {
      g = 0.0f; u = 0.0f;
      for (int s = 0; s < n_parts; ++s) {
        g += parts[s * part_stride + at];
        u += parts[s * part_stride + at + block];
      }
    }
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_f32<T>(s * u);
  }
}

// The same for an intermediate size and a block that are multiples of 8: 16-byte loads and stores.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, const float* __restrict__ parts, int n_parts,
                                  size_t part_stride, T* __restrict__ out, int inter, int block, size_t total8) {
  pdl_trigger();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const int per_row = inter / 8;
  for (; idx < total8; idx += stride) {
    const size_t t = idx / per_row;
    const int j = (int)(idx - t * per_row) * 8;
    const size_t at = t * 2 * inter + (size_t)(j / block) * 2 * block + (j % block);
    float g[8], u[8], y[8];
    if (parts == nullptr) {
      Vec8<T>::load(gu + at, g);
      Vec8<T>::load(gu + at + block, u);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) { g[e] = 0.0f; u[e] = 0.0f; }
      for (int s = 0; s < n_parts; ++s) {
        float a[8], b[8];
        Vec8<float>::load(parts + s * part_stride + at, a);
        Vec8<float>::load(parts + s * part_stride + at + block, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) { g[e] += a[e]; u[e] += b[e]; }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = g[e] / (1.0f + expf(-g[e])) * u[e];
    Vec8<T>::store(out + t * inter + j, y);
  }
}

}  // namespace tk

TK_TIMELINE_SETTER(elementwise)

TK_API int tk_embed_gather(const void* table, int dtype, const int* ids, float* resid, int n_tokens,
                           int hidden, int vocab, int* err, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::embed_gather_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream,
                                       (const T*)table, ids, resid, hidden, vocab, err));
  return (int)e;
}

// delta: branch output in the activation type, or null.  parts: float32 partial sums of the
// branch output [n_parts, rows of resid, hidden] (part_stride elements apart), or null.
TK_API int tk_add_rmsnorm(float* resid, const void* delta, const float* parts, int n_parts,
                          long long part_stride, const float* weight, void* out, const int* rows,
                          int n_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (parts != nullptr && (delta != nullptr || n_parts < 1)) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  if (hidden % 8 == 0 && hidden <= 4 * 512 * 8) {
    // one pass with the row in registers: threads * 8 * ITERS >= hidden
    int threads = ((hidden / 8 + 31) / 32) * 32;
    int iters = 1;
    if (threads > 512) { iters = (hidden / 8 + 511) / 512; threads = 512; }
    if (threads > 256 && iters == 1 && n_rows >= 64) { threads = (threads / 2 + 31) / 32 * 32; iters = 2; }
    if (iters == 3) iters = 4;
#define TK_LAUNCH_VEC(IT)                                                                       \
    TK_DISPATCH_DTYPE(dtype, T,                                                                 \
                      (e = tk::launch(tk::add_rmsnorm_vec_kernel<T, IT>, dim3(n_rows), dim3(threads), 0, \
                                      stream, resid, (const T*)delta, parts, n_parts,             \
                                      (size_t)part_stride, weight, (T*)out, rows, hidden, eps)))
    if (iters == 1) { TK_LAUNCH_VEC(1); } else if (iters == 2) { TK_LAUNCH_VEC(2); } else { TK_LAUNCH_VEC(4); }
#undef TK_LAUNCH_VEC
    return (int)e;
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  TK_DISPATCH_DTYPE(dtype, T,
                    (e = tk::launch(tk::add_rmsnorm_kernel<T, T>, dim3(n_rows), dim3(threads), 0, stream,
                                    resid, (const T*)delta, parts, n_parts, (size_t)part_stride, weight,
                                    (T*)out, rows, hidden, eps)));
  return (int)e;
}

TK_API int tk_swiglu(const void* gate_up, const float* parts, int n_parts, long long part_stride,
                     void* out, int n_tokens, int inter, int block, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (block <= 0 || inter % block != 0) return (int)cudaErrorInvalidValue;
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  cudaError_t e = cudaSuccess;
  if (inter % 8 == 0 && block % 8 == 0) {
    const size_t total8 = total / 8;
    size_t vblocks = (total8 + threads - 1) / threads;
    if (vblocks > 148 * 32) vblocks = 148 * 32;
    TK_DISPATCH_DTYPE(dtype, T,
                      e = tk::launch(tk::swiglu_vec_kernel<T>, dim3((unsigned)vblocks), dim3(threads), 0, stream,
                                     (const T*)gate_up, parts, n_parts, (size_t)part_stride, (T*)out, inter,
                                     block, total8));
    return (int)e;
  }
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::swiglu_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                                   (const T*)gate_up, parts, n_parts, (size_t)part_stride, (T*)out, inter,
                                   block, total));
  return (int)e;
}
