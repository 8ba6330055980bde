// Embedding lookup, residual add + RMSNorm, and the SwiGLU gate.
//
// The residual stream is float32 in every engine dtype, so the residual sum is
// always a 32-bit sum; the normalised output is rounded once to the activation
// type.  RMSNorm statistics are 32-bit as in the reference
// (src/tokamak/model/layers.py:28-33).
#include "common.cuh"

namespace tk {

// resid[t, :] = float(table[ids[t], :])                 (src/tokamak/model/transformer.py:140)
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ resid, int hidden, int vocab, int* err) {
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
                                   const float* __restrict__ weight, TOut* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  const TDelta* d = delta ? delta + (size_t)r * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  float ss = 0.0f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float v = x[h];
    if (d) v += to_f32<TDelta>(d[h]);
    if (write_back) x[h] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  TOut* o = out + (size_t)i * hidden;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float v;
    if (write_back || d == nullptr) {
      v = x[h];
    } else {
      v = x[h] + to_f32<TDelta>(d[h]);
    }
    o[h] = from_f32<TOut>(v * rstd * weight[h]);
  }
}

// out[t, j] = silu(gu[t, j]) * gu[t, inter + j]           (src/tokamak/model/layers.py:103)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const float g = to_f32<T>(gu[t * 2 * inter + j]);
    const float u = to_f32<T>(gu[t * 2 * inter + inter + j]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_f32<T>(s * u);
  }
}

}  // namespace tk

TK_API int tk_embed_gather(const void* table, int dtype, const int* ids, float* resid, int n_tokens,
                           int hidden, int vocab, int* err, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  TK_DISPATCH_DTYPE(dtype, T,
                    tk::embed_gather_kernel<T><<<n_tokens, threads, 0, stream>>>(
                        (const T*)table, ids, resid, hidden, vocab, err));
  return (int)cudaGetLastError();
}

TK_API int tk_add_rmsnorm(float* resid, const void* delta, const float* weight, void* out,
                          const int* rows, int n_rows, int hidden, float eps, int dtype,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  TK_DISPATCH_DTYPE(dtype, T,
                    (tk::add_rmsnorm_kernel<T, T><<<n_rows, threads, 0, stream>>>(
                        resid, (const T*)delta, weight, (T*)out, rows, hidden, eps)));
  return (int)cudaGetLastError();
}

TK_API int tk_swiglu(const void* gate_up, void* out, int n_tokens, int inter, int dtype,
                     cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  TK_DISPATCH_DTYPE(dtype, T,
                    tk::swiglu_kernel<T><<<(int)blocks, threads, 0, stream>>>(
                        (const T*)gate_up, (T*)out, inter, total));
  return (int)cudaGetLastError();
}
