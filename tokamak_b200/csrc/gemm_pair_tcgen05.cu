// bfloat16 matrix product for many tokens on pairs of SMs (tcgen05.mma.cta_group::2):
//   D[t, n] = sum_k X[t, k] * W[n, k]      (both operands K-major, float32 accumulation)
//
// The grid is persistent: thread-block clusters of two blocks walk the 256 x 256 output tiles,
// token tiles fastest, so that the pairs that run at the same time share weight tiles in L2.
// Of a tile's operands each block of the pair loads its own half by TMA (128 token rows and
// 128 weight rows of 64 k-elements per stage, 128-byte swizzle, every block for itself) into its own
// shared memory; both halves complete on the full-barrier of the pair's first block, whose
// single issuing thread runs tcgen05.mma with M = 256, N = 256 over both blocks' shared memory.
// Each block ends up with the 128 x 256 float32 accumulator of its own token rows in its own
// tensor memory.  Half as many operand bytes per SM cross the L2 as with one block per tile,
// which is what a 128 x 256 tile on one SM is short of.
//
// Tensor memory holds two accumulators: the four epilogue warps of both blocks read one
// (tcgen05.ld) and store the result while the next tile is multiplied into the other.
//
// Epilogues: bfloat16 output [tokens, n]; or, for a stacked gate/up weight whose rows alternate
// in blocks of 64 (64 gate rows, then the 64 up rows of the same outputs),
// bf16(silu(gate) * up) as [tokens, n / 2]: the activation costs no pass over memory
// (src/tokamak/model/layers.py:103).
//
// tcgen05.commit with cluster multicast gives a stage back to both blocks; every wait on an
// mbarrier is bounded, reports kErrWait and lets the block leave through the common exit, which
// meets the other block at a cluster barrier before tensor memory is freed.
#include "tcgen05_utils.cuh"

namespace tk {

constexpr int kGpBM = 128;          // token rows per block; the pair's tile has 256
constexpr int kGpBNHalf = 128;      // weight rows per block; the pair's tile has 256
constexpr int kGpBN = 256;
constexpr int kGpBK = 64;
constexpr int kGpStages = 6;
constexpr int kGpThreads = 192;     // warp 0: TMA, warp 1: MMA (first block only), warps 2..5: epilogue
constexpr uint32_t kGpStageBytes = (kGpBM + kGpBNHalf) * kGpBK * 2;
constexpr uint32_t kGpPeerMask = 0xFEFFFFFFu;   // clears the bit that tells the pair's blocks apart in a
                                                // shared::cluster address: the first block's barrier

struct GemmPairParams {
  void* out;
  int* err;
  int rows, cols, k;
  long long ld_out;
  int mode;                 // 0: bf16 [rows, cols]; 1: gated activation, bf16 [rows, cols / 2]
};

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar & kGpPeerMask)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in both blocks of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_first_block(uint32_t local_bar) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_bar), "r"(0u));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(remote) : "memory");
}

__global__ void __launch_bounds__(kGpThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 GemmPairParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t raw = gt_smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;         // the same offset in both blocks
  unsigned char* smem = smem_raw + (base - raw);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kGpStages * kGpStageBytes);
  uint64_t* empty_bar = full_bar + kGpStages;
  uint64_t* acc_full = empty_bar + kGpStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int n_tm = (p.rows + 2 * kGpBM - 1) / (2 * kGpBM);
  const int n_tn = (p.cols + kGpBN - 1) / kGpBN;
  const int n_tiles = n_tm * n_tn;
  const int n_kb = (p.k + kGpBK - 1) / kGpBK;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGpStages; ++s) {
      mbar_init(gt_smem_u32(&full_bar[s]), 1);
      mbar_init(gt_smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(gt_smem_u32(&acc_full[b]), 1);
      mbar_init(gt_smem_u32(&acc_empty[b]), 8);       // four epilogue warps of each block
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(gt_smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // both blocks' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer of this block's halves ---------------------------------------------------
    if (lane == 0) {
      pdl_wait();                // the activations come from the kernel before this one
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        const int tm = tile % n_tm, tn = tile / n_tm;
        const int x_row = tm * 2 * kGpBM + (int)rank * kGpBM;
        const int w_row = tn * kGpBN + (int)rank * kGpBNHalf;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const uint32_t s = it % kGpStages, round = it / kGpStages;
          if (round > 0 && !mbar_wait(gt_smem_u32(&empty_bar[s]), (round - 1) & 1u, abort_flag)) {
            set_error(p.err, kErrWait, 20, (int)it, (int)s);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = gt_smem_u32(&full_bar[s]);
          if (rank == 0) mbar_expect_tx(full, 2 * kGpStageBytes);     // both blocks' halves land here
          const uint32_t dst = base + s * kGpStageBytes;
          tma_load_2d_pair(dst, &map_x, kb * kGpBK, x_row, full);
          tma_load_2d_pair(dst + kGpBM * kGpBK * 2, &map_w, kb * kGpBK, w_row, full);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the pair's first block only --------------------------------------------------
    if (lane == 0 && rank == 0) {
      // bf16 x bf16 -> f32, K-major operands, M = 256 over the pair, N = 256
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kGpBN >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);
      uint32_t it = 0;
      int lt = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++lt) {
        const int b = lt & 1, use = lt >> 1;
        if (use > 0 && !mbar_wait(gt_smem_u32(&acc_empty[b]), (uint32_t)(use - 1) & 1u, abort_flag)) {
          set_error(p.err, kErrWait, 21, lt, b);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const uint32_t s = it % kGpStages, round = it / kGpStages;
          if (!mbar_wait(gt_smem_u32(&full_bar[s]), round & 1u, abort_flag)) {
            set_error(p.err, kErrWait, 22, (int)it, (int)s);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = base + s * kGpStageBytes;
          const uint64_t desc_a = umma_desc_sw128(a_addr);
          const uint64_t desc_b = umma_desc_sw128(a_addr + kGpBM * kGpBK * 2);
#pragma unroll
          for (int k = 0; k < kGpBK / 16; ++k) {
            umma_bf16_pair(tmem_base + (uint32_t)(b * kGpBN), desc_a + (uint64_t)(2 * k), desc_b + (uint64_t)(2 * k),
                           idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(gt_smem_u32(&empty_bar[s]));      // both blocks may refill the stage
        }
        if (ok) umma_commit_pair(gt_smem_u32(&acc_full[b]));  // both blocks may read their accumulator
      }
    }
  } else {
    // ---- epilogue: warps 2..5 of both blocks, each owning 32 accumulator lanes -----------------------
    const int quarter = warp & 3;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    int lt = 0;
    bool ok = true;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++lt) {
      const int tm = tile % n_tm, tn = tile / n_tm;
      const int b = lt & 1, use = lt >> 1;
      ok = __all_sync(0xffffffffu, mbar_wait(gt_smem_u32(&acc_full[b]), (uint32_t)use & 1u, abort_flag));
      if (!ok) {
        if (lane == 0) { set_error(p.err, kErrWait, 23, lt, b); *abort_flag = 1; }
        break;
      }
      tc_fence_after();
      const int row = tm * 2 * kGpBM + (int)rank * kGpBM + quarter * 32 + lane;
      const uint32_t tacc = tmem_base + lane_addr + (uint32_t)(b * kGpBN);
      if (p.mode == 1) {
        // columns [0, 64) and [128, 192) of the tile are gate values, [64, 128) and [192, 256) the up
        // values of the same outputs
        const int inter = p.cols >> 1;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.ld_out;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t g[32], u[32];
            tmem_ld32(tacc + (uint32_t)(blk * 128 + c0), g);
            tmem_ld32(tacc + (uint32_t)(blk * 128 + 64 + c0), u);
            tmem_wait_ld();
            const int oc = tn * (kGpBN / 2) + blk * 64 + c0;
            if (row < p.rows && oc < inter) {     // inter is a multiple of 64: the 32 outputs exist together
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 v;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float g0 = __uint_as_float(g[q * 8 + 2 * e]), g1 = __uint_as_float(g[q * 8 + 2 * e + 1]);
                  const float u0 = __uint_as_float(u[q * 8 + 2 * e]), u1 = __uint_as_float(u[q * 8 + 2 * e + 1]);
                  h2[e] = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
                }
                *reinterpret_cast<uint4*>(orow + oc + q * 8) = v;
              }
            }
          }
        }
      } else {
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.ld_out;
#pragma unroll 2
        for (int c0 = 0; c0 < kGpBN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tacc + (uint32_t)c0, v);
          tmem_wait_ld();
          const int col0 = tn * kGpBN + c0;
          if (row >= p.rows) continue;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = col0 + q * 8;
            if (col + 8 <= p.cols) {
              uint4 o;
              __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                h2[e] = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2 * e]), __uint_as_float(v[q * 8 + 2 * e + 1]));
              }
              *reinterpret_cast<uint4*>(orow + col) = o;
            } else {
              for (int e = 0; e < 8; ++e) {
                if (col + e < p.cols) orow[col + e] = __float2bfloat16_rn(__uint_as_float(v[q * 8 + e]));
              }
            }
          }
        }
      }
      // the accumulator has been read: the first block's issuer may multiply into it again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_first_block(gt_smem_u32(&acc_empty[b]));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither block leaves while the other may still reach into it
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

static int make_pair_map(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if (((uintptr_t)ptr & 15u) != 0 || (ld * 2) % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kGpBK, (cuuint32_t)kGpBM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace tk

// out = x * w^T on pairs of SMs.  x: [rows, k] bf16 (row stride ld_x), w: [cols, k] bf16 (row stride
// ld_w).  mode 0: out is bf16 [rows, cols]; mode 1 (cols a multiple of 128, gate and up rows of w
// alternating in blocks of 64): out is bf16 [rows, cols / 2] = silu(gate) * up.  ld_out: elements
// between output rows, a multiple of 8.
TK_API int tk_gemm_bf16_pair(const void* x, const void* w, void* out, int* err, int rows, int cols, int k,
                             long long ld_x, long long ld_w, long long ld_out, int mode, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (k <= 0 || k % 8 != 0 || ld_out % 8 != 0 || (mode != 0 && mode != 1) || (mode == 1 && cols % 128 != 0) ||
      ((uintptr_t)out & 15u) != 0) {
    return (int)cudaErrorInvalidValue;
  }
  CUtensorMap map_x, map_w;
  int rc = tk::make_pair_map(&map_x, x, rows, k, ld_x);
  if (rc != 0) return rc;
  rc = tk::make_pair_map(&map_w, w, cols, k, ld_w);
  if (rc != 0) return rc;
  const size_t smem_bytes = (size_t)tk::kGpStages * tk::kGpStageBytes + 1024 /* alignment */ + 256 /* barriers */;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(tk::gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148, 1, 1);
    cfg.blockDim = dim3(tk::kGpThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, tk::gemm_pair_kernel, &cfg);
    if (e != cudaSuccess) return (int)e;
    if (n < 1) return (int)cudaErrorLaunchOutOfResources;
    max_pairs = n;
  }
  const int n_tiles = ((rows + 255) / 256) * ((cols + 255) / 256);
  const int pairs = n_tiles < max_pairs ? n_tiles : max_pairs;
  tk::GemmPairParams p;
  p.out = out; p.err = err; p.rows = rows; p.cols = cols; p.k = k; p.ld_out = ld_out; p.mode = mode;
  // the two blocks of a pair are neighbours along x, as tcgen05's cta_group::2 wants them
  return (int)tk::launch_cluster(tk::gemm_pair_kernel, dim3(2 * pairs, 1, 1), dim3(tk::kGpThreads), smem_bytes, stream,
                                 dim3(2, 1, 1), map_x, map_w, p);
}
