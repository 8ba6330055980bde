// Optional time stamps from inside the kernels, compiled in with -DTK_TIMELINE (set
// TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE before the library is built; off by default, and then
// every mark below is nothing at all).
//
// Kernels of a decode step overlap under programmatic dependent launch, so neither a profiler
// that serialises launches nor CUDA events around single kernels show where a step's time goes.
// With the marks, chosen threads of a block write (global timer, kernel, phase, SM, block) records
// into a buffer that the host hands over with tk_timeline_set_<file>; the host reads them back
// and lays the blocks of all kernels out on one time axis.
#pragma once

#include "common.cuh"

#ifdef TK_TIMELINE
namespace tk {

struct TimelineBuf {
  unsigned long long* buf;   // [1 + 2 * cap]: count, then (time in ns, packed record) pairs
  unsigned int cap;
};
static __device__ TimelineBuf g_timeline = {nullptr, 0u};

__device__ __forceinline__ void tl_mark(int kernel, int phase) {
  const TimelineBuf tl = g_timeline;
  if (tl.buf == nullptr) return;
  unsigned long long t;
  unsigned int sm;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  asm volatile("mov.u32 %0, %%smid;\n" : "=r"(sm));
  const unsigned long long i = atomicAdd(tl.buf, 1ull);
  if (i < tl.cap) {
    const unsigned long long block =
        (unsigned long long)blockIdx.x + gridDim.x * ((unsigned long long)blockIdx.y + gridDim.y * blockIdx.z);
    tl.buf[1 + 2 * i] = t;
    tl.buf[2 + 2 * i] = ((unsigned long long)(kernel & 0xFF) << 56) | ((unsigned long long)(phase & 0xFF) << 48) |
                        ((unsigned long long)(sm & 0xFFFF) << 32) | (block & 0xFFFFFFFFull);
  }
}

// A record that carries a number (e.g. nanoseconds spent waiting) in place of the block index.
__device__ __forceinline__ void tl_value(int kernel, int phase, unsigned int value) {
  const TimelineBuf tl = g_timeline;
  if (tl.buf == nullptr) return;
  unsigned long long t;
  unsigned int sm;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  asm volatile("mov.u32 %0, %%smid;\n" : "=r"(sm));
  const unsigned long long i = atomicAdd(tl.buf, 1ull);
  if (i < tl.cap) {
    tl.buf[1 + 2 * i] = t;
    tl.buf[2 + 2 * i] = ((unsigned long long)(kernel & 0xFF) << 56) | ((unsigned long long)(phase & 0xFF) << 48) |
                        ((unsigned long long)(sm & 0xFFFF) << 32) | (unsigned long long)value;
  }
}
__device__ __forceinline__ unsigned long long tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// A cheap mark for one chosen thread: no atomic, the thread counts its own records (`count`) in
// its own range of 1,024 records at the end of the buffer (`lane` picks the range).  The host sets the buffer's count to
// its capacity before it reads, and skips the empty records.
__device__ __forceinline__ void tl_own(int lane, unsigned int& count, int kernel, int phase, unsigned int value) {
  const TimelineBuf tl = g_timeline;
  if (tl.buf == nullptr || count >= 1024u) return;
  if (tl.cap < 1024u * (unsigned)(lane + 1)) return;
  const unsigned long long i = tl.cap - 1024ull * (unsigned)(lane + 1) + count++;     // from the buffer's end
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  tl.buf[1 + 2 * i] = t;
  tl.buf[2 + 2 * i] = ((unsigned long long)(kernel & 0xFF) << 56) | ((unsigned long long)(phase & 0xFF) << 48) |
                      (unsigned long long)value;
}

}  // namespace tk

#define TK_TIMELINE_SETTER(name)                                                        \
  TK_API int tk_timeline_set_##name(unsigned long long* buf, unsigned int cap) {        \
    tk::TimelineBuf h{buf, cap};                                                        \
    return (int)cudaMemcpyToSymbol(tk::g_timeline, &h, sizeof(h));                      \
  }
#else
namespace tk {
__device__ __forceinline__ void tl_mark(int, int) {}
__device__ __forceinline__ void tl_value(int, int, unsigned int) {}
__device__ __forceinline__ unsigned long long tl_now() { return 0ull; }
__device__ __forceinline__ void tl_own(int, unsigned int&, int, int, unsigned int) {}
}
#define TK_TIMELINE_SETTER(name)
#endif
