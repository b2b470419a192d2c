// Device-side timeline trace: when a trace buffer is installed, thread 0 of block (0,0,0) of every instrumented
// kernel records (globaltimer ns, kernel id, phase) at its first instruction, after its stream-dependency wait and
// at its end. Inside a CUDA graph this is the only way to see how kernels overlap under programmatic dependent
// launch; with no buffer installed a mark is one predictable branch on a cached word.
//
// The control block is a per-translation-unit static (the library is built without relocatable device code), so
// every .cu file that uses trace_mark() instantiates its own installer with EREDU_TRACE_INSTALLER(name); the host
// tracer (utils/trace.py) calls all of them. Plays the role of the reference's device timing hooks
// (doc/device-timing.md; safemlx/src/transforms async_eval timed variants).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace eredu {

struct TraceCtl {
  unsigned long long* buf;  // [cap][2]: {time ns, (kernel id << 8) | phase}
  unsigned int* count;
  unsigned int cap;
};

enum TraceKernel : unsigned int {
  kTraceGemm = 1, kTraceGemmPersistent = 2, kTraceQGemm = 3, kTraceAttnDecode = 4, kTraceAttnPrefill = 5,
  kTraceRope = 6, kTraceRmsNorm = 7, kTraceEmbedding = 8, kTraceSampler = 9, kTraceAdvance = 10, kTraceMoe = 11,
  kTraceSiluMul = 12, kTraceComm = 13,
};
enum TracePhase : unsigned int { kTraceStart = 0, kTraceAfterWait = 1, kTraceEnd = 2 };

static __constant__ TraceCtl g_trace_ctl;  // constant bank: a disabled mark costs one cached constant load

__device__ __forceinline__ void trace_mark(unsigned int kernel, unsigned int phase) {
  if (g_trace_ctl.buf == nullptr) return;
  if ((threadIdx.x | threadIdx.y | blockIdx.x | blockIdx.y | blockIdx.z) != 0u) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned int i = atomicAdd(g_trace_ctl.count, 1u);
  if (i < g_trace_ctl.cap) {
    g_trace_ctl.buf[2 * i] = t;
    g_trace_ctl.buf[2 * i + 1] = (static_cast<unsigned long long>(kernel) << 8) | phase;
  }
}

// Same, from a chosen thread of block (0,0,0) (pipeline roles live in different warps); phases >= 3 are
// kernel-specific sub-steps.
__device__ __forceinline__ void trace_mark_thread(unsigned int kernel, unsigned int phase, unsigned int tid) {
#ifndef EREDU_TRACE_FINE
  (void)kernel;
  (void)phase;
  (void)tid;
  return;  // sub-step marks sit on the pipeline's critical path: compiled in only for -DEREDU_TRACE_FINE builds
#endif
  if (g_trace_ctl.buf == nullptr) return;
  if (threadIdx.x != tid || (blockIdx.x | blockIdx.y | blockIdx.z) != 0u) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned int i = atomicAdd(g_trace_ctl.count, 1u);
  if (i < g_trace_ctl.cap) {
    g_trace_ctl.buf[2 * i] = t;
    g_trace_ctl.buf[2 * i + 1] = (static_cast<unsigned long long>(kernel) << 8) | phase;
  }
}

}  // namespace eredu

#define EREDU_TRACE_INSTALLER(name)                                                                              \
  extern "C" int eredu_trace_install_##name(unsigned long long* buf, unsigned int* count, unsigned int cap) {     \
    eredu::TraceCtl c{buf, count, cap};                                                                          \
    return static_cast<int>(cudaMemcpyToSymbol(eredu::g_trace_ctl, &c, sizeof(c)));                              \
  }
