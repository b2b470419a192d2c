// Self-test of the bounded-wait discipline: a kernel spins on a flag that nothing sets and must give up
// after `limit_cycles`, record kStatusPeerFlagTimeout and return, leaving the context usable.
#include "../common/launch_count.h"
#include "../common/ptx.cuh"

namespace eredu {

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void bounded_wait_selftest_kernel(int* status, int* flag, long long limit_cycles) {
  const long long t0 = clock64();
  while (ld_acquire_sys(flag) != 1) {
    if (clock64() - t0 > limit_cycles) {
      report_status(status, kStatusPeerFlagTimeout);
      return;
    }
  }
}

}  // namespace eredu

// `status` must be a zeroed device int; the flag waited on is status[0]'s neighbour is not used: the kernel
// waits on a private zero word (`status` itself is only written on give-up, with a value != 1 ... so the wait
// can only end by the limit).
extern "C" int eredu_selftest_bounded_wait(int* status, long long limit_cycles, cudaStream_t stream) {
  static int* flag = nullptr;
  if (flag == nullptr) {
    if (cudaMalloc(&flag, sizeof(int)) != cudaSuccess) return -1;
    cudaMemset(flag, 0, sizeof(int));
  }
  eredu::bounded_wait_selftest_kernel<<<1, 1, 0, stream>>>(status, flag, limit_cycles);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
