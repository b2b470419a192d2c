// Symmetric peer memory over CUDA IPC, and the stand-alone collectives built on it:
//   * two-shot all-reduce (reduce-scatter by P2P loads + all-gather by P2P stores) for large activations,
//   * all-gather of row blocks,
//   * a cross-GPU barrier.
// They replace the reference's NCCL calls for the tensor/expert-parallel hot path (all_sum after row-parallel
// projections: eredu/src/backend/mlx/nn/parallel.rs:736-757,824-841; logits all_gather :1382-1409). Pipeline
// stage hand-off stays on NCCL p2p. Waits are bounded; nothing here uses TMA multicast.
#include <cuda_runtime.h>

#include <cstring>

#include "../common/launch_count.h"
#include "../common/peer.cuh"

namespace eredu {

// Every CTA synchronises with the same-index CTA of every peer (needs the same grid on all ranks and all
// CTAs resident). `slot` selects which flag row to use so that two barriers of one kernel do not alias.
__device__ __forceinline__ void cta_peer_barrier(const PeerComm& c, int parity, unsigned int seq, int slot, int* status) {
  __syncthreads();
  const int idx = (blockIdx.x * 2 + slot) % kMaxFlags;
  if (threadIdx.x < c.size) {
    __threadfence_system();
    st_release_sys(peer_flag(c, threadIdx.x, parity, c.rank, idx), seq + 1u);
    wait_flag(c, parity, threadIdx.x, idx, seq + 1u, status);
  }
  __syncthreads();
}

// x_off: byte offset (inside the symmetric buffer) of this call's input [M, N] bf16, identical on all ranks.
// Rank r reduces rows [r*M/size, (r+1)*M/size) (16-byte chunks), adds bias / residual, and stores the bf16
// result into every peer's `out` region (and optionally a local tensor y).
__global__ void __launch_bounds__(512) allreduce_twoshot_kernel(PeerComm c, long long x_off, const __nv_bfloat16* residual,
                                                                  const __nv_bfloat16* bias, __nv_bfloat16* y, int M, int N,
                                                                  int ldr, int* status) {
  const unsigned int seq = *c.seq;
  const int parity = static_cast<int>(seq & 1u);
  cta_peer_barrier(c, parity, seq, 0, status);  // every rank's partial is complete
  const int chunks_per_row = N >> 3;
  const long long total = static_cast<long long>(M) * chunks_per_row;
  const long long per = (total + c.size - 1) / c.size;
  const long long lo = per * c.rank, hi = min(total, lo + per);
  for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int src = 0; src < c.size; ++src) {
      const uint4 v = ld_cg_u4(c.base[src] + x_off + i * 16);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(u[j]);
        acc[2 * j + 1] += bf16_hi(u[j]);
      }
    }
    const long long m = i / chunks_per_row;
    const int n0 = static_cast<int>(i % chunks_per_row) * 8;
    if (bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(bias[n0 + j]);
    }
    if (residual != nullptr) {
      const uint4 rv = *reinterpret_cast<const uint4*>(residual + m * ldr + n0);
      const uint32_t u[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(u[j]);
        acc[2 * j + 1] += bf16_hi(u[j]);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    for (int peer = 0; peer < c.size; ++peer) *reinterpret_cast<uint4*>(c.base[peer] + c.out_off + i * 16) = o;
  }
  cta_peer_barrier(c, parity, seq, 1, status);  // every slice has landed everywhere
  if (y != nullptr) {
    const uint4* src = reinterpret_cast<const uint4*>(c.base[c.rank] + c.out_off);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      reinterpret_cast<uint4*>(y)[i] = ld_cg_u4(src + i);
  }
  if (threadIdx.x == 0) finish_call(c, seq, gridDim.x);
}

// Gather `bytes` (multiple of 16) from every rank's local `src` into every rank's out region at rank * bytes.
__global__ void __launch_bounds__(512) allgather_kernel(PeerComm c, const uint4* src, long long bytes, int* status) {
  const unsigned int seq = *c.seq;
  const int parity = static_cast<int>(seq & 1u);
  const long long n = bytes >> 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int peer = 0; peer < c.size; ++peer)
      *reinterpret_cast<uint4*>(c.base[peer] + c.out_off + c.rank * bytes + i * 16) = v;
  }
  cta_peer_barrier(c, parity, seq, 0, status);
  if (threadIdx.x == 0) finish_call(c, seq, gridDim.x);
}

__global__ void peer_barrier_kernel(PeerComm c, int* status) {
  const unsigned int seq = *c.seq;
  cta_peer_barrier(c, static_cast<int>(seq & 1u), seq, 0, status);
  if (threadIdx.x == 0) finish_call(c, seq, gridDim.x);
}

}  // namespace eredu

using namespace eredu;

extern "C" int eredu_peer_alloc(long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*out, 0, static_cast<size_t>(bytes)));
}
extern "C" int eredu_peer_free(void* p) { return static_cast<int>(cudaFree(p)); }
extern "C" int eredu_ipc_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
extern "C" int eredu_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  std::memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int eredu_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int eredu_ipc_close(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

// Build the host-side PeerComm. `bases[size]`: mapped base pointers in rank order (bases[rank] = own buffer);
// `local_words`: device pointer to 2 zeroed u32 (seq, done) that peers never touch.
extern "C" void* eredu_comm_create(void** bases, int rank, int size, long long slot_bytes, long long out_bytes,
                                   unsigned int* local_words) {
  if (size < 1 || size > kMaxRanks || rank < 0 || rank >= size) return nullptr;
  PeerComm* c = new PeerComm();
  for (int i = 0; i < kMaxRanks; ++i) c->base[i] = i < size ? static_cast<uint8_t*>(bases[i]) : nullptr;
  c->rank = rank;
  c->size = size;
  c->flags_off = 0;
  const long long flag_bytes = 2LL * kMaxRanks * kMaxFlags * 4;
  c->data_off = flag_bytes;
  c->slot_bytes = (slot_bytes + 255) / 256 * 256;
  c->out_off = c->data_off + 2LL * kMaxRanks * c->slot_bytes;
  c->seq = local_words;
  c->done = local_words + 1;
  (void)out_bytes;
  return c;
}
extern "C" void eredu_comm_destroy(void* c) { delete static_cast<PeerComm*>(c); }
extern "C" long long eredu_comm_buffer_bytes(long long slot_bytes, long long out_bytes) {
  const long long sb = (slot_bytes + 255) / 256 * 256;
  return 2LL * kMaxRanks * kMaxFlags * 4 + 2LL * kMaxRanks * sb + (out_bytes + 255) / 256 * 256;
}
extern "C" long long eredu_comm_out_offset(const void* c) { return static_cast<const PeerComm*>(c)->out_off; }
extern "C" long long eredu_comm_data_offset(const void* c, int parity, int src) {
  const PeerComm* pc = static_cast<const PeerComm*>(c);
  return pc->data_off + (static_cast<long long>(parity) * kMaxRanks + src) * pc->slot_bytes;
}

static int comm_grid(long long work_items, int sm_count) {
  long long g = (work_items + 511) / 512;
  const long long cap = sm_count > 0 ? sm_count : 148;  // one CTA per SM: all CTAs are resident
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

// All-reduce of [M, N] bf16 partials that every rank has already written at byte offset `x_off` of its own
// symmetric buffer. The result (+bias +residual) is in every rank's out region and, if y != null, copied to y.
extern "C" int eredu_allreduce_twoshot(const void* comm, long long x_off, const void* residual, const void* bias,
                                       void* y, int M, int N, int ldr, int sm_count, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  if (N % 8 != 0) return -1;
  const long long chunks = static_cast<long long>(M) * (N / 8);
  const int grid = comm_grid((chunks + c->size - 1) / c->size, sm_count);
  if (grid * 2 > kMaxFlags) return -2;
  allreduce_twoshot_kernel<<<grid, 512, 0, stream>>>(*c, x_off, static_cast<const __nv_bfloat16*>(residual),
                                                     static_cast<const __nv_bfloat16*>(bias),
                                                     static_cast<__nv_bfloat16*>(y), M, N, ldr, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_allgather(const void* comm, const void* src, long long bytes, int sm_count, int* status,
                               cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  if (bytes % 16 != 0) return -1;
  const int grid = comm_grid(bytes / 16, sm_count);
  allgather_kernel<<<grid, 512, 0, stream>>>(*c, static_cast<const uint4*>(src), bytes, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_peer_barrier(const void* comm, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  peer_barrier_kernel<<<1, 32, 0, stream>>>(*c, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
