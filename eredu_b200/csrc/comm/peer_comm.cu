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
    // every rank's copy is requested before the first one is used: a peer load takes microseconds, and a warp that adds
    // as it goes has one of them in flight at a time
    uint4 v[kMaxRanks];
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src)
      if (src < c.size) v[src] = ld_cg_u4(c.base[src] + x_off + i * 16);
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src) {
      if (src < c.size) {
        const uint32_t u[4] = {v[src].x, v[src].y, v[src].z, v[src].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += bf16_lo(u[j]);
          acc[2 * j + 1] += bf16_hi(u[j]);
        }
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
    if (y != nullptr) reinterpret_cast<uint4*>(y)[i] = o;  // this rank's own slice goes straight to y
  }
  cta_peer_barrier(c, parity, seq, 1, status);  // CTA k of every peer has stored its chunks everywhere
  if (y != nullptr) {
    // The barrier orders this CTA only against the same-index CTA of each peer, so the copy walks each peer's
    // slice with the writer's own partition: CTA k reads exactly the chunks that CTA k of rank `src` stored.
    const uint4* from = reinterpret_cast<const uint4*>(c.base[c.rank] + c.out_off);
    for (int src = 0; src < c.size; ++src) {
      if (src == c.rank) continue;
      const long long slo = per * src, shi = min(total, slo + per);
      for (long long i = slo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < shi;
           i += static_cast<long long>(gridDim.x) * blockDim.x)
        reinterpret_cast<uint4*>(y)[i] = ld_cg_u4(from + i);
    }
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

// One-shot all-reduce of a small [M, N] bf16 partial (decode steps: M * N * 4 bytes fit one staging slot). Every
// thread pushes 8 values to every peer as four self-validating 8-byte words {bf16x2, sequence tag}, then collects
// the same words of all ranks from its own slots and sums them in rank order (bitwise identical everywhere),
// adds bias and residual once and stores: no flag, no fence, no barrier.
__global__ void __launch_bounds__(128) allreduce_ll_kernel(PeerComm c, const __nv_bfloat16* __restrict__ partial, int ldp,
                                                            const __nv_bfloat16* __restrict__ residual, int ldr,
                                                            const __nv_bfloat16* __restrict__ bias,
                                                            __nv_bfloat16* __restrict__ y, int ldy, int M, int N, int* status) {
  const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(c.seq);
  const int parity = static_cast<int>(seq & 1u);
  const uint32_t tag = seq + 1u;
  const int chunks_per_row = N >> 3;
  const int id = blockIdx.x * blockDim.x + threadIdx.x;
  if (id < M * chunks_per_row) {
    const int m = id / chunks_per_row, n0 = (id % chunks_per_row) * 8;
    const uint4 pv = *reinterpret_cast<const uint4*>(partial + static_cast<size_t>(m) * ldp + n0);
    const size_t word = static_cast<size_t>(id) * 32;  // four 8-byte words per thread
    for (int peer = 0; peer < c.size; ++peer) {
      uint8_t* dst = peer_slot(c, peer, parity, c.rank) + word;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(pv.x), "r"(tag), "r"(pv.y), "r"(tag) : "memory");
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 16), "r"(pv.z), "r"(tag), "r"(pv.w), "r"(tag) : "memory");
    }
    uint4 rv = make_uint4(0u, 0u, 0u, 0u);
    if (residual != nullptr) rv = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(m) * ldr + n0);
    uint32_t val[kMaxRanks][4];
    uint32_t missing = (1u << c.size) - 1u;
    const long long t0 = clock64();
    while (missing != 0u) {
#pragma unroll
      for (int src = 0; src < kMaxRanks; ++src) {
        if (src < c.size && ((missing >> src) & 1u)) {
          const uint8_t* from = peer_slot(c, c.rank, parity, src) + word;
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "l"(from) : "memory");
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "l"(from + 16) : "memory");
          if (a1 == tag && a3 == tag && b1 == tag && b3 == tag) {
            val[src][0] = a0;
            val[src][1] = a2;
            val[src][2] = b0;
            val[src][3] = b2;
            missing &= ~(1u << src);
          }
        }
      }
      if (missing != 0u && clock64() - t0 > kWaitCycleLimit) {
        report_status(status, kStatusPeerFlagTimeout);
        break;
      }
    }
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src) {
      if (src < c.size && !((missing >> src) & 1u)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sum[2 * j] += bf16_lo(val[src][j]);
          sum[2 * j + 1] += bf16_hi(val[src][j]);
        }
      }
    }
    const uint32_t r[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sum[2 * j] += bf16_lo(r[j]);
      sum[2 * j + 1] += bf16_hi(r[j]);
    }
    if (bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sum[j] += __bfloat162float(bias[n0 + j]);
    }
    uint4 o;
    o.x = pack_bf16x2(sum[0], sum[1]);
    o.y = pack_bf16x2(sum[2], sum[3]);
    o.z = pack_bf16x2(sum[4], sum[5]);
    o.w = pack_bf16x2(sum[6], sum[7]);
    *reinterpret_cast<uint4*>(y + static_cast<size_t>(m) * ldy + n0) = o;
  }
  __syncthreads();
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
  c->lam_bytes = (c->slot_bytes / 2 + 255) / 256 * 256;
  c->lam_off = c->out_off + (out_bytes + 255) / 256 * 256;
  c->seq = local_words;
  c->done = local_words + 1;
  return c;
}
extern "C" void eredu_comm_destroy(void* c) { delete static_cast<PeerComm*>(c); }
extern "C" long long eredu_comm_buffer_bytes(long long slot_bytes, long long out_bytes) {
  const long long sb = (slot_bytes + 255) / 256 * 256;
  const long long lam = (sb / 2 + 255) / 256 * 256;
  return 2LL * kMaxRanks * kMaxFlags * 4 + 2LL * kMaxRanks * sb + (out_bytes + 255) / 256 * 256 + 2LL * kMaxRanks * lam;
}
// Fill the tag-free region of a freshly allocated symmetric buffer with its "empty" pattern. Call on the owner's
// buffer before any peer maps it.
extern "C" int eredu_comm_init_buffer(void* base, long long slot_bytes, long long out_bytes) {
  const long long sb = (slot_bytes + 255) / 256 * 256;
  const long long lam = (sb / 2 + 255) / 256 * 256;
  const long long off = 2LL * kMaxRanks * kMaxFlags * 4 + 2LL * kMaxRanks * sb + (out_bytes + 255) / 256 * 256;
  cudaError_t e = cudaMemset(static_cast<uint8_t*>(base) + off, 0xFF, static_cast<size_t>(2LL * kMaxRanks * lam));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaDeviceSynchronize());
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

// ------------------------------------------------------------------------------------------ point-to-point messages
// Pipeline hand-off without the host: a message is copied into the receiver's staging slot with plain peer stores and
// published with a release store of its sequence number; the receiver waits (bounded), copies it out and acknowledges,
// which lets the sender reuse that slot two messages later. Both sides are ordinary kernels on the caller's stream,
// so a pipeline stage's decode step - hand-off included - can be captured in a CUDA graph. Counters live in device
// memory of the calling rank ([peer][sent | received][channel]); channel 0 owns the slot from its start, channels
// 1..3 own 4 KB each at its end (token ids and other small control messages).
constexpr int kP2PChannels = 4;
constexpr int kP2PAckFlag = 64;

__device__ __forceinline__ long long p2p_channel_offset(const PeerComm& c, int channel) {
  return channel == 0 ? 0 : c.slot_bytes - 4096LL * channel;
}

__global__ void __launch_bounds__(512) peer_send_kernel(PeerComm c, int dst, int channel, const uint4* __restrict__ src,
                                                        long long bytes, unsigned int* counters, unsigned int* done, int* status) {
  unsigned int* cnt = counters + (dst * 2 + 0) * kP2PChannels + channel;
  const unsigned int n = *cnt;                      // messages already sent to `dst` on this channel
  const int parity = static_cast<int>(n & 1u);
  if (n >= 2u) {
    // the slot of this parity still holds message n - 2 until the receiver has acknowledged it
    if (threadIdx.x == 0) wait_flag(c, parity, dst, kP2PAckFlag + channel, n - 1u, status);
    __syncthreads();
  }
  uint4* slot = reinterpret_cast<uint4*>(peer_slot(c, dst, parity, c.rank) + p2p_channel_offset(c, channel));
  const long long words = bytes >> 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < words;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    slot[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
    *done = 0u;
    *cnt = n + 1u;
    st_release_sys(peer_flag(c, dst, parity, c.rank, channel), n + 1u);
  }
}

__global__ void __launch_bounds__(512) peer_recv_kernel(PeerComm c, int src, int channel, uint4* __restrict__ dst, long long bytes,
                                                        unsigned int* counters, unsigned int* done, int* status) {
  unsigned int* cnt = counters + (src * 2 + 1) * kP2PChannels + channel;
  const unsigned int m = *cnt;                      // messages already received from `src` on this channel
  const int parity = static_cast<int>(m & 1u);
  if (threadIdx.x == 0) wait_flag(c, parity, src, channel, m + 1u, status);
  __syncthreads();
  const uint8_t* slot = peer_slot(c, c.rank, parity, src) + p2p_channel_offset(c, channel);
  const long long words = bytes >> 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < words;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = ld_cg_u4(slot + i * 16);
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
    *done = 0u;
    *cnt = m + 1u;
    st_release_sys(peer_flag(c, src, parity, c.rank, kP2PAckFlag + channel), m + 1u);   // the sender may reuse the slot
  }
}

// `counters`: zero-initialised device words of the calling rank, [kMaxRanks][2][4] message counts followed by two words
// the kernels use to find their last CTA. bytes: a multiple of 16; channel 0 up to slot_bytes - 12 KB, channels 1..3 up
// to 4 KB. `peer` is the group rank of the other side.
static int p2p_check(const PeerComm* c, int peer, int channel, long long bytes) {
  if (peer < 0 || peer >= c->size || peer == c->rank || channel < 0 || channel >= kP2PChannels || bytes <= 0 || bytes % 16 != 0) return -1;
  if (bytes > (channel == 0 ? c->slot_bytes - 4096LL * (kP2PChannels - 1) : 4096LL)) return -2;
  return 0;
}

extern "C" int eredu_peer_send(const void* comm, int dst, int channel, const void* src, long long bytes, void* counters,
                               int sm_count, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  const int bad = p2p_check(c, dst, channel, bytes);
  if (bad != 0) return bad;
  unsigned int* cnt = static_cast<unsigned int*>(counters);
  const int grid = comm_grid(bytes / 16, sm_count);
  peer_send_kernel<<<grid, 512, 0, stream>>>(*c, dst, channel, static_cast<const uint4*>(src), bytes, cnt,
                                             cnt + kMaxRanks * 2 * kP2PChannels, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_peer_recv(const void* comm, int src, int channel, void* dst, long long bytes, void* counters,
                               int sm_count, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  const int bad = p2p_check(c, src, channel, bytes);
  if (bad != 0) return bad;
  unsigned int* cnt = static_cast<unsigned int*>(counters);
  const int grid = comm_grid(bytes / 16, sm_count);
  peer_recv_kernel<<<grid, 512, 0, stream>>>(*c, src, channel, static_cast<uint4*>(dst), bytes, cnt,
                                             cnt + kMaxRanks * 2 * kP2PChannels + 1, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_peer_barrier(const void* comm, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  peer_barrier_kernel<<<1, 32, 0, stream>>>(*c, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

// One-shot ("LL") all-reduce of a local [M, N] bf16 partial, for M * N * 4 bytes <= one staging slot (decode and
// verify steps). y = sum over ranks (+bias +residual). Returns -2 when the partial is too large (use the two-shot).
extern "C" int eredu_allreduce_ll(const void* comm, const void* partial, int ldp, const void* residual, int ldr,
                                  const void* bias, void* y, int ldy, int M, int N, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  if (N % 8 != 0 || ldp % 8 != 0 || ldy % 8 != 0 || (residual != nullptr && ldr % 8 != 0)) return -1;
  if (static_cast<long long>(M) * N * 4 > c->slot_bytes) return -2;
  const int items = M * (N / 8);
  allreduce_ll_kernel<<<(items + 127) / 128, 128, 0, stream>>>(
      *c, static_cast<const __nv_bfloat16*>(partial), ldp, static_cast<const __nv_bfloat16*>(residual), ldr,
      static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y), ldy, M, N, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
