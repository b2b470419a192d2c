// Mixture-of-experts routing and data movement, all on the device (no host synchronisation anywhere):
//   route   : router logits -> scores (softmax | sigmoid | sqrt-softplus | top-k-then-softmax) (+ selection
//             bias) -> top-k ids + weights (optional renormalisation, scale)
//   plan    : routes of the locally owned experts -> per-expert segments, row positions, GEMM work items
//   gather  : token rows -> expert-contiguous rows (the routing permute)
//   combine : out[t] = residual[t] + sum_k w[t,k] * y[pos(t,k)]  summed in slot order (deterministic)
//
// Semantics follow eredu/src/backend/mlx/nn/moe.rs:433-507,652-738 (router variants, renormalisation,
// weighted route sum in stable slot order) and safemlx/src/ops/moe.rs:36-106 (sort by expert, gather rows,
// grouped GEMM, scatter back). The reference synchronises the host for route compaction
// (runtime/distributed/expert.rs:575) and for the count matrix (:805-808); here both stay on the device.
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/peer.cuh"
#include "../common/ptx.cuh"

namespace eredu {

enum { SCORE_SOFTMAX = 0, SCORE_SIGMOID = 1, SCORE_SQRT_SOFTPLUS = 2, SCORE_TOPK_SOFTMAX = 3 };

// One warp routes one token, up to 512 experts (16 per lane).
__device__ __forceinline__ void route_token(const float* __restrict__ logits, const float* __restrict__ sel_bias,
                                            int* __restrict__ ids, float* __restrict__ weights, int t, int lane, int E, int k,
                                            int scoring, int renorm, float scale) {
  constexpr int PER = 16;
  float score[PER];   // value reported as the route weight
  float select[PER];  // value used for selection (score + bias)
  const float* row = logits + static_cast<size_t>(t) * E;
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    score[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, score[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (scoring == SCORE_SOFTMAX) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      score[j] = (lane + 32 * j < E) ? __expf(score[j] - mx) : 0.f;
      sum += score[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) score[j] *= inv;
  } else if (scoring == SCORE_SIGMOID) {
#pragma unroll
    for (int j = 0; j < PER; ++j) score[j] = (lane + 32 * j < E) ? 1.f / (1.f + __expf(-score[j])) : -INFINITY;
  } else if (scoring == SCORE_SQRT_SOFTPLUS) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const float x = score[j];
      score[j] = (lane + 32 * j < E) ? sqrtf(x > 20.f ? x : log1pf(__expf(x))) : -INFINITY;
    }
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    select[j] = (e < E) ? score[j] + (sel_bias != nullptr ? sel_bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;  // lane i keeps the weight of slot i
  int my_id = 0;
  for (int slot = 0; slot < k; ++slot) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (select[j] > best || (select[j] == best && e < best_e)) { best = select[j]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    // owner lane reports the score and retires the expert
    float w = 0.f;
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        if (lane + 32 * j == best_e) { w = score[j]; select[j] = -INFINITY; }
      }
    }
    w = __shfl_sync(0xffffffffu, w, best_e & 31);
    if (lane == (slot & 31)) { my_w = w; my_id = best_e; }
    wsum += w;
    if (slot >= 31) break;  // k <= 32
  }
  if (scoring == SCORE_TOPK_SOFTMAX) {
    // softmax over the selected logits only
    float m2 = lane < k ? my_w : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m2 = fmaxf(m2, __shfl_xor_sync(0xffffffffu, m2, o));
    float ex = lane < k ? __expf(my_w - m2) : 0.f;
    float s2 = ex;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    my_w = ex / s2;
  } else if (renorm) {
    my_w = my_w / fmaxf(wsum, 1e-20f);
  }
  if (lane < k) {
    ids[static_cast<size_t>(t) * k + lane] = my_id;
    weights[static_cast<size_t>(t) * k + lane] = my_w * scale;
  }
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ sel_bias,
                                                         int* __restrict__ ids, float* __restrict__ weights, int T, int E,
                                                         int k, int scoring, int renorm, float scale) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= T) return;
  route_token(logits, sel_bias, ids, weights, t, threadIdx.x & 31, E, k, scoring, renorm, scale);
}

// Single CTA. routes = T*k. Experts [e0, e1) are local. Outputs:
//   seg[0..n_local]      : first row of each local expert's segment (seg[n_local] = number of local routes)
//   route_pos[r]         : row of route r in the permuted buffers, -1 when its expert is not local
//   row_token[pos]       : token index of the row
//   work[n_work_cap] int4: {local expert, row0, rows, 0} one item per `tile` rows of a segment, rest zeroed
//   counts[2]            : {local routes, work items used}
__device__ __forceinline__ void plan_block(const int* __restrict__ ids, int routes, int k, int e0, int e1, int tile,
                                           int* __restrict__ seg, int* __restrict__ route_pos, int* __restrict__ row_token,
                                           int4* __restrict__ work, int n_work_cap, int* __restrict__ counts) {
  __shared__ int cnt[512];
  __shared__ int start[513];
  __shared__ int cursor[512];
  __shared__ int item0[513];
  const int n_local = e1 - e0;
  for (int i = threadIdx.x; i < n_local; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = ids[r] - e0;
    if (e >= 0 && e < n_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, items = 0;
    for (int e = 0; e < n_local; ++e) {
      start[e] = acc;
      item0[e] = items;
      acc += cnt[e];
      items += (cnt[e] + tile - 1) / tile;
    }
    start[n_local] = acc;
    item0[n_local] = items;
    counts[0] = acc;
    counts[1] = items;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= n_local; i += blockDim.x) {
    seg[i] = start[i];
    if (i < n_local) cursor[i] = 0;
  }
  for (int i = threadIdx.x; i < n_work_cap; i += blockDim.x) work[i] = make_int4(0, 0, 0, 0);
  __syncthreads();
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) {
    const int n_items = item0[e + 1] - item0[e];
    for (int j = 0; j < n_items; ++j) {
      const int idx = item0[e] + j;
      if (idx < n_work_cap) work[idx] = make_int4(e, start[e] + j * tile, min(tile, cnt[e] - j * tile), 0);
    }
  }
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = ids[r] - e0;
    int pos = -1;
    if (e >= 0 && e < n_local) {
      pos = start[e] + atomicAdd(&cursor[e], 1);
      row_token[pos] = r / k;
    }
    route_pos[r] = pos;
  }
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, int routes, int k, int e0, int e1,
                                                         int tile, int* __restrict__ seg, int* __restrict__ route_pos,
                                                         int* __restrict__ row_token, int4* __restrict__ work,
                                                         int n_work_cap, int* __restrict__ counts) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  plan_block(ids, routes, k, e0, e1, tile, seg, route_pos, row_token, work, n_work_cap, counts);
}

// Decode-sized steps (T <= 64 tokens): routing, planning and the row gather in ONE single-CTA kernel instead of
// three dependent launches. 32 warps route the tokens, the block plans the local experts' segments in shared
// memory, then copies the token rows into expert order.
__global__ void __launch_bounds__(1024) moe_route_plan_gather_kernel(
    const float* __restrict__ logits, const float* __restrict__ sel_bias, int* __restrict__ ids, float* __restrict__ weights,
    int T, int E, int k, int scoring, int renorm, float scale, int e0, int e1, int tile, int* __restrict__ seg,
    int* __restrict__ route_pos, int* __restrict__ row_token, int4* __restrict__ work, int n_work_cap, int* __restrict__ counts,
    const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ xp, int H) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = warp; t < T; t += 32) route_token(logits, sel_bias, ids, weights, t, lane, E, k, scoring, renorm, scale);
  __syncthreads();  // ids written by this block are visible to it
  plan_block(ids, T * k, k, e0, e1, tile, seg, route_pos, row_token, work, n_work_cap, counts);
  __syncthreads();
  const int n_rows = xp != nullptr ? counts[0] : 0;  // large steps gather with the many-CTA kernel instead
  for (int pos = warp; pos < n_rows; pos += 32) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row_token[pos]) * H);
    uint4* dst = reinterpret_cast<uint4*>(xp + static_cast<size_t>(pos) * H);
    for (int c = lane; c < (H >> 3); c += 32) dst[c] = src[c];
  }
}

// xp[pos, :] = x[row_token[pos], :] for pos < counts[0]. grid = rows_cap CTAs.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                  const int* __restrict__ counts, __nv_bfloat16* __restrict__ xp, int H) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int pos = blockIdx.x;
  if (pos >= counts[0]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row_token[pos]) * H);
  uint4* dst = reinterpret_cast<uint4*>(xp + static_cast<size_t>(pos) * H);
  // L2 loads: the rows may have been stored by another GPU into a buffer this SM read before
  for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) dst[c] = ld_cg_u4(src + c);
}

// out[t, :] = (residual[t, :]) + (extra[t, :]) + sum_k w[t,k] * y[route_pos[t*k + slot], :]  (local routes only),
// slots in ascending order. grid = T CTAs.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_pos,
                                   const float* __restrict__ weights, const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ extra, __nv_bfloat16* __restrict__ out, int k, int H) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int slot = 0; slot < k; ++slot) {
      const int pos = route_pos[t * k + slot];
      if (pos < 0) continue;
      const float w = weights[t * k + slot];
      const uint4 v = reinterpret_cast<const uint4*>(y + static_cast<size_t>(pos) * H)[c];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += w * bf16_lo(u[j]);
        acc[2 * j + 1] += w * bf16_hi(u[j]);
      }
    }
    const __nv_bfloat16* adds[2] = {residual, extra};
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      if (adds[a] != nullptr) {
        const uint4 v = reinterpret_cast<const uint4*>(adds[a] + t * H)[c];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += bf16_lo(u[j]);
          acc[2 * j + 1] += bf16_hi(u[j]);
        }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + t * H)[c] = o;
  }
}

// Expert-parallel combine fused with the all-reduce over the expert group (replicated-token expert
// parallelism: every rank routed all tokens and ran its own experts). Each thread forms the weighted sum of
// its token's LOCAL routes for 8 columns, pushes it to every peer's staging slot as four 8-byte
// {bf16x2, sequence tag} words (two 16-byte stores; every 8-byte half validates itself, so no fence, flag or
// barrier is needed), then collects the same words from all ranks out of its own slots, sums them in rank order
// (bitwise identical on every rank), adds the residual once and stores. T <= 64 tokens (decode / verify steps).
// grid = (T, ceil(H / 8 / 128)).
__global__ void __launch_bounds__(128) moe_combine_ar_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_pos,
                                                              const float* __restrict__ weights,
                                                              const __nv_bfloat16* __restrict__ residual,
                                                              const __nv_bfloat16* __restrict__ extra,
                                                              __nv_bfloat16* __restrict__ out, int k, int H, PeerComm comm,
                                                              int* status) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(comm.seq);
  const int parity = static_cast<int>(seq & 1u);
  const uint32_t tag = seq + 1u;
  const size_t t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c < (H >> 3)) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int slot = 0; slot < k; ++slot) {
      const int pos = route_pos[t * k + slot];
      if (pos < 0) continue;
      const float w = weights[t * k + slot];
      const uint4 v = reinterpret_cast<const uint4*>(y + static_cast<size_t>(pos) * H)[c];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += w * bf16_lo(u[j]);
        acc[2 * j + 1] += w * bf16_hi(u[j]);
      }
    }
    if (extra != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(extra + t * H)[c];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(u[j]);
        acc[2 * j + 1] += bf16_hi(u[j]);
      }
    }
    uint32_t pk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pk[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
    const size_t word = (t * (H >> 1) + static_cast<size_t>(c) * 4) * 8;  // byte offset of this thread's four words
    for (int peer = 0; peer < comm.size; ++peer) {
      uint8_t* dst = peer_slot(comm, peer, parity, comm.rank) + word;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(pk[0]), "r"(tag), "r"(pk[1]), "r"(tag)
                   : "memory");
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 16), "r"(pk[2]), "r"(tag), "r"(pk[3]),
                   "r"(tag)
                   : "memory");
    }
    uint32_t val[kMaxRanks][4];
    uint32_t missing = (1u << comm.size) - 1u;
    const long long t0 = clock64();
    while (missing != 0u) {
#pragma unroll
      for (int src = 0; src < kMaxRanks; ++src) {
        if (src < comm.size && ((missing >> src) & 1u)) {
          const uint8_t* from = peer_slot(comm, comm.rank, parity, src) + word;
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "l"(from) : "memory");
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                       : "l"(from + 16)
                       : "memory");
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
      if (src < comm.size && !((missing >> src) & 1u)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sum[2 * j] += bf16_lo(val[src][j]);
          sum[2 * j + 1] += bf16_hi(val[src][j]);
        }
      }
    }
    if (residual != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(residual + t * H)[c];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sum[2 * j] += bf16_lo(u[j]);
        sum[2 * j + 1] += bf16_hi(u[j]);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(sum[0], sum[1]);
    o.y = pack_bf16x2(sum[2], sum[3]);
    o.z = pack_bf16x2(sum[4], sum[5]);
    o.w = pack_bf16x2(sum[6], sum[7]);
    reinterpret_cast<uint4*>(out + t * H)[c] = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) finish_call(comm, seq, gridDim.x * gridDim.y);
}


// ============================================================================ expert-parallel all-to-all (sharded tokens)
// The token-sharded form of expert parallelism (the reference's `dispatch_sharded`: a count all-gather with a host sync,
// four forward and two reverse all_to_all_v exchanges - eredu/src/backend/mlx/runtime/distributed/expert.rs:781-842,
// 1054-1222) as four kernels over NVLink peer memory with every count kept on the device:
//   dispatch : the SOURCE rank of a token walks its top-k routes, claims a row in the owner rank's receive area (one
//              region per source, so a device-side cursor per owner is all the bookkeeping) and stores the hidden row and
//              {expert id, route index} straight into the owner's memory - the routing permute IS the transfer; the last
//              CTA publishes the per-owner counts and one flag per owner;
//   recv_plan: the OWNER waits (bounded) for the flags of all sources, reads the counts and builds the grouped-GEMM plan
//              over the received rows;
//   return   : after the expert GEMMs the owner stores every output row into the source's return area at the route's
//              own slot [token, k] (no atomics; a flag per source follows);
//   combine  : the source waits for all owners, forms residual + sum_k w_k * row_k in slot order (deterministic), stores
//              the finished token row into EVERY rank's output (the all-gather that restores replicated activations),
//              and the kernel ends once the rows of all sources have arrived.
// Sequence numbers as in the other peer kernels: dispatch, return and combine each advance the communicator by one.
struct A2AView {
  long long recv_off;  // [size src][cap][H] bf16   rows received from every source
  long long meta_off;  // [size src][cap] int2      {global expert id, route index at the source}
  long long cnt_off;   // [2 parity][size src] int  rows sent by each source in this call
  long long ret_off;   // [cap][H] bf16             rows returned to this source, slot = its route index
  long long out_off;   // [2][T_max][H] bf16        gathered token rows (double-buffered by call)
  long long out_half_bytes;
  int T, T_src, k, H, E_local, cap;
  int out_parity;
};

__device__ __forceinline__ void copy_row16(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
  for (int i = lane * 16; i < bytes; i += 32 * 16) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
}

// grid = max(1, n_own) CTAs of 128 threads; token `blockIdx.x` of this rank's slice, one warp per route.
__global__ void __launch_bounds__(128) moe_a2a_dispatch_kernel(PeerComm c, A2AView v, const __nv_bfloat16* __restrict__ x_own,
                                                               const int* __restrict__ ids, int n_own,
                                                               int* __restrict__ cursor, int* status) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(c.seq);
  const int parity = static_cast<int>(seq & 1u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  if (t < n_own) {
    for (int s = warp; s < v.k; s += 4) {
      int e = 0, idx = 0;
      if (lane == 0) {
        e = ids[t * v.k + s];
        idx = atomicAdd(&cursor[e / v.E_local], 1);
      }
      e = __shfl_sync(0xffffffffu, e, 0);
      idx = __shfl_sync(0xffffffffu, idx, 0);
      const int owner = e / v.E_local;
      if (idx < v.cap) {  // cap = every route of the slice: cannot overflow
        const size_t row = static_cast<size_t>(c.rank) * v.cap + idx;
        copy_row16(c.base[owner] + v.recv_off + row * v.H * 2, reinterpret_cast<const uint8_t*>(x_own + static_cast<size_t>(t) * v.H),
                   v.H * 2, lane);
        if (lane == 0) *reinterpret_cast<int2*>(c.base[owner] + v.meta_off + row * 8) = make_int2(e, t * v.k + s);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(c.done, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {  // every CTA's rows are out: publish how many each owner got, then the flag
    __threadfence_system();
    if (threadIdx.x < c.size) {
      const int owner = threadIdx.x;
      const int n = atomicAdd(&cursor[owner], 0);
      *reinterpret_cast<volatile int*>(c.base[owner] + v.cnt_off + (static_cast<size_t>(parity) * kMaxRanks + c.rank) * 4) = n;
      cursor[owner] = 0;
      __threadfence_system();
      st_release_sys(peer_flag(c, owner, parity, c.rank, 0), seq + 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *c.done = 0u;
      __threadfence();
      *c.seq = seq + 1u;
    }
  }
  (void)status;
}

// Single CTA (1024 threads). Waits for the dispatch flags of all sources, then plans the local experts over the received
// rows: flat row r = src * cap + i is a route when i < count[src]. `ids_flat` is scratch [size * cap].
__global__ void __launch_bounds__(1024) moe_a2a_recv_plan_kernel(PeerComm c, A2AView v, int e0, int e1, int tile,
                                                                 int* __restrict__ ids_flat, int* __restrict__ seg,
                                                                 int* __restrict__ route_pos, int* __restrict__ row_token,
                                                                 int4* __restrict__ work, int n_work_cap, int* __restrict__ counts,
                                                                 int* status) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const unsigned int want = *reinterpret_cast<volatile unsigned int*>(c.seq);  // the dispatch kernel already advanced it
  const int parity = static_cast<int>((want - 1u) & 1u);
  __shared__ int s_cnt[kMaxRanks];
  if (threadIdx.x < c.size) {
    wait_flag(c, parity, threadIdx.x, 0, want, status);
    s_cnt[threadIdx.x] = *reinterpret_cast<volatile int*>(c.base[c.rank] + v.cnt_off + (static_cast<size_t>(parity) * kMaxRanks + threadIdx.x) * 4);
  }
  __syncthreads();
  const int total = c.size * v.cap;
  const int2* meta = reinterpret_cast<const int2*>(c.base[c.rank] + v.meta_off);
  for (int r = threadIdx.x; r < total; r += blockDim.x) {
    const int src = r / v.cap, i = r - src * v.cap;
    ids_flat[r] = (i < min(s_cnt[src], v.cap)) ? __ldcg(&meta[r].x) : -1;
  }
  __syncthreads();
  plan_block(ids_flat, total, 1, e0, e1, tile, seg, route_pos, row_token, work, n_work_cap, counts);
}

// grid = size * cap CTAs of 128 threads (one per receive slot). Output row of slot r goes back to its source.
__global__ void __launch_bounds__(128) moe_a2a_return_kernel(PeerComm c, A2AView v, const __nv_bfloat16* __restrict__ y,
                                                             const int* __restrict__ route_pos, int* status) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(c.seq);
  const int parity = static_cast<int>(seq & 1u);
  const int r = blockIdx.x;
  const int pos = route_pos[r];
  if (pos >= 0) {
    const int src = r / v.cap;
    const int2 m = __ldcg(reinterpret_cast<const int2*>(c.base[c.rank] + v.meta_off) + r);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* dst = c.base[src] + v.ret_off + static_cast<size_t>(m.y) * v.H * 2;
    const uint8_t* from = reinterpret_cast<const uint8_t*>(y + static_cast<size_t>(pos) * v.H);
    const int quarter = (v.H * 2 / 64) * 16;  // each warp copies a quarter of the row (H * 2 bytes, multiple of 64)
    copy_row16(dst + warp * quarter, from + warp * quarter, quarter, lane);
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(c.done, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < c.size) st_release_sys(peer_flag(c, threadIdx.x, parity, c.rank, 1), seq + 1u);
    __syncthreads();
    if (threadIdx.x == 0) {
      *c.done = 0u;
      __threadfence();
      *c.seq = seq + 1u;
    }
  }
  (void)status;
}

// grid = max(1, n_own) CTAs of 128 threads. Token t (local index) -> out[t0 + t] on every rank.
__global__ void __launch_bounds__(128) moe_a2a_combine_kernel(PeerComm c, A2AView v, const float* __restrict__ weights,
                                                              const __nv_bfloat16* __restrict__ residual_own,
                                                              const __nv_bfloat16* __restrict__ extra_own, int n_own, int t0,
                                                              int* status) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(c.seq);  // the return kernel's flags carry this value
  const int parity = static_cast<int>(seq & 1u);
  if (threadIdx.x < c.size) wait_flag(c, static_cast<int>((seq - 1u) & 1u), threadIdx.x, 1, seq, status);
  __syncthreads();
  const int t = blockIdx.x;
  if (t < n_own) {
    const uint8_t* ret = c.base[c.rank] + v.ret_off;
    for (int ch = threadIdx.x; ch < (v.H >> 3); ch += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < v.k; ++s) {  // slot order: the same bits whatever the arrival order was
        const float w = weights[t * v.k + s];
        const uint4 q = ld_cg_u4(ret + (static_cast<size_t>(t) * v.k + s) * v.H * 2 + static_cast<size_t>(ch) * 16);
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += w * bf16_lo(u[j]);
          acc[2 * j + 1] += w * bf16_hi(u[j]);
        }
      }
      const __nv_bfloat16* adds[2] = {residual_own, extra_own};
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        if (adds[a] != nullptr) {
          const uint4 q = reinterpret_cast<const uint4*>(adds[a] + static_cast<size_t>(t) * v.H)[ch];
          const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += bf16_lo(u[j]);
            acc[2 * j + 1] += bf16_hi(u[j]);
          }
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      const size_t off = v.out_off + static_cast<size_t>(v.out_parity) * v.out_half_bytes +
                         (static_cast<size_t>(t0 + t) * v.H) * 2 + static_cast<size_t>(ch) * 16;
      for (int peer = 0; peer < c.size; ++peer) *reinterpret_cast<uint4*>(c.base[peer] + off) = o;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(c.done, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {  // this rank's rows are everywhere: tell everyone, then wait for everyone's rows
    __threadfence_system();
    if (threadIdx.x < c.size) {
      st_release_sys(peer_flag(c, threadIdx.x, parity, c.rank, 2), seq + 1u);
      wait_flag(c, parity, threadIdx.x, 2, seq + 1u, status);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *c.done = 0u;
      __threadfence();
      *c.seq = seq + 1u;
    }
  }
}

}  // namespace eredu

using namespace eredu;

extern "C" int eredu_moe_route(const float* logits, const float* sel_bias, int* ids, float* weights, int T, int E, int k,
                               int scoring, int renorm, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 512 || k > 32 || k > E) return -1;
  launch_pdl(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, logits, sel_bias, ids, weights, T, E, k, scoring,
             renorm, scale);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_moe_plan(const int* ids, int routes, int k, int e0, int e1, int tile, int* seg, int* route_pos,
                              int* row_token, int* work, int n_work_cap, int* counts, cudaStream_t stream) {
  if (e1 - e0 > 512 || e1 <= e0) return -1;
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, routes, k, e0, e1, tile, seg, route_pos, row_token,
             reinterpret_cast<int4*>(work), n_work_cap, counts);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_moe_gather(const void* x, const int* row_token, const int* counts, void* xp, int rows_cap, int H,
                                cudaStream_t stream) {
  if (rows_cap <= 0) return 0;
  if (H % 8 != 0) return -1;
  launch_pdl(moe_gather_kernel, dim3(rows_cap), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(x), row_token,
             counts, static_cast<__nv_bfloat16*>(xp), H);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_moe_combine(const void* y, const int* route_pos, const float* weights, const void* residual,
                                 const void* extra, void* out, int T, int k, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  launch_pdl(moe_combine_kernel, dim3(T), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(y), route_pos, weights,
             static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(extra),
             static_cast<__nv_bfloat16*>(out), k, H);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

// Combine + all-reduce over the expert group in one kernel (see moe_combine_ar_kernel). `comm` is the peer
// communication context of the group; T * H * 4 bytes must fit one staging slot.
extern "C" int eredu_moe_combine_ar(const void* y, const int* route_pos, const float* weights, const void* residual,
                                    const void* extra, void* out, int T, int k, int H, const void* comm, int* status,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  if (H % 8 != 0 || c == nullptr) return -1;
  if (static_cast<long long>(T) * H * 4 > c->slot_bytes) return -2;
  const int chunks = H / 8;
  launch_pdl(moe_combine_ar_kernel, dim3(T, (chunks + 127) / 128), dim3(128), 0, stream,
             static_cast<const __nv_bfloat16*>(y), route_pos, weights, static_cast<const __nv_bfloat16*>(residual),
             static_cast<const __nv_bfloat16*>(extra), static_cast<__nv_bfloat16*>(out), k, H, *c, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_moe_route_plan_gather(const float* logits, const float* sel_bias, int* ids, float* weights, int T, int E,
                                           int k, int scoring, int renorm, float scale, int e0, int e1, int tile, int* seg,
                                           int* route_pos, int* row_token, int* work, int n_work_cap, int* counts,
                                           const void* x, void* xp, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 512 || k > 32 || k > E || e1 - e0 > 512 || e1 <= e0 || H % 8 != 0 || T > 64) return -1;
  launch_pdl(moe_route_plan_gather_kernel, dim3(1), dim3(1024), 0, stream, logits, sel_bias, ids, weights, T, E, k, scoring,
             renorm, scale, e0, e1, tile, seg, route_pos, row_token, reinterpret_cast<int4*>(work), n_work_cap, counts,
             static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(xp), H);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

// ---- expert-parallel all-to-all over peer memory. `view`: 13 values {recv_off, meta_off, cnt_off, ret_off, out_off,
// out_half_bytes, T, T_src, k, H, E_local, cap, out_parity} as int64.
static A2AView a2a_view(const long long* p) {
  A2AView v;
  v.recv_off = p[0];
  v.meta_off = p[1];
  v.cnt_off = p[2];
  v.ret_off = p[3];
  v.out_off = p[4];
  v.out_half_bytes = p[5];
  v.T = static_cast<int>(p[6]);
  v.T_src = static_cast<int>(p[7]);
  v.k = static_cast<int>(p[8]);
  v.H = static_cast<int>(p[9]);
  v.E_local = static_cast<int>(p[10]);
  v.cap = static_cast<int>(p[11]);
  v.out_parity = static_cast<int>(p[12]);
  return v;
}
extern "C" int eredu_moe_a2a_dispatch(const void* comm, const long long* view, const void* x_own, const int* ids, int n_own,
                                      int* cursor, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  const A2AView v = a2a_view(view);
  if (c == nullptr || v.H % 32 != 0 || v.k > 32 || v.E_local <= 0) return -1;
  launch_pdl(moe_a2a_dispatch_kernel, dim3(n_own > 0 ? n_own : 1), dim3(128), 0, stream, *c, v,
             static_cast<const __nv_bfloat16*>(x_own), ids, n_own, cursor, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int eredu_moe_a2a_recv_plan(const void* comm, const long long* view, int e0, int e1, int tile, int* ids_flat, int* seg,
                                       int* route_pos, int* row_token, int* work, int n_work_cap, int* counts, int* status,
                                       cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  const A2AView v = a2a_view(view);
  if (c == nullptr || e1 - e0 > 512 || e1 <= e0) return -1;
  launch_pdl(moe_a2a_recv_plan_kernel, dim3(1), dim3(1024), 0, stream, *c, v, e0, e1, tile, ids_flat, seg, route_pos, row_token,
             reinterpret_cast<int4*>(work), n_work_cap, counts, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int eredu_moe_a2a_return(const void* comm, const long long* view, const void* y, const int* route_pos, int* status,
                                    cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  const A2AView v = a2a_view(view);
  if (c == nullptr) return -1;
  launch_pdl(moe_a2a_return_kernel, dim3(c->size * v.cap), dim3(128), 0, stream, *c, v, static_cast<const __nv_bfloat16*>(y),
             route_pos, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int eredu_moe_a2a_combine(const void* comm, const long long* view, const float* weights, const void* residual_own,
                                     const void* extra_own, int n_own, int t0, int* status, cudaStream_t stream) {
  const PeerComm* c = static_cast<const PeerComm*>(comm);
  const A2AView v = a2a_view(view);
  if (c == nullptr) return -1;
  launch_pdl(moe_a2a_combine_kernel, dim3(n_own > 0 ? n_own : 1), dim3(128), 0, stream, *c, v, weights,
             static_cast<const __nv_bfloat16*>(residual_own), static_cast<const __nv_bfloat16*>(extra_own), n_own, t0, status);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
