// Dense bf16 linear layer  Y[M,N] = X[M,K] · W[N,K]^T  on the 5th-gen tensor cores.
//
// Design ("weight-stationary, swap-AB"): the 128-row weight tile is the MMA's M operand and the
// token tile (16..256 rows of X) is the MMA's N operand, so that one kernel covers decode
// (M = 1..64 tokens, a pure weight-streaming problem) and prefill (thousands of tokens).
//   * TMA (cp.async.bulk.tensor, 128B swizzle, no multicast) streams W and X tiles into a
//     multi-stage shared-memory ring; one thread issues tcgen05.mma; accumulators live in TMEM;
//     four epilogue warps read them back with tcgen05.ld.
//   * DUAL mode multiplies the same X tile against two weight tiles (gate rows and up rows of a
//     concatenated [2I,K] matrix) into two TMEM regions and the epilogue writes silu(g)*u — the
//     SwiGLU activation never round-trips through HBM.
//   * Split-K for the decode regime runs as a thread-block cluster along z: every CTA of the
//     cluster accumulates a K slice, the partials are exchanged through distributed shared
//     memory and each CTA reduces and stores a share of the token columns. No atomics, no
//     global scratch, bitwise deterministic.
//   * Epilogue fusions: bias, residual add, SwiGLU, bf16 or fp32 output.
//
// Replaces the reference's dense matmul call sites (eredu-architectures/src/llama.rs:270-286,
// 418-431; eredu/src/backend/mlx/nn/parallel.rs:794-796) and its silu(gate)*up composition
// (eredu/src/backend/mlx/nn/layers.rs:21-24).
#include <cooperative_groups.h>

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/peer.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "../common/trace.cuh"
#include "gemm_persistent.h"

namespace cg = cooperative_groups;

namespace eredu {

struct GemmParams {
  void* y;               // [M, ldy] bf16 or fp32
  const void* residual;  // optional [M, ldr] bf16, added after activation
  const void* bias;      // optional [N] bf16 (DUAL: [2*N_out], gate part then up part)
  int M, N, K;           // N = output columns (DUAL: columns of the activation output)
  int ldy, ldr;
  int dual_row_offset;  // DUAL: row of W where the "up" matrix starts
  int out_fp32;
  int* status;
  int col_offset;  // COMM_AG: column of the gathered output where this rank's N columns start
  // RMSNorm folded around the GEMMs of a decoder block (norm weights are pre-multiplied into W):
  //   consumer: y[m,:] = rsqrt(sum_j ssq_in[m, j] * norm_inv_dim + norm_eps) * (x[m,:] W^T)
  //   producer: ssq_out[m, tile_n] = sum over this tile's columns of (stored y[m, n])^2
  const float* ssq_in;
  int ssq_parts;
  float norm_eps;
  float norm_inv_dim;
  float* ssq_out;
  // Grouped (MoE) mode: blockIdx.y indexes a work item {expert, first row, row count, -} built on the device;
  // the expert's weights start at row expert * w_rows_per_expert of W, its tokens are rows [row0, row0+rows)
  // of X and Y. Items with rows == 0 exit at once.
  const int* work;
  int w_rows_per_expert;
  // Large token tiles: the epilogue goes through shared memory so that the output (and the residual) move as
  // 16-byte row chunks instead of one 2-byte element per thread. Needs 16-byte aligned rows (host-checked).
  int staged;
  // Gated activation of DUAL tiles: 0 = silu(g) * u (SwiGLU); 1 = g * sigmoid(1.702 g) * (u + 1) (GPT-OSS). With
  // act_limit > 0 the gate is clamped from above and the linear branch to [-limit, limit] first
  // (eredu/src/backend/mlx/architectures/gpt_oss/model.rs:748-753; nn/moe.rs swiglu_limit).
  int act;
  float act_limit;
  int bias_expert_stride;  // grouped mode: elements between two experts' bias vectors (0 = one shared vector)
  // Weights that no kernel of the stream rewrites (every model weight): their first tiles are fetched, and the
  // rest prefetched into L2, BEFORE the kernel waits for its producer under programmatic dependent launch, so
  // the weight stream of this kernel overlaps the tail of the previous one.
  int w_static;
  PeerComm comm;   // COMM modes only
};

// Collective fused into the epilogue (tensor parallelism over NVLink peer memory, small token counts):
//   COMM_AR: every rank holds a K-slice; partial tiles are pushed to all peers' slots as they leave TMEM, as 4-byte
//            bf16x2 words into a sentinel-initialised region (a word is valid once it differs from the sentinel: no
//            tag, no fence, no flag - the whole word is payload), and each rank sums the `size` partials in rank
//            order (bitwise identical on all ranks), adds bias/residual once and stores.
//   COMM_AG: every rank holds an N-slice; finished tiles are stored straight into every peer's gathered
//            output at the rank's column offset.
enum { COMM_NONE = 0, COMM_AR = 1, COMM_AG = 2 };

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int TN, bool DUAL>
struct GemmCfg {
  static constexpr int kATile = 128 * 64 * 2;
  static constexpr int kBTile = TN * 64 * 2;
  static constexpr int kStageBytes = kATile * (DUAL ? 2 : 1) + kBTile;
  // Decode-sized tiles keep shared memory under half an SM so that two CTAs are co-resident: the whole grid
  // (<= 296 CTAs) then runs as one wave and HBM bandwidth is shared evenly instead of paying a partial wave.
  static constexpr int kBudget = (TN <= 32) ? (DUAL ? 3 * kStageBytes : 100 * 1024) : (TN == 64 && !DUAL) ? 100 * 1024 : 196 * 1024;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccCols = TN * (DUAL ? 2 : 1);
  static constexpr int kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
  static constexpr int kCtrlBytes = 1024;
  static constexpr int kSmemBytes = 1024 + kCtrlBytes + kStages * kStageBytes;
  static_assert(kStages >= 2, "pipeline too shallow");
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ float gated_act(const GemmParams& p, float g, float u) {
  if (p.act_limit > 0.f) {
    g = fminf(g, p.act_limit);
    u = fminf(fmaxf(u, -p.act_limit), p.act_limit);
  }
  if (p.act == 1) return g / (1.0f + __expf(-1.702f * g)) * (u + 1.0f);
  return silu_f(g) * u;
}

// Applies row scale, bias, activation and residual, stores, and returns the value as stored (after rounding).
__device__ __forceinline__ float residual_at(const GemmParams& p, int m, int n) {
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p.residual)[static_cast<size_t>(m) * p.ldr + n]);
}

// `rv`: the residual value of the element (0 when there is none), loaded by the caller ahead of time so that
// the load does not sit between two dependent stores.
template <bool DUAL>
__device__ __forceinline__ float epilogue_store(const GemmParams& p, float g, float u, int m, int n, float scale, float rv) {
  g *= scale;
  if (DUAL) u *= scale;
  if (p.bias != nullptr) {
    const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(p.bias);
    g += __bfloat162float(b[n]);
    if (DUAL) u += __bfloat162float(b[p.N + n]);
  }
  float v = (DUAL ? gated_act(p, g, u) : g) + rv;
  if (p.out_fp32) {
    static_cast<float*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = v;
    return v;
  }
  const __nv_bfloat16 r = __float2bfloat16(v);
  static_cast<__nv_bfloat16*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = r;
  return __bfloat162float(r);
}

// COMM_AG: the finished value goes straight into every peer's gathered output.
template <int COMM>
__device__ __forceinline__ void comm_emit(const GemmParams& p, int parity, float g, int m, int n, float scale) {
  (void)parity;
  float v = g * scale;
  if (p.bias != nullptr) v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
  const size_t idx = static_cast<size_t>(m) * p.ldy + p.col_offset + n;
  for (int peer = 0; peer < p.comm.size; ++peer) {
    uint8_t* out = p.comm.base[peer] + p.comm.out_off;
    if (p.out_fp32) reinterpret_cast<float*>(out)[idx] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16(v);
  }
}

template <int TN, bool DUAL, bool SPLIT, int COMM>
__global__ void __launch_bounds__(192, 1)
gemm_wt_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmParams p) {
  using Cfg = GemmCfg<TN, DUAL>;
  pdl_launch_early();
  trace_mark(kTraceGemm, kTraceStart);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);            // [kStages]
  uint64_t* empty_bar = full_bar + Cfg::kStages;                     // [kStages]
  uint64_t* accum_bar = empty_bar + Cfg::kStages;                    // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);  // [1]
  uint8_t* stages = smem + Cfg::kCtrlBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x;
  const int tile_m = blockIdx.y;
  int m_base = tile_m * TN;   // first token row of this tile
  int m_limit = p.M;          // rows >= m_limit are not stored
  int w_row0 = tile_n * 128;  // first weight row of this tile
  if (p.work != nullptr) {
    pdl_wait();  // the work table comes from the routing kernels
    const int4 item = reinterpret_cast<const int4*>(p.work)[tile_m];
    if (item.z <= 0) return;  // uniform over the CTA (and over its cluster: same blockIdx.y)
    m_base = item.y;
    m_limit = item.y + item.z;
    w_row0 += item.x * p.w_rows_per_expert;
    if (p.bias != nullptr)
      p.bias = static_cast<const __nv_bfloat16*>(p.bias) + static_cast<size_t>(item.x) * p.bias_expert_stride;
  }
  const int nsplit = SPLIT ? gridDim.z : 1;
  const int split = SPLIT ? blockIdx.z : 0;

  const int kblocks = (p.K + 63) >> 6;
  const int kb_per = (kblocks + nsplit - 1) / nsplit;
  const int kb0 = split * kb_per;
  const int kb1 = min(kblocks, kb0 + kb_per);
  const int niter = max(0, kb1 - kb0);

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Weight tiles do not depend on the producer kernels: start them before the wait.
  int n_pre = 0;
  if (p.w_static && p.work == nullptr) {
    n_pre = min(niter, Cfg::kStages);
    if (warp == 0 && lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      for (int it = 0; it < niter; ++it) {
        const int kx = (kb0 + it) * 64;
        if (it < n_pre) {
          uint8_t* a = stages + it * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[it], Cfg::kStageBytes);
          tma_load_2d_hint(a, &tmW, kx, w_row0, &full_bar[it], pol_w);
          if (DUAL) tma_load_2d_hint(a + Cfg::kATile, &tmW, kx, p.dual_row_offset + w_row0, &full_bar[it], pol_w);
        } else if (p.w_static > 1) {
          tma_prefetch_l2_2d(&tmW, kx, w_row0);
          if (DUAL) tma_prefetch_l2_2d(&tmW, kx, p.dual_row_offset + w_row0);
        }
      }
    }
  }
  // Everything above touched only this CTA's own resources and constant weights; wait for the producer kernels here.
  pdl_wait();
  trace_mark(kTraceGemm, kTraceAfterWait);
  pdl_launch_dependents();
  unsigned int seq = 0;
  if (COMM != COMM_NONE) seq = *p.comm.seq;
  const int parity = static_cast<int>(seq & 1u);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      int issued = n_pre;
      bool ok = true;
      for (int it = 0; it < niter && ok; ++it) {
        const int s = it % Cfg::kStages;
        const uint32_t ph = (it / Cfg::kStages) & 1;
        uint8_t* a = stages + s * Cfg::kStageBytes;
        const int kx = (kb0 + it) * 64;
        if (it >= n_pre) {  // the first n_pre stages already hold (or are receiving) their weight tiles
          ok = mbar_wait(&empty_bar[s], ph ^ 1, p.status, kStatusSmemEmptyTimeout);
          if (!ok) break;
          mbar_arrive_expect_tx(&full_bar[s], Cfg::kStageBytes);
          tma_load_2d_hint(a, &tmW, kx, w_row0, &full_bar[s], pol_w);
          if (DUAL) tma_load_2d_hint(a + Cfg::kATile, &tmW, kx, p.dual_row_offset + w_row0, &full_bar[s], pol_w);
        }
        tma_load_2d_hint(a + Cfg::kATile * (DUAL ? 2 : 1), &tmX, kx, m_base, &full_bar[s], pol_x);
        issued = it + 1;
      }
      if (!ok) {
        // Give up cleanly: wait (bounded) for the copies still in flight before shared memory dies.
        const int first = max(0, issued - Cfg::kStages);
        for (int it = first; it < issued; ++it) {
          mbar_wait(&full_bar[it % Cfg::kStages], (it / Cfg::kStages) & 1, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, TN);
      bool ok = true;
      for (int it = 0; it < niter; ++it) {
        const int s = it % Cfg::kStages;
        const uint32_t ph = (it / Cfg::kStages) & 1;
        ok = mbar_wait(&full_bar[s], ph, p.status, kStatusTmaFullTimeout);
        if (!ok) break;
        if (it == 0) trace_mark_thread(kTraceGemm, 3, 32);       // first operands landed
        if (it == niter - 1) trace_mark_thread(kTraceGemm, 4, 32);  // last operands landed
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(stages + s * Cfg::kStageBytes);
        const uint64_t da = umma_desc_k_sw128(a_addr);
        const uint64_t da2 = umma_desc_k_sw128(a_addr + Cfg::kATile);
        const uint64_t db = umma_desc_k_sw128(a_addr + Cfg::kATile * (DUAL ? 2 : 1));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          if (DUAL) umma_f16(tmem_base + TN, da2 + 2 * k, db + 2 * k, idesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(accum_bar);
    }
  }
  __syncwarp();  // lanes 1..31 of the producer / MMA warps rejoin lane 0 before any block or cluster barrier

  // ------------------------------------------------------------ epilogue (warps 2..5)
  const int q = warp & 3;  // TMEM lane quarter this warp may read
  const int row = q * 32 + lane;
  const int n = tile_n * 128 + row;
  bool acc_ok = false;
  float* red = reinterpret_cast<float*>(stages);  // SPLIT: [DUAL?2:1][TN][128] fp32, aliases the ring

  __shared__ float s_scale[TN];
  __shared__ float s_ssq[4][TN];
  const int et = threadIdx.x - 64;  // epilogue thread index 0..127 (warps 2..5)
  const bool in_n = n < p.N;
  constexpr bool kCanStage = (TN >= 64) && !SPLIT && COMM == COMM_NONE;
  // Columns (tokens) of the tile whose final value this CTA produces: all of them, or with cluster split-K
  // every nsplit-th one (COMM_AR: every nsplit-th PAIR of columns, because partials travel as bf16x2).
  const int m_end = min(TN, m_limit - m_base);
  const int own_first = SPLIT ? split : 0, own_step = SPLIT ? nsplit : 1;
  constexpr int kPre = 8;
  float rpre[2 * kPre];
#pragma unroll
  for (int j = 0; j < 2 * kPre; ++j) rpre[j] = 0.f;
  const bool has_res = p.residual != nullptr && in_n;

  // Final value of element (column c of the tile, this thread's row): store it (or hand it to the
  // collective) and add its square to the per-column sum kept for a following RMSNorm. Executed by whole warps.
  auto finish = [&](float g, float u, int c, bool valid, float rv) {
    const int m = m_base + c;
    const bool ok = valid && in_n && m < m_limit;
    float v = 0.f;
    if (ok) {
      const float sc = (p.ssq_in != nullptr) ? s_scale[c] : 1.f;
      if (COMM == COMM_NONE) v = epilogue_store<DUAL>(p, g, u, m, n, sc, rv);
      else comm_emit<COMM>(p, parity, g, m, n, sc);
    }
    if (COMM == COMM_NONE && p.ssq_out != nullptr) {
      float sq = v * v;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0) s_ssq[q][c] = sq;
    }
  };
  // After every owned column went through finish(): publish the per-row partial sums of squares.
  auto publish_ssq = [&](int c_first, int c_step) {
    if (p.ssq_out == nullptr) return;
    epi_barrier();
    for (int c = et; c < TN; c += 128) {
      if (c >= c_first && (c - c_first) % c_step == 0 && m_base + c < m_limit)
        p.ssq_out[static_cast<size_t>(m_base + c) * gridDim.x + tile_n] = s_ssq[0][c] + s_ssq[1][c] + s_ssq[2][c] + s_ssq[3][c];
    }
  };

  if (warp >= 2) {
    if (p.ssq_in != nullptr) {
      for (int c = et; c < TN; c += 128) {
        float t = 0.f;
        if (m_base + c < m_limit) {
          const float* src = p.ssq_in + static_cast<size_t>(m_base + c) * p.ssq_parts;
          for (int j = 0; j < p.ssq_parts; ++j) t += src[j];
        }
        s_scale[c] = rsqrtf(t * p.norm_inv_dim + p.norm_eps);
      }
      epi_barrier();
    }
    // Residual values of the first kPre columns (COMM_AR: column pairs) this thread will finish: the loads are
    // in flight while the tensor cores work, instead of one dependent load per finished column.
    if (has_res) {
#pragma unroll
      for (int j = 0; j < kPre; ++j) {
        if (COMM == COMM_AR) {
          const int c = 2 * (own_first + j * own_step);
          if (c < m_end) rpre[2 * j] = residual_at(p, m_base + c, n);
          if (c + 1 < m_end) rpre[2 * j + 1] = residual_at(p, m_base + c + 1, n);
        } else if (SPLIT) {
          const int c = own_first + j * own_step;
          if (c < m_end) rpre[j] = residual_at(p, m_base + c, n);
        }
      }
    }
    acc_ok = (niter > 0) && mbar_wait(accum_bar, 0, p.status, kStatusAccumTimeout);
    acc_ok = __all_sync(0xffffffffu, acc_ok);
    trace_mark_thread(kTraceGemm, 5, 64);  // accumulator complete
    tc_fence_after_sync();
    if (acc_ok) {
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t g[16];
        uint32_t u[16];
        tmem_ld16(taddr + c0, g);
        if (DUAL) tmem_ld16(taddr + TN + c0, u);
        tmem_wait_ld();
        if (SPLIT || COMM == COMM_AR) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            red[(c0 + j) * 128 + row] = __uint_as_float(g[j]);
            if (DUAL) red[(TN + c0 + j) * 128 + row] = __uint_as_float(u[j]);
          }
        } else if (kCanStage && p.staged) {
          // value before the residual, fp32, [column][row]: conflict-free writes, coalesced second pass
          float bg = 0.f, bu = 0.f;
          if (p.bias != nullptr && in_n) {
            const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(p.bias);
            bg = __bfloat162float(b[n]);
            if (DUAL) bu = __bfloat162float(b[p.N + n]);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float sc = (p.ssq_in != nullptr) ? s_scale[c0 + j] : 1.f;
            const float gg = __uint_as_float(g[j]) * sc + bg;
            red[(c0 + j) * 128 + row] = DUAL ? gated_act(p, gg, __uint_as_float(u[j]) * sc + bu) : gg;
          }
        } else {
          float rr[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) rr[j] = (has_res && c0 + j < m_end) ? residual_at(p, m_base + c0 + j, n) : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) finish(__uint_as_float(g[j]), DUAL ? __uint_as_float(u[j]) : 0.f, c0 + j, true, rr[j]);
        }
      }
    }
    if (kCanStage && p.staged) {
      epi_barrier();  // the whole tile is staged (or the accumulator never arrived: nothing is stored)
      if (acc_ok) {
        const int m_cnt = min(TN, m_limit - m_base);
        const int limit = (m_cnt * 16 + 31) & ~31;  // 16 chunks of 8 columns per token row; warp-uniform bound
        const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(p.residual);
        __nv_bfloat16* yout = static_cast<__nv_bfloat16*>(p.y);
        constexpr int kBatch = 4;
        for (int ch0 = et; ch0 < limit; ch0 += 128 * kBatch) {
          uint4 rv[kBatch];
          bool ok[kBatch];
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            const int ch = ch0 + 128 * b;
            const int c = ch >> 4, gn = tile_n * 128 + (ch & 15) * 8;
            ok[b] = ch < limit && c < m_cnt && gn < p.N;
            rv[b] = make_uint4(0u, 0u, 0u, 0u);
            if (ok[b] && res != nullptr) rv[b] = *reinterpret_cast<const uint4*>(res + static_cast<size_t>(m_base + c) * p.ldr + gn);
          }
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            const int ch = ch0 + 128 * b;
            if (ch >= limit) break;  // warp-uniform
            const int c = ch >> 4, n0 = (ch & 15) * 8;
            const float4 a0 = *reinterpret_cast<const float4*>(red + c * 128 + n0);
            const float4 a1 = *reinterpret_cast<const float4*>(red + c * 128 + n0 + 4);
            const uint32_t r[4] = {rv[b].x, rv[b].y, rv[b].z, rv[b].w};
            uint4 o;
            o.x = pack_bf16x2(a0.x + bf16_lo(r[0]), a0.y + bf16_hi(r[0]));
            o.y = pack_bf16x2(a0.z + bf16_lo(r[1]), a0.w + bf16_hi(r[1]));
            o.z = pack_bf16x2(a1.x + bf16_lo(r[2]), a1.y + bf16_hi(r[2]));
            o.w = pack_bf16x2(a1.z + bf16_lo(r[3]), a1.w + bf16_hi(r[3]));
            if (ok[b]) *reinterpret_cast<uint4*>(yout + static_cast<size_t>(m_base + c) * p.ldy + tile_n * 128 + n0) = o;
            if (p.ssq_out != nullptr) {
              const uint32_t w[4] = {o.x, o.y, o.z, o.w};
              float sq = 0.f;
              if (ok[b]) {
#pragma unroll
                for (int j = 0; j < 4; ++j) sq += bf16_lo(w[j]) * bf16_lo(w[j]) + bf16_hi(w[j]) * bf16_hi(w[j]);
              }
#pragma unroll
              for (int o2 = 8; o2 > 0; o2 >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o2);
              if ((lane & 15) == 0 && c < m_cnt) p.ssq_out[static_cast<size_t>(m_base + c) * gridDim.x + tile_n] = sq;
            }
          }
        }
      }
    } else if (!SPLIT && COMM == COMM_NONE) {
      publish_ssq(0, 1);
    }
  }

  if (SPLIT) {
    // Every thread of every CTA of the cluster reaches both barriers, whatever happened above.
    cg::cluster_group cluster = cg::this_cluster();
    trace_mark_thread(kTraceGemm, 6, 64);  // partials staged
    cluster.sync();
    trace_mark_thread(kTraceGemm, 7, 64);  // cluster barrier 1 passed
  }
  if (COMM == COMM_AR) {
    // ---- all-reduce, one shot: every partial pair of token columns is one 4-byte bf16x2 word stored into each
    // peer's sentinel-initialised slot; a word is complete when it differs from the sentinel, so there is no fence,
    // no flag and no barrier between the tensor-core tile and the reduction.
    if (warp >= 2) {
      cg::cluster_group cluster = cg::this_cluster();
      const int p_first = SPLIT ? split : 0, p_step = SPLIT ? nsplit : 1;
      for (int pi = p_first; 2 * pi < m_end; pi += p_step) {
        float g0 = 0.f, g1 = 0.f;
        if (SPLIT) {
          float a0[8], a1[8];
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const float* peer = cluster.map_shared_rank(red, r < nsplit ? r : 0);
            a0[r] = (r < nsplit) ? peer[(2 * pi) * 128 + row] : 0.f;
            a1[r] = (r < nsplit) ? peer[(2 * pi + 1) * 128 + row] : 0.f;
          }
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            g0 += a0[r];
            g1 += a1[r];
          }
        } else {
          g0 = red[(2 * pi) * 128 + row];
          g1 = red[(2 * pi + 1) * 128 + row];
        }
        if (in_n) {
          const uint32_t packed = lamport_payload(pack_bf16x2(g0, g1));
          const size_t word = (static_cast<size_t>(m_base / 2 + pi) * p.N + n) * 4;
          for (int peer = 0; peer < p.comm.size; ++peer) {
            asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(lamport_slot(p.comm, peer, parity, p.comm.rank) + word),
                         "r"(packed)
                         : "memory");
          }
        }
      }
    }
  } else if (SPLIT) {
    if (warp >= 2) {
      cg::cluster_group cluster = cg::this_cluster();
      const float* peers[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) peers[r] = cluster.map_shared_rank(red, r < nsplit ? r : 0);
      // all remote loads of a column are issued together; the sum runs in cluster-rank order (deterministic)
      auto reduce_col = [&](int c, float& g, float& u) {
        float pg[8], pu[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          pg[r] = (r < nsplit) ? peers[r][c * 128 + row] : 0.f;
          if (DUAL) pu[r] = (r < nsplit) ? peers[r][(TN + c) * 128 + row] : 0.f;
        }
        g = 0.f;
        u = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          g += pg[r];
          if (DUAL) u += pu[r];
        }
      };
#pragma unroll
      for (int j = 0; j < kPre; ++j) {
        const int c = split + j * nsplit;
        if (c < m_end) {  // warp-uniform
          float g, u;
          reduce_col(c, g, u);
          finish(g, u, c, true, rpre[j]);
        }
      }
      for (int c = split + kPre * nsplit; c < m_end; c += nsplit) {
        float g, u;
        reduce_col(c, g, u);
        finish(g, u, c, true, has_res ? residual_at(p, m_base + c, n) : 0.f);
      }
      if (COMM == COMM_NONE) publish_ssq(split, nsplit);
    }
  }
  if (SPLIT) {
    cg::cluster_group cluster = cg::this_cluster();
    trace_mark_thread(kTraceGemm, 8, 64);  // reduced and stored
    cluster.sync();
    trace_mark_thread(kTraceGemm, 9, 64);  // cluster barrier 2 passed
  }

  if (COMM == COMM_AR) {
    if (warp >= 2) {
      const int p_first = SPLIT ? split : 0, p_step = SPLIT ? nsplit : 1;
      // Pairs are collected four at a time: the first poll of a chunk issues every (pair, source rank) load before
      // any word is looked at, so one memory round trip usually brings all 32 words; stragglers are re-polled. The
      // single reader of a word writes the sentinel back as soon as it has the value (the slot of this parity is
      // written again two calls later).
      constexpr int kPB = 4;
      for (int pi0 = p_first; 2 * pi0 < m_end; pi0 += kPB * p_step) {
        float r0[kPB], r1[kPB];
        uint32_t lo[kPB][kMaxRanks], miss[kPB];
        size_t word[kPB];
#pragma unroll
        for (int j = 0; j < kPB; ++j) {
          const int pi = pi0 + j * p_step;
          const bool live = in_n && 2 * pi < m_end;
          miss[j] = live ? (1u << p.comm.size) - 1u : 0u;
          word[j] = (static_cast<size_t>(m_base / 2 + pi) * p.N + n) * 4;
          r0[j] = (live && has_res) ? residual_at(p, m_base + 2 * pi, n) : 0.f;
          r1[j] = (live && has_res && 2 * pi + 1 < m_end) ? residual_at(p, m_base + 2 * pi + 1, n) : 0.f;
        }
        const long long t0 = clock64();
        bool first_pass = true;
        while (true) {
          // words still missing are (re)loaded straight into their final registers; a word that is still the sentinel
          // keeps its `miss` bit and is simply loaded again on the next pass
#pragma unroll
          for (int j = 0; j < kPB; ++j) {
#pragma unroll
            for (int src = 0; src < kMaxRanks; ++src) {
              if ((miss[j] >> src) & 1u) {
                asm volatile("ld.volatile.global.u32 %0, [%1];"
                             : "=r"(lo[j][src])
                             : "l"(lamport_slot(p.comm, p.comm.rank, parity, src) + word[j])
                             : "memory");
              }
            }
          }
          uint32_t pending = 0u;
#pragma unroll
          for (int j = 0; j < kPB; ++j) {
#pragma unroll
            for (int src = 0; src < kMaxRanks; ++src) {
              if (((miss[j] >> src) & 1u) && lo[j][src] != kLamportEmpty) {
                miss[j] &= ~(1u << src);
                asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(lamport_slot(p.comm, p.comm.rank, parity, src) + word[j]),
                             "r"(kLamportEmpty)
                             : "memory");
              }
            }
            pending |= miss[j];
          }
          if (pending == 0u) break;
          if (!first_pass && clock64() - t0 > kWaitCycleLimit) {
            report_status(p.status, kStatusPeerFlagTimeout);
            break;
          }
          first_pass = false;
        }
#pragma unroll
        for (int j = 0; j < kPB; ++j) {
          const int pi = pi0 + j * p_step;
          if (2 * pi >= m_end) break;  // warp-uniform
          float v0 = 0.f, v1 = 0.f;
          if (in_n) {
#pragma unroll
            for (int src = 0; src < kMaxRanks; ++src) {  // rank order: every rank computes the same bits
              if (src < p.comm.size && !((miss[j] >> src) & 1u)) {
                v0 += bf16_lo(lo[j][src]);
                v1 += bf16_hi(lo[j][src]);
              }
            }
            v0 = epilogue_store<false>(p, v0, 0.f, m_base + 2 * pi, n, 1.f, r0[j]);
            v1 = (2 * pi + 1 < m_end) ? epilogue_store<false>(p, v1, 0.f, m_base + 2 * pi + 1, n, 1.f, r1[j]) : 0.f;
          }
          if (p.ssq_out != nullptr) {
            float s0 = in_n ? v0 * v0 : 0.f, s1 = in_n ? v1 * v1 : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              s0 += __shfl_xor_sync(0xffffffffu, s0, o);
              s1 += __shfl_xor_sync(0xffffffffu, s1, o);
            }
            if (lane == 0) {
              s_ssq[q][2 * pi] = s0;
              if (2 * pi + 1 < TN) s_ssq[q][2 * pi + 1] = s1;
            }
          }
        }
      }
      // publish the sums of squares of the columns this CTA finished (pairs p_first, p_first + p_step, ...)
      if (p.ssq_out != nullptr) {
        epi_barrier();
        for (int c = et; c < m_end; c += 128) {
          const int pi = c >> 1;
          if (pi >= p_first && (pi - p_first) % p_step == 0)
            p.ssq_out[static_cast<size_t>(m_base + c) * gridDim.x + tile_n] = s_ssq[0][c] + s_ssq[1][c] + s_ssq[2][c] + s_ssq[3][c];
        }
      }
    }
  } else if (COMM == COMM_AG) {
    // ---- all-gather: publish this CTA's stores with one flag per peer, wait for the peers' same tile
    const int flag_id = ((tile_n * gridDim.y + tile_m) * (SPLIT ? 8 : 1) + split) % kMaxFlags;
    const bool has_share = (SPLIT ? split : 0) < m_end;
    if (warp >= 2 && has_share) {
      epi_barrier();
      if (et < p.comm.size) {
        __threadfence_system();
        st_release_sys(peer_flag(p.comm, et, parity, p.comm.rank, flag_id), seq + 1u);
        wait_flag(p.comm, parity, et, flag_id, seq + 1u, p.status);
      }
      epi_barrier();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (COMM != COMM_NONE && threadIdx.x == 0) finish_call(p.comm, seq, gridDim.x * gridDim.y * gridDim.z);
  trace_mark(kTraceGemm, kTraceEnd);
}

template <int TN, bool DUAL, bool SPLIT, int COMM = COMM_NONE>
static cudaError_t launch_gemm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int n_tiles,
                               int m_tiles, int nsplit, cudaStream_t stream) {
  using Cfg = GemmCfg<TN, DUAL>;
  auto kern = gemm_wt_kernel<TN, DUAL, SPLIT, COMM>;
  static bool configured[64] = {};  // the attribute is a per-device setting
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return ce;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (ce != cudaSuccess) return ce;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, m_tiles, nsplit);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (pdl_enabled()) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (SPLIT) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = 1;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = nsplit;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p);
}

template <int TN, bool DUAL, int COMM = COMM_NONE>
static cudaError_t launch_gemm_split(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                                     int n_tiles, int m_tiles, int nsplit, cudaStream_t stream) {
  if (nsplit > 1) {
    if constexpr (TN <= 64) return launch_gemm<TN, DUAL, true, COMM>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream);
  }
  return launch_gemm<TN, DUAL, false, COMM>(tmW, tmX, p, n_tiles, m_tiles, 1, stream);
}

}  // namespace eredu

using namespace eredu;

EREDU_TRACE_INSTALLER(gemm)

// EREDU_GEMM_PERSISTENT=0 keeps prefill-sized GEMMs on the one-tile-per-CTA kernel (for A/B measurements).
static bool persistent_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("EREDU_GEMM_PERSISTENT");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

static int prefetch_level(long long weight_bytes) {
  static int forced = -2;
  if (forced == -2) {
    const char* e = std::getenv("EREDU_GEMM_PREFETCH");
    forced = (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : -1;
  }
  if (forced >= 0) return forced;
  return weight_bytes <= (16LL << 20) ? 2 : 1;
}

static bool staged_epilogue_ok(const void* Y, const void* residual, int N, int ldy, int ldr, int out_fp32) {
  if (out_fp32 || N % 8 != 0 || ldy % 8 != 0 || (reinterpret_cast<uintptr_t>(Y) & 15) != 0) return false;
  if (residual != nullptr && (ldr % 8 != 0 || (reinterpret_cast<uintptr_t>(residual) & 15) != 0)) return false;
  return true;
}

// Number of K splits the launcher would use (exposed for tests and tuning).
extern "C" int eredu_gemm_pick_split(int M, int N, int K, int sm_count) {
  const int tn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  if (tn > 64) return 1;
  const int tiles = ((N + 127) / 128) * ((M + tn - 1) / tn);
  const int kblocks = (K + 63) / 64;
  int s = 1;
  // Split while the grid still fits two CTAs per SM: besides streaming the weights in parallel, a split CTA
  // finishes only every s-th token column, and the serial per-column epilogue is what a small GEMM pays for.
  while (s < 8 && tiles * s * 2 <= 2 * sm_count && kblocks / (s * 2) >= 2) s *= 2;
  return s;
}

// Y = X W^T (+bias) (+residual), or with dual != 0: Y = silu(X Wg^T) * (X Wu^T) where Wg = W[0:N],
// Wu = W[dual_row_offset : dual_row_offset+N]. X: [M,K] bf16 (row stride ldx), W: [rows,K] bf16 (row
// stride ldw). `force_split` > 0 overrides the split-K heuristic (1,2,4,8). With `ssq_in` the output rows are
// scaled by rsqrt(sum(ssq_in[m, 0:ssq_parts]) / norm_dim + norm_eps) (RMSNorm whose weights were folded into
// W); with `ssq_out` ([M, ceil(N/128)] fp32) the kernel also writes per-tile sums of squares of the stored
// output for the next such GEMM. Returns a cudaError_t or a negative tensor-map error.
extern "C" int eredu_gemm_bf16(const void* X, const void* W, void* Y, const void* residual, const void* bias, int M,
                               int N, int K, int ldx, int ldw, int ldy, int ldr, int w_rows, int dual,
                               int dual_row_offset, int out_fp32, int force_split, int sm_count, int* status,
                               const float* ssq_in, int ssq_parts, float norm_eps, int norm_dim, float* ssq_out,
                               int flags, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int tn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  if (tn == 256 && !out_fp32 && force_split <= 1 && persistent_enabled()) {
    // prefill-sized: persistent kernel with double-buffered accumulators
    const int pr = launch_gemm_persistent(X, W, Y, residual, bias, M, N, K, ldx, ldw, ldy, ldr, w_rows, dual, dual_row_offset,
                                          sm_count, status, ssq_in, ssq_parts, norm_eps, norm_dim, ssq_out, stream);
    if (pr != kPersistentUnsupported) return pr;
  }
  CUtensorMap tmW, tmX;
  int r = make_tma_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_rows, K, ldw, 128, 64);
  if (r != 0) return -100 + r;
  r = make_tma_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, tn, 64);
  if (r != 0) return -200 + r;
  GemmParams p;
  p.y = Y;
  p.residual = residual;
  p.bias = bias;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.ldr = ldr;
  p.dual_row_offset = dual_row_offset;
  p.out_fp32 = out_fp32;
  p.status = status;
  p.col_offset = 0;
  p.ssq_in = ssq_in;
  p.ssq_parts = ssq_parts;
  p.norm_eps = norm_eps;
  p.norm_inv_dim = norm_dim > 0 ? 1.0f / static_cast<float>(norm_dim) : 0.f;
  p.ssq_out = ssq_out;
  p.work = nullptr;
  p.w_rows_per_expert = 0;
  p.staged = 0;
  p.act = 0;
  p.act_limit = 0.f;
  p.bias_expert_stride = 0;
  // flag bit 0: W was produced by a preceding kernel of the stream (no early fetch at all). Otherwise the ring's
  // first stages are fetched before the dependency wait (level 1), and for matrices that fit L2 many times over
  // the remaining tiles are prefetched into L2 as well (level 2). EREDU_GEMM_PREFETCH overrides the level.
  p.w_static = (flags & 1) ? 0 : prefetch_level(static_cast<long long>(w_rows) * K * 2);
  const int n_tiles = (N + 127) / 128;
  const int m_tiles = (M + tn - 1) / tn;
  int nsplit = force_split > 0 ? force_split : eredu_gemm_pick_split(M, N, K, sm_count > 0 ? sm_count : 148);
  const int kblocks = (K + 63) / 64;
  while (nsplit > 1 && (kblocks + nsplit - 1) / nsplit * (nsplit - 1) >= kblocks) nsplit >>= 1;  // no empty split
  p.staged = staged_epilogue_ok(Y, residual, N, ldy, ldr, out_fp32) && tn >= 64 && nsplit == 1;
  cudaError_t e;
#define ER_DISPATCH(TN_)                                                                     \
  case TN_:                                                                                  \
    e = dual ? launch_gemm_split<TN_, true>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream)   \
             : launch_gemm_split<TN_, false>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream); \
    break;
  switch (tn) {
    ER_DISPATCH(16)
    ER_DISPATCH(32)
    ER_DISPATCH(64)
    ER_DISPATCH(128)
    default:
      // DUAL with 256-token tiles would need 512 TMEM columns and a 2-stage ring; use 128-token tiles.
      if (dual) {
        CUtensorMap tmX2;
        r = make_tma_2d(&tmX2, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, 128, 64);
        if (r != 0) return -200 + r;
        e = launch_gemm_split<128, true>(tmW, tmX2, p, n_tiles, (M + 127) / 128, 1, stream);
      } else {
        e = launch_gemm_split<256, false>(tmW, tmX, p, n_tiles, m_tiles, 1, stream);
      }
      break;
  }
#undef ER_DISPATCH
  eredu_count_launches(1);
  return static_cast<int>(e);
}

// Row-parallel (mode 1: GEMM + all-reduce) or column-parallel (mode 2: GEMM + all-gather) linear layer of a
// tensor-parallel group, collective fused into the epilogue over NVLink peer memory. M <= 64 tokens.
//   mode 1: X [M, K_local], W [N, K_local]; Y [M, N] (local, bf16/fp32) = sum over ranks (+bias +residual).
//   mode 2: X [M, K], W [N_local, K]; the gathered [M, ldy] result lands in every rank's symmetric `out`
//           region at column `col_offset` (+bias); Y is unused.
// `comm` points to a host PeerComm (see eredu_comm_create). Every rank of the group must call this with the
// same shapes in the same order.
extern "C" int eredu_gemm_bf16_comm(const void* X, const void* W, void* Y, const void* residual, const void* bias,
                                    int M, int N, int K, int ldx, int ldw, int ldy, int ldr, int w_rows, int out_fp32,
                                    int mode, int col_offset, const void* comm, int force_split, int sm_count,
                                    int* status, const float* ssq_in, int ssq_parts, float norm_eps, int norm_dim,
                                    float* ssq_out, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 64 || comm == nullptr || (mode != COMM_AR && mode != COMM_AG)) return -1;
  const PeerComm* pc = static_cast<const PeerComm*>(comm);
  const int tn = M <= 16 ? 16 : M <= 32 ? 32 : 64;
  CUtensorMap tmW, tmX;
  int r = make_tma_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_rows, K, ldw, 128, 64);
  if (r != 0) return -100 + r;
  r = make_tma_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, tn, 64);
  if (r != 0) return -200 + r;
  GemmParams p;
  p.y = Y;
  p.residual = residual;
  p.bias = bias;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.ldr = ldr;
  p.dual_row_offset = 0;
  p.out_fp32 = out_fp32;
  p.status = status;
  p.col_offset = col_offset;
  p.ssq_in = ssq_in;
  p.ssq_parts = ssq_parts;
  p.norm_eps = norm_eps;
  p.norm_inv_dim = norm_dim > 0 ? 1.0f / static_cast<float>(norm_dim) : 0.f;
  p.ssq_out = ssq_out;
  p.work = nullptr;
  p.w_rows_per_expert = 0;
  p.staged = 0;
  p.act = 0;
  p.act_limit = 0.f;
  p.bias_expert_stride = 0;
  p.w_static = prefetch_level(static_cast<long long>(w_rows) * K * 2);
  p.comm = *pc;
  const int n_tiles = (N + 127) / 128;
  const int m_tiles = 1;
  if (mode == COMM_AR && static_cast<long long>((M + 1) / 2) * N * 4 > pc->lam_bytes) return -2;
  int nsplit = force_split > 0 ? force_split : eredu_gemm_pick_split(M, N, K, sm_count > 0 ? sm_count : 148);
  const int kblocks = (K + 63) / 64;
  while (nsplit > 1 && (kblocks + nsplit - 1) / nsplit * (nsplit - 1) >= kblocks) nsplit >>= 1;
  if (mode == COMM_AG && n_tiles * (nsplit > 1 ? 8 : 1) > kMaxFlags) return -3;
  cudaError_t e;
#define ER_COMM(TN_)                                                                                        \
  case TN_:                                                                                                 \
    e = mode == COMM_AR ? launch_gemm_split<TN_, false, COMM_AR>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream) \
                        : launch_gemm_split<TN_, false, COMM_AG>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream); \
    break;
  switch (tn) {
    ER_COMM(16)
    ER_COMM(32)
    default:
      e = mode == COMM_AR ? launch_gemm_split<64, false, COMM_AR>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream)
                          : launch_gemm_split<64, false, COMM_AG>(tmW, tmX, p, n_tiles, m_tiles, nsplit, stream);
      break;
  }
#undef ER_COMM
  eredu_count_launches(1);
  return static_cast<int>(e);
}

// Grouped (mixture-of-experts) linear layer. X: [rows_cap, K] token rows already permuted so that each
// expert's tokens are contiguous; W: [n_experts * rows_per_expert, K] (expert-major); `work`: device table of
// n_work int4 items {expert, row0, rows, 0} (rows <= tile, rows == 0 = unused item), built without a host
// round trip; `tile` = 16/32/64/128: token rows per item. dual: gate rows then up rows inside each expert
// block (dual_row_offset = N). Y: [rows_cap, N].
extern "C" int eredu_gemm_bf16_grouped(const void* X, const void* W, void* Y, const int* work, int n_work, int tile,
                                       int rows_cap, int N, int K, int ldx, int ldw, int ldy, int w_rows_total,
                                       int w_rows_per_expert, int dual, int force_split, int sm_count, int* status,
                                       const void* bias, int bias_expert_stride, int act, float act_limit,
                                       cudaStream_t stream) {
  if (n_work <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap tmW, tmX;
  int r = make_tma_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_rows_total, K, ldw, 128, 64);
  if (r != 0) return -100 + r;
  r = make_tma_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_cap, K, ldx, tile, 64);
  if (r != 0) return -200 + r;
  GemmParams p = {};
  p.y = Y;
  p.M = rows_cap;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.dual_row_offset = N;
  p.status = status;
  p.work = work;
  p.w_rows_per_expert = w_rows_per_expert;
  p.bias = bias;  // per expert: [w_rows_per_expert] (dual: gate part then up part), bias_expert_stride apart
  p.bias_expert_stride = bias_expert_stride;
  p.act = act;
  p.act_limit = act_limit;
  const int n_tiles = (N + 127) / 128;
  const int kblocks = (K + 63) / 64;
  int nsplit = 1;
  if (tile <= 64) {
    nsplit = force_split > 0 ? force_split : 1;
    if (force_split <= 0) {
      const int sm = sm_count > 0 ? sm_count : 148;
      while (nsplit < 8 && n_tiles * n_work * nsplit * 2 <= 2 * sm && kblocks / (nsplit * 2) >= 2) nsplit *= 2;
    }
    while (nsplit > 1 && (kblocks + nsplit - 1) / nsplit * (nsplit - 1) >= kblocks) nsplit >>= 1;
  }
  p.staged = staged_epilogue_ok(Y, nullptr, N, ldy, 0, 0) && tile >= 64 && nsplit == 1;
  cudaError_t e;
#define ER_GROUPED(TN_)                                                                      \
  case TN_:                                                                                  \
    e = dual ? launch_gemm_split<TN_, true>(tmW, tmX, p, n_tiles, n_work, nsplit, stream)    \
             : launch_gemm_split<TN_, false>(tmW, tmX, p, n_tiles, n_work, nsplit, stream);  \
    break;
  switch (tile) {
    ER_GROUPED(16)
    ER_GROUPED(32)
    ER_GROUPED(64)
    ER_GROUPED(128)
    default: return -1;
  }
#undef ER_GROUPED
  eredu_count_launches(1);
  return static_cast<int>(e);
}
