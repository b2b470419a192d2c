// Persistent tcgen05 GEMM for prefill-sized problems (more than 128 tokens): Y = X W^T with the same fused
// epilogues as the one-tile-per-CTA kernel (RMSNorm row scale, bias, residual, SwiGLU, sums of squares for the
// next norm), built so that the tensor cores never wait for an epilogue:
//
//   * one CTA per SM walks a list of [128 weight rows x 256 tokens] tiles (swap-AB: the weight tile is the MMA M
//     operand, the token tile the MMA N operand);
//   * the fp32 accumulator is double-buffered in TMEM (2 x 256 columns): while the epilogue warps drain tile i,
//     the MMA warp already accumulates tile i+1;
//   * a 4-stage TMA ring (48 KB per stage) runs ahead across tile boundaries;
//   * the epilogue transposes through a 16 KB staging buffer so that Y leaves the SM as 16-byte row chunks;
//   * SwiGLU ("dual") tiles load 64 gate rows and 64 up rows into ONE 128-row operand tile, so gate and up use the
//     same single 128x256 MMA stream as a plain GEMM; silu(gate) * up is formed when the staged rows are combined.
//
// Replaces the cuBLASLt matmul behind the reference's dense projections at prefill sizes
// (eredu-architectures/src/llama.rs:270-286,418-431; safemlx/src/ops/arithmetic.rs matmul).
#include "gemm_persistent.h"

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "../common/trace.cuh"

namespace eredu {

namespace {

constexpr int kTN = 256;                         // tokens per tile (MMA N)
constexpr int kStages = 4;
constexpr int kATile = 128 * 64 * 2;             // 16 KB: 128 weight rows x 64 k
constexpr int kBTile = kTN * 64 * 2;             // 32 KB: 256 tokens x 64 k
constexpr int kStageBytes = kATile + kBTile;     // 48 KB
constexpr int kStagingBytes = 16 * 1024;
constexpr int kCtrlBytes = 1024;
constexpr int kSmemBytes = 1024 + kCtrlBytes + kStages * kStageBytes + kStagingBytes;

struct PGemmParams {
  void* y;
  const void* residual;
  const void* bias;
  int M, N, K;
  int ldy, ldr;
  int dual_row_offset;
  int* status;
  const float* ssq_in;
  int ssq_parts;
  float norm_eps;
  float norm_inv_dim;
  float* ssq_out;
  int n_tiles, m_tiles;
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

template <bool DUAL>
__global__ void __launch_bounds__(192, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, PGemmParams p) {
  pdl_launch_early();
  trace_mark(kTraceGemmPersistent, kTraceStart);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);   // [kStages]  TMA -> MMA
  uint64_t* empty_bar = full_bar + kStages;                 // [kStages]  MMA -> TMA
  uint64_t* tfull_bar = empty_bar + kStages;                // [2]        MMA -> epilogue (accumulator ready)
  uint64_t* tempty_bar = tfull_bar + 2;                     // [2]        epilogue -> MMA (accumulator drained)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  uint8_t* stages = smem + kCtrlBytes;
  uint8_t* staging = stages + kStages * kStageBytes;
  __shared__ float s_scale[kTN];
  __shared__ int s_fail;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kblocks = (p.K + 63) >> 6;
  const int total = p.n_tiles * p.m_tiles;
  constexpr int kRowsPerTile = DUAL ? 64 : 128;  // output columns (weight rows of the result) per tile

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 128);
    }
    s_fail = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  trace_mark(kTraceGemmPersistent, kTraceAfterWait);
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_last();   // both operands are re-read by other CTAs from L2
      const uint64_t pol_x = l2_policy_evict_last();
      int it = 0, issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int tile_m = t / p.n_tiles, tile_n = t % p.n_tiles;
        const int w_row0 = tile_n * kRowsPerTile, m_base = tile_m * kTN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          ok = mbar_wait(&empty_bar[s], ph ^ 1, p.status, kStatusSmemEmptyTimeout);
          if (!ok) break;
          uint8_t* a = stages + s * kStageBytes;
          mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
          if (DUAL) {
            tma_load_2d_hint(a, &tmW, kb * 64, w_row0, &full_bar[s], pol_w);
            tma_load_2d_hint(a + kATile / 2, &tmW, kb * 64, p.dual_row_offset + w_row0, &full_bar[s], pol_w);
          } else {
            tma_load_2d_hint(a, &tmW, kb * 64, w_row0, &full_bar[s], pol_w);
          }
          tma_load_2d_hint(a + kATile, &tmX, kb * 64, m_base, &full_bar[s], pol_x);
          issued = it + 1;
        }
      }
      if (!ok) {  // wait (bounded) for the copies still in flight before shared memory goes away
        for (int j = max(0, issued - kStages); j < issued; ++j) mbar_wait(&full_bar[j % kStages], (j / kStages) & 1, nullptr, 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, kTN);
      int it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++lt) {
        const int buf = lt & 1;
        const uint32_t bph = (lt >> 1) & 1;
        ok = mbar_wait(&tempty_bar[buf], bph ^ 1, p.status, kStatusAccumTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc_addr = tmem_base + buf * kTN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          ok = mbar_wait(&full_bar[s], ph, p.status, kStatusTmaFullTimeout);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(stages + s * kStageBytes);
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + kATile);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(acc_addr, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;   // accumulator lane = weight row inside the tile
    const int et = threadIdx.x - 64;
    const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(p.residual);
    const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(p.bias);
    __nv_bfloat16* yout = static_cast<__nv_bfloat16*>(p.y);
    int lt = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++lt) {
      const int tile_m = t / p.n_tiles, tile_n = t % p.n_tiles;
      const int m_base = tile_m * kTN;
      const int m_cnt = min(kTN, p.M - m_base);
      const int buf = lt & 1;
      const uint32_t bph = (lt >> 1) & 1;
      if (p.ssq_in != nullptr) {
        for (int c = et; c < kTN; c += 128) {
          float s = 0.f;
          if (c < m_cnt) {
            const float* src = p.ssq_in + static_cast<size_t>(m_base + c) * p.ssq_parts;
            for (int j = 0; j < p.ssq_parts; ++j) s += src[j];
          }
          s_scale[c] = rsqrtf(s * p.norm_inv_dim + p.norm_eps);
        }
      }
      if (!mbar_wait(&tfull_bar[buf], bph, p.status, kStatusAccumTimeout)) s_fail = 1;
      epi_bar();  // s_scale is complete; the failure flag is agreed on by all epilogue threads
      if (s_fail) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + buf * kTN + (static_cast<uint32_t>(q * 32) << 16);
      // this thread's weight row: output column n (DUAL: gate rows are lanes 0..63, up rows lanes 64..127)
      const int n = DUAL ? tile_n * 64 + (row & 63) : tile_n * 128 + row;
      const bool in_n = n < p.N;
      float b_row = 0.f;
      if (bias != nullptr && in_n) b_row = __bfloat162float(bias[DUAL && row >= 64 ? p.N + n : n]);
      constexpr int kChunkCols = 32;  // tokens per staging pass: 32 x 128 fp32 = 16 KB
      const int last_cc = ((m_cnt - 1) / kChunkCols) * kChunkCols;  // chunks past the last token are skipped
      for (int cc = 0; cc <= last_cc; cc += kChunkCols) {
        // Second-pass work items of this thread (16-byte pieces of output rows); their residual is fetched now
        // so that the loads are in flight while the accumulator is read.
        constexpr int kItems = DUAL ? 2 : 4;
        uint4 rv[kItems];
        bool item_ok[kItems];
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
          const int id = et + 128 * i;
          const int c = DUAL ? id >> 3 : id >> 4;
          const int gn = DUAL ? tile_n * 64 + (id & 7) * 8 : tile_n * 128 + (id & 15) * 8;
          item_ok[i] = cc + c < m_cnt && gn < p.N;
          rv[i] = make_uint4(0u, 0u, 0u, 0u);
          if (item_ok[i] && res != nullptr) rv[i] = *reinterpret_cast<const uint4*>(res + static_cast<size_t>(m_base + cc + c) * p.ldr + gn);
        }
        float* stf = reinterpret_cast<float*>(staging);
#pragma unroll
        for (int c0 = 0; c0 < kChunkCols; c0 += 16) {
          uint32_t g[16];
          tmem_ld16(taddr + cc + c0, g);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float sc = (p.ssq_in != nullptr) ? s_scale[cc + c0 + j] : 1.f;
            stf[(c0 + j) * 128 + row] = __uint_as_float(g[j]) * sc + b_row;
          }
        }
        if (cc == last_cc) {
          // this thread has read everything it needs from TMEM: hand the accumulator back to the MMA warp
          tc_fence_before_sync();
          mbar_arrive(&tempty_bar[buf]);
        }
        epi_bar();
        const float* st = reinterpret_cast<const float*>(staging);
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
          const int id = et + 128 * i;
          const int c = DUAL ? id >> 3 : id >> 4;
          const int n0 = DUAL ? (id & 7) * 8 : (id & 15) * 8;
          const int m = m_base + cc + c;
          const int gn = tile_n * kRowsPerTile + n0;
          const float4 g0 = *reinterpret_cast<const float4*>(st + c * 128 + n0);
          const float4 g1 = *reinterpret_cast<const float4*>(st + c * 128 + n0 + 4);
          float v[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
          if (DUAL) {
            const float4 u0 = *reinterpret_cast<const float4*>(st + c * 128 + 64 + n0);
            const float4 u1 = *reinterpret_cast<const float4*>(st + c * 128 + 64 + n0 + 4);
            const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = silu_f(v[j]) * u[j];
          }
          const uint32_t r[4] = {rv[i].x, rv[i].y, rv[i].z, rv[i].w};
          uint4 o;
          o.x = pack_bf16x2(v[0] + bf16_lo(r[0]), v[1] + bf16_hi(r[0]));
          o.y = pack_bf16x2(v[2] + bf16_lo(r[1]), v[3] + bf16_hi(r[1]));
          o.z = pack_bf16x2(v[4] + bf16_lo(r[2]), v[5] + bf16_hi(r[2]));
          o.w = pack_bf16x2(v[6] + bf16_lo(r[3]), v[7] + bf16_hi(r[3]));
          if (item_ok[i]) *reinterpret_cast<uint4*>(yout + static_cast<size_t>(m) * p.ldy + gn) = o;
          if (!DUAL && p.ssq_out != nullptr) {
            const uint32_t w[4] = {o.x, o.y, o.z, o.w};
            float sq = 0.f;
            if (item_ok[i]) {
#pragma unroll
              for (int j = 0; j < 4; ++j) sq += bf16_lo(w[j]) * bf16_lo(w[j]) + bf16_hi(w[j]) * bf16_hi(w[j]);
            }
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o2);
            if ((lane & 15) == 0 && cc + c < m_cnt) p.ssq_out[static_cast<size_t>(m) * p.n_tiles + tile_n] = sq;
          }
        }
        epi_bar();  // staging may be overwritten
      }
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
  trace_mark(kTraceGemmPersistent, kTraceEnd);
}

}  // namespace

int launch_gemm_persistent(const void* X, const void* W, void* Y, const void* residual, const void* bias, int M, int N,
                           int K, int ldx, int ldw, int ldy, int ldr, int w_rows, int dual, int dual_row_offset,
                           int sm_count, int* status, const float* ssq_in, int ssq_parts, float norm_eps, int norm_dim,
                           float* ssq_out, cudaStream_t stream) {
  if (N % 8 != 0 || ldy % 8 != 0 || (reinterpret_cast<uintptr_t>(Y) & 15) != 0) return kPersistentUnsupported;
  if (dual && (ssq_out != nullptr || N % 64 != 0 || dual_row_offset % 8 != 0)) return kPersistentUnsupported;
  if (residual != nullptr && (ldr % 8 != 0 || (reinterpret_cast<uintptr_t>(residual) & 15) != 0)) return kPersistentUnsupported;
  CUtensorMap tmW, tmX;
  int r = make_tma_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_rows, K, ldw, dual ? 64 : 128, 64);
  if (r != 0) return -100 + r;
  r = make_tma_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, kTN, 64);
  if (r != 0) return -200 + r;
  PGemmParams p = {};
  p.y = Y;
  p.residual = residual;
  p.bias = bias;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.ldr = ldr;
  p.dual_row_offset = dual_row_offset;
  p.status = status;
  p.ssq_in = ssq_in;
  p.ssq_parts = ssq_parts;
  p.norm_eps = norm_eps;
  p.norm_inv_dim = norm_dim > 0 ? 1.0f / static_cast<float>(norm_dim) : 0.f;
  p.ssq_out = ssq_out;
  p.n_tiles = dual ? (N + 63) / 64 : (N + 127) / 128;
  p.m_tiles = (M + kTN - 1) / kTN;
  const int total = p.n_tiles * p.m_tiles;
  const int sms = sm_count > 0 ? sm_count : 148;
  // equal rounds for every CTA where possible: ceil(total / rounds) CTAs, never more than the SM count
  const int rounds = (total + sms - 1) / sms;
  const int grid = (total + rounds - 1) / rounds;
  auto launch = [&](auto kern) -> cudaError_t {
    static bool configured_plain = false, configured_dual = false;
    bool& configured = dual ? configured_dual : configured_plain;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e != cudaSuccess) return e;
      configured = true;
    }
    return launch_pdl(kern, dim3(grid), dim3(192), kSmemBytes, stream, tmW, tmX, p);
  };
  const cudaError_t e = dual ? launch(gemm_persistent_kernel<true>) : launch(gemm_persistent_kernel<false>);
  eredu_count_launches(1);
  return static_cast<int>(e);
}

}  // namespace eredu

EREDU_TRACE_INSTALLER(gemm_persistent)
