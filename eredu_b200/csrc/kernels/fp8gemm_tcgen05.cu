// Block-scaled FP8 GEMM on the FP8 tensor cores: Y = (Xq * sx) (Wq * sw)^T (+bias) (+residual).
//
//   Xq  E4M3 [M, K] with one fp32 scale per row per 128 input columns, table sx_t [K/128, ld_sx] with ld_sx = M rounded
//       up to 128 (dynamic quantisation of the bf16 activations, act_quant_fp8_kernel below: scale = max(|x|, 1e-4) / 448, as the reference's
//       block_fp8_activation_quantization kernel, eredu/src/backend/mlx/nn/fp8.rs:291-323)
//   Wq  E4M3 [N, K] with one fp32 scale per 128 x 128 block, table sw [K/128, N/128] (the checkpoint's own blocks;
//       eredu/src/backend/mlx/nn/fp8.rs:330-345 is the decoding rule)
//
// The scales differ from one 128-wide K block to the next, so the tensor core cannot sum over the whole K: every K block
// is one tcgen05.mma.kind::f8f6f4 group (four K = 32 instructions) into its own tensor-memory buffer, and the epilogue
// warps fold each partial tile into fp32 registers with the factor sx[m, kb] * sw[kb, tile] (one FMA per element per K
// block). Four 128-column buffers rotate, so the tensor core runs up to three K blocks ahead of the folding.
//
// One CTA per 128 x 128 output tile (m fastest, so CTAs that are resident together share the B tile in L2):
//   warp 0      TMA producer: A and B tiles of 128 rows x 128 bytes, 128-byte swizzled, six stages; with every stage the
//               128 activation scales of that K block (one 512-byte bulk copy into a 16-deep ring: the folding warps read a
//               K block's scales up to four accumulator buffers after its operand stage was handed back)
//   warp 1      MMA issuer (one thread)
//   warps 2..9  folding and store: lane quarter = warp % 4 (rows), column half = (warp - 2) / 4; a thread owns 64
//               columns of one output row
// Every wait is bounded; on expiry the status word is set and the CTA leaves through the common exit.
//
// Measured (B200, M = 8192): 1.1-1.3 PFLOP/s, i.e. 0.8-0.98 of this repository's bf16 tcgen05 GEMM on the same shapes, and
// ahead of it only around 512 tokens. Folding reads every partial tile out of tensor memory once per K block (64 KB per
// 128 x 128 x 128 block), and that read path, not the tensor pipe (27 % active under ncu) nor instruction issue (27 %),
// sets the pace: sixteen folding warps with the next block's loads in flight were slower (0.7 PFLOP/s) than these eight.
// The form that would pass the bf16 kernel keeps the sum over K inside the tensor core with power-of-two block scales
// (the block-scaled MMA kinds); weight scales of block-FP8 checkpoints are arbitrary fp32 values, so that needs a
// re-encoding of the weights and is not built.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/tma_host.h"

namespace eredu {

struct Fp8GemmParams {
  const float* sx_t;            // [K/128, ld_sx]
  int ld_sx;                    // M rounded up to a multiple of 128
  const float* sw;              // [K/128, N/128]
  void* y;                      // bf16 or fp32 [M, ldy]
  const __nv_bfloat16* residual;
  const __nv_bfloat16* bias;
  int M, N, K;
  int ldy, ldr;
  int out_fp32;
  int* status;
};

constexpr int kF8Threads = 320;
constexpr int kF8Stages = 6;
constexpr int kF8Tile = 128 * 128;      // one operand tile: 128 rows x 128 E4M3 bytes
constexpr int kF8ScaleRing = 16;        // > stages + accumulator buffers
constexpr int kF8MaxKBlocks = 512;      // weight scales of one tile column, staged once
constexpr int kF8Smem = 1024 + kF8Stages * 2 * kF8Tile + kF8ScaleRing * 512 + kF8MaxKBlocks * 4 + 256;

__device__ __forceinline__ void f8_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
constexpr uint32_t kF8Idesc = umma_idesc_e4m3(128, 128);

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  float* sx_s = reinterpret_cast<float*>(smem + kF8Stages * 2 * kF8Tile);       // [ring][128]
  float* sw_s = sx_s + kF8ScaleRing * 128;                                     // [kblocks]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sw_s + kF8MaxKBlocks);
  uint64_t* full = bars;                        // [stages]
  uint64_t* empty = bars + kF8Stages;           // [stages]
  uint64_t* acc_full = bars + 2 * kF8Stages;    // [4]
  uint64_t* acc_empty = acc_full + 4;           // [4], one arrival per folding warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 4);

  pdl_launch_early();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_m = blockIdx.x, tile_n = blockIdx.y;
  const int kblocks = p.K / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 8);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int s = kb % kF8Stages;
        if (kb >= kF8Stages) ok = mbar_wait(&empty[s], ((kb / kF8Stages) - 1) & 1, p.status, kStatusSmemEmptyTimeout);
        if (!ok) break;
        uint8_t* st = smem + s * 2 * kF8Tile;
        mbar_arrive_expect_tx(&full[s], 2 * kF8Tile + 512);
        f8_bulk_load(sx_s + (kb % kF8ScaleRing) * 128, p.sx_t + static_cast<size_t>(kb) * p.ld_sx + tile_m * 128, 512, &full[s]);
        tma_load_2d(st, &tmA, kb * 128, tile_m * 128, &full[s]);
        tma_load_2d(st + kF8Tile, &tmB, kb * 128, tile_n * 128, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int s = kb % kF8Stages, buf = kb & 3;
        ok = mbar_wait(&full[s], (kb / kF8Stages) & 1, p.status, kStatusTmaFullTimeout);
        if (ok && kb >= 4) ok = mbar_wait(&acc_empty[buf], ((kb >> 2) - 1) & 1, p.status, kStatusAccumTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * 2 * kF8Tile), b_addr = a_addr + kF8Tile;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)               // K = 32 bytes per instruction
          umma_f8(tmem + buf * 128, umma_desc_k_sw128(a_addr + kk * 32), umma_desc_k_sw128(b_addr + kk * 32), kF8Idesc, kk > 0 ? 1u : 0u);
        umma_commit(&empty[s]);
        umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = tile_m * 128 + quarter * 32 + lane;
    const bool live = row < p.M;
    const uint32_t t_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
    const int n_blocks = p.N / 128;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    // this tile column's weight scales: one per K block, staged once by the folding warps themselves
    for (int i = threadIdx.x - 64; i < kblocks; i += 256) sw_s[i] = p.sw[static_cast<size_t>(i) * n_blocks + tile_n];
    asm volatile("bar.sync 1, 256;" ::: "memory");
    for (int kb = 0; kb < kblocks && ok; ++kb) {
      const int buf = kb & 3;
      ok = mbar_wait(&acc_full[buf], (kb >> 2) & 1, p.status, kStatusAccumTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t part[4][16];
#pragma unroll
      for (int h = 0; h < 4; ++h) tmem_ld16(t_addr + buf * 128 + h * 16, part[h]);
      // acc_full follows the stage's full barrier, so the K block's scales have landed
      const float c = sx_s[(kb % kF8ScaleRing) * 128 + quarter * 32 + lane] * sw_s[kb];
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);                     // the buffer is in registers: the tensor core may refill it
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[h * 16 + i] = fmaf(c, __uint_as_float(part[h][i]), acc[h * 16 + i]);
    }
    if (ok && live) {
      const int col0 = tile_n * 128 + half * 64;
      if (p.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] += __bfloat162float(p.bias[col0 + i]);
      }
      if (p.residual != nullptr) {
        const uint4* r = reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.ldr + col0);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = r[c];
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[c * 8 + 2 * i] += bf16_lo(w[i]);
            acc[c * 8 + 2 * i + 1] += bf16_hi(w[i]);
          }
        }
      }
      if (p.out_fp32) {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.y) + static_cast<size_t>(row) * p.ldy + col0);
#pragma unroll
        for (int c = 0; c < 16; ++c) dst[c] = make_float4(acc[c * 4], acc[c * 4 + 1], acc[c * 4 + 2], acc[c * 4 + 3]);
      } else {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.y) + static_cast<size_t>(row) * p.ldy + col0);
#pragma unroll
        for (int c = 0; c < 8; ++c)
          dst[c] = make_uint4(pack_bf16x2(acc[c * 8], acc[c * 8 + 1]), pack_bf16x2(acc[c * 8 + 2], acc[c * 8 + 3]),
                              pack_bf16x2(acc[c * 8 + 4], acc[c * 8 + 5]), pack_bf16x2(acc[c * 8 + 6], acc[c * 8 + 7]));
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// One warp per (row, 128-column block): 4 bf16 per lane, maximum by shuffles, E4M3 codes and the block's scale.
__global__ void __launch_bounds__(256) act_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, int ldx, uint8_t* __restrict__ xq,
                                                            float* __restrict__ sx_t, int ld_sx, int M, int K) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int kb = blockIdx.x, row = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(row) * ldx + kb * 128 + lane * 4);
  const float v0 = bf16_lo(raw.x), v1 = bf16_hi(raw.x), v2 = bf16_lo(raw.y), v3 = bf16_hi(raw.y);
  float mx = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float scale = fmaxf(mx, 1.0e-4f) / 448.0f;
  const float inv = 1.f / scale;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v0 * inv, v1 * inv), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v2 * inv, v3 * inv), __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(row) * K + kb * 128 + lane * 4) = lo | (hi << 16);
  if (lane == 0) sx_t[static_cast<size_t>(kb) * ld_sx + row] = scale;
}

}  // namespace eredu

using namespace eredu;

// Dynamic 1 x 128 quantisation of bf16 activations x [M, K] (row stride ldx) to E4M3 xq [M, K] and scales sx_t [K/128, ld_sx].
extern "C" int eredu_fp8_quant_act(const void* x, int ldx, void* xq, float* sx_t, int ld_sx, int M, int K, cudaStream_t stream) {
  if (M <= 0 || K <= 0 || K % 128 != 0 || ldx % 4 != 0 || ld_sx < M) return -2;
  dim3 grid(K / 128, (M + 7) / 8);
  const cudaError_t e = launch_pdl(act_quant_fp8_kernel, grid, dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), ldx,
                                   static_cast<uint8_t*>(xq), sx_t, ld_sx, M, K);
  eredu_count_launches(1);
  return static_cast<int>(e);
}

// Y [M, N] = (xq * sx) (wq * sw)^T (+bias) (+residual); xq E4M3 [M, K], sx_t fp32 [K/128, ld_sx] (ld_sx: M rounded up to 128), wq E4M3 [N, K], sw fp32
// [K/128, N/128]; N and K multiples of 128. Returns -2 for shapes it does not take.
extern "C" int eredu_gemm_fp8_tc(const void* xq, const float* sx_t, int ld_sx, const void* wq, const float* sw, void* Y, const void* residual,
                                 const void* bias, int M, int N, int K, int ldy, int ldr, int out_fp32, int* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || N % 128 != 0 || K % 128 != 0 || ldy % 8 != 0 || (residual != nullptr && ldr % 8 != 0)) return -2;
  if (K / 128 > kF8MaxKBlocks || ld_sx % 128 != 0 || ld_sx < M) return -2;
  CUtensorMap tmA, tmB;
  int r = make_tma_2d(&tmA, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(M), static_cast<uint64_t>(K),
                      static_cast<uint64_t>(K), 128, 128);
  if (r != 0) return -100 + r;
  r = make_tma_2d(&tmB, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(N), static_cast<uint64_t>(K),
                  static_cast<uint64_t>(K), 128, 128);
  if (r != 0) return -200 + r;
  Fp8GemmParams p = {};
  p.sx_t = sx_t;
  p.ld_sx = ld_sx;
  p.sw = sw;
  p.y = Y;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.ldr = ldr;
  p.out_fp32 = out_fp32;
  p.status = status;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(gemm_fp8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem) != cudaSuccess) return -1;
    configured[dev] = true;
  }
  dim3 grid((M + 127) / 128, N / 128);
  const cudaError_t e = launch_pdl(gemm_fp8_tc_kernel, grid, dim3(kF8Threads), kF8Smem, stream, tmA, tmB, p);
  eredu_count_launches(1);
  return static_cast<int>(e);
}
