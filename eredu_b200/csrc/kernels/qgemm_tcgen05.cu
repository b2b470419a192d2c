// Quantised-weight linear layer  Y[M,N] = X[M,K] · dequant(Wq)[N,K]^T  on tcgen05, weights dequantised on the fly.
//
// Pipeline per 64-wide K block (same weight-stationary "swap-AB" tiling as gemm_tcgen05.cu):
//   TMA      : packed weight bytes of 128 rows + the bf16 X tile  -> shared memory (raw ring)
//   8 warps  : decode the packed block to bf16 and write it as the 128B-swizzled K-major operand tile
//   1 thread : tcgen05.mma (accumulators in TMEM)
//   4 warps  : epilogue (bias, residual, cluster split-K reduction through distributed shared memory)
// so HBM only ever sees the packed bytes (0.5 B / weight for 4-bit) while the tensor cores see bf16.
//
// Formats (FMT), both "affine" (w = scale * q + bias per group of 16/32/64/128 along K; contract:
// eredu/src/backend/mlx/runtime/checkpoint/quantization.rs:1-8,137-232), in a kernel layout made once at load:
//   QF_AFFINE4: codes tiled as [ceil(N/16)][K/64][16 rows][32 bytes] (a 16-row x 64-column tile is 512 contiguous
//     bytes, so both this kernel's TMA boxes and the decode kernel's per-warp streams read whole DRAM bursts instead
//     of 32-byte pieces 4 KB apart); inside each u32 the eight nibbles are stored as (n0,n2,n4,n6,n1,n3,n5,n7)
//   QF_AFFINE8: codes [N, K] bytes (also the container for 2/3/5/6-bit codes and for GGUF Q5/Q6 blocks)
//   scales / biases bf16, transposed to [K/group, N] so that a K block's 128 values are contiguous.
//   QF_FP8: E4M3 bytes [N, K] with one fp32 scale per weight row per 128 input columns, table [K/128, N]
//     (the 128x128 block scales of an FP8 checkpoint expanded along the rows, so that tensor-parallel row slices
//     need no alignment; weight = e4m3 * scale, eredu/src/backend/mlx/nn/fp8.rs:330-345). Activations stay bf16.
// GGUF Q4_0/Q4_1/Q4_K map to QF_AFFINE4 with group 32, Q8_0 to QF_AFFINE8 (conversion rule:
// eredu-gguf/src/convert.rs:124-152); the codes are the file's codes, only the layout changes.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/tma_host.h"

namespace cg = cooperative_groups;

namespace eredu {

enum { QF_AFFINE4 = 0, QF_AFFINE8 = 3, QF_FP8 = 5 };

struct QGemmParams {
  void* y;
  const void* residual;
  const void* bias;
  const __nv_bfloat16* scales_t;  // affine: [K/group, N]
  const __nv_bfloat16* biases_t;  // affine: [K/group, N]
  const float* scales_f32;        // QF_FP8: [K/128, N]
  int M, N, K;
  int ldy, ldr;
  int group;
  int group_shift;  // log2(group) when the group size is a power of two, else -1 (general division)
  int sb_rows;      // > 0: scales / biases of a K block arrive by TMA as sb_rows x 128 tiles next to the packed weights
  int out_fp32;
  int* status;
};

template <int FMT>
struct QRaw {
  // bytes of packed payload per weight row per 64-wide K block
  static constexpr int kBox0 = FMT == QF_AFFINE4 ? 32 : 64;
  static constexpr int kRowBytes = kBox0;
  static constexpr int kBytes = 128 * kRowBytes;
};

// Two rings. The packed weights (with the activation tile of the same K block) land in a DEEP ring of small
// slots: at 4 bits a K block is only 4 KB per tile, and HBM needs tens of KB in flight per SM to run at full
// bandwidth. The dequantised bf16 operand tiles live in a SHALLOW ring of 16 KB slots that only has to cover the
// dequant -> MMA hand-off.
template <int TN, int FMT>
struct QCfg {
  static constexpr int kATile = 128 * 64 * 2;
  static constexpr int kBTile = TN * 64 * 2;
  static constexpr int kRaw = QRaw<FMT>::kBytes;
  static constexpr int kSbBytes = 4 * 128 * 2;  // up to 4 groups per 64-wide K block, one bf16 per weight row
  static constexpr int kRawSlot = ((kRaw + kBTile + 2 * kSbBytes + 1023) / 1024) * 1024;  // [X][packed][scales][biases]
  // decode-sized tiles stay under half an SM's shared memory: two resident CTAs per SM (twice the dequant warps,
  // one full wave for grids of up to 296 CTAs)
  static constexpr int kAStages = 4;
  static constexpr int kBudget = TN <= 32 ? 108 * 1024 : 200 * 1024;
  static constexpr int kRawStagesMax = (kBudget - kAStages * kATile) / kRawSlot;
  static constexpr int kRawStages = kRawStagesMax > 16 ? 16 : kRawStagesMax;
  static constexpr int kTmemCols = TN <= 32 ? 32 : TN <= 64 ? 64 : TN <= 128 ? 128 : 256;
  static constexpr int kCtrlBytes = 1024;
  static constexpr int kSmemBytes = 1024 + kCtrlBytes + kAStages * kATile + kRawStages * kRawSlot;
  static_assert(kRawStages >= 2, "pipeline too shallow");
  static_assert(kBTile % 1024 == 0, "the packed bytes must start 1024-byte aligned behind the X tile");
};

constexpr int kDequantWarps = 8;
constexpr int kQThreads = 32 * (6 + kDequantWarps);

__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ void store_chunk(uint8_t* a_tile, int r, int c, uint4 v) {
  // K-major SW128 operand tile: 128-byte rows, 16-byte chunk c of row r lives at chunk (c ^ (r & 7))
  *reinterpret_cast<uint4*>(a_tile + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}

// ---------------------------------------------------------------------------------------------- dequant
// 256 dequant threads: thread t owns row t>>1 and the 32-weight half t&1 of the 64-wide K block.
// AFFINE4 kernel layout: inside each u32 the nibbles are stored in the order (n0,n2,n4,n6,n1,n3,n5,n7) so that
// one lop3 with 0x000F000F yields the bf16 pair (128+n_{2i}, 128+n_{2i+1}) without any byte shuffling.
__device__ __forceinline__ int group_of(const QGemmParams& p, int k) {
  return p.group_shift >= 0 ? (k >> p.group_shift) : (k / p.group);
}

// Scale and bias (as bf16x2 splats) of the group that holds element k of row n; zero outside the matrix.
__device__ __forceinline__ void load_scale_bias(const QGemmParams& p, int n, int k, uint32_t& s2, uint32_t& b2) {
  uint32_t s = 0, b = 0;
  if (n < p.N && k < p.K) {
    const size_t idx = static_cast<size_t>(group_of(p, k)) * p.N + n;
    s = reinterpret_cast<const uint16_t*>(p.scales_t)[idx];
    b = reinterpret_cast<const uint16_t*>(p.biases_t)[idx];
  }
  s2 = s | (s << 16);
  b2 = b | (b << 16);
}

// `s_sm` / `b_sm` (non-null): this K block's scales and biases in shared memory, [group within the block][128 rows],
// delivered by TMA together with the packed weights, so no global load sits inside the dequant loop.
template <int FMT>
__device__ __forceinline__ void dequant_half_row(const QGemmParams& p, const uint8_t* raw, uint8_t* a_tile, int r, int half,
                                                 int n, int kb, const uint16_t* s_sm = nullptr, const uint16_t* b_sm = nullptr) {
  const int k0 = kb * 64 + half * 32;
  const bool live = n < p.N && k0 < p.K;
  if (FMT == QF_AFFINE4 && s_sm != nullptr && p.group >= 32) {
    // fast path: one scale / bias pair for the whole half-row, read from shared memory; no group bookkeeping
    const uint4 w4 = *reinterpret_cast<const uint4*>(raw + r * 32 + half * 16);
    const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
    const int gl = p.group < 64 ? half : 0;
    const uint32_t s2 = __byte_perm(s_sm[gl * 128 + r], 0, 0x1010);  // bf16 -> (bf16, bf16)
    const uint32_t b2 = __byte_perm(b_sm[gl * 128 + r], 0, 0x1010);
    uint8_t* row = a_tile + r * 128;
    const int sw = r & 7;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t x = words[w];
      uint4 o;
      uint32_t p0 = (x & 0x000F000Fu) | 0x43004300u;          // (128 + n_2i, 128 + n_2i+1)
      uint32_t p1 = ((x >> 4) & 0x000F000Fu) | 0x43004300u;
      uint32_t p2 = ((x >> 8) & 0x000F000Fu) | 0x43004300u;
      uint32_t p3 = ((x >> 12) & 0x000F000Fu) | 0x43004300u;
      asm("sub.bf16x2 %0, %0, %1;" : "+r"(p0) : "r"(0x43004300u));
      asm("sub.bf16x2 %0, %0, %1;" : "+r"(p1) : "r"(0x43004300u));
      asm("sub.bf16x2 %0, %0, %1;" : "+r"(p2) : "r"(0x43004300u));
      asm("sub.bf16x2 %0, %0, %1;" : "+r"(p3) : "r"(0x43004300u));
      o.x = bf16x2_fma(p0, s2, b2);
      o.y = bf16x2_fma(p1, s2, b2);
      o.z = bf16x2_fma(p2, s2, b2);
      o.w = bf16x2_fma(p3, s2, b2);
      *reinterpret_cast<uint4*>(row + (((half * 4 + w) ^ sw) << 4)) = o;
    }
  } else if (FMT == QF_AFFINE4) {
    const uint4 w4 = *reinterpret_cast<const uint4*>(raw + r * 32 + half * 16);
    const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
    uint32_t s2 = 0, b2 = 0;
    int cur_group = -1;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int g = group_of(p, k0 + w * 8);
      if (g != cur_group) {
        cur_group = g;
        uint32_t s = 0, b = 0;
        if (s_sm != nullptr) {
          const int gl = p.group < 64 ? ((half * 32 + w * 8) >> p.group_shift) : 0;
          s = s_sm[gl * 128 + r];
          b = b_sm[gl * 128 + r];
        } else if (live) {
          s = reinterpret_cast<const uint16_t*>(p.scales_t)[static_cast<size_t>(g) * p.N + n];
          b = reinterpret_cast<const uint16_t*>(p.biases_t)[static_cast<size_t>(g) * p.N + n];
        }
        s2 = s | (s << 16);
        b2 = b | (b << 16);
      }
      uint32_t x = words[w];
      uint4 o;
      uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t pair = (x & 0x000F000Fu) | 0x43004300u;           // (128 + n_2i, 128 + n_2i+1)
        asm("sub.bf16x2 %0, %0, %1;" : "+r"(pair) : "r"(0x43004300u));
        ov[i] = bf16x2_fma(pair, s2, b2);
        x >>= 4;
      }
      store_chunk(a_tile, r, half * 4 + w, o);
    }
  } else if (FMT == QF_FP8) {  // 64 E4M3 bytes per row per K block, this thread takes 32; one scale for all of them
    const uint4 lo = *reinterpret_cast<const uint4*>(raw + r * 64 + half * 32);
    const uint4 hi = *reinterpret_cast<const uint4*>(raw + r * 64 + half * 32 + 16);
    const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    float sc = 0.f;
    if (s_sm != nullptr) sc = reinterpret_cast<const float*>(s_sm)[r];
    else if (live) sc = p.scales_f32[static_cast<size_t>(k0 >> 7) * p.N + n];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 o;
      uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int hw = 0; hw < 2; ++hw) {
        const uint32_t x = words[c * 2 + hw];
        uint32_t h01, h23;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"(static_cast<uint16_t>(x & 0xFFFFu)));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"(static_cast<uint16_t>(x >> 16)));
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
        const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
        ov[hw * 2] = pack_bf16x2(f01.x * sc, f01.y * sc);
        ov[hw * 2 + 1] = pack_bf16x2(f23.x * sc, f23.y * sc);
      }
      store_chunk(a_tile, r, half * 4 + c, o);
    }
  } else {  // QF_AFFINE8: 64 bytes per row per K block, this thread takes 32 of them
    const uint4 lo = *reinterpret_cast<const uint4*>(raw + r * 64 + half * 32);
    const uint4 hi = *reinterpret_cast<const uint4*>(raw + r * 64 + half * 32 + 16);
    const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint32_t s2 = 0, b2 = 0;
    int cur_group = -1;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 o;
      uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int hw = 0; hw < 2; ++hw) {
        const int g = group_of(p, k0 + c * 8 + hw * 4);
        if (g != cur_group) {
          cur_group = g;
          uint32_t s = 0, b = 0;
          if (s_sm != nullptr) {
            const int gl = p.group < 64 ? ((half * 32 + c * 8 + hw * 4) >> p.group_shift) : 0;
            s = s_sm[gl * 128 + r];
            b = b_sm[gl * 128 + r];
          } else if (live) {
            s = reinterpret_cast<const uint16_t*>(p.scales_t)[static_cast<size_t>(g) * p.N + n];
            b = reinterpret_cast<const uint16_t*>(p.biases_t)[static_cast<size_t>(g) * p.N + n];
          }
          s2 = s | (s << 16);
          b2 = b | (b << 16);
        }
        const uint32_t x = words[c * 2 + hw];
        // bytes -> exact floats through the 2^23 trick, no integer-to-float conversion unit involved
        const float f0 = __uint_as_float(0x4B000000u | (x & 0xFFu)) - 8388608.f;
        const float f1 = __uint_as_float(0x4B000000u | ((x >> 8) & 0xFFu)) - 8388608.f;
        const float f2 = __uint_as_float(0x4B000000u | ((x >> 16) & 0xFFu)) - 8388608.f;
        const float f3 = __uint_as_float(0x4B000000u | (x >> 24)) - 8388608.f;
        ov[hw * 2] = bf16x2_fma(pack_bf16x2(f0, f1), s2, b2);
        ov[hw * 2 + 1] = bf16x2_fma(pack_bf16x2(f2, f3), s2, b2);
      }
      store_chunk(a_tile, r, half * 4 + c, o);
    }
  }
}

// ---------------------------------------------------------------------------------------------- kernel
// warps: 0 TMA producer, 1 MMA issuer (+TMEM alloc), 2..5 epilogue, 6..13 dequant.
template <int TN, int FMT, bool SPLIT>
__global__ void __launch_bounds__(kQThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmX,
             const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmB, QGemmParams p) {
  using Cfg = QCfg<TN, FMT>;
  constexpr int R = Cfg::kRawStages, A = Cfg::kAStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem);  // [R] TMA landed (packed weights + X tile)
  uint64_t* raw_empty = raw_full + R;                      // [R] the MMAs that read the slot's X tile retired
  uint64_t* a_full = raw_empty + R;                        // [A] bf16 operand tile written (8 warp arrivals)
  uint64_t* a_empty = a_full + A;                          // [A] the MMAs that read the operand tile retired
  uint64_t* accum_bar = a_empty + A;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  uint8_t* a_ring = smem + Cfg::kCtrlBytes;                // [A][16 KB] K-major SW128 operand tiles
  uint8_t* raw_ring = a_ring + A * Cfg::kATile;            // [R][X tile | packed weights]
  constexpr int kRawOff = Cfg::kBTile, kScaleOff = Cfg::kBTile + Cfg::kRaw, kBiasOff = kScaleOff + Cfg::kSbBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.y;
  const int nsplit = SPLIT ? gridDim.z : 1;
  const int split = SPLIT ? blockIdx.z : 0;
  const int kblocks = (p.K + 63) >> 6;
  const int kb_per = (kblocks + nsplit - 1) / nsplit;
  const int kb0 = split * kb_per;
  const int niter = max(0, min(kblocks, kb0 + kb_per) - kb0);

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmX);
    for (int s = 0; s < R; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 1);
    }
    for (int s = 0; s < A; ++s) {
      mbar_init(&a_full[s], kDequantWarps);
      mbar_init(&a_empty[s], 1);
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
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < niter; ++it) {
        const int s = it % R;
        const uint32_t ph = (it / R) & 1;
        ok = mbar_wait(&raw_empty[s], ph ^ 1, p.status, kStatusSmemEmptyTimeout);
        if (!ok) break;
        uint8_t* st = raw_ring + s * Cfg::kRawSlot;
        const int kb = kb0 + it;
        mbar_arrive_expect_tx(&raw_full[s], Cfg::kRaw + Cfg::kBTile + (FMT == QF_FP8 ? p.sb_rows * 512 : 2 * p.sb_rows * 256));
        // packed weights: byte tensor [N, row_bytes]; x coordinate in bytes (a multiple of 32)
        if (FMT == QF_AFFINE4) tma_load_3d_hint(st + kRawOff, &tmQ, 0, kb, tile_n * 8, &raw_full[s], pol_w);  // 8 tiles of 16 rows
        else tma_load_2d_hint(st + kRawOff, &tmQ, kb * QRaw<FMT>::kBox0, tile_n * 128, &raw_full[s], pol_w);
        tma_load_2d_hint(st, &tmX, kb * 64, tile_m * TN, &raw_full[s], pol_x);
        if (p.sb_rows > 0) {
          const int grow = (kb * 64) >> p.group_shift;
          tma_load_2d_hint(st + kScaleOff, &tmS, tile_n * 128, grow, &raw_full[s], pol_w);
          if (FMT != QF_FP8) tma_load_2d_hint(st + kBiasOff, &tmB, tile_n * 128, grow, &raw_full[s], pol_w);
        }
        issued = it + 1;
      }
      if (!ok) {
        for (int it = max(0, issued - R); it < issued; ++it) mbar_wait(&raw_full[it % R], (it / R) & 1, nullptr, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, TN);
      bool ok = true;
      for (int it = 0; it < niter; ++it) {
        const int rs = it % R, as = it % A;
        ok = mbar_wait(&raw_full[rs], (it / R) & 1, p.status, kStatusTmaFullTimeout) &&
             mbar_wait(&a_full[as], (it / A) & 1, p.status, kStatusTmaFullTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t da = umma_desc_k_sw128(smem_u32(a_ring + as * Cfg::kATile));
        const uint64_t db = umma_desc_k_sw128(smem_u32(raw_ring + rs * Cfg::kRawSlot));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(&a_empty[as]);
        umma_commit(&raw_empty[rs]);
      }
      if (ok) umma_commit(accum_bar);
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ dequant warps
    // 256 threads: thread t converts the 32-weight half t&1 of row t>>1 of every K block. (Giving each warp whole
    // blocks of its own - fewer hand-offs, more work per wait - measured slower: the conversion of one half-row
    // is a dependent chain, and eight warps sharing a block overlap those chains better.)
    const int dt = threadIdx.x - 6 * 32;  // 0..255
    const int r = dt >> 1, half = dt & 1;
    const int n = tile_n * 128 + r;
    bool ok = true;
    for (int it = 0; it < niter; ++it) {
      const int rs = it % R, as = it % A;
      ok = mbar_wait(&raw_full[rs], (it / R) & 1, p.status, kStatusTmaFullTimeout) &&
           mbar_wait(&a_empty[as], ((it / A) & 1) ^ 1, p.status, kStatusSmemEmptyTimeout);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint8_t* slot = raw_ring + rs * Cfg::kRawSlot;
      const uint16_t* s_sm = p.sb_rows > 0 ? reinterpret_cast<const uint16_t*>(slot + kScaleOff) : nullptr;
      const uint16_t* b_sm = p.sb_rows > 0 ? reinterpret_cast<const uint16_t*>(slot + kBiasOff) : nullptr;
      dequant_half_row<FMT>(p, slot + kRawOff, a_ring + as * Cfg::kATile, r, half, n, kb0 + it, s_sm, b_sm);
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[as]);
    }
  }
  __syncwarp();

  // ------------------------------------------------------------ epilogue (warps 2..5)
  const int q = warp & 3;
  const int row = q * 32 + lane;
  const int n = tile_n * 128 + row;
  const int m_base = tile_m * TN;
  float* red = reinterpret_cast<float*>(a_ring);  // SPLIT: [TN][128] fp32, aliases the operand ring after the main loop

  auto store = [&](float v, int m) {
    if (p.bias != nullptr) v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
    if (p.residual != nullptr)
      v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.residual)[static_cast<size_t>(m) * p.ldr + n]);
    if (p.out_fp32) static_cast<float*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = v;
    else static_cast<__nv_bfloat16*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = __float2bfloat16(v);
  };

  if (warp >= 2 && warp < 6) {
    bool acc_ok = (niter > 0) && mbar_wait(accum_bar, 0, p.status, kStatusAccumTimeout);
    acc_ok = __all_sync(0xffffffffu, acc_ok);
    tc_fence_after_sync();
    if (acc_ok) {
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t g[16];
        tmem_ld16(taddr + c0, g);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (SPLIT) {
            red[(c0 + j) * 128 + row] = __uint_as_float(g[j]);
          } else {
            const int m = m_base + c0 + j;
            if (m < p.M && n < p.N) store(__uint_as_float(g[j]), m);
          }
        }
      }
    }
  }
  if (SPLIT) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (warp >= 2 && warp < 6 && n < p.N) {
      const int m_end = min(TN, p.M - m_base);
      for (int c = split; c < m_end; c += nsplit) {
        float v = 0.f;
        for (int rr = 0; rr < nsplit; ++rr) v += cluster.map_shared_rank(red, rr)[c * 128 + row];
        store(v, m_base + c);
      }
    }
    cluster.sync();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int TN, int FMT, bool SPLIT>
static cudaError_t launch_q(const CUtensorMap& tmQ, const CUtensorMap& tmX, const CUtensorMap& tmS, const CUtensorMap& tmB,
                            const QGemmParams& p, int n_tiles, int m_tiles, int nsplit, cudaStream_t stream) {
  using Cfg = QCfg<TN, FMT>;
  auto kern = qgemm_kernel<TN, FMT, SPLIT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, m_tiles, nsplit);
  cfg.blockDim = dim3(kQThreads, 1, 1);
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
  return cudaLaunchKernelEx(&cfg, kern, tmQ, tmX, tmS, tmB, p);
}

template <int FMT>
static cudaError_t dispatch_q(int tn, const CUtensorMap& tmQ, const CUtensorMap& tmX, const CUtensorMap& tmS,
                              const CUtensorMap& tmB, const QGemmParams& p, int n_tiles, int m_tiles, int nsplit,
                              cudaStream_t stream) {
  switch (tn) {
    case 16: return nsplit > 1 ? launch_q<16, FMT, true>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, nsplit, stream)
                               : launch_q<16, FMT, false>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, 1, stream);
    case 32: return nsplit > 1 ? launch_q<32, FMT, true>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, nsplit, stream)
                               : launch_q<32, FMT, false>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, 1, stream);
    case 64: return nsplit > 1 ? launch_q<64, FMT, true>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, nsplit, stream)
                               : launch_q<64, FMT, false>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, 1, stream);
    default: return launch_q<128, FMT, false>(tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, 1, stream);
  }
}

// Whole-matrix dequantisation to bf16 [N, K] (prefill with many tokens: decode once, then the dense GEMM).
// grid (K/64, ceil(N/128)), 256 threads: same thread mapping as the in-pipeline decoder.
template <int FMT>
__global__ void __launch_bounds__(256) dequant_matrix_kernel(const uint8_t* __restrict__ wq, QGemmParams p,
                                                             __nv_bfloat16* __restrict__ out) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int kb = blockIdx.x, r = threadIdx.x >> 1, half = threadIdx.x & 1;
  const int n = blockIdx.y * 128 + r;
  if (n >= p.N) return;
  constexpr int kRowK = FMT == QF_AFFINE4 ? 2 : 1;  // weights per byte
  const size_t row_bytes = static_cast<size_t>(p.K) / kRowK;
  const uint8_t* src = FMT == QF_AFFINE4
                           ? wq + (static_cast<size_t>(n >> 4) * (p.K >> 6) + kb) * 512 + (n & 15) * 32 + half * 16
                           : wq + static_cast<size_t>(n) * row_bytes + static_cast<size_t>(kb) * (64 / kRowK) + half * (32 / kRowK);
  __align__(16) uint8_t raw[64];
  __align__(16) uint8_t tile[128];
  // stage this thread's 32 weights as "row 0, half `half`" of a private one-row tile
  if (FMT == QF_AFFINE4) *reinterpret_cast<uint4*>(raw + half * 16) = *reinterpret_cast<const uint4*>(src);
  else {
    *reinterpret_cast<uint4*>(raw + half * 32) = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(raw + half * 32 + 16) = *reinterpret_cast<const uint4*>(src + 16);
  }
  dequant_half_row<FMT>(p, raw, tile, 0, half, n, kb);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(n) * p.K + kb * 64 + half * 32);
#pragma unroll
  for (int c = 0; c < 4; ++c) dst[c] = *reinterpret_cast<const uint4*>(tile + ((half * 4 + c) << 4));
}

}  // namespace eredu

using namespace eredu;

static int dequant_impl(int fmt, const void* wq, const void* scales_t, const void* biases_t, void* out, int N, int K, int group,
                        cudaStream_t stream) {
  if (K % 64 != 0 || group <= 0 || K % group != 0) return -1;
  QGemmParams p = {};
  p.scales_t = static_cast<const __nv_bfloat16*>(scales_t);
  p.biases_t = static_cast<const __nv_bfloat16*>(biases_t);
  p.scales_f32 = static_cast<const float*>(scales_t);
  p.N = N;
  p.K = K;
  p.group = group;
  p.group_shift = (group & (group - 1)) == 0 ? __builtin_ctz(static_cast<unsigned>(group)) : -1;
  dim3 grid(K / 64, (N + 127) / 128);
  const uint8_t* w = static_cast<const uint8_t*>(wq);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  if (fmt == QF_AFFINE4) launch_pdl(dequant_matrix_kernel<QF_AFFINE4>, grid, dim3(256), 0, stream, w, p, o);
  else if (fmt == QF_FP8) launch_pdl(dequant_matrix_kernel<QF_FP8>, grid, dim3(256), 0, stream, w, p, o);
  else launch_pdl(dequant_matrix_kernel<QF_AFFINE8>, grid, dim3(256), 0, stream, w, p, o);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_dequant_affine(const void* wq, const void* scales_t, const void* biases_t, void* out, int N, int K,
                                    int bits, int group, cudaStream_t stream) {
  if (bits != 4 && bits != 8) return -1;
  return dequant_impl(bits == 4 ? QF_AFFINE4 : QF_AFFINE8, wq, scales_t, biases_t, out, N, K, group, stream);
}

// Block-scaled E4M3 weights [N, K] with the fp32 row-scale table [K/128, N] -> bf16 [N, K].
extern "C" int eredu_dequant_fp8(const void* wq, const void* scales_f32_t, void* out, int N, int K, cudaStream_t stream) {
  if (K % 128 != 0) return -1;
  return dequant_impl(QF_FP8, wq, scales_f32_t, nullptr, out, N, K, 128, stream);
}

static int qgemm_impl(int fmt, const void* X, const void* wq, const void* scales_t, const void* biases_t, void* Y,
                      const void* residual, const void* bias, int M, int N, int K, int ldx, int ldy, int ldr, int group,
                      int out_fp32, int force_split, int sm_count, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 64 != 0 || group <= 0 || K % group != 0 || (group != 16 && group % 32 != 0)) return -1;
  const int tn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  const int row_bytes = fmt == QF_AFFINE4 ? K / 2 : K;
  const int box0 = fmt == QF_AFFINE4 ? 32 : 64;
  CUtensorMap tmQ, tmX;
  int r;
  if (fmt == QF_AFFINE4) {
    // tiled codes [ceil(N/16)][K/64][16 rows x 32 bytes]: eight consecutive row tiles of one K block are the 128 x 32
    // byte block the decoder expects, and each of them is one contiguous 512-byte read
    const uint64_t kb_count = static_cast<uint64_t>(K / 64), tiles = static_cast<uint64_t>((N + 15) / 16);
    r = make_tma_3d(&tmQ, wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, 128, kb_count, tiles, 512, kb_count * 512, 128, 1, 8,
                    CU_TENSOR_MAP_SWIZZLE_NONE);
  } else {
    r = make_tma_2d(&tmQ, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, row_bytes, row_bytes, 128, box0, CU_TENSOR_MAP_SWIZZLE_NONE);
  }
  if (r != 0) return -100 + r;
  r = make_tma_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, tn, 64);
  if (r != 0) return -200 + r;
  QGemmParams p = {};
  p.y = Y;
  p.residual = residual;
  p.bias = bias;
  p.scales_t = static_cast<const __nv_bfloat16*>(scales_t);
  p.biases_t = static_cast<const __nv_bfloat16*>(biases_t);
  p.scales_f32 = static_cast<const float*>(scales_t);
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldy = ldy;
  p.ldr = ldr;
  p.group = group;
  p.group_shift = (group & (group - 1)) == 0 ? __builtin_ctz(static_cast<unsigned>(group)) : -1;
  p.out_fp32 = out_fp32;
  p.status = status;
  // scales / biases by TMA: power-of-two groups (1, 2 or 4 per 64-wide K block, or one row shared by several
  // blocks) and 16-byte aligned rows of the transposed tables
  CUtensorMap tmS = tmX, tmB = tmX;
  p.sb_rows = 0;
  if (fmt == QF_FP8) {
    if (N % 4 == 0 && make_tma_2d(&tmS, scales_t, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, static_cast<uint64_t>(K / 128), N, N, 1, 128,
                                  CU_TENSOR_MAP_SWIZZLE_NONE) == 0)
      p.sb_rows = 1;
  } else if (p.group_shift >= 0 && group >= 16 && N % 8 == 0) {
    const int rows = group >= 64 ? 1 : 64 / group;
    const uint64_t table_rows = static_cast<uint64_t>(K / group);
    if (make_tma_2d(&tmS, scales_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, table_rows, N, N, rows, 128, CU_TENSOR_MAP_SWIZZLE_NONE) == 0 &&
        make_tma_2d(&tmB, biases_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, table_rows, N, N, rows, 128, CU_TENSOR_MAP_SWIZZLE_NONE) == 0)
      p.sb_rows = rows;
  }
  const int n_tiles = (N + 127) / 128;
  const int m_tiles = (M + tn - 1) / tn;
  const int kblocks = K / 64;
  int nsplit = 1;
  if (tn <= 64) {
    if (force_split > 0) nsplit = force_split;
    else {
      const int sm = sm_count > 0 ? sm_count : 148;
      while (nsplit < 8 && n_tiles * m_tiles * nsplit * 2 <= 2 * sm && kblocks / (nsplit * 2) >= 2) nsplit *= 2;
    }
    while (nsplit > 1 && (kblocks + nsplit - 1) / nsplit * (nsplit - 1) >= kblocks) nsplit >>= 1;
  }
  cudaError_t e = fmt == QF_AFFINE4 ? dispatch_q<QF_AFFINE4>(tn, tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, nsplit, stream)
                  : fmt == QF_FP8   ? dispatch_q<QF_FP8>(tn, tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, nsplit, stream)
                                    : dispatch_q<QF_AFFINE8>(tn, tmQ, tmX, tmS, tmB, p, n_tiles, m_tiles, nsplit, stream);
  eredu_count_launches(1);
  return static_cast<int>(e);
}

// Y = X dequant(Wq)^T (+bias) (+residual). `wq`: packed codes in kernel layout (4-bit: tiles [ceil(N/16)][K/64][16][32]
// bytes with the nibbles of every u32 interleaved (n0,n2,n4,n6,n1,n3,n5,n7); [N, K] bytes for 8-bit); scales_t / biases_t: bf16
// [K/group, N]. bits: 4 or 8. K must be a multiple of 64 and of the group size.
extern "C" int eredu_qgemm(const void* X, const void* wq, const void* scales_t, const void* biases_t, void* Y,
                           const void* residual, const void* bias, int M, int N, int K, int ldx, int ldy, int ldr, int bits,
                           int group, int out_fp32, int force_split, int sm_count, int* status, cudaStream_t stream) {
  if (bits != 4 && bits != 8) return -1;
  return qgemm_impl(bits == 4 ? QF_AFFINE4 : QF_AFFINE8, X, wq, scales_t, biases_t, Y, residual, bias, M, N, K, ldx, ldy, ldr,
                    group, out_fp32, force_split, sm_count, status, stream);
}

// Y = X (e4m3(Wq) * scale)^T (+bias) (+residual) for block-scaled FP8 weights: wq E4M3 bytes [N, K], scales_f32_t fp32
// [K/128, N]. K must be a multiple of 128.
extern "C" int eredu_qgemm_fp8(const void* X, const void* wq, const void* scales_f32_t, void* Y, const void* residual,
                               const void* bias, int M, int N, int K, int ldx, int ldy, int ldr, int out_fp32, int force_split,
                               int sm_count, int* status, cudaStream_t stream) {
  if (K % 128 != 0) return -1;
  return qgemm_impl(QF_FP8, X, wq, scales_f32_t, nullptr, Y, residual, bias, M, N, K, ldx, ldy, ldr, 128, out_fp32, force_split,
                    sm_count, status, stream);
}
