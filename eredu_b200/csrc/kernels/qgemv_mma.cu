// Decode-regime quantised linear layer: Y[M,N] = X[M,K] · dequant(Wq)[N,K]^T for M <= 16 tokens and 4-bit affine weights.
//
// With so few tokens the layer is a stream over the packed weights (0.5 B per weight), and what matters is that nothing
// but HBM sits on the critical path. This kernel therefore keeps the weights in registers from the load to the tensor
// core: no shared-memory operand tiles, no TMEM round trip, no producer / consumer hand-off (the tcgen05 pipeline of
// qgemm_tcgen05.cu serves M > 16, where the MMA is worth the staging).
//
//   warp          : a 16-row weight tile x a K range; every 64-wide K block is two 8-byte loads per lane (rows g and
//                   g + 8 of the tile, 16 consecutive codes each), prefetched several blocks ahead in registers
//   dequant       : one shift + one lop3 place two nibbles into the mantissas of a bf16 pair (1 + n/16), one
//                   fma.rn.bf16x2 with the per-group pair (16·scale, bias − 16·scale) turns it into the weights
//   mma.sync      : m16n8k16, the weight tile as A (16 rows x 16 k), eight tokens as B; the k slots of an instruction
//                   are filled lane by lane with the codes that lane loaded, and the activations follow the same map, so
//                   no data is exchanged between lanes
//   split K       : across the warps of a CTA (through shared memory) and across the CTAs of a cluster (through
//                   distributed shared memory); the reducing threads add bias / residual or apply SwiGLU and store
//
// GATED: the weight holds gate rows [0, I) and up rows [I, 2I); a warp computes both tiles of its 16 output columns and
// the epilogue writes silu(gate) * up, so the activation never exists unfused.
//
// Numerics: weights are rounded to bf16 after dequantisation like in the tcgen05 kernel; the bias constant
// bias − 16·scale is rounded to bf16 when the table is built (error <= scale / 32, a thirtieth of a quantisation step).
// The affine contract is eredu/src/backend/mlx/runtime/checkpoint/quantization.rs:1-8,137-232.
#include <cuda_bf16.h>

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/trace.cuh"

namespace eredu {

struct QGemvParams {
  const __nv_bfloat16* x;
  const uint8_t* wq;    // [N, K/2], kernel nibble order (n0,n2,n4,n6,n1,n3,n5,n7) inside each u32
  const uint32_t* dq;   // [K/group, N]: bf16(16·scale) | bf16(bias − 16·scale) << 16
  void* y;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* bias;
  int M, N, n_out, K;
  int ldx, ldy, ldr;
  int group_shift;
  int kblocks, blocks_per_split;
  int wk;               // warps of a CTA that share a row tile and split K (1, 2, 4 or 8)
  int ns;               // CTAs of a cluster that split K
  int out_fp32;
  float limit;          // GATED: clamp (0 = off): gate <= limit, |up| <= limit
};

constexpr int kGemvThreads = 256;
constexpr int kGemvDepth = 4;  // 64-wide K blocks of packed weights in flight per warp

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return d;
}

// Eight codes of one u32 -> four bf16 pairs (k, k+1), (k+2, k+3), ... already scaled: pair j sits in nibbles j and j + 4.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t s2, uint32_t c2, uint32_t* out) {
  constexpr uint32_t kMask = 0x00780078u, kOne = 0x3F803F80u;
  out[0] = fma_bf16x2(lop3_and_or(w << 3, kMask, kOne), s2, c2);
  out[1] = fma_bf16x2(lop3_and_or(w >> 1, kMask, kOne), s2, c2);
  out[2] = fma_bf16x2(lop3_and_or(w >> 5, kMask, kOne), s2, c2);
  out[3] = fma_bf16x2(lop3_and_or(w >> 9, kMask, kOne), s2, c2);
}

__device__ __forceinline__ void mma_bf16_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ldg_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// One stage of the register prefetch ring: packed codes and the dequantisation pair of rows g and g + 8 (x2 when GATED).
template <int S>
struct GemvStage {
  uint2 w[S][2];
  uint32_t sc[S][2];
};

template <int NT, bool GATED>
__global__ void __launch_bounds__(kGemvThreads, 2) qgemv4_kernel(const QGemvParams p) {
  constexpr int S = GATED ? 2 : 1;
  constexpr int TOK = NT * 8;
  // partial tiles [wk][S][TOK][rows + 4]: rows = 128 / wk, so one plane holds at most TOK * 160 floats
  __shared__ float red[S * TOK * 160];

  pdl_launch_early();
  trace_mark(kTraceQGemm, kTraceStart);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tiles_per_cta = 8 / p.wk;              // row tiles (16 rows) of this CTA
  const int rows_cta = tiles_per_cta * 16;
  const int wr = warp % tiles_per_cta, wkk = warp / tiles_per_cta;
  uint32_t crank = 0;
  if (p.ns > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int n0 = blockIdx.x * rows_cta + wr * 16;
  const int split = static_cast<int>(crank) * p.wk + wkk;
  const int kb0 = min(split * p.blocks_per_split, p.kblocks);
  const int kb1 = min(kb0 + p.blocks_per_split, p.kblocks);

  // rows beyond the matrix read the last row and are dropped at the store
  const int r_lo = min(n0 + g, p.n_out - 1), r_hi = min(n0 + g + 8, p.n_out - 1);
  const size_t row_bytes = static_cast<size_t>(p.K) >> 1;
  const uint8_t* wrow[S][2];
  const uint32_t* dqrow[S][2];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    const int off = s * p.n_out;                   // GATED: the up rows follow the n_out gate rows
    wrow[s][0] = p.wq + static_cast<size_t>(r_lo + off) * row_bytes + t * 8;
    wrow[s][1] = p.wq + static_cast<size_t>(r_hi + off) * row_bytes + t * 8;
    dqrow[s][0] = p.dq + r_lo + off;
    dqrow[s][1] = p.dq + r_hi + off;
  }

  auto load_stage = [&](GemvStage<S>& st, int kb) {
    const size_t grp = static_cast<size_t>((kb * 64 + t * 16) >> p.group_shift) * p.N;
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        st.w[s][h] = ldg_stream_u2(wrow[s][h] + static_cast<size_t>(kb) * 32);
        st.sc[s][h] = ldg_stream_u32(dqrow[s][h] + grp);
      }
  };

  // weights do not depend on the previous kernel: their first loads are in flight before the dependency wait
  GemvStage<S> ring[kGemvDepth];
#pragma unroll
  for (int d = 0; d < kGemvDepth; ++d)
    if (kb0 + d < kb1) load_stage(ring[d], kb0 + d);

  pdl_wait();
  trace_mark(kTraceQGemm, kTraceAfterWait);
  pdl_launch_dependents();

  // activations: token nt*8 + g, the 16 values that match this lane's codes
  const __nv_bfloat16* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) xrow[nt] = p.x + static_cast<size_t>(min(nt * 8 + g, p.M - 1)) * p.ldx + t * 16;

  float acc[S][NT][4];
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[s][nt][j] = 0.f;

  uint4 xn[NT][2];
  if (kb0 < kb1) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      xn[nt][0] = *reinterpret_cast<const uint4*>(xrow[nt] + kb0 * 64);
      xn[nt][1] = *reinterpret_cast<const uint4*>(xrow[nt] + kb0 * 64 + 8);
    }
  }

  for (int kb = kb0; kb < kb1; kb += kGemvDepth) {
#pragma unroll
    for (int d = 0; d < kGemvDepth; ++d) {
      const int k = kb + d;
      if (k < kb1) {
        const GemvStage<S> cur = ring[d];
        if (k + kGemvDepth < kb1) load_stage(ring[d], k + kGemvDepth);
        uint4 xc[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          xc[nt][0] = xn[nt][0];
          xc[nt][1] = xn[nt][1];
        }
        if (k + 1 < kb1) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            xn[nt][0] = *reinterpret_cast<const uint4*>(xrow[nt] + (k + 1) * 64);
            xn[nt][1] = *reinterpret_cast<const uint4*>(xrow[nt] + (k + 1) * 64 + 8);
          }
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
          uint32_t a[2][8];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t sc = cur.sc[s][h];
            const uint32_t s2 = __byte_perm(sc, sc, 0x1010), c2 = __byte_perm(sc, sc, 0x3232);
            dequant_word(cur.w[s][h].x, s2, c2, &a[h][0]);
            dequant_word(cur.w[s][h].y, s2, c2, &a[h][4]);
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t xb[8] = {xc[nt][0].x, xc[nt][0].y, xc[nt][0].z, xc[nt][0].w,
                                    xc[nt][1].x, xc[nt][1].y, xc[nt][1].z, xc[nt][1].w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_bf16_16816(acc[s][nt], a[0][2 * i], a[1][2 * i], a[0][2 * i + 1], a[1][2 * i + 1], xb[2 * i], xb[2 * i + 1]);
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ reduction over the K splits and epilogue
  // plane of this warp's K split: [S][TOK][rows_cta + 4]; lane holds rows g / g + 8 and tokens 2t, 2t + 1 of each tile
  const int ldn = rows_cta + 4;
  const int plane = S * TOK * ldn;
  float* mine = red + wkk * plane;
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float* base = mine + (s * TOK + nt * 8 + 2 * t) * ldn + wr * 16 + g;
      base[0] = acc[s][nt][0];
      base[ldn] = acc[s][nt][1];
      base[8] = acc[s][nt][2];
      base[ldn + 8] = acc[s][nt][3];
    }
  if (p.ns > 1) {
    cluster_arrive_release();
    cluster_wait_acquire();
  } else {
    __syncthreads();
  }
  // cluster rank r finishes columns [r * cols, (r + 1) * cols) of the CTA's rows_cta output columns
  const int cols = rows_cta / p.ns;
  const int items = p.M * cols;
  const uint32_t red_addr = smem_u32(red);
  for (int idx = threadIdx.x; idx < items; idx += kGemvThreads) {
    const int m = idx / cols, c = static_cast<int>(crank) * cols + idx % cols;
    const int n = blockIdx.x * rows_cta + c;
    if (n >= p.n_out) continue;
    float v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      float sum = 0.f;
      const int off = (s * TOK + m) * ldn + c;
      for (int q = 0; q < p.ns; ++q) {
        if (p.ns > 1) {
          const uint32_t remote = mapa_shared(red_addr, static_cast<uint32_t>(q));
          for (int w = 0; w < p.wk; ++w) sum += ld_dsmem_f32(remote + static_cast<uint32_t>(w * plane + off) * 4u);
        } else {
          for (int w = 0; w < p.wk; ++w) sum += red[w * plane + off];
        }
      }
      v[s] = sum;
    }
    float out;
    if (GATED) {
      float gate = v[0], up = v[S - 1];
      if (p.bias != nullptr) {
        gate += __bfloat162float(p.bias[n]);
        up += __bfloat162float(p.bias[p.n_out + n]);
      }
      if (p.limit > 0.f) {
        gate = fminf(gate, p.limit);
        up = fminf(fmaxf(up, -p.limit), p.limit);
      }
      out = gate / (1.f + __expf(-gate)) * up;
    } else {
      out = v[0];
      if (p.bias != nullptr) out += __bfloat162float(p.bias[n]);
      if (p.residual != nullptr) out += __bfloat162float(p.residual[static_cast<size_t>(m) * p.ldr + n]);
    }
    if (p.out_fp32) static_cast<float*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = out;
    else static_cast<__nv_bfloat16*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = __float2bfloat16(out);
  }
  if (p.ns > 1) {
    // nobody leaves while a peer may still read its partial tiles
    cluster_arrive_release();
    cluster_wait_acquire();
  }
  trace_mark(kTraceQGemm, kTraceEnd);
}

template <int NT, bool GATED>
static cudaError_t launch_gemv(const QGemvParams& p, int n_ctas, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ctas, p.ns, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (pdl_enabled()) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (p.ns > 1) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = 1;
    attr[nattr].val.clusterDim.y = p.ns;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  return cudaLaunchKernelEx(&cfg, qgemv4_kernel<NT, GATED>, p);
}

}  // namespace eredu

using namespace eredu;

// Y = X dequant(Wq)^T (+bias) (+residual), or with gated != 0 Y[M, N/2] = silu(X Wgate^T) * (X Wup^T), for M <= 16.
// wq: 4-bit codes [N, K/2] in kernel nibble order; dq: u32 [K/group, N] holding bf16(16·scale) in the low and
// bf16(bias − 16·scale) in the high half; group a power of two >= 16; K a multiple of 64. Returns -2 for shapes this
// kernel does not take (the caller then uses eredu_qgemm).
extern "C" int eredu_qgemv4(const void* X, const void* wq, const void* dq, void* Y, const void* residual, const void* bias,
                            int M, int N, int K, int ldx, int ldy, int ldr, int group, int out_fp32, int gated, float limit,
                            int force_wk, int force_ns, int sm_count, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 16 || K % 64 != 0 || group < 16 || (group & (group - 1)) != 0 || K % group != 0 || ldx % 8 != 0) return -2;
  if (gated && (N % 2 != 0 || residual != nullptr)) return -2;
  QGemvParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(X);
  p.wq = static_cast<const uint8_t*>(wq);
  p.dq = static_cast<const uint32_t*>(dq);
  p.y = Y;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M;
  p.N = N;
  p.n_out = gated ? N / 2 : N;
  p.K = K;
  p.ldx = ldx;
  p.ldy = ldy;
  p.ldr = ldr;
  p.group_shift = __builtin_ctz(static_cast<unsigned>(group));
  p.kblocks = K / 64;
  p.out_fp32 = out_fp32;
  p.limit = limit;
  // K splits: enough warps to cover the machine twice over, at least four K blocks each where the matrix allows it
  const int sm = sm_count > 0 ? sm_count : 148;
  const int row_tiles = (p.n_out + 15) / 16;
  int ks = 1;
  while (ks < 64 && row_tiles * ks < sm * 16 && p.kblocks / (ks * 2) >= 4) ks *= 2;
  int wk = ks < 8 ? ks : 8, ns = ks / wk;
  if (force_wk > 0) wk = force_wk;
  if (force_ns > 0) ns = force_ns;
  if ((wk != 1 && wk != 2 && wk != 4 && wk != 8) || ns < 1 || ns > 8 || (ns & (ns - 1)) != 0) return -1;
  // a cluster rank finishes rows_cta / ns whole columns
  while (ns > 1 && (128 / wk) % ns != 0) ns >>= 1;
  p.wk = wk;
  p.ns = ns;
  p.blocks_per_split = (p.kblocks + wk * ns - 1) / (wk * ns);
  const int n_ctas = (p.n_out + 128 / wk - 1) / (128 / wk);
  cudaError_t e;
  if (M <= 8) e = gated ? launch_gemv<1, true>(p, n_ctas, stream) : launch_gemv<1, false>(p, n_ctas, stream);
  else e = gated ? launch_gemv<2, true>(p, n_ctas, stream) : launch_gemv<2, false>(p, n_ctas, stream);
  eredu_count_launches(1);
  return static_cast<int>(e);
}
