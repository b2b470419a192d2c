// Decode-regime quantised linear layer: Y[M,N] = X[M,K] · dequant(Wq)[N,K]^T for M <= 8 tokens and 4-bit affine weights.
//
// With so few tokens the layer is a stream over the packed weights (0.5 B per weight), and what matters is that nothing
// but HBM sits on the critical path. This kernel therefore keeps the weights in registers from the load to the tensor
// core: no shared-memory operand tiles, no TMEM round trip, no producer / consumer hand-off (the tcgen05 pipeline of
// qgemm_tcgen05.cu serves M > 8, where the MMA is worth the staging).
//
//   warp          : a 16-row weight tile x a K range. The codes are stored tile by tile (16 rows x 64 columns = 512
//                   contiguous bytes, consecutive K blocks of a row tile adjacent), so the warp's stream is one contiguous
//                   run that it fetches with bulk copies (cp.async.bulk, 2 KB each) into a private four-slot ring in
//                   shared memory: several KB in flight per warp at no register cost. A lane then reads its 16 codes of
//                   rows g and g + 8 with two 8-byte shared-memory loads.
//   dequant       : one shift + one lop3 place two nibbles into the mantissas of a bf16 pair (128 + n). Groups of 64 or
//                   128 codes feed that to the tensor core as it is and apply scale and bias to the fp32 accumulators of
//                   the K block (RAW); smaller groups subtract 128 and apply (scale, bias) with one fma.rn.bf16x2 per pair
//   mma.sync      : m16n8k16, the weight tile as A (16 rows x 16 k), eight tokens as B; the k slots of an instruction
//                   are filled lane by lane with the codes that lane loaded, and the activations follow the same map, so
//                   no data is exchanged between lanes
//   split K       : across the warps of a CTA (through shared memory) and across the CTAs of a cluster (through
//                   distributed shared memory); the reducing threads add bias / residual or apply SwiGLU and store
//
// GATED: the weight holds gate rows [0, I) and up rows [I, 2I); a warp computes both tiles of its 16 output columns and
// the epilogue writes silu(gate) * up, so the activation never exists unfused.
//
// Numerics: weights are rounded to bf16 once after dequantisation, like in the tcgen05 kernel. The affine contract is eredu/src/backend/mlx/runtime/checkpoint/quantization.rs:1-8,137-232.
#include <cuda_bf16.h>

#include <algorithm>

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/peer.cuh"
#include "../common/ptx.cuh"
#include "../common/trace.cuh"

namespace eredu {

struct QGemvParams {
  const __nv_bfloat16* x;
  const uint8_t* wq;    // tiles [ceil(N/16)][K/64][16 rows][32 bytes], nibble order (n0,n2,n4,n6,n1,n3,n5,n7) in each u32
  const uint32_t* dq;   // tiles [ceil(N/16)][K/group][16 rows]: bf16 scale | bf16 bias << 16
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
  int* status;
  int use_comm;         // row-parallel shard: sum the result over the tensor-parallel group inside the kernel
  PeerComm comm;
};

constexpr int kGemvThreads = 256;

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

// Eight codes of one u32 -> four bf16 pairs (k, k+1), (k+2, k+3), ...: pair j sits in nibbles j and j + 4. A nibble
// OR-ed into the mantissa of 128.0 is 128 + code exactly; subtracting 128 and one fused multiply-add with (scale, bias)
// round once, like dequantising in fp32 and converting to bf16.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t s2, uint32_t b2, uint32_t* out) {
  constexpr uint32_t kMask = 0x000F000Fu, kBase = 0x43004300u, kOne = 0x3F803F80u, kMinus128 = 0xC300C300u;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t q = fma_bf16x2(lop3_and_or(w >> (4 * j), kMask, kBase), kOne, kMinus128);
    out[j] = fma_bf16x2(q, s2, b2);
  }
}

__device__ __forceinline__ void mma_bf16_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// Raw variant for groups of 64 or 128 codes: the tensor core multiplies 128 + code (the lop3 result as it is), and the
// affine map moves behind the MMA, where it is exact fp32 arithmetic on four accumulators per 64-wide K block:
//   sum_k (s (128 + n_k) + (b - 128 s)) x_k  =  s * sum_k (128 + n_k) x_k  +  (b - 128 s) * sum_k x_k
// The sums of the activations come from the tensor core too (an all-ones A operand). No bf16 arithmetic is left in the
// dequantisation (HFMA2 issues at half rate), and the weights are not rounded to bf16 at all.
__device__ __forceinline__ void raw_word(uint32_t w, uint32_t* out) {
  constexpr uint32_t kMask = 0x000F000Fu, kBase = 0x43004300u;
#pragma unroll
  for (int j = 0; j < 4; ++j) out[j] = lop3_and_or(w >> (4 * j), kMask, kBase);
}

__device__ __forceinline__ void mma_bf16_16816_zero(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                    uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Per-warp ring of bulk copies. A slot holds four consecutive K blocks of the warp's row tile(s): the codes (512 bytes
// per block and tile) followed by their (scale, bias) words (64 bytes per group and tile). Both are contiguous in global
// memory (tiled layouts), so a slot is filled by one bulk copy per tile and table: no registers are spent on prefetch
// and a warp keeps several KB in flight, which is what the HBM latency asks for.
constexpr int kGemvChunk = 4;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// GATED: two row tiles per warp (gate and up). RAW: accumulator-side affine map (group 64 / 128), else the weights are
// dequantised to bf16 in registers (any power-of-two group from 16).
template <bool GATED, bool RAW>
__global__ void __launch_bounds__(kGemvThreads, 2) qgemv4_kernel(const QGemvParams p) {
  constexpr int S = GATED ? 2 : 1;
  constexpr int TOK = 8;
  constexpr int C = kGemvChunk;
  constexpr int SLOTS = GATED ? 2 : 4;       // 9 KB of ring per warp either way
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                  // [8 warps][SLOTS]
  uint8_t* ring = smem + 256;
  float* red = reinterpret_cast<float*>(smem + 256);                  // partial tiles reuse the ring after the main loop

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
  const int kb1 = (n0 < p.n_out) ? min(kb0 + p.blocks_per_split, p.kblocks) : kb0;   // tiles beyond the matrix do nothing
  const int nchunks = (kb1 - kb0 + C - 1) / C;

  // slot layout: codes [S][C][512] | dq [S][gpc][16] words; gpc = groups per chunk
  const int gpc = max(1, (C * 64) >> p.group_shift);
  const int slot_bytes = S * C * 512 + S * gpc * 64;
  uint8_t* my_ring = ring + warp * SLOTS * slot_bytes;
  uint64_t* my_bars = bars + warp * SLOTS;
  const int groups_total = (p.kblocks * 64) >> p.group_shift;
  const int tile0 = n0 >> 4;

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) mbar_init(&my_bars[i], 1);
    fence_mbar_init();
  }
  __syncwarp();

  auto issue = [&](int c) {   // lane 0 only
    const int kb = kb0 + c * C;
    const int nb = min(C, kb1 - kb);
    const int g0 = (kb * 64) >> p.group_shift;
    const int ng = max(1, (nb * 64) >> p.group_shift);
    uint8_t* slot = my_ring + (c % SLOTS) * slot_bytes;
    uint64_t* bar = &my_bars[c % SLOTS];
    mbar_arrive_expect_tx(bar, static_cast<uint32_t>(S * (nb * 512 + ng * 64)));
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const size_t tile = static_cast<size_t>(tile0 + s * (p.n_out >> 4));   // GATED: the up tiles follow the gate tiles
      bulk_load(slot + s * C * 512, p.wq + (tile * p.kblocks + kb) * 512, static_cast<uint32_t>(nb * 512), bar);
      bulk_load(slot + S * C * 512 + s * gpc * 64, p.dq + (tile * groups_total + g0) * 16, static_cast<uint32_t>(ng * 64), bar);
    }
  };

  // weights do not depend on the previous kernel: the ring is full before the dependency wait
  if (lane == 0)
    for (int c = 0; c < min(SLOTS, nchunks); ++c) issue(c);

  pdl_wait();
  trace_mark(kTraceQGemm, kTraceAfterWait);
  pdl_launch_dependents();
  const unsigned int seq = p.use_comm ? *p.comm.seq : 0u;

  // activations: token g, the 16 values that match this lane's codes; one chunk (four blocks) ahead in registers
  const __nv_bfloat16* xrow = p.x + static_cast<size_t>(min(g, p.M - 1)) * p.ldx + t * 16;
  uint4 xq[C][2];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    const int k = min(kb0 + j, p.kblocks - 1);
    xq[j][0] = *reinterpret_cast<const uint4*>(xrow + k * 64);
    xq[j][1] = *reinterpret_cast<const uint4*>(xrow + k * 64 + 8);
  }

  float acc[S][4];
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[s][j] = 0.f;

  // this lane's fixed offsets inside a slot
  const uint32_t code_off = g * 32 + t * 8;
  const int lane_group = (t * 16) >> p.group_shift;          // group of the lane's codes inside a block (groups below 64)
  constexpr uint32_t kOnes = 0x3F803F80u;

  bool ok = true;
  for (int c = 0; c < nchunks; ++c) {
    const uint8_t* slot = my_ring + (c % SLOTS) * slot_bytes;
    ok = mbar_wait(&my_bars[c % SLOTS], (c / SLOTS) & 1, p.status, kStatusTmaFullTimeout);
    if (!ok) break;
    const int kbc = kb0 + c * C;
    const int nb = min(C, kb1 - kbc);
#pragma unroll
    for (int j = 0; j < C; ++j) {
      if (j < nb) {
        const uint32_t xb[8] = {xq[j][0].x, xq[j][0].y, xq[j][0].z, xq[j][0].w, xq[j][1].x, xq[j][1].y, xq[j][1].z, xq[j][1].w};
        {
          // the same block of the next chunk (clamped: a value that is never used)
          const int k = min(kbc + C + j, p.kblocks - 1);
          xq[j][0] = *reinterpret_cast<const uint4*>(xrow + k * 64);
          xq[j][1] = *reinterpret_cast<const uint4*>(xrow + k * 64 + 8);
        }
        const int gi = RAW ? ((j * 64) >> p.group_shift) : (((j * 64) >> p.group_shift) + lane_group);
        float tx[4];
        if (RAW) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (i == 0) mma_bf16_16816_zero(tx, kOnes, kOnes, kOnes, kOnes, xb[0], xb[1]);
            else mma_bf16_16816(tx, kOnes, kOnes, kOnes, kOnes, xb[2 * i], xb[2 * i + 1]);
          }
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
          const uint8_t* codes = slot + (s * C + j) * 512 + code_off;
          const uint32_t* dq = reinterpret_cast<const uint32_t*>(slot + S * C * 512 + s * gpc * 64) + gi * 16 + g;
          const uint2 w_lo = *reinterpret_cast<const uint2*>(codes);
          const uint2 w_hi = *reinterpret_cast<const uint2*>(codes + 8 * 32);
          const uint32_t sc_lo = dq[0], sc_hi = dq[8];
          uint32_t a[2][8];
          if (RAW) {
            raw_word(w_lo.x, &a[0][0]);
            raw_word(w_lo.y, &a[0][4]);
            raw_word(w_hi.x, &a[1][0]);
            raw_word(w_hi.y, &a[1][4]);
            float tmp[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (i == 0) mma_bf16_16816_zero(tmp, a[0][0], a[1][0], a[0][1], a[1][1], xb[0], xb[1]);
              else mma_bf16_16816(tmp, a[0][2 * i], a[1][2 * i], a[0][2 * i + 1], a[1][2 * i + 1], xb[2 * i], xb[2 * i + 1]);
            }
            const float s_lo = __uint_as_float(sc_lo << 16), b_lo = __uint_as_float(sc_lo & 0xFFFF0000u);
            const float s_hi = __uint_as_float(sc_hi << 16), b_hi = __uint_as_float(sc_hi & 0xFFFF0000u);
            const float c_lo = fmaf(-128.f, s_lo, b_lo), c_hi = fmaf(-128.f, s_hi, b_hi);
            acc[s][0] = fmaf(s_lo, tmp[0], fmaf(c_lo, tx[0], acc[s][0]));
            acc[s][1] = fmaf(s_lo, tmp[1], fmaf(c_lo, tx[1], acc[s][1]));
            acc[s][2] = fmaf(s_hi, tmp[2], fmaf(c_hi, tx[2], acc[s][2]));
            acc[s][3] = fmaf(s_hi, tmp[3], fmaf(c_hi, tx[3], acc[s][3]));
          } else {
            const uint32_t s2l = __byte_perm(sc_lo, sc_lo, 0x1010), b2l = __byte_perm(sc_lo, sc_lo, 0x3232);
            const uint32_t s2h = __byte_perm(sc_hi, sc_hi, 0x1010), b2h = __byte_perm(sc_hi, sc_hi, 0x3232);
            dequant_word(w_lo.x, s2l, b2l, &a[0][0]);
            dequant_word(w_lo.y, s2l, b2l, &a[0][4]);
            dequant_word(w_hi.x, s2h, b2h, &a[1][0]);
            dequant_word(w_hi.y, s2h, b2h, &a[1][4]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_bf16_16816(acc[s], a[0][2 * i], a[1][2 * i], a[0][2 * i + 1], a[1][2 * i + 1], xb[2 * i], xb[2 * i + 1]);
          }
        }
      }
    }
    __syncwarp();                                   // every lane has its fragments of this slot in registers
    if (lane == 0 && c + SLOTS < nchunks) issue(c + SLOTS);
  }
  if (!ok) {
    // a copy never landed (status recorded): give the other copies of this warp their bounded wait before the ring is reused
    for (int c = 0; c < min(SLOTS, nchunks); ++c) mbar_wait(&my_bars[c], 0, p.status, kStatusTmaFullTimeout);
  }

  // ------------------------------------------------------------------ reduction over the K splits and epilogue
  // plane of this warp's K split: [S][TOK][rows_cta + 4]; lane holds rows g / g + 8 and tokens 2t, 2t + 1 of each tile
  __syncthreads();                                  // every warp is done with its ring: the partial tiles take its place
  const int ldn = rows_cta + 4;
  const int plane = S * TOK * ldn;
  float* mine = red + wkk * plane;
#pragma unroll
  for (int s = 0; s < S; ++s) {
    float* base = mine + (s * TOK + 2 * t) * ldn + wr * 16 + g;
    base[0] = acc[s][0];
    base[ldn] = acc[s][1];
    base[8] = acc[s][2];
    base[ldn + 8] = acc[s][3];
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
  if (!GATED && p.use_comm) {
    // ---- row-parallel shard: one-shot all-reduce over peer memory in the same kernel. A pair of tokens of one output
    // column travels as a 4-byte bf16x2 word into the sentinel-initialised slot of every peer (complete once it differs
    // from the sentinel: no flag, fence or barrier); then this rank sums the words of all ranks in rank order, so every
    // rank holds the same bits. The word layout and the parity protocol are those of the dense GEMM's fused all-reduce.
    const int parity = static_cast<int>(seq & 1u);
    const int pair_items = ((p.M + 1) / 2) * cols;
    auto local_sum = [&](int m, int c) {
      float sum = 0.f;
      if (m >= p.M) return sum;
      const int off = m * ldn + c;
      for (int q = 0; q < p.ns; ++q) {
        if (p.ns > 1) {
          const uint32_t remote = mapa_shared(red_addr, static_cast<uint32_t>(q));
          for (int w = 0; w < p.wk; ++w) sum += ld_dsmem_f32(remote + static_cast<uint32_t>(w * plane + off) * 4u);
        } else {
          for (int w = 0; w < p.wk; ++w) sum += red[w * plane + off];
        }
      }
      return sum;
    };
    for (int idx = threadIdx.x; idx < pair_items; idx += kGemvThreads) {
      const int pi = idx / cols, c = static_cast<int>(crank) * cols + idx % cols;
      const int n = blockIdx.x * rows_cta + c;
      if (n >= p.n_out) continue;
      const uint32_t packed = lamport_payload(pack_bf16x2(local_sum(2 * pi, c), local_sum(2 * pi + 1, c)));
      const size_t word = (static_cast<size_t>(pi) * p.N + n) * 4;
      for (int peer = 0; peer < p.comm.size; ++peer)
        asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(lamport_slot(p.comm, peer, parity, p.comm.rank) + word), "r"(packed)
                     : "memory");
    }
    for (int idx = threadIdx.x; idx < pair_items; idx += kGemvThreads) {
      const int pi = idx / cols, c = static_cast<int>(crank) * cols + idx % cols;
      const int n = blockIdx.x * rows_cta + c;
      if (n >= p.n_out) continue;
      const size_t word = (static_cast<size_t>(pi) * p.N + n) * 4;
      uint32_t got[kMaxRanks];
      uint32_t miss = (1u << p.comm.size) - 1u;
      const long long t0 = clock64();
      bool first_pass = true;
      while (true) {
#pragma unroll
        for (int src = 0; src < kMaxRanks; ++src)
          if ((miss >> src) & 1u)
            asm volatile("ld.volatile.global.u32 %0, [%1];"
                         : "=r"(got[src])
                         : "l"(lamport_slot(p.comm, p.comm.rank, parity, src) + word)
                         : "memory");
#pragma unroll
        for (int src = 0; src < kMaxRanks; ++src)
          if (((miss >> src) & 1u) && got[src] != kLamportEmpty) {
            miss &= ~(1u << src);
            asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(lamport_slot(p.comm, p.comm.rank, parity, src) + word),
                         "r"(kLamportEmpty)
                         : "memory");
          }
        if (miss == 0u) break;
        if (!first_pass && clock64() - t0 > kWaitCycleLimit) {
          report_status(p.status, kStatusPeerFlagTimeout);
          break;
        }
        first_pass = false;
      }
      float v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int src = 0; src < kMaxRanks; ++src)
        if (src < p.comm.size && !((miss >> src) & 1u)) {
          v0 += bf16_lo(got[src]);
          v1 += bf16_hi(got[src]);
        }
      const float bv = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int m = 2 * pi + h;
        if (m >= p.M) break;
        float out = (h == 0 ? v0 : v1) + bv;
        if (p.residual != nullptr) out += __bfloat162float(p.residual[static_cast<size_t>(m) * p.ldr + n]);
        if (p.out_fp32) static_cast<float*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = out;
        else static_cast<__nv_bfloat16*>(p.y)[static_cast<size_t>(m) * p.ldy + n] = __float2bfloat16(out);
      }
    }
  } else
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
  if (p.use_comm && threadIdx.x == 0) finish_call(p.comm, seq, gridDim.x * gridDim.y);
  trace_mark(kTraceQGemm, kTraceEnd);
}

// Dynamic shared memory of a launch: barriers, then the larger of the eight per-warp rings and the partial tiles.
static int gemv_smem_bytes(const QGemvParams& p, bool gated) {
  const int S = gated ? 2 : 1, C = kGemvChunk, slots = gated ? 2 : 4;
  const int gpc = std::max(1, (C * 64) >> p.group_shift);
  const int ring = 8 * slots * (S * C * 512 + S * gpc * 64);
  const int red = p.wk * S * 8 * (128 / p.wk + 4) * 4;
  return 256 + std::max(ring, red);
}

template <bool GATED, bool RAW>
static cudaError_t launch_gemv(const QGemvParams& p, int n_ctas, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ctas, p.ns, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  const int smem = gemv_smem_bytes(p, GATED);
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qgemv4_kernel<GATED, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cfg.dynamicSmemBytes = smem;
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
  return cudaLaunchKernelEx(&cfg, qgemv4_kernel<GATED, RAW>, p);
}

}  // namespace eredu

using namespace eredu;

// Y = X dequant(Wq)^T (+bias) (+residual), or with gated != 0 Y[M, N/2] = silu(X Wgate^T) * (X Wup^T), for M <= 8.
// wq: 4-bit codes in the tiled kernel layout ([ceil(N/16)][K/64][16][32] bytes); dq: u32 [K/group, N] holding the bf16
// scale in the low and the bf16 bias in the high half; group a power of two >= 16; K a multiple of 64. Returns -2 for shapes this
// kernel does not take (the caller then uses eredu_qgemm). `comm` (a PeerComm, or null): the rank's result is a partial sum
// of a row-parallel shard and is summed over the group inside the kernel (bias and residual added once, after the sum).
extern "C" int eredu_qgemv4(const void* X, const void* wq, const void* dq, void* Y, const void* residual, const void* bias,
                            int M, int N, int K, int ldx, int ldy, int ldr, int group, int out_fp32, int gated, float limit,
                            int force_wk, int force_ns, int force_exact_bf16, int sm_count, const void* comm, int* status,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 8 || K % 64 != 0 || group < 16 || group > 128 || (group & (group - 1)) != 0 || K % group != 0 || ldx % 8 != 0)
    return -2;
  if (gated && (N % 32 != 0 || residual != nullptr)) return -2;   // the up rows start on a row-tile boundary
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
  p.status = status;
  if (comm != nullptr) {
    // the sum over the group runs in the epilogue; residual and bias are added once, after it
    const PeerComm* pc = static_cast<const PeerComm*>(comm);
    if (gated || out_fp32) return -2;
    if (static_cast<long long>((M + 1) / 2) * N * 4 > pc->lam_bytes) return -2;
    p.use_comm = 1;
    p.comm = *pc;
  }
  // K splits. A warp streams best when it has many K blocks to itself, but an SM wants two CTAs (sixteen warps) to fill
  // its issue slots, small CTAs spread more evenly over the SMs, and every further round of CTAs on an SM pays the fixed
  // costs again (first data from HBM, reduction, epilogue: worth about sixteen K blocks). Estimate for each power-of-two
  // split: the evenly spread work + half a CTA of imbalance + the fixed cost per round; take the smallest.
  const int sm = sm_count > 0 ? sm_count : 148;
  const int row_tiles = (p.n_out + 15) / 16;
  int ks = 1;
  {
    double best = 1e30;
    for (int cand = 1; cand <= 64; cand *= 2) {
      const int cwk = cand < 8 ? cand : 8, cns = cand / cwk;
      if ((128 / cwk) % cns != 0) continue;
      const int bps = ((p.kblocks + cand - 1) / cand + 3) / 4 * 4;
      if (cand > 1 && bps * (cand - 1) >= p.kblocks) break;          // the last split would be empty
      const long ctas = static_cast<long>((row_tiles + 8 / cwk - 1) / (8 / cwk)) * cns;
      const long n = (ctas + sm - 1) / sm;                           // CTAs of the busiest SM
      const double work = static_cast<double>(ctas) * 8.0 * bps / sm;   // warp-blocks per SM when spread evenly
      const double t = work / 10.0 + 0.5 * bps + 16.0 * ((n + 1) / 2) + 2.0 * (cns - 1);
      if (t < best) {
        best = t;
        ks = cand;
      }
    }
  }
  int wk = ks < 8 ? ks : 8, ns = ks / wk;
  if (force_wk > 0) wk = force_wk;
  if (force_ns > 0) ns = force_ns;
  if ((wk != 1 && wk != 2 && wk != 4 && wk != 8) || ns < 1 || ns > 8 || (ns & (ns - 1)) != 0) return -1;
  // a cluster rank finishes rows_cta / ns whole columns
  while (ns > 1 && (128 / wk) % ns != 0) ns >>= 1;
  p.wk = wk;
  p.ns = ns;
  // splits start on multiples of four K blocks: a slot of the copy ring then starts on a group boundary for every group size
  p.blocks_per_split = ((p.kblocks + wk * ns - 1) / (wk * ns) + 3) / 4 * 4;
  const int n_ctas = (p.n_out + 128 / wk - 1) / (128 / wk);
  const bool raw = group >= 64 && force_exact_bf16 == 0;
  cudaError_t e = gated ? (raw ? launch_gemv<true, true>(p, n_ctas, stream) : launch_gemv<true, false>(p, n_ctas, stream))
                        : (raw ? launch_gemv<false, true>(p, n_ctas, stream) : launch_gemv<false, false>(p, n_ctas, stream));
  eredu_count_launches(1);
  return static_cast<int>(e);
}
