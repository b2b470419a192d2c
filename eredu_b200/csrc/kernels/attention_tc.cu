// Prefill attention on the 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma with the accumulators in
// tensor memory, K / V pages arrive by TMA straight from the paged cache.
//
// One CTA = 256 query rows (two tiles of 128, "a" and "b") of one (sequence, query head); keys are walked in tiles of 128
// (eight 16-token pages). The two query tiles share every K / V tile and alternate on the tensor core, so the softmax of
// one runs while the MMAs of the other execute.
//   warp 0      : TMA producer - both Q tiles once, then per key tile sixteen boxes for K and sixteen for V (a page is
//                 [16 keys x 64 values] per half of the head dimension, 128-byte swizzled); K and V have their own
//                 two-deep rings, because a K tile is free a whole step before its V tile
//   warp 1      : MMA issuer (one thread) - S_w = Q_w K_j^T into tile w's score columns, O_w += P_w V_j with P_w read
//                 from tensor memory (the A operand) and V as it lies in the cache ([key][value], MN-major B operand)
//   warps 2..5  : softmax of tile a, warps 6..9 of tile b, one query row per thread (TMEM lane = row): the whole score
//                 row comes into registers with one wait, P = exp2(S * scale - m) goes back as packed bf16 over the
//                 first 64 score columns. The output accumulator stays in tensor memory; it is rescaled only when a
//                 row's maximum has grown by more than 2^8 since the scale in use was chosen (the probabilities are
//                 then at most 256, exact enough in bf16, and the final division by the row sum takes the scale out).
// TMEM columns: S_a [0,128) | S_b [128,256) | O_a [256,384) | O_b [384,512).
// Causal masking by position (queries are the last q_len positions of their sequence, so chunked prefill and cached
// prefixes work); key tiles beyond a query tile's last position are never loaded. CTAs with the most key tiles are
// scheduled first.
//
// Head size 64 or 128, optional sliding window (key tiles before the window are skipped) and sink logits. Same
// online-softmax recurrence and semantics as attn_prefill_kernel in attention.cu and as the reference's blockwise attention (eredu/src/backend/mlx/nn/attention.rs:346-436,
// runtime/cache/kv.rs:2267-2436). Every wait is bounded; on expiry the status word is set and the CTA leaves through the
// common exit (TMEM is freed there).
#include <cuda_bf16.h>

#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "../common/trace.cuh"

namespace eredu {

struct AttnTcParams {
  __nv_bfloat16* out;          // [tokens, n_q, 128]
  const int* block_table;      // [batch, max_pages]
  const int* seq_lens;         // kv length after this call, per sequence
  const int* cu_q;             // [batch + 1] query-row offsets
  const float* sinks;          // optional [n_q_heads]: logit of a virtual key with zero value (enters the normaliser only)
  int max_pages;
  int n_q_heads, n_kv_heads;
  int window;                  // 0: none; else a query at position p sees keys in (p - window, p]
  float scale_log2;
  int* status;
};

constexpr int kTcThreads = 320;
constexpr int kTcTile = 128;            // query rows per tile and keys per tile
constexpr int kTcRows = 2 * kTcTile;    // query rows per CTA
constexpr int kTcHalf = 128 * 64 * 2;   // one [128 rows][64 bf16] swizzled half tile: 16 KB
// shared memory: Q_a, Q_b (D / 64 halves each) | K ring (2 x D / 64 halves) | V ring (2 x D / 64 halves) | barriers
constexpr int tc_smem(int d) { return 1024 + 3 * 2 * (d / 64) * kTcHalf + 256; }
// A quarter of the exponentials as a polynomial on the FMA pipe (build option). Measured slower here (1153 against 1192
// TFLOP/s at 32k tokens, 1112 against 1170 at 8k): the softmax warps are bound by instruction issue, not by the
// special-function unit, so the extra FMA-pipe instructions cost more than the unit they relieve.
#ifndef EREDU_ATTN_POLY_EXP
#define EREDU_ATTN_POLY_EXP 0
#endif
constexpr bool kTcPolyExp = EREDU_ATTN_POLY_EXP != 0;
constexpr float kTcRescale = 8.f;       // log2 units a row maximum may outgrow the scale in use

// MN-major operand tile stored as [k rows][64 bf16] (128-byte rows, 128B swizzle): 64-element blocks along MN are `lbo`
// bytes apart, 8-row groups along K are 1024 bytes apart. Advancing K by 16 = +2048 bytes on the start address.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
constexpr uint32_t kIdescQK = umma_idesc_bf16(128, 128);                 // both operands K-major

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, int w, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const AttnTcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr int NH = D / 64;                                           // 64-wide halves of the head dimension
  constexpr uint32_t kIdescPV = umma_idesc_bf16(128, D) | (1u << 16);  // B (= V) MN-major, N = head dimension
  uint8_t* q_s = smem;                                                 // tile w at + w * NH halves
  uint8_t* k_s = q_s + 2 * NH * kTcHalf;                               // stage s at + s * NH halves
  uint8_t* v_s = k_s + 2 * NH * kTcHalf;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * NH * kTcHalf);
  uint64_t* q_full = bars;                  // 1
  uint64_t* k_full = bars + 1;              // [2]
  uint64_t* k_empty = bars + 3;             // [2]
  uint64_t* v_full = bars + 5;              // [2]
  uint64_t* v_empty = bars + 7;             // [2]
  uint64_t* s_full = bars + 9;              // [2] per query tile
  uint64_t* p_full = bars + 11;             // [2] per query tile, 128 arrivals
  uint64_t* o_final = bars + 13;            // [2] per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  pdl_launch_early();
  trace_mark(kTraceAttnPrefill, kTraceStart);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads vary fastest: the first wave holds the longest query tiles of every head (longest-first balances the causal
  // triangle), and neighbouring CTAs are query heads of one key / value head reading the same pages
  const int b = blockIdx.z, head = blockIdx.x, qt = gridDim.y - 1 - blockIdx.y;
  const int q0 = p.cu_q[b], q_len = p.cu_q[b + 1] - q0;
  const int kv_len = p.seq_lens[b];
  const int row0 = qt * kTcRows;
  if (row0 >= q_len) return;                                            // uniform: before any barrier or allocation
  const int kv_head = head / (p.n_q_heads / p.n_kv_heads);
  const int pos0 = kv_len - q_len + row0;                               // position of the CTA's first query row
  // causal: nothing beyond the position of a tile's last row
  const int n_a = min(kv_len - 1, pos0 + kTcTile - 1) / kTcTile + 1;
  const int n_b = row0 + kTcTile < q_len ? min(kv_len - 1, pos0 + kTcRows - 1) / kTcTile + 1 : 0;
  const int n_tiles = max(n_a, n_b);
  // sliding window: key tiles that lie wholly before the window of a tile's FIRST row are skipped
  const int j0_a = p.window > 0 ? max(0, pos0 - p.window + 1) / kTcTile : 0;
  const int j0_b = p.window > 0 ? max(0, pos0 + kTcTile - p.window + 1) / kTcTile : 0;
  const int j0 = n_b > 0 ? min(j0_a, j0_b) : j0_a;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&o_final[s], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
  trace_mark(kTraceAttnPrefill, kTraceAfterWait);
  pdl_launch_dependents();

  bool ok = true;
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * NH * kTcHalf);
      for (int w = 0; w < 2; ++w)
        for (int h = 0; h < NH; ++h)
          tma_load_3d(q_s + (w * NH + h) * kTcHalf, &tmQ, h * 64, head, q0 + row0 + w * kTcTile, q_full);
      const int* pages = p.block_table + static_cast<size_t>(b) * p.max_pages;
      for (int jj = 0; j0 + jj < n_tiles && ok; ++jj) {
        const int j = j0 + jj;                                           // key tile; jj counts this CTA's iterations
        const int s = jj & 1;
        const uint32_t reuse_parity = ((jj >> 1) - 1) & 1;
        int page[8];
#pragma unroll
        for (int pg = 0; pg < 8; ++pg) {
          const int page_index = j * 8 + pg;
          page[pg] = page_index < p.max_pages ? pages[page_index] : 0;            // beyond the table: the reserved page (masked)
        }
        if (jj >= 2) ok = mbar_wait(&k_empty[s], reuse_parity, p.status, kStatusSmemEmptyTimeout);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[s], NH * kTcHalf);
#pragma unroll
        for (int pg = 0; pg < 8; ++pg)
          for (int h = 0; h < NH; ++h) tma_load_4d(k_s + (s * NH + h) * kTcHalf + pg * 2048, &tmK, h * 64, 0, kv_head, page[pg], &k_full[s]);
        if (jj >= 2) ok = mbar_wait(&v_empty[s], reuse_parity, p.status, kStatusSmemEmptyTimeout);
        if (!ok) break;
        mbar_arrive_expect_tx(&v_full[s], NH * kTcHalf);
#pragma unroll
        for (int pg = 0; pg < 8; ++pg)
          for (int h = 0; h < NH; ++h) tma_load_4d(v_s + (s * NH + h) * kTcHalf + pg * 2048, &tmV, h * 64, 0, kv_head, page[pg], &v_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(q_s);
      // jj: this CTA's iteration (selects the K / V stage); tile w is active on key tiles [first_w, n_w)
      const int first[2] = {j0_a, j0_b}, last[2] = {n_a, n_b};
      auto issue_s = [&](int w, int jj) {
        const uint32_t qa = q_addr + w * NH * kTcHalf;
        const uint32_t ka = smem_u32(k_s + (jj & 1) * NH * kTcHalf);
        const uint32_t d = tmem + w * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {      // K = head dimension: four 16-steps per 64-wide half
          const uint32_t off = (kk >> 2) * kTcHalf + (kk & 3) * 32;
          umma_f16(d, umma_desc_k_sw128(qa + off), umma_desc_k_sw128(ka + off), kIdescQK, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[w]);
      };
      auto issue_pv = [&](int w, int jj, bool fresh) {
        const uint32_t va = smem_u32(v_s + (jj & 1) * NH * kTcHalf);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)             // K = keys: P from tensor memory (8 columns per step), V MN-major (2048 bytes per step)
          umma_f16_ts(tmem + 256 + w * 128, tmem + w * 128 + kk * 8, umma_desc_mn_sw128(va + kk * 2048, kTcHalf), kIdescPV,
                      (!fresh || kk > 0) ? 1u : 0u);
      };
      auto active = [&](int w, int j) { return j >= first[w] && j < last[w]; };
      ok = mbar_wait(q_full, 0, p.status, kStatusTmaFullTimeout);
      if (ok) ok = mbar_wait(&k_full[0], 0, p.status, kStatusTmaFullTimeout);
      if (ok) {
        tc_fence_after_sync();
        if (active(0, j0)) issue_s(0, 0);
        if (active(1, j0)) issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      int done[2] = {0, 0};                        // softmax rounds completed per tile: parity of p_full
      for (int jj = 0; j0 + jj < n_tiles && ok; ++jj) {
        const int j = j0 + jj;
        const bool next = j + 1 < n_tiles;
        bool k_ready = false;
        ok = mbar_wait(&v_full[jj & 1], (jj >> 1) & 1, p.status, kStatusTmaFullTimeout);
        for (int w = 0; w < 2 && ok; ++w) {
          if (active(w, j)) {
            ok = mbar_wait(&p_full[w], done[w] & 1, p.status, kStatusAccumTimeout);   // P_w(j) is in tensor memory, O_w is rescaled
            if (!ok) break;
            tc_fence_after_sync();
            issue_pv(w, jj, done[w] == 0);
            ++done[w];
          }
          if (w == 1) umma_commit(&v_empty[jj & 1]);
          if (active(w, j + 1)) {
            if (!k_ready) {
              ok = mbar_wait(&k_full[(jj + 1) & 1], ((jj + 1) >> 1) & 1, p.status, kStatusTmaFullTimeout);
              if (!ok) break;
              tc_fence_after_sync();
              k_ready = true;
            }
            issue_s(w, jj + 1);
          } else if (j + 1 == last[w]) {
            umma_commit(&o_final[w]);
          }
        }
        if (ok && next) umma_commit(&k_empty[(jj + 1) & 1]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, one row per thread
    const int w = (warp - 2) >> 2;                                       // query tile of this warp
    const int n_w = w == 0 ? n_a : n_b;
    const int j0_w = w == 0 ? j0_a : j0_b;
    const int quarter = warp & 3;                                        // TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;
    const int tile_row0 = row0 + w * kTcTile;
    const int tile_pos0 = pos0 + w * kTcTile;
    const int qpos = tile_pos0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + w * 128;
    const uint32_t o_addr = tmem + lane_addr + 256 + w * 128;
    float m = 0.f, l = 0.f;
    for (int j = j0_w; j < n_w && ok; ++j) {
      const int it = j - j0_w;                                           // this tile's round: parity of its barriers
      ok = mbar_wait(&s_full[w], it & 1, p.status, kStatusAccumTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sc[8][16];
#pragma unroll
      for (int c = 0; c < 8; ++c) tmem_ld16(s_addr + c * 16, sc[c]);
      tmem_wait_ld();
      const int key0 = j * kTcTile;
      const bool before = p.window > 0 && key0 <= tile_pos0 + kTcTile - 1 - p.window;     // some row's window starts inside or after this tile
      if (key0 + kTcTile - 1 > tile_pos0 || key0 + kTcTile > kv_len || before) {   // some (row, key) of the tile is masked: -inf gives p = 0
        const int visible = min(qpos, kv_len - 1) - key0;                // keys hidden .. visible of this tile are seen by this row
        const int hidden = p.window > 0 ? qpos - p.window + 1 - key0 : 0;
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c * 16 + i > visible || c * 16 + i < hidden) sc[c][i] = 0xFF800000u;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains of three-input maxima
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int i = 0; i < 16; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sc[c][i]), __uint_as_float(sc[c][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = mx * p.scale_log2;                             // -inf for a fully masked row: every comparison below is false
      if (it == 0) {
        m = m_new == -INFINITY ? 0.f : m_new;
      } else {
        const bool grow = m_new > m + kTcRescale;
        if (__any_sync(0xffffffffu, grow)) {                             // O_w(j - 1) is complete: s_full followed it on the tensor core
          const float alpha = grow ? ex2_approx(m - m_new) : 1.f;
          if (grow) m = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t r[16];
            tmem_ld16(o_addr + c * 16, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st16(o_addr + c * 16, r);
          }
        }
      }
      // p = exp2(s * scale - m), two values per FMA / add; sums in four chains
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), shift2 = pack_f32x2(-m, -m);
      uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c2 = 0; c2 < 4; ++c2) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int c = c2 * 2 + (i >> 4), e = i & 15;
          float t0, t1;
          unpack_f32x2(fma_f32x2(pack_b32x2(sc[c][e], sc[c][e + 1]), scale2, shift2), t0, t1);
          // every fourth pair takes the polynomial on the FMA pipe instead of the special-function unit
          const bool poly = kTcPolyExp && ((i >> 1) & 3) == 3;
          const float p0 = poly ? ex2_poly(t0) : ex2_approx(t0), p1 = poly ? ex2_poly(t1) : ex2_approx(t1);
          acc[(i >> 1) & 3] = add_f32x2(acc[(i >> 1) & 3], pack_f32x2(p0, p1));
          packed[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st16(s_addr + c2 * 16, packed);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[w]);
      float s0, s1;
      unpack_f32x2(add_f32x2(add_f32x2(acc[0], acc[1]), add_f32x2(acc[2], acc[3])), s0, s1);
      l += s0 + s1;
    }
    if (ok && n_w > 0) ok = mbar_wait(&o_final[w], 0, p.status, kStatusAccumTimeout);
    if (ok && n_w > 0) {
      tc_fence_after_sync();
      const bool store = tile_row0 + row < q_len;
      if (p.sinks != nullptr) l += ex2_approx(p.sinks[head] * 1.4426950408889634f - m);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(q0 + tile_row0 + row) * p.n_q_heads + head) * D);
#pragma unroll 1
      for (int c = 0; c < D / 16; ++c) {
        uint32_t r[16];
        tmem_ld16(o_addr + c * 16, r);
        tmem_wait_ld();
        if (store) {
          uint4 v0, v1;
          v0.x = pack_bf16x2(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
          v0.y = pack_bf16x2(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
          v0.z = pack_bf16x2(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
          v0.w = pack_bf16x2(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
          v1.x = pack_bf16x2(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
          v1.y = pack_bf16x2(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
          v1.z = pack_bf16x2(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
          v1.w = pack_bf16x2(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
          dst[c * 2] = v0;
          dst[c * 2 + 1] = v1;
        }
      }
    }
  }
  // common exit: every role comes here, also after a timed-out wait; the tensor memory goes back
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  trace_mark(kTraceAttnPrefill, kTraceEnd);
}

}  // namespace eredu

using namespace eredu;

// Causal prefill attention over the paged cache, head size 64 or 128, optional sliding window and sink logits.
// q: [tokens, n_q, D] bf16 (contiguous); k_cache / v_cache: [pages, n_kv, 16, D] bf16 (contiguous); sinks: fp32 [n_q] or
// null. Same arguments as eredu_attn_prefill otherwise. Returns -2 for shapes it does not take.
template <int D>
static int launch_attn_tc(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnTcParams& p, dim3 grid,
                          cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem(D)) != cudaSuccess) return -1;
    configured[dev] = true;
  }
  return static_cast<int>(launch_pdl(attn_prefill_tc_kernel<D>, grid, dim3(kTcThreads), tc_smem(D), stream, tmQ, tmK, tmV, p));
}

extern "C" int eredu_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                                     const int* seq_lens, const int* cu_q, const float* sinks, int batch, int total_q, int max_q_len,
                                     int max_pages, int num_pages, int n_q_heads, int n_kv_heads, int head_dim, int window, float scale,
                                     int* status, cudaStream_t stream) {
  if ((head_dim != 128 && head_dim != 64) || batch <= 0 || total_q <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 || window < 0)
    return -2;
  const uint64_t D = static_cast<uint64_t>(head_dim);
  CUtensorMap tmQ, tmK, tmV;
  // q as [tokens][heads][D]: box = 128 tokens x 1 head x 64 values
  int r = make_tma_3d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, static_cast<uint64_t>(n_q_heads),
                      static_cast<uint64_t>(total_q), D * 2, static_cast<uint64_t>(n_q_heads) * D * 2, 64, 1, 128);
  if (r != 0) return -100 + r;
  r = make_tma_4d(&tmK, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, 16, static_cast<uint64_t>(n_kv_heads),
                  static_cast<uint64_t>(num_pages), D * 2, 16 * D * 2, static_cast<uint64_t>(n_kv_heads) * 16 * D * 2, 64, 16, 1, 1);
  if (r != 0) return -200 + r;
  r = make_tma_4d(&tmV, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, 16, static_cast<uint64_t>(n_kv_heads),
                  static_cast<uint64_t>(num_pages), D * 2, 16 * D * 2, static_cast<uint64_t>(n_kv_heads) * 16 * D * 2, 64, 16, 1, 1);
  if (r != 0) return -300 + r;
  AttnTcParams p = {};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.cu_q = cu_q;
  p.sinks = sinks;
  p.max_pages = max_pages;
  p.n_q_heads = n_q_heads;
  p.n_kv_heads = n_kv_heads;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid(n_q_heads, (max_q_len + kTcRows - 1) / kTcRows, batch);
  const int e = head_dim == 128 ? launch_attn_tc<128>(tmQ, tmK, tmV, p, grid, stream) : launch_attn_tc<64>(tmQ, tmK, tmV, p, grid, stream);
  eredu_count_launches(1);
  return e;
}
