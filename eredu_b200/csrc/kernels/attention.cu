// Paged-KV attention for prefill (causal / sliding window, GQA) and decode (split-KV, 1..k+1 query
// tokens per sequence for speculative verification).
//
// KV cache layout per layer: K and V are [num_pages, n_kv_heads, page_size = 16, head_dim] bf16, so one
// (page, kv head) is a contiguous 16 x head_dim slab. A block table [batch, max_pages] (int32) maps
// logical page -> physical page; everything stays on the device — there is no host loop over cache
// blocks (the reference evaluates once per block from the host: eredu/src/backend/mlx/runtime/cache/
// kv.rs:2017-2128, recurrence :2267-2436).
//
// Both kernels use the exact blockwise online-softmax recurrence (running max m, running sum l,
// rescaled accumulator) with bf16 tensor-core MMAs and fp32 state.
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/trace.cuh"

namespace eredu {

constexpr int kPage = 16;

struct AttnParams {
  const __nv_bfloat16* q;  // [total_q, n_q_heads, D]
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;       // [total_q, n_q_heads, D]
  const int* block_table;   // [B, max_pages]
  const int* seq_lens;      // [B] kv length including the new tokens
  const int* cu_q;          // [B+1] prefix sums of query lengths (prefill); null for decode
  const float* sinks;       // optional [n_q_heads] attention-sink logits
  float* part_o;            // decode scratch [B*rows_total, splits, D]
  float* part_ml;           // decode scratch [B*rows_total, splits, 2]
  int* counters;            // decode scratch [B * n_kv_heads], zero between launches (split arrival tickets)
  int max_pages;
  int n_q_heads, n_kv_heads;
  int q_per_seq;  // decode: query tokens per sequence
  int t0, t_count;  // decode: token sub-range handled by this launch
  int splits;
  int window;  // 0 = full attention, else sliding window width
  float scale_log2;  // softmax scale * log2(e)
  // Decode with the projection output taken as is (qkv != null): the kernel applies the per-head q/k RMSNorm and RoPE
  // itself and appends the new K/V rows to their pages, so no separate RoPE / append launch precedes it.
  const __nv_bfloat16* qkv;   // [B * q_per_seq, ld_qkv] = [q heads | k heads | v heads] x D
  const int* positions;       // [B * q_per_seq] rotary position of every new token
  const long long* slots;     // [B * q_per_seq] page * 16 + offset of every new token, < 0 = do not store
  const float* inv_freq;      // [rot / 2]
  const float* q_norm_w;      // optional [D]
  const float* k_norm_w;      // optional [D]
  int ld_qkv, rot, interleaved;
  float attn_factor, norm_eps, norm_w_off;
  // splits > 1: 1 = the `splits` CTAs of a (sequence, kv head) form a thread-block cluster and combine their partial
  // results through distributed shared memory (no global scratch, no arrival tickets); 0 = scratch + last-arriver.
  int cluster_reduce;
};
constexpr int kMaxFusedNew = 8;       // new tokens per sequence the fused (RoPE + append) decode path handles
constexpr int kMaxClusterSplits = 8;  // portable cluster size

__device__ __forceinline__ float ld_dsmem_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// One head row of the projection output: optional RMSNorm over D (result rounded to bf16 like a module boundary),
// rotation of the first `rot` dims by the token's position. Executed by one warp; lane l owns the pairs l, l + 32, ...
// `store(i0, a, i1, b)` receives the finished element pairs.
template <int D, typename Store>
__device__ __forceinline__ void rope_head_row(const AttnParams& p, const __nv_bfloat16* src, const float* nw, int pos,
                                              int lane, Store store) {
  constexpr int PER = D / 64;  // pairs per lane
  const int rh = p.rot >> 1;
  float a[PER], b[PER];
  int i0[PER], i1[PER];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    if (i < rh) {
      i0[j] = p.interleaved ? 2 * i : i;
      i1[j] = p.interleaved ? 2 * i + 1 : i + rh;
    } else {  // pass-through tail beyond the rotary dims
      i0[j] = p.rot + 2 * (i - rh);
      i1[j] = i0[j] + 1;
    }
    a[j] = __bfloat162float(src[i0[j]]);
    b[j] = __bfloat162float(src[i1[j]]);
    ss += a[j] * a[j] + b[j] * b[j];
  }
  if (nw != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / static_cast<float>(D) + p.norm_eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      a[j] = __bfloat162float(__float2bfloat16(a[j] * inv * (nw[i0[j]] + p.norm_w_off)));
      b[j] = __bfloat162float(__float2bfloat16(b[j] * inv * (nw[i1[j]] + p.norm_w_off)));
    }
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    if (i < rh) {
      float sn, cs;
      sincosf(static_cast<float>(pos) * p.inv_freq[i], &sn, &cs);
      sn *= p.attn_factor;
      cs *= p.attn_factor;
      const float ra = a[j] * cs - b[j] * sn;
      const float rb = b[j] * cs + a[j] * sn;
      a[j] = ra;
      b[j] = rb;
    }
    store(i0[j], a[j], i1[j], b[j]);
  }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `c` of row `r` in a [rows][D] bf16 tile with XOR swizzle.
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return static_cast<uint32_t>(r * (D * 2) + (((c & ~7) | ((c ^ r) & 7)) << 4));
}

// ============================================================================ prefill
// grid (q_tiles, n_q_heads, B), 128 threads; each warp owns 16 query tokens of one head.
template <int D>
__global__ void __launch_bounds__(128) attn_prefill_kernel(AttnParams p) {
  constexpr int CH = D / 8;       // 16-byte chunks per row
  constexpr int KS = D / 16;      // k-steps over head_dim
  constexpr int BM = 64, BN = 64;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + BM * D * 2;            // [2][BN][D]
  uint8_t* v_s = k_s + 2 * BN * D * 2;        // [2][BN][D]

  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  if (qt * BM >= q_len) return;
  const int kv_len = p.seq_lens[b];
  const int q_pos0 = kv_len - q_len;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int kvh = h / group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int* bt = p.block_table + static_cast<size_t>(b) * p.max_pages;

  // ---- Q tile
  for (int i = threadIdx.x; i < BM * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    const int tok = qt * BM + r;
    const bool ok = tok < q_len;
    const __nv_bfloat16* src = p.q + (static_cast<size_t>(q_begin + (ok ? tok : 0)) * p.n_q_heads + h) * D + c * 8;
    cp_async16(q_s + swz<D>(r, c), src, ok ? 16 : 0);
  }
  cp_async_commit();

  const int last_q_pos = q_pos0 + min(q_len, qt * BM + BM) - 1;
  const int first_q_pos = q_pos0 + qt * BM;
  int kv_hi = min(kv_len, last_q_pos + 1);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, first_q_pos - p.window + 1);
  const int chunk_lo = kv_lo / BN;
  const int chunk_hi = (kv_hi + BN - 1) / BN;

  auto load_chunk = [&](int chunk, int buf) {
    uint8_t* kd = k_s + buf * BN * D * 2;
    uint8_t* vd = v_s + buf * BN * D * 2;
    for (int i = threadIdx.x; i < BN * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      const int tok = chunk * BN + r;
      const bool ok = tok < kv_len;
      size_t off = 0;
      if (ok) {
        const int page = bt[tok / kPage];
        off = ((static_cast<size_t>(page) * p.n_kv_heads + kvh) * kPage + (tok % kPage)) * D + c * 8;
      }
      cp_async16(kd + swz<D>(r, c), p.k_cache + off, ok ? 16 : 0);
      cp_async16(vd + swz<D>(r, c), p.v_cache + off, ok ? 16 : 0);
    }
  };

  load_chunk(chunk_lo, 0);
  cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  if (p.sinks != nullptr) {
    // A sink is a virtual key with logit sinks[h] and zero value: it only enters the normaliser.
    // (l_run holds per-lane partial sums that are added across the quad at the end, so the
    // sink's unit mass goes to one lane of each quad only.)
    m_run[0] = m_run[1] = p.sinks[h] * 1.4426950408889634f;
    l_run[0] = l_run[1] = (tig == 0) ? 1.f : 0.f;
  }
  const int row_tok0 = qt * BM + warp * 16 + g;  // token index (within the sequence's new tokens)
  const int qpos0 = q_pos0 + row_tok0, qpos1 = qpos0 + 8;
  const uint32_t q_base = smem_u32(q_s);

  for (int chunk = chunk_lo; chunk < chunk_hi; ++chunk) {
    const int buf = (chunk - chunk_lo) & 1;
    if (chunk + 1 < chunk_hi) load_chunk(chunk + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const uint32_t k_base = smem_u32(k_s + buf * BN * D * 2);
    const uint32_t v_base = smem_u32(v_s + buf * BN * D * 2);
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_base + swz<D>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
#pragma unroll
      for (int nt = 0; nt < BN / 8; nt += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(k_base + swz<D>(nt * 8 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma16816(s[nt], a0, a1, a2, a3, b0, b1);
        mma16816(s[nt + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- mask + online softmax
    const int kv0 = chunk * BN;
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = kv0 + nt * 8 + tig * 2 + (e & 1);
        const int qp = (e < 2) ? qpos0 : qpos1;
        bool ok = (j <= qp) && (j < kv_len);
        if (p.window > 0) ok = ok && (j > qp - p.window);
        const float v = ok ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      msafe[r] = (mx[r] == -INFINITY) ? 0.f : mx[r];
      corr[r] = exp2f(m_run[r] - msafe[r]);  // m_run = -inf -> 0
      m_run[r] = mx[r];
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[nt][e] - msafe[e >> 1]);
        s[nt][e] = pv;
        ls[e >> 1] += pv;
      }
    }
    l_run[0] += ls[0];
    l_run[1] += ls[1];
    // ---- O += P V
#pragma unroll
    for (int kt = 0; kt < BN / 16; ++kt) {
      const uint32_t a0 = pack_bf16x2(s[2 * kt][0], s[2 * kt][1]);
      const uint32_t a1 = pack_bf16x2(s[2 * kt][2], s[2 * kt][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kt + 1][0], s[2 * kt + 1][1]);
      const uint32_t a3 = pack_bf16x2(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
      for (int dn = 0; dn < D / 8; dn += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_base + swz<D>(kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dn + (lane >> 4)), b0, b1, b2, b3);
        mma16816(o[dn], a0, a1, a2, a3, b0, b1);
        mma16816(o[dn + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- finalize: row sums live in the 4 lanes of a quad
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int tok = row_tok0 + r * 8;
    if (tok < q_len) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<size_t>(q_begin + tok) * p.n_q_heads + h) * D;
#pragma unroll
      for (int dn = 0; dn < D / 8; ++dn) {
        *reinterpret_cast<uint32_t*>(dst + dn * 8 + tig * 2) =
            pack_bf16x2(o[dn][2 * r] * inv, o[dn][2 * r + 1] * inv);
      }
    }
  }
}

// ============================================================================ decode (split-KV)
// grid (splits, n_kv_heads, B). The MT*16 MMA rows hold (query token t, head-in-group g) pairs,
// row = (t - t0) * group + g. Each of the 4 warps streams every 4th page through its own 3-stage
// cp.async ring and keeps private (m, l, O); the warps are merged through shared memory at the end.
template <int D, int MT>
__global__ void __launch_bounds__(128) attn_decode_kernel(AttnParams p) {
  constexpr int CH = D / 8;
  constexpr int KS = D / 16;
  constexpr int NSTAGE = 3;
  constexpr int ROWS = 16 * MT;
  constexpr int PAGE_BYTES = kPage * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_s = smem;                   // [ROWS][D] bf16
  uint8_t* newkv_s = smem + ROWS * D * 2;                    // [kMaxFusedNew][K row, V row] bf16 (fused path)
  uint8_t* ring = newkv_s + kMaxFusedNew * 2 * D * 2;        // [4 warps][NSTAGE][K page, V page]

  __shared__ int s_last;
  pdl_launch_early();
  trace_mark(kTraceAttnDecode, kTraceStart);
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int rows = p.t_count * group;
  const int* bt = p.block_table + static_cast<size_t>(b) * p.max_pages;
  pdl_wait();
  trace_mark(kTraceAttnDecode, kTraceAfterWait);
  pdl_launch_dependents();
  const int kv_len = p.seq_lens[b];
  const int npages = (kv_len + kPage - 1) / kPage;
  int pps = (npages + p.splits - 1) / p.splits;
  pps = (pps + 3) & ~3;
  const int page0 = split * pps;
  const int page1 = min(npages, page0 + pps);

  const bool fused = p.qkv != nullptr;
  // The launch that handles the first query tokens also appends the new K / V rows. A page fetched from the cache may
  // then still hold the old bytes of a new row, so the rows are patched into the shared-memory copy of their page
  // (from `newkv_s`) after it has landed: no fence and no ordering between the append and the page fetches is needed.
  const bool appending = fused && p.t0 == 0;
  const int new_pos0 = kv_len - p.q_per_seq;
  const int first_new_page = appending ? new_pos0 / kPage : 0x7fffffff;
  if (!fused) {
    for (int i = threadIdx.x; i < ROWS * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      const bool ok = r < rows;
      const int t = p.t0 + (ok ? r / group : 0), hg = ok ? r % group : 0;
      const __nv_bfloat16* src =
          p.q + (static_cast<size_t>(b * p.q_per_seq + t) * p.n_q_heads + kvh * group + hg) * D + c * 8;
      cp_async16(q_s + swz<D>(r, c), src, ok ? 16 : 0);
    }
  }
  cp_async_commit();

  uint8_t* my_ring = ring + warp * NSTAGE * 2 * PAGE_BYTES;
  auto load_page = [&](int pg, int stage) {
    if (pg < page1) {
      const int phys = bt[pg];
      const __nv_bfloat16* ksrc = p.k_cache + (static_cast<size_t>(phys) * p.n_kv_heads + kvh) * kPage * D;
      const __nv_bfloat16* vsrc = p.v_cache + (static_cast<size_t>(phys) * p.n_kv_heads + kvh) * kPage * D;
      uint8_t* kd = my_ring + stage * 2 * PAGE_BYTES;
      uint8_t* vd = kd + PAGE_BYTES;
      for (int i = lane; i < kPage * CH; i += 32) {
        const int r = i / CH, c = i % CH;
        cp_async16(kd + swz<D>(r, c), ksrc + r * D + c * 8, 16);
        cp_async16(vd + swz<D>(r, c), vsrc + r * D + c * 8, 16);
      }
    }
  };

  float o[MT][D / 8][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
  }

  const int first = page0 + warp;
  load_page(first, 0);
  cp_async_commit();
  load_page(first + 4, 1);
  cp_async_commit();
  if (fused) {
    // ---- q rows: norm + RoPE straight into the swizzled tile (rows beyond `rows` are zero)
    for (int r = warp; r < ROWS; r += 4) {
      auto put = [&](int i0, float a, int i1, float bb) {
        *reinterpret_cast<__nv_bfloat16*>(q_s + swz<D>(r, i0 >> 3) + (i0 & 7) * 2) = __float2bfloat16(a);
        *reinterpret_cast<__nv_bfloat16*>(q_s + swz<D>(r, i1 >> 3) + (i1 & 7) * 2) = __float2bfloat16(bb);
      };
      if (r < rows) {
        const int t = p.t0 + r / group, hg = r % group;
        const size_t m = static_cast<size_t>(b) * p.q_per_seq + t;
        rope_head_row<D>(p, p.qkv + m * p.ld_qkv + static_cast<size_t>(kvh * group + hg) * D, p.q_norm_w, p.positions[m],
                         lane, put);
      } else {
        for (int i = lane; i < D / 2; i += 32) put(2 * i, 0.f, 2 * i + 1, 0.f);
      }
    }
    // ---- new K / V rows whose page lies in this CTA's range: norm + RoPE on K; both go to the cache (for later
    // steps) and to `newkv_s` (for this step's own use)
    if (appending) {
      for (int t = warp; t < p.q_per_seq; t += 4) {
        const int pg = (new_pos0 + t) / kPage;
        const size_t m = static_cast<size_t>(b) * p.q_per_seq + t;
        const long long slot = p.slots[m];
        if (pg < page0 || pg >= page1 || slot < 0) continue;  // warp-uniform
        const size_t dst = ((static_cast<size_t>(slot >> 4) * p.n_kv_heads + kvh) * kPage + static_cast<size_t>(slot & 15)) * D;
        __nv_bfloat16* kd = const_cast<__nv_bfloat16*>(p.k_cache) + dst;
        __nv_bfloat16* vd = const_cast<__nv_bfloat16*>(p.v_cache) + dst;
        __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(newkv_s) + static_cast<size_t>(t) * 2 * D;
        const __nv_bfloat16* krow = p.qkv + m * p.ld_qkv + static_cast<size_t>(p.n_q_heads + kvh) * D;
        const __nv_bfloat16* vrow = p.qkv + m * p.ld_qkv + static_cast<size_t>(p.n_q_heads + p.n_kv_heads + kvh) * D;
        rope_head_row<D>(p, krow, p.k_norm_w, p.positions[m], lane, [&](int i0, float a, int i1, float bb) {
          const __nv_bfloat16 ha = __float2bfloat16(a), hb = __float2bfloat16(bb);
          kd[i0] = ha;
          kd[i1] = hb;
          ks[i0] = ha;
          ks[i1] = hb;
        });
        for (int i = lane; i < D / 2; i += 32) {
          const uint32_t vv = reinterpret_cast<const uint32_t*>(vrow)[i];
          reinterpret_cast<uint32_t*>(vd)[i] = vv;
          reinterpret_cast<uint32_t*>(ks + D)[i] = vv;
        }
      }
    }
  }
  cp_async_wait<2>();  // the Q tile (the oldest group)
  __syncthreads();     // Q tile and new rows visible to every warp

  const uint32_t q_base = smem_u32(q_s);
  int it = 0;
  for (int pg = first; pg < page1; pg += 4, ++it) {
    load_page(pg + 8, (it + 2) % NSTAGE);
    cp_async_commit();
    cp_async_wait<2>();
    __syncwarp();
    if (pg >= first_new_page) {
      // this page holds rows appended in this step: overwrite them in the landed copy (16-byte chunks, lanes 0-15 the
      // K row, 16-31 the V row; D / 8 chunks per row)
      uint8_t* kst = my_ring + (it % NSTAGE) * 2 * PAGE_BYTES;
      for (int t = 0; t < p.q_per_seq; ++t) {
        const int pos = new_pos0 + t;
        if (pos / kPage != pg || p.slots[static_cast<size_t>(b) * p.q_per_seq + t] < 0) continue;  // warp-uniform
        const uint4* src = reinterpret_cast<const uint4*>(newkv_s + static_cast<size_t>(t) * 2 * D * 2);
        for (int i = lane; i < 2 * CH; i += 32) {
          const int which = i / CH, c = i % CH;
          *reinterpret_cast<uint4*>(kst + which * PAGE_BYTES + swz<D>(pos & (kPage - 1), c)) = src[i];
        }
      }
      __syncwarp();
    }
    const uint32_t k_base = smem_u32(my_ring + (it % NSTAGE) * 2 * PAGE_BYTES);
    const uint32_t v_base = k_base + PAGE_BYTES;

    float s[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(k_base + swz<D>((lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4(q_base + swz<D>(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
        mma16816(s[mt][0], a0, a1, a2, a3, b0, b1);
        mma16816(s[mt][1], a0, a1, a2, a3, b2, b3);
      }
    }
    const int kv0 = pg * kPage;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float mx[2] = {m_run[mt][0], m_run[mt][1]};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = kv0 + nt * 8 + tig * 2 + (e & 1);
          const int r = mt * 16 + g + (e >> 1) * 8;
          const int qp = kv_len - p.q_per_seq + p.t0 + r / group;
          bool ok = (r < rows) && (j <= qp) && (j < kv_len);
          if (p.window > 0) ok = ok && (j > qp - p.window);
          const float v = ok ? s[mt][nt][e] * p.scale_log2 : -INFINITY;
          s[mt][nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], msafe[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        msafe[r] = (mx[r] == -INFINITY) ? 0.f : mx[r];
        corr[r] = exp2f(m_run[mt][r] - msafe[r]);
        m_run[mt][r] = mx[r];
        l_run[mt][r] *= corr[r];
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[mt][i][0] *= corr[0];
        o[mt][i][1] *= corr[0];
        o[mt][i][2] *= corr[1];
        o[mt][i][3] *= corr[1];
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[mt][nt][e] - msafe[e >> 1]);
          s[mt][nt][e] = pv;
          l_run[mt][e >> 1] += pv;
        }
    }
#pragma unroll
    for (int dn = 0; dn < D / 8; dn += 2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(v_base + swz<D>((lane & 7) + ((lane >> 3) & 1) * 8, dn + (lane >> 4)), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint32_t a0 = pack_bf16x2(s[mt][0][0], s[mt][0][1]);
        const uint32_t a1 = pack_bf16x2(s[mt][0][2], s[mt][0][3]);
        const uint32_t a2 = pack_bf16x2(s[mt][1][0], s[mt][1][1]);
        const uint32_t a3 = pack_bf16x2(s[mt][1][2], s[mt][1][3]);
        mma16816(o[mt][dn], a0, a1, a2, a3, b0, b1);
        mma16816(o[mt][dn + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: reuse it for the merge

  // ---- merge the 4 warps: mo[w][row][D] fp32, mm/ml[w][row]; then this CTA's merged partial (cluster mode)
  float* mo = reinterpret_cast<float*>(ring);
  float* mm = mo + 4 * ROWS * D;
  float* ml = mm + 4 * ROWS;
  float* part_s = ml + 4 * ROWS;   // [ROWS][D]
  float* part_m = part_s + ROWS * D;
  float* part_l = part_m + ROWS;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_run[mt][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int row = mt * 16 + g + r * 8;
      if (tig == 0) {
        mm[warp * ROWS + row] = m_run[mt][r];
        ml[warp * ROWS + row] = l;
      }
#pragma unroll
      for (int dn = 0; dn < D / 8; ++dn) {
        float2 v = make_float2(o[mt][dn][2 * r], o[mt][dn][2 * r + 1]);
        *reinterpret_cast<float2*>(&mo[(warp * ROWS + row) * D + dn * 8 + tig * 2]) = v;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rows * D; i += 128) {
    const int row = i / D, d = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * ROWS + row]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float e = exp2f(mm[w * ROWS + row] - Ms);
      L += ml[w * ROWS + row] * e;
      acc += mo[(w * ROWS + row) * D + d] * e;
    }
    const int t = p.t0 + row / group, hg = row % group;
    const int head = kvh * group + hg;
    const size_t qrow = static_cast<size_t>(b * p.q_per_seq + t) * p.n_q_heads + head;
    if (p.splits == 1) {
      float Lf = L;
      if (p.sinks != nullptr) Lf += exp2f(p.sinks[head] * 1.4426950408889634f - Ms);
      p.out[qrow * D + d] = __float2bfloat16(Lf > 0.f ? acc / Lf : 0.f);
    } else if (p.cluster_reduce) {
      part_s[row * D + d] = acc;
      if (d == 0) {
        part_m[row] = M;
        part_l[row] = L;
      }
    } else {
      p.part_o[(qrow * p.splits + split) * D + d] = acc;
      if (d == 0) {
        p.part_ml[(qrow * p.splits + split) * 2 + 0] = M;
        p.part_ml[(qrow * p.splits + split) * 2 + 1] = L;
      }
    }
  }
  if (p.splits > 1 && p.cluster_reduce) {
    // The splits of this (sequence, kv head) are one cluster: every CTA combines a share of the rows, reading the
    // partials of all splits out of their shared memory.
    cluster_arrive_release();
    cluster_wait_acquire();
    const uint32_t a_s = smem_u32(part_s), a_m = smem_u32(part_m), a_l = smem_u32(part_l);
    for (int i = threadIdx.x + split * 128; i < rows * D; i += 128 * p.splits) {  // row-major: a warp stays in one row
      const int row = i / D, d = i % D;
      float M = -INFINITY;
      float ms[kMaxClusterSplits], pv[kMaxClusterSplits], ls[kMaxClusterSplits];
#pragma unroll
      for (int sp = 0; sp < kMaxClusterSplits; ++sp) {
        if (sp < p.splits) {
          ms[sp] = ld_dsmem_f32(mapa_shared(a_m + row * 4, sp));
          ls[sp] = ld_dsmem_f32(mapa_shared(a_l + row * 4, sp));
          pv[sp] = ld_dsmem_f32(mapa_shared(a_s + (row * D + d) * 4, sp));
          M = fmaxf(M, ms[sp]);
        }
      }
      const float Ms = (M == -INFINITY) ? 0.f : M;
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int sp = 0; sp < kMaxClusterSplits; ++sp) {
        if (sp < p.splits) {
          const float e = exp2f(ms[sp] - Ms);
          L += ls[sp] * e;
          acc += pv[sp] * e;
        }
      }
      const int t = p.t0 + row / group, hg = row % group;
      const int head = kvh * group + hg;
      if (p.sinks != nullptr) L += exp2f(p.sinks[head] * 1.4426950408889634f - Ms);
      p.out[(static_cast<size_t>(b * p.q_per_seq + t) * p.n_q_heads + head) * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
    }
    cluster_arrive_release();  // done reading the peers' shared memory
    cluster_wait_acquire();    // and nobody reads this CTA's any more
  } else if (p.splits > 1) {
    // The last split to arrive for this (sequence, kv head) combines all partials: no second launch.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int ticket = atomicAdd(&p.counters[b * gridDim.y + kvh], 1);
      s_last = (ticket == p.splits - 1) ? 1 : 0;
      if (s_last) p.counters[b * gridDim.y + kvh] = 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      // per (row, split) weights first (rows * splits <= 32 * 64 values, in the free merge area), then the
      // D-wide accumulation with independent loads
      float* wgt = mo;                       // [rows][splits]  exp2(m_s - M)
      float* linv = mo + ROWS * 64;          // [rows]          1 / L
      __syncthreads();
      for (int row = threadIdx.x; row < rows; row += 128) {
        const int t = p.t0 + row / group, hg = row % group;
        const int head = kvh * group + hg;
        const size_t qrow = static_cast<size_t>(b * p.q_per_seq + t) * p.n_q_heads + head;
        float M = -INFINITY;
        for (int sp = 0; sp < p.splits; ++sp) M = fmaxf(M, __ldcg(&p.part_ml[(qrow * p.splits + sp) * 2]));
        const float Ms = (M == -INFINITY) ? 0.f : M;
        float L = 0.f;
        for (int sp = 0; sp < p.splits; ++sp) {
          const size_t idx = qrow * p.splits + sp;
          const float e = exp2f(__ldcg(&p.part_ml[idx * 2]) - Ms);
          wgt[row * 64 + sp] = e;
          L += __ldcg(&p.part_ml[idx * 2 + 1]) * e;
        }
        if (p.sinks != nullptr) L += exp2f(p.sinks[head] * 1.4426950408889634f - Ms);
        linv[row] = L > 0.f ? 1.f / L : 0.f;
      }
      __syncthreads();
      for (int i = threadIdx.x; i < rows * D; i += 128) {
        const int row = i / D, d = i % D;
        const int t = p.t0 + row / group, hg = row % group;
        const size_t qrow = static_cast<size_t>(b * p.q_per_seq + t) * p.n_q_heads + kvh * group + hg;
        const float* po = p.part_o + qrow * p.splits * D + d;
        float acc = 0.f;
        int sp = 0;
        for (; sp + 4 <= p.splits; sp += 4) {
          const float a0 = __ldcg(po + (sp + 0) * D), a1 = __ldcg(po + (sp + 1) * D);
          const float a2 = __ldcg(po + (sp + 2) * D), a3 = __ldcg(po + (sp + 3) * D);
          acc += a0 * wgt[row * 64 + sp] + a1 * wgt[row * 64 + sp + 1] + a2 * wgt[row * 64 + sp + 2] +
                 a3 * wgt[row * 64 + sp + 3];
        }
        for (; sp < p.splits; ++sp) acc += __ldcg(po + sp * D) * wgt[row * 64 + sp];
        p.out[qrow * D + d] = __float2bfloat16(acc * linv[row]);
      }
    }
  }
  trace_mark(kTraceAttnDecode, kTraceEnd);
}

template <int D>
static size_t prefill_smem() {
  return 64 * D * 2 + 4 * 64 * D * 2;
}
template <int D, int MT>
static size_t decode_smem() {
  const size_t ring = 4 * 3 * 2 * kPage * D * 2;
  const size_t merge = (4 * 16 * MT * D + 2 * 4 * 16 * MT + 16 * MT * D + 2 * 16 * MT) * sizeof(float);
  return 16 * MT * D * 2 + kMaxFusedNew * 2 * D * 2 + (ring > merge ? ring : merge);
}

}  // namespace eredu

using namespace eredu;

// Bytes of fp32 scratch (part_o, part_ml) a decode launch with `splits` > 1 needs.
EREDU_TRACE_INSTALLER(attention)

// cudaFuncSetAttribute is a per-device setting: one "configured" flag per device of the process.
constexpr int kMaxDevices = 64;
template <typename K>
static bool configure_once(bool (&done)[kMaxDevices], K kernel, size_t smem) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
  if (!done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return false;
    done[dev] = true;
  }
  return true;
}

extern "C" void eredu_attn_decode_scratch_elems(int batch, int q_per_seq, int n_q_heads, int head_dim, int splits,
                                                long long* part_o_elems, long long* part_ml_elems) {
  const long long rows = static_cast<long long>(batch) * q_per_seq * n_q_heads;
  *part_o_elems = rows * splits * head_dim;
  *part_ml_elems = rows * splits * 2;
}

extern "C" int eredu_attn_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  const int* block_table, const int* seq_lens, const int* cu_q, const float* sinks,
                                  int batch, int max_q_len, int max_pages, int n_q_heads, int n_kv_heads,
                                  int head_dim, int window, float scale, cudaStream_t stream) {
  AttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
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
  dim3 grid((max_q_len + 63) / 64, n_q_heads, batch);
  cudaError_t e;
  if (head_dim == 128) {
    static bool cfg[kMaxDevices] = {};
    if (!configure_once(cfg, attn_prefill_kernel<128>, prefill_smem<128>())) return -1;
    e = launch_pdl(attn_prefill_kernel<128>, grid, dim3(128), prefill_smem<128>(), stream, p);
  } else if (head_dim == 64) {
    static bool cfg[kMaxDevices] = {};
    if (!configure_once(cfg, attn_prefill_kernel<64>, prefill_smem<64>())) return -1;
    e = launch_pdl(attn_prefill_kernel<64>, grid, dim3(128), prefill_smem<64>(), stream, p);
  } else {
    return -1;
  }
  eredu_count_launches(1);
  return static_cast<int>(e);
}

template <int D, int MT>
static cudaError_t launch_decode(const AttnParams& p, dim3 grid, cudaStream_t stream) {
  static bool cfg[kMaxDevices] = {};
  if (!configure_once(cfg, attn_decode_kernel<D, MT>, decode_smem<D, MT>())) return cudaErrorInvalidValue;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = dim3(128);
  lc.dynamicSmemBytes = decode_smem<D, MT>();
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (pdl_enabled()) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (p.cluster_reduce) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = grid.x;  // the splits of one (sequence, kv head)
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  lc.attrs = attr;
  lc.numAttrs = nattr;
  const cudaError_t e = cudaLaunchKernelEx(&lc, attn_decode_kernel<D, MT>, p);
  eredu_count_launches(1);
  return e;
}

// q: [batch * q_per_seq, n_q_heads, D]; every sequence contributes exactly q_per_seq query tokens whose
// positions are the last q_per_seq positions of its kv (causal among themselves). part_o / part_ml are
// caller-provided fp32 scratch (see eredu_attn_decode_scratch_elems) and `counters` a zeroed int32
// [batch * n_kv_heads] array (left zeroed again on return); all unused when splits == 1.
static int launch_decode_all(AttnParams p, int batch, int q_per_seq, int n_q_heads, int n_kv_heads, int head_dim,
                             cudaStream_t stream, bool force_scratch = false) {
  if (n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads != 0) return -1;
  const int group = n_q_heads / n_kv_heads;
  if (group > 32 || (head_dim != 128 && head_dim != 64)) return -1;
  const int t_per = group > 16 ? 1 : (32 / group < q_per_seq ? 32 / group : q_per_seq);
  if (p.qkv != nullptr && q_per_seq > kMaxFusedNew) return -1;
  // Few splits: a cluster per (sequence, kv head) combines the partials in shared memory. More splits than a portable
  // cluster holds (or a caller that asks for it by passing scratch and force_scratch): global scratch + last arriver.
  p.cluster_reduce = (p.splits > 1 && p.splits <= kMaxClusterSplits && !force_scratch) ? 1 : 0;
  if (p.splits > 1 && !p.cluster_reduce && (p.part_o == nullptr || p.part_ml == nullptr || p.counters == nullptr)) return -1;
  dim3 grid(p.splits, n_kv_heads, batch);
  for (int t0 = 0; t0 < q_per_seq; t0 += t_per) {
    p.t0 = t0;
    p.t_count = (q_per_seq - t0 < t_per) ? q_per_seq - t0 : t_per;
    const int rows = p.t_count * group;
    cudaError_t e;
    if (head_dim == 128) e = rows <= 16 ? launch_decode<128, 1>(p, grid, stream) : launch_decode<128, 2>(p, grid, stream);
    else e = rows <= 16 ? launch_decode<64, 1>(p, grid, stream) : launch_decode<64, 2>(p, grid, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return 0;
}

static int attn_decode_impl(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                            const int* seq_lens, const float* sinks, float* part_o, float* part_ml, int* counters,
                            int batch, int q_per_seq, int max_pages, int n_q_heads, int n_kv_heads, int head_dim,
                            int splits, int window, float scale, cudaStream_t stream, bool force_scratch) {
  AttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.sinks = sinks;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.counters = counters;
  p.max_pages = max_pages;
  p.n_q_heads = n_q_heads;
  p.n_kv_heads = n_kv_heads;
  p.q_per_seq = q_per_seq;
  p.splits = splits < 1 ? 1 : (splits > 64 ? 64 : splits);
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  return launch_decode_all(p, batch, q_per_seq, n_q_heads, n_kv_heads, head_dim, stream, force_scratch);
}

// Up to 8 splits combine inside a thread-block cluster and ignore the scratch arguments (they may be null); more
// splits need them.
extern "C" int eredu_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                 const int* block_table, const int* seq_lens, const float* sinks, float* part_o,
                                 float* part_ml, int* counters, int batch, int q_per_seq, int max_pages, int n_q_heads,
                                 int n_kv_heads, int head_dim, int splits, int window, float scale,
                                 cudaStream_t stream) {
  return attn_decode_impl(q, k_cache, v_cache, out, block_table, seq_lens, sinks, part_o, part_ml, counters, batch,
                          q_per_seq, max_pages, n_q_heads, n_kv_heads, head_dim, splits, window, scale, stream, false);
}

// Decode attention that starts from the projection output: qkv [batch * q_per_seq, ld_qkv] = [q heads | k heads |
// v heads] x D as the qkv GEMM wrote it. The kernel normalises (optional per-head RMSNorm weights) and rotates q and
// the new k rows by `positions`, appends the new k / v rows at `slots` (page * 16 + offset; negative: not stored)
// and attends - the RoPE + KV-append launch of the unfused path disappears. Every new row is appended by the one CTA
// whose page range contains it, before that CTA fetches the page. Other arguments as eredu_attn_decode.
extern "C" int eredu_attn_decode_rope(const void* qkv, int ld_qkv, void* k_cache, void* v_cache, void* out,
                                      const int* block_table, const int* seq_lens, const float* sinks, float* part_o,
                                      float* part_ml, int* counters, const int* positions, const long long* slots,
                                      const float* inv_freq, const float* q_norm_w, const float* k_norm_w, int batch,
                                      int q_per_seq, int max_pages, int n_q_heads, int n_kv_heads, int head_dim, int rot,
                                      int interleaved, int splits, int window, float scale, float attn_factor,
                                      float norm_eps, float norm_w_off, cudaStream_t stream) {
  if (qkv == nullptr || positions == nullptr || slots == nullptr || inv_freq == nullptr) return -1;
  if (rot <= 0 || rot > head_dim || rot % 2 != 0 || ld_qkv % 2 != 0) return -1;
  AttnParams p = {};
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.ld_qkv = ld_qkv;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.sinks = sinks;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.counters = counters;
  p.positions = positions;
  p.slots = slots;
  p.inv_freq = inv_freq;
  p.q_norm_w = q_norm_w;
  p.k_norm_w = k_norm_w;
  p.rot = rot;
  p.interleaved = interleaved;
  p.attn_factor = attn_factor;
  p.norm_eps = norm_eps;
  p.norm_w_off = norm_w_off;
  p.max_pages = max_pages;
  p.n_q_heads = n_q_heads;
  p.n_kv_heads = n_kv_heads;
  p.q_per_seq = q_per_seq;
  p.splits = splits < 1 ? 1 : (splits > 64 ? 64 : splits);
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  return launch_decode_all(p, batch, q_per_seq, n_q_heads, n_kv_heads, head_dim, stream);
}

// ---------------------------------------------------------------------------------------------- no-allocation variant
#include "attention_noalloc.h"

namespace {
constexpr size_t kNoAllocCounterBytes = EREDU_NOALLOC_MAX_GROUPS * sizeof(int);
constexpr size_t kNoAllocMlBytes = static_cast<size_t>(EREDU_NOALLOC_MAX_ROW_SPLITS) * 2 * sizeof(float);
constexpr size_t kNoAllocOBytes = static_cast<size_t>(EREDU_NOALLOC_MAX_ROW_SPLITS) * 128 * sizeof(float);
}  // namespace

// Scratch of eredu_attn_decode_static: [arrival counters | (max, sum) pairs | partial outputs].
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocCounterBytes + kNoAllocMlBytes + kNoAllocOBytes];

extern "C" int eredu_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* block_table, const int* seq_lens, const float* sinks, int batch,
                                        int q_per_seq, int max_pages, int n_q_heads, int n_kv_heads, int head_dim,
                                        int splits, int window, float scale, cudaStream_t stream) {
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  if (head_dim != 64 && head_dim != 128) return -1;
  if (batch <= 0 || q_per_seq <= 0 || n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads != 0) return -1;
  const long long row_splits = static_cast<long long>(batch) * q_per_seq * n_q_heads * splits;
  if (row_splits > EREDU_NOALLOC_MAX_ROW_SPLITS || static_cast<long long>(batch) * n_kv_heads > EREDU_NOALLOC_MAX_GROUPS)
    return -2;
  // The array's name is only a host-side handle: resolve its device address once per device.
  static unsigned char* base[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -1;
  if (base[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    base[dev] = static_cast<unsigned char*>(p);
  }
  int* counters = reinterpret_cast<int*>(base[dev]);
  float* part_ml = reinterpret_cast<float*>(base[dev] + kNoAllocCounterBytes);
  float* part_o = reinterpret_cast<float*>(base[dev] + kNoAllocCounterBytes + kNoAllocMlBytes);
  if (splits > 1) {
    e = cudaMemsetAsync(counters, 0, static_cast<size_t>(batch) * n_kv_heads * sizeof(int), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  // always the scratch form of the split reduction: that is the form whose scratch this entry point provides
  return attn_decode_impl(q, k_cache, v_cache, out, block_table, seq_lens, sinks, part_o, part_ml, counters, batch,
                          q_per_seq, max_pages, n_q_heads, n_kv_heads, head_dim, splits, window, scale, stream, true);
}
