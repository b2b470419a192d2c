// Fused sampler: token-filter mask -> repetition/frequency/presence penalties -> top-k -> top-p ->
// min-p -> temperature -> argmax | categorical, one launch per step, no host synchronisation, plus
// the speculative-decoding verify rule (accept with min(1, p_t/p_d), residual resample, bonus token).
//
// Semantics follow the reference sampler chain (eredu/src/backend/mlx/runtime/generation/
// sampler.rs:690-923): top-k keeps logits >= the k-th largest; top-p keeps the sorted prefix whose
// mass *before* each token is <= top_p, computed at temperature 1 on the top-k survivors; min-p keeps
// p >= min_p * p_max; temperature is applied last. The verify rule is the reference's
// (eredu/src/backend/mlx/speculative.rs:520-574) without its four host synchronisations per proposal.
//
// Randomness is position addressed: the uniform for (seed, stream, position, purpose) is a pure
// function (Philox4x32-10), so batching and scheduling never change committed tokens.
//
// One CTA (1024 threads) per logits row. The top-k/top-p path selects at most 1024 candidates with an
// exact 4-pass radix select (integer histograms: deterministic), sorts them in shared memory and
// scans them. With top-k disabled and top-p < 1 the candidate set is the 1024 largest logits with
// probabilities normalised over the full vocabulary. With both disabled the kernel samples the
// full (min-p filtered) vocabulary in index order.
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/trace.cuh"

namespace eredu {

struct SamplerRow {
  float temperature;
  float top_p;
  float min_p;
  float repeat_penalty;
  float frequency_penalty;
  float presence_penalty;
  int top_k;
  int repeat_last_n;   // < 0: whole history
  int hist_len;        // valid entries of this row's history
  int position;        // RNG position (index of the token being sampled)
  unsigned int seed_lo, seed_hi;
  unsigned int stream_id;
  int pad;
};

constexpr int kSampThreads = 1024;
constexpr int kCand = 1024;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
// Uniform in [0,1) for (seed, stream, position, purpose).
__device__ __forceinline__ float philox_uniform(uint32_t seed_lo, uint32_t seed_hi, uint32_t stream, uint32_t position,
                                                uint32_t purpose) {
  uint32_t c[4] = {position, stream, purpose, 0x45524544u};
  uint32_t k0 = seed_lo, k1 = seed_hi;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return static_cast<float>(c[0] >> 8) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ uint32_t f2key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(b);
}

struct BlockScratch {
  float fbuf[32];
  int ibuf[32];
  float fval;
  int ival;
};

__device__ __forceinline__ float block_sum(float v, BlockScratch& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.fbuf[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = s.fbuf[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) s.fval = t;
  }
  __syncthreads();
  return s.fval;
}

// Inclusive prefix sum over the 1024 threads (deterministic tree order).
__device__ __forceinline__ float block_scan_incl(float v, BlockScratch& s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) s.fbuf[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = s.fbuf[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += u;
    }
    s.fbuf[lane] = t;
  }
  __syncthreads();
  if (warp > 0) v += s.fbuf[warp - 1];
  return v;
}

// (max value, smallest index attaining it)
__device__ __forceinline__ void block_argmax(float& v, int& idx, BlockScratch& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { s.fbuf[threadIdx.x >> 5] = v; s.ibuf[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = s.fbuf[threadIdx.x];
    int ti = s.ibuf[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, t, o);
      const int oi = __shfl_xor_sync(0xffffffffu, ti, o);
      if (ov > t || (ov == t && oi < ti)) { t = ov; ti = oi; }
    }
    if (threadIdx.x == 0) { s.fval = t; s.ival = ti; }
  }
  __syncthreads();
  v = s.fval;
  idx = s.ival;
}

__device__ __forceinline__ int block_min_int(int v, BlockScratch& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.ibuf[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    int t = s.ibuf[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (threadIdx.x == 0) s.ival = t;
  }
  __syncthreads();
  return s.ival;
}

struct SamplerParams {
  float* logits;             // [rows, V] fp32, modified in place by penalties
  const uint32_t* allow;     // optional bitmask [rows or 1, ceil(V/32)]: bit set = token allowed
  int allow_stride;          // words between rows (0 = one mask for all rows)
  const SamplerRow* rows;    // [rows]
  const int* history;        // [rows, hist_stride] generated tokens (most recent last)
  int hist_stride;
  int* tokens;               // [rows] sampled ids
  float* probs;              // optional [rows, V]: final distribution (dense)
  int V;
};

__device__ __forceinline__ float load_logit(const SamplerParams& p, const float* row, const uint32_t* allow, int i) {
  float x = row[i];
  if (allow != nullptr && !((allow[i >> 5] >> (i & 31)) & 1u)) x = -INFINITY;
  return x;
}

__global__ void __launch_bounds__(kSampThreads) sampler_kernel(SamplerParams p) {
  __shared__ __align__(16) BlockScratch scr;
  __shared__ __align__(16) int hist[256];
  __shared__ __align__(16) uint32_t cand_key[kCand];
  __shared__ __align__(16) uint32_t cand_idx[kCand];
  __shared__ int sh_count;
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_krem;
  __shared__ int sh_pick;

  pdl_launch_early();
  trace_mark(kTraceSampler, kTraceStart);
  pdl_wait();
  trace_mark(kTraceSampler, kTraceAfterWait);
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int tid = threadIdx.x;
  SamplerRow cfg;
  {
    const int* src = reinterpret_cast<const int*>(p.rows + r);
    int* dst = reinterpret_cast<int*>(&cfg);
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(SamplerRow) / 4); ++i) dst[i] = src[i];
  }
  float* row = p.logits + static_cast<size_t>(r) * p.V;
  const uint32_t* allow = p.allow ? p.allow + static_cast<size_t>(r) * p.allow_stride : nullptr;
  float* prow = p.probs ? p.probs + static_cast<size_t>(r) * p.V : nullptr;
  const int V = p.V;

  // ---- 1. penalties, in place, once per distinct token of the window
  const bool pen = (cfg.repeat_penalty != 1.f || cfg.frequency_penalty != 0.f || cfg.presence_penalty != 0.f) &&
                   cfg.hist_len > 0 && p.history != nullptr;
  if (pen) {
    const int* h = p.history + static_cast<size_t>(r) * p.hist_stride;
    const int start = cfg.repeat_last_n < 0 ? 0 : max(0, cfg.hist_len - cfg.repeat_last_n);
    for (int j = start + tid; j < cfg.hist_len; j += kSampThreads) {
      const int tok = h[j];
      if (tok < 0 || tok >= V) continue;
      int count = 0;
      bool first = true;
      for (int q = start; q < cfg.hist_len; ++q) {
        if (h[q] == tok) {
          ++count;
          if (q < j) first = false;
        }
      }
      if (first) {
        float x = row[tok];
        if (cfg.repeat_penalty != 1.f) x = x > 0.f ? x / cfg.repeat_penalty : x * cfg.repeat_penalty;
        x -= cfg.frequency_penalty * static_cast<float>(count) + cfg.presence_penalty;
        row[tok] = x;
      }
    }
    __syncthreads();
  }

  // ---- 2. max / argmax (the greedy answer; also the softmax shift)
  float vmax = -INFINITY;
  int imax = 0x7fffffff;
  for (int i = tid; i < V; i += kSampThreads) {
    const float x = load_logit(p, row, allow, i);
    if (x > vmax) { vmax = x; imax = i; }
  }
  block_argmax(vmax, imax, scr);
  if (imax == 0x7fffffff) imax = 0;

  if (cfg.temperature == 0.f) {
    if (tid == 0) p.tokens[r] = imax;
    if (prow != nullptr) {
      for (int i = tid; i < V; i += kSampThreads) prow[i] = (i == imax) ? 1.f : 0.f;
    }
    return;
  }

  const float inv_t = 1.f / cfg.temperature;
  const bool use_topk = cfg.top_k > 0 && cfg.top_k < V;
  const bool use_topp = cfg.top_p < 1.f;
  const float minp_thr = cfg.min_p > 0.f ? vmax + __logf(cfg.min_p) : -INFINITY;
  const float u = philox_uniform(cfg.seed_lo, cfg.seed_hi, cfg.stream_id, static_cast<uint32_t>(cfg.position), 0u);

  if (!use_topk && !use_topp) {
    // ---- dense path: categorical over {x >= min-p threshold} in index order
    const int seg = (V + kSampThreads - 1) / kSampThreads;
    const int lo = tid * seg, hi = min(V, lo + seg);
    float local = 0.f;
    for (int i = lo; i < hi; ++i) {
      const float x = load_logit(p, row, allow, i);
      if (x >= minp_thr) local += __expf((x - vmax) * inv_t);
    }
    const float incl = block_scan_incl(local, scr);
    const float total = block_sum(local, scr);
    const float target = u * total;
    // the first thread whose inclusive sum exceeds the target owns the sample
    const int owner = block_min_int((incl > target && local > 0.f) ? tid : kSampThreads, scr);
    if (tid == 0) sh_pick = imax;
    __syncthreads();
    if (tid == owner) {
      float run = incl - local;
      int pick = -1;
      for (int i = lo; i < hi; ++i) {
        const float x = load_logit(p, row, allow, i);
        if (x >= minp_thr) {
          run += __expf((x - vmax) * inv_t);
          pick = i;
          if (run > target) break;
        }
      }
      if (pick >= 0) sh_pick = pick;
    }
    __syncthreads();
    if (tid == 0) p.tokens[r] = sh_pick;
    if (prow != nullptr) {
      const float inv_total = 1.f / total;
      for (int i = tid; i < V; i += kSampThreads) {
        const float x = load_logit(p, row, allow, i);
        prow[i] = (x >= minp_thr) ? __expf((x - vmax) * inv_t) * inv_total : 0.f;
      }
    }
    return;
  }

  // ---- 3. radix select: key of the K-th largest logit
  const int K = use_topk ? min(cfg.top_k, kCand) : min(V, kCand);
  if (tid == 0) { sh_prefix = 0u; sh_krem = K; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    const uint32_t himask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += kSampThreads) {
      const uint32_t k = f2key(load_logit(p, row, allow, i));
      if ((k & himask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int krem = sh_krem;
      int b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= krem) break;
        krem -= hist[b];
      }
      sh_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      sh_krem = krem;
    }
    __syncthreads();
  }
  const uint32_t thr_key = sh_prefix;

  // ---- 4. gather candidates (key >= threshold), sort descending by (key, then smaller index first)
  if (tid == 0) sh_count = 0;
  cand_key[tid] = 0u;
  cand_idx[tid] = 0xFFFFFFFFu;
  __syncthreads();
  for (int i = tid; i < V; i += kSampThreads) {
    const uint32_t k = f2key(load_logit(p, row, allow, i));
    if (k >= thr_key && k > f2key(-INFINITY)) {
      const int slot = atomicAdd(&sh_count, 1);
      if (slot < kCand) {
        cand_key[slot] = k;
        cand_idx[slot] = static_cast<uint32_t>(i);
      }
    }
  }
  __syncthreads();
  // bitonic sort, descending by key, ties by ascending index (empty slots: key 0 sorts last)
  for (int k = 2; k <= kCand; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      const int ixj = tid ^ j;
      if (ixj > tid) {
        const uint32_t ka = cand_key[tid], kb = cand_key[ixj];
        const uint32_t ia = cand_idx[tid], ib = cand_idx[ixj];
        const bool a_before_b = (ka > kb) || (ka == kb && ia < ib);  // a ranks ahead of b
        const bool desc = (tid & k) == 0;
        if (desc ? !a_before_b : a_before_b) {
          cand_key[tid] = kb; cand_idx[tid] = ib;
          cand_key[ixj] = ka; cand_idx[ixj] = ia;
        }
      }
      __syncthreads();
    }
  }
  const int ncand = min(sh_count, kCand);
  const bool valid = tid < ncand;
  const float x = valid ? key2f(cand_key[tid]) : -INFINITY;
  const int tok = valid ? static_cast<int>(cand_idx[tid]) : 0;

  // ---- 5. top-p at temperature 1 on the top-k survivors
  const float p1 = valid ? __expf(x - vmax) : 0.f;
  float z1;
  if (use_topk) {
    z1 = block_sum(p1, scr);
  } else {
    float local = 0.f;
    for (int i = tid; i < V; i += kSampThreads) local += __expf(load_logit(p, row, allow, i) - vmax);
    z1 = block_sum(local, scr);
  }
  const float cum = block_scan_incl(p1, scr);
  bool keep = valid;
  if (use_topp) keep = keep && ((cum - p1) <= fmaxf(cfg.top_p, 0.f) * z1);
  keep = keep && (x >= minp_thr);
  if (tid == 0) keep = valid;  // the most likely token always survives

  // ---- 6. temperature + categorical over the survivors (sorted order)
  const float w = keep ? __expf((x - vmax) * inv_t) : 0.f;
  const float wcum = block_scan_incl(w, scr);
  const float wtot = block_sum(w, scr);
  const float target = u * wtot;
  int pick = block_min_int((keep && wcum > target) ? tid : kCand, scr);
  if (pick >= kCand) {  // rounding at the upper end: last survivor
    pick = kCand - 1 - block_min_int(keep ? (kCand - 1 - tid) : kCand, scr);
    if (pick < 0 || pick >= kCand) pick = 0;
  }
  if (tid == pick) p.tokens[r] = tok;
  if (prow != nullptr) {
    for (int i = tid; i < V; i += kSampThreads) prow[i] = 0.f;
    __syncthreads();
    if (keep) prow[tok] = w / wtot;
  }
}

// ------------------------------------------------------------------ speculative verify
// One CTA per sequence. p_t: [n_draft + 1, V] target distributions, p_d: [n_draft, V] draft
// distributions (both dense, as written by sampler_kernel), drafted: [n_draft].
// out[0] = number of accepted drafts a (0..n_draft), out[1] = the token that follows them
// (a residual resample on rejection, or the bonus token sampled from p_t[n_draft] on full acceptance).
// Greedy rows (one-hot p_t) reduce to "argmax == proposed".
struct VerifyParams {
  const float* p_t;
  const float* p_d;
  const int* drafted;
  const SamplerRow* rows;  // one per sequence (seed / stream / position of the first drafted token)
  int* out;                // [B, 2]
  int n_draft;
  int V;
};

__global__ void __launch_bounds__(kSampThreads) spec_verify_kernel(VerifyParams p) {
  __shared__ BlockScratch scr;
  __shared__ int sh_pick;
  pdl_launch_early();
  trace_mark(kTraceSampler, kTraceStart);
  pdl_wait();
  trace_mark(kTraceSampler, kTraceAfterWait);
  pdl_launch_dependents();
  const int b = blockIdx.x, tid = threadIdx.x;
  SamplerRow cfg;
  {
    const int* src = reinterpret_cast<const int*>(p.rows + b);
    int* dst = reinterpret_cast<int*>(&cfg);
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(SamplerRow) / 4); ++i) dst[i] = src[i];
  }
  const int V = p.V;
  const float* pt = p.p_t + static_cast<size_t>(b) * (p.n_draft + 1) * V;
  const float* pd = p.p_d + static_cast<size_t>(b) * p.n_draft * V;
  const int* dr = p.drafted + static_cast<size_t>(b) * p.n_draft;
  int accepted = 0;
  int next = -1;
  for (int i = 0; i < p.n_draft; ++i) {
    const int tok = dr[i];
    const float t = pt[static_cast<size_t>(i) * V + tok];
    const float d = pd[static_cast<size_t>(i) * V + tok];
    const float u = philox_uniform(cfg.seed_lo, cfg.seed_hi, cfg.stream_id, static_cast<uint32_t>(cfg.position + i), 1u);
    const bool accept = (d > 0.f) ? (u * d < t) : (t > 0.f);
    if (accept) { ++accepted; continue; }
    // residual distribution max(p_t - p_d, 0), sampled in index order
    const float* ti = pt + static_cast<size_t>(i) * V;
    const float* di = pd + static_cast<size_t>(i) * V;
    const int seg = (V + kSampThreads - 1) / kSampThreads;
    const int lo = tid * seg, hi = min(V, lo + seg);
    float local = 0.f;
    for (int j = lo; j < hi; ++j) local += fmaxf(ti[j] - di[j], 0.f);
    const float incl = block_scan_incl(local, scr);
    const float total = block_sum(local, scr);
    const float u2 = philox_uniform(cfg.seed_lo, cfg.seed_hi, cfg.stream_id, static_cast<uint32_t>(cfg.position + i), 2u);
    if (tid == 0) sh_pick = -1;
    __syncthreads();
    if (total > 0.f) {
      const float target = u2 * total;
      const int owner = block_min_int((incl > target && local > 0.f) ? tid : kSampThreads, scr);
      if (tid == owner) {
        float run = incl - local;
        int pick = -1;
        for (int j = lo; j < hi; ++j) {
          const float rj = fmaxf(ti[j] - di[j], 0.f);
          if (rj > 0.f) { run += rj; pick = j; if (run > target) break; }
        }
        sh_pick = pick;
      }
      __syncthreads();
    }
    next = sh_pick;
    if (next < 0) {  // degenerate residual (p_t == p_d): fall back to the target's most likely token
      float v = -1.f; int vi = 0x7fffffff;
      for (int j = tid; j < V; j += kSampThreads) if (ti[j] > v) { v = ti[j]; vi = j; }
      block_argmax(v, vi, scr);
      next = vi;
    }
    break;
  }
  if (next < 0) {
    // every draft accepted: bonus token from p_t[n_draft]
    const float* ti = pt + static_cast<size_t>(p.n_draft) * V;
    const int seg = (V + kSampThreads - 1) / kSampThreads;
    const int lo = tid * seg, hi = min(V, lo + seg);
    float local = 0.f;
    for (int j = lo; j < hi; ++j) local += ti[j];
    const float incl = block_scan_incl(local, scr);
    const float total = block_sum(local, scr);
    const float u3 = philox_uniform(cfg.seed_lo, cfg.seed_hi, cfg.stream_id, static_cast<uint32_t>(cfg.position + p.n_draft), 0u);
    const float target = u3 * total;
    const int owner = block_min_int((incl > target && local > 0.f) ? tid : kSampThreads, scr);
    if (tid == 0) sh_pick = -1;
    __syncthreads();
    if (tid == owner) {
      float run = incl - local;
      int pick = -1;
      for (int j = lo; j < hi; ++j) {
        if (ti[j] > 0.f) { run += ti[j]; pick = j; if (run > target) break; }
      }
      sh_pick = pick;
    }
    __syncthreads();
    next = sh_pick;
    if (next < 0) {
      float v = -1.f; int vi = 0x7fffffff;
      for (int j = tid; j < V; j += kSampThreads) if (ti[j] > v) { v = ti[j]; vi = j; }
      block_argmax(v, vi, scr);
      next = vi;
    }
  }
  if (tid == 0) {
    p.out[b * 2 + 0] = accepted;
    p.out[b * 2 + 1] = next;
  }
}

}  // namespace eredu

using namespace eredu;

EREDU_TRACE_INSTALLER(sampler)

extern "C" int eredu_sampler_row_bytes() { return static_cast<int>(sizeof(SamplerRow)); }

extern "C" int eredu_sample(float* logits, const unsigned int* allow, int allow_stride, const void* rows,
                            const int* history, int hist_stride, int* tokens, float* probs, int n_rows, int V,
                            cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  SamplerParams p;
  p.logits = logits;
  p.allow = allow;
  p.allow_stride = allow_stride;
  p.rows = static_cast<const SamplerRow*>(rows);
  p.history = history;
  p.hist_stride = hist_stride;
  p.tokens = tokens;
  p.probs = probs;
  p.V = V;
  launch_pdl(sampler_kernel, dim3(n_rows), dim3(kSampThreads), 0, stream, p);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_spec_verify(const float* p_t, const float* p_d, const int* drafted, const void* rows, int* out,
                                 int batch, int n_draft, int V, cudaStream_t stream) {
  if (batch <= 0) return 0;
  VerifyParams p;
  p.p_t = p_t;
  p.p_d = p_d;
  p.drafted = drafted;
  p.rows = static_cast<const SamplerRow*>(rows);
  p.out = out;
  p.n_draft = n_draft;
  p.V = V;
  launch_pdl(spec_verify_kernel, dim3(batch), dim3(kSampThreads), 0, stream, p);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
