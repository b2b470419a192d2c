// Memory-bound glue kernels of the decoder block, each fused as far as the data flow allows:
//   * (residual add +) RMSNorm                       (reference: safemlx/src/fast.rs:1119-1148,
//                                                      eredu/src/backend/mlx/nn/shared.rs:121-140)
//   * per-head q/k RMSNorm + RoPE + paged KV append   (nn/rope.rs:111-226, qwen/dense.rs:739-790,
//                                                      runtime/cache/kv.rs:2781-2860)
//   * embedding gather with vocab-parallel masking    (nn/parallel.rs:980-1018)
//   * silu(gate) * up for paths whose GEMM cannot fuse it (nn/layers.rs:21-24)
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"
#include "../common/trace.cuh"

namespace eredu {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One CTA per row. h = x (+ residual); h_out = h (optional); y = h * rsqrt(mean(h^2) + eps) * (w + w_off).
template <int THREADS, int MAXCH>
__global__ void __launch_bounds__(THREADS) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ residual,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                           __nv_bfloat16* __restrict__ h_out, int H, float eps,
                                                           float w_off) {
  __shared__ float red[32];
  pdl_launch_early();
  trace_mark(kTraceRmsNorm, kTraceStart);
  pdl_wait();
  trace_mark(kTraceRmsNorm, kTraceAfterWait);
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  const int nch = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + row * H) : nullptr;
  float vals[MAXCH][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXCH; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < nch) {
      uint4 v = xr[c];
      uint32_t u[4] = {v.x, v.y, v.z, v.w};
      uint32_t ru[4] = {0, 0, 0, 0};
      if (rr) {
        uint4 r = rr[c];
        ru[0] = r.x; ru[1] = r.y; ru[2] = r.z; ru[3] = r.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a = bf16_lo(u[j]) + bf16_lo(ru[j]);
        float b = bf16_hi(u[j]) + bf16_hi(ru[j]);
        if (rr) {  // the residual stream is stored in bf16: normalise exactly what is stored
          a = __bfloat162float(__float2bfloat16(a));
          b = __bfloat162float(__float2bfloat16(b));
        }
        vals[i][2 * j] = a;
        vals[i][2 * j + 1] = b;
        ss += a * a + b * b;
      }
      if (h_out) {
        uint4 o;
        o.x = pack_bf16x2(vals[i][0], vals[i][1]);
        o.y = pack_bf16x2(vals[i][2], vals[i][3]);
        o.z = pack_bf16x2(vals[i][4], vals[i][5]);
        o.w = pack_bf16x2(vals[i][6], vals[i][7]);
        reinterpret_cast<uint4*>(h_out + row * H)[c] = o;
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < THREADS / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  const float inv = rsqrtf(red[0] / static_cast<float>(H) + eps);
#pragma unroll
  for (int i = 0; i < MAXCH; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < nch) {
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * c];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * c + 1];
      uint4 o;
      o.x = pack_bf16x2(vals[i][0] * inv * (w0.x + w_off), vals[i][1] * inv * (w0.y + w_off));
      o.y = pack_bf16x2(vals[i][2] * inv * (w0.z + w_off), vals[i][3] * inv * (w0.w + w_off));
      o.z = pack_bf16x2(vals[i][4] * inv * (w1.x + w_off), vals[i][5] * inv * (w1.y + w_off));
      o.w = pack_bf16x2(vals[i][6] * inv * (w1.z + w_off), vals[i][7] * inv * (w1.w + w_off));
      reinterpret_cast<uint4*>(y + row * H)[c] = o;
    }
  }
}

struct RopeParams {
  const __nv_bfloat16* qkv;  // [M, ld] = [q heads | k heads | v heads] x D
  __nv_bfloat16* q_out;      // [M, n_q, D]
  __nv_bfloat16* k_cache;    // [pages, n_kv, 16, D]
  __nv_bfloat16* v_cache;
  const int* positions;      // [M]
  const long long* slots;    // [M] page * 16 + offset, < 0 = do not store
  const float* inv_freq;     // [rot/2]
  const float* q_norm_w;     // optional [D]
  const float* k_norm_w;     // optional [D]
  int ld, n_q, n_kv, D, rot;  // rot = rotary dims (<= D)
  int interleaved;            // 0: pairs (i, i+rot/2) ("split-half"), 1: pairs (2i, 2i+1)
  float attn_factor;          // multiplies cos/sin (YaRN mscale), 1 otherwise
  float norm_eps;
  float norm_w_off;
};

// grid (M, n_q + 2 n_kv), D/2 threads: thread i owns one rotation pair (or a pass-through pair).
__global__ void rope_kv_kernel(RopeParams p) {
  __shared__ float red[8];
  pdl_launch_early();
  trace_mark(kTraceRope, kTraceStart);
  pdl_wait();
  trace_mark(kTraceRope, kTraceAfterWait);
  pdl_launch_dependents();
  const int m = blockIdx.x, head = blockIdx.y;
  const int i = threadIdx.x;
  const int half = p.D >> 1;
  const bool is_q = head < p.n_q;
  const bool is_k = !is_q && head < p.n_q + p.n_kv;
  const __nv_bfloat16* src = p.qkv + static_cast<size_t>(m) * p.ld + static_cast<size_t>(head) * p.D;
  int i0, i1;
  const int rh = p.rot >> 1;
  if (i < rh) {
    i0 = p.interleaved ? 2 * i : i;
    i1 = p.interleaved ? 2 * i + 1 : i + rh;
  } else {  // pass-through tail beyond the rotary dims
    i0 = p.rot + 2 * (i - rh);
    i1 = i0 + 1;
  }
  float a = __bfloat162float(src[i0]);
  float b = __bfloat162float(src[i1]);
  const float* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
  if (nw != nullptr) {
    float ss = warp_sum(a * a + b * b);
    if ((i & 31) == 0) red[i >> 5] = ss;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (half + 31) / 32; ++w) t += red[w];
    const float inv = rsqrtf(t / static_cast<float>(p.D) + p.norm_eps);
    // match a bf16 module boundary: the normalised head is rounded before the rotation
    a = __bfloat162float(__float2bfloat16(a * inv * (nw[i0] + p.norm_w_off)));
    b = __bfloat162float(__float2bfloat16(b * inv * (nw[i1] + p.norm_w_off)));
  }
  if ((is_q || is_k) && i < rh) {
    float sn, cs;
    sincosf(static_cast<float>(p.positions[m]) * p.inv_freq[i], &sn, &cs);
    sn *= p.attn_factor;
    cs *= p.attn_factor;
    const float ra = a * cs - b * sn;
    const float rb = b * cs + a * sn;
    a = ra;
    b = rb;
  }
  if (is_q) {
    __nv_bfloat16* dst = p.q_out + (static_cast<size_t>(m) * p.n_q + head) * p.D;
    dst[i0] = __float2bfloat16(a);
    dst[i1] = __float2bfloat16(b);
  } else {
    const long long slot = p.slots[m];
    if (slot >= 0) {
      const int kvh = is_k ? head - p.n_q : head - p.n_q - p.n_kv;
      __nv_bfloat16* cache = is_k ? p.k_cache : p.v_cache;
      const long long page = slot >> 4;
      const int off = static_cast<int>(slot & 15);
      __nv_bfloat16* dst = cache + ((page * p.n_kv + kvh) * 16 + off) * p.D;
      dst[i0] = __float2bfloat16(a);
      dst[i1] = __float2bfloat16(b);
    }
  }
}

// out[m, :] = table[ids[m] - vocab_start, :] when the id falls in [vocab_start, vocab_start + rows), else 0.
// ssq_out (optional, [M]) receives the sum of squares of the stored row, for an RMSNorm fused into the
// first GEMM of the first layer.
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int H, int vocab_start, int rows, float scale,
                                 float* __restrict__ ssq_out) {
  __shared__ float red[8];
  pdl_launch_early();
  trace_mark(kTraceEmbedding, kTraceStart);
  pdl_wait();
  trace_mark(kTraceEmbedding, kTraceAfterWait);
  pdl_launch_dependents();
  const size_t m = blockIdx.x;
  const int id = ids[m] - vocab_start;
  const bool ok = id >= 0 && id < rows;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(ok ? id : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + m * H);
  float ss = 0.f;
  for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) {
    uint4 v = ok ? src[c] : make_uint4(0, 0, 0, 0);
    if (scale != 1.f) {
      v.x = pack_bf16x2(bf16_lo(v.x) * scale, bf16_hi(v.x) * scale);
      v.y = pack_bf16x2(bf16_lo(v.y) * scale, bf16_hi(v.y) * scale);
      v.z = pack_bf16x2(bf16_lo(v.z) * scale, bf16_hi(v.z) * scale);
      v.w = pack_bf16x2(bf16_lo(v.w) * scale, bf16_hi(v.w) * scale);
    }
    dst[c] = v;
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += bf16_lo(u[j]) * bf16_lo(u[j]) + bf16_hi(u[j]) * bf16_hi(u[j]);
  }
  if (ssq_out != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t += red[w];
      ssq_out[m] = t;
    }
  }
}

// y[m, i] = silu(x[m, i]) * x[m, I + i], optional clamp of both branches (swiglu_limit).
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int I, int ldx,
                                float limit) {
  pdl_launch_early();
  trace_mark(kTraceSiluMul, kTraceStart);
  pdl_wait();
  trace_mark(kTraceSiluMul, kTraceAfterWait);
  pdl_launch_dependents();
  const size_t m = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= (I >> 3)) return;
  const uint4 g = reinterpret_cast<const uint4*>(x + m * ldx)[c];
  const uint4 u = reinterpret_cast<const uint4*>(x + m * ldx + I)[c];
  const uint32_t gv[4] = {g.x, g.y, g.z, g.w};
  const uint32_t uv[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float g0 = bf16_lo(gv[j]), g1 = bf16_hi(gv[j]), u0 = bf16_lo(uv[j]), u1 = bf16_hi(uv[j]);
    if (limit > 0.f) {
      g0 = fminf(g0, limit); g1 = fminf(g1, limit);
      u0 = fminf(fmaxf(u0, -limit), limit); u1 = fminf(fmaxf(u1, -limit), limit);
    }
    o[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
  }
  reinterpret_cast<uint4*>(y + m * I)[c] = make_uint4(o[0], o[1], o[2], o[3]);
}


// Device-side bookkeeping between two decode steps, so that a captured decode graph replays with
// no host work: feed the sampled token back, advance position / kv length, derive the next KV
// slot from the (pre-reserved) block table, append to the penalty history and advance the RNG
// position stored in the packed sampler row (int32 index 9 = position, 8 = hist_len).
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ token_ids,
                                      int* __restrict__ positions, int* __restrict__ seq_lens,
                                      long long* __restrict__ slots, const int* __restrict__ block_table,
                                      int max_pages, const int* __restrict__ active, int* __restrict__ sampler_rows,
                                      int row_ints, int* __restrict__ history, int hist_stride, int B) {
  pdl_launch_early();
  trace_mark(kTraceAdvance, kTraceStart);
  pdl_wait();
  trace_mark(kTraceAdvance, kTraceAfterWait);
  pdl_launch_dependents();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (active != nullptr && active[b] == 0) {
    slots[b] = -1;
    return;
  }
  const int tok = sampled[b];
  token_ids[b] = tok;
  const int pos = positions[b] + 1;
  positions[b] = pos;
  seq_lens[b] = pos + 1;
  const int page = block_table[static_cast<size_t>(b) * max_pages + (pos >> 4)];
  slots[b] = static_cast<long long>(page) * 16 + (pos & 15);
  if (sampler_rows != nullptr) {
    int* row = sampler_rows + static_cast<size_t>(b) * row_ints;
    if (history != nullptr) {
      const int n = row[8];
      if (n < hist_stride) {
        history[static_cast<size_t>(b) * hist_stride + n] = tok;
        row[8] = n + 1;
      }
    }
    row[9] += 1;
  }
}

}  // namespace eredu

using namespace eredu;

EREDU_TRACE_INSTALLER(norm_rope)

extern "C" int eredu_rmsnorm(const void* x, const void* residual, const float* w, void* y, void* h_out, int M, int H,
                             float eps, float w_off, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H % 8 != 0 || H > 256 * 8 * 8) return -1;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto Ho = static_cast<__nv_bfloat16*>(h_out);
  const int nch = H / 8;
  if (nch <= 128) launch_pdl(rmsnorm_kernel<128, 1>, dim3(M), dim3(128), 0, stream, X, R, w, Y, Ho, H, eps, w_off);
  else if (nch <= 256) launch_pdl(rmsnorm_kernel<256, 1>, dim3(M), dim3(256), 0, stream, X, R, w, Y, Ho, H, eps, w_off);
  else if (nch <= 512) launch_pdl(rmsnorm_kernel<256, 2>, dim3(M), dim3(256), 0, stream, X, R, w, Y, Ho, H, eps, w_off);
  else if (nch <= 1024) launch_pdl(rmsnorm_kernel<256, 4>, dim3(M), dim3(256), 0, stream, X, R, w, Y, Ho, H, eps, w_off);
  else launch_pdl(rmsnorm_kernel<256, 8>, dim3(M), dim3(256), 0, stream, X, R, w, Y, Ho, H, eps, w_off);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_rope_kv(const void* qkv, void* q_out, void* k_cache, void* v_cache, const int* positions,
                             const long long* slots, const float* inv_freq, const float* q_norm_w,
                             const float* k_norm_w, int M, int ld, int n_q, int n_kv, int D, int rot, int interleaved,
                             float attn_factor, float norm_eps, float norm_w_off, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (D % 2 != 0 || D > 512 || rot > D || rot % 2 != 0) return -1;
  RopeParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.positions = positions;
  p.slots = slots;
  p.inv_freq = inv_freq;
  p.q_norm_w = q_norm_w;
  p.k_norm_w = k_norm_w;
  p.ld = ld;
  p.n_q = n_q;
  p.n_kv = n_kv;
  p.D = D;
  p.rot = rot;
  p.interleaved = interleaved;
  p.attn_factor = attn_factor;
  p.norm_eps = norm_eps;
  p.norm_w_off = norm_w_off;
  launch_pdl(rope_kv_kernel, dim3(M, n_q + 2 * n_kv), dim3(D / 2), 0, stream, p);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_embedding(const int* ids, const void* table, void* out, int M, int H, int vocab_start, int rows,
                               float scale, float* ssq_out, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H % 8 != 0) return -1;
  launch_pdl(embedding_kernel, dim3(M), dim3(256), 0, stream, ids, static_cast<const __nv_bfloat16*>(table),
             static_cast<__nv_bfloat16*>(out), H, vocab_start, rows, scale, ssq_out);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_silu_mul(const void* x, void* y, int M, int I, int ldx, float limit, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (I % 8 != 0) return -1;
  dim3 grid((I / 8 + 255) / 256, M);
  launch_pdl(silu_mul_kernel, grid, dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x),
             static_cast<__nv_bfloat16*>(y), I, ldx, limit);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int eredu_decode_advance(const int* sampled, int* token_ids, int* positions, int* seq_lens,
                                    long long* slots, const int* block_table, int max_pages, const int* active,
                                    int* sampler_rows, int row_ints, int* history, int hist_stride, int B,
                                    cudaStream_t stream) {
  if (B <= 0) return 0;
  launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, sampled, token_ids, positions,
             seq_lens, slots, block_table, max_pages, active, sampler_rows, row_ints, history, hist_stride, B);
  eredu_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}
