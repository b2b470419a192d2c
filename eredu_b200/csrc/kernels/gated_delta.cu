// Gated delta-rule recurrence of linear-attention layers (Qwen3-Next / Kimi-Linear style), one token after another:
//   S  <- S * exp(g_t)                      (g_t: one log decay per head, or one per key channel)
//   m   = S^T k_t                            (what the memory currently returns for this key)
//   S  <- S + k_t (beta_t * (v_t - m))^T     (delta rule: move the stored value toward v_t)
//   o_t = S^T q_t
// with S [Dk, Dv] per (sequence, head) kept in fp32 (eredu/src/backend/mlx/nn/gated_delta.rs:135-183 is the step,
// :295-360 the scan). A quad of lanes owns one value column of S in registers for the whole scan; the token's key, query and
// decay vectors are staged in shared memory once per token for all columns of the block. Sequential in the tokens by construction:
// the kernel serves decode steps and short chunks, a chunk-parallel form is a separate piece of work.
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"

namespace eredu {

struct GatedDeltaParams {
  const __nv_bfloat16* q;   // [B, T, H, DK]
  const __nv_bfloat16* k;   // [B, T, H, DK]
  const __nv_bfloat16* v;   // [B, T, H, Dv]
  const float* log_decay;   // [B, T, H] or [B, T, H, DK]
  const float* beta;        // [B, T, H]
  float* state;             // [B, H, DK, Dv], updated in place
  __nv_bfloat16* out;       // [B, T, H, Dv]
  int B, T, H, Dv;
  int vector_decay;
};

// Four consecutive lanes share one value column: lane `sub` of the quad keeps the rows i = 4 r + sub of that column
// (DK / 4 registers), and the two dot products of a step are finished with two shuffles inside the quad.
template <int DK>
__global__ void __launch_bounds__(128) gated_delta_kernel(GatedDeltaParams p) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  constexpr int R = DK / 4;
  __shared__ float ks[DK], qs[DK], ds[DK];
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int sub = threadIdx.x & 3;
  const int j = blockIdx.x * 32 + (threadIdx.x >> 2);
  const bool live = j < p.Dv;
  float S[R];
  float* st = p.state + (static_cast<size_t>(bh) * DK) * p.Dv + (live ? j : 0);
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = live ? st[static_cast<size_t>(4 * r + sub) * p.Dv] : 0.f;

  for (int t = 0; t < p.T; ++t) {
    const size_t row = (static_cast<size_t>(b) * p.T + t) * p.H + h;
    for (int i = threadIdx.x; i < DK; i += 128) {
      ks[i] = __bfloat162float(p.k[row * DK + i]);
      qs[i] = __bfloat162float(p.q[row * DK + i]);
      ds[i] = __expf(p.vector_decay ? p.log_decay[row * DK + i] : p.log_decay[row]);
    }
    __syncthreads();
    float mem = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      S[r] *= ds[4 * r + sub];
      mem += S[r] * ks[4 * r + sub];
    }
    mem += __shfl_xor_sync(0xffffffffu, mem, 1);
    mem += __shfl_xor_sync(0xffffffffu, mem, 2);
    const float vj = live ? __bfloat162float(p.v[row * p.Dv + j]) : 0.f;
    const float delta = p.beta[row] * (vj - mem);
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      S[r] += ks[4 * r + sub] * delta;
      o += S[r] * qs[4 * r + sub];
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    if (live && sub == 0) p.out[row * p.Dv + j] = __float2bfloat16(o);
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) st[static_cast<size_t>(4 * r + sub) * p.Dv] = S[r];
  }
}

}  // namespace eredu

using namespace eredu;

// q, k [B, T, H, Dk] bf16; v, out [B, T, H, Dv] bf16; log_decay fp32 [B, T, H] (vector_decay = 0) or [B, T, H, Dk];
// beta fp32 [B, T, H]; state fp32 [B, H, Dk, Dv] read and written. Dk is 64 or 128.
extern "C" int eredu_gated_delta_scan(const void* q, const void* k, const void* v, const float* log_decay, const float* beta,
                                      float* state, void* out, int B, int T, int H, int Dk, int Dv, int vector_decay,
                                      cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || Dv <= 0) return 0;
  if (Dk != 64 && Dk != 128) return -1;
  GatedDeltaParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.log_decay = log_decay;
  p.beta = beta;
  p.state = state;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.B = B;
  p.T = T;
  p.H = H;
  p.Dv = Dv;
  p.vector_decay = vector_decay;
  dim3 grid((Dv + 31) / 32, B * H);
  cudaError_t e = Dk == 64 ? launch_pdl(gated_delta_kernel<64>, grid, dim3(128), 0, stream, p)
                           : launch_pdl(gated_delta_kernel<128>, grid, dim3(128), 0, stream, p);
  eredu_count_launches(1);
  return static_cast<int>(e);
}
