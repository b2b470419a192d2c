// Mamba-2 selective state-space recurrence, one token after another (Nemotron-H mixer layers):
//   S  <- S * exp(dt_t A) + x_t (dt_t B_t)^T        S [P, N] per (sequence, head), fp32
//   y_t = S C_t + D x_t
// with one scalar decay per head and step (eredu/src/backend/mlx/architectures/nemotron_h/model.rs:1929-1962 is the
// reference recurrence). A quad of lanes owns one state row p in registers for the whole scan (lane `sub` keeps the columns
// n = 4 r + sub); the token's B and C vectors are staged in shared memory once per token for all rows of the block, the row
// dot product with C is finished by two shuffles inside the quad. B and C come per group (G groups, H / G heads each).
// Sequential in the tokens by construction: decode steps and short chunks; a chunk-parallel (SSD) form is separate work.
#include "../common/launch.h"
#include "../common/launch_count.h"
#include "../common/ptx.cuh"

namespace eredu {

struct Mamba2Params {
  const __nv_bfloat16* x;    // [B, T, H, P]
  const __nv_bfloat16* Bm;   // [B, T, G, N]
  const __nv_bfloat16* Cm;   // [B, T, G, N]
  const float* dt;           // [B, T, H]  (after softplus and limits)
  const float* A;            // [H]        (negative)
  const float* D;            // [H]
  float* state;              // [B, H, P, N], updated in place
  __nv_bfloat16* out;        // [B, T, H, P]
  int B, T, H, G, P;
};

template <int N>
__global__ void __launch_bounds__(128) mamba2_scan_kernel(Mamba2Params p) {
  pdl_launch_early();
  pdl_wait();
  pdl_launch_dependents();
  constexpr int R = N / 4;
  __shared__ float bs[N], cs[N];
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int g = h / (p.H / p.G);
  const int sub = threadIdx.x & 3;
  const int row_p = blockIdx.x * 32 + (threadIdx.x >> 2);
  const bool live = row_p < p.P;
  float S[R];
  float* st = p.state + (static_cast<size_t>(bh) * p.P + (live ? row_p : 0)) * N;
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = live ? st[4 * r + sub] : 0.f;
  const float a = p.A[h], d_skip = p.D[h];

  for (int t = 0; t < p.T; ++t) {
    const size_t tok = static_cast<size_t>(b) * p.T + t;
    const size_t grow = (tok * p.G + g) * N;
    for (int i = threadIdx.x; i < N; i += 128) {
      bs[i] = __bfloat162float(p.Bm[grow + i]);
      cs[i] = __bfloat162float(p.Cm[grow + i]);
    }
    __syncthreads();
    const size_t hrow = tok * p.H + h;
    const float dt = p.dt[hrow];
    const float xv = live ? __bfloat162float(p.x[hrow * p.P + row_p]) : 0.f;
    const float decay = __expf(dt * a), dx = dt * xv;
    float y = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      S[r] = S[r] * decay + dx * bs[4 * r + sub];
      y += S[r] * cs[4 * r + sub];
    }
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    if (live && sub == 0) p.out[hrow * p.P + row_p] = __float2bfloat16(y + d_skip * xv);
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) st[4 * r + sub] = S[r];
  }
}

}  // namespace eredu

using namespace eredu;

// x, out [B, T, H, P] bf16; Bm, Cm [B, T, G, N] bf16 (G divides H); dt fp32 [B, T, H]; A, D fp32 [H]; state fp32
// [B, H, P, N] read and written. N is 64, 128 or 256.
extern "C" int eredu_mamba2_scan(const void* x, const void* Bm, const void* Cm, const float* dt, const float* A, const float* D,
                                 float* state, void* out, int B, int T, int H, int G, int P, int N, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || P <= 0) return 0;
  if (G <= 0 || H % G != 0) return -1;
  if (N != 64 && N != 128 && N != 256) return -1;
  Mamba2Params p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.Bm = static_cast<const __nv_bfloat16*>(Bm);
  p.Cm = static_cast<const __nv_bfloat16*>(Cm);
  p.dt = dt;
  p.A = A;
  p.D = D;
  p.state = state;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.B = B;
  p.T = T;
  p.H = H;
  p.G = G;
  p.P = P;
  dim3 grid((P + 31) / 32, B * H);
  cudaError_t e = N == 64    ? launch_pdl(mamba2_scan_kernel<64>, grid, dim3(128), 0, stream, p)
                  : N == 128 ? launch_pdl(mamba2_scan_kernel<128>, grid, dim3(128), 0, stream, p)
                             : launch_pdl(mamba2_scan_kernel<256>, grid, dim3(128), 0, stream, p);
  eredu_count_launches(1);
  return static_cast<int>(e);
}
