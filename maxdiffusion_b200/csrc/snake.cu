// Anti-aliased Snake activation of the BigVGAN-style vocoder as ONE kernel:
//   up-sample x2 (zero stuffing + 12-tap Kaiser-sinc FIR, replicate padding)  ->  snake(u) = u + sin^2(alpha u) / beta
//   ->  low-pass + decimate x2 (12-tap FIR, stride 2, replicate padding).
// The reference runs three XLA ops with the 2x-rate signal materialised in HBM between them
// (src/maxdiffusion/models/ltx2/vocoder_ltx2.py:75-270: UpSample1d, SnakeBeta, DownSample1d, AntiAliasAct1d);
// here the 2x-rate signal only ever exists in shared memory.
//
// Index arithmetic (K = 12, ratio 2; L input samples per row):
//   x_pad[p]  = x[clamp(p - 5, 0, L-1)]                         p in [0, L+10)
//   u[j]      = 2 * sum_{m, (j+15-m) even} f_up[m] * x_pad[(j + 15 - m) / 2]        j in [0, 2L)
//   a[j]      = snake(u[j])
//   out[t]    = sum_{k<12} f_dn[k] * a[clamp(2t + k - 5, 0, 2L-1)]                   t in [0, L)
#include "host_common.h"

namespace mdb {
namespace snake {

constexpr int K = 12;
constexpr int TILE = 256;           // outputs per block
constexpr int U_LEN = 2 * TILE + K; // activated samples needed by a tile

struct Filters {
  float up[K];
  float dn[K];
};

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

// rows = B * C contiguous rows of L samples; alpha / inv_beta are per channel (row % C). mode 0 = snake, 1 = leaky relu
// with slope `alpha[0]` (the anti-aliased path of the plain activation).
template <typename T>
__global__ void __launch_bounds__(256)
snake_aa_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ alpha,
                const float* __restrict__ inv_beta, Filters f, int C, int L, int mode) {
  __shared__ float xs[TILE + 16];
  __shared__ float us[U_LEN];
  const long long row = blockIdx.y;
  const int t0 = blockIdx.x * TILE;
  const int c = static_cast<int>(row % C);
  const T* xr = x + row * L;
  // input samples x[t0 - 8 .. t0 + TILE + 7], clamped
  for (int i = threadIdx.x; i < TILE + 16; i += blockDim.x) {
    int idx = t0 - 8 + i;
    idx = idx < 0 ? 0 : (idx > L - 1 ? L - 1 : idx);
    xs[i] = ldf<T>(xr, idx);
  }
  __syncthreads();
  const float a = mode == 0 ? alpha[c] : alpha[0];
  const float ib = mode == 0 ? inv_beta[c] : 0.0f;
  const int j0 = 2 * t0 - 5;  // first activated sample of this tile (before clamping)
  for (int i = threadIdx.x; i < U_LEN; i += blockDim.x) {
    int j = j0 + i;
    j = j < 0 ? 0 : (j > 2 * L - 1 ? 2 * L - 1 : j);
    float u = 0.0f;
    // taps with (j + 15 - m) even: m has the parity of (j + 15)
    const int m0 = (j + 15) & 1;
#pragma unroll
    for (int q = 0; q < K / 2; ++q) {
      const int m = m0 + 2 * q;
      int p = ((j + 15 - m) >> 1) - 5;               // index into x
      p = p < 0 ? 0 : (p > L - 1 ? L - 1 : p);
      u = fmaf(f.up[m], xs[p - (t0 - 8)], u);
    }
    u *= 2.0f;
    if (mode == 0) {
      const float s = __sinf(u * a);
      u = fmaf(ib, s * s, u);
    } else {
      u = u > 0.0f ? u : a * u;
    }
    us[i] = u;
  }
  __syncthreads();
  const int t = t0 + threadIdx.x;
  if (t < L) {
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) acc = fmaf(f.dn[k], us[2 * threadIdx.x + k], acc);
    stf<T>(out + row * L, t, acc);
  }
}

}  // namespace snake
}  // namespace mdb

// x, out: [rows, L] contiguous (rows = batch * channels), fp32 or bf16. f_up / f_dn: 12 host floats each.
// alpha, inv_beta: device fp32 [C] (already exponentiated; inv_beta = 1 / (beta + eps)).
extern "C" int mdb_snake_aa(const void* x, void* out, int is_f32, const float* alpha, const float* inv_beta,
                            const float* f_up, const float* f_dn, long long rows, int C, int L, int mode,
                            void* stream_ptr) {
  using namespace mdb::snake;
  if (rows <= 0 || L <= 0) return 0;
  if (rows > 65535 || C < 1 || L > (1 << 29)) return 3201;  // grid.y limit; callers chunk the rows
  Filters f;
  for (int i = 0; i < K; ++i) {
    f.up[i] = f_up[i];
    f.dn[i] = f_dn[i];
  }
  dim3 grid((L + TILE - 1) / TILE, static_cast<unsigned int>(rows));
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (is_f32)
    snake_aa_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(out), alpha, inv_beta, f, C, L, mode);
  else
    snake_aa_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out),
                                                        alpha, inv_beta, f, C, L, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
