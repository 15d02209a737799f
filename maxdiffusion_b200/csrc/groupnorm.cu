// GroupNorm (+ optional fused SiLU), forward and backward, for channels-first activations
// [N, C, *spatial] whose (n, c) rows of `hw` elements are contiguous (UNet ResNet blocks, VAE blocks:
// reference src/maxdiffusion/models/resnet_flax.py:97-186, src/maxdiffusion/models/vae_flax.py).
//
// Two streaming passes, both with one CTA per (n, c, split) slice so that small-batch, high-resolution
// VAE shapes (32 groups only) still fill 148 SMs:
//   stats : partial[n, c, s] = {sum x, sum x^2}                       (bwd: {sum dy', sum dy' * xhat})
//   apply : group statistics = ordered sum of the group's partials (bitwise reproducible), then
//           y = act(xhat * gamma + beta)                               (bwd: dx from the two group sums)
// dgamma / dbeta are the per-channel sums of the backward partials (folded on the host side from the
// [N, C, S, 2] partial array). Statistics are fp32; IO is bf16 or fp32.
#include "host_common.h"

namespace mdb {
namespace gn {

__device__ __forceinline__ float ld(const void* p, int f32, long long i) {
  return f32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st(void* p, int f32, long long i, float v) {
  if (f32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// V consecutive elements starting at element index i (i a multiple of V; V = 8 needs 16-byte aligned rows)
template <int V> __device__ __forceinline__ void ldv(const void* p, int f32, long long i, float (&f)[V]) {
  if constexpr (V == 1) {
    f[0] = ld(p, f32, i);
  } else if (f32) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    const float4 a = q[0], b = q[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
  }
}
template <int V> __device__ __forceinline__ void stv(void* p, int f32, long long i, const float (&f)[V]) {
  if constexpr (V == 1) {
    st(p, f32, i, f[0]);
  } else if (f32) {
    float4* q = reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i);
    q[0] = make_float4(f[0], f[1], f[2], f[3]);
    q[1] = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = u;
  }
}

__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = make_float2(a, b);
  __syncthreads();
  float2 t = make_float2(0.f, 0.f);
  if (w == 0) {
    if (l < (blockDim.x >> 5)) t = red[l];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      t.x += __shfl_xor_sync(0xffffffffu, t.x, o);
      t.y += __shfl_xor_sync(0xffffffffu, t.y, o);
    }
  }
  __syncthreads();
  return t;
}

struct Shape {
  int N, C, G, S;      // S = splits of a row
  long long hw;        // elements per (n, c) row
  long long slice;     // elements per split (last may be short)
};

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }
__device__ __forceinline__ float dsilu(float v) {
  const float s = 1.0f / (1.0f + __expf(-v));
  return s * (1.0f + v * (1.0f - s));
}

// grid = N*C*S. Forward statistics.
template <int V> __global__ void __launch_bounds__(256)
stats_fwd_kernel(const void* __restrict__ x, int x_f32, Shape sh, float2* __restrict__ partial) {
  __shared__ float2 red[8];
  const long long row = blockIdx.x / sh.S;
  const int s = blockIdx.x % sh.S;
  const long long lo = s * sh.slice, hi = min(sh.hw, lo + sh.slice);
  const long long base = row * sh.hw;
  float a = 0.f, b = 0.f;
  for (long long i = lo + static_cast<long long>(threadIdx.x) * V; i < hi; i += static_cast<long long>(blockDim.x) * V) {
    float f[V];
    ldv<V>(x, x_f32, base + i, f);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      a += f[j];
      b = fmaf(f[j], f[j], b);
    }
  }
  const float2 t = block_sum2(a, b, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// Ordered sum of the partials of group (n, g): Cg * S consecutive entries starting at (n*C + g*Cg) * S.
__device__ __forceinline__ float2 group_sum(const float2* __restrict__ partial, const Shape& sh, int n, int g,
                                            float2* sm) {
  const int Cg = sh.C / sh.G;
  const int cnt = Cg * sh.S;
  const float2* p = partial + (static_cast<long long>(n) * sh.C + g * Cg) * sh.S;
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int i = 0; i < cnt; ++i) {
      a += p[i].x;
      b += p[i].y;
    }
    *sm = make_float2(a, b);
  }
  __syncthreads();
  return *sm;
}

template <int V> __global__ void __launch_bounds__(256)
apply_fwd_kernel(const void* __restrict__ x, int x_f32, void* __restrict__ y, int y_f32,
                 const float* __restrict__ gamma, const float* __restrict__ beta, Shape sh, float eps, int act,
                 const float2* __restrict__ partial, float2* __restrict__ mean_rstd) {
  __shared__ float2 sm;
  const long long row = blockIdx.x / sh.S;
  const int s = blockIdx.x % sh.S;
  const int n = static_cast<int>(row / sh.C), c = static_cast<int>(row % sh.C);
  const int Cg = sh.C / sh.G, g = c / Cg;
  const float2 t = group_sum(partial, sh, n, g, &sm);
  const float cnt = static_cast<float>(Cg) * static_cast<float>(sh.hw);
  const float mean = t.x / cnt;
  const float var = fmaxf(t.y / cnt - mean * mean, 0.0f);
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0 && s == 0 && c == g * Cg && mean_rstd != nullptr)
    mean_rstd[n * sh.G + g] = make_float2(mean, rstd);
  const float ga = gamma != nullptr ? gamma[c] : 1.0f, be = beta != nullptr ? beta[c] : 0.0f;
  const float a = rstd * ga, b = be - mean * rstd * ga;
  const long long lo = s * sh.slice, hi = min(sh.hw, lo + sh.slice);
  const long long base = row * sh.hw;
  for (long long i = lo + static_cast<long long>(threadIdx.x) * V; i < hi; i += static_cast<long long>(blockDim.x) * V) {
    float f[V];
    ldv<V>(x, x_f32, base + i, f);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      f[j] = fmaf(f[j], a, b);
      if (act) f[j] = silu(f[j]);
    }
    stv<V>(y, y_f32, base + i, f);
  }
}

// Backward statistics: partial[n,c,s] = {sum dy', sum dy' * xhat}, dy' = dy * silu'(xhat*gamma+beta) when act.
template <int V> __global__ void __launch_bounds__(256)
stats_bwd_kernel(const void* __restrict__ dy, int dy_f32, const void* __restrict__ x, int x_f32,
                 const float* __restrict__ gamma, const float* __restrict__ beta, Shape sh, int act,
                 const float2* __restrict__ mean_rstd, float2* __restrict__ partial) {
  __shared__ float2 red[8];
  const long long row = blockIdx.x / sh.S;
  const int s = blockIdx.x % sh.S;
  const int n = static_cast<int>(row / sh.C), c = static_cast<int>(row % sh.C);
  const int g = c / (sh.C / sh.G);
  const float2 mr = mean_rstd[n * sh.G + g];
  const float ga = gamma != nullptr ? gamma[c] : 1.0f, be = beta != nullptr ? beta[c] : 0.0f;
  const long long lo = s * sh.slice, hi = min(sh.hw, lo + sh.slice);
  const long long base = row * sh.hw;
  float a = 0.f, b = 0.f;
  for (long long i = lo + static_cast<long long>(threadIdx.x) * V; i < hi; i += static_cast<long long>(blockDim.x) * V) {
    float fx[V], fd[V];
    ldv<V>(x, x_f32, base + i, fx);
    ldv<V>(dy, dy_f32, base + i, fd);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float xh = (fx[j] - mr.x) * mr.y;
      float d = fd[j];
      if (act) d *= dsilu(fmaf(xh, ga, be));
      a += d;
      b = fmaf(d, xh, b);
    }
  }
  const float2 t = block_sum2(a, b, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// dx = rstd * (gamma*dy' - mean_g(gamma*dy') - xhat * mean_g(gamma*dy'*xhat)); the group means are ordered sums of
// gamma[c] * partial[n, c, s].
template <int V> __global__ void __launch_bounds__(256)
apply_bwd_kernel(const void* __restrict__ dy, int dy_f32, const void* __restrict__ x, int x_f32,
                 void* __restrict__ dx, int dx_f32, const float* __restrict__ gamma, const float* __restrict__ beta,
                 Shape sh, int act, const float2* __restrict__ mean_rstd, const float2* __restrict__ partial) {
  __shared__ float2 sm;
  const long long row = blockIdx.x / sh.S;
  const int s = blockIdx.x % sh.S;
  const int n = static_cast<int>(row / sh.C), c = static_cast<int>(row % sh.C);
  const int Cg = sh.C / sh.G, g = c / Cg;
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    const float2* p = partial + (static_cast<long long>(n) * sh.C + g * Cg) * sh.S;
    for (int cc = 0; cc < Cg; ++cc) {
      const float gm = gamma != nullptr ? gamma[g * Cg + cc] : 1.0f;
      for (int k = 0; k < sh.S; ++k) {
        a = fmaf(gm, p[cc * sh.S + k].x, a);
        b = fmaf(gm, p[cc * sh.S + k].y, b);
      }
    }
    sm = make_float2(a, b);
  }
  __syncthreads();
  const float cnt = static_cast<float>(Cg) * static_cast<float>(sh.hw);
  const float m1 = sm.x / cnt, m2 = sm.y / cnt;
  const float2 mr = mean_rstd[n * sh.G + g];
  const float ga = gamma != nullptr ? gamma[c] : 1.0f, be = beta != nullptr ? beta[c] : 0.0f;
  const long long lo = s * sh.slice, hi = min(sh.hw, lo + sh.slice);
  const long long base = row * sh.hw;
  for (long long i = lo + static_cast<long long>(threadIdx.x) * V; i < hi; i += static_cast<long long>(blockDim.x) * V) {
    float fx[V], fd[V];
    ldv<V>(x, x_f32, base + i, fx);
    ldv<V>(dy, dy_f32, base + i, fd);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float xh = (fx[j] - mr.x) * mr.y;
      float d = fd[j];
      if (act) d *= dsilu(fmaf(xh, ga, be));
      fd[j] = mr.y * (ga * d - m1 - xh * m2);
    }
    stv<V>(dx, dx_f32, base + i, fd);
  }
}

inline Shape make_shape(int N, int C, int G, long long hw, int S) {
  Shape sh;
  sh.N = N; sh.C = C; sh.G = G; sh.S = S; sh.hw = hw;
  sh.slice = (((hw + S - 1) / S) + 7) / 8 * 8;  // slices start on 8-element boundaries (vector path)
  return sh;
}

inline bool vector_ok(long long hw, const void* a, const void* b, const void* c) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  return (hw & 7) == 0 && al(a) && al(b) && al(c);
}

}  // namespace gn
}  // namespace mdb

using namespace mdb;

// partial: [N*C*S] float2 scratch owned by the caller; mean_rstd: [N*G] float2 (saved for backward; may be null).
extern "C" int mdb_groupnorm_fwd(const void* x, int x_f32, void* y, int y_f32, const float* gamma, const float* beta,
                                 int N, int C, int G, long long hw, int S, float eps, int act, void* partial,
                                 void* mean_rstd, cudaStream_t stream) {
  if (N < 1 || C < 1 || G < 1 || C % G != 0 || hw < 1 || S < 1) return 1;
  const gn::Shape sh = gn::make_shape(N, C, G, hw, S);
  const long long blocks = static_cast<long long>(N) * C * S;
  if (blocks > 0x7fffffffLL) return 1;
  const bool vec = gn::vector_ok(hw, x, y, nullptr);
  if (vec) {
    gn::stats_fwd_kernel<8><<<static_cast<int>(blocks), 256, 0, stream>>>(x, x_f32, sh, static_cast<float2*>(partial));
    gn::apply_fwd_kernel<8><<<static_cast<int>(blocks), 256, 0, stream>>>(
        x, x_f32, y, y_f32, gamma, beta, sh, eps, act, static_cast<const float2*>(partial),
        static_cast<float2*>(mean_rstd));
  } else {
    gn::stats_fwd_kernel<1><<<static_cast<int>(blocks), 256, 0, stream>>>(x, x_f32, sh, static_cast<float2*>(partial));
    gn::apply_fwd_kernel<1><<<static_cast<int>(blocks), 256, 0, stream>>>(
        x, x_f32, y, y_f32, gamma, beta, sh, eps, act, static_cast<const float2*>(partial),
        static_cast<float2*>(mean_rstd));
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// partial receives {sum dy', sum dy'*xhat} per (n, c, s): the caller folds it into dbeta / dgamma.
extern "C" int mdb_groupnorm_bwd(const void* dy, int dy_f32, const void* x, int x_f32, void* dx, int dx_f32,
                                 const float* gamma, const float* beta, int N, int C, int G, long long hw, int S,
                                 int act, const void* mean_rstd, void* partial, cudaStream_t stream) {
  if (N < 1 || C < 1 || G < 1 || C % G != 0 || hw < 1 || S < 1) return 1;
  const gn::Shape sh = gn::make_shape(N, C, G, hw, S);
  const long long blocks = static_cast<long long>(N) * C * S;
  if (blocks > 0x7fffffffLL) return 1;
  const auto* mr = static_cast<const float2*>(mean_rstd);
  auto* pt = static_cast<float2*>(partial);
  if (gn::vector_ok(hw, x, dy, dx)) {
    gn::stats_bwd_kernel<8><<<static_cast<int>(blocks), 256, 0, stream>>>(dy, dy_f32, x, x_f32, gamma, beta, sh, act, mr, pt);
    gn::apply_bwd_kernel<8><<<static_cast<int>(blocks), 256, 0, stream>>>(dy, dy_f32, x, x_f32, dx, dx_f32, gamma, beta,
                                                                           sh, act, mr, pt);
  } else {
    gn::stats_bwd_kernel<1><<<static_cast<int>(blocks), 256, 0, stream>>>(dy, dy_f32, x, x_f32, gamma, beta, sh, act, mr, pt);
    gn::apply_bwd_kernel<1><<<static_cast<int>(blocks), 256, 0, stream>>>(dy, dy_f32, x, x_f32, dx, dx_f32, gamma, beta,
                                                                           sh, act, mr, pt);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
