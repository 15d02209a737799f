// Streaming elementwise kernels of the sampling / training step (memory-bound; 16-byte vectors,
// grid sized to the SM count). One templated family covers what the reference leaves to XLA fusions:
//
//   lincomb        : out = sum_i c[b][i] * x_i   (up to 6 inputs, bf16 or f32 each, per-sample coefficients).
//                    Classifier-free-guidance combine, Euler / UniPC predictor-corrector updates with
//                    host-computed coefficients, flow-match noising, residual-cache add/sub, STG blend.
//                    Optionally emits per-block sum(out^2) partials (residual-cache relative-L1/L2 tests).
//                    reference: src/maxdiffusion/pipelines/wan/wan_pipeline.py:1314-1369 (CFG inside the jitted
//                    forward), src/maxdiffusion/schedulers/scheduling_unipc_multistep_flax.py:332-623.
//   mse_fwd_bwd    : loss partials of sum_b w_b * (pred - target)^2 and d(pred) in the same pass
//                    (reference: src/maxdiffusion/trainers/wan_trainer.py:136-189 computes the loss and lets
//                    autodiff produce the gradient in separate fusions).
//   channel_affine : out = (x - mean[c]) * scale[c] or x * scale[c] + mean[c] (latent normalise / de-normalise,
//                    reference: src/maxdiffusion/models/wan/autoencoder_kl_wan.py:1022-1057).
//   to_uint8       : clamp(x * 0.5 + 0.5, 0, 1) * 255 -> uint8 (video post-process).
//   blend_ramp     : linear cross-fade of two tiles along one axis (tiled VAE decode,
//                    reference: src/maxdiffusion/models/ltx2/autoencoder_kl_ltx2.py:1292-1368).
#include "host_common.h"

namespace mdb {
namespace ew {

constexpr int MAX_IN = 6;
constexpr int MAX_B = 16;

struct LinArgs {
  const void* x[MAX_IN];
  int is_f32[MAX_IN];
  float c[MAX_B][MAX_IN];
  int n_in;
  long long per_batch;  // elements per sample (multiple of 8)
};

__device__ __forceinline__ void load8(const void* base, int is_f32, long long vec, float (&f)[8]) {
  if (is_f32) {
    const float4* p = reinterpret_cast<const float4*>(base) + vec * 2;
    float4 a = p[0], b = p[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    uint4 u = reinterpret_cast<const uint4*>(base)[vec];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
  }
}

__device__ __forceinline__ void store8(void* base, int is_f32, long long vec, const float (&f)[8]) {
  if (is_f32) {
    float4* p = reinterpret_cast<float4*>(base) + vec * 2;
    p[0] = make_float4(f[0], f[1], f[2], f[3]);
    p[1] = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    reinterpret_cast<uint4*>(base)[vec] = u;
  }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.0f;
  if (w == 0) {
    t = l < (blockDim.x >> 5) ? red[l] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  __syncthreads();
  return t;  // valid in warp 0
}

__global__ void __launch_bounds__(256)
lincomb_kernel(LinArgs a, void* __restrict__ out, int out_f32, long long nvec, float* __restrict__ sumsq_partial) {
  __shared__ float red[8];
  const long long vec_per_batch = a.per_batch >> 3;
  float sq = 0.0f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(i / vec_per_batch);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < MAX_IN; ++k) {
      if (k < a.n_in) {
        float f[8];
        load8(a.x[k], a.is_f32[k], i, f);
        const float c = a.c[b][k];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(c, f[j], acc[j]);
      }
    }
    store8(out, out_f32, i, acc);
#pragma unroll
    for (int j = 0; j < 8; ++j) sq = fmaf(acc[j], acc[j], sq);
  }
  if (sumsq_partial != nullptr) {
    const float t = block_sum(sq, red);
    if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = t;
  }
}

// partial[block] = sum over the block's elements of w[b] * (pred - target)^2; dpred = gscale * w[b] * (pred - target).
struct MseArgs {
  float w[MAX_B];
  long long per_batch;
};
__global__ void __launch_bounds__(256)
mse_kernel(const void* __restrict__ pred, int pred_f32, const void* __restrict__ target, int target_f32,
           void* __restrict__ dpred, int dpred_f32, MseArgs a, float gscale, long long nvec,
           float* __restrict__ partial) {
  __shared__ float red[8];
  const long long vec_per_batch = a.per_batch >> 3;
  float acc = 0.0f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float w = a.w[static_cast<int>(i / vec_per_batch)];
    float p[8], t[8], d[8];
    load8(pred, pred_f32, i, p);
    load8(target, target_f32, i, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float e = p[j] - t[j];
      acc = fmaf(w * e, e, acc);
      d[j] = gscale * w * e;
    }
    if (dpred != nullptr) store8(dpred, dpred_f32, i, d);
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// element i belongs to channel (i / inner) % C
__global__ void __launch_bounds__(256)
channel_affine_kernel(const void* __restrict__ x, int x_f32, void* __restrict__ out, int out_f32,
                      const float* __restrict__ mean, const float* __restrict__ scale, int C, long long inner,
                      int denorm, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>((i / inner) % C);
    const float v = x_f32 ? reinterpret_cast<const float*>(x)[i]
                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    const float r = denorm ? fmaf(v, scale[c], mean[c]) : (v - mean[c]) * scale[c];
    if (out_f32) reinterpret_cast<float*>(out)[i] = r;
    else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(r);
  }
}

__global__ void __launch_bounds__(256)
to_uint8_kernel(const void* __restrict__ x, int x_f32, unsigned char* __restrict__ out, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8];
    load8(x, x_f32, i, f);
    unsigned int lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= static_cast<unsigned int>(__float2uint_rn(__saturatef(fmaf(f[j], 0.5f, 0.5f)) * 255.0f)) << (8 * j);
      hi |= static_cast<unsigned int>(__float2uint_rn(__saturatef(fmaf(f[j + 4], 0.5f, 0.5f)) * 255.0f)) << (8 * j);
    }
    reinterpret_cast<uint2*>(out)[i] = make_uint2(lo, hi);
  }
}

// out[o, e, i] = a[o, e, i] * (1 - e / extent) + b[o, e, i] * (e / extent); tensors are [outer, extent, inner]
__global__ void __launch_bounds__(256)
blend_ramp_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out, int is_f32,
                  long long a_outer_stride, long long b_outer_stride, long long o_outer_stride,
                  long long a_ext_stride, long long b_ext_stride, long long o_ext_stride, int extent, long long inner,
                  long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long in = i % inner;
    const long long e = (i / inner) % extent;
    const long long o = i / (inner * extent);
    const float w = static_cast<float>(e) / static_cast<float>(extent);
    const long long ia = o * a_outer_stride + e * a_ext_stride + in;
    const long long ib = o * b_outer_stride + e * b_ext_stride + in;
    const long long io = o * o_outer_stride + e * o_ext_stride + in;
    if (is_f32) {
      const float va = reinterpret_cast<const float*>(a)[ia], vb = reinterpret_cast<const float*>(b)[ib];
      reinterpret_cast<float*>(out)[io] = va * (1.0f - w) + vb * w;
    } else {
      const float va = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a)[ia]);
      const float vb = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[ib]);
      reinterpret_cast<__nv_bfloat16*>(out)[io] = __float2bfloat16_rn(va * (1.0f - w) + vb * w);
    }
  }
}

inline int grid_for(long long work, int per_block, int cap_blocks) {
  long long g = (work + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > cap_blocks) g = cap_blocks;
  return static_cast<int>(g);
}

}  // namespace ew
}  // namespace mdb

using namespace mdb;

// coefs: host array [batch][n_in]; n = batch * per_batch elements, per_batch a multiple of 8.
// sumsq_partial (optional): `partial_blocks` floats; the launch uses exactly that many blocks.
extern "C" int mdb_lincomb(void* out, int out_f32, int n_in, const void* const* xs, const int* is_f32,
                           const float* coefs, int batch, long long per_batch, float* sumsq_partial,
                           int partial_blocks, cudaStream_t stream) {
  if (n_in < 1 || n_in > ew::MAX_IN || batch < 1 || batch > ew::MAX_B || (per_batch & 7) != 0) return 1;
  ew::LinArgs a{};
  a.n_in = n_in;
  a.per_batch = per_batch;
  for (int k = 0; k < n_in; ++k) {
    a.x[k] = xs[k];
    a.is_f32[k] = is_f32[k];
    for (int b = 0; b < batch; ++b) a.c[b][k] = coefs[b * n_in + k];
  }
  const long long nvec = batch * per_batch / 8;
  const int grid = sumsq_partial != nullptr ? partial_blocks : ew::grid_for(nvec, 256 * 4, sm_count() * 8);
  ew::lincomb_kernel<<<grid, 256, 0, stream>>>(a, out, out_f32, nvec, sumsq_partial);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int mdb_mse_fwd_bwd(const void* pred, int pred_f32, const void* target, int target_f32, void* dpred,
                               int dpred_f32, const float* weights, int batch, long long per_batch, float gscale,
                               float* partial, int partial_blocks, cudaStream_t stream) {
  if (batch < 1 || batch > ew::MAX_B || (per_batch & 7) != 0 || partial_blocks < 1) return 1;
  ew::MseArgs a{};
  a.per_batch = per_batch;
  for (int b = 0; b < batch; ++b) a.w[b] = weights[b];
  ew::mse_kernel<<<partial_blocks, 256, 0, stream>>>(pred, pred_f32, target, target_f32, dpred, dpred_f32, a, gscale,
                                                     batch * per_batch / 8, partial);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int mdb_channel_affine(const void* x, int x_f32, void* out, int out_f32, const float* mean,
                                  const float* scale, int C, long long inner, int denorm, long long n,
                                  cudaStream_t stream) {
  if (C < 1 || inner < 1) return 1;
  ew::channel_affine_kernel<<<ew::grid_for(n, 256 * 8, sm_count() * 8), 256, 0, stream>>>(x, x_f32, out, out_f32, mean,
                                                                                        scale, C, inner, denorm, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int mdb_to_uint8(const void* x, int x_f32, unsigned char* out, long long n, cudaStream_t stream) {
  if ((n & 7) != 0) return 1;
  ew::to_uint8_kernel<<<ew::grid_for(n / 8, 256 * 4, sm_count() * 8), 256, 0, stream>>>(x, x_f32, out, n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int mdb_blend_ramp(const void* a, const void* b, void* out, int is_f32, long long outer,
                              const long long* strides6, int extent, long long inner, cudaStream_t stream) {
  if (extent < 1 || inner < 1 || outer < 1) return 1;
  const long long n = outer * extent * inner;
  ew::blend_ramp_kernel<<<ew::grid_for(n, 256 * 8, sm_count() * 8), 256, 0, stream>>>(
      a, b, out, is_f32, strides6[0], strides6[1], strides6[2], strides6[3], strides6[4], strides6[5], extent, inner, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
