// Optimizer-side streaming kernels over flat parameter buffers: fused AdamW on a (sharded)
// flat buffer, gradient sum-of-squares / max-abs reduction, scaled accumulate.
//
// Reference behaviour: optax.adamw with optional global-norm / value clipping
// (src/maxdiffusion/max_utils.py:683-696) and the gradient metrics of the Wan trainer
// (src/maxdiffusion/trainers/wan_trainer.py:169-189).
#include "host_common.h"

namespace mdb {
namespace opt {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return static_cast<uint32_t>(x);
}
// fp32 -> bf16 with stochastic rounding (unbiased for updates far below one ulp).
__device__ __forceinline__ __nv_bfloat16 stochastic_bf16(float v, uint32_t rnd) {
  uint32_t bits = __float_as_uint(v);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16_rn(v);
  bits += rnd & 0xffffu;
  return __ushort_as_bfloat16(static_cast<unsigned short>(bits >> 16));
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, grad_scale, clip_value;
  unsigned long long seed;
  int stochastic;
};

template <typename GT, typename ST>
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, const GT* __restrict__ g, ST* __restrict__ m,
                             ST* __restrict__ v, long long n, AdamArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float gi = to_f<GT>(g[i]) * a.grad_scale;
    if (a.clip_value > 0.0f) gi = fminf(fmaxf(gi, -a.clip_value), a.clip_value);
    const float mi = a.b1 * to_f<ST>(m[i]) + (1.0f - a.b1) * gi;
    const float vi = a.b2 * to_f<ST>(v[i]) + (1.0f - a.b2) * gi * gi;
    m[i] = from_f<ST>(mi);
    v[i] = from_f<ST>(vi);
    const float mhat = mi / a.bc1;
    const float vhat = vi / a.bc2;
    float w = __bfloat162float(p[i]);
    w -= a.lr * (mhat / (sqrtf(vhat) + a.eps) + a.wd * w);
    p[i] = a.stochastic ? stochastic_bf16(w, hash32(a.seed + static_cast<uint64_t>(i))) : __float2bfloat16_rn(w);
  }
}

// All-bf16 variant, 8 elements per thread through 16-byte loads and stores (the scalar kernel moves 2 bytes per
// access and reaches about a third of the copy bandwidth). n8 = n / 8; the host runs the scalar kernel on the tail.
__global__ void __launch_bounds__(256) adamw_bf16x8_kernel(uint4* __restrict__ p, const uint4* __restrict__ g,
                                                           uint4* __restrict__ m, uint4* __restrict__ v, long long n8,
                                                           AdamArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 pv = p[i], gv = g[i], mv = m[i], vv = v[i];
    const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
    uint32_t po[4], mo[4], vo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 pf = unpack_bf16x2(pw[e]), gf = unpack_bf16x2(gw[e]), mf = unpack_bf16x2(mw[e]), vf = unpack_bf16x2(vw[e]);
      float w2[2], m2[2], v2[2];
      const float pin[2] = {pf.x, pf.y}, gin[2] = {gf.x, gf.y}, min_[2] = {mf.x, mf.y}, vin[2] = {vf.x, vf.y};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float gi = gin[h] * a.grad_scale;
        if (a.clip_value > 0.0f) gi = fminf(fmaxf(gi, -a.clip_value), a.clip_value);
        const float mi = a.b1 * min_[h] + (1.0f - a.b1) * gi;
        const float vi = a.b2 * vin[h] + (1.0f - a.b2) * gi * gi;
        // the moments are stored in bf16: the update uses the stored values' fp32 originals, as the scalar kernel does
        m2[h] = mi;
        v2[h] = vi;
        float w = pin[h];
        w -= a.lr * ((mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps) + a.wd * w);  // same arithmetic as the scalar kernel
        w2[h] = w;
      }
      mo[e] = pack_bf16x2(m2[0], m2[1]);
      vo[e] = pack_bf16x2(v2[0], v2[1]);
      if (a.stochastic) {
        const uint64_t idx = static_cast<uint64_t>(i) * 8 + 2 * e;
        const __nv_bfloat16 lo = stochastic_bf16(w2[0], hash32(a.seed + idx));
        const __nv_bfloat16 hi = stochastic_bf16(w2[1], hash32(a.seed + idx + 1));
        po[e] = static_cast<uint32_t>(__bfloat16_as_ushort(lo)) | (static_cast<uint32_t>(__bfloat16_as_ushort(hi)) << 16);
      } else {
        po[e] = pack_bf16x2(w2[0], w2[1]);
      }
    }
    p[i] = make_uint4(po[0], po[1], po[2], po[3]);
    m[i] = make_uint4(mo[0], mo[1], mo[2], mo[3]);
    v[i] = make_uint4(vo[0], vo[1], vo[2], vo[3]);
  }
}

// partial[block] = {sum x^2, max |x|}
template <typename T>
__global__ void sumsq_maxabs_kernel(const T* __restrict__ x, long long n, float2* __restrict__ partial) {
  float s = 0.0f, mx = 0.0f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = to_f<T>(x[i]);
    s += v * v;
    mx = fmaxf(mx, fabsf(v));
  }
  __shared__ float ss[32], sm[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0) { ss[threadIdx.x >> 5] = s; sm[threadIdx.x >> 5] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ts = 0.0f, tm = 0.0f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) { ts += ss[i]; tm = fmaxf(tm, sm[i]); }
    partial[blockIdx.x] = make_float2(ts, tm);
  }
}
// out[0] += sum, out[1] = max(out[1], max)  -- single thread block, fixed order
__global__ void fold_sumsq_kernel(const float2* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float ts = 0.0f, tm = 0.0f;
    for (int i = 0; i < n; ++i) { ts += partial[i].x; tm = fmaxf(tm, partial[i].y); }
    if (accumulate) { out[0] += ts; out[1] = fmaxf(out[1], tm); } else { out[0] = ts; out[1] = tm; }
  }
}

}  // namespace opt
}  // namespace mdb

using namespace mdb::opt;

// p: bf16 [n]; g: bf16 (g_f32=0) or fp32; m, v: bf16 (state_f32=0) or fp32. bc1 = 1-b1^t, bc2 = 1-b2^t.
extern "C" int mdb_adamw(void* p, const void* g, void* m, void* v, long long n, float lr, float b1, float b2,
                         float eps, float wd, float bc1, float bc2, float grad_scale, float clip_value,
                         unsigned long long seed, int stochastic, int g_f32, int state_f32, void* stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, b1, b2, eps, wd, bc1, bc2, grad_scale, clip_value, seed, stochastic};
  const int blocks = static_cast<int>((n + 1023) / 1024 < 148 * 16 ? (n + 1023) / 1024 : 148 * 16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* pp = static_cast<__nv_bfloat16*>(p);
  if (g_f32 && state_f32)
    adamw_kernel<float, float><<<blocks, 256, 0, st>>>(pp, static_cast<const float*>(g), static_cast<float*>(m),
                                                       static_cast<float*>(v), n, a);
  else if (g_f32)
    adamw_kernel<float, __nv_bfloat16><<<blocks, 256, 0, st>>>(pp, static_cast<const float*>(g),
                                                               static_cast<__nv_bfloat16*>(m),
                                                               static_cast<__nv_bfloat16*>(v), n, a);
  else if (state_f32)
    adamw_kernel<__nv_bfloat16, float><<<blocks, 256, 0, st>>>(pp, static_cast<const __nv_bfloat16*>(g),
                                                               static_cast<float*>(m), static_cast<float*>(v), n, a);
  else {
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                           reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    const long long n8 = aligned ? n / 8 : 0;
    if (n8 > 0) {
      const int vb = static_cast<int>((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
      adamw_bf16x8_kernel<<<vb, 256, 0, st>>>(static_cast<uint4*>(p), static_cast<const uint4*>(g), static_cast<uint4*>(m),
                                              static_cast<uint4*>(v), n8, a);
    }
    const long long done = n8 * 8;
    if (done < n) {  // tail (or everything when a pointer is not 16-byte aligned); the hash index continues at `done`
      AdamArgs t = a;
      t.seed = a.seed + static_cast<unsigned long long>(done);
      const long long rest = n - done;
      const int tb = static_cast<int>((rest + 1023) / 1024 < 148 * 16 ? (rest + 1023) / 1024 : 148 * 16);
      adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<tb, 256, 0, st>>>(
          pp + done, static_cast<const __nv_bfloat16*>(g) + done, static_cast<__nv_bfloat16*>(m) + done,
          static_cast<__nv_bfloat16*>(v) + done, rest, t);
    }
  }
  return static_cast<int>(cudaGetLastError());
}

// out: fp32 [2] = {sum of squares, max abs}; scratch: 2 * 1024 floats. accumulate != 0 adds to / maxes with out.
extern "C" int mdb_sumsq_maxabs(const void* x, long long n, int is_f32, float* out, float* scratch, int accumulate,
                                void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = static_cast<int>((n + 2047) / 2048 < 1024 ? (n + 2047) / 2048 : 1024);
  float2* part = reinterpret_cast<float2*>(scratch);
  if (is_f32)
    sumsq_maxabs_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), n, part);
  else
    sumsq_maxabs_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, part);
  fold_sumsq_kernel<<<1, 32, 0, st>>>(part, blocks, out, accumulate);
  return static_cast<int>(cudaGetLastError());
}
