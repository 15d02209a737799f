// Memory-bound row-wise kernels (one pass over HBM each): fp32 LayerNorm + AdaLN modulation,
// RMSNorm (+ rotary embedding), their backward passes with deterministic column reductions,
// GELU, gated residual, bias-gradient column sums.
//
// They stand in for the XLA fusions the reference relies on:
//   LayerNorm*(1+scale)+shift  src/maxdiffusion/models/wan/transformers/transformer_wan.py:486-489,519-522
//   gated residual             :499,526-528
//   RMSNorm + RoPE on q/k      src/maxdiffusion/models/attention_flax.py:2596-2620,2655-2677
//
// Shape convention: x is [rows, C] bf16 row-major, C a multiple of 8 and at most 8192. Each CTA
// (256 threads) walks a strip of rows; thread t owns the 8-element vectors t, t+256, ... of every
// row, so per-column partial sums live in registers for the whole strip and are written once per
// CTA to a scratch buffer [gridDim.x * gridDim.y, n_sums, C]; a second kernel folds the partials
// in a fixed order (bitwise reproducible).
#include "host_common.h"

namespace mdb {
namespace rw {

constexpr int THREADS = 256;
constexpr int MAXV = 4;  // vectors of 8 per thread -> C <= 8192

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16x2(w[j]);
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16x2(w[j]);
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
  uint4 v;
  v.x = pack_bf16x2(x[0], x[1]);
  v.y = pack_bf16x2(x[2], x[3]);
  v.z = pack_bf16x2(x[4], x[5]);
  v.w = pack_bf16x2(x[6], x[7]);
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ void loadf8(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void storef8(float* p, const float (&x)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over the CTA; every thread gets the result. `red` is 8 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += red[i];
  return t;
}
// The same with ONE barrier per call: the warp partials go to red[parity] and the parity flips on every call, so
// a warp that runs ahead into its next call writes the other half; it can reach the call after that only once
// every warp has passed the barrier in between, i.e. has finished reading this half. `red` is 2 x 8 float2.
__device__ __forceinline__ float2 block_sum2(float a, float b, float2 (*red)[THREADS / 32], int& parity) {
  a = warp_sum(a);
  b = warp_sum(b);
  if ((threadIdx.x & 31) == 0) red[parity][threadIdx.x >> 5] = make_float2(a, b);
  __syncthreads();
  float2 t = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) {
    t.x += red[parity][i].x;
    t.y += red[parity][i].y;
  }
  parity ^= 1;
  return t;
}
// Sum over aligned groups of 16 lanes (one 128-channel head).
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Strip {
  long long begin, end;  // rows of this CTA
  int batch;
};
// grid = (ctas_per_batch, num_batches); rows of one batch are contiguous.
__device__ __forceinline__ Strip my_strip(int rows_per_batch) {
  Strip s;
  const int per = (rows_per_batch + gridDim.x - 1) / gridDim.x;
  const long long base = static_cast<long long>(blockIdx.y) * rows_per_batch;
  const int b = min(rows_per_batch, static_cast<int>(blockIdx.x) * per);
  const int e = min(rows_per_batch, b + per);
  s.begin = base + b;
  s.end = base + e;
  s.batch = blockIdx.y;
  return s;
}

// ---------------------------------------------------------------------------------------
// LayerNorm (fp32 statistics) with optional affine (gamma, beta: bf16 [C]) and optional
// modulation (scale, shift: fp32 [num_batches, mod_ld]):  y = ((x-mean)*rstd*gamma+beta)*(1+scale)+shift
// ---------------------------------------------------------------------------------------
// Destination of a head-scattering store (the Ulysses all-to-all folded into the producer): n ranks, this rank's
// index, heads per rank, and every rank's receive buffer [B, n * S, hn, 128].
struct HeadScatter {
  int n, me, hn;
  __nv_bfloat16* base[8];
};

// NV = 16-byte vectors per thread (C <= NV*8*THREADS). Four CTAs fit on an SM, so a grid of 4 x 148 is one wave.
template <int NV>
__global__ void __launch_bounds__(THREADS, 4)
ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
              const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
              const float* __restrict__ scale, const float* __restrict__ shift, long long mod_ld, int rows_per_batch,
              int C, float eps, float* __restrict__ mean_out, float* __restrict__ rstd_out) {
  __shared__ float2 red[2][THREADS / 32];
  int parity = 0;
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  const float inv_c = 1.0f / C;
  for (long long row = s.begin; row < s.end; ++row) {
    float v[NV][8];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
        load8(x + row * C + vi * 8, v[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += v[k][j];
      }
    }
    const float mean = block_sum2(sum, 0.0f, red, parity).x * inv_c;
    float sq = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[k][j] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(block_sum2(sq, 0.0f, red, parity).x * inv_c + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mean) * rstd;
        if (gamma) {
          float g[8];
          load8(gamma + vi * 8, g);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] *= g[j];
        }
        if (beta) {
          float b[8];
          load8(beta + vi * 8, b);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += b[j];
        }
        if (scale) {
          float sc[8], sh[8];
          loadf8(scale + s.batch * mod_ld + vi * 8, sc);
          loadf8(shift + s.batch * mod_ld + vi * 8, sh);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = o[j] * (1.0f + sc[j]) + sh[j];
        }
        store8(y + row * C + vi * 8, o);
      }
    }
  }
}

// Backward of the above. Writes dx and per-CTA partial column sums
//   partial[cta][0][c] = sum_rows dy*xhat (-> dscale, or dgamma when affine)
//   partial[cta][1][c] = sum_rows dy      (-> dshift, or dbeta)
// (for the modulated form the first sum is taken after the affine, i.e. d/dscale of y).
// Between the two passes over a row a thread keeps only the packed bf16 inputs (the fp32 terms are recomputed),
// which together with the 2*NV*8 column accumulators leaves room for two CTAs per SM; the two row sums share
// one reduction with one barrier.
template <int NV>
__global__ void __launch_bounds__(THREADS, 2)
ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
              const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
              const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ scale, long long mod_ld,
              int rows_per_batch, int C, __nv_bfloat16* __restrict__ dx, float* __restrict__ partial) {
  __shared__ float2 red[2][THREADS / 32];
  int parity = 0;
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  const float inv_c = 1.0f / C;
  float acc0[NV][8], acc1[NV][8];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc0[k][j] = acc1[k][j] = 0.0f;

  // w = (1+scale)*gamma of a vector of 8 columns (re-read from L1 in both passes).
  auto weights = [&](int vi, float (&w)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = 1.0f;
    if (scale) {
      float sc[8];
      loadf8(scale + s.batch * mod_ld + vi * 8, sc);
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = 1.0f + sc[j];
    }
    if (gamma) {
      float gm[8];
      load8(gamma + vi * 8, gm);
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] *= gm[j];
    }
  };

  for (long long row = s.begin; row < s.end; ++row) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    uint4 rd[NV], rx[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
        rd[k] = *reinterpret_cast<const uint4*>(dy + row * C + vi * 8);
        rx[k] = *reinterpret_cast<const uint4*>(x + row * C + vi * 8);
      }
    }
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
        float d[8], xv[8], w[8];
        unpack8(rd[k], d);
        unpack8(rx[k], xv);
        weights(vi, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float g = d[j] * w[j];
          s1 += g;
          s2 += g * xh;
          acc0[k][j] += d[j] * xh;
          acc1[k][j] += d[j];
        }
      }
    }
    const float2 m = block_sum2(s1, s2, red, parity);
    const float m1 = m.x * inv_c, m2 = m.y * inv_c;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
        float d[8], xv[8], w[8], o[8];
        unpack8(rd[k], d);
        unpack8(rx[k], xv);
        weights(vi, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          o[j] = rstd * (d[j] * w[j] - m1 - xh * m2);
        }
        store8(dx + row * C + vi * 8, o);
      }
    }
  }
  if (partial) {
    const long long cta = static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) {
        storef8(partial + (cta * 2 + 0) * C + vi * 8, acc0[k]);
        storef8(partial + (cta * 2 + 1) * C + vi * 8, acc1[k]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Plain affine LayerNorm for rows of at most 2048 channels (UNet / DiT blocks of 320 .. 1280 channels): one warp
// per row instead of one CTA per row. A row of 1280 channels is 160 vectors, which leaves 96 of a CTA's 256 threads
// idle and pays two block barriers per row; with a warp per row the reductions are shuffles, eight rows of a CTA
// are in flight at once and nothing waits on a barrier. Same grid (strips of a batch's rows per CTA), same outputs
// and the same partial-sum layout as the CTA-per-row kernels, so the fold kernel and the callers do not change.
// ---------------------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(THREADS)
ln_rows_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                   const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta, int rows_per_batch,
                   int C, float eps, float* __restrict__ mean_out, float* __restrict__ rstd_out) {
  const Strip s = my_strip(rows_per_batch);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nvec = C >> 3;
  const float inv_c = 1.0f / C;
  for (long long row = s.begin + warp; row < s.end; row += THREADS / 32) {
    float v[VPL][8];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        load8(x + row * C + vi * 8, v[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += v[k][j];
      }
    }
    const float mean = warp_sum(sum) * inv_c;
    float sq = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      if (lane + k * 32 < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[k][j] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_c + eps);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        float g[8], b[8], o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 1.0f, b[j] = 0.0f;
        if (gamma) load8(gamma + vi * 8, g);
        if (beta) load8(beta + vi * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mean) * rstd * g[j] + b[j];
        store8(y + row * C + vi * 8, o);
      }
    }
    if (lane == 0 && mean_out) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(THREADS)
ln_rows_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ gamma, int rows_per_batch, int C, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ partial) {
  extern __shared__ float fold[];  // [2][C]: the CTA's column sums, added warp by warp in warp order
  const Strip s = my_strip(rows_per_batch);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nvec = C >> 3;
  const float inv_c = 1.0f / C;
  float acc0[VPL][8], acc1[VPL][8];
#pragma unroll
  for (int k = 0; k < VPL; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc0[k][j] = acc1[k][j] = 0.0f;
  for (long long row = s.begin + warp; row < s.end; row += THREADS / 32) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    uint4 rd[VPL], rx[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        rd[k] = *reinterpret_cast<const uint4*>(dy + row * C + vi * 8);
        rx[k] = *reinterpret_cast<const uint4*>(x + row * C + vi * 8);
      }
    }
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        float d[8], xv[8], g[8];
        unpack8(rd[k], d);
        unpack8(rx[k], xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 1.0f;
        if (gamma) load8(gamma + vi * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float gd = d[j] * g[j];
          s1 += gd;
          s2 += gd * xh;
          acc0[k][j] += d[j] * xh;
          acc1[k][j] += d[j];
        }
      }
    }
    const float m1 = warp_sum(s1) * inv_c, m2 = warp_sum(s2) * inv_c;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        float d[8], xv[8], g[8], o[8];
        unpack8(rd[k], d);
        unpack8(rx[k], xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 1.0f;
        if (gamma) load8(gamma + vi * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          o[j] = rstd * (d[j] * g[j] - m1 - xh * m2);
        }
        store8(dx + row * C + vi * 8, o);
      }
    }
  }
  if (partial) {
    for (int w = 0; w < THREADS / 32; ++w) {
      if (warp == w) {
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
          const int vi = lane + k * 32;
          if (vi < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = vi * 8 + j;
              fold[c] = (w == 0 ? 0.0f : fold[c]) + acc0[k][j];
              fold[C + c] = (w == 0 ? 0.0f : fold[C + c]) + acc1[k][j];
            }
          }
        }
      }
      __syncthreads();
    }
    const long long cta = static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x;
    for (int i = threadIdx.x; i < 2 * C; i += THREADS) partial[cta * 2 * C + i] = fold[i];
  }
}

// out[b][s][c] = sum over the CTAs of batch b of partial[cta][s][c]  (fixed order, hence reproducible).
// A block covers 32 columns; its 8 warps each sum every 8th partial (4 loads in flight per thread) and the 8
// slice sums are added in slice order through shared memory.
__global__ void __launch_bounds__(256) fold_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                            int ctas_per_batch, int n_sums, int C, int accumulate) {
  __shared__ float red[8][32];
  const int cx = threadIdx.x & 31, sy = threadIdx.x >> 5;
  const int idx = blockIdx.x * 32 + cx;  // over n_sums*C
  const int b = blockIdx.y;
  const int width = n_sums * C;
  float t = 0.0f;
  if (idx < width) {
    const float* src = partial + static_cast<long long>(b) * ctas_per_batch * width + idx;
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    int i = sy;
    for (; i + 24 < ctas_per_batch; i += 32) {
      a0 += src[static_cast<long long>(i) * width];
      a1 += src[static_cast<long long>(i + 8) * width];
      a2 += src[static_cast<long long>(i + 16) * width];
      a3 += src[static_cast<long long>(i + 24) * width];
    }
    for (; i < ctas_per_batch; i += 8) a0 += src[static_cast<long long>(i) * width];
    t = (a0 + a1) + (a2 + a3);
  }
  red[sy][cx] = t;
  __syncthreads();
  if (sy == 0 && idx < width) {
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += red[k][cx];
    float* o = out + static_cast<long long>(b) * width + idx;
    *o = accumulate ? (*o + tot) : tot;
  }
}

// ---------------------------------------------------------------------------------------
// RMSNorm over groups of `group` channels (group == C: across all heads; group == 128: per head),
// learned weight w [C or 128], followed by an optional rotary embedding on interleaved pairs of
// each 128-wide head: cos/sin are fp32 [rows_per_batch, 64].
// ---------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(THREADS, 4)
rms_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y, long long ldy,
                    const __nv_bfloat16* __restrict__ w, int w_per_head, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int rows_per_batch, int C, int group, float eps,
                    float* __restrict__ rstd_out, const HeadScatter sc) {
  __shared__ float2 red[2][THREADS / 32];
  int parity = 0;
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  for (long long row = s.begin; row < s.end; ++row) {
    const int pos = static_cast<int>(row - static_cast<long long>(s.batch) * rows_per_batch);
    float v[NV][8];
    float sq[NV];
    float total = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      sq[k] = 0.0f;
      if (vi < nvec) {
        load8(x + row * ldx + vi * 8, v[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) sq[k] += v[k][j] * v[k][j];
      }
      total += sq[k];
    }
    float rstd_all = 1.0f;  // group == 0: no normalisation (the value projection only changes layout)
    if (group == C) rstd_all = rsqrtf(block_sum2(total, 0.0f, red, parity).x / C + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      float rstd = rstd_all;
      if (group != C && group != 0) rstd = rsqrtf(half_warp_sum(sq[k]) / 128.0f + eps);  // all lanes take part
      if (vi < nvec) {
        if (rstd_out) {
          if (group == C) {
            if (threadIdx.x == 0 && k == 0) rstd_out[row] = rstd;
          } else if ((vi & 15) == 0) {
            rstd_out[row * (C >> 7) + (vi >> 4)] = rstd;
          }
        }
        float o[8];
        if (w) {
          float wv[8];
          load8(w + (w_per_head ? (vi & 15) * 8 : vi * 8), wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[k][j] * rstd * wv[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[k][j] * rstd;
        }
        if (cos_t) {
          const int pair0 = (vi & 15) * 4;  // 4 pairs per vector, 64 pairs per head
          const float4 cv = *reinterpret_cast<const float4*>(cos_t + static_cast<long long>(pos) * 64 + pair0);
          const float4 sv = *reinterpret_cast<const float4*>(sin_t + static_cast<long long>(pos) * 64 + pair0);
          const float c4[4] = {cv.x, cv.y, cv.z, cv.w};
          const float s4[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = o[2 * j], b = o[2 * j + 1];
            o[2 * j] = a * c4[j] - b * s4[j];
            o[2 * j + 1] = a * s4[j] + b * c4[j];
          }
        }
        if (sc.n > 0) {
          // Ulysses exchange folded into the store: head h goes to rank h / hn, where it is head h % hn of the
          // [B, n * S, hn, 128] tensor, at sequence position me * S + pos (16-byte peer stores over NVLink)
          const int head = vi >> 4;
          const int r = head / sc.hn;
          const long long drow = (static_cast<long long>(s.batch) * sc.n + sc.me) * rows_per_batch + pos;
          store8(sc.base[r] + (drow * sc.hn + (head - r * sc.hn)) * 128 + (vi & 15) * 8, o);
        } else {
          store8(y + row * ldy + vi * 8, o);
        }
      }
    }
  }
}

// Backward: dy is the gradient w.r.t. the rotated output. partial[cta][0][c] = sum_rows dyn*xhat
// (gradient of w before folding heads when w_per_head).
template <int NV>
__global__ void __launch_bounds__(THREADS, 2)
rms_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy, const __nv_bfloat16* __restrict__ x,
                    long long ldx, const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ w,
                    int w_per_head, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                    int rows_per_batch, int C, int group, __nv_bfloat16* __restrict__ dx, long long lddx,
                    float* __restrict__ partial) {
  __shared__ float2 red[2][THREADS / 32];
  int parity = 0;
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  float acc[NV][8];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[k][j] = 0.0f;

  for (long long row = s.begin; row < s.end; ++row) {
    const int pos = static_cast<int>(row - static_cast<long long>(s.batch) * rows_per_batch);
    float g[NV][8], xh[NV][8];
    float dot[NV];
    float total = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      dot[k] = 0.0f;
      if (vi < nvec) {
        float d[8], xv[8];
        load8(dy + row * lddy + vi * 8, d);
        load8(x + row * ldx + vi * 8, xv);
        if (cos_t) {
          const int pair0 = (vi & 15) * 4;
          const float4 cv = *reinterpret_cast<const float4*>(cos_t + static_cast<long long>(pos) * 64 + pair0);
          const float4 sv = *reinterpret_cast<const float4*>(sin_t + static_cast<long long>(pos) * 64 + pair0);
          const float c4[4] = {cv.x, cv.y, cv.z, cv.w};
          const float s4[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = d[2 * j], b = d[2 * j + 1];
            d[2 * j] = a * c4[j] + b * s4[j];
            d[2 * j + 1] = -a * s4[j] + b * c4[j];
          }
        }
        const float rstd = (group == C) ? rstd_in[row] : rstd_in[row * (C >> 7) + (vi >> 4)];
        float wv[8];
        if (w) {
          load8(w + (w_per_head ? (vi & 15) * 8 : vi * 8), wv);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[j] = 1.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] = xv[j] * rstd;
          g[k][j] = d[j] * wv[j];
          dot[k] += g[k][j] * xh[k][j];
          acc[k][j] += d[j] * xh[k][j];
          g[k][j] *= rstd;
        }
      }
      total += dot[k];
    }
    float mean_all = 0.0f;
    if (group == C) mean_all = block_sum2(total, 0.0f, red, parity).x / C;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      float mdot = mean_all;
      if (group != C) mdot = half_warp_sum(dot[k]) / 128.0f;
      if (vi < nvec) {
        const float rstd = (group == C) ? rstd_in[row] : rstd_in[row * (C >> 7) + (vi >> 4)];
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = g[k][j] - xh[k][j] * mdot * rstd;
        store8(dx + row * lddx + vi * 8, o);
      }
    }
  }
  if (partial) {
    const long long cta = static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = threadIdx.x + k * THREADS;
      if (vi < nvec) storef8(partial + cta * C + vi * 8, acc[k]);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Gated residual:  out = res + gate[b] * y   (gate fp32 [num_batches, gate_ld], may be nullptr -> 1)
// backward: dy = dout * gate ; partial[cta][0][c] = sum_rows dout * y (-> dgate)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
gated_res_fwd_kernel(const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ y,
                     const float* __restrict__ gate, long long gate_ld, int rows_per_batch, int C,
                     __nv_bfloat16* __restrict__ out) {
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  for (int k = 0; k < MAXV; ++k) {
    const int vi = threadIdx.x + k * THREADS;
    if (vi >= nvec) break;
    float g[8];
    if (gate) {
      loadf8(gate + s.batch * gate_ld + vi * 8, g);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 1.0f;
    }
    for (long long row = s.begin; row < s.end; ++row) {
      float r[8], v[8], o[8];
      load8(res + row * C + vi * 8, r);
      load8(y + row * C + vi * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = r[j] + g[j] * v[j];
      store8(out + row * C + vi * 8, o);
    }
  }
}

__global__ void __launch_bounds__(THREADS)
gated_res_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                     const float* __restrict__ gate, long long gate_ld, int rows_per_batch, int C,
                     __nv_bfloat16* __restrict__ dy, float* __restrict__ partial) {
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  const long long cta = static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x;
  for (int k = 0; k < MAXV; ++k) {
    const int vi = threadIdx.x + k * THREADS;
    if (vi >= nvec) break;
    float g[8], acc[8];
    loadf8(gate + s.batch * gate_ld + vi * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (long long row = s.begin; row < s.end; ++row) {
      float d[8], v[8], o[8];
      load8(dout + row * C + vi * 8, d);
      load8(y + row * C + vi * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = d[j] * g[j];
        acc[j] += d[j] * v[j];
      }
      store8(dy + row * C + vi * 8, o);
    }
    storef8(partial + cta * C + vi * 8, acc);
  }
}

// Column sums of a bf16 matrix (bias gradient): partial[cta][0][c] = sum_rows x
__global__ void __launch_bounds__(THREADS)
colsum_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int rows_per_batch, int C,
              float* __restrict__ partial) {
  const Strip s = my_strip(rows_per_batch);
  const int nvec = C >> 3;
  const long long cta = static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x;
  for (int vi = threadIdx.x; vi < nvec; vi += THREADS) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 4
    for (long long row = s.begin; row < s.end; ++row) {
      float v[8];
      load8(x + row * ldx + vi * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    storef8(partial + cta * C + vi * 8, acc);
  }
}

// ---------------------------------------------------------------------------------------
// Flat elementwise: GELU(tanh) forward / backward, SiLU-gate (a * silu(b)), plain add.
// ---------------------------------------------------------------------------------------
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ y, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v[8];
    load8(u + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
    store8(y + i * 8, v);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ u,
                                __nv_bfloat16* __restrict__ du, long long nvec) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float d[8], v[8], o[8];
    load8(dy + i * 8, d);
    load8(u + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x = v[j];
      const float t = tanhf(k0 * (x + k1 * x * x * x));
      const float dt = (1.0f - t * t) * k0 * (1.0f + 3.0f * k1 * x * x);
      o[j] = d[j] * (0.5f * (1.0f + t) + 0.5f * x * dt);
    }
    store8(du + i * 8, o);
  }
}

// GEGLU of the UNet feed-forward (reference: `FlaxGEGLU`, src/maxdiffusion/models/attention_flax.py:3537-3570):
// u [rows, 2 * inner] holds (h | gate) side by side; y = h * gelu(gate) with the exact (erf) GELU. One pass instead
// of slice + gelu + mul, and one pass for the backward: du = (dy * gelu(gate) | dy * h * gelu'(gate)).
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f)); }
__device__ __forceinline__ float gelu_erf_grad(float x) {
  return 0.5f * (1.0f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
__global__ void geglu_fwd_kernel(const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ y, long long rows,
                                 int inner_vecs) {
  const long long total = rows * inner_vecs;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / inner_vecs;
    const int c = static_cast<int>(i - r * inner_vecs);
    const __nv_bfloat16* row = u + r * inner_vecs * 16;
    float h[8], g[8];
    load8(row + c * 8, h);
    load8(row + (inner_vecs + c) * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] *= gelu_erf(g[j]);
    store8(y + i * 8, h);
  }
}
__global__ void geglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ u,
                                 __nv_bfloat16* __restrict__ du, long long rows, int inner_vecs) {
  const long long total = rows * inner_vecs;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / inner_vecs;
    const int c = static_cast<int>(i - r * inner_vecs);
    const long long off_h = r * inner_vecs * 16 + c * 8, off_g = off_h + inner_vecs * 8;
    float d[8], h[8], g[8], dh[8], dg[8];
    load8(dy + i * 8, d);
    load8(u + off_h, h);
    load8(u + off_g, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dh[j] = d[j] * gelu_erf(g[j]);
      dg[j] = d[j] * h[j] * gelu_erf_grad(g[j]);
    }
    store8(du + off_h, dh);
    store8(du + off_g, dg);
  }
}

}  // namespace rw
}  // namespace mdb

// ---------------------------------------------------------------------------------------
// C entry points. `ctas_per_batch` chooses the strip width; `scratch` must hold
// ctas_per_batch * num_batches * n_sums * C floats. Return 0 or a CUDA error code.
// ---------------------------------------------------------------------------------------
using namespace mdb;
using namespace mdb::rw;

static inline int check_c(int C) { return (C <= 0 || (C & 7) || C > THREADS * MAXV * 8) ? 3201 : 0; }
static inline int vectors_per_thread(int C) { return ((C >> 3) + THREADS - 1) / THREADS; }

extern "C" int mdb_ln_fwd(const void* x, void* y, const void* gamma, const void* beta, const float* scale,
                          const float* shift, long long mod_ld, int num_batches, int rows_per_batch, int C, float eps,
                          float* mean_out, float* rstd_out, int ctas_per_batch, void* stream) {
  if (int rc = check_c(C)) return rc;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  dim3 grid(ctas_per_batch, num_batches);
  if (scale == nullptr && shift == nullptr && C <= 2048) {  // plain affine, short rows: a warp per row
    const int vpl = ((C >> 3) + 31) / 32;
#define MDB_LN_ROWS_FWD(V)                                                                                          \
  ln_rows_fwd_kernel<V><<<grid, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(                                   \
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(gamma), \
      static_cast<const __nv_bfloat16*>(beta), rows_per_batch, C, eps, mean_out, rstd_out)
    if (vpl <= 1) MDB_LN_ROWS_FWD(1);
    else if (vpl == 2) MDB_LN_ROWS_FWD(2);
    else if (vpl <= 4) MDB_LN_ROWS_FWD(4);
    else if (vpl <= 5) MDB_LN_ROWS_FWD(5);
    else MDB_LN_ROWS_FWD(8);
#undef MDB_LN_ROWS_FWD
    return static_cast<int>(cudaGetLastError());
  }
#define MDB_LN_FWD(NV)                                                                                          \
  ln_fwd_kernel<NV><<<grid, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(                                   \
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(gamma), \
      static_cast<const __nv_bfloat16*>(beta), scale, shift, mod_ld, rows_per_batch, C, eps, mean_out, rstd_out)
  switch (vectors_per_thread(C)) {
    case 1: MDB_LN_FWD(1); break;
    case 2: MDB_LN_FWD(2); break;
    case 3: MDB_LN_FWD(3); break;
    default: MDB_LN_FWD(4); break;
  }
#undef MDB_LN_FWD
  return static_cast<int>(cudaGetLastError());
}

// out_sums: fp32 [num_batches, 2, C] (dscale/dshift per batch, or dgamma/dbeta with num_batches folded by caller)
extern "C" int mdb_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                          const float* scale, long long mod_ld, int num_batches, int rows_per_batch, int C, void* dx,
                          float* out_sums, float* scratch, int ctas_per_batch, void* stream) {
  if (int rc = check_c(C)) return rc;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(ctas_per_batch, num_batches);
  if (scale == nullptr && C <= 2048) {  // plain affine, short rows: a warp per row
    const int vpl = ((C >> 3) + 31) / 32;
    const size_t smem = out_sums ? 2 * static_cast<size_t>(C) * sizeof(float) : 0;
#define MDB_LN_ROWS_BWD(V)                                                                                        \
  ln_rows_bwd_kernel<V><<<grid, THREADS, smem, st>>>(static_cast<const __nv_bfloat16*>(dy),                       \
                                                     static_cast<const __nv_bfloat16*>(x), mean, rstd,             \
                                                     static_cast<const __nv_bfloat16*>(gamma), rows_per_batch, C,  \
                                                     static_cast<__nv_bfloat16*>(dx), out_sums ? scratch : nullptr)
    if (vpl <= 1) MDB_LN_ROWS_BWD(1);
    else if (vpl == 2) MDB_LN_ROWS_BWD(2);
    else if (vpl <= 4) MDB_LN_ROWS_BWD(4);
    else if (vpl <= 5) MDB_LN_ROWS_BWD(5);
    else MDB_LN_ROWS_BWD(8);
#undef MDB_LN_ROWS_BWD
    if (out_sums) {
      dim3 g2((2 * C + 31) / 32, num_batches);
      fold_partials_kernel<<<g2, 256, 0, st>>>(scratch, out_sums, ctas_per_batch, 2, C, 0);
    }
    return static_cast<int>(cudaGetLastError());
  }
#define MDB_LN_BWD(NV)                                                                                          \
  ln_bwd_kernel<NV><<<grid, THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(dy),                            \
                                              static_cast<const __nv_bfloat16*>(x), mean, rstd,                  \
                                              static_cast<const __nv_bfloat16*>(gamma), scale, mod_ld,           \
                                              rows_per_batch, C, static_cast<__nv_bfloat16*>(dx),                \
                                              out_sums ? scratch : nullptr)
  switch (vectors_per_thread(C)) {
    case 1: MDB_LN_BWD(1); break;
    case 2: MDB_LN_BWD(2); break;
    case 3: MDB_LN_BWD(3); break;
    default: MDB_LN_BWD(4); break;
  }
#undef MDB_LN_BWD
  if (out_sums) {
    dim3 g2((2 * C + 31) / 32, num_batches);
    fold_partials_kernel<<<g2, 256, 0, st>>>(scratch, out_sums, ctas_per_batch, 2, C, 0);
  }
  return static_cast<int>(cudaGetLastError());
}

static int launch_rms_rope_fwd(const void* x, long long ldx, void* y, long long ldy, const void* w, int w_per_head,
                               const float* cos_t, const float* sin_t, int num_batches, int rows_per_batch, int C, int group,
                               float eps, float* rstd_out, const mdb::rw::HeadScatter& sc, int ctas_per_batch, void* stream) {
  using namespace mdb::rw;
  dim3 grid(ctas_per_batch, num_batches);
#define MDB_RMS_FWD(NV)                                                                                 \
  rms_rope_fwd_kernel<NV><<<grid, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(                     \
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_bfloat16*>(y), ldy,                   \
      static_cast<const __nv_bfloat16*>(w), w_per_head, cos_t, sin_t, rows_per_batch, C, group, eps, rstd_out, sc)
  switch (vectors_per_thread(C)) {
    case 1: MDB_RMS_FWD(1); break;
    case 2: MDB_RMS_FWD(2); break;
    case 3: MDB_RMS_FWD(3); break;
    default: MDB_RMS_FWD(4); break;
  }
#undef MDB_RMS_FWD
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_rms_rope_fwd(const void* x, long long ldx, void* y, long long ldy, const void* w, int w_per_head,
                                const float* cos_t, const float* sin_t, int num_batches, int rows_per_batch, int C,
                                int group, float eps, float* rstd_out, int ctas_per_batch, void* stream) {
  if (int rc = check_c(C)) return rc;
  if ((group != C && group != 128) || (C & 127)) return 3202;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  HeadScatter sc;
  sc.n = 0; sc.me = 0; sc.hn = 1;
  for (int i = 0; i < 8; ++i) sc.base[i] = nullptr;
  return launch_rms_rope_fwd(x, ldx, y, ldy, w, w_per_head, cos_t, sin_t, num_batches, rows_per_batch, C, group, eps, rstd_out,
                             sc, ctas_per_batch, stream);
}

// The same kernel with the Ulysses head <-> sequence exchange folded into its stores: nothing is written locally; head
// h of row (b, s) goes to peer_ptrs[h / (H / n)], a [B, n * S, H / n, 128] buffer, at sequence position me * S + s.
// group = C (RMS over the row), 128 (per head) or 0 (no normalisation: the value projection). w / cos_t may be null.
extern "C" int mdb_rms_rope_fwd_scatter(const void* x, long long ldx, const void* w, int w_per_head, const float* cos_t,
                                        const float* sin_t, int num_batches, int rows_per_batch, int C, int group,
                                        float eps, const unsigned long long* peer_ptrs, int n, int me, int ctas_per_batch,
                                        void* stream) {
  if (int rc = check_c(C)) return rc;
  if ((group != C && group != 128 && group != 0) || (C & 127)) return 3202;
  const int heads = C >> 7;
  if (n < 1 || n > 8 || me < 0 || me >= n || heads % n != 0) return 3204;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  HeadScatter sc;
  sc.n = n; sc.me = me; sc.hn = heads / n;
  for (int i = 0; i < 8; ++i) sc.base[i] = i < n ? reinterpret_cast<__nv_bfloat16*>(peer_ptrs[i]) : nullptr;
  return launch_rms_rope_fwd(x, ldx, nullptr, 0, w, w_per_head, cos_t, sin_t, num_batches, rows_per_batch, C, group, eps,
                             nullptr, sc, ctas_per_batch, stream);
}

// dw_out: fp32 [C] summed over batches (accumulated over `num_batches` folds).
extern "C" int mdb_rms_rope_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* rstd,
                                const void* w, int w_per_head, const float* cos_t, const float* sin_t,
                                int num_batches, int rows_per_batch, int C, int group, void* dx, long long lddx,
                                float* dw_out, float* scratch, int ctas_per_batch, void* stream) {
  if (int rc = check_c(C)) return rc;
  if ((group != C && group != 128) || (C & 127)) return 3202;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(ctas_per_batch, num_batches);
#define MDB_RMS_BWD(NV)                                                                                 \
  rms_rope_bwd_kernel<NV><<<grid, THREADS, 0, st>>>(                                                    \
      static_cast<const __nv_bfloat16*>(dy), lddy, static_cast<const __nv_bfloat16*>(x), ldx, rstd,     \
      static_cast<const __nv_bfloat16*>(w), w_per_head, cos_t, sin_t, rows_per_batch, C, group,         \
      static_cast<__nv_bfloat16*>(dx), lddx, dw_out ? scratch : nullptr)
  switch (vectors_per_thread(C)) {
    case 1: MDB_RMS_BWD(1); break;
    case 2: MDB_RMS_BWD(2); break;
    case 3: MDB_RMS_BWD(3); break;
    default: MDB_RMS_BWD(4); break;
  }
#undef MDB_RMS_BWD
  if (dw_out) {
    // fold all CTAs of all batches into one [C] vector
    dim3 g2((C + 31) / 32, 1);
    fold_partials_kernel<<<g2, 256, 0, st>>>(scratch, dw_out, ctas_per_batch * num_batches, 1, C, 0);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_gated_res_fwd(const void* res, const void* y, const float* gate, long long gate_ld,
                                 int num_batches, int rows_per_batch, int C, void* out, int ctas_per_batch,
                                 void* stream) {
  if (int rc = check_c(C)) return rc;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  dim3 grid(ctas_per_batch, num_batches);
  gated_res_fwd_kernel<<<grid, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(y), gate, gate_ld, rows_per_batch, C,
      static_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

// dgate_out: fp32 [num_batches, C]
extern "C" int mdb_gated_res_bwd(const void* dout, const void* y, const float* gate, long long gate_ld,
                                 int num_batches, int rows_per_batch, int C, void* dy, float* dgate_out,
                                 float* scratch, int ctas_per_batch, void* stream) {
  if (int rc = check_c(C)) return rc;
  if (num_batches <= 0 || rows_per_batch <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(ctas_per_batch, num_batches);
  gated_res_bwd_kernel<<<grid, THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(dout),
                                                 static_cast<const __nv_bfloat16*>(y), gate, gate_ld, rows_per_batch,
                                                 C, static_cast<__nv_bfloat16*>(dy), scratch);
  dim3 g2((C + 31) / 32, num_batches);
  fold_partials_kernel<<<g2, 256, 0, st>>>(scratch, dgate_out, ctas_per_batch, 1, C, 0);
  return static_cast<int>(cudaGetLastError());
}

// out: fp32 [C] = column sums of x [rows, C] (leading dimension ldx)
extern "C" int mdb_colsum(const void* x, long long ldx, int rows, int C, float* out, float* scratch,
                          int ctas, void* stream) {
  if (C <= 0 || (C & 7)) return 3201;
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(ctas, 1);
  colsum_kernel<<<grid, THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows, C, scratch);
  dim3 g2((C + 31) / 32, 1);
  fold_partials_kernel<<<g2, 256, 0, st>>>(scratch, out, ctas, 1, C, 0);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_gelu_fwd(const void* u, void* y, long long n, void* stream) {
  if (n & 7) return 3203;
  if (n == 0) return 0;
  const long long nvec = n >> 3;
  const int blocks = static_cast<int>(nvec / 256 + 1 < 148 * 8 ? nvec / 256 + 1 : 148 * 8);
  gelu_fwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(u),
                                                                          static_cast<__nv_bfloat16*>(y), nvec);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int mdb_gelu_bwd(const void* dy, const void* u, void* du, long long n, void* stream) {
  if (n & 7) return 3203;
  if (n == 0) return 0;
  const long long nvec = n >> 3;
  const int blocks = static_cast<int>(nvec / 256 + 1 < 148 * 8 ? nvec / 256 + 1 : 148 * 8);
  gelu_bwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(du),
      nvec);
  return static_cast<int>(cudaGetLastError());
}

// u: bf16 [rows, 2 * inner] contiguous, inner a multiple of 8; y: [rows, inner]; du: like u.
extern "C" int mdb_geglu_fwd(const void* u, void* y, long long rows, int inner, void* stream) {
  if ((inner & 7) || inner <= 0) return 3204;
  if (rows <= 0) return 0;
  const long long total = rows * (inner >> 3);
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 8 ? total / 256 + 1 : 148 * 8);
  geglu_fwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(y), rows, inner >> 3);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int mdb_geglu_bwd(const void* dy, const void* u, void* du, long long rows, int inner, void* stream) {
  if ((inner & 7) || inner <= 0) return 3204;
  if (rows <= 0) return 0;
  const long long total = rows * (inner >> 3);
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 8 ? total / 256 + 1 : 148 * 8);
  geglu_bwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(du), rows,
      inner >> 3);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// Allocation-free column sums (declared and documented in no_alloc.h).
// ---------------------------------------------------------------------------------------
#include "no_alloc.h"

namespace {
// Scratch of the allocation-free entry point: one partial row per CTA. Device code may name the array directly;
// host code must not pass `g_colsum_scratch` to a kernel (in host code the name is only a stand-in for the
// symbol) and uses the address obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_colsum_scratch[MDB_COLSUM_NOALLOC_CTAS * MDB_COLSUM_NOALLOC_MAX_COLS];

constexpr int kNoAllocMaxDevices = 64;
float* g_colsum_scratch_addr[kNoAllocMaxDevices] = {nullptr};
}  // namespace

extern "C" const char* mdb_colsum_noalloc_strerror(int code) {
  switch (code) {
    case MDB_NOALLOC_OK: return "ok";
    case MDB_NOALLOC_ERR_TOO_WIDE: return "mdb_colsum_noalloc: more than 8192 columns do not fit the built-in scratch array";
    case MDB_NOALLOC_ERR_BAD_SHAPE: return "mdb_colsum_noalloc: cols must be a positive multiple of 8 and ldx >= cols";
    case MDB_NOALLOC_ERR_SETUP: return "mdb_colsum_noalloc: cudaGetSymbolAddress failed for the scratch array";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "mdb_colsum_noalloc: unknown code";
  }
}

extern "C" int mdb_colsum_noalloc(const void* x, long long ldx, int rows, int cols, float* out, void* stream) {
  if (cols > MDB_COLSUM_NOALLOC_MAX_COLS) return MDB_NOALLOC_ERR_TOO_WIDE;
  if (cols <= 0 || (cols & 7) || ldx < cols) return MDB_NOALLOC_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0) {
    // the sum over no rows is zero: the caller still gets a defined result
    return static_cast<int>(cudaMemsetAsync(out, 0, sizeof(float) * static_cast<size_t>(cols), st));
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return MDB_NOALLOC_ERR_SETUP;
  float* scratch = g_colsum_scratch_addr[dev];
  if (scratch == nullptr) {
    // set-up, once per device and with that device current: translate the symbol into its device address
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_colsum_scratch) != cudaSuccess || addr == nullptr) return MDB_NOALLOC_ERR_SETUP;
    scratch = static_cast<float*>(addr);
    g_colsum_scratch_addr[dev] = scratch;
  }
  const int ctas = rows < MDB_COLSUM_NOALLOC_CTAS ? rows : MDB_COLSUM_NOALLOC_CTAS;
  colsum_kernel<<<dim3(ctas, 1), THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows, cols, scratch);
  const cudaError_t first = cudaGetLastError();  // each launch is checked: the second must not hide the first
  if (first != cudaSuccess) return static_cast<int>(first);
  fold_partials_kernel<<<dim3((cols + 31) / 32, 1), 256, 0, st>>>(scratch, out, ctas, 1, cols, 0);
  return static_cast<int>(cudaGetLastError());
}
