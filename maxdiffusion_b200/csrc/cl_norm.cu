// Row kernels for channels-last activations [rows, C] (a row is one pixel / voxel):
//   rms_act : y = act( x / max(||x||_2, eps) * sqrt(C) * gamma + beta ),  act = identity or SiLU
// This is the `WanRMS_norm` + SiLU that precedes every convolution of the Wan VAE's residual blocks
// (src/maxdiffusion/models/wan/autoencoder_kl_wan.py:150-183, 452-484): memory bound, one read and one write of the
// activation. A row of C channels (16 .. 1024) is handled by a group of G = 2 .. 32 lanes, each lane holding VPL
// 16-byte vectors, with G * VPL equal to the row's vector count wherever it factors that way (96 channels = 12
// vectors = 4 lanes x 3, 384 = 16 x 3, 320 = 8 x 5), so that no lane of a warp is idle; the sum of squares is
// reduced with shuffles inside the group, statistics in fp32.
#include "host_common.h"

namespace mdb {
namespace cln {

constexpr int MAX_VPL = 5;  // vectors (8 bf16) per lane

// R rows per group and iteration are loaded before any of them is reduced: a memory-bound kernel needs tens of
// kilobytes in flight per SM, and one 16-byte load per thread is not enough of them.
template <int G, int VPL, int R>
__global__ void __launch_bounds__(256)
rms_act_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y, long long ldy,
               const float* __restrict__ gamma, const float* __restrict__ beta, long long rows, int C, float eps,
               int act, int out_w, int out_halo) {
  const int vecs = C >> 3;
  const int lane_in_group = threadIdx.x % G;
  const long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  const long long n_groups = static_cast<long long>(gridDim.x) * blockDim.x / G;
  const float scale = sqrtf(static_cast<float>(C));
  // every lane of a warp runs the same number of iterations (the shuffles below name all 32 lanes)
  const long long iters = (rows + n_groups * R - 1) / (n_groups * R);
  for (long long it = 0; it < iters; ++it) {
    uint4 v[R][VPL];
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long long row = group + (it * R + r) * n_groups;
      ss[r] = 0.0f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int vi = lane_in_group + i * G;
        if (row < rows && vi < vecs) v[r][i] = *reinterpret_cast<const uint4*>(x + row * ldx + vi * 8);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long long row = group + (it * R + r) * n_groups;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int vi = lane_in_group + i * G;
        if (row < rows && vi < vecs) {
          const uint32_t w[4] = {v[r][i].x, v[r][i].y, v[r][i].z, v[r][i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(w[j]);
            ss[r] += f.x * f.x + f.y * f.y;
          }
        }
      }
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], o);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long long row = group + (it * R + r) * n_groups;
      const float inv = scale / fmaxf(sqrtf(ss[r]), eps);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int vi = lane_in_group + i * G;
        if (row < rows && vi < vecs) {
          const uint32_t w[4] = {v[r][i].x, v[r][i].y, v[r][i].z, v[r][i].w};
          float o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(w[j]);
            o[2 * j] = f.x * inv;
            o[2 * j + 1] = f.y * inv;
          }
          const float4 g0 = *reinterpret_cast<const float4*>(gamma + vi * 8);
          const float4 g1 = *reinterpret_cast<const float4*>(gamma + vi * 8 + 4);
          o[0] *= g0.x; o[1] *= g0.y; o[2] *= g0.z; o[3] *= g0.w;
          o[4] *= g1.x; o[5] *= g1.y; o[6] *= g1.z; o[7] *= g1.w;
          if (beta != nullptr) {
            const float4 b0 = *reinterpret_cast<const float4*>(beta + vi * 8);
            const float4 b1 = *reinterpret_cast<const float4*>(beta + vi * 8 + 4);
            o[0] += b0.x; o[1] += b0.y; o[2] += b0.z; o[3] += b0.w;
            o[4] += b1.x; o[5] += b1.y; o[6] += b1.z; o[7] += b1.w;
          }
          if (act) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = o[j] / (1.0f + __expf(-o[j]));
          }
          uint4 ov;
          ov.x = pack_bf16x2(o[0], o[1]);
          ov.y = pack_bf16x2(o[2], o[3]);
          ov.z = pack_bf16x2(o[4], o[5]);
          ov.w = pack_bf16x2(o[6], o[7]);
          // out_w > 0: the output is the interior of a tensor whose width axis carries out_halo extra columns per side
          const long long yrow = out_w > 0 ? (row / out_w) * (out_w + 2 * out_halo) + out_halo + row % out_w : row;
          *reinterpret_cast<uint4*>(y + yrow * ldy + vi * 8) = ov;
        }
      }
    }
  }
}

}  // namespace cln
}  // namespace mdb

// x, y: bf16 [rows, C] with leading dimensions ldx / ldy (elements, multiples of 8); gamma / beta: fp32 [C]
// (beta may be null); C a multiple of 8, at most 1024. act: 0 identity, 1 SiLU. out_w > 0: x is [.., out_w, C] and y
// is the interior of a [.., out_w + 2 out_halo, C] tensor (y points at its first row, halo column included).
extern "C" int mdb_rms_act_cl(const void* x, long long ldx, void* y, long long ldy, const float* gamma,
                              const float* beta, long long rows, int C, float eps, int act, int out_w, int out_halo,
                              void* stream) {
  using namespace mdb::cln;
  if (rows <= 0) return 0;
  if ((C & 7) || C <= 0 || C > 8 * 32 * MAX_VPL || (ldx & 7) || (ldy & 7) || gamma == nullptr || out_halo < 0 ||
      (out_w > 0 && rows % out_w))
    return 3701;
  const int vecs = C >> 3;
  // widest group whose lanes are all busy; rows that do not factor fall back to a full warp with a ragged last pass
  int G = 0, vpl = 0;
  for (int g = 32; g >= 2 && G == 0; g >>= 1)
    if (vecs % g == 0 && vecs / g <= MAX_VPL && (vecs / g == 1 || vecs / g == 3 || vecs / g == 5 || g == 32)) G = g, vpl = vecs / g;
  if (G == 0) {
    G = vecs <= 8 ? 8 : (vecs <= 16 ? 16 : 32);
    vpl = (vecs + G - 1) / G;
  }
  const int R = vpl <= 2 ? 4 : (vpl <= 4 ? 2 : 1);
  const long long groups_per_block = 256 / G;
  long long blocks = (rows + groups_per_block * R - 1) / (groups_per_block * R);
  const long long cap = static_cast<long long>(mdb::sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  const int nb = static_cast<int>(blocks);
#define MDB_RMS_ACT(GG, VV, RR) \
  rms_act_kernel<GG, VV, RR><<<nb, 256, 0, st>>>(xp, ldx, yp, ldy, gamma, beta, rows, C, eps, act, out_w, out_halo)
#define MDB_RMS_ACT_G(GG)                         \
  if (G == GG) {                                  \
    if (vpl == 1) MDB_RMS_ACT(GG, 1, 4);          \
    else if (vpl == 3) MDB_RMS_ACT(GG, 3, 2);     \
    else if (vpl == 5) MDB_RMS_ACT(GG, 5, 1);     \
    else return 3701;                             \
  }
  if (G == 32) {
    if (vpl == 1) MDB_RMS_ACT(32, 1, 4);
    else if (vpl == 2) MDB_RMS_ACT(32, 2, 4);
    else if (vpl == 3) MDB_RMS_ACT(32, 3, 2);
    else if (vpl == 4) MDB_RMS_ACT(32, 4, 2);
    else MDB_RMS_ACT(32, 5, 1);
  }
  else MDB_RMS_ACT_G(16)
  else MDB_RMS_ACT_G(8)
  else MDB_RMS_ACT_G(4)
  else MDB_RMS_ACT_G(2)
  else return 3701;
#undef MDB_RMS_ACT_G
#undef MDB_RMS_ACT
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------
// GroupNorm (+ SiLU) for channels-last activations [N, HW, C], forward and backward
// (UNet ResNet blocks and the image VAE: src/maxdiffusion/models/resnet_flax.py:97-186, vae_flax.py).
//
// A group's channels are neither contiguous over a pixel nor aligned to 16-byte vectors (320 channels in 32 groups
// are 10 channels each), so both passes work per CHANNEL and the groups appear only in a tiny fold in between:
//   sums  : partial[n, split, c] = {sum f1, sum f2} over a strip of pixels; forward (f1, f2) = (x, x^2), backward
//           (f1, f2) = (dy', dy' * x) with dy' = dy * silu'(x * scale + shift) when the activation is fused
//   fold  : (host side, on [N, C]-sized arrays) group statistics -> per-(n, c) coefficients
//   apply : forward y = act(x * a + b); backward dx = dy' * a + b + x * c, coefficients fp32 [N, C]
// One strip of pixels per CTA, a thread keeps one 8-channel vector in registers over the rows of the strip; partial
// sums are combined in a fixed order, so results are bitwise reproducible.
// ---------------------------------------------------------------------------------------------------------------
namespace mdb {
namespace cln {

__device__ __forceinline__ float silu_grad(float z) {
  const float s = 1.0f / (1.0f + __expf(-z));
  return s * (1.0f + z * (1.0f - s));
}

// grid (splits, N), block = rows_per_pass * vecs threads. act_a / act_b: forward coefficients for the fused SiLU of the
// backward pass (null: none). dy null: forward sums of x.
__global__ void __launch_bounds__(256)
gn_cl_sums_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ act_a,
                  const float* __restrict__ act_b, float2* __restrict__ partial, int HW, int C, int rows_per_pass) {
  extern __shared__ float red[];  // [rows_per_pass][vecs][16]
  const int vecs = C >> 3;
  const int v = threadIdx.x % vecs, r = threadIdx.x / vecs;
  const int n = blockIdx.y, splits = gridDim.x;
  const int per = (HW + splits - 1) / splits;
  const int row0 = blockIdx.x * per, row1 = min(HW, row0 + per);
  float s1[8], s2[8], a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s1[j] = s2[j] = 0.0f;
  if (dy != nullptr && act_a != nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a[j] = act_a[static_cast<long long>(n) * C + v * 8 + j];
      b[j] = act_b[static_cast<long long>(n) * C + v * 8 + j];
    }
  }
  for (int row = row0 + r; row < row1; row += rows_per_pass) {
    const long long off = (static_cast<long long>(n) * HW + row) * C + v * 8;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + off);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    float xf[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(xw[j]);
      xf[2 * j] = f.x;
      xf[2 * j + 1] = f.y;
    }
    if (dy == nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s1[j] += xf[j];
        s2[j] += xf[j] * xf[j];
      }
    } else {
      const uint4 dv = *reinterpret_cast<const uint4*>(dy + off);
      const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(dw[j]);
        float d0 = f.x, d1 = f.y;
        if (act_a != nullptr) {
          d0 *= silu_grad(xf[2 * j] * a[2 * j] + b[2 * j]);
          d1 *= silu_grad(xf[2 * j + 1] * a[2 * j + 1] + b[2 * j + 1]);
        }
        s1[2 * j] += d0;
        s1[2 * j + 1] += d1;
        s2[2 * j] += d0 * xf[2 * j];
        s2[2 * j + 1] += d1 * xf[2 * j + 1];
      }
    }
  }
  float* mine = red + (static_cast<size_t>(r) * vecs + v) * 16;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    mine[j] = s1[j];
    mine[8 + j] = s2[j];
  }
  __syncthreads();
  if (r == 0) {
    for (int rr = 1; rr < rows_per_pass; ++rr) {  // fixed order
      const float* o = red + (static_cast<size_t>(rr) * vecs + v) * 16;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s1[j] += o[j];
        s2[j] += o[8 + j];
      }
    }
    float2* dst = partial + (static_cast<long long>(n) * splits + blockIdx.x) * C + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float2(s1[j], s2[j]);
  }
}

// forward: y = act(x * a + b). backward (dy != null): dx = dy' * a + b + x * c, dy' = dy * silu'(x * fa + fb) if fa.
__global__ void __launch_bounds__(256)
gn_cl_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ out,
                   const float* __restrict__ ca, const float* __restrict__ cb, const float* __restrict__ cc,
                   const float* __restrict__ fa, const float* __restrict__ fb, long long total_vecs, int HW, int C,
                   int act) {
  const int vecs = C >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total_vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vecs);
    const long long row = i / vecs;
    const int n = static_cast<int>(row / HW);
    const long long cbase = static_cast<long long>(n) * C + v * 8;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + i * 8);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    float xf[8], o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(xw[j]);
      xf[2 * j] = f.x;
      xf[2 * j + 1] = f.y;
    }
    const float4 a0 = *reinterpret_cast<const float4*>(ca + cbase), a1 = *reinterpret_cast<const float4*>(ca + cbase + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(cb + cbase), b1 = *reinterpret_cast<const float4*>(cb + cbase + 4);
    const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    if (dy == nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float z = xf[j] * av[j] + bv[j];
        o[j] = act ? z / (1.0f + __expf(-z)) : z;
      }
    } else {
      const uint4 dv = *reinterpret_cast<const uint4*>(dy + i * 8);
      const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
      float df[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(dw[j]);
        df[2 * j] = f.x;
        df[2 * j + 1] = f.y;
      }
      if (fa != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) df[j] *= silu_grad(xf[j] * fa[cbase + j] + fb[cbase + j]);
      }
      const float4 c0 = *reinterpret_cast<const float4*>(cc + cbase), c1 = *reinterpret_cast<const float4*>(cc + cbase + 4);
      const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = df[j] * av[j] + bv[j] + xf[j] * cv[j];
    }
    uint4 ov;
    ov.x = pack_bf16x2(o[0], o[1]);
    ov.y = pack_bf16x2(o[2], o[3]);
    ov.z = pack_bf16x2(o[4], o[5]);
    ov.w = pack_bf16x2(o[6], o[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = ov;
  }
}

}  // namespace cln
}  // namespace mdb

// Per-channel partial sums over `splits` strips of pixels: partial fp32 [N, splits, C, 2]. x (and dy) bf16 [N, HW, C],
// contiguous, C a multiple of 8 and at most 2048. act_a / act_b (fp32 [N, C], may be null) select the fused-SiLU form
// of the backward sums.
extern "C" int mdb_gn_cl_sums(const void* x, const void* dy, const float* act_a, const float* act_b, float* partial, int N,
                              int HW, int C, int splits, void* stream) {
  using namespace mdb::cln;
  if (N <= 0 || HW <= 0) return 0;
  const int vecs = C >> 3;
  if ((C & 7) || vecs < 1 || vecs > 256 || splits < 1) return 3702;
  const int rows_per_pass = 256 / vecs;
  const int threads = rows_per_pass * vecs;
  const size_t smem = static_cast<size_t>(threads) * 16 * sizeof(float);
  gn_cl_sums_kernel<<<dim3(splits, N), threads, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), act_a, act_b,
      reinterpret_cast<float2*>(partial), HW, C, rows_per_pass);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_gn_cl_apply(const void* x, const void* dy, void* out, const float* ca, const float* cb, const float* cc,
                               const float* fa, const float* fb, int N, int HW, int C, int act, void* stream) {
  using namespace mdb::cln;
  if (N <= 0 || HW <= 0) return 0;
  if ((C & 7) || ca == nullptr || cb == nullptr || (dy != nullptr && cc == nullptr)) return 3703;
  const long long total = static_cast<long long>(N) * HW * (C >> 3);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(mdb::sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  gn_cl_apply_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(out), ca, cb,
      cc, fa, fb, total, HW, C, act);
  return static_cast<int>(cudaGetLastError());
}

// The fold between the two passes, one CTA per sample: per-channel partial sums [N, splits, C, 2] -> group statistics
// -> per-(n, c) coefficients. The arithmetic is a few thousand values; as PyTorch ops it was a dozen launches per
// normalisation (twenty in the backward), which at the UNet's 176 normalisations per step cost more than the passes.
namespace mdb {
namespace cln {

__device__ __forceinline__ float param_at(const void* p, int is_bf16, int c) {
  if (p == nullptr) return 1.0f;
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[c]) : static_cast<const float*>(p)[c];
}

// forward: a = rstd * gamma, b = beta - mean * a; also mean / rstd [N, G] for the backward
__global__ void __launch_bounds__(256)
gn_cl_fold_fwd_kernel(const float2* __restrict__ partial, int splits, int C, int groups, float count, float eps,
                      const void* gamma, const void* beta, int params_bf16, float* __restrict__ a, float* __restrict__ b,
                      float* __restrict__ mean_out, float* __restrict__ rstd_out) {
  extern __shared__ float sm[];  // [C][2] channel sums, then [G][2] group (mean, rstd)
  float* ch = sm;
  float* gr = sm + 2 * C;
  const int n = blockIdx.x, cg = C / groups;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float s1 = 0.0f, s2 = 0.0f;
    for (int s = 0; s < splits; ++s) {  // fixed order
      const float2 v = partial[(static_cast<long long>(n) * splits + s) * C + c];
      s1 += v.x;
      s2 += v.y;
    }
    ch[2 * c] = s1;
    ch[2 * c + 1] = s2;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float s1 = 0.0f, s2 = 0.0f;
    for (int j = 0; j < cg; ++j) {
      s1 += ch[2 * (g * cg + j)];
      s2 += ch[2 * (g * cg + j) + 1];
    }
    const float mean = s1 / count;
    const float rstd = rsqrtf(fmaxf(s2 / count - mean * mean, 0.0f) + eps);
    gr[2 * g] = mean;
    gr[2 * g + 1] = rstd;
    mean_out[n * groups + g] = mean;
    rstd_out[n * groups + g] = rstd;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int g = c / cg;
    const float av = gr[2 * g + 1] * param_at(gamma, params_bf16, c);
    a[static_cast<long long>(n) * C + c] = av;
    b[static_cast<long long>(n) * C + c] = (beta != nullptr ? param_at(beta, params_bf16, c) : 0.0f) - gr[2 * g] * av;
  }
}

// backward: from d1 = sum dy', d2 = sum dy' * x per channel: dx = dy' * ca + cb + x * cc, and the per-sample terms of
// dgamma (sum dy' * xhat) and dbeta (sum dy')
__global__ void __launch_bounds__(256)
gn_cl_fold_bwd_kernel(const float2* __restrict__ partial, int splits, int C, int groups, float count, const void* gamma,
                      int params_bf16, const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                      float* __restrict__ ca, float* __restrict__ cb, float* __restrict__ cc, float* __restrict__ dgamma_n,
                      float* __restrict__ dbeta_n) {
  extern __shared__ float sm[];  // [C][2]: (d1, dxhat) per channel, then [G][2]: (s1, s2)
  float* ch = sm;
  float* gr = sm + 2 * C;
  const int n = blockIdx.x, cg = C / groups;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float d1 = 0.0f, d2 = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float2 v = partial[(static_cast<long long>(n) * splits + s) * C + c];
      d1 += v.x;
      d2 += v.y;
    }
    const int g = c / cg;
    const float mean = mean_in[n * groups + g], rstd = rstd_in[n * groups + g];
    const float dxhat = rstd * (d2 - mean * d1);
    ch[2 * c] = d1;
    ch[2 * c + 1] = dxhat;
    dbeta_n[static_cast<long long>(n) * C + c] = d1;
    dgamma_n[static_cast<long long>(n) * C + c] = dxhat;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float s1 = 0.0f, s2 = 0.0f;
    for (int j = 0; j < cg; ++j) {
      const int c = g * cg + j;
      const float gm = param_at(gamma, params_bf16, c);
      s1 += gm * ch[2 * c];
      s2 += gm * ch[2 * c + 1];
    }
    gr[2 * g] = s1 / count;
    gr[2 * g + 1] = s2 / count;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int g = c / cg;
    const float mean = mean_in[n * groups + g], rstd = rstd_in[n * groups + g];
    const float s1 = gr[2 * g], s2 = gr[2 * g + 1];
    const long long o = static_cast<long long>(n) * C + c;
    ca[o] = rstd * param_at(gamma, params_bf16, c);
    cb[o] = -rstd * s1 + mean * rstd * rstd * s2;
    cc[o] = -rstd * rstd * s2;
  }
}

}  // namespace cln
}  // namespace mdb

// partial: fp32 [N, splits, C, 2] from mdb_gn_cl_sums; gamma / beta: [C] bf16 (params_bf16 = 1) or fp32, may be null;
// a, b: fp32 [N, C]; mean, rstd: fp32 [N, groups]. count = pixels * channels per group.
extern "C" int mdb_gn_cl_fold_fwd(const float* partial, int N, int splits, int C, int groups, float count, float eps,
                                  const void* gamma, const void* beta, int params_bf16, float* a, float* b, float* mean,
                                  float* rstd, void* stream) {
  if (N <= 0) return 0;
  if (groups <= 0 || C % groups || splits < 1 || C > 8192) return 3704;
  const size_t smem = (2 * static_cast<size_t>(C) + 2 * groups) * sizeof(float);
  mdb::cln::gn_cl_fold_fwd_kernel<<<N, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2*>(partial), splits, C, groups, count, eps, gamma, beta, params_bf16, a, b, mean, rstd);
  return static_cast<int>(cudaGetLastError());
}

// ca, cb, cc, dgamma_n, dbeta_n: fp32 [N, C] (the caller sums the last two over N).
extern "C" int mdb_gn_cl_fold_bwd(const float* partial, int N, int splits, int C, int groups, float count, const void* gamma,
                                  int params_bf16, const float* mean, const float* rstd, float* ca, float* cb, float* cc,
                                  float* dgamma_n, float* dbeta_n, void* stream) {
  if (N <= 0) return 0;
  if (groups <= 0 || C % groups || splits < 1 || C > 8192) return 3704;
  const size_t smem = (2 * static_cast<size_t>(C) + 2 * groups) * sizeof(float);
  mdb::cln::gn_cl_fold_bwd_kernel<<<N, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2*>(partial), splits, C, groups, count, gamma, params_bf16, mean, rstd, ca, cb, cc, dgamma_n,
      dbeta_n);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------
// Row softmax, in place or out of place: y[r, :] = softmax(x[r, :]) for bf16 rows of up to 32768 columns, fp32 math.
// One CTA per row, the row lives in registers between the two reductions (one read, one write). It sits between the two
// GEMMs of attention with a head size the flash kernels are not built for (the Wan VAE's single 384-wide head,
// src/maxdiffusion/models/wan/autoencoder_kl_wan.py:487-546): scores = Q K^T on the GEMM kernel, this, then P V.
// ---------------------------------------------------------------------------------------------------------------
namespace mdb {
namespace cln {

constexpr int SM_THREADS = 256;
constexpr int SM_MAX_VPT = 16;  // vectors of 8 per thread

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int i = 1; i < SM_THREADS / 32; ++i) t = is_max ? fmaxf(t, red[i]) : t + red[i];
  return t;
}

template <int VPT>
__global__ void __launch_bounds__(SM_THREADS)
softmax_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y, long long ldy, int cols) {
  __shared__ float red[SM_THREADS / 32];
  const long long row = blockIdx.x;
  const int vecs = cols >> 3;
  float v[VPT][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * SM_THREADS;
    if (vi < vecs) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + row * ldx + vi * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        v[i][2 * j] = f.x;
        v[i][2 * j + 1] = f.y;
        mx = fmaxf(mx, fmaxf(f.x, f.y));
      }
    }
  }
  mx = block_reduce(mx, true, red);
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * SM_THREADS;
    if (vi < vecs) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = __expf(v[i][j] - mx);
        sum += v[i][j];
      }
    }
  }
  sum = block_reduce(sum, false, red);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * SM_THREADS;
    if (vi < vecs) {
      uint4 o;
      o.x = pack_bf16x2(v[i][0] * inv, v[i][1] * inv);
      o.y = pack_bf16x2(v[i][2] * inv, v[i][3] * inv);
      o.z = pack_bf16x2(v[i][4] * inv, v[i][5] * inv);
      o.w = pack_bf16x2(v[i][6] * inv, v[i][7] * inv);
      *reinterpret_cast<uint4*>(y + row * ldy + vi * 8) = o;
    }
  }
}

}  // namespace cln
}  // namespace mdb

// x, y: bf16 [rows, cols] with leading dimensions ldx / ldy (multiples of 8); cols a multiple of 8, at most 32768.
extern "C" int mdb_softmax_rows(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols, void* stream) {
  using namespace mdb::cln;
  if (rows <= 0) return 0;
  if ((cols & 7) || cols <= 0 || cols > 8 * SM_THREADS * SM_MAX_VPT || (ldx & 7) || (ldy & 7) || rows >= (1ll << 31)) return 3704;
  const int vpt = ((cols >> 3) + SM_THREADS - 1) / SM_THREADS;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  const int grid = static_cast<int>(rows);
  if (vpt <= 1) softmax_rows_kernel<1><<<grid, SM_THREADS, 0, st>>>(xp, ldx, yp, ldy, cols);
  else if (vpt <= 2) softmax_rows_kernel<2><<<grid, SM_THREADS, 0, st>>>(xp, ldx, yp, ldy, cols);
  else if (vpt <= 4) softmax_rows_kernel<4><<<grid, SM_THREADS, 0, st>>>(xp, ldx, yp, ldy, cols);
  else if (vpt <= 8) softmax_rows_kernel<8><<<grid, SM_THREADS, 0, st>>>(xp, ldx, yp, ldy, cols);
  else softmax_rows_kernel<16><<<grid, SM_THREADS, 0, st>>>(xp, ldx, yp, ldy, cols);
  return static_cast<int>(cudaGetLastError());
}
