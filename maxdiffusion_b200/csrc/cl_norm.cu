// Row kernels for channels-last activations [rows, C] (a row is one pixel / voxel):
//   rms_act : y = act( x / max(||x||_2, eps) * sqrt(C) * gamma + beta ),  act = identity or SiLU
// This is the `WanRMS_norm` + SiLU that precedes every convolution of the Wan VAE's residual blocks
// (src/maxdiffusion/models/wan/autoencoder_kl_wan.py:150-183, 452-484): memory bound, one read and one write of the
// activation. A row of C channels (96 .. 1024) is handled by a group of G = 8, 16 or 32 lanes, each lane holding up
// to four 16-byte vectors, so that narrow rows (96 channels = 12 vectors) do not leave most of a warp idle; the
// sum of squares is reduced with shuffles inside the group, statistics in fp32.
#include "host_common.h"

namespace mdb {
namespace cln {

constexpr int MAX_VPL = 4;  // vectors (8 bf16) per lane

template <int G>
__global__ void __launch_bounds__(256)
rms_act_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y, long long ldy,
               const float* __restrict__ gamma, const float* __restrict__ beta, long long rows, int C, float eps,
               int act) {
  const int vecs = C >> 3;
  const int lane_in_group = threadIdx.x % G;
  const long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  const long long n_groups = static_cast<long long>(gridDim.x) * blockDim.x / G;
  const float scale = sqrtf(static_cast<float>(C));
  // every lane of a warp runs the same number of iterations (the shuffles below name all 32 lanes)
  const long long iters = (rows + n_groups - 1) / n_groups;
  for (long long it = 0; it < iters; ++it) {
    const long long row = group + it * n_groups;
    const bool on = row < rows;
    uint4 v[MAX_VPL];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_VPL; ++i) {
      const int vi = lane_in_group + i * G;
      if (on && vi < vecs) {
        v[i] = *reinterpret_cast<const uint4*>(x + row * ldx + vi * 8);
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = scale / fmaxf(sqrtf(ss), eps);
#pragma unroll
    for (int i = 0; i < MAX_VPL; ++i) {
      const int vi = lane_in_group + i * G;
      if (on && vi < vecs) {
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
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
        *reinterpret_cast<uint4*>(y + row * ldy + vi * 8) = ov;
      }
    }
  }
}

}  // namespace cln
}  // namespace mdb

// x, y: bf16 [rows, C] with leading dimensions ldx / ldy (elements, multiples of 8); gamma / beta: fp32 [C]
// (beta may be null); C a multiple of 8, at most 1024. act: 0 identity, 1 SiLU.
extern "C" int mdb_rms_act_cl(const void* x, long long ldx, void* y, long long ldy, const float* gamma,
                              const float* beta, long long rows, int C, float eps, int act, void* stream) {
  using namespace mdb::cln;
  if (rows <= 0) return 0;
  if ((C & 7) || C <= 0 || C > 8 * 32 * MAX_VPL || (ldx & 7) || (ldy & 7) || gamma == nullptr) return 3701;
  const int vecs = C >> 3;
  const int G = vecs <= 8 ? 8 : (vecs <= 16 ? 16 : 32);
  const long long groups_per_block = 256 / G;
  long long blocks = (rows + groups_per_block - 1) / groups_per_block;
  const long long cap = static_cast<long long>(mdb::sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  if (G == 8) rms_act_kernel<8><<<static_cast<int>(blocks), 256, 0, st>>>(xp, ldx, yp, ldy, gamma, beta, rows, C, eps, act);
  else if (G == 16) rms_act_kernel<16><<<static_cast<int>(blocks), 256, 0, st>>>(xp, ldx, yp, ldy, gamma, beta, rows, C, eps, act);
  else rms_act_kernel<32><<<static_cast<int>(blocks), 256, 0, st>>>(xp, ldx, yp, ldy, gamma, beta, rows, C, eps, act);
  return static_cast<int>(cudaGetLastError());
}
