// fp8 GEMM for sm_100a with per-tensor absmax scales, and the quantiser that feeds it:
//     D[M,N] (bf16) = (sa * sb) * ( Aq[M,K] * Bq[N,K]^T ) + bias
// Aq / Bq hold e4m3 (forward operands) or e5m2 (gradients) values; sa, sb are the de-quantisation
// scales (absmax / fp8_max) written to device memory by the quantiser, so no host round trip sits between
// quantisation and the product. tcgen05.mma.kind::f8f6f4 runs at twice the bf16 rate: one instruction is
// 128 x 256 x 32; a pipeline stage holds 128 bytes of K per row (128-byte swizzle), i.e. K = 128.
//
// Same structure as the bf16 kernel (persistent, TMA producer warp / MMA warp / 4 epilogue warps,
// TMEM accumulators double buffered), K-major operands only.
// Replaces the reference's qwix fp8 / int8 paths, which quantise around XLA dot_general
// (src/maxdiffusion/pipelines/wan/wan_pipeline.py:569-651, src/maxdiffusion/models/quantizations.py:88-131).
#include <cuda_fp8.h>

#include "host_common.h"

namespace mdb {
namespace gemm8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // elements = bytes
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
  int M, N, K;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;
  const float* scale_a;  // device scalars
  const float* scale_b;
  int a_e5m2, b_e5m2;
  int int8;  // 1: operands are signed 8-bit integers (tcgen05 kind::i8, int32 accumulators)
  DeviceStatus* status;
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_idx, int& n_idx) {
  const int tiles_per_group = GROUP_M * num_n;
  const int group = tile / tiles_per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int local = tile - group * tiles_per_group;
  m_idx = first_m + local % rows;
  n_idx = local / rows;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr_smem, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, num_m, num_n, m_idx, n_idx);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 50)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m_idx * BM);
          tma_load_2d(sa + A_BYTES, &tmap_b, &full_bar[stage], kb * BK, n_idx * BN);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          int s = (stage - 1 - i + 2 * STAGES) % STAGES;
          uint32_t ph = (i < stage) ? phase : (phase ^ 1u);
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(&full_bar[s], ph); ++spin) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = p.int8 ? make_idesc_i8(BM, BN) : make_idesc_f8(BM, BN, p.a_e5m2, p.b_e5m2);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 51)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 52)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {  // 32 bytes of K per instruction
            const uint64_t da = make_smem_desc(sa + k * 32, 16, 1024), db = make_smem_desc(sb + k * 32, 16, 1024);
            if (p.int8) umma_ss_i8(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_ss_f8(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const float alpha = (*p.scale_a) * (*p.scale_b);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int m_idx, n_idx;
      tile_coords(tile, num_m, num_n, m_idx, n_idx);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, 53)) { ok = false; break; }
      tc_fence_after_sync();
      const long long row = static_cast<long long>(m_idx) * BM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n_idx * BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col >= p.N) break;
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              x[j] = (p.int8 ? static_cast<float>(static_cast<int>(r[v * 8 + j])) : __uint_as_float(r[v * 8 + j])) * alpha;
            if (p.bias) {
              const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
              const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16x2(bw[j]);
                x[2 * j] += f.x;
                x[2 * j + 1] += f.y;
              }
            }
            uint4 ov;
            ov.x = pack_bf16x2(x[0], x[1]);
            ov.y = pack_bf16x2(x[2], x[3]);
            ov.z = pack_bf16x2(x[4], x[5]);
            ov.w = pack_bf16x2(x[6], x[7]);
            *reinterpret_cast<uint4*>(p.out + row * p.ldo + col) = ov;
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// q = fp8(x * fp8_max / absmax); scale_out = absmax / fp8_max. stats[1] holds max |x| (from sumsq_maxabs).
__global__ void __launch_bounds__(256)
quantize_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, long long nvec,
                    const float* __restrict__ stats, float* __restrict__ scale_out, int e5m2) {
  const float fmax = e5m2 ? 57344.0f : 448.0f;
  const float amax = fmaxf(stats[1], 1e-12f);
  const float mul = fmax / amax;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = amax / fmax;
  const __nv_fp8_interpretation_t kind = e5m2 ? __NV_E5M2 : __NV_E4M3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(f.x * mul, f.y * mul), __NV_SATFINITE, kind);
      if (j < 2) lo |= pair << (16 * j);
      else hi |= pair << (16 * (j - 2));
    }
    reinterpret_cast<uint2*>(q)[i] = make_uint2(lo, hi);
  }
}

// q = round(x * 127 / absmax) in [-127, 127]; scale_out = absmax / 127 (symmetric per-tensor int8).
__global__ void __launch_bounds__(256)
quantize_int8_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q, long long nvec,
                     const float* __restrict__ stats, float* __restrict__ scale_out) {
  const float amax = fmaxf(stats[1], 1e-12f);
  const float mul = 127.0f / amax;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = amax / 127.0f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      const int a = max(-127, min(127, __float2int_rn(f.x * mul)));
      const int b = max(-127, min(127, __float2int_rn(f.y * mul)));
      const uint32_t pair = (static_cast<uint32_t>(a) & 0xffu) | ((static_cast<uint32_t>(b) & 0xffu) << 8);
      out[j >> 1] |= pair << (16 * (j & 1));
    }
    reinterpret_cast<uint2*>(q)[i] = make_uint2(out[0], out[1]);
  }
}

}  // namespace gemm8
}  // namespace mdb

// Aq: [M, K] fp8 bytes (leading dimension lda, a multiple of 16); Bq: [N, K]; out: bf16 [M, N]; N % 8 == 0.
// scale_a / scale_b: device floats. a_e5m2 / b_e5m2 select the 8-bit format of each operand.
static int gemm8_impl(const void* Aq, const void* Bq, void* out, const void* bias, const float* scale_a,
                      const float* scale_b, int M, int N, int K, long long lda, long long ldb, long long ldo, int a_e5m2,
                      int b_e5m2, int int8, void* stream_ptr);

extern "C" int mdb_gemm_fp8(const void* Aq, const void* Bq, void* out, const void* bias, const float* scale_a,
                            const float* scale_b, int M, int N, int K, long long lda, long long ldb, long long ldo,
                            int a_e5m2, int b_e5m2, void* stream_ptr) {
  return gemm8_impl(Aq, Bq, out, bias, scale_a, scale_b, M, N, K, lda, ldb, ldo, a_e5m2, b_e5m2, 0, stream_ptr);
}

// The same kernel on signed 8-bit integers (tcgen05 kind::i8, exact int32 accumulation): Aq [M, K], Bq [N, K] int8,
// out = scale_a * scale_b * (Aq Bq^T) + bias in bf16. The reference's int8 quantisation modes
// (src/maxdiffusion/pyconfig.py `quantization: int8`, models/quantizations.py:88-131) run on it.
extern "C" int mdb_gemm_int8(const void* Aq, const void* Bq, void* out, const void* bias, const float* scale_a,
                             const float* scale_b, int M, int N, int K, long long lda, long long ldb, long long ldo,
                             void* stream_ptr) {
  return gemm8_impl(Aq, Bq, out, bias, scale_a, scale_b, M, N, K, lda, ldb, ldo, 0, 0, 1, stream_ptr);
}

static int gemm8_impl(const void* Aq, const void* Bq, void* out, const void* bias, const float* scale_a,
                      const float* scale_b, int M, int N, int K, long long lda, long long ldb, long long ldo, int a_e5m2,
                      int b_e5m2, int int8, void* stream_ptr) {
  using namespace mdb;
  using namespace mdb::gemm8;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (lda & 15) || (ldb & 15) || (ldo & 7) || !scale_a || !scale_b) return 3101;
  CUtensorMap ta, tb;
  uint64_t dims_a[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  uint64_t str_a[1] = {static_cast<uint64_t>(lda)};
  uint32_t box_a[2] = {BK, BM};
  int rc = encode_tmap_u8(&ta, Aq, 2, dims_a, str_a, box_a);
  if (rc) return rc;
  uint64_t dims_b[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
  uint64_t str_b[1] = {static_cast<uint64_t>(ldb)};
  uint32_t box_b[2] = {BK, BN};
  rc = encode_tmap_u8(&tb, Bq, 2, dims_b, str_b, box_b);
  if (rc) return rc;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.a_e5m2 = a_e5m2;
  p.b_e5m2 = b_e5m2;
  p.int8 = int8;
  p.status = status_buffer();
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  gemm_fp8_kernel<<<grid, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream_ptr)>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// x: bf16 [n] (n % 8 == 0); stats: device {sum x^2, max |x|} as produced by mdb_sumsq_maxabs.
extern "C" int mdb_quantize_fp8(const void* x, void* q, long long n, const float* stats, float* scale_out, int e5m2,
                                void* stream_ptr) {
  using namespace mdb;
  if (n <= 0) return 0;
  if (n & 7) return 3102;
  const long long nvec = n >> 3;
  long long blocks = (nvec + 1023) / 1024;
  const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks > sm_count() * 8 ? sm_count() * 8 : blocks));
  gemm8::quantize_fp8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), nvec, stats, scale_out, e5m2);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_quantize_int8(const void* x, void* q, long long n, const float* stats, float* scale_out,
                                 void* stream_ptr) {
  using namespace mdb;
  if (n <= 0) return 0;
  if (n & 7) return 3102;
  const long long nvec = n >> 3;
  long long blocks = (nvec + 1023) / 1024;
  const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks > sm_count() * 8 ? sm_count() * 8 : blocks));
  gemm8::quantize_int8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<int8_t*>(q), nvec, stats, scale_out);
  return static_cast<int>(cudaGetLastError());
}
