// Weight gradient of a channels-last convolution on sm_100a (tcgen05 + TMEM + TMA):
//
//     dW[tap][co][ci] = sum over pixels p of  dY[p, co] * X[p + shift(tap), ci]
//
// Both tensors are laid out on the same zero-bordered pixel grid ([B, H + 2, W + 2, C] flattened to rows), so that the
// spatial shift of a tap is ONE constant row offset of X and the border rows of dY (zeros) cancel whatever the offset
// reaches across an image edge. Each tap is then a GEMM with the pixel axis as K:  A = dY seen as [K, M = Cout],
// B = X seen as [K, N = Cin] at the tap's row offset, both "MN-major" operands fetched by plain 2-D TMA boxes (rows
// outside the tensor read as zeros). K is tens of thousands of pixels while M x N is only a handful of tiles, so
// the pixel axis is split: a work item is (tap, K split, M tile, N tile) and writes an fp32 partial tile; the caller
// sums the splits in a fixed order (bitwise reproducible). Stride-2 convolutions use the same kernel on the four
// parity planes of X (plane choice = one more row offset).
//
// The boxed form (`mdb_conv_wgrad_boxed`) needs no bordered copies at all: a K block is a box of 64 output pixels
// (BW x BH of one image) fetched from the unpadded channels-last tensors by 5-D TMA; a tap moves X's box by its
// (row, column) shift and whatever falls outside the image is the tensor map's zero fill, exactly the padding the
// forward convolution read. Stride 2 views X as [B, H/2, 2, W/2, 2C]: the row parity is a coordinate of its own and
// the column parity an offset into the doubled channel axis.
// Roles per CTA (persistent): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..5 epilogue; accumulators
// double buffered in TMEM.
//
// Replaces the weight-gradient convolutions XLA:GPU / cuDNN run for the reference's UNet and VAE training
// (src/maxdiffusion/models/resnet_flax.py:37-186, src/maxdiffusion/trainers/sdxl_trainer.py:294-391).
#include "host_common.h"

namespace mdb {
namespace wgrad {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BK * BM * 2;  // 16 KiB: two 64-column chunks of 64 K rows
constexpr int NUM_THREADS = 192;
constexpr int MAX_TAPS = 9;
constexpr int ACC_COLS = 256;

struct Params {
  int M, N;                 // Cout, Cin
  int BN;                   // 64, 128, 192 or 256
  int stages;
  int n_taps, splits;
  int kb_total;             // 64-row blocks of the pixel grid
  long long b_row_off[MAX_TAPS];
  float* out;               // [n_taps, splits, M, N] fp32
  DeviceStatus* status;
  // boxed form: K block kb = (image, row block, column block) of the output pixel grid
  int boxed, BW, BH, n_wb, n_hb;
  int tap_c[MAX_TAPS], tap_w[MAX_TAPS], tap_par[MAX_TAPS], tap_h[MAX_TAPS];  // channel offset, column shift, row parity, row shift
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int STAGES = p.stages;
  const int STAGE_BYTES = A_BYTES + p.BN * BK * 2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                // [8]
  uint64_t* empty_bar = bars + 8;           // [8]
  uint64_t* tmem_full = bars + 16;          // [2]
  uint64_t* tmem_empty = bars + 18;         // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + p.BN - 1) / p.BN;
  const int num_items = p.n_taps * p.splits * num_m * num_n;
  const int kb_per_split = (p.kb_total + p.splits - 1) / p.splits;

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
    tmem_alloc(tmem_ptr_smem, 2 * ACC_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // item -> (n tile, m tile, split, tap), n fastest: the CTAs of a wave share the dY / X rows of one K range in L2
  auto decode = [&](int item, int& n_idx, int& m_idx, int& split, int& tap) {
    n_idx = item % num_n; item /= num_n;
    m_idx = item % num_m; item /= num_m;
    tap = item % p.n_taps; item /= p.n_taps;
    split = item;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int n_idx, m_idx, split, tap;
        decode(item, n_idx, m_idx, split, tap);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        const long long off = p.b_row_off[tap];
        // boxed form: (image, row block, column block) of the first K block, advanced without divisions
        int wb = 0, hb = 0, img = 0;
        if (p.boxed) {
          wb = kb0 % p.n_wb;
          const int t = kb0 / p.n_wb;
          hb = t % p.n_hb;
          img = t / p.n_hb;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 140)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          if (p.boxed) {
            const int w0 = wb * p.BW, h0 = hb * p.BH;
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_5d(sa + c * (BK * 128), &tmap_a, &full_bar[stage], m_idx * BM + c * 64, w0, 0, h0, img);
            for (int c = 0; c < p.BN / 64; ++c)
              tma_load_5d(sb + c * (BK * 128), &tmap_b, &full_bar[stage], p.tap_c[tap] + n_idx * p.BN + c * 64,
                          w0 + p.tap_w[tap], p.tap_par[tap], h0 + p.tap_h[tap], img);
            if (++wb == p.n_wb) {
              wb = 0;
              if (++hb == p.n_hb) { hb = 0; ++img; }
            }
            ++issued;
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          const int k0 = kb * BK;
#pragma unroll
          for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmap_a, &full_bar[stage], m_idx * BM + c * 64, k0);
          for (int c = 0; c < p.BN / 64; ++c)
            tma_load_2d(sb + c * (BK * 128), &tmap_b, &full_bar[stage], n_idx * p.BN + c * 64, static_cast<int>(k0 + off));
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
      const uint32_t idesc = make_idesc_bf16(BM, p.BN, true, true);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
        int n_idx, m_idx, split, tap;
        decode(item, n_idx, m_idx, split, tap);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 150)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 151)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa, BK * 128, 1024);
          const uint64_t db = make_smem_desc(sa + A_BYTES, BK * 128, 1024);
          // one K step = 16 rows of 128 bytes = 2048 bytes = 128 units of the descriptor's address field
          umma_ss(d_tmem, da, db, idesc, accumulate);
          umma_ss(d_tmem, da + 128, db + 128, idesc, 1u);
          umma_ss(d_tmem, da + 256, db + 256, idesc, 1u);
          umma_ss(d_tmem, da + 384, db + 384, idesc, 1u);
          accumulate = 1u;
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    int it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
      int n_idx, m_idx, split, tap;
      decode(item, n_idx, m_idx, split, tap);
      const int kb0 = split * kb_per_split;
      const bool empty = kb0 >= p.kb_total;  // a split past the end of the pixel axis contributes zeros
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, 160)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m_idx * BM + row_in_tile;
      const bool row_ok = row < p.M;
      float* orow = p.out + (static_cast<long long>(tap) * p.splits + split) * p.M * p.N + static_cast<long long>(row) * p.N;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * ACC_COLS;
#pragma unroll 1
      for (int c = 0; c < p.BN / 16; ++c) {
        const int col0 = n_idx * p.BN + c * 16;
        if (col0 >= p.N) break;  // uniform across the CTA
        uint32_t v[16];
        tmem_ld_x16(taddr + c * 16, v);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = col0 + q * 4;
            if (col >= p.N) break;  // N is a multiple of 8
            float4 o = make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]), __uint_as_float(v[q * 4 + 2]),
                                   __uint_as_float(v[q * 4 + 3]));
            if (empty) o = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(orow + col) = o;
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
    tmem_dealloc(tmem_base, 2 * ACC_COLS);
  }
}

}  // namespace wgrad
}  // namespace mdb

// dy: [rows_a, M] bf16 (rows = pixels of the zero-bordered grid, border rows zero); x: [rows_b, N] bf16 (the same grid,
// or several such planes stacked); b_row_off[tap]: row of x that pairs with row 0 of dy for that tap (may be negative:
// rows outside x read as zeros). out: fp32 [n_taps, splits, M, N]. M and N multiples of 8.
extern "C" int mdb_conv_wgrad(const void* dy, const void* x, float* out, long long rows_a, long long rows_b, int M, int N,
                              int n_taps, const long long* b_row_off, int splits, void* stream_ptr) {
  using namespace mdb;
  using namespace mdb::wgrad;
  if (M <= 0 || N <= 0 || rows_a <= 0) return 0;
  if ((M & 7) || (N & 7) || n_taps < 1 || n_taps > MAX_TAPS || splits < 1) return 3801;
  if (rows_a >= (1ll << 31) || rows_b >= (1ll << 31)) return 3802;
  Params p;
  p.M = M; p.N = N;
  // tile width: a multiple of 64 (MN-major operand chunks); fewest padded columns, with a penalty for narrow tiles
  int best = 64;
  double best_cost = -1.0;
  for (int bn = 64; bn <= 256; bn += 64) {
    const double cost = static_cast<double>((N + bn - 1) / bn * bn) * (1.0 + 64.0 / bn);
    if (best_cost < 0 || cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && bn > best)) { best = bn; best_cost = cost; }
  }
  p.BN = best;
  p.stages = p.BN > 128 ? 4 : 6;
  p.n_taps = n_taps;
  p.splits = splits;
  p.kb_total = static_cast<int>((rows_a + BK - 1) / BK);
  for (int t = 0; t < MAX_TAPS; ++t) p.b_row_off[t] = t < n_taps ? b_row_off[t] : 0;
  p.out = out;
  p.status = status_buffer();
  p.boxed = 0;
  p.BW = p.BH = p.n_wb = p.n_hb = 1;
  for (int t = 0; t < MAX_TAPS; ++t) p.tap_c[t] = p.tap_w[t] = p.tap_par[t] = p.tap_h[t] = 0;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(rows_a)};
    uint64_t str[1] = {static_cast<uint64_t>(M) * 2};
    uint32_t box[2] = {64, BK};
    int rc = encode_tmap_bf16(&ta, dy, 2, dims, str, box);
    if (rc) return rc;
    uint64_t dimsb[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(rows_b)};
    uint64_t strb[1] = {static_cast<uint64_t>(N) * 2};
    rc = encode_tmap_bf16(&tb, x, 2, dimsb, strb, box);
    if (rc) return rc;
  }
  int smem = p.stages * (A_BYTES + p.BN * BK * 2) + 1024 + 256;
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: every CTA allocates all of TMEM
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  const long long items = static_cast<long long>(n_taps) * splits * ((M + BM - 1) / BM) * ((N + p.BN - 1) / p.BN);
  const int grid = items < sm_count() ? static_cast<int>(items) : sm_count();
  conv_wgrad_kernel<<<grid, NUM_THREADS, smem, static_cast<cudaStream_t>(stream_ptr)>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// The same products from the UNPADDED channels-last tensors. dy: [B, Ho, Wo, M] bf16 (strides in elements: dy_sb,
// dy_sh, dy_sw; channels dense); x: [B, H, W, C] bf16 with strides x_sb, x_sh, x_sw, N = C rounded up to 8 (the
// tensor itself must hold N channels). stride 1 or 2 (2 needs even H and W). taps: n_taps x {column parity (0 / 1),
// column shift, row parity, row shift} in units of the (possibly halved) grid of x; a K block is a BW x BH box of
// output pixels with BW * BH = 64. out: fp32 [n_taps, splits, M, N].
extern "C" int mdb_conv_wgrad_boxed(const void* dy, const void* x, float* out, int B, int Ho, int Wo, int H, int W, int M,
                                    int N, long long dy_sb, long long dy_sh, long long dy_sw, long long x_sb,
                                    long long x_sh, long long x_sw, int stride, int n_taps, const int* taps, int BW, int BH,
                                    int splits, void* stream_ptr) {
  using namespace mdb;
  using namespace mdb::wgrad;
  if (M <= 0 || N <= 0 || B <= 0 || Ho <= 0 || Wo <= 0) return 0;
  if ((M & 7) || (N & 7) || n_taps < 1 || n_taps > MAX_TAPS || splits < 1 || BW * BH != BK || BW > 256 || BH > 256) return 3801;
  if ((stride != 1 && stride != 2) || (stride == 2 && ((H | W) & 1))) return 3803;
  if ((dy_sb | dy_sh | dy_sw | x_sb | x_sh | x_sw) & 7) return 3804;
  Params p;
  p.M = M; p.N = N;
  int best = 64;
  double best_cost = -1.0;
  for (int bn = 64; bn <= 256; bn += 64) {
    const double cost = static_cast<double>((N + bn - 1) / bn * bn) * (1.0 + 64.0 / bn);
    if (best_cost < 0 || cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && bn > best)) { best = bn; best_cost = cost; }
  }
  p.BN = best;
  p.stages = p.BN > 128 ? 4 : 6;
  p.n_taps = n_taps;
  p.splits = splits;
  p.boxed = 1;
  p.BW = BW; p.BH = BH;
  p.n_wb = (Wo + BW - 1) / BW;
  p.n_hb = (Ho + BH - 1) / BH;
  p.kb_total = B * p.n_hb * p.n_wb;
  for (int t = 0; t < MAX_TAPS; ++t) {
    p.b_row_off[t] = 0;
    p.tap_c[t] = t < n_taps ? taps[4 * t] * N : 0;  // the column parity selects one half of the doubled channel axis
    p.tap_w[t] = t < n_taps ? taps[4 * t + 1] : 0;
    p.tap_par[t] = t < n_taps ? taps[4 * t + 2] : 0;
    p.tap_h[t] = t < n_taps ? taps[4 * t + 3] : 0;
  }
  p.out = out;
  p.status = status_buffer();
  CUtensorMap ta, tb;
  {
    uint64_t dims[5] = {static_cast<uint64_t>(M), static_cast<uint64_t>(Wo), 1, static_cast<uint64_t>(Ho), static_cast<uint64_t>(B)};
    uint64_t str[4] = {static_cast<uint64_t>(dy_sw) * 2, static_cast<uint64_t>(dy_sh) * 2, static_cast<uint64_t>(dy_sh) * 2,
                       static_cast<uint64_t>(dy_sb) * 2};
    uint32_t box[5] = {64, static_cast<uint32_t>(BW), 1, static_cast<uint32_t>(BH), 1};
    int rc = encode_tmap_bf16(&ta, dy, 5, dims, str, box);
    if (rc) return rc;
    // x: stride 1 -> [N, W, 1, H, B]; stride 2 -> [2N (column parity x channel), W/2, 2 (row parity), H/2, B]
    const int s = stride;
    uint64_t dimsb[5] = {static_cast<uint64_t>(N) * s, static_cast<uint64_t>(W / s), static_cast<uint64_t>(s),
                         static_cast<uint64_t>(H / s), static_cast<uint64_t>(B)};
    uint64_t strb[4] = {static_cast<uint64_t>(x_sw) * s * 2, static_cast<uint64_t>(x_sh) * 2, static_cast<uint64_t>(x_sh) * s * 2,
                        static_cast<uint64_t>(x_sb) * 2};
    if (stride == 2 && x_sw != N) return 3805;  // the column parity rides on the channel axis: pixels must be N apart
    rc = encode_tmap_bf16(&tb, x, 5, dimsb, strb, box);
    if (rc) return rc;
  }
  int smem = p.stages * (A_BYTES + p.BN * BK * 2) + 1024 + 256;
  if (smem < 120 * 1024) smem = 120 * 1024;
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  const long long items = static_cast<long long>(n_taps) * splits * ((M + BM - 1) / BM) * ((N + p.BN - 1) / p.BN);
  const int grid = items < sm_count() ? static_cast<int>(items) : sm_count();
  conv_wgrad_kernel<<<grid, NUM_THREADS, smem, static_cast<cudaStream_t>(stream_ptr)>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}
