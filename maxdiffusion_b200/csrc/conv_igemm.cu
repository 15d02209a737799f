// Convolution as an implicit GEMM on sm_100a (tcgen05 + TMEM + TMA), channels-last, bf16 in / fp32 accumulate.
//
//     Y[pixel, co] = epilogue( sum_{tap, ci} X[pixel + shift(tap), ci] * W[co, tap, ci] )
//
// There is no im2col buffer and no gather pass. The activation tensor is described to TMA as a 5-D array
// (channels innermost) and an M-tile is a BOX of 128 output positions (e.g. 4 rows x 32 columns of one frame).
// The A operand of one (tap, channel block) step is that box fetched at coordinates shifted by the tap's offset:
// positions that fall outside the tensor are filled with zeros by TMA, which is exactly the zero padding of the
// convolution, and the box lands in shared memory as a K-major, 128-byte-swizzled 128 x 64 tile that `tcgen05.mma`
// consumes directly. The weights are a plain K-major matrix [Cout, taps * Cpad]. Everything that distinguishes one
// convolution from another is a table of tap offsets prepared on the host:
//   * 3x3x3 causal conv3d: 27 taps over (t, h, w); a tap that reaches before the chunk's first frame reads the
//     2-frame history ("feature cache") through a second tensor map, or zeros when there is none;
//   * 3x3 / 1x1 conv2d, (3,1,1) time convolution: the same with fewer taps;
//   * stride 2: the input is viewed as [.., H/2, 2, W/2, 2*C], so that a tap becomes (row pair, parity, column pair,
//     parity * C + channel) and the box stays dense;
//   * nearest-2x upsample + 3x3 conv: four output-parity classes, each a 2x2 convolution of the LOW resolution
//     input with pre-summed weights (2.25x fewer FLOPs than up-sampling first), written with stride 2.
// Roles per CTA (persistent, one per SM): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..5 epilogue
// (bias, SiLU, residual add, ragged-edge masking). Accumulators are double buffered in TMEM.
// Channel counts that are not multiples of 64 (96, 192, 320) cost no tensor work: the last channel block is
// fetched with zero fill and only its valid 16-wide K steps are issued.
// The lane that issues the MMAs pays a fixed price per pipeline stage (barrier wait, fence, commit: several hundred
// cycles) besides the price per instruction, and with few output channels (N <= 128) a stage of one 64-channel block
// holds less tensor work than that. Narrow tiles therefore put TWO (tap, channel block) units into a stage.
//
// Replaces the XLA:GPU / cuDNN convolutions behind the reference's `WanCausalConv3d`, `WanResample`,
// `WanResidualBlock` (src/maxdiffusion/models/wan/autoencoder_kl_wan.py:70-147, 245-389, 452-484) and the UNet /
// VAE `nn.Conv` layers (src/maxdiffusion/models/resnet_flax.py:37-186).
#include "host_common.h"

namespace mdb {
namespace conv {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int NUM_THREADS = 192;
constexpr int MAX_STAGES = 6;
constexpr int MAX_TAPS = 36;      // 27 (3x3x3) or 4 classes x 9
constexpr int MAX_CLASSES = 4;
// TMEM columns per accumulator: 256 (two accumulators = all 512 columns, one CTA per SM) for wide tiles, 128 for
// tiles of at most 128 output channels, which run TWO CTAs per SM (256 columns and half the shared memory each).
// One thread can issue a tcgen05.mma only every ~100 ns whatever its width, so with narrow tiles a single issuing
// lane leaves the tensor pipe half idle; two co-resident CTAs are two issuing lanes, each tile still accumulated
// by one thread in a fixed order (bitwise reproducible).

struct Tap {
  int o0;              // added to the channel coordinate (parity * C in the stride-2 view, else 0)
  short o1, o2, o3, o4;  // added to the tile's base coordinates along dims 1..4
  int koff;            // first K index of this tap in the weight matrix
};

enum Epilogue : int { kEpiNone = 0, kEpiSilu = 1 };

struct Params {
  int n_classes;
  int tap_begin[MAX_CLASSES + 1];
  Tap taps[MAX_TAPS];
  int box1, box2, box3;          // tile extents along dims 1..3, product 128
  int ext1, ext2, ext3, ext4;    // output positions along dims 1..4 (per class)
  int C;                         // input channels, multiple of 16
  int N;                         // output channels, multiple of 8
  int BN;                        // tile width: multiple of 16, <= 256
  int stages;
  int ups;                       // (tap, channel block) units per pipeline stage: 1 or 2
  int acc_cols;                  // TMEM columns per accumulator: 128 or 256
  int alt_dim, alt_shift, has_alt;  // a tap whose coordinate along alt_dim is negative reads the second map at +alt_shift
  long long os1, os2, os3, os4;  // output strides (elements) along dims 1..4
  long long class_off[MAX_CLASSES];
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;      // [N] or nullptr
  const __nv_bfloat16* residual;  // addressed like out, or nullptr
  int epi;
  DeviceStatus* status;
};

struct TileCoord {
  int cls, n_idx, m1, m2, m3, m4;
};

__device__ __forceinline__ TileCoord decode_tile(int tile, const Params& p, int nt1, int nt2, int nt3, int num_n) {
  TileCoord c;
  c.n_idx = tile % num_n; tile /= num_n;
  c.m1 = (tile % nt1) * p.box1; tile /= nt1;
  c.m2 = (tile % nt2) * p.box2; tile /= nt2;
  c.m3 = (tile % nt3) * p.box3; tile /= nt3;
  c.m4 = tile % p.ext4; tile /= p.ext4;
  c.cls = tile;
  return c;
}

__global__ void __launch_bounds__(NUM_THREADS, 2)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_alt,
                  const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int STAGES = p.stages;
  const int B_BYTES = p.BN * BK * 2;
  const int UNIT_BYTES = A_BYTES + B_BYTES;   // a multiple of 1024: BN is a multiple of 16
  const int STAGE_BYTES = p.ups * UNIT_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                          // [MAX_STAGES]
  uint64_t* empty_bar = bars + MAX_STAGES;            // [MAX_STAGES]
  uint64_t* tmem_full = bars + 2 * MAX_STAGES;        // [2]
  uint64_t* tmem_empty = bars + 2 * MAX_STAGES + 2;   // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nt1 = (p.ext1 + p.box1 - 1) / p.box1;
  const int nt2 = (p.ext2 + p.box2 - 1) / p.box2;
  const int nt3 = (p.ext3 + p.box3 - 1) / p.box3;
  const int num_n = (p.N + p.BN - 1) / p.BN;
  const int num_tiles = p.n_classes * p.ext4 * nt3 * nt2 * nt1 * num_n;
  const int num_kb = (p.C + BK - 1) / BK;

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
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_w);
  }
  const int ACC_COLS = p.acc_cols;
  if (warp == 1) {
    tmem_alloc(tmem_ptr_smem, 2 * ACC_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile(tile, p, nt1, nt2, nt3, num_n);
        const int n0 = tc.n_idx * p.BN;
        const int t0 = p.tap_begin[tc.cls];
        const int n_units = (p.tap_begin[tc.cls + 1] - t0) * num_kb;
        int ti = t0, kb = 0;
        Tap tap = p.taps[ti];
        for (int u0 = 0; u0 < n_units && ok; u0 += p.ups) {
          const int nu = min(p.ups, n_units - u0);
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 110)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], nu * UNIT_BYTES);
          uint8_t* sa = smem + stage * STAGE_BYTES;
          for (int j = 0; j < nu; ++j, sa += UNIT_BYTES) {
            int c1 = tc.m1 + tap.o1, c2 = tc.m2 + tap.o2, c3 = tc.m3 + tap.o3, c4 = tc.m4 + tap.o4;
            const CUtensorMap* map = &tmap_x;
            if (p.has_alt) {
              // a tap that reaches before the first position along alt_dim reads the history tensor instead
              if (p.alt_dim == 3 && c3 < 0) { c3 += p.alt_shift; map = &tmap_alt; }
              else if (p.alt_dim == 2 && c2 < 0) { c2 += p.alt_shift; map = &tmap_alt; }
            }
            tma_load_5d(sa, map, &full_bar[stage], tap.o0 + kb * BK, c1, c2, c3, c4);
            tma_load_2d(sa + A_BYTES, &tmap_w, &full_bar[stage], tap.koff + kb * BK, n0);
            if (++kb == num_kb) {
              kb = 0;
              ++ti;
              if (ti < p.tap_begin[tc.cls + 1]) tap = p.taps[ti];
            }
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give the copies already in flight a bounded chance to land before the CTA exits.
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          int s = (stage - 1 - i + 2 * STAGES) % STAGES;
          uint32_t ph = (i < stage) ? phase : (phase ^ 1u);
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(&full_bar[s], ph); ++spin) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, p.BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int cls = tile / (num_tiles / p.n_classes);
        const int n_taps = p.tap_begin[cls + 1] - p.tap_begin[cls];
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 120)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        uint32_t accumulate = 0;
        const int n_units = n_taps * num_kb;
        // this lane is the critical resource of the kernel: no divisions, descriptors advance by addition
        const int last_ksteps = (p.C - (num_kb - 1) * BK + 15) / 16;
        int kb = 0;
        for (int u0 = 0; u0 < n_units; u0 += p.ups) {
          const int nu = min(p.ups, n_units - u0);
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 121)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          for (int j = 0; j < nu; ++j, sa += UNIT_BYTES) {
            const uint64_t da = make_smem_desc(sa, 16, 1024);
            const uint64_t db = make_smem_desc(sa + A_BYTES, 16, 1024);
            const bool last = (kb + 1 == num_kb);
            if (!last || last_ksteps == BK / 16) {
              // one K step (16 bf16 = 32 bytes) advances the descriptors' address field (units of 16 bytes) by 2
              umma_ss(d_tmem, da, db, idesc, accumulate);
              umma_ss(d_tmem, da + 2, db + 2, idesc, 1u);
              umma_ss(d_tmem, da + 4, db + 4, idesc, 1u);
              umma_ss(d_tmem, da + 6, db + 6, idesc, 1u);
            } else {
              for (int k = 0; k < last_ksteps; ++k) umma_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, k ? 1u : accumulate);
            }
            accumulate = 1u;
            kb = last ? 0 : kb + 1;
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------ Epilogue ----------------------------------
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are reachable from this warp
    const int r = quarter * 32 + lane;
    const int r1 = r % p.box1;
    const int r2 = (r / p.box1) % p.box2;
    const int r3 = r / (p.box1 * p.box2);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      const TileCoord tc = decode_tile(tile, p, nt1, nt2, nt3, num_n);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, 130)) { ok = false; break; }
      tc_fence_after_sync();
      const int p1 = tc.m1 + r1, p2 = tc.m2 + r2, p3 = tc.m3 + r3;
      const bool row_ok = p1 < p.ext1 && p2 < p.ext2 && p3 < p.ext3;
      const long long off = tc.m4 * p.os4 + p3 * p.os3 + p2 * p.os2 + p1 * p.os1 + p.class_off[tc.cls];
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * ACC_COLS;
      const int n0 = tc.n_idx * p.BN;
#pragma unroll 1
      for (int c = 0; c < p.BN / 16; ++c) {
        const int col0 = n0 + c * 16;
        if (col0 >= p.N) break;  // uniform across the CTA
        uint32_t v[16];
        tmem_ld_x16(taddr + c * 16, v);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col = col0 + h * 8;
            if (col >= p.N) break;
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[h * 8 + j]);
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
            if (p.epi == kEpiSilu) {
#pragma unroll
              for (int j = 0; j < 8; ++j) x[j] = x[j] / (1.0f + __expf(-x[j]));
            }
            if (p.residual) {
              const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + off + col);
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16x2(rw[j]);
                x[2 * j] += f.x;
                x[2 * j + 1] += f.y;
              }
            }
            uint4 ov;
            ov.x = pack_bf16x2(x[0], x[1]);
            ov.y = pack_bf16x2(x[2], x[3]);
            ov.z = pack_bf16x2(x[4], x[5]);
            ov.w = pack_bf16x2(x[6], x[7]);
            *reinterpret_cast<uint4*>(p.out + off + col) = ov;
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

// Tile width for N output channels: the multiple of 16 (<= 256) that wastes the fewest padded columns, the widest
// among equals (a wider tile moves fewer operand bytes per FLOP).
static int pick_bn(int N) {
  int best = 16;
  long long best_cost = -1;
  for (int bn = 16; bn <= 256; bn += 16) {
    const long long cost = static_cast<long long>((N + bn - 1) / bn) * bn;
    if (best_cost < 0 || cost < best_cost || (cost == best_cost && bn > best)) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

}  // namespace conv
}  // namespace mdb

// Tuning overrides for the tile search and the benchmarks (0 = the launcher's own choice): units per stage (1 / 2),
// an upper limit on the pipeline stages, CTAs per SM (1 / 2; 2 only applies to tiles of at most 128 channels).
static int g_tune_ups = 0, g_tune_stages = 0, g_tune_ctas = 0;

extern "C" int mdb_conv_igemm_tune(int ups, int stages, int ctas_per_sm) {
  if (ups < 0 || ups > 2 || stages < 0 || stages > 6 || ctas_per_sm < 0 || ctas_per_sm > 2) return 3609;
  g_tune_ups = ups;
  g_tune_stages = stages;
  g_tune_ctas = ctas_per_sm;
  return 0;
}

// Generic entry point; `ops/conv.py` builds the descriptions for the concrete convolutions.
//   x / x_alt : activation tensor and optional history tensor, both seen as 5-D arrays with `dims` / `alt_dims`
//               (innermost first, dim 0 = channels, contiguous) and element strides `strides` / `alt_strides` of dims 1..4
//   w         : [N, k_total] bf16, row-major (K-major); the K range of tap i starts at taps[i].koff and spans Cpad
//   box       : tile extents along dims 1..3 (product 128);  ext: output positions along dims 1..4
//   taps      : n_taps_total x 6 ints (o0, o1, o2, o3, o4, koff);  tap_begin: n_classes + 1 ints
//   out_strides (dims 1..4, elements), class_off (n_classes): where output position (p1..p4) of a class goes
// All channel counts and strides must keep 16-byte alignment (multiples of 8 elements); C a multiple of 16.
extern "C" int mdb_conv_igemm(const void* x, const void* x_alt, const void* w, void* out, const void* bias,
                              const void* residual, const long long* dims, const long long* strides,
                              const long long* alt_dims, const long long* alt_strides, const int* box, const int* ext,
                              int C, int N, long long k_total, int n_classes, const int* tap_begin, const int* taps,
                              int alt_dim, int alt_shift, const long long* out_strides, const long long* class_off,
                              int epi, void* stream_ptr) {
  using namespace mdb;
  using namespace mdb::conv;
  if (n_classes < 1 || n_classes > MAX_CLASSES) return 3601;
  const int n_taps = tap_begin[n_classes];
  if (n_taps < 1 || n_taps > MAX_TAPS) return 3602;
  if ((C & 15) || (N & 7) || C <= 0 || N <= 0) return 3603;
  if (box[0] * box[1] * box[2] != BM || box[0] > 256 || box[1] > 256 || box[2] > 256) return 3604;
  for (int i = 0; i < 4; ++i) {
    if (ext[i] <= 0) return 0;  // nothing to compute
    if ((strides[i] & 7) || (out_strides[i] & 7)) return 3605;
  }
  if (k_total & 7) return 3605;
  Params p;
  p.n_classes = n_classes;
  for (int c = 0; c <= MAX_CLASSES; ++c) p.tap_begin[c] = tap_begin[c <= n_classes ? c : n_classes];
  for (int c = 0; c < n_classes; ++c) {
    if (tap_begin[c + 1] <= tap_begin[c]) return 3602;
    p.class_off[c] = class_off[c];
    if (class_off[c] & 7) return 3605;
  }
  for (int i = 0; i < n_taps; ++i) {
    const int* t = taps + 6 * i;
    if (t[0] & 7) return 3606;  // the innermost TMA coordinate must stay 16-byte aligned
    p.taps[i].o0 = t[0];
    p.taps[i].o1 = static_cast<short>(t[1]);
    p.taps[i].o2 = static_cast<short>(t[2]);
    p.taps[i].o3 = static_cast<short>(t[3]);
    p.taps[i].o4 = static_cast<short>(t[4]);
    p.taps[i].koff = t[5];
    if (t[5] & 7) return 3606;
  }
  p.box1 = box[0]; p.box2 = box[1]; p.box3 = box[2];
  p.ext1 = ext[0]; p.ext2 = ext[1]; p.ext3 = ext[2]; p.ext4 = ext[3];
  p.C = C; p.N = N;
  p.BN = pick_bn(N);
  const int unit_bytes = A_BYTES + p.BN * BK * 2;
  int ctas_per_sm = p.BN <= 128 ? 2 : 1;
  if (g_tune_ctas > 0) ctas_per_sm = (g_tune_ctas == 2 && p.BN <= 128) ? 2 : 1;
  p.acc_cols = ctas_per_sm == 2 ? 128 : 256;
  const int budget = (ctas_per_sm == 2 ? 112 : 226) * 1024 - 1024 - 256;
  p.ups = g_tune_ups > 0 ? g_tune_ups : (ctas_per_sm == 2 ? 1 : (p.BN <= 128 ? 2 : 1));
  if (p.ups < 1 || p.ups > 2) return 3608;
  p.stages = budget / (p.ups * unit_bytes);
  if (g_tune_stages > 0 && g_tune_stages < p.stages) p.stages = g_tune_stages;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  if (p.stages < 2) return 3608;
  p.alt_dim = alt_dim; p.alt_shift = alt_shift; p.has_alt = (x_alt != nullptr && alt_dim >= 2 && alt_dim <= 3) ? 1 : 0;
  p.os1 = out_strides[0]; p.os2 = out_strides[1]; p.os3 = out_strides[2]; p.os4 = out_strides[3];
  p.out = static_cast<__nv_bfloat16*>(out);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.epi = epi;
  p.status = status_buffer();

  CUtensorMap tx, talt, tw;
  {
    uint64_t d[5], s[4];
    uint32_t b[5] = {BK, static_cast<uint32_t>(box[0]), static_cast<uint32_t>(box[1]), static_cast<uint32_t>(box[2]), 1};
    for (int i = 0; i < 5; ++i) d[i] = static_cast<uint64_t>(dims[i]);
    for (int i = 0; i < 4; ++i) s[i] = static_cast<uint64_t>(strides[i]) * 2;
    int rc = encode_tmap_bf16(&tx, x, 5, d, s, b);
    if (rc) return rc;
    if (p.has_alt) {
      if ((alt_strides[0] | alt_strides[1] | alt_strides[2] | alt_strides[3]) & 7) return 3605;
      for (int i = 0; i < 5; ++i) d[i] = static_cast<uint64_t>(alt_dims[i]);
      for (int i = 0; i < 4; ++i) s[i] = static_cast<uint64_t>(alt_strides[i]) * 2;
      rc = encode_tmap_bf16(&talt, x_alt, 5, d, s, b);
      if (rc) return rc;
    } else {
      talt = tx;
    }
    uint64_t wd[2] = {static_cast<uint64_t>(k_total), static_cast<uint64_t>(N)};
    uint64_t ws[1] = {static_cast<uint64_t>(k_total) * 2};
    uint32_t wb[2] = {BK, static_cast<uint32_t>(p.BN)};
    rc = encode_tmap_bf16(&tw, w, 2, wd, ws, wb);
    if (rc) return rc;
  }
  int smem = p.stages * p.ups * unit_bytes + 1024 + 256;
  // the shared-memory request decides how many CTAs share an SM; it has to agree with the TMEM each one allocates
  if (ctas_per_sm == 1 && smem < 120 * 1024) smem = 120 * 1024;
  if (ctas_per_sm == 2 && smem < 80 * 1024) smem = 80 * 1024;
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(conv_igemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  const auto cdiv = [](long long a, long long b) { return (a + b - 1) / b; };
  const long long tiles = static_cast<long long>(n_classes) * ext[3] * cdiv(ext[2], box[2]) * cdiv(ext[1], box[1]) *
                          cdiv(ext[0], box[0]) * cdiv(N, p.BN);
  if (tiles >= (1ll << 31)) return 3607;
  const long long slots = static_cast<long long>(sm_count()) * ctas_per_sm;
  const int grid = tiles < slots ? static_cast<int>(tiles) : static_cast<int>(slots);
  conv_igemm_kernel<<<grid, NUM_THREADS, smem, static_cast<cudaStream_t>(stream_ptr)>>>(tx, talt, tw, p);
  return static_cast<int>(cudaGetLastError());
}
