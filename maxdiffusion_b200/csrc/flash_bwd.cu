// Flash-attention backward for head_dim 128 on sm_100a (tcgen05 + TMEM + TMA), as two
// deterministic passes built from one kernel template:
//
//   DKV pass : a CTA keeps one 128-key block (K_j, V_j) resident and streams 64-row blocks of
//              (Q_i, dO_i):  S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T  ->  dV += P^T dO, dK += dS^T Q
//   DQ  pass : a CTA keeps one 128-row block (Q_i, dO_i) resident and streams 64-key blocks of
//              (K_j, V_j) over every KV segment:  S = Q K^T, dP = dO V^T -> dS -> dQ += dS K
//
// with P = exp2(S*c - lse2) and dS = P * (dP - delta), delta = rowsum(dO * O). No atomics and no
// cross-CTA reduction are needed, so results are bitwise reproducible. The two score tiles of a
// step are double buffered in TMEM so the elementwise warps (16 warps, each warp group owns 16 of
// the 64 columns) overlap with the tensor core. The streamed tile is used twice from the same
// shared memory: as a K-major operand of the score MMAs and as an MN-major operand of the
// accumulating MMAs whose A operand (P^T / dS as packed bf16) is read from TMEM.
//
// Replaces the reference's fused Pallas-TPU backward `_flash_attention_dkv_kernel`
// (src/maxdiffusion/kernels/splash_attention/splash_attention_kernel.py:1394-1602, launcher :1605-1995)
// and the ring backward around it (ring_attention_kernel.py:181-289).
#include "host_common.h"

namespace mdb {
namespace fab {

constexpr int BX = 128;   // resident rows
constexpr int BY = 64;    // streamed rows per step
constexpr int Y_STAGES = 4;
// A tile is stored as head_dim / 64 chunks of 64 columns (128-byte rows, 128-byte swizzle).
constexpr int X_CHUNK_BYTES = BX * 128;         // 16 KiB
constexpr int Y_CHUNK_BYTES = BY * 128;         // 8 KiB
constexpr int MAX_SEGMENTS = 8;
constexpr int EW_GROUPS = 4;                    // elementwise warp groups, 16 of the 64 columns each
constexpr int NUM_THREADS = 128 + EW_GROUPS * 128;  // warp 0 TMA, warp 1 score MMAs, warp 2 accumulating MMAs, warps 4.. elementwise
template <int HD>
constexpr int smem_bytes() {
  return 2 * (HD / 64) * X_CHUNK_BYTES + Y_STAGES * 2 * (HD / 64) * Y_CHUNK_BYTES + Y_STAGES * 128 * 4 + 1024 + 256;
}

struct Maps {
  CUtensorMap x1, x2;
  CUtensorMap y1[MAX_SEGMENTS];
  CUtensorMap y2[MAX_SEGMENTS];
};

struct Params {
  int B, H;
  int x_len;                       // resident-side sequence length (kv_len for DKV, q_len for DQ)
  int num_segments;
  int y_len[MAX_SEGMENTS];         // streamed-side lengths (q_len for DKV; kv_len per segment for DQ)
  const float* lse;                // [B, H, q_len] log2 domain
  const float* delta;              // [B, H, q_len]
  int q_len;
  void* out0;                      // DKV: dV, DQ: dQ
  void* out1;                      // DKV: dK
  long long o0_sb, o0_ss, o0_sh, o1_sb, o1_ss, o1_sh;
  int out_f32;
  float scale, scale_log2;
  // DKV pass over several stacked KV segments in ONE launch (seg_batches > 0): blockIdx.z = seg * seg_batches + b
  // selects the K/V rows; queries, dO, lse and delta are those of batch b for every segment; the outputs of segment
  // seg go to slice (out_rot + seg * out_step) % n_seg of the output buffers, slices o_seg_stride elements apart.
  int seg_batches, n_seg, out_rot, out_step;
  int x_len_seg[MAX_SEGMENTS];
  long long o_seg_stride;
  DeviceStatus* status;
};

template <bool DKV, int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ Maps maps, const Params p) {
  constexpr int D = HD;                        // head_dim: 64 or 128
  constexpr int CH = HD / 64;                  // chunks per tile
  constexpr int X_TILE_BYTES = CH * X_CHUNK_BYTES;
  constexpr int Y_TILE_BYTES = CH * Y_CHUNK_BYTES;
  // Score-tile buffers: the hand-over chain score product -> elementwise -> accumulating product -> next score product
  // of one buffer is several times longer than the tensor work of a step, so the pipe is kept busy by the other
  // buffers. The DKV pass has TMEM for two (two accumulators), the DQ pass for three.
  constexpr int NBUF = DKV ? 2 : 3;
  constexpr uint32_t T2C = NBUF * 64, ACC = 2 * NBUF * 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sx1 = smem;
  uint8_t* sx2 = smem + X_TILE_BYTES;
  uint8_t* sy = smem + 2 * X_TILE_BYTES;  // [Y_STAGES][y1 | y2]
  float* stat_s = reinterpret_cast<float*>(sy + Y_STAGES * 2 * Y_TILE_BYTES);  // [Y_STAGES][lse 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stat_s + Y_STAGES * 128);
  uint64_t* x_full = bars;          // [1]
  uint64_t* y_full = bars + 1;                      // [Y_STAGES]
  uint64_t* y_empty = y_full + Y_STAGES;            // [Y_STAGES]
  uint64_t* t1_full = y_empty + Y_STAGES;           // [NBUF] first score tile (S) written
  uint64_t* t2_full = t1_full + NBUF;               // [NBUF] second score tile (dP) written
  uint64_t* p_ready = t2_full + NBUF;               // [NBUF] DKV: P^T stored over the first tile
  uint64_t* ds_ready = p_ready + NBUF;              // [NBUF] dS stored over the second tile
  uint64_t* t1_free = ds_ready + NBUF;              // [NBUF] first tile may be overwritten (DKV: dV product done; DQ: loaded)
  uint64_t* t2_free = t1_free + NBUF;               // [NBUF] second tile may be overwritten (dK / dQ product done)
  uint64_t* acc_final = t2_free + NBUF;             // [1]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_final + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int x0 = blockIdx.x * BX;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  int ybatch = batch;       // batch index of the streamed side, the statistics and the outputs
  int x_len = p.x_len;      // valid rows of the resident side
  long long o_base = 0;     // offset of the output slice
  if (DKV && p.seg_batches > 0) {
    const int seg = batch / p.seg_batches;
    ybatch = batch - seg * p.seg_batches;
    x_len = p.x_len_seg[seg];
    o_base = static_cast<long long>((p.out_rot + seg * p.out_step) % p.n_seg) * p.o_seg_stride;
  }

  int total_steps = 0;
  for (int s = 0; s < p.num_segments; ++s) total_steps += (p.y_len[s] + BY - 1) / BY;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int i = 0; i < Y_STAGES; ++i) {
      mbar_init(&y_full[i], 1);  // lane 0 of the producer: TMA transaction bytes (tiles, and lse / delta in the DKV pass)
      mbar_init(&y_empty[i], 1);
    }
    for (int i = 0; i < NBUF; ++i) {
      mbar_init(&t1_full[i], 1);
      mbar_init(&t2_full[i], 1);
      mbar_init(&p_ready[i], EW_GROUPS * 4);   // one elected lane per elementwise warp
      mbar_init(&ds_ready[i], EW_GROUPS * 4);
      mbar_init(&t1_free[i], DKV ? 1 : EW_GROUPS * 4);
      mbar_init(&t2_free[i], 1);
    }
    mbar_init(acc_final, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // TMEM columns: T1[b] = b*64, T2[b] = T2C + b*64, accumulators from ACC (DKV: 2 buffers, acc 256 / 384; DQ: 3 buffers, acc 384).

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // Lane 0 issues the TMA loads; in the DKV pass all 32 lanes also stage lse / delta of the 64
    // streamed query rows next to the tile, so their lifetime is that of the stage.
    if (total_steps > 0) {
      if (lane == 0) {
        mbar_expect_tx(x_full, 2 * X_TILE_BYTES);
        for (int c = 0; c < CH; ++c) {
          tma_load_4d(sx1 + c * X_CHUNK_BYTES, &maps.x1, x_full, c * 64, head, x0, batch);
          tma_load_4d(sx2 + c * X_CHUNK_BYTES, &maps.x2, x_full, c * 64, head, x0, batch);
        }
      }
      const long long stat_base = (static_cast<long long>(ybatch) * p.H + head) * p.q_len;
      // lse / delta of the streamed query rows ride in the stage. When the rows start on 16-byte boundaries they are
      // fetched by bulk copies that complete on the stage's barrier; otherwise the lanes copy them by hand.
      const bool stat_bulk = DKV && (p.q_len % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.lse) & 15) == 0) &&
                             ((reinterpret_cast<uintptr_t>(p.delta) & 15) == 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int seg = 0; seg < p.num_segments && ok; ++seg) {
        const int nblk = (p.y_len[seg] + BY - 1) / BY;
        for (int jb = 0; jb < nblk; ++jb) {
          if (!mbar_wait(&y_empty[stage], phase ^ 1u, abort_flag, p.status, 70)) { ok = false; break; }
          float* st = stat_s + stage * 128;
          const uint32_t stat_bytes = stat_bulk ? static_cast<uint32_t>(min(BY, p.q_len - jb * BY)) * 4u : 0u;
          if (DKV && !stat_bulk) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int qi = lane + 32 * h;
              const int q = jb * BY + qi;
              st[qi] = (q < p.q_len) ? p.lse[stat_base + q] : 0.0f;
              st[64 + qi] = (q < p.q_len) ? p.delta[stat_base + q] : 0.0f;
            }
            __syncwarp();
          }
          if (lane == 0) {
            uint8_t* d1 = sy + stage * 2 * Y_TILE_BYTES;
            uint8_t* d2 = d1 + Y_TILE_BYTES;
            mbar_expect_tx(&y_full[stage], 2 * Y_TILE_BYTES + 2 * stat_bytes);
            for (int c = 0; c < CH; ++c) {
              tma_load_4d(d1 + c * Y_CHUNK_BYTES, &maps.y1[seg], &y_full[stage], c * 64, head, jb * BY, ybatch);
              tma_load_4d(d2 + c * Y_CHUNK_BYTES, &maps.y2[seg], &y_full[stage], c * 64, head, jb * BY, ybatch);
            }
            if (stat_bytes) {
              bulk_load_1d(st, p.lse + stat_base + jb * BY, stat_bytes, &y_full[stage]);
              bulk_load_1d(st + 64, p.delta + stat_base + jb * BY, stat_bytes, &y_full[stage]);
            }
          }
          if (++stage == Y_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------ issuing lanes A1 / A2: score products ---------
    // Three lanes in different warps feed the tensor pipe: a step's waits, commits and MMA instructions cost an
    // issuing lane more cycles than the products take to execute. Warp 1 issues X1 Y1^T (S), warp 3 issues
    // X2 Y2^T (dP), warp 2 the accumulating products. Every dependency between them is an mbarrier.
    if (lane == 0 && total_steps > 0) {
      constexpr uint32_t idesc_t = make_idesc_bf16(128, BY, false, false);   // score tiles, N = 64
      const bool second = warp == 3;
      bool ok = mbar_wait(x_full, 0, abort_flag, p.status, 80);
      tc_fence_after_sync();
      // Shared-memory descriptors are built once: the address field (bits 0-13, units of 16 bytes) of a
      // descriptor advances by plain addition.
      const uint64_t xd = make_smem_desc(smem_u32(second ? sx2 : sx1), 16, 1024);
      const uint64_t ys0 = make_smem_desc(smem_u32(sy + (second ? Y_TILE_BYTES : 0)), 16, 1024);
      const uint32_t tcol = tmem_base + (second ? T2C : 0u);
      constexpr uint32_t STAGE_STEP = (2 * Y_TILE_BYTES) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < total_steps && ok; ++i) {
        const int b = i % NBUF, use = i / NBUF;
        const uint64_t yd = ys0 + stage * STAGE_STEP;
        if (!mbar_wait(&y_full[stage], phase, abort_flag, p.status, 81)) { ok = false; break; }
        // the buffer was last used by step i - NBUF: its reader (a product, or in the DQ pass the elementwise load of
        // the first tile) must be done
        if (use > 0 && !mbar_wait(second ? &t2_free[b] : &t1_free[b], (use - 1) & 1, abort_flag, p.status, 82)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t xo = ((k >> 2) * X_CHUNK_BYTES + (k & 3) * 32) >> 4;
          const uint32_t yo = ((k >> 2) * Y_CHUNK_BYTES + (k & 3) * 32) >> 4;
          umma_ss(tcol + b * 64, xd + xo, yd + yo, idesc_t, k > 0 ? 1u : 0u);
        }
        umma_commit(second ? &t2_full[b] : &t1_full[b]);
        if (++stage == Y_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 2) {
    // ------------------------------ issuing lane B: accumulating products --------
    if (lane == 0 && total_steps > 0) {
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, false, true); // B operand MN-major
      const uint64_t ym0 = make_smem_desc(smem_u32(sy), Y_CHUNK_BYTES, 1024);
      constexpr uint32_t STAGE_STEP = (2 * Y_TILE_BYTES) >> 4, TILE_STEP = Y_TILE_BYTES >> 4;
      int stage = 0;
      bool ok = true;
      for (int i = 0; i < total_steps && ok; ++i) {
        const int b = i % NBUF, use = i / NBUF;
        const uint64_t y1d = ym0 + stage * STAGE_STEP, y2d = y1d + TILE_STEP;
        if (DKV) {
          // dV += P^T dO_i as soon as P^T is stored; the first score tile is free afterwards
          if (!mbar_wait(&p_ready[b], use & 1, abort_flag, p.status, 83)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < BY / 16; ++k)  // packed bf16 columns of K-step k were written by column group k
            umma_ts(tmem_base + ACC, tmem_base + b * 64 + k * 16, y2d + k * (2048 >> 4), idesc_acc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(&t1_free[b]);
        }
        if (!mbar_wait(&ds_ready[b], use & 1, abort_flag, p.status, 84)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < BY / 16; ++k)  // DKV: dK += dS^T Q_i;  DQ: dQ += dS K_j
          umma_ts(tmem_base + ACC + (DKV ? 128 : 0), tmem_base + T2C + b * 64 + k * 16, y1d + k * (2048 >> 4), idesc_acc,
                  (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&t2_free[b]);
        umma_commit(&y_empty[stage]);
        if (++stage == Y_STAGES) stage = 0;
      }
      if (ok) umma_commit(acc_final);
    }
  } else if (warp >= 4) {
    // ------------------------------ Elementwise + epilogue --------------------
    const int wg = (warp - 4) >> 2;       // column group: 16 * wg .. +15
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int x_row = x0 + row_in_tile;
    const bool row_ok = x_row < x_len;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    if (total_steps > 0) {
      const long long stat_base = (static_cast<long long>(ybatch) * p.H + head) * p.q_len;
      float lse_r = 0.0f, delta_r = 0.0f;
      if (!DKV && row_ok) {
        lse_r = p.lse[stat_base + x_row];
        delta_r = p.delta[stat_base + x_row];
      }
      bool ok = true;
      int i = 0;
      for (int seg = 0; seg < p.num_segments && ok; ++seg) {
        const int nblk = (p.y_len[seg] + BY - 1) / BY;
        for (int jb = 0; jb < nblk; ++jb, ++i) {
          const int b = i % NBUF, use = i / NBUF;
          const int valid = min(BY, p.y_len[seg] - jb * BY);
          const int ystage = i % Y_STAGES;
          const float* st = stat_s + ystage * 128;
          if (DKV) {
            if (!mbar_wait(&y_full[ystage], (i / Y_STAGES) & 1, abort_flag, p.status, 92)) { ok = false; break; }
          }
          const bool full_tile = (valid == BY) && (x0 + BX <= x_len);  // uniform over the CTA
          const uint32_t t1a = tmem_base + lane_off + b * 64 + wg * 16;
          const uint32_t t2a = tmem_base + lane_off + T2C + b * 64 + wg * 16;
          // ---- phase 1: P of this thread's 16 columns from the first score tile
          if (!mbar_wait(&t1_full[b], use & 1, abort_flag, p.status, 90)) { ok = false; break; }
          if (!DKV) {  // the DQ pass has nothing to hand over between the tiles: one phase, both tiles loaded at once
            if (!mbar_wait(&t2_full[b], use & 1, abort_flag, p.status, 93)) { ok = false; break; }
          }
          tc_fence_after_sync();
          uint32_t t1[16], t2[16], ds[8];
          tmem_ld_x16(t1a, t1);
          if (!DKV) tmem_ld_x16(t2a, t2);
          tmem_wait_ld();
          if (!DKV) {  // nothing else reads the first tile in the DQ pass: the next S may be multiplied into it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&t1_free[b]);
          }
          float pr[16];
          if (full_tile) {
            if (DKV) {
              const float4* lse4 = reinterpret_cast<const float4*>(st + wg * 16);
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                const float4 l = lse4[c4];
                pr[4 * c4 + 0] = fast_exp2(__uint_as_float(t1[4 * c4 + 0]) * p.scale_log2 - l.x);
                pr[4 * c4 + 1] = fast_exp2(__uint_as_float(t1[4 * c4 + 1]) * p.scale_log2 - l.y);
                pr[4 * c4 + 2] = fast_exp2(__uint_as_float(t1[4 * c4 + 2]) * p.scale_log2 - l.z);
                pr[4 * c4 + 3] = fast_exp2(__uint_as_float(t1[4 * c4 + 3]) * p.scale_log2 - l.w);
              }
            } else {
#pragma unroll
              for (int c = 0; c < 16; ++c) pr[c] = fast_exp2(__uint_as_float(t1[c]) * p.scale_log2 - lse_r);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const int col = wg * 16 + c;
              const bool col_ok = col < valid;
              const float lse = DKV ? (col_ok ? st[col] : 0.0f) : lse_r;
              const float pe = fast_exp2(__uint_as_float(t1[c]) * p.scale_log2 - lse);
              pr[c] = (row_ok && col_ok) ? pe : 0.0f;
            }
          }
          if (DKV) {
            uint32_t pp[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) pp[c] = pack_bf16x2(pr[2 * c], pr[2 * c + 1]);
            tmem_st_x8(t1a, pp);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
          }
          // ---- phase 2: dS = P * (dP - delta) over the second score tile
          if (DKV) {
            if (!mbar_wait(&t2_full[b], use & 1, abort_flag, p.status, 93)) { ok = false; break; }
            tc_fence_after_sync();
            tmem_ld_x16(t2a, t2);
            tmem_wait_ld();
          }
          if (DKV) {
            if (full_tile) {
              const float4* del4 = reinterpret_cast<const float4*>(st + 64 + wg * 16);
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                const float4 d = del4[c4];
                ds[2 * c4] = pack_bf16x2(pr[4 * c4 + 0] * (__uint_as_float(t2[4 * c4 + 0]) - d.x),
                                         pr[4 * c4 + 1] * (__uint_as_float(t2[4 * c4 + 1]) - d.y));
                ds[2 * c4 + 1] = pack_bf16x2(pr[4 * c4 + 2] * (__uint_as_float(t2[4 * c4 + 2]) - d.z),
                                             pr[4 * c4 + 3] * (__uint_as_float(t2[4 * c4 + 3]) - d.w));
              }
            } else {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const int col = wg * 16 + 2 * c;
                const float d0 = col < valid ? st[64 + col] : 0.0f;
                const float d1 = col + 1 < valid ? st[64 + col + 1] : 0.0f;
                ds[c] = pack_bf16x2(pr[2 * c] * (__uint_as_float(t2[2 * c]) - d0),
                                    pr[2 * c + 1] * (__uint_as_float(t2[2 * c + 1]) - d1));
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 8; ++c)
              ds[c] = pack_bf16x2(pr[2 * c] * (__uint_as_float(t2[2 * c]) - delta_r),
                                  pr[2 * c + 1] * (__uint_as_float(t2[2 * c + 1]) - delta_r));
          }
          tmem_st_x8(t2a, ds);
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ds_ready[b]);
        }
      }
      if (ok && mbar_wait(acc_final, 0, abort_flag, p.status, 91)) {
        tc_fence_after_sync();
        // each column group writes a quarter of the output columns of every accumulator, 16 at a time
        const int n_acc = DKV ? 2 : 1;
        for (int a = 0; a < n_acc; ++a) {
          const float mul = (DKV && a == 0) ? 1.0f : p.scale;
          void* outp = a == 0 ? p.out0 : p.out1;
          const long long sb = a == 0 ? p.o0_sb : p.o1_sb, ss = a == 0 ? p.o0_ss : p.o1_ss,
                          sh = a == 0 ? p.o0_sh : p.o1_sh;
          const long long off = o_base + ybatch * sb + static_cast<long long>(x_row) * ss + head * sh;
#pragma unroll 1
          for (int c = 0; c < CH; ++c) {
            const int col0 = wg * (D / 4) + c * 16;
            uint32_t r[16];
            tmem_ld_x16(tmem_base + lane_off + ACC + a * 128 + col0, r);
            tmem_wait_ld();
            if (row_ok) {
              if (p.out_f32) {
                float* o = reinterpret_cast<float*>(outp) + off + col0;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  *reinterpret_cast<float4*>(o + v * 4) =
                      make_float4(__uint_as_float(r[v * 4]) * mul, __uint_as_float(r[v * 4 + 1]) * mul,
                                  __uint_as_float(r[v * 4 + 2]) * mul, __uint_as_float(r[v * 4 + 3]) * mul);
                }
              } else {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(outp) + off + col0;
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                  uint4 ov;
                  ov.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * mul, __uint_as_float(r[v * 8 + 1]) * mul);
                  ov.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * mul, __uint_as_float(r[v * 8 + 3]) * mul);
                  ov.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * mul, __uint_as_float(r[v * 8 + 5]) * mul);
                  ov.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * mul, __uint_as_float(r[v * 8 + 7]) * mul);
                  *reinterpret_cast<uint4*>(o + v * 8) = ov;
                }
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d]; one warp per (b,s,h) row of HD elements.
template <int HD>
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                             float* __restrict__ delta, int B, int S, int H, long long o_sb, long long o_ss,
                             long long o_sh, long long g_sb, long long g_ss, long long g_sh) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * S * H;
  if (row >= total) return;
  const int h = static_cast<int>(row % H);
  const long long bs = row / H;
  const int s = static_cast<int>(bs % S);
  const int b = static_cast<int>(bs / S);
  float acc;
  if (HD == 128) {
    const uint2 ov = *reinterpret_cast<const uint2*>(o + b * o_sb + s * o_ss + h * o_sh + lane * 4);
    const uint2 gv = *reinterpret_cast<const uint2*>(d_o + b * g_sb + s * g_ss + h * g_sh + lane * 4);
    const float2 o0 = unpack_bf16x2(ov.x), o1 = unpack_bf16x2(ov.y);
    const float2 g0 = unpack_bf16x2(gv.x), g1 = unpack_bf16x2(gv.y);
    acc = o0.x * g0.x + o0.y * g0.y + o1.x * g1.x + o1.y * g1.y;
  } else {
    const uint32_t ov = *reinterpret_cast<const uint32_t*>(o + b * o_sb + s * o_ss + h * o_sh + lane * 2);
    const uint32_t gv = *reinterpret_cast<const uint32_t*>(d_o + b * g_sb + s * g_ss + h * g_sh + lane * 2);
    const float2 o0 = unpack_bf16x2(ov), g0 = unpack_bf16x2(gv);
    acc = o0.x * g0.x + o0.y * g0.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * S + s] = acc;
}

static int make_map(CUtensorMap* map, const void* ptr, int D, int B, int S, int H, long long sb, long long ss, long long sh,
                    int box_rows) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                      static_cast<uint64_t>(B)};
  uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return encode_tmap_bf16(map, ptr, 4, dims, str, box);
}

template <int HD>
static int make_map_d(CUtensorMap* map, const void* ptr, int B, int S, int H, long long sb, long long ss, long long sh,
                      int box_rows) {
  return make_map(map, ptr, HD, B, S, H, sb, ss, sh, box_rows);
}

}  // namespace fab
}  // namespace mdb

using namespace mdb;
using namespace mdb::fab;

template <int HD>
static int flash_delta_launch(const void* o, const void* d_o, float* delta, int B, int S, int H, long long o_sb,
                              long long o_ss, long long o_sh, long long g_sb, long long g_ss, long long g_sh,
                              void* stream) {
  if ((o_sb | o_ss | o_sh | g_sb | g_ss | g_sh) & 3) return 3301;
  const long long rows = static_cast<long long>(B) * S * H;
  if (rows <= 0) return 0;
  const int blocks = static_cast<int>((rows * 32 + 255) / 256);
  delta_kernel<HD><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, B, S, H, o_sb, o_ss, o_sh,
      g_sb, g_ss, g_sh);
  return static_cast<int>(cudaGetLastError());
}

// dK, dV of one KV segment from all local queries. Strides in elements (batch, seq, head).
// q/dO share q strides `qs`, k/v share `ks`; outputs share `os`. out_f32 selects fp32 outputs.
template <int HD>
static int flash_bwd_dkv_launch(const void* q, const void* d_o, const void* k, const void* v, const float* lse,
                                const float* delta, void* dk, void* dv, int B, int H, int q_len, int kv_len,
                                const long long* qs, const long long* gs, const long long* ks, const long long* vs,
                                const long long* dks, const long long* dvs, float softmax_scale, int out_f32,
                                void* stream, int n_seg = 0, const int* seg_lens = nullptr, int out_rot = 0,
                                int out_step = 1, long long o_seg_stride = 0) {
  if (B <= 0 || H <= 0 || q_len <= 0 || kv_len <= 0) return 0;
  if (n_seg < 0 || n_seg > MAX_SEGMENTS || (n_seg > 0 && seg_lens == nullptr)) return 3250;
  // stacked form: K and V are [n_seg * B, kv_len, H, D] with one batch stride across segments
  const int x_batches = n_seg > 0 ? n_seg * B : B;
  Maps maps;
  Params p;
  int rc = make_map_d<HD>(&maps.x1, k, x_batches, kv_len, H, ks[0], ks[1], ks[2], BX);
  if (rc) return rc;
  rc = make_map_d<HD>(&maps.x2, v, x_batches, kv_len, H, vs[0], vs[1], vs[2], BX);
  if (rc) return rc;
  for (int s = 0; s < MAX_SEGMENTS; ++s) {
    rc = make_map_d<HD>(&maps.y1[s], q, B, q_len, H, qs[0], qs[1], qs[2], BY);
    if (rc) return rc;
    rc = make_map_d<HD>(&maps.y2[s], d_o, B, q_len, H, gs[0], gs[1], gs[2], BY);
    if (rc) return rc;
    p.y_len[s] = s == 0 ? q_len : 0;
  }
  p.B = B; p.H = H; p.x_len = kv_len; p.num_segments = 1;
  p.lse = lse; p.delta = delta; p.q_len = q_len;
  p.out0 = dv; p.out1 = dk;
  p.o0_sb = dvs[0]; p.o0_ss = dvs[1]; p.o0_sh = dvs[2];
  p.o1_sb = dks[0]; p.o1_ss = dks[1]; p.o1_sh = dks[2];
  p.out_f32 = out_f32;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.seg_batches = n_seg > 0 ? B : 0;
  p.n_seg = n_seg > 0 ? n_seg : 1;
  p.out_rot = n_seg > 0 ? ((out_rot % n_seg) + n_seg) % n_seg : 0;
  p.out_step = n_seg > 0 ? ((out_step % n_seg) + n_seg) % n_seg : 0;
  p.o_seg_stride = o_seg_stride;
  for (int s = 0; s < MAX_SEGMENTS; ++s) {
    const int len = (s < n_seg) ? seg_lens[s] : 0;
    if (len < 0 || len > kv_len) return 3250;
    p.x_len_seg[s] = len;
  }
  p.status = status_buffer();
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(flash_bwd_kernel<true, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<HD>()));
    configured = true;
  }
  dim3 grid((kv_len + BX - 1) / BX, H, x_batches);
  flash_bwd_kernel<true, HD><<<grid, NUM_THREADS, smem_bytes<HD>(), static_cast<cudaStream_t>(stream)>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

// dQ of the local queries over every KV segment.
template <int HD>
static int flash_bwd_dq_launch(const void* q, const void* d_o, const void* const* k_ptrs, const void* const* v_ptrs,
                               const float* lse, const float* delta, void* dq, int B, int H, int q_len,
                               int num_segments, const int* kv_lens, const long long* qs, const long long* gs,
                               const long long* ks, const long long* vs, const long long* dqs, float softmax_scale,
                               int out_f32, void* stream) {
  if (B <= 0 || H <= 0 || q_len <= 0) return 0;
  if (num_segments < 1 || num_segments > MAX_SEGMENTS) return 3302;
  Maps maps;
  Params p;
  int rc = make_map_d<HD>(&maps.x1, q, B, q_len, H, qs[0], qs[1], qs[2], BX);
  if (rc) return rc;
  rc = make_map_d<HD>(&maps.x2, d_o, B, q_len, H, gs[0], gs[1], gs[2], BX);
  if (rc) return rc;
  for (int s = 0; s < MAX_SEGMENTS; ++s) {
    const int src = s < num_segments ? s : 0;
    const int len = kv_lens[src] > 0 ? kv_lens[src] : 1;
    rc = make_map_d<HD>(&maps.y1[s], k_ptrs[src], B, len, H, ks[0], ks[1], ks[2], BY);
    if (rc) return rc;
    rc = make_map_d<HD>(&maps.y2[s], v_ptrs[src], B, len, H, vs[0], vs[1], vs[2], BY);
    if (rc) return rc;
    p.y_len[s] = s < num_segments ? kv_lens[s] : 0;
  }
  p.B = B; p.H = H; p.x_len = q_len; p.num_segments = num_segments;
  p.seg_batches = 0; p.n_seg = 1; p.out_rot = 0; p.out_step = 0; p.o_seg_stride = 0;
  for (int s = 0; s < MAX_SEGMENTS; ++s) p.x_len_seg[s] = 0;
  p.lse = lse; p.delta = delta; p.q_len = q_len;
  p.out0 = dq; p.out1 = nullptr;
  p.o0_sb = dqs[0]; p.o0_ss = dqs[1]; p.o0_sh = dqs[2];
  p.o1_sb = p.o1_ss = p.o1_sh = 0;
  p.out_f32 = out_f32;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status_buffer();
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(flash_bwd_kernel<false, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<HD>()));
    configured = true;
  }
  dim3 grid((q_len + BX - 1) / BX, H, B);
  flash_bwd_kernel<false, HD><<<grid, NUM_THREADS, smem_bytes<HD>(), static_cast<cudaStream_t>(stream)>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

// C entry points: head_dim 128, and `_d64` for head_dim 64 (Stable Diffusion / SDXL / LTX-Video heads).
#define MDB_FAB_ENTRY(SUFFIX, HD)                                                                                        \
  extern "C" int mdb_flash_delta##SUFFIX(const void* o, const void* d_o, float* delta, int B, int S, int H,               \
                                         long long o_sb, long long o_ss, long long o_sh, long long g_sb, long long g_ss,  \
                                         long long g_sh, void* stream) {                                                  \
    return flash_delta_launch<HD>(o, d_o, delta, B, S, H, o_sb, o_ss, o_sh, g_sb, g_ss, g_sh, stream);                    \
  }                                                                                                                       \
  extern "C" int mdb_flash_bwd_dkv##SUFFIX(const void* q, const void* d_o, const void* k, const void* v,                  \
                                           const float* lse, const float* delta, void* dk, void* dv, int B, int H,        \
                                           int q_len, int kv_len, const long long* qs, const long long* gs,               \
                                           const long long* ks, const long long* vs, const long long* dks,                \
                                           const long long* dvs, float softmax_scale, int out_f32, void* stream) {        \
    return flash_bwd_dkv_launch<HD>(q, d_o, k, v, lse, delta, dk, dv, B, H, q_len, kv_len, qs, gs, ks, vs, dks, dvs,      \
                                    softmax_scale, out_f32, stream);                                                      \
  }                                                                                                                       \
  extern "C" int mdb_flash_bwd_dkv_stacked##SUFFIX(                                                                      \
      const void* q, const void* d_o, const void* k, const void* v, const float* lse, const float* delta, void* dk,       \
      void* dv, int B, int H, int q_len, int kv_len, const long long* qs, const long long* gs, const long long* ks,       \
      const long long* vs, const long long* dks, const long long* dvs, float softmax_scale, int out_f32, void* stream,    \
      int n_seg, const int* seg_lens, int out_rot, int out_step, long long o_seg_stride) {                                \
    if (n_seg < 1) return 3250;                                                                                           \
    return flash_bwd_dkv_launch<HD>(q, d_o, k, v, lse, delta, dk, dv, B, H, q_len, kv_len, qs, gs, ks, vs, dks, dvs,      \
                                    softmax_scale, out_f32, stream, n_seg, seg_lens, out_rot, out_step, o_seg_stride);    \
  }                                                                                                                       \
  extern "C" int mdb_flash_bwd_dq##SUFFIX(const void* q, const void* d_o, const void* const* k_ptrs,                      \
                                          const void* const* v_ptrs, const float* lse, const float* delta, void* dq,      \
                                          int B, int H, int q_len, int num_segments, const int* kv_lens,                  \
                                          const long long* qs, const long long* gs, const long long* ks,                  \
                                          const long long* vs, const long long* dqs, float softmax_scale, int out_f32,    \
                                          void* stream) {                                                                 \
    return flash_bwd_dq_launch<HD>(q, d_o, k_ptrs, v_ptrs, lse, delta, dq, B, H, q_len, num_segments, kv_lens, qs, gs,    \
                                   ks, vs, dqs, softmax_scale, out_f32, stream);                                          \
  }
MDB_FAB_ENTRY(, 128)
MDB_FAB_ENTRY(_d64, 64)
