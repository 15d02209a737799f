// Persistent, warp-specialised bf16 GEMM for sm_100a:
//     D[M,N] = epilogue( A[M,K] * B[N,K]^T )
// Operands come through (non-multicast) TMA into 128-byte-swizzled shared memory, the product is
// issued by one thread with tcgen05.mma (128 x 256 x 16 per instruction), fp32 accumulators sit in
// TMEM and are double buffered (2 x 256 columns) so that the epilogue of tile i overlaps the main
// loop of tile i+1.
//
// Either operand may be "MN-major" (stored transposed, i.e. A as [K,M] or B as [K,N]); this is what
// lets dgrad (dX = dY * W) and wgrad (dW = dY^T * X) run on the same kernel without transposes.
//
// Roles:  warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 and 6..9 = two epilogue groups, each
// taking one column half of every tile (own staging slab, named barrier and TMA-store issuing thread).
// Covers the reference's XLA:GPU / cuBLAS matmuls behind every Dense layer
// (src/maxdiffusion/models/attention_flax.py:2471-2525, models/wan/transformers/transformer_wan.py:220-330)
// together with the elementwise fusions XLA places after them (bias, GELU-tanh, gated residual).
#include "host_common.h"

namespace mdb {

namespace gemm {
constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int NUM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..5 and 6..9: two epilogue groups (one column half each)
constexpr int GROUP_M = 8;
// The tile is 128 x BN with BN = 256 (the default) or 128 (on request). The narrower tile fills the waves of the
// 148 persistent CTAs better at small M, but it moves a third more operand bytes per FLOP from L2 into shared
// memory and measured 1.3-1.5x SLOWER on every shape of an 8-way sequence split (4095 x 5120 x 5120: 0.228 ms
// against 0.173 ms), so the launcher never picks it by itself: operand traffic, not wave fill, is the limit.
__host__ __device__ constexpr int stages_for(int bn) { return bn == 256 ? 4 : 6; }                    // 4 x 48 KiB or 6 x 32 KiB
__host__ __device__ constexpr int stage_bytes(int bn) { return A_BYTES + bn * BK * 2; }
// Output staging of the epilogue: one 128-row x 128-byte slab (64 bf16 or 32 fp32 columns) per epilogue group in the
// 128-byte swizzle, written by the group's warps and drained by its TMA stores.
constexpr int SLAB_BYTES = BM * 128;
constexpr int STAGING_BYTES = 2 * SLAB_BYTES;
constexpr int BIAS_BYTES = 256 * 4;  // the tile's bias columns as fp32
__host__ __device__ constexpr int smem_bytes(int bn) {
  return stages_for(bn) * stage_bytes(bn) + STAGING_BYTES + BIAS_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
}

enum Epilogue : int {
  kEpiNone = 0,       // out = acc*alpha + bias
  kEpiGeluTanh = 1,   // out = gelu_tanh(acc*alpha + bias)
  kEpiGatedRes = 2,   // out = residual + gate[batch(row), col] * (acc*alpha + bias)
  kEpiSilu = 3,       // out = silu(acc*alpha + bias)
  kEpiAddRes = 4,     // out = residual + acc*alpha + bias
};

struct Params {
  int M, N, K;
  void* out;
  long long ldo;
  const __nv_bfloat16* bias;      // [N] or nullptr
  const __nv_bfloat16* residual;  // [M, ldr] or nullptr
  long long ldr;
  const float* gate;              // [num_batches, gate_ld] fp32 or nullptr
  long long gate_ld;
  int rows_per_batch;
  int epi;
  int out_f32;
  float alpha;
  DeviceStatus* status;
  // split-K (weight gradients: a small output with a long contraction): work item w covers k-blocks
  // [split * kb_per_split, ..) of tile w % num_tiles with split = w / num_tiles and writes fp32 partials
  // [splits, M, N]; `splitk_fold_kernel` sums them in split order (deterministic, no atomics)
  int splits;
  int kb_per_split;
  float* partial;
  int partial_rows;  // rows per split in `partial` (M rounded up to the tile height when TMA stores write it)
  // 1: the epilogue stages 128-byte-wide slabs in shared memory and writes them with TMA stores (full lines, clipped
  // at the edges of the tensor) instead of 16-byte stores from one thread per row
  int tma_store;
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_idx, int& n_idx) {
  // Grouped rasterisation: GROUP_M row-blocks share each sweep over the column-blocks so that
  // concurrently running CTAs reuse both operands out of L2.
  const int tiles_per_group = GROUP_M * num_n;
  const int group = tile / tiles_per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int local = tile - group * tiles_per_group;
  m_idx = first_m + local % rows;
  n_idx = local / rows;
}

template <bool A_MN, bool B_MN, int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  constexpr int STAGES = stages_for(BN);
  constexpr int STAGE_BYTES = stage_bytes(BN);
  constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // 1024-byte aligned: every stage is a multiple of 1024 bytes
  float* bias_s = reinterpret_cast<float*>(staging + STAGING_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + STAGING_BYTES + BIAS_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;      // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_work = num_tiles * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 256);  // both epilogue groups have read the accumulator
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if (p.tma_store) prefetch_tensormap(&tmap_c);
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
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        int m_idx, n_idx;
        const int split = work / num_tiles;
        tile_coords(work - split * num_tiles, num_m, num_n, m_idx, n_idx);
        const int m0 = m_idx * BM, n0 = n_idx * BN;
        const int kb_begin = split * p.kb_per_split, kb_end = min(num_kb, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 10)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmap_a, &full_bar[stage], m0 + c * 64, k0);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmap_b, &full_bar[stage], n0 + c * 64, k0);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
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
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 20)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb_begin = (work / num_tiles) * p.kb_per_split, kb_end = min(num_kb, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 21)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            umma_ss(d_tmem, da, db, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------ Epilogue ----------------------------------
    // Two groups of four warps share a tile: group g takes the columns [g BN/2, (g + 1) BN/2). With short
    // contractions (10-20 K blocks) a tile's epilogue lasts as long as its main loop; two groups halve it. Each group
    // has its own staging slab, named barrier and store-issuing thread.
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are reachable from this warp
    const int row_in_tile = quarter * 32 + lane;
    const int egroup = (warp - 2) >> 2;
    const int group_thread = static_cast<int>(threadIdx.x) - 64 - egroup * 128;
    const int col_begin = egroup * (BN / 2), col_end = col_begin + BN / 2;
    int it = 0;
    bool ok = true;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x, ++it) {
      int m_idx, n_idx;
      const int split = work / num_tiles;
      tile_coords(work - split * num_tiles, num_m, num_n, m_idx, n_idx);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, 30)) { ok = false; break; }
      tc_fence_after_sync();
      const long long row = static_cast<long long>(m_idx) * BM + row_in_tile;
      const bool row_ok = row < p.M;
      const int batch = (p.rows_per_batch > 0) ? static_cast<int>(row / p.rows_per_batch) : 0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (p.tma_store) {
        // ---- staged epilogue: 128 bytes of every row per slab, swizzled, one TMA store per slab ----
        const bool f32 = p.out_f32 || p.splits > 1;
        const int slab_cols = f32 ? 32 : 64;
        const bool leader = group_thread == 0;  // the group's first thread issues and tracks its stores
        const long long out_row0 = (p.splits > 1 ? static_cast<long long>(split) * p.partial_rows : 0) +
                                   static_cast<long long>(m_idx) * BM;
        const int sw = row_in_tile & 7;
        const bool use_bias = p.bias != nullptr && p.splits == 1;
        const bool res_epi = (p.epi == kEpiGatedRes || p.epi == kEpiAddRes) && p.splits == 1;
        // bf16 output: the residual slab is fetched by coalesced loads (8 lanes per 128-byte row) and handed to the
        // row-owning threads through the staging slab; a warp touches only its own 32 rows, so a warp sync suffices
        const bool res_staged = res_epi && !f32;
        if (use_bias) {
          // the tile's bias columns once, as fp32 (the previous tile's readers passed its last slab barrier)
          for (int c = col_begin + group_thread; c < col_end; c += 128) {
            const int col = n_idx * BN + c;
            bias_s[c] = col < p.N ? __bfloat162float(p.bias[col]) : 0.0f;
          }
        }
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end; c0 += slab_cols) {
          const int col0 = n_idx * BN + c0;
          if (col0 >= p.N) break;  // uniform across the group
          uint8_t* slab = staging + egroup * SLAB_BYTES;
          uint4 rv[8];
          if (res_staged) {  // issued before the barrier: their latency overlaps the wait for the slab
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = quarter * 32 + i * 4 + (lane >> 3);
              const long long grow = static_cast<long long>(m_idx) * BM + rl;
              const int gcol = col0 + (lane & 7) * 8;
              rv[i] = (grow < p.M && gcol < p.N) ? *reinterpret_cast<const uint4*>(p.residual + grow * p.ldr + gcol)
                                                 : make_uint4(0u, 0u, 0u, 0u);
            }
          }
          if (leader) tma_store_wait_read<0>();  // the group's previous store is done reading the slab
          named_bar_sync(1 + egroup, 128);
          if (res_staged) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = quarter * 32 + i * 4 + (lane >> 3);
              *reinterpret_cast<uint4*>(slab + rl * 128 + ((((lane & 7) ^ (rl & 7))) << 4)) = rv[i];
            }
            __syncwarp();
          }
          uint8_t* my_row = slab + row_in_tile * 128;
#pragma unroll
          for (int h = 0; h < 2; ++h) {  // bf16: two 32-column loads per slab; fp32: one
            if (f32 && h == 1) break;
            uint32_t r[32];
            tmem_ld_x32(taddr + c0 + h * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = col0 + h * 32 + v * 8;
              float x[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(r[v * 8 + j]) * p.alpha;
              if (p.splits == 1 && col < p.N) {
                if (use_bias) {
                  const float4 b0 = *reinterpret_cast<const float4*>(bias_s + c0 + h * 32 + v * 8);
                  const float4 b1 = *reinterpret_cast<const float4*>(bias_s + c0 + h * 32 + v * 8 + 4);
                  x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w;
                  x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
                }
                if (p.epi == kEpiGeluTanh) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) x[j] = gelu_tanh(x[j]);
                } else if (p.epi == kEpiSilu) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) x[j] = x[j] / (1.0f + __expf(-x[j]));
                } else if (res_epi && row_ok) {
                  const uint4 rres = res_staged ? *reinterpret_cast<const uint4*>(my_row + (((h * 4 + v) ^ sw) << 4))
                                                : *reinterpret_cast<const uint4*>(p.residual + row * p.ldr + col);
                  const uint32_t rw[4] = {rres.x, rres.y, rres.z, rres.w};
                  float g[8];
                  if (p.epi == kEpiGatedRes) {
                    const float4 g0 = *reinterpret_cast<const float4*>(p.gate + batch * p.gate_ld + col);
                    const float4 g1 = *reinterpret_cast<const float4*>(p.gate + batch * p.gate_ld + col + 4);
                    g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w;
                    g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
                  } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) g[j] = 1.0f;
                  }
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 f = unpack_bf16x2(rw[j]);
                    x[2 * j] = f.x + g[2 * j] * x[2 * j];
                    x[2 * j + 1] = f.y + g[2 * j + 1] * x[2 * j + 1];
                  }
                }
              }
              if (f32) {  // 8 values = two 16-byte chunks of the row's 128 bytes
                const int ch = v * 2;
                *reinterpret_cast<float4*>(my_row + (((ch) ^ sw) << 4)) = make_float4(x[0], x[1], x[2], x[3]);
                *reinterpret_cast<float4*>(my_row + (((ch + 1) ^ sw) << 4)) = make_float4(x[4], x[5], x[6], x[7]);
              } else {
                const int ch = h * 4 + v;
                uint4 ov;
                ov.x = pack_bf16x2(x[0], x[1]);
                ov.y = pack_bf16x2(x[2], x[3]);
                ov.z = pack_bf16x2(x[4], x[5]);
                ov.w = pack_bf16x2(x[6], x[7]);
                *reinterpret_cast<uint4*>(my_row + ((ch ^ sw) << 4)) = ov;
              }
            }
          }
          fence_proxy_async_smem();
          named_bar_sync(1 + egroup, 128);
          if (leader) {
            tma_store_2d(&tmap_c, slab, col0, static_cast<int>(out_row0));
            tma_store_commit();
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tmem_empty[acc]);
        continue;
      }
#pragma unroll 1
      for (int c = egroup * (BN / 64); c < (egroup + 1) * (BN / 64); ++c) {
        const int col0 = n_idx * BN + c * 32;
        if (col0 >= p.N) break;  // uniform across the group
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {  // 4 groups of 8 columns
            const int col = col0 + v * 8;
            if (col >= p.N) break;
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(r[v * 8 + j]) * p.alpha;
            if (p.splits > 1) {
              float* o = p.partial + (static_cast<long long>(split) * p.partial_rows + row) * p.N + col;
              *reinterpret_cast<float4*>(o) = make_float4(x[0], x[1], x[2], x[3]);
              *reinterpret_cast<float4*>(o + 4) = make_float4(x[4], x[5], x[6], x[7]);
              continue;
            }
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
            if (p.epi == kEpiGeluTanh) {
#pragma unroll
              for (int j = 0; j < 8; ++j) x[j] = gelu_tanh(x[j]);
            } else if (p.epi == kEpiSilu) {
#pragma unroll
              for (int j = 0; j < 8; ++j) x[j] = x[j] / (1.0f + __expf(-x[j]));
            } else if (p.epi == kEpiGatedRes || p.epi == kEpiAddRes) {
              const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + row * p.ldr + col);
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
              float g[8];
              if (p.epi == kEpiGatedRes) {
                const float4 g0 = *reinterpret_cast<const float4*>(p.gate + batch * p.gate_ld + col);
                const float4 g1 = *reinterpret_cast<const float4*>(p.gate + batch * p.gate_ld + col + 4);
                g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w;
                g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] = 1.0f;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16x2(rw[j]);
                x[2 * j] = f.x + g[2 * j] * x[2 * j];
                x[2 * j + 1] = f.y + g[2 * j + 1] * x[2 * j + 1];
              }
            }
            if (p.out_f32) {
              float* o = reinterpret_cast<float*>(p.out) + row * p.ldo + col;
              *reinterpret_cast<float4*>(o) = make_float4(x[0], x[1], x[2], x[3]);
              *reinterpret_cast<float4*>(o + 4) = make_float4(x[4], x[5], x[6], x[7]);
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + col;
              uint4 ov;
              ov.x = pack_bf16x2(x[0], x[1]);
              ov.y = pack_bf16x2(x[2], x[3]);
              ov.z = pack_bf16x2(x[4], x[5]);
              ov.w = pack_bf16x2(x[6], x[7]);
              *reinterpret_cast<uint4*>(o) = ov;
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[acc]);
    }
    if (p.tma_store && group_thread == 0) tma_store_wait_read<0>();  // shared memory stays valid until the stores have read it
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out[i] = sum over splits of partial[s][i], in split order; n8 = M * N / 8 vectors of 8 values.
__global__ void splitk_fold_kernel(const float* __restrict__ partial, void* __restrict__ out, long long ldo, int M, int N,
                                   int splits, int out_f32, int partial_rows) {
  const long long n8 = static_cast<long long>(M) * N / 8;
  const long long split_stride = static_cast<long long>(partial_rows) * N;
  const int n_vec = N / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
      const float4* src = reinterpret_cast<const float4*>(partial + s * split_stride + i * 8);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    const long long row = i / n_vec;
    const int col = static_cast<int>(i - row * n_vec) * 8;
    if (out_f32) {
      float* o = reinterpret_cast<float*>(out) + row * ldo + col;
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      uint4 ov;
      ov.x = pack_bf16x2(acc[0], acc[1]);
      ov.y = pack_bf16x2(acc[2], acc[3]);
      ov.z = pack_bf16x2(acc[4], acc[5]);
      ov.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + row * ldo + col) = ov;
    }
  }
}

template <bool A_MN, bool B_MN, int BN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const Params& p, cudaStream_t stream) {
  auto kern = gemm_kernel<A_MN, B_MN, BN>;
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(BN)));
    configured = true;
  }
  const int num_work = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.splits;
  const int grid = num_work < sm_count() ? num_work : sm_count();
  kern<<<grid, NUM_THREADS, smem_bytes(BN), stream>>>(ta, tb, tc, p);
  if (p.splits > 1) {
    const long long n8 = static_cast<long long>(p.M) * p.N / 8;
    const int blocks = static_cast<int>(n8 / 256 + 1 < sm_count() * 4 ? n8 / 256 + 1 : sm_count() * 4);
    splitk_fold_kernel<<<blocks, 256, 0, stream>>>(p.partial, p.out, p.ldo, p.M, p.N, p.splits, p.out_f32, p.partial_rows);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm
}  // namespace mdb

static int g_force_tile_n = 0;
static int g_epilogue_mode = 0;  // 0: TMA-store epilogue where the output allows it; 1: always direct stores

// Tile search / benchmarks: 1 pins the direct-store epilogue (one thread per row, 16-byte stores), 0 restores the default.
extern "C" int mdb_gemm_epilogue_mode(int mode) {
  if (mode != 0 && mode != 1) return 3006;
  g_epilogue_mode = mode;
  return 0;
}

// C entry point. A is [M,K] with leading dimension lda (a_mn_major = 0) or [K,M] (a_mn_major = 1);
// B is [N,K] (b_mn_major = 0) or [K,N] (b_mn_major = 1). All leading dimensions are in elements and
// must be multiples of 8; N must be a multiple of 8. Returns 0 or a CUDA / encoder error code.
static int gemm_impl(const void* A, const void* B, void* out, const void* bias, const void* residual, const void* gate,
                     int M, int N, int K, long long lda, long long ldb, long long ldo, long long ldr, long long gate_ld,
                     int rows_per_batch, int a_mn_major, int b_mn_major, int epi, int out_f32, float alpha,
                     float* partial, int splits, void* stream_ptr);

extern "C" int mdb_gemm_bf16(const void* A, const void* B, void* out, const void* bias, const void* residual,
                             const void* gate, int M, int N, int K, long long lda, long long ldb, long long ldo,
                             long long ldr, long long gate_ld, int rows_per_batch, int a_mn_major, int b_mn_major,
                             int epi, int out_f32, float alpha, void* stream_ptr) {
  return gemm_impl(A, B, out, bias, residual, gate, M, N, K, lda, ldb, ldo, ldr, gate_ld, rows_per_batch, a_mn_major,
                   b_mn_major, epi, out_f32, alpha, nullptr, 1, stream_ptr);
}

// Split-K form: out = alpha * A B^T with the contraction cut into `splits` ranges that run as separate work items
// (for products whose output has fewer tiles than the GPU has SMs: weight gradients). `partial` is a caller-provided
// fp32 workspace of splits * M * N values; no bias / epilogue. The sum over splits runs in split order.
extern "C" int mdb_gemm_bf16_splitk(const void* A, const void* B, void* out, int M, int N, int K, long long lda,
                                    long long ldb, long long ldo, int a_mn_major, int b_mn_major, int out_f32,
                                    float alpha, void* partial, int splits, void* stream_ptr) {
  if (splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) return 3005;
  return gemm_impl(A, B, out, nullptr, nullptr, nullptr, M, N, K, lda, ldb, ldo, 0, 0, 0, a_mn_major, b_mn_major, 0,
                   out_f32, alpha, static_cast<float*>(partial), splits, stream_ptr);
}

static int gemm_impl(const void* A, const void* B, void* out, const void* bias, const void* residual, const void* gate,
                     int M, int N, int K, long long lda, long long ldb, long long ldo, long long ldr, long long gate_ld,
                     int rows_per_batch, int a_mn_major, int b_mn_major, int epi, int out_f32, float alpha,
                     float* partial, int splits, void* stream_ptr) {
  using namespace mdb;
  using namespace mdb::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int BN = g_force_tile_n ? g_force_tile_n : 256;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldo & 3) || (!out_f32 && (ldo & 7))) return 3001;
  if ((epi == kEpiGatedRes || epi == kEpiAddRes) && (!residual || (ldr & 7))) return 3002;
  if (epi == kEpiGatedRes && (!gate || (gate_ld & 3))) return 3003;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn_major) {
    uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(K)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, BK};
    rc = encode_tmap_bf16(&ta, A, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {BK, BM};
    rc = encode_tmap_bf16(&ta, A, 2, dims, str, box);
  }
  if (rc) return rc;
  if (b_mn_major) {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, BK};
    rc = encode_tmap_bf16(&tb, B, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {BK, static_cast<uint32_t>(BN)};
    rc = encode_tmap_bf16(&tb, B, 2, dims, str, box);
  }
  if (rc) return rc;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.gate = static_cast<const float*>(gate);
  p.gate_ld = gate_ld;
  p.rows_per_batch = rows_per_batch;
  p.epi = epi;
  p.out_f32 = out_f32;
  p.alpha = alpha;
  p.status = status_buffer();
  {
    // every split gets at least one k-block: the count is recomputed from the rounded-up range
    const int num_kb = (K + BK - 1) / BK;
    int per = (num_kb + splits - 1) / splits;
    if (per < 1) per = 1;
    p.kb_per_split = per;
    p.splits = (num_kb + per - 1) / per;
    p.partial = partial;
    if (p.splits <= 1) { p.splits = 1; p.kb_per_split = num_kb; }
  }
  // Output map for the TMA-store epilogue: [N (inner), rows], 128-byte-wide boxes of 128 rows. With split-K it
  // covers the fp32 partials, whose splits are `partial_rows` = M rounded up to the tile height apart, so that a
  // tile's rows beyond M fall into padding instead of the next split.
  CUtensorMap tc;
  p.partial_rows = (M + BM - 1) / BM * BM;
  {
    const bool f32 = out_f32 || p.splits > 1;
    const void* base = p.splits > 1 ? static_cast<const void*>(partial) : out;
    const long long ld = p.splits > 1 ? N : ldo;
    const uint64_t rows = p.splits > 1 ? static_cast<uint64_t>(p.splits) * p.partial_rows : static_cast<uint64_t>(M);
    const int esz = f32 ? 4 : 2;
    p.tma_store = g_epilogue_mode == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0 && ((ld * esz) & 15) == 0;
    if (p.tma_store) {
      uint64_t dims[2] = {static_cast<uint64_t>(N), rows};
      uint64_t str[1] = {static_cast<uint64_t>(ld) * esz};
      uint32_t box[2] = {static_cast<uint32_t>(128 / esz), BM};
      rc = f32 ? encode_tmap_f32(&tc, base, 2, dims, str, box, 1) : encode_tmap_bf16(&tc, base, 2, dims, str, box);
      if (rc) return rc;
    } else {
      tc = ta;  // unused by the kernel; any valid map
      if (p.splits > 1) p.partial_rows = M;
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (BN == 256) {
    if (a_mn_major) {
      return b_mn_major ? launch<true, true, 256>(ta, tb, tc, p, stream) : launch<true, false, 256>(ta, tb, tc, p, stream);
    }
    return b_mn_major ? launch<false, true, 256>(ta, tb, tc, p, stream) : launch<false, false, 256>(ta, tb, tc, p, stream);
  }
  if (a_mn_major) {
    return b_mn_major ? launch<true, true, 128>(ta, tb, tc, p, stream) : launch<true, false, 128>(ta, tb, tc, p, stream);
  }
  return b_mn_major ? launch<false, true, 128>(ta, tb, tc, p, stream) : launch<false, false, 128>(ta, tb, tc, p, stream);
}

// 0: the default width (256); 128 or 256: use that tile width (tile search, benchmarks, tests).
extern "C" int mdb_gemm_force_tile_n(int bn) {
  if (bn != 0 && bn != 128 && bn != 256) return 3004;
  g_force_tile_n = bn;
  return 0;
}
