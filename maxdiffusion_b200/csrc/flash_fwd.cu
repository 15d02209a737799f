// Non-causal flash-attention forward for head_dim 128 on sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles that ping-pong on the
// tensor core: while the softmax warps of tile 0 work on S0, the MMA warp runs tile 1.
//   S_t = Q_t K_j^T      SS-form UMMA, fp32 in TMEM (128 columns per tile)
//   P_t = exp2(S_t*c - m) written back over S_t as packed bf16 (tcgen05.st)
//   O_t += P_t V_j       TS-form UMMA (A from TMEM, V is an MN-major smem operand)
// The running row max is refreshed lazily (only when it moves by more than 2^8), so the
// accumulator rescale is rare. The KV sequence may consist of several segments (one per ring
// hop / context shard); (O, m, l) stay on chip across segments and the merge costs nothing.
// A segment can be guarded by a ready flag in global memory that the loader warp waits on
// (bounded) before its first TMA load of that segment.
//
// Layout: q, k, v, o are [B, S, H, 128] bf16 with arbitrary (16-byte aligned) strides for
// B, S, H, so the [B, S, H*D] projections are consumed without a transpose.
// Ragged tails: rows >= q_len are not stored, keys >= kv_len of a segment are masked.
//
// Replaces the reference's Pallas-TPU kernels `_flash_attention_kernel`
// (src/maxdiffusion/kernels/custom_splash_attention.py:69-320) and the per-hop ring variant
// (:568-685) plus the online-softmax merge around it
// (src/maxdiffusion/kernels/splash_attention/ring_attention_kernel.py:1099-1131).
#include "host_common.h"

namespace mdb {
namespace fa {

constexpr int D = 128;
constexpr int BQ = 128;          // rows per q tile
constexpr int BKV = 128;         // keys per block
constexpr int KV_STAGES = 2;
constexpr int TILE_BYTES = 128 * D * 2;  // 32 KiB: two 64-column chunks of 128 rows x 128 B
constexpr int CHUNK_BYTES = 128 * 128;   // 16 KiB
constexpr int MAX_SEGMENTS = 8;
constexpr int NUM_THREADS = 384;         // warp 0 TMA, warp 1 MMA, warps 4-7 / 8-11 softmax
constexpr int SMEM_BYTES = 2 * TILE_BYTES + 2 * KV_STAGES * TILE_BYTES + 1024 + 256;
constexpr float kRescaleThreshold = 8.0f;

struct KVMaps {
  CUtensorMap k[MAX_SEGMENTS];
  CUtensorMap v[MAX_SEGMENTS];
};

struct Params {
  int B, H, q_len;
  int num_segments;
  int kv_len[MAX_SEGMENTS];
  __nv_bfloat16* out;
  long long o_stride_b, o_stride_s, o_stride_h;
  float* lse;  // [B, H, q_len] in the log2 domain (m + log2 l), may be nullptr
  float scale_log2;
  const unsigned int* seg_flags;  // [num_segments] or nullptr
  unsigned int flag_target;       // segment s is ready once seg_flags[s] >= flag_target
  DeviceStatus* status;
};

__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int target, volatile int* abort_flag,
                                          DeviceStatus* st, unsigned int detail) {
  uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if ((++spins & 0xffu) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        report_status(st, kStatusFlagTimeout, 40, detail);
        return false;
      }
    }
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ KVMaps maps, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;                                  // [2 tiles][2 chunks][128][128 B]
  uint8_t* sk = smem + 2 * TILE_BYTES;                 // [KV_STAGES] tiles
  uint8_t* sv = sk + KV_STAGES * TILE_BYTES;           // [KV_STAGES] tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sv + KV_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] per q tile
  uint64_t* p_full = bars + 11;       // [2] per q tile
  uint64_t* o_final = bars + 13;      // [2] per q tile
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 2 * BQ;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int n_tiles = (p.q_len - q0 > BQ) ? 2 : 1;

  int total_blocks = 0;
  for (int s = 0; s < p.num_segments; ++s) total_blocks += (p.kv_len[s] + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_final[i], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_q);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t aliases S_t.

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && total_blocks > 0) {
      mbar_expect_tx(q_full, n_tiles * TILE_BYTES);
      for (int t = 0; t < n_tiles; ++t) {
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(sq + t * TILE_BYTES + c * CHUNK_BYTES, &tmap_q, q_full, c * 64, head, q0 + t * BQ, batch);
        }
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int seg = 0; seg < p.num_segments && ok; ++seg) {
        const int nblk = (p.kv_len[seg] + BKV - 1) / BKV;
        if (nblk > 0 && p.seg_flags != nullptr) {
          if (!wait_flag(p.seg_flags + seg, p.flag_target, abort_flag, p.status, seg)) { ok = false; break; }
        }
        for (int jb = 0; jb < nblk; ++jb) {
          if (!mbar_wait(&k_empty[stage], phase ^ 1u, abort_flag, p.status, 41)) { ok = false; break; }
          mbar_expect_tx(&k_full[stage], TILE_BYTES);
          for (int c = 0; c < 2; ++c) {
            tma_load_4d(sk + stage * TILE_BYTES + c * CHUNK_BYTES, &maps.k[seg], &k_full[stage], c * 64, head,
                        jb * BKV, batch);
          }
          if (!mbar_wait(&v_empty[stage], phase ^ 1u, abort_flag, p.status, 42)) { ok = false; break; }
          mbar_expect_tx(&v_full[stage], TILE_BYTES);
          for (int c = 0; c < 2; ++c) {
            tma_load_4d(sv + stage * TILE_BYTES + c * CHUNK_BYTES, &maps.v[seg], &v_full[stage], c * 64, head,
                        jb * BKV, batch);
          }
          if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && total_blocks > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, false, true);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 50);
      tc_fence_after_sync();
      auto issue_s = [&](int t, int stage) {
        const uint32_t qa = smem_u32(sq + t * TILE_BYTES);
        const uint32_t ka = smem_u32(sk + stage * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
          umma_ss(tmem_base + t * 128, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024),
                  idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, p.status, 51);
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < n_tiles; ++t) issue_s(t, 0);
        umma_commit(&k_empty[0]);  // K block 0 is free once both S MMAs have read it
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < total_blocks && ok; ++j) {
        const int nstage = (stage + 1 == KV_STAGES) ? 0 : stage + 1;
        const uint32_t nphase = (stage + 1 == KV_STAGES) ? (phase ^ 1u) : phase;
        if (!mbar_wait(&v_full[stage], phase, abort_flag, p.status, 52)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t va = smem_u32(sv + stage * TILE_BYTES);
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (!mbar_wait(&p_full[t], j & 1, abort_flag, p.status, 53)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            umma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8,
                    make_smem_desc(va + k * 2048, CHUNK_BYTES, 1024), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          }
          if (j + 1 < total_blocks) {
            if (t == 0) {
              if (!mbar_wait(&k_full[nstage], nphase, abort_flag, p.status, 54)) { ok = false; break; }
              tc_fence_after_sync();
            }
            issue_s(t, nstage);
            if (t == n_tiles - 1) umma_commit(&k_empty[nstage]);
          } else {
            umma_commit(&o_final[t]);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[stage]);
        stage = nstage;
        phase = nphase;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ Softmax / correction / epilogue ------------
    const int t = (warp - 4) >> 2;         // q tile of this warp group
    const int quarter = warp & 3;          // TMEM lanes 32*quarter..+31
    const int row_in_tile = quarter * 32 + lane;
    const int q_row = q0 + t * BQ + row_in_tile;
    if (t < n_tiles && total_blocks > 0) {
      const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t s_addr = tmem_base + lane_off + t * 128;
      const uint32_t o_addr = tmem_base + lane_off + 256 + t * 128;
      float m = -INFINITY, l = 0.0f;
      bool ok = true;
      int j = 0;
      for (int seg = 0; seg < p.num_segments && ok; ++seg) {
        const int nblk = (p.kv_len[seg] + BKV - 1) / BKV;
        for (int jb = 0; jb < nblk; ++jb, ++j) {
          const int valid = min(BKV, p.kv_len[seg] - jb * BKV);
          if (!mbar_wait(&s_full[t], j & 1, abort_flag, p.status, 60)) { ok = false; break; }
          tc_fence_after_sync();
          // the whole 128-column row of S goes to registers with one wait, so the TMEM latency is paid once
          uint32_t sv[4][32];
          tmem_ld_x32(s_addr, sv[0]);
          tmem_ld_x32(s_addr + 32, sv[1]);
          tmem_ld_x32(s_addr + 64, sv[2]);
          tmem_ld_x32(s_addr + 96, sv[3]);
          tmem_wait_ld();
          float mx = -INFINITY;
          if (valid == BKV) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[c][i]));
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (c * 32 + i < valid) mx = fmaxf(mx, __uint_as_float(sv[c][i]));
              }
          }
          const float m_new = fmaxf(m, mx * p.scale_log2);
          if (j == 0) {
            m = m_new;
          } else {
            const bool need = (m_new - m) > kRescaleThreshold;
            if (__any_sync(0xffffffffu, need)) {
              const float alpha = fast_exp2(m - m_new);
              l *= alpha;
              m = m_new;
#pragma unroll 1
              for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld_x32(o_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                tmem_st_x32(o_addr + c * 32, r);
              }
              tmem_wait_st();
            }
          }
          // probabilities, written over S as packed bf16
          float rowsum = 0.0f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
            if (valid == BKV) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float p0 = fast_exp2(__uint_as_float(sv[c][2 * i]) * p.scale_log2 - m);
                const float p1 = fast_exp2(__uint_as_float(sv[c][2 * i + 1]) * p.scale_log2 - m);
                rowsum += p0 + p1;
                pk[i] = pack_bf16x2(p0, p1);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int col = c * 32 + 2 * i;
                float p0 = fast_exp2(__uint_as_float(sv[c][2 * i]) * p.scale_log2 - m);
                float p1 = fast_exp2(__uint_as_float(sv[c][2 * i + 1]) * p.scale_log2 - m);
                if (col >= valid) p0 = 0.0f;
                if (col + 1 >= valid) p1 = 0.0f;
                rowsum += p0 + p1;
                pk[i] = pack_bf16x2(p0, p1);
              }
            }
            tmem_st_x16(s_addr + c * 16, pk);
          }
          l += rowsum;
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&p_full[t]);
        }
      }
      if (ok && mbar_wait(&o_final[t], 0, abort_flag, p.status, 61)) {
        tc_fence_after_sync();
        const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
        const bool row_ok = q_row < p.q_len;
        __nv_bfloat16* orow = p.out + batch * p.o_stride_b + static_cast<long long>(q_row) * p.o_stride_s +
                              head * p.o_stride_h;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_x32(o_addr + c * 32, r);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 ov;
              ov.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
              ov.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
              ov.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
              ov.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = ov;
            }
          }
        }
        if (row_ok && p.lse != nullptr) {
          p.lse[(static_cast<long long>(batch) * p.H + head) * p.q_len + q_row] = m + log2f(l);
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

static int make_map(CUtensorMap* map, const void* ptr, int B, int S, int H, long long sb, long long ss, long long sh) {
  // dims innermost first: (D, H, S, B)
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                      static_cast<uint64_t>(B)};
  uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap_bf16(map, ptr, 4, dims, str, box);
}

}  // namespace fa
}  // namespace mdb

// q: [B, q_len, H, 128]; k/v segment s: [B, kv_len[s], H, 128]; out like q. Strides are in elements
// (batch, sequence, head); the head_dim stride is 1. Every segment shares the k strides / v strides
// given here. Returns 0 or an error code.
extern "C" int mdb_flash_fwd(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* out,
                             float* lse, int B, int H, int q_len, int num_segments, const int* kv_lens,
                             long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                             long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_sb,
                             long long o_ss, long long o_sh, float softmax_scale, const unsigned int* seg_flags,
                             unsigned int flag_target, void* stream_ptr) {
  using namespace mdb;
  using namespace mdb::fa;
  if (B <= 0 || H <= 0 || q_len <= 0) return 0;
  if (num_segments < 1 || num_segments > MAX_SEGMENTS) return 3101;
  if ((q_sb | q_ss | q_sh | k_sb | k_ss | k_sh | v_sb | v_ss | v_sh | o_sb | o_ss | o_sh) & 7) return 3102;
  CUtensorMap tq;
  KVMaps maps;
  Params p;
  int rc = make_map(&tq, q, B, q_len, H, q_sb, q_ss, q_sh);
  if (rc) return rc;
  for (int s = 0; s < MAX_SEGMENTS; ++s) {
    const int src = s < num_segments ? s : 0;
    p.kv_len[s] = s < num_segments ? kv_lens[s] : 0;
    const int len = kv_lens[src] > 0 ? kv_lens[src] : 1;
    rc = make_map(&maps.k[s], k_ptrs[src], B, len, H, k_sb, k_ss, k_sh);
    if (rc) return rc;
    rc = make_map(&maps.v[s], v_ptrs[src], B, len, H, v_sb, v_ss, v_sh);
    if (rc) return rc;
  }
  p.B = B; p.H = H; p.q_len = q_len;
  p.num_segments = num_segments;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.o_stride_b = o_sb; p.o_stride_s = o_ss; p.o_stride_h = o_sh;
  p.lse = lse;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.seg_flags = seg_flags;
  p.flag_target = flag_target;
  p.status = status_buffer();
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  dim3 grid((q_len + 2 * BQ - 1) / (2 * BQ), H, B);
  flash_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream_ptr)>>>(tq, maps, p);
  return static_cast<int>(cudaGetLastError());
}
