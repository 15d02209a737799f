// Non-causal flash-attention forward for head_dim 128 on sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles, and streams K / V in blocks of 64 keys:
//   S_t = Q_t K_j^T      SS-form UMMA, fp32 in TMEM (64 columns), two buffers per tile
//   P_t = exp2(S_t*c - m) written back over S_t as packed bf16 (tcgen05.st)
//   O_t += P_t V_j       TS-form UMMA (A from TMEM, V is an MN-major smem operand)
// The softmax is bound by the exponential unit (16 results per clock and SM, as many cycles per tile as both
// products together), so the layout keeps the softmax warps of both tiles busy all the time: S of block j+1 is
// multiplied into the tile's second buffer while block j is exponentiated, and four lanes in different warps issue
// the products (S and P V of either tile), because the waits, commits and MMA instructions of a block cost one
// issuing lane more cycles than the products take to run. Every hand-over is an mbarrier.
// The running row max is refreshed lazily (only when it moves by more than 2^8), so the
// accumulator rescale is rare; it waits for the tile's previous P V product first. The KV sequence may consist of several segments (one per ring
// hop / context shard); (O, m, l) stay on chip across segments and the merge costs nothing.
// A segment can be guarded by a ready flag in global memory that the loader warp waits on
// (bounded) before its first TMA load of that segment.
//
// The kernel is persistent: at most one CTA per SM, each compute CTA walks a static list of
// (q-block, head, batch) tiles. When the K/V segments of other ranks have to be fetched (ring /
// context-parallel attention) the last `n_copy` CTAs of the same launch are copy CTAs: they wait for
// the owner's epoch flag, pull its K/V shard over NVLink with 16-byte loads into this GPU's staging
// buffer, and raise ready flags; afterwards they acknowledge to the owners. The shards are pulled in
// units of (head group, segment), head group outermost, and a unit's flag is raised as soon as it is
// staged: the compute CTAs walk the work list head by head, so the first round of work items needs only
// the first group's heads of every segment (a fraction of the bytes) and the later groups arrive while
// the earlier ones are being multiplied. Transfer and math therefore overlap unit by unit inside ONE
// kernel whose CTAs are all co-resident, and no remote tile crosses NVLink more than once.
//
// Layout: q, k, v, o are [B, S, H, 128] bf16 with arbitrary (16-byte aligned) strides for
// B, S, H, so the [B, S, H*D] projections are consumed without a transpose.
// Ragged tails: rows >= q_len are not stored, keys >= kv_len of a segment are masked.
//
// Replaces the reference's Pallas-TPU kernels `_flash_attention_kernel`
// (src/maxdiffusion/kernels/custom_splash_attention.py:69-320) and the per-hop ring variant
// (:568-685) plus the online-softmax merge around it
// (src/maxdiffusion/kernels/splash_attention/ring_attention_kernel.py:1099-1131).
#include <string.h>

#include "host_common.h"

namespace mdb {
namespace fa {

constexpr int BQ = 128;          // rows per q tile
constexpr int BKV = 64;          // keys per block
constexpr int DEFAULT_KV_STAGES = 4;  // K / V pipeline depth; 2..5 are built and selectable (tile search)
// A tile is stored as head_dim / 64 chunks of 64 columns (128-byte rows, 128-byte swizzle).
constexpr int CHUNK_BYTES = 128 * 128;       // 16 KiB: one chunk of a 128-row Q tile
constexpr int KV_CHUNK_BYTES = BKV * 128;    // 8 KiB: one chunk of a 64-key K / V tile
constexpr int MAX_SEGMENTS = 8;
constexpr int ROLE_WARPS = 5;            // warp 0 TMA, warps 1 / 3 issue S of tile 0 / 1, warps 2 / 4 issue P V of tile 0 / 1
constexpr int NUM_THREADS = ROLE_WARPS * 32 + 256;  // + softmax warps 5-8 (tile 0), 9-12 (tile 1)
template <int HD, int KV_STAGES>
constexpr int smem_bytes() { return 2 * (HD / 64) * CHUNK_BYTES + 2 * KV_STAGES * (HD / 64) * KV_CHUNK_BYTES + 1024 + 512; }
constexpr float kRescaleThreshold = 8.0f;

struct KVMaps {
  CUtensorMap k[MAX_SEGMENTS];
  CUtensorMap v[MAX_SEGMENTS];
};

constexpr int MAX_REMOTE = MAX_SEGMENTS - 1;
constexpr int MAX_GROUPS = 8;            // head groups of a copy plan; also the stride of the per-segment flag rows
constexpr int NUM_COUNTERS = MAX_REMOTE * MAX_GROUPS + 1;

// Work of the copy CTAs: remote segment i (KV segment 1 + i of the launch) is pulled from src to dst, as n_groups
// column slabs (head groups) of the [rows, row_vecs] tensors; slab g covers vectors [g * group_vecs, ...) of a row.
struct CopyPlan {
  int n_remote;                         // 0: no copy CTAs
  int n_copy_ctas;
  int n_groups;                         // 1 .. MAX_GROUPS
  unsigned int rows;                    // token rows per tensor (B * S)
  unsigned int row_vecs;                // 16-byte vectors per row (H * D * 2 / 16)
  unsigned int group_vecs;              // vectors per row of one head group (the last group may be narrower)
  const uint4* src[MAX_REMOTE][2];      // peer addresses of K and V
  uint4* dst[MAX_REMOTE][2];            // local staging
  const unsigned int* ready[MAX_REMOTE];  // local signal-pad slot the owner raises
  unsigned int epoch;
  unsigned int* counters;               // [NUM_COUNTERS], zero at launch
  unsigned int* seg_flags;              // flag (1 + i) * MAX_GROUPS + g is raised once slab g of segment i is staged
  unsigned int* ack[MAX_SEGMENTS];      // peers' pad slots to acknowledge into (n_ack entries)
  int n_ack;
};

struct Params {
  int B, H, q_len;
  int num_segments;
  int kv_len[MAX_SEGMENTS];
  __nv_bfloat16* out;
  long long o_stride_b, o_stride_s, o_stride_h;
  float* lse;  // [B, H, q_len] in the log2 domain (m + log2 l), may be nullptr
  float scale_log2;
  const unsigned int* seg_flags;  // [num_segments * flag_stride] or nullptr
  unsigned int flag_target;       // heads [g*hpg, (g+1)*hpg) of segment s are ready once seg_flags[s*flag_stride + g] >= flag_target
  int flag_stride;                // 1: one flag per segment; MAX_GROUPS: one per (segment, head group)
  int heads_per_group;            // hpg above (>= H when flag_stride is 1)
  // Fixed-exponent softmax (both nullptr: off). Rows of the heads with fixed_heads[h] != 0 subtract the given
  // m_fixed[b, h, row] (log2 domain) instead of a running maximum: no row maximum, no accumulator rescale.
  // The caller guarantees  s*scale_log2 - m_fixed <= 126  for every score of such a head.
  const float* m_fixed;    // [B, H, q_len]
  const int* fixed_heads;  // [H]
  // Output scatter (0: off). The reverse Ulysses exchange folded into the epilogue: query row r of this launch is row
  // r % rows_per_rank of rank r / rows_per_rank, whose output tensor [B, rows_per_rank, heads_total, D] is addressed
  // with the o strides above; this launch's head h is head out_head_off + h there (16-byte peer stores).
  int out_scatter_n, out_rows_per_rank, out_head_off;
  __nv_bfloat16* out_peers[MAX_SEGMENTS];
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
      if (status_failed(st)) {
        *abort_flag = 1;
        return false;
      }
      if (global_timer_ns() - t0 > kPeerWaitBudgetNs + kWaitBudgetNs) {  // outlasts the copy CTAs' own wait
        *abort_flag = 1;
        report_status(st, kStatusFlagTimeout, 40, detail);
        return false;
      }
    }
  }
}

// One (head group, segment) unit: this CTA's share of slab `g` of both tensors. Vector `idx` of the slab is column
// idx % gv of row idx / gv; the pair advances by NUM_THREADS per load without a division.
__device__ __forceinline__ void copy_slab(const uint4* __restrict__ src, uint4* __restrict__ dst, unsigned int begin,
                                          unsigned int end, unsigned int gv, unsigned int row_vecs, unsigned int col0) {
  const unsigned int step_row = NUM_THREADS / gv, step_col = NUM_THREADS % gv;
  unsigned int idx = begin + threadIdx.x;
  unsigned int row = idx / gv, col = idx % gv;
  // 16 independent 16-byte loads in flight per thread (a copy CTA then holds about 100 KB in flight, which a round
  // trip of a few microseconds over NVLink turns into 25-30 GB/s per CTA); peer data bypasses L1
  while (idx + 15u * NUM_THREADS < end) {
    uint4 r[16];
    unsigned long long off[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      off[u] = static_cast<unsigned long long>(row) * row_vecs + col0 + col;
      r[u] = __ldcg(src + off[u]);
      row += step_row;
      col += step_col;
      if (col >= gv) { col -= gv; ++row; }
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) dst[off[u]] = r[u];
    idx += 16u * NUM_THREADS;
  }
  while (idx < end) {
    const unsigned long long off = static_cast<unsigned long long>(row) * row_vecs + col0 + col;
    dst[off] = __ldcg(src + off);
    row += step_row;
    col += step_col;
    if (col >= gv) { col -= gv; ++row; }
    idx += NUM_THREADS;
  }
}

__device__ __forceinline__ void copy_cta(const CopyPlan& cp, int ci, DeviceStatus* status) {
  __shared__ int ok_s;
  unsigned int owner_seen = 0;  // remote segments whose owner flag has been observed (uniform over the CTA)
  const int n_units = cp.n_remote * cp.n_groups;
  for (int u = 0; u < n_units; ++u) {
    const int g = u / cp.n_remote;  // head group outermost: every segment's first slab before any second slab
    const int i = u - g * cp.n_remote;
    if (!((owner_seen >> i) & 1u)) {
      if (threadIdx.x == 0) {
        int ok = 1;
        const uint64_t t0 = global_timer_ns();
        unsigned int spins = 0;
        while (true) {
          unsigned int v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(cp.ready[i]) : "memory");
          if (v >= cp.epoch) break;
          if ((++spins & 0xffu) == 0u) {
            if (status_failed(status)) {
              ok = 0;
              break;
            }
            if (global_timer_ns() - t0 > kPeerWaitBudgetNs) {
              report_status(status, kStatusFlagTimeout, 45, static_cast<unsigned int>(i));
              ok = 0;
              break;
            }
          }
        }
        ok_s = ok;
      }
      __syncthreads();
      if (!ok_s) return;
      owner_seen |= 1u << i;
    }
    const unsigned int col0 = static_cast<unsigned int>(g) * cp.group_vecs;
    const unsigned int gv = min(cp.group_vecs, cp.row_vecs - col0);
    const unsigned int total = cp.rows * gv;
    const unsigned int per = (total + cp.n_copy_ctas - 1) / cp.n_copy_ctas;
    const unsigned int begin = min(total, static_cast<unsigned int>(ci) * per);
    const unsigned int end = min(total, begin + per);
    for (int t = 0; t < 2; ++t) copy_slab(cp.src[i][t], cp.dst[i][t], begin, end, gv, cp.row_vecs, col0);
    asm volatile("fence.proxy.async.global;" ::: "memory");  // staged data is read back through TMA
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int old = atomicAdd(cp.counters + u, 1u);
      if (old == static_cast<unsigned int>(cp.n_copy_ctas - 1)) {
        __threadfence();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(cp.seg_flags + (1 + i) * MAX_GROUPS + g), "r"(cp.epoch)
                     : "memory");
      }
    }
  }
  if (threadIdx.x == 0) {
    const unsigned int old = atomicAdd(cp.counters + NUM_COUNTERS - 1, 1u);
    if (old == static_cast<unsigned int>(cp.n_copy_ctas - 1)) {
      // every remote shard has been read: tell the owners that their buffer may be overwritten
      for (int a = 0; a < cp.n_ack; ++a) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(cp.ack[a]), "r"(cp.epoch) : "memory");
      }
    }
  }
}

template <int HD, int KV_STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ KVMaps maps, const Params p,
                 const __grid_constant__ CopyPlan cp) {
  const int n_copy = cp.n_remote > 0 ? cp.n_copy_ctas : 0;
  const int n_compute = static_cast<int>(gridDim.x) - n_copy;
  if (static_cast<int>(blockIdx.x) >= n_compute) {
    copy_cta(cp, static_cast<int>(blockIdx.x) - n_compute, p.status);
    return;
  }

  constexpr int D = HD;                       // head_dim: 64 or 128
  constexpr int CH = HD / 64;                 // chunks per tile
  constexpr int TILE_BYTES = CH * CHUNK_BYTES;        // Q tile of 128 rows
  constexpr int KV_TILE_BYTES = CH * KV_CHUNK_BYTES;  // K / V tile of 64 keys
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;                                  // [2 tiles][2 chunks][128][128 B]
  uint8_t* sk = smem + 2 * TILE_BYTES;                 // [KV_STAGES] tiles of 64 keys
  uint8_t* sv = sk + KV_STAGES * KV_TILE_BYTES;        // [KV_STAGES] tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sv + KV_STAGES * KV_TILE_BYTES);
  uint64_t* q_full = bars;                        // [1]
  uint64_t* q_empty = bars + 1;                   // [1] both S lanes
  uint64_t* k_full = bars + 2;                    // [KV_STAGES]
  uint64_t* k_empty = k_full + KV_STAGES;         // [KV_STAGES] both S lanes
  uint64_t* v_full = k_empty + KV_STAGES;         // [KV_STAGES]
  uint64_t* v_empty = v_full + KV_STAGES;         // [KV_STAGES] both P V lanes
  uint64_t* s_full = v_empty + KV_STAGES;         // [2 tiles][2 buffers] S written
  uint64_t* p_full = s_full + 4;                  // [2][2] P stored over S
  uint64_t* s_free = p_full + 4;                  // [2][2] P V product that reads the buffer (and adds into O) completed
  uint64_t* o_final = s_free + 4;                 // [2] per q tile
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(o_final + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_qb = (p.q_len + 2 * BQ - 1) / (2 * BQ);
  const int total_work = n_qb * p.H * p.B;

  int total_blocks = 0;
  for (int s = 0; s < p.num_segments; ++s) total_blocks += (p.kv_len[s] + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one elected lane per softmax warp
      mbar_init(&s_free[i], 1);
    }
    mbar_init(&o_final[0], 1);
    mbar_init(&o_final[1], 1);
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
  // TMEM columns: S(t, b) = t*128 + b*64 (P aliases it as 32 packed columns), O(t) = 256 + t*128.

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && total_blocks > 0) {
      int stage = 0;
      uint32_t phase = 0;
      unsigned long long seen = 0;  // (segment, head group) flags that have been observed
      bool ok = true;
      int it = 0;
      for (int work = blockIdx.x; work < total_work && ok; work += n_compute, ++it) {
        const int qb = work % n_qb;
        const int head = (work / n_qb) % p.H;
        const int batch = work / (n_qb * p.H);
        const int q0 = qb * 2 * BQ;
        const int n_tiles = (p.q_len - q0 > BQ) ? 2 : 1;
        if (!mbar_wait(q_empty, (it & 1) ^ 1u, abort_flag, p.status, 43)) { ok = false; break; }
        mbar_expect_tx(q_full, n_tiles * TILE_BYTES);
        for (int t = 0; t < n_tiles; ++t) {
          for (int c = 0; c < CH; ++c) {
            tma_load_4d(sq + t * TILE_BYTES + c * CHUNK_BYTES, &tmap_q, q_full, c * 64, head, q0 + t * BQ, batch);
          }
        }
        for (int seg = 0; seg < p.num_segments && ok; ++seg) {
          const int nblk = (p.kv_len[seg] + BKV - 1) / BKV;
          if (nblk > 0 && p.seg_flags != nullptr) {
            const int fi = seg * p.flag_stride + head / p.heads_per_group;  // < MAX_SEGMENTS * MAX_GROUPS = 64
            if (!((seen >> fi) & 1ull)) {
              if (!wait_flag(p.seg_flags + fi, p.flag_target, abort_flag, p.status, fi)) { ok = false; break; }
              asm volatile("fence.proxy.async.global;" ::: "memory");
              seen |= 1ull << fi;
            }
          }
          for (int jb = 0; jb < nblk; ++jb) {
            if (!mbar_wait(&k_empty[stage], phase ^ 1u, abort_flag, p.status, 41)) { ok = false; break; }
            mbar_expect_tx(&k_full[stage], KV_TILE_BYTES);
            for (int c = 0; c < CH; ++c) {
              tma_load_4d(sk + stage * KV_TILE_BYTES + c * KV_CHUNK_BYTES, &maps.k[seg], &k_full[stage], c * 64, head,
                          jb * BKV, batch);
            }
            if (!mbar_wait(&v_empty[stage], phase ^ 1u, abort_flag, p.status, 42)) { ok = false; break; }
            mbar_expect_tx(&v_full[stage], KV_TILE_BYTES);
            for (int c = 0; c < CH; ++c) {
              tma_load_4d(sv + stage * KV_TILE_BYTES + c * KV_CHUNK_BYTES, &maps.v[seg], &v_full[stage], c * 64, head,
                          jb * BKV, batch);
            }
            if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------ issuing lanes: S_t = Q_t K_j^T --------------
    if (lane == 0 && total_blocks > 0) {
      const int t = warp >> 1;  // warp 1 -> tile 0, warp 3 -> tile 1
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BKV, false, false);
      // descriptors are built once; the address field (units of 16 bytes) advances by addition
      const uint64_t qd = make_smem_desc(smem_u32(sq + t * TILE_BYTES), 16, 1024);
      const uint64_t kd0 = make_smem_desc(smem_u32(sk), 16, 1024);
      constexpr uint32_t STAGE_STEP = KV_TILE_BYTES >> 4;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t n = 0;  // blocks of this tile so far, over all work items: buffer n & 1, use n >> 1
      bool ok = true;
      int it = 0;
      for (int work = blockIdx.x; work < total_work && ok; work += n_compute, ++it) {
        const int q0 = (work % n_qb) * 2 * BQ;
        const bool active = t < ((p.q_len - q0 > BQ) ? 2 : 1);
        if (!mbar_wait(q_full, it & 1, abort_flag, p.status, 50)) { ok = false; break; }
        for (int j = 0; j < total_blocks; ++j) {
          if (!mbar_wait(&k_full[stage], phase, abort_flag, p.status, 51)) { ok = false; break; }
          if (active) {
            const uint32_t b = n & 1u;
            // the buffer last held P of block n - 2: its P V product must have completed
            if (n >= 2 && !mbar_wait(&s_free[t * 2 + b], ((n >> 1) - 1) & 1u, abort_flag, p.status, 55)) { ok = false; break; }
            tc_fence_after_sync();
            const uint64_t kd = kd0 + stage * STAGE_STEP;
            const uint32_t s_col = tmem_base + t * 128 + b * 64;
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint32_t qo = ((k >> 2) * CHUNK_BYTES + (k & 3) * 32) >> 4;
              const uint32_t ko = ((k >> 2) * KV_CHUNK_BYTES + (k & 3) * 32) >> 4;
              umma_ss(s_col, qd + qo, kd + ko, idesc_s, k > 0 ? 1u : 0u);
            }
            umma_commit(&s_full[t * 2 + b]);
            umma_commit(&k_empty[stage]);  // this K block is free once the S MMAs have read it
            // the S MMAs of the last block are the last readers of the Q tile: free it for the next work item
            if (j + 1 == total_blocks) umma_commit(q_empty);
            ++n;
          } else {
            mbar_arrive(&k_empty[stage]);
            if (j + 1 == total_blocks) mbar_arrive(q_empty);
          }
          if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 2 || warp == 4) {
    // ------------------------------ issuing lanes: O_t += P_t V_j ----------------
    if (lane == 0 && total_blocks > 0) {
      const int t = (warp >> 1) - 1;  // warp 2 -> tile 0, warp 4 -> tile 1
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      const uint64_t vd0 = make_smem_desc(smem_u32(sv), KV_CHUNK_BYTES, 1024);
      constexpr uint32_t STAGE_STEP = KV_TILE_BYTES >> 4;
      const uint32_t o_col = tmem_base + 256 + t * 128;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t n = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < total_work && ok; work += n_compute) {
        const int q0 = (work % n_qb) * 2 * BQ;
        const bool active = t < ((p.q_len - q0 > BQ) ? 2 : 1);
        for (int j = 0; j < total_blocks; ++j) {
          if (!mbar_wait(&v_full[stage], phase, abort_flag, p.status, 52)) { ok = false; break; }
          if (active) {
            const uint32_t b = n & 1u;
            if (!mbar_wait(&p_full[t * 2 + b], (n >> 1) & 1u, abort_flag, p.status, 53)) { ok = false; break; }
            tc_fence_after_sync();
            const uint64_t vd = vd0 + stage * STAGE_STEP;
            const uint32_t p_col = tmem_base + t * 128 + b * 64;
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
              umma_ts(o_col, p_col + k * 8, vd + k * (2048 >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
            umma_commit(&s_free[t * 2 + b]);
            umma_commit(&v_empty[stage]);
            if (j + 1 == total_blocks) umma_commit(&o_final[t]);
            ++n;
          } else {
            mbar_arrive(&v_empty[stage]);
          }
          if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp >= ROLE_WARPS) {
    // ------------------------------ Softmax / correction / epilogue ------------
    const int t = (warp - ROLE_WARPS) >> 2;  // q tile of this warp group
    const int quarter = warp & 3;            // TMEM lanes 32*quarter..+31
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem_base + lane_off + 256 + t * 128;
    uint32_t n = 0, oc = 0;  // blocks of this tile so far; parity of o_final
    bool ok = total_blocks > 0;
    for (int work = blockIdx.x; work < total_work && ok; work += n_compute) {
      const int qb = work % n_qb;
      const int head = (work / n_qb) % p.H;
      const int batch = work / (n_qb * p.H);
      const int q0 = qb * 2 * BQ;
      const int n_tiles = (p.q_len - q0 > BQ) ? 2 : 1;
      if (t >= n_tiles) continue;
      const int q_row = q0 + t * BQ + row_in_tile;
      float m = -INFINITY, l = 0.0f;
      const bool fixed = p.m_fixed != nullptr && p.fixed_heads[head] != 0;  // uniform over the CTA
      if (fixed) {
        m = (q_row < p.q_len) ? p.m_fixed[(static_cast<long long>(batch) * p.H + head) * p.q_len + q_row] : 0.0f;
      }
      int j = 0;
      for (int seg = 0; seg < p.num_segments && ok; ++seg) {
        const int nblk = (p.kv_len[seg] + BKV - 1) / BKV;
        for (int jb = 0; jb < nblk; ++jb, ++j, ++n) {
          const int valid = min(BKV, p.kv_len[seg] - jb * BKV);
          const uint32_t b = n & 1u;
          const uint32_t s_addr = tmem_base + lane_off + t * 128 + b * 64;
          if (!mbar_wait(&s_full[t * 2 + b], (n >> 1) & 1u, abort_flag, p.status, 60)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t sv2[2][32];
          tmem_ld_x32(s_addr, sv2[0]);
          tmem_ld_x32(s_addr + 32, sv2[1]);
          tmem_wait_ld();
          if (!fixed) {
            float mx0 = -INFINITY, mx1 = -INFINITY;  // two chains
            if (valid == BKV) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(sv2[0][i]));
                mx1 = fmaxf(mx1, __uint_as_float(sv2[1][i]));
              }
            } else {
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  if (c * 32 + i < valid) mx0 = fmaxf(mx0, __uint_as_float(sv2[c][i]));
                }
            }
            const float m_new = fmaxf(m, fmaxf(mx0, mx1) * p.scale_log2);
            if (j == 0) {
              m = m_new;
            } else {
              const bool need = (m_new - m) > kRescaleThreshold;
              if (__any_sync(0xffffffffu, need)) {
                // O must be at rest: the P V product of the previous block (the other buffer) has to be complete
                if (!mbar_wait(&s_free[t * 2 + (b ^ 1u)], ((n - 1) >> 1) & 1u, abort_flag, p.status, 62)) { ok = false; break; }
                tc_fence_after_sync();
                const float alpha = fast_exp2(m - m_new);
                l *= alpha;
                m = m_new;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
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
          }
          // probabilities, written over S as packed bf16 (32 columns)
          float rs0 = 0.0f, rs1 = 0.0f;
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float p0 = fast_exp2(__uint_as_float(sv2[c][2 * i]) * p.scale_log2 - m);
              float p1 = fast_exp2(__uint_as_float(sv2[c][2 * i + 1]) * p.scale_log2 - m);
              if (valid != BKV) {
                const int col = c * 32 + 2 * i;
                if (col >= valid) p0 = 0.0f;
                if (col + 1 >= valid) p1 = 0.0f;
              }
              rs0 += p0;
              rs1 += p1;
              pk[c * 16 + i] = pack_bf16x2(p0, p1);
            }
          }
          tmem_st_x32(s_addr, pk);
          l += rs0 + rs1;
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[t * 2 + b]);
        }
      }
      if (!ok) break;
      if (!mbar_wait(&o_final[t], oc & 1u, abort_flag, p.status, 61)) { ok = false; break; }
      ++oc;
      tc_fence_after_sync();
      const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
      const bool row_ok = q_row < p.q_len;
      __nv_bfloat16* obase = p.out;
      int orow_idx = q_row, ohead = head;
      if (p.out_scatter_n > 0) {
        const int r = min(q_row / p.out_rows_per_rank, p.out_scatter_n - 1);
        obase = p.out_peers[r];
        orow_idx = q_row - r * p.out_rows_per_rank;
        ohead = head + p.out_head_off;
      }
      __nv_bfloat16* orow = obase + batch * p.o_stride_b + static_cast<long long>(orow_idx) * p.o_stride_s +
                            ohead * p.o_stride_h;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
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
      // the next tile's first P*V overwrites O only after this warp group has arrived on p_full again
      tc_fence_before_sync();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

static int make_map(CUtensorMap* map, const void* ptr, int D, int B, int S, int H, long long sb, long long ss, long long sh,
                    int box_rows) {
  // dims innermost first: (D, H, S, B)
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                      static_cast<uint64_t>(B)};
  uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return encode_tmap_bf16(map, ptr, 4, dims, str, box);
}

}  // namespace fa
}  // namespace mdb

// Host-side description of the output scatter (see Params::out_scatter_n).
struct MdbOutScatter {
  int n, rows_per_rank, head_off;
  unsigned long long ptrs[8];
};

// Host-side description of the copy CTAs' work (all addresses as integers); see CopyPlan.
struct MdbCopyPlan {
  int n_remote;
  int n_copy_ctas;
  unsigned long long src[7][2];
  unsigned long long dst[7][2];
  long long nbytes;                 // per tensor, multiple of 16; source and staging are contiguous [B, S, H, D]
  unsigned long long ready[7];
  unsigned int epoch;
  unsigned long long counters;      // device uint32[57] (7 segments x 8 head groups + 1), zero at launch
  unsigned long long seg_flags;     // device uint32[num_segments * 8]: flag seg * 8 + g; row 0 (own shard) raised
  unsigned long long ack[8];
  int n_ack;
  int n_groups;                     // head groups: 0 lets the launcher choose, 1 copies whole segments in order
};

// Launch-shape overrides for the tile search (0 = default): K / V pipeline stages (2..5) and the number of copy CTAs.
static int g_tune_stages = 0, g_tune_copy_ctas = 0;
static int g_last_stages = 0, g_last_copy_ctas = 0;  // what the most recent launch used (for the tile-search tests)

extern "C" int mdb_flash_fwd_last_variant(int* kv_stages, int* copy_ctas) {
  *kv_stages = g_last_stages;
  *copy_ctas = g_last_copy_ctas;
  return 0;
}

extern "C" int mdb_flash_fwd_tune(int kv_stages, int copy_ctas) {
  if (kv_stages != 0 && (kv_stages < 2 || kv_stages > 5)) return 3108;
  if (copy_ctas < 0 || copy_ctas > 64) return 3108;
  g_tune_stages = kv_stages;
  g_tune_copy_ctas = copy_ctas;
  return 0;
}

template <int HD, int STAGES>
static int launch_variant(dim3 grid, cudaStream_t st, const CUtensorMap& tq, const mdb::fa::KVMaps& maps, const mdb::fa::Params& p,
                          const mdb::fa::CopyPlan& cp) {
  using namespace mdb::fa;
  static bool configured = false;
  if (!configured) {
    MDB_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        smem_bytes<HD, STAGES>()));
    configured = true;
  }
  flash_fwd_kernel<HD, STAGES><<<grid, NUM_THREADS, smem_bytes<HD, STAGES>(), st>>>(tq, maps, p, cp);
  return static_cast<int>(cudaGetLastError());
}

// q: [B, q_len, H, 128]; k/v segment s: [B, kv_len[s], H, 128]; out like q. Strides are in elements
// (batch, sequence, head); the head_dim stride is 1. Every segment shares the k strides / v strides
// given here. `plan` (may be null) adds copy CTAs that stage the remote segments 1.. from peer memory.
// Returns 0 or an error code.
template <int HD>
static int flash_fwd_launch(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* out,
                            float* lse, int B, int H, int q_len, int num_segments, const int* kv_lens,
                            long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                            long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_sb,
                            long long o_ss, long long o_sh, float softmax_scale, const unsigned int* seg_flags,
                            unsigned int flag_target, const MdbCopyPlan* plan, void* stream_ptr,
                            const float* m_fixed = nullptr, const int* fixed_heads = nullptr,
                            const MdbOutScatter* scatter = nullptr) {
  using namespace mdb;
  using namespace mdb::fa;
  if (B <= 0 || H <= 0 || q_len <= 0) return 0;
  if (num_segments < 1 || num_segments > MAX_SEGMENTS) return 3101;
  if ((q_sb | q_ss | q_sh | k_sb | k_ss | k_sh | v_sb | v_ss | v_sh | o_sb | o_ss | o_sh) & 7) return 3102;
  CUtensorMap tq;
  KVMaps maps;
  Params p;
  int rc = make_map(&tq, q, HD, B, q_len, H, q_sb, q_ss, q_sh, BQ);
  if (rc) return rc;
  for (int s = 0; s < MAX_SEGMENTS; ++s) {
    const int src = s < num_segments ? s : 0;
    p.kv_len[s] = s < num_segments ? kv_lens[s] : 0;
    const int len = kv_lens[src] > 0 ? kv_lens[src] : 1;
    rc = make_map(&maps.k[s], k_ptrs[src], HD, B, len, H, k_sb, k_ss, k_sh, BKV);
    if (rc) return rc;
    rc = make_map(&maps.v[s], v_ptrs[src], HD, B, len, H, v_sb, v_ss, v_sh, BKV);
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
  p.flag_stride = 1;
  p.heads_per_group = H;
  if ((m_fixed == nullptr) != (fixed_heads == nullptr)) return 3105;
  p.m_fixed = m_fixed;
  p.fixed_heads = fixed_heads;
  p.out_scatter_n = 0;
  p.out_rows_per_rank = 1;
  p.out_head_off = 0;
  for (int i = 0; i < MAX_SEGMENTS; ++i) p.out_peers[i] = nullptr;
  if (scatter != nullptr && scatter->n > 0) {
    if (scatter->n > MAX_SEGMENTS || scatter->rows_per_rank <= 0 || lse != nullptr) return 3109;
    if (static_cast<long long>(scatter->n) * scatter->rows_per_rank < q_len) return 3109;
    p.out_scatter_n = scatter->n;
    p.out_rows_per_rank = scatter->rows_per_rank;
    p.out_head_off = scatter->head_off;
    for (int i = 0; i < scatter->n; ++i) p.out_peers[i] = reinterpret_cast<__nv_bfloat16*>(scatter->ptrs[i]);
  }
  p.status = status_buffer();
  CopyPlan cp;
  memset(&cp, 0, sizeof(cp));
  if (plan != nullptr && plan->n_remote > 0) {
    if (plan->n_remote > MAX_REMOTE || plan->n_remote != num_segments - 1 || (plan->nbytes & 15) ||
        plan->n_copy_ctas < 1 || plan->n_ack > MAX_SEGMENTS || seg_flags == nullptr)
      return 3103;
    cp.n_remote = plan->n_remote;
    cp.n_copy_ctas = plan->n_copy_ctas;
    for (int i = 0; i < plan->n_remote; ++i) {
      for (int t = 0; t < 2; ++t) {
        cp.src[i][t] = reinterpret_cast<const uint4*>(plan->src[i][t]);
        cp.dst[i][t] = reinterpret_cast<uint4*>(plan->dst[i][t]);
      }
      cp.ready[i] = reinterpret_cast<const unsigned int*>(plan->ready[i]);
    }
    cp.epoch = plan->epoch;
    cp.counters = reinterpret_cast<unsigned int*>(plan->counters);
    cp.seg_flags = reinterpret_cast<unsigned int*>(plan->seg_flags);
    cp.n_ack = plan->n_ack;
    for (int a = 0; a < plan->n_ack; ++a) cp.ack[a] = reinterpret_cast<unsigned int*>(plan->ack[a]);
  }
  const int n_qb = (q_len + 2 * BQ - 1) / (2 * BQ);
  const long long total_work = static_cast<long long>(n_qb) * H * B;
  int n_copy = cp.n_remote > 0 ? cp.n_copy_ctas : 0;
  if (n_copy > 0) {
    // Copy CTAs that cost no extra wave of work items are free: 640 items (8 ranks, 4096 queries each) take 5 rounds
    // on anything from 128 to 148 compute CTAs, so the copies may have 20 SMs instead of 12.
    const auto rounds = [&](int copy) { return (total_work + sm_count() - copy - 1) / (sm_count() - copy); };
    while (n_copy < 32 && sm_count() - (n_copy + 1) >= 1 && rounds(n_copy + 1) == rounds(cp.n_copy_ctas)) ++n_copy;
    cp.n_copy_ctas = n_copy;
  }
  int n_compute = sm_count() - n_copy;
  if (n_compute < 1) return 3104;
  if (total_work < n_compute) n_compute = static_cast<int>(total_work);
  if (n_copy > 0) {
    // Head groups. The compute CTAs take the work list in rounds of n_compute items and the list runs through the
    // q blocks of head 0, then head 1, ...: a round covers n_compute / n_qb heads. One group per round lets the first
    // round start after 1 / rounds of the bytes; more than MAX_GROUPS rounds share groups.
    const long long row_bytes = static_cast<long long>(H) * HD * 2;
    if (plan->nbytes % row_bytes != 0) return 3106;
    int hpg = n_compute / n_qb;
    if (hpg < 1) hpg = 1;
    if (hpg > H) hpg = H;
    if ((H + hpg - 1) / hpg > MAX_GROUPS) hpg = (H + MAX_GROUPS - 1) / MAX_GROUPS;
    if (plan->n_groups == 1) hpg = H;
    else if (plan->n_groups > 1 && plan->n_groups <= MAX_GROUPS) hpg = (H + plan->n_groups - 1) / plan->n_groups;
    cp.n_groups = (H + hpg - 1) / hpg;
    cp.rows = static_cast<unsigned int>(plan->nbytes / row_bytes);
    cp.row_vecs = static_cast<unsigned int>(row_bytes >> 4);
    cp.group_vecs = static_cast<unsigned int>((static_cast<long long>(hpg) * HD * 2) >> 4);
    if (static_cast<long long>(cp.rows) * cp.row_vecs >= (1ll << 31)) return 3107;  // slab indices are 32-bit
    p.flag_stride = MAX_GROUPS;
    p.heads_per_group = hpg;
  }
  if (g_tune_copy_ctas > 0 && n_copy > 0) {
    // the tile search pins the number of copy CTAs (the automatic choice above is bypassed)
    n_copy = g_tune_copy_ctas < sm_count() - 1 ? g_tune_copy_ctas : sm_count() - 1;
    cp.n_copy_ctas = n_copy;
    n_compute = sm_count() - n_copy;
    if (total_work < n_compute) n_compute = static_cast<int>(total_work);
  }
  const dim3 grid(n_compute + n_copy);
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  g_last_stages = g_tune_stages > 0 ? g_tune_stages : DEFAULT_KV_STAGES;
  g_last_copy_ctas = n_copy;
  switch (g_tune_stages > 0 ? g_tune_stages : DEFAULT_KV_STAGES) {
    case 2: return launch_variant<HD, 2>(grid, st, tq, maps, p, cp);
    case 3: return launch_variant<HD, 3>(grid, st, tq, maps, p, cp);
    case 5: return launch_variant<HD, 5>(grid, st, tq, maps, p, cp);
    default: return launch_variant<HD, 4>(grid, st, tq, maps, p, cp);
  }
}

extern "C" int mdb_flash_fwd(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* out,
                             float* lse, int B, int H, int q_len, int num_segments, const int* kv_lens,
                             long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                             long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_sb,
                             long long o_ss, long long o_sh, float softmax_scale, const unsigned int* seg_flags,
                             unsigned int flag_target, const MdbCopyPlan* plan, void* stream_ptr) {
  return flash_fwd_launch<128>(q, k_ptrs, v_ptrs, out, lse, B, H, q_len, num_segments, kv_lens, q_sb, q_ss, q_sh, k_sb,
                               k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, softmax_scale, seg_flags, flag_target,
                               plan, stream_ptr);
}

// head_dim 128 with the output scattered to the sequence owners (the reverse Ulysses exchange in the epilogue): `out`
// is unused, the o strides describe every peer's [B, rows_per_rank, heads_total, 128] output, no log-sum-exp is written.
extern "C" int mdb_flash_fwd_scatter(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, int B, int H,
                                     int q_len, int num_segments, const int* kv_lens, long long q_sb, long long q_ss,
                                     long long q_sh, long long k_sb, long long k_ss, long long k_sh, long long v_sb,
                                     long long v_ss, long long v_sh, long long o_sb, long long o_ss, long long o_sh,
                                     float softmax_scale, const unsigned int* seg_flags, unsigned int flag_target,
                                     const MdbCopyPlan* plan, const MdbOutScatter* scatter, void* stream_ptr) {
  if (scatter == nullptr || scatter->n < 1) return 3109;
  return flash_fwd_launch<128>(q, k_ptrs, v_ptrs, nullptr, nullptr, B, H, q_len, num_segments, kv_lens, q_sb, q_ss, q_sh, k_sb,
                               k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, softmax_scale, seg_flags, flag_target,
                               plan, stream_ptr, nullptr, nullptr, scatter);
}

// Same for head_dim 64 (Stable Diffusion / SDXL / LTX-Video heads).
extern "C" int mdb_flash_fwd_d64(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* out,
                                 float* lse, int B, int H, int q_len, int num_segments, const int* kv_lens,
                                 long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                                 long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_sb,
                                 long long o_ss, long long o_sh, float softmax_scale, const unsigned int* seg_flags,
                                 unsigned int flag_target, const MdbCopyPlan* plan, void* stream_ptr) {
  return flash_fwd_launch<64>(q, k_ptrs, v_ptrs, out, lse, B, H, q_len, num_segments, kv_lens, q_sb, q_ss, q_sh, k_sb,
                              k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, softmax_scale, seg_flags, flag_target,
                              plan, stream_ptr);
}

// The same kernels with the fixed-exponent softmax: m_fixed fp32 [B, H, q_len] (log2 domain), fixed_heads
// int32 [H] (non-zero: the head uses m_fixed; zero: the head keeps the running maximum).
extern "C" int mdb_flash_fwd_fixed_m(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* out,
                                     float* lse, int B, int H, int q_len, int num_segments, const int* kv_lens,
                                     long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                                     long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_sb,
                                     long long o_ss, long long o_sh, float softmax_scale,
                                     const unsigned int* seg_flags, unsigned int flag_target, const MdbCopyPlan* plan,
                                     void* stream_ptr, const float* m_fixed, const int* fixed_heads) {
  if (m_fixed == nullptr || fixed_heads == nullptr) return 3105;
  return flash_fwd_launch<128>(q, k_ptrs, v_ptrs, out, lse, B, H, q_len, num_segments, kv_lens, q_sb, q_ss, q_sh, k_sb,
                               k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, softmax_scale, seg_flags, flag_target,
                               plan, stream_ptr, m_fixed, fixed_heads);
}
extern "C" int mdb_flash_fwd_fixed_m_d64(const void* q, const void* const* k_ptrs, const void* const* v_ptrs,
                                         void* out, float* lse, int B, int H, int q_len, int num_segments,
                                         const int* kv_lens, long long q_sb, long long q_ss, long long q_sh,
                                         long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                                         long long v_sh, long long o_sb, long long o_ss, long long o_sh,
                                         float softmax_scale, const unsigned int* seg_flags, unsigned int flag_target,
                                         const MdbCopyPlan* plan, void* stream_ptr, const float* m_fixed,
                                         const int* fixed_heads) {
  if (m_fixed == nullptr || fixed_heads == nullptr) return 3105;
  return flash_fwd_launch<64>(q, k_ptrs, v_ptrs, out, lse, B, H, q_len, num_segments, kv_lens, q_sb, q_ss, q_sh, k_sb,
                              k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, softmax_scale, seg_flags, flag_target,
                              plan, stream_ptr, m_fixed, fixed_heads);
}
