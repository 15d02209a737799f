// Peer-memory communication kernels over NVLink / NVSwitch. All pointers named "peer" are device
// addresses of other GPUs' symmetric buffers mapped into this process; they are accessed with plain
// loads / stores (and st.release.sys / ld.acquire.sys for flags) — never through a TMA multicast.
//
//   signal_peers   : publish an epoch number in a slot of every peer's signal pad
//   wait_flags     : bounded wait until a set of local signal slots reached an epoch (status on timeout)
//   set_flag       : stream-ordered release store of one flag (marks a staged segment as ready)
//   rs_adamw       : fused gradient reduce-scatter + statistics + AdamW. The owner of a parameter slice
//                    pulls that slice of every rank's gradient buffer, sums the ranks in a fixed order
//                    (bitwise reproducible), accumulates sum-of-squares / max-abs of the reduced gradient
//                    and applies AdamW to its slice of weights and moments in the same pass.
//   small_allreduce: one-shot all-reduce (sum / max) of a few KB: every rank publishes its vector in its own
//                    symmetric buffer, signals, waits (bounded) for the others and reduces all vectors in rank order,
//                    so every rank gets bitwise the same result. One launch, one CTA; two buffer halves alternate by
//                    epoch so that a fast rank cannot overwrite data a slow rank still reads. Replaces the scalar
//                    NCCL all-reduces of the gradient norm / max-abs / loss (reference: optax global-norm clipping,
//                    src/maxdiffusion/max_utils.py:683-696) and the `process_allgather` of tile-search timings.
//   peer_copy      : pull copy peer -> local with 16-byte vectors (used where a copy engine is not wanted)
//
// rs_adamw replaces NCCL reduce-scatter followed by the optax update of the reference
// (src/maxdiffusion/trainers/wan_trainer.py:169-189, src/maxdiffusion/max_utils.py:683-696).
#include "host_common.h"

namespace mdb {
namespace comm {

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  const void* p[MAX_RANKS];
};
struct PeerFlagPtrs {
  unsigned int* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(unsigned int* addr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__global__ void signal_peers_kernel(PeerFlagPtrs flags, int n, int slot, unsigned int value) {
  const int i = threadIdx.x;
  if (i < n && flags.p[i] != nullptr) {
    __threadfence_system();
    st_release_sys(flags.p[i] + slot, value);
  }
}

// Thread i waits until flags[i * stride] >= target. A wait that runs out of its budget reports
// {where = 100, detail = i} in the status word; the host turns that into an exception. Once a failure is recorded
// every later wait returns at once: a sequence of exchanges queued behind a failed one costs one budget, not one each.
__global__ void wait_flags_kernel(const unsigned int* flags, int n, int stride, unsigned int target,
                                  unsigned long long budget_ns, DeviceStatus* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  if (status_failed(status)) return;
  const uint64_t t0 = global_timer_ns();
  unsigned int spins = 0;
  while (ld_acquire_sys(flags + static_cast<long long>(i) * stride) < target) {
    if ((++spins & 0x3fu) == 0u) {
      __nanosleep(200);
      if (status_failed(status)) return;
      if (global_timer_ns() - t0 > budget_ns) {
        report_status(status, kStatusFlagTimeout, 100, static_cast<unsigned int>(i));
        return;
      }
    }
  }
}

__global__ void set_flag_kernel(unsigned int* flag, unsigned int value) {
  if (threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys(flag, value);
  }
}

__global__ void peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    dst[i] = src[i];
  }
}

// All-gather by pulls: dst[r * nvec + i] = srcs.p[r][i] for every rank r; blockIdx.y selects the source, so all
// peers are read concurrently and every byte crosses NVLink once. 4 loads of 16 bytes in flight per thread.
__global__ void __launch_bounds__(512) pull_gather_kernel(PeerFlagPtrs srcs, uint4* __restrict__ dst, long long nvec) {
  const uint4* __restrict__ src = reinterpret_cast<const uint4*>(srcs.p[blockIdx.y]);
  uint4* __restrict__ out = dst + static_cast<long long>(blockIdx.y) * nvec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) r[u] = __ldcg(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u) out[i + u * stride] = r[u];
  }
  for (; i < nvec; i += stride) out[i] = __ldcg(src + i);
}

// All-to-all by pulls with the layout change fused (the Ulysses exchange). For every source rank r (blockIdx.y) a
// block of n_b x n_s rows of row_vecs 16-byte vectors is read from srcs.p[r] (row (b, s) at b * src_sb + s * src_ss)
// and written to dst + r * dst_sr + b * dst_sb + s * dst_ss; all strides in 16-byte vectors. With the right strides
// this is [B, S, H, D] -> [B, n S, H / n, D] (rows = the H / n heads this rank keeps) and its inverse, without the
// permute + contiguous passes that a library all-to-all needs on both sides.
__global__ void __launch_bounds__(512) pull_a2a_kernel(PeerFlagPtrs srcs, uint4* __restrict__ dst, int n_b, int n_s,
                                                       int row_vecs, long long src_sb, long long src_ss,
                                                       long long dst_sr, long long dst_sb, long long dst_ss) {
  const uint4* __restrict__ src = reinterpret_cast<const uint4*>(srcs.p[blockIdx.y]);
  uint4* __restrict__ out = dst + static_cast<long long>(blockIdx.y) * dst_sr;
  const long long total = static_cast<long long>(n_b) * n_s * row_vecs;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += 4 * stride) {
    uint4 r[4];
    long long d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long j = i + u * stride;
      if (j < total) {
        const int v = static_cast<int>(j % row_vecs);
        const long long row = j / row_vecs;
        const int sidx = static_cast<int>(row % n_s);
        const int b = static_cast<int>(row / n_s);
        r[u] = __ldcg(src + b * src_sb + sidx * src_ss + v);
        d[u] = b * dst_sb + sidx * dst_ss + v;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i + u * stride < total) out[d[u]] = r[u];
    }
  }
}

// Owner-side reduce of a reduce-scatter: out[i] = sum over ranks r (in rank order, fp32) of srcs.p[r][i], bf16 in and
// out. srcs.p[r] is the address, in rank r's symmetric buffer, of the slice that belongs to this rank, so every byte
// crosses NVLink once and the sum is rounded once. 16-byte loads, 4 ranks in flight per thread.
__global__ void __launch_bounds__(512) pull_reduce_kernel(PeerFlagPtrs srcs, int world, uint4* __restrict__ out,
                                                          long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
    for (int r0 = 0; r0 < world; r0 += 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u < world) v[u] = __ldcg(reinterpret_cast<const uint4*>(srcs.p[r0 + u]) + i);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u < world) {
          const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(w[e]);
            acc[2 * e] += f.x;
            acc[2 * e + 1] += f.y;
          }
        }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    out[i] = o;
  }
}

__device__ __forceinline__ float ld_relaxed_sys_f32(const float* addr) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(addr) : "memory");
  return v;
}

// bufs.p[r]: rank r's symmetric float buffer of 2 * cap elements; flags.p[r]: rank r's signal pad.
// op 0 = sum, 1 = max. A wait that runs out reports {where = 110, detail = source rank} and leaves `out` untouched.
__global__ void __launch_bounds__(256)
small_allreduce_kernel(const float* __restrict__ in, float* __restrict__ out, int n, int op, PeerPtrs bufs,
                       PeerFlagPtrs flags, int world, int rank, int slot_base, int cap, unsigned int epoch,
                       unsigned long long budget_ns, DeviceStatus* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  const int half = static_cast<int>(epoch & 1u) * cap;
  float* mine = const_cast<float*>(static_cast<const float*>(bufs.p[rank])) + half;
  for (int i = threadIdx.x; i < n; i += blockDim.x) mine[i] = in[i];
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flags.p[threadIdx.x] + slot_base + rank, epoch);
    const unsigned int* my_flag = flags.p[rank] + slot_base + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    unsigned int spins = 0;
    while (ld_acquire_sys(my_flag) < epoch) {
      if ((++spins & 0x3fu) == 0u) {
        __nanosleep(100);
        if (status_failed(status)) {
          atomicExch(&failed, 1);
          break;
        }
        if (global_timer_ns() - t0 > budget_ns) {
          report_status(status, kStatusFlagTimeout, 110, threadIdx.x);
          atomicExch(&failed, 1);
          break;
        }
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  if (failed) return;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float acc = ld_relaxed_sys_f32(static_cast<const float*>(bufs.p[0]) + half + i);
    for (int r = 1; r < world; ++r) {
      const float v = ld_relaxed_sys_f32(static_cast<const float*>(bufs.p[r]) + half + i);
      acc = op == 0 ? acc + v : fmaxf(acc, v);
    }
    out[i] = acc;
  }
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, grad_scale, clip_value;
  unsigned long long seed;
  int stochastic;
};

__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return static_cast<uint32_t>(x);
}
__device__ __forceinline__ __nv_bfloat16 round_bf16(float v, int stochastic, uint64_t key) {
  if (!stochastic) return __float2bfloat16_rn(v);
  uint32_t bits = __float_as_uint(v);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16_rn(v);
  bits += hash32(key) & 0xffffu;
  return __ushort_as_bfloat16(static_cast<unsigned short>(bits >> 16));
}

template <typename ST> __device__ __forceinline__ float st_to_f(ST v);
template <> __device__ __forceinline__ float st_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float st_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename ST> __device__ __forceinline__ ST f_to_st(float v);
template <> __device__ __forceinline__ float f_to_st<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 f_to_st<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// grads.p[r] points at rank r's bf16 gradient buffer, already offset to this owner's slice.
// n is a multiple of 8. partial[block] = {sum g^2, max |g|} of the reduced gradient. When `apply` is 0
// only the reduced gradient (bf16, to `reduced_out`) and the statistics are produced.
template <typename ST>
__global__ void __launch_bounds__(512)
rs_adamw_kernel(PeerPtrs grads, int world, long long n, __nv_bfloat16* __restrict__ p, ST* __restrict__ m,
                ST* __restrict__ v, __nv_bfloat16* __restrict__ reduced_out, float2* __restrict__ partial,
                int apply, AdamArgs a) {
  float sq = 0.0f, mx = 0.0f;
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = 0.0f;
    uint4 buf[MAX_RANKS];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < world) buf[r] = reinterpret_cast<const uint4*>(grads.p[r])[i];
    }
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < world) {
        const uint32_t w[4] = {buf[r].x, buf[r].y, buf[r].z, buf[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          g[2 * j] += f.x;
          g[2 * j + 1] += f.y;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      g[j] *= a.grad_scale;
      sq += g[j] * g[j];
      mx = fmaxf(mx, fabsf(g[j]));
    }
    if (reduced_out != nullptr) {
      uint4 o;
      o.x = pack_bf16x2(g[0], g[1]); o.y = pack_bf16x2(g[2], g[3]);
      o.z = pack_bf16x2(g[4], g[5]); o.w = pack_bf16x2(g[6], g[7]);
      reinterpret_cast<uint4*>(reduced_out)[i] = o;
    }
    if (apply) {
      const long long e0 = i * 8;
      const uint4 pw = reinterpret_cast<const uint4*>(p)[i];
      const uint32_t pwv[4] = {pw.x, pw.y, pw.z, pw.w};
      float w8[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(pwv[j]);
        w8[2 * j] = f.x;
        w8[2 * j + 1] = f.y;
      }
      __nv_bfloat16 outw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float gj = g[j];
        if (a.clip_value > 0.0f) gj = fminf(fmaxf(gj, -a.clip_value), a.clip_value);
        const float mi = a.b1 * st_to_f<ST>(m[e0 + j]) + (1.0f - a.b1) * gj;
        const float vi = a.b2 * st_to_f<ST>(v[e0 + j]) + (1.0f - a.b2) * gj * gj;
        m[e0 + j] = f_to_st<ST>(mi);
        v[e0 + j] = f_to_st<ST>(vi);
        float w = w8[j];
        w -= a.lr * ((mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps) + a.wd * w);
        outw[j] = round_bf16(w, a.stochastic, a.seed + static_cast<uint64_t>(e0 + j));
      }
      reinterpret_cast<uint4*>(p)[i] = *reinterpret_cast<uint4*>(outw);
    }
  }
  __shared__ float ss[16], sm[16];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0) { ss[threadIdx.x >> 5] = sq; sm[threadIdx.x >> 5] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ts = 0.0f, tm = 0.0f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) { ts += ss[i]; tm = fmaxf(tm, sm[i]); }
    partial[blockIdx.x] = make_float2(ts, tm);
  }
}

__global__ void fold_stats_kernel(const float2* __restrict__ partial, int n, float* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float ts = 0.0f, tm = 0.0f;
    for (int i = 0; i < n; ++i) { ts += partial[i].x; tm = fmaxf(tm, partial[i].y); }
    out[0] += ts;
    out[1] = fmaxf(out[1], tm);
  }
}

}  // namespace comm
}  // namespace mdb

using namespace mdb;
using namespace mdb::comm;

extern "C" int mdb_signal_peers(const unsigned long long* peer_flag_ptrs, int n, int slot, unsigned int value,
                                void* stream) {
  if (n < 0 || n > MAX_RANKS) return 3401;
  PeerFlagPtrs f;
  for (int i = 0; i < MAX_RANKS; ++i) f.p[i] = i < n ? reinterpret_cast<unsigned int*>(peer_flag_ptrs[i]) : nullptr;
  signal_peers_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, n, slot, value);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_wait_flags(const unsigned int* flags, int n, int stride, unsigned int target, double budget_s,
                              void* stream) {
  if (n <= 0) return 0;
  if (n > 32) return 3402;
  wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flags, n, stride, target, static_cast<unsigned long long>(budget_s * 1e9), status_buffer());
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_set_flag(unsigned int* flag, unsigned int value, void* stream) {
  set_flag_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag, value);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_peer_copy(const void* src, void* dst, long long nbytes, int ctas, void* stream) {
  if (nbytes & 15) return 3403;
  if (nbytes == 0) return 0;
  peer_copy_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), nbytes >> 4);
  return static_cast<int>(cudaGetLastError());
}

// src_ptrs: `world` device addresses (rank order) of this rank's slice in every rank's buffer; n_elems bf16 elements,
// a multiple of 8. The caller has waited for the producers' ready flags on this stream.
extern "C" int mdb_pull_reduce(const unsigned long long* src_ptrs, int world, void* out, long long n_elems, int ctas,
                               void* stream) {
  if (world < 1 || world > MAX_RANKS) return 3410;
  if (n_elems & 7) return 3411;
  if (n_elems == 0) return 0;
  PeerFlagPtrs srcs;
  for (int r = 0; r < world; ++r) {
    if (src_ptrs[r] & 15) return 3412;
    srcs.p[r] = reinterpret_cast<unsigned int*>(src_ptrs[r]);
  }
  pull_reduce_kernel<<<ctas > 0 ? ctas : 64, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      srcs, world, static_cast<uint4*>(out), n_elems >> 3);
  return static_cast<int>(cudaGetLastError());
}

// src_ptrs: the address of every rank's shard (rank order, this rank's own included); nbytes per shard, a multiple of
// 16. The caller has waited for the owners' ready flags on this stream.
extern "C" int mdb_pull_gather(const unsigned long long* src_ptrs, int world, void* dst, long long nbytes, int ctas,
                               void* stream) {
  if (world < 1 || world > MAX_RANKS) return 3420;
  if (nbytes & 15) return 3421;
  if (nbytes == 0) return 0;
  PeerFlagPtrs srcs;
  for (int r = 0; r < world; ++r) {
    if (src_ptrs[r] & 15) return 3422;
    srcs.p[r] = reinterpret_cast<unsigned int*>(src_ptrs[r]);
  }
  dim3 grid(ctas > 0 ? ctas : 16, world);
  pull_gather_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(srcs, static_cast<uint4*>(dst), nbytes >> 4);
  return static_cast<int>(cudaGetLastError());
}

// See pull_a2a_kernel; src_ptrs are peer addresses already offset to the first row this rank pulls.
extern "C" int mdb_pull_a2a(const unsigned long long* src_ptrs, int world, void* dst, int n_b, int n_s, int row_bytes,
                            long long src_sb_bytes, long long src_ss_bytes, long long dst_sr_bytes,
                            long long dst_sb_bytes, long long dst_ss_bytes, int ctas, void* stream) {
  if (world < 1 || world > MAX_RANKS) return 3430;
  if ((row_bytes | src_sb_bytes | src_ss_bytes | dst_sr_bytes | dst_sb_bytes | dst_ss_bytes) & 15) return 3431;
  if (n_b <= 0 || n_s <= 0 || row_bytes <= 0) return 0;
  PeerFlagPtrs srcs;
  for (int r = 0; r < world; ++r) {
    if (src_ptrs[r] & 15) return 3432;
    srcs.p[r] = reinterpret_cast<unsigned int*>(src_ptrs[r]);
  }
  dim3 grid(ctas > 0 ? ctas : 16, world);
  pull_a2a_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      srcs, static_cast<uint4*>(dst), n_b, n_s, row_bytes >> 4, src_sb_bytes >> 4, src_ss_bytes >> 4, dst_sr_bytes >> 4,
      dst_sb_bytes >> 4, dst_ss_bytes >> 4);
  return static_cast<int>(cudaGetLastError());
}

// Copy-engine copy between two device addresses of this process (local or peer-mapped); no SM is used.
extern "C" int mdb_memcpy_async(void* dst, const void* src, long long nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  return static_cast<int>(cudaMemcpyAsync(dst, src, static_cast<size_t>(nbytes), cudaMemcpyDeviceToDevice,
                                          static_cast<cudaStream_t>(stream)));
}

// 32-bit store into device memory, issued by the stream itself (a stream memory operation: no kernel, no SM). It runs
// after every earlier operation of the stream, behind a system-wide fence, so a kernel of another stream that polls the
// word with an acquire load sees the copies that precede it in this stream.
extern "C" int mdb_stream_write_value32(void* addr, unsigned int value, void* stream) {
  typedef CUresult (*WriteFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  static WriteFn fn = nullptr;
  if (fn == nullptr) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || f == nullptr) {
      return 3407;
    }
    fn = reinterpret_cast<WriteFn>(f);
  }
  if (addr == nullptr || (reinterpret_cast<uintptr_t>(addr) & 3u) != 0) return 3408;
  const CUresult r = fn(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(addr), value, 0u);
  return r == CUDA_SUCCESS ? 0 : 3409;
}

// buf_ptrs / flag_ptrs: `world` device addresses (this rank's own included). n <= cap floats; epoch must grow by
// one per call on every rank of the group.
extern "C" int mdb_small_allreduce(const float* in, float* out, int n, int op, const unsigned long long* buf_ptrs,
                                   const unsigned long long* flag_ptrs, int world, int rank, int slot_base, int cap,
                                   unsigned int epoch, double budget_s, void* stream) {
  if (world < 1 || world > MAX_RANKS || n < 1 || n > cap || rank < 0 || rank >= world || epoch == 0) return 3405;
  PeerPtrs b;
  PeerFlagPtrs f;
  for (int i = 0; i < MAX_RANKS; ++i) {
    b.p[i] = i < world ? reinterpret_cast<const void*>(buf_ptrs[i]) : nullptr;
    f.p[i] = i < world ? reinterpret_cast<unsigned int*>(flag_ptrs[i]) : nullptr;
  }
  small_allreduce_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      in, out, n, op, b, f, world, rank, slot_base, cap, epoch, static_cast<unsigned long long>(budget_s * 1e9),
      status_buffer());
  return static_cast<int>(cudaGetLastError());
}

// grad_ptrs[r]: address of rank r's gradient slice for this owner (bf16, n elements, n % 8 == 0).
// stats: fp32 [2] accumulated in place; scratch: 2 * ctas floats.
extern "C" int mdb_rs_adamw(const unsigned long long* grad_ptrs, int world, long long n, void* p, void* m, void* v,
                            void* reduced_out, float* stats, float* scratch, int apply, float lr, float b1, float b2,
                            float eps, float wd, float bc1, float bc2, float grad_scale, float clip_value,
                            unsigned long long seed, int stochastic, int state_f32, int ctas, void* stream) {
  if (world < 1 || world > MAX_RANKS || (n & 7)) return 3404;
  if (n == 0) return 0;
  PeerPtrs g;
  for (int i = 0; i < MAX_RANKS; ++i) g.p[i] = i < world ? reinterpret_cast<const void*>(grad_ptrs[i]) : nullptr;
  AdamArgs a{lr, b1, b2, eps, wd, bc1, bc2, grad_scale, clip_value, seed, stochastic};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float2* part = reinterpret_cast<float2*>(scratch);
  if (state_f32)
    rs_adamw_kernel<float><<<ctas, 512, 0, st>>>(g, world, n, static_cast<__nv_bfloat16*>(p), static_cast<float*>(m),
                                                 static_cast<float*>(v), static_cast<__nv_bfloat16*>(reduced_out), part,
                                                 apply, a);
  else
    rs_adamw_kernel<__nv_bfloat16><<<ctas, 512, 0, st>>>(
        g, world, n, static_cast<__nv_bfloat16*>(p), static_cast<__nv_bfloat16*>(m), static_cast<__nv_bfloat16*>(v),
        static_cast<__nv_bfloat16*>(reduced_out), part, apply, a);
  fold_stats_kernel<<<1, 32, 0, st>>>(part, ctas, stats);
  return static_cast<int>(cudaGetLastError());
}
