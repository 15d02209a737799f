// Runtime glue: per-device status buffer, tensor-map encoder, device properties.
#include <mutex>

#include "host_common.h"

namespace mdb {

namespace {
constexpr int kMaxDevices = 16;
DeviceStatus* g_status_dev[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

DeviceStatus* status_buffer() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status_dev[dev]) return g_status_dev[dev];
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_status_dev[dev]) return g_status_dev[dev];
  DeviceStatus* p = nullptr;
  if (cudaMalloc(&p, sizeof(DeviceStatus)) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, sizeof(DeviceStatus));
  g_status_dev[dev] = p;
  return p;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

static int encode_common(CUtensorMap* map, CUtensorMapDataType dt, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return 1001;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2000 + static_cast<int>(r);
}

int encode_tmap_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_common(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box,
                       CU_TENSOR_MAP_SWIZZLE_128B);
}

int encode_tmap_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_common(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, rank, dims, strides_bytes, box,
                       CU_TENSOR_MAP_SWIZZLE_128B);
}

int encode_tmap_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int swizzle128) {
  return encode_common(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box,
                       swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace mdb

// Reads the device status into `out` (4 uints) and optionally clears it. Synchronises the
// current stream of the calling thread's device only through the copy itself.
extern "C" int mdb_read_status(unsigned int* out, int clear) {
  mdb::DeviceStatus* p = mdb::status_buffer();
  if (!p) return -1;
  mdb::DeviceStatus h;
  cudaError_t e = cudaMemcpy(&h, p, sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  out[0] = h.code;
  out[1] = h.where;
  out[2] = h.block;
  out[3] = h.detail;
  if (clear && h.code != 0) cudaMemset(p, 0, sizeof(h));
  return 0;
}

extern "C" int mdb_sm_count() { return mdb::sm_count(); }
