// Host-side helpers shared by the tcgen05 translation units: TMA descriptor encoding, per-device
// caches (compute capability, SM count, kernel attributes).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace faws {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// (rows, 64 x 16-bit) boxes out of a (B, H, S, D) view
inline bool make_map_bhsd(CUtensorMap* m, const void* base, int D, int rows, int H, int B, int64_t ss, int64_t sh,
                   int64_t sb, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t row_bytes = (cuuint64_t)ss * 2;
  cuuint64_t strides[3] = {row_bytes, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  if (H == 1) strides[1] = row_bytes * (cuuint64_t)rows;
  if (B == 1) strides[2] = strides[1] * (cuuint64_t)H;
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 32 x 32 fp32 boxes into a (BH, rows, cols) tensor whose rows are `row_stride` floats apart
// (esize = 2: 32-row x 64-column boxes of 16-bit elements, same 128-byte box rows)
inline bool make_map_store_f32(CUtensorMap* m, void* base, int cols, int rows, int64_t row_stride,
                        int64_t bh_stride, int BH, int esize = 4) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride * esize, (cuuint64_t)bh_stride * esize};
  cuuint32_t box[3] = {(cuuint32_t)(128 / esize), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

inline bool ok16(const void* ptr, int64_t a, int64_t b, int64_t c) {
  return (reinterpret_cast<uintptr_t>(ptr) % 16 == 0) && a % 8 == 0 && b % 8 == 0 && c % 8 == 0;
}

constexpr int kMaxDevices = 64;

// Current device ordinal, or -1.
inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// Compute capability 10.x of the current device (looked up once per device).
inline bool device_is_sm100() {
  static int cached[kMaxDevices];  // 0 = unknown, 1 = yes, 2 = no
  static std::mutex mu;
  const int dev = current_device();
  if (dev < 0) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
    cached[dev] = (major == 10) ? 1 : 2;
  }
  return cached[dev] == 1;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device setting of a kernel: one flag per
// (kernel instantiation, device), so the first launch on every device of the process sets it.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[kMaxDevices] = {};
};
template <typename K>
inline cudaError_t set_max_smem_once(PerDeviceOnce& once, K kernel, int bytes) {
  const int dev = current_device();
  if (dev < 0) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(once.mu);
  if (!once.done[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    once.done[dev] = true;
  }
  return cudaSuccess;
}

inline int sm_count() {
  static int cached[kMaxDevices];
  const int dev = current_device();
  if (dev < 0) return 148;
  if (cached[dev] == 0) {
    int sms = 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    cached[dev] = sms;
  }
  return cached[dev];
}


// Device address of the per-device status word the tcgen05 kernels raise when a bounded wait gives up.
int* tc_status_word();

}  // namespace faws
