// Host-side helpers shared by the launchers: tensor-map encoding through the driver entry
// point (resolved at run time, so the library links without libcuda), device attributes and
// a small per-pointer cache of encoded maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "launch.cuh"

namespace plow {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

inline CUtensorMapDataType tmap_dtype(int esize) {
  return esize == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
         : esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
}

// Row-major [rows, cols] matrix of `esize`-byte elements with row pitch `ld_bytes`; the box is
// [box_rows, swizzle_bytes] with a swizzle span equal to the box width (128 or 64 bytes), the
// layouts the UMMA descriptors in ptx.cuh assume.  Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* out, const void* base, int esize, uint64_t rows,
                        uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                        uint32_t swizzle_bytes = 128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(swizzle_bytes / esize), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, tmap_dtype(esize), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// [d2, d1, d0] tensor, innermost d0 contiguous; box [box2, box1, swizzle_bytes].
inline int make_tmap_3d(CUtensorMap* out, const void* base, int esize, uint64_t d0, uint64_t d1,
                        uint64_t d2, uint64_t ld1_bytes, uint64_t ld2_bytes, uint32_t box1,
                        uint32_t box2 = 1, uint32_t swizzle_bytes = 128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1_bytes, ld2_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(swizzle_bytes / esize), box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, tmap_dtype(esize), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// SM count of the current device (cached per device: a process may drive several GPUs).
inline int sm_count() {
  static int n[kMaxDevices] = {};
  const int dev = current_device();
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

}  // namespace plow
