// Host runtime of libugemm_b200.so: raw device allocations that can be shared
// between the ranks of one node through legacy CUDA IPC handles (the symmetric
// heap the reference obtains from nvshmem.tensor / get_peer_tensor in
// dtensor_scratch.py:19 and dtensor_utils.py:546-552), and TMA descriptor
// encoding through the driver entry point (no link-time dependency on libcuda,
// so the library also loads on a machine without a GPU).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "ugemm_b200.h"

namespace {

thread_local char g_last_error[512] = "";

void set_error(const char* what, int code, const char* detail) {
  snprintf(g_last_error, sizeof(g_last_error), "%s failed with code %d (%s)", what, code, detail ? detail : "");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    set_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", static_cast<int>(e), cudaGetErrorString(e));
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

}  // namespace

extern "C" int ug_version(void) { return 1; }

extern "C" const char* ug_last_error(void) { return g_last_error; }

extern "C" int ug_malloc(uint64_t bytes, uint64_t* out_ptr) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    set_error("cudaMalloc", static_cast<int>(e), cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  *out_ptr = reinterpret_cast<uint64_t>(p);
  return 0;
}

extern "C" int ug_free(uint64_t ptr) {
  cudaError_t e = cudaFree(reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) set_error("cudaFree", static_cast<int>(e), cudaGetErrorString(e));
  return static_cast<int>(e);
}

extern "C" int ug_ipc_get_handle(uint64_t ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) {
    set_error("cudaIpcGetMemHandle", static_cast<int>(e), cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

extern "C" int ug_ipc_open(const void* handle64, uint64_t* out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error("cudaIpcOpenMemHandle", static_cast<int>(e), cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  *out_ptr = reinterpret_cast<uint64_t>(p);
  return 0;
}

extern "C" int ug_ipc_close(uint64_t ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) set_error("cudaIpcCloseMemHandle", static_cast<int>(e), cudaGetErrorString(e));
  return static_cast<int>(e);
}

extern "C" int ug_encode_tensor_map(void* out128, uint64_t base, int dtype, uint64_t inner, uint64_t outer,
                                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                                    int swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  const CUtensorMapDataType dt = dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUtensorMapSwizzle sw = swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  alignas(64) CUtensorMap map;
  CUresult r = fn(&map, dt, 2, reinterpret_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled", static_cast<int>(r), "check alignment of base / stride and box extents");
    return static_cast<int>(r);
  }
  memcpy(out128, &map, sizeof(map));
  return 0;
}
