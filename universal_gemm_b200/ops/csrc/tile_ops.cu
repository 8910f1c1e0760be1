// Stand-alone tile kernels for sm_100a: zeroing, one-sided 2-D copy (pull),
// one-sided 2-D accumulate (push with red.add) and dtype-converting pack/unpack.
//
// They back the tile-level API (get_tile / accumulate_tile / reduce_replicas and
// the redistribute path).  Counterparts in the reference: nvshmem.get in
// dtensor_utils.py:358-366, the Triton atomic-add kernel accumulate_kernels.py:12-60
// and the ATen zero_ / clone calls in stationary_{b,c}_plan.py.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "ugemm_b200.h"

using namespace ugptx;

namespace {

constexpr int kThreads = 256;

__host__ __device__ __forceinline__ bool aligned16(uint64_t a) { return (a & 15ull) == 0ull; }

// ---------------------------------------------------------------- zero
__global__ void __launch_bounds__(kThreads) zero_2d_kernel(uint64_t dst, int64_t ld_bytes, int32_t rows,
                                                           int64_t row_bytes, int vec) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  char* base = reinterpret_cast<char*>(dst);
  if (vec) {
    const int64_t vpr = row_bytes >> 4;
    const int64_t total = vpr * rows;
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int64_t i = tid; i < total; i += stride) {
      const int64_t r = i / vpr, c = i - r * vpr;
      *reinterpret_cast<uint4*>(base + r * ld_bytes + (c << 4)) = z;
    }
  } else {
    const int64_t hpr = row_bytes >> 1;   // 2-byte granules (all supported dtypes are >= 2 bytes)
    const int64_t total = hpr * rows;
    for (int64_t i = tid; i < total; i += stride) {
      const int64_t r = i / hpr, c = i - r * hpr;
      *reinterpret_cast<uint16_t*>(base + r * ld_bytes + (c << 1)) = 0;
    }
  }
}

// ---------------------------------------------------------------- pull (copy)
// Eight 16-byte loads in flight per thread so that a few hundred CTAs cover the
// NVLink round trip when `src` is a peer's memory.
__global__ void __launch_bounds__(kThreads) pull_2d_vec_kernel(uint64_t dst, int64_t dst_ld, uint64_t src,
                                                               int64_t src_ld, int32_t rows, int64_t row_bytes) {
  constexpr int U = 8;
  const int64_t vpr = row_bytes >> 4;
  const int64_t total = vpr * rows;
  const char* s = reinterpret_cast<const char*>(src);
  char* d = reinterpret_cast<char*>(dst);
  const int64_t span = static_cast<int64_t>(blockDim.x) * U;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * span; base < total;
       base += static_cast<int64_t>(gridDim.x) * span) {
    uint4 buf[U];
    int64_t off[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x + threadIdx.x;
      off[u] = -1;
      if (i < total) {
        const int64_t r = i / vpr, c = i - r * vpr;
        buf[u] = ld_stream_v4(s + r * src_ld + (c << 4));
        off[u] = r * dst_ld + (c << 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (off[u] >= 0) *reinterpret_cast<uint4*>(d + off[u]) = buf[u];
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) pull_2d_elem_kernel(uint64_t dst, int64_t dst_ld, uint64_t src,
                                                                int64_t src_ld, int32_t rows, int64_t cols) {
  const int64_t total = cols * rows;
  const char* s = reinterpret_cast<const char*>(src);
  char* d = reinterpret_cast<char*>(dst);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    *reinterpret_cast<T*>(d + r * dst_ld + c * sizeof(T)) =
        *reinterpret_cast<const T*>(s + r * src_ld + c * sizeof(T));
  }
}

// ---------------------------------------------------------------- accumulate (push)
__global__ void __launch_bounds__(kThreads) accumulate_f32_kernel(float* dst, int64_t dst_ld, const float* src,
                                                                  int64_t src_ld, int32_t rows, int32_t cols,
                                                                  int vec) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const int64_t vpr = cols >> 2;
    const int64_t total = vpr * rows;
    for (int64_t i = tid; i < total; i += stride) {
      const int64_t r = i / vpr, c = (i - r * vpr) << 2;
      const float4 v = *reinterpret_cast<const float4*>(src + r * src_ld + c);
      red_add_v4_f32(dst + r * dst_ld + c, v.x, v.y, v.z, v.w);
    }
  } else {
    const int64_t total = static_cast<int64_t>(cols) * rows;
    for (int64_t i = tid; i < total; i += stride) {
      const int64_t r = i / cols, c = i - r * cols;
      red_add_f32(dst + r * dst_ld + c, src[r * src_ld + c]);
    }
  }
}

__global__ void __launch_bounds__(kThreads) accumulate_bf16_kernel(__nv_bfloat16* dst, int64_t dst_ld,
                                                                   const __nv_bfloat16* src, int64_t src_ld,
                                                                   int32_t rows, int32_t cols, int vec) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const int64_t vpr = cols >> 3;
    const int64_t total = vpr * rows;
    for (int64_t i = tid; i < total; i += stride) {
      const int64_t r = i / vpr, c = (i - r * vpr) << 3;
      const uint4 v = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
      red_add_v4_bf16x2(dst + r * dst_ld + c, v.x, v.y, v.z, v.w);
    }
  } else {
    const int64_t total = static_cast<int64_t>(cols) * rows;
    for (int64_t i = tid; i < total; i += stride) {
      const int64_t r = i / cols, c = i - r * cols;
      atomicAdd(dst + r * dst_ld + c, src[r * src_ld + c]);
    }
  }
}

// ---------------------------------------------------------------- convert (pack / unpack)
template <typename D, typename S>
__device__ __forceinline__ D cvt(S v);
template <> __device__ __forceinline__ float cvt<float, float>(float v) { return v; }
template <> __device__ __forceinline__ float cvt<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16, __nv_bfloat16>(__nv_bfloat16 v) { return v; }

template <typename D, typename S>
__global__ void __launch_bounds__(kThreads) convert_2d_kernel(D* dst, int64_t dst_ld, const S* src, int64_t src_ld,
                                                              int32_t rows, int32_t cols) {
  const int64_t total = static_cast<int64_t>(cols) * rows;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    dst[r * dst_ld + c] = cvt<D, S>(src[r * src_ld + c]);
  }
}

// Eight elements per thread with 16-byte accesses on the 2-byte side (both sides 16-byte aligned, cols % 8 == 0).
__global__ void __launch_bounds__(kThreads) convert_f32_to_bf16_vec_kernel(__nv_bfloat16* dst, int64_t dst_ld,
                                                                           const float* src, int64_t src_ld,
                                                                           int32_t rows, int32_t cols) {
  const int64_t vpr = cols >> 3;
  const int64_t total = vpr * rows;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vpr, c = (i - r * vpr) << 3;
    const float4 lo = *reinterpret_cast<const float4*>(src + r * src_ld + c);
    const float4 hi = *reinterpret_cast<const float4*>(src + r * src_ld + c + 4);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
    uint4 out;
    out.x = *reinterpret_cast<uint32_t*>(&p0); out.y = *reinterpret_cast<uint32_t*>(&p1);
    out.z = *reinterpret_cast<uint32_t*>(&p2); out.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(dst + r * dst_ld + c) = out;
  }
}

__global__ void __launch_bounds__(kThreads) convert_bf16_to_f32_vec_kernel(float* dst, int64_t dst_ld,
                                                                           const __nv_bfloat16* src, int64_t src_ld,
                                                                           int32_t rows, int32_t cols) {
  const int64_t vpr = cols >> 3;
  const int64_t total = vpr * rows;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vpr, c = (i - r * vpr) << 3;
    const uint4 in = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    const float2 c2 = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
    *reinterpret_cast<float4*>(dst + r * dst_ld + c) = make_float4(a.x, a.y, b.x, b.y);
    *reinterpret_cast<float4*>(dst + r * dst_ld + c + 4) = make_float4(c2.x, c2.y, d.x, d.y);
  }
}

int grid_for(int64_t work_items, int per_thread) {
  int64_t blocks = (work_items + static_cast<int64_t>(kThreads) * per_thread - 1) / (static_cast<int64_t>(kThreads) * per_thread);
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return static_cast<int>(blocks);
}

}  // namespace

extern "C" int ug_zero_2d(uint64_t dst, int64_t ld_bytes, int32_t rows, int64_t row_bytes, void* stream) {
  if (rows <= 0 || row_bytes <= 0) return 0;
  if (row_bytes & 1) return static_cast<int>(cudaErrorInvalidValue);
  const int vec = ((dst & 15ull) == 0 && (ld_bytes & 15) == 0 && (row_bytes & 15) == 0) ? 1 : 0;
  const int64_t items = vec ? (row_bytes >> 4) * rows : (row_bytes >> 1) * rows;
  zero_2d_kernel<<<grid_for(items, 4), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(dst, ld_bytes, rows,
                                                                                        row_bytes, vec);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ug_pull_2d(uint64_t dst, int64_t dst_ld_bytes, uint64_t src, int64_t src_ld_bytes, int32_t rows,
                          int64_t row_bytes, int32_t elem_bytes, void* stream) {
  if (rows <= 0 || row_bytes <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = (dst & 15ull) == 0 && (src & 15ull) == 0 && (dst_ld_bytes & 15) == 0 &&
                   (src_ld_bytes & 15) == 0 && (row_bytes & 15) == 0;
  if (vec) {
    pull_2d_vec_kernel<<<grid_for((row_bytes >> 4) * rows, 8), kThreads, 0, st>>>(dst, dst_ld_bytes, src,
                                                                                 src_ld_bytes, rows, row_bytes);
  } else if (elem_bytes == 2) {
    pull_2d_elem_kernel<uint16_t><<<grid_for((row_bytes >> 1) * rows, 4), kThreads, 0, st>>>(
        dst, dst_ld_bytes, src, src_ld_bytes, rows, row_bytes >> 1);
  } else if (elem_bytes == 4) {
    pull_2d_elem_kernel<uint32_t><<<grid_for((row_bytes >> 2) * rows, 4), kThreads, 0, st>>>(
        dst, dst_ld_bytes, src, src_ld_bytes, rows, row_bytes >> 2);
  } else {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ug_accumulate_2d(uint64_t dst, int64_t dst_ld_elems, uint64_t src, int64_t src_ld_elems,
                                int32_t rows, int32_t cols, int32_t dtype, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    const int vec = (aligned16(dst) && aligned16(src) && (dst_ld_elems & 3) == 0 && (src_ld_elems & 3) == 0 &&
                     (cols & 3) == 0) ? 1 : 0;
    const int64_t items = vec ? static_cast<int64_t>(cols >> 2) * rows : static_cast<int64_t>(cols) * rows;
    accumulate_f32_kernel<<<grid_for(items, 4), kThreads, 0, st>>>(
        reinterpret_cast<float*>(dst), dst_ld_elems, reinterpret_cast<const float*>(src), src_ld_elems, rows,
        cols, vec);
  } else if (dtype == 1) {
    const int vec = (aligned16(dst) && aligned16(src) && (dst_ld_elems & 7) == 0 && (src_ld_elems & 7) == 0 &&
                     (cols & 7) == 0) ? 1 : 0;
    const int64_t items = vec ? static_cast<int64_t>(cols >> 3) * rows : static_cast<int64_t>(cols) * rows;
    accumulate_bf16_kernel<<<grid_for(items, 4), kThreads, 0, st>>>(
        reinterpret_cast<__nv_bfloat16*>(dst), dst_ld_elems, reinterpret_cast<const __nv_bfloat16*>(src),
        src_ld_elems, rows, cols, vec);
  } else {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ug_convert_2d(uint64_t dst, int64_t dst_ld_elems, int32_t dst_dtype, uint64_t src,
                             int64_t src_ld_elems, int32_t src_dtype, int32_t rows, int32_t cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = (cols & 7) == 0 && aligned16(dst) && aligned16(src) && (dst_ld_elems & 7) == 0 && (src_ld_elems & 7) == 0;
  if (vec && dst_dtype == 1 && src_dtype == 0) {
    convert_f32_to_bf16_vec_kernel<<<grid_for(static_cast<int64_t>(rows) * (cols >> 3), 2), kThreads, 0, st>>>(
        reinterpret_cast<__nv_bfloat16*>(dst), dst_ld_elems, reinterpret_cast<const float*>(src), src_ld_elems, rows, cols);
    return static_cast<int>(cudaGetLastError());
  }
  if (vec && dst_dtype == 0 && src_dtype == 1) {
    convert_bf16_to_f32_vec_kernel<<<grid_for(static_cast<int64_t>(rows) * (cols >> 3), 2), kThreads, 0, st>>>(
        reinterpret_cast<float*>(dst), dst_ld_elems, reinterpret_cast<const __nv_bfloat16*>(src), src_ld_elems, rows, cols);
    return static_cast<int>(cudaGetLastError());
  }
  const int g = grid_for(static_cast<int64_t>(rows) * cols, 4);
#define UG_CVT(D, S)                                                                                   \
  convert_2d_kernel<D, S><<<g, kThreads, 0, st>>>(reinterpret_cast<D*>(dst), dst_ld_elems,             \
                                                  reinterpret_cast<const S*>(src), src_ld_elems, rows, cols)
  if (dst_dtype == 0 && src_dtype == 0) UG_CVT(float, float);
  else if (dst_dtype == 0 && src_dtype == 1) UG_CVT(float, __nv_bfloat16);
  else if (dst_dtype == 1 && src_dtype == 0) UG_CVT(__nv_bfloat16, float);
  else if (dst_dtype == 1 && src_dtype == 1) UG_CVT(__nv_bfloat16, __nv_bfloat16);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef UG_CVT
  return static_cast<int>(cudaGetLastError());
}
