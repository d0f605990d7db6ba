// Pieces shared by the tcgen05 MatMul kernels (dsd_tc.cu, sdd_tc.cu): 16-bit packing, the
// 3-D TMA load and the host-side tensor-map encoder (128-byte swizzle, as the MMA descriptors
// of tc.cuh expect, or the 64-byte one for tiles whose rows hold 32 elements).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "common.h"
#include "tc.cuh"

namespace bsp {
namespace mmtc {

using namespace tc;

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ T cvt1(float a);
template <> __device__ __forceinline__ __half cvt1<__half>(float a) { return __float2half_rn(a); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt1<__nv_bfloat16>(float a) { return __float2bfloat16_rn(a); }
template <typename T> struct Bf { static constexpr int v = 0; };
template <> struct Bf<__nv_bfloat16> { static constexpr int v = 1; };

BSP_DEVI void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(saddr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(saddr(bar)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}


// ---- host ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
}

inline int encode(CUtensorMap* m, const void* ptr, int dtype, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
           const cuuint32_t* box, int swizzle_bytes = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(BSP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  // The encoder is a driver call and needs the primary context bound to this thread; a thread
  // that has made no runtime call yet (a worker thread of the caller) has none.
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  cuuint32_t es[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(m, dtype == BSP_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank,
                  const_cast<void*>(ptr), dims, strides_bytes, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BSP_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return BSP_OK;
}


}  // namespace mmtc
}  // namespace bsp
