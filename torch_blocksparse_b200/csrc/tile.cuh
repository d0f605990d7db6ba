// Device building blocks shared by the block-sparse GEMM kernels:
//   * cp.async tile loader (16-byte chunks, zero fill for out-of-range parts)
//   * warp-level tile product: mma.sync m16n8k16 (FP16 / BF16, FP32 accumulate)
//     fed by ldmatrix, or FFMA for FP32 operands
//   * accumulator -> (row, col, value) iteration for the epilogues
//
// Shared-memory tiles keep the orientation the operand has in global memory,
// so that every copy is a plain 16-byte cp.async:
//   "K-contiguous"  tile[nonK][K]   pitch = TK + PAD
//   "K-strided"     tile[K][nonK]   pitch = extent + PAD
// PAD is 16 bytes, which makes the pitch an odd multiple of 16 bytes: eight
// consecutive rows fall into eight different 16-byte bank groups, so ldmatrix
// and the FP32 reads are conflict free.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace bsp {

template <typename T> struct Elem;
template <> struct Elem<float> { static constexpr int VEC = 4; static constexpr bool MMA = false; };
template <> struct Elem<__half> { static constexpr int VEC = 8; static constexpr bool MMA = true; };
template <> struct Elem<__nv_bfloat16> { static constexpr int VEC = 8; static constexpr bool MMA = true; };

template <typename T> __device__ __forceinline__ T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 2^x on the special-function unit (ex2.approx: about 2 ulp, denormals flushed).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy; copies nothing and zero-fills when !pred.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Copies a tile of ROWS x CONT elements (CONT along the unit-stride direction
// of global memory) into shared memory with row pitch PITCH.  Rows >= rows_ok
// and columns >= cont_ok are zero-filled; `src` always stays a valid address.
template <typename T, int ROWS, int CONT, int PITCH, int NTHREADS>
__device__ __forceinline__ void load_tile(T* smem, const T* src, int64_t row_stride, int tid,
                                          int rows_ok, int cont_ok) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int CPR = CONT / VEC;            // chunks per row
  constexpr int TOTAL = ROWS * CPR;
#pragma unroll
  for (int it = 0; it < (TOTAL + NTHREADS - 1) / NTHREADS; ++it) {
    const int ch = tid + it * NTHREADS;
    if (TOTAL % NTHREADS == 0 || ch < TOTAL) {
      const int r = ch / CPR, c = (ch % CPR) * VEC;
      const bool ok = r < rows_ok && c < cont_ok;
      cp_async16(smem + r * PITCH + c, ok ? src + r * row_stride + c : src, ok);
    }
  }
}

// ---------------------------------------------------------------------------
// Warp tile product.  A is the [M][K] operand, B the [K][N] operand; AKC / BKC
// say whether their shared-memory tiles are K-contiguous.  The accumulator
// layout differs between the two back-ends; use for_each_acc to walk it.
// ---------------------------------------------------------------------------
template <typename T, int WM, int WN> struct Acc {
  static constexpr int COUNT = WM * WN / 32;
  float v[COUNT];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < COUNT; ++i) v[i] = 0.f;
  }
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One K-chunk (TK elements) of the warp tile at rows [m0, m0+WM), cols [n0, n0+WN).
// As / Bs point at the CTA tiles of the current stage; PA / PB are their pitches.
template <typename T, int WM, int WN, int TK, bool AKC, bool BKC, int PA, int PB>
__device__ __forceinline__ void warp_tile_mma(Acc<T, WM, WN>& acc, const T* As, const T* Bs,
                                              int m0, int n0, int lane) {
  if constexpr (Elem<T>::MMA) {
    constexpr int MI = WM / 16, NI = WN / 8;
    static_assert(WM % 16 == 0 && WN % 16 == 0 && TK % 16 == 0, "mma tile shape");
    const int l7 = lane & 7, mi4 = lane >> 3;
#pragma unroll
    for (int k0 = 0; k0 < TK; k0 += 16) {
      uint32_t a[MI][4];
#pragma unroll
      for (int i = 0; i < MI; ++i) {
        const int mb = m0 + i * 16;
        if constexpr (AKC) {
          // matrices: (m+0,k+0) (m+8,k+0) (m+0,k+8) (m+8,k+8)
          ldsm_x4(a[i], smem_u32(As + (mb + (mi4 & 1) * 8 + l7) * PA + k0 + (mi4 >> 1) * 8));
        } else {
          // stored [k][m]: same four matrices, read transposed
          ldsm_x4_t(a[i], smem_u32(As + (k0 + (mi4 >> 1) * 8 + l7) * PA + mb + (mi4 & 1) * 8));
        }
      }
#pragma unroll
      for (int j = 0; j < NI; j += 2) {
        const int nb = n0 + j * 8;
        uint32_t b[4];
        if constexpr (BKC) {
          // stored [n][k]; matrices: (n+0,k+0) (n+0,k+8) (n+8,k+0) (n+8,k+8)
          ldsm_x4(b, smem_u32(Bs + (nb + (mi4 >> 1) * 8 + l7) * PB + k0 + (mi4 & 1) * 8));
        } else {
          // stored [k][n]; same four matrices, read transposed
          ldsm_x4_t(b, smem_u32(Bs + (k0 + (mi4 & 1) * 8 + l7) * PB + nb + (mi4 >> 1) * 8));
        }
#pragma unroll
        for (int i = 0; i < MI; ++i) {
          mma16816<T>(*reinterpret_cast<float(*)[4]>(&acc.v[(i * NI + j) * 4]), a[i], b[0], b[1]);
          mma16816<T>(*reinterpret_cast<float(*)[4]>(&acc.v[(i * NI + j + 1) * 4]), a[i], b[2], b[3]);
        }
      }
    }
  } else {
    // FP32: lane (ty, tx) = (lane / 4, lane % 4) owns rows ty + 8i and cols tx + 4j.
    constexpr int RI = WM / 8, CJ = WN / 4;
    const int ty = lane >> 2, tx = lane & 3;
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float av[RI], bv[CJ];
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        const int m = m0 + ty + 8 * i;
        av[i] = AKC ? As[m * PA + k] : As[k * PA + m];
      }
#pragma unroll
      for (int j = 0; j < CJ; ++j) {
        const int n = n0 + tx + 4 * j;
        bv[j] = BKC ? Bs[n * PB + k] : Bs[k * PB + n];
      }
#pragma unroll
      for (int i = 0; i < RI; ++i)
#pragma unroll
        for (int j = 0; j < CJ; ++j) acc.v[i * CJ + j] = fmaf(av[i], bv[j], acc.v[i * CJ + j]);
    }
  }
}

// Calls f(row, col, value) for every accumulator element of the warp tile
// (row / col relative to the warp tile origin).
template <typename T, int WM, int WN, typename F>
__device__ __forceinline__ void for_each_acc(const Acc<T, WM, WN>& acc, int lane, F&& f) {
  if constexpr (Elem<T>::MMA) {
    constexpr int MI = WM / 16, NI = WN / 8;
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r)
          f(i * 16 + g + 8 * (r >> 1), j * 8 + 2 * t + (r & 1), acc.v[(i * NI + j) * 4 + r]);
  } else {
    constexpr int RI = WM / 8, CJ = WN / 4;
    const int ty = lane >> 2, tx = lane & 3;
#pragma unroll
    for (int i = 0; i < RI; ++i)
#pragma unroll
      for (int j = 0; j < CJ; ++j) f(ty + 8 * i, tx + 4 * j, acc.v[i * CJ + j]);
  }
}

}  // namespace bsp
