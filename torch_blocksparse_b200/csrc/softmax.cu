// Block-sparse row softmax, forward and backward, for sm_100a.
//
// Replaces softmax_fwd / softmax_bwd of the reference
// (torch_blocksparse/softmax.py:7-138, 144-194) and their launch code
// (softmax.py:253-326).
//
// A row of block-row (h, i) is made of `size` chunks of `block` contiguous
// elements, one per nonzero block, read with 16-byte vector loads.  Three
// work decompositions, picked by the longest row of the layout:
//   * up to 8 blocks per row: a group of block/VEC lanes per row (see
//     softmax_fwd_group), several rows per warp;
//   * longer rows: one warp per row with the row held in registers (NV vectors
//     per lane, compile-time), consecutive warps on consecutive rows;
//   * rows beyond the largest NV: one warp per row, two sweeps, x re-read.
// In the first two x is read once and written once.
// The kernel is pure streaming: its roofline is HBM bandwidth.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "common.h"

namespace bsp {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr float kNegInf = -__builtin_huge_valf();

template <typename T> struct Vec;   // 16 bytes of T
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte load of Vec<T>::N elements, converted to float.
template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[Vec<T>::N]) {
  constexpr int N = Vec<T>::N;
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = to_f(e[i]);
}

// Streaming variant for data that is read exactly once (x, dy).
template <typename T>
__device__ __forceinline__ void load_vec_stream(const T* p, float (&f)[Vec<T>::N]) {
  constexpr int N = Vec<T>::N;
  uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = to_f(e[i]);
}

template <typename T>
__device__ __forceinline__ void load_scalar(const T* p, float (&f)[Vec<T>::N]) {
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) f[i] = to_f(p[i]);
}

template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[Vec<T>::N]) {
  constexpr int N = Vec<T>::N;
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = from_f<T>(f[i]);
  __stcs(reinterpret_cast<uint4*>(p), raw);
}

// Two 16-bit values of one 32-bit word <-> a pair of floats.
template <typename T> __device__ __forceinline__ float2 word_to_f2(uint32_t w);
template <> __device__ __forceinline__ float2 word_to_f2<__half>(uint32_t w) { return __half22float2(*reinterpret_cast<__half2*>(&w)); }
template <> __device__ __forceinline__ float2 word_to_f2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 word_to_f2<float>(uint32_t w) { return make_float2(__uint_as_float(w), 0.f); }
template <typename T> __device__ __forceinline__ uint32_t f2_to_word(float2 v);
template <> __device__ __forceinline__ uint32_t f2_to_word<__half>(float2 v) {
  __half2 h = __floats2half2_rn(v.x, v.y);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t f2_to_word<__nv_bfloat16>(float2 v) {
  __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t f2_to_word<float>(float2 v) { return __float_as_uint(v.x); }
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// 2^x on the special-function unit (ex2.approx: about 2 ulp, denormals flushed).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct FwdArgs {
  void* x; int64_t x_sz;
  const int32_t* lut;
  int rows;            // H * Mb * block
  int block_log2;
  float scale;
  const void* rpe; int64_t rpe_sz, rpe_sh, rpe_sr;
  const void* kpm; int64_t kpm_sz; int kpm_mul;
  const void* am; int64_t am_sr; int am_mul;
  int mask_vec;        // masks may be read with 16-byte loads
};

// Computes the pre-softmax values of one vector slot: x*scale + rpe + kpm + am.
template <typename T>
__device__ __forceinline__ void fwd_slot(const FwdArgs& a, const T* xrow, int z, int rxm, const int32_t* ent,
                                         int c, int block_log2, float (&f)[Vec<T>::N]) {
  constexpr int N = Vec<T>::N;
  const int blockid = ent[0], col = ent[1], row = ent[2], head = ent[3];
  load_vec_stream(xrow + ((int64_t)blockid << (2 * block_log2)) + c, f);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] *= a.scale;
  const int64_t gcol = ((int64_t)col << block_log2) + c;
  const int64_t grow = ((int64_t)row << block_log2) + rxm;
  if (a.rpe) {
    float r[N];
    const T* p = reinterpret_cast<const T*>(a.rpe) + z * a.rpe_sz + head * a.rpe_sh + grow * a.rpe_sr + gcol;
    if (a.mask_vec) load_vec(p, r); else load_scalar(p, r);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] += r[i];
  }
  if (a.kpm) {
    float r[N];
    const T* p = reinterpret_cast<const T*>(a.kpm) + z * a.kpm_sz + gcol;
    if (a.mask_vec) load_vec(p, r); else load_scalar(p, r);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] += a.kpm_mul ? (r[i] == 0.f ? kNegInf : 0.f) : r[i];
  }
  if (a.am) {
    float r[N];
    const T* p = reinterpret_cast<const T*>(a.am) + grow * a.am_sr + gcol;
    if (a.mask_vec) load_vec(p, r); else load_scalar(p, r);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] += a.am_mul ? (r[i] == 0.f ? kNegInf : 0.f) : r[i];
  }
}

// Rows of up to 32 * NV vectors, held in registers.
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32) softmax_fwd_reg(FwdArgs a) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int z = blockIdx.y;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int size = a.lut[2 * rbm], offset = a.lut[2 * rbm + 1];
  if (size == 0) return;
  const int nvec = size << (bl - (N == 8 ? 3 : 2));   // vectors in this row
  T* xrow = reinterpret_cast<T*>(a.x) + z * a.x_sz + ((int64_t)rxm << bl);
  float f[NV][N];
  float m = kNegInf;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int s = lane + 32 * k;
    if (s < nvec) {
      const int e = s * N;
      fwd_slot<T>(a, xrow, z, rxm, a.lut + offset + 4 * (e >> bl), e & ((1 << bl) - 1), bl, f[k]);
#pragma unroll
      for (int i = 0; i < N; ++i) m = fmaxf(m, f[k][i]);
    }
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    if (lane + 32 * k < nvec) {
#pragma unroll
      for (int i = 0; i < N; ++i) { f[k][i] = __expf(f[k][i] - m); sum += f[k][i]; }
    }
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int s = lane + 32 * k;
    if (s < nvec) {
      const int e = s * N;
      const int blockid = a.lut[offset + 4 * (e >> bl)];
#pragma unroll
      for (int i = 0; i < N; ++i) f[k][i] *= inv;
      store_vec(xrow + ((int64_t)blockid << (2 * bl)) + (e & ((1 << bl) - 1)), f[k]);
    }
  }
}

// Rows of any length: one sweep for max and sum (rescaled on the fly), one to
// recompute and store.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32) softmax_fwd_loop(FwdArgs a) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int z = blockIdx.y;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int size = a.lut[2 * rbm], offset = a.lut[2 * rbm + 1];
  if (size == 0) return;
  const int nvec = size << (bl - (N == 8 ? 3 : 2));
  T* xrow = reinterpret_cast<T*>(a.x) + z * a.x_sz + ((int64_t)rxm << bl);
  float m = kNegInf, sum = 0.f;
  for (int s = lane; s < nvec; s += 32) {
    float f[N];
    const int e = s * N;
    fwd_slot<T>(a, xrow, z, rxm, a.lut + offset + 4 * (e >> bl), e & ((1 << bl) - 1), bl, f);
    float vm = f[0];
#pragma unroll
    for (int i = 1; i < N; ++i) vm = fmaxf(vm, f[i]);
    const float nm = fmaxf(m, vm);
    if (nm != kNegInf) {
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) part += __expf(f[i] - nm);
      sum = sum * __expf(m - nm) + part;
      m = nm;
    }
  }
  const float gm = warp_max(m);
  sum = (m == kNegInf) ? 0.f : sum * __expf(m - gm);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int s = lane; s < nvec; s += 32) {
    float f[N];
    const int e = s * N;
    const int32_t* ent = a.lut + offset + 4 * (e >> bl);
    fwd_slot<T>(a, xrow, z, rxm, ent, e & ((1 << bl) - 1), bl, f);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = __expf(f[i] - gm) * inv;
    store_vec(xrow + ((int64_t)ent[0] << (2 * bl)) + (e & ((1 << bl) - 1)), f);
  }
}

struct BwdArgs {
  const void* y; void* dy; int64_t y_sz, dy_sz;
  const int32_t* lut;
  int rows;
  int block_log2;
  float scale;
};

template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32) softmax_bwd_reg(BwdArgs a) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int z = blockIdx.y;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int size = a.lut[2 * rbm], offset = a.lut[2 * rbm + 1];
  if (size == 0) return;
  const int nvec = size << (bl - (N == 8 ? 3 : 2));
  const T* yrow = reinterpret_cast<const T*>(a.y) + z * a.y_sz + ((int64_t)rxm << bl);
  T* drow = reinterpret_cast<T*>(a.dy) + z * a.dy_sz + ((int64_t)rxm << bl);
  float y[NV][N], d[NV][N];
  float dot = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int s = lane + 32 * k;
    if (s < nvec) {
      const int e = s * N;
      const int64_t off = ((int64_t)a.lut[offset + 4 * (e >> bl)] << (2 * bl)) + (e & ((1 << bl) - 1));
      load_vec_stream(yrow + off, y[k]);
      load_vec_stream(drow + off, d[k]);
#pragma unroll
      for (int i = 0; i < N; ++i) dot += y[k][i] * d[k][i];
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int s = lane + 32 * k;
    if (s < nvec) {
      const int e = s * N;
      const int64_t off = ((int64_t)a.lut[offset + 4 * (e >> bl)] << (2 * bl)) + (e & ((1 << bl) - 1));
#pragma unroll
      for (int i = 0; i < N; ++i) d[k][i] = y[k][i] * (d[k][i] - dot) * a.scale;
      store_vec(drow + off, d[k]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32) softmax_bwd_loop(BwdArgs a) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int z = blockIdx.y;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int size = a.lut[2 * rbm], offset = a.lut[2 * rbm + 1];
  if (size == 0) return;
  const int nvec = size << (bl - (N == 8 ? 3 : 2));
  const T* yrow = reinterpret_cast<const T*>(a.y) + z * a.y_sz + ((int64_t)rxm << bl);
  T* drow = reinterpret_cast<T*>(a.dy) + z * a.dy_sz + ((int64_t)rxm << bl);
  float dot = 0.f;
  for (int s = lane; s < nvec; s += 32) {
    float y[N], d[N];
    const int e = s * N;
    const int64_t off = ((int64_t)a.lut[offset + 4 * (e >> bl)] << (2 * bl)) + (e & ((1 << bl) - 1));
    load_vec(yrow + off, y);
    load_vec(drow + off, d);
#pragma unroll
    for (int i = 0; i < N; ++i) dot += y[i] * d[i];
  }
  dot = warp_sum(dot);
  for (int s = lane; s < nvec; s += 32) {
    float y[N], d[N];
    const int e = s * N;
    const int64_t off = ((int64_t)a.lut[offset + 4 * (e >> bl)] << (2 * bl)) + (e & ((1 << bl) - 1));
    load_vec(yrow + off, y);
    load_vec(drow + off, d);
#pragma unroll
    for (int i = 0; i < N; ++i) d[i] = y[i] * (d[i] - dot) * a.scale;
    store_vec(drow + off, d);
  }
}

// ---------------------------------------------------------------------------
// Short rows (at most 8 nonzero blocks): a group of block/VEC lanes owns one
// row and walks its chunks, so a warp covers 32/(block/VEC) consecutive rows
// of one block at full lane utilisation and reads 512 contiguous bytes per
// chunk.  The batch index is the fastest grid dimension: CTAs that run
// together read the same rpe / attention-mask rows, which then stay in L2.
// ---------------------------------------------------------------------------
constexpr int kGroupWarps = 4;     // warps per CTA of the short-row kernels

// CTAs per SM the short-row kernels are compiled for: the register budget grows
// with the number of vectors a thread keeps in flight.
constexpr int fwd_ctas(int nv) { return nv <= 1 ? 12 : nv <= 2 ? 10 : nv <= 4 ? 8 : nv <= 6 ? 6 : 5; }
constexpr int bwd_ctas(int nv) { return nv <= 1 ? 16 : nv <= 2 ? 12 : nv <= 4 ? 9 : nv <= 6 ? 8 : 6; }

// Raw 16-byte vectors are kept packed while they are in flight, so that the
// registers of a thread hold as many outstanding bytes as possible; they are
// expanded to FP32 only when consumed.
template <typename T>
__device__ __forceinline__ void expand(const uint4& raw, float (&f)[Vec<T>::N]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) f[i] = to_f(e[i]);
}

template <typename T>
__device__ __forceinline__ uint4 load_raw(const T* p, bool vec) {
  if (vec) return __ldg(reinterpret_cast<const uint4*>(p));
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) e[i] = p[i];
  return raw;
}

// The table lists the blocks of a block-row consecutively and numbers them in
// the same order (block id = position in the table), so the id of the k-th
// block of a row follows from the row's table offset: no per-block table read
// sits between the header load and the data loads.
__device__ __forceinline__ int first_block_of_row(int offset, int header_ints) { return (offset - header_ints) >> 2; }

// Compile-time description of the optional inputs of the forward, so that no
// per-element work depends on a run-time flag: RPE present or not; key-padding
// and attention mask each absent (0), added (1) or in 'mul' mode (2); VEC says
// that every optional input may be read with 16-byte loads.
template <bool RPE_, int KPM_, int AM_, bool VEC_> struct FwdSpec {
  static constexpr bool RPE = RPE_, VEC = VEC_;
  static constexpr int KPM = KPM_, AM = AM_;
};

template <typename T, int NV, typename S>
__global__ void __launch_bounds__(kGroupWarps * 32, fwd_ctas(NV))
softmax_fwd_group(FwdArgs a, int Z, int lpr_log2, int header_ints) {
  constexpr int N = Vec<T>::N;
  constexpr float kLog2e = 1.4426950408889634f;
  const int lane = threadIdx.x & 31;
  const int z = blockIdx.x % Z;
  const int wg = blockIdx.x / Z * kGroupWarps + (threadIdx.x >> 5);
  const int row = (wg << (5 - lpr_log2)) + (lane >> lpr_log2);
  if (row >= a.rows) return;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int2 hdr = __ldg(reinterpret_cast<const int2*>(a.lut) + rbm);
  const int size = hdr.x, offset = hdr.y;
  if (size == 0) return;
  const int c = (lane & ((1 << lpr_log2) - 1)) * N;
  T* xp = reinterpret_cast<T*>(a.x) + z * a.x_sz + ((int64_t)first_block_of_row(offset, header_ints) << (2 * bl)) +
          ((int64_t)rxm << bl) + c;
  uint4 xr[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (k < size) xr[k] = __ldcs(reinterpret_cast<const uint4*>(xp + ((int64_t)k << (2 * bl))));
  float f[NV][N];
  float m = kNegInf;
  if constexpr (S::RPE || S::KPM != 0 || S::AM != 0) {
    // row and head are the same for all blocks of this block-row
    const int64_t grow = ((int64_t)__ldg(a.lut + offset + 2) << bl) + rxm;
    const T* rpe = nullptr;
    if constexpr (S::RPE)
      rpe = reinterpret_cast<const T*>(a.rpe) + z * a.rpe_sz + __ldg(a.lut + offset + 3) * a.rpe_sh + grow * a.rpe_sr + c;
    const T* kpm = reinterpret_cast<const T*>(a.kpm) + z * a.kpm_sz + c;
    const T* am = reinterpret_cast<const T*>(a.am) + grow * a.am_sr + c;
    int col[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k)
      if (k < size) col[k] = __ldg(a.lut + offset + 4 * k + 1) << bl;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (k < size) {
        expand<T>(xr[k], f[k]);
        float r[N];
        if constexpr (S::RPE) {
          expand<T>(load_raw(rpe + col[k], S::VEC), r);
#pragma unroll
          for (int i = 0; i < N; ++i) f[k][i] = fmaf(f[k][i], a.scale, r[i]);
        } else {
#pragma unroll
          for (int i = 0; i < N; ++i) f[k][i] *= a.scale;
        }
        if constexpr (S::KPM != 0) {
          expand<T>(load_raw(kpm + col[k], S::VEC), r);
#pragma unroll
          for (int i = 0; i < N; ++i) f[k][i] = S::KPM == 2 ? (r[i] == 0.f ? kNegInf : f[k][i]) : f[k][i] + r[i];
        }
        if constexpr (S::AM != 0) {
          expand<T>(load_raw(am + col[k], S::VEC), r);
#pragma unroll
          for (int i = 0; i < N; ++i) f[k][i] = S::AM == 2 ? (r[i] == 0.f ? kNegInf : f[k][i]) : f[k][i] + r[i];
        }
#pragma unroll
        for (int i = 0; i < N; ++i) m = fmaxf(m, f[k][i]);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (k < size) {
        expand<T>(xr[k], f[k]);
#pragma unroll
        for (int i = 0; i < N; ++i) { f[k][i] *= a.scale; m = fmaxf(m, f[k][i]); }
      }
    }
  }
  for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  // exp(f - m) = 2^(f*log2(e) - m*log2(e)); a row that is masked everywhere has
  // m = -inf and yields NaN, as the reference's kernel does
  const float ml2 = m * kLog2e;
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    if (k < size) {
#pragma unroll
      for (int i = 0; i < N; ++i) { f[k][i] = fast_exp2(fmaf(f[k][i], kLog2e, -ml2)); sum += f[k][i]; }
    }
  }
  for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    if (k < size) {
#pragma unroll
      for (int i = 0; i < N; ++i) f[k][i] *= inv;
      store_vec(xp + ((int64_t)k << (2 * bl)), f[k]);
    }
  }
}

// Same row decomposition, but the batch is walked inside the kernel: whatever
// does not depend on the batch entry (the attention mask, an rpe that is
// broadcast over the batch, the table look-ups) is read and converted once and
// kept in registers as one term per element, and the x vectors of the next two
// batch entries are in flight while the current one is reduced.
template <typename T, int NV, typename S>
// (measured: four CTAs per SM spill and take 198 us instead of 146; x of one batch entry in
// flight instead of two 157 us)
__global__ void __launch_bounds__(kGroupWarps * 32, 3)
softmax_fwd_zloop(FwdArgs a, int Z, int lpr_log2, int header_ints) {
  constexpr int N = Vec<T>::N;
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr bool TERM = S::RPE || S::AM != 0;
  const int lane = threadIdx.x & 31;
  const int wg = blockIdx.x * kGroupWarps + (threadIdx.x >> 5);
  const int row = (wg << (5 - lpr_log2)) + (lane >> lpr_log2);
  if (row >= a.rows) return;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int2 hdr = __ldg(reinterpret_cast<const int2*>(a.lut) + rbm);
  const int size = hdr.x, offset = hdr.y;
  if (size == 0) return;
  const int c = (lane & ((1 << lpr_log2) - 1)) * N;
  T* xp = reinterpret_cast<T*>(a.x) + ((int64_t)first_block_of_row(offset, header_ints) << (2 * bl)) + ((int64_t)rxm << bl) + c;
  // Loads are issued in the order of their dependences and none is consumed before all
  // independent ones are in flight: table entries of the row, then x of the first two batch
  // entries, then the optional inputs.
  int ck[NV];
  int hb[2] = {0, 0};
  if constexpr (TERM || S::KPM != 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k)
      if (k < size) ck[k] = __ldg(a.lut + offset + 4 * k + 1);
    if constexpr (TERM) { hb[0] = __ldg(a.lut + offset + 2); hb[1] = __ldg(a.lut + offset + 3); }
  }
  uint4 cur[NV], nxt[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (k < size) cur[k] = __ldcs(reinterpret_cast<const uint4*>(xp + ((int64_t)k << (2 * bl))));
  if (Z > 1) {
#pragma unroll
    for (int k = 0; k < NV; ++k)
      if (k < size) nxt[k] = __ldcs(reinterpret_cast<const uint4*>(xp + a.x_sz + ((int64_t)k << (2 * bl))));
  }
  int col[S::KPM != 0 ? NV : 1];
  // The batch-independent term stays in registers.  It is kept in the storage type, which
  // is exact, unless rpe and an additive attention mask are both present: their sum is an
  // FP32 value.  (A 'mul' mask only turns elements of the term into -inf.)
  constexpr bool PACKED = TERM && !(S::RPE && S::AM == 1) && N == 8;
  float term[TERM && !PACKED ? NV : 1][N];
  uint4 pterm[PACKED ? NV : 1];
  const T* kpm = reinterpret_cast<const T*>(a.kpm) + c;
  uint4 kcur[S::KPM != 0 ? NV : 1];
  if constexpr (TERM || S::KPM != 0) {
    const int64_t grow = ((int64_t)hb[0] << bl) + rxm;
    const T* rpe = nullptr;
    if constexpr (S::RPE) rpe = reinterpret_cast<const T*>(a.rpe) + hb[1] * a.rpe_sh + grow * a.rpe_sr + c;
    const T* am = reinterpret_cast<const T*>(a.am) + grow * a.am_sr + c;
    uint4 rraw[S::RPE ? NV : 1], mraw[S::AM != 0 ? NV : 1];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (k < size) {
        const int cc = ck[k] << bl;
        if constexpr (S::KPM != 0) { col[k] = cc; kcur[k] = load_raw(kpm + cc, true); }
        if constexpr (S::RPE) rraw[k] = load_raw(rpe + cc, true);
        if constexpr (S::AM != 0) mraw[k] = load_raw(am + cc, true);
      }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (k < size) {
        if constexpr (PACKED) {
          if constexpr (S::RPE) {
            pterm[k] = rraw[k];
            if constexpr (S::AM == 2) {
              const T* me = reinterpret_cast<const T*>(&mraw[k]);
              T* te = reinterpret_cast<T*>(&pterm[k]);
#pragma unroll
              for (int i = 0; i < N; ++i) if (to_f(me[i]) == 0.f) te[i] = from_f<T>(kNegInf);
            }
          } else {                                           // the attention mask alone
            pterm[k] = mraw[k];
            if constexpr (S::AM == 2) {
              T* te = reinterpret_cast<T*>(&pterm[k]);
#pragma unroll
              for (int i = 0; i < N; ++i) te[i] = from_f<T>(to_f(te[i]) == 0.f ? kNegInf : 0.f);
            }
          }
        } else if constexpr (TERM) {
          float r[N];
#pragma unroll
          for (int i = 0; i < N; ++i) term[k][i] = 0.f;
          if constexpr (S::RPE) {
            expand<T>(rraw[k], r);
#pragma unroll
            for (int i = 0; i < N; ++i) term[k][i] = r[i];
          }
          if constexpr (S::AM != 0) {
            expand<T>(mraw[k], r);
#pragma unroll
            for (int i = 0; i < N; ++i) term[k][i] = S::AM == 2 ? (r[i] == 0.f ? kNegInf : term[k][i]) : term[k][i] + r[i];
          }
        }
      }
    }
  }
  // x of the next two batch entries is in flight while this one is reduced
  for (int z = 0; z < Z; ++z) {
    uint4 nx2[NV];
    if (z + 2 < Z) {
#pragma unroll
      for (int k = 0; k < NV; ++k)
        if (k < size) nx2[k] = __ldcs(reinterpret_cast<const uint4*>(xp + 2 * a.x_sz + ((int64_t)k << (2 * bl))));
    }
    if constexpr (N == 8) {
      // 16-bit storage: two elements per instruction through the packed FP32 operations of
      // sm_100 (multiply-add, add, multiply) and three-input maxima; per pair of elements
      // about fifteen instructions, most of them the conversions from and to 16 bits.
      float2 f[NV][4];
      float m0 = kNegInf, m1 = kNegInf;
      const float2 sc2 = make_float2(a.scale, a.scale);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (k < size) {
          const uint32_t* xw = reinterpret_cast<const uint32_t*>(&cur[k]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 v = word_to_f2<T>(xw[i]);
            if constexpr (PACKED) v = __ffma2_rn(v, sc2, word_to_f2<T>(reinterpret_cast<const uint32_t*>(&pterm[k])[i]));
            else if constexpr (TERM) v = __ffma2_rn(v, sc2, make_float2(term[k][2 * i], term[k][2 * i + 1]));
            else v = __fmul2_rn(v, sc2);
            if constexpr (S::KPM != 0) {
              const float2 r = word_to_f2<T>(reinterpret_cast<const uint32_t*>(&kcur[k])[i]);
              if constexpr (S::KPM == 2) { v.x = r.x == 0.f ? kNegInf : v.x; v.y = r.y == 0.f ? kNegInf : v.y; }
              else v = __fadd2_rn(v, r);
            }
            f[k][i] = v;
            if (i & 1) m1 = max3f(m1, v.x, v.y); else m0 = max3f(m0, v.x, v.y);
          }
        }
      }
      float m = fmaxf(m0, m1);
      kpm += a.kpm_sz;
      if constexpr (S::KPM != 0) {
        if (z + 1 < Z) {
#pragma unroll
          for (int k = 0; k < NV; ++k)
            if (k < size) kcur[k] = load_raw(kpm + col[k], true);
        }
      }
      for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float ml2 = m * kLog2e;
      const float2 l2 = make_float2(kLog2e, kLog2e), nm2 = make_float2(-ml2, -ml2);
      float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (k < size) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 y = __ffma2_rn(f[k][i], l2, nm2);
            f[k][i] = make_float2(fast_exp2(y.x), fast_exp2(y.y));
            s2 = __fadd2_rn(s2, f[k][i]);
          }
        }
      }
      float sum = s2.x + s2.y;
      for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float inv = 1.f / sum;
      const float2 inv2 = make_float2(inv, inv);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (k < size) {
          uint4 o;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int i = 0; i < 4; ++i) ow[i] = f2_to_word<T>(__fmul2_rn(f[k][i], inv2));
          __stcs(reinterpret_cast<uint4*>(xp + ((int64_t)k << (2 * bl))), o);
        }
      }
    } else {
      float f[NV][N];
      float m = kNegInf;
  #pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (k < size) {
          expand<T>(cur[k], f[k]);
          if constexpr (PACKED) {
            float r[N];
            expand<T>(pterm[k], r);
  #pragma unroll
            for (int i = 0; i < N; ++i) f[k][i] = fmaf(f[k][i], a.scale, r[i]);
          } else if constexpr (TERM) {
  #pragma unroll
            for (int i = 0; i < N; ++i) f[k][i] = fmaf(f[k][i], a.scale, term[k][i]);
          } else {
  #pragma unroll
            for (int i = 0; i < N; ++i) f[k][i] *= a.scale;
          }
          if constexpr (S::KPM != 0) {
            float r[N];
            expand<T>(kcur[k], r);
  #pragma unroll
            for (int i = 0; i < N; ++i) f[k][i] = S::KPM == 2 ? (r[i] == 0.f ? kNegInf : f[k][i]) : f[k][i] + r[i];
          }
  #pragma unroll
          for (int i = 0; i < N; ++i) m = fmaxf(m, f[k][i]);
        }
      }
      // the key-padding vectors of the next batch entry take over the registers of
      // the current ones as soon as those are consumed
      kpm += a.kpm_sz;
      if constexpr (S::KPM != 0) {
        if (z + 1 < Z) {
  #pragma unroll
          for (int k = 0; k < NV; ++k)
            if (k < size) kcur[k] = load_raw(kpm + col[k], true);
        }
      }
      for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float ml2 = m * kLog2e;
      float sum = 0.f;
  #pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (k < size) {
  #pragma unroll
          for (int i = 0; i < N; ++i) { f[k][i] = fast_exp2(fmaf(f[k][i], kLog2e, -ml2)); sum += f[k][i]; }
        }
      }
      for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float inv = 1.f / sum;
  #pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (k < size) {
  #pragma unroll
          for (int i = 0; i < N; ++i) f[k][i] *= inv;
          store_vec(xp + ((int64_t)k << (2 * bl)), f[k]);
        }
      }
    }
    xp += a.x_sz;
#pragma unroll
    for (int k = 0; k < NV; ++k) { cur[k] = nxt[k]; nxt[k] = nx2[k]; }
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(kGroupWarps * 32, bwd_ctas(NV))
softmax_bwd_group(BwdArgs a, int Z, int lpr_log2, int header_ints) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int z = blockIdx.x % Z;
  const int wg = blockIdx.x / Z * kGroupWarps + (threadIdx.x >> 5);
  const int row = (wg << (5 - lpr_log2)) + (lane >> lpr_log2);
  if (row >= a.rows) return;
  const int bl = a.block_log2;
  const int rbm = row >> bl, rxm = row & ((1 << bl) - 1);
  const int2 hdr = __ldg(reinterpret_cast<const int2*>(a.lut) + rbm);
  const int size = hdr.x;
  if (size == 0) return;
  const int64_t off = ((int64_t)first_block_of_row(hdr.y, header_ints) << (2 * bl)) + ((int64_t)rxm << bl) +
                      (lane & ((1 << lpr_log2) - 1)) * N;
  const T* yp = reinterpret_cast<const T*>(a.y) + z * a.y_sz + off;
  T* dp = reinterpret_cast<T*>(a.dy) + z * a.dy_sz + off;
  uint4 yr[NV], dr[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (k < size) {
      yr[k] = __ldcs(reinterpret_cast<const uint4*>(yp + ((int64_t)k << (2 * bl))));
      dr[k] = __ldcs(reinterpret_cast<const uint4*>(dp + ((int64_t)k << (2 * bl))));
    }
  float dot = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (k < size) {
      float y[N], d[N];
      expand<T>(yr[k], y);
      expand<T>(dr[k], d);
#pragma unroll
      for (int i = 0; i < N; ++i) dot += y[i] * d[i];
    }
  for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (k < size) {
      float y[N], d[N];
      expand<T>(yr[k], y);
      expand<T>(dr[k], d);
#pragma unroll
      for (int i = 0; i < N; ++i) d[i] = y[i] * (d[i] - dot) * a.scale;
      store_vec(dp + ((int64_t)k << (2 * bl)), d);
    }
}

constexpr int kGroupMaxBlocks = 8;

template <typename T, typename S>
void launch_fwd_group(const FwdArgs& a, int maxlut, int Z, int block, int header_ints, cudaStream_t st) {
  int lpr_log2 = 0;
  while ((Vec<T>::N << lpr_log2) < block) ++lpr_log2;
  const int rows_per_cta = kGroupWarps << (5 - lpr_log2);
  if (S::RPE && Z >= 4 && a.rpe_sz == 0 && maxlut > 1) {
    const unsigned grid = (unsigned)((a.rows + rows_per_cta - 1) / rows_per_cta);
    if (maxlut <= 2) softmax_fwd_zloop<T, 2, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
    else if (maxlut <= 4) softmax_fwd_zloop<T, 4, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
    else if (maxlut <= 5) softmax_fwd_zloop<T, 5, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
    else if (maxlut <= 6) softmax_fwd_zloop<T, 6, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
    else softmax_fwd_zloop<T, 8, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
    return;
  }
  const unsigned grid = (unsigned)((a.rows + rows_per_cta - 1) / rows_per_cta) * Z;
  if (maxlut <= 1) softmax_fwd_group<T, 1, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else if (maxlut <= 2) softmax_fwd_group<T, 2, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else if (maxlut <= 4) softmax_fwd_group<T, 4, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else if (maxlut <= 6) softmax_fwd_group<T, 6, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else softmax_fwd_group<T, 8, S><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
}

// Maps the run-time description of the optional inputs onto a FwdSpec.
template <typename T, bool RPE, int KPM>
void pick_am(const FwdArgs& a, int maxlut, int Z, int block, int header_ints, cudaStream_t st) {
  const int am = a.am ? (a.am_mul ? 2 : 1) : 0;
  if (am == 0) launch_fwd_group<T, FwdSpec<RPE, KPM, 0, true>>(a, maxlut, Z, block, header_ints, st);
  else if (am == 1) launch_fwd_group<T, FwdSpec<RPE, KPM, 1, true>>(a, maxlut, Z, block, header_ints, st);
  else launch_fwd_group<T, FwdSpec<RPE, KPM, 2, true>>(a, maxlut, Z, block, header_ints, st);
}
template <typename T>
void dispatch_fwd_group(const FwdArgs& a, int maxlut, int Z, int block, int header_ints, cudaStream_t st) {
  const int kpm = a.kpm ? (a.kpm_mul ? 2 : 1) : 0;
  if (a.rpe) {
    if (kpm == 0) pick_am<T, true, 0>(a, maxlut, Z, block, header_ints, st);
    else if (kpm == 1) pick_am<T, true, 1>(a, maxlut, Z, block, header_ints, st);
    else pick_am<T, true, 2>(a, maxlut, Z, block, header_ints, st);
  } else {
    if (kpm == 0) pick_am<T, false, 0>(a, maxlut, Z, block, header_ints, st);
    else if (kpm == 1) pick_am<T, false, 1>(a, maxlut, Z, block, header_ints, st);
    else pick_am<T, false, 2>(a, maxlut, Z, block, header_ints, st);
  }
}
template <typename T>
void dispatch_bwd_group(const BwdArgs& a, int maxlut, int Z, int block, int header_ints, cudaStream_t st) {
  int lpr_log2 = 0;
  while ((Vec<T>::N << lpr_log2) < block) ++lpr_log2;
  const int rows_per_cta = kGroupWarps << (5 - lpr_log2);
  const unsigned grid = (unsigned)((a.rows + rows_per_cta - 1) / rows_per_cta) * Z;
  if (maxlut <= 1) softmax_bwd_group<T, 1><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else if (maxlut <= 2) softmax_bwd_group<T, 2><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else if (maxlut <= 4) softmax_bwd_group<T, 4><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else if (maxlut <= 6) softmax_bwd_group<T, 6><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
  else softmax_bwd_group<T, 8><<<grid, kGroupWarps * 32, 0, st>>>(a, Z, lpr_log2, header_ints);
}

inline int log2i(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, int NV>
void launch_fwd_reg(const FwdArgs& a, dim3 grid, cudaStream_t st) {
  softmax_fwd_reg<T, NV><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
}
template <typename T, int NV>
void launch_bwd_reg(const BwdArgs& a, dim3 grid, cudaStream_t st) {
  softmax_bwd_reg<T, NV><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
}

// Picks the smallest register variant that holds a row of `nvec` vectors.
template <typename T>
void dispatch_fwd(const FwdArgs& a, int nvec, dim3 grid, cudaStream_t st) {
  const int need = (nvec + 31) / 32;
  if (need <= 1) launch_fwd_reg<T, 1>(a, grid, st);
  else if (need <= 2) launch_fwd_reg<T, 2>(a, grid, st);
  else if (need <= 3) launch_fwd_reg<T, 3>(a, grid, st);
  else if (need <= 4) launch_fwd_reg<T, 4>(a, grid, st);
  else if (need <= 6) launch_fwd_reg<T, 6>(a, grid, st);
  else if (need <= 9) launch_fwd_reg<T, 9>(a, grid, st);
  else if (need <= 12) launch_fwd_reg<T, 12>(a, grid, st);
  else if (need <= 16) launch_fwd_reg<T, 16>(a, grid, st);
  else softmax_fwd_loop<T><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
}
template <typename T>
void dispatch_bwd(const BwdArgs& a, int nvec, dim3 grid, cudaStream_t st) {
  const int need = (nvec + 31) / 32;
  if (need <= 1) launch_bwd_reg<T, 1>(a, grid, st);
  else if (need <= 2) launch_bwd_reg<T, 2>(a, grid, st);
  else if (need <= 3) launch_bwd_reg<T, 3>(a, grid, st);
  else if (need <= 4) launch_bwd_reg<T, 4>(a, grid, st);
  else if (need <= 6) launch_bwd_reg<T, 6>(a, grid, st);
  else if (need <= 8) launch_bwd_reg<T, 8>(a, grid, st);
  else softmax_bwd_loop<T><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
}

int check_common(int dtype, int Z, int block, int H, int Mb, const int32_t* lut, int maxlut) {
  if (!valid_dtype(dtype)) return fail(BSP_ERR_INVALID, "unknown dtype %d", dtype);
  if (!valid_block(block)) return fail(BSP_ERR_INVALID, "block must be 16, 32, 64 or 128 (got %d)", block);
  if (Z <= 0 || H <= 0 || Mb <= 0 || maxlut < 0) return fail(BSP_ERR_INVALID, "non-positive size");
  if (Z > 65535) return fail(BSP_ERR_UNSUPPORTED, "batch %d exceeds the grid limit 65535", Z);
  if (!lut) return fail(BSP_ERR_INVALID, "lut is NULL");
  if ((int64_t)maxlut * block >= 32768)
    return fail(BSP_ERR_UNSUPPORTED, "Reductions larger than 32768 elements are not yet implemented");
  return BSP_OK;
}

int finish(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return BSP_OK;
}

}  // namespace
}  // namespace bsp

using namespace bsp;

extern "C" int bsp_softmax_fwd(void* x, int dtype, int Z, int64_t x_sz, int block,
                               int H, int Mb, const int32_t* lut, int maxlut, float scale,
                               const void* rpe, int64_t rpe_sz, int64_t rpe_sh, int64_t rpe_sr,
                               const void* kpm, int64_t kpm_sz, int kpm_mul,
                               const void* am, int64_t am_sr, int am_mul, void* stream) {
  if (int rc = check_common(dtype, Z, block, H, Mb, lut, maxlut)) return rc;
  if (!x) return fail(BSP_ERR_INVALID, "x is NULL");
  if (!aligned16(x)) return fail(BSP_ERR_INVALID, "x must be 16-byte aligned");
  if (maxlut == 0) return BSP_OK;
  const int vec = dtype == BSP_F32 ? 4 : 8;
  if (x_sz % vec) return fail(BSP_ERR_INVALID, "batch stride of x must be a multiple of %d elements", vec);
  FwdArgs a;
  a.x = x; a.x_sz = x_sz; a.lut = lut; a.rows = H * Mb * block; a.block_log2 = log2i(block); a.scale = scale;
  a.rpe = rpe; a.rpe_sz = rpe_sz; a.rpe_sh = rpe_sh; a.rpe_sr = rpe_sr;
  a.kpm = kpm; a.kpm_sz = kpm_sz; a.kpm_mul = kpm_mul;
  a.am = am; a.am_sr = am_sr; a.am_mul = am_mul;
  bool mv = true;
  if (rpe) mv = mv && aligned16(rpe) && rpe_sz % vec == 0 && rpe_sh % vec == 0 && rpe_sr % vec == 0;
  if (kpm) mv = mv && aligned16(kpm) && kpm_sz % vec == 0;
  if (am) mv = mv && aligned16(am) && am_sr % vec == 0;
  a.mask_vec = mv ? 1 : 0;
  const dim3 grid((a.rows + kWarpsPerCta - 1) / kWarpsPerCta, Z);
  const int nvec = maxlut * block / vec;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (maxlut <= kGroupMaxBlocks && a.mask_vec) {
    if (dtype == BSP_F32) dispatch_fwd_group<float>(a, maxlut, Z, block, 2 * H * Mb, st);
    else if (dtype == BSP_F16) dispatch_fwd_group<__half>(a, maxlut, Z, block, 2 * H * Mb, st);
    else dispatch_fwd_group<__nv_bfloat16>(a, maxlut, Z, block, 2 * H * Mb, st);
  } else if (dtype == BSP_F32) dispatch_fwd<float>(a, nvec, grid, st);
  else if (dtype == BSP_F16) dispatch_fwd<__half>(a, nvec, grid, st);
  else dispatch_fwd<__nv_bfloat16>(a, nvec, grid, st);
  return finish("softmax forward");
}

extern "C" int bsp_softmax_bwd(const void* y, void* dy, int dtype, int Z, int64_t y_sz, int64_t dy_sz,
                               int block, int H, int Mb, const int32_t* lut, int maxlut, float scale,
                               void* stream) {
  if (int rc = check_common(dtype, Z, block, H, Mb, lut, maxlut)) return rc;
  if (!y || !dy) return fail(BSP_ERR_INVALID, "y or dy is NULL");
  if (!aligned16(y) || !aligned16(dy)) return fail(BSP_ERR_INVALID, "y and dy must be 16-byte aligned");
  if (maxlut == 0) return BSP_OK;
  const int vec = dtype == BSP_F32 ? 4 : 8;
  if (y_sz % vec || dy_sz % vec) return fail(BSP_ERR_INVALID, "batch strides must be multiples of %d elements", vec);
  BwdArgs a;
  a.y = y; a.dy = dy; a.y_sz = y_sz; a.dy_sz = dy_sz; a.lut = lut;
  a.rows = H * Mb * block; a.block_log2 = log2i(block); a.scale = scale;
  const dim3 grid((a.rows + kWarpsPerCta - 1) / kWarpsPerCta, Z);
  const int nvec = maxlut * block / vec;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (maxlut <= kGroupMaxBlocks) {
    if (dtype == BSP_F32) dispatch_bwd_group<float>(a, maxlut, Z, block, 2 * H * Mb, st);
    else if (dtype == BSP_F16) dispatch_bwd_group<__half>(a, maxlut, Z, block, 2 * H * Mb, st);
    else dispatch_bwd_group<__nv_bfloat16>(a, maxlut, Z, block, 2 * H * Mb, st);
  } else if (dtype == BSP_F32) dispatch_bwd<float>(a, nvec, grid, st);
  else if (dtype == BSP_F16) dispatch_bwd<__half>(a, nvec, grid, st);
  else dispatch_bwd<__nv_bfloat16>(a, nvec, grid, st);
  return finish("softmax backward");
}
