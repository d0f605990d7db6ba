// SDD: sparse = dense x dense, sampled on the layout (mma.sync / FFMA path).
//
// Replaces the SDD variant of the reference kernel and its launch code
// (torch_blocksparse/matmul.py:30-54, 128-175, 299-364).
//
// A CTA computes G nonzero blocks with consecutive block ids as G independent
// block x block products that share one K loop (G = 4 for block 16 and 32,
// 1 for 64 and 128).  Each product reads its own block-row of A and
// block-column of B (looked up per block id in the execution metadata, so
// there is no packing table and no duplicate work), staged through a
// three-stage cp.async pipeline.  Both operands are addressed through element
// strides, which is how trans_a / trans_b / trans_c of the reference reach
// this kernel; the shared-memory tile keeps the global orientation and the
// fragment loads transpose on the fly.
#pragma once
#include "common.h"
#include "tile.cuh"

namespace bsp {
namespace {

struct SddArgs {
  const void* a; const void* b; void* c;
  int64_t a_sz, a_sh, a_sm, a_sk;
  int64_t b_sz, b_sh, b_sk, b_sn;
  int64_t c_sz;
  int K, nnz;
  const int32_t* blk_row; const int32_t* blk_col; const int32_t* blk_head;
};

template <int B> struct SddShape;
template <> struct SddShape<16>  { static constexpr int WM = 16, WN = 16, NW = 4, G = 4; };
template <> struct SddShape<32>  { static constexpr int WM = 32, WN = 32, NW = 4, G = 4; };
template <> struct SddShape<64>  { static constexpr int WM = 32, WN = 32, NW = 4, G = 1; };
template <> struct SddShape<128> { static constexpr int WM = 64, WN = 32, NW = 8, G = 1; };

constexpr int kStages = 3;

template <typename T, int B, bool AKC, bool BKC>
struct SddSmem {
  static constexpr int VEC = Elem<T>::VEC;
  static constexpr int TK = Elem<T>::MMA ? (B >= 32 ? 32 : 16) : 16;
  static constexpr int PAD = VEC;                            // 16 bytes
  static constexpr int PA = (AKC ? TK : B) + PAD;
  static constexpr int PB = (BKC ? TK : B) + PAD;
  static constexpr int A_ELEMS = (AKC ? B : TK) * PA;        // one block product
  static constexpr int B_ELEMS = (BKC ? B : TK) * PB;
  static constexpr int G = SddShape<B>::G;
  static constexpr int STAGE = G * (A_ELEMS + B_ELEMS);
  static constexpr int BYTES = kStages * STAGE * int(sizeof(T));
};

template <typename T, int B, bool AKC, bool BKC>
__global__ void __launch_bounds__(SddShape<B>::NW * 32) sdd_kernel(SddArgs p) {
  using S = SddSmem<T, B, AKC, BKC>;
  using Sh = SddShape<B>;
  constexpr int TK = S::TK, G = S::G, NT = Sh::NW * 32;
  constexpr int WPB = Sh::NW / G;                 // warps per block product
  constexpr int WCOLS = B / Sh::WN;               // warp grid inside one product
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* smem = reinterpret_cast<T*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int z = blockIdx.y;
  const int bid0 = blockIdx.x * G;

  // operand bases of the G products
  __shared__ const T* a_base[G];
  __shared__ const T* b_base[G];
  if (tid < G) {
    const int bid = bid0 + tid;
    if (bid < p.nnz) {
      const int h = p.blk_head[bid];
      a_base[tid] = reinterpret_cast<const T*>(p.a) + z * p.a_sz + h * p.a_sh + (int64_t)p.blk_row[bid] * B * p.a_sm;
      b_base[tid] = reinterpret_cast<const T*>(p.b) + z * p.b_sz + h * p.b_sh + (int64_t)p.blk_col[bid] * B * p.b_sn;
    } else {
      a_base[tid] = reinterpret_cast<const T*>(p.a);
      b_base[tid] = reinterpret_cast<const T*>(p.b);
    }
  }
  __syncthreads();

  auto issue = [&](int chunk, int stage) {
    T* st = smem + stage * S::STAGE;
    const int k0 = chunk * TK;
    const int kk = min(TK, p.K - k0);            // the last chunk may be partial; the rest is zero-filled
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const bool ok = bid0 + g < p.nnz;
      T* as = st + g * (S::A_ELEMS + S::B_ELEMS);
      T* bs = as + S::A_ELEMS;
      if constexpr (AKC) load_tile<T, B, TK, S::PA, NT>(as, a_base[g] + k0, p.a_sm, tid, ok ? B : 0, kk);
      else               load_tile<T, TK, B, S::PA, NT>(as, a_base[g] + k0 * p.a_sk, p.a_sk, tid, ok ? kk : 0, B);
      if constexpr (BKC) load_tile<T, B, TK, S::PB, NT>(bs, b_base[g] + k0, p.b_sn, tid, ok ? B : 0, kk);
      else               load_tile<T, TK, B, S::PB, NT>(bs, b_base[g] + k0 * p.b_sk, p.b_sk, tid, ok ? kk : 0, B);
    }
  };

  const int g_w = warp / WPB;                      // product this warp works on
  const int wi = warp % WPB;
  const int m0 = (wi / WCOLS) * Sh::WM, n0 = (wi % WCOLS) * Sh::WN;
  Acc<T, Sh::WM, Sh::WN> acc;
  acc.clear();

  const int nchunks = (p.K + TK - 1) / TK;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < nchunks) issue(s, s);
    cp_async_commit();
  }
  for (int c = 0; c < nchunks; ++c) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    const int nx = c + kStages - 1;
    if (nx < nchunks) issue(nx, nx % kStages);
    cp_async_commit();
    const T* st = smem + (c % kStages) * S::STAGE + g_w * (S::A_ELEMS + S::B_ELEMS);
    warp_tile_mma<T, Sh::WM, Sh::WN, TK, AKC, BKC, S::PA, S::PB>(acc, st, st + S::A_ELEMS, m0, n0, lane);
  }
  cp_async_wait<0>();

  const int bid = bid0 + g_w;
  if (bid < p.nnz) {
    T* cb = reinterpret_cast<T*>(p.c) + z * p.c_sz + (int64_t)bid * B * B;
    for_each_acc<T, Sh::WM, Sh::WN>(acc, lane, [&](int r, int cidx, float v) {
      cb[(m0 + r) * B + n0 + cidx] = cvt_out<T>(v);
    });
  }
}

template <typename T, int B, bool AKC, bool BKC>
int launch(const SddArgs& p, int Z, cudaStream_t st) {
  using S = SddSmem<T, B, AKC, BKC>;
  auto kern = sdd_kernel<T, B, AKC, BKC>;
  if (S::BYTES > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::BYTES);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "sdd: cannot reserve %d bytes of shared memory: %s", S::BYTES, cudaGetErrorString(e));
  }
  const dim3 grid((p.nnz + S::G - 1) / S::G, Z);
  kern<<<grid, SddShape<B>::NW * 32, S::BYTES, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "sdd launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

template <typename T, int B>
int launch_layout(const SddArgs& p, int Z, cudaStream_t st) {
  const bool akc = p.a_sk == 1, bkc = p.b_sk == 1;
  if (akc && bkc) return launch<T, B, true, true>(p, Z, st);
  if (akc) return launch<T, B, true, false>(p, Z, st);
  if (bkc) return launch<T, B, false, true>(p, Z, st);
  return launch<T, B, false, false>(p, Z, st);
}

template <typename T>
int launch_block(const SddArgs& p, int block, int Z, cudaStream_t st) {
  switch (block) {
    case 16: return launch_layout<T, 16>(p, Z, st);
    case 32: return launch_layout<T, 32>(p, Z, st);
    case 64: return launch_layout<T, 64>(p, Z, st);
    default: return launch_layout<T, 128>(p, Z, st);
  }
}

}  // namespace

// One instance per element type (sdd_f32.cu, sdd_f16.cu, sdd_bf16.cu).
template <typename T>
int sdd_mma_t(const void* a, const void* b, void* c, int block, int Z, int K,
            int64_t a_sz, int64_t a_sh, int64_t a_sm, int64_t a_sk,
            int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
            int64_t c_sz, const Meta& m, cudaStream_t st) {
  SddArgs p;
  p.a = a; p.b = b; p.c = c;
  p.a_sz = a_sz; p.a_sh = a_sh; p.a_sm = a_sm; p.a_sk = a_sk;
  p.b_sz = b_sz; p.b_sh = b_sh; p.b_sk = b_sk; p.b_sn = b_sn;
  p.c_sz = c_sz; p.K = K; p.nnz = m.nnz;
  p.blk_row = m.blk_row; p.blk_col = m.blk_col; p.blk_head = m.blk_head;
  return launch_block<T>(p, block, Z, st);
}

}  // namespace bsp
