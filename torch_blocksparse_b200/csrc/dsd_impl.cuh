// DSD: dense = op(sparse) x dense (mma.sync / FFMA path).  DDS runs through the
// same kernel on the transposed problem (C^T = op(S)^T x A^T).
//
// Replaces the DSD / DDS variants of the reference kernel and their launch
// code (torch_blocksparse/matmul.py:57-99, 128-184, 460-552).
//
// A CTA owns one block-row of op(S) (a block-column of S when it is used
// transposed) and TN dense columns: it walks that row's nonzero blocks (CSR,
// or CSC for the transposed use) and accumulates block x TN products in
// registers, so every output element is produced by exactly one CTA in a fixed
// order -- no locks, no atomics, bitwise reproducible.  Rows without any
// nonzero block store zeros.  Block-rows are scheduled longest first.
#pragma once
#include "common.h"
#include "tile.cuh"

namespace bsp {
namespace {

struct DsdArgs {
  const void* s; const void* b; void* c;
  int64_t s_sz;
  int64_t b_sz, b_sh, b_sk, b_sn;
  int64_t c_sz, c_sh, c_sm, c_sn;
  int N;               // dense columns
  int outer;           // block-rows of op(S) per head
  int n_tiles;         // ceil(N / TN)
  const int32_t* ptr;  // CSR row_ptr or CSC col_ptr, indexed by head*outer + o
  const int32_t* kidx; // block index along K of every listed block
  const int32_t* bid;  // canonical block id of every listed block (NULL: the list position)
  const int32_t* order;// schedule: (head*outer + o) longest first
};

template <int B, int TN> struct DsdShape;
template <> struct DsdShape<16, 128>  { static constexpr int WM = 16, WN = 32; };
template <> struct DsdShape<32, 128>  { static constexpr int WM = 32, WN = 32; };
template <> struct DsdShape<64, 128>  { static constexpr int WM = 32, WN = 64; };
template <> struct DsdShape<128, 128> { static constexpr int WM = 64, WN = 32; };
template <> struct DsdShape<16, 64>   { static constexpr int WM = 16, WN = 16; };
template <> struct DsdShape<32, 64>   { static constexpr int WM = 32, WN = 16; };
template <> struct DsdShape<64, 64>   { static constexpr int WM = 32, WN = 32; };
template <> struct DsdShape<128, 64>  { static constexpr int WM = 64, WN = 32; };

constexpr int kDsdStages = 3;

template <typename T, int B, int TN, bool AKC, bool BKC>
struct DsdCfg {
  using Sh = DsdShape<B, TN>;
  static constexpr int NW = (B / Sh::WM) * (TN / Sh::WN);
  static constexpr int VEC = Elem<T>::VEC;
  static constexpr int TK = Elem<T>::MMA ? (B >= 32 ? 32 : 16) : 16;
  static constexpr int SUB = B / TK;                        // K chunks per block
  static constexpr int PAD = VEC;
  static constexpr int PA = (AKC ? TK : B) + PAD;
  static constexpr int PB = (BKC ? TK : TN) + PAD;
  static constexpr int A_ELEMS = (AKC ? B : TK) * PA;
  static constexpr int B_ELEMS = (BKC ? TN : TK) * PB;
  static constexpr int STAGE = A_ELEMS + B_ELEMS;
  static constexpr int BYTES = kDsdStages * STAGE * int(sizeof(T));
};

template <typename T, int B, int TN, bool AKC, bool BKC>
__global__ void __launch_bounds__(DsdCfg<T, B, TN, AKC, BKC>::NW * 32) dsd_kernel(DsdArgs p) {
  using C = DsdCfg<T, B, TN, AKC, BKC>;
  using Sh = typename C::Sh;
  constexpr int TK = C::TK, NT = C::NW * 32, SUB = C::SUB;
  constexpr int WCOLS = TN / Sh::WN;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* smem = reinterpret_cast<T*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int z = blockIdx.y;
  const int item = blockIdx.x / p.n_tiles, nt = blockIdx.x % p.n_tiles;
  const int ho = p.order[item];                  // head * outer + o
  const int h = ho / p.outer, o = ho % p.outer;
  const int first = p.ptr[ho], count = p.ptr[ho + 1] - first;
  const int n0g = nt * TN;
  const int n_ok = min(TN, p.N - n0g);

  const T* sblk = reinterpret_cast<const T*>(p.s) + z * p.s_sz;
  const T* bmat = reinterpret_cast<const T*>(p.b) + z * p.b_sz + h * p.b_sh + (int64_t)n0g * p.b_sn;

  auto issue = [&](int chunk, int stage) {
    T* as = smem + stage * C::STAGE;
    T* bs = as + C::A_ELEMS;
    const int pos = first + chunk / SUB, sub = chunk % SUB;
    const int kb = p.kidx[pos];
    const int id = p.bid ? p.bid[pos] : pos;
    const T* blk = sblk + (int64_t)id * B * B;
    // op(S)[m][k]: stored [m][k] when used as is, [k][m] when used transposed
    if constexpr (AKC) load_tile<T, B, TK, C::PA, NT>(as, blk + sub * TK, B, tid, B, TK);
    else               load_tile<T, TK, B, C::PA, NT>(as, blk + sub * TK * B, B, tid, TK, B);
    const int64_t k0 = (int64_t)kb * B + sub * TK;
    if constexpr (BKC) load_tile<T, TN, TK, C::PB, NT>(bs, bmat + k0, p.b_sn, tid, n_ok, TK);
    else               load_tile<T, TK, TN, C::PB, NT>(bs, bmat + k0 * p.b_sk, p.b_sk, tid, TK, n_ok);
  };

  const int m0 = (warp / WCOLS) * Sh::WM, n0 = (warp % WCOLS) * Sh::WN;
  Acc<T, Sh::WM, Sh::WN> acc;
  acc.clear();

  const int nchunks = count * SUB;
#pragma unroll
  for (int s = 0; s < kDsdStages - 1; ++s) {
    if (s < nchunks) issue(s, s);
    cp_async_commit();
  }
  for (int c = 0; c < nchunks; ++c) {
    cp_async_wait<kDsdStages - 2>();
    __syncthreads();
    const int nx = c + kDsdStages - 1;
    if (nx < nchunks) issue(nx, nx % kDsdStages);
    cp_async_commit();
    const T* st = smem + (c % kDsdStages) * C::STAGE;
    warp_tile_mma<T, Sh::WM, Sh::WN, TK, AKC, BKC, C::PA, C::PB>(acc, st, st + C::A_ELEMS, m0, n0, lane);
  }
  cp_async_wait<0>();

  T* cmat = reinterpret_cast<T*>(p.c) + z * p.c_sz + h * p.c_sh + ((int64_t)o * B + m0) * p.c_sm +
            ((int64_t)n0g + n0) * p.c_sn;
  const int n_lim = n_ok - n0;
  for_each_acc<T, Sh::WM, Sh::WN>(acc, lane, [&](int r, int cidx, float v) {
    if (cidx < n_lim) cmat[r * p.c_sm + cidx * p.c_sn] = cvt_out<T>(v);
  });
}

template <typename T, int B, int TN, bool AKC, bool BKC>
int dsd_launch(const DsdArgs& p0, int Z, int H, cudaStream_t st) {
  using C = DsdCfg<T, B, TN, AKC, BKC>;
  DsdArgs p = p0;
  p.n_tiles = (p.N + TN - 1) / TN;
  auto kern = dsd_kernel<T, B, TN, AKC, BKC>;
  if (C::BYTES > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::BYTES);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "dsd: cannot reserve %d bytes of shared memory: %s", C::BYTES, cudaGetErrorString(e));
  }
  const dim3 grid((unsigned)((int64_t)H * p.outer * p.n_tiles), Z);
  kern<<<grid, C::NW * 32, C::BYTES, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "dsd launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

template <typename T, int B, int TN>
int dsd_layout(const DsdArgs& p, bool trans_s, int Z, int H, cudaStream_t st) {
  const bool bkc = p.b_sk == 1 && p.b_sn != 1;
  if (!trans_s && bkc) return dsd_launch<T, B, TN, true, true>(p, Z, H, st);
  if (!trans_s) return dsd_launch<T, B, TN, true, false>(p, Z, H, st);
  if (bkc) return dsd_launch<T, B, TN, false, true>(p, Z, H, st);
  return dsd_launch<T, B, TN, false, false>(p, Z, H, st);
}

template <typename T, int B>
int dsd_tn(const DsdArgs& p, bool trans_s, int Z, int H, cudaStream_t st) {
  if (p.N <= 64) return dsd_layout<T, B, 64>(p, trans_s, Z, H, st);
  return dsd_layout<T, B, 128>(p, trans_s, Z, H, st);
}

}  // namespace

// One instance per element type (dsd_f32.cu, dsd_f16.cu, dsd_bf16.cu).
template <typename T>
int dsd_mma_t(const void* s, const void* b, void* c, int block, int Z, int N,
              int64_t s_sz, int trans_s,
              int64_t b_sz, int64_t b_sh, int64_t b_sk, int64_t b_sn,
              int64_t c_sz, int64_t c_sh, int64_t c_sm, int64_t c_sn,
              const Meta& m, cudaStream_t st) {
  DsdArgs p;
  p.s = s; p.b = b; p.c = c; p.s_sz = s_sz;
  p.b_sz = b_sz; p.b_sh = b_sh; p.b_sk = b_sk; p.b_sn = b_sn;
  p.c_sz = c_sz; p.c_sh = c_sh; p.c_sm = c_sm; p.c_sn = c_sn;
  p.N = N; p.n_tiles = 0;
  if (trans_s) {
    p.outer = m.Nb; p.ptr = m.col_ptr; p.kidx = m.col_row; p.bid = m.col_bid; p.order = m.col_order;
  } else {
    p.outer = m.Mb; p.ptr = m.row_ptr; p.kidx = m.blk_col; p.bid = nullptr; p.order = m.row_order;
  }
  switch (block) {
    case 16: return dsd_tn<T, 16>(p, trans_s != 0, Z, m.H, st);
    case 32: return dsd_tn<T, 32>(p, trans_s != 0, Z, m.H, st);
    case 64: return dsd_tn<T, 64>(p, trans_s != 0, Z, m.H, st);
    default: return dsd_tn<T, 128>(p, trans_s != 0, Z, m.H, st);
  }
}

}  // namespace bsp
