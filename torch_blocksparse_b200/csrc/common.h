// Shared host-side helpers of the block-sparse library: error reporting and
// argument checks used by every C-ABI entry point.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include "../../include/bsp.h"

#ifdef __CUDACC__
#define BSP_HD __host__ __device__
#else
#define BSP_HD
#endif

namespace bsp {

// Stores a printf-style message in the calling thread's error slot and
// returns `code`, so that entry points can `return fail(code, ...)`.
int fail(int code, const char* fmt, ...);

inline bool valid_block(int b) { return b == 16 || b == 32 || b == 64 || b == 128; }
inline bool valid_dtype(int d) { return d == BSP_F32 || d == BSP_F16 || d == BSP_BF16; }
inline int dtype_bytes(int d) { return d == BSP_F32 ? 4 : 2; }

// Decoded view of the execution metadata written by bsp_meta_build; all
// pointers are DEVICE pointers into the caller's metadata buffer, the scalar
// fields come from the host-side copy the caller passes along.
struct Meta {
  int H, Mb, Nb, nnz, max_row, max_col;
  const int32_t* row_ptr;
  const int32_t* blk_row;
  const int32_t* blk_col;
  const int32_t* blk_head;
  const int32_t* col_ptr;
  const int32_t* col_row;
  const int32_t* col_bid;
  const int32_t* row_order;
  const int32_t* col_order;
};

BSP_HD inline int64_t meta_total(int H, int Mb, int Nb, int64_t nnz) {
  return BSP_META_HEADER + (int64_t)(H * Mb + 1) + 3 * nnz + (int64_t)(H * Nb + 1) + 2 * nnz +
         (int64_t)H * Mb + (int64_t)H * Nb;
}

// Lays the section pointers of a metadata buffer out from its base address.
BSP_HD inline Meta meta_view(const int32_t* base, int H, int Mb, int Nb, int nnz, int max_row, int max_col) {
  Meta m;
  m.H = H; m.Mb = Mb; m.Nb = Nb; m.nnz = nnz; m.max_row = max_row; m.max_col = max_col;
  const int32_t* p = base + BSP_META_HEADER;
  m.row_ptr = p;   p += H * Mb + 1;
  m.blk_row = p;   p += nnz;
  m.blk_col = p;   p += nnz;
  m.blk_head = p;  p += nnz;
  m.col_ptr = p;   p += H * Nb + 1;
  m.col_row = p;   p += nnz;
  m.col_bid = p;   p += nnz;
  m.row_order = p; p += H * Mb;
  m.col_order = p;
  return m;
}

}  // namespace bsp
