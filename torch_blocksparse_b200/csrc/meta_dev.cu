// Execution metadata (the buffer bsp_meta_build writes on the host) built on the device from a
// layout that lives in device memory: no copy of the layout to the host, no upload of the
// result.  Replaces, for the kernels' own metadata, the reference's host-side rebuild and
// upload of its tables per (dtype, device) (torch_blocksparse/matmul.py:611-641, with the
// `.to(device)` of matmul.py:293,455 and softmax.py:220).
//
// The buffer is bit-identical to bsp_meta_build's: header, CSR (row_ptr, blk_row, blk_col,
// blk_head), CSC (col_ptr, col_row, col_bid), longest-first orders of the block-rows and
// block-columns (stable).  Section offsets depend on the number of nonzero blocks, which is
// only known on the device, so every kernel after the count derives them from the header the
// scan kernel wrote.  Layout sizes are small (H * Mb * Nb positions, typically < 10^6): the
// kernels favour simplicity over throughput and the whole build takes tens of microseconds.
#include <cuda_runtime.h>
#include <algorithm>
#include "common.h"

namespace bsp {
namespace {

template <typename L>
__global__ void meta_count_kernel(const L* __restrict__ lay, int H, int Mb, int Nb, int32_t* __restrict__ row_cnt,
                                  int32_t* __restrict__ col_cnt) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < H * Mb) {                                   // one thread per block-row
    const L* p = lay + (size_t)i * Nb;
    int c = 0;
    for (int n = 0; n < Nb; ++n) c += p[n] != 0;
    row_cnt[i] = c;
  }
  if (i < H * Nb) {                                   // one thread per block-column
    const int h = i / Nb, n = i % Nb;
    const L* p = lay + (size_t)h * Mb * Nb + n;
    int c = 0;
    for (int m = 0; m < Mb; ++m) c += p[(size_t)m * Nb] != 0;
    col_cnt[i] = c;
  }
}

// Exclusive scan of `n` counts into ptr[0 .. n] by one block of 1024 threads; returns the total
// in every thread and the maximum count through *mx.
__device__ int block_scan(const int32_t* cnt, int n, int32_t* ptr, int* mx) {
  __shared__ int warp_sums[32];
  __shared__ int carry, vmax;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { carry = 0; vmax = 0; }
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + tid;
    const int v = i < n ? cnt[i] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int s = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += y;
      }
      warp_sums[lane] = s;
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + x - v;
    if (i < n) ptr[i] = before;
    atomicMax(&vmax, v);
    __syncthreads();
    if (tid == 1023) carry = before + v;
    __syncthreads();
  }
  if (tid == 0) ptr[n] = carry;
  __syncthreads();
  *mx = vmax;
  const int total = carry;
  __syncthreads();
  return total;
}

__global__ void __launch_bounds__(1024) meta_scan_kernel(const int32_t* __restrict__ row_cnt, const int32_t* __restrict__ col_cnt,
                                                          int H, int Mb, int Nb, int32_t* __restrict__ out) {
  int max_row = 0, max_col = 0;
  const int nnz = block_scan(row_cnt, H * Mb, out + BSP_META_HEADER, &max_row);
  int32_t* col_ptr = out + BSP_META_HEADER + (H * Mb + 1) + 3 * (size_t)nnz;
  block_scan(col_cnt, H * Nb, col_ptr, &max_col);
  if (threadIdx.x == 0) {
    out[0] = BSP_META_MAGIC; out[1] = H; out[2] = Mb; out[3] = Nb; out[4] = nnz; out[5] = max_row; out[6] = max_col; out[7] = 0;
  }
}

template <typename L>
__global__ void meta_fill_kernel(const L* __restrict__ lay, int H, int Mb, int Nb, int32_t* __restrict__ out) {
  const int nnz = out[4];
  const int32_t* row_ptr = out + BSP_META_HEADER;
  int32_t* blk_row = out + BSP_META_HEADER + (H * Mb + 1);
  int32_t* blk_col = blk_row + nnz;
  int32_t* blk_head = blk_col + nnz;
  const int32_t* col_ptr = blk_head + nnz;
  int32_t* col_row = blk_head + nnz + (H * Nb + 1);
  int32_t* col_bid = col_row + nnz;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < H * Mb) {                                   // CSR entries of one block-row, in column order
    const int h = i / Mb, m = i % Mb;
    const L* p = lay + (size_t)i * Nb;
    int b = row_ptr[i];
    for (int n = 0; n < Nb; ++n)
      if (p[n] != 0) { blk_row[b] = m; blk_col[b] = n; blk_head[b] = h; ++b; }
  }
  if (i < H * Nb) {                                   // CSC entries of one block-column, in row order
    const int h = i / Nb, n = i % Nb;
    const L* base = lay + (size_t)h * Mb * Nb;
    int c = col_ptr[i];
    for (int m = 0; m < Mb; ++m) {
      const L* row = base + (size_t)m * Nb;
      if (row[n] == 0) continue;
      int rank = 0;                                    // nonzeros of the row before this column
      for (int k = 0; k < n; ++k) rank += row[k] != 0;
      col_row[c] = m;
      col_bid[c] = row_ptr[h * Mb + m] + rank;
      ++c;
    }
  }
}

// order[pos] = x with pos = rank of x in the stable sort by descending length.
__global__ void meta_order_kernel(int H, int Mb, int Nb, int32_t* __restrict__ out) {
  const int nnz = out[4];
  const int32_t* row_ptr = out + BSP_META_HEADER;
  const int32_t* col_ptr = out + BSP_META_HEADER + (H * Mb + 1) + 3 * (size_t)nnz;
  int32_t* row_order = out + BSP_META_HEADER + (H * Mb + 1) + 3 * (size_t)nnz + (H * Nb + 1) + 2 * (size_t)nnz;
  int32_t* col_order = row_order + H * Mb;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool rows = blockIdx.y == 0;
  const int n = rows ? H * Mb : H * Nb;
  if (i >= n) return;
  const int32_t* ptr = rows ? row_ptr : col_ptr;
  const int mine = ptr[i + 1] - ptr[i];
  int pos = 0;
  for (int y = 0; y < n; ++y) {
    const int len = ptr[y + 1] - ptr[y];
    pos += (len > mine) || (len == mine && y < i);
  }
  (rows ? row_order : col_order)[pos] = i;
}

template <typename L>
int build(const L* lay, int H, int Mb, int Nb, int32_t* out, int32_t* scratch, cudaStream_t st) {
  const int n = std::max(H * Mb, H * Nb);
  const int grid = (n + 255) / 256;
  meta_count_kernel<L><<<grid, 256, 0, st>>>(lay, H, Mb, Nb, scratch, scratch + H * Mb);
  meta_scan_kernel<<<1, 1024, 0, st>>>(scratch, scratch + H * Mb, H, Mb, Nb, out);
  meta_fill_kernel<L><<<grid, 256, 0, st>>>(lay, H, Mb, Nb, out);
  meta_order_kernel<<<dim3(grid, 2), 256, 0, st>>>(H, Mb, Nb, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device metadata build: launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

// ---- validation -----------------------------------------------------------------------------
// Every index a compute kernel will derive from a metadata buffer or from attention tile
// lists, checked against the sizes in the buffer's header: the first violation found is
// recorded as (code, position) in `err` (two ints, zero on entry).  Used instead of a memory
// checker: a corrupt table shows up as an error code before any kernel dereferences it.
__device__ void report(int* err, int code, int pos) {
  if (atomicCAS(&err[0], 0, code) == 0) err[1] = pos;
}

__global__ void meta_validate_kernel(const int32_t* __restrict__ m, int64_t len, int* err) {
  const int H = m[1], Mb = m[2], Nb = m[3], nnz = m[4];
  if (m[0] != BSP_META_MAGIC || H <= 0 || Mb <= 0 || Nb <= 0 || nnz < 0 || meta_total(H, Mb, Nb, nnz) > len) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report(err, 1, 0);
    return;
  }
  const Meta v = meta_view(m, H, Mb, Nb, nnz, m[5], m[6]);
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i <= H * Mb) {
    if (i == 0 && v.row_ptr[0] != 0) report(err, 2, 0);
    if (i == H * Mb && v.row_ptr[i] != nnz) report(err, 2, (int)i);
    if (i < H * Mb && (v.row_ptr[i + 1] < v.row_ptr[i] || v.row_ptr[i + 1] - v.row_ptr[i] > m[5])) report(err, 3, (int)i);
    if (i < H * Mb && (v.row_order[i] < 0 || v.row_order[i] >= H * Mb)) report(err, 8, (int)i);
  }
  if (i <= H * Nb) {
    if (i == 0 && v.col_ptr[0] != 0) report(err, 4, 0);
    if (i == H * Nb && v.col_ptr[i] != nnz) report(err, 4, (int)i);
    if (i < H * Nb && (v.col_ptr[i + 1] < v.col_ptr[i] || v.col_ptr[i + 1] - v.col_ptr[i] > m[6])) report(err, 5, (int)i);
    if (i < H * Nb && (v.col_order[i] < 0 || v.col_order[i] >= H * Nb)) report(err, 9, (int)i);
  }
  if (i < nnz) {
    if (v.blk_row[i] < 0 || v.blk_row[i] >= Mb || v.blk_col[i] < 0 || v.blk_col[i] >= Nb || v.blk_head[i] < 0 || v.blk_head[i] >= H)
      report(err, 6, (int)i);
    if (v.col_row[i] < 0 || v.col_row[i] >= Mb || v.col_bid[i] < 0 || v.col_bid[i] >= nnz) report(err, 7, (int)i);
  }
}

__global__ void tiles_validate_kernel(const int32_t* __restrict__ t, int64_t len, int* err) {
  const int H = t[1], nb = t[2], block = t[3], nt = t[4], er = t[5], ec = t[6];
  const int64_t n = (int64_t)H * nt;
  if (t[0] != BSP_TILES_MAGIC || H <= 0 || nb <= 0 || nt <= 0 || er < 0 || ec < 0 || (block != 64 && block != 128) ||
      BSP_TILES_HEADER + 2 * (4 * n + 1) + 3 * (int64_t)er + 3 * (int64_t)ec > len) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report(err, 11, 0);
    return;
  }
  const int chunks = nb * (block / 64);                   // 64-row chunks per side
  const int32_t* p = t + BSP_TILES_HEADER;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int set = 0; set < 2; ++set) {
    const int e = set == 0 ? er : ec;
    const int32_t *c01 = p, *ptr = c01 + 2 * n, *chunk = ptr + n + 1, *mask = chunk + e, *order = mask + 2 * (int64_t)e;
    if (i < 2 * n && (c01[i] < -1 || c01[i] >= chunks)) report(err, 12 + 10 * set, (int)i);
    if (i <= n) {
      if (i == 0 && ptr[0] != 0) report(err, 13 + 10 * set, 0);
      if (i == n && ptr[i] != e) report(err, 13 + 10 * set, (int)i);
      if (i < n && ptr[i + 1] < ptr[i]) report(err, 14 + 10 * set, (int)i);
      if (i < n && (order[i] < 0 || order[i] >= n)) report(err, 15 + 10 * set, (int)i);
    }
    if (i < e && (chunk[i] < 0 || chunk[i] >= chunks || mask[i] < 0 || mask[i] > 3)) report(err, 16 + 10 * set, (int)i);
    p = order + n;
  }
}

int validate(bool tiles, const int32_t* buf, int64_t len, int* code, int* pos, cudaStream_t st) {
  if (!buf || len < 8 || !code || !pos) return fail(BSP_ERR_INVALID, "validation: NULL buffer or result pointer");
  int* err = nullptr;
  cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&err), 2 * sizeof(int), st);
  if (e == cudaSuccess) e = cudaMemsetAsync(err, 0, 2 * sizeof(int), st);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "validation: scratch allocation failed: %s", cudaGetErrorString(e));
  const int grid = (int)((len + 255) / 256);
  if (tiles) tiles_validate_kernel<<<grid, 256, 0, st>>>(buf, len, err);
  else meta_validate_kernel<<<grid, 256, 0, st>>>(buf, len, err);
  int host[2] = {0, 0};
  e = cudaMemcpyAsync(host, err, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFreeAsync(err, st);
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "validation failed to run: %s", cudaGetErrorString(e));
  *code = host[0]; *pos = host[1];
  if (host[0]) return fail(BSP_ERR_INVALID, "%s buffer is corrupt: check %d failed at entry %d",
                           tiles ? "attention tile-list" : "metadata", host[0], host[1]);
  return BSP_OK;
}

}  // namespace
}  // namespace bsp

using namespace bsp;

extern "C" int bsp_meta_validate(const int32_t* meta, int64_t len, int* code, int* pos, void* stream) {
  return validate(false, meta, len, code, pos, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int bsp_attn_tiles_validate(const int32_t* tiles, int64_t len, int* code, int* pos, void* stream) {
  return validate(true, tiles, len, code, pos, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int64_t bsp_meta_device_capacity(int H, int Mb, int Nb) {
  if (H <= 0 || Mb <= 0 || Nb <= 0) return 0;
  return meta_total(H, Mb, Nb, (int64_t)H * Mb * Nb) + (int64_t)H * Mb + (int64_t)H * Nb;
}

extern "C" int bsp_meta_build_device(const void* layout, int elem_bytes, int H, int Mb, int Nb,
                                     int32_t* out, int64_t out_cap, int32_t* hdr_host, void* stream) {
  if (!layout || !out) return fail(BSP_ERR_INVALID, "device metadata build: NULL pointer");
  if (H <= 0 || Mb <= 0 || Nb <= 0) return fail(BSP_ERR_INVALID, "layout shape [%d,%d,%d] is not positive", H, Mb, Nb);
  if (elem_bytes != 1 && elem_bytes != 4 && elem_bytes != 8)
    return fail(BSP_ERR_INVALID, "device metadata build: layout elements of 1, 4 or 8 bytes (got %d)", elem_bytes);
  if ((int64_t)H * Mb * Nb > (int64_t)1 << 28) return fail(BSP_ERR_UNSUPPORTED, "device metadata build: layout too large");
  const int64_t need = bsp_meta_device_capacity(H, Mb, Nb);
  if (out_cap < need)
    return fail(BSP_ERR_CAPACITY, "device metadata build needs a buffer of %lld ints (worst case), got %lld",
                (long long)need, (long long)out_cap);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // counts live past the worst-case end of the metadata: never overlapped by it
  int32_t* scratch = out + meta_total(H, Mb, Nb, (int64_t)H * Mb * Nb);
  int rc;
  if (elem_bytes == 8) rc = build(static_cast<const int64_t*>(layout), H, Mb, Nb, out, scratch, st);
  else if (elem_bytes == 4) rc = build(static_cast<const int32_t*>(layout), H, Mb, Nb, out, scratch, st);
  else rc = build(static_cast<const uint8_t*>(layout), H, Mb, Nb, out, scratch, st);
  if (rc) return rc;
  if (hdr_host) {                                    // the launch code needs the sizes: 32 bytes come back
    cudaError_t e = cudaMemcpyAsync(hdr_host, out, BSP_META_HEADER * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device metadata build: reading the header failed: %s", cudaGetErrorString(e));
  }
  return BSP_OK;
}
