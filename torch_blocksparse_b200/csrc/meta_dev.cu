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

// ---------------------------------------------------------------------------------------------
// Attention tile lists (the buffer bsp_attn_tiles_build writes on the host) built on the device,
// for blocks 64 and 128 and at most kTilesMaxNb blocks per side.  Bit-identical to the host
// builder: per head and side (rows, columns) the block-rows are sorted by size (stable,
// descending) and paired greedily, each with the unused later one whose nonzero set is most
// similar (|A and B| / |A or B|, first best wins); a tile's list is the union of its two sets in
// ascending order with a 2-bit mask per entry.  One CTA per (head, side) does the pairing; the
// candidates of a row are scored in parallel, the rows are taken one after the other as the
// greedy rule demands.
// ---------------------------------------------------------------------------------------------
namespace bsp {
namespace {

constexpr int kTilesMaxNb = 512;
constexpr int kTilesWords = kTilesMaxNb / 64;

template <typename L>
__device__ __forceinline__ bool present(const L* lay, int nb, int side, int h, int outer, int inner) {
  // side 0: outer = row, inner = column; side 1: outer = column, inner = row
  const size_t r = side == 0 ? outer : inner, c = side == 0 ? inner : outer;
  return lay[((size_t)h * nb + r) * nb + c] != 0;
}

// c01s: [2][H * nt][2] pairs; lens: [2][H * nt] list lengths
template <typename L>
__global__ void __launch_bounds__(256) tiles_pair_kernel(const L* __restrict__ lay, int H, int nb, int block, int nt,
                                                         int32_t* __restrict__ c01s, int32_t* __restrict__ lens) {
  const int h = blockIdx.x, side = blockIdx.y, tid = threadIdx.x;
  const int words = (nb + 63) / 64;
  __shared__ unsigned long long bits[kTilesMaxNb][kTilesWords];
  __shared__ short size[kTilesMaxNb], order[kTilesMaxNb];
  __shared__ unsigned char used[kTilesMaxNb];
  __shared__ int red_inter[256], red_uni[256], red_oj[256];
  int32_t* c01 = c01s + ((size_t)side * H * nt + (size_t)h * nt) * 2;
  int32_t* len = lens + (size_t)side * H * nt + (size_t)h * nt;
  for (int i = tid; i < nb; i += 256) {
    int cnt = 0;
    for (int w = 0; w < words; ++w) {
      unsigned long long b = 0;
      for (int k = 0; k < 64 && w * 64 + k < nb; ++k)
        if (present(lay, nb, side, h, i, w * 64 + k)) { b |= 1ull << k; ++cnt; }
      bits[i][w] = b;
    }
    size[i] = (short)cnt;
    used[i] = 0;
  }
  __syncthreads();
  if (block == 128) {                                 // a tile is one block-row; every block brings two chunks
    for (int i = tid; i < nb; i += 256) { c01[2 * i] = 2 * i; c01[2 * i + 1] = 2 * i + 1; len[i] = 2 * size[i]; }
    return;
  }
  for (int i = tid; i < nb; i += 256) {               // stable order by descending size
    int pos = 0;
    for (int y = 0; y < nb; ++y) pos += (size[y] > size[i]) || (size[y] == size[i] && y < i);
    order[pos] = (short)i;
  }
  __syncthreads();
  int tile = 0;
  for (int oi = 0; oi < nb; ++oi) {
    const int u = order[oi];
    if (used[u]) continue;                            // (uniform: shared memory, read after a barrier)
    // every thread scores its share of the later unused rows; the best is the highest
    // |A and B| / |A or B| (two empty sets count as 1), the first in the order among equals
    int bi = -1, bu = 1, boj = 1 << 30;
    for (int oj = oi + 1 + tid; oj < nb; oj += 256) {
      const int v = order[oj];
      if (used[v]) continue;
      int inter = 0, uni = 0;
      for (int w = 0; w < words; ++w) {
        inter += __popcll(bits[u][w] & bits[v][w]);
        uni += __popcll(bits[u][w] | bits[v][w]);
      }
      if (uni == 0) { inter = 1; uni = 1; }
      if (bi < 0 || inter * bu > bi * uni) { bi = inter; bu = uni; boj = oj; }      // (own candidates come in order)
    }
    red_inter[tid] = bi; red_uni[tid] = bu; red_oj[tid] = boj;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
      if (tid < s) {
        const int ai = red_inter[tid], au = red_uni[tid], ao = red_oj[tid];
        const int ci = red_inter[tid + s], cu = red_uni[tid + s], co = red_oj[tid + s];
        bool take = false;
        if (ci >= 0) {
          if (ai < 0) take = true;
          else {
            const int lhs = ci * au, rhs = ai * cu;   // c better than a?
            take = lhs > rhs || (lhs == rhs && co < ao);
          }
        }
        if (take) { red_inter[tid] = ci; red_uni[tid] = cu; red_oj[tid] = co; }
      }
      __syncthreads();
    }
    const int best = red_inter[0] >= 0 ? order[red_oj[0]] : -1;
    if (tid == 0) {
      used[u] = 1;
      if (best >= 0) used[best] = 1;
      c01[2 * tile] = best < 0 ? u : min(u, best);
      c01[2 * tile + 1] = best < 0 ? -1 : max(u, best);
      int n = 0;
      for (int w = 0; w < words; ++w) n += __popcll(bits[u][w] | (best >= 0 ? bits[best][w] : 0ull));
      len[tile] = n;
    }
    ++tile;
    __syncthreads();
  }
}

// ptr arrays of both sides (exclusive scans of the list lengths), totals, header; one CTA
__global__ void __launch_bounds__(1024) tiles_scan_kernel(const int32_t* __restrict__ lens, int H, int nb, int block, int nt,
                                                          int fine_block, int32_t* __restrict__ out) {
  const int n = H * nt;
  int mx = 0;
  int32_t* ptr_r = out + BSP_TILES_HEADER + 2 * n;
  const int er = block_scan(lens, n, ptr_r, &mx);
  int32_t* ptr_c = out + BSP_TILES_HEADER + (4 * (size_t)n + 1) + 3 * (size_t)er + 2 * n;
  const int ec = block_scan(lens + n, n, ptr_c, &mx);
  if (threadIdx.x == 0) {
    out[0] = BSP_TILES_MAGIC; out[1] = H; out[2] = nb; out[3] = block; out[4] = nt; out[5] = er; out[6] = ec; out[7] = fine_block;
  }
}

template <typename L>
__global__ void tiles_fill_kernel(const L* __restrict__ lay, int H, int nb, int block, int nt,
                                  const int32_t* __restrict__ c01s, int32_t* __restrict__ out) {
  const int n = H * nt;
  const int side = blockIdx.y;
  const int ti = blockIdx.x * blockDim.x + threadIdx.x;
  if (ti >= n) return;
  const int er = out[5], ec = out[6];
  const int e = side == 0 ? er : ec;
  int32_t* base = out + BSP_TILES_HEADER + (side == 0 ? 0 : (4 * (size_t)n + 1) + 3 * (size_t)er);
  int32_t *c01 = base, *ptr = c01 + 2 * n, *chunk = ptr + n + 1, *mask = chunk + e, *sub = mask + e;
  const int a = c01s[((size_t)side * n + ti) * 2], b = c01s[((size_t)side * n + ti) * 2 + 1];
  c01[2 * ti] = a; c01[2 * ti + 1] = b;
  const int h = ti / nt;
  int p = ptr[ti];
  if (block == 128) {
    const int i = a / 2;
    for (int j = 0; j < nb; ++j)
      if (present(lay, nb, side, h, i, j))
        for (int c = 0; c < 2; ++c) { chunk[p] = 2 * j + c; mask[p] = 3; sub[p] = -1; ++p; }
    return;
  }
  for (int j = 0; j < nb; ++j) {
    int m = present(lay, nb, side, h, a, j) ? 1 : 0;
    if (b >= 0 && present(lay, nb, side, h, b, j)) m |= 2;
    if (!m) continue;
    chunk[p] = j; mask[p] = m;
    sub[p] = (int32_t)(((m & 1) ? 0xFFFFu : 0u) | ((m & 2) ? 0xFFFF0000u : 0u));
    ++p;
  }
}

// order[pos] = tile with pos = its rank in the stable sort by descending list length
__global__ void tiles_order_kernel(int H, int nt, int32_t* __restrict__ out) {
  const int n = H * nt;
  const int side = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int er = out[5], ec = out[6];
  const int e = side == 0 ? er : ec;
  int32_t* base = out + BSP_TILES_HEADER + (side == 0 ? 0 : (4 * (size_t)n + 1) + 3 * (size_t)er);
  const int32_t* ptr = base + 2 * n;
  int32_t* order = base + 2 * n + (n + 1) + 3 * (size_t)e;
  const int mine = ptr[i + 1] - ptr[i];
  int pos = 0;
  for (int y = 0; y < n; ++y) {
    const int len = ptr[y + 1] - ptr[y];
    pos += (len > mine) || (len == mine && y < i);
  }
  order[pos] = i;
}

// Blocks 16 and 32: the layout coarsened to 64 x 64 positions (present = some piece present) and,
// per position, which of its 16 x 16 pieces lie in a nonzero block: pr[h][q][k] with bit 4 a + b
// for query group a and key group b (the row tiles' view), pc[h][k][q] with bit 4 a + b for key
// group a and query group b (the column tiles' view).
template <typename L>
__global__ void tiles_coarsen_kernel(const L* __restrict__ lay, int H, int nbf, int fine_block, int nb,
                                     uint8_t* __restrict__ coarse, uint16_t* __restrict__ pr, uint16_t* __restrict__ pc) {
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= (int64_t)H * nb * nb) return;
  const int j = (int)(idx % nb), i = (int)((idx / nb) % nb), h = (int)(idx / ((int64_t)nb * nb));
  const L* hl = lay + (size_t)h * nbf * nbf;
  int vr = 0, vc = 0;
  for (int a = 0; a < 4; ++a)
    for (int b = 0; b < 4; ++b) {
      const int fi = (i * 64 + a * 16) / fine_block, fj = (j * 64 + b * 16) / fine_block;
      if (hl[(size_t)fi * nbf + fj] != 0) { vr |= 1 << (4 * a + b); vc |= 1 << (4 * b + a); }
    }
  coarse[idx] = vr != 0;
  pr[idx] = (uint16_t)vr;
  pc[((size_t)h * nb + j) * nb + i] = (uint16_t)vc;
}

// sub of every entry from the piece masks (blocks 16 and 32); one thread per tile and side
__global__ void tiles_sub_kernel(int H, int nb, int nt, const uint16_t* __restrict__ pr, const uint16_t* __restrict__ pc,
                                 int32_t* __restrict__ out) {
  const int n = H * nt;
  const int side = blockIdx.y;
  const int ti = blockIdx.x * blockDim.x + threadIdx.x;
  if (ti >= n) return;
  const int er = out[5], ec = out[6];
  const int e = side == 0 ? er : ec;
  int32_t* base = out + BSP_TILES_HEADER + (side == 0 ? 0 : (4 * (size_t)n + 1) + 3 * (size_t)er);
  const int32_t *c01 = base, *ptr = c01 + 2 * n, *chunk = ptr + n + 1, *mask = chunk + e;
  int32_t* sub = base + 2 * n + (n + 1) + 2 * (size_t)e;
  const uint16_t* P = (side == 0 ? pr : pc) + (size_t)(ti / nt) * nb * nb;
  const int a = c01[2 * ti], b = c01[2 * ti + 1];
  for (int p = ptr[ti]; p < ptr[ti + 1]; ++p) {
    const int j = chunk[p], m = mask[p];
    const uint32_t lo = (m & 1) ? P[(size_t)a * nb + j] : 0u, hi = (m & 2) ? P[(size_t)b * nb + j] : 0u;
    sub[p] = (int32_t)(lo | (hi << 16));
  }
}

template <typename L>
int build_tiles(const L* lay, int H, int nb, int block, int nt, int32_t* out, int32_t* scratch, cudaStream_t st,
                int fine_block = 0) {
  const int n = H * nt;
  int32_t* c01s = scratch;
  int32_t* lens = scratch + 4 * (size_t)n;
  tiles_pair_kernel<L><<<dim3(H, 2), 256, 0, st>>>(lay, H, nb, block, nt, c01s, lens);
  tiles_scan_kernel<<<1, 1024, 0, st>>>(lens, H, nb, block, nt, fine_block ? fine_block : block, out);
  const int grid = (n + 127) / 128;
  tiles_fill_kernel<L><<<dim3(grid, 2), 128, 0, st>>>(lay, H, nb, block, nt, c01s, out);
  tiles_order_kernel<<<dim3(grid, 2), 128, 0, st>>>(H, nt, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device tile-list build: launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}

int64_t tiles_worst_case(int H, int nb, int block) {
  const int64_t nt = block == 128 ? nb : (nb + 1) / 2, n = (int64_t)H * nt;
  const int64_t e = block == 128 ? 2 * (int64_t)H * nb * nb : n * nb;       // entries of one side at most
  return BSP_TILES_HEADER + 2 * (4 * n + 1) + 6 * e;
}

}  // namespace
}  // namespace bsp

extern "C" int64_t bsp_attn_tiles_device_capacity(int H, int nb, int block) {
  if (H <= 0 || nb <= 0 || (block != 16 && block != 32 && block != 64 && block != 128)) return 0;
  int64_t extra = 0;
  if (block < 64) {                                                          // coarsened layout and piece masks
    const int f = 64 / block;
    if (nb % f) return 0;
    nb /= f; block = 64;
    extra = (5 * (int64_t)H * nb * nb + 3) / 4 + 4;
  }
  const int64_t nt = block == 128 ? nb : (nb + 1) / 2;
  return tiles_worst_case(H, nb, block) + 6 * (int64_t)H * nt + extra;       // + pairs and lengths of both sides
}

extern "C" int bsp_attn_tiles_build_device(const void* layout, int elem_bytes, int H, int nb, int block,
                                           int32_t* out, int64_t out_cap, int32_t* hdr_host, void* stream) {
  if (!layout || !out) return fail(BSP_ERR_INVALID, "device tile-list build: NULL pointer");
  if (H <= 0 || nb <= 0) return fail(BSP_ERR_INVALID, "layout shape [%d,%d,%d] is not positive", H, nb, nb);
  if (block != 16 && block != 32 && block != 64 && block != 128)
    return fail(BSP_ERR_UNSUPPORTED, "attention tiles exist for block 16, 32, 64 and 128 (got %d)", block);
  const int fine_block = block, nbf = nb, f = block < 64 ? 64 / block : 1;
  if (nb % f) return fail(BSP_ERR_UNSUPPORTED, "attention tiles for block %d need a number of blocks per side that is a multiple of %d (got %d)", block, f, nb);
  if (f > 1) { nb /= f; block = 64; }
  if (nb > kTilesMaxNb) return fail(BSP_ERR_UNSUPPORTED, "device tile-list build: at most %d positions of 64 or 128 per side (got %d)", kTilesMaxNb, nb);
  if (elem_bytes != 1 && elem_bytes != 4 && elem_bytes != 8)
    return fail(BSP_ERR_INVALID, "device tile-list build: layout elements of 1, 4 or 8 bytes (got %d)", elem_bytes);
  const int64_t need = bsp_attn_tiles_device_capacity(H, nbf, fine_block);
  if (out_cap < need)
    return fail(BSP_ERR_CAPACITY, "device tile-list build needs a buffer of %lld ints (worst case), got %lld",
                (long long)need, (long long)out_cap);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nt = block == 128 ? nb : (nb + 1) / 2;
  int32_t* scratch = out + tiles_worst_case(H, nb, block);
  int rc;
  if (f > 1) {
    // blocks 16 / 32: block-64 lists of the coarsened layout, then the piece masks of every entry
    const int64_t pos = (int64_t)H * nb * nb;
    uint16_t* pr = reinterpret_cast<uint16_t*>(scratch + 6 * (size_t)H * nt);
    uint16_t* pc = pr + pos;
    uint8_t* coarse = reinterpret_cast<uint8_t*>(pc + pos);
    const unsigned grid = (unsigned)((pos + 255) / 256);
    if (elem_bytes == 8) tiles_coarsen_kernel<<<grid, 256, 0, st>>>(static_cast<const int64_t*>(layout), H, nbf, fine_block, nb, coarse, pr, pc);
    else if (elem_bytes == 4) tiles_coarsen_kernel<<<grid, 256, 0, st>>>(static_cast<const int32_t*>(layout), H, nbf, fine_block, nb, coarse, pr, pc);
    else tiles_coarsen_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(layout), H, nbf, fine_block, nb, coarse, pr, pc);
    rc = build_tiles(coarse, H, nb, block, nt, out, scratch, st, fine_block);
    if (rc) return rc;
    tiles_sub_kernel<<<dim3((H * nt + 127) / 128, 2), 128, 0, st>>>(H, nb, nt, pr, pc, out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device tile-list build: launch failed: %s", cudaGetErrorString(e));
  } else {
    if (elem_bytes == 8) rc = build_tiles(static_cast<const int64_t*>(layout), H, nb, block, nt, out, scratch, st);
    else if (elem_bytes == 4) rc = build_tiles(static_cast<const int32_t*>(layout), H, nb, block, nt, out, scratch, st);
    else rc = build_tiles(static_cast<const uint8_t*>(layout), H, nb, block, nt, out, scratch, st);
    if (rc) return rc;
  }
  if (hdr_host) {
    cudaError_t e = cudaMemcpyAsync(hdr_host, out, BSP_TILES_HEADER * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "device tile-list build: reading the header failed: %s", cudaGetErrorString(e));
  }
  return BSP_OK;
}

// ---- softmax table from the execution metadata ------------------------------------------
namespace bsp {
namespace {

// One thread per row header and per block entry of the table bsp_softmax_lut_build writes.
__global__ void softmax_lut_kernel(Meta m, int32_t* out) {
  const int64_t rows = (int64_t)m.H * m.Mb;
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < rows) {
    const int first = m.row_ptr[i];
    out[2 * i] = m.row_ptr[i + 1] - first;
    out[2 * i + 1] = (int32_t)(4 * (int64_t)first + 2 * rows);
  }
  if (i < m.nnz) {
    int32_t* e = out + 2 * rows + 4 * i;
    e[0] = (int32_t)i; e[1] = m.blk_col[i]; e[2] = m.blk_row[i]; e[3] = m.blk_head[i];
  }
}

}  // namespace
}  // namespace bsp

extern "C" int bsp_softmax_lut_from_meta(const int32_t* meta_hdr, const int32_t* meta, int32_t* out, int64_t out_cap,
                                         int64_t* total, int* maxlut, void* stream) {
  using namespace bsp;
  if (!meta_hdr || !meta || !total || !maxlut) return fail(BSP_ERR_INVALID, "softmax table from metadata: NULL pointer");
  if (meta_hdr[0] != BSP_META_MAGIC || meta_hdr[1] <= 0 || meta_hdr[2] <= 0 || meta_hdr[3] <= 0 || meta_hdr[4] < 0)
    return fail(BSP_ERR_INVALID, "metadata header is corrupt");
  const Meta m = meta_view(meta, meta_hdr[1], meta_hdr[2], meta_hdr[3], meta_hdr[4], meta_hdr[5], meta_hdr[6]);
  const int64_t rows = (int64_t)m.H * m.Mb;
  *total = 2 * rows + 4 * (int64_t)m.nnz;
  *maxlut = m.max_row;
  if (!out) return BSP_OK;
  if (out_cap < *total)
    return fail(BSP_ERR_CAPACITY, "softmax table needs %lld ints, buffer holds %lld", (long long)*total, (long long)out_cap);
  const int64_t n = rows > m.nnz ? rows : m.nnz;
  softmax_lut_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(m, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSP_ERR_CUDA, "softmax table from metadata: launch failed: %s", cudaGetErrorString(e));
  return BSP_OK;
}
