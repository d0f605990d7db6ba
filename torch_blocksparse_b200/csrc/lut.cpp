// Host-side layout -> table builders of the block-sparse library.
//
// The three reference-format tables (SDD, DSD/DDS, softmax) are reproduced
// bit for bit from the reference's builders:
//   SDD      torch_blocksparse/matmul.py:281-297 + csrc/utils.cpp:11-120
//   DSD/DDS  torch_blocksparse/matmul.py:221-267, 372-458
//   softmax  torch_blocksparse/softmax.py:201-221
// plus the "fixed" layout generator
//   torch_blocksparse/deepspeedsparseselfattention.py:33-65
// and the CSR/CSC execution metadata the compute kernels of this library read.
//
// Heads are independent in every builder; the SDD packer (the only one with a
// sequential scan) runs its heads on a small pool of std::threads.
#include <algorithm>
#include <climits>
#include <cstring>
#include <numeric>
#include <thread>
#include <functional>
#include <vector>
#include "common.h"

namespace bsp {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

namespace {

struct Entry { int32_t h, i, j, b; };

// Greedy w x w packing of one head for one pass.
//   present : Mb*Nb flags of this head, consumed (packed blocks are cleared)
//   ids     : canonical block id of every position of this head
// The scan keeps, as the reference does, a history of the last w nonzero columns
// visited (carried across rows) and, per column, of the last w nonzero rows.
void pack_head(int h, int Mb, int Nb, int w, uint8_t* present, const int32_t* ids,
               std::vector<Entry>& out) {
  std::vector<int32_t> run(size_t(Mb) * Nb, 0);        // side of the square ending at (m, n)
  std::vector<int32_t> hist_col(w, -1);                // circular, newest at (head_c - 1) mod w
  std::vector<int32_t> hist_row(size_t(w) * Nb, -1);   // [n][k] circular per column
  std::vector<int32_t> row_pos(Nb, 0);                 // write cursor per column
  int col_pos = 0;
  auto last_col = [&](int age) { return hist_col[((col_pos - 1 - age) % w + w) % w]; };
  auto last_row = [&](int n, int age) {
    return hist_row[size_t(n) * w + ((row_pos[n] - 1 - age) % w + w) % w];
  };
  for (int m = 0; m < Mb; ++m) {
    for (int n = 0; n < Nb; ++n) {
      if (!present[size_t(m) * Nb + n]) continue;
      const int pn = last_col(0);
      const int pm = last_row(n, 0);
      const int up = pm >= 0 ? run[size_t(pm) * Nb + n] : 0;
      const int lf = pn >= 0 ? run[size_t(m) * Nb + pn] : 0;
      const int dg = (pm >= 0 && pn >= 0) ? run[size_t(pm) * Nb + pn] : 0;
      int side = std::min(lf, std::min(up, dg)) + 1;
      // a column strictly between the previous visited column and this one whose
      // latest row is more recent than this column's breaks the square
      for (int c = pn + 1; c < n; ++c)
        if (last_row(c, 0) > pm) side = 1;
      run[size_t(m) * Nb + n] = side;
      hist_col[col_pos % w] = n;
      col_pos = (col_pos + 1) % w + w;  // keep positive, congruent mod w
      hist_row[size_t(n) * w + row_pos[n] % w] = m;
      row_pos[n] = (row_pos[n] + 1) % w + w;
      if (side != w) continue;
      for (int km = 0; km < w; ++km) {
        const int mm = last_row(n, w - 1 - km);
        for (int kn = 0; kn < w; ++kn) {
          const int nn = last_col(w - 1 - kn);
          if (mm < 0 || nn < 0) continue;
          present[size_t(mm) * Nb + nn] = 0;
          run[size_t(mm) * Nb + nn] = 0;
          out.push_back({h, mm, nn, ids[size_t(mm) * Nb + nn]});
        }
      }
    }
  }
}

template <class F>
void parallel_heads(int H, F&& fn) {
  unsigned hw = std::thread::hardware_concurrency();
  int nt = std::max(1, std::min<int>(H, hw ? int(hw) : 1));
  if (nt == 1) { for (int h = 0; h < H; ++h) fn(h); return; }
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; ++t)
    pool.emplace_back([&, t] { for (int h = t; h < H; h += nt) fn(h); });
  for (auto& th : pool) th.join();
}

int check_layout_args(const int64_t* layout, int H, int Mb, int Nb) {
  if (!layout) return fail(BSP_ERR_INVALID, "layout is NULL");
  if (H <= 0 || Mb <= 0 || Nb <= 0) return fail(BSP_ERR_INVALID, "layout shape [%d,%d,%d] is not positive", H, Mb, Nb);
  return BSP_OK;
}

// One column (or row) of the reduction split into segments, following
// matmul.py:233-264 with seg_max = the largest reduction of the head.
struct Segment { int64_t len, column, lockid, maxid; };

int balance(const std::vector<int64_t>& sizes, std::vector<Segment>& segs) {
  int64_t seg_max = 0;
  bool any = false;
  for (int64_t s : sizes) { seg_max = std::max(seg_max, s); any |= (s != 0); }
  if (!any) return BSP_ERR_EMPTY_HEAD;
  const int64_t seg_min = std::max<int64_t>((seg_max + 3) / 4, 4);
  int64_t nlocks = 0;
  for (size_t c = 0; c < sizes.size(); ++c) {
    const int64_t s = sizes[c], d = s / seg_max, r = s % seg_max;
    const bool tiny = s < seg_min;
    const int64_t n = d + (r >= seg_min ? 1 : 0) + (tiny ? 1 : 0);
    const size_t first = segs.size();
    segs.resize(first + n, Segment{0, int64_t(c), 0, 0});
    for (int64_t k = 0; k < d; ++k) segs[first + k].len = seg_max;
    if (r < seg_min && !tiny) segs[first + d - 1].len += r;
    if (r >= seg_min || tiny) segs[first + d].len = r;
    if (d > 1 || (d == 1 && r >= seg_min)) {
      ++nlocks;
      for (int64_t k = 0; k < n; ++k) { segs[first + k].lockid = nlocks; segs[first + k].maxid = n; }
    }
  }
  return BSP_OK;
}

}  // namespace
}  // namespace bsp

using namespace bsp;

extern "C" {

const char* bsp_last_error(void) { return g_err; }

int bsp_abi_version(void) { return 1; }

int bsp_sdd_lut_build(const int64_t* layout, int H, int Mb, int Nb, int block,
                      int32_t* out, int64_t out_cap,
                      int32_t* packs, int64_t* widths, int64_t* offsets,
                      int* n_packs, int64_t* total) {
  if (int rc = check_layout_args(layout, H, Mb, Nb)) return rc;
  if (!valid_block(block)) return fail(BSP_ERR_INVALID, "block must be 16, 32, 64 or 128 (got %d)", block);
  if (!packs || !widths || !offsets || !n_packs || !total) return fail(BSP_ERR_INVALID, "NULL result pointer");
  const size_t per_head = size_t(Mb) * Nb;
  std::vector<uint8_t> present(size_t(H) * per_head);
  std::vector<int32_t> ids(size_t(H) * per_head, 0);
  int32_t next = 0;
  for (size_t p = 0; p < present.size(); ++p) {
    present[p] = layout[p] != 0;
    if (present[p]) ids[p] = next++;
  }
  *n_packs = 0;
  int64_t cursor = 0;
  bool overflow = false;
  for (int w = 64 / block; w > 0; w /= 2) {
    std::vector<std::vector<Entry>> per(H);
    parallel_heads(H, [&](int h) {
      pack_head(h, Mb, Nb, w, present.data() + h * per_head, ids.data() + h * per_head, per[h]);
    });
    int64_t rows = 0;
    for (auto& v : per) rows += int64_t(v.size());
    if (rows == 0) continue;
    if (*n_packs >= BSP_MAX_PACKS) return fail(BSP_ERR_INVALID, "too many pack sizes");
    packs[*n_packs] = w;
    widths[*n_packs] = rows / (int64_t(w) * w);
    offsets[*n_packs] = cursor;
    ++*n_packs;
    if (out && cursor + 4 * rows <= out_cap) {
      int32_t* dst = out + cursor;
      for (auto& v : per)
        for (const Entry& e : v) { *dst++ = e.h; *dst++ = e.i; *dst++ = e.j; *dst++ = e.b; }
    } else if (out) {
      overflow = true;
    }
    cursor += 4 * rows;
  }
  *total = cursor;
  if (overflow) return fail(BSP_ERR_CAPACITY, "SDD table needs %lld ints, buffer holds %lld", (long long)cursor, (long long)out_cap);
  return BSP_OK;
}

int bsp_dxx_lut_build(const int64_t* layout, int H, int Mb, int Nb, int block,
                      int step, int trans,
                      int32_t* out, int64_t out_cap, int64_t* total,
                      int* num_locks, int* width) {
  if (int rc = check_layout_args(layout, H, Mb, Nb)) return rc;
  if (!valid_block(block)) return fail(BSP_ERR_INVALID, "block must be 16, 32, 64 or 128 (got %d)", block);
  if (step <= 0 || block % step) return fail(BSP_ERR_INVALID, "step %d must divide block %d", step, block);
  if (!total || !num_locks || !width) return fail(BSP_ERR_INVALID, "NULL result pointer");
  const int64_t div = block / step;
  const int outer = trans ? Mb : Nb;   // reductions are per block-row (trans) or per block-column
  const int inner = trans ? Nb : Mb;
  auto at = [&](int h, int o, int i) -> bool {
    return trans ? layout[(size_t(h) * Mb + o) * Nb + i] != 0 : layout[(size_t(h) * Mb + i) * Nb + o] != 0;
  };
  // canonical (row-major) block ids
  std::vector<int64_t> head_base(H + 1, 0);
  std::vector<int32_t> ids(size_t(H) * Mb * Nb, -1);
  {
    int32_t next = 0;
    for (int h = 0; h < H; ++h) {
      head_base[h] = next;
      for (size_t p = 0; p < size_t(Mb) * Nb; ++p)
        if (layout[size_t(h) * Mb * Nb + p] != 0) ids[size_t(h) * Mb * Nb + p] = next++;
    }
    head_base[H] = next;
  }
  const int64_t nnz = head_base[H];
  // traversal list: (dense-side index, block id) of every block, head by head,
  // reduction by reduction
  std::vector<int64_t> dense_idx; dense_idx.reserve(nnz);
  std::vector<int64_t> blk_id;    blk_id.reserve(nnz);
  struct Hdr { int64_t off, len, column, depth, lockid, maxid; };
  std::vector<Hdr> hdr;
  int64_t lock_base = 0;
  for (int h = 0; h < H; ++h) {
    std::vector<int64_t> sizes(outer, 0);
    for (int o = 0; o < outer; ++o)
      for (int i = 0; i < inner; ++i)
        if (at(h, o, i)) {
          ++sizes[o];
          dense_idx.push_back(int64_t(i) * block);
          blk_id.push_back(trans ? ids[(size_t(h) * Mb + o) * Nb + i] : ids[(size_t(h) * Mb + i) * Nb + o]);
        }
    std::vector<Segment> segs;
    if (balance(sizes, segs) != BSP_OK)
      return fail(BSP_ERR_EMPTY_HEAD, "head %d of the layout has no nonzero block", h);
    int64_t run = head_base[h], head_lock_max = 0;
    for (const Segment& s : segs) {
      const int64_t lk = s.lockid > 0 ? s.lockid + lock_base : 0;
      head_lock_max = std::max(head_lock_max, lk);
      hdr.push_back({run, s.len, s.column, int64_t(h), lk, s.maxid});
      run += s.len;
    }
    lock_base = head_lock_max;   // running maximum, as matmul.py:391-392
  }
  const int64_t W = int64_t(hdr.size());
  const int64_t need = 6 * W + 2 * nnz * div + 2;
  *total = need;
  *width = int(W);
  int64_t lk_max = 0;
  for (const Hdr& s : hdr) lk_max = std::max(lk_max, s.lockid);
  *num_locks = int(std::max<int64_t>(1, lk_max));
  if (!out) return BSP_OK;
  if (out_cap < need) return fail(BSP_ERR_CAPACITY, "DSD/DDS table needs %lld ints, buffer holds %lld", (long long)need, (long long)out_cap);
  // increments: deltas between consecutive blocks of the traversal, split in
  // `div` sub-steps; the first pair of every non-empty reduction is absolute
  int32_t* pairs = out + 6 * W;
  for (int64_t b = 0; b < nnz; ++b) {
    const int64_t dx = dense_idx[b] - (b ? dense_idx[b - 1] : 0);
    const int64_t dw = (blk_id[b] - (b ? blk_id[b - 1] : 0)) * block * block;
    const int64_t wstep = trans ? step : int64_t(step) * block;
    pairs[2 * (b * div)] = int32_t(dx - (div - 1) * step);
    pairs[2 * (b * div) + 1] = int32_t(dw - (div - 1) * wstep);
    for (int64_t k = 1; k < div; ++k) {
      pairs[2 * (b * div + k)] = int32_t(step);
      pairs[2 * (b * div + k) + 1] = int32_t(wstep);
    }
  }
  pairs[2 * nnz * div] = 0;
  pairs[2 * nnz * div + 1] = 0;
  for (int64_t s = 0; s < W; ++s) {
    const int64_t first = std::min(hdr[s].off, nnz - 1);
    if (hdr[s].len > 0) {
      pairs[2 * (first * div)] = int32_t(dense_idx[first]);
      pairs[2 * (first * div) + 1] = int32_t(blk_id[first]);
    }
    int32_t* hp = out + 6 * s;
    hp[0] = int32_t(first * 2 * div + 6 * W);
    hp[1] = int32_t(hdr[s].len * block);
    hp[2] = int32_t(hdr[s].column);
    hp[3] = int32_t(hdr[s].depth);
    hp[4] = int32_t(hdr[s].lockid);
    hp[5] = int32_t(hdr[s].maxid);
  }
  return BSP_OK;
}

int bsp_softmax_lut_build(const int64_t* layout, int H, int Mb, int Nb,
                          int32_t* out, int64_t out_cap, int64_t* total, int* maxlut) {
  if (int rc = check_layout_args(layout, H, Mb, Nb)) return rc;
  if (!total || !maxlut) return fail(BSP_ERR_INVALID, "NULL result pointer");
  const int64_t rows = int64_t(H) * Mb;
  int64_t nnz = 0;
  int mx = 0;
  for (int64_t r = 0; r < rows; ++r) {
    int s = 0;
    for (int n = 0; n < Nb; ++n) s += layout[r * Nb + n] != 0;
    nnz += s;
    mx = std::max(mx, s);
  }
  *total = 2 * rows + 4 * nnz;
  *maxlut = mx;
  if (!out) return BSP_OK;
  if (out_cap < *total) return fail(BSP_ERR_CAPACITY, "softmax table needs %lld ints, buffer holds %lld", (long long)*total, (long long)out_cap);
  int32_t* core = out + 2 * rows;
  int64_t b = 0;
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t first = b;
    for (int n = 0; n < Nb; ++n)
      if (layout[r * Nb + n] != 0) {
        core[4 * b + 0] = int32_t(b);
        core[4 * b + 1] = int32_t(n);
        core[4 * b + 2] = int32_t(r % Mb);
        core[4 * b + 3] = int32_t(r / Mb);
        ++b;
      }
    out[2 * r] = int32_t(b - first);
    out[2 * r + 1] = int32_t(first * 4 + 2 * rows);
  }
  return BSP_OK;
}

int bsp_fixed_layout_build(int num_heads, int num_blocks, int mode, int block_stride,
                           int unidirectional, int numverts, int vertsize, int64_t* out) {
  if (!out) return fail(BSP_ERR_INVALID, "out is NULL");
  if (num_heads <= 0 || num_blocks <= 0) return fail(BSP_ERR_INVALID, "num_heads and num_blocks must be positive");
  const size_t n = size_t(num_heads) * num_blocks * num_blocks;
  if (mode == 0) { std::fill(out, out + n, int64_t(1)); return BSP_OK; }
  if (mode != 1) return fail(BSP_ERR_UNSUPPORTED, "only \"dense\" and \"fixed\" modes are supported for now");
  if (block_stride <= 0 || vertsize <= 0 || numverts <= 0) return fail(BSP_ERR_INVALID, "stride, numverts and vertsize must be positive");
  if (block_stride % vertsize)
    return fail(BSP_ERR_INVALID, "Number of blocks in a stride window %d must be dividable by vertical block size %d", block_stride, vertsize);
  if (numverts > block_stride / vertsize)
    return fail(BSP_ERR_INVALID, "Number of layout versions %d cannot be larger than blocks in a stride window divided by vertical block size %d / %d", numverts, block_stride, vertsize);
  if (num_blocks % block_stride)
    return fail(BSP_ERR_INVALID, "number of blocks %d must be a multiple of the stride window %d", num_blocks, block_stride);
  std::fill(out, out + n, int64_t(0));
  for (int h = 0; h < num_heads; ++h) {
    int64_t* L = out + size_t(h) * num_blocks * num_blocks;
    // local windows: block-row i sees its own window, up to the diagonal when unidirectional
    for (int i = 0; i < num_blocks; ++i) {
      const int w0 = (i / block_stride) * block_stride;
      const int w1 = unidirectional ? i + 1 : w0 + block_stride;
      for (int j = w0; j < w1; ++j) L[size_t(i) * num_blocks + j] = 1;
    }
    // vertical stripes: the last columns of every window, rotated by head
    const int start = block_stride - (1 + h % numverts) * vertsize;
    for (int i = 0; i < num_blocks; ++i) {
      const int end = unidirectional ? i : num_blocks;
      for (int j = start; j < end; j += block_stride)
        for (int k = j; k < std::min(j + vertsize, num_blocks); ++k) L[size_t(i) * num_blocks + k] = 1;
    }
  }
  return BSP_OK;
}

int bsp_window_layout_build(int num_heads, int num_blocks, int below, int above, int global_rows, int global_cols,
                            const int32_t* random_cols, int num_random, int64_t* out) {
  if (!out) return fail(BSP_ERR_INVALID, "out is NULL");
  if (num_heads <= 0 || num_blocks <= 0) return fail(BSP_ERR_INVALID, "num_heads and num_blocks must be positive");
  if (below < 0 || above < 0 || global_rows < 0 || global_cols < 0 || num_random < 0)
    return fail(BSP_ERR_INVALID, "window, global and random counts must not be negative");
  if (num_random > 0 && !random_cols) return fail(BSP_ERR_INVALID, "random_cols is NULL");
  const size_t nb = size_t(num_blocks);
  for (size_t k = 0; k < size_t(num_heads) * nb * size_t(num_random); ++k)
    if (random_cols[k] < 0 || random_cols[k] >= num_blocks)
      return fail(BSP_ERR_INVALID, "random column %d is outside [0, %d)", int(random_cols[k]), num_blocks);
  parallel_heads(num_heads, [&](int h) {
    int64_t* L = out + size_t(h) * nb * nb;
    for (int i = 0; i < num_blocks; ++i) {
      int64_t* row = L + size_t(i) * nb;
      if (i < global_rows) { std::fill(row, row + nb, int64_t(1)); continue; }
      std::fill(row, row + nb, int64_t(0));
      const int j0 = std::max(0, i - below), j1 = std::min(num_blocks - 1, i + above);
      for (int j = j0; j <= j1; ++j) row[j] = 1;
      for (int j = 0; j < std::min(global_cols, num_blocks); ++j) row[j] = 1;
      const int32_t* rc = random_cols + (size_t(h) * nb + i) * size_t(num_random);
      for (int r = 0; r < num_random; ++r) row[rc[r]] = 1;
    }
  });
  return BSP_OK;
}

int bsp_meta_build(const int64_t* layout, int H, int Mb, int Nb,
                   int32_t* out, int64_t out_cap, int64_t* total) {
  if (int rc = check_layout_args(layout, H, Mb, Nb)) return rc;
  if (!total) return fail(BSP_ERR_INVALID, "NULL result pointer");
  int64_t nnz = 0;
  for (size_t p = 0; p < size_t(H) * Mb * Nb; ++p) nnz += layout[p] != 0;
  *total = meta_total(H, Mb, Nb, nnz);
  if (!out) return BSP_OK;
  if (out_cap < *total) return fail(BSP_ERR_CAPACITY, "metadata needs %lld ints, buffer holds %lld", (long long)*total, (long long)out_cap);
  int32_t* row_ptr = out + BSP_META_HEADER;
  int32_t* blk_row = row_ptr + (H * Mb + 1);
  int32_t* blk_col = blk_row + nnz;
  int32_t* blk_head = blk_col + nnz;
  int32_t* col_ptr = blk_head + nnz;
  int32_t* col_row = col_ptr + (H * Nb + 1);
  int32_t* col_bid = col_row + nnz;
  int32_t* row_order = col_bid + nnz;
  int32_t* col_order = row_order + H * Mb;
  // CSR (canonical order)
  int32_t b = 0;
  int max_row = 0;
  std::vector<int32_t> col_cnt(size_t(H) * Nb, 0);
  for (int h = 0; h < H; ++h)
    for (int m = 0; m < Mb; ++m) {
      row_ptr[h * Mb + m] = b;
      for (int n = 0; n < Nb; ++n)
        if (layout[(size_t(h) * Mb + m) * Nb + n] != 0) {
          blk_row[b] = m; blk_col[b] = n; blk_head[b] = h;
          ++col_cnt[size_t(h) * Nb + n];
          ++b;
        }
      max_row = std::max(max_row, b - row_ptr[h * Mb + m]);
    }
  row_ptr[H * Mb] = b;
  // CSC
  int max_col = 0;
  col_ptr[0] = 0;
  for (int c = 0; c < H * Nb; ++c) {
    col_ptr[c + 1] = col_ptr[c] + col_cnt[c];
    max_col = std::max(max_col, col_cnt[c]);
  }
  std::vector<int32_t> cursor(col_ptr, col_ptr + H * Nb);
  for (int32_t k = 0; k < b; ++k) {
    const int c = blk_head[k] * Nb + blk_col[k];
    col_row[cursor[c]] = blk_row[k];
    col_bid[cursor[c]] = k;
    ++cursor[c];
  }
  // longest-first work orders
  std::iota(row_order, row_order + H * Mb, 0);
  std::stable_sort(row_order, row_order + H * Mb, [&](int32_t x, int32_t y) {
    return row_ptr[x + 1] - row_ptr[x] > row_ptr[y + 1] - row_ptr[y];
  });
  std::iota(col_order, col_order + H * Nb, 0);
  std::stable_sort(col_order, col_order + H * Nb, [&](int32_t x, int32_t y) {
    return col_ptr[x + 1] - col_ptr[x] > col_ptr[y + 1] - col_ptr[y];
  });
  out[0] = BSP_META_MAGIC; out[1] = H; out[2] = Mb; out[3] = Nb; out[4] = int32_t(nnz);
  out[5] = max_row; out[6] = max_col; out[7] = 0;
  return BSP_OK;
}


// Tile lists of the tcgen05 attention kernels.  Those kernels work on tiles of
// 128 query rows (forward, dQ) or 128 key rows (dK / dV), made of two 64-row
// chunks, and walk 64-row chunks of the other operand.  With block 128 a tile
// is one block-row and every nonzero block contributes two chunks.  With block
// 64 a tile is a PAIR of block-rows (block-columns) of one head, not
// necessarily adjacent: the list is the union of their nonzero positions with a
// 2-bit mask saying which half owns the block.  Pairs are chosen greedily by
// similarity of their nonzero sets, since every position only one of the two
// owns is computed for nothing in the other half.
namespace {

struct TileLists {
  std::vector<int32_t> c01, ptr{0}, chunk, mask, sub;   // c01: two outer chunk ids per tile (-1: none)
};

// rows[i] = sorted nonzero positions of block-row (or block-column) i of one head
void pair_blocks(const std::vector<std::vector<int>>& sets, int nb, std::vector<std::pair<int, int>>& pairs) {
  const int words = (nb + 63) / 64;
  std::vector<std::vector<uint64_t>> bits(sets.size(), std::vector<uint64_t>(words, 0));
  for (size_t i = 0; i < sets.size(); ++i)
    for (int j : sets[i]) bits[i][j >> 6] |= uint64_t(1) << (j & 63);
  std::vector<int> order(sets.size());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return sets[x].size() > sets[y].size(); });
  std::vector<char> used(sets.size(), 0);
  for (size_t oi = 0; oi < order.size(); ++oi) {
    const int u = order[oi];
    if (used[u]) continue;
    used[u] = 1;
    int best = -1;
    double best_score = -1.0;
    for (size_t oj = oi + 1; oj < order.size(); ++oj) {
      const int v = order[oj];
      if (used[v]) continue;
      int inter = 0, uni = 0;
      for (int w = 0; w < words; ++w) {
        inter += __builtin_popcountll(bits[u][w] & bits[v][w]);
        uni += __builtin_popcountll(bits[u][w] | bits[v][w]);
      }
      const double score = uni ? double(inter) / uni : 1.0;
      if (score > best_score) { best_score = score; best = v; }
      if (inter == uni) break;                      // cannot do better than identical sets
    }
    if (best >= 0) used[best] = 1;
    pairs.push_back({std::min(u, best < 0 ? u : best), best < 0 ? -1 : std::max(u, best)});
  }
}

// `fine(outer, inner)`: for blocks 16 and 32, which 16 x 16 pieces of the coarse 64 x 64 position
// (outer block of this side, inner block of the other side) lie in a nonzero block of the
// layout: bit 4 a + b for outer group a and inner group b of 16; NULL: all of them.  `sub`
// holds these 16 bits for the first half of the tile in its low half-word and for the second
// half in its high half-word.
void build_lists(const std::vector<std::vector<int>>& sets, int nb, int block, TileLists& out,
                 const std::function<int(int, int)>* fine = nullptr) {
  if (block == 128) {
    for (size_t i = 0; i < sets.size(); ++i) {
      out.c01.push_back(int32_t(2 * i)); out.c01.push_back(int32_t(2 * i + 1));
      for (int j : sets[i]) {
        for (int c = 0; c < 2; ++c) { out.chunk.push_back(2 * j + c); out.mask.push_back(3); out.sub.push_back(-1); }
      }
      out.ptr.push_back(int32_t(out.chunk.size()));
    }
    return;
  }
  std::vector<std::pair<int, int>> pairs;
  pair_blocks(sets, nb, pairs);
  for (auto& pr : pairs) {
    out.c01.push_back(pr.first); out.c01.push_back(pr.second);
    const std::vector<int>& A = sets[pr.first];
    static const std::vector<int> none;
    const std::vector<int>& B = pr.second >= 0 ? sets[pr.second] : none;
    size_t ia = 0, ib = 0;
    while (ia < A.size() || ib < B.size()) {
      const int ja = ia < A.size() ? A[ia] : INT32_MAX, jb = ib < B.size() ? B[ib] : INT32_MAX;
      const int j = std::min(ja, jb);
      int m = 0;
      if (ja == j) { m |= 1; ++ia; }
      if (jb == j) { m |= 2; ++ib; }
      uint32_t sub = ((m & 1) ? 0xFFFFu : 0u) | ((m & 2) ? 0xFFFF0000u : 0u);
      if (fine) sub = uint32_t((m & 1) ? (*fine)(pr.first, j) : 0) | (uint32_t((m & 2) ? (*fine)(pr.second, j) : 0) << 16);
      out.chunk.push_back(j); out.mask.push_back(m); out.sub.push_back(int32_t(sub));
    }
    out.ptr.push_back(int32_t(out.chunk.size()));
  }
}

}  // namespace

int bsp_attn_tiles_build(const int64_t* layout, int H, int nb, int block,
                         int32_t* out, int64_t out_cap, int64_t* total) {
  if (int rc = check_layout_args(layout, H, nb, nb)) return rc;
  if (!total) return fail(BSP_ERR_INVALID, "NULL result pointer");
  if (block != 16 && block != 32 && block != 64 && block != 128)
    return fail(BSP_ERR_UNSUPPORTED, "attention tiles exist for block 16, 32, 64 and 128 (got %d)", block);
  // blocks 16 and 32 are handled as block 64 on the coarsened layout, with the presence of the
  // 16 x 16 pieces of every position in `sub`
  const int fine_nb = nb, fine_block = block, f = block < 64 ? 64 / block : 1;
  if (nb % f) return fail(BSP_ERR_UNSUPPORTED, "attention tiles for block %d need a number of blocks per side that is a multiple of %d (got %d)", block, f, nb);
  if (f > 1) { nb /= f; block = 64; }
  const int nt = block == 128 ? nb : (nb + 1) / 2;   // tiles per head
  std::vector<TileLists> rt(H), ct(H);
  parallel_heads(H, [&](int h) {
    std::vector<std::vector<int>> rows(nb), cols(nb);
    const int64_t* lay = layout + size_t(h) * fine_nb * fine_nb;
    if (f == 1) {
      for (int i = 0; i < nb; ++i)
        for (int j = 0; j < nb; ++j)
          if (lay[size_t(i) * nb + j] != 0) { rows[i].push_back(j); cols[j].push_back(i); }
      build_lists(rows, nb, block, rt[h]);
      build_lists(cols, nb, block, ct[h]);
    } else {
      // 16 bits of a coarse position: piece (a, b) of 16 rows x 16 columns lies in fine block (a * block16, ...)
      auto piece = [&](int i, int j, int a, int b) {   // a, b: groups of 16 inside coarse position (i, j)
        const int fi = (i * 64 + a * 16) / fine_block, fj = (j * 64 + b * 16) / fine_block;
        return lay[size_t(fi) * fine_nb + fj] != 0 ? 1 : 0;
      };
      const std::function<int(int, int)> by_row = [&](int i, int j) {   // outer = query block, inner = key block
        int v = 0;
        for (int a = 0; a < 4; ++a) for (int b = 0; b < 4; ++b) v |= piece(i, j, a, b) << (4 * a + b);
        return v;
      };
      const std::function<int(int, int)> by_col = [&](int j, int i) {   // outer = key block, inner = query block
        int v = 0;
        for (int a = 0; a < 4; ++a) for (int b = 0; b < 4; ++b) v |= piece(i, j, b, a) << (4 * a + b);
        return v;
      };
      for (int i = 0; i < nb; ++i)
        for (int j = 0; j < nb; ++j)
          if (by_row(i, j)) { rows[i].push_back(j); cols[j].push_back(i); }
      build_lists(rows, nb, block, rt[h], &by_row);
      build_lists(cols, nb, block, ct[h], &by_col);
    }
  });
  int64_t er = 0, ec = 0;
  for (int h = 0; h < H; ++h) { er += int64_t(rt[h].chunk.size()); ec += int64_t(ct[h].chunk.size()); }
  const int64_t n = int64_t(H) * nt;
  const int64_t need = BSP_TILES_HEADER + 2 * (2 * n + (n + 1) + n) + 3 * er + 3 * ec;
  *total = need;
  if (!out) return BSP_OK;
  if (out_cap < need) return fail(BSP_ERR_CAPACITY, "attention tile lists need %lld ints, buffer holds %lld", (long long)need, (long long)out_cap);
  int32_t* p = out;
  p[0] = BSP_TILES_MAGIC; p[1] = H; p[2] = nb; p[3] = block; p[4] = nt; p[5] = int32_t(er); p[6] = int32_t(ec); p[7] = fine_block;
  p += BSP_TILES_HEADER;
  auto emit = [&](std::vector<TileLists>& v, int64_t entries) {
    int32_t* c01 = p; p += 2 * n;
    int32_t* ptr = p; p += n + 1;
    int32_t* chunk = p; p += entries;
    int32_t* mask = p; p += entries;
    int32_t* sub = p; p += entries;
    int32_t* order = p; p += n;
    int32_t base = 0;
    ptr[0] = 0;
    for (int h = 0; h < H; ++h) {
      std::copy(v[h].c01.begin(), v[h].c01.end(), c01 + size_t(h) * nt * 2);
      for (int t = 0; t < nt; ++t) ptr[size_t(h) * nt + t + 1] = base + v[h].ptr[t + 1];
      std::copy(v[h].chunk.begin(), v[h].chunk.end(), chunk + base);
      std::copy(v[h].mask.begin(), v[h].mask.end(), mask + base);
      std::copy(v[h].sub.begin(), v[h].sub.end(), sub + base);
      base += int32_t(v[h].chunk.size());
    }
    std::iota(order, order + n, 0);
    std::stable_sort(order, order + n, [&](int32_t x, int32_t y) { return ptr[x + 1] - ptr[x] > ptr[y + 1] - ptr[y]; });
  };
  emit(rt, er);
  emit(ct, ec);
  return BSP_OK;
}

}  // extern "C"
