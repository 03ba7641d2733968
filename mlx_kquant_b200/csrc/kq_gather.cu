// gather_qmm (mixture-of-experts matmul): for every index entry b,
//   y[b] [M, N] = x[lhs[b]] [M, K] . dequant(w[rhs[b]])^T
// replacing KQuantGatherQMM::eval_cpu (src/kquant_gather.cpp:470-746). Like the
// reference, entries are grouped by expert so each expert's wire bytes are
// streamed once per 16 rows instead of once per entry; unlike the reference
// the grouping happens on the device, inside the caller's stream, with no host
// round trip:
//   1. histogram of rhs -> rows per expert
//   2. one-CTA exclusive scan -> entry offsets and task offsets per expert
//   3. scatter of entry ids into expert order
//   4. task build: each expert's c*M rows are cut into GemvTask slices of 16
//   5. the skinny-M kernel runs over (row tile, k-slice, task)
// Prefill-sized calls (on average 16 or more rows per expert) take the tensor-core
// route instead: steps 1-3, then a tile list of 256 sorted rows per entry, an
// expert-sorted fp16 copy of the activations (the tile kernel streams it with TMA),
// and the tcgen05 tile kernel with a row-index scatter in its epilogue.
// All of it lives in a caller-provided workspace laid out by gather_layout().
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "../../include/kquant_b200.h"
#include "kq_common.cuh"
#include "kq_launch.h"

namespace kq {

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Which regime a call takes is decided on the host from sizes alone (no device round trip).
static bool use_grouped(long long n_entries, int M, int n_experts, int K) {
  const long long rows = n_entries * (long long)M;
  return K > 0 && (K % 8) == 0 && rows >= 512 && rows >= 16LL * n_experts && rows < (1LL << 31);
}

GatherLayout gather_layout(long long n_entries, int M, int n_experts, int K) {
  GatherLayout L;
  const long long rows = n_entries * (long long)M;
  // every task but at most one per expert is full, and no task is empty
  long long mt = rows / 16 + (n_entries < n_experts ? n_entries : n_experts);
  if (mt > rows) mt = rows;
  if (mt < 1) mt = 1;
  L.max_tasks = mt;
  L.grouped = use_grouped(n_entries, M, n_experts, K);
  L.max_tiles = rows / kGroupedTileRows + n_experts;
  size_t off = 0;
  L.counts = off;    off = align_up(off + sizeof(int) * (size_t)n_experts, 256);
  L.cursor = off;    off = align_up(off + sizeof(int) * (size_t)n_experts, 256);
  L.offsets = off;   off = align_up(off + sizeof(int) * ((size_t)n_experts + 1), 256);
  L.task_base = off; off = align_up(off + sizeof(int) * ((size_t)n_experts + 1), 256);
  L.n_tasks = off;   off = align_up(off + sizeof(int), 256);
  L.order = off;     off = align_up(off + sizeof(int) * (size_t)(n_entries > 0 ? n_entries : 1), 256);
  L.xh = L.row_scale = L.yrow = L.tiles = 0;
  if (L.grouped) {
    L.tasks = off;  // unused in this regime
    L.tiles = off;     off = align_up(off + 16 * (size_t)L.max_tiles, 256);
    L.yrow = off;      off = align_up(off + sizeof(int) * (size_t)rows, 256);
    L.row_scale = off; off = align_up(off + sizeof(float) * (size_t)rows, 256);
    L.xh = off;        off = align_up(off + 2 * (size_t)rows * (size_t)K, 256);
  } else {
    L.tasks = off;     off = align_up(off + sizeof(GemvTask) * (size_t)mt, 256);
    if (K > 0 && (K % 8) == 0) {
      // room for an fp16 copy of the routed rows: q4_k task lists with bf16 / f32 rows run on the
      // fp16 tensor-core decode kernel (sixteen rows per pass over an expert's weights)
      L.row_scale = off; off = align_up(off + sizeof(float) * (size_t)rows, 256);
      L.xh = off;        off = align_up(off + 2 * (size_t)rows * (size_t)K, 256);
    }
  }
  L.total = off;
  return L;
}

// Entries whose expert index or activation index is out of range take no part (their output rows stay unwritten).
__global__ void gather_hist_kernel(const uint32_t* __restrict__ rhs, const uint32_t* __restrict__ lhs,
                                   long long x_batch, long long n, int n_experts, int* counts) {
  const long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (b < n) {
    const uint32_t e = rhs[b];
    if (e < (uint32_t)n_experts && (lhs == nullptr || (long long)lhs[b] < x_batch)) atomicAdd(&counts[e], 1);
  }
}

// One CTA: exclusive scans of counts (entry offsets) and of ceil(count*M/unit)
// (task or tile offsets; unit = rows per task or tile). n_experts is small (hundreds), a serial chunked scan is enough.
__global__ void gather_scan_kernel(const int* __restrict__ counts, int n_experts, int M, int unit, int* offsets,
                                   int* task_base, int* n_tasks) {
  __shared__ int s_cnt[1024], s_tsk[1024];
  __shared__ int carry_c, carry_t;
  if (threadIdx.x == 0) carry_c = carry_t = 0;
  __syncthreads();
  for (int base = 0; base < n_experts; base += 1024) {
    const int e = base + threadIdx.x;
    const int c = e < n_experts ? counts[e] : 0;
    const int tk = (int)(((long long)c * M + unit - 1) / unit);
    s_cnt[threadIdx.x] = c;
    s_tsk[threadIdx.x] = tk;
    __syncthreads();
    // Hillis-Steele inclusive scan over 1024 slots
    for (int d = 1; d < 1024; d <<= 1) {
      int vc = 0, vt = 0;
      if ((int)threadIdx.x >= d) {
        vc = s_cnt[threadIdx.x - d];
        vt = s_tsk[threadIdx.x - d];
      }
      __syncthreads();
      s_cnt[threadIdx.x] += vc;
      s_tsk[threadIdx.x] += vt;
      __syncthreads();
    }
    if (e < n_experts) {
      offsets[e] = carry_c + s_cnt[threadIdx.x] - c;
      task_base[e] = carry_t + s_tsk[threadIdx.x] - tk;
    }
    __syncthreads();
    if (threadIdx.x == 1023) {
      carry_c += s_cnt[1023];
      carry_t += s_tsk[1023];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    offsets[n_experts] = carry_c;
    task_base[n_experts] = carry_t;
    *n_tasks = carry_t;
  }
}

__global__ void gather_scatter_kernel(const uint32_t* __restrict__ rhs, const uint32_t* __restrict__ lhs,
                                      long long x_batch, long long n, int n_experts, const int* __restrict__ offsets,
                                      int* cursor, int* order) {
  const long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (b < n) {
    const uint32_t e = rhs[b];
    if (e < (uint32_t)n_experts && (lhs == nullptr || (long long)lhs[b] < x_batch))
      order[offsets[e] + atomicAdd(&cursor[e], 1)] = (int)b;
  }
}

// grid.x = expert. The scatter's atomics leave each expert's entries in an
// arbitrary order; that is harmless because an output row depends only on its
// own activation row and the weights, never on which rows share its task.
// entry_order_x != 0: the activations are a copy in entry order (row = entry * M + i), not the caller's x.
__global__ void gather_tasks_kernel(const uint8_t* w, long long expert_stride, int M, const uint32_t* __restrict__ lhs,
                                    const int* __restrict__ offsets, const int* __restrict__ task_base,
                                    const int* __restrict__ order, GemvTask* tasks, int entry_order_x) {
  const int e = blockIdx.x;
  const int o0 = offsets[e], c = offsets[e + 1] - o0;
  if (c == 0) return;
  const long long rows = (long long)c * M;
  const int nt = (int)((rows + 15) / 16);
  const int tb = task_base[e];
  for (int idx = threadIdx.x; idx < nt * 16; idx += blockDim.x) {
    const int tk = idx >> 4, slot = idx & 15;
    GemvTask& t = tasks[tb + tk];
    const long long r = (long long)tk * 16 + slot;
    if (slot == 0) {
      t.w = w + (long long)e * expert_stride;
      t.m = (int)min(16LL, rows - (long long)tk * 16);
      t.pad = 0;
    }
    if (r < rows) {
      const int entry = order[o0 + (int)(r / M)];
      const int i = (int)(r % M);
      t.xrow[slot] = entry_order_x ? entry * M + i : (int)lhs[entry] * M + i;
      t.yrow[slot] = entry * M + i;
    } else {
      t.xrow[slot] = 0;
      t.yrow[slot] = 0;
    }
  }
}

// grid.x = expert: the expert's c*M sorted rows cut into tiles of kGroupedTileRows
struct GatherTile {
  int expert, row_start, rows, pad;
};
__global__ void gather_tiles_kernel(int M, const int* __restrict__ offsets, const int* __restrict__ tile_base,
                                    GatherTile* tiles) {
  const int e = blockIdx.x;
  const long long start = (long long)offsets[e] * M, rows = (long long)(offsets[e + 1] - offsets[e]) * M;
  const int nt = (int)((rows + kGroupedTileRows - 1) / kGroupedTileRows);
  for (int j = threadIdx.x; j < nt; j += blockDim.x) {
    GatherTile t;
    t.expert = e;
    t.row_start = (int)(start + (long long)j * kGroupedTileRows);
    t.rows = (int)min((long long)kGroupedTileRows, rows - (long long)j * kGroupedTileRows);
    t.pad = 0;
    tiles[tile_base[e] + j] = t;
  }
}

// ---------------------------------------------------------------- tile map + segment product
// expert_tile_map (src/kquant_ops.cpp:422-447): rows sorted by expert -> (expert, row_start, num_rows) triples of
// at most 64 rows each and their count. grid.x = expert.
__global__ void tile_map_kernel(const int* __restrict__ offsets, const int* __restrict__ tile_base, uint32_t* map) {
  const int e = blockIdx.x;
  const int start = offsets[e], rows = offsets[e + 1] - offsets[e];
  const int nt = (rows + kSegMapTileRows - 1) / kSegMapTileRows;
  for (int j = threadIdx.x; j < nt; j += blockDim.x) {
    uint32_t* t = map + 3 * (size_t)(tile_base[e] + j);
    t[0] = (uint32_t)e;
    t[1] = (uint32_t)(start + j * kSegMapTileRows);
    t[2] = (uint32_t)min(kSegMapTileRows, rows - j * kSegMapTileRows);
  }
}

// Group n entries by expert on the stream: counts / cursor / offsets / unit_base are n_experts + 1 ints each
// (counts and cursor adjacent, cleared here), order n ints, n_units one int. unit_base[e] = first unit of expert e
// when every expert's entries are cut into units of `unit` entries; *n_units = their total.
cudaError_t launch_group_by_expert(const uint32_t* rhs, long long n, int n_experts, int unit, int* counts, int* cursor,
                                   int* offsets, int* unit_base, int* n_units, int* order, cudaStream_t st) {
  cudaError_t err = cudaMemsetAsync(counts, 0, (size_t)(reinterpret_cast<char*>(cursor) - reinterpret_cast<char*>(counts)) +
                                                   (size_t)(n_experts + 1) * 4, st);
  if (err != cudaSuccess) return err;
  const int th = 256;
  const unsigned nb = (unsigned)((n + th - 1) / th);
  gather_hist_kernel<<<nb, th, 0, st>>>(rhs, nullptr, 0, n, n_experts, counts);
  gather_scan_kernel<<<1, 1024, 0, st>>>(counts, n_experts, 1, unit, offsets, unit_base, n_units);
  gather_scatter_kernel<<<nb, th, 0, st>>>(rhs, nullptr, 0, n, n_experts, offsets, cursor, order);
  return cudaGetLastError();
}

size_t tile_map_workspace_bytes(int n_experts) { return ((size_t)(3 * (n_experts + 1) + 1) * 4 + 255) & ~(size_t)255; }

cudaError_t launch_tile_map(const uint32_t* indices, long long rows, int n_experts, uint32_t* map, uint32_t* count,
                            void* workspace, cudaStream_t st) {
  int* counts = static_cast<int*>(workspace);
  int* offsets = counts + n_experts + 1;
  int* tile_base = offsets + n_experts + 1;
  cudaError_t err = cudaMemsetAsync(counts, 0, (size_t)(n_experts + 1) * 4, st);
  if (err != cudaSuccess) return err;
  const int th = 256;
  gather_hist_kernel<<<(unsigned)((rows + th - 1) / th), th, 0, st>>>(indices, nullptr, 0, rows, n_experts, counts);
  gather_scan_kernel<<<1, 1024, 0, st>>>(counts, n_experts, 1, kSegMapTileRows, offsets, tile_base,
                                         reinterpret_cast<int*>(count));
  tile_map_kernel<<<n_experts, 64, 0, st>>>(offsets, tile_base, map);
  return cudaGetLastError();
}

// gather_qmm_seg (src/kquant_ops.cpp:466-548): the caller's map becomes the tile kernel's list. Maps built by
// expert_tile_map or by the host recipe (mlx_kquant/nn.py:33-47) give every expert ONE run of consecutive rows cut in
// 64-row pieces; such a run is re-cut into tiles of kGroupedTileRows rows, so that a weight tile is dequantized once
// per 256 rows instead of once per 64. A map whose pieces of an expert do not add up to one run is taken piece by
// piece (pieces longer than a tile are split). One CTA; seg = 3 n_experts ints of scratch.
__global__ void __launch_bounds__(1024)
seg_tiles_kernel(const uint32_t* __restrict__ map, const uint32_t* __restrict__ count, int cap, int n_experts,
                 long long rows_total, int* seg, GatherTile* tiles, int max_tiles, int* n_tiles) {
  __shared__ int s_scan[1024];
  __shared__ int irregular, carry, appended;
  int* seg_start = seg;
  int* seg_end = seg + n_experts;
  int* seg_len = seg + 2 * n_experts;
  const int n = (int)min((unsigned)cap, *count);
  if (threadIdx.x == 0) irregular = carry = appended = 0;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    seg_start[e] = 0x7fffffff;
    seg_end[e] = 0;
    seg_len[e] = 0;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < n; t += blockDim.x) {
    const uint32_t e = map[3 * t], r0 = map[3 * t + 1], nr = map[3 * t + 2];
    if (nr == 0 || e >= (uint32_t)n_experts || (long long)r0 + nr > rows_total) continue;  // dead or invalid piece
    atomicMin(&seg_start[e], (int)r0);
    atomicMax(&seg_end[e], (int)(r0 + nr));
    atomicAdd(&seg_len[e], (int)nr);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
    if (seg_len[e] > 0 && seg_end[e] - seg_start[e] != seg_len[e]) irregular = 1;
  __syncthreads();
  if (!irregular) {
    for (int base = 0; base < n_experts; base += 1024) {
      const int e = base + threadIdx.x;
      const int len = e < n_experts ? seg_len[e] : 0;
      const int nt = (len + kGroupedTileRows - 1) / kGroupedTileRows;
      s_scan[threadIdx.x] = nt;
      __syncthreads();
      for (int d = 1; d < 1024; d <<= 1) {
        const int v = (int)threadIdx.x >= d ? s_scan[threadIdx.x - d] : 0;
        __syncthreads();
        s_scan[threadIdx.x] += v;
        __syncthreads();
      }
      const int first = carry + s_scan[threadIdx.x] - nt;
      for (int j = 0; j < nt; j++) {
        if (first + j >= max_tiles) break;
        GatherTile t;
        t.expert = e;
        t.row_start = seg_start[e] + j * kGroupedTileRows;
        t.rows = min(kGroupedTileRows, len - j * kGroupedTileRows);
        t.pad = 0;
        tiles[first + j] = t;
      }
      __syncthreads();
      if (threadIdx.x == 1023) carry += s_scan[1023];
      __syncthreads();
    }
    if (threadIdx.x == 0) *n_tiles = min(carry, max_tiles);
  } else {
    for (int t = threadIdx.x; t < n; t += blockDim.x) {
      const uint32_t e = map[3 * t], r0 = map[3 * t + 1], nr = map[3 * t + 2];
      if (nr == 0 || e >= (uint32_t)n_experts || (long long)r0 + nr > rows_total) continue;
      for (uint32_t off = 0; off < nr; off += kGroupedTileRows) {
        const int slot = atomicAdd(&appended, 1);
        if (slot >= max_tiles) break;
        GatherTile g;
        g.expert = (int)e;
        g.row_start = (int)(r0 + off);
        g.rows = (int)min((uint32_t)kGroupedTileRows, nr - off);
        g.pad = 0;
        tiles[slot] = g;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) *n_tiles = min(appended, max_tiles);
  }
}

static long long seg_max_tiles(long long rows, long long cap) { return cap + rows / kGroupedTileRows + 1; }

size_t gather_seg_workspace_bytes(int x_dtype, long long rows, int K, int n_experts, long long cap) {
  size_t b = ((size_t)(3 * n_experts + 1) * 4 + 255) & ~(size_t)255;                        // seg + n_tiles
  b += ((size_t)seg_max_tiles(rows, cap) * sizeof(GatherTile) + 255) & ~(size_t)255;        // tiles
  if (x_dtype != F16) {
    b += ((size_t)rows * (size_t)K * 2 + 255) & ~(size_t)255;                               // fp16 copy of x
    b += ((size_t)rows * 4 + 255) & ~(size_t)255;                                           // row factors
  }
  return b;
}

cudaError_t launch_gather_seg(int codec, int x_dtype, const void* x, long long rows, int K, const uint8_t* w,
                              int n_experts, long long expert_stride, long long row_bytes, int N, const uint32_t* map,
                              const uint32_t* count, long long cap, void* y, void* workspace, cudaStream_t st) {
  if (rows <= 0 || N <= 0) return cudaSuccess;
  if (rows >= (1LL << 31)) return cudaErrorInvalidValue;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* seg = reinterpret_cast<int*>(ws);
  int* n_tiles = seg + 3 * n_experts;
  size_t off = ((size_t)(3 * n_experts + 1) * 4 + 255) & ~(size_t)255;
  GatherTile* tiles = reinterpret_cast<GatherTile*>(ws + off);
  const long long max_tiles = seg_max_tiles(rows, cap);
  if (max_tiles > 65535) return cudaErrorInvalidConfiguration;
  off += ((size_t)max_tiles * sizeof(GatherTile) + 255) & ~(size_t)255;
  seg_tiles_kernel<<<1, 1024, 0, st>>>(map, count, (int)cap, n_experts, rows, seg, tiles, (int)max_tiles, n_tiles);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  const void* xh = x;
  const float* rs = nullptr;
  if (x_dtype != F16) {
    void* xc = ws + off;
    off += ((size_t)rows * (size_t)K * 2 + 255) & ~(size_t)255;
    float* rsw = reinterpret_cast<float*>(ws + off);
    if ((err = launch_convert_rows(x_dtype, x, K, K, rows, nullptr, 1, xc, rsw, st)) != cudaSuccess) return err;
    xh = xc;
    rs = rsw;
  }
  return launch_gemm_tiles(codec, x_dtype == F16, xh, rows, K, w, expert_stride, row_bytes, N, y, rs, nullptr, tiles,
                           n_tiles, (int)max_tiles, st);
}

cudaError_t launch_gather(int codec, int x_dtype, const void* x, long long x_batch, int M, int K, const uint8_t* w,
                          int n_experts,
                          long long expert_stride, long long row_bytes, int N, const uint32_t* lhs,
                          const uint32_t* rhs, long long n_entries, void* y, void* workspace, bool allow_grouped,
                          cudaStream_t st) {
  if (n_entries <= 0 || M <= 0) return cudaSuccess;
  const GatherLayout L = gather_layout(n_entries, M, n_experts, allow_grouped ? K : 0);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* counts = reinterpret_cast<int*>(ws + L.counts);
  int* cursor = reinterpret_cast<int*>(ws + L.cursor);
  int* offsets = reinterpret_cast<int*>(ws + L.offsets);
  int* task_base = reinterpret_cast<int*>(ws + L.task_base);
  int* n_tasks = reinterpret_cast<int*>(ws + L.n_tasks);
  int* order = reinterpret_cast<int*>(ws + L.order);

  cudaError_t err = cudaMemsetAsync(ws + L.counts, 0, L.offsets - L.counts, st);  // counts + cursor
  if (err != cudaSuccess) return err;
  const int th = 256;
  const unsigned nb = (unsigned)((n_entries + th - 1) / th);
  gather_hist_kernel<<<nb, th, 0, st>>>(rhs, lhs, x_batch, n_entries, n_experts, counts);
  gather_scan_kernel<<<1, 1024, 0, st>>>(counts, n_experts, M, L.grouped ? kGroupedTileRows : 16, offsets, task_base,
                                         n_tasks);
  gather_scatter_kernel<<<nb, th, 0, st>>>(rhs, lhs, x_batch, n_entries, n_experts, offsets, cursor, order);

  if (L.grouped) {
    GatherTile* tiles = reinterpret_cast<GatherTile*>(ws + L.tiles);
    gather_tiles_kernel<<<n_experts, 64, 0, st>>>(M, offsets, task_base, tiles);
    if ((err = cudaGetLastError()) != cudaSuccess) return err;
    if (L.max_tiles > 65535) return cudaErrorInvalidConfiguration;
    return launch_gemm_grouped(codec, x_dtype, x, M, K, w, expert_stride, row_bytes, N, lhs, order,
                               n_entries * (long long)M, y, reinterpret_cast<__half*>(ws + L.xh),
                               reinterpret_cast<float*>(ws + L.row_scale), reinterpret_cast<int*>(ws + L.yrow), tiles,
                               n_tasks, (int)L.max_tiles, offsets + n_experts, st);
  }

  GemvTask* tasks = reinterpret_cast<GemvTask*>(ws + L.tasks);
  const bool w16 = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (expert_stride & 15) == 0;
  // q4_k with bf16 / f32 rows: exact fp16 copy of the routed rows (per-row power-of-two factor), then the
  // fp16 tensor-core decode kernel, which writes bf16(sum * factor). Measured 2-4x faster than the paths
  // that take bf16 rows directly.
  const bool to_half = codec == Q4_K && x_dtype != F16 && w16 && L.xh != 0 && (row_bytes & 15) == 0;
  gather_tasks_kernel<<<n_experts, 256, 0, st>>>(w, expert_stride, M, lhs, offsets, task_base, order, tasks,
                                                 to_half ? 1 : 0);
  if ((err = cudaGetLastError()) != cudaSuccess) return err;

  GemvArgs a{};
  a.x = x;
  if (to_half) {
    __half* xh = reinterpret_cast<__half*>(ws + L.xh);
    float* rs = reinterpret_cast<float*>(ws + L.row_scale);
    if ((err = launch_convert_rows(x_dtype, x, K, K, n_entries * (long long)M, lhs, M, xh, rs, st)) != cudaSuccess)
      return err;
    a.x = xh;
    a.out_bf16 = 1;
    a.row_scale = rs;
    x_dtype = F16;
  }
  a.avg_rows = (int)((n_entries * (long long)M + n_experts - 1) / n_experts);
  a.x_row_stride = K;
  a.y = y;
  a.y_row_stride = N;
  a.w = w;
  a.w_align16 = w16 ? 1 : 0;
  a.row_bytes = row_bytes;
  a.N = N;
  a.K = K;
  a.M = 0;
  a.n_tasks_dev = n_tasks;
  a.max_m = (int)(n_entries * M < 16 ? n_entries * M : 16);
  // grid.z is capped at 65535: cover the task list in slices
  for (long long t0 = 0; t0 < L.max_tasks; t0 += 65535) {
    a.tasks = tasks + t0;
    a.n_tasks = (int)((L.max_tasks - t0) < 65535 ? (L.max_tasks - t0) : 65535);
    a.task_offset = (int)t0;
    if ((err = launch_gemv(codec, x_dtype, a, st)) != cudaSuccess) return err;
  }
  return cudaSuccess;
}


// ---------------------------------------------------------------- a whole SwiGLU block on the tile kernel
// The composition gather_qmm(gate | up) -> silu * up -> gather_qmm(down) -> weighted sum groups the same
// entries twice, scatters the first product back to entry order only to gather it again, and makes two
// elementwise passes in between. Here the routed rows are grouped once, the gate | up product stays in
// expert order, the activation is computed inside the fp16 pre-pass of the down product (with the same
// roundings as the separate kernels, so the two forms give the same bits), and only the down product is
// scattered back to entry order for the per-token sum.
namespace {
struct MoeBlockLayout {
  size_t counts, cursor, offsets, tile_base, n_tiles, order, tiles, yrow, scale1, scale2, xh, gu, hh, total;
  long long max_tiles;
};
MoeBlockLayout moe_block_layout(long long T, int k, int E, int H, int F) {
  MoeBlockLayout L;
  const size_t rows = (size_t)(T * k);
  L.max_tiles = (long long)rows / kGroupedTileRows + E;
  size_t off = 0;
  L.counts = off;    off = align_up(off + 4 * (size_t)E, 256);
  L.cursor = off;    off = align_up(off + 4 * (size_t)E, 256);
  L.offsets = off;   off = align_up(off + 4 * ((size_t)E + 1), 256);
  L.tile_base = off; off = align_up(off + 4 * ((size_t)E + 1), 256);
  L.n_tiles = off;   off = align_up(off + 4, 256);
  L.order = off;     off = align_up(off + 4 * rows, 256);
  L.tiles = off;     off = align_up(off + 16 * (size_t)L.max_tiles, 256);
  L.yrow = off;      off = align_up(off + 4 * rows, 256);
  L.scale1 = off;    off = align_up(off + 4 * rows, 256);
  L.scale2 = off;    off = align_up(off + 4 * rows, 256);
  L.xh = off;        off = align_up(off + 2 * rows * (size_t)H, 256);  // later the down product in entry order
  L.gu = off;        off = align_up(off + 4 * rows * (size_t)F, 256);
  L.hh = off;        off = align_up(off + 2 * rows * (size_t)F, 256);
  L.total = off;
  return L;
}
}  // namespace

bool moe_block_supported(int x_dtype, long long T, int k, int n_experts, int H, int F) {
  if (x_dtype != F16 && x_dtype != BF16) return false;
  if (T <= 0 || k <= 0 || n_experts <= 0 || H <= 0 || F <= 0 || (H % 8) != 0 || (F % 8) != 0) return false;
  if (T > (long long)INT32_MAX / k) return false;
  if (!use_grouped(T * k, 1, n_experts, H)) return false;
  return T * k / kGroupedTileRows + n_experts <= 65535;
}

size_t moe_block_workspace_bytes(long long T, int k, int n_experts, int H, int F) {
  return moe_block_supported(F16, T, k, n_experts, H, F) ? moe_block_layout(T, k, n_experts, H, F).total : 0;
}

cudaError_t launch_moe_block(int codec, int x_dtype, const void* x, long long x_row_stride, const uint32_t* token_rows,
                             long long T, int H, const uint8_t* wgu, long long stride_gu, long long rb_h, int F,
                             const uint8_t* wd, long long stride_d, long long rb_f, int n_experts, const uint32_t* idx,
                             const float* scores, int k, void* y, bool y_f32, void* workspace, cudaStream_t st,
                             const MoeScatter* scatter) {
  if (!moe_block_supported(x_dtype, T, k, n_experts, H, F)) return cudaErrorInvalidValue;
  const MoeBlockLayout L = moe_block_layout(T, k, n_experts, H, F);
  const long long n = T * k;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* counts = reinterpret_cast<int*>(ws + L.counts);
  int* cursor = reinterpret_cast<int*>(ws + L.cursor);
  int* offsets = reinterpret_cast<int*>(ws + L.offsets);
  int* tile_base = reinterpret_cast<int*>(ws + L.tile_base);
  int* n_tiles = reinterpret_cast<int*>(ws + L.n_tiles);
  int* order = reinterpret_cast<int*>(ws + L.order);
  GatherTile* tiles = reinterpret_cast<GatherTile*>(ws + L.tiles);
  int* yrow = reinterpret_cast<int*>(ws + L.yrow);
  float* scale1 = reinterpret_cast<float*>(ws + L.scale1);
  float* scale2 = reinterpret_cast<float*>(ws + L.scale2);
  __half* xh = reinterpret_cast<__half*>(ws + L.xh);
  void* gu = ws + L.gu;
  __half* hh = reinterpret_cast<__half*>(ws + L.hh);
  void* d = ws + L.xh;  // the sorted copy of x is dead once the gate | up product has run

  cudaError_t err = cudaMemsetAsync(ws + L.counts, 0, L.offsets - L.counts, st);
  if (err != cudaSuccess) return err;
  const int th = 256;
  const unsigned nb = (unsigned)((n + th - 1) / th);
  gather_hist_kernel<<<nb, th, 0, st>>>(idx, nullptr, 0, n, n_experts, counts);
  gather_scan_kernel<<<1, 1024, 0, st>>>(counts, n_experts, 1, kGroupedTileRows, offsets, tile_base, n_tiles);
  gather_scatter_kernel<<<nb, th, 0, st>>>(idx, nullptr, 0, n, n_experts, offsets, cursor, order);
  gather_tiles_kernel<<<n_experts, 64, 0, st>>>(1, offsets, tile_base, tiles);
  if ((err = cudaGetLastError()) != cudaSuccess) return err;
  const int* n_valid = offsets + n_experts;  // entries whose expert is in range: the sorted rows that exist
  const bool half = x_dtype == F16;
  // routed rows in expert order (token of entry b = b / k), yrow[r] = entry of sorted row r
  if ((err = launch_convert(x_dtype, x, x_row_stride, H, n, order, token_rows, k, 1, xh, scale1, yrow, n_valid, false,
                            st)) != cudaSuccess)
    return err;
  if ((err = launch_gemm_tiles(codec, half, xh, n, H, wgu, stride_gu, rb_h, 2 * F, gu, half ? nullptr : scale1, nullptr,
                               tiles, n_tiles, (int)L.max_tiles, st)) != cudaSuccess)
    return err;
  if ((err = launch_convert(x_dtype, gu, 2LL * F, F, n, nullptr, nullptr, 1, 1, hh, scale2, nullptr, n_valid, true, st)) !=
      cudaSuccess)
    return err;
  if ((err = launch_gemm_tiles(codec, half, hh, n, F, wd, stride_d, rb_f, H, d, half ? nullptr : scale2, yrow, tiles,
                               n_tiles, (int)L.max_tiles, st)) != cudaSuccess)
    return err;
  if (scatter != nullptr)
    return launch_moe_combine_scatter(x_dtype, d, scores, idx, (uint32_t)n_experts, T, k, H, scatter->tokens_per_rank,
                                      scatter->my_rank, scatter->slots, scatter->slot_f32, st);
  return launch_moe_combine(x_dtype, d, scores, T, k, H, y, y_f32, st, idx, (uint32_t)n_experts);
}

}  // namespace kq

// ---- gather_qmm for callers that may not allocate ---------------------------
// The grouping scratch of launch_gather(), as a fixed array inside the library
// image: every GPU that loads the library carries these bytes until the
// process exits, whether or not this entry point is ever called.
static __device__ __align__(256) unsigned char g_gather_static_ws[KQ_GATHER_STATIC_WS_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_ws_mutex;
void* g_static_ws_addr[kMaxDevices] = {};

// Device address of g_gather_static_ws on the CURRENT device. The symbol name is
// only a host-side handle: handing it to a kernel would pass a host address, so
// the real address is asked for once per device and remembered.
cudaError_t static_ws_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_ws_mutex);
  if (g_static_ws_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_gather_static_ws);
    if (e != cudaSuccess) return e;
    g_static_ws_addr[dev] = p;
  }
  *out = g_static_ws_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int kq_gather_qmm_noalloc(const void* x, int x_dtype, long long x_batch, int M, int K, const void* w,
                                     int n_experts, long long w_expert_stride_bytes, size_t w_row_bytes, int N,
                                     const char* kquant_type, const uint32_t* lhs_indices,
                                     const uint32_t* rhs_indices, long long n_entries, int transpose, int rhs_sorted,
                                     void* y, void* stream) {
  void* ws = nullptr;
  const cudaError_t e = static_ws_address(&ws);
  if (e != cudaSuccess) {
    char msg[256];
    std::snprintf(msg, sizeof(msg), "[mlx_kquant] gather_qmm: cannot resolve the built-in scratch: %s",
                  cudaGetErrorString(e));
    return kq::set_error(KQ_ERR_CUDA, msg);
  }
  // From here on it is the ordinary path (argument checks first, then the size limit of the fixed array for
  // the orientation that needs scratch; it clears the counters it needs on the stream). This entry point
  // always takes the decode regime (the skinny kernel over task lists).
  return kq::gather_qmm_entry(x, x_dtype, x_batch, M, K, w, n_experts, w_expert_stride_bytes, w_row_bytes, N,
                              kquant_type, lhs_indices, rhs_indices, n_entries, transpose, rhs_sorted, y, ws,
                              KQ_GATHER_STATIC_WS_BYTES, stream, /*allow_grouped=*/false, /*builtin_scratch=*/true);
}

