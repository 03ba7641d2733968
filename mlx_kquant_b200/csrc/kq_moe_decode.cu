// Fused mixture-of-experts decode kernels for q4_k expert stacks (the B200 counterparts of the reference's
// Metal-only ops moe_glu_gather_kq, gather_qmv_mix_ns_kq and moe_router_topk, src/kquant.h:335-357, 549-558,
// 560-585), for calls of a few tokens where every routed (token, expert) entry streams its own expert's rows:
//
//   moe_glu_kernel     h[entry, f] = act(x[token] . Wg[e][f]) * (x[token] . Wu[e][f])
//                      grid (F / 16, entries): one CTA multiplies 16 gate rows and the 16 up rows of the same
//                      features by one activation row (the two 16-row fragments share every activation
//                      fragment) and applies the activation before its single rounding.
//   moe_mix_kernel     y[token, n] = sum_s score[token, s] * (h[token, s] . Wd[e_s][n])
//                      grid (N / 16, tokens): warp w owns slot s = w, w + 8, ...: it quantizes that slot's
//                      activation row, multiplies the slot's expert rows, and the score-weighted float32 sum
//                      over the slots is taken in slot order before the single rounding.
//   router_topk_kernel one warp per token, the E scores in registers, top_k rounds of a warp arg-max with the
//                      lowest index winning ties.
//
// Both product kernels start their weight copies before griddepcontrol.wait, from the expert indices as they
// are in memory then; after the wait the indices are read again and a CTA whose expert changed copies again
// (its first copy has landed by then). The activations are only read after the wait.
// Arithmetic and shared-memory layout of the products: kq_imma_q4k.cuh / kq_gemv_stream.cu.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_imma_q4k.cuh"
#include "kq_launch.h"

namespace kq {

namespace {

constexpr int kMdWarps = 8, kMdThreads = 32 * kMdWarps;

inline int md_group_stride(long long row_bytes) {
  const long long gb = 4 * row_bytes;
  return (int)(gb + ((32 - (gb & 127)) & 127));
}

__device__ __forceinline__ uint32_t md_ld_cg32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// bounded wait for a bulk-copy barrier; false (and a raised flag) after two seconds
__device__ __forceinline__ bool md_wait(uint64_t* bar, uint32_t parity, int* error_word) {
  if (st_mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = st_gtime();
  for (int spin = 0; !st_mbar_try_wait(bar, parity); spin++) {
    if ((spin & 63) == 63 && st_gtime() - t0 > 2000000000ull) {
      atomicOr(error_word, 0x100);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ float md_act(float g, float u, int act, float limit) {
  if (act == 1) {  // tanh-approximated gelu
    const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return (0.5f * g * (1.0f + t)) * u;
  }
  if (act == 2) {  // limited SwiGLU: gate clamped from above, up clamped on both sides
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return (g / (1.0f + expf(-g))) * u;
}

template <typename T>
__device__ __forceinline__ void md_store(T* p, float v) {
  if constexpr (std::is_same<T, __half>::value) *p = __float2half_rn(v);
  else *p = __float2bfloat16_rn(v);
}

// copies of up to 16 rows of one matrix in groups of four (group i at dst + i * GS)
__device__ __forceinline__ void md_copy_tile(uint8_t* dst, const uint8_t* src, int rows, int RB, int GS, uint64_t* bar) {
  for (int r = 0; r < rows; r += 4) st_bulk_g2s(dst + (r >> 2) * GS, src + (long long)r * RB, (uint32_t)(min(4, rows - r) * RB), bar);
}

struct GluArgs {
  const void* x;            // [T, K]
  const uint8_t* wg;
  const uint8_t* wu;
  long long stride_g, stride_u;
  int row_bytes, K, F, R, n_entries, n_experts;
  const uint32_t* idx;      // [T * R]
  void* y;                  // [T * R, F]
  int act;
  float limit;
  int tiles_per_cta;        // grouped kernel only: consecutive 16-feature tiles a CTA walks
};

// shared memory: gate tile | up tile (4 groups each) | planes 2 K | XS K / 32 | SX K / 256 (padded) | red 8 x 32 | mbar
inline int glu_smem_bytes(int K, int row_bytes) {
  return 8 * md_group_stride(row_bytes) + 2 * K + (K / 32) * 4 + (((K / 256) + 3) & ~3) * 4 + kMdWarps * 32 * 4 + 16;
}

template <typename XT>
__global__ void __launch_bounds__(kMdThreads, 3) moe_glu_kernel(const GluArgs a, int* __restrict__ error_word) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  extern __shared__ __align__(128) uint8_t md_dyn[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, nchunks = K >> 8, RB = a.row_bytes;
  const int gb = 4 * RB, GS = gb + ((32 - (gb & 127)) & 127);
  uint8_t* wbuf = md_dyn;
  uint8_t* planes = wbuf + 8 * GS;
  float* XS = reinterpret_cast<float*>(planes + 2 * K);
  float* SX = XS + (K / 32);
  float* red = SX + ((nchunks + 3) & ~3);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + kMdWarps * 32);
  const int entry = blockIdx.y, f0 = blockIdx.x * 16;
  const int rows = min(16, a.F - f0);
  __shared__ int s_parity;

  // expert as it is now; the copies start before the preceding kernel has finished
  const uint32_t e0 = md_ld_cg32(a.idx + entry);
  const bool v0 = e0 < (uint32_t)a.n_experts;
  auto issue = [&](uint32_t e) {
    st_mbar_expect_tx(mbar, (uint32_t)(2 * rows * RB));
    md_copy_tile(wbuf, a.wg + (long long)e * a.stride_g + (long long)f0 * RB, rows, RB, GS, mbar);
    md_copy_tile(wbuf + 4 * GS, a.wu + (long long)e * a.stride_u + (long long)f0 * RB, rows, RB, GS, mbar);
  };
  if (threadIdx.x == 0) {
    st_mbar_init(mbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (v0) issue(e0);
  }
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const uint32_t e = md_ld_cg32(a.idx + entry);
  const bool valid = e < (uint32_t)a.n_experts;
  if (threadIdx.x == 0) {
    int parity = 0;
    bool ok = true;
    if (v0 && e != e0) {  // the first copy must land before its buffer is reused or the CTA leaves
      ok = md_wait(mbar, 0, error_word);
      parity = 1;
      if (valid && ok) issue(e);
    } else if (!v0 && valid) {
      issue(e);
    }
    s_parity = ok ? parity : -1;
  }
  __syncthreads();
  const int parity = s_parity;
  if (!valid || parity < 0) return;

  const XT* x = static_cast<const XT*>(a.x) + (long long)(entry / a.R) * K;
  for (int sb = warp; sb < nchunks; sb += kMdWarps)
    st_quantize<XT>(st_ld_cg16(x + sb * 256 + lane * 8), sb, lane, K, planes, XS, SX);
  __syncwarp();
  if (!md_wait(mbar, (uint32_t)parity, error_word)) return;

  const uint8_t* bplane = planes + min(g, 1) * K + 8 * t;
  const int lrA = min(4 * (g & 3) + (g >> 2), rows - 1), lrB = min(4 * (g & 3) + (g >> 2) + 2, rows - 1);
  const uint8_t* base[4] = {wbuf + (lrA >> 2) * GS + (lrA & 3) * RB, wbuf + (lrB >> 2) * GS + (lrB & 3) * RB,
                            wbuf + (4 + (lrA >> 2)) * GS + (lrA & 3) * RB, wbuf + (4 + (lrB >> 2)) * GS + (lrB & 3) * RB};
  float y4[4] = {0.f, 0.f, 0.f, 0.f};
  for (int sb = warp; sb < nchunks; sb += kMdWarps) {
    const uint8_t* const blk[4] = {base[0] + sb * 144, base[1] + sb * 144, base[2] + sb * 144, base[3] + sb * 144};
    st_unit<2>(blk, bplane + sb * 256, XS + sb * 8, SX[sb], t, y4);
  }
#pragma unroll
  for (int r = 0; r < 4; r++) {
    y4[r] += __shfl_xor_sync(0xffffffffu, y4[r], 1);
    y4[r] += __shfl_xor_sync(0xffffffffu, y4[r], 2);
  }
  if (t == 0) {
    const int rA = 4 * (g & 3) + (g >> 2), rB = rA + 2;   // unclamped: rows past the tile are never read back
    red[warp * 32 + rA] = y4[0];
    red[warp * 32 + rB] = y4[1];
    red[warp * 32 + 16 + rA] = y4[2];
    red[warp * 32 + 16 + rB] = y4[3];
  }
  __syncthreads();
  if (threadIdx.x < rows) {
    float gs = 0.f, us = 0.f;
#pragma unroll
    for (int w = 0; w < kMdWarps; w++) {
      gs += red[w * 32 + threadIdx.x];
      us += red[w * 32 + 16 + threadIdx.x];
    }
    md_store(static_cast<XT*>(a.y) + (long long)entry * a.F + f0 + threadIdx.x, md_act(gs, us, a.act, a.limit));
  }
}

struct MixArgs {
  const void* x;            // [T * S, K]
  const uint8_t* w;
  long long stride_w;
  int row_bytes, K, N, S, n_experts;
  const uint32_t* idx;      // [T * S]
  const float* scores;      // [T * S]
  void* y;                  // [T, N]
};

// shared memory per warp: one 16-row tile (4 groups) | planes 2 K | XS | SX; then red 8 x 16 | 8 mbarriers
inline int mix_warp_bytes(int K, int row_bytes) {
  return 4 * md_group_stride(row_bytes) + 2 * K + (K / 32) * 4 + (((K / 256) + 3) & ~3) * 4;
}
inline int mix_smem_bytes(int K, int row_bytes) { return kMdWarps * mix_warp_bytes(K, row_bytes) + kMdWarps * 16 * 4 + kMdWarps * 8; }

template <typename XT>
__global__ void __launch_bounds__(kMdThreads, 2) moe_mix_kernel(const MixArgs a, int* __restrict__ error_word) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  extern __shared__ __align__(128) uint8_t md_dyn[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, nchunks = K >> 8, RB = a.row_bytes;
  const int gb = 4 * RB, GS = gb + ((32 - (gb & 127)) & 127);
  const int wbytes = 4 * GS + 2 * K + (K / 32) * 4 + ((nchunks + 3) & ~3) * 4;
  uint8_t* wbuf = md_dyn + warp * wbytes;
  uint8_t* planes = wbuf + 4 * GS;
  float* XS = reinterpret_cast<float*>(planes + 2 * K);
  float* SX = XS + (K / 32);
  float* red = reinterpret_cast<float*>(md_dyn + kMdWarps * wbytes);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + kMdWarps * 16) + warp;
  const int token = blockIdx.y, n0 = blockIdx.x * 16;
  const int rows = min(16, a.N - n0);
  const int lrA = min(4 * (g & 3) + (g >> 2), rows - 1), lrB = min(4 * (g & 3) + (g >> 2) + 2, rows - 1);
  const uint8_t* bplane = planes + min(g, 1) * K + 8 * t;
  const long long slot0 = (long long)token * a.S;

  auto issue = [&](uint32_t e) {
    st_mbar_expect_tx(mbar, (uint32_t)(rows * RB));
    md_copy_tile(wbuf, a.w + (long long)e * a.stride_w + (long long)n0 * RB, rows, RB, GS, mbar);
  };
  // first slot of this warp: its copy starts before the preceding kernel has finished
  uint32_t e0 = 0xffffffffu;
  if (warp < a.S) e0 = md_ld_cg32(a.idx + slot0 + warp);
  bool v0 = e0 < (uint32_t)a.n_experts;
  if (lane == 0) {
    st_mbar_init(mbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (v0) issue(e0);
  }
  __syncwarp();
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

  float yA = 0.f, yB = 0.f;   // score-weighted sums of this warp's slots (rows lrA, lrB), complete in lanes t = 0
  uint32_t parity = 0;
  bool dead = false;
  for (int s = warp; s < a.S; s += kMdWarps) {
    const uint32_t e = md_ld_cg32(a.idx + slot0 + s);
    const bool valid = e < (uint32_t)a.n_experts;
    // copies: the first slot's may already be in flight for another expert
    if (lane == 0) {
      bool ok = true;
      if (s == warp) {
        if (v0 && e != e0) {
          ok = md_wait(mbar, 0, error_word);
          if (ok && valid) issue(e);
        } else if (!v0 && valid) {
          issue(e);
        }
      } else if (valid) {
        issue(e);
      }
      if (!ok) atomicOr(error_word, 0x100);
    }
    if (s == warp && v0 && e != e0) parity ^= 1;
    __syncwarp();
    if (valid) {
      const XT* x = static_cast<const XT*>(a.x) + (slot0 + s) * K;
      for (int sb = 0; sb < nchunks; sb++)
        st_quantize<XT>(st_ld_cg16(x + sb * 256 + lane * 8), sb, lane, K, planes, XS, SX);
      __syncwarp();
      if (!md_wait(mbar, parity, error_word)) {
        dead = true;
        break;
      }
      parity ^= 1;
      const uint8_t* pA = wbuf + (lrA >> 2) * GS + (lrA & 3) * RB;
      const uint8_t* pB = wbuf + (lrB >> 2) * GS + (lrB & 3) * RB;
      float y2[2] = {0.f, 0.f};
      for (int sb = 0; sb < nchunks; sb++) {
        const uint8_t* const blk[2] = {pA + sb * 144, pB + sb * 144};
        st_unit<1>(blk, bplane + sb * 256, XS + sb * 8, SX[sb], t, y2);
      }
      const float sc = a.scores[slot0 + s];
      yA = fmaf(sc, y2[0], yA);
      yB = fmaf(sc, y2[1], yB);
      __syncwarp();   // the tile and the planes are free for the next slot
    }
  }
  yA += __shfl_xor_sync(0xffffffffu, yA, 1);
  yA += __shfl_xor_sync(0xffffffffu, yA, 2);
  yB += __shfl_xor_sync(0xffffffffu, yB, 1);
  yB += __shfl_xor_sync(0xffffffffu, yB, 2);
  if (t == 0) {
    const int rA = 4 * (g & 3) + (g >> 2);
    red[warp * 16 + rA] = yA;
    red[warp * 16 + rA + 2] = yB;
  }
  (void)dead;   // every copy that was started has been waited for above (the stale one by lane 0)
  __syncthreads();
  if (threadIdx.x < rows) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kMdWarps; w++) sum += red[w * 16 + threadIdx.x];
    md_store(static_cast<XT*>(a.y) + (long long)token * a.N + n0 + threadIdx.x, sum);
  }
}

// ---------------------------------------------------------------------------------- grouped by expert
// From a few dozen routed entries on, entries that share an expert share its weight stream: the entries are
// grouped by expert on the device (kq_gather.cu) and cut into tasks of at most kTaskEntries entries. A CTA brings
// its rows of the task's expert into shared memory once and multiplies them by the task's activation rows four
// at a time (the B operand has room for four rows' byte planes).
constexpr int kTaskEntries = 16;
struct Task4 {
  int expert, m;
  int ent[kTaskEntries];   // entry indices; slots past m repeat the last one
};

__global__ void moe_tasks4_kernel(const int* __restrict__ offsets, const int* __restrict__ task_base,
                                  const int* __restrict__ order, Task4* tasks) {
  const int e = blockIdx.x;
  const int o0 = offsets[e], c = offsets[e + 1] - o0;
  const int nt = (c + kTaskEntries - 1) / kTaskEntries, tb = task_base[e];
  for (int k = threadIdx.x; k < nt; k += blockDim.x) {
    Task4 t;
    t.expert = e;
    t.m = min(kTaskEntries, c - kTaskEntries * k);
#pragma unroll
    for (int j = 0; j < kTaskEntries; j++) t.ent[j] = order[o0 + kTaskEntries * k + min(j, t.m - 1)];
    tasks[tb + k] = t;
  }
}

__device__ __forceinline__ float md_pick4(const float (&v)[4], int t) {
  return t == 0 ? v[0] : (t == 1 ? v[1] : (t == 2 ? v[2] : v[3]));
}

// shared memory: gate tile | up tile | planes 4 x 2 K | XS 4 x K / 32 | SX 4 x padded K / 256 | red 8 x 32 x 4 | mbar
// Feature tiles per CTA of the grouped gate | up kernel: a CTA keeps its task's quantized activations and walks
// kGluTiles consecutive 16-feature tiles through a two-deep ring of weight buffers, the copy of tile i + 2 issued
// as soon as tile i has been used. (One tile per CTA left the CTA's ~10 us of serial latencies - task load, copy
// issue, activation fetch and quantization, first weight bytes, reduction - in front of every 36 KB of weights.)
constexpr int kGluTiles = 4;
inline int glu4_smem_bytes(int K, int row_bytes) {
  return 16 * md_group_stride(row_bytes) + 8 * K + (K / 32) * 16 + (((K / 256) + 3) & ~3) * 16 + kMdWarps * 32 * 16 + 32;
}

template <typename XT>
__global__ void __launch_bounds__(kMdThreads, 2)
moe_glu_tasks_kernel(const GluArgs a, const Task4* __restrict__ tasks, const int* __restrict__ n_tasks,
                     int* __restrict__ error_word) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  if ((int)blockIdx.y >= *n_tasks) return;
  extern __shared__ __align__(128) uint8_t md_dyn[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, nchunks = K >> 8, ncp = (nchunks + 3) & ~3, RB = a.row_bytes;
  const int gb = 4 * RB, GS = gb + ((32 - (gb & 127)) & 127);
  uint8_t* wbuf = md_dyn;                       // two buffers of (gate tile | up tile), 4 groups each
  uint8_t* planes = wbuf + 16 * GS;
  float* XS = reinterpret_cast<float*>(planes + 8 * K);
  float* SX = XS + 4 * (K / 32);
  float* red = SX + 4 * ncp;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + kMdWarps * 32 * 4);   // [2]
  const Task4 tk = tasks[blockIdx.y];
  const int all_tiles = (a.F + 15) >> 4;
  const int tile0 = blockIdx.x * a.tiles_per_cta, ntile = min(a.tiles_per_cta, all_tiles - tile0);
  const int npass = (tk.m + 3) >> 2, total = npass * ntile;   // weight copies: tiles of a pass, pass after pass
  // Warp 0 issues a tile's eight bulk copies (four-row groups of the gate and of the up rows), one per lane: a
  // single thread issuing all eight kept the other warps waiting at the tile's barrier for its issue time.
  auto issue = [&](int seq) {
    const int f0 = (tile0 + seq % ntile) * 16, rows = min(16, a.F - f0);
    uint8_t* wb = wbuf + (seq & 1) * 8 * GS;
    if (lane == 0) st_mbar_expect_tx(&mbar[seq & 1], (uint32_t)(2 * rows * RB));
    __syncwarp();
    if (lane < 8) {
      const int grp = lane & 3, r = 4 * grp;
      if (r < rows) {
        const uint8_t* src = (lane < 4 ? a.wg + (long long)tk.expert * a.stride_g : a.wu + (long long)tk.expert * a.stride_u) +
                             (long long)(f0 + r) * RB;
        st_bulk_g2s(wb + (lane < 4 ? 0 : 4 * GS) + grp * GS, src, (uint32_t)(min(4, rows - r) * RB), &mbar[seq & 1]);
      }
    }
  };
  if (warp == 0) {
    if (lane == 0) {
      st_mbar_init(&mbar[0], 1);
      st_mbar_init(&mbar[1], 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    issue(0);
    if (total > 1) issue(1);
  }
  const uint8_t* bcol = planes + min(g >> 1, 3) * 2 * K + (g & 1) * K + 8 * t;
  const int rA = 4 * (g & 3) + (g >> 2);
  const int rrow[4] = {rA, rA + 2, 16 + rA, 16 + rA + 2};
  int seq = 0;
  for (int m0 = 0; m0 < tk.m; m0 += 4) {   // four activation rows per pass over the CTA's tiles
    for (int sb = warp; sb < nchunks; sb += kMdWarps) {
      uint4 raw[4];   // the four loads in flight together
#pragma unroll
      for (int m = 0; m < 4; m++) {
        const XT* x = static_cast<const XT*>(a.x) + (long long)(tk.ent[min(m0 + m, kTaskEntries - 1)] / a.R) * K;
        raw[m] = st_ld_cg16(x + sb * 256 + lane * 8);
      }
#pragma unroll
      for (int m = 0; m < 4; m++)
        st_quantize<XT>(raw[m], sb, lane, K, planes + m * 2 * K, XS + m * (K / 32), SX + m * ncp);
    }
    __syncthreads();  // first pass: the barriers are initialised
    for (int ti = 0; ti < ntile; ti++, seq++) {
      const int f0 = (tile0 + ti) * 16, rows = min(16, a.F - f0);
      const uint8_t* wb = wbuf + (seq & 1) * 8 * GS;
      if (!md_wait(&mbar[seq & 1], (uint32_t)((seq >> 1) & 1), error_word)) return;
      const int lrA = min(rA, rows - 1), lrB = min(rA + 2, rows - 1);
      const uint8_t* base[4] = {wb + (lrA >> 2) * GS + (lrA & 3) * RB, wb + (lrB >> 2) * GS + (lrB & 3) * RB,
                                wb + (4 + (lrA >> 2)) * GS + (lrA & 3) * RB, wb + (4 + (lrB >> 2)) * GS + (lrB & 3) * RB};
      float ydot[4] = {0.f, 0.f, 0.f, 0.f}, ymin[4][4] = {};
      for (int sb = warp; sb < nchunks; sb += kMdWarps) {
        const uint8_t* const blk[4] = {base[0] + sb * 144, base[1] + sb * 144, base[2] + sb * 144, base[3] + sb * 144};
        st_unit_mx<2, 4>(blk, bcol + sb * 256, XS + sb * 8, K / 32, SX + sb, ncp, t, ydot, ymin);
      }
#pragma unroll
      for (int r = 0; r < 4; r++) {
#pragma unroll
        for (int m = 0; m < 4; m++) {
          ymin[r][m] += __shfl_xor_sync(0xffffffffu, ymin[r][m], 1);
          ymin[r][m] += __shfl_xor_sync(0xffffffffu, ymin[r][m], 2);
        }
        red[(warp * 32 + rrow[r]) * 4 + t] = ydot[r] - md_pick4(ymin[r], t);   // activation row m0 + t of this lane
      }
      __syncthreads();   // every warp has read this tile's weights and left its partial sums
      if (warp == 0 && seq + 2 < total) issue(seq + 2);   // the buffer is free: the copy after next goes in
      if (threadIdx.x < 64) {
        const int r = threadIdx.x & 15, m = threadIdx.x >> 4;
        if (r < rows && m0 + m < tk.m) {
          float gs = 0.f, us = 0.f;
#pragma unroll
          for (int w = 0; w < kMdWarps; w++) {
            gs += red[(w * 32 + r) * 4 + m];
            us += red[(w * 32 + 16 + r) * 4 + m];
          }
          md_store(static_cast<XT*>(a.y) + (long long)tk.ent[m0 + m] * a.F + f0 + r, md_act(gs, us, a.act, a.limit));
        }
      }
      __syncthreads();   // red (and, after the last tile, the planes) are free again
    }
  }
}

struct RowsArgs {
  const void* x;            // [entries, K]: row of entry b = x + b * K
  const uint8_t* w;
  long long stride_w;
  int row_bytes, K, N;
  void* y;                  // [entries, N]
};

// 128 rows per CTA, one 16-row tile per warp (for short rows: few superblocks, nothing to split over the warps)
// shared memory: 32 groups | planes 4 x 2 K | XS 4 x K / 32 | SX 4 x padded K / 256 | mbar
inline int rows4_smem_bytes(int K, int row_bytes) {
  return 32 * md_group_stride(row_bytes) + 8 * K + (K / 32) * 16 + (((K / 256) + 3) & ~3) * 16 + 16;
}

template <typename XT>
__global__ void __launch_bounds__(kMdThreads, 3)
moe_rows_tasks_kernel(const RowsArgs a, const Task4* __restrict__ tasks, const int* __restrict__ n_tasks,
                      int* __restrict__ error_word) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  if ((int)blockIdx.y >= *n_tasks) return;
  extern __shared__ __align__(128) uint8_t md_dyn[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, nchunks = K >> 8, ncp = (nchunks + 3) & ~3, RB = a.row_bytes;
  const int gb = 4 * RB, GS = gb + ((32 - (gb & 127)) & 127);
  uint8_t* wbuf = md_dyn;
  uint8_t* planes = wbuf + 32 * GS;
  float* XS = reinterpret_cast<float*>(planes + 8 * K);
  float* SX = XS + 4 * (K / 32);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(SX + 4 * ncp);
  const Task4 tk = tasks[blockIdx.y];
  const int n0 = blockIdx.x * 128, rows = min(128, a.N - n0);
  if (warp == 0) {
    if (lane == 0) {
      st_mbar_init(mbar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
      st_mbar_expect_tx(mbar, (uint32_t)(rows * RB));
    }
    __syncwarp();
    const int r = 4 * lane;   // one group of four rows per lane
    if (r < rows)
      st_bulk_g2s(wbuf + lane * GS, a.w + (long long)tk.expert * a.stride_w + (long long)(n0 + r) * RB,
                  (uint32_t)(min(4, rows - r) * RB), mbar);
  }
  const int rowsT = rows - 16 * warp;   // rows of this warp's tile (<= 0: the warp only helps quantizing)
  const uint8_t* bcol = planes + min(g >> 1, 3) * 2 * K + (g & 1) * K + 8 * t;
  const int rA = 4 * (g & 3) + (g >> 2);
  const int hi = max(min(rowsT, 16) - 1, 0);
  const int lrA = 16 * warp + min(rA, hi), lrB = 16 * warp + min(rA + 2, hi);
  const uint8_t* pA = wbuf + (lrA >> 2) * GS + (lrA & 3) * RB;
  const uint8_t* pB = wbuf + (lrB >> 2) * GS + (lrB & 3) * RB;
  for (int m0 = 0; m0 < tk.m; m0 += 4) {
    for (int u = warp; u < 4 * nchunks; u += kMdWarps) {
      const int m = u / nchunks, sb = u - m * nchunks;
      const XT* x = static_cast<const XT*>(a.x) + (long long)tk.ent[min(m0 + m, kTaskEntries - 1)] * K;
      st_quantize<XT>(st_ld_cg16(x + sb * 256 + lane * 8), sb, lane, K, planes + m * 2 * K, XS + m * (K / 32),
                      SX + m * ncp);
    }
    __syncthreads();
    if (m0 == 0 && !md_wait(mbar, 0, error_word)) return;
    if (rowsT > 0) {
      float ydot[2] = {0.f, 0.f}, ymin[2][4] = {};
      for (int sb = 0; sb < nchunks; sb++) {
        const uint8_t* const blk[2] = {pA + sb * 144, pB + sb * 144};
        st_unit_mx<1, 4>(blk, bcol + sb * 256, XS + sb * 8, K / 32, SX + sb, ncp, t, ydot, ymin);
      }
#pragma unroll
      for (int r = 0; r < 2; r++) {
#pragma unroll
        for (int m = 0; m < 4; m++) {
          ymin[r][m] += __shfl_xor_sync(0xffffffffu, ymin[r][m], 1);
          ymin[r][m] += __shfl_xor_sync(0xffffffffu, ymin[r][m], 2);
        }
      }
      if (m0 + t < tk.m) {
        XT* out = static_cast<XT*>(a.y) + (long long)tk.ent[m0 + t] * a.N + n0 + 16 * warp;
        if (rA < rowsT) md_store(out + rA, ydot[0] - md_pick4(ymin[0], t));
        if (rA + 2 < rowsT) md_store(out + rA + 2, ydot[1] - md_pick4(ymin[1], t));
      }
    }
    __syncthreads();   // the planes are free for the next pass
  }
}

// ------------------------------------------------------------------------------------------------ router
struct RouterArgs {
  const void* logits;       // [T, E + shared]
  int dtype, T, E, top_k, norm, shared, scoring;
  const float* pes;         // per-expert scale [E] or nullptr
  const float* bias;        // selection bias [E] or nullptr
  float scale;
  uint32_t* indices;        // [T, top_k]
  float* scores;            // [T, top_k + shared]
};

__device__ __forceinline__ float md_logit(const void* p, int dtype, long long i) {
  if (dtype == F32) return static_cast<const float*>(p)[i];
  if (dtype == F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

// One warp per token; lane l holds experts l, l + 32, ... (E <= 1024: at most 32 per lane).
__global__ void __launch_bounds__(256) router_topk_kernel(const RouterArgs a) {
  // the kernel that consumes the indices may start its prologue now; it reads them again after this grid is done
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= a.T) return;
  const long long row = (long long)token * (a.E + a.shared);
  float p[32], rk[32];
  float gsum = 1.f;
  if (a.scoring == 1) {   // sqrt(softplus(x)), softplus in its overflow-free form
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const int e = lane + 32 * i;
      float v = -INFINITY;
      if (e < a.E) {
        const float x = md_logit(a.logits, a.dtype, row + e);
        v = sqrtf(fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))));
      }
      p[i] = v;
    }
  } else {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const int e = lane + 32 * i;
      p[i] = e < a.E ? md_logit(a.logits, a.dtype, row + e) : -INFINITY;
      m = fmaxf(m, p[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const int e = lane + 32 * i;
      const float v = e < a.E ? expf(p[i] - m) : 0.f;
      p[i] = e < a.E ? v : -INFINITY;
      s += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    gsum = s;
  }
#pragma unroll
  for (int i = 0; i < 32; i++) {
    const int e = lane + 32 * i;
    rk[i] = (a.bias != nullptr && e < a.E) ? p[i] + a.bias[e] : p[i];
  }
  float win_v = 0.f;        // lane r keeps the r-th winner
  uint32_t win_i = 0;
  float psum = 0.f;
  for (int r = 0; r < a.top_k; r++) {
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < 32; i++) {   // ascending expert index within the lane: '>' keeps the lowest on ties
      if (rk[i] > bv) {
        bv = rk[i];
        bi = (uint32_t)(lane + 32 * i);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    // the emitted score is the unbiased one; its owner lane removes the expert from the ranking
    float pv = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
      if ((uint32_t)(lane + 32 * i) == bi) {
        pv = p[i];
        rk[i] = -INFINITY;
      }
    }
    pv = __shfl_sync(0xffffffffu, pv, bi & 31);
    psum += pv;
    if (lane == r) {
      win_v = pv;
      win_i = bi;
    }
  }
  const float denom = a.norm ? (a.scoring == 1 ? psum + 1e-20f : psum) : gsum;
  if (lane < a.top_k) {
    float sv = win_v / denom;
    if (a.pes != nullptr && win_i < (uint32_t)a.E) sv *= a.pes[win_i];
    a.indices[(long long)token * a.top_k + lane] = win_i;
    a.scores[(long long)token * (a.top_k + a.shared) + lane] = sv * a.scale;
  }
  if (a.shared && lane == 0)
    a.scores[(long long)token * (a.top_k + 1) + a.top_k] = 1.f / (1.f + expf(-md_logit(a.logits, a.dtype, row + a.E)));
}

template <typename KernelT>
cudaError_t md_set_smem(KernelT kern, int bytes, bool (&done)[16]) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return cudaErrorInvalidDevice;
  if (!done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done[dev] = true;
  }
  return cudaSuccess;
}

constexpr int kMdMaxSmem = 200 * 1024;

template <typename KernelT, typename ArgsT>
cudaError_t md_launch(KernelT kern, dim3 grid, int smem, const ArgsT& a, cudaStream_t st) {
  int* err = device_error_word();
  if (err == nullptr) return cudaErrorUnknown;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kMdThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, a, err);
}

}  // namespace

// ---- grouped forms: scratch = grouping arrays + task list (+ the per-entry products of the down stage)
struct MoeWs {
  size_t counts, cursor, offsets, task_base, n_tasks, order, tasks, d, total;
  long long max_tasks;
};
static MoeWs moe_ws_layout(long long n_entries, int n_experts, long long d_bytes) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  MoeWs L{};
  const size_t e1 = (size_t)(n_experts + 1) * 4;
  L.counts = 0;
  L.cursor = e1;
  L.offsets = 2 * e1;
  L.task_base = 3 * e1;
  L.n_tasks = 4 * e1;
  L.order = up(4 * e1 + 4);
  L.max_tasks = n_entries / kTaskEntries + n_experts + 1;
  L.tasks = up(L.order + (size_t)n_entries * 4);
  L.d = up(L.tasks + (size_t)L.max_tasks * sizeof(Task4));
  L.total = up(L.d + (size_t)d_bytes);
  return L;
}

size_t moe_grouped_workspace_bytes(long long n_entries, int n_experts, long long d_bytes) {
  return moe_ws_layout(n_entries, n_experts, d_bytes).total;
}

static cudaError_t moe_build_tasks(const uint32_t* idx, long long n_entries, int n_experts, uint8_t* ws, const MoeWs& L,
                                   cudaStream_t st) {
  int* offsets = reinterpret_cast<int*>(ws + L.offsets);
  int* task_base = reinterpret_cast<int*>(ws + L.task_base);
  int* order = reinterpret_cast<int*>(ws + L.order);
  cudaError_t e = launch_group_by_expert(idx, n_entries, n_experts, kTaskEntries, reinterpret_cast<int*>(ws + L.counts),
                                         reinterpret_cast<int*>(ws + L.cursor), offsets, task_base,
                                         reinterpret_cast<int*>(ws + L.n_tasks), order, st);
  if (e != cudaSuccess) return e;
  moe_tasks4_kernel<<<n_experts, 64, 0, st>>>(offsets, task_base, order, reinterpret_cast<Task4*>(ws + L.tasks));
  return cudaGetLastError();
}

template <typename KernelT, typename ArgsT>
static cudaError_t md_launch_tasks(KernelT kern, dim3 grid, int smem, const ArgsT& a, const Task4* tasks,
                                   const int* n_tasks, cudaStream_t st) {
  int* err = device_error_word();
  if (err == nullptr) return cudaErrorUnknown;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kMdThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  return cudaLaunchKernelEx(&cfg, kern, a, tasks, n_tasks, err);
}

// the grouping alone (for a caller whose own grouped kernel does not apply but whose workspace is handed on)
cudaError_t launch_moe_grouping_only(const uint32_t* idx, long long n_entries, int n_experts, void* workspace,
                                     cudaStream_t st) {
  const MoeWs L = moe_ws_layout(n_entries, n_experts, 0);
  return moe_build_tasks(idx, n_entries, n_experts, static_cast<uint8_t*>(workspace), L, st);
}

bool moe_grouped_supported(int K, long long row_bytes, bool rows_kernel) {
  const int smem = rows_kernel ? rows4_smem_bytes(K, (int)row_bytes) : glu4_smem_bytes(K, (int)row_bytes);
  return smem <= 110 * 1024;   // two CTAs per SM
}

cudaError_t launch_moe_glu_grouped(int x_dtype, const void* x, int K, const uint8_t* wg, long long stride_g,
                                   const uint8_t* wu, long long stride_u, long long row_bytes, int F, int n_experts,
                                   const uint32_t* idx, long long n_entries, int R, int act, float limit, void* y,
                                   void* workspace, cudaStream_t st) {
  if (n_entries <= 0 || F <= 0) return cudaSuccess;
  const MoeWs L = moe_ws_layout(n_entries, n_experts, 0);
  if (L.max_tasks > 65535) return cudaErrorInvalidConfiguration;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaError_t e = moe_build_tasks(idx, n_entries, n_experts, ws, L, st);
  if (e != cudaSuccess) return e;
  static const int tiles_env = [] {
    const char* e = std::getenv("KQ_MOE_GLU_TILES");   // A/B lever
    const int v = e ? std::atoi(e) : 0;
    return v >= 1 && v <= 64 ? v : kGluTiles;
  }();
  GluArgs a{x, wg, wu, stride_g, stride_u, (int)row_bytes, K, F, R, (int)n_entries, n_experts, idx, y, act, limit,
            tiles_env};
  const int smem = glu4_smem_bytes(K, (int)row_bytes);
  const dim3 grid(((F + 15) / 16 + tiles_env - 1) / tiles_env, (unsigned)L.max_tasks, 1);
  const Task4* tasks = reinterpret_cast<const Task4*>(ws + L.tasks);
  const int* nt = reinterpret_cast<const int*>(ws + L.n_tasks);
  static bool done_h[16] = {}, done_b[16] = {};
  if (x_dtype == F16) {
    if ((e = md_set_smem(moe_glu_tasks_kernel<__half>, kMdMaxSmem, done_h)) != cudaSuccess) return e;
    return md_launch_tasks(moe_glu_tasks_kernel<__half>, grid, smem, a, tasks, nt, st);
  }
  if ((e = md_set_smem(moe_glu_tasks_kernel<__nv_bfloat16>, kMdMaxSmem, done_b)) != cudaSuccess) return e;
  return md_launch_tasks(moe_glu_tasks_kernel<__nv_bfloat16>, grid, smem, a, tasks, nt, st);
}

// d[b] = x[b] . W[idx[b]]^T for every entry b (entries grouped by expert), then y[t] = sum_s scores[t, s] d[t S + s]
cudaError_t launch_moe_mix_grouped(int x_dtype, const void* x, int K, const uint8_t* w, long long stride_w,
                                   long long row_bytes, int N, int n_experts, const uint32_t* idx, const float* scores,
                                   long long T, int S, void* y, void* workspace, bool reuse_grouping,
                                   cudaStream_t st) {
  const long long n_entries = T * S;
  if (n_entries <= 0 || N <= 0) return cudaSuccess;
  const MoeWs L = moe_ws_layout(n_entries, n_experts, n_entries * (long long)N * 2);
  if (L.max_tasks > 65535) return cudaErrorInvalidConfiguration;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaError_t e = cudaSuccess;
  // reuse_grouping: the workspace still holds the task list that launch_moe_glu_grouped built from these indices
  if (!reuse_grouping && (e = moe_build_tasks(idx, n_entries, n_experts, ws, L, st)) != cudaSuccess) return e;
  // entries of experts out of range get no task: their d rows must not carry old bytes into the weighted sum
  if ((e = cudaMemsetAsync(ws + L.d, 0, (size_t)n_entries * N * 2, st)) != cudaSuccess) return e;
  RowsArgs a{x, w, stride_w, (int)row_bytes, K, N, ws + L.d};
  const int smem = rows4_smem_bytes(K, (int)row_bytes);
  const dim3 grid((N + 127) / 128, (unsigned)L.max_tasks, 1);
  const Task4* tasks = reinterpret_cast<const Task4*>(ws + L.tasks);
  const int* nt = reinterpret_cast<const int*>(ws + L.n_tasks);
  static bool done_h[16] = {}, done_b[16] = {};
  if (x_dtype == F16) {
    if ((e = md_set_smem(moe_rows_tasks_kernel<__half>, kMdMaxSmem, done_h)) != cudaSuccess) return e;
    e = md_launch_tasks(moe_rows_tasks_kernel<__half>, grid, smem, a, tasks, nt, st);
  } else {
    if ((e = md_set_smem(moe_rows_tasks_kernel<__nv_bfloat16>, kMdMaxSmem, done_b)) != cudaSuccess) return e;
    e = md_launch_tasks(moe_rows_tasks_kernel<__nv_bfloat16>, grid, smem, a, tasks, nt, st);
  }
  if (e != cudaSuccess) return e;
  return launch_moe_combine(x_dtype, ws + L.d, scores, T, S, N, y, false, st);
}

bool moe_decode_supported(int codec, int x_dtype, int K, long long row_bytes, const void* x, const void* w0,
                          long long stride0, const void* w1, long long stride1) {
  if (codec != Q4_K || (x_dtype != F16 && x_dtype != BF16)) return false;
  if (K < 256 || (K & 255) != 0 || row_bytes != (long long)(K >> 8) * 144) return false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return false;
  if ((reinterpret_cast<uintptr_t>(w0) & 15) != 0 || (stride0 & 15) != 0) return false;
  if (w1 != nullptr && ((reinterpret_cast<uintptr_t>(w1) & 15) != 0 || (stride1 & 15) != 0)) return false;
  return glu_smem_bytes(K, (int)row_bytes) <= kMdMaxSmem && mix_smem_bytes(K, (int)row_bytes) <= kMdMaxSmem;
}

cudaError_t launch_moe_glu(int x_dtype, const void* x, int K, const uint8_t* wg, long long stride_g, const uint8_t* wu,
                           long long stride_u, long long row_bytes, int F, int n_experts, const uint32_t* idx,
                           long long n_entries, int R, int act, float limit, void* y, cudaStream_t st) {
  if (n_entries <= 0 || F <= 0) return cudaSuccess;
  if (n_entries > 65535) return cudaErrorInvalidConfiguration;
  GluArgs a{x, wg, wu, stride_g, stride_u, (int)row_bytes, K, F, R, (int)n_entries, n_experts, idx, y, act, limit};
  const int smem = glu_smem_bytes(K, (int)row_bytes);
  const dim3 grid((F + 15) / 16, (unsigned)n_entries, 1);
  static bool done_h[16] = {}, done_b[16] = {};
  cudaError_t e;
  if (x_dtype == F16) {
    if ((e = md_set_smem(moe_glu_kernel<__half>, kMdMaxSmem, done_h)) != cudaSuccess) return e;
    return md_launch(moe_glu_kernel<__half>, grid, smem, a, st);
  }
  if ((e = md_set_smem(moe_glu_kernel<__nv_bfloat16>, kMdMaxSmem, done_b)) != cudaSuccess) return e;
  return md_launch(moe_glu_kernel<__nv_bfloat16>, grid, smem, a, st);
}

cudaError_t launch_moe_mix(int x_dtype, const void* x, int K, const uint8_t* w, long long stride_w, long long row_bytes,
                           int N, int n_experts, const uint32_t* idx, const float* scores, long long T, int S, void* y,
                           cudaStream_t st) {
  if (T <= 0 || N <= 0) return cudaSuccess;
  if (T > 65535) return cudaErrorInvalidConfiguration;
  MixArgs a{x, w, stride_w, (int)row_bytes, K, N, S, n_experts, idx, scores, y};
  const int smem = mix_smem_bytes(K, (int)row_bytes);
  const dim3 grid((N + 15) / 16, (unsigned)T, 1);
  static bool done_h[16] = {}, done_b[16] = {};
  cudaError_t e;
  if (x_dtype == F16) {
    if ((e = md_set_smem(moe_mix_kernel<__half>, kMdMaxSmem, done_h)) != cudaSuccess) return e;
    return md_launch(moe_mix_kernel<__half>, grid, smem, a, st);
  }
  if ((e = md_set_smem(moe_mix_kernel<__nv_bfloat16>, kMdMaxSmem, done_b)) != cudaSuccess) return e;
  return md_launch(moe_mix_kernel<__nv_bfloat16>, grid, smem, a, st);
}

cudaError_t launch_router_topk(const void* logits, int dtype, int T, int E, int top_k, int norm, int shared, int scoring,
                               const float* pes, const float* bias, float scale, uint32_t* indices, float* scores,
                               cudaStream_t st) {
  if (T <= 0) return cudaSuccess;
  RouterArgs a{logits, dtype, T, E, top_k, norm, shared, scoring, pes, bias, scale, indices, scores};
  router_topk_kernel<<<(T + 7) / 8, 256, 0, st>>>(a);
  return cudaGetLastError();
}

}  // namespace kq
