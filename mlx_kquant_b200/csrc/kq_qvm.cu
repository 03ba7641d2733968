// quantized_matmul with transpose == 0: W is [K, N / weights_per_block * bytes_per_block], every one of its
// K rows a quantized vector of N weights, and y[m, n] = sum_k x[m, k] * dequant(W)[k, n]
// (src/kquant_ops.cpp:140-155; the reference's qvm / qmm_n Metal kernels, src/kquant_matmul.cpp:705-751, and on
// the CPU dequantize-then-GEMM, src/kquant_cpu_decode.cpp:1299-1352). A rarely used orientation (the layers
// of the reference's own models keep [N, K] weights), served by one streaming CUDA-core kernel:
// a CTA owns 256 output columns and a slice of K; its eight warps take the slice's rows in turn, lane j
// decodes the eight weights 8 j .. 8 j + 7 of the row's 256-column chunk in fp32 (decode8, the dequantize
// kernel's arithmetic) and multiplies them by up to four activations x[m, k]; warps meet in shared memory,
// K slices (a cluster of up to 8 CTAs) through distributed shared memory. More than four rows are
// further passes over the weights (grid.z): correct for any M, efficient for decode-sized M only.
#include <cooperative_groups.h>

#include <type_traits>

#include "kq_common.cuh"
#include "kq_launch.h"

namespace cg = cooperative_groups;

namespace kq {

namespace {

constexpr int kWarps = 8, kThreads = 256, kMT = 4, kMaxSplit = 8, kCols = 256;

struct QvmGather {
  const uint32_t* lhs;
  const uint32_t* rhs;   // nullptr = dense call
  long long entry0, x_batch, expert_stride;
  int n_experts, m_tiles;
};

template <typename XT>
__device__ __forceinline__ float load_x(const XT* p) {
  if constexpr (std::is_same<XT, __half>::value) return __half2float(*p);
  else if constexpr (std::is_same<XT, __nv_bfloat16>::value) return __bfloat162float(*p);
  else return __bfloat162float(__float2bfloat16_rn(*p));  // float rows are rounded to bf16 first, as the op does
}

template <int C, int A, typename XT>
__global__ void __launch_bounds__(kThreads)
qvm_kernel(const XT* __restrict__ x, long long x_row_stride, void* __restrict__ y, long long y_row_stride,
           const uint8_t* __restrict__ w, long long row_bytes, int M, int N, int K, QvmGather gq) {
  using OT = typename std::conditional<std::is_same<XT, __half>::value, __half, __nv_bfloat16>::type;
  constexpr int WPB = wpb_of(C), BPB = bpb_of(C);
  __shared__ float red[kWarps][kMT][kCols];
  __shared__ float part[kMT][kCols];
  __shared__ __align__(16) uint8_t s_tabs[(C == IQ4_NL || C == IQ4_XS || C == IQ2_XXS) ? kIqSmemBytes : 16];
  cg::cluster_group cluster = cg::this_cluster();
  IqTables tabs = global_iq_tables();
  if constexpr (C == IQ4_NL || C == IQ4_XS || C == IQ2_XXS) {
    tabs = stage_iq_tables(s_tabs, threadIdx.x, kThreads);
    __syncthreads();
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int S = gridDim.y, slice = blockIdx.y;
  const int c0 = blockIdx.x * kCols + 8 * lane;  // this lane's eight output columns
  int mtile = blockIdx.z;
  if (gq.rhs != nullptr) {
    // gather form: grid.z = entries x row tiles; entry e multiplies x[lhs[e]] ([M, K]) by matrix rhs[e] into y[e].
    // An index out of range leaves the entry's rows unwritten (uniform over the cluster, which spans grid.y only).
    const long long e = gq.entry0 + blockIdx.z / gq.m_tiles;
    mtile = blockIdx.z % gq.m_tiles;
    const uint32_t l = gq.lhs[e], r = gq.rhs[e];
    if (r >= (uint32_t)gq.n_experts || (long long)l >= gq.x_batch) return;
    x += (long long)l * M * x_row_stride;
    w += (long long)r * gq.expert_stride;
    y = static_cast<OT*>(y) + e * M * y_row_stride;
  }
  const int m0 = mtile * kMT, m = min(kMT, M - m0);
  const int per = (K + S - 1) / S;
  const int k0 = min(slice * per, K), k1 = min(k0 + per, K);

  float acc[kMT][8];
#pragma unroll
  for (int t = 0; t < kMT; t++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[t][i] = 0.f;
  // this lane's eight columns: 256 blockIdx.x + 8 lane .. + 7
  const long long blk_off = block_of<C>(256ll * blockIdx.x + 8 * lane) * BPB;
  const int oct = octet_of<C>(8 * lane);
  if (c0 < N) {
    for (int k = k0 + warp; k < k1; k += kWarps) {
      float v[8];
      decode8<C, A>(w + (long long)k * row_bytes + blk_off, oct, v, tabs);
#pragma unroll
      for (int t = 0; t < kMT; t++) {
        if (t < m) {
          const float xv = load_x<XT>(x + (long long)(m0 + t) * x_row_stride + k);
#pragma unroll
          for (int i = 0; i < 8; i++) acc[t][i] = fmaf(xv, v[i], acc[t][i]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kMT; t++)
#pragma unroll
    for (int i = 0; i < 8; i++) red[warp][t][8 * lane + i] = acc[t][i];
  __syncthreads();
  for (int idx = threadIdx.x; idx < kMT * kCols; idx += kThreads) {
    const int t = idx / kCols, c = idx % kCols;
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < kWarps; wv++) s += red[wv][t][c];
    part[t][c] = s;
  }
  cluster.sync();  // every K slice's partial sums are in its shared memory
  const float* peer[kMaxSplit];
#pragma unroll
  for (int s = 0; s < kMaxSplit; s++) peer[s] = s < S ? cluster.map_shared_rank(&part[0][0], s) : &part[0][0];
  for (int idx = slice + S * threadIdx.x; idx < kMT * kCols; idx += S * kThreads) {
    const int t = idx / kCols, c = blockIdx.x * kCols + idx % kCols;
    if (t < m && c < N) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxSplit; s++)
        if (s < S) sum += peer[s][idx];
      OT* out = static_cast<OT*>(y) + (long long)(m0 + t) * y_row_stride + c;
      if constexpr (std::is_same<OT, __half>::value) *out = __float2half_rn(sum);
      else *out = __float2bfloat16_rn(sum);
    }
  }
  cluster.sync();  // peers may still be reading this CTA's partial sums
}

template <int C, int A, typename XT>
cudaError_t launch_one(const void* x, long long x_row_stride, void* y, long long y_row_stride, const uint8_t* w,
                       long long row_bytes, int M, int N, int K, cudaStream_t st, QvmGather gq = QvmGather{},
                       long long entries = 1) {
  const int col_ctas = (N + kCols - 1) / kCols, m_tiles = (M + kMT - 1) / kMT;
  int S = 1;
  while (S < kMaxSplit && (long long)col_ctas * m_tiles * entries * S < 2 * 148 && K / (S * 2) >= 4 * kWarps) S *= 2;
  gq.m_tiles = m_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(col_ctas, S, (unsigned)(m_tiles * entries));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = S;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, qvm_kernel<C, A, XT>, static_cast<const XT*>(x), x_row_stride, y, y_row_stride, w,
                            row_bytes, M, N, K, gq);
}

template <int C, int NAT>
cudaError_t launch_codec(int x_dtype, const void* x, long long x_row_stride, void* y, long long y_row_stride,
                         const uint8_t* w, long long row_bytes, int M, int N, int K, cudaStream_t st,
                         QvmGather gq = QvmGather{}, long long entries = 1) {
  const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (row_bytes & 15) == 0 && (gq.expert_stride & 15) == 0;
#define KQ_QVM(XT)                                                                                                    \
  return aligned ? launch_one<C, NAT, XT>(x, x_row_stride, y, y_row_stride, w, row_bytes, M, N, K, st, gq, entries)  \
                 : launch_one<C, 1, XT>(x, x_row_stride, y, y_row_stride, w, row_bytes, M, N, K, st, gq, entries)
  if (x_dtype == F16) KQ_QVM(__half);
  if (x_dtype == BF16) KQ_QVM(__nv_bfloat16);
  KQ_QVM(float);
#undef KQ_QVM
}

}  // namespace

cudaError_t launch_qvm(int codec, int x_dtype, const void* x, long long x_row_stride, void* y, long long y_row_stride,
                       const uint8_t* w, long long row_bytes, int M, int N, int K, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaSuccess;
  if ((M + kMT - 1) / kMT > 65535) return cudaErrorInvalidConfiguration;
#define KQ_CASE(CODEC, NAT) \
  case CODEC: return launch_codec<CODEC, NAT>(x_dtype, x, x_row_stride, y, y_row_stride, w, row_bytes, M, N, K, st)
  switch (codec) {
    KQ_CASE(Q2_K, 4);
    KQ_CASE(Q3_K, 2);
    KQ_CASE(Q4_K, 16);
    KQ_CASE(Q5_K, 16);
    KQ_CASE(Q6_K, 2);
    KQ_CASE(Q4_0, 2);
    KQ_CASE(Q8_0, 2);
    KQ_CASE(IQ4_NL, 2);
    KQ_CASE(IQ4_XS, 8);
    KQ_CASE(IQ2_XXS, 2);
    KQ_CASE(Q4_1, 4);
    KQ_CASE(Q5_0, 2);
    KQ_CASE(Q5_1, 8);
    KQ_CASE(IQ3_XXS, 2);
    KQ_CASE(IQ3_S, 2);
    KQ_CASE(IQ2_XS, 2);
    KQ_CASE(IQ2_S, 2);
    KQ_CASE(IQ1_S, 2);
    KQ_CASE(IQ1_M, 8);
    KQ_CASE(MXFP4, 1);
    KQ_CASE(NVFP4, 4);
  }
#undef KQ_CASE
  return cudaErrorInvalidValue;
}

// gather form of the same kernel: entry e is x[lhs[e]] ([M, K]) @ dequant(w[rhs[e]]) ([K, N]) -> y[e] ([M, N])
cudaError_t launch_qvm_gather(int codec, int x_dtype, const void* x, long long x_batch, void* y, const uint8_t* w,
                              int n_experts, long long expert_stride, long long row_bytes, int M, int N, int K,
                              const uint32_t* lhs, const uint32_t* rhs, long long n_entries, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || n_entries <= 0) return cudaSuccess;
  const int m_tiles = (M + kMT - 1) / kMT;
  if (m_tiles > 65535) return cudaErrorInvalidConfiguration;
  const long long per_launch = 65535 / m_tiles;
  for (long long e0 = 0; e0 < n_entries; e0 += per_launch) {
    const long long cnt = n_entries - e0 < per_launch ? n_entries - e0 : per_launch;
    QvmGather gq{lhs, rhs, e0, x_batch, expert_stride, n_experts, m_tiles};
    cudaError_t err = cudaErrorInvalidValue;
#define KQ_CASE(CODEC, NAT) \
  case CODEC: err = launch_codec<CODEC, NAT>(x_dtype, x, K, y, N, w, row_bytes, M, N, K, st, gq, cnt); break
    switch (codec) {
      KQ_CASE(Q2_K, 4);
      KQ_CASE(Q3_K, 2);
      KQ_CASE(Q4_K, 16);
      KQ_CASE(Q5_K, 16);
      KQ_CASE(Q6_K, 2);
      KQ_CASE(Q4_0, 2);
      KQ_CASE(Q8_0, 2);
      KQ_CASE(IQ4_NL, 2);
      KQ_CASE(IQ4_XS, 8);
      KQ_CASE(IQ2_XXS, 2);
      KQ_CASE(Q4_1, 4);
      KQ_CASE(Q5_0, 2);
      KQ_CASE(Q5_1, 8);
      KQ_CASE(IQ3_XXS, 2);
      KQ_CASE(IQ3_S, 2);
      KQ_CASE(IQ2_XS, 2);
      KQ_CASE(IQ2_S, 2);
      KQ_CASE(IQ1_S, 2);
      KQ_CASE(IQ1_M, 8);
      KQ_CASE(MXFP4, 1);
      KQ_CASE(NVFP4, 4);
    }
#undef KQ_CASE
    if (err != cudaSuccess) return err;
  }
  return cudaSuccess;
}

}  // namespace kq
