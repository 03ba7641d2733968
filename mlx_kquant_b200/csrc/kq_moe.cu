// The two elementwise stages of a mixture-of-experts SwiGLU block that sit between the three
// gather_qmm calls: h = silu(gate) * up, and y[t] = sum_j p[t, j] * d[t k + j]. The reference fuses
// them into its Metal MoE op (src/kquant.h:335-357; no CPU evaluation, src/kquant_moe_glu.cpp:1-8); here
// they are two streaming kernels so that a block built from gather_qmm calls does not pay a dozen
// generic elementwise passes. fp32 arithmetic, one rounding to the activation dtype (where the
// three-call composition of the reference rounds too, src/kquant_ops.cpp:354).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kq_common.cuh"
#include "kq_launch.h"

namespace kq {

namespace {

template <typename T>
__device__ __forceinline__ float2 pair_to_float(uint32_t v);
template <>
__device__ __forceinline__ float2 pair_to_float<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <>
__device__ __forceinline__ float2 pair_to_float<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}
template <typename T>
__device__ __forceinline__ uint32_t float_to_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t float_to_pair<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t float_to_pair<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}


// eight elements per thread; F % 8 == 0, rows 16-byte aligned
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                    long long in_row_stride, long long rows, int F,
                                                    T* __restrict__ out, const uint32_t* __restrict__ row_expert,
                                                    uint32_t n_experts) {
  const int per_row = F / 8;
  const long long n = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    // a row routed to an expert outside [0, n_experts) has no product: gather_qmm left it unwritten
    if (row_expert != nullptr && row_expert[r] >= n_experts) continue;
    const uint4 g = *reinterpret_cast<const uint4*>(gate + r * in_row_stride + c);
    const uint4 u = *reinterpret_cast<const uint4*>(up + r * in_row_stride + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 a = pair_to_float<T>(gw[j]), b = pair_to_float<T>(uw[j]);
      o[j] = float_to_pair<T>(silu_f(a.x) * b.x, silu_f(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(out + r * (long long)F + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <typename OT>
__device__ __forceinline__ void store8(OT* o, const float (&acc)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* o, const float (&acc)[8]) {
  reinterpret_cast<float4*>(o)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  reinterpret_cast<float4*>(o)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half* o, const float (&acc)[8]) {
  *reinterpret_cast<uint4*>(o) =
      make_uint4(float_to_pair<__half>(acc[0], acc[1]), float_to_pair<__half>(acc[2], acc[3]),
                 float_to_pair<__half>(acc[4], acc[5]), float_to_pair<__half>(acc[6], acc[7]));
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* o, const float (&acc)[8]) {
  *reinterpret_cast<uint4*>(o) =
      make_uint4(float_to_pair<__nv_bfloat16>(acc[0], acc[1]), float_to_pair<__nv_bfloat16>(acc[2], acc[3]),
                 float_to_pair<__nv_bfloat16>(acc[4], acc[5]), float_to_pair<__nv_bfloat16>(acc[6], acc[7]));
}

// one CTA per token: y[t, :] = sum_j p[t, j] * d[t k + j, :]; H % 8 == 0. A row whose weight is exactly zero
// is not read (an expert-parallel rank zeroes the weights of the rows other ranks own, and those rows of d
// were never written); with idx given, neither is a row whose expert index is outside [0, n_experts).
template <typename T, typename OT>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ d, const float* __restrict__ p,
                                                     const uint32_t* __restrict__ idx, uint32_t n_experts, int k, int H,
                                                     OT* __restrict__ y) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; j++) {
      const float w = p[t * k + j];
      if (w == 0.f) continue;
      if (idx != nullptr && idx[t * k + j] >= n_experts) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(d + (t * k + j) * (long long)H + c);
      const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float2 f = pair_to_float<T>(vw[q]);
        acc[2 * q] = fmaf(w, f.x, acc[2 * q]);
        acc[2 * q + 1] = fmaf(w, f.y, acc[2 * q + 1]);
      }
    }
    store8<OT>(y + t * (long long)H + c, acc);
  }
}


// ---- expert-parallel combine over peer memory -------------------------------------------------
// The weighted sum of an expert-parallel rank, written straight into the memory of the rank that owns the
// token instead of into a local buffer that a reduce-scatter then moves: token g = w * tokens_per_rank + t
// belongs to rank w, and this rank's partial row goes to slots[w][my_rank][t] (slots[w] = that rank's
// [world, tokens_per_rank, H] buffer, reached through a peer mapping; plain 16-byte stores, no multicast).
// A token none of whose experts lives here writes nothing: the owner knows from its own routing table
// which ranks contribute to each of its tokens (slot_sum_kernel below) and never reads the other slots.
template <typename T, typename OT>
__global__ void __launch_bounds__(256)
combine_scatter_kernel(const T* __restrict__ d, const float* __restrict__ p, const uint32_t* __restrict__ idx,
                       uint32_t n_experts, int k, int H, long long tokens_per_rank, int my_rank,
                       OT* const* __restrict__ slots) {
  const long long g = blockIdx.x;
  int mine = 0;
  if ((int)threadIdx.x < k) mine = (idx[g * k + threadIdx.x] < n_experts && p[g * k + threadIdx.x] != 0.f) ? 1 : 0;
  if (!__syncthreads_or(mine)) return;
  const long long w = g / tokens_per_rank, t = g % tokens_per_rank;
  OT* out = slots[w] + ((long long)my_rank * tokens_per_rank + t) * (long long)H;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; j++) {
      const float wj = p[g * k + j];
      if (wj == 0.f || idx[g * k + j] >= n_experts) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(d + (g * k + j) * (long long)H + c);
      const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float2 f = pair_to_float<T>(vw[q]);
        acc[2 * q] = fmaf(wj, f.x, acc[2 * q]);
        acc[2 * q + 1] = fmaf(wj, f.y, acc[2 * q + 1]);
      }
    }
    store8<OT>(out + c, acc);
  }
  // No fence here: the stores are complete when the grid is, and the host orders "every rank's grid has finished"
  // before anyone reads its slots (a collective queued behind this kernel on every rank's stream).
}

// y[t, :] = sum over the ranks r that own at least one of token t's experts, in rank order, of slots[r][t, :]
// (float32 accumulation, one rounding). rank_lo [world + 1]: first expert of each rank's contiguous share.
template <typename ST, typename OT>
__global__ void __launch_bounds__(256)
slot_sum_kernel(const ST* __restrict__ slots, const uint32_t* __restrict__ ids, const int* __restrict__ rank_lo, int world,
                long long T, int k, int H, OT* __restrict__ y) {
  const long long t = blockIdx.x;
  __shared__ unsigned s_mask;
  if (threadIdx.x == 0) s_mask = 0u;
  __syncthreads();
  if ((int)threadIdx.x < k) {
    const int e = (int)ids[t * k + threadIdx.x];
    for (int r = 0; r < world; r++)
      if (e >= rank_lo[r] && e < rank_lo[r + 1]) atomicOr(&s_mask, 1u << r);
  }
  __syncthreads();
  const unsigned mask = s_mask;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; r++) {
      if (!((mask >> r) & 1u)) continue;
      const ST* src = slots + ((long long)r * T + t) * (long long)H + c;
      if constexpr (sizeof(ST) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
        acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w;
        acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
      } else {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float2 f = pair_to_float<ST>(vw[q]);
          acc[2 * q] += f.x;
          acc[2 * q + 1] += f.y;
        }
      }
    }
    store8<OT>(y + t * (long long)H + c, acc);
  }
}

}  // namespace

cudaError_t launch_swiglu(int dtype, const void* gate, const void* up, long long in_row_stride, long long rows, int F,
                          void* out, const uint32_t* row_expert, uint32_t n_experts, cudaStream_t st) {
  if (rows <= 0 || F <= 0) return cudaSuccess;
  const long long n = rows * (F / 8);
  const unsigned blocks = (unsigned)std::min<long long>((n + 255) / 256, 148 * 16);
  if (dtype == F16)
    swiglu_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(gate), static_cast<const __half*>(up),
                                                  in_row_stride, rows, F, static_cast<__half*>(out), row_expert, n_experts);
  else
    swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gate),
                                                         static_cast<const __nv_bfloat16*>(up), in_row_stride, rows, F,
                                                         static_cast<__nv_bfloat16*>(out), row_expert, n_experts);
  return cudaGetLastError();
}

cudaError_t launch_moe_combine(int dtype, const void* d, const float* probs, long long tokens, int k, int H, void* y,
                               bool y_f32, cudaStream_t st, const uint32_t* idx, uint32_t n_experts) {
  if (tokens <= 0 || H <= 0 || k <= 0) return cudaSuccess;
  const unsigned g = (unsigned)tokens;
  if (dtype == F16) {
    const __half* dp = static_cast<const __half*>(d);
    if (y_f32) combine_kernel<__half, float><<<g, 256, 0, st>>>(dp, probs, idx, n_experts, k, H, static_cast<float*>(y));
    else combine_kernel<__half, __half><<<g, 256, 0, st>>>(dp, probs, idx, n_experts, k, H, static_cast<__half*>(y));
  } else {
    const __nv_bfloat16* dp = static_cast<const __nv_bfloat16*>(d);
    if (y_f32) combine_kernel<__nv_bfloat16, float><<<g, 256, 0, st>>>(dp, probs, idx, n_experts, k, H, static_cast<float*>(y));
    else combine_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, st>>>(dp, probs, idx, n_experts, k, H, static_cast<__nv_bfloat16*>(y));
  }
  return cudaGetLastError();
}

// d [tokens * k, H] of dtype -> partial rows in the owners' slot buffers (slot_f32: float32 slots, else dtype).
cudaError_t launch_moe_combine_scatter(int dtype, const void* d, const float* probs, const uint32_t* idx,
                                       uint32_t n_experts, long long tokens, int k, int H, long long tokens_per_rank,
                                       int my_rank, void* const* slots, bool slot_f32, cudaStream_t st) {
  if (tokens <= 0 || H <= 0 || k <= 0) return cudaSuccess;
  if (k > 256 || tokens_per_rank <= 0) return cudaErrorInvalidValue;
  const unsigned g = (unsigned)tokens;
#define KQ_CS(T, OT)                                                                                          \
  combine_scatter_kernel<T, OT><<<g, 256, 0, st>>>(static_cast<const T*>(d), probs, idx, n_experts, k, H,      \
                                                   tokens_per_rank, my_rank, reinterpret_cast<OT* const*>(slots))
  if (dtype == F16) {
    if (slot_f32) KQ_CS(__half, float);
    else KQ_CS(__half, __half);
  } else {
    if (slot_f32) KQ_CS(__nv_bfloat16, float);
    else KQ_CS(__nv_bfloat16, __nv_bfloat16);
  }
#undef KQ_CS
  return cudaGetLastError();
}

// slots [world, T, H] (slot_dtype F32 / F16 / BF16), ids [T, k] global expert indices -> y [T, H] (F16 / BF16 / F32)
cudaError_t launch_moe_slot_sum(int slot_dtype, const void* slots, const uint32_t* ids, const int* rank_lo, int world,
                                long long T, int k, int H, int y_dtype, void* y, cudaStream_t st) {
  if (T <= 0 || H <= 0 || k <= 0) return cudaSuccess;
  if (k > 256 || world <= 0 || world > 32) return cudaErrorInvalidValue;
  const unsigned g = (unsigned)T;
#define KQ_SS(ST, OT) \
  slot_sum_kernel<ST, OT><<<g, 256, 0, st>>>(static_cast<const ST*>(slots), ids, rank_lo, world, T, k, H, static_cast<OT*>(y))
#define KQ_SS_OUT(ST)                        \
  do {                                       \
    if (y_dtype == F32) KQ_SS(ST, float);    \
    else if (y_dtype == F16) KQ_SS(ST, __half); \
    else KQ_SS(ST, __nv_bfloat16);           \
  } while (0)
  if (slot_dtype == F32) KQ_SS_OUT(float);
  else if (slot_dtype == F16) KQ_SS_OUT(__half);
  else KQ_SS_OUT(__nv_bfloat16);
#undef KQ_SS_OUT
#undef KQ_SS
  return cudaGetLastError();
}

}  // namespace kq
