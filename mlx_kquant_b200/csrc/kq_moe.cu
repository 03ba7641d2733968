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

}  // namespace kq
