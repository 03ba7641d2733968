// q4_k decode product of ONE activation row for matrices of about one wave of CTAs (N <= 32 x SM count rows,
// K <= 4096): the kernel behind the [4096, 4096] decode benchmark.
//
// A launch of this size is shorter than the latencies around it (launch, first DRAM bytes, the wait for the
// preceding kernel), so the kernel is built to overlap consecutive launches of a stream three deep:
//
//   * griddepcontrol.launch_dependents is the first instruction: the next kernel of the stream may start as
//     soon as every CTA of this one has started.
//   * One CTA per <= 32 consecutive weight rows (N / SM count, so one CTA per SM and launch). Thread 0 brings
//     the CTA's whole weight span into shared memory with a few bulk copies (cp.async.bulk, one per group of
//     four rows, completion on an mbarrier; plain copies of this GPU's memory, no multicast). Groups lie
//     32 bytes apart modulo 128 and a fragment's rows come from different groups, so the 8-byte reads of a
//     warp fall into different banks without per-row padding.
//   * The products run BEFORE griddepcontrol.wait, on the activations as they are in memory at that moment.
//     After the wait (the preceding kernel has finished and its writes are visible) every warp reads its
//     activations again with an L2 load and compares them bit for bit with what it used; a warp whose
//     activations changed quantizes and multiplies again. The result is therefore always the product with
//     the final activations; when they did not change after the CTA started (the producer ran earlier in the
//     stream, or does not trigger its dependents early) only the comparison and the store remain after the
//     wait. Nothing is written before the wait.
//   * 75 KB of shared memory and 80 registers x 256 threads per CTA: three launches are resident per SM.
//
// Arithmetic: as kq_gemv_imma.cu. The activations of a superblock are quantized to 16-bit integers
// xi = rint(x * 32639 / amax) in two signed byte planes (xi = 256 xh + xl); mma.sync.m16n8k32 (u8 x s8 -> s32)
// multiplies sixteen weight rows x one 32-weight sub-block by the two planes; the exact integer dot products
// are weighted by the 6-bit sub-block scales in integer arithmetic and turned to float once per superblock:
// y += d * sx * sum_j sc_j dot_j - dmin * sum_j mn_j xsum_j (decode: src/kquant_cpu_decode.cpp:177-202).
// Two row tiles share each activation fragment.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_imma_q4k.cuh"
#include "kq_launch.h"

namespace kq {

namespace {

constexpr int kStWarps = 8, kStThreads = 32 * kStWarps;
constexpr int kStMaxRows = 32;        // rows per CTA: two 16-row fragments
constexpr int kStMaxK = 4096;         // two superblocks per warp: their raw activations stay in registers for the check
constexpr int kStMaxSmem = 75 * 1024; // three CTAs per SM

// rows are copied four at a time; groups lie 32 bytes apart modulo 128
inline int st_group_stride(long long row_bytes) {
  const long long gb = 4 * row_bytes;
  return (int)(gb + ((32 - (gb & 127)) & 127));
}
// weights | byte planes (2 K) | sub-block sums (K / 32 floats) | superblock scales (K / 256) | partial sums | mbarrier
inline int st_smem_bytes(int rpc, int K, long long row_bytes) {
  return ((rpc + 3) / 4) * st_group_stride(row_bytes) + 2 * K + (K / 32) * 4 + (((K / 256) + 3) & ~3) * 4 +
         kStWarps * 32 * 4 + 16;
}

template <typename XT>
__global__ void __launch_bounds__(kStThreads, 3)
gemv_q4k_stream_kernel(const GemvArgs a, const int rpc, int* __restrict__ error_word) {
  using OT = XT;
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  extern __shared__ __align__(128) uint8_t st_dyn[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, nchunks = K >> 8;
  const int RB = (int)a.row_bytes;
  const int gb = 4 * RB;
  const int GS = gb + ((32 - (gb & 127)) & 127);
  uint8_t* wbuf = st_dyn;
  uint8_t* planes = wbuf + ((rpc + 3) >> 2) * GS;
  float* XS = reinterpret_cast<float*>(planes + 2 * K);
  float* SX = XS + (K / 32);
  float* red = SX + ((nchunks + 3) & ~3);  // keeps the mbarrier 8-byte aligned
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + kStWarps * 32);
  const int row0 = (int)blockIdx.x * rpc;
  const int rows = min(rpc, a.N - row0);
  const XT* x = static_cast<const XT*>(a.x);

  if (threadIdx.x == 0) {
    st_mbar_init(mbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    st_mbar_expect_tx(mbar, (uint32_t)(rows * RB));
    for (int r = 0; r < rows; r += 4)
      st_bulk_g2s(wbuf + (r >> 2) * GS, a.w + (long long)(row0 + r) * RB, (uint32_t)(min(4, rows - r) * RB), mbar);
  }
  // this warp's superblocks of x as they are now (at most two: K <= 4096)
  uint4 raw[2];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int sb = warp + i * kStWarps;
    raw[i] = sb < nchunks ? st_ld_cg16(x + sb * 256 + lane * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  const int ntiles = (rows + 15) >> 4;
  const uint8_t* bplane = planes + min(g, 1) * K + 8 * t;
  // tile row of this lane's two fragment rows: rows g and g + 8 of a fragment come from different four-row groups
  const int lrA = 4 * (g & 3) + (g >> 2), lrB = lrA + 2;
  bool gave_up = false;

  auto compute = [&](bool first) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int sb = warp + i * kStWarps;
      if (sb < nchunks) {
        if (!first) raw[i] = st_ld_cg16(x + sb * 256 + lane * 8);
        st_quantize<XT>(raw[i], sb, lane, K, planes, XS, SX);
      }
    }
    __syncwarp();
    if (first) {
      // weights landed? Bounded: after two seconds the CTA raises a flag and goes on (results undefined).
      if (!st_mbar_try_wait(mbar, 0)) {
        const unsigned long long t0 = st_gtime();
        for (int spin = 0; !st_mbar_try_wait(mbar, 0); spin++) {
          if ((spin & 63) == 63 && st_gtime() - t0 > 2000000000ull) {
            if (lane == 0) atomicOr(error_word, 0x80);
            gave_up = true;
            break;
          }
        }
      }
    }
    if (ntiles == 2) {
      const int r2 = min(16 + lrA, rows - 1), r3 = min(16 + lrB, rows - 1);
      const uint8_t* base[4] = {wbuf + (lrA >> 2) * GS + (lrA & 3) * RB, wbuf + (lrB >> 2) * GS + (lrB & 3) * RB,
                                wbuf + (r2 >> 2) * GS + (r2 & 3) * RB, wbuf + (r3 >> 2) * GS + (r3 & 3) * RB};
      float y4[4] = {0.f, 0.f, 0.f, 0.f};
      for (int sb = warp; sb < nchunks; sb += kStWarps) {
        const uint8_t* const blk[4] = {base[0] + sb * 144, base[1] + sb * 144, base[2] + sb * 144, base[3] + sb * 144};
        st_unit<2>(blk, bplane + sb * 256, XS + sb * 8, SX[sb], t, y4);
      }
#pragma unroll
      for (int r = 0; r < 4; r++) {
        y4[r] += __shfl_xor_sync(0xffffffffu, y4[r], 1);
        y4[r] += __shfl_xor_sync(0xffffffffu, y4[r], 2);
      }
      if (t == 0) {
        red[warp * 32 + lrA] = y4[0];
        red[warp * 32 + lrB] = y4[1];
        red[warp * 32 + 16 + lrA] = y4[2];
        red[warp * 32 + 16 + lrB] = y4[3];
      }
    } else {
      const int r0 = min(lrA, rows - 1), r1 = min(lrB, rows - 1);
      float y2[2] = {0.f, 0.f};
      for (int sb = warp; sb < nchunks; sb += kStWarps) {
        const uint8_t* const blk[2] = {wbuf + (r0 >> 2) * GS + (r0 & 3) * RB + sb * 144,
                                       wbuf + (r1 >> 2) * GS + (r1 & 3) * RB + sb * 144};
        st_unit<1>(blk, bplane + sb * 256, XS + sb * 8, SX[sb], t, y2);
      }
#pragma unroll
      for (int r = 0; r < 2; r++) {
        y2[r] += __shfl_xor_sync(0xffffffffu, y2[r], 1);
        y2[r] += __shfl_xor_sync(0xffffffffu, y2[r], 2);
      }
      if (t == 0) {
        red[warp * 32 + lrA] = y2[0];
        red[warp * 32 + lrB] = y2[1];
      }
    }
  };
  auto total = [&]() {  // fixed order over the warps
    float s = 0.f;
    if (threadIdx.x < 32) {
#pragma unroll
      for (int w = 0; w < kStWarps; w++) s += red[w * 32 + threadIdx.x];
    }
    return s;
  };

  __syncthreads();  // the barrier is initialised
  compute(true);
  __syncthreads();
  float ysum = total();
  asm volatile("griddepcontrol.wait;\n" ::: "memory");  // the preceding kernel has finished: x is final
  bool same = true;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int sb = warp + i * kStWarps;
    if (sb < nchunks) {
      const uint4 r = st_ld_cg16(x + sb * 256 + lane * 8);
      same = same && r.x == raw[i].x && r.y == raw[i].y && r.z == raw[i].z && r.w == raw[i].w;
    }
  }
  const bool warp_same = __all_sync(0xffffffffu, same);
  if (__syncthreads_or(!warp_same)) {
    if (!warp_same) compute(false);
    __syncthreads();
    ysum = total();
  }
  if (threadIdx.x < rows && !gave_up) {
    OT* out = static_cast<OT*>(a.y) + row0 + threadIdx.x;
    if constexpr (std::is_same<OT, __half>::value) *out = __float2half_rn(ysum);
    else *out = __float2bfloat16_rn(ysum);
  }
}

template <typename XT>
cudaError_t launch_stream(const GemvArgs& a, int rpc, cudaStream_t st) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_stream_kernel<XT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kStMaxSmem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  int* err = device_error_word();
  if (err == nullptr) return cudaErrorUnknown;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + rpc - 1) / rpc, 1, 1);
  cfg.blockDim = dim3(kStThreads);
  cfg.dynamicSmemBytes = st_smem_bytes(rpc, a.K, a.row_bytes);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, gemv_q4k_stream_kernel<XT>, a, rpc, err);
}

int stream_rows_per_cta(const GemvArgs& a) {
  static int sms[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 0;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
    sms[dev] = n;
  }
  return (a.N + sms[dev] - 1) / sms[dev];
}

}  // namespace

bool gemv_stream_supported(int codec, int x_dtype, const GemvArgs& a) {
  if (!(codec == Q4_K && (x_dtype == F16 || x_dtype == BF16) && a.tasks == nullptr && a.M == 1 && a.w_align16 != 0 &&
        (a.K & 255) == 0 && a.K >= 256 && a.K <= kStMaxK && a.row_bytes == (long long)(a.K >> 8) * 144 &&
        (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && a.out_bf16 == 0 && a.row_scale == nullptr &&
        a.bias == nullptr && a.N >= 256))
    return false;
  const int rpc = stream_rows_per_cta(a);
  return rpc >= 1 && rpc <= kStMaxRows && st_smem_bytes(rpc, a.K, a.row_bytes) <= kStMaxSmem;
}

cudaError_t launch_gemv_stream(int x_dtype, const GemvArgs& a, cudaStream_t st) {
  const int rpc = stream_rows_per_cta(a);
  if (x_dtype == F16) return launch_stream<__half>(a, rpc, st);
  return launch_stream<__nv_bfloat16>(a, rpc, st);
}

}  // namespace kq
