// q4_k decode product (one to four activation rows) on the integer tensor pipe.
//
// Same arithmetic as the integer dot-product kernel of kq_gemv.cu, with mma.sync.m16n8k32 (u8 x s8 ->
// s32) doing the products: the activations of every 256-weight superblock are quantized to 16-bit
// integers xi = rint(x * 32639 / amax) (one scale per superblock) and split into two signed byte
// planes xi = 256 xh + xl, xl = (int8)(xi & 255); the 4-bit quants are the A operand as they lie in
// the wire bytes (low nibbles masked, high nibbles kept in place as 16 q), sixteen weight rows by one
// 32-weight sub-block per instruction; the planes are the B operand, columns 2m and 2m + 1 for
// activation row m. Each instruction yields the exact integer products of one sub-block, which are
// weighted by the sub-block's 6-bit scale in integer arithmetic and turned to float once per
// superblock: y += d * sx * (sum_j sc_j dot_j) - dmin * sum_j mn_j * xsum_j, with xsum_j the float
// sums of the activations of sub-block j (src/kquant_cpu_decode.cpp:177-202 is the decode this
// reproduces; the op rounds float32 activations to bfloat16 first, src/kquant_ops.cpp:159-168).
//
// Against the dp4a kernel: 590 instead of 726 warp instructions per 32 rows x 256 weights (the products of
// 512 weights in one instruction instead of 128 in two). Measured on one GPU, same run: 3-7 % faster up
// to ~60 M weights, slower beyond; the dispatcher uses it in that range (KQ_GEMV_IMMA=0|1 forces the choice).
//
// CTA = 8 warps x up to 32 weight rows; the warps split K in superblock columns; every warp streams
// its columns through a cp.async ring of D slots (32 rows x 160 bytes: the 144 wire bytes of a block
// plus 16 of padding, so that the eight rows a quarter-warp reads lie in different banks).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_launch.h"

namespace kq {

namespace {

constexpr int kImWarps = 8, kImThreads = 32 * kImWarps, kImRows = 32;
constexpr int kImRowStride = 160;
constexpr int kImSlot = kImRows * kImRowStride;
constexpr int kImMaxK = 16384;

// byte planes, sub-block sums and superblock scales of MX activation rows
constexpr int im_x_bytes(int K, int MX) { return MX * (2 * K + (K / 32) * 4 + (K / 256) * 4); }
inline int im_dyn_smem(int K, int D, int MX) { return kImWarps * D * kImSlot + im_x_bytes(K, MX); }

__device__ __forceinline__ void im_cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void im_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void im_wait(int n) {
  if (n <= 0) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  else asm volatile("cp.async.wait_group 1;\n" ::: "memory");
}

// D(16 x 8, s32) = A(16 x 32, u8, row) * B(32 x 8, s8, col)
__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ int byte_of(uint32_t v, int j) { return (int)__byte_perm(v, 0u, 0x4440u + j); }

struct ScaleWords {
  uint32_t scl, sch, mnl, mnh;  // 6-bit scales of sub-blocks 0-3, 4-7; mins likewise; one byte each
};
__device__ __forceinline__ ScaleWords unpack_scales(const uint4& hdr) {
  const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
  ScaleWords s;
  s.scl = u0 & 0x3f3f3f3fu;
  s.mnl = u1 & 0x3f3f3f3fu;
  s.sch = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
  s.mnh = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
  return s;
}

// eight activations of one lane, as loaded
template <typename XT>
struct XRaw {
  uint4 a, b;  // b only for float
};
template <typename XT>
__device__ __forceinline__ XRaw<XT> x_load(const XT* p) {
  XRaw<XT> r;
  r.a = __ldg(reinterpret_cast<const uint4*>(p));
  if constexpr (std::is_same<XT, float>::value) r.b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  else r.b = r.a;
  return r;
}
template <typename XT>
__device__ __forceinline__ void x_unpack(const XRaw<XT>& r, float (&v)[8]) {
  if constexpr (std::is_same<XT, float>::value) {
    const uint32_t f[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(f[i])));
  } else {
    const uint32_t w4[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 f;
      if constexpr (std::is_same<XT, __half>::value) f = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
      else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
}

// grid.x CTAs; CTA b takes the row blocks b, b + grid.x, ... of rpc <= 32 rows each (n_blocks in all).
template <typename XT, int MX>
__global__ void __launch_bounds__(kImThreads, 2)
gemv_q4k_imma_kernel(const GemvArgs a, const int D, const int rpc, const int n_blocks) {
  using OT = typename std::conditional<std::is_same<XT, __half>::value, __half, __nv_bfloat16>::type;
  __shared__ float red[2][kImWarps][MX][kImRows];
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K, nchunks = K >> 8;
  uint8_t* planes = dyn_smem + kImWarps * D * kImSlot;              // plane 2m: high bytes of row m, 2m + 1: low
  float* XS = reinterpret_cast<float*>(planes + 2 * MX * K);         // [MX][K / 32] sums of the sub-blocks
  float* SX = XS + MX * (K / 32);                                    // [MX][K / 256] scale of each superblock
  const int per = (nchunks + kImWarps - 1) / kImWarps;
  const int ch0 = min(warp * per, nchunks), ch1 = min(ch0 + per, nchunks);
  const int perw = ch1 - ch0;                                        // superblock columns of this warp
  const int my_blocks = ((int)blockIdx.x < n_blocks) ? (n_blocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total = my_blocks * perw;                                // slots this warp consumes

  // Per-warp ring of D slots (one superblock column x 32 rows each); every issue() commits exactly one group.
  uint8_t* ring = dyn_smem + warp * D * kImSlot;
  // piece j = lane + 32 i (288 pieces of 16 bytes per slot) is piece j % 9 of row r = j / 9: it comes from
  // r * row_bytes + 16 (j - 9 r) and goes to r * 160 + 16 (j - 9 r) = 16 (j + r)
  int rr[9];
#pragma unroll
  for (int i = 0; i < 9; i++) rr[i] = (lane + 32 * i) / 9;
  const int row_gap = (int)a.row_bytes - 144;
  int q_issue = 0, blk_issue = 0, sb_issue = ch0;
  auto issue = [&]() {
    if (q_issue < total) {
      const int brow0 = ((int)blockIdx.x + blk_issue * (int)gridDim.x) * rpc;
      const int rows = min(rpc, a.N - brow0);
      const uint8_t* base = a.w + (long long)brow0 * a.row_bytes + (long long)sb_issue * 144;
      uint8_t* slot = ring + (q_issue % D) * kImSlot;
#pragma unroll
      for (int i = 0; i < 9; i++)  // rows past the block stay unset
        if (rr[i] < rows) im_cp16(slot + 16 * (lane + 32 * i + rr[i]), base + (rr[i] * row_gap + 16 * (lane + 32 * i)));
      q_issue++;
      if (++sb_issue == ch1) {
        sb_issue = ch0;
        blk_issue++;
      }
    }
    im_commit();
  };
  for (int d = 0; d < D; d++) issue();
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");  // activations may come from the kernel before this one

  // ---- quantize the activations: one warp per superblock, eight values per lane, the next load in flight
#pragma unroll 1
  for (int m = 0; m < MX; m++) {
    const XT* xrow = static_cast<const XT*>(a.x) + (long long)m * a.x_row_stride + lane * 8;
    XRaw<XT> cur{};
    if (warp < nchunks) cur = x_load<XT>(xrow + warp * 256);
    for (int c = warp; c < nchunks; c += kImWarps) {
      XRaw<XT> nxt = cur;
      if (c + kImWarps < nchunks) nxt = x_load<XT>(xrow + (c + kImWarps) * 256);
      const int e0 = c * 256 + lane * 8;
      float v[8];
      x_unpack<XT>(cur, v);
      cur = nxt;
      float amax = 0.f, sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        amax = fmaxf(amax, fabsf(v[i]));
        sum += v[i];
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      // NaN must survive the maximum: fmaxf drops it, so carry it separately
      bool bad = !(amax < INFINITY);
#pragma unroll
      for (int i = 0; i < 8; i++) bad = bad || (v[i] != v[i]);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      bad = __any_sync(0xffffffffu, bad);
      const bool finite = amax > 0.f && !bad;
      const float inv = finite ? 32639.f * __frcp_rn(amax) : 0.f;
      uint32_t h[2] = {0u, 0u}, l[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int xi = __float2int_rn(v[i] * inv);
        h[i >> 2] |= ((uint32_t)((xi + 128) >> 8) & 0xffu) << (8 * (i & 3));
        l[i >> 2] |= ((uint32_t)xi & 0xffu) << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(planes + (2 * m) * K + e0) = make_uint2(h[0], h[1]);
      *reinterpret_cast<uint2*>(planes + (2 * m + 1) * K + e0) = make_uint2(l[0], l[1]);
      if (t == 0) XS[m * (K / 32) + c * 8 + g] = sum;
      // a superblock holding inf / nan: the products are 0 and the scale carries the non-finite value
      if (lane == 0) SX[m * nchunks + c] = finite ? amax * (1.f / 32639.f) : (bad ? __int_as_float(0x7fc00000) : 0.f);
    }
  }
  __syncthreads();

  const int mrow = MX == 1 ? 0 : min(t, MX - 1);     // activation row whose columns this lane holds
  const uint8_t* bplane = planes + min(g, 2 * MX - 1) * K + 8 * t;
  int q = 0;
  for (int blk = 0; blk < my_blocks; blk++) {
    float ydot[4] = {0.f, 0.f, 0.f, 0.f}, ymin[4] = {0.f, 0.f, 0.f, 0.f};  // weight rows g, g + 8, g + 16, g + 24
    for (int sb = ch0; sb < ch1; sb++, q++) {
      im_wait(D - 1);
      __syncwarp();
      const uint8_t* slot = ring + (q % D) * kImSlot;
      const uint8_t* bsb = bplane + sb * 256;
      const float sx = SX[mrow * nchunks + sb];
#pragma unroll
      for (int T = 0; T < 2; T++) {
        const uint8_t* rowA = slot + (16 * T + g) * kImRowStride;
        const uint8_t* rowB = rowA + 8 * kImRowStride;
        const uint4 hdrA = *reinterpret_cast<const uint4*>(rowA), hdrB = *reinterpret_cast<const uint4*>(rowB);
        const ScaleWords sA = unpack_scales(hdrA), sB = unpack_scales(hdrB);
        int ahA[2] = {0, 0}, alA[2] = {0, 0}, ahB[2] = {0, 0}, alB[2] = {0, 0};  // [low | high nibbles]
#pragma unroll
        for (int p = 0; p < 4; p++) {
          // 32 quant bytes: low nibbles are sub-block 2p, high nibbles sub-block 2p + 1; this lane holds bytes
          // 8t .. 8t + 7 of both rows, which are K-slots 4t .. 4t + 3 and 16 + 4t .. 16 + 4t + 3 of the fragment
          const uint2 wa = *reinterpret_cast<const uint2*>(rowA + 16 + 32 * p + 8 * t);
          const uint2 wb = *reinterpret_cast<const uint2*>(rowB + 16 + 32 * p + 8 * t);
          const uint32_t scwA = p < 2 ? sA.scl : sA.sch, scwB = p < 2 ? sB.scl : sB.sch;
          const uint2 bl = *reinterpret_cast<const uint2*>(bsb + 64 * p);
          const uint2 bh = *reinterpret_cast<const uint2*>(bsb + 64 * p + 32);
          int c[4];
          imma(c, wa.x & 0x0f0f0f0fu, wb.x & 0x0f0f0f0fu, wa.y & 0x0f0f0f0fu, wb.y & 0x0f0f0f0fu, bl.x, bl.y);
          int scA = byte_of(scwA, 2 * (p & 1)), scB = byte_of(scwB, 2 * (p & 1));
          ahA[0] += c[0] * scA;
          alA[0] += c[1] * scA;
          ahB[0] += c[2] * scB;
          alB[0] += c[3] * scB;
          imma(c, wa.x & 0xf0f0f0f0u, wb.x & 0xf0f0f0f0u, wa.y & 0xf0f0f0f0u, wb.y & 0xf0f0f0f0u, bh.x, bh.y);
          scA = byte_of(scwA, 2 * (p & 1) + 1);
          scB = byte_of(scwB, 2 * (p & 1) + 1);
          ahA[1] += c[0] * scA;
          alA[1] += c[1] * scA;
          ahB[1] += c[2] * scB;
          alB[1] += c[3] * scB;
        }
        const float2 ddA = __half22float2(*reinterpret_cast<const __half2*>(&hdrA.x));  // (d, dmin)
        const float2 ddB = __half22float2(*reinterpret_cast<const __half2*>(&hdrB.x));
        const float fA = fmaf((float)ahA[0], 256.f, (float)alA[0]) + fmaf((float)ahA[1], 256.f, (float)alA[1]) * 0.0625f;
        const float fB = fmaf((float)ahB[0], 256.f, (float)alB[0]) + fmaf((float)ahB[1], 256.f, (float)alB[1]) * 0.0625f;
        ydot[2 * T] = fmaf(ddA.x * sx, fA, ydot[2 * T]);
        ydot[2 * T + 1] = fmaf(ddB.x * sx, fB, ydot[2 * T + 1]);
        if constexpr (MX == 1) {
          // the mins of sub-blocks 2t and 2t + 1 are this lane's share; the quad is summed at the end
          const float2 xs = *reinterpret_cast<const float2*>(XS + sb * 8 + 2 * t);
          const uint32_t mwA = (t & 2) ? sA.mnh : sA.mnl, mwB = (t & 2) ? sB.mnh : sB.mnl;
          const int sh = 16 * (t & 1);
          const float mA = fmaf((float)((mwA >> (sh + 8)) & 0xffu), xs.y, (float)((mwA >> sh) & 0xffu) * xs.x);
          const float mB = fmaf((float)((mwB >> (sh + 8)) & 0xffu), xs.y, (float)((mwB >> sh) & 0xffu) * xs.x);
          ymin[2 * T] = fmaf(ddA.y, mA, ymin[2 * T]);
          ymin[2 * T + 1] = fmaf(ddB.y, mB, ymin[2 * T + 1]);
        } else {
          const float4* xs4 = reinterpret_cast<const float4*>(XS + mrow * (K / 32) + sb * 8);
          const float4 x0 = xs4[0], x1 = xs4[1];
          const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          float mA = 0.f, mB = 0.f;
#pragma unroll
          for (int j = 0; j < 8; j++) {
            mA = fmaf((float)byte_of(j < 4 ? sA.mnl : sA.mnh, j & 3), xv[j], mA);
            mB = fmaf((float)byte_of(j < 4 ? sB.mnl : sB.mnh, j & 3), xv[j], mB);
          }
          ymin[2 * T] = fmaf(ddA.y, mA, ymin[2 * T]);
          ymin[2 * T + 1] = fmaf(ddB.y, mB, ymin[2 * T + 1]);
        }
      }
      __syncwarp();  // the slot is free again
      issue();
    }

    // ---- block result: columns 2m, 2m + 1 of the fragments live in lanes t = m
    float(*rb)[MX][kImRows] = red[blk & 1];
    if constexpr (MX == 1) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        float v = (t == 0 ? ydot[i] : 0.f) - ymin[i];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (t == 0) rb[warp][0][g + 8 * i] = v;
      }
    } else {
      if (t < MX) {
#pragma unroll
        for (int i = 0; i < 4; i++) rb[warp][t][g + 8 * i] = ydot[i] - ymin[i];
      }
    }
    __syncthreads();  // one barrier per block: the buffer written two blocks later was read before the next barrier
    const int brow0 = ((int)blockIdx.x + blk * (int)gridDim.x) * rpc;
    if (warp < MX && lane < rpc && brow0 + lane < a.N) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kImWarps; w++) sum += rb[w][warp][lane];
      OT* out = static_cast<OT*>(a.y) + (long long)warp * a.y_row_stride + brow0 + lane;
      if constexpr (std::is_same<OT, __half>::value) *out = __float2half_rn(sum);
      else *out = __float2bfloat16_rn(sum);
    }
  }
}

template <typename XT, int MX>
cudaError_t launch_imma(const GemvArgs& a, cudaStream_t st) {
  const int nchunks = a.K >> 8;
  const int per = (nchunks + kImWarps - 1) / kImWarps;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_imma_kernel<XT, MX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         im_dyn_smem(kImMaxK, 2, MX));
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  // Up to one 32-row block per SM: one CTA per block, rows spread over all 148 SMs (28 each for N = 4096), which
  // leaves the second CTA slot of every SM to the next launch's prefetch. Up to two blocks per SM: one CTA per
  // block. Larger matrices: 296 persistent CTAs (two per SM) that share the blocks evenly: `waves` blocks each,
  // of as many rows as that takes (measured: [14336, 4096] 11.8 -> 10.5 us).
  int rpc = kImRows, grid;
  const int blocks32 = (a.N + kImRows - 1) / kImRows;
  if (blocks32 <= 296) {
    if (blocks32 < 148 && a.N >= 148 * 16) rpc = (a.N + 147) / 148;
    grid = (a.N + rpc - 1) / rpc;
  } else {
    const int waves = (blocks32 + 295) / 296;
    rpc = (a.N + 296 * waves - 1) / (296 * waves);
    grid = std::min((a.N + rpc - 1) / rpc, 296);
  }
  const int n_blocks = (a.N + rpc - 1) / rpc;
  const int D = (per * ((n_blocks + grid - 1) / grid)) < 2 ? 1 : 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kImThreads);
  cfg.dynamicSmemBytes = im_dyn_smem(a.K, D, MX);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, gemv_q4k_imma_kernel<XT, MX>, a, D, rpc, n_blocks);
}

template <typename XT>
cudaError_t launch_imma_rows(const GemvArgs& a, cudaStream_t st) {
  if (a.M == 1) return launch_imma<XT, 1>(a, st);
  if (a.M == 2) return launch_imma<XT, 2>(a, st);
  return cudaErrorInvalidValue;
}

}  // namespace

bool gemv_imma_supported(int codec, int x_dtype, const GemvArgs& a) {
  (void)x_dtype;
  return codec == Q4_K && a.tasks == nullptr && a.M >= 1 && a.M <= 2 && a.w_align16 != 0 && (a.K & 255) == 0 &&
         a.K <= kImMaxK && (a.row_bytes & 15) == 0 && (a.x_row_stride & 7) == 0 &&
         (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && a.out_bf16 == 0;
}

cudaError_t launch_gemv_imma(int x_dtype, const GemvArgs& a, cudaStream_t st) {
  if (x_dtype == F16) return launch_imma_rows<__half>(a, st);
  if (x_dtype == BF16) return launch_imma_rows<__nv_bfloat16>(a, st);
  return launch_imma_rows<float>(a, st);
}

}  // namespace kq
