// Skinny-M quantized matmul (decode regime, M <= 16 rows per weight matrix):
//   y[m, n] = sum_k x[m, k] * dequant(w)[n, k]
// replacing the reference's fused decode-then-dot CPU path
// (src/kquant_matmul.cpp:1104-1164 -> src/kquant_cpu_decode.cpp:1032-1065,
// 1254-1297) and, through GemvTask lists, its batched MoE decode
// (src/kquant_cpu_decode.cpp:1362-1527).
//
// The kernel is HBM-bound: every wire byte is read exactly once. Work layout:
// one CTA of 8 warps owns 16 consecutive weight rows; the warps split K in
// 256-weight chunks round-robin and their partial sums meet in shared memory.
// Inside a warp the 16 rows x 16 K-slice products run on mma.sync m16n8k16 with
// the WEIGHTS as the A operand (lane (g, t) holds rows g and g+8) and up to 8
// (or 16) activation rows as the B operand, so the cost per weight does not
// grow with M up to 16 and accumulation is fp32 throughout.
//
//  * gemv_q4k_f16_kernel (q4_k, fp16 activations): lane t of each quad owns
//    sub-block pair (2t, 2t+1) of the superblock, so it issues two 16-byte
//    loads of quants per row and unpacks only its own two 6-bit scales. The
//    A operand is the exact integer sc*q (<= 63*15, exact in fp16) built by one
//    HFMA2 from the 0x6400|q half trick; a second MMA chain with A = mn gives
//    sum(mn * x); the fp16 block scales d and dmin are applied in fp32 once per
//    superblock: y += d * sum(sc*q*x) - dmin * sum(mn*x).
//  * gemv_generic_kernel (every codec, f16 / bf16 / f32-as-bf16 activations):
//    decode8<> produces bit-exact fp32 weights which are rounded to fp16 (fp16
//    activations) or split into bf16 hi + lo (bf16 activations, two MMAs), so
//    the weight error stays below 2^-12 relative either way.
#include <type_traits>

#include "kq_common.cuh"
#include "kq_launch.h"

namespace kq {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Eight consecutive activations as four packed 16-bit pairs. p == nullptr
// (a padding row of the 8-wide B tile) yields zeros. float input is rounded to
// bf16 first, as the reference's op does before its matmul
// (src/kquant_ops.cpp:159-168).
template <typename XT>
__device__ __forceinline__ void load_x8(const XT* p, uint32_t (&r)[4]) {
  if (p == nullptr) {
    r[0] = r[1] = r[2] = r[3] = 0u;
    return;
  }
  if constexpr (sizeof(XT) == 2) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    r[0] = pack_bf2(a.x, a.y); r[1] = pack_bf2(a.z, a.w);
    r[2] = pack_bf2(b.x, b.y); r[3] = pack_bf2(b.z, b.w);
  }
}

struct TaskView {
  const uint8_t* w;
  int m;
};

// Resolve this CTA's row group into shared memory; returns false when the CTA
// has nothing to do (a task index at or beyond the device-side task count).
__device__ __forceinline__ bool resolve_task(const GemvArgs& a, int* s_xrow, int* s_yrow, TaskView& tv) {
  if (a.tasks != nullptr) {
    if (a.n_tasks_dev != nullptr && (int)blockIdx.y + a.task_offset >= *a.n_tasks_dev) return false;
    const GemvTask& t = a.tasks[blockIdx.y];
    tv.w = t.w;
    tv.m = t.m;
    if (threadIdx.x < 16) {
      s_xrow[threadIdx.x] = t.xrow[threadIdx.x];
      s_yrow[threadIdx.x] = t.yrow[threadIdx.x];
    }
  } else {
    const int r0 = blockIdx.y * 16;
    tv.w = a.w;
    tv.m = min(16, a.M - r0);
    if (threadIdx.x < 16) {
      s_xrow[threadIdx.x] = r0 + threadIdx.x;
      s_yrow[threadIdx.x] = r0 + threadIdx.x;
    }
  }
  __syncthreads();
  return tv.m > 0;
}

// Cross-warp sum of the per-warp D fragments and the store of the finished
// 16-row x (8*NT)-token tile. OT is the output element type.
template <int NT, typename OT>
__device__ __forceinline__ void reduce_store(float (&acc)[NT][4], float* red, const GemvArgs& a, const int* s_yrow,
                                             int m, int row0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  constexpr int kTile = NT * 8 * 16;
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int tok = nt * 8 + 2 * t + (i & 1);
      const int row = g + 8 * (i >> 1);
      red[warp * kTile + tok * 16 + row] = acc[nt][i];
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kTile; idx += kGemvThreads) {
    const int tok = idx >> 4, row = idx & 15;
    if (tok < m && row0 + row < a.N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; w++) s += red[w * kTile + idx];
      OT* y = static_cast<OT*>(a.y) + (long long)s_yrow[tok] * a.y_row_stride + row0 + row;
      if constexpr (sizeof(OT) == 2 && !std::is_same<OT, __half>::value) {
        *y = __float2bfloat16_rn(s);
      } else {
        *y = __float2half_rn(s);
      }
    }
  }
}

// ------------------------------------------------------------------ generic
template <int C, int A, typename XT, int NT>
__global__ void __launch_bounds__(kGemvThreads) gemv_generic_kernel(const GemvArgs a) {
  constexpr bool kHalf = std::is_same<XT, __half>::value;
  using OT = typename std::conditional<kHalf, __half, __nv_bfloat16>::type;
  constexpr int WPB = wpb_of(C), BPB = bpb_of(C);
  __shared__ int s_xrow[16], s_yrow[16];
  __shared__ float red[kGemvWarps * NT * 8 * 16];
  __shared__ __align__(16) uint8_t s_tabs[kIqSmemBytes];

  IqTables tabs{};
  if constexpr (C == IQ4_NL || C == IQ4_XS || C == IQ2_XXS) {
    tabs = stage_iq_tables(s_tabs, threadIdx.x, kGemvThreads);
  }
  TaskView tv;
  if (!resolve_task(a, s_xrow, s_yrow, tv)) return;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  const uint8_t* pA = tv.w + (long long)min(row0 + g, a.N - 1) * a.row_bytes;
  const uint8_t* pB = tv.w + (long long)min(row0 + g + 8, a.N - 1) * a.row_bytes;
  const XT* xp[NT];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const int tok = nt * 8 + g;
    xp[nt] = tok < tv.m ? static_cast<const XT*>(a.x) + (long long)s_xrow[tok] * a.x_row_stride : nullptr;
  }

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[nt][i] = 0.f;

  const int ngroups = a.K / 32;  // 32-weight groups along K
  for (int g0 = warp * 8; g0 < ngroups; g0 += kGemvWarps * 8) {
#pragma unroll 2
    for (int G = 0; G < 8; G++) {
      const int gi = g0 + G;
      if (gi >= ngroups) break;
      long long boff;
      int oct;
      if constexpr (WPB == 256) {
        boff = (long long)(gi >> 3) * BPB;
        oct = (gi & 7) * 4 + t;
      } else {
        boff = (long long)gi * BPB;
        oct = t;
      }
      float va[8], vb[8];
      decode8<C, A>(pA + boff, oct, va, tabs);
      decode8<C, A>(pB + boff, oct, vb, tabs);
      uint32_t xb[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; nt++) load_x8<XT>(xp[nt] ? xp[nt] + gi * 32 + t * 8 : nullptr, xb[nt]);
      uint32_t ha[4], hb[4];
      if constexpr (kHalf) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          ha[i] = pack_h2(va[2 * i], va[2 * i + 1]);
          hb[i] = pack_h2(vb[2 * i], vb[2 * i + 1]);
        }
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
            mma_f16(acc[nt], ha[2 * s], hb[2 * s], ha[2 * s + 1], hb[2 * s + 1], xb[nt][2 * s], xb[nt][2 * s + 1]);
      } else {
        uint32_t la[4], lb[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const __nv_bfloat162 h1 = __floats2bfloat162_rn(va[2 * i], va[2 * i + 1]);
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(vb[2 * i], vb[2 * i + 1]);
          ha[i] = *reinterpret_cast<const uint32_t*>(&h1);
          hb[i] = *reinterpret_cast<const uint32_t*>(&h2);
          la[i] = pack_bf2(va[2 * i] - __low2float(h1), va[2 * i + 1] - __high2float(h1));
          lb[i] = pack_bf2(vb[2 * i] - __low2float(h2), vb[2 * i + 1] - __high2float(h2));
        }
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            mma_bf16(acc[nt], ha[2 * s], hb[2 * s], ha[2 * s + 1], hb[2 * s + 1], xb[nt][2 * s], xb[nt][2 * s + 1]);
            mma_bf16(acc[nt], la[2 * s], lb[2 * s], la[2 * s + 1], lb[2 * s + 1], xb[nt][2 * s], xb[nt][2 * s + 1]);
          }
      }
    }
  }
  reduce_store<NT, OT>(acc, red, a, s_yrow, tv.m, row0);
}

// ------------------------------------------------------------------ q4_k, fp16
// (1024 + q) pairs from one byte pair: bytes {i, i+1} of `nib` (each holding a
// 4-bit value) become the low bytes of two halves whose high byte is 0x64.
__device__ __forceinline__ uint32_t h2_magic01(uint32_t nib) { return __byte_perm(nib, 0x64646464u, 0x4140); }
__device__ __forceinline__ uint32_t h2_magic23(uint32_t nib) { return __byte_perm(nib, 0x64646464u, 0x4342); }

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, __half2 b, __half2 c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), b, c);
  return *reinterpret_cast<uint32_t*>(&r);
}

struct Q4kRow {
  __half2 sc0, off0, sc1, off1;  // sub-blocks 2t and 2t+1: scale and -1024*scale, both lanes of a half2
  uint32_t mn0, mn1;             // the two mins as half2 broadcasts
  float d, dmin;
};

__device__ __forceinline__ Q4kRow q4k_row_prep(const uint4& hdr, int t) {
  Q4kRow r;
  r.d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
  r.dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
  uint32_t sc0, mn0, sc1, mn1;
  k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * t, sc0, mn0);
  k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * t + 1, sc1, mn1);
  const __half2 m1024 = __float2half2_rn(-1024.f);
  r.sc0 = __half2half2(__ushort2half_rn((unsigned short)sc0));
  r.sc1 = __half2half2(__ushort2half_rn((unsigned short)sc1));
  r.off0 = __hmul2(r.sc0, m1024);
  r.off1 = __hmul2(r.sc1, m1024);
  const __half2 m0 = __half2half2(__ushort2half_rn((unsigned short)mn0));
  const __half2 m1 = __half2half2(__ushort2half_rn((unsigned short)mn1));
  r.mn0 = *reinterpret_cast<const uint32_t*>(&m0);
  r.mn1 = *reinterpret_cast<const uint32_t*>(&m1);
  return r;
}

template <int NT>
__global__ void __launch_bounds__(kGemvThreads) gemv_q4k_f16_kernel(const GemvArgs a) {
  __shared__ int s_xrow[16], s_yrow[16];
  __shared__ float red[kGemvWarps * NT * 8 * 16];
  TaskView tv;
  if (!resolve_task(a, s_xrow, s_yrow, tv)) return;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  const uint8_t* pA = tv.w + (long long)min(row0 + g, a.N - 1) * a.row_bytes;
  const uint8_t* pB = tv.w + (long long)min(row0 + g + 8, a.N - 1) * a.row_bytes;
  const __half* xp[NT];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const int tok = nt * 8 + g;
    xp[nt] = tok < tv.m ? static_cast<const __half*>(a.x) + (long long)s_xrow[tok] * a.x_row_stride + 64 * t
                        : nullptr;
  }

  float fin[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) fin[nt][i] = 0.f;

  const int nsb = a.K >> 8;
#pragma unroll 2
  for (int sb = warp; sb < nsb; sb += kGemvWarps) {
    const uint4* bA = reinterpret_cast<const uint4*>(pA + (long long)sb * 144);
    const uint4* bB = reinterpret_cast<const uint4*>(pB + (long long)sb * 144);
    // quants of sub-block pair t: bytes [32t, 32t+32) of the 128
    const uint4 qa0 = __ldg(bA + 1 + 2 * t), qa1 = __ldg(bA + 2 + 2 * t);
    const uint4 qb0 = __ldg(bB + 1 + 2 * t), qb1 = __ldg(bB + 2 + 2 * t);
    const uint4 hA = __ldg(bA), hB = __ldg(bB);
    const Q4kRow ra = q4k_row_prep(hA, t), rb = q4k_row_prep(hB, t);
    const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};

    float accq[NT][4], accm[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int i = 0; i < 4; i++) accq[nt][i] = accm[nt][i] = 0.f;

#pragma unroll
    for (int ip = 0; ip < 4; ip++) {  // two words (8 weights per sub-block) per step
      uint32_t x0[NT][4], x1[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        load_x8<__half>(xp[nt] ? xp[nt] + sb * 256 + ip * 8 : nullptr, x0[nt]);        // sub-block 2t
        load_x8<__half>(xp[nt] ? xp[nt] + sb * 256 + 32 + ip * 8 : nullptr, x1[nt]);   // sub-block 2t+1
      }
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const uint32_t Wa = wa[2 * ip + h], Wb = wb[2 * ip + h];
        const uint32_t la = Wa & 0x0f0f0f0fu, ua = (Wa >> 4) & 0x0f0f0f0fu;
        const uint32_t lb = Wb & 0x0f0f0f0fu, ub = (Wb >> 4) & 0x0f0f0f0fu;
        // sub-block 2t (low nibbles)
        const uint32_t a0 = hfma2_u(h2_magic01(la), ra.sc0, ra.off0), a2 = hfma2_u(h2_magic23(la), ra.sc0, ra.off0);
        const uint32_t a1 = hfma2_u(h2_magic01(lb), rb.sc0, rb.off0), a3 = hfma2_u(h2_magic23(lb), rb.sc0, rb.off0);
        // sub-block 2t+1 (high nibbles)
        const uint32_t c0 = hfma2_u(h2_magic01(ua), ra.sc1, ra.off1), c2 = hfma2_u(h2_magic23(ua), ra.sc1, ra.off1);
        const uint32_t c1 = hfma2_u(h2_magic01(ub), rb.sc1, rb.off1), c3 = hfma2_u(h2_magic23(ub), rb.sc1, rb.off1);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          mma_f16(accq[nt], a0, a1, a2, a3, x0[nt][2 * h], x0[nt][2 * h + 1]);
          mma_f16(accm[nt], ra.mn0, rb.mn0, ra.mn0, rb.mn0, x0[nt][2 * h], x0[nt][2 * h + 1]);
          mma_f16(accq[nt], c0, c1, c2, c3, x1[nt][2 * h], x1[nt][2 * h + 1]);
          mma_f16(accm[nt], ra.mn1, rb.mn1, ra.mn1, rb.mn1, x1[nt][2 * h], x1[nt][2 * h + 1]);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      fin[nt][0] += ra.d * accq[nt][0] - ra.dmin * accm[nt][0];
      fin[nt][1] += ra.d * accq[nt][1] - ra.dmin * accm[nt][1];
      fin[nt][2] += rb.d * accq[nt][2] - rb.dmin * accm[nt][2];
      fin[nt][3] += rb.d * accq[nt][3] - rb.dmin * accm[nt][3];
    }
  }
  reduce_store<NT, __half>(fin, red, a, s_yrow, tv.m, row0);
}

// ------------------------------------------------------------------ launch
template <int C, int NAT>
static cudaError_t launch_generic(int x_dtype, const GemvArgs& a, dim3 grid, bool nt2, bool aligned, cudaStream_t st) {
#define KQ_GV(AL, XT)                                                             \
  do {                                                                            \
    if (nt2) gemv_generic_kernel<C, AL, XT, 2><<<grid, kGemvThreads, 0, st>>>(a); \
    else gemv_generic_kernel<C, AL, XT, 1><<<grid, kGemvThreads, 0, st>>>(a);     \
    return cudaGetLastError();                                                    \
  } while (0)
  if (aligned) {
    if (x_dtype == F16) KQ_GV(NAT, __half);
    if (x_dtype == BF16) KQ_GV(NAT, __nv_bfloat16);
    KQ_GV(NAT, float);
  } else {
    if (x_dtype == F16) KQ_GV(1, __half);
    if (x_dtype == BF16) KQ_GV(1, __nv_bfloat16);
    KQ_GV(1, float);
  }
#undef KQ_GV
}

cudaError_t launch_gemv(int codec, int x_dtype, const GemvArgs& a, cudaStream_t st) {
  if (a.N <= 0 || a.K <= 0) return cudaSuccess;
  const int groups = a.tasks ? a.n_tasks : (a.M + 15) / 16;
  if (groups <= 0) return cudaSuccess;
  if (groups > 65535) return cudaErrorInvalidConfiguration;
  const dim3 grid((a.N + 15) / 16, groups);
  const bool nt2 = a.tasks ? true : (a.M > 8);
  // Block starts keep their natural alignment when the base pointer is 16-byte
  // aligned and rows are a whole number of blocks (always true).
  const bool aligned = a.w_align16 != 0;

  if (codec == Q4_K && x_dtype == F16 && aligned) {
    if (nt2) gemv_q4k_f16_kernel<2><<<grid, kGemvThreads, 0, st>>>(a);
    else gemv_q4k_f16_kernel<1><<<grid, kGemvThreads, 0, st>>>(a);
    return cudaGetLastError();
  }
  switch (codec) {
    case Q2_K: return launch_generic<Q2_K, 4>(x_dtype, a, grid, nt2, aligned, st);
    case Q3_K: return launch_generic<Q3_K, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q4_K: return launch_generic<Q4_K, 16>(x_dtype, a, grid, nt2, aligned, st);
    case Q5_K: return launch_generic<Q5_K, 16>(x_dtype, a, grid, nt2, aligned, st);
    case Q6_K: return launch_generic<Q6_K, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q4_0: return launch_generic<Q4_0, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q8_0: return launch_generic<Q8_0, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ4_NL: return launch_generic<IQ4_NL, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ4_XS: return launch_generic<IQ4_XS, 8>(x_dtype, a, grid, nt2, aligned, st);
    case IQ2_XXS: return launch_generic<IQ2_XXS, 2>(x_dtype, a, grid, nt2, aligned, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace kq
