// Building blocks of the q4_k decode kernels on the integer tensor pipe (mma.sync.m16n8k32, u8 x s8 -> s32),
// shared by the one-wave dense kernel (kq_gemv_stream.cu) and the mixture-of-experts decode kernels
// (kq_moe_decode.cu): bulk copies into shared memory, the 16-bit quantization of an activation superblock into
// two signed byte planes, and the product of 16-row weight fragments with one superblock.
//
// Arithmetic (decode being reproduced: src/kquant_cpu_decode.cpp:177-202): the activations of a superblock are
// xi = rint(x * 32639 / amax) = 256 xh + xl; every instruction multiplies sixteen weight rows x one 32-weight
// sub-block by the planes (columns 2 m and 2 m + 1 of the B operand belong to activation row m); the exact integer
// dot products are weighted by the 6-bit sub-block scales in integer arithmetic and turned to float once per
// superblock: y += d * sx * sum_j sc_j dot_j - dmin * sum_j mn_j xsum_j.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

namespace kq {

__device__ __forceinline__ uint32_t st_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void st_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(st_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void st_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(st_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool st_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok)
               : "r"(st_smem(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// plain bulk copy global -> this CTA's shared memory (16-byte aligned addresses, size a multiple of 16)
__device__ __forceinline__ void st_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   st_smem(dst)),
               "l"(src), "r"(bytes), "r"(st_smem(bar))
               : "memory");
}
__device__ __forceinline__ unsigned long long st_gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// L2 load: the activations are read twice, before and after the preceding kernel has finished; the second
// read must not be served from a line the first one left in L1
__device__ __forceinline__ uint4 st_ld_cg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// D(16 x 8, s32) = A(16 x 32, u8, row) * B(32 x 8, s8, col)
__device__ __forceinline__ void st_imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ int st_byte(uint32_t v, int j) { return (int)__byte_perm(v, 0u, 0x4440u + j); }

// Quantize superblock sb (eight values per lane, as loaded): maximum and non-finite test on packed halves,
// rounding by the float32 magic constant (the integer sits in the low mantissa bits).
template <typename XT>
__device__ __forceinline__ void st_quantize(const uint4 raw, int sb, int lane, int K, uint8_t* planes, float* XS,
                                            float* SX) {
  const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
  uint32_t am;
  if constexpr (std::is_same<XT, __half>::value) {
    __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t ab = w4[i] & 0x7fff7fffu;
      m2 = __hmax2_nan(m2, *reinterpret_cast<const __half2*>(&ab));
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
    am = __float_as_uint(__half2float(__hmax_nan(__low2half(m2), __high2half(m2))));  // NaN if any value is NaN
  } else {
    // bfloat16: the magnitude bits of the two halves of a word order like unsigned integers (NaN above inf)
    uint32_t m = 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t ab = w4[i] & 0x7fff7fffu;
      m = max(m, max(ab << 16, ab & 0xffff0000u));
      v[2 * i] = __uint_as_float(w4[i] << 16);
      v[2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
    }
    am = m;
  }
  float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  // non-negative floats order like unsigned integers, NaN above inf: the maximum keeps a non-finite value
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) am = max(am, __shfl_xor_sync(0xffffffffu, am, o));
  const float amax = __uint_as_float(am);
  const bool finite = am > 0u && am < 0x7f800000u;
  const float inv = finite ? 32639.f * __frcp_rn(amax) : 0.f;
  uint32_t yi[8], xi[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    xi[i] = __float_as_uint(fmaf(v[i], inv, 12582912.f));          // low 16 bits: two's complement of rint(v * inv)
    yi[i] = __float_as_uint(fmaf(v[i], inv, 12582912.f + 128.f));  // ... of rint(v * inv) + 128
  }
  // high plane = byte 1 of xi + 128, low plane = byte 0 of xi: xi = 256 xh + (int8)xl
  const uint32_t h0 = __byte_perm(__byte_perm(yi[0], yi[1], 0x0051), __byte_perm(yi[2], yi[3], 0x0051), 0x5410);
  const uint32_t h1 = __byte_perm(__byte_perm(yi[4], yi[5], 0x0051), __byte_perm(yi[6], yi[7], 0x0051), 0x5410);
  const uint32_t l0 = __byte_perm(__byte_perm(xi[0], xi[1], 0x0040), __byte_perm(xi[2], xi[3], 0x0040), 0x5410);
  const uint32_t l1 = __byte_perm(__byte_perm(xi[4], xi[5], 0x0040), __byte_perm(xi[6], xi[7], 0x0040), 0x5410);
  const int e0 = sb * 256 + lane * 8;
  *reinterpret_cast<uint2*>(planes + e0) = make_uint2(h0, h1);
  *reinterpret_cast<uint2*>(planes + K + e0) = make_uint2(l0, l1);
  if ((lane & 3) == 0) XS[sb * 8 + (lane >> 2)] = sum;
  // a superblock holding inf / nan: the products are 0 and the scale carries the non-finite value
  if (lane == 0) SX[sb] = finite ? amax * (1.f / 32639.f) : (am != 0u ? __int_as_float(0x7fc00000) : 0.f);
}

struct StScales {
  uint32_t scl, sch, mnl, mnh;  // 6-bit scales of sub-blocks 0-3, 4-7; mins likewise; one byte each
};
__device__ __forceinline__ StScales st_unpack(const uint4& hdr) {
  const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
  StScales s;
  s.scl = u0 & 0x3f3f3f3fu;
  s.mnl = u1 & 0x3f3f3f3fu;
  s.sch = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
  s.mnh = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
  return s;
}

// NT row tiles x one superblock. blk[2 T], blk[2 T + 1]: the 144-byte blocks of the lane's two fragment rows of
// tile T; bsb: the lane's plane (high for g = 0, low otherwise) at the superblock + 8 t; xs: the eight
// sub-block sums. Adds to y[r] what this lane contributes to fragment row r: the dot part is complete in lanes
// t = 0, the min part is spread over the quad.
template <int NT>
__device__ __forceinline__ void st_unit(const uint8_t* const (&blk)[2 * NT], const uint8_t* bsb, const float* xs,
                                        float sx, int t, float (&y)[2 * NT]) {
  uint4 hdr[2 * NT];
  StScales sw[2 * NT];
#pragma unroll
  for (int r = 0; r < 2 * NT; r++) {
    hdr[r] = *reinterpret_cast<const uint4*>(blk[r]);
    sw[r] = st_unpack(hdr[r]);
  }
  int acc[2 * NT][4];  // [high plane | low plane] x [low-nibble | high-nibble sub-blocks]
#pragma unroll
  for (int r = 0; r < 2 * NT; r++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[r][j] = 0;
#pragma unroll
  for (int p = 0; p < 4; p++) {
    // 32 quant bytes: low nibbles are sub-block 2p, high nibbles sub-block 2p + 1; this lane holds bytes
    // 8t .. 8t + 7 of its rows, which are K-slots 4t .. 4t + 3 and 16 + 4t .. 16 + 4t + 3 of the fragment
    const uint2 bl = *reinterpret_cast<const uint2*>(bsb + 64 * p);
    const uint2 bh = *reinterpret_cast<const uint2*>(bsb + 64 * p + 32);
#pragma unroll
    for (int T = 0; T < NT; T++) {
      const uint2 wa = *reinterpret_cast<const uint2*>(blk[2 * T] + 16 + 32 * p + 8 * t);
      const uint2 wb = *reinterpret_cast<const uint2*>(blk[2 * T + 1] + 16 + 32 * p + 8 * t);
      const uint32_t scwA = p < 2 ? sw[2 * T].scl : sw[2 * T].sch, scwB = p < 2 ? sw[2 * T + 1].scl : sw[2 * T + 1].sch;
      int c[4], d[4];
      st_imma(c, wa.x & 0x0f0f0f0fu, wb.x & 0x0f0f0f0fu, wa.y & 0x0f0f0f0fu, wb.y & 0x0f0f0f0fu, bl.x, bl.y);
      st_imma(d, wa.x & 0xf0f0f0f0u, wb.x & 0xf0f0f0f0u, wa.y & 0xf0f0f0f0u, wb.y & 0xf0f0f0f0u, bh.x, bh.y);
      int scA = st_byte(scwA, 2 * (p & 1)), scB = st_byte(scwB, 2 * (p & 1));
      acc[2 * T][0] += c[0] * scA;
      acc[2 * T][1] += c[1] * scA;
      acc[2 * T + 1][0] += c[2] * scB;
      acc[2 * T + 1][1] += c[3] * scB;
      scA = st_byte(scwA, 2 * (p & 1) + 1);
      scB = st_byte(scwB, 2 * (p & 1) + 1);
      acc[2 * T][2] += d[0] * scA;  // high nibbles stay in place: 16 q, undone below
      acc[2 * T][3] += d[1] * scA;
      acc[2 * T + 1][2] += d[2] * scB;
      acc[2 * T + 1][3] += d[3] * scB;
    }
  }
  // the mins of sub-blocks 2t and 2t + 1 are this lane's share
  const float2 xv = *reinterpret_cast<const float2*>(xs + 2 * t);
  const int sh = 16 * (t & 1);
#pragma unroll
  for (int r = 0; r < 2 * NT; r++) {
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr[r].x));  // (d, dmin)
    const float f =
        fmaf((float)acc[r][0], 256.f, (float)acc[r][1]) + fmaf((float)acc[r][2], 256.f, (float)acc[r][3]) * 0.0625f;
    const uint32_t mw = (t & 2) ? sw[r].mnh : sw[r].mnl;
    const float m = fmaf((float)((mw >> (sh + 8)) & 0xffu), xv.y, (float)((mw >> sh) & 0xffu) * xv.x);
    y[r] += (t == 0 ? dd.x * sx * f : 0.f) - dd.y * m;
  }
}


// The same product for MX <= 4 activation rows at once: B columns 2 m and 2 m + 1 carry the planes of row m, so
// the instructions are those of one row. bsb: this lane's column (planes of row min(g / 2, MX - 1), high plane for
// even g) at the superblock + 8 t; xs: sub-block sums of row 0 at this superblock, row m at xs + m * xs_stride;
// sx: superblock scale of row 0, row m at sx[m * sx_stride].
// ydot[r]: dot part of fragment row r for activation row m = t (lanes t >= MX hold nothing useful);
// ymin[r][m]: this lane's share (sub-blocks 2 t, 2 t + 1) of the min part of fragment row r, activation row m -
// sum it over the quad at the end.
template <int NT, int MX>
__device__ __forceinline__ void st_unit_mx(const uint8_t* const (&blk)[2 * NT], const uint8_t* bsb, const float* xs,
                                           int xs_stride, const float* sx, int sx_stride, int t, float (&ydot)[2 * NT],
                                           float (&ymin)[2 * NT][MX]) {
  uint4 hdr[2 * NT];
  StScales sw[2 * NT];
#pragma unroll
  for (int r = 0; r < 2 * NT; r++) {
    hdr[r] = *reinterpret_cast<const uint4*>(blk[r]);
    sw[r] = st_unpack(hdr[r]);
  }
  int acc[2 * NT][4];
#pragma unroll
  for (int r = 0; r < 2 * NT; r++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[r][j] = 0;
#pragma unroll
  for (int p = 0; p < 4; p++) {
    const uint2 bl = *reinterpret_cast<const uint2*>(bsb + 64 * p);
    const uint2 bh = *reinterpret_cast<const uint2*>(bsb + 64 * p + 32);
#pragma unroll
    for (int T = 0; T < NT; T++) {
      const uint2 wa = *reinterpret_cast<const uint2*>(blk[2 * T] + 16 + 32 * p + 8 * t);
      const uint2 wb = *reinterpret_cast<const uint2*>(blk[2 * T + 1] + 16 + 32 * p + 8 * t);
      const uint32_t scwA = p < 2 ? sw[2 * T].scl : sw[2 * T].sch, scwB = p < 2 ? sw[2 * T + 1].scl : sw[2 * T + 1].sch;
      int c[4], d[4];
      st_imma(c, wa.x & 0x0f0f0f0fu, wb.x & 0x0f0f0f0fu, wa.y & 0x0f0f0f0fu, wb.y & 0x0f0f0f0fu, bl.x, bl.y);
      st_imma(d, wa.x & 0xf0f0f0f0u, wb.x & 0xf0f0f0f0u, wa.y & 0xf0f0f0f0u, wb.y & 0xf0f0f0f0u, bh.x, bh.y);
      int scA = st_byte(scwA, 2 * (p & 1)), scB = st_byte(scwB, 2 * (p & 1));
      acc[2 * T][0] += c[0] * scA;
      acc[2 * T][1] += c[1] * scA;
      acc[2 * T + 1][0] += c[2] * scB;
      acc[2 * T + 1][1] += c[3] * scB;
      scA = st_byte(scwA, 2 * (p & 1) + 1);
      scB = st_byte(scwB, 2 * (p & 1) + 1);
      acc[2 * T][2] += d[0] * scA;
      acc[2 * T][3] += d[1] * scA;
      acc[2 * T + 1][2] += d[2] * scB;
      acc[2 * T + 1][3] += d[3] * scB;
    }
  }
  const int sh = 16 * (t & 1);
  const float sxt = sx[min(t, MX - 1) * sx_stride];
  float2 xv[MX];
#pragma unroll
  for (int m = 0; m < MX; m++) xv[m] = *reinterpret_cast<const float2*>(xs + m * xs_stride + 2 * t);
#pragma unroll
  for (int r = 0; r < 2 * NT; r++) {
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr[r].x));  // (d, dmin)
    const float f =
        fmaf((float)acc[r][0], 256.f, (float)acc[r][1]) + fmaf((float)acc[r][2], 256.f, (float)acc[r][3]) * 0.0625f;
    ydot[r] = fmaf(dd.x * sxt, f, ydot[r]);
    const uint32_t mw = (t & 2) ? sw[r].mnh : sw[r].mnl;
    const float m0 = dd.y * (float)((mw >> sh) & 0xffu), m1 = dd.y * (float)((mw >> (sh + 8)) & 0xffu);
#pragma unroll
    for (int m = 0; m < MX; m++) ymin[r][m] = fmaf(m1, xv[m].y, fmaf(m0, xv[m].x, ymin[r][m]));
  }
}

}  // namespace kq
