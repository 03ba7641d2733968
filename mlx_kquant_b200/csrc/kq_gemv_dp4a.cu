// Decode products for one to four activation rows on the integer dot-product pipe, for the codecs
// that have no tensor-core fast path: q2_k q3_k q5_k q6_k q4_0 q8_0 iq4_nl iq4_xs iq2_xxs.
//
// Every one of these formats stores small integers times a per-group scale (minus a per-group
// minimum for q2_k / q5_k; iq2_xxs: signed 8-weight lattice points), src/kquant_cpu_decode.cpp:50-82,
// 205-377, 383-465, 557-584. So
//   y[n] = sum_groups  scale_g * sum_k (q_k - off) x_k  -  min_g * sum_k x_k
// and the inner sums run on dp4a once the activations are integers too: each 32-group of x is
// quantized once per CTA to 16 bits with the group's own scale (xi = rint(x * 32767 / max|x|),
// |error| <= 2^-16 of the group maximum - far below the fp16 / bf16 rounding the activations
// already carry) and stored as two int8 planes (xi = 256 xh + xl). A few logic ops unpack FOUR
// weights into one register, one dp4a per plane multiplies them; integer sums are exact, scales are
// applied in fp32 per 16- or 32-weight sub-group. "- off" costs nothing: off * sum_k xi is taken
// from the per-16 integer sums of x.
//
// Thread = weight row (a warp owns 32 rows); the eight warps of a CTA split K in 256-weight
// chunks and meet in shared memory. Wire bytes stream through a per-warp cp.async ring of
// 16-byte-aligned windows (chunk sizes such as 210 or 110 bytes are not multiples of 16; readers
// add the chunk's phase inside its window, which is the same for all rows of a warp).
#include <cstdlib>
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kq_common.cuh"
#include "kq_launch.h"

namespace kq {

namespace {

constexpr int kWarps = 8, kThreads = 32 * kWarps, kRows = 32;
constexpr int kMaxK = 16384;

__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_wait(int n) {  // at most n groups still pending
  if (n <= 0) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  else asm volatile("cp.async.wait_group 1;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
// signed weights x unsigned low plane
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ float f16_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// bytes of a 256-weight chunk and 16-byte pieces of its aligned window (odd: fewer bank conflicts)
template <int C>
struct Geom;
template <> struct Geom<Q2_K> { static constexpr int kCB = 84, kP = 7; };
template <> struct Geom<Q3_K> { static constexpr int kCB = 110, kP = 9; };
template <> struct Geom<Q4_K> { static constexpr int kCB = 144, kP = 9; };
template <> struct Geom<Q5_K> { static constexpr int kCB = 176, kP = 11; };
template <> struct Geom<Q6_K> { static constexpr int kCB = 210, kP = 15; };
template <> struct Geom<Q4_0> { static constexpr int kCB = 144, kP = 9; };
template <> struct Geom<Q8_0> { static constexpr int kCB = 272, kP = 17; };
template <> struct Geom<IQ4_NL> { static constexpr int kCB = 144, kP = 9; };
template <> struct Geom<IQ4_XS> { static constexpr int kCB = 136, kP = 9; };
template <> struct Geom<IQ2_XXS> { static constexpr int kCB = 66, kP = 5; };
template <> struct Geom<Q4_1> { static constexpr int kCB = 160, kP = 11; };
template <> struct Geom<Q5_0> { static constexpr int kCB = 176, kP = 11; };
template <> struct Geom<Q5_1> { static constexpr int kCB = 192, kP = 13; };

// The activations of one chunk for MT rows of x, as the products need them. Row t is t * stride further.
struct XChunk {
  const uint4* xh;    // 16 uint4: high bytes, four weights per word, a 16-group per uint4
  const uint4* xl;    // 16 uint4: low bytes
  const float* sg;    // 8: scale of each 32-group
  const int* xi16;    // 16: integer sum of each 16-group
  const float* xs16;  // 16: float sum of each 16-group
  int plane_stride;   // uint4 between rows of x in xh / xl
  int sg_stride, s16_stride;
};

// Reader of a chunk whose first byte sits PH2 (0 or 2) bytes after the 4-byte-aligned `base`.
template <int PH2>
struct Bytes {
  const uint32_t* base;
  __device__ __forceinline__ uint32_t w(int off) const {  // 32 bits at even byte offset `off`
    const int abs = off + PH2;
    if (abs & 2) return __funnelshift_r(base[abs >> 2], base[(abs >> 2) + 1], 16);
    return base[abs >> 2];
  }
  __device__ __forceinline__ uint32_t h(int off) const {  // 16 bits at even byte offset
    const int abs = off + PH2;
    return (base[abs >> 2] >> ((abs & 2) * 8)) & 0xffffu;
  }
  __device__ __forceinline__ uint32_t b(int off) const {  // one byte
    const int abs = off + PH2;
    return (base[abs >> 2] >> ((abs & 3) * 8)) & 0xffu;
  }
};

// dot of 16 weights (four words) with the two planes of x: exact integer sum_k q_k xi_k
template <bool SIGNED>
__device__ __forceinline__ int dot16(const uint32_t (&q)[4], const uint4 xh, const uint4 xl) {
  int hi = 0, lo = 0;
  const uint32_t h[4] = {xh.x, xh.y, xh.z, xh.w}, l[4] = {xl.x, xl.y, xl.z, xl.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    hi = dp4a_ss(q[i], h[i], hi);
    if constexpr (SIGNED) lo = dp4a_su(q[i], l[i], lo);
    else lo = (int)__dp4a(q[i], l[i], (unsigned)lo);
  }
  return hi * 256 + lo;
}

// acc[t] += scale * sum_k (q_k - off) x_k over 16-group g16, for every row t of x
template <bool SIGNED, int MT>
__device__ __forceinline__ void accum16(const uint32_t (&q)[4], int g16, float scale, int off, const XChunk& X,
                                        float (&acc)[MT]) {
#pragma unroll
  for (int t = 0; t < MT; t++) {
    int s = dot16<SIGNED>(q, X.xh[t * X.plane_stride + g16], X.xl[t * X.plane_stride + g16]);
    if (off != 0) s -= off * X.xi16[t * X.s16_stride + g16];
    acc[t] = fmaf(scale * X.sg[t * X.sg_stride + (g16 >> 1)], (float)s, acc[t]);
  }
}
// acc[t] -= mn * sum_k x_k over 16-group g16
template <int MT>
__device__ __forceinline__ void accum_min(int g16, float mn, const XChunk& X, float (&acc)[MT]) {
#pragma unroll
  for (int t = 0; t < MT; t++) acc[t] = fmaf(-mn, X.xs16[t * X.s16_stride + g16], acc[t]);
}

// ---- per-codec chunk products: adds this chunk's contribution to acc[t] ---------------------
// T: the 16-level table of the iq4 codecs in four registers; grid: the iq2_xxs lattice in shared memory.
template <int C, int PH2, int MT>
__device__ __forceinline__ void chunk_dot(const Bytes<PH2> B, const XChunk& X, const uint32_t (&T)[4],
                                          const uint2* grid, float (&acc)[MT]) {
  if constexpr (C == Q8_0) {
    // eight blocks [f16 d][32 x int8]
#pragma unroll
    for (int b = 0; b < 8; b++) {
      const float d = f16_bits(B.h(34 * b));
#pragma unroll
      for (int hlf = 0; hlf < 2; hlf++) {
        uint32_t q[4];
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = B.w(34 * b + 2 + 16 * hlf + 4 * i);
        accum16<true, MT>(q, 2 * b + hlf, d, 0, X, acc);
      }
    }
  } else if constexpr (C == Q4_0) {
    // eight blocks [f16 d][16 B]: low nibble -> weight i, high nibble -> weight i + 16, minus 8
#pragma unroll
    for (int b = 0; b < 8; b++) {
      const float d = f16_bits(B.h(18 * b));
      uint32_t lo[4], hi[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t W = B.w(18 * b + 2 + 4 * i);
        lo[i] = W & 0x0f0f0f0fu;
        hi[i] = (W >> 4) & 0x0f0f0f0fu;
      }
      accum16<false, MT>(lo, 2 * b, d, 8, X, acc);
      accum16<false, MT>(hi, 2 * b + 1, d, 8, X, acc);
    }
  } else if constexpr (C == Q4_1 || C == Q5_0 || C == Q5_1) {
    // eight blocks [f16 d]([f16 m])([u32 qh])[16 B]: nibbles as q4_0; bit i of qh is the fifth bit of weight i
    // (src/kquant_cpu_decode.cpp:84-153). q5_0 subtracts 16 through the integer sums of x, the codecs with a
    // minimum add m * sum x through the float sums.
    constexpr int kBlk = C == Q4_1 ? 20 : (C == Q5_0 ? 22 : 24);
    constexpr int kQs = C == Q4_1 ? 4 : (C == Q5_0 ? 6 : 8);
#pragma unroll
    for (int b = 0; b < 8; b++) {
      const float d = f16_bits(B.h(kBlk * b));
      uint32_t qh = 0;
      if constexpr (C == Q5_0) qh = B.w(kBlk * b + 2);
      if constexpr (C == Q5_1) qh = B.w(kBlk * b + 4);
      uint32_t lo[4], hi[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t W = B.w(kBlk * b + kQs + 4 * i);
        lo[i] = W & 0x0f0f0f0fu;
        hi[i] = (W >> 4) & 0x0f0f0f0fu;
        if constexpr (C != Q4_1) {
          // four consecutive bits of qh -> bit 4 of the four bytes
          lo[i] |= ((((qh >> (4 * i)) & 0xfu) * 0x00204081u) & 0x01010101u) << 4;
          hi[i] |= ((((qh >> (16 + 4 * i)) & 0xfu) * 0x00204081u) & 0x01010101u) << 4;
        }
      }
      accum16<false, MT>(lo, 2 * b, d, C == Q5_0 ? 16 : 0, X, acc);
      accum16<false, MT>(hi, 2 * b + 1, d, C == Q5_0 ? 16 : 0, X, acc);
      if constexpr (C != Q5_0) {
        const float m = f16_bits(B.h(kBlk * b + 2));
        accum_min<MT>(2 * b, -m, X, acc);
        accum_min<MT>(2 * b + 1, -m, X, acc);
      }
    }
  } else if constexpr (C == IQ4_NL || C == IQ4_XS) {
    // 16 bytes per 32-group: low nibble -> weight i, high nibble -> weight i + 16, through the 16-level
    // table. Two bytes = four nibbles = one byte-permute selector; the result bytes come out in the
    // order (i, i+16, i+1, i+17), which is the order the planes of x are stored in for these codecs.
    auto lut4 = [&](uint32_t Xs) {
      const uint32_t sel = Xs & 0x7777u;
      const uint32_t vlo = __byte_perm(T[0], T[1], sel), vhi = __byte_perm(T[2], T[3], sel);
      uint32_t m, v;
      asm("prmt.b32 %0, %1, %2, 0xD9C8;\n" : "=r"(m) : "r"(Xs << 4), "r"(Xs));  // bit 3 of each nibble -> byte mask
      asm("lop3.b32 %0, %1, %2, %3, 0xCA;\n" : "=r"(v) : "r"(m), "r"(vhi), "r"(vlo));
      return v;
    };
    float d = 0.f;
    uint32_t sh = 0, sl = 0;
    if constexpr (C == IQ4_XS) {
      d = f16_bits(B.h(0));
      sh = B.h(2);
      sl = B.w(4);
    }
#pragma unroll
    for (int g = 0; g < 8; g++) {
      const int qoff = (C == IQ4_XS) ? 8 + 16 * g : 18 * g + 2;
      float dl;
      if constexpr (C == IQ4_XS) {
        const int ls = (int)(((sl >> (4 * g)) & 15u) | (((sh >> (2 * g)) & 3u) << 4)) - 32;
        dl = d * (float)ls;
      } else {
        dl = f16_bits(B.h(18 * g));
      }
      uint32_t q0[4], q1[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t W = B.w(qoff + 4 * i);
        if (i < 2) {
          q0[2 * i] = lut4(W);
          q0[2 * i + 1] = lut4(W >> 16);
        } else {
          q1[2 * (i - 2)] = lut4(W);
          q1[2 * (i - 2) + 1] = lut4(W >> 16);
        }
      }
      accum16<true, MT>(q0, 2 * g, dl, 0, X, acc);
      accum16<true, MT>(q1, 2 * g + 1, dl, 0, X, acc);
    }
  } else if constexpr (C == IQ2_XXS) {
    // [f16 d][8 x (4 lattice-index bytes, u32: 4 x 7-bit sign field + 4-bit scale @28)]. A lattice entry is
    // eight bytes out of {8, 25, 43}; the eighth sign is the parity of the seven stored ones.
    const float d = f16_bits(B.h(0));
#pragma unroll
    for (int g = 0; g < 8; g++) {
      const uint32_t aux0 = B.w(2 + 8 * g), aux1 = B.w(6 + 8 * g);
      const float db = d * (0.5f + (float)(aux1 >> 28)) * 0.25f;
      uint32_t q[8];
#pragma unroll
      for (int l = 0; l < 4; l++) {
        const uint2 gv = grid[(aux0 >> (8 * l)) & 0xffu];
        const uint32_t s7 = (aux1 >> (7 * l)) & 127u;
        const uint32_t s8 = s7 | ((__popc(s7) & 1u) << 7);
        // sign bit -> 0x01 in its byte -> negate that byte: (v ^ 0xff) + 1 (bytes are 8..43: no carry out)
        const uint32_t b0 = ((s8 & 15u) * 0x00204081u) & 0x01010101u, b1 = ((s8 >> 4) * 0x00204081u) & 0x01010101u;
        q[2 * l] = (gv.x ^ (b0 * 255u)) + b0;
        q[2 * l + 1] = (gv.y ^ (b1 * 255u)) + b1;
      }
      const uint32_t qa[4] = {q[0], q[1], q[2], q[3]}, qb[4] = {q[4], q[5], q[6], q[7]};
      accum16<true, MT>(qa, 2 * g, db, 0, X, acc);
      accum16<true, MT>(qb, 2 * g + 1, db, 0, X, acc);
    }
  } else if constexpr (C == Q5_K || C == Q4_K) {
    // q4_k: [d][dmin][12 B scales][qs 128], low nibbles sub-block 2p, high nibbles 2p + 1;
    // q5_k: [d][dmin][12 B scales][qh 32][qs 128], plus bit s of qh[i] as the fifth bit of sub-block s
    const uint32_t hd = B.w(0);
    const float d = f16_bits(hd & 0xffffu), dmin = f16_bits(hd >> 16);
    const uint32_t u0 = B.w(4), u1 = B.w(8), u2 = B.w(12);
    const uint32_t scl = u0 & 0x3f3f3f3fu, mnl = u1 & 0x3f3f3f3fu;
    const uint32_t sch = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
    const uint32_t mnh = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
#pragma unroll
    for (int p = 0; p < 4; p++) {
      uint32_t lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const uint32_t W = B.w((C == Q5_K ? 48 : 16) + 32 * p + 4 * i), H = (C == Q5_K) ? B.w(16 + 4 * i) : 0u;
        // bit 2p of H -> bit 4 of the low-nibble weights, bit 2p+1 -> bit 4 of the high-nibble ones
        const uint32_t hl = (p <= 2) ? (H << ((p <= 2) ? 4 - 2 * p : 0)) : (H >> ((p > 2) ? 2 * p - 4 : 0));
        const uint32_t hh = (p <= 1) ? (H << ((p <= 1) ? 3 - 2 * p : 0)) : (H >> ((p > 1) ? 2 * p - 3 : 0));
        lo[i] = (W & 0x0f0f0f0fu) | (hl & 0x10101010u);
        hi[i] = ((W >> 4) & 0x0f0f0f0fu) | (hh & 0x10101010u);
      }
      const uint32_t la[4] = {lo[0], lo[1], lo[2], lo[3]}, lb[4] = {lo[4], lo[5], lo[6], lo[7]};
      const uint32_t ha[4] = {hi[0], hi[1], hi[2], hi[3]}, hb[4] = {hi[4], hi[5], hi[6], hi[7]};
      const uint32_t scw = p < 2 ? scl : sch, mnw = p < 2 ? mnl : mnh;
      const float sc_lo = d * (float)((scw >> (16 * (p & 1))) & 0xffu), sc_hi = d * (float)((scw >> (16 * (p & 1) + 8)) & 0xffu);
      const float mn_lo = dmin * (float)((mnw >> (16 * (p & 1))) & 0xffu), mn_hi = dmin * (float)((mnw >> (16 * (p & 1) + 8)) & 0xffu);
      accum16<false, MT>(la, 4 * p, sc_lo, 0, X, acc);
      accum16<false, MT>(lb, 4 * p + 1, sc_lo, 0, X, acc);
      accum16<false, MT>(ha, 4 * p + 2, sc_hi, 0, X, acc);
      accum16<false, MT>(hb, 4 * p + 3, sc_hi, 0, X, acc);
      accum_min<MT>(4 * p, mn_lo, X, acc);
      accum_min<MT>(4 * p + 1, mn_lo, X, acc);
      accum_min<MT>(4 * p + 2, mn_hi, X, acc);
      accum_min<MT>(4 * p + 3, mn_hi, X, acc);
    }
  } else if constexpr (C == Q6_K) {
    // [ql 128][qh 64][int8 sc 16][f16 d @208]: 16-weight scales, q - 32
    const float d = f16_bits(B.h(208));
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
#pragma unroll
      for (int qd = 0; qd < 4; qd++) {
        // 32 weights 128 hf + 32 qd + l: nibbles of ql[64 hf + 32 (qd & 1) + l], two bits 2 qd of qh[32 hf + l]
#pragma unroll
        for (int sub = 0; sub < 2; sub++) {
          uint32_t q[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint32_t L = B.w(64 * hf + 32 * (qd & 1) + 16 * sub + 4 * i);
            const uint32_t H = B.w(128 + 32 * hf + 16 * sub + 4 * i);
            const uint32_t nib = (qd & 2) ? (L >> 4) : L;
            const uint32_t hb = (qd < 2) ? (H << ((qd < 2) ? 4 - 2 * qd : 0)) : (H >> ((qd >= 2) ? 2 * qd - 4 : 0));
            q[i] = (nib & 0x0f0f0f0fu) | (hb & 0x30303030u);
          }
          const int g16 = 8 * hf + 2 * qd + sub;  // 16-group of the chunk = index of its scale
          accum16<false, MT>(q, g16, d * (float)(int)(int8_t)B.b(192 + g16), 32, X, acc);
        }
      }
    }
  } else if constexpr (C == Q2_K) {
    // [scales 16: 4-bit scale | 4-bit min << 4][qs 64][d @80][dmin @82]: 16-weight groups
    const uint32_t dd = B.w(80);
    const float d = f16_bits(dd & 0xffffu), dmin = f16_bits(dd >> 16);
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
#pragma unroll
      for (int si = 0; si < 4; si++) {
#pragma unroll
        for (int sub = 0; sub < 2; sub++) {
          uint32_t q[4];
#pragma unroll
          for (int i = 0; i < 4; i++) q[i] = (B.w(16 + 32 * hf + 16 * sub + 4 * i) >> (2 * si)) & 0x03030303u;
          const int g16 = 8 * hf + 2 * si + sub;
          const uint32_t scb = B.b(g16);
          accum16<false, MT>(q, g16, d * (float)(scb & 15u), 0, X, acc);
          accum_min<MT>(g16, dmin * (float)(scb >> 4), X, acc);
        }
      }
    }
  } else {
    static_assert(C == Q3_K, "codec without an integer dot-product path");
    // [hmask 32][qs 64][scales 12][d @108]: two bits of qs, bit 4 hf + si of hmask as the third, minus 4;
    // sixteen 6-bit scales minus 32: scale k takes its low four bits from byte k % 8 (low nibble for k < 8,
    // high nibble otherwise) and its high two bits from byte 8 + k % 4, shifted by 2 (k / 4)
    const float d = f16_bits(B.h(108));
    const uint32_t s0 = B.w(96), s1 = B.w(100), s2 = B.w(104);
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
#pragma unroll
      for (int si = 0; si < 4; si++) {
#pragma unroll
        for (int sub = 0; sub < 2; sub++) {
          uint32_t q[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint32_t Q = (B.w(32 + 32 * hf + 16 * sub + 4 * i) >> (2 * si)) & 0x03030303u;
            const uint32_t M = B.w(16 * sub + 4 * i);
            const int sh = 4 * hf + si;  // mask bit -> bit 2
            const uint32_t mb = (sh <= 2) ? (M << ((sh <= 2) ? 2 - sh : 0)) : (M >> ((sh > 2) ? sh - 2 : 0));
            q[i] = Q | (mb & 0x04040404u);
          }
          const int k = 8 * hf + 2 * si + sub;
          const uint32_t lw = (k & 4) ? s1 : s0;
          const uint32_t lo4 = ((lw >> (8 * (k & 3))) >> ((k & 8) ? 4 : 0)) & 15u;
          const uint32_t hi2 = ((s2 >> (8 * (k & 3))) >> (2 * (k >> 2))) & 3u;
          accum16<false, MT>(q, k, d * (float)((int)(lo4 | (hi2 << 4)) - 32), 4, X, acc);
        }
      }
    }
  }
}

// dyn smem: ring [8 warps][D][32 rows x 16 P] | per row of x: XH [K] | XL [K] | SG [K/32] | XI16 [K/16] | XS16 [K/16]
template <int C>
constexpr int slot_bytes() { return kRows * 16 * Geom<C>::kP; }
__host__ __device__ static inline int x_bytes(int K) { return 2 * K + (K / 32) * 4 + 2 * (K / 16) * 4; }
template <int C>
int dyn_smem(int K, int D, int MT) { return kWarps * D * slot_bytes<C>() + MT * x_bytes(K); }

template <int C, typename XT, int MT>
__global__ void __launch_bounds__(kThreads, 2) gemv_dp4a_kernel(const GemvArgs a, const int D) {
  using OT = typename std::conditional<std::is_same<XT, __half>::value, __half, __nv_bfloat16>::type;
  using G = Geom<C>;
  constexpr int kSlot = slot_bytes<C>(), kStride = 16 * G::kP;
  constexpr bool kPerm = (C == IQ4_NL || C == IQ4_XS);  // planes of x in the (i, i+16, i+1, i+17) order
  __shared__ float red[kWarps][MT][kRows];
  __shared__ __align__(16) uint2 s_grid[C == IQ2_XXS ? 256 : 1];
  extern __shared__ __align__(16) uint8_t dyn[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nchunks = a.K >> 8;
  const int K = a.K;
  uint8_t* xbase = dyn + kWarps * D * kSlot;
  const int xb = x_bytes(K);
  const int row0 = blockIdx.x * kRows;
  const int per = (nchunks + kWarps - 1) / kWarps;
  const int ch0 = min(warp * per, nchunks), ch1 = min(ch0 + per, nchunks);
  // dense: rows 0 .. M-1 of x against a.w; task list: task blockIdx.y, its rows MT blockIdx.z .. +MT-1
  int m = min(a.M, MT);
  const uint8_t* wmat = a.w;
  int xr[MT], yr[MT];
#pragma unroll
  for (int t = 0; t < MT; t++) xr[t] = yr[t] = t;
  if (a.tasks != nullptr) {
    if (a.n_tasks_dev != nullptr && (int)blockIdx.y + a.task_offset >= *a.n_tasks_dev) return;  // whole CTA
    const GemvTask& tk = a.tasks[blockIdx.y];
    const int t0 = MT * (int)blockIdx.z;
    m = min(MT, tk.m - t0);
    if (m <= 0) return;
    wmat = tk.w;
#pragma unroll
    for (int t = 0; t < MT; t++) {
      xr[t] = tk.xrow[min(t0 + t, 15)];
      yr[t] = tk.yrow[min(t0 + t, 15)];
    }
  }

  // the 16-level table of the iq4 codecs in four registers; the iq2_xxs lattice in shared memory
  uint32_t T[4] = {0u, 0u, 0u, 0u};
  if constexpr (kPerm) {
#pragma unroll
    for (int i = 0; i < 16; i++) T[i >> 2] |= ((uint32_t)(uint8_t)kq_tab_iq4nl[i]) << (8 * (i & 3));
  }
  if constexpr (C == IQ2_XXS) {
    for (int i = threadIdx.x; i < 256; i += kThreads) {
      const unsigned long long gv = kq_tab_iq2xxs_grid[i];
      s_grid[i] = make_uint2((uint32_t)gv, (uint32_t)(gv >> 32));
    }
  }

  // ring: window of chunk sb starts at the 16-byte boundary below it, pulled back for the last chunk
  // so that it never leaves the row; piece j = lane + 32 i is bytes [16 (j % P), +16) of row j / P
  uint8_t* ring = dyn + warp * D * kSlot;
  constexpr int kPerLane = G::kP;  // 32 P pieces per slot
  int roff[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; i++) {
    const int j = lane + 32 * i;
    roff[i] = min(row0 + j / G::kP, a.N - 1) - row0;  // row of the piece, clamped at the matrix end
    roff[i] = roff[i] * 64 + (j % G::kP);             // packed: row * 64 + piece
  }
  const uint8_t* wbase = wmat + (long long)row0 * a.row_bytes;
  const int last_ws = (int)a.row_bytes - kStride;
  auto window_start = [&](int sb) { return min((sb * G::kCB) & ~15, last_ws); };
  int issued = ch0;
  auto issue = [&](uint8_t* slot) {
    if (issued < ch1) {
      const int ws = window_start(issued);
#pragma unroll
      for (int i = 0; i < kPerLane; i++)
        cp16(slot + 16 * (lane + 32 * i), wbase + (long long)(roff[i] >> 6) * a.row_bytes + ws + 16 * (roff[i] & 63));
      issued++;
    }
    cp_commit();
  };
  for (int d = 0; d < D; d++) issue(ring + d * kSlot);
  pdl_launch_dependents();
  if (a.tasks == nullptr) pdl_wait();  // activations may come from the kernel before this one

#pragma unroll
  for (int t = 0; t < MT; t++) {
    // quantize all of K: eight activations per thread and step, four threads per 32-group.
    // Rows past M are zeros.
    uint32_t* XH = reinterpret_cast<uint32_t*>(xbase + t * xb);
    uint32_t* XL = XH + K / 4;
    float* SG = reinterpret_cast<float*>(XL + K / 4);
    int* XI16 = reinterpret_cast<int*>(SG + K / 32);
    float* XS16 = reinterpret_cast<float*>(XI16 + K / 16);
    const XT* xrow = static_cast<const XT*>(a.x) + (long long)xr[t] * a.x_row_stride;
    for (int c = threadIdx.x; c < K / 8; c += kThreads) {
      float v[8];
      if (t >= m) {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = 0.f;
      } else if constexpr (std::is_same<XT, float>::value) {
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(xrow + 8 * c));
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(xrow + 8 * c) + 1);
        const float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __bfloat162float(__float2bfloat16_rn(f[i]));
      } else {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(xrow + 8 * c));
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float2 f;
          if constexpr (std::is_same<XT, __half>::value) f = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
          else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[i]));
          v[2 * i] = f.x;
          v[2 * i + 1] = f.y;
        }
      }
      float amax = 0.f, sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        amax = fmaxf(amax, fabsf(v[i]));
        sum += v[i];
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // 16-group
      const bool finite = amax > 0.f && amax < INFINITY;
      const float inv = finite ? 32767.f * __frcp_rn(amax) : 0.f;
      int xi[8], isum = 0;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        xi[i] = __float2int_rn(v[i] * inv);
        isum += xi[i];
      }
      isum += __shfl_xor_sync(0xffffffffu, isum, 1);
      if constexpr (kPerm) {
        // word w of a 32-group holds x[2w], x[16 + 2w], x[2w + 1], x[17 + 2w]: quarters 0 and 2 of the
        // group make words 0-3, quarters 1 and 3 words 4-7; the lower quarter of each pair writes them
        int other[8];
#pragma unroll
        for (int i = 0; i < 8; i++) other[i] = __shfl_xor_sync(0xffffffffu, xi[i], 2);
        if ((c & 2) == 0) {
          const int gbase = (c >> 2) * 8 + (c & 1) * 4;  // first word of the four this thread writes
#pragma unroll
          for (int w = 0; w < 4; w++) {
            const int e[4] = {xi[2 * w], other[2 * w], xi[2 * w + 1], other[2 * w + 1]};
            uint32_t hw = 0u, lw = 0u;
#pragma unroll
            for (int i = 0; i < 4; i++) {
              hw |= ((uint32_t)(e[i] >> 8) & 0xffu) << (8 * i);
              lw |= ((uint32_t)e[i] & 0xffu) << (8 * i);
            }
            XH[gbase + w] = hw;
            XL[gbase + w] = lw;
          }
        }
      } else {
        uint32_t h[2] = {0u, 0u}, l[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; i++) {
          h[i >> 2] |= ((uint32_t)(xi[i] >> 8) & 0xffu) << (8 * (i & 3));
          l[i >> 2] |= ((uint32_t)xi[i] & 0xffu) << (8 * (i & 3));
        }
        *reinterpret_cast<uint2*>(XH + 2 * c) = make_uint2(h[0], h[1]);
        *reinterpret_cast<uint2*>(XL + 2 * c) = make_uint2(l[0], l[1]);
      }
      if ((c & 1) == 0) {
        XI16[c >> 1] = isum;
        XS16[c >> 1] = sum;
      }
      // a group holding inf / nan keeps them: the scale carries the non-finite value into the sum
      if ((c & 3) == 0) SG[c >> 2] = finite ? amax * (1.f / 32767.f) : (amax > 0.f ? amax : 0.f);
    }
  }
  __syncthreads();

  float y[MT];
#pragma unroll
  for (int t = 0; t < MT; t++) y[t] = 0.f;
  for (int sb = ch0; sb < ch1; sb++) {
    const int rel = sb - ch0;
    cp_wait(D - 1);
    __syncwarp();
    uint8_t* slot = ring + (rel % D) * kSlot;
    const int phase = sb * G::kCB - window_start(sb);  // same for every row; even
    const uint8_t* blk = slot + lane * kStride + (phase & ~3);
    XChunk X;
    uint32_t* XH = reinterpret_cast<uint32_t*>(xbase);
    X.xh = reinterpret_cast<const uint4*>(XH + sb * 64);
    X.xl = reinterpret_cast<const uint4*>(XH + K / 4 + sb * 64);
    X.sg = reinterpret_cast<const float*>(XH + K / 2) + sb * 8;
    X.xi16 = reinterpret_cast<const int*>(XH + K / 2 + K / 32) + sb * 16;
    X.xs16 = reinterpret_cast<const float*>(XH + K / 2 + K / 32 + K / 16) + sb * 16;
    X.plane_stride = xb / 16;
    X.sg_stride = xb / 4;
    X.s16_stride = xb / 4;
    if (phase & 2) chunk_dot<C, 2, MT>(Bytes<2>{reinterpret_cast<const uint32_t*>(blk)}, X, T, s_grid, y);
    else chunk_dot<C, 0, MT>(Bytes<0>{reinterpret_cast<const uint32_t*>(blk)}, X, T, s_grid, y);
    __syncwarp();  // the slot is free again
    issue(slot);
  }
#pragma unroll
  for (int t = 0; t < MT; t++) red[warp][t][lane] = y[t];
  __syncthreads();
  for (int idx = threadIdx.x; idx < MT * kRows; idx += kThreads) {
    const int t = idx / kRows, r = idx % kRows;
    if (t < m && row0 + r < a.N) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) sum += red[w][t][r];
      int yrow = yr[0];
#pragma unroll
      for (int u = 1; u < MT; u++)
        if (t == u) yrow = yr[u];
      OT* out = static_cast<OT*>(a.y) + (long long)yrow * a.y_row_stride + row0 + r;
      if (a.bias != nullptr) sum += (float)static_cast<const OT*>(a.bias)[row0 + r];
      if constexpr (std::is_same<OT, __half>::value) *out = __float2half_rn(sum);
      else *out = __float2bfloat16_rn(sum);
    }
  }
}

template <int C, typename XT, int MT>
cudaError_t launch_mt(const GemvArgs& a, cudaStream_t st) {
  const int nchunks = a.K >> 8;
  const int per = (nchunks + kWarps - 1) / kWarps;
  int D = per < 2 ? 1 : 2;
  if (dyn_smem<C>(a.K, D, MT) > 110 * 1024) D = 1;  // two CTAs per SM where the ring allows it
  const int dyn = dyn_smem<C>(a.K, D, MT);
  if (dyn > 200 * 1024) return cudaErrorInvalidConfiguration;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(gemv_dp4a_kernel<C, XT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = a.tasks ? dim3((a.N + kRows - 1) / kRows, a.n_tasks, (a.max_m + MT - 1) / MT)
                        : dim3((a.N + kRows - 1) / kRows, 1, 1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = (no_pdl || a.tasks != nullptr) ? 0 : 1;  // a task list comes from the kernel before: plain stream order
  return cudaLaunchKernelEx(&cfg, gemv_dp4a_kernel<C, XT, MT>, a, D);
}

template <int C, typename XT>
cudaError_t launch_one(const GemvArgs& a, cudaStream_t st) {
  const int rows = a.tasks ? a.max_m : a.M;
  if (rows == 1) return launch_mt<C, XT, 1>(a, st);
  if (rows == 2) return launch_mt<C, XT, 2>(a, st);
  return launch_mt<C, XT, 4>(a, st);
}

template <int C>
cudaError_t launch_codec(int x_dtype, const GemvArgs& a, cudaStream_t st) {
  if (x_dtype == F16) return launch_one<C, __half>(a, st);
  if (x_dtype == BF16) return launch_one<C, __nv_bfloat16>(a, st);
  return launch_one<C, float>(a, st);
}

}  // namespace

bool gemv_dp4a_supported(int codec, int x_dtype, const GemvArgs& a) {
  if (codec > Q5_1) return false;   // the codecs added after the integer kernels were written use the generic path
  if (!a.w_align16 || (a.K & 255) != 0 || a.K > kMaxK || (a.row_bytes & 15) != 0 || a.row_bytes < 16 * 17) return false;
  if (a.tasks != nullptr) {
    // task lists (gather_qmm): rows in slices of four. q4_k with fp16 rows and the two table codecs keep
    // their tensor-core kernels, which take sixteen rows per pass over the weights.
    if ((codec == Q4_K && x_dtype == F16) || codec == IQ4_XS || codec == IQ2_XXS) return false;
    if (a.n_tasks > 65535) return false;
    // measured on a 128-expert block: a win at ~4 rows per expert, a loss at 16 (every four-row slice
    // streams the expert's weights again)
    if (a.avg_rows > 4) return false;
    return 4 * x_bytes(a.K) <= 96 * 1024;
  }
  if (codec == Q4_K) return false;  // dense q4_k has its own kernels (kq_gemv.cu)
  if (codec > Q5_1) return false;   // the codecs added after the integer kernels were written use the generic path
  if (a.M < 1 || a.M > 4) return false;
  // measured: with more than one row the table-driven tensor-core kernels of kq_gemv.cu win for these two,
  // and so they do for iq2_xxs matrices too small to hide the lattice lookups
  if ((codec == IQ4_XS || codec == IQ2_XXS) && a.M > 1) return false;
  if (codec == IQ2_XXS && (long long)a.N * a.K < (48ll << 20)) return false;
  // the activations of all rows are staged whole: 2.6 bytes per activation
  const int mt = a.M == 3 ? 4 : a.M;
  return mt * x_bytes(a.K) <= 96 * 1024;
}

cudaError_t launch_gemv_dp4a(int codec, int x_dtype, const GemvArgs& a, cudaStream_t st) {
  switch (codec) {
    case Q2_K: return launch_codec<Q2_K>(x_dtype, a, st);
    case Q3_K: return launch_codec<Q3_K>(x_dtype, a, st);
    case Q4_K: return launch_codec<Q4_K>(x_dtype, a, st);
    case Q5_K: return launch_codec<Q5_K>(x_dtype, a, st);
    case Q6_K: return launch_codec<Q6_K>(x_dtype, a, st);
    case Q4_0: return launch_codec<Q4_0>(x_dtype, a, st);
    case Q8_0: return launch_codec<Q8_0>(x_dtype, a, st);
    case IQ4_NL: return launch_codec<IQ4_NL>(x_dtype, a, st);
    case IQ4_XS: return launch_codec<IQ4_XS>(x_dtype, a, st);
    case IQ2_XXS: return launch_codec<IQ2_XXS>(x_dtype, a, st);
    case Q4_1: return launch_codec<Q4_1>(x_dtype, a, st);
    case Q5_0: return launch_codec<Q5_0>(x_dtype, a, st);
    case Q5_1: return launch_codec<Q5_1>(x_dtype, a, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace kq
