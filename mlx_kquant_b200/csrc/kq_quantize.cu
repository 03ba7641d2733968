// kq_quantize_cpu: float weights -> GGUF wire bytes on the HOST, the producer of everything the GPU
// kernels read. The reference's `quantize` is a CPU-only op too (src/kquant_ops.cpp:550-631 ->
// src/kquant_encode.cpp:48-98 -> src/kquant_cpu_encode.cpp:824-859); this file restates the ggml
// block-fitting searches it uses, in the same operation order, so that the bytes are identical:
//   q8_0, q4_0     absmax scale, round-half-away (src/kquant_cpu_encode.cpp:38-91)
//   q4_k, q5_k     per-32 (scale, min) by the 37-step grid search, 6-bit super-scales (:445-540)
//   q6_k, q3_k     per-16 signed scale by the 19-step search, 8- / 6-bit super-scales (:542-734)
//   q2_k           per-16 (scale, min), 4-bit super-scales (:736-822)
//   iq4_nl, iq4_xs 16-level table, per-32 scale by a 15-step search (src/kquant_iq_encode.cpp:49-223)
//   iq2_xxs        8-weight lattice points with parity-constrained signs; nearest-neighbour lists of
//                  off-lattice points built once from the decode lattice (:228-598)
// Everything is plain float arithmetic without contraction (no FMA on the host build), one thread
// per group of rows; blocks are independent, so threading does not change a byte.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "kq_common.cuh"
#include "kq_launch.h"

// a host copy of the generated tables (kq_common.cuh holds the device copy)
#undef KQ_IQ_TABLES_INC
#undef KQ_TAB_QUAL
#define KQ_TAB_QUAL static
namespace kq_host_tabs {
#include "kq_iq_tables.inc"
}

namespace kq {

namespace {

inline void put_f16(uint8_t* p, float v) {
  const __half h = __float2half_rn(v);
  std::memcpy(p, &h, 2);
}
inline float get_f16(const uint8_t* p) {
  __half h;
  std::memcpy(&h, p, 2);
  return __half2float(h);
}
inline int rne(float v) { return (int)std::rint(v); }
inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---- the three fitting searches ------------------------------------------------------------
// All follow ggml's routines of the same purpose; comments name the reference's copy.

// (scale, min) of n values with levels 0..nmax, weights wt: start from the min / max line, then try
// 37 inverse scales around it and keep the weighted-least-squares (scale, min) with the smallest
// weighted squared error. Returns the scale, *neg_min = -min. (kq_make_qkx3_quants, :250-336)
float fit_scale_min(const float* x, const float* wt, int n, int nmax, float* neg_min) {
  float lo = x[0], hi = x[0], sw = wt[0], sx = sw * x[0];
  for (int i = 1; i < n; i++) {
    if (x[i] < lo) lo = x[i];
    if (x[i] > hi) hi = x[i];
    sw += wt[i];
    sx += wt[i] * x[i];
  }
  if (lo > 0.f) lo = 0.f;
  if (hi <= lo) {
    *neg_min = -lo;
    return 0.f;
  }
  float inv = (float)nmax / (hi - lo);
  float scale = 1.f / inv;
  float best_err = 0.f;
  for (int i = 0; i < n; i++) {
    const int l = clampi(rne(inv * (x[i] - lo)), 0, nmax);
    const float e = scale * (float)l + lo - x[i];
    best_err += wt[i] * e * e;
  }
  float best_min = lo;
  uint8_t lv[32];
  for (int step = 0; step <= 36; step++) {
    const float inv_s = (-0.9f + 0.05f * (float)step + (float)nmax) / (hi - lo);
    float sl = 0.f, sl2 = 0.f, sxl = 0.f;
    for (int i = 0; i < n; i++) {
      const int l = clampi(rne(inv_s * (x[i] - lo)), 0, nmax);
      lv[i] = (uint8_t)l;
      sl += wt[i] * (float)l;
      sl2 += wt[i] * (float)l * (float)l;
      sxl += wt[i] * (float)l * x[i];
    }
    const float det = sw * sl2 - sl * sl;
    if (det > 0.f) {
      float s = (sw * sxl - sx * sl) / det;
      float m = (sl2 * sx - sl * sxl) / det;
      if (m > 0.f) {
        m = 0.f;
        s = sxl / sl2;
      }
      float err = 0.f;
      for (int i = 0; i < n; i++) {
        const float e = s * (float)lv[i] + m - x[i];
        err += wt[i] * e * e;
      }
      if (err < best_err) {
        best_err = err;
        scale = s;
        best_min = m;
      }
    }
  }
  *neg_min = -best_min;
  return scale;
}

// Signed scale of 16 values with levels -nmax..nmax-1 (weights wt, or x^2 when wt is null): the
// scale that maps the largest magnitude to -nmax, then 18 neighbours, keeping the one that
// maximises (sum w x l)^2 / (sum w l^2). (kq_make_qx_quants_16, :338-397)
float fit_signed16(const float* x, const float* wt, int nmax) {
  float big = 0.f, amax = 0.f;
  for (int i = 0; i < 16; i++) {
    const float a = std::fabs(x[i]);
    if (a > amax) {
      amax = a;
      big = x[i];
    }
  }
  if (amax < 1e-30f) return 0.f;
  auto sums = [&](float inv, float& slx, float& sl2) {
    slx = 0.f;
    sl2 = 0.f;
    for (int i = 0; i < 16; i++) {
      const int l = clampi(rne(inv * x[i]), -nmax, nmax - 1);
      const float w = wt ? wt[i] : x[i] * x[i];
      slx += w * x[i] * (float)l;
      sl2 += w * (float)l * (float)l;
    }
  };
  float slx, sl2;
  sums(-(float)nmax / big, slx, sl2);
  float scale = sl2 > 0.f ? slx / sl2 : 0.f;
  float best = scale * slx;
  for (int step = -9; step <= 9; step++) {
    if (step == 0) continue;
    sums(-((float)nmax + 0.1f * (float)step) / big, slx, sl2);
    if (sl2 > 0.f && slx * slx > best * sl2) {
      scale = slx / sl2;
      best = scale * slx;
    }
  }
  return scale;
}

// One non-negative scale for n non-negative values with levels 0..nmax: eight neighbours of
// nmax / max, then up to five rounds of single-level refinement. Writes the levels, returns the
// scale. (kq_make_qp_quants, src/kquant_cpu_encode_util.h:57-144)
float fit_positive(const float* x, const float* wt, int n, int nmax, uint8_t* levels, float eps = 1e-30f) {
  float top = 0.f;
  for (int i = 0; i < n; i++)
    if (x[i] > top) top = x[i];
  if (top < eps) {
    for (int i = 0; i < n; i++) levels[i] = 0;
    return 0.f;
  }
  float inv = (float)nmax / top;
  uint8_t lv[32];
  for (int i = 0; i < n; i++) lv[i] = (uint8_t)clampi(rne(inv * x[i]), 0, nmax);
  const float s0 = 1.f / inv;
  float best = 0.f;
  for (int i = 0; i < n; i++) {
    const float e = x[i] - s0 * (float)lv[i];
    best += wt[i] * e * e;
  }
  for (int step = -4; step <= 4; step++) {
    if (step == 0) continue;
    const float inv_s = (0.1f * (float)step + (float)nmax) / top;
    const float s = 1.f / inv_s;
    float err = 0.f;
    for (int i = 0; i < n; i++) {
      const int l = std::min(nmax, rne(inv_s * x[i]));
      const float e = x[i] - s * (float)l;
      err += wt[i] * e * e;
    }
    if (err < best) {
      best = err;
      inv = inv_s;
    }
  }
  float slx = 0.f, sl2 = 0.f;
  for (int i = 0; i < n; i++) {
    const int l = std::min(nmax, rne(inv * x[i]));
    lv[i] = (uint8_t)l;
    slx += wt[i] * x[i] * (float)l;
    sl2 += wt[i] * (float)l * (float)l;
  }
  for (int round = 0; round < 5; round++) {
    int changed = 0;
    for (int i = 0; i < n; i++) {
      const float w = wt[i];
      float a = slx - w * x[i] * (float)lv[i];
      float b = sl2 - w * (float)lv[i] * (float)lv[i];
      if (a > 0.f && b > 0.f) {
        const int nl = std::min(nmax, rne(x[i] * b / a));
        if (nl != (int)lv[i]) {
          a += w * x[i] * (float)nl;
          b += w * (float)nl * (float)nl;
          if (a * a * sl2 > slx * slx * b) {
            lv[i] = (uint8_t)nl;
            slx = a;
            sl2 = b;
            changed++;
          }
        }
      }
    }
    if (changed == 0) break;
  }
  for (int i = 0; i < n; i++) levels[i] = lv[i];
  return sl2 > 0.f ? slx / sl2 : 0.f;
}

// importance weights of a superblock: imatrix[k] * sqrt(sigma2 + x^2), or av_x + |x| without one;
// sigma2 = factor * sum(x^2) / 256 (compute_sigma2_av_x, :237-248)
void importance(const float* x, const float* im, float factor, bool need_default, float* wt) {
  float total = 0.f;
  for (int i = 0; i < 256; i++) total += x[i] * x[i];
  const float sigma2 = factor * total / 256.0f;
  if (im) {
    for (int i = 0; i < 256; i++) wt[i] = im[i] * std::sqrt(sigma2 + x[i] * x[i]);
  } else if (need_default) {
    const float av = std::sqrt(sigma2);
    for (int i = 0; i < 256; i++) wt[i] = av + std::fabs(x[i]);
  }
}

// ---- block encoders (x: 32 or 256 floats, im: the matching slice of the imatrix or null) ----
void enc_q8_0(const float* x, const float*, uint8_t* b) {
  float amax = 0.f;
  for (int j = 0; j < 32; j++) amax = std::max(amax, std::fabs(x[j]));
  const float d = amax / 127.0f, id = d != 0.f ? 1.0f / d : 0.f;
  put_f16(b, d);
  for (int j = 0; j < 32; j++)
    b[2 + j] = (uint8_t)(int8_t)std::min(127.0f, std::max(-127.0f, std::round(x[j] * id)));
}

void enc_q4_0(const float* x, const float*, uint8_t* b) {
  float amax = 0.f;
  for (int j = 0; j < 32; j++) amax = std::max(amax, std::fabs(x[j]));
  const float d = amax / 7.0f, id = d != 0.f ? 1.0f / d : 0.f;
  put_f16(b, d);
  for (int j = 0; j < 16; j++) {
    const uint8_t q0 = (uint8_t)std::min(15.0f, std::max(0.0f, std::round(x[j] * id) + 8.0f));
    const uint8_t q1 = (uint8_t)std::min(15.0f, std::max(0.0f, std::round(x[j + 16] * id) + 8.0f));
    b[2 + j] = (uint8_t)(q0 | (q1 << 4));
  }
}

// q4_1, q5_0, q5_1 (src/kquant_cpu_encode.cpp:93-205): round-half-away like the other flat codecs
void enc_q4_1(const float* x, const float*, uint8_t* b) {
  float vmin = x[0], vmax = x[0];
  for (int j = 1; j < 32; j++) {
    vmin = std::min(vmin, x[j]);
    vmax = std::max(vmax, x[j]);
  }
  const float d = (vmax - vmin) / 15.0f, id = d != 0.f ? 1.0f / d : 0.f;
  put_f16(b, d);
  put_f16(b + 2, vmin);
  for (int j = 0; j < 16; j++) {
    const uint8_t q0 = (uint8_t)std::min(15.0f, std::max(0.0f, std::round((x[j] - vmin) * id)));
    const uint8_t q1 = (uint8_t)std::min(15.0f, std::max(0.0f, std::round((x[j + 16] - vmin) * id)));
    b[4 + j] = (uint8_t)(q0 | (q1 << 4));
  }
}

template <bool WITH_MIN>
void enc_q5_01(const float* x, const float*, uint8_t* b) {
  float d, off;
  if constexpr (WITH_MIN) {
    float vmin = x[0], vmax = x[0];
    for (int j = 1; j < 32; j++) {
      vmin = std::min(vmin, x[j]);
      vmax = std::max(vmax, x[j]);
    }
    d = (vmax - vmin) / 31.0f;
    off = vmin;
    put_f16(b + 2, vmin);
  } else {
    float amax = 0.f;
    for (int j = 0; j < 32; j++) amax = std::max(amax, std::fabs(x[j]));
    d = amax / 15.0f;
    off = 0.f;
  }
  const float id = d != 0.f ? 1.0f / d : 0.f;
  put_f16(b, d);
  uint8_t* qhp = b + (WITH_MIN ? 4 : 2);
  uint8_t* qs = b + (WITH_MIN ? 8 : 6);
  uint32_t qh = 0;
  for (int j = 0; j < 16; j++) {
    float v0, v1;
    if constexpr (WITH_MIN) {
      v0 = std::round((x[j] - off) * id);
      v1 = std::round((x[j + 16] - off) * id);
    } else {
      v0 = std::round(x[j] * id) + 16.0f;
      v1 = std::round(x[j + 16] * id) + 16.0f;
    }
    const uint8_t q0 = (uint8_t)std::min(31.0f, std::max(0.0f, v0));
    const uint8_t q1 = (uint8_t)std::min(31.0f, std::max(0.0f, v1));
    qs[j] = (uint8_t)((q0 & 0x0F) | ((q1 & 0x0F) << 4));
    qh |= (uint32_t)(q0 >> 4) << j;
    qh |= (uint32_t)(q1 >> 4) << (j + 16);
  }
  for (int i = 0; i < 4; i++) qhp[i] = (uint8_t)(qh >> (8 * i));
}

// q4_k (bits = 4) and q5_k (bits = 5)
template <int BITS>
void enc_q45_k(const float* x, const float* im, uint8_t* b) {
  constexpr int nmax = BITS == 4 ? 15 : 31;
  constexpr int kQs = BITS == 4 ? 16 : 48;
  float wt[256];
  importance(x, im, 2.0f, true, wt);
  float sc[8], mn[8], sw[8];
  for (int s = 0; s < 8; s++) {
    float t = 0.f;
    for (int l = 0; l < 32; l++) t += wt[32 * s + l];
    sw[s] = t;
    sc[s] = fit_scale_min(x + 32 * s, wt + 32 * s, 32, nmax, &mn[s]);
  }
  uint8_t ls[8], lm[8];
  put_f16(b, fit_positive(sc, sw, 8, 63, ls));
  put_f16(b + 2, fit_positive(mn, sw, 8, 63, lm));
  // twelve bytes of 6-bit pairs (inverse of the decoder's unpacking, src/kquant_cpu_decode.cpp:155-174)
  uint8_t* p = b + 4;
  std::memset(p, 0, 12);
  for (int j = 0; j < 8; j++) {
    if (j < 4) {
      p[j] = ls[j];
      p[j + 4] = lm[j];
    } else {
      p[j + 4] = (uint8_t)((ls[j] & 15) | ((lm[j] & 15) << 4));
      p[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
      p[j] |= (uint8_t)((lm[j] >> 4) << 6);
    }
  }
  // levels against the scales as the decoder will see them (fp16 d / dmin, 6-bit integers)
  const float d = get_f16(b), dmin = get_f16(b + 2);
  uint8_t L[256];
  for (int s = 0; s < 8; s++) {
    const float ds = d * (float)ls[s], ms = dmin * (float)lm[s];
    for (int l = 0; l < 32; l++) {
      const int i = 32 * s + l;
      L[i] = ds == 0.f ? 0 : (uint8_t)clampi(rne((x[i] + ms) / ds), 0, nmax);
    }
  }
  for (int g = 0; g < 4; g++)
    for (int l = 0; l < 32; l++) b[kQs + 32 * g + l] = (uint8_t)((L[64 * g + l] & 15) | ((L[64 * g + 32 + l] & 15) << 4));
  if (BITS == 5) {
    for (int j = 0; j < 32; j++) {
      uint8_t bits = 0;
      for (int s = 0; s < 8; s++)
        if (L[32 * s + j] > 15) bits |= (uint8_t)(1u << s);
      b[16 + j] = bits;
    }
  }
}

void enc_q6_k(const float* x, const float* im, uint8_t* b) {
  float sc[16];
  for (int s = 0; s < 16; s++) sc[s] = fit_signed16(x + 16 * s, im ? im + 16 * s : nullptr, 32);
  float top = 0.f, atop = 0.f;
  for (int s = 0; s < 16; s++) {
    const float a = std::fabs(sc[s]);
    if (a > atop) {
      atop = a;
      top = sc[s];
    }
  }
  if (atop < 1e-30f) {
    std::memset(b, 0, 210);
    return;
  }
  const float inv = -128.0f / top;
  put_f16(b + 208, 1.0f / inv);
  int8_t* so = reinterpret_cast<int8_t*>(b + 192);
  for (int s = 0; s < 16; s++) so[s] = (int8_t)std::min(127, rne(inv * sc[s]));
  const float d = get_f16(b + 208);
  uint8_t L[256];
  for (int i = 0; i < 256; i++) {
    const float de = d * (float)so[i / 16];
    L[i] = de == 0.f ? 32 : (uint8_t)(clampi(rne(x[i] / de), -32, 31) + 32);
  }
  for (int h = 0; h < 2; h++) {
    for (int l = 0; l < 32; l++) {
      const uint8_t a = L[128 * h + l], bb = L[128 * h + 32 + l], c = L[128 * h + 64 + l], e = L[128 * h + 96 + l];
      b[64 * h + l] = (uint8_t)((a & 15) | ((c & 15) << 4));
      b[64 * h + 32 + l] = (uint8_t)((bb & 15) | ((e & 15) << 4));
      b[128 + 32 * h + l] = (uint8_t)((a >> 4) | ((bb >> 4) << 2) | ((c >> 4) << 4) | ((e >> 4) << 6));
    }
  }
}

void enc_q3_k(const float* x, const float* im, uint8_t* b) {
  float wt[256];
  if (im) importance(x, im, 2.0f, false, wt);
  float sc[16];
  for (int s = 0; s < 16; s++) sc[s] = fit_signed16(x + 16 * s, im ? wt + 16 * s : nullptr, 4);
  float top = 0.f, atop = 0.f;
  for (int s = 0; s < 16; s++) {
    const float a = std::fabs(sc[s]);
    if (a > atop) {
      atop = a;
      top = sc[s];
    }
  }
  uint8_t* p = b + 96;
  std::memset(p, 0, 12);
  float dblk = 0.f;
  int lsc[16];
  for (int s = 0; s < 16; s++) lsc[s] = 0;
  if (top != 0.f) {
    const float inv = -32.0f / top;
    for (int s = 0; s < 16; s++) {
      const int l = clampi(rne(inv * sc[s]), -32, 31) + 32;  // biased, 0..63
      lsc[s] = l;
      if (s < 8) p[s] = (uint8_t)(l & 15);
      else p[s - 8] |= (uint8_t)((l & 15) << 4);
      p[8 + (s & 3)] |= (uint8_t)(((l >> 4) & 3) << (2 * (s >> 2)));
    }
    dblk = 1.0f / inv;
  }
  put_f16(b + 108, dblk);
  const float d = get_f16(b + 108);
  uint8_t L[256];
  for (int i = 0; i < 256; i++) {
    const float de = d * (float)(lsc[i / 16] - 32);
    L[i] = de == 0.f ? 4 : (uint8_t)(clampi(rne(x[i] / de), -4, 3) + 4);
  }
  for (int h = 0; h < 2; h++)
    for (int l = 0; l < 32; l++) {
      uint8_t v = 0;
      for (int k = 0; k < 4; k++) v |= (uint8_t)((L[128 * h + 32 * k + l] & 3) << (2 * k));
      b[32 + 32 * h + l] = v;
    }
  for (int l = 0; l < 32; l++) {
    uint8_t v = 0;
    for (int bit = 0; bit < 8; bit++) v |= (uint8_t)(((L[128 * (bit >> 2) + 32 * (bit & 3) + l] >> 2) & 1) << bit);
    b[l] = v;
  }
}

void enc_q2_k(const float* x, const float* im, uint8_t* b) {
  float wt[256];
  importance(x, im, 1.0f, true, wt);
  float sc[16], mn[16], sw[16];
  for (int s = 0; s < 16; s++) {
    float t = 0.f;
    for (int l = 0; l < 16; l++) t += wt[16 * s + l];
    sw[s] = t;
    sc[s] = fit_scale_min(x + 16 * s, wt + 16 * s, 16, 3, &mn[s]);
  }
  uint8_t ls[16], lm[16];
  put_f16(b + 80, fit_positive(sc, sw, 16, 15, ls));
  put_f16(b + 82, fit_positive(mn, sw, 16, 15, lm));
  for (int s = 0; s < 16; s++) b[s] = (uint8_t)((ls[s] & 15) | ((lm[s] & 15) << 4));
  const float d = get_f16(b + 80), dmin = get_f16(b + 82);
  uint8_t L[256];
  for (int i = 0; i < 256; i++) {
    const float de = d * (float)(b[i / 16] & 15), me = dmin * (float)(b[i / 16] >> 4);
    L[i] = de == 0.f ? 0 : (uint8_t)clampi(rne((x[i] + me) / de), 0, 3);
  }
  for (int h = 0; h < 2; h++)
    for (int l = 0; l < 32; l++) {
      uint8_t v = 0;
      for (int k = 0; k < 4; k++) v |= (uint8_t)((L[128 * h + 32 * k + l] & 3) << (2 * k));
      b[16 + 32 * h + l] = v;
    }
}

// ---- iq4_nl / iq4_xs: the 16 non-uniform levels of ggml's kvalues_iq4nl ------------------------
const int8_t kLevels[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// index of the level nearest to v; ties go to the lower index (best_index_int8, :49-68)
inline int nearest_level(float v) {
  if (v <= (float)kLevels[0]) return 0;
  if (v >= (float)kLevels[15]) return 15;
  int lo = 0, hi = 15;
  while (hi - lo > 1) {
    const int mid = (lo + hi) / 2;
    if (v < (float)kLevels[mid]) hi = mid;
    else lo = mid;
  }
  return v - (float)kLevels[hi - 1] < (float)kLevels[hi] - v ? hi - 1 : hi;
}

// n = 32 (iq4_nl: [f16 d][16 B]) or 256 (iq4_xs: [f16 d][u16 high scale bits][4 B low nibbles][128 B]).
// Per 32 weights: the scale that maps the largest magnitude to level -127, then 15 neighbours, keeping
// the one with the largest (sum w q x)^2 / (sum w q^2). (quantize_iq4_block, :73-223, ntry = 7)
template <int N>
void enc_iq4(const float* x, const float* im, uint8_t* b) {
  constexpr int nsb = N / 32;
  float sigma2 = 0.f;
  for (int j = 0; j < N; j++) sigma2 += x[j] * x[j];
  sigma2 *= 2.f / (float)N;
  float scales[8];
  float top = 0.f, atop = 0.f;
  for (int ib = 0; ib < nsb; ib++) {
    const float* xb = x + 32 * ib;
    float wt[32];
    for (int j = 0; j < 32; j++) wt[j] = im ? im[32 * ib + j] * std::sqrt(sigma2 + xb[j] * xb[j]) : xb[j] * xb[j];
    float amax = 0.f, big = 0.f;
    for (int j = 0; j < 32; j++) {
      const float a = std::fabs(xb[j]);
      if (a > amax) {
        amax = a;
        big = xb[j];
      }
    }
    if (amax < 1e-15f) {
      scales[ib] = 0.f;
      continue;
    }
    auto sums = [&](float inv, float& sqx, float& sq2) {
      sqx = 0.f;
      sq2 = 0.f;
      for (int j = 0; j < 32; j++) {
        const float q = (float)kLevels[nearest_level(inv * xb[j])];
        sqx += wt[j] * q * xb[j];
        sq2 += wt[j] * q * q;
      }
    };
    float d = -big / (float)kLevels[0];
    float sqx, sq2;
    sums(1.f / d, sqx, sq2);
    d = sq2 > 0.f ? sqx / sq2 : 0.f;
    float best = d * sqx;
    for (int step = -7; step <= 7; step++) {
      sums(((float)step + (float)kLevels[0]) / big, sqx, sq2);
      if (sq2 > 0.f && sqx * sqx > best * sq2) {
        d = sqx / sq2;
        best = d * sqx;
      }
    }
    scales[ib] = d;
    if (std::fabs(d) > atop) {
      atop = std::fabs(d);
      top = d;
    }
  }
  uint8_t L[256];
  uint8_t* q4;
  if (nsb > 1) {
    q4 = b + 8;
    std::memset(b + 4, 0, 4);
    uint32_t high = 0;
    const float d = -top / 32.f;
    put_f16(b, d);
    const float id = d != 0.f ? 1.f / d : 0.f;
    for (int ib = 0; ib < nsb; ib++) {
      int l = clampi(rne(id * scales[ib]), -32, 31);
      const float dl = d * (float)l;
      const float idl = dl != 0.f ? 1.f / dl : 0.f;
      for (int j = 0; j < 32; j++) L[32 * ib + j] = (uint8_t)nearest_level(idl * x[32 * ib + j]);
      l += 32;
      b[4 + ib / 2] |= (uint8_t)((l & 15) << (4 * (ib & 1)));
      high |= (uint32_t)(l >> 4) << (2 * ib);
    }
    b[2] = (uint8_t)(high & 0xff);
    b[3] = (uint8_t)(high >> 8);
  } else {
    q4 = b + 2;
    put_f16(b, scales[0]);
    const float id = scales[0] != 0.f ? 1.f / scales[0] : 0.f;
    for (int j = 0; j < 32; j++) L[j] = (uint8_t)nearest_level(id * x[j]);
  }
  for (int i = 0; i < nsb; i++)
    for (int j = 0; j < 16; j++) q4[16 * i + j] = (uint8_t)(L[32 * i + j] | (L[32 * i + 16 + j] << 4));
}

// ---- iq2_xxs --------------------------------------------------------------------------------------
// Search space: eight levels l in {0, 1, 2} (decoded as 8, 25, 43), searched as 2 l + 1, packed two bits
// each into an index < 43692. `slot[index]` is the lattice entry, or -(offset + 1) into `near`, where a
// count and that many entries list the lattice points at the two smallest distances (ties by entry
// number). Built once from the decode lattice. (build_iq_grid_index, :235-330, nwant = 2)
struct Lattice {
  int8_t point[256][8];
  std::vector<int> slot;
  std::vector<uint16_t> near;
  Lattice() : slot(43692, -1) {
    for (int e = 0; e < 256; e++) {
      int index = 0;
      for (int i = 0; i < 8; i++) {
        const int byte = (int)((kq_host_tabs::kq_tab_iq2xxs_grid[e] >> (8 * i)) & 0xff);
        const int l = byte == 8 ? 0 : (byte == 25 ? 1 : 2);
        point[e][i] = (int8_t)(2 * l + 1);
        index |= l << (2 * i);
      }
      slot[index] = e;
    }
    std::vector<std::pair<int, int>> dist(256);
    for (int idx = 0; idx < (int)slot.size(); idx++) {
      if (slot[idx] >= 0) continue;
      for (int e = 0; e < 256; e++) {
        int d2 = 0;
        for (int i = 0; i < 8; i++) {
          const int diff = point[e][i] - (2 * ((idx >> (2 * i)) & 3) + 1);
          d2 += diff * diff;
        }
        dist[e] = {d2, e};
      }
      std::sort(dist.begin(), dist.end());
      const int at = (int)near.size();
      near.push_back(0);
      int d2 = dist[0].first, have = 1;
      for (int e = 0; e < 256; e++) {
        if (dist[e].first > d2) {
          if (have == 2) break;
          d2 = dist[e].first;
          have++;
        }
        near.push_back((uint16_t)dist[e].second);
      }
      near[at] = (uint16_t)(near.size() - at - 1);
      slot[idx] = -(at + 1);
    }
  }
};
const Lattice& lattice() {
  static const Lattice l;  // thread-safe one-time construction
  return l;
}

// lattice entry for the packed levels u; off-lattice: the listed neighbour with the smallest weighted
// squared error to the scaled point (iq2_find_best_neighbour, :359-389)
inline int lattice_entry(const Lattice& G, int u, const float* xv, const float* w, float scale) {
  int e = G.slot[u];
  if (e >= 0) return e;
  const uint16_t* nb = G.near.data() + (-e - 1);
  float best = 3.402823466e+38f;
  e = -1;
  for (int j = 1; j <= (int)nb[0]; j++) {
    const int8_t* pg = G.point[nb[j]];
    float d2 = 0.f;
    for (int i = 0; i < 8; i++) {
      const float diff = scale * (float)pg[i] - xv[i];
      d2 += w[i] * diff * diff;
    }
    if (d2 < best) {
      best = d2;
      e = nb[j];
    }
  }
  return e;
}

// (quantize_iq2_xxs_block, :392-598)
void enc_iq2_xxs(const float* x, const float* im, uint8_t* b) {
  const Lattice& G = lattice();
  uint32_t q2[16];
  std::memset(q2, 0, sizeof(q2));
  float total = 0.f;
  for (int i = 0; i < 256; i++) total += x[i] * x[i];
  const float sigma2 = total / 256.0f;
  float scales[8], top = 0.f;
  for (int ib = 0; ib < 8; ib++) {
    const float* xb = x + 32 * ib;
    float wt[32], wsq[32], xv[32];
    for (int i = 0; i < 32; i++) wt[i] = im[32 * ib + i] * std::sqrt(sigma2 + xb[i] * xb[i]);
    for (int i = 0; i < 32; i++) wsq[i] = std::sqrt(wt[i]);
    // magnitudes and sign bits; an odd number of negatives flips the least important weight so that the
    // eighth sign is the parity of the other seven
    uint8_t signs[4];
    for (int k = 0; k < 4; k++) {
      int flips = 0;
      uint8_t sb = 0;
      for (int i = 0; i < 8; i++) {
        const float v = xb[8 * k + i];
        if (v >= 0.f) {
          xv[8 * k + i] = v;
        } else {
          xv[8 * k + i] = -v;
          flips++;
          sb |= (uint8_t)(1 << i);
        }
      }
      if (flips & 1) {
        int imin = 0;
        float least = wt[8 * k] * xb[8 * k] * xb[8 * k];
        for (int i = 1; i < 8; i++) {
          const float a = wt[8 * k + i] * xb[8 * k + i] * xb[8 * k + i];
          if (a < least) {
            least = a;
            imin = i;
          }
        }
        xv[8 * k + imin] = -xv[8 * k + imin];
        sb ^= (uint8_t)(1 << imin);
      }
      signs[k] = sb & 127;
    }
    float mx = xv[0];
    for (int i = 1; i < 32; i++) mx = std::max(mx, xv[i]);
    scales[ib] = 0.f;
    if (mx < 1e-15f) continue;
    int8_t L[32], La[32];
    float scale = fit_positive(xv, wt, 32, 4, reinterpret_cast<uint8_t*>(L), 1e-15f);
    const float eff_max = scale * 3;
    if (eff_max <= 0.f) continue;
    auto levels_of = [&](float id, int k, int8_t* out) {
      int u = 0;
      for (int i = 0; i < 8; i++) {
        const int l = clampi(rne(0.5f * (id * xv[8 * k + i] - 1)), 0, 2);
        out[i] = (int8_t)l;
        u |= l << (2 * i);
      }
      return u;
    };
    auto score = [&](const int8_t* lv, float& sqx, float& sq2) {
      sqx = 0.f;
      sq2 = 0.f;
      for (int i = 0; i < 32; i++) {
        const float q = (float)(2 * lv[i] + 1);
        sqx += wt[i] * xv[i] * q;
        sq2 += wt[i] * q * q;
      }
    };
    float best = 0.f, sqx, sq2;
    for (int step = -6; step <= 6; step++) {
      const float id = (5 + step * 0.1f) / eff_max;
      const float this_scale = 1 / id;
      for (int k = 0; k < 4; k++) {
        const int u = levels_of(id, k, La + 8 * k);
        if (G.slot[u] < 0) {
          const int8_t* pg = G.point[lattice_entry(G, u, xv + 8 * k, wsq + 8 * k, this_scale)];
          for (int i = 0; i < 8; i++) La[8 * k + i] = (int8_t)((pg[i] - 1) / 2);
        }
      }
      score(La, sqx, sq2);
      if (sq2 > 0.f && sqx * sqx > best * sq2) {
        scale = sqx / sq2;
        best = scale * sqx;
        std::memcpy(L, La, 32);
      }
    }
    if (scale > 0.f) {
      const float id = 1 / scale;
      for (int k = 0; k < 4; k++) {
        int8_t tmp[8];
        const int u = levels_of(id, k, tmp);
        const int8_t* pg = G.point[lattice_entry(G, u, xv + 8 * k, wsq + 8 * k, scale)];
        for (int i = 0; i < 8; i++) L[8 * k + i] = (int8_t)((pg[i] - 1) / 2);
      }
      score(L, sqx, sq2);
      if (sq2 > 0.f) scale = sqx / sq2;
    }
    if (scale < 0.f) {  // the wire holds an unsigned scale: move the sign into the sign bits
      scale = -scale;
      for (int k = 0; k < 4; k++) signs[k] = (uint8_t)((~signs[k]) & 127);
    }
    for (int k = 0; k < 4; k++) {
      int u = 0;
      for (int i = 0; i < 8; i++) u |= L[8 * k + i] << (2 * i);
      const int e = G.slot[u] >= 0 ? G.slot[u] : 0;  // always on the lattice after the step above
      q2[2 * ib] |= (uint32_t)e << (8 * k);
      q2[2 * ib + 1] |= (uint32_t)signs[k] << (7 * k);
    }
    scales[ib] = scale;
    top = std::max(top, scale);
  }
  if (!(top != 0.f)) {
    put_f16(b, 0.f);
    std::memset(b + 2, 0, 64);
    return;
  }
  const float d = top / 31;
  put_f16(b, d);
  const float id = 1 / d;
  for (int ib = 0; ib < 8; ib++) q2[2 * ib + 1] |= (uint32_t)clampi(rne(0.5f * (id * scales[ib] - 1)), 0, 15) << 28;
  std::memcpy(b + 2, q2, 64);
}

using BlockFn = void (*)(const float*, const float*, uint8_t*);
BlockFn block_encoder(int codec) {
  switch (codec) {
    case Q8_0: return enc_q8_0;
    case Q4_0: return enc_q4_0;
    case Q4_K: return enc_q45_k<4>;
    case Q5_K: return enc_q45_k<5>;
    case Q6_K: return enc_q6_k;
    case Q3_K: return enc_q3_k;
    case Q2_K: return enc_q2_k;
    case IQ4_NL: return enc_iq4<32>;
    case IQ4_XS: return enc_iq4<256>;
    case IQ2_XXS: return enc_iq2_xxs;
    case Q4_1: return enc_q4_1;
    case Q5_0: return enc_q5_01<false>;
    case Q5_1: return enc_q5_01<true>;
  }
  return nullptr;
}

inline float load_as_float(const void* w, int dtype, long long i) {
  if (dtype == F32) return static_cast<const float*>(w)[i];
  if (dtype == F16) return __half2float(static_cast<const __half*>(w)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]);
}

}  // namespace

bool quantize_supported(int codec) { return block_encoder(codec) != nullptr; }

// w: n_weights values of dtype (0 f32, 1 f16, 2 bf16) in host memory, rows of K; imatrix: K floats
// or null; out: n_weights / wpb * bpb bytes. Block b of the flat array uses imatrix[(b * wpb) % K ...]
// (src/kquant_cpu_encode.cpp:471).
void quantize_host(int codec, const void* w, int dtype, long long n_weights, long long K, const float* imatrix,
                   uint8_t* out, int threads) {
  const BlockFn fn = block_encoder(codec);
  const int wpb = kCodecs[codec].wpb, bpb = kCodecs[codec].bpb;
  const long long n_blocks = n_weights / wpb;
  if (fn == nullptr || n_blocks <= 0) return;
  const bool uses_imatrix = !(codec == Q8_0 || codec == Q4_0 || codec == Q4_1 || codec == Q5_0 || codec == Q5_1);  // the flat codecs ignore it (src/kquant_cpu_encode.cpp:832-834)
  auto run = [&](long long b0, long long b1) {
    float x[256];
    for (long long b = b0; b < b1; b++) {
      for (int i = 0; i < wpb; i++) x[i] = load_as_float(w, dtype, b * wpb + i);
      const float* im = (imatrix && uses_imatrix) ? imatrix + (b * wpb) % K : nullptr;
      fn(x, im, out + b * bpb);
    }
  };
  int nt = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  nt = (int)std::max(1LL, std::min<long long>(nt > 0 ? nt : 1, n_blocks / 64));
  if (nt == 1) {
    run(0, n_blocks);
    return;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; t++) pool.emplace_back(run, n_blocks * t / nt, n_blocks * (t + 1) / nt);
  for (auto& th : pool) th.join();
}

}  // namespace kq
