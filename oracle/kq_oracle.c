/* TEST INFRASTRUCTURE - CPU restatement of the reference's quantized-weight
 * path, used only as the checker for the CUDA kernels (tests, the smoke check,
 * the benchmark's CPU-baseline leg). The shipped library never links, loads or
 * calls this file.
 *
 * Parity status: PINNED. tests/test_oracle.py checks every decoder here
 * bit-for-bit (f32, f16, bf16) against (a) the reference's own compiled CPU
 * library (oracle/_ref/libkqref.so) where it has been built, (b) gguf-py's
 * independent decoders, and (c) the committed golden vectors made from the
 * reference's fixtures.
 *
 * Each function cites the reference lines it restates (paths relative to the
 * reference checkout). All arithmetic is fp32 in the association order the
 * reference writes, followed by exactly one rounding to the output type.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#include "kq_iq_tables.inc"

/* ---- a minimal parallel-for over [0, n): threads are created per call ----
 * KQO_THREADS (default: online cores, capped at 64 like the reference's pool,
 * src/kquant_cpu_decode.cpp:797-810) sets the width. Work items are
 * independent output rows or blocks, so results do not depend on the width. */
typedef void (*range_fn)(long long begin, long long end, void* ctx);
typedef struct {
  range_fn fn;
  void* ctx;
  long long b, e;
} par_job;

static void* par_tramp(void* p) {
  par_job* j = (par_job*)p;
  j->fn(j->b, j->e, j->ctx);
  return NULL;
}

int kqo_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  const char* env = getenv("KQO_THREADS");
  if (env && atoi(env) > 0) n = atoi(env);
  if (n < 1) n = 1;
  if (n > 64) n = 64;
  return (int)n;
}

static void par_for(long long n, range_fn fn, void* ctx) {
  int nt = kqo_threads();
  if (nt > n) nt = (int)(n > 0 ? n : 1);
  if (nt <= 1) {
    fn(0, n, ctx);
    return;
  }
  pthread_t th[64];
  par_job jobs[64];
  long long chunk = (n + nt - 1) / nt;
  int started = 0;
  for (int t = 0; t < nt; t++) {
    jobs[t].fn = fn;
    jobs[t].ctx = ctx;
    jobs[t].b = t * chunk;
    jobs[t].e = jobs[t].b + chunk < n ? jobs[t].b + chunk : n;
    if (jobs[t].b >= jobs[t].e) break;
    if (t == nt - 1 || pthread_create(&th[t], NULL, par_tramp, &jobs[t]) != 0) {
      fn(jobs[t].b, n, ctx); /* the last part (or everything left after a failed spawn) runs inline */
      break;
    }
    started++;
  }
  for (int t = 0; t < started; t++) pthread_join(th[t], NULL);
}

/* ---- registry: src/kquant_codec.cpp:12-37, the ten in-scope rows ---- */
typedef struct {
  const char* name;
  int wpb; /* weights per block */
  int bpb; /* bytes per block */
  int bits;
  int requires_imatrix;
} kqo_codec;

static const kqo_codec KQO_CODECS[] = {
    {"q2_k", 256, 84, 2, 0},   {"q3_k", 256, 110, 3, 0},
    {"q4_k", 256, 144, 4, 0},  {"q5_k", 256, 176, 5, 0},
    {"q6_k", 256, 210, 6, 0},  {"q4_0", 32, 18, 4, 0},
    {"q8_0", 32, 34, 8, 0},    {"iq4_nl", 32, 18, 4, 0},
    {"iq4_xs", 256, 136, 4, 0}, {"iq2_xxs", 256, 66, 2, 1},
    {"q4_1", 32, 20, 4, 0},    {"q5_0", 32, 22, 5, 0},
    {"q5_1", 32, 24, 5, 0},    {"iq3_xxs", 256, 98, 3, 0},
    {"iq3_s", 256, 110, 3, 0}, {"iq2_xs", 256, 74, 2, 1},
    {"iq2_s", 256, 82, 2, 0},  {"iq1_s", 256, 50, 1, 1},
    {"iq1_m", 256, 56, 1, 0},  {"mxfp4", 32, 17, 4, 0},
    {"nvfp4", 64, 36, 4, 0},
};
#define KQO_NCODECS ((int)(sizeof(KQO_CODECS) / sizeof(KQO_CODECS[0])))

int kqo_codec_count(void) { return KQO_NCODECS; }

int kqo_codec_info(int i, const char** name, int* wpb, int* bpb, int* bits, int* req_imat) {
  if (i < 0 || i >= KQO_NCODECS) return 1;
  *name = KQO_CODECS[i].name;
  *wpb = KQO_CODECS[i].wpb;
  *bpb = KQO_CODECS[i].bpb;
  *bits = KQO_CODECS[i].bits;
  *req_imat = KQO_CODECS[i].requires_imatrix;
  return 0;
}

static int codec_index(const char* name) {
  for (int i = 0; i < KQO_NCODECS; i++)
    if (strcmp(KQO_CODECS[i].name, name) == 0) return i;
  return -1;
}

/* src/kquant_cpu_decode.cpp:43-47 */
static float rd_f16(const uint8_t* p) {
  _Float16 h;
  memcpy(&h, p, 2);
  return (float)h;
}

/* ---- block decoders, one block -> wpb floats ---- */

/* src/kquant_cpu_decode.cpp:50-63 */
static void blk_q8_0(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  const int8_t* qs = (const int8_t*)(b + 2);
  for (int i = 0; i < 32; i++) o[i] = d * (float)qs[i];
}

/* src/kquant_cpu_decode.cpp:66-82 */
static void blk_q4_0(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  const uint8_t* qs = b + 2;
  for (int j = 0; j < 16; j++) {
    o[j] = d * (float)((int)(qs[j] & 15) - 8);
    o[j + 16] = d * (float)((int)(qs[j] >> 4) - 8);
  }
}

/* src/kquant_cpu_decode.cpp:84-103 */
static void blk_q4_1(const uint8_t* b, float* o) {
  float d = rd_f16(b), m = rd_f16(b + 2);
  const uint8_t* qs = b + 4;
  for (int j = 0; j < 16; j++) {
    o[j] = d * (float)(qs[j] & 15) + m;
    o[j + 16] = d * (float)(qs[j] >> 4) + m;
  }
}

/* src/kquant_cpu_decode.cpp:105-128 (with_min = 0) and 130-153 (with_min = 1) */
static void blk_q5(const uint8_t* b, float* o, int with_min) {
  float d = rd_f16(b), m = with_min ? rd_f16(b + 2) : 0.f;
  const uint8_t* qhp = b + (with_min ? 4 : 2);
  const uint8_t* qs = b + (with_min ? 8 : 6);
  uint32_t qh = (uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24);
  for (int j = 0; j < 16; j++) {
    int x0 = (qs[j] & 15) | (int)(((qh >> j) << 4) & 0x10);
    int x1 = (qs[j] >> 4) | (int)((qh >> (j + 12)) & 0x10);
    if (with_min) {
      o[j] = d * (float)x0 + m;
      o[j + 16] = d * (float)x1 + m;
    } else {
      o[j] = d * (float)(x0 - 16);
      o[j + 16] = d * (float)(x1 - 16);
    }
  }
}
static void blk_q5_0(const uint8_t* b, float* o) { blk_q5(b, o, 0); }
static void blk_q5_1(const uint8_t* b, float* o) { blk_q5(b, o, 1); }

/* src/kquant_cpu_decode.cpp:383-397 */
static void blk_iq4_nl(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  const uint8_t* qs = b + 2;
  for (int j = 0; j < 16; j++) {
    o[j] = d * (float)kq_tab_iq4nl[qs[j] & 15];
    o[j + 16] = d * (float)kq_tab_iq4nl[qs[j] >> 4];
  }
}

/* src/kquant_cpu_decode.cpp:155-174: eight 6-bit (scale, min) pairs in 12 B */
static void q4k_scales(const uint8_t* s, float d, float dmin, float* sc, float* mn) {
  for (int i = 0; i < 8; i++) {
    int rs, rm;
    if (i < 4) {
      rs = s[i] & 63;
      rm = s[i + 4] & 63;
    } else {
      rs = (s[i + 4] & 15) | ((s[i - 4] >> 6) << 4);
      rm = (s[i + 4] >> 4) | ((s[i] >> 6) << 4);
    }
    sc[i] = d * (float)rs;
    mn[i] = dmin * (float)rm;
  }
}

/* src/kquant_cpu_decode.cpp:177-202 */
static void blk_q4_k(const uint8_t* b, float* o) {
  float sc[8], mn[8];
  q4k_scales(b + 4, rd_f16(b), rd_f16(b + 2), sc, mn);
  const uint8_t* qs = b + 16;
  for (int g = 0; g < 4; g++)
    for (int i = 0; i < 32; i++) {
      o[(2 * g) * 32 + i] = sc[2 * g] * (float)(qs[g * 32 + i] & 15) - mn[2 * g];
      o[(2 * g + 1) * 32 + i] = sc[2 * g + 1] * (float)(qs[g * 32 + i] >> 4) - mn[2 * g + 1];
    }
}

/* src/kquant_cpu_decode.cpp:205-235 */
static void blk_q5_k(const uint8_t* b, float* o) {
  float sc[8], mn[8];
  q4k_scales(b + 4, rd_f16(b), rd_f16(b + 2), sc, mn);
  const uint8_t* qh = b + 16;
  const uint8_t* qs = b + 48;
  for (int g = 0; g < 4; g++)
    for (int i = 0; i < 32; i++) {
      int lo0 = qs[g * 32 + i] & 15, lo1 = qs[g * 32 + i] >> 4;
      int hi0 = (qh[i] >> (2 * g)) & 1, hi1 = (qh[i] >> (2 * g + 1)) & 1;
      o[(2 * g) * 32 + i] = sc[2 * g] * (float)(lo0 | (hi0 << 4)) - mn[2 * g];
      o[(2 * g + 1) * 32 + i] = sc[2 * g + 1] * (float)(lo1 | (hi1 << 4)) - mn[2 * g + 1];
    }
}

/* src/kquant_cpu_decode.cpp:238-280; note (d * sc) * q, left to right */
static void blk_q6_k(const uint8_t* b, float* o) {
  const int8_t* scales = (const int8_t*)(b + 192);
  float d = rd_f16(b + 208);
  for (int h = 0; h < 2; h++) {
    const uint8_t* ql = b + h * 64;
    const uint8_t* qh = b + 128 + h * 32;
    const int8_t* sc = scales + h * 8;
    float* oh = o + h * 128;
    for (int l = 0; l < 32; l++) {
      int is0 = l / 16;
      int q1 = (int)(int8_t)((ql[l] & 15) | (((qh[l] >> 0) & 3) << 4)) - 32;
      int q2 = (int)(int8_t)((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
      int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      oh[l] = d * (float)sc[is0] * (float)q1;
      oh[l + 32] = d * (float)sc[is0 + 2] * (float)q2;
      oh[l + 64] = d * (float)sc[is0 + 4] * (float)q3;
      oh[l + 96] = d * (float)sc[is0 + 6] * (float)q4;
    }
  }
}

/* src/kquant_cpu_decode.cpp:282-337 */
static void blk_q3_k(const uint8_t* b, float* o) {
  const uint8_t* hmask = b;
  const uint8_t* qs = b + 32;
  const uint8_t* s = b + 96;
  float d = rd_f16(b + 108);
  int sc[16];
  for (int k = 0; k < 4; k++) {
    sc[k] = (s[k] & 15) | ((s[8 + k] & 3) << 4);
    sc[k + 4] = (s[k + 4] & 15) | (((s[8 + k] >> 2) & 3) << 4);
    sc[k + 8] = ((s[k] >> 4) & 15) | (((s[8 + k] >> 4) & 3) << 4);
    sc[k + 12] = ((s[k + 4] >> 4) & 15) | (((s[8 + k] >> 6) & 3) << 4);
  }
  for (int i = 0; i < 16; i++) sc[i] -= 32;
  int oi = 0;
  for (int h = 0; h < 2; h++) {
    const uint8_t* q = qs + h * 32;
    for (int si = 0; si < 4; si++) {
      int shift = si * 2;
      uint8_t m = (uint8_t)(1 << (h * 4 + si));
      int is = h * 8 + si * 2;
      float dl = d * (float)sc[is];
      for (int l = 0; l < 16; l++) {
        int q2 = (q[l] >> shift) & 3;
        int hh = (hmask[l] & m) ? 0 : 4;
        o[oi++] = dl * (float)(q2 - hh);
      }
      float dr = d * (float)sc[is + 1];
      for (int l = 0; l < 16; l++) {
        int q2 = (q[l + 16] >> shift) & 3;
        int hh = (hmask[l + 16] & m) ? 0 : 4;
        o[oi++] = dr * (float)(q2 - hh);
      }
    }
  }
}

/* src/kquant_cpu_decode.cpp:340-377 */
static void blk_q2_k(const uint8_t* b, float* o) {
  const uint8_t* scales = b;
  const uint8_t* qs = b + 16;
  float d = rd_f16(b + 80), dmin = rd_f16(b + 82);
  int oi = 0, is = 0;
  for (int h = 0; h < 2; h++) {
    const uint8_t* q = qs + h * 32;
    for (int si = 0; si < 4; si++) {
      int shift = si * 2;
      uint8_t sl = scales[is++];
      float dl = d * (float)(sl & 15), ml = dmin * (float)(sl >> 4);
      for (int l = 0; l < 16; l++) o[oi++] = dl * (float)((q[l] >> shift) & 3) - ml;
      uint8_t sr = scales[is++];
      float dr = d * (float)(sr & 15), mr = dmin * (float)(sr >> 4);
      for (int l = 0; l < 16; l++) o[oi++] = dr * (float)((q[l + 16] >> shift) & 3) - mr;
    }
  }
}

/* src/kquant_cpu_decode.cpp:441-465 */
static void blk_iq4_xs(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  uint16_t sh;
  memcpy(&sh, b + 2, 2);
  const uint8_t* sl = b + 4;
  const uint8_t* qs = b + 8;
  for (int ib = 0; ib < 8; ib++) {
    int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4);
    float dl = d * (float)(ls - 32);
    const uint8_t* q = qs + ib * 16;
    float* oo = o + ib * 32;
    for (int j = 0; j < 16; j++) {
      oo[j] = dl * (float)kq_tab_iq4nl[q[j] & 15];
      oo[j + 16] = dl * (float)kq_tab_iq4nl[q[j] >> 4];
    }
  }
}

/* src/kquant_cpu_decode.cpp:557-584 */
static void blk_iq2_xxs(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  const uint8_t* qs = b + 2;
  for (int ib = 0; ib < 8; ib++) {
    uint32_t aux[2];
    memcpy(aux, qs + 8 * ib, 8);
    const uint8_t* a8 = (const uint8_t*)aux;
    float db = d * (0.5f + (float)(aux[1] >> 28)) * 0.25f;
    for (int l = 0; l < 4; l++) {
      const uint8_t* g = (const uint8_t*)(kq_tab_iq2xxs_grid + a8[l]);
      uint8_t signs = kq_tab_ksigns[(aux[1] >> (7 * l)) & 127];
      for (int j = 0; j < 8; j++)
        o[j] = db * (float)g[j] * ((signs & kq_tab_kmask[j]) ? -1.f : 1.f);
      o += 8;
    }
  }
}


/* sign of weight j of an eight-weight group whose sign bits are `signs` */
static float sgn(uint8_t signs, int j) { return (signs & kq_tab_kmask[j]) ? -1.f : 1.f; }

/* src/kquant_cpu_decode.cpp:468-503: [d][qs 64][8 x u32 = 4 x 7-bit sign index + 4-bit scale] */
static void blk_iq3_xxs(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  for (int ib = 0; ib < 8; ib++) {
    uint32_t aux;
    memcpy(&aux, b + 66 + 4 * ib, 4);
    float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    const uint8_t* q = b + 2 + 8 * ib;
    for (int l = 0; l < 4; l++, o += 8) {
      uint8_t signs = kq_tab_ksigns[(aux >> (7 * l)) & 127];
      const uint8_t* g1 = (const uint8_t*)(kq_tab_iq3xxs_grid + q[2 * l]);
      const uint8_t* g2 = (const uint8_t*)(kq_tab_iq3xxs_grid + q[2 * l + 1]);
      for (int j = 0; j < 4; j++) {
        o[j] = db * (float)g1[j] * sgn(signs, j);
        o[j + 4] = db * (float)g2[j] * sgn(signs, j + 4);
      }
    }
  }
}

/* src/kquant_cpu_decode.cpp:505-556: [d][qs 64][qh 8][signs 32][scales 4] */
static void blk_iq3_s(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  for (int ib = 0; ib < 8; ib++) {
    uint8_t sb = b[106 + ib / 2];
    float db = d * (float)(1 + 2 * ((ib & 1) ? (sb >> 4) : (sb & 15)));
    const uint8_t* q = b + 2 + 8 * ib;
    const uint8_t* sg = b + 74 + 4 * ib;
    uint32_t qh = b[66 + ib];
    for (int l = 0; l < 4; l++, o += 8) {
      const uint8_t* g1 = (const uint8_t*)(kq_tab_iq3s_grid + (q[2 * l] | ((qh << (8 - 2 * l)) & 256)));
      const uint8_t* g2 = (const uint8_t*)(kq_tab_iq3s_grid + (q[2 * l + 1] | ((qh << (7 - 2 * l)) & 256)));
      for (int j = 0; j < 4; j++) {
        o[j] = db * (float)g1[j] * sgn(sg[l], j);
        o[j + 4] = db * (float)g2[j] * sgn(sg[l], j + 4);
      }
    }
  }
}

/* src/kquant_cpu_decode.cpp:586-616: [d][32 x u16 = 9-bit lattice index | 7-bit sign index][scales 8] */
static void blk_iq2_xs(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  for (int ib = 0; ib < 8; ib++) {
    uint8_t sb = b[66 + ib];
    float db[2] = {d * (0.5f + (float)(sb & 15)) * 0.25f, d * (0.5f + (float)(sb >> 4)) * 0.25f};
    for (int l = 0; l < 4; l++, o += 8) {
      uint16_t q;
      memcpy(&q, b + 2 + 2 * (4 * ib + l), 2);
      const uint8_t* g = (const uint8_t*)(kq_tab_iq2xs_grid + (q & 511));
      uint8_t signs = kq_tab_ksigns[q >> 9];
      for (int j = 0; j < 8; j++) o[j] = db[l / 2] * (float)g[j] * sgn(signs, j);
    }
  }
}

/* src/kquant_cpu_decode.cpp:618-649: [d][qs 32][signs 32][qh 8][scales 8] */
static void blk_iq2_s(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  for (int ib = 0; ib < 8; ib++) {
    uint8_t sb = b[74 + ib];
    float db[2] = {d * (0.5f + (float)(sb & 15)) * 0.25f, d * (0.5f + (float)(sb >> 4)) * 0.25f};
    uint32_t qh = b[66 + ib];
    for (int l = 0; l < 4; l++, o += 8) {
      const uint8_t* g = (const uint8_t*)(kq_tab_iq2s_grid + (b[2 + 4 * ib + l] | ((qh << (8 - 2 * l)) & 0x300)));
      uint8_t signs = b[34 + 4 * ib + l];
      for (int j = 0; j < 8; j++) o[j] = db[l / 2] * (float)g[j] * sgn(signs, j);
    }
  }
}

/* src/kquant_cpu_decode.cpp:658-685: [d][qs 32][8 x u16 qh]; lattice bytes are signed, + or - 1/8 added */
static void blk_iq1_s(const uint8_t* b, float* o) {
  float d = rd_f16(b);
  for (int ib = 0; ib < 8; ib++) {
    uint16_t qh;
    memcpy(&qh, b + 34 + 2 * ib, 2);
    float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
    float delta = (qh & 0x8000) ? -0.125f : 0.125f;
    for (int l = 0; l < 4; l++, o += 8) {
      const int8_t* g = (const int8_t*)(kq_tab_iq1s_grid + (b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)));
      for (int j = 0; j < 8; j++) o[j] = dl * ((float)g[j] + delta);
    }
  }
}

/* src/kquant_cpu_decode.cpp:687-735: [qs 32][qh 16][4 x u16 scales]; the fp16 super-scale is the four top nibbles */
static void blk_iq1_m(const uint8_t* b, float* o) {
  uint16_t sc[4];
  memcpy(sc, b + 48, 8);
  uint16_t dbits = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000));
  float d = rd_f16((const uint8_t*)&dbits);
  for (int ib = 0; ib < 8; ib++) {
    float dl[2] = {d * (float)(2 * ((sc[ib / 2] >> (6 * (ib % 2))) & 7) + 1),
                   d * (float)(2 * ((sc[ib / 2] >> (6 * (ib % 2) + 3)) & 7) + 1)};
    for (int l = 0; l < 4; l++, o += 8) {
      uint32_t qh = b[32 + 2 * ib + l / 2];
      uint32_t idx = b[4 * ib + l] | ((qh << ((l & 1) ? 4 : 8)) & 0x700);
      float delta = (qh & ((l & 1) ? 0x80 : 0x08)) ? -0.125f : 0.125f;
      const int8_t* g = (const int8_t*)(kq_tab_iq1s_grid + idx);
      for (int j = 0; j < 8; j++) o[j] = dl[l / 2] * ((float)g[j] + delta);
    }
  }
}

/* src/kquant_fp_tables.h:24-31: E8M0 byte -> 2^(e - 127) / 2, subnormal results built from the bits */
static float e8m0_half(uint8_t e) {
  uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
/* src/kquant_fp_tables.h:36-45: unsigned E4M3 (bias 7) byte -> value / 2; 0x00 and 0x7f give 0 */
static float ue4m3_half(uint8_t x) {
  if (x == 0 || x == 0x7f) return 0.f;
  int ex = (x >> 3) & 15;
  float man = (float)(x & 7);
  float raw = ex == 0 ? man * 0x1p-9f : ldexpf(1.0f + man * 0.125f, ex - 7);
  return raw * 0.5f;
}
/* src/kquant_cpu_decode.cpp:404-419 */
static void blk_mxfp4(const uint8_t* b, float* o) {
  float d = e8m0_half(b[0]);
  for (int j = 0; j < 16; j++) {
    o[j] = d * (float)kq_tab_mxfp4[b[1 + j] & 15];
    o[j + 16] = d * (float)kq_tab_mxfp4[b[1 + j] >> 4];
  }
}
/* src/kquant_cpu_decode.cpp:421-438: four groups of sixteen weights, one scale byte each */
static void blk_nvfp4(const uint8_t* b, float* o) {
  for (int g = 0; g < 4; g++) {
    float d = ue4m3_half(b[g]);
    const uint8_t* q = b + 4 + 8 * g;
    for (int j = 0; j < 8; j++) {
      o[16 * g + j] = d * (float)kq_tab_mxfp4[q[j] & 15];
      o[16 * g + j + 8] = d * (float)kq_tab_mxfp4[q[j] >> 4];
    }
  }
}

typedef void (*blk_fn)(const uint8_t*, float*);
static const blk_fn BLK_FNS[] = {blk_q2_k, blk_q3_k, blk_q4_k, blk_q5_k,   blk_q6_k,
                                 blk_q4_0, blk_q8_0, blk_iq4_nl, blk_iq4_xs, blk_iq2_xxs,
                                 blk_q4_1, blk_q5_0, blk_q5_1, blk_iq3_xxs, blk_iq3_s,
                                 blk_iq2_xs, blk_iq2_s, blk_iq1_s, blk_iq1_m, blk_mxfp4, blk_nvfp4};

/* ---- output rounding: one IEEE RNE rounding of the exact f32 value ---- */
static uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static void store(void* out, size_t i, float v, int dtype) {
  if (dtype == 0) {
    ((float*)out)[i] = v;
  } else if (dtype == 1) {
    ((_Float16*)out)[i] = (_Float16)v;
  } else {
    ((uint16_t*)out)[i] = f32_to_bf16(v);
  }
}
static float load(const void* in, size_t i, int dtype) {
  if (dtype == 0) return ((const float*)in)[i];
  if (dtype == 1) return (float)((const _Float16*)in)[i];
  return bf16_to_f32(((const uint16_t*)in)[i]);
}

typedef struct {
  const uint8_t* w;
  void* out;
  int wpb, bpb;
  blk_fn fn;
  int dtype;
} deq_ctx;

static void deq_range(long long b0, long long b1, void* p) {
  deq_ctx* c = (deq_ctx*)p;
  float buf[256];
  for (long long b = b0; b < b1; b++) {
    c->fn(c->w + (size_t)b * c->bpb, buf);
    for (int i = 0; i < c->wpb; i++) store(c->out, (size_t)b * c->wpb + i, buf[i], c->dtype);
  }
}

/* src/kquant_cpu_decode.cpp:1136-1207 (dispatch + block-parallel driver).
 * dtype: 0 f32, 1 f16, 2 bf16. Returns 0, or 1 for an unknown codec/dtype. */
int kqo_dequantize(const uint8_t* w, void* out, size_t num_weights, const char* codec, int dtype) {
  int ci = codec_index(codec);
  if (ci < 0 || dtype < 0 || dtype > 2) return 1;
  const int wpb = KQO_CODECS[ci].wpb, bpb = KQO_CODECS[ci].bpb;
  const blk_fn fn = BLK_FNS[ci];
  deq_ctx c = {w, out, wpb, bpb, fn, dtype};
  par_for((long long)(num_weights / (size_t)wpb), deq_range, &c);
  return 0;
}

/* src/kquant_cpu_decode.cpp:1010-1024: eight strided partial sums, fixed tree */
static float dot_block(const float* a, const float* b, int n) {
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int i = 0; i < n; i += 8)
    for (int j = 0; j < 8; j++) s[j] += a[i + j] * b[i + j];
  return ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
}

typedef struct {
  float* of;
  const float* xf;
  const uint8_t* w;
  float* wd;
  int M, N, K, transpose, wpb, bpb, w_cols;
  size_t row_bytes;
  blk_fn fn;
} qmm_ctx;

/* src/kquant_cpu_decode.cpp:1032-1065 (qmv_fused_rows) over rows [n0, n1) */
static void qmm_fused_range(long long n0, long long n1, void* p) {
  qmm_ctx* c = (qmm_ctx*)p;
  float buf[256], acc[16];
  const int nblocks = c->K / c->wpb;
  for (long long n = n0; n < n1; n++) {
    const uint8_t* wr = c->w + (size_t)n * c->row_bytes;
    for (int m = 0; m < c->M; m++) acc[m] = 0.f;
    for (int b = 0; b < nblocks; b++) {
      c->fn(wr + (size_t)b * c->bpb, buf);
      const float* xb = c->xf + (size_t)b * c->wpb;
      for (int m = 0; m < c->M; m++) acc[m] += dot_block(xb + (size_t)m * c->K, buf, c->wpb);
    }
    for (int m = 0; m < c->M; m++) c->of[(size_t)m * c->N + n] = acc[m];
  }
}

/* src/kquant_cpu_decode.cpp:1301-1312: dequantize weight rows [r0, r1) */
static void qmm_decode_range(long long r0, long long r1, void* p) {
  qmm_ctx* c = (qmm_ctx*)p;
  for (long long r = r0; r < r1; r++)
    for (int b = 0; b < c->w_cols / c->wpb; b++)
      c->fn(c->w + (size_t)r * c->row_bytes + (size_t)b * c->bpb,
            c->wd + (size_t)r * c->w_cols + (size_t)b * c->wpb);
}

/* src/kquant_cpu_decode.cpp:1333-1352: sequential-K scalar GEMM, columns [n0, n1) */
static void qmm_gemm_range(long long n0, long long n1, void* p) {
  qmm_ctx* c = (qmm_ctx*)p;
  for (int m = 0; m < c->M; m++) {
    const float* xm = c->xf + (size_t)m * c->K;
    for (long long n = n0; n < n1; n++) {
      float acc = 0.f;
      if (c->transpose) {
        const float* wn = c->wd + (size_t)n * c->K;
        for (int k = 0; k < c->K; k++) acc += xm[k] * wn[k];
      } else {
        for (int k = 0; k < c->K; k++) acc += xm[k] * c->wd[(size_t)k * c->N + n];
      }
      c->of[(size_t)m * c->N + n] = acc;
    }
  }
}

/* Row-major fp32 core of kquant_qmm_cpu: of[M,N] = xf[M,K] . dequant(w)^T (or
 * . dequant(w) when !transpose). fused != 0 selects the decode-then-dot GEMV
 * (needs transpose and M <= 16), else dequantize-once + sequential-K GEMM. */
static int qmm_f32(float* of, const float* xf, const uint8_t* w, int M, int N, int K,
                   int transpose, int ci, int fused) {
  qmm_ctx c;
  c.of = of;
  c.xf = xf;
  c.w = w;
  c.wd = NULL;
  c.M = M;
  c.N = N;
  c.K = K;
  c.transpose = transpose;
  c.wpb = KQO_CODECS[ci].wpb;
  c.bpb = KQO_CODECS[ci].bpb;
  c.fn = BLK_FNS[ci];
  const int w_rows = transpose ? N : K;
  c.w_cols = transpose ? K : N;
  c.row_bytes = (size_t)(c.w_cols / c.wpb) * c.bpb;
  if (fused) {
    par_for(N, qmm_fused_range, &c);
    return 0;
  }
  c.wd = (float*)malloc(((size_t)w_rows * c.w_cols + 1) * sizeof(float));
  if (!c.wd) return 2;
  par_for(w_rows, qmm_decode_range, &c);
  par_for(N, qmm_gemm_range, &c);
  free(c.wd);
  return 0;
}

/* src/kquant_cpu_decode.cpp:1210-1359 (kquant_qmm_cpu): stage x in f32, pick
 * the regime by M <= 16 (kQmvFusedMaxM, src/kquant_cpu_decode.h:72), round the
 * f32 result once to the x dtype. */
int kqo_qmm(void* result, const void* x, const uint8_t* w, int M, int N, int K, int transpose,
            const char* codec, int dtype) {
  int ci = codec_index(codec);
  if (ci < 0 || dtype < 0 || dtype > 2) return 1;
  size_t xe = (size_t)M * K, oe = (size_t)M * N;
  float* xf = (float*)malloc((xe ? xe : 1) * sizeof(float));
  float* of = (float*)malloc((oe ? oe : 1) * sizeof(float));
  if (!xf || !of) return 2;
  for (size_t i = 0; i < xe; i++) xf[i] = load(x, i, dtype);
  int rc = qmm_f32(of, xf, w, M, N, K, transpose, ci, transpose && M <= 16);
  for (size_t i = 0; i < oe; i++) store(result, i, of[i], dtype);
  free(xf);
  free(of);
  return rc;
}

/* src/kquant_gather.cpp:496-731 (KQuantGatherQMM::eval_cpu), restated.
 *   out[b] [M,N] = x[lhs[b]] [M,K] . dequant(w[rhs[b]])^T,  b in [0, n_entries)
 * x is [x_batch, M, K] dense; w is E experts, expert e at w + e*w_expert_stride
 * bytes (64-bit, so strided or >2 GiB stacks work, cf. kquant_gather.cpp:548-563).
 * The reference groups entries by expert and then picks the accumulation order
 * per group, which is all that matters numerically:
 *   - if transpose and every group has rg*M <= 16 rows, all groups go through
 *     the fused GEMV (kquant_qmm_cpu_batch, src/kquant_cpu_decode.cpp:1362-1527);
 *   - otherwise each group runs kquant_qmm_cpu on its packed rg*M rows, which
 *     is again the fused GEMV when transpose and rg*M <= 16 and the
 *     sequential-K GEMM otherwise.
 * Both cases reduce to one rule per group: fused iff transpose && rg*M <= 16.
 * Duplicate (lhs, rhs) entries produce identical rows either way, so the
 * reference's dedupe needs no restating. */
int kqo_gather_qmm(void* out, const void* x, const uint8_t* w, const uint32_t* lhs,
                   const uint32_t* rhs, long long n_entries, int M, int N, int K, int n_experts,
                   long long w_expert_stride, int transpose, const char* codec, int dtype) {
  int ci = codec_index(codec);
  if (ci < 0 || dtype < 0 || dtype > 2) return 1;
  long long* count = (long long*)calloc((size_t)n_experts + 1, sizeof(long long));
  if (!count) return 2;
  for (long long b = 0; b < n_entries; b++) {
    if ((int)rhs[b] >= n_experts) {
      free(count);
      return 3;
    }
    count[rhs[b]]++;
  }
  /* stable grouping by expert: order[] lists entries expert by expert */
  long long* start = (long long*)malloc(((size_t)n_experts + 1) * sizeof(long long));
  long long* order = (long long*)malloc((size_t)(n_entries ? n_entries : 1) * sizeof(long long));
  long long acc = 0;
  for (int e = 0; e < n_experts; e++) {
    start[e] = acc;
    acc += count[e];
  }
  start[n_experts] = acc;
  long long* fill = (long long*)calloc((size_t)n_experts + 1, sizeof(long long));
  for (long long b = 0; b < n_entries; b++) order[start[rhs[b]] + fill[rhs[b]]++] = b;
  int rc = 0;
  for (int e = 0; e < n_experts && rc == 0; e++) {
    long long rg = count[e];
    if (rg == 0) continue;
    int rows = (int)rg * M;
    int fused = transpose && rows <= 16;
    float* xf = (float*)malloc((size_t)rows * K * sizeof(float));
    float* of = (float*)malloc((size_t)rows * N * sizeof(float));
    for (long long r = 0; r < rg; r++) {
      long long b = order[start[e] + r];
      for (size_t i = 0; i < (size_t)M * K; i++)
        xf[(size_t)r * M * K + i] = load(x, (size_t)lhs[b] * M * K + i, dtype);
    }
    rc = qmm_f32(of, xf, w + (size_t)e * (size_t)w_expert_stride, rows, N, K, transpose, ci, fused);
    for (long long r = 0; r < rg; r++) {
      long long b = order[start[e] + r];
      for (size_t i = 0; i < (size_t)M * N; i++)
        store(out, (size_t)b * M * N + i, of[(size_t)r * M * N + i], dtype);
    }
    free(xf);
    free(of);
  }
  free(count);
  free(start);
  free(order);
  free(fill);
  return rc;
}
