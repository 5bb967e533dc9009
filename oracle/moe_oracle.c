/* CPU oracle of the MoE expert layer: test infrastructure and the timed CPU baseline, never the product path.
 * What each function restates is cited beside it; moe_oracle.h says what is pinned and what is not. */
#include "moe_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "iq3s_grid.h" /* generated at build time from gguf-py, sha256-checked: kIq3sGrid[512] */

#define QK_K 256
#define ORC_PIECES 8 /* the router product's pieces */

static inline float h2f(uint16_t h) { return _cvtsh_ss(h); }
static inline uint16_t f2h(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
static inline uint16_t rd16(const uint8_t *p) {
  uint16_t v;
  memcpy(&v, p, 2);
  return v;
}
static inline float rdf(const uint8_t *p) {
  float v;
  memcpy(&v, p, 4);
  return v;
}

int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* The threads every later parallel loop takes. The reference sizes its pool from the cores the process may run on
 * (docs/DESIGN.md:694-696), not from an environment variable: the caller counts them and says so here. */
void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* shared/quant.h:36-75 */
uint32_t orc_block_values(uint32_t t) {
  switch (t) {
    case ORC_Q8_0: case ORC_IQ4_NL: return 32;
    case ORC_Q2_0: return 64;
    case ORC_Q4_K: case ORC_Q6_K: case ORC_Q8_K: case ORC_IQ3_S: case ORC_IQ4_XS: case ORC_IQ3_XXS: case ORC_IQ2_S: return 256;
    default: return 0;
  }
}
uint32_t orc_block_bytes(uint32_t t) {
  switch (t) {
    case ORC_Q8_0: return 34;
    case ORC_Q4_K: return 144;
    case ORC_Q6_K: return 210;
    case ORC_Q8_K: return 292;
    case ORC_IQ3_S: return 110;
    case ORC_IQ4_NL: return 18;
    case ORC_IQ4_XS: return 136;
    case ORC_IQ3_XXS: return 98;
    case ORC_IQ2_S: return 82;
    case ORC_Q2_0: return 18;
    default: return 0;
  }
}
uint32_t orc_vec_dot_type(uint32_t t) { return t == ORC_Q8_0 || t == ORC_IQ4_NL || t == ORC_Q2_0 ? ORC_Q8_0 : ORC_Q8_K; }
uint64_t orc_row_bytes(uint32_t t, uint64_t n) { return n / orc_block_values(t) * orc_block_bytes(t); }

/* The fields of a block in run order, (offset, size): shared/quant.h:78-169. */
static uint32_t fields(uint32_t t, uint32_t off[5], uint32_t sz[5]) {
  switch (t) {
    case ORC_Q8_0: off[0] = 2, sz[0] = 32, off[1] = 0, sz[1] = 2; return 2;
    case ORC_Q4_K: off[0] = 16, sz[0] = 128, off[1] = 4, sz[1] = 12, off[2] = 0, sz[2] = 4; return 3;
    case ORC_Q6_K: off[0] = 0, sz[0] = 128, off[1] = 128, sz[1] = 64, off[2] = 192, sz[2] = 16, off[3] = 208, sz[3] = 2; return 4;
    case ORC_IQ3_S:
      off[0] = 2, sz[0] = 64, off[1] = 74, sz[1] = 32, off[2] = 66, sz[2] = 8, off[3] = 106, sz[3] = 4, off[4] = 0, sz[4] = 2;
      return 5;
    case ORC_IQ4_NL: case ORC_Q2_0: off[0] = 2, sz[0] = 16, off[1] = 0, sz[1] = 2; return 2;
    case ORC_IQ4_XS: off[0] = 8, sz[0] = 128, off[1] = 4, sz[1] = 4, off[2] = 2, sz[2] = 2, off[3] = 0, sz[3] = 2; return 4;
    /* grid indices, scale-and-sign words, d; and grid index low bits, signs, qh, scales, d (QUANT_FORMATS.md:602-603) */
    case ORC_IQ3_XXS: off[0] = 2, sz[0] = 64, off[1] = 66, sz[1] = 32, off[2] = 0, sz[2] = 2; return 3;
    case ORC_IQ2_S: off[0] = 2, sz[0] = 32, off[1] = 34, sz[1] = 32, off[2] = 66, sz[2] = 8, off[3] = 74, sz[3] = 8, off[4] = 0, sz[4] = 2; return 5;
    default: return 0;
  }
}

void orc_to_runs(uint32_t t, const uint8_t *src, uint64_t n, uint8_t *dst) {
  uint32_t off[5], sz[5];
  const uint32_t nf = fields(t, off, sz), bb = orc_block_bytes(t);
  uint64_t run = 0;
  for (uint32_t f = 0; f < nf; f++) {
    for (uint64_t k = 0; k < n; k++) memcpy(dst + run + k * sz[f], src + k * bb + off[f], sz[f]);
    run += (uint64_t)sz[f] * n;
  }
}
void orc_from_runs(uint32_t t, const uint8_t *src, uint64_t n, uint8_t *dst) {
  uint32_t off[5], sz[5];
  const uint32_t nf = fields(t, off, sz), bb = orc_block_bytes(t);
  uint64_t run = 0;
  for (uint32_t f = 0; f < nf; f++) {
    for (uint64_t k = 0; k < n; k++) memcpy(dst + k * bb + off[f], src + run + k * sz[f], sz[f]);
    run += (uint64_t)sz[f] * n;
  }
}

/* ksigns_iq2xs[k]: k with bit 7 set when k has an odd number of set bits, so that every sign byte has even parity
 * (QUANT_FORMATS.md:167-168; the table's sha256, :548, is checked against this rule in the tests). */
static inline uint8_t ksigns(uint32_t k) {
  uint32_t p = k ^ (k >> 4);
  p ^= p >> 2, p ^= p >> 1;
  return (uint8_t)(k | ((p & 1u) << 7));
}

/* Q4_K's packed 6-bit scale and minimum of sub-block j (QUANT_FORMATS.md:386-392). */
static inline void q4k_scale_min(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* ------------------------------------------------------------------------------------------------------------
 * Dequantisation (QUANT_FORMATS.md: Q8_0 :461, Q4_K :394, Q6_K :441, IQ3_S :199-207). */
void orc_dequantize_row(uint32_t t, const void *vb, float *y, int64_t n) {
  const uint8_t *b = (const uint8_t *)vb;
  const int64_t nb = n / orc_block_values(t);
  for (int64_t i = 0; i < nb; i++, b += orc_block_bytes(t)) {
    if (t == ORC_Q8_0) {
      const float d = h2f(rd16(b));
      for (int j = 0; j < 32; j++) y[i * 32 + j] = d * (float)(int8_t)b[2 + j];
    } else if (t == ORC_Q4_K) {
      const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
      const uint8_t *scales = b + 4, *qs = b + 16;
      float *yy = y + i * QK_K;
      for (int c = 0; c < 4; c++) {
        uint8_t sc, m;
        q4k_scale_min(2 * c, scales, &sc, &m);
        const float d1 = d * sc, m1 = dmin * m;
        q4k_scale_min(2 * c + 1, scales, &sc, &m);
        const float d2 = d * sc, m2 = dmin * m;
        for (int l = 0; l < 32; l++) yy[64 * c + l] = d1 * (float)(qs[32 * c + l] & 0xF) - m1;
        for (int l = 0; l < 32; l++) yy[64 * c + 32 + l] = d2 * (float)(qs[32 * c + l] >> 4) - m2;
      }
    } else if (t == ORC_Q6_K) {
      const uint8_t *ql = b, *qh = b + 128;
      const int8_t *sc = (const int8_t *)(b + 192);
      const float d = h2f(rd16(b + 208));
      float *yy = y + i * QK_K;
      for (int h = 0; h < 2; h++)
        for (int l = 0; l < 32; l++) {
          const int is = 8 * h + l / 16;
          const uint8_t hb = qh[32 * h + l];
          const int q1 = (int)((ql[64 * h + l] & 0xF) | (((hb >> 0) & 3) << 4)) - 32;
          const int q2 = (int)((ql[64 * h + 32 + l] & 0xF) | (((hb >> 2) & 3) << 4)) - 32;
          const int q3 = (int)((ql[64 * h + l] >> 4) | (((hb >> 4) & 3) << 4)) - 32;
          const int q4 = (int)((ql[64 * h + 32 + l] >> 4) | (((hb >> 6) & 3) << 4)) - 32;
          yy[128 * h + l] = d * sc[is] * q1;
          yy[128 * h + 32 + l] = d * sc[is + 2] * q2;
          yy[128 * h + 64 + l] = d * sc[is + 4] * q3;
          yy[128 * h + 96 + l] = d * sc[is + 6] * q4;
        }
    } else if (t == ORC_IQ3_S) {
      const float d = h2f(rd16(b));
      const uint8_t *qs = b + 2, *qh = b + 66, *signs = b + 74, *scales = b + 106;
      float *yy = y + i * QK_K;
      for (int sb = 0; sb < 8; sb++) {
        const int ls = (scales[sb / 2] >> (4 * (sb % 2))) & 0xF;
        const float db = d * (float)(1 + 2 * ls);
        for (int k = 0; k < 8; k++) {
          const uint32_t idx = qs[8 * sb + k] | (((uint32_t)(qh[sb] >> k) & 1u) << 8);
          const uint32_t g = kIq3sGrid[idx];
          const uint8_t sg = signs[4 * sb + k / 2];
          for (int v = 0; v < 4; v++) {
            const int neg = (sg >> (4 * (k % 2) + v)) & 1;
            yy[32 * sb + 4 * k + v] = db * (float)((g >> (8 * v)) & 0xFF) * (neg ? -1.0f : 1.0f);
          }
        }
      }
    } else if (t == ORC_IQ4_NL) {
      /* y = d * kvalues[nibble]; byte j: low nibble value j, high nibble value j + 16 (QUANT_FORMATS.md:234-244). */
      const float d = h2f(rd16(b));
      for (int j = 0; j < 16; j++) {
        y[i * 32 + j] = d * (float)kIq4nlValues[b[2 + j] & 0xF];
        y[i * 32 + 16 + j] = d * (float)kIq4nlValues[b[2 + j] >> 4];
      }
    } else if (t == ORC_IQ4_XS) {
      /* y = d * (ls - 32) * kvalues[nibble], ls the sub-block's 6-bit scale: low 4 bits in scales_l, high 2 in scales_h
       * (QUANT_FORMATS.md:213-226). */
      const float d = h2f(rd16(b));
      const uint32_t sh = rd16(b + 2);
      const uint8_t *sl = b + 4, *qs = b + 8;
      for (int ib = 0; ib < 8; ib++) {
        const int ls = (int)(((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
        const float dl = d * (float)ls;
        for (int j = 0; j < 16; j++) {
          y[i * QK_K + 32 * ib + j] = dl * (float)kIq4nlValues[qs[16 * ib + j] & 0xF];
          y[i * QK_K + 32 * ib + 16 + j] = dl * (float)kIq4nlValues[qs[16 * ib + j] >> 4];
        }
      }
    } else if (t == ORC_Q2_0) {
      /* y = (q - 1) * d, q the 2-bit code: value j is bits 2 (j mod 4) .. of byte j / 4 (QUANT_FORMATS.md:251-263). */
      const float d = h2f(rd16(b));
      for (int j = 0; j < 64; j++) y[i * 64 + j] = (float)((int)((b[2 + j / 4] >> (2 * (j % 4))) & 3) - 1) * d;
    } else if (t == ORC_IQ3_XXS) {
      /* y = d * (0.5 + s) / 2 * grid byte * sign; sub-block sb's word holds four 7-bit sign indices, each completed to
       * 8 signs by parity, and the scale s in bits 28-31 (QUANT_FORMATS.md:147-168). */
      const float d = h2f(rd16(b));
      const uint8_t *qs = b + 2, *gas = b + 66;
      for (int sb = 0; sb < 8; sb++) {
        uint32_t w32;
        memcpy(&w32, gas + 4 * sb, 4);
        const float db = d * (0.5f + (float)(w32 >> 28)) * 0.5f;
        for (int l = 0; l < 4; l++) {
          const uint8_t signs = ksigns((w32 >> (7 * l)) & 127);
          for (int k = 0; k < 2; k++) {
            const uint32_t g = kIq3xxsGrid[qs[8 * sb + 2 * l + k]];
            for (int v = 0; v < 4; v++)
              y[i * QK_K + 32 * sb + 8 * l + 4 * k + v] = db * (float)((g >> (8 * v)) & 0xFF) * (((signs >> (4 * k + v)) & 1) ? -1.0f : 1.0f);
          }
        }
      }
    } else if (t == ORC_IQ2_S) {
      /* y = d * (0.5 + s) / 4 * grid byte * sign: groups of 8 values from a 10-bit index (qs and two bits of qh), a
       * byte of signs a group, a scale nibble per 16 values (QUANT_FORMATS.md:115-137). */
      const float d = h2f(rd16(b));
      const uint8_t *qs = b + 2, *sg = b + 34, *qh = b + 66, *sc = b + 74;
      for (int sb = 0; sb < 8; sb++) {
        for (int g = 0; g < 4; g++) {
          const float db = d * (0.5f + (float)((sc[sb] >> (4 * (g / 2))) & 0xF)) * 0.25f;
          const uint32_t idx = qs[4 * sb + g] | ((((uint32_t)qh[sb] >> (2 * g)) & 3u) << 8);
          const uint8_t signs = sg[4 * sb + g];
          for (int v = 0; v < 8; v++) {
            const uint32_t word = kIq2sGrid[2 * idx + v / 4];
            y[i * QK_K + 32 * sb + 8 * g + v] = db * (float)((word >> (8 * (v % 4))) & 0xFF) * (((signs >> v) & 1) ? -1.0f : 1.0f);
          }
        }
      }
    }
  }
}

/* ------------------------------------------------------------------------------------------------------------
 * Activation quantisers. q8_0: {f16 d; int8 qs[32]}, d = max|x| / 127, q = round(x * (1/d)), 0 when d is 0
 * (QUANT_FORMATS.md:463-465, :525-526). q8_K: {f32 d; int8 qs[256]; int16 bsums[16]}, iscale = -127 / max with max
 * the value of largest magnitude, q = min(127, nearest(iscale * x)), d = 1 / iscale (QUANT_FORMATS.md:528-535). */
static inline int nearest_even(float v) {
  /* Adding 1.5 * 2^23 leaves the integer nearest v (ties to even) in the low mantissa bits, for |v| < 2^22. */
  const float s = v + 12582912.0f;
  int32_t i;
  memcpy(&i, &s, 4);
  return (i & 0x007fffff) - 0x00400000;
}

void orc_quantize_row(uint32_t at, const float *x, void *vy, int64_t n) {
  uint8_t *y = (uint8_t *)vy;
  if (at == ORC_Q8_0) {
    for (int64_t i = 0; i < n / 32; i++, y += 34, x += 32) {
      float amax = 0.0f;
      for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(x[j]));
      const float d = amax / 127.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
      const uint16_t hd = f2h(d);
      memcpy(y, &hd, 2);
      for (int j = 0; j < 32; j++) ((int8_t *)y)[2 + j] = (int8_t)roundf(x[j] * id);
    }
    return;
  }
  for (int64_t i = 0; i < n / QK_K; i++, y += 292, x += QK_K) {
    float max = 0.0f, amax = 0.0f;
    for (int j = 0; j < QK_K; j++) {
      const float ax = fabsf(x[j]);
      if (ax > amax) amax = ax, max = x[j];
    }
    int8_t *qs = (int8_t *)(y + 4);
    int16_t bs[16];
    if (amax == 0.0f) {
      memset(y, 0, 292);
      continue;
    }
    const float iscale = -127.0f / max;
    for (int j = 0; j < QK_K; j++) {
      const int v = nearest_even(iscale * x[j]);
      qs[j] = (int8_t)(v < 127 ? v : 127);
    }
    for (int j = 0; j < 16; j++) {
      int s = 0;
      for (int l = 0; l < 16; l++) s += qs[16 * j + l];
      bs[j] = (int16_t)s;
    }
    const float d = 1.0f / iscale;
    memcpy(y, &d, 4);
    memcpy(y + 260, bs, 32);
  }
}

/* ------------------------------------------------------------------------------------------------------------
 * Dots: integer block sums, scaled and summed in f32 (docs/spec/MODEL_LAYER.md, section 6). */
static float dot_q8_0(int64_t n, const uint8_t *w, const uint8_t *a) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < n / 32; i++, w += 34, a += 34) {
    const int8_t *q = (const int8_t *)(w + 2), *p = (const int8_t *)(a + 2);
    int sumi = 0;
    for (int j = 0; j < 32; j++) sumi += (int)q[j] * (int)p[j];
    sumf += (float)sumi * (h2f(rd16(w)) * h2f(rd16(a)));
  }
  return sumf;
}

/* d * sum(sc * sum(q * qa)) - dmin * sum(m * sum(qa)) per block (QUANT_FORMATS.md:396-399). */
static float dot_q4_K(int64_t n, const uint8_t *w, const uint8_t *a) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < n / QK_K; i++, w += 144, a += 292) {
    const uint8_t *scales = w + 4, *qs = w + 16;
    const int8_t *p = (const int8_t *)(a + 4);
    int16_t bs[16];
    memcpy(bs, a + 260, 32);
    int isum = 0, msum = 0;
    for (int c = 0; c < 4; c++) {
      uint8_t sc1, m1, sc2, m2;
      q4k_scale_min(2 * c, scales, &sc1, &m1);
      q4k_scale_min(2 * c + 1, scales, &sc2, &m2);
      int s1 = 0, s2 = 0;
      for (int l = 0; l < 32; l++) {
        s1 += (int)(qs[32 * c + l] & 0xF) * (int)p[64 * c + l];
        s2 += (int)(qs[32 * c + l] >> 4) * (int)p[64 * c + 32 + l];
      }
      isum += sc1 * s1 + sc2 * s2;
      msum += m1 * (bs[4 * c] + bs[4 * c + 1]) + m2 * (bs[4 * c + 2] + bs[4 * c + 3]);
    }
    const float da = rdf(a);
    sumf += (h2f(rd16(w)) * da) * (float)isum - (h2f(rd16(w + 2)) * da) * (float)msum;
  }
  return sumf;
}

/* d * sum(scale16 * sum((q - 32) * qa)) per block (QUANT_FORMATS.md:443-445). */
static float dot_q6_K(int64_t n, const uint8_t *w, const uint8_t *a) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < n / QK_K; i++, w += 210, a += 292) {
    const uint8_t *ql = w, *qh = w + 128;
    const int8_t *sc = (const int8_t *)(w + 192), *p = (const int8_t *)(a + 4);
    int isum = 0;
    for (int h = 0; h < 2; h++) {
      int s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int l = 0; l < 32; l++) {
        const uint8_t hb = qh[32 * h + l];
        const int q1 = (int)((ql[64 * h + l] & 0xF) | (((hb >> 0) & 3) << 4)) - 32;
        const int q2 = (int)((ql[64 * h + 32 + l] & 0xF) | (((hb >> 2) & 3) << 4)) - 32;
        const int q3 = (int)((ql[64 * h + l] >> 4) | (((hb >> 4) & 3) << 4)) - 32;
        const int q4 = (int)((ql[64 * h + 32 + l] >> 4) | (((hb >> 6) & 3) << 4)) - 32;
        const int is = l / 16;
        s[is] += q1 * p[128 * h + l];
        s[is + 2] += q2 * p[128 * h + 32 + l];
        s[is + 4] += q3 * p[128 * h + 64 + l];
        s[is + 6] += q4 * p[128 * h + 96 + l];
      }
      for (int j = 0; j < 8; j++) isum += sc[8 * h + j] * s[j];
    }
    sumf += (h2f(rd16(w + 208)) * rdf(a)) * (float)isum;
  }
  return sumf;
}

/* core/cpu/multirow.cpp:180-245 in scalar form: eight f32 lanes, lane L taking values 4L .. 4L+3 of every sub-block
 * of 32; per block lane += (d_w * d_a) * (its integer sum), fused; the lanes then added as the AVX2 horizontal sum
 * adds them: (l0+l4 + l2+l6) + (l1+l5 + l3+l7). */
static float dot_iq3_s(int64_t n, const uint8_t *w, const uint8_t *a) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t i = 0; i < n / QK_K; i++, w += 110, a += 292) {
    const uint8_t *qs = w + 2, *qh = w + 66, *signs = w + 74, *scales = w + 106;
    const int8_t *p = (const int8_t *)(a + 4);
    int32_t lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sb = 0; sb < 8; sb++) {
      const int sc = 2 * ((scales[sb / 2] >> (4 * (sb % 2))) & 0xF) + 1;
      for (int k = 0; k < 8; k++) {
        const uint32_t g = kIq3sGrid[qs[8 * sb + k] | (((uint32_t)(qh[sb] >> k) & 1u) << 8)];
        const uint8_t sg = signs[4 * sb + k / 2] >> (4 * (k % 2));
        int s = 0;
        for (int v = 0; v < 4; v++) {
          const int q = p[32 * sb + 4 * k + v];
          s += (int)((g >> (8 * v)) & 0xFF) * (((sg >> v) & 1) ? -q : q);
        }
        lane[k] += sc * s;
      }
    }
    const float d = h2f(rd16(w)) * rdf(a);
    for (int L = 0; L < 8; L++) acc[L] = fmaf(d, (float)lane[L], acc[L]);
  }
  const float r0 = acc[4] + acc[0], r1 = acc[5] + acc[1], r2 = acc[6] + acc[2], r3 = acc[7] + acc[3];
  return (r0 + r2) + (r1 + r3);
}

/* core/cpu/multirow.cpp:128-177 in scalar form, the same lanes and order as dot_iq3_s: lane L takes values 4L .. 4L+3 of
 * every sub-block of 32 times the sub-block's 2 s + 1; the quarter comes last. */
static float dot_iq3_xxs(int64_t n, const uint8_t *w, const uint8_t *a) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t i = 0; i < n / QK_K; i++, w += 98, a += 292) {
    const uint8_t *qs = w + 2, *gas = w + 66;
    const int8_t *p = (const int8_t *)(a + 4);
    int32_t lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sb = 0; sb < 8; sb++) {
      uint32_t w32;
      memcpy(&w32, gas + 4 * sb, 4);
      const int sc = 2 * (int)(w32 >> 28) + 1;
      for (int k = 0; k < 8; k++) {
        const uint32_t g = kIq3xxsGrid[qs[8 * sb + k]];
        const uint8_t sg = ksigns((w32 >> (7 * (k / 2))) & 127) >> (4 * (k % 2));
        int s = 0;
        for (int v = 0; v < 4; v++) {
          const int q = p[32 * sb + 4 * k + v];
          s += (int)((g >> (8 * v)) & 0xFF) * (((sg >> v) & 1) ? -q : q);
        }
        lane[k] += sc * s;
      }
    }
    const float d = h2f(rd16(w)) * rdf(a);
    for (int L = 0; L < 8; L++) acc[L] = fmaf(d, (float)lane[L], acc[L]);
  }
  const float r0 = acc[4] + acc[0], r1 = acc[5] + acc[1], r2 = acc[6] + acc[2], r3 = acc[7] + acc[3];
  return 0.25f * ((r0 + r2) + (r1 + r3));
}

/* core/cpu/multirow.cpp:65-125 in scalar form: lane L takes values 4L .. 4L+3 of every sub-block times 2 s + 1 of the
 * half (values 0-15 or 16-31) they are in; the eighth comes last. */
static float dot_iq2_s(int64_t n, const uint8_t *w, const uint8_t *a) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t i = 0; i < n / QK_K; i++, w += 82, a += 292) {
    const uint8_t *qs = w + 2, *sg = w + 34, *qh = w + 66, *scl = w + 74;
    const int8_t *p = (const int8_t *)(a + 4);
    int32_t lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sb = 0; sb < 8; sb++) {
      for (int k = 0; k < 8; k++) { /* values 4k .. 4k+3: half k % 2 of group k / 2 */
        const int g = k / 2;
        const int sc = 2 * (int)((scl[sb] >> (4 * (g / 2))) & 0xF) + 1;
        const uint32_t idx = qs[4 * sb + g] | ((((uint32_t)qh[sb] >> (2 * g)) & 3u) << 8);
        const uint32_t word = kIq2sGrid[2 * idx + k % 2];
        const uint8_t bits = sg[4 * sb + g] >> (4 * (k % 2));
        int s = 0;
        for (int v = 0; v < 4; v++) {
          const int q = p[32 * sb + 4 * k + v];
          s += (int)((word >> (8 * v)) & 0xFF) * (((bits >> v) & 1) ? -q : q);
        }
        lane[k] += sc * s;
      }
    }
    const float d = h2f(rd16(w)) * rdf(a);
    for (int L = 0; L < 8; L++) acc[L] = fmaf(d, (float)lane[L], acc[L]);
  }
  const float r0 = acc[4] + acc[0], r1 = acc[5] + acc[1], r2 = acc[6] + acc[2], r3 = acc[7] + acc[3];
  return 0.125f * ((r0 + r2) + (r1 + r3));
}

/* Q2_0 against q8_0: a block of 64 meets two activation blocks of 32; each half's integer sum of (q - 1) * code times
 * d_w * d_a of its half, as the single-token GPU kernel states it (QUANT_FORMATS.md:265-270). The type is the
 * reference's fork's; neither gguf-py nor the reference's own CPU kernels (core/cpu/multirow.cpp) have it, so the order
 * in which ggml's CPU dot adds the halves is not pinned here. */
static float dot_q2_0(int64_t n, const uint8_t *w, const uint8_t *a) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < n / 64; i++, w += 18, a += 68) {
    const float d = h2f(rd16(w));
    for (int h = 0; h < 2; h++) {
      const int8_t *p = (const int8_t *)(a + 34 * h + 2);
      int sumi = 0;
      for (int j = 0; j < 32; j++) sumi += ((int)((w[2 + 8 * h + j / 4] >> (2 * (j % 4))) & 3) - 1) * p[j];
      sumf += (float)sumi * (d * h2f(rd16(a + 34 * h)));
    }
  }
  return sumf;
}

/* IQ4_NL against q8_0: per block the integer sum of table values times codes, times d_w * d_a (QUANT_FORMATS.md:246-247). */
static float dot_iq4_nl(int64_t n, const uint8_t *w, const uint8_t *a) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < n / 32; i++, w += 18, a += 34) {
    const int8_t *p = (const int8_t *)(a + 2);
    int sumi = 0;
    for (int j = 0; j < 16; j++) sumi += (int)kIq4nlValues[w[2 + j] & 0xF] * p[j] + (int)kIq4nlValues[w[2 + j] >> 4] * p[16 + j];
    sumf += (float)sumi * (h2f(rd16(w)) * h2f(rd16(a)));
  }
  return sumf;
}

/* IQ4_XS against q8_K: per block sum over sub-blocks of (ls - 32) * integer sum, times d_w * d_a (QUANT_FORMATS.md:228-232). */
static float dot_iq4_xs(int64_t n, const uint8_t *w, const uint8_t *a) {
  float sumf = 0.0f;
  for (int64_t i = 0; i < n / QK_K; i++, w += 136, a += 292) {
    const uint32_t sh = rd16(w + 2);
    const uint8_t *sl = w + 4, *qs = w + 8;
    const int8_t *p = (const int8_t *)(a + 4);
    int isum = 0;
    for (int ib = 0; ib < 8; ib++) {
      const int ls = (int)(((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
      int s = 0;
      for (int j = 0; j < 16; j++)
        s += (int)kIq4nlValues[qs[16 * ib + j] & 0xF] * p[32 * ib + j] + (int)kIq4nlValues[qs[16 * ib + j] >> 4] * p[32 * ib + 16 + j];
      isum += ls * s;
    }
    sumf += (h2f(rd16(w)) * rdf(a)) * (float)isum;
  }
  return sumf;
}

float orc_vec_dot(uint32_t t, int64_t n, const void *w, const void *a) {
  switch (t) {
    case ORC_Q8_0: return dot_q8_0(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_Q4_K: return dot_q4_K(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_Q6_K: return dot_q6_K(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_IQ3_S: return dot_iq3_s(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_IQ4_NL: return dot_iq4_nl(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_IQ4_XS: return dot_iq4_xs(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_IQ3_XXS: return dot_iq3_xxs(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_IQ2_S: return dot_iq2_s(n, (const uint8_t *)w, (const uint8_t *)a);
    case ORC_Q2_0: return dot_q2_0(n, (const uint8_t *)w, (const uint8_t *)a);
    default: return NAN;
  }
}

/* ------------------------------------------------------------------------------------------------------------
 * Router. */
void orc_router_logits(const float *x, uint32_t T, uint32_t E, const float *W, const float *wsg, const float *bias,
                       uint32_t NE, float *rl) {
  const uint32_t N = NE + 1, piece = E / ORC_PIECES;
  float *Wt = (float *)malloc((size_t)E * N * sizeof(float)); /* Wt[k][e], so a row of experts is contiguous */
  for (uint32_t e = 0; e < NE; e++)
    for (uint32_t k = 0; k < E; k++) Wt[(size_t)k * N + e] = W[(size_t)e * E + k];
  for (uint32_t k = 0; k < E; k++) Wt[(size_t)k * N + NE] = wsg ? wsg[k] : 0.0f;
#pragma omp parallel
  {
    float *p = (float *)malloc(N * sizeof(float));
#pragma omp for schedule(static)
    for (uint32_t t = 0; t < T; t++) {
      const float *xt = x + (size_t)t * E;
      float *out = rl + (size_t)t * N;
      for (uint32_t s = 0; s < ORC_PIECES; s++) {
        for (uint32_t e = 0; e < N; e++) p[e] = 0.0f;
        for (uint32_t k = s * piece; k < (s + 1) * piece; k++) {
          const float xk = xt[k];
          const float *wr = Wt + (size_t)k * N;
          for (uint32_t e = 0; e < N; e++) p[e] = fmaf(xk, wr[e], p[e]);
        }
        if (s == 0)
          for (uint32_t e = 0; e < N; e++) out[e] = p[e];
        else
          for (uint32_t e = 0; e < N; e++) out[e] = out[e] + p[e];
      }
      if (bias)
        for (uint32_t e = 0; e < NE; e++) out[e] = out[e] + bias[e];
    }
    free(p);
  }
  free(Wt);
}

/* kernels/include/topk.h:12-15 */
static inline uint32_t topk_key(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

void orc_router_topk(const float *rl, uint32_t T, uint32_t NE, uint32_t K, int32_t *ids, float *w, float *gs) {
#pragma omp parallel for schedule(static)
  for (uint32_t t = 0; t < T; t++) {
    const float *v = rl + (size_t)t * (NE + 1);
    /* layer.cl:765-777: the maximum, and the sum of exp(v - max) in f32. */
    float mx = -INFINITY;
    for (uint32_t e = 0; e < NE; e++) mx = fmaxf(mx, v[e]);
    float sum = 0.0f;
    for (uint32_t e = 0; e < NE; e++) sum += expf(v[e] - mx);
    /* route.h:33-38: the K largest keys, largest first, ties to the lower expert; -0 as +0 (prompt.cl:669). */
    uint32_t taken[16];
    float p[16], tot = 0.0f;
    for (uint32_t k = 0; k < K; k++) {
      uint32_t best = 0, bi = NE;
      for (uint32_t e = 0; e < NE; e++) {
        int used = 0;
        for (uint32_t j = 0; j < k; j++) used |= taken[j] == e;
        if (used) continue;
        const uint32_t key = topk_key(v[e] + 0.0f);
        if (bi == NE || key > best) best = key, bi = e;
      }
      taken[k] = bi;
      p[k] = expf(v[bi] - mx) / sum;
    }
    /* layer.cl:784-787 */
    for (uint32_t k = 0; k < K; k++) tot += p[k];
    for (uint32_t k = 0; k < K; k++) {
      ids[(size_t)t * K + k] = (int32_t)taken[k];
      w[(size_t)t * K + k] = p[k] / fmaxf(tot, 6.1035e-5f);
    }
    if (gs) gs[t] = 1.0f / (1.0f + expf(-v[NE]));
  }
}

/* prompt.cl:682-738, with the order inside an expert's run fixed: ascending assignment. */
uint32_t orc_pack(const int32_t *ids, uint32_t A, uint32_t NE, uint32_t first_expert, uint32_t *cnt, uint32_t *base,
                  uint32_t *inv, orc_tile *tiles) {
  uint32_t *cursor = (uint32_t *)calloc(NE, sizeof(uint32_t));
  for (uint32_t e = 0; e < NE; e++) cnt[e] = 0;
  for (uint32_t a = 0; a < A; a++) cnt[ids[a]]++;
  uint32_t run = 0, nt = 0;
  for (uint32_t e = 0; e < NE; e++) {
    base[e] = run;
    if (tiles)
      for (uint32_t i = 0; i * 64 < cnt[e]; i++) {
        const uint32_t left = cnt[e] - i * 64;
        tiles[nt++] = (orc_tile){e, e - first_expert, run + i * 64, left < 64 ? left : 64};
      }
    run += cnt[e];
  }
  for (uint32_t a = 0; a < A; a++) inv[a] = base[ids[a]] + cursor[ids[a]]++;
  free(cursor);
  return nt;
}

/* ------------------------------------------------------------------------------------------------------------
 * Experts. core/cpu/experts.cpp:21-27 */
static inline float swiglu_one(float g, float u, float limit) {
  if (limit > 0.0f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return g / (1.0f + expf(-g)) * u;
}

/* core/cpu/experts.cpp:152-284. Tasks of 32 rows (kRowsH, kRowsDown); an expert's weights are read once for all its
 * jobs; a token's jobs are summed in the order given. */
void orc_compute_many(const orc_shape *s, const orc_job *jobs, uint32_t n, uint32_t ntok, const float *x,
                      uint64_t x_stride, float *y, uint64_t y_stride, int threads) {
  const uint32_t E = s->n_embd, F = s->n_ff;
  if (threads <= 0) threads = orc_threads();
  if (n == 0) {
    for (uint32_t t = 0; t < ntok; t++) memset(y + t * y_stride, 0, E * sizeof(float));
    return;
  }
  const uint32_t gat = orc_vec_dot_type(s->gate_type), dat = orc_vec_dot_type(s->down_type);
  const uint64_t grow = orc_row_bytes(s->gate_type, E), drow = orc_row_bytes(s->down_type, F);
  const uint64_t xqb = orc_row_bytes(gat, E), hqb = orc_row_bytes(dat, F);
  uint8_t *xq = (uint8_t *)malloc((size_t)ntok * xqb);
  uint8_t *hq = (uint8_t *)malloc((size_t)n * hqb);
  float *hf = (float *)malloc((size_t)n * F * sizeof(float));
#pragma omp parallel for schedule(static) num_threads(threads)
  for (uint32_t t = 0; t < ntok; t++) orc_quantize_row(gat, x + t * x_stride, xq + (size_t)t * xqb, E);

  /* The distinct experts, each with its jobs in order (experts.cpp:169-178). An open-addressed table on the gate
   * pointer keeps this linear in the jobs. */
  uint32_t cap = 1;
  while (cap < 2 * n) cap <<= 1;
  int32_t *table = (int32_t *)malloc(cap * sizeof(int32_t));
  for (uint32_t i = 0; i < cap; i++) table[i] = -1;
  uint32_t *dof = (uint32_t *)malloc(n * sizeof(uint32_t)); /* job -> distinct expert */
  uint32_t *dfirst = (uint32_t *)malloc(n * sizeof(uint32_t)), nd = 0;
  for (uint32_t j = 0; j < n; j++) {
    uint32_t hpos = (uint32_t)(((uintptr_t)jobs[j].gate >> 4) * 2654435761u) & (cap - 1);
    while (table[hpos] >= 0 && jobs[dfirst[table[hpos]]].gate != jobs[j].gate) hpos = (hpos + 1) & (cap - 1);
    if (table[hpos] < 0) table[hpos] = (int32_t)nd, dfirst[nd++] = j;
    dof[j] = (uint32_t)table[hpos];
  }
  uint32_t *dstart = (uint32_t *)calloc(nd + 1, sizeof(uint32_t)), *djobs = (uint32_t *)malloc(n * sizeof(uint32_t));
  for (uint32_t j = 0; j < n; j++) dstart[dof[j] + 1]++;
  for (uint32_t d = 0; d < nd; d++) dstart[d + 1] += dstart[d];
  {
    uint32_t *cur = (uint32_t *)malloc(nd * sizeof(uint32_t));
    memcpy(cur, dstart, nd * sizeof(uint32_t));
    for (uint32_t j = 0; j < n; j++) djobs[cur[dof[j]]++] = j;
    free(cur);
  }

  /* Gate and up: one task per (expert, 32 rows), for all its jobs, and their h (experts.cpp:215-228). */
  const uint32_t ft = (F + 31) / 32;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
  for (uint64_t task = 0; task < (uint64_t)nd * ft; task++) {
    const uint32_t d = (uint32_t)(task / ft), r0 = (uint32_t)(task % ft) * 32, r1 = r0 + 32 < F ? r0 + 32 : F;
    const orc_job *lead = &jobs[dfirst[d]];
    for (uint32_t r = r0; r < r1; r++)
      for (uint32_t i = dstart[d]; i < dstart[d + 1]; i++) {
        const uint32_t j = djobs[i];
        const uint8_t *xa = xq + (size_t)jobs[j].tok * xqb;
        const float g = orc_vec_dot(s->gate_type, E, lead->gate + r * grow, xa);
        const float u = orc_vec_dot(s->gate_type, E, lead->up + r * grow, xa);
        hf[(size_t)j * F + r] = swiglu_one(g, u, s->swiglu_limit);
      }
  }
  /* h in the down type's dot format: blocks never straddle rows of h, so quantising a job's whole row gives the bits
   * the reference's blockwise quantising does (experts.cpp:185-188). */
#pragma omp parallel for schedule(static) num_threads(threads)
  for (uint32_t j = 0; j < n; j++) orc_quantize_row(dat, hf + (size_t)j * F, hq + (size_t)j * hqb, F);

  /* Down: one task per 32 rows of every expert; y summed over the jobs in order (experts.cpp:241-263). */
  const uint32_t et = (E + 31) / 32;
#pragma omp parallel num_threads(threads)
  {
    float *out = (float *)malloc((size_t)n * 32 * sizeof(float));
#pragma omp for schedule(dynamic, 1)
    for (uint32_t task = 0; task < et; task++) {
      const uint32_t r0 = task * 32, r1 = r0 + 32 < E ? r0 + 32 : E;
      for (uint32_t d = 0; d < nd; d++) {
        const orc_job *lead = &jobs[dfirst[d]];
        for (uint32_t r = r0; r < r1; r++)
          for (uint32_t i = dstart[d]; i < dstart[d + 1]; i++) {
            const uint32_t j = djobs[i];
            out[(size_t)j * 32 + (r - r0)] = orc_vec_dot(s->down_type, F, lead->down + r * drow, hq + (size_t)j * hqb);
          }
      }
      for (uint32_t t = 0; t < ntok; t++)
        for (uint32_t r = r0; r < r1; r++) y[t * y_stride + r] = 0.0f;
      for (uint32_t j = 0; j < n; j++) {
        float *yt = y + jobs[j].tok * y_stride;
        for (uint32_t r = r0; r < r1; r++) yt[r] += jobs[j].w * out[(size_t)j * 32 + (r - r0)];
      }
    }
    free(out);
  }
  free(xq), free(hq), free(hf), free(table), free(dof), free(dfirst), free(dstart), free(djobs);
}

/* The block: router, pack, routed experts summed in rank order, shared expert gated by sigmoid of the router's last
 * logit (layer.cl:869-883; docs/spec/MODEL_LAYER.md 4.2-4.4). */
void orc_moe_forward(const orc_layer *L, const float *x, uint32_t T, float *out, int32_t *ids_out, float *w_out,
                     uint32_t *inv_out, orc_tile *tiles_out, uint32_t *ntiles_out, int threads) {
  const uint32_t E = L->n_embd, F = L->n_ff, NE = L->n_experts, K = L->n_used, A = T * K;
  float *rl = (float *)malloc((size_t)T * (NE + 1) * sizeof(float));
  int32_t *ids = (int32_t *)malloc((size_t)A * sizeof(int32_t));
  float *w = (float *)malloc((size_t)A * sizeof(float)), *gs = (float *)malloc(T * sizeof(float));
  orc_router_logits(x, T, E, L->router, L->shexp_gate_inp, L->router_bias, NE, rl);
  orc_router_topk(rl, T, NE, K, ids, w, gs);
  if (ids_out) memcpy(ids_out, ids, (size_t)A * sizeof(int32_t));
  if (w_out) memcpy(w_out, w, (size_t)A * sizeof(float));
  if (inv_out) {
    uint32_t *cnt = (uint32_t *)malloc(NE * sizeof(uint32_t)), *base = (uint32_t *)malloc(NE * sizeof(uint32_t));
    const uint32_t nt = orc_pack(ids, A, NE, 0, cnt, base, inv_out, tiles_out);
    if (ntiles_out) *ntiles_out = nt;
    free(cnt), free(base);
  }
  const uint64_t gsl = (uint64_t)F * orc_row_bytes(L->gate_type, E), dsl = (uint64_t)E * orc_row_bytes(L->down_type, F);
  orc_job *jobs = (orc_job *)malloc(((size_t)A > T ? A : T) * sizeof(orc_job));
  for (uint32_t a = 0; a < A; a++) {
    const uint64_t e = (uint64_t)ids[a];
    jobs[a] = (orc_job){L->gate_exps + e * gsl, L->up_exps + e * gsl, L->down_exps + e * dsl, a / K, w[a]};
  }
  const orc_shape rs = {L->gate_type, L->down_type, E, F, L->swiglu_limit};
  orc_compute_many(&rs, jobs, A, T, x, E, out, E, threads);
  if (L->gate_shexp) {
    float *sh = (float *)malloc((size_t)T * E * sizeof(float));
    for (uint32_t t = 0; t < T; t++) jobs[t] = (orc_job){L->gate_shexp, L->up_shexp, L->down_shexp, t, 1.0f};
    const orc_shape ss = {L->shexp_gate_type, L->shexp_down_type, E, F, L->swiglu_limit};
    orc_compute_many(&ss, jobs, T, T, x, E, sh, E, threads);
    for (uint32_t t = 0; t < T; t++)
      for (uint32_t i = 0; i < E; i++) out[(size_t)t * E + i] += gs[t] * sh[(size_t)t * E + i];
    free(sh);
  }
  free(rl), free(ids), free(w), free(gs), free(jobs);
}
