/* CPU oracle for the int8-activation x GGUF block-quantised weight matrix product (Q8_0, Q4_K).
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of the reference engine
 * (rizagp/arcinferzero) for the one path the CUDA library accelerates.  Only the tests, the smoke check and the
 * benchmark's cpu-baseline leg load it; the shipped library never links or calls it.
 *
 * Parity is pinned: tests/golden/ holds vectors produced by the reference's own src/quants.h (compiled in place by
 * oracle/Makefile into oracle/_ref/libizb_ref.so); tests/test_oracle_golden.py checks every function here against
 * them, and against the live _ref library when it is present.
 *
 * Each function cites the reference file:line it follows (paths inside the reference project).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <omp.h>

/* Worker threads of the loops below (a launcher may have exported OMP_NUM_THREADS=1: the benchmark's CPU baseline sets
 * the count it reports). */
void orc_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}
int orc_max_threads(void) { return omp_get_max_threads(); }

#define ORC_Q8_0 8
#define ORC_Q4_K 12
#define ORC_Q4_0 2   /* further ggml types: decoded into the reference's generic view below */
#define ORC_Q5_K 13
#define ORC_Q6_K 14
#define ORC_IQ4_XS 23

/* ---------------------------------------------------------------- fp16 <-> f32 (src/quants.h:17-52) */
float orc_fp16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, f;
  if (e == 0) {
    if (m == 0) f = sign;
    else {
      e = 127 - 15 + 1;
      while (!(m & 0x400u)) { m <<= 1; --e; }
      f = sign | (e << 23) | ((m & 0x3FFu) << 13);
    }
  } else if (e == 31) f = sign | 0x7F800000u | (m << 13);
  else f = sign | ((e + 127 - 15) << 23) | (m << 13);
  float r;
  memcpy(&r, &f, 4);
  return r;
}

uint16_t orc_f32_to_fp16(float x) {
  uint32_t f;
  memcpy(&f, &x, 4);
  uint32_t sign = (f >> 16) & 0x8000u;
  int32_t e = (int32_t)((f >> 23) & 0xFF) - 127 + 15;
  uint32_t m = f & 0x7FFFFFu;
  if (((f >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0));
  if (e >= 31) return (uint16_t)(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    m |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t h = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = sign | ((uint32_t)e << 10) | (m >> 13), rem = m & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return (uint16_t)h;
}

/* ---------------------------------------------------------------- block formats */
/* bytes of 256 weights in GGUF form (src/gguf.h:48-70) */
int orc_sb_bytes(int type) {
  switch (type) {
    case ORC_Q4_K: return 144;
    case ORC_Q8_0: return 8 * 34;
    case ORC_Q4_0: return 8 * 18;
    case ORC_Q5_K: return 176;
    case ORC_Q6_K: return 210;
    case ORC_IQ4_XS: return 136;
    default: return -1;
  }
}
static int orc_generic(int type) { return type == ORC_Q5_K || type == ORC_Q6_K || type == ORC_IQ4_XS; }

/* 6-bit scale / min j of a Q4_K superblock's 12 packed bytes (src/quants.h:61-69) */
void orc_q4k_scale_min(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = s[j] & 63;
    *mn = s[j + 4] & 63;
  } else {
    *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
    *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
  }
}

/* Q4_K superblock (144 B) -> d, dmin, 8 scales, 8 mins, 256 quants 0..15 (src/quants.h:91-114) */
void orc_q4k_decode_sb(const uint8_t* p, float* d, float* dmin, uint8_t* sc, uint8_t* mn, uint8_t* q) {
  uint16_t dh, mh;
  memcpy(&dh, p, 2);
  memcpy(&mh, p + 2, 2);
  *d = orc_fp16_to_f32(dh);
  *dmin = orc_fp16_to_f32(mh);
  for (int b = 0; b < 8; ++b) orc_q4k_scale_min(b, p + 4, &sc[b], &mn[b]);
  const uint8_t* qs = p + 16;
  for (int j = 0; j < 4; ++j)
    for (int l = 0; l < 32; ++l) {
      q[64 * j + l] = qs[32 * j + l] & 0xF;
      q[64 * j + 32 + l] = qs[32 * j + l] >> 4;
    }
}

/* eight Q8_0 blocks (8 x 34 B) -> 8 scales, 256 signed quants (src/quants.h:149-158) */
void orc_q8_0_decode_sb(const uint8_t* p, float* d8, int8_t* q) {
  for (int b = 0; b < 8; ++b) {
    uint16_t dh;
    memcpy(&dh, p + 34 * b, 2);
    d8[b] = orc_fp16_to_f32(dh);
    memcpy(q + 32 * b, p + 34 * b + 2, 32);
  }
}

/* inverse of orc_q4k_decode_sb: the generator's packer (inverse of src/quants.h:61-69,103-112) */
void orc_q4k_pack_sb(uint16_t d, uint16_t dmin, const uint8_t* sc, const uint8_t* mn, const uint8_t* q, uint8_t* out) {
  memcpy(out, &d, 2);
  memcpy(out + 2, &dmin, 2);
  uint8_t* s = out + 4;
  memset(s, 0, 12);
  for (int j = 0; j < 4; ++j) {
    s[j] = sc[j] & 63;
    s[j + 4] = mn[j] & 63;
  }
  for (int j = 4; j < 8; ++j) {
    s[j + 4] = (uint8_t)((sc[j] & 15) | ((mn[j] & 15) << 4));
    s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
    s[j] |= (uint8_t)((mn[j] >> 4) << 6);
  }
  for (int j = 0; j < 4; ++j)
    for (int l = 0; l < 32; ++l) out[16 + 32 * j + l] = (uint8_t)((q[64 * j + l] & 15) | ((q[64 * j + 32 + l] & 15) << 4));
}

/* ---------------------------------------------------------------- further weight types
 * The reference gives every K-quant and codebook type one generic view of a superblock (DecodedSB, src/quants.h:72-87):
 *   w[e] = wd * wsc[e/16] * (q[e] - qoff) - wdmin * wmn[e/16]
 * with an integer scale and min per 16 elements.  orc_decode_generic_sb fills it for Q5_K (src/quants.h:91-114), Q6_K
 * (:115-135) and IQ4_XS (:297-312), with qoff already subtracted from q.  Q4_0 (:136-148) is a Q8_0 with 4-bit quants
 * q - 8: orc_q4_0_to_q8_0 rewrites its blocks as Q8_0 blocks, exactly. */
static const int8_t orc_iq4nl_values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

int orc_decode_generic_sb(int type, const uint8_t* p, float* wd, float* wdmin, int8_t* wsc, uint8_t* wmn, int* has_min, int16_t* q) {
  uint16_t h;
  memset(wmn, 0, 16);
  *wdmin = 0.0f;
  *has_min = 0;
  if (type == ORC_Q5_K) { /* fp16 d, dmin | 12 B 6-bit scales / mins | 32 B fifth bits | 128 B nibbles */
    uint8_t sc[8], mn[8];
    memcpy(&h, p, 2);
    *wd = orc_fp16_to_f32(h);
    memcpy(&h, p + 2, 2);
    *wdmin = orc_fp16_to_f32(h);
    *has_min = 1;
    for (int b = 0; b < 8; ++b) orc_q4k_scale_min(b, p + 4, &sc[b], &mn[b]);
    for (int i = 0; i < 16; ++i) { wsc[i] = (int8_t)sc[i / 2]; wmn[i] = mn[i / 2]; }
    const uint8_t* qh = p + 16;
    const uint8_t* qs = p + 48;
    for (int j = 0; j < 4; ++j)
      for (int l = 0; l < 32; ++l) {
        q[64 * j + l] = (int16_t)((qs[32 * j + l] & 0xF) | (((qh[l] >> (2 * j)) & 1) << 4));
        q[64 * j + 32 + l] = (int16_t)((qs[32 * j + l] >> 4) | (((qh[l] >> (2 * j + 1)) & 1) << 4));
      }
    return 0;
  }
  if (type == ORC_Q6_K) { /* 128 B low nibbles | 64 B upper two bits | 16 int8 scales | fp16 d; value q - 32 */
    const uint8_t* ql = p;
    const uint8_t* qh = p + 128;
    memcpy(&h, p + 208, 2);
    *wd = orc_fp16_to_f32(h);
    for (int i = 0; i < 16; ++i) wsc[i] = (int8_t)p[192 + i];
    for (int n = 0; n < 2; ++n)
      for (int l = 0; l < 32; ++l) {
        const uint8_t* L = ql + 64 * n;
        const uint8_t* H = qh + 32 * n;
        q[128 * n + l] = (int16_t)(((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32);
        q[128 * n + l + 32] = (int16_t)(((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32);
        q[128 * n + l + 64] = (int16_t)(((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32);
        q[128 * n + l + 96] = (int16_t)(((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32);
      }
    return 0;
  }
  if (type == ORC_IQ4_XS) { /* fp16 d | u16 upper scale bits | 4 B lower scale nibbles | 128 B codebook indices */
    uint16_t sh;
    memcpy(&h, p, 2);
    memcpy(&sh, p + 2, 2);
    *wd = orc_fp16_to_f32(h);
    const uint8_t* sl = p + 4;
    const uint8_t* qs = p + 8;
    for (int ib = 0; ib < 8; ++ib) {
      const int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
      wsc[2 * ib] = wsc[2 * ib + 1] = (int8_t)(ls - 32);
      for (int j = 0; j < 16; ++j) {
        q[32 * ib + j] = orc_iq4nl_values[qs[16 * ib + j] & 0xF];
        q[32 * ib + 16 + j] = orc_iq4nl_values[qs[16 * ib + j] >> 4];
      }
    }
    return 0;
  }
  return -1;
}

/* Q4_0 rows (18-byte blocks: fp16 d, low nibbles = elements 0..15, high nibbles = 16..31, value q - 8) as Q8_0 rows */
void orc_q4_0_to_q8_0(const uint8_t* src, size_t n_blocks, uint8_t* dst) {
  for (size_t b = 0; b < n_blocks; ++b) {
    const uint8_t* s8 = src + 18 * b;
    uint8_t* d8 = dst + 34 * b;
    d8[0] = s8[0];
    d8[1] = s8[1];
    for (int i = 0; i < 16; ++i) {
      d8[2 + i] = (uint8_t)(int8_t)((s8[2 + i] & 0xF) - 8);
      d8[2 + 16 + i] = (uint8_t)(int8_t)((s8[2 + i] >> 4) - 8);
    }
  }
}

/* one weight row -> f32 (src/quants.h:519-616 dequant_row, :319-326 dequant_value) */
void orc_dequant_row(int type, const uint8_t* row, int K, float* out) {
  for (int s = 0; s < K / 256; ++s) {
    if (orc_generic(type)) { /* src/quants.h:319-324: d * scale * q - dmin * min, left to right */
      float wd, wdmin;
      int8_t wsc[16];
      uint8_t wmn[16];
      int has_min;
      int16_t q[256];
      orc_decode_generic_sb(type, row + (size_t)s * orc_sb_bytes(type), &wd, &wdmin, wsc, wmn, &has_min, q);
      for (int e = 0; e < 256; ++e)
        out[s * 256 + e] = wd * wsc[e / 16] * q[e] - (has_min ? wdmin * wmn[e / 16] : 0.0f);
    } else if (type == ORC_Q4_0) {
      for (int b = 0; b < 8; ++b) {
        const uint8_t* blk = row + (size_t)s * 144 + 18 * b;
        uint16_t dh;
        memcpy(&dh, blk, 2);
        const float d = orc_fp16_to_f32(dh);
        for (int i = 0; i < 16; ++i) {
          out[s * 256 + 32 * b + i] = d * (float)((blk[2 + i] & 0xF) - 8);
          out[s * 256 + 32 * b + 16 + i] = d * (float)((blk[2 + i] >> 4) - 8);
        }
      }
    } else if (type == ORC_Q4_K) {
      float d, dmin;
      uint8_t sc[8], mn[8], q[256];
      orc_q4k_decode_sb(row + (size_t)s * 144, &d, &dmin, sc, mn, q);
      for (int e = 0; e < 256; ++e) out[s * 256 + e] = d * sc[e / 32] * q[e] - dmin * mn[e / 32];
    } else {
      float d8[8];
      int8_t q[256];
      orc_q8_0_decode_sb(row + (size_t)s * 272, d8, q);
      for (int e = 0; e < 256; ++e) out[s * 256 + e] = d8[e / 32] * q[e];
    }
  }
}

/* ---------------------------------------------------------------- activation quantiser
 * src/quants.h:626-643 (quantize_act_cpu, act32 = true) == zero/kernels/ops.cl:38-72 (quant_store16).
 * x: [M][ldx] f32.  aq: [Mp][K] int8.  asc: [K/32][Mp] f32.  absum: [K/16][Mp] int16 (may be NULL).
 * Rows M..Mp-1 are padding: zeros with scale 0 (zero/kernels/ops.cl:132-135). */
void orc_quantize_act(const float* x, int M, int K, int ldx, int Mp, int8_t* aq, float* asc, int16_t* absum) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < Mp; ++m) {
    for (int b0 = 0; b0 < K; b0 += 32) {
      int8_t* o = aq + (size_t)m * K + b0;
      if (m >= M) {
        memset(o, 0, 32);
        asc[(size_t)(b0 / 32) * Mp + m] = 0.0f;
      } else {
        const float* v = x + (size_t)m * ldx + b0;
        float amax = 0;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        const float inv = amax > 0 ? 127.0f / amax : 0.0f;
        asc[(size_t)(b0 / 32) * Mp + m] = amax / 127.0f;
        for (int i = 0; i < 32; ++i) o[i] = (int8_t)lrintf(v[i] * inv);
      }
      if (absum)
        for (int h = 0; h < 2; ++h) {
          int sum = 0;
          for (int i = 0; i < 16; ++i) sum += o[16 * h + i];
          absum[(size_t)(b0 / 16 + h) * Mp + m] = (int16_t)sum;
        }
    }
  }
}

/* ---------------------------------------------------------------- fused producers
 * sum of v[i]^2 in the CUDA kernels' order: 256 strided chains of fused multiply-adds, xor butterfly over each group of 32,
 * the eight group sums added in order */
static float ordered_sumsq(const float* v, int K) {
  float part[256];
  for (int t = 0; t < 256; ++t) {
    float ss = 0.0f;
    for (int i = t; i < K; i += 256) ss = fmaf(v[i], v[i], ss);
    part[t] = ss;
  }
  float total = 0.0f;
  for (int g = 0; g < 8; ++g) {
    float a[32], n[32];
    memcpy(a, part + 32 * g, sizeof a);
    for (int o = 16; o > 0; o >>= 1) {
      for (int l = 0; l < 32; ++l) n[l] = a[l] + a[l ^ o];
      memcpy(a, n, sizeof a);
    }
    total = g == 0 ? a[0] : total + a[0];
  }
  return total;
}

/* the same with the chains of the rmsnorm_quant kernel: chain t takes the groups of 8 consecutive values t, t + 256, ... */
static float ordered_sumsq8(const float* v, int K) {
  float part[256];
  for (int t = 0; t < 256; ++t) {
    float ss = 0.0f;
    for (int g = t; g < K / 8; g += 256)
      for (int e = 0; e < 8; ++e) ss = fmaf(v[8 * g + e], v[8 * g + e], ss);
    part[t] = ss;
  }
  float total = 0.0f;
  for (int g = 0; g < 8; ++g) {
    float a[32], n[32];
    memcpy(a, part + 32 * g, sizeof a);
    for (int o = 16; o > 0; o >>= 1) {
      for (int l = 0; l < 32; ++l) n[l] = a[l] + a[l ^ o];
      memcpy(a, n, sizeof a);
    }
    total = g == 0 ? a[0] : total + a[0];
  }
  return total;
}

/* add_norm_quant, zero/kernels/ops_attn_g.cl:617-680: x = (x + (t * r) * w) * s, r = rsqrt(sum(t^2)/K + eps); then the next
 * GEMV input y = w2 ? (x * r2) * w2 : x with r2 from the new x, quantised per 32.  x is updated in place. */
void orc_add_norm_quant(float* x, const float* t, const float* w, float eps, float s, const float* w2, int M, int K, int Mp,
                        int8_t* aq, float* asc, int16_t* absum) {
  float* y = (float*)malloc((size_t)(M > 0 ? M : 1) * K * sizeof(float));
  for (int m = 0; m < M; ++m) {
    float* xr = x + (size_t)m * K;
    const float* tr = t + (size_t)m * K;
    const float r = 1.0f / sqrtf(ordered_sumsq(tr, K) / (float)K + eps);
    for (int i = 0; i < K; ++i) {
      const float a = tr[i] * r;
      const float b = a * w[i];
      const float c = xr[i] + b;
      xr[i] = c * s;
    }
    float r2 = 1.0f;
    if (w2) r2 = 1.0f / sqrtf(ordered_sumsq(xr, K) / (float)K + eps);
    for (int i = 0; i < K; ++i) {
      const float a = xr[i] * r2;
      y[(size_t)m * K + i] = w2 ? a * w2[i] : xr[i];
    }
  }
  orc_quantize_act(y, M, K, K, Mp, aq, asc, absum);
  free(y);
}

/* ---------------------------------------------------------------- RMSNorm + quantise
 * rmsnorm_quant, zero/kernels/ops.cl:104-141: r = rsqrt(sum(x^2) / K + eps); y = x * r * w; then quant_store16.  The
 * kernel leaves the order of the sum to the OpenCL work-group reduction; the order written here is the CUDA kernel's
 * (256 chains of fused multiply-adds over groups of 8 values, xor butterfly over each group of 32 chains, the eight group
 * sums in order), so that both produce the same bits.  hout (may be NULL): y as f32 [M][K]. */
void orc_rmsnorm_quant(const float* x, int M, int K, int ldx, const float* w, float eps, int Mp, float* hout, int8_t* aq,
                       float* asc, int16_t* absum) {
  float* y = (float*)malloc((size_t)(M > 0 ? M : 1) * K * sizeof(float));
  for (int m = 0; m < M; ++m) {
    const float* xr = x + (size_t)m * ldx;
    const float total = ordered_sumsq8(xr, K);
    const float r = 1.0f / sqrtf(total / (float)K + eps);
    for (int i = 0; i < K; ++i) {
      const float xr_r = xr[i] * r;
      y[(size_t)m * K + i] = xr_r * w[i];
    }
  }
  if (hout) memcpy(hout, y, (size_t)M * K * sizeof(float));
  orc_quantize_act(y, M, K, K, Mp, aq, asc, absum);
  free(y);
}

/* ---------------------------------------------------------------- per-block integer dots
 * zero/kernels/decode.cl:992-999, zero/kernels/gemm.cl:413-423: dot[m][n][b] = sum_i aq[m][32b+i] * qw[n][32b+i] (int32),
 * asum[m][b] = sum_i aq[m][32b+i].  These are the values every GPU kernel must reproduce bit for bit. */
static void decode_row_q(int type, const uint8_t* row, int K, int16_t* q, float* dd, float* dm, uint8_t* sc, uint8_t* mn) {
  /* q[K]; Q4_K: dd/dm per superblock, sc/mn per block. Q8_0: dd per block. */
  for (int s = 0; s < K / 256; ++s) {
    if (type == ORC_Q4_K) {
      uint8_t qq[256];
      orc_q4k_decode_sb(row + (size_t)s * 144, &dd[s], &dm[s], sc + 8 * s, mn + 8 * s, qq);
      for (int e = 0; e < 256; ++e) q[s * 256 + e] = qq[e];
    } else {
      int8_t qq[256];
      orc_q8_0_decode_sb(row + (size_t)s * 272, dd + 8 * s, qq);
      for (int e = 0; e < 256; ++e) q[s * 256 + e] = qq[e];
    }
  }
}

static inline int32_t dot32(const int8_t* a, const int16_t* w) {
  int32_t s = 0;
  for (int i = 0; i < 32; ++i) s += (int32_t)a[i] * (int32_t)w[i];
  return s;
}

void orc_block_dots(int type, const uint8_t* w, int N, int K, const int8_t* aq, int M, int32_t* dots, int32_t* asum) {
  const int nb = K / 32;
  const size_t rb = (size_t)(K / 256) * orc_sb_bytes(type);
  if (asum)
    for (int m = 0; m < M; ++m)
      for (int b = 0; b < nb; ++b) {
        int32_t s = 0;
        for (int i = 0; i < 32; ++i) s += aq[(size_t)m * K + 32 * b + i];
        asum[(size_t)m * nb + b] = s;
      }
#pragma omp parallel
  {
    int16_t* q = (int16_t*)malloc((size_t)K * 2);
    float* dd = (float*)malloc((size_t)nb * 4 * 2);
    uint8_t* sm = (uint8_t*)malloc((size_t)nb * 2);
#pragma omp for schedule(dynamic, 8)
    for (int n = 0; n < N; ++n) {
      decode_row_q(type, w + (size_t)n * rb, K, q, dd, dd + nb, sm, sm + nb);
      for (int m = 0; m < M; ++m)
        for (int b = 0; b < nb; ++b) dots[((size_t)m * N + n) * nb + b] = dot32(aq + (size_t)m * K + 32 * b, q + 32 * b);
    }
    free(q);
    free(dd);
    free(sm);
  }
}

/* ---------------------------------------------------------------- f32 combine, two orders of the reference
 * store modes (zero/kernels/gemm.cl:556-567): acc 0: C = v; 1: C += v; 2: C = v * silu(C) (C holds the gate) */
static inline float store_mode(float old, float v, int acc) {
  if (acc == 1) return v + old;
  if (acc == 2) return v * (old / (1.0f + expf(-old)));
  return v;
}

/* GEMV order (zero/kernels/decode.cl:913-1034 and :1581-1694): sixteen lanes, lane l owns the blocks b == l (mod 16)
 * in increasing b (two superblocks per step), the lanes are then summed (sub_group_reduce_add: order unspecified;
 * here lane 0..15).  Q4_K term: sa*(d*(float)(sc*dot) - dmin*(float)(mn*asum)); Q8_0 term: sa*d*(float)dot. */
void orc_matmul_gemv_order(int type, const uint8_t* w, int N, int K, const int8_t* aq, const float* asc, int Mp, int T,
                           float* C, int ldc, int c_off, int acc) {
  const int nb = K / 32;
  const size_t rb = (size_t)(K / 256) * orc_sb_bytes(type);
#pragma omp parallel
  {
    int16_t* q = (int16_t*)malloc((size_t)K * 2);
    float* dd = (float*)malloc((size_t)nb * 4 * 2);
    uint8_t* sm = (uint8_t*)malloc((size_t)nb * 2);
#pragma omp for schedule(dynamic, 8)
    for (int n = 0; n < N; ++n) {
      decode_row_q(type, w + (size_t)n * rb, K, q, dd, dd + nb, sm, sm + nb);
      for (int t = 0; t < T; ++t) {
        float lane[16];
        for (int l = 0; l < 16; ++l) lane[l] = 0.0f;
        for (int b = 0; b < nb; ++b) {
          const int8_t* a = aq + (size_t)t * K + 32 * b;
          const float sa = asc[(size_t)b * Mp + t];
          const int32_t dot = dot32(a, q + 32 * b);
          if (type == ORC_Q4_K) {
            int32_t as = 0;
            for (int i = 0; i < 32; ++i) as += a[i];
            const float d = dd[b / 8], dmin = dd[nb + b / 8];
            lane[b % 16] += sa * (d * (float)((int32_t)sm[b] * dot) - dmin * (float)((int32_t)sm[nb + b] * as));
          } else {
            lane[b % 16] += sa * dd[b] * (float)dot;
          }
        }
        float v = 0.0f;
        for (int l = 0; l < 16; ++l) v += lane[l];
        float* c = C + (size_t)t * ldc + c_off + n;
        *c = acc ? *c + v : v;
      }
    }
    free(q);
    free(dd);
    free(sm);
  }
}

/* GEMM order (zero/kernels/gemm.cl:441-487, -DACT32): superblock s, chunk j of 64 = blocks 2j (lo), 2j+1 (hi):
 *   Q8_0: res = fma(asc_lo*d_lo, (float)dot_lo, fma(asc_hi*d_hi, (float)dot_hi, res))
 *   Q4_K: tq  = fma(asc_lo, (float)(sc_lo*dot_lo), fma(asc_hi, (float)(sc_hi*dot_hi), tq))
 *         tmn = fma(asc_lo, (float)(mn_lo*asum_lo), fma(asc_hi, (float)(mn_hi*asum_hi), tmn))
 *         per superblock: res = fma(d, tq, fma(-dmin, tmn, res))
 * [k0, k1) in superblocks restates the split-K pieces (zero/engine.h:1242-1250); rows M valid of Mp. */
void orc_matmul_gemm_order(int type, const uint8_t* w, int N, int K, const int8_t* aq, const float* asc, int Mp, int M,
                           float* C, int ldc, int c_off, int acc) {
  const int nb = K / 32, nsb = K / 256;
  const size_t rb = (size_t)nsb * orc_sb_bytes(type);
#pragma omp parallel
  {
    int16_t* q = (int16_t*)malloc((size_t)K * 2);
    float* dd = (float*)malloc((size_t)nb * 4 * 2);
    uint8_t* sm = (uint8_t*)malloc((size_t)nb * 2);
#pragma omp for schedule(dynamic, 8)
    for (int n = 0; n < N; ++n) {
      decode_row_q(type, w + (size_t)n * rb, K, q, dd, dd + nb, sm, sm + nb);
      for (int m = 0; m < M; ++m) {
        float res = 0.0f;
        for (int s = 0; s < nsb; ++s) {
          float tq = 0.0f, tmn = 0.0f;
          for (int j = 0; j < 4; ++j) {
            const int bl = 8 * s + 2 * j, bh = bl + 1;
            const int8_t* al = aq + (size_t)m * K + 32 * bl;
            const int8_t* ah = al + 32;
            const float sl = asc[(size_t)bl * Mp + m], sh = asc[(size_t)bh * Mp + m];
            const int32_t dl = dot32(al, q + 32 * bl), dh = dot32(ah, q + 32 * bh);
            if (type == ORC_Q4_K) {
              int32_t sl_sum = 0, sh_sum = 0;
              for (int i = 0; i < 32; ++i) { sl_sum += al[i]; sh_sum += ah[i]; }
              tq = fmaf(sl, (float)((int32_t)sm[bl] * dl), fmaf(sh, (float)((int32_t)sm[bh] * dh), tq));
              tmn = fmaf(sl, (float)((int32_t)sm[nb + bl] * sl_sum), fmaf(sh, (float)((int32_t)sm[nb + bh] * sh_sum), tmn));
            } else {
              res = fmaf(sl * dd[bl], (float)dl, fmaf(sh * dd[bh], (float)dh, res));
            }
          }
          if (type == ORC_Q4_K) res = fmaf(dd[s], tq, fmaf(-dd[nb + s], tmn, res));
        }
        float* c = C + (size_t)m * ldc + c_off + n;
        *c = store_mode(*c, res, acc);
      }
    }
    free(q);
    free(dd);
    free(sm);
  }
}

/* ---------------------------------------------------------------- the same for the generic view (Q5_K, Q6_K, IQ4_XS)
 * Per 32-block with its two 16-element halves (zero/kernels/decode.cl:992-1004): lo / hi = integer dots of the halves,
 * bs0 / bs1 = sums of the activations of the halves,
 *   with mins:    term = sa * (d * (float)(sc0*lo + sc1*hi) - dmin * (float)(mn0*bs0 + mn1*bs1))
 *   without:      term = sa * d * (float)(sc0*lo + sc1*hi)
 * order 0 ("gemv"): sixteen lanes as in orc_matmul_gemv_order.  order 1 ("gemm"): the reference has no exact GEMM for these
 * types (it requantises them, src/quants.h:683-686); the order defined here is the Q4_K one with per-16 scales:
 *   tq = fma(sl, (float)(sc0*lo + sc1*hi), fma(sh, (float)(...), tq)), tmn likewise, res = fma(d, tq, fma(-dmin, tmn, res)). */
typedef struct {
  int16_t* q;      /* [K], offset subtracted */
  float* wd;       /* [K/256] d, then [K/256] dmin */
  int8_t* wsc;     /* [K/16] */
  uint8_t* wmn;    /* [K/16] */
  int has_min;
} orc_grow;

static void grow_alloc(orc_grow* g, int K) {
  g->q = (int16_t*)malloc((size_t)K * 2);
  g->wd = (float*)malloc((size_t)(K / 256) * 8);
  g->wsc = (int8_t*)malloc((size_t)K / 16);
  g->wmn = (uint8_t*)malloc((size_t)K / 16);
}
static void grow_free(orc_grow* g) { free(g->q); free(g->wd); free(g->wsc); free(g->wmn); }
static void grow_decode(orc_grow* g, int type, const uint8_t* row, int K) {
  const int nsb = K / 256;
  for (int s = 0; s < nsb; ++s)
    orc_decode_generic_sb(type, row + (size_t)s * orc_sb_bytes(type), &g->wd[s], &g->wd[nsb + s], g->wsc + 16 * s, g->wmn + 16 * s,
                          &g->has_min, g->q + 256 * s);
}
static inline int32_t dot16(const int8_t* a, const int16_t* w) {
  int32_t s = 0;
  for (int i = 0; i < 16; ++i) s += (int32_t)a[i] * (int32_t)w[i];
  return s;
}
static inline int32_t sum16(const int8_t* a) {
  int32_t s = 0;
  for (int i = 0; i < 16; ++i) s += a[i];
  return s;
}

void orc_block_dots_generic(int type, const uint8_t* w, int N, int K, const int8_t* aq, int M, int32_t* dots) {
  const int nb = K / 32;
  const size_t rb = (size_t)(K / 256) * orc_sb_bytes(type);
#pragma omp parallel
  {
    orc_grow g;
    grow_alloc(&g, K);
#pragma omp for schedule(dynamic, 8)
    for (int n = 0; n < N; ++n) {
      grow_decode(&g, type, w + (size_t)n * rb, K);
      for (int m = 0; m < M; ++m)
        for (int b = 0; b < nb; ++b) dots[((size_t)m * N + n) * nb + b] = dot32(aq + (size_t)m * K + 32 * b, g.q + 32 * b);
    }
    grow_free(&g);
  }
}

void orc_matmul_generic(int type, const uint8_t* w, int N, int K, const int8_t* aq, const float* asc, int Mp, int T, float* C,
                        int ldc, int c_off, int acc, int order) {
  const int nb = K / 32, nsb = K / 256;
  const size_t rb = (size_t)nsb * orc_sb_bytes(type);
#pragma omp parallel
  {
    orc_grow g;
    grow_alloc(&g, K);
#pragma omp for schedule(dynamic, 8)
    for (int n = 0; n < N; ++n) {
      grow_decode(&g, type, w + (size_t)n * rb, K);
      for (int t = 0; t < T; ++t) {
        float v = 0.0f;
        if (order == 0) {
          float lane[16];
          for (int l = 0; l < 16; ++l) lane[l] = 0.0f;
          for (int b = 0; b < nb; ++b) {
            const int8_t* a = aq + (size_t)t * K + 32 * b;
            const float sa = asc[(size_t)b * Mp + t], d = g.wd[b / 8], dmin = g.wd[nsb + b / 8];
            const int32_t x = (int32_t)g.wsc[2 * b] * dot16(a, g.q + 32 * b) + (int32_t)g.wsc[2 * b + 1] * dot16(a + 16, g.q + 32 * b + 16);
            if (g.has_min) {
              const int32_t y = (int32_t)g.wmn[2 * b] * sum16(a) + (int32_t)g.wmn[2 * b + 1] * sum16(a + 16);
              lane[b % 16] += sa * (d * (float)x - dmin * (float)y);
            } else {
              lane[b % 16] += sa * d * (float)x;
            }
          }
          for (int l = 0; l < 16; ++l) v += lane[l];
        } else {
          for (int s = 0; s < nsb; ++s) {
            float tq = 0.0f, tmn = 0.0f;
            for (int j = 0; j < 4; ++j) {
              int32_t x[2], y[2];
              float sc2[2];
              for (int h = 0; h < 2; ++h) {
                const int b = 8 * s + 2 * j + h;
                const int8_t* a = aq + (size_t)t * K + 32 * b;
                sc2[h] = asc[(size_t)b * Mp + t];
                x[h] = (int32_t)g.wsc[2 * b] * dot16(a, g.q + 32 * b) + (int32_t)g.wsc[2 * b + 1] * dot16(a + 16, g.q + 32 * b + 16);
                y[h] = (int32_t)g.wmn[2 * b] * sum16(a) + (int32_t)g.wmn[2 * b + 1] * sum16(a + 16);
              }
              tq = fmaf(sc2[0], (float)x[0], fmaf(sc2[1], (float)x[1], tq));
              tmn = fmaf(sc2[0], (float)y[0], fmaf(sc2[1], (float)y[1], tmn));
            }
            v = fmaf(g.wd[s], tq, fmaf(-g.wd[nsb + s], tmn, v));
          }
        }
        float* c = C + (size_t)t * ldc + c_off + n;
        *c = order == 0 ? (acc ? *c + v : v) : store_mode(*c, v, acc);
      }
    }
    grow_free(&g);
  }
}

/* f32 CPU model (tools/ref_forward.cpp:251-305 matmul with REF_Q=all REF_QB=32, i.e. round_int8 :109-126):
 * weights through dequant_row, activations de-quantised (scale * int8), double accumulation, cast to float. */
void orc_matmul_f64(int type, const uint8_t* w, int N, int K, const int8_t* aq, const float* asc, int Mp, int M, float* Y,
                    int ldy) {
  const size_t rb = (size_t)(K / 256) * orc_sb_bytes(type);
  float* X = (float*)malloc((size_t)M * K * 4);
  for (int m = 0; m < M; ++m)
    for (int k = 0; k < K; ++k) X[(size_t)m * K + k] = asc[(size_t)(k / 32) * Mp + m] * (float)aq[(size_t)m * K + k];
#pragma omp parallel
  {
    float* wf = (float*)malloc((size_t)K * 4);
#pragma omp for schedule(dynamic, 16)
    for (int n = 0; n < N; ++n) {
      orc_dequant_row(type, w + (size_t)n * rb, K, wf);
      for (int m = 0; m < M; ++m) {
        double a = 0;
        const float* x = X + (size_t)m * K;
        for (int k = 0; k < K; ++k) a += (double)wf[k] * x[k];
        Y[(size_t)m * ldy + n] = (float)a;
      }
    }
    free(wf);
  }
  free(X);
}

/* ---------------------------------------------------------------- mixture of experts
 * routing (zero/kernels/moe.cl:50-89): softmax numerators exp(l - max) of the NU largest logits (ties: lower expert
 * id), weights renormalised over the selection; counts per expert. */
void orc_moe_route(const float* logits, int ldl, int T, int NE, int NU, int32_t* ids, float* wts, int32_t* counts) {
  for (int e = 0; e < NE; ++e) counts[e] = 0;
  float* v = (float*)malloc((size_t)NE * 4);
  float* p = (float*)malloc((size_t)NU * 4);
  for (int t = 0; t < T; ++t) {
    const float* lg = logits + (size_t)t * ldl;
    float mx = -INFINITY;
    for (int e = 0; e < NE; ++e) { v[e] = lg[e]; mx = fmaxf(mx, v[e]); }
    float sum = 0.0f;
    for (int k = 0; k < NU; ++k) {
      float bv = -INFINITY;
      int bi = NE;
      for (int e = 0; e < NE; ++e)
        if (v[e] > bv) { bv = v[e]; bi = e; }
      if (bi < NE) v[bi] = -INFINITY;
      const int sel = bi < NE - 1 ? bi : NE - 1;
      ids[t * NU + k] = sel;
      p[k] = expf(bv - mx);
      sum += p[k];
      counts[sel]++;
    }
    for (int k = 0; k < NU; ++k) wts[t * NU + k] = p[k] / sum;
  }
  free(v);
  free(p);
}

/* counting sort of the (token, choice) pairs into expert slots (zero/kernels/moe.cl:141-179).  The reference places
 * pairs with atomic_inc (order inside an expert unspecified); here: increasing pair index, the deterministic choice.
 * tiles: tiles[0] = count, then (expert, first slot, rows<=TM) per tile.  offs[NE+1]. */
void orc_moe_sort(const int32_t* ids, const float* wts, int T, int NE, int NU, int TM, const int32_t* counts,
                  int32_t* offs, int32_t* tiles, int32_t* stok, float* swt, int32_t* inv) {
  int nt = 0, off = 0;
  for (int e = 0; e < NE; ++e) {
    offs[e] = off;
    for (int i = 0; i * TM < counts[e]; ++i) {
      int32_t* tp = tiles + 1 + 3 * nt++;
      tp[0] = e;
      tp[1] = off + i * TM;
      tp[2] = counts[e] - i * TM < TM ? counts[e] - i * TM : TM;
    }
    off += counts[e];
  }
  offs[NE] = off;
  tiles[0] = nt;
  int32_t* cur = (int32_t*)malloc((size_t)NE * 4);
  memcpy(cur, offs, (size_t)NE * 4);
  for (int i = 0; i < T * NU; ++i) {
    const int s = cur[ids[i]]++;
    stok[s] = i / NU;
    swt[s] = wts[i];
    inv[i] = s;
  }
  free(cur);
}

/* h[slot][F] = silu(g) * u with g = x_tok Wg_e^T, u = x_tok Wu_e^T in the GEMV order
 * (zero/kernels/decode_moe.cl:58-72 moe_term, :92-260 moe_gateup_q, silu at :257).  wg, wu: [NE][F] rows of K. */
void orc_moe_gateup(int type, const uint8_t* wg, const uint8_t* wu, int F, int K, const int8_t* aq, const float* asc,
                    int Mp, int S, const int32_t* slot_expert, const int32_t* stok, float* h, float* g_out, float* u_out) {
  const size_t rb = (size_t)(K / 256) * orc_sb_bytes(type);
#pragma omp parallel for schedule(dynamic, 4)
  for (int s = 0; s < S; ++s) {
    const int e = slot_expert[s], t = stok[s];
    float* g = (float*)malloc((size_t)F * 4 * 2);
    float* u = g + F;
    orc_matmul_gemv_order(type, wg + (size_t)e * F * rb, F, K, aq + (size_t)t * K, asc + t, Mp, 1, g, F, 0, 0);
    orc_matmul_gemv_order(type, wu + (size_t)e * F * rb, F, K, aq + (size_t)t * K, asc + t, Mp, 1, u, F, 0, 0);
    for (int f = 0; f < F; ++f) {
      h[(size_t)s * F + f] = g[f] / (1.0f + expf(-g[f])) * u[f];
      if (g_out) g_out[(size_t)s * F + f] = g[f];
      if (u_out) u_out[(size_t)s * F + f] = u[f];
    }
    free(g);
  }
}

/* y[slot][E] = swt[slot] * (hq[slot] Wd_e^T) (zero/kernels/decode_moe.cl:269-449, scaling at :446).  wd: [NE][E] rows
 * of F; hq [S][F] int8, hsc [F/32][S]. */
void orc_moe_down(int type, const uint8_t* wd, int E, int F, const int8_t* hq, const float* hsc, int S,
                  const int32_t* slot_expert, const float* swt, float* y) {
  const size_t rb = (size_t)(F / 256) * orc_sb_bytes(type);
#pragma omp parallel for schedule(dynamic, 4)
  for (int s = 0; s < S; ++s) {
    const int e = slot_expert[s];
    orc_matmul_gemv_order(type, wd + (size_t)e * E * rb, E, F, hq + (size_t)s * F, hsc + s, S, 1, y + (size_t)s * E, E, 0, 0);
    for (int c = 0; c < E; ++c) y[(size_t)s * E + c] *= swt[s];
  }
}

/* x[t] += sum_k y[inv[t*NU+k]] in choice order (zero/kernels/moe.cl:344-352; no shared expert) */
/* the shared expert's gate (SGATE, zero/kernels/moe.cl:44,88): the sigmoid of the logit that follows the experts' */
void orc_moe_sgate(const float* logits, int ldl, int T, int NE, float* sgate) {
  for (int t = 0; t < T; ++t) sgate[t] = 1.0f / (1.0f + expf(-logits[(size_t)t * ldl + NE]));
}

/* expert-parallel sort (zero/kernels/tp.cl:55-78): experts outside [e0, e1) count as empty, their pairs get inv = -1, and a
 * tile names its expert by its index in the rank's own stack (e - e0) */
void orc_moe_sort_range(const int32_t* ids, const float* wts, int T, int NE, int NU, int TM, const int32_t* counts, int e0, int e1,
                        int32_t* offs, int32_t* tiles, int32_t* stok, float* swt, int32_t* inv) {
  int nt = 0, off = 0;
  for (int e = 0; e < NE; ++e) {
    const int c = (e >= e0 && e < e1) ? counts[e] : 0;
    offs[e] = off;
    for (int i = 0; i * TM < c; ++i) {
      int32_t* tp = tiles + 1 + 3 * nt++;
      tp[0] = e - e0;
      tp[1] = off + i * TM;
      tp[2] = c - i * TM < TM ? c - i * TM : TM;
    }
    off += c;
  }
  offs[NE] = off;
  tiles[0] = nt;
  int32_t* cur = (int32_t*)malloc((size_t)NE * 4);
  memcpy(cur, offs, (size_t)NE * 4);
  for (int i = 0; i < T * NU; ++i) {
    const int e = ids[i];
    if (e < e0 || e >= e1) { inv[i] = -1; continue; }
    const int s = cur[e]++;
    stok[s] = i / NU;
    swt[s] = wts[i];
    inv[i] = s;
  }
  free(cur);
}

/* moe_combine with the shared expert (zero/kernels/moe.cl:344-352) and the partial form of the expert-parallel split
 * (tp_moe_combine, zero/kernels/tp.cl:100-111): v = sum of the token's slots >= 0 in choice order (+ sgate * sh);
 * x += v, or x = v when partial */
void orc_moe_combine_ex(float* x, const float* y, const int32_t* inv, int T, int NU, int E, const float* sh, const float* sgate,
                        int partial) {
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < E; ++c) {
      float v = 0.0f;
      for (int k = 0; k < NU; ++k) {
        const int s = inv[t * NU + k];
        if (s >= 0) v += y[(size_t)s * E + c];
      }
      if (sh) v += sgate[t] * sh[(size_t)t * E + c];
      x[(size_t)t * E + c] = partial ? v : x[(size_t)t * E + c] + v;
    }
}

void orc_moe_combine(float* x, const float* y, const int32_t* inv, int T, int NU, int E) {
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < E; ++c) {
      float v = 0.0f;
      for (int k = 0; k < NU; ++k) v += y[(size_t)inv[t * NU + k] * E + c];
      x[(size_t)t * E + c] += v;
    }
}

/* ---------------------------------------------------------------- SwiGLU (zero/kernels/ops.cl:272-315, fused = 0) */
void orc_swiglu(const float* g, const float* u, size_t n, float* h) {
  for (size_t i = 0; i < n; ++i) h[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
}

/* ---------------------------------------------------------------- logit soft-cap (zero/kernels/ops_attn_g.cl:724-729;
 * zero/kernels/decode.cl:882-887 HEAD_OUT): v = cap * tanh(v * (1 / cap)) on columns off .. off+N-1 of `rows` rows */
void orc_softcap_rows(float* c, int rows, int ld, int off, int N, float cap) {
  const float rcap = 1.0f / cap;
  for (int r = 0; r < rows; ++r)
    for (int n = 0; n < N; ++n) {
      float* p = c + (size_t)r * ld + off + n;
      *p = cap * tanhf(*p * rcap);
    }
}

/* ---------------------------------------------------------------- tensor parallel
 * rank r's part of `total` in whole units (zero/mgpu/engine_tp_shard.h:68-72) */
void orc_tp_range(int64_t total, int64_t unit, int N, int r, int64_t* begin, int64_t* end) {
  const int64_t units = total / unit, base = units / N, extra = units % N;
  const int64_t b = r * base + (r < extra ? r : extra), e = b + base + (r < extra ? 1 : 0);
  *begin = b * unit;
  *end = e * unit;
}

/* x[i] += part_0[i] + part_1[i] + ... in rank order (zero/kernels/tp.cl:5-11) */
void orc_tp_add(float* x, const float* parts, size_t n, int np, size_t stride) {
  for (size_t i = 0; i < n; ++i) {
    float s = x[i];
    for (int k = 0; k < np; ++k) s += parts[(size_t)k * stride + i];
    x[i] = s;
  }
}
