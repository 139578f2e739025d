// Further GGUF weight types through the path: Q4_0, Q5_K, Q6_K, IQ4_XS.
//
// The reference decodes every K-quant and codebook type with one table-driven per-block decoder into a generic view
// (DecodedSB, src/quants.h:72-87; device twin decode32, zero/kernels/decode.cl:183-478):
//     w[e] = wd * wsc[e/16] * (q[e] - qoff) - wdmin * wmn[e/16]          (an integer scale and min per 16 elements)
// and runs the per-32-block integer arithmetic on it (zero/kernels/decode.cl:992-1004):
//     term = sa * (d * (float)(sc0*lo + sc1*hi) - dmin * (float)(mn0*bs0 + mn1*bs1)),   lo / hi = dots of the two halves.
// Here that view IS the device format ("K16"): the loader decodes the file's superblocks once, on the host, into
//     f32 wd | f32 wdmin | int8 wsc[16] | uint8 wmn[16] | 8 pad | int8 (q - qoff)[256]           = 304 bytes per 256 weights
// so that the kernels need no per-type bit fiddling: 16-byte aligned int8 quants for dp4a, scales a lane reads with two
// small loads.  Exact for every type whose quants minus offset fit int8: Q5_K (0..31), Q6_K (-32..31), IQ4_XS (codebook
// values -127..113).  Q4_0 is a Q8_0 with 4-bit quants q - 8 (src/quants.h:136-148): it is rewritten as Q8_0 blocks and
// takes the Q8_0 kernels, tensor-core GEMM included.
//
// Q6_K is the exception to "the view is the device format": it stays packed (kQ6pSbBytes = 224 per superblock, the file's
// 210 bytes padded) and the kernels unpack a 32-block from 32 bytes of low nibbles and 32 bytes of high bit pairs into
// the same int8 quants -- a decode step over the Q6_K output head streams 0.875 instead of 1.19 bytes per weight.
//
// Kernels: a GEMV for 1..8 activation rows (warp per weight row, lane per 32-block, activations staged in shared memory)
// and a CUDA-core GEMM with the per-superblock combine of the Q4_K kernel.  The tensor-core GEMM does not take K16 (its
// exact-integer fp16 operand trick needs |scale * quant| < 2048; Q6_K reaches 4096).
#include <string.h>

#include <vector>

#include "izb_common.cuh"

// ---------------------------------------------------------------------------------------------- host: decoders
namespace {

float h2f(const uint8_t* p) {  // fp16 -> f32, subnormals included
  const uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
  const uint32_t sign = (h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
  uint32_t f;
  if (e == 0) {
    if (m == 0) {
      f = sign;
    } else {
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 1024u)) { mm <<= 1; ++sh; }
      f = sign | ((uint32_t)(113 - sh) << 23) | ((mm & 1023u) << 13);
    }
  } else if (e == 31) {
    f = sign | 0x7F800000u | (m << 13);
  } else {
    f = sign | ((e + 112u) << 23) | (m << 13);
  }
  float r;
  memcpy(&r, &f, 4);
  return r;
}

void k4_scale_min(int j, const uint8_t* s, int& sc, int& mn) {  // src/quants.h:61-69
  if (j < 4) {
    sc = s[j] & 63;
    mn = s[j + 4] & 63;
  } else {
    sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
    mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
  }
}

const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};  // the IQ4_NL / IQ4_XS codebook

struct K16Sb {  // the device superblock, 304 bytes
  float wd, wdmin;
  int8_t wsc[16];
  uint8_t wmn[16];
  uint8_t pad[8];
  int8_t q[256];
};
static_assert(sizeof(K16Sb) == kK16SbBytes, "K16 superblock");

void decode_q5_k(const uint8_t* p, K16Sb& o) {  // src/quants.h:91-114
  o.wd = h2f(p);
  o.wdmin = h2f(p + 2);
  for (int b = 0; b < 8; ++b) {
    int sc, mn;
    k4_scale_min(b, p + 4, sc, mn);
    o.wsc[2 * b] = o.wsc[2 * b + 1] = (int8_t)sc;
    o.wmn[2 * b] = o.wmn[2 * b + 1] = (uint8_t)mn;
  }
  const uint8_t* qh = p + 16;
  const uint8_t* qs = p + 48;
  for (int j = 0; j < 4; ++j)
    for (int l = 0; l < 32; ++l) {
      o.q[64 * j + l] = (int8_t)((qs[32 * j + l] & 0xF) | (((qh[l] >> (2 * j)) & 1) << 4));
      o.q[64 * j + 32 + l] = (int8_t)((qs[32 * j + l] >> 4) | (((qh[l] >> (2 * j + 1)) & 1) << 4));
    }
}

void decode_iq4_xs(const uint8_t* p, K16Sb& o) {  // src/quants.h:297-312
  o.wd = h2f(p);
  o.wdmin = 0.0f;
  const uint32_t sh = (uint32_t)p[2] | ((uint32_t)p[3] << 8);
  const uint8_t* sl = p + 4;
  const uint8_t* qs = p + 8;
  for (int ib = 0; ib < 8; ++ib) {
    const int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
    o.wsc[2 * ib] = o.wsc[2 * ib + 1] = (int8_t)(ls - 32);
    o.wmn[2 * ib] = o.wmn[2 * ib + 1] = 0;
    for (int j = 0; j < 16; ++j) {
      o.q[32 * ib + j] = kIq4nl[qs[16 * ib + j] & 0xF];
      o.q[32 * ib + 16 + j] = kIq4nl[qs[16 * ib + j] >> 4];
    }
  }
}

}  // namespace

// bytes of 256 weights of a ggml type in the file, or 0 when the library does not take the type (src/gguf.h:48-70)
int izb_gguf_sb_bytes(int ggml_type) {
  switch (ggml_type) {
    case IZB_Q8_0: return 8 * 34;
    case IZB_Q4_K: return 144;
    case IZB_Q4_0: return 8 * 18;
    case IZB_Q5_K: return 176;
    case IZB_Q6_K: return 210;
    case IZB_IQ4_XS: return 136;
    default: return 0;
  }
}

// `n_sb` superblocks of the file's form -> the device's source form (GGUF Q8_0 blocks for Q4_0, K16 for the rest)
void izb_transcode_sb(int ggml_type, const uint8_t* src, size_t n_sb, uint8_t* dst) {
  if (ggml_type == IZB_Q4_0) {
    for (size_t b = 0; b < n_sb * 8; ++b) {
      const uint8_t* s = src + 18 * b;
      uint8_t* d = dst + 34 * b;
      d[0] = s[0];
      d[1] = s[1];
      for (int i = 0; i < 16; ++i) {
        d[2 + i] = (uint8_t)(int8_t)((s[2 + i] & 0xF) - 8);
        d[18 + i] = (uint8_t)(int8_t)((s[2 + i] >> 4) - 8);
      }
    }
    return;
  }
  if (ggml_type == IZB_Q6_K) {  // kept packed: the 210 bytes as they are (ql | qh | scales | d), padded to 224
    for (size_t i = 0; i < n_sb; ++i) {
      memcpy(dst + i * kQ6pSbBytes, src + i * 210, 210);
      memset(dst + i * kQ6pSbBytes + 210, 0, kQ6pSbBytes - 210);
    }
    return;
  }
  const int sbb = izb_gguf_sb_bytes(ggml_type);
  for (size_t i = 0; i < n_sb; ++i) {
    K16Sb o;
    memset(&o, 0, sizeof o);
    if (ggml_type == IZB_Q5_K) decode_q5_k(src + i * sbb, o);
    else decode_iq4_xs(src + i * sbb, o);
    memcpy(dst + i * kK16SbBytes, &o, sizeof o);
  }
}

// ---------------------------------------------------------------------------------------------- device: GEMV, 1..8 rows
namespace {

constexpr int kGvWarps = 8;

// One warp per weight row (rows warp, warp + W, ... of a persistent grid), one lane per 32-block: a step of the warp
// covers four superblocks.  A lane reads its block's 32 int8 quants (two 128-bit streaming loads), the two scales and
// mins of the block's halves, and multiplies them into the T activation rows the CTA staged in shared memory at start.
template <int T, bool kMin>
__global__ void __launch_bounds__(kGvWarps * 32) gemv_k16_kernel(const uint8_t* __restrict__ raw, int N, int K,
                                                                 const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp,
                                                                 float* __restrict__ C, int ldc, int c_off, int acc) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int nb = K >> 5, nsb = K >> 8;
  int8_t* s_a = reinterpret_cast<int8_t*>(smem);                          // [T][K]
  float* s_sc = reinterpret_cast<float*>(smem + (size_t)T * K);           // [T][K/32]
  for (int i = threadIdx.x; i < T * (K / 16); i += blockDim.x) {
    const int t = i / (K / 16), pc = i % (K / 16);
    reinterpret_cast<uint4*>(s_a)[i] = *reinterpret_cast<const uint4*>(aq + (size_t)t * K + 16 * pc);
  }
  for (int i = threadIdx.x; i < T * nb; i += blockDim.x) {
    const int t = i / nb, b = i % nb;
    s_sc[i] = asc[(size_t)b * Mp + t];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t row_bytes = (size_t)nsb * kK16SbBytes;
  for (int n = blockIdx.x * kGvWarps + warp; n < N; n += gridDim.x * kGvWarps) {
    const uint8_t* row = raw + (size_t)n * row_bytes;
    float sum[T];
#pragma unroll
    for (int t = 0; t < T; ++t) sum[t] = 0.0f;
    for (int sb = lane >> 3; sb < nsb; sb += 4) {
      const int blk = lane & 7;
      const uint8_t* p = row + (size_t)sb * kK16SbBytes;
      const float wd = *reinterpret_cast<const float*>(p), wdmin = *reinterpret_cast<const float*>(p + 4);
      const int sc0 = (int)(int8_t)p[8 + 2 * blk], sc1 = (int)(int8_t)p[9 + 2 * blk];
      const int mn0 = kMin ? (int)p[24 + 2 * blk] : 0, mn1 = kMin ? (int)p[25 + 2 * blk] : 0;
      const uint4 q0 = ldg_stream_v4(p + 48 + 32 * blk), q1 = ldg_stream_v4(p + 64 + 32 * blk);
      const int gb = sb * 8 + blk;
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const uint4 a0 = *reinterpret_cast<const uint4*>(s_a + (size_t)t * K + 32 * gb);
        const uint4 a1 = *reinterpret_cast<const uint4*>(s_a + (size_t)t * K + 32 * gb + 16);
        int lo = __dp4a((int)a0.x, (int)q0.x, 0);
        lo = __dp4a((int)a0.y, (int)q0.y, lo);
        lo = __dp4a((int)a0.z, (int)q0.z, lo);
        lo = __dp4a((int)a0.w, (int)q0.w, lo);
        int hi = __dp4a((int)a1.x, (int)q1.x, 0);
        hi = __dp4a((int)a1.y, (int)q1.y, hi);
        hi = __dp4a((int)a1.z, (int)q1.z, hi);
        hi = __dp4a((int)a1.w, (int)q1.w, hi);
        const float sa = s_sc[t * nb + gb];
        const float x = (float)(sc0 * lo + sc1 * hi);
        if (kMin) {
          int bs0 = __dp4a((int)a0.x, 0x01010101, 0);
          bs0 = __dp4a((int)a0.y, 0x01010101, bs0);
          bs0 = __dp4a((int)a0.z, 0x01010101, bs0);
          bs0 = __dp4a((int)a0.w, 0x01010101, bs0);
          int bs1 = __dp4a((int)a1.x, 0x01010101, 0);
          bs1 = __dp4a((int)a1.y, 0x01010101, bs1);
          bs1 = __dp4a((int)a1.z, 0x01010101, bs1);
          bs1 = __dp4a((int)a1.w, 0x01010101, bs1);
          sum[t] = __fadd_rn(sum[t], __fmul_rn(sa, __fsub_rn(__fmul_rn(wd, x), __fmul_rn(wdmin, (float)(mn0 * bs0 + mn1 * bs1)))));
        } else {
          sum[t] = __fadd_rn(sum[t], __fmul_rn(__fmul_rn(sa, wd), x));
        }
      }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(sum[t]);
      if (lane == 0) {
        float* c = C + (size_t)t * ldc + c_off + n;
        *c = acc ? __fadd_rn(*c, v) : v;
      }
    }
  }
}

// ---- Q6_K packed (kQ6pSbBytes per superblock).  Element e = 128 n + 32 sub + l of a superblock (src/quants.h:115-135):
//   low nibble:  ql[64 n + 32 (sub & 1) + l] >> 4 (sub >> 1);   high two bits: qh[32 n + l] >> 2 sub;   value - 32;
//   scale[8 n + 2 sub + l / 16].  Four weights per 32-bit word:
__device__ __forceinline__ uint32_t q6p_word(uint32_t ql, uint32_t qh, int sub) {
  const uint32_t qu = ((ql >> (4 * (sub >> 1))) & 0x0F0F0F0Fu) | (((qh >> (2 * sub)) & 0x03030303u) << 4);  // 0..63 per byte
  return ((qu | 0x80808080u) - 0x20202020u) ^ 0x80808080u;                                                  // - 32 per byte, no borrow
}

// Same warp / lane mapping and the same arithmetic as gemv_k16_kernel (so the two device forms give identical bits); a
// lane unpacks its 32-block from 32 bytes of ql and 32 bytes of qh.  Lanes that share bytes (sub and sub + 2 share ql, the
// four sub-blocks of a half share qh) read the same addresses in the same instruction: one transaction.
template <int T>
__global__ void __launch_bounds__(kGvWarps * 32, T <= 2 ? 4 : T <= 4 ? 3 : 2) gemv_q6p_kernel(const uint8_t* __restrict__ raw, int N, int K,
                                                                 const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp,
                                                                 float* __restrict__ C, int ldc, int c_off, int acc) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int nb = K >> 5, nsb = K >> 8;
  int8_t* s_a = reinterpret_cast<int8_t*>(smem);                          // [T][K]
  float* s_sc = reinterpret_cast<float*>(smem + (size_t)T * K);           // [T][K/32]
  for (int i = threadIdx.x; i < T * (K / 16); i += blockDim.x) {
    const int t = i / (K / 16), pc = i % (K / 16);
    reinterpret_cast<uint4*>(s_a)[i] = *reinterpret_cast<const uint4*>(aq + (size_t)t * K + 16 * pc);
  }
  for (int i = threadIdx.x; i < T * nb; i += blockDim.x) {
    const int t = i / nb, b = i % nb;
    s_sc[i] = asc[(size_t)b * Mp + t];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t row_bytes = (size_t)nsb * kQ6pSbBytes;
  const int blk = lane & 7, nh = blk >> 2, sub = blk & 3;
  for (int n = blockIdx.x * kGvWarps + warp; n < N; n += gridDim.x * kGvWarps) {
    const uint8_t* row = raw + (size_t)n * row_bytes;
    float sum[T];
#pragma unroll
    for (int t = 0; t < T; ++t) sum[t] = 0.0f;
    for (int sb = lane >> 3; sb < nsb; sb += 4) {
      const uint8_t* p = row + (size_t)sb * kQ6pSbBytes;
      const uint4 l0 = ldg_stream_v4(p + 64 * nh + 32 * (sub & 1)), l1 = ldg_stream_v4(p + 64 * nh + 32 * (sub & 1) + 16);
      const uint4 h0 = ldg_stream_v4(p + 128 + 32 * nh), h1 = ldg_stream_v4(p + 128 + 32 * nh + 16);
      const uint4 tail = ldg_stream_v4(p + 192);  // the 16 scales; d follows in the next 16 bytes
      const uint32_t scw[4] = {tail.x, tail.y, tail.z, tail.w};
      const uint32_t sc2 = scw[blk >> 1] >> (16 * (blk & 1));
      const int sc0 = (int)(int8_t)(sc2 & 0xFFu), sc1 = (int)(int8_t)((sc2 >> 8) & 0xFFu);
      const float wd = half_bits_to_float((uint32_t)*reinterpret_cast<const unsigned short*>(p + 208));
      const uint32_t q[8] = {q6p_word(l0.x, h0.x, sub), q6p_word(l0.y, h0.y, sub), q6p_word(l0.z, h0.z, sub), q6p_word(l0.w, h0.w, sub),
                             q6p_word(l1.x, h1.x, sub), q6p_word(l1.y, h1.y, sub), q6p_word(l1.z, h1.z, sub), q6p_word(l1.w, h1.w, sub)};
      const int gb = sb * 8 + blk;
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const uint4 a0 = *reinterpret_cast<const uint4*>(s_a + (size_t)t * K + 32 * gb);
        const uint4 a1 = *reinterpret_cast<const uint4*>(s_a + (size_t)t * K + 32 * gb + 16);
        int lo = __dp4a((int)a0.x, (int)q[0], 0);
        lo = __dp4a((int)a0.y, (int)q[1], lo);
        lo = __dp4a((int)a0.z, (int)q[2], lo);
        lo = __dp4a((int)a0.w, (int)q[3], lo);
        int hi = __dp4a((int)a1.x, (int)q[4], 0);
        hi = __dp4a((int)a1.y, (int)q[5], hi);
        hi = __dp4a((int)a1.z, (int)q[6], hi);
        hi = __dp4a((int)a1.w, (int)q[7], hi);
        const float sa = s_sc[t * nb + gb];
        sum[t] = __fadd_rn(sum[t], __fmul_rn(__fmul_rn(sa, wd), (float)(sc0 * lo + sc1 * hi)));
      }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(sum[t]);
      if (lane == 0) {
        float* c = C + (size_t)t * ldc + c_off + n;
        *c = acc ? __fadd_rn(*c, v) : v;
      }
    }
  }
}

template <int T>
int launch_gemv_k16(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc,
                    int c_off, int acc, cudaStream_t st) {
  const size_t smem = (size_t)T * w->K + (size_t)T * (w->K / 32) * 4;
  if (smem > 200 * 1024) IZB_FAIL(IZB_ERR_LIMIT, "gemv: %d rows of K = %d do not fit in shared memory", T, w->K);
  int grid = izb_sm_count(w->device) * (smem <= 100 * 1024 ? 2 : 1);
  // (the packed form needs more loads in flight per SM than two CTAs issue: four, or three for 3..4 rows, where the
  //  activations leave room -- 151936 x 5120, one row: 300 us with two CTAs per SM, 142 us with four)
  if (w->packed6 && T <= 4 && smem <= 48 * 1024) grid = izb_sm_count(w->device) * (T <= 2 ? 4 : 3);
  const int need = (w->N + kGvWarps - 1) / kGvWarps;
  if (grid > need) grid = need;
  if (w->packed6) {
    IZB_SMEM_OPTIN((gemv_q6p_kernel<T>), 200 * 1024, w->device);
    IZB_LAUNCH("gemv_q6p", st, gemv_q6p_kernel<T><<<grid, kGvWarps * 32, smem, st>>>(raw, w->N, w->K, aq, asc, Mp, C, ldc, c_off, acc));
  } else if (w->has_min) {
    IZB_SMEM_OPTIN((gemv_k16_kernel<T, true>), 200 * 1024, w->device);
    IZB_LAUNCH("gemv_k16", st, gemv_k16_kernel<T, true><<<grid, kGvWarps * 32, smem, st>>>(raw, w->N, w->K, aq, asc, Mp, C, ldc, c_off, acc));
  } else {
    IZB_SMEM_OPTIN((gemv_k16_kernel<T, false>), 200 * 1024, w->device);
    IZB_LAUNCH("gemv_k16", st, gemv_k16_kernel<T, false><<<grid, kGvWarps * 32, smem, st>>>(raw, w->N, w->K, aq, asc, Mp, C, ldc, c_off, acc));
  }
  return IZB_OK;
}

}  // namespace

int izb_gemv_k16_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int T, int Mp, float* C, int ldc,
                        int c_off, int acc, cudaStream_t st) {
  switch (T) {
    case 1: return launch_gemv_k16<1>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 2: return launch_gemv_k16<2>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 3: return launch_gemv_k16<3>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 4: return launch_gemv_k16<4>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 5: return launch_gemv_k16<5>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 6: return launch_gemv_k16<6>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 7: return launch_gemv_k16<7>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    default: return launch_gemv_k16<8>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
  }
}

// ---------------------------------------------------------------------------------------------- device: GEMM on the CUDA cores
// 64 tokens x 64 weight rows per CTA, one superblock per step staged in shared memory, 4 x 4 outputs per thread, dp4a over
// the 16-element halves; combine in the order of the Q4_K kernel with a scale and min per half:
//   tq  = fma(sl, (float)(sc0*lo + sc1*hi), fma(sh, (float)(...), tq)),  tmn likewise with the mins and activation sums,
//   res = fma(wd, tq, fma(-wdmin, tmn, res))   per superblock
// (without mins wdmin = 0 and every wmn = 0: the second fma leaves res as it is).  kDots: the per-32-block integer dots.
namespace {

constexpr int GM = 64, GN = 64, GP = 65;  // tile, words per staged row (256 B + 4)

template <bool kDots, bool kPacked6>
__global__ void __launch_bounds__(256) gemm_k16_kernel(const uint8_t* __restrict__ raw, int N, int K, const int8_t* __restrict__ aq,
                                                       const float* __restrict__ asc, int Mp, int M, float* __restrict__ C, int ldc,
                                                       int c_off, int acc, int32_t* __restrict__ dots) {
  __shared__ uint32_t sA[GM * GP], sW[GN * GP];
  __shared__ float s_asc[8][GM];
  __shared__ int s_asum[16][GM];
  __shared__ float s_d[GN][2];
  __shared__ int8_t s_sc[GN][16];
  __shared__ uint8_t s_mn[GN][16];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * GN, m0 = blockIdx.y * GM;
  const int nsb = K >> 8, nb = K >> 5;
  constexpr int kSb = kPacked6 ? kQ6pSbBytes : kK16SbBytes;
  const size_t row_bytes = (size_t)nsb * kSb;
  float res[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) res[i][j] = 0.0f;
  for (int s = 0; s < nsb; ++s) {
    __syncthreads();
    for (int i = tid; i < GM * 16; i += 256) {
      const int m = i >> 4, pc = i & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m0 + m < Mp) v = *reinterpret_cast<const uint4*>(aq + (size_t)(m0 + m) * K + s * 256 + pc * 16);
      uint32_t* dst = sA + m * GP + pc * 4;
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    if (!kDots)
      for (int i = tid; i < 8 * GM; i += 256) {
        const int b = i / GM, m = i % GM;
        s_asc[b][m] = m0 + m < Mp ? asc[(size_t)(s * 8 + b) * Mp + m0 + m] : 0.0f;
      }
    for (int i = tid; i < GN * 16; i += 256) {
      const int n = i >> 4, pc = i & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (n0 + n < N) {
        const uint8_t* p = raw + (size_t)(n0 + n) * row_bytes + (size_t)s * kSb;
        if (kPacked6) {  // elements 16 pc .. 16 pc + 15: block j = pc / 2, its half pc % 2
          const int j = pc >> 1, hl = pc & 1, nh = j >> 2, sub = j & 3;
          const uint4 l = ldg_stream_v4(p + 64 * nh + 32 * (sub & 1) + 16 * hl), h = ldg_stream_v4(p + 128 + 32 * nh + 16 * hl);
          v = make_uint4(q6p_word(l.x, h.x, sub), q6p_word(l.y, h.y, sub), q6p_word(l.z, h.z, sub), q6p_word(l.w, h.w, sub));
        } else {
          v = ldg_stream_v4(p + 48 + 16 * pc);
        }
      }
      uint32_t* dst = sW + n * GP + pc * 4;
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    if (tid < GN) {
      uint4 h0 = make_uint4(0, 0, 0, 0), h1 = h0, h2 = h0;
      if (n0 + tid < N) {
        const uint8_t* p = raw + (size_t)(n0 + tid) * row_bytes + (size_t)s * kSb;
        if (kPacked6) {  // (brought into the generic header's form: d, dmin = 0, 16 scales, 16 mins = 0)
          const uint4 sc = ldg_stream_v4(p + 192);
          h0 = make_uint4(__float_as_uint(half_bits_to_float((uint32_t)*reinterpret_cast<const unsigned short*>(p + 208))), 0u, sc.x, sc.y);
          h1 = make_uint4(sc.z, sc.w, 0u, 0u);
        } else {
          h0 = ldg_stream_v4(p);
          h1 = ldg_stream_v4(p + 16);
          h2 = ldg_stream_v4(p + 32);
        }
      }
      s_d[tid][0] = __uint_as_float(h0.x);
      s_d[tid][1] = __uint_as_float(h0.y);
      const uint32_t scw[4] = {h0.z, h0.w, h1.x, h1.y}, mnw[4] = {h1.z, h1.w, h2.x, h2.y};
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        s_sc[tid][k] = (int8_t)(scw[k >> 2] >> (8 * (k & 3)));
        s_mn[tid][k] = (uint8_t)(mnw[k >> 2] >> (8 * (k & 3)));
      }
    }
    __syncthreads();
    if (!kDots) {
      for (int i = tid; i < 16 * GM; i += 256) {
        const int hb = i / GM, m = i % GM;
        int sum = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) sum = __dp4a((int)sA[m * GP + hb * 4 + k], 0x01010101, sum);
        s_asum[hb][m] = sum;
      }
      __syncthreads();
    }
    float tq[4][4], tmn[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) tq[i][c] = tmn[i][c] = 0.0f;
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {  // chunks of 64 = (lo block, hi block), each block two halves of 16
      int x[2][4][4], raw32[2][4][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int b = 2 * j + h;
        int d0[4][4], d1[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) d0[i][c] = d1[i][c] = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t a0[4], a1[4], w0[4], w1[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            a0[i] = sA[(i * 16 + ty) * GP + b * 8 + k];
            a1[i] = sA[(i * 16 + ty) * GP + b * 8 + 4 + k];
            w0[i] = sW[(i * 16 + tx) * GP + b * 8 + k];
            w1[i] = sW[(i * 16 + tx) * GP + b * 8 + 4 + k];
          }
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              d0[i][c] = __dp4a((int)a0[i], (int)w0[c], d0[i][c]);
              d1[i][c] = __dp4a((int)a1[i], (int)w1[c], d1[i][c]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int n = c * 16 + tx;
            raw32[h][i][c] = d0[i][c] + d1[i][c];
            x[h][i][c] = (int)s_sc[n][2 * b] * d0[i][c] + (int)s_sc[n][2 * b + 1] * d1[i][c];
          }
      }
      const int bl = 2 * j, bh = 2 * j + 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = i * 16 + ty;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = c * 16 + tx;
          if (kDots) {
            if (m0 + m < M && n0 + n < N) {
              int32_t* o = dots + ((size_t)(m0 + m) * N + n0 + n) * nb + s * 8;
              o[bl] = raw32[0][i][c];
              o[bh] = raw32[1][i][c];
            }
          } else {
            const float sl = s_asc[bl][m], sh = s_asc[bh][m];
            const int yl = (int)s_mn[n][2 * bl] * s_asum[2 * bl][m] + (int)s_mn[n][2 * bl + 1] * s_asum[2 * bl + 1][m];
            const int yh = (int)s_mn[n][2 * bh] * s_asum[2 * bh][m] + (int)s_mn[n][2 * bh + 1] * s_asum[2 * bh + 1][m];
            tq[i][c] = fmaf(sl, (float)x[0][i][c], fmaf(sh, (float)x[1][i][c], tq[i][c]));
            tmn[i][c] = fmaf(sl, (float)yl, fmaf(sh, (float)yh, tmn[i][c]));
          }
        }
      }
    }
    if (!kDots) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = c * 16 + tx;
          res[i][c] = fmaf(s_d[n][0], tq[i][c], fmaf(-s_d[n][1], tmn[i][c], res[i][c]));
        }
    }
  }
  if (kDots) return;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int m = m0 + i * 16 + ty, n = n0 + c * 16 + tx;
      if (m < M && n < N) {
        float* pc = C + (size_t)m * ldc + c_off + n;
        float v = res[i][c];
        if (acc == 1) v = __fadd_rn(v, *pc);
        else if (acc == 2) {
          const float g = *pc;
          v = __fmul_rn(v, __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
        }
        *pc = v;
      }
    }
}

}  // namespace

int izb_gemm_k16_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int M, int Mp, float* C, int ldc,
                        int c_off, int acc, int32_t* dots, cudaStream_t st) {
  dim3 grid((w->N + GN - 1) / GN, (M + GM - 1) / GM);
  if (grid.y > 65535) IZB_FAIL(IZB_ERR_LIMIT, "gemm: %d rows (at most %d per call for this weight type)", M, 65535 * GM);
  if (w->packed6) {
    if (dots) IZB_LAUNCH("gemm_k16_dots", st, (gemm_k16_kernel<true, true><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots)));
    else IZB_LAUNCH("gemm_k16", st, (gemm_k16_kernel<false, true><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots)));
    return IZB_OK;
  }
  if (dots) IZB_LAUNCH("gemm_k16_dots", st, (gemm_k16_kernel<true, false><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots)));
  else IZB_LAUNCH("gemm_k16", st, (gemm_k16_kernel<false, false><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots)));
  return IZB_OK;
}
