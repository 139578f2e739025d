// CUDA-core GEMM (dp4a) with the f32 combine in exactly the reference's order, and the per-block integer dots.
//
// This is the check kernel of the library, the role the reference gives its DP4a GEMM next to the XMX one
// (Engine::xmx_check, zero/engine_setup.h:424): the tensor-core kernel must reproduce its block dots bit for bit and its
// outputs to 1e-5.  Because every f32 operation below is written as an explicit fmaf / __fmul_rn in the order of
// zero/kernels/gemm.cl:441-487 (-DACT32), its outputs equal the CPU restatement of that kernel bit for bit:
//   Q8_0: res = fma(asc_lo*d_lo, (float)dot_lo, fma(asc_hi*d_hi, (float)dot_hi, res))        per 64-chunk
//   Q4_K: tq  = fma(asc_lo, (float)(sc_lo*dot_lo), fma(asc_hi, (float)(sc_hi*dot_hi), tq))
//         tmn = fma(asc_lo, (float)(mn_lo*asum_lo), fma(asc_hi, (float)(mn_hi*asum_hi), tmn))
//         res = fma(d, tq, fma(-dmin, tmn, res))                                              per superblock
// store modes (gemm.cl:556-567): 0 store, 1 add, 2 C = res * silu(C).
//
// Tiling: 64 tokens x 64 weight rows per CTA, one 256-element superblock per step staged in shared memory as int8
// (weights already unpacked), 256 threads with a 4 x 4 register tile each (rows i*16+ty, columns j*16+tx so that the
// 65-word row pitch makes both operand reads conflict-free).
#include "izb_common.cuh"

namespace {

constexpr int TM = 64, TN = 64, PITCH = 65;  // words per staged row (256 B + 4)

template <int QT, bool kDots>
__global__ void __launch_bounds__(256) gemm_core_kernel(const uint8_t* __restrict__ raw, int N, int K,
                                                        const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp,
                                                        int M, float* __restrict__ C, int ldc, int c_off, int acc,
                                                        int32_t* __restrict__ dots) {
  __shared__ uint32_t sA[TM * PITCH], sW[TN * PITCH];
  __shared__ float s_asc[8][TM];
  __shared__ int s_asum[8][TM];
  __shared__ float s_d[TN][8];     // Q8_0: d per block; Q4_K: [0] = d, [1] = dmin
  __shared__ uint8_t s_sc[TN][8], s_mn[TN][8];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * TN, m0 = blockIdx.y * TM;
  const int nsb = K >> 8, nb = K >> 5;
  constexpr int SBB = QT == IZB_Q4_K ? 144 : 272;
  const size_t row_bytes = (size_t)nsb * SBB;
  float res[4][4], tq[4][4], tmn[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) res[i][j] = tq[i][j] = tmn[i][j] = 0.0f;

  for (int s = 0; s < nsb; ++s) {
    __syncthreads();
    // ---- activations: 64 rows x 256 bytes
    for (int i = tid; i < TM * 16; i += 256) {
      const int m = i >> 4, pc = i & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m0 + m < Mp) v = *reinterpret_cast<const uint4*>(aq + (size_t)(m0 + m) * K + s * 256 + pc * 16);
      uint32_t* dst = sA + m * PITCH + pc * 4;
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    if (!kDots)
      for (int i = tid; i < 8 * TM; i += 256) {
        const int b = i / TM, m = i % TM;
        s_asc[b][m] = m0 + m < Mp ? asc[(size_t)(s * 8 + b) * Mp + m0 + m] : 0.0f;
      }
    // ---- weights
    if (QT == IZB_Q4_K) {
      for (int i = tid; i < TN * 8; i += 256) {
        const int n = i >> 3, pc = i & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n0 + n < N) v = ldg_stream_v4(raw + (size_t)(n0 + n) * row_bytes + (size_t)s * 144 + 16 + 16 * pc);
        uint32_t* lo = sW + n * PITCH + (pc >> 1) * 16 + (pc & 1) * 4;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          lo[k] = w[k] & 0x0F0F0F0Fu;
          lo[8 + k] = (w[k] >> 4) & 0x0F0F0F0Fu;
        }
      }
      if (tid < TN) {
        uint4 h = make_uint4(0, 0, 0, 0);
        if (n0 + tid < N) h = ldg_stream_v4(raw + (size_t)(n0 + tid) * row_bytes + (size_t)s * 144);
        s_d[tid][0] = half_bits_to_float(h.x & 0xFFFFu);
        s_d[tid][1] = half_bits_to_float(h.x >> 16);
        const uint32_t s3[3] = {h.y, h.z, h.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          int sc, mn;
          q4k_scale_min(s3, j, sc, mn);
          s_sc[tid][j] = (uint8_t)sc;
          s_mn[tid][j] = (uint8_t)mn;
        }
      }
    } else {
      for (int i = tid; i < TN * 16; i += 256) {
        const int n = i >> 4, pc = i & 15;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n0 + n < N) v = ldg_stream_v4(raw + (size_t)(n0 + n) * row_bytes + (size_t)s * 272 + 16 + 16 * pc);
        uint32_t* dst = sW + n * PITCH + pc * 4;
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
      }
      if (tid < TN) {
        uint4 h = make_uint4(0, 0, 0, 0);
        if (n0 + tid < N) h = ldg_stream_v4(raw + (size_t)(n0 + tid) * row_bytes + (size_t)s * 272);
        const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
        for (int b = 0; b < 8; ++b) s_d[tid][b] = half_bits_to_float((b & 1) ? hw[b >> 1] >> 16 : hw[b >> 1] & 0xFFFFu);
      }
    }
    __syncthreads();
    if (QT == IZB_Q4_K) {
      for (int i = tid; i < 8 * TM; i += 256) {
        const int b = i / TM, m = i % TM;
        int sum = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) sum = __dp4a((int)sA[m * PITCH + b * 8 + k], 0x01010101, sum);
        s_asum[b][m] = sum;
      }
      __syncthreads();
    }
    // ---- 4 chunks of 64 = (lo block, hi block)
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      int dl[4][4], dh[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) dl[i][c] = dh[i][c] = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint32_t al[4], ah[4], wl[4], wh[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          al[i] = sA[(i * 16 + ty) * PITCH + j * 16 + k];
          ah[i] = sA[(i * 16 + ty) * PITCH + j * 16 + 8 + k];
          wl[i] = sW[(i * 16 + tx) * PITCH + j * 16 + k];
          wh[i] = sW[(i * 16 + tx) * PITCH + j * 16 + 8 + k];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            dl[i][c] = __dp4a((int)al[i], (int)wl[c], dl[i][c]);
            dh[i][c] = __dp4a((int)ah[i], (int)wh[c], dh[i][c]);
          }
      }
      const int bl = 2 * j, bh = 2 * j + 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = i * 16 + ty;
        const float sl = s_asc[bl][m], sh = s_asc[bh][m];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = c * 16 + tx;
          if (kDots) {
            if (m0 + m < M && n0 + n < N) {
              int32_t* o = dots + ((size_t)(m0 + m) * N + n0 + n) * nb + s * 8;
              o[bl] = dl[i][c];
              o[bh] = dh[i][c];
            }
          } else if (QT == IZB_Q4_K) {
            tq[i][c] = fmaf(sl, (float)((int)s_sc[n][bl] * dl[i][c]), fmaf(sh, (float)((int)s_sc[n][bh] * dh[i][c]), tq[i][c]));
            tmn[i][c] = fmaf(sl, (float)((int)s_mn[n][bl] * s_asum[bl][m]), fmaf(sh, (float)((int)s_mn[n][bh] * s_asum[bh][m]), tmn[i][c]));
          } else {
            res[i][c] = fmaf(__fmul_rn(sl, s_d[n][bl]), (float)dl[i][c], fmaf(__fmul_rn(sh, s_d[n][bh]), (float)dh[i][c], res[i][c]));
          }
        }
      }
    }
    if (!kDots && QT == IZB_Q4_K) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = c * 16 + tx;
          res[i][c] = fmaf(s_d[n][0], tq[i][c], fmaf(-s_d[n][1], tmn[i][c], res[i][c]));
          tq[i][c] = tmn[i][c] = 0.0f;
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
        float* p = C + (size_t)m * ldc + c_off + n;
        float v = res[i][c];
        if (acc == 1) v = __fadd_rn(v, *p);
        else if (acc == 2) {
          const float g = *p;
          v = __fmul_rn(v, __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
        }
        *p = v;
      }
    }
}

}  // namespace

int izb_gemm_core_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int M, int Mp, float* C,
                         int ldc, int c_off, int acc, int32_t* dots, cudaStream_t st) {
  dim3 grid((w->N + TN - 1) / TN, (M + TM - 1) / TM);
  izb_prof_begin(dots ? "gemm_core_dots" : "gemm_core", st);
  if (w->type == IZB_Q4_K) {
    if (dots) gemm_core_kernel<IZB_Q4_K, true><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots);
    else gemm_core_kernel<IZB_Q4_K, false><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots);
  } else {
    if (dots) gemm_core_kernel<IZB_Q8_0, true><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots);
    else gemm_core_kernel<IZB_Q8_0, false><<<grid, 256, 0, st>>>(raw, w->N, w->K, aq, asc, Mp, M, C, ldc, c_off, acc, dots);
  }
  izb_prof_end(st);
  IZB_LAUNCHED();
  return IZB_OK;
}
