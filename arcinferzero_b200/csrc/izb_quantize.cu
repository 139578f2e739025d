// Activation quantiser: f32 rows -> int8 per 32-block + f32 scale (+ int16 sums per 16), HBM-bound.
// Arithmetic of quantize_act_cpu (src/quants.h:626-643) = quant_store16 (zero/kernels/ops.cl:38-72), bit for bit:
//   amax = max|x|;  inv = amax > 0 ? 127.0f / amax : 0;  q = rint(x * inv);  scale = amax / 127.0f
// The divisions and the product are written with the round-to-nearest intrinsics so no contraction or reciprocal
// approximation can change a bit.
//
// One CTA covers 32 token rows x 256 columns: every lane owns 8 consecutive values (two 128-bit loads), four lanes make
// a 32-block.  The int8 row stores are 256 contiguous bytes per warp; the scales, whose layout is block-major
// ([K/32][Mp]), go through shared memory so that each block's 32 token scales leave as one 128-byte line.
#include "izb_common.cuh"

namespace {

// kMode 0: quantise x.  1 (SwiGLU): x holds gate | up at column offset F, quantise h = silu(gate) * up; hout: optional
// f32 copy of h.
template <int kMode>
__global__ void __launch_bounds__(256) quantize_act_kernel(const float* __restrict__ x, int ldx, int M, int Mp, int K,
                                                           int8_t* __restrict__ aq, float* __restrict__ asc,
                                                           int16_t* __restrict__ absum, float* __restrict__ hout,
                                                           int F /* mode 1: up projection at column offset F */) {
  constexpr bool kSwiglu = kMode == 1;
  __shared__ float s_sc[8][33];
  __shared__ int16_t s_sum[16][34];
  const int sb = blockIdx.x, m0 = blockIdx.y * 32, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = sb * 256 + lane * 8;
  float v[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + warp + 8 * i;
    if (m < M) {
      const float4* p = reinterpret_cast<const float4*>(x + (size_t)m * ldx + col);
      const float4 a = __ldcs(p), b = __ldcs(p + 1);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
      v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
      if (kSwiglu) {  // v holds the gate g: h = g / (1 + exp(-g)) * u   (zero/kernels/ops.cl:272-315)
        const float4* pu = reinterpret_cast<const float4*>(x + (size_t)m * ldx + F + col);
        const float4 c = __ldcs(pu), d = __ldcs(pu + 1);
        const float u[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] = __fmul_rn(__fdiv_rn(v[i][k], __fadd_rn(1.0f, expf(-v[i][k]))), u[k]);
        if (hout) {
          float4* ph = reinterpret_cast<float4*>(hout + (size_t)m * F + col);
          ph[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          ph[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[i][k] = 0.0f;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp + 8 * i, m = m0 + r;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[i][k]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int q[8], s8 = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // lrintf's x86 result for products outside the int range or NaN (only when amax is so small that 127 / amax
      // overflows): INT_MIN, whose low byte is 0
      const float p = __fmul_rn(v[i][k], inv);
      q[k] = fabsf(p) <= 2147483520.0f ? __float2int_rn(p) : 0;
      s8 += q[k];
    }
    const int s16 = s8 + __shfl_xor_sync(0xFFFFFFFFu, s8, 1);
    if (m < Mp) {
      uint2 pk;
      pk.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
      pk.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
      *reinterpret_cast<uint2*>(aq + (size_t)m * K + col) = pk;
    }
    if ((lane & 3) == 0) s_sc[lane >> 2][r] = __fdiv_rn(amax, 127.0f);
    if ((lane & 1) == 0) s_sum[lane >> 1][r] = (int16_t)s16;
  }
  __syncthreads();
  {
    const int b = threadIdx.x >> 5, r = threadIdx.x & 31;
    if (m0 + r < Mp) {
      asc[(size_t)(sb * 8 + b) * Mp + m0 + r] = s_sc[b][r];
      if (absum) {
        absum[(size_t)(sb * 16 + b) * Mp + m0 + r] = s_sum[b][r];
        absum[(size_t)(sb * 16 + 8 + b) * Mp + m0 + r] = s_sum[8 + b][r];
      }
    }
  }
}

// Sum over the CTA's 256 threads in the defined order: xor butterfly 16, 8, 4, 2, 1 inside every warp, then the eight
// warp sums added in warp order; every thread returns the same value.  s_w: 8 floats of shared memory.
__device__ __forceinline__ float cta_sum_ordered(float v, float* s_w) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  __syncthreads();  // (s_w may still be read from a call before)
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = s_w[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) t = __fadd_rn(t, s_w[w]);
  return t;
}

// add_norm_quant (zero/kernels/ops_attn_g.cl:617-680), one CTA of 256 threads per row, K <= 256 * kAnqMax:
//   x = (x + (t * r) * w) * s with r = 1/sqrt(sum(t^2)/K + eps);  y = w2 ? (x * r2) * w2 : x with r2 from the new x;
//   y quantised per 32-block.  Thread j owns elements j, j + 256, ...: a warp owns one 32-block per step, so the
// block maximum is a warp reduction; the new x stays in registers between the two steps.  Both sums of squares are
// taken in the defined order of cta_sum_ordered over per-thread fused-multiply-add chains.
constexpr int kAnqMax = 64;
__global__ void __launch_bounds__(256) add_norm_quant_kernel(float* __restrict__ x, const float* __restrict__ t,
                                                             const float* __restrict__ w, int K, float eps, float s,
                                                             const float* __restrict__ w2, int Mp, int8_t* __restrict__ aq,
                                                             float* __restrict__ asc, int16_t* __restrict__ absum) {
  __shared__ float s_w[8];
  const int m = blockIdx.x, lane = threadIdx.x & 31;
  float* xr = x + (size_t)m * K;
  const float* tr = t + (size_t)m * K;
  const int nk = K / 256;
  float ss = 0.0f;
  for (int k = 0; k < nk; ++k) {
    const float v = tr[threadIdx.x + 256 * k];
    ss = __fmaf_rn(v, v, ss);
  }
  ss = cta_sum_ordered(ss, s_w);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
  float xv[kAnqMax];
  float s2 = 0.0f;
#pragma unroll
  for (int k = 0; k < kAnqMax; ++k) {
    if (k < nk) {
      const int i = threadIdx.x + 256 * k;
      const float v = __fmul_rn(__fadd_rn(xr[i], __fmul_rn(__fmul_rn(tr[i], r), w[i])), s);
      xv[k] = v;
      xr[i] = v;
      s2 = __fmaf_rn(v, v, s2);
    }
  }
  float r2 = 1.0f;
  if (w2) {
    s2 = cta_sum_ordered(s2, s_w);
    r2 = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s2, (float)K), eps)));
  }
#pragma unroll
  for (int k = 0; k < kAnqMax; ++k) {
    if (k < nk) {
      const int i = threadIdx.x + 256 * k;
      const float y = w2 ? __fmul_rn(__fmul_rn(xv[k], r2), w2[i]) : xv[k];
      float amax = fabsf(y);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
      const float p = __fmul_rn(y, inv);
      const int q = fabsf(p) <= 2147483520.0f ? __float2int_rn(p) : 0;  // (see quantize_act_kernel)
      aq[(size_t)m * K + i] = (int8_t)q;
      int s16 = q;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) s16 += __shfl_xor_sync(0xFFFFFFFFu, s16, o);
      const int b = i >> 5;
      if (lane == 0) asc[(size_t)b * Mp + m] = __fdiv_rn(amax, 127.0f);
      if (absum && (lane & 15) == 0) absum[(size_t)(2 * b + (lane >> 4)) * Mp + m] = (int16_t)s16;
    }
  }
}

// rmsnorm_quant (zero/kernels/ops.cl:104-141), one CTA of 256 threads per row: the row is read from HBM once (the second
// pass finds it in L1 / L2).  Both passes use the quantiser's lane layout: thread j owns the groups of 8 consecutive values
// j, j + 256, ... .  Pass 1: the sum of squares, a chain of fused multiply-adds over the thread's values in index order,
// then cta_sum_ordered (this order is part of the definition: the oracle repeats it).  Pass 2: y = (x * r) * w, optional
// f32 copy, and per 32-block (four adjacent threads) int8 + scale + sums of 16.
__global__ void __launch_bounds__(256) rmsnorm_quant_row_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w,
                                                                int K, float eps, int Mp, float* __restrict__ hout,
                                                                int8_t* __restrict__ aq, float* __restrict__ asc,
                                                                int16_t* __restrict__ absum) {
  __shared__ float s_w[8];
  const int m = blockIdx.x;
  const float* xr = x + (size_t)m * ldx;
  float ss = 0.0f;
  for (int g = threadIdx.x; g < K / 8; g += 256) {
    const float4 a = *reinterpret_cast<const float4*>(xr + 8 * g), b = *reinterpret_cast<const float4*>(xr + 8 * g + 4);
    ss = __fmaf_rn(a.x, a.x, ss); ss = __fmaf_rn(a.y, a.y, ss); ss = __fmaf_rn(a.z, a.z, ss); ss = __fmaf_rn(a.w, a.w, ss);
    ss = __fmaf_rn(b.x, b.x, ss); ss = __fmaf_rn(b.y, b.y, ss); ss = __fmaf_rn(b.z, b.z, ss); ss = __fmaf_rn(b.w, b.w, ss);
  }
  ss = cta_sum_ordered(ss, s_w);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
  for (int g = threadIdx.x; g < K / 8; g += 256) {  // (K / 8 is a multiple of 32: whole warps take part in the shuffles)
    const int col = 8 * g;
    const float4 a = *reinterpret_cast<const float4*>(xr + col), b = *reinterpret_cast<const float4*>(xr + col + 4);
    const float4 wa = *reinterpret_cast<const float4*>(w + col), wb = *reinterpret_cast<const float4*>(w + col + 4);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      v[k] = __fmul_rn(__fmul_rn(v[k], r), wv[k]);
      amax = fmaxf(amax, fabsf(v[k]));
    }
    if (hout) {
      float4* ph = reinterpret_cast<float4*>(hout + (size_t)m * K + col);
      ph[0] = make_float4(v[0], v[1], v[2], v[3]);
      ph[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int q[8], s8 = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float p = __fmul_rn(v[k], inv);
      q[k] = fabsf(p) <= 2147483520.0f ? __float2int_rn(p) : 0;  // (see quantize_act_kernel)
      s8 += q[k];
    }
    const int s16 = s8 + __shfl_xor_sync(0xFFFFFFFFu, s8, 1);
    uint2 pk;
    pk.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    pk.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    *reinterpret_cast<uint2*>(aq + (size_t)m * K + col) = pk;
    if ((g & 3) == 0) asc[(size_t)(g >> 2) * Mp + m] = __fdiv_rn(amax, 127.0f);
    if (absum && (g & 1) == 0) absum[(size_t)(g >> 1) * Mp + m] = (int16_t)s16;
  }
}

// rows M..Mp-1 of a quantised activation buffer: zeros with scale 0
__global__ void zero_pad_rows_kernel(int M, int Mp, int K, int8_t* __restrict__ aq, float* __restrict__ asc, int16_t* __restrict__ absum) {
  const int m = M + blockIdx.x;
  for (int i = threadIdx.x; i < K; i += blockDim.x) aq[(size_t)m * K + i] = 0;
  for (int b = threadIdx.x; b < K / 32; b += blockDim.x) asc[(size_t)b * Mp + m] = 0.0f;
  if (absum)
    for (int b = threadIdx.x; b < K / 16; b += blockDim.x) absum[(size_t)b * Mp + m] = 0;
}

int check_quant_args(const float* x, int ldx, int M, int Mp, int K, const int8_t* aq, const float* asc, int width_needed) {
  if (!x || !aq || !asc) IZB_FAIL(IZB_ERR_ARG, "quantize: null pointer");
  if (K <= 0 || K % 256) IZB_FAIL(IZB_ERR_SHAPE, "quantize: K = %d is not a positive multiple of 256", K);
  if (Mp <= 0 || Mp % 16 || M < 0 || M > Mp) IZB_FAIL(IZB_ERR_SHAPE, "quantize: rows %d of Mp = %d (Mp must be a multiple of 16)", M, Mp);
  if (ldx < width_needed) IZB_FAIL(IZB_ERR_SHAPE, "quantize: row stride %d shorter than the row (%d)", ldx, width_needed);
  if (ldx % 4 || !izb_aligned(x, 16)) IZB_FAIL(IZB_ERR_ALIGN, "quantize: input rows must be 16-byte aligned (ldx %% 4 == 0)");
  if (!izb_aligned(aq, 16) || !izb_aligned(asc, 4)) IZB_FAIL(IZB_ERR_ALIGN, "quantize: outputs not aligned");
  return IZB_OK;
}

}  // namespace

extern "C" int izb_quantize_act(const float* d_x, int ldx, int M_valid, int Mp, int K, int8_t* d_aq, float* d_asc,
                                int16_t* d_absum, void* stream) {
  if (int rc = check_quant_args(d_x, ldx, M_valid, Mp, K, d_aq, d_asc, K)) return rc;
  dim3 grid(K / 256, (Mp + 31) / 32);
  IZB_LAUNCH("quantize_act", (cudaStream_t)stream, quantize_act_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>(d_x, ldx, M_valid, Mp, K, d_aq, d_asc, d_absum, nullptr, 0));
  return IZB_OK;
}

extern "C" int izb_swiglu_quant(const float* d_gu, int ldgu, int split, int M_valid, int Mp, int F, float* d_h, int8_t* d_aq,
                                float* d_asc, int16_t* d_absum, void* stream) {
  if (int rc = check_quant_args(d_gu, ldgu, M_valid, Mp, F, d_aq, d_asc, split ? 2 * F : F)) return rc;
  if (d_h && !izb_aligned(d_h, 16)) IZB_FAIL(IZB_ERR_ALIGN, "swiglu_quant: h not 16-byte aligned");
  dim3 grid(F / 256, (Mp + 31) / 32);
  cudaStream_t st = (cudaStream_t)stream;
  if (split)
    IZB_LAUNCH("swiglu_quant", st, quantize_act_kernel<1><<<grid, 256, 0, st>>>(d_gu, ldgu, M_valid, Mp, F, d_aq, d_asc, d_absum, d_h, F));
  else
    IZB_LAUNCH("quantize_act", st, quantize_act_kernel<0><<<grid, 256, 0, st>>>(d_gu, ldgu, M_valid, Mp, F, d_aq, d_asc, d_absum, nullptr, 0));
  return IZB_OK;
}

extern "C" int izb_rmsnorm_quant(const float* d_x, int ldx, const float* d_w, float eps, int M_valid, int Mp, int K, float* d_h,
                                 int8_t* d_aq, float* d_asc, int16_t* d_absum, void* stream) {
  if (int rc = check_quant_args(d_x, ldx, M_valid, Mp, K, d_aq, d_asc, K)) return rc;
  if (!d_w) IZB_FAIL(IZB_ERR_ARG, "rmsnorm_quant: null weight");
  if (!izb_aligned(d_w, 16) || (d_h && !izb_aligned(d_h, 16))) IZB_FAIL(IZB_ERR_ALIGN, "rmsnorm_quant: w and h must be 16-byte aligned");
  if (!(eps >= 0.0f)) IZB_FAIL(IZB_ERR_ARG, "rmsnorm_quant: eps = %g", (double)eps);
  cudaStream_t st = (cudaStream_t)stream;
  if (M_valid > 0)
    IZB_LAUNCH("rmsnorm_quant", st, rmsnorm_quant_row_kernel<<<M_valid, 256, 0, st>>>(d_x, ldx, d_w, K, eps, Mp, d_h, d_aq, d_asc, d_absum));
  if (Mp > M_valid) IZB_LAUNCH("zero_pad_rows", st, zero_pad_rows_kernel<<<Mp - M_valid, 256, 0, st>>>(M_valid, Mp, K, d_aq, d_asc, d_absum));
  return IZB_OK;
}

extern "C" int izb_add_norm_quant(float* d_x, const float* d_t, const float* d_w, float eps, float s, const float* d_w2, int M_valid,
                                  int Mp, int K, int8_t* d_aq, float* d_asc, int16_t* d_absum, void* stream) {
  if (!d_x || !d_t || !d_w || !d_aq || !d_asc) IZB_FAIL(IZB_ERR_ARG, "add_norm_quant: null pointer");
  if (K <= 0 || K % 256 || K > 256 * kAnqMax) IZB_FAIL(IZB_ERR_SHAPE, "add_norm_quant: K = %d (a multiple of 256 up to %d)", K, 256 * kAnqMax);
  if (Mp <= 0 || Mp % 16 || M_valid < 0 || M_valid > Mp) IZB_FAIL(IZB_ERR_SHAPE, "add_norm_quant: rows %d of Mp = %d (Mp must be a multiple of 16)", M_valid, Mp);
  if (!(eps >= 0.0f)) IZB_FAIL(IZB_ERR_ARG, "add_norm_quant: eps = %g", (double)eps);
  cudaStream_t st = (cudaStream_t)stream;
  if (M_valid > 0)
    IZB_LAUNCH("add_norm_quant", st, add_norm_quant_kernel<<<M_valid, 256, 0, st>>>(d_x, d_t, d_w, K, eps, s, d_w2, Mp, d_aq, d_asc, d_absum));
  if (Mp > M_valid) IZB_LAUNCH("zero_pad_rows", st, zero_pad_rows_kernel<<<Mp - M_valid, 256, 0, st>>>(M_valid, Mp, K, d_aq, d_asc, d_absum));
  return IZB_OK;
}

// ---------------------------------------------------------------------------------------------- logit soft-cap
// softcap_rows (zero/kernels/ops_attn_g.cl:724) and the output head's HEAD_OUT (zero/kernels/decode.cl:882-887):
// v = cap * tanh(v * (1 / cap)) on columns off .. off+N-1 of `rows` rows.  One float4 per thread where the row start is
// 16-byte aligned, scalars otherwise.
namespace {
__global__ void __launch_bounds__(256) softcap_rows_kernel(float* __restrict__ C, int ld, int off, int N, float cap, float rcap, int vec) {
  float* p = C + (size_t)blockIdx.y * ld + off;
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (vec) {
    if (4 * i + 3 < N) {
      float4 v = *reinterpret_cast<float4*>(p + 4 * i);
      v.x = __fmul_rn(cap, tanhf(__fmul_rn(v.x, rcap)));
      v.y = __fmul_rn(cap, tanhf(__fmul_rn(v.y, rcap)));
      v.z = __fmul_rn(cap, tanhf(__fmul_rn(v.z, rcap)));
      v.w = __fmul_rn(cap, tanhf(__fmul_rn(v.w, rcap)));
      *reinterpret_cast<float4*>(p + 4 * i) = v;
    } else {
      for (int n = 4 * i; n < N; ++n) p[n] = __fmul_rn(cap, tanhf(__fmul_rn(p[n], rcap)));
    }
  } else if (i < N) {
    p[i] = __fmul_rn(cap, tanhf(__fmul_rn(p[i], rcap)));
  }
}
}  // namespace

extern "C" int izb_softcap_rows(float* d_C, int rows, int ld, int off, int N, float cap, void* stream) {
  if (!d_C) IZB_FAIL(IZB_ERR_ARG, "softcap_rows: null pointer");
  if (rows < 0 || N < 0 || off < 0 || (rows > 1 && ld < off + N)) IZB_FAIL(IZB_ERR_SHAPE, "softcap_rows: rows=%d ld=%d off=%d N=%d", rows, ld, off, N);
  if (!(cap > 0.0f)) IZB_FAIL(IZB_ERR_ARG, "softcap_rows: cap = %g (must be positive)", (double)cap);
  if (rows == 0 || N == 0) return IZB_OK;
  if (rows > 65535) IZB_FAIL(IZB_ERR_LIMIT, "softcap_rows: %d rows (at most 65535 per call)", rows);
  cudaStream_t st = (cudaStream_t)stream;
  const int vec = izb_aligned(d_C, 16) && ld % 4 == 0 && off % 4 == 0;
  const int per_row = vec ? (N + 3) / 4 : N;
  dim3 grid((per_row + 255) / 256, rows);
  IZB_LAUNCH("softcap_rows", st, softcap_rows_kernel<<<grid, 256, 0, st>>>(d_C, ld, off, N, cap, 1.0f / cap, vec));
  return IZB_OK;
}

// ---------------------------------------------------------------------------------------------- SwiGLU of interleaved columns
// gu [M][ldgu]: the outputs of a gate | up weight whose rows alternate in groups of 32 (izb_weight_create_gateup): columns
// 64 j .. 64 j + 31 are gate outputs, 64 j + 32 .. 64 j + 63 the up outputs of the same FFN rows.
// C[m][c_off + 32 j + i] = up * silu(gate) (zero/kernels/gemm.cl:562-565).  Used where the tensor-core GEMM, which forms
// this product in its epilogue, does not take the call.
namespace {
__global__ void __launch_bounds__(256) swiglu_pairs_kernel(const float* __restrict__ gu, int ldgu, int F, float* __restrict__ C, int ldc, int c_off) {
  const int f = blockIdx.x * 256 + threadIdx.x;
  if (f >= F) return;
  const float* row = gu + (size_t)blockIdx.y * ldgu + 64 * (f >> 5) + (f & 31);
  const float g = row[0], u = row[32];
  C[(size_t)blockIdx.y * ldc + c_off + f] = __fmul_rn(u, __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
}
}  // namespace

int izb_swiglu_pairs_launch(const float* gu, int ldgu, int M, int F, float* C, int ldc, int c_off, cudaStream_t st) {
  dim3 grid((F + 255) / 256, M);
  IZB_LAUNCH("swiglu_pairs", st, swiglu_pairs_kernel<<<grid, 256, 0, st>>>(gu, ldgu, F, C, ldc, c_off));
  return IZB_OK;
}
