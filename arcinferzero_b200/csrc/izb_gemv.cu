// Decode GEMV for 1..8 activation rows: C[t][n] (+)= sum_b asc[b][t] * f(block b of row n), weights read once.
// Bandwidth-bound: no tensor cores; 128-bit streaming weight loads, nibble unpack in registers, dp4a, one warp shuffle
// reduction per output.  Arithmetic of zero/kernels/decode.cl gemv (:913-1034) and gemv_mt (:1581-1694):
//   Q4_K  term = sa * (d * (float)(sc * dot) - dmin * (float)(mn * asum))
//   Q8_0  term = sa * d * (float)dot
// with dot / asum exact int32.  A lane holds a 16-element half of a block, so it adds the term of its half; the sum
// over lanes is a different order of the same f32 terms (the reference leaves that order unspecified as well).
//
// Work split: a warp owns kRows consecutive weight rows for the whole K; the 32 lanes cover 512 weight bytes per step
// (Q4_K: the nibbles of 4 superblocks, lane -> superblock lane/8, 16-byte piece lane%8; Q8_0: 2 superblocks, lane ->
// superblock lane/16, piece lane%16).  The CTA first stages the T activation rows in shared memory, permuted so that
// every lane's operands are one conflict-free 128-bit read, with the per-lane block scales and (Q4_K) the sums of the
// 16 int8 values each lane pairs with a min.
#include "izb_gemv_body.cuh"

int izb_gemv_k16_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int T, int Mp, float* C, int ldc,
                        int c_off, int acc, cudaStream_t st);
int izb_gemv_stream_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int T, int Mp, float* C,
                           int ldc, int c_off, int acc, cudaStream_t st);

namespace {
using namespace izb_gemvk;

template <int QT, int T>
__global__ void __launch_bounds__(kWarps * 32) gemv_kernel(const uint8_t* __restrict__ raw, int N, int K,
                                                           const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp,
                                                           float* __restrict__ C, int ldc, int c_off, int acc, int spc) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int tok[T];
  if (threadIdx.x < T) tok[threadIdx.x] = threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = (blockIdx.x * kWarps + warp) * kRows;
  float accv[kRows][T];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) accv[r][t] = 0.0f;
  gemv_body<QT, T>(smem, raw, N, K, aq, asc, Mp, tok, row0, spc, accv);
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(accv[r][t]);
      const int n = row0 + r;
      if (lane == 0 && n < N) {
        float* c = C + (size_t)t * ldc + c_off + n;
        *c = acc ? *c + v : v;
      }
    }
}

template <int QT, int T>
int launch_qt(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc, int c_off,
              int acc, cudaStream_t st) {
  const int grid = (w->N + kWarps * kRows - 1) / (kWarps * kRows);
  size_t smem = 0;
  const int spc = steps_per_chunk(QT, w->K, T, &smem);
  IZB_SMEM_OPTIN((gemv_kernel<QT, T>), kMaxSmem, w->device);
  IZB_LAUNCH("gemv", st, gemv_kernel<QT, T><<<grid, kWarps * 32, smem, st>>>(raw, w->N, w->K, aq, asc, Mp, C, ldc, c_off, acc, spc));
  return IZB_OK;
}

template <int T>
int launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc, int c_off,
           int acc, cudaStream_t st) {
  return w->type == IZB_Q4_K ? launch_qt<IZB_Q4_K, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st)
                             : launch_qt<IZB_Q8_0, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
}

}  // namespace
extern "C" int izb_gemv(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, int T, int Mp, float* d_C,
                        int ldc, int c_off, int acc, void* stream) {
  if (!w || !d_aq || !d_asc || !d_C) IZB_FAIL(IZB_ERR_ARG, "gemv: null pointer");
  if (mat < 0 || mat >= w->n_mats) IZB_FAIL(IZB_ERR_ARG, "gemv: matrix %d of %d", mat, w->n_mats);
  if (T < 1 || T > 8) IZB_FAIL(IZB_ERR_SHAPE, "gemv: T = %d outside 1..8", T);
  if (Mp < T) IZB_FAIL(IZB_ERR_SHAPE, "gemv: Mp = %d < T = %d", Mp, T);
  if (acc != 0 && acc != 1) IZB_FAIL(IZB_ERR_ARG, "gemv: store mode %d (the GEMV stores or adds, zero/kernels/decode.cl:1031)", acc);
  if (ldc < c_off + w->N && T > 1) IZB_FAIL(IZB_ERR_SHAPE, "gemv: ldc = %d < c_off + N = %d", ldc, c_off + w->N);
  if (!izb_aligned(d_aq, 16)) IZB_FAIL(IZB_ERR_ALIGN, "gemv: aq not 16-byte aligned");
  if (int rc = izb_require_device(w->device, "gemv")) return rc;
  const uint8_t* raw = w->raw + (size_t)mat * w->N * w->row_bytes;
  cudaStream_t st = (cudaStream_t)stream;
  if (w->type == IZB_K16) return izb_gemv_k16_launch(w, raw, d_aq, d_asc, T, Mp, d_C, ldc, c_off, acc, st);
  {  // the streaming kernel takes every call whose staged activations fit in shared memory
    const int rc = izb_gemv_stream_launch(w, raw, d_aq, d_asc, T, Mp, d_C, ldc, c_off, acc, st);
    if (rc <= 0) return rc;
  }
  switch (T) {
    case 1: return launch<1>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    case 2: return launch<2>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    case 3: return launch<3>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    case 4: return launch<4>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    case 5: return launch<5>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    case 6: return launch<6>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    case 7: return launch<7>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
    default: return launch<8>(w, raw, d_aq, d_asc, Mp, d_C, ldc, c_off, acc, st);
  }
}
