// Device bodies of the few-row GEMV (see izb_gemv.cu for the design): shared by the dense GEMV kernels and by the
// per-tile mixture-of-experts kernels, which run the same loop over the rows of one expert with gathered token rows.
#pragma once
#include "izb_common.cuh"

namespace izb_gemvk {


constexpr int kWarps = 8;
constexpr int kRows = 2;  // rows per warp, interleaved for loads in flight

// bytes of shared memory per (step, token): Q4_K 32 lanes x (2 x 16 B values + 8 B scales + 8 B sums)
constexpr int kQ4StepBytes = 32 * 48;
// Q8_0: 32 lanes x (16 B values + 4 B scale)
constexpr int kQ8StepBytes = 32 * 20;

// Accumulates accv[r][t] = partial (this lane's) sums of rows row0 + r (< N) against the T activation rows tok[t]
// (row indices into aq / columns of asc).  All threads of the CTA must call it together (it synchronises).
template <int T>
__device__ __forceinline__ void gemv_q4k_body(unsigned char* smem, const uint8_t* __restrict__ raw, int N, int K,
                                              const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp,
                                              const int* tok, int row0, int steps_per_chunk, float (&accv)[kRows][T]) {
  const int nsb = K >> 8, nsteps = (nsb + 3) >> 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row_bytes = (size_t)nsb * 144;
  const int piece = lane & 7, chunk64 = piece >> 1;  // 16-byte piece of the 128 nibble bytes; 64-element chunk
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) accv[r][t] = 0.0f;
  const uint8_t* rp[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) rp[r] = raw + (size_t)min(row0 + r, N - 1) * row_bytes;

  for (int s0 = 0; s0 < nsteps; s0 += steps_per_chunk) {
    const int s1 = min(nsteps, s0 + steps_per_chunk);
    // the first step's weights are requested before the activations are staged, so both latencies overlap
    uint4 hdr[kRows], qv[kRows];
    auto load = [&](int step, uint4* h, uint4* q) {
      const int sb = step * 4 + (lane >> 3);
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (sb < nsb) {
          const uint8_t* p = rp[r] + (size_t)sb * 144;
          h[r] = ldg_stream_v4(p);
          q[r] = ldg_stream_v4(p + 16 + 16 * piece);
        } else {
          h[r] = make_uint4(0, 0, 0, 0);
          q[r] = make_uint4(0, 0, 0, 0);
        }
      }
    };
    load(s0, hdr, qv);
    __syncthreads();
    // ---- stage activations of steps [s0, s1): entry (step, t, lane)
    for (int i = threadIdx.x; i < (s1 - s0) * T * 32; i += blockDim.x) {
      const int l = i & 31, t = (i >> 5) % T, st = (i >> 5) / T;
      const int sb = (s0 + st) * 4 + (l >> 3), pc = l & 7;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      float2 sc = make_float2(0.0f, 0.0f);
      int2 sm = make_int2(0, 0);
      if (sb < nsb) {
        const int e = sb * 256 + (pc >> 1) * 64 + (pc & 1) * 16;  // low-nibble elements; the high nibbles are 32 further
        lo = *reinterpret_cast<const uint4*>(aq + (size_t)tok[t] * K + e);
        hi = *reinterpret_cast<const uint4*>(aq + (size_t)tok[t] * K + e + 32);
        const int b = sb * 8 + (pc >> 1) * 2;
        sc.x = asc[(size_t)b * Mp + tok[t]];
        sc.y = asc[(size_t)(b + 1) * Mp + tok[t]];
        sm.x = __dp4a((int)lo.x, 0x01010101, __dp4a((int)lo.y, 0x01010101, __dp4a((int)lo.z, 0x01010101, __dp4a((int)lo.w, 0x01010101, 0))));
        sm.y = __dp4a((int)hi.x, 0x01010101, __dp4a((int)hi.y, 0x01010101, __dp4a((int)hi.z, 0x01010101, __dp4a((int)hi.w, 0x01010101, 0))));
      }
      unsigned char* base = smem + (size_t)(st * T + t) * kQ4StepBytes;
      reinterpret_cast<uint4*>(base)[l] = lo;
      reinterpret_cast<uint4*>(base + 512)[l] = hi;
      reinterpret_cast<float2*>(base + 1024)[l] = sc;
      reinterpret_cast<int2*>(base + 1280)[l] = sm;
    }
    __syncthreads();

    for (int step = s0; step < s1; ++step) {
      uint4 hn[kRows], qn[kRows];
      if (step + 1 < s1) load(step + 1, hn, qn);
      const unsigned char* sbase = smem + (size_t)(step - s0) * T * kQ4StepBytes;
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const float d = half_bits_to_float(hdr[r].x & 0xFFFFu), dmin = half_bits_to_float(hdr[r].x >> 16);
        const uint32_t s3[3] = {hdr[r].y, hdr[r].z, hdr[r].w};
        int sc_lo, mn_lo, sc_hi, mn_hi;
        q4k_scale_min(s3, 2 * chunk64, sc_lo, mn_lo);
        q4k_scale_min(s3, 2 * chunk64 + 1, sc_hi, mn_hi);
        const uint32_t w[4] = {qv[r].x, qv[r].y, qv[r].z, qv[r].w};
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const unsigned char* b = sbase + (size_t)t * kQ4StepBytes;
          const uint4 alo = reinterpret_cast<const uint4*>(b)[lane];
          const uint4 ahi = reinterpret_cast<const uint4*>(b + 512)[lane];
          const float2 sa = reinterpret_cast<const float2*>(b + 1024)[lane];
          const int2 as = reinterpret_cast<const int2*>(b + 1280)[lane];
          const uint32_t al[4] = {alo.x, alo.y, alo.z, alo.w}, ah[4] = {ahi.x, ahi.y, ahi.z, ahi.w};
          int lo = 0, hi = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            lo = __dp4a((int)al[k], (int)(w[k] & 0x0F0F0F0Fu), lo);
            hi = __dp4a((int)ah[k], (int)((w[k] >> 4) & 0x0F0F0F0Fu), hi);
          }
          accv[r][t] += sa.x * (d * (float)(sc_lo * lo) - dmin * (float)(mn_lo * as.x)) +
                        sa.y * (d * (float)(sc_hi * hi) - dmin * (float)(mn_hi * as.y));
        }
      }
      if (step + 1 < s1) {
#pragma unroll
        for (int r = 0; r < kRows; ++r) { hdr[r] = hn[r]; qv[r] = qn[r]; }
      }
    }
  }
}

template <int T>
__device__ __forceinline__ void gemv_q8_0_body(unsigned char* smem, const uint8_t* __restrict__ raw, int N, int K,
                                               const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp,
                                               const int* tok, int row0, int steps_per_chunk, float (&accv)[kRows][T]) {
  const int nsb = K >> 8, nsteps = (nsb + 1) >> 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row_bytes = (size_t)nsb * 272;
  const int piece = lane & 15, blk = piece >> 1;
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) accv[r][t] = 0.0f;
  const uint8_t* rp[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) rp[r] = raw + (size_t)min(row0 + r, N - 1) * row_bytes;

  for (int s0 = 0; s0 < nsteps; s0 += steps_per_chunk) {
    const int s1 = min(nsteps, s0 + steps_per_chunk);
    // the first step's weights are requested before the activations are staged, so both latencies overlap
    uint4 hdr[kRows], qv[kRows];
    auto load = [&](int step, uint4* h, uint4* q) {
      const int sb = step * 2 + (lane >> 4);
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (sb < nsb) {
          const uint8_t* p = rp[r] + (size_t)sb * 272;
          h[r] = ldg_stream_v4(p);
          q[r] = ldg_stream_v4(p + 16 + 16 * piece);
        } else {
          h[r] = make_uint4(0, 0, 0, 0);
          q[r] = make_uint4(0, 0, 0, 0);
        }
      }
    };
    load(s0, hdr, qv);
    __syncthreads();
    for (int i = threadIdx.x; i < (s1 - s0) * T * 32; i += blockDim.x) {
      const int l = i & 31, t = (i >> 5) % T, st = (i >> 5) / T;
      const int sb = (s0 + st) * 2 + (l >> 4), pc = l & 15;
      uint4 a = make_uint4(0, 0, 0, 0);
      float sc = 0.0f;
      if (sb < nsb) {
        a = *reinterpret_cast<const uint4*>(aq + (size_t)tok[t] * K + sb * 256 + pc * 16);
        sc = asc[(size_t)(sb * 8 + (pc >> 1)) * Mp + tok[t]];
      }
      unsigned char* base = smem + (size_t)(st * T + t) * kQ8StepBytes;
      reinterpret_cast<uint4*>(base)[l] = a;
      reinterpret_cast<float*>(base + 512)[l] = sc;
    }
    __syncthreads();

    for (int step = s0; step < s1; ++step) {
      uint4 hn[kRows], qn[kRows];
      if (step + 1 < s1) load(step + 1, hn, qn);
      const unsigned char* sbase = smem + (size_t)(step - s0) * T * kQ8StepBytes;
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint32_t hw[4] = {hdr[r].x, hdr[r].y, hdr[r].z, hdr[r].w};
        const uint32_t pair = hw[blk >> 1];
        const float d = half_bits_to_float((blk & 1) ? (pair >> 16) : (pair & 0xFFFFu));
        const uint32_t w[4] = {qv[r].x, qv[r].y, qv[r].z, qv[r].w};
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const unsigned char* b = sbase + (size_t)t * kQ8StepBytes;
          const uint4 a4 = reinterpret_cast<const uint4*>(b)[lane];
          const float sa = reinterpret_cast<const float*>(b + 512)[lane];
          const uint32_t a[4] = {a4.x, a4.y, a4.z, a4.w};
          int dot = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) dot = __dp4a((int)a[k], (int)w[k], dot);
          accv[r][t] += sa * d * (float)dot;
        }
      }
      if (step + 1 < s1) {
#pragma unroll
        for (int r = 0; r < kRows; ++r) { hdr[r] = hn[r]; qv[r] = qn[r]; }
      }
    }
  }
}


template <int QT, int T>
__device__ __forceinline__ void gemv_body(unsigned char* smem, const uint8_t* __restrict__ raw, int N, int K,
                                          const int8_t* __restrict__ aq, const float* __restrict__ asc, int Mp, const int* tok,
                                          int row0, int steps_per_chunk, float (&accv)[kRows][T]) {
  if (QT == IZB_Q4_K) gemv_q4k_body<T>(smem, raw, N, K, aq, asc, Mp, tok, row0, steps_per_chunk, accv);
  else gemv_q8_0_body<T>(smem, raw, N, K, aq, asc, Mp, tok, row0, steps_per_chunk, accv);
}

constexpr int kMaxSmem = 96 * 1024;
// K-steps staged per pass and the dynamic shared memory that takes
inline int steps_per_chunk(int type, int K, int T, size_t* smem) {
  const int nsb = K / 256;
  const int nsteps = type == IZB_Q4_K ? (nsb + 3) / 4 : (nsb + 1) / 2;
  const int sb = type == IZB_Q4_K ? kQ4StepBytes : kQ8StepBytes;
  int spc = kMaxSmem / (T * sb);
  if (spc > nsteps) spc = nsteps;
  *smem = (size_t)spc * T * sb;
  return spc;
}
}  // namespace izb_gemvk
