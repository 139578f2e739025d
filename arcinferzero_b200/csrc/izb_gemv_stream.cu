// Streaming decode GEMV (1..8 activation rows): the kernel izb_gemv uses whenever its shared-memory plan fits.
// Same arithmetic as izb_gemv_body.cuh (zero/kernels/decode.cl:913-1034, :1581-1694); different data movement.
//
// A decode matrix streams in a few microseconds at HBM speed, so what decides the achieved bandwidth is how many weight
// bytes are in flight from the first cycle to the last, not the arithmetic.  Registers cannot hold enough, shared
// memory can:
//   * one persistent CTA of 16 warps per SM; warp w of the grid owns weight rows w, w + W, w + 2W, ... (W = warps in the
//     grid), so every SM holds the same share of every part of the matrix;
//   * every warp has its own ring of kSlots row buffers in shared memory, filled by the TMA engine (cp.async.bulk, one
//     copy per weight row: a row of K/256 superblocks is contiguous and a multiple of 16 bytes) and tracked by one
//     mbarrier per slot: all its rows (~190 KB) are in flight per SM at any time, across row boundaries;
//   * the first ring fill is issued before the CTA stages the activation rows, so the two latencies overlap.
// Per lane and step: Q4_K lane = (superblock lane/8 of the step's four, 16-byte nibble piece lane%8);
//                    Q8_0 lane = (superblock lane/16 of the step's two, 16-byte piece lane%16).
// Waits are bounded; a wait that gives up sets the device error word and the warp stops (izb_device_status).
#include "izb_gemv_body.cuh"

namespace {
using namespace izb_gemvk;

constexpr uint32_t kSpin = 1u << 24;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void row_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar) : "memory");
}

// warps per CTA (32 with half the ring slots measured slower for every shape but one)
template <int T> __host__ __device__ constexpr int stream_warps() { return 16; }

template <int QT, int T>
__global__ void __launch_bounds__(stream_warps<T>() * 32, 1) gemv_stream_kernel(const uint8_t* __restrict__ raw, int N, int K,
                                                                      const int8_t* __restrict__ aq, const float* __restrict__ asc,
                                                                      int Mp, float* __restrict__ C, int ldc, int c_off, int acc,
                                                                      int slots, int slot_bytes, uint32_t* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int SBS = QT == IZB_Q4_K ? 4 : 2;  // superblocks per step
  constexpr int SBB = QT == IZB_Q4_K ? 144 : 272;
  constexpr int STEP = QT == IZB_Q4_K ? kQ4StepBytes : kQ8StepBytes;
  constexpr int kSWarps = stream_warps<T>();
  const int nsb = K >> 8, nsteps = (nsb + SBS - 1) / SBS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int W = gridDim.x * kSWarps, w0 = blockIdx.x * kSWarps + warp;
  const uint32_t row_bytes = (uint32_t)nsb * SBB;
  const int my_rows = w0 < N ? (N - w0 + W - 1) / W : 0;
  const int sub = QT == IZB_Q4_K ? lane >> 3 : lane >> 4;   // superblock of the step
  const int piece = QT == IZB_Q4_K ? lane & 7 : lane & 15;  // 16-byte piece of its quants
  // shared memory: [activation staging: nsteps * T * STEP][16 warps x slots x slot_bytes][16 x slots mbarriers]
  unsigned char* act = smem;
  unsigned char* ring = smem + (((size_t)nsteps * T * STEP + 127) & ~(size_t)127) + (size_t)warp * slots * slot_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (((size_t)nsteps * T * STEP + 127) & ~(size_t)127) +
                                               (size_t)kSWarps * slots * slot_bytes) + warp * slots;
  if (lane == 0) {
    for (int s = 0; s < slots; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int s = 0; s < slots && s < my_rows; ++s)
      row_copy(s_u32(ring + (size_t)s * slot_bytes), raw + (size_t)(w0 + s * W) * row_bytes, row_bytes, s_u32(&bars[s]));
  }
  // ---- stage the T activation rows for all steps: entry (step, t, lane), laid out as in izb_gemv_body.cuh
  for (int i = threadIdx.x; i < nsteps * T * 32; i += blockDim.x) {
    const int l = i & 31, t = (i >> 5) % T, st = (i >> 5) / T;
    unsigned char* base = act + (size_t)(st * T + t) * STEP;
    if (QT == IZB_Q4_K) {
      const int sb = st * 4 + (l >> 3), pc = l & 7;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      float2 sc = make_float2(0.0f, 0.0f);
      int2 sm = make_int2(0, 0);
      if (sb < nsb) {
        const int e = sb * 256 + (pc >> 1) * 64 + (pc & 1) * 16;
        lo = *reinterpret_cast<const uint4*>(aq + (size_t)t * K + e);
        hi = *reinterpret_cast<const uint4*>(aq + (size_t)t * K + e + 32);
        const int b = sb * 8 + (pc >> 1) * 2;
        sc.x = asc[(size_t)b * Mp + t];
        sc.y = asc[(size_t)(b + 1) * Mp + t];
        sm.x = __dp4a((int)lo.x, 0x01010101, __dp4a((int)lo.y, 0x01010101, __dp4a((int)lo.z, 0x01010101, __dp4a((int)lo.w, 0x01010101, 0))));
        sm.y = __dp4a((int)hi.x, 0x01010101, __dp4a((int)hi.y, 0x01010101, __dp4a((int)hi.z, 0x01010101, __dp4a((int)hi.w, 0x01010101, 0))));
      }
      reinterpret_cast<uint4*>(base)[l] = lo;
      reinterpret_cast<uint4*>(base + 512)[l] = hi;
      reinterpret_cast<float2*>(base + 1024)[l] = sc;
      reinterpret_cast<int2*>(base + 1280)[l] = sm;
    } else {
      const int sb = st * 2 + (l >> 4), pc = l & 15;
      uint4 a = make_uint4(0, 0, 0, 0);
      float sc = 0.0f;
      if (sb < nsb) {
        a = *reinterpret_cast<const uint4*>(aq + (size_t)t * K + sb * 256 + pc * 16);
        sc = asc[(size_t)(sb * 8 + (pc >> 1)) * Mp + t];
      }
      reinterpret_cast<uint4*>(base)[l] = a;
      reinterpret_cast<float*>(base + 512)[l] = sc;
    }
  }
  __syncthreads();

  int slot = 0;
  uint32_t parity = 0;
  for (int i = 0; i < my_rows; ++i) {
    const int row = w0 + i * W;
    bool ready = false;
    for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[slot]), parity);
    if (!ready) {  // (bounded wait gave up)
      if (lane == 0) atomicOr(err, 64u);
      break;
    }
    const unsigned char* wrow = ring + (size_t)slot * slot_bytes;
    float accv[T];
#pragma unroll
    for (int t = 0; t < T; ++t) accv[t] = 0.0f;
    for (int step = 0; step < nsteps; ++step) {
      const int sb = step * SBS + sub;
      if (sb < nsb) {
        const uint4 h = *reinterpret_cast<const uint4*>(wrow + sb * SBB);
        const uint4 qw = *reinterpret_cast<const uint4*>(wrow + sb * SBB + 16 + 16 * piece);
        const unsigned char* sbase = act + (size_t)step * T * STEP;
        const uint32_t w[4] = {qw.x, qw.y, qw.z, qw.w};
        if (QT == IZB_Q4_K) {
          const float d = half_bits_to_float(h.x & 0xFFFFu), dmin = half_bits_to_float(h.x >> 16);
          const uint32_t s3[3] = {h.y, h.z, h.w};
          int sc_lo, mn_lo, sc_hi, mn_hi;
          q4k_scale_min(s3, 2 * (piece >> 1), sc_lo, mn_lo);
          q4k_scale_min(s3, 2 * (piece >> 1) + 1, sc_hi, mn_hi);
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const unsigned char* b = sbase + (size_t)t * STEP;
            const uint4 alo = reinterpret_cast<const uint4*>(b)[lane];
            const uint4 ahi = reinterpret_cast<const uint4*>(b + 512)[lane];
            const float2 sa = reinterpret_cast<const float2*>(b + 1024)[lane];
            const int2 as = reinterpret_cast<const int2*>(b + 1280)[lane];
            const uint32_t al[4] = {alo.x, alo.y, alo.z, alo.w}, ah[4] = {ahi.x, ahi.y, ahi.z, ahi.w};
            int lo = 0, hi = 0;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              lo = __dp4a((int)al[kk], (int)(w[kk] & 0x0F0F0F0Fu), lo);
              hi = __dp4a((int)ah[kk], (int)((w[kk] >> 4) & 0x0F0F0F0Fu), hi);
            }
            accv[t] += sa.x * (d * (float)(sc_lo * lo) - dmin * (float)(mn_lo * as.x)) +
                       sa.y * (d * (float)(sc_hi * hi) - dmin * (float)(mn_hi * as.y));
          }
        } else {
          const int blk = piece >> 1;
          const uint32_t pair = blk < 2 ? h.x : blk < 4 ? h.y : blk < 6 ? h.z : h.w;
          const float d = half_bits_to_float((blk & 1) ? (pair >> 16) : (pair & 0xFFFFu));
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const unsigned char* b = sbase + (size_t)t * STEP;
            const uint4 a4 = reinterpret_cast<const uint4*>(b)[lane];
            const float sa = reinterpret_cast<const float*>(b + 512)[lane];
            const uint32_t a[4] = {a4.x, a4.y, a4.z, a4.w};
            int dot = 0;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) dot = __dp4a((int)a[kk], (int)w[kk], dot);
            accv[t] += sa * d * (float)dot;
          }
        }
      }
    }
    // the slot is read: request the row `slots` ahead into it, then reduce and store this one
    __syncwarp();
    if (lane == 0 && i + slots < my_rows)
      row_copy(s_u32(ring + (size_t)slot * slot_bytes), raw + (size_t)(row + slots * W) * row_bytes, row_bytes, s_u32(&bars[slot]));
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(accv[t]);
      if (lane == 0) {
        float* c = C + (size_t)t * ldc + c_off + row;
        *c = acc ? *c + v : v;
      }
    }
    if (++slot == slots) { slot = 0; parity ^= 1; }
  }
}


// ---------------------------------------------------------------------------------------------- Q4_K, one activation row
// The decode case proper (batch 1, K a multiple of 1024 up to 5120).  Same ring of TMA-filled row buffers per warp, but
//   * a lane owns one pair of 32-blocks (32 bytes of nibbles) of one of the eight superblocks of a step, so the superblock
//     header is decoded by four lanes, not eight, and it meets the same activation bytes in every weight row: it keeps
//     them -- 64 int8 values, two block scales and the two scaled block sums per step -- in registers for the whole
//     kernel: nothing is staged in shared memory and the CTA never synchronises;
//   * a warp works on two weight rows at a time, so that two independent dependency chains hide each other's latencies
//     and the per-row bookkeeping (waits, re-arming the copies, the warp reduction) is paid once per pair;
//   * the pair of 6-bit (scale, min) values a lane needs is unpacked without branches (q4k_pair).
// Per 32-block: acc += d * (asc * (float)(sc * dot)) - dmin * ((asc * (float)asum) * (float)mn), the factors that depend
// only on the activations precomputed.

// Q4_K: the 6-bit (scale, min) values of sub-blocks 2*pp and 2*pp + 1 (pp = 0..3) as two bytes each.  Sub-blocks 0..3
// keep their values in the low six bits of bytes 0..7; sub-blocks 4..7 have the low four bits in bytes 8..11 and the high
// two in the top bits of bytes 0..7 (get_scale_min_k4, src/quants.h:61-69).
__device__ __forceinline__ void q4k_pair(const uint4 h, int sh, bool upper, uint32_t& sc2, uint32_t& mn2) {
  const uint32_t a = h.y >> sh, b = h.z >> sh, c = h.w >> sh;
  sc2 = upper ? ((c & 0x0F0Fu) | ((a >> 2) & 0x3030u)) : (a & 0x3F3Fu);
  mn2 = upper ? (((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u)) : (b & 0x3F3Fu);
}

// signed x unsigned byte dot product
__device__ __forceinline__ int dp4a_su(int a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Two CTAs of eight warps per SM rather than one of sixteen: with programmatic dependent launch the next kernel's CTAs
// move in, and start their first ring fill, as soon as half an SM is free.
constexpr int kRegWarps = 8;

template <int NSB4>  // K / 1024
__global__ void __launch_bounds__(kRegWarps * 32, 2) gemv_q4k_reg_kernel(const uint8_t* __restrict__ raw, int N,
                                                                         const int8_t* __restrict__ aq, const float* __restrict__ asc,
                                                                         int Mp, float* __restrict__ C, int c_off, int acc,
                                                                         int slots, int slot_bytes, uint32_t* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int nsb = 4 * NSB4, WS = (nsb + 7) / 8, FS = nsb / 8;  // steps of eight superblocks: FS full ones, and for an odd
  constexpr bool kHalf = (nsb % 8) != 0;                            // K / 1024 a last step of four
  // The half step does not leave half the warp idle: when a warp works on two rows, lanes 0..15 take the last four
  // superblocks of the first row and lanes 16..31 those of the second, so a pair of rows costs 2 FS + 1 steps.
  constexpr uint32_t row_bytes = nsb * 144;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int W = gridDim.x * kRegWarps, w0 = blockIdx.x * kRegWarps + warp;
  const int my_rows = w0 < N ? (N - w0 + W - 1) / W : 0;
  const int sub = lane >> 2, pp = lane & 3;  // superblock of the step, pair of 32-blocks (2 pp, 2 pp + 1) inside it
  unsigned char* ring = smem + (size_t)warp * slots * slot_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kRegWarps * slots * slot_bytes) + warp * slots;
  if (lane == 0) {
    for (int s = 0; s < slots; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int s = 0; s < slots && s < my_rows; ++s)
      row_copy(s_u32(ring + (size_t)s * slot_bytes), raw + (size_t)(w0 + s * W) * row_bytes, row_bytes, s_u32(&bars[s]));
  }
  __syncwarp();
  // Programmatic dependent launch: the weights do not depend on the kernel before this one in the stream, so the ring
  // fill above may run while that kernel drains; its results (the activations, and C when accumulating) are read only
  // after griddepcontrol.wait.  launch_dependents lets the next kernel of the stream do the same with this one.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // ---- this lane's activations: per step the 2 x 32 int8 values of its block pair, the two block scales (the second one
  // divided by 16, see below) and the two scaled block sums
  uint4 alo[WS][2], ahi[WS][2];
  float sx[WS], sy16[WS], px[WS], py[WS];
#pragma unroll
  for (int st = 0; st < WS; ++st) {
    const int sb = st < FS ? st * 8 + sub : st * 8 + (sub & 3);  // (the half step: both half warps hold the same four)
    {
      const int8_t* a = aq + sb * 256 + pp * 64;
      alo[st][0] = *reinterpret_cast<const uint4*>(a);
      alo[st][1] = *reinterpret_cast<const uint4*>(a + 16);
      ahi[st][0] = *reinterpret_cast<const uint4*>(a + 32);
      ahi[st][1] = *reinterpret_cast<const uint4*>(a + 48);
      const int b = sb * 8 + pp * 2;
      const float s0 = asc[(size_t)b * Mp], s1 = asc[(size_t)(b + 1) * Mp];
      const uint32_t l[8] = {alo[st][0].x, alo[st][0].y, alo[st][0].z, alo[st][0].w, alo[st][1].x, alo[st][1].y, alo[st][1].z, alo[st][1].w};
      const uint32_t g[8] = {ahi[st][0].x, ahi[st][0].y, ahi[st][0].z, ahi[st][0].w, ahi[st][1].x, ahi[st][1].y, ahi[st][1].z, ahi[st][1].w};
      int sl = 0, sh = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        sl = __dp4a((int)l[k], 0x01010101, sl);
        sh = __dp4a((int)g[k], 0x01010101, sh);
      }
      sx[st] = s0;
      sy16[st] = s1 * 0.0625f;
      px[st] = s0 * (float)sl;
      py[st] = s1 * (float)sh;
    }
  }
  const int pp_sh = 16 * (pp & 1);  // where this lane's pair of sub-block scales sits in the packed words
  const bool pp_upper = pp >= 2;
  const uint32_t h_off = sub * 144, q_off = sub * 144 + 16 + 32 * pp;
  const uint32_t h_off_half = (sub & 3) * 144, q_off_half = (sub & 3) * 144 + 16 + 32 * pp;

  int slot = 0;
  uint32_t parity = 0;
  for (int i = 0; i < my_rows; i += 2) {
    const bool two = i + 1 < my_rows;  // (uniform over the warp)
    bool ready = false;
    for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[slot]), parity);
    if (ready && two) {
      ready = false;
      for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[slot + 1]), parity);
    }
    if (!ready) {  // (bounded wait gave up)
      if (lane == 0) atomicOr(err, 64u);
      break;
    }
    const unsigned char* w0p = ring + (size_t)slot * slot_bytes;
    const unsigned char* w1p = two ? w0p + slot_bytes : w0p;  // (a lone last row is computed twice, stored once)
    float acc0 = 0.0f, acc1 = 0.0f;
    auto one = [&](int st, const unsigned char* wp, uint32_t ho, uint32_t qo, float accv) -> float {
      const uint32_t al[8] = {alo[st][0].x, alo[st][0].y, alo[st][0].z, alo[st][0].w, alo[st][1].x, alo[st][1].y, alo[st][1].z, alo[st][1].w};
      const uint32_t ah[8] = {ahi[st][0].x, ahi[st][0].y, ahi[st][0].z, ahi[st][0].w, ahi[st][1].x, ahi[st][1].y, ahi[st][1].z, ahi[st][1].w};
      const uint4 h = *reinterpret_cast<const uint4*>(wp + st * 1152 + ho);
      const uint4 qa = *reinterpret_cast<const uint4*>(wp + st * 1152 + qo);
      const uint4 qb = *reinterpret_cast<const uint4*>(wp + st * 1152 + qo + 16);
      const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&h.x));  // (d, dmin)
      uint32_t sc2, mn2;
      q4k_pair(h, pp_sh, pp_upper, sc2, mn2);
      const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      // low nibbles against the first block; the high nibbles stay where they are, as unsigned bytes 16 * q, against
      // the second block: hi = 16 * dot, and the factor 1/16 sits in the activation scale
      int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        lo0 = __dp4a((int)al[kk], (int)(w[kk] & 0x0F0F0F0Fu), lo0);
        lo1 = __dp4a((int)al[4 + kk], (int)(w[4 + kk] & 0x0F0F0F0Fu), lo1);
        hi0 = dp4a_su((int)ah[kk], w[kk] & 0xF0F0F0F0u, hi0);
        hi1 = dp4a_su((int)ah[4 + kk], w[4 + kk] & 0xF0F0F0F0u, hi1);
      }
      const float tq = fmaf(sx[st], (float)((int)(sc2 & 0xFFu) * (lo0 + lo1)), sy16[st] * (float)((int)(sc2 >> 8) * (hi0 + hi1)));
      const float tm = fmaf(px[st], (float)(mn2 & 0xFFu), py[st] * (float)(mn2 >> 8));
      return fmaf(df.x, tq, fmaf(-df.y, tm, accv));
    };
#pragma unroll
    for (int st = 0; st < FS; ++st) {
      acc0 = one(st, w0p, h_off, q_off, acc0);
      acc1 = one(st, w1p, h_off, q_off, acc1);
    }
    if (kHalf) {  // (for a lone last row w1p == w0p: lanes 16..31 repeat the work and their sum is dropped)
      const float r = one(FS, lane < 16 ? w0p : w1p, h_off_half, q_off_half, 0.0f);
      acc0 += lane < 16 ? r : 0.0f;
      acc1 += lane < 16 ? 0.0f : r;
    }
    // the slots are read: request the rows `slots` ahead into them, then reduce and store
    __syncwarp();
    const int row = w0 + i * W;
    if (lane == 0) {
      if (i + slots < my_rows)
        row_copy(s_u32(ring + (size_t)slot * slot_bytes), raw + (size_t)(row + slots * W) * row_bytes, row_bytes, s_u32(&bars[slot]));
      if (i + 1 + slots < my_rows)
        row_copy(s_u32(ring + (size_t)(slot + 1) * slot_bytes), raw + (size_t)(row + (slots + 1) * W) * row_bytes, row_bytes, s_u32(&bars[slot + 1]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, o);
      acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, o);
    }
    if (lane < 2 && (lane == 0 || two)) {
      float* c = C + c_off + row + lane * W;
      const float v = lane ? acc1 : acc0;
      *c = acc ? *c + v : v;
    }
    slot += 2;
    if (slot >= slots) { slot = 0; parity ^= 1; }
  }
}

template <int NSTEPS>
int launch_q4k_reg(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int c_off, int acc,
                   cudaStream_t st) {
  constexpr size_t kBudget = 100 * 1024;  // per CTA, two CTAs per SM
  const int slot_bytes = (int)((w->row_bytes + 127) & ~(size_t)127);
  int slots = (int)((kBudget - 4096) / ((size_t)kRegWarps * slot_bytes));
  slots = slots > 8 ? 8 : (slots & ~1);  // rows are taken two at a time
  if (slots < 2) return 1;
  const size_t smem = (size_t)kRegWarps * slots * slot_bytes + (size_t)kRegWarps * slots * 8;
  IZB_SMEM_OPTIN((gemv_q4k_reg_kernel<NSTEPS>), kBudget + 8192, w->device);
  const int sms = izb_sm_count(w->device);
  int grid = 2 * sms;
  const int need = (w->N + kRegWarps - 1) / kRegWarps;
  if (grid > need) grid = need;
  uint32_t* err = izb_device_error_word(w->device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "gemv: no device error word");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kRegWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int N = w->N;
  IZB_LAUNCH("gemv", st, cudaLaunchKernelEx(&cfg, gemv_q4k_reg_kernel<NSTEPS>, raw, N, aq, asc, Mp, C, c_off, acc, slots, slot_bytes, err));
  return IZB_OK;
}

// ---------------------------------------------------------------------------------------------- Q4_K, 2..4 activation rows
// The same lane mapping, row pairs and ring as gemv_q4k_reg_kernel, for a few activation rows: their bytes do not fit
// the registers, so each CTA stages them once in shared memory in the per-lane form the loop reads (per step and
// token: four 16-byte pieces, the two block scales -- the second one / 16 -- and the two scaled block sums per lane).
// A weight row's nibbles are masked once and multiplied into every token's accumulators.
constexpr int kPairWarps = 16;
constexpr int kPairActBytes = 4 * 512 + 4 * 128;  // per (step, token)

template <int NSB4, int T>
__global__ void __launch_bounds__(kPairWarps * 32, 1) gemv_q4k_pair_kernel(const uint8_t* __restrict__ raw, int N,
                                                                          const int8_t* __restrict__ aq, const float* __restrict__ asc,
                                                                          int Mp, float* __restrict__ C, int ldc, int c_off, int acc,
                                                                          int slots, int slot_bytes, uint32_t* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int nsb = 4 * NSB4, WS = (nsb + 7) / 8, FS = nsb / 8, K = nsb * 256;
  constexpr bool kHalf = (nsb % 8) != 0;  // a last step of four superblocks: shared by the two rows of a pair (half a warp each)
  constexpr uint32_t row_bytes = nsb * 144;
  constexpr int kActBytes = WS * T * kPairActBytes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int W = gridDim.x * kPairWarps, w0 = blockIdx.x * kPairWarps + warp;
  const int my_rows = w0 < N ? (N - w0 + W - 1) / W : 0;
  const int sub = lane >> 2, pp = lane & 3;
  unsigned char* act = smem;
  unsigned char* ring = smem + kActBytes + (size_t)warp * slots * slot_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kActBytes + (size_t)kPairWarps * slots * slot_bytes) + warp * slots;
  if (lane == 0) {
    for (int s = 0; s < slots; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int s = 0; s < slots && s < my_rows; ++s)
      row_copy(s_u32(ring + (size_t)s * slot_bytes), raw + (size_t)(w0 + s * W) * row_bytes, row_bytes, s_u32(&bars[s]));
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // (see gemv_q4k_reg_kernel: the ring fill above runs ahead of it)
  // ---- stage the activations: entry (step, token, lane)
  for (int i = threadIdx.x; i < WS * T * 32; i += blockDim.x) {
    const int l = i & 31, t = (i >> 5) % T, st = (i >> 5) / T;
    const int sb = st < FS ? st * 8 + (l >> 2) : st * 8 + ((l >> 2) & 3), p2 = l & 3;
    uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0, a2 = a0, a3 = a0;
    float4 sc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (sb < nsb) {
      const int8_t* a = aq + (size_t)t * K + sb * 256 + p2 * 64;
      a0 = *reinterpret_cast<const uint4*>(a);
      a1 = *reinterpret_cast<const uint4*>(a + 16);
      a2 = *reinterpret_cast<const uint4*>(a + 32);
      a3 = *reinterpret_cast<const uint4*>(a + 48);
      const int b = sb * 8 + p2 * 2;
      const float s0 = asc[(size_t)b * Mp + t], s1 = asc[(size_t)(b + 1) * Mp + t];
      const uint32_t lw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, hw[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
      int sl = 0, sh = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        sl = __dp4a((int)lw[k], 0x01010101, sl);
        sh = __dp4a((int)hw[k], 0x01010101, sh);
      }
      sc = make_float4(s0, s1 * 0.0625f, s0 * (float)sl, s1 * (float)sh);
    }
    unsigned char* base = act + (size_t)(st * T + t) * kPairActBytes;
    reinterpret_cast<uint4*>(base)[l] = a0;
    reinterpret_cast<uint4*>(base + 512)[l] = a1;
    reinterpret_cast<uint4*>(base + 1024)[l] = a2;
    reinterpret_cast<uint4*>(base + 1536)[l] = a3;
    reinterpret_cast<float4*>(base + 2048)[l] = sc;
  }
  __syncthreads();
  const int pp_sh = 16 * (pp & 1);
  const bool pp_upper = pp >= 2;
  const uint32_t h_off = sub * 144, q_off = sub * 144 + 16 + 32 * pp;
  const uint32_t h_off_half = (sub & 3) * 144, q_off_half = (sub & 3) * 144 + 16 + 32 * pp;

  int slot = 0;
  uint32_t parity = 0;
  for (int i = 0; i < my_rows; i += 2) {
    const bool two = i + 1 < my_rows;  // (uniform over the warp)
    bool ready = false;
    for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[slot]), parity);
    if (ready && two) {
      ready = false;
      for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[slot + 1]), parity);
    }
    if (!ready) {  // (bounded wait gave up)
      if (lane == 0) atomicOr(err, 64u);
      break;
    }
    const unsigned char* wp[2] = {ring + (size_t)slot * slot_bytes, ring + (size_t)(two ? slot + 1 : slot) * slot_bytes};
    float accv[2][T];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) accv[r][t] = 0.0f;
#pragma unroll
    for (int st = 0; st < FS; ++st) {
      {
        uint32_t wl[2][8], wh[2][8], sc2[2], mn2[2];
        float2 df[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint4 h = *reinterpret_cast<const uint4*>(wp[r] + st * 1152 + h_off);
          const uint4 qa = *reinterpret_cast<const uint4*>(wp[r] + st * 1152 + q_off);
          const uint4 qb = *reinterpret_cast<const uint4*>(wp[r] + st * 1152 + q_off + 16);
          df[r] = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
          q4k_pair(h, pp_sh, pp_upper, sc2[r], mn2[r]);
          const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            wl[r][kk] = w[kk] & 0x0F0F0F0Fu;
            wh[r][kk] = w[kk] & 0xF0F0F0F0u;
          }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const unsigned char* base = act + (size_t)(st * T + t) * kPairActBytes;
          const uint4 a0 = reinterpret_cast<const uint4*>(base)[lane], a1 = reinterpret_cast<const uint4*>(base + 512)[lane];
          const uint4 a2 = reinterpret_cast<const uint4*>(base + 1024)[lane], a3 = reinterpret_cast<const uint4*>(base + 1536)[lane];
          const float4 sc = reinterpret_cast<const float4*>(base + 2048)[lane];  // (s0, s1/16, s0*sum0, s1*sum1)
          const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              lo0 = __dp4a((int)al[kk], (int)wl[r][kk], lo0);
              lo1 = __dp4a((int)al[4 + kk], (int)wl[r][4 + kk], lo1);
              hi0 = dp4a_su((int)ah[kk], wh[r][kk], hi0);
              hi1 = dp4a_su((int)ah[4 + kk], wh[r][4 + kk], hi1);
            }
            const float tq = fmaf(sc.x, (float)((int)(sc2[r] & 0xFFu) * (lo0 + lo1)), sc.y * (float)((int)(sc2[r] >> 8) * (hi0 + hi1)));
            const float tm = fmaf(sc.z, (float)(mn2[r] & 0xFFu), sc.w * (float)(mn2[r] >> 8));
            accv[r][t] = fmaf(df[r].x, tq, fmaf(-df[r].y, tm, accv[r][t]));
          }
        }
      }
    }
    if (kHalf) {  // lanes 0..15: the first row's last four superblocks, lanes 16..31: the second row's
      const unsigned char* wph = lane < 16 ? wp[0] : wp[1];
      const uint4 h = *reinterpret_cast<const uint4*>(wph + FS * 1152 + h_off_half);
      const uint4 qa = *reinterpret_cast<const uint4*>(wph + FS * 1152 + q_off_half);
      const uint4 qb = *reinterpret_cast<const uint4*>(wph + FS * 1152 + q_off_half + 16);
      const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
      uint32_t sc2, mn2;
      q4k_pair(h, pp_sh, pp_upper, sc2, mn2);
      const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      uint32_t wl[8], wh[8];
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        wl[kk] = w[kk] & 0x0F0F0F0Fu;
        wh[kk] = w[kk] & 0xF0F0F0F0u;
      }
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const unsigned char* base = act + (size_t)(FS * T + t) * kPairActBytes;
        const uint4 a0 = reinterpret_cast<const uint4*>(base)[lane], a1 = reinterpret_cast<const uint4*>(base + 512)[lane];
        const uint4 a2 = reinterpret_cast<const uint4*>(base + 1024)[lane], a3 = reinterpret_cast<const uint4*>(base + 1536)[lane];
        const float4 sc = reinterpret_cast<const float4*>(base + 2048)[lane];
        const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
        int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          lo0 = __dp4a((int)al[kk], (int)wl[kk], lo0);
          lo1 = __dp4a((int)al[4 + kk], (int)wl[4 + kk], lo1);
          hi0 = dp4a_su((int)ah[kk], wh[kk], hi0);
          hi1 = dp4a_su((int)ah[4 + kk], wh[4 + kk], hi1);
        }
        const float tq = fmaf(sc.x, (float)((int)(sc2 & 0xFFu) * (lo0 + lo1)), sc.y * (float)((int)(sc2 >> 8) * (hi0 + hi1)));
        const float tm = fmaf(sc.z, (float)(mn2 & 0xFFu), sc.w * (float)(mn2 >> 8));
        const float r = fmaf(df.x, tq, -df.y * tm);
        accv[0][t] += lane < 16 ? r : 0.0f;
        accv[1][t] += lane < 16 ? 0.0f : r;
      }
    }
    __syncwarp();
    const int row = w0 + i * W;
    if (lane == 0) {
      if (i + slots < my_rows)
        row_copy(s_u32(ring + (size_t)slot * slot_bytes), raw + (size_t)(row + slots * W) * row_bytes, row_bytes, s_u32(&bars[slot]));
      if (i + 1 + slots < my_rows)
        row_copy(s_u32(ring + (size_t)(slot + 1) * slot_bytes), raw + (size_t)(row + (slots + 1) * W) * row_bytes, row_bytes, s_u32(&bars[slot + 1]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float v = warp_sum(accv[r][t]);
        if (lane == 0 && (r == 0 || two)) {
          float* c = C + (size_t)t * ldc + c_off + row + r * W;
          *c = acc ? *c + v : v;
        }
      }
    slot += 2;
    if (slot >= slots) { slot = 0; parity ^= 1; }
  }
}

template <int NSB4, int T>
int launch_q4k_pair(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc, int c_off,
                    int acc, cudaStream_t st) {
  constexpr size_t kBudget = 216 * 1024;
  constexpr int WS = (4 * NSB4 + 7) / 8;
  const size_t act = (size_t)WS * T * kPairActBytes;
  const int slot_bytes = (int)((w->row_bytes + 127) & ~(size_t)127);
  int slots = (int)((kBudget - act - 4096) / ((size_t)kPairWarps * slot_bytes));
  slots = slots > 8 ? 8 : (slots & ~1);
  if (slots < 2) return 1;
  const size_t smem = act + (size_t)kPairWarps * slots * slot_bytes + (size_t)kPairWarps * slots * 8;
  IZB_SMEM_OPTIN((gemv_q4k_pair_kernel<NSB4, T>), kBudget + 8192, w->device);
  const int sms = izb_sm_count(w->device);
  int grid = sms;
  const int need = (w->N + kPairWarps - 1) / kPairWarps;
  if (grid > need) grid = need;
  uint32_t* err = izb_device_error_word(w->device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "gemv: no device error word");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kPairWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int N = w->N;
  IZB_LAUNCH("gemv", st, cudaLaunchKernelEx(&cfg, gemv_q4k_pair_kernel<NSB4, T>, raw, N, aq, asc, Mp, C, ldc, c_off, acc, slots, slot_bytes, err));
  return IZB_OK;
}

template <int T>
int launch_q4k_pair_k(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc, int c_off,
                      int acc, cudaStream_t st) {
  switch (w->K / 1024) {
    case 1: return launch_q4k_pair<1, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 2: return launch_q4k_pair<2, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 3: return launch_q4k_pair<3, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 4: return launch_q4k_pair<4, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    default: return launch_q4k_pair<5, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
  }
}

// ---------------------------------------------------------------------------------------------- Q4_K, long rows (K > 5120)
// A row of a down projection (K = 17408: 9.8 KB) is too long for a ring of whole rows per warp, and such matrices have few
// rows per warp (5120 rows over 2368 warps), so rows are not paired either.  Here the ring holds chunks of eight
// superblocks (1152 B, one step of the lane mapping of gemv_q4k_pair_kernel) and a warp takes two consecutive chunks of
// ONE row per pass (two independent dependency chains), its rows one after the other; the copies of the chunks
// `slots / 2` passes ahead are in flight, across row boundaries.  K = 1024 * odd ends in a chunk of four superblocks
// (lanes 16..31 repeat lanes 0..15 there and are dropped).  Activations staged per lane in shared memory (1..4 rows).
constexpr int kChunkBytes = 8 * 144;

template <int T>
__global__ void __launch_bounds__(kPairWarps * 32, 1) gemv_q4k_chunk_kernel(const uint8_t* __restrict__ raw, int N, int K,
                                                                           const int8_t* __restrict__ aq, const float* __restrict__ asc,
                                                                           int Mp, float* __restrict__ C, int ldc, int c_off, int acc,
                                                                           int slots, uint32_t* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int nsb = K >> 8, FS = nsb >> 3, WS = (nsb + 7) >> 3;  // chunks per row: FS whole ones (+ one of four superblocks)
  const int PP = (WS + 1) >> 1;                                 // passes per row (two chunks each, the last maybe one)
  const uint32_t row_bytes = (uint32_t)nsb * 144;
  const int act_bytes = WS * T * kPairActBytes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int W = gridDim.x * kPairWarps, w0 = blockIdx.x * kPairWarps + warp;
  const int my_rows = w0 < N ? (N - w0 + W - 1) / W : 0;
  const int total = my_rows * PP;  // passes of this warp, in order (row, pass)
  const int sub = lane >> 2, pp = lane & 3, hs = slots >> 1;
  unsigned char* act = smem;
  unsigned char* ring = smem + act_bytes + (size_t)warp * slots * kChunkBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + act_bytes + (size_t)kPairWarps * slots * kChunkBytes) + warp * slots;
  // pass n -> copies of chunks 2 * (n % PP), + 1 of row n / PP into slots 2 * (n % hs), + 1
  auto issue = [&](int n) {
    const int ri = n / PP, c0 = 2 * (n - ri * PP), q = n % hs;
    const uint8_t* src = raw + (size_t)(w0 + ri * W) * row_bytes + (size_t)c0 * kChunkBytes;
    row_copy(s_u32(ring + (size_t)(2 * q) * kChunkBytes), src, c0 < FS ? kChunkBytes : kChunkBytes / 2, s_u32(&bars[2 * q]));
    if (c0 + 1 < WS)
      row_copy(s_u32(ring + (size_t)(2 * q + 1) * kChunkBytes), src + kChunkBytes, c0 + 1 < FS ? kChunkBytes : kChunkBytes / 2, s_u32(&bars[2 * q + 1]));
    else  // (no second chunk in this pass: the slot's barrier still completes its phase, so that its parity keeps step)
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_u32(&bars[2 * q + 1])) : "memory");
  };
  if (lane == 0) {
    for (int s = 0; s < slots; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(&bars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int n = 0; n < hs && n < total; ++n) issue(n);
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // (see gemv_q4k_reg_kernel: the ring fill above runs ahead of it)
  for (int i = threadIdx.x; i < WS * T * 32; i += blockDim.x) {
    const int l = i & 31, t = (i >> 5) % T, st = (i >> 5) / T;
    const int sb = st < FS ? st * 8 + (l >> 2) : st * 8 + ((l >> 2) & 3), p2 = l & 3;
    const int8_t* a = aq + (size_t)t * K + sb * 256 + p2 * 64;
    const uint4 a0 = *reinterpret_cast<const uint4*>(a), a1 = *reinterpret_cast<const uint4*>(a + 16);
    const uint4 a2 = *reinterpret_cast<const uint4*>(a + 32), a3 = *reinterpret_cast<const uint4*>(a + 48);
    const int b = sb * 8 + p2 * 2;
    const float s0 = asc[(size_t)b * Mp + t], s1 = asc[(size_t)(b + 1) * Mp + t];
    const uint32_t lw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, hw[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
    int sl = 0, sh = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      sl = __dp4a((int)lw[k], 0x01010101, sl);
      sh = __dp4a((int)hw[k], 0x01010101, sh);
    }
    unsigned char* base = act + (size_t)(st * T + t) * kPairActBytes;
    reinterpret_cast<uint4*>(base)[l] = a0;
    reinterpret_cast<uint4*>(base + 512)[l] = a1;
    reinterpret_cast<uint4*>(base + 1024)[l] = a2;
    reinterpret_cast<uint4*>(base + 1536)[l] = a3;
    reinterpret_cast<float4*>(base + 2048)[l] = make_float4(s0, s1 * 0.0625f, s0 * (float)sl, s1 * (float)sh);
  }
  __syncthreads();
  const int pp_sh = 16 * (pp & 1);
  const bool pp_upper = pp >= 2;
  const uint32_t h_off = sub * 144, q_off = sub * 144 + 16 + 32 * pp;
  const uint32_t h_off_half = (sub & 3) * 144, q_off_half = (sub & 3) * 144 + 16 + 32 * pp;

  float accv[T];
#pragma unroll
  for (int t = 0; t < T; ++t) accv[t] = 0.0f;
  // one chunk against every token: the chunk's nibbles are masked once
  auto chunk = [&](const unsigned char* wp, uint32_t ho, uint32_t qo, const unsigned char* abase, float (&out)[T]) {
    const uint4 h = *reinterpret_cast<const uint4*>(wp + ho);
    const uint4 qa = *reinterpret_cast<const uint4*>(wp + qo), qb = *reinterpret_cast<const uint4*>(wp + qo + 16);
    const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
    uint32_t sc2, mn2;
    q4k_pair(h, pp_sh, pp_upper, sc2, mn2);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    uint32_t wl[8], wh[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      wl[kk] = w[kk] & 0x0F0F0F0Fu;
      wh[kk] = w[kk] & 0xF0F0F0F0u;
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const unsigned char* base = abase + (size_t)t * kPairActBytes;
      const uint4 a0 = reinterpret_cast<const uint4*>(base)[lane], a1 = reinterpret_cast<const uint4*>(base + 512)[lane];
      const uint4 a2 = reinterpret_cast<const uint4*>(base + 1024)[lane], a3 = reinterpret_cast<const uint4*>(base + 1536)[lane];
      const float4 sc = reinterpret_cast<const float4*>(base + 2048)[lane];
      const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
      int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        lo0 = __dp4a((int)al[kk], (int)wl[kk], lo0);
        lo1 = __dp4a((int)al[4 + kk], (int)wl[4 + kk], lo1);
        hi0 = dp4a_su((int)ah[kk], wh[kk], hi0);
        hi1 = dp4a_su((int)ah[4 + kk], wh[4 + kk], hi1);
      }
      const float tq = fmaf(sc.x, (float)((int)(sc2 & 0xFFu) * (lo0 + lo1)), sc.y * (float)((int)(sc2 >> 8) * (hi0 + hi1)));
      const float tm = fmaf(sc.z, (float)(mn2 & 0xFFu), sc.w * (float)(mn2 >> 8));
      out[t] = fmaf(df.x, tq, -df.y * tm);
    }
  };
  for (int n = 0; n < total; ++n) {
    const int ri = n / PP, c0 = 2 * (n - ri * PP), q = n % hs;
    const uint32_t parity = (uint32_t)(n / hs) & 1u;
    const bool two = c0 + 1 < WS;  // (uniform over the warp)
    bool ready = false;
    for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[2 * q]), parity);
    if (ready && two) {
      ready = false;
      for (uint32_t it = 0; it < kSpin && !ready; ++it) ready = try_wait(s_u32(&bars[2 * q + 1]), parity);
    }
    if (!ready) {  // (bounded wait gave up)
      if (lane == 0) atomicOr(err, 64u);
      break;
    }
    const unsigned char* wa = ring + (size_t)(2 * q) * kChunkBytes;
    const unsigned char* abase = act + (size_t)c0 * T * kPairActBytes;
    float r0[T], r1[T];
    // a chunk of four superblocks is read with the half-warp mapping by all lanes; lanes 16..31 are dropped
    const bool h0 = c0 >= FS, h1 = c0 + 1 >= FS;
    chunk(wa, h0 ? h_off_half : h_off, h0 ? q_off_half : q_off, abase, r0);
    const float k0 = (h0 && lane >= 16) ? 0.0f : 1.0f;
    if (two) {
      chunk(wa + kChunkBytes, h1 ? h_off_half : h_off, h1 ? q_off_half : q_off, abase + (size_t)T * kPairActBytes, r1);
      const float k1 = (h1 && lane >= 16) ? 0.0f : 1.0f;
#pragma unroll
      for (int t = 0; t < T; ++t) accv[t] += k0 * r0[t] + k1 * r1[t];
    } else {
#pragma unroll
      for (int t = 0; t < T; ++t) accv[t] += k0 * r0[t];
    }
    __syncwarp();
    if (lane == 0 && n + hs < total) issue(n + hs);  // the slots are read: the pass `hs` ahead goes into them
    if (c0 + 2 >= WS) {  // the row is complete
      const int row = w0 + ri * W;
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float v = warp_sum(accv[t]);
        if (lane == 0) {
          float* cp = C + (size_t)t * ldc + c_off + row;
          *cp = acc ? *cp + v : v;
        }
        accv[t] = 0.0f;
      }
    }
  }
}

template <int T>
int launch_q4k_chunk(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc, int c_off,
                     int acc, cudaStream_t st) {
  constexpr size_t kBudget = 216 * 1024;
  const int nsb = w->K / 256, WS = (nsb + 7) / 8;
  const size_t act = (size_t)WS * T * kPairActBytes;
  if (act + 4096 + (size_t)kPairWarps * 4 * kChunkBytes > kBudget) return 1;
  int slots = (int)((kBudget - act - 4096) / ((size_t)kPairWarps * kChunkBytes));
  slots = slots > 12 ? 12 : (slots & ~1);
  const size_t smem = act + (size_t)kPairWarps * slots * kChunkBytes + (size_t)kPairWarps * slots * 8;
  IZB_SMEM_OPTIN((gemv_q4k_chunk_kernel<T>), kBudget + 8192, w->device);
  const int sms = izb_sm_count(w->device);
  int grid = sms;
  const int need = (w->N + kPairWarps - 1) / kPairWarps;
  if (grid > need) grid = need;
  uint32_t* err = izb_device_error_word(w->device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "gemv: no device error word");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kPairWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int N = w->N, K = w->K;
  IZB_LAUNCH("gemv", st, cudaLaunchKernelEx(&cfg, gemv_q4k_chunk_kernel<T>, raw, N, K, aq, asc, Mp, C, ldc, c_off, acc, slots, err));
  return IZB_OK;
}

template <int QT, int T>
int launch_stream(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc,
                  int c_off, int acc, cudaStream_t st) {
  constexpr int STEP = QT == IZB_Q4_K ? kQ4StepBytes : kQ8StepBytes;
  constexpr size_t kBudget = 200 * 1024;
  constexpr int kSWarps = stream_warps<T>();
  const int nsb = w->K / 256, nsteps = QT == IZB_Q4_K ? (nsb + 3) / 4 : (nsb + 1) / 2;
  const size_t act = ((size_t)nsteps * T * STEP + 127) & ~(size_t)127;
  const int slot_bytes = (int)((w->row_bytes + 127) & ~(size_t)127);
  if (act + 4096 >= kBudget) return 1;
  int slots = (int)((kBudget - act - 4096) / ((size_t)kSWarps * slot_bytes));
  if (slots < 2) return 1;  // (rows too long for a ring: the chunked kernel takes the call)
  if (slots > 8) slots = 8;
  const size_t smem = act + (size_t)kSWarps * slots * slot_bytes + (size_t)kSWarps * slots * 8;
  IZB_SMEM_OPTIN((gemv_stream_kernel<QT, T>), kBudget + 8192, w->device);
  const int sms = izb_sm_count(w->device);
  int grid = sms;
  const int need = (w->N + kSWarps - 1) / kSWarps;
  if (grid > need) grid = need;
  uint32_t* err = izb_device_error_word(w->device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "gemv: no device error word");
  IZB_LAUNCH("gemv", st, gemv_stream_kernel<QT, T><<<grid, kSWarps * 32, smem, st>>>(raw, w->N, w->K, aq, asc, Mp, C, ldc, c_off, acc,
                                                                                    slots, slot_bytes, err));
  return IZB_OK;
}

}  // namespace

// +1: the shared-memory plan does not fit (the chunked kernel of izb_gemv.cu takes the call)
template <int T>
static int stream_t(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int Mp, float* C, int ldc,
                    int c_off, int acc, cudaStream_t st) {
  return w->type == IZB_Q4_K ? launch_stream<IZB_Q4_K, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st)
                             : launch_stream<IZB_Q8_0, T>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
}

#ifndef IZB_MANY_ROWS
#define IZB_MANY_ROWS 1024
#endif
constexpr int kManyRows = IZB_MANY_ROWS;  // below it the matrix is a few hundred KB and the generic kernel does as well

int izb_gemv_stream_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int T, int Mp, float* C,
                           int ldc, int c_off, int acc, cudaStream_t st) {
  if (T == 1 && w->type == IZB_Q4_K && w->K % 1024 == 0 && w->K <= 5120 && w->N >= kManyRows) {
    switch (w->K / 1024) {
      case 1: return launch_q4k_reg<1>(w, raw, aq, asc, Mp, C, c_off, acc, st);
      case 2: return launch_q4k_reg<2>(w, raw, aq, asc, Mp, C, c_off, acc, st);
      case 3: return launch_q4k_reg<3>(w, raw, aq, asc, Mp, C, c_off, acc, st);
      case 4: return launch_q4k_reg<4>(w, raw, aq, asc, Mp, C, c_off, acc, st);
      default: return launch_q4k_reg<5>(w, raw, aq, asc, Mp, C, c_off, acc, st);
    }
  }
  if (T <= 4 && w->type == IZB_Q4_K && w->K % 1024 == 0 && w->K > 5120 && w->N >= kManyRows) {  // long rows: ring of chunks
    int rc = 1;
    switch (T) {
      case 1: rc = launch_q4k_chunk<1>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st); break;
      case 2: rc = launch_q4k_chunk<2>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st); break;
      case 3: rc = launch_q4k_chunk<3>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st); break;
      default: rc = launch_q4k_chunk<4>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st); break;
    }
    if (rc != 1) return rc;  // (+1: the activations alone do not fit: the kernels below take the call)
  }
  if (T >= 2 && T <= 4 && w->type == IZB_Q4_K && w->K % 1024 == 0 && w->K <= 5120 && w->N >= kManyRows) {
    switch (T) {
      case 2: return launch_q4k_pair_k<2>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
      case 3: return launch_q4k_pair_k<3>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
      default: return launch_q4k_pair_k<4>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    }
  }
  switch (T) {
    case 1: return stream_t<1>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 2: return stream_t<2>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 3: return stream_t<3>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 4: return stream_t<4>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 5: return stream_t<5>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 6: return stream_t<6>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    case 7: return stream_t<7>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
    default: return stream_t<8>(w, raw, aq, asc, Mp, C, ldc, c_off, acc, st);
  }
}
