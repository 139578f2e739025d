// Mixture-of-experts around the quantised matmul: routing, the counting sort of (token, choice) pairs into expert
// slots, the per-tile expert kernels on raw GGUF rows, and the combine.
//   moe_route    zero/kernels/moe.cl:50-89     softmax numerators of the NU largest logits, ties -> lower expert id
//   moe_sort     zero/kernels/moe.cl:141-179   exclusive scan of the counts, tile list, scatter (here deterministic)
//   moe_gateup   zero/kernels/decode_moe.cl:92-260   h = silu(x Wg^T) * (x Wu^T) per tile of <= TM slots of one expert
//   moe_down     zero/kernels/decode_moe.cl:269-449  y = swt * (hq Wd^T)
//   moe_combine  zero/kernels/moe.cl:344-352   x[t] += sum_k y[inv[t*NU+k]] in choice order
// The per-tile kernels run the few-row GEMV loop (izb_gemv_body.cuh) over the rows of the tile's expert, with the
// activation rows gathered through the slot -> token map, as the reference's moe_gateup_q / moe_down_q do.
#include "izb_gemv_body.cuh"

namespace {
using namespace izb_gemvk;

constexpr int kMaxPerLane = 16;  // experts per lane: NE <= 512

// Routing.  The rule (zero/kernels/moe.cl:56-86; CPU twin tools/ref_forward.cpp:1660-1690): choice k is the largest logit
// not chosen yet, the lower expert id winning a tie; p_k = exp(l_k - l_0) where l_0, the first choice, is the maximum;
// w_k = p_k / (p_0 + ... + p_{NU-1}), the sum taken in choice order.
//
// One warp per token.  A logit and its expert id travel as ONE 64-bit key -- the order-preserving integer image of the
// float in the high word, the complemented id in the low word -- so a single warp-wide maximum per choice yields the
// winner and applies the tie rule at once.  Every lane keeps the key of its own best candidate and only the lane that
// owned the winner rescans its (at most 16) experts.
__device__ __forceinline__ unsigned long long route_key(float v, int e) {
  uint32_t u = __float_as_uint(__fadd_rn(v, 0.0f));  // (-0 becomes +0: the two compare equal, so they must tie)
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (uint32_t)(~(uint32_t)e);
}
__device__ __forceinline__ float route_key_value(unsigned long long k) {
  const uint32_t u = (uint32_t)(k >> 32);
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
}

__global__ void __launch_bounds__(256) moe_route_kernel(const float* __restrict__ logits, int ldl, int T, int NE, int NU,
                                                        int32_t* __restrict__ ids, float* __restrict__ wts,
                                                        int32_t* __restrict__ counts, float* __restrict__ sgate) {
  const int token = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (token >= T) return;
  const float* row = logits + (size_t)token * ldl;
  // the shared expert's gate: the sigmoid of the logit after the experts' (SGATE, zero/kernels/moe.cl:44,88)
  if (sgate && lane == 0) sgate[token] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-row[NE])));
  unsigned long long key[kMaxPerLane];  // 0 = no candidate (past NE, or already chosen)
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    key[i] = e < NE ? route_key(row[e], e) : 0ull;
  }
  auto lane_best = [&]() {
    unsigned long long b = 0ull;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) b = key[i] > b ? key[i] : b;
    return b;
  };
  unsigned long long mine = lane_best();
  float top = 0.0f, denom = 0.0f, p_keep = 0.0f;
  int e_keep = 0;
  for (int k = 0; k < NU; ++k) {
    unsigned long long win = mine;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, win, o);
      win = other > win ? other : win;
    }
    const int e = (int)(~(uint32_t)win);
    const float l = route_key_value(win);
    if (k == 0) top = l;
    if ((e & 31) == lane) {  // the owner strikes the winner out and looks for its next candidate
#pragma unroll
      for (int i = 0; i < kMaxPerLane; ++i)
        if (i == (e >> 5)) key[i] = 0ull;
      mine = lane_best();
    }
    const float p = expf(l - top);
    denom += p;  // (every lane adds the same terms in choice order)
    if (lane == k) { p_keep = p; e_keep = e; }
  }
  if (lane < NU) {
    ids[token * NU + lane] = e_keep;
    wts[token * NU + lane] = __fdiv_rn(p_keep, denom);
    atomicAdd(&counts[e_keep], 1);
  }
}

// One thread per expert: offsets (exclusive scan, serial: NE is a few hundred) and the expert's tiles.
// With an expert range [e0, e1) (the expert-parallel split, tp_moe_mask, zero/kernels/tp.cl:61-64) the other experts count
// as empty and a tile names its expert by its index in this rank's stack, e - e0.
__global__ void moe_scan_kernel(const int32_t* __restrict__ counts, int NE, int TM, int32_t* __restrict__ offs,
                                int32_t* __restrict__ tiles, int max_tiles, int e0, int e1) {
  const int e = threadIdx.x;
  int off = 0, toff = 0;
  for (int i = 0; i < e && i < NE; ++i) {
    const int ci = (i >= e0 && i < e1) ? counts[i] : 0;
    off += ci;
    toff += (ci + TM - 1) / TM;
  }
  if (e < NE) {
    const int c = (e >= e0 && e < e1) ? counts[e] : 0, nt = (c + TM - 1) / TM;
    offs[e] = off;
    for (int i = 0; i < nt; ++i) {
      if (toff + i >= max_tiles) break;
      int32_t* tp = tiles + 1 + 3 * (toff + i);
      tp[0] = e - e0;
      tp[1] = off + i * TM;
      tp[2] = min(TM, c - i * TM);
    }
    if (e == NE - 1) {
      offs[NE] = off + c;
      tiles[0] = min(toff + nt, max_tiles);
    }
  }
}

// One CTA per expert: its pairs in increasing pair index take consecutive slots (a deterministic atomic_inc order).
// A thread looks at four consecutive pairs per pass (one 128-bit load), so a pass covers 1024 pairs: an exclusive scan of
// the per-thread counts over the warp (shuffles) and over the eight warps (shared memory, double-buffered so that one
// barrier per pass is enough) gives every pair of the expert its slot.
__global__ void __launch_bounds__(256) moe_scatter_kernel(const int32_t* __restrict__ ids, const float* __restrict__ wts, int n,
                                                          int NU, const int32_t* __restrict__ offs, int32_t* __restrict__ stok,
                                                          float* __restrict__ swt, int32_t* __restrict__ inv, int e0, int e1) {
  __shared__ int s_warp[2][8];
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (e < e0 || e >= e1) {  // another rank's expert: its pairs get no slot (tp_moe_scatter, zero/kernels/tp.cl:67-78)
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      if (ids[i] == e) inv[i] = -1;
    return;
  }
  int base = offs[e];  // (every thread keeps the running base: no broadcast needed)
  int buf = 0;
  for (int i0 = 0; i0 < n; i0 += 1024, buf ^= 1) {
    const int i = i0 + 4 * threadIdx.x;
    int4 v = make_int4(-1, -1, -1, -1);
    if (i + 3 < n) {
      v = *reinterpret_cast<const int4*>(ids + i);
    } else {
      if (i < n) v.x = ids[i];
      if (i + 1 < n) v.y = ids[i + 1];
      if (i + 2 < n) v.z = ids[i + 2];
    }
    const int m0 = v.x == e, m1 = v.y == e, m2 = v.z == e, m3 = v.w == e;
    const int cnt = m0 + m1 + m2 + m3;
    int incl = cnt;  // inclusive scan over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[buf][warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = s_warp[buf][w];
      if (w < warp) before += c;
      total += c;
    }
    int s = base + before + incl - cnt;
    if (m0) { stok[s] = i / NU; swt[s] = wts[i]; inv[i] = s; ++s; }
    if (m1) { stok[s] = (i + 1) / NU; swt[s] = wts[i + 1]; inv[i + 1] = s; ++s; }
    if (m2) { stok[s] = (i + 2) / NU; swt[s] = wts[i + 2]; inv[i + 2] = s; ++s; }
    if (m3) { stok[s] = (i + 3) / NU; swt[s] = wts[i + 3]; inv[i + 3] = s; }
    base += total;
  }
}

template <int QT>
__global__ void __launch_bounds__(kWarps * 32) moe_gateup_kernel(const uint8_t* __restrict__ rg, const uint8_t* __restrict__ ru,
                                                                 int F, int K, size_t mat_bytes, const int8_t* __restrict__ aq,
                                                                 const float* __restrict__ asc, int Mp,
                                                                 const int32_t* __restrict__ tiles,
                                                                 const int32_t* __restrict__ stok, float* __restrict__ h, int spc) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int tok[8];
  const int ti = blockIdx.y;
  if (ti >= tiles[0]) return;  // uniform over the CTA
  const int e = tiles[1 + 3 * ti], r0 = tiles[2 + 3 * ti], nr = tiles[3 + 3 * ti];
  if (threadIdx.x < 8) tok[threadIdx.x] = stok[r0 + min((int)threadIdx.x, nr - 1)];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = (blockIdx.x * kWarps + warp) * kRows;
  float ag[kRows][8], au[kRows][8];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < 8; ++t) ag[r][t] = au[r][t] = 0.0f;
  gemv_body<QT, 8>(smem, rg + (size_t)e * mat_bytes, F, K, aq, asc, Mp, tok, row0, spc, ag);
  gemv_body<QT, 8>(smem, ru + (size_t)e * mat_bytes, F, K, aq, asc, Mp, tok, row0, spc, au);
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float g = warp_sum(ag[r][t]), u = warp_sum(au[r][t]);
      const int n = row0 + r;
      if (lane == 0 && n < F && t < nr) h[(size_t)(r0 + t) * F + n] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
    }
}

template <int QT>
__global__ void __launch_bounds__(kWarps * 32) moe_down_kernel(const uint8_t* __restrict__ rd, int E, int F, size_t mat_bytes,
                                                               const int8_t* __restrict__ hq, const float* __restrict__ hsc,
                                                               int Sp, const int32_t* __restrict__ tiles,
                                                               const float* __restrict__ swt, float* __restrict__ y, int spc) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int tok[8];
  const int ti = blockIdx.y;
  if (ti >= tiles[0]) return;
  const int e = tiles[1 + 3 * ti], r0 = tiles[2 + 3 * ti], nr = tiles[3 + 3 * ti];
  if (threadIdx.x < 8) tok[threadIdx.x] = r0 + min((int)threadIdx.x, nr - 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = (blockIdx.x * kWarps + warp) * kRows;
  float a[kRows][8];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < 8; ++t) a[r][t] = 0.0f;
  gemv_body<QT, 8>(smem, rd + (size_t)e * mat_bytes, E, F, hq, hsc, Sp, tok, row0, spc, a);
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float v = warp_sum(a[r][t]);
      const int n = row0 + r;
      if (lane == 0 && n < E && t < nr) y[(size_t)(r0 + t) * E + n] = __fmul_rn(swt[r0 + t], v);
    }
}

// x[t] += v, v = sum over the token's choices (in choice order, slots < 0 left out) + sgate[t] * sh[t] when a shared expert is
// given (moe_combine, zero/kernels/moe.cl:344-352); partial: x[t] = v, a rank's share of the sum in the expert-parallel
// split (tp_moe_combine, zero/kernels/tp.cl:100-111).
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, const int32_t* __restrict__ inv, int T,
                                   int NU, int E, const float* __restrict__ sh, const float* __restrict__ sgate, int partial) {
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4, t = blockIdx.x;  // (tokens on x: no 65535 limit)
  if (c >= E) return;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < NU; ++k) {
    const int s = inv[t * NU + k];
    if (s < 0) continue;
    const float4 a = *reinterpret_cast<const float4*>(y + (size_t)s * E + c);
    v.x = __fadd_rn(v.x, a.x); v.y = __fadd_rn(v.y, a.y); v.z = __fadd_rn(v.z, a.z); v.w = __fadd_rn(v.w, a.w);
  }
  if (sh) {
    const float g = sgate[t];
    const float4 a = *reinterpret_cast<const float4*>(sh + (size_t)t * E + c);
    v.x = __fadd_rn(v.x, __fmul_rn(g, a.x)); v.y = __fadd_rn(v.y, __fmul_rn(g, a.y));
    v.z = __fadd_rn(v.z, __fmul_rn(g, a.z)); v.w = __fadd_rn(v.w, __fmul_rn(g, a.w));
  }
  float4* px = reinterpret_cast<float4*>(x + (size_t)t * E + c);
  if (!partial) {
    const float4 o = *px;
    v.x = __fadd_rn(o.x, v.x); v.y = __fadd_rn(o.y, v.y); v.z = __fadd_rn(o.z, v.z); v.w = __fadd_rn(o.w, v.w);
  }
  *px = v;
}

}  // namespace

extern "C" int izb_moe_route_ex(const float* d_logits, int ldl, int T, int NE, int NU, int32_t* d_ids, float* d_wts,
                                int32_t* d_counts, float* d_sgate, void* stream) {
  if (!d_logits || !d_ids || !d_wts || !d_counts) IZB_FAIL(IZB_ERR_ARG, "moe_route: null pointer");
  if (T < 1 || NE < 1 || NE > 32 * kMaxPerLane || NU < 1 || NU > 32 || NU > NE || ldl < NE + (d_sgate ? 1 : 0))
    IZB_FAIL(IZB_ERR_SHAPE, "moe_route: T=%d NE=%d NU=%d ldl=%d (NE <= 512, NU <= 32, ldl >= NE, + 1 with a shared-expert gate)", T, NE, NU, ldl);
  cudaStream_t st = (cudaStream_t)stream;
  IZB_CUDA(cudaMemsetAsync(d_counts, 0, (size_t)NE * 4, st));
  IZB_LAUNCH("moe_route", st, moe_route_kernel<<<(T + 7) / 8, 256, 0, st>>>(d_logits, ldl, T, NE, NU, d_ids, d_wts, d_counts, d_sgate));
  return IZB_OK;
}

extern "C" int izb_moe_route(const float* d_logits, int ldl, int T, int NE, int NU, int32_t* d_ids, float* d_wts,
                             int32_t* d_counts, void* stream) {
  return izb_moe_route_ex(d_logits, ldl, T, NE, NU, d_ids, d_wts, d_counts, nullptr, stream);
}

extern "C" int izb_moe_sort_ex(const int32_t* d_ids, const float* d_wts, const int32_t* d_counts, int T, int NE, int NU, int TM,
                               int e0, int e1, int32_t* d_offs, int32_t* d_tiles, int max_tiles, int32_t* d_stok, float* d_swt,
                               int32_t* d_inv, void* stream) {
  if (!d_ids || !d_wts || !d_counts || !d_offs || !d_tiles || !d_stok || !d_swt || !d_inv) IZB_FAIL(IZB_ERR_ARG, "moe_sort: null pointer");
  if (T < 1 || NE < 1 || NE > 1024 || NU < 1 || TM < 1) IZB_FAIL(IZB_ERR_SHAPE, "moe_sort: T=%d NE=%d NU=%d TM=%d", T, NE, NU, TM);
  if (e0 < 0 || e1 > NE || e0 >= e1) IZB_FAIL(IZB_ERR_SHAPE, "moe_sort: expert range [%d, %d) of %d", e0, e1, NE);
  if (!izb_aligned(d_ids, 16)) IZB_FAIL(IZB_ERR_ALIGN, "moe_sort: ids must be 16-byte aligned (read four at a time)");
  if (max_tiles < (T * NU + TM - 1) / TM + NE) IZB_FAIL(IZB_ERR_LIMIT, "moe_sort: max_tiles = %d < %d (pairs/TM + NE)", max_tiles, (T * NU + TM - 1) / TM + NE);
  cudaStream_t st = (cudaStream_t)stream;
  IZB_LAUNCH("moe_scan", st, moe_scan_kernel<<<1, 1024, 0, st>>>(d_counts, NE, TM, d_offs, d_tiles, max_tiles, e0, e1));
  IZB_LAUNCH("moe_scatter", st, moe_scatter_kernel<<<NE, 256, 0, st>>>(d_ids, d_wts, T * NU, NU, d_offs, d_stok, d_swt, d_inv, e0, e1));
  return IZB_OK;
}

extern "C" int izb_moe_sort(const int32_t* d_ids, const float* d_wts, const int32_t* d_counts, int T, int NE, int NU, int TM,
                            int32_t* d_offs, int32_t* d_tiles, int max_tiles, int32_t* d_stok, float* d_swt, int32_t* d_inv,
                            void* stream) {
  return izb_moe_sort_ex(d_ids, d_wts, d_counts, T, NE, NU, TM, 0, NE, d_offs, d_tiles, max_tiles, d_stok, d_swt, d_inv, stream);
}

int izb_moe_gateup_tiles(const izb_weight* wg, const izb_weight* wu, const int8_t* d_aq, const float* d_asc, int Mp,
                         const int32_t* d_tiles, int max_tiles, const int32_t* d_stok, float* d_h, cudaStream_t st) {
  const int F = wg->N, K = wg->K;
  size_t smem = 0;
  const int spc = steps_per_chunk(wg->type, K, 8, &smem);
  dim3 grid((F + kWarps * kRows - 1) / (kWarps * kRows), max_tiles);
  const size_t mat_bytes = (size_t)F * wg->row_bytes;
  if (wg->type == IZB_Q4_K) {
    IZB_SMEM_OPTIN((moe_gateup_kernel<IZB_Q4_K>), kMaxSmem, wg->device);
    moe_gateup_kernel<IZB_Q4_K><<<grid, kWarps * 32, smem, st>>>(wg->raw, wu->raw, F, K, mat_bytes, d_aq, d_asc, Mp, d_tiles, d_stok, d_h, spc);
  } else {
    IZB_SMEM_OPTIN((moe_gateup_kernel<IZB_Q8_0>), kMaxSmem, wg->device);
    moe_gateup_kernel<IZB_Q8_0><<<grid, kWarps * 32, smem, st>>>(wg->raw, wu->raw, F, K, mat_bytes, d_aq, d_asc, Mp, d_tiles, d_stok, d_h, spc);
  }
  IZB_LAUNCHED();
  return IZB_OK;
}

int izb_moe_down_tiles(const izb_weight* wd, const int8_t* d_hq, const float* d_hsc, int Sp, const int32_t* d_tiles,
                       int max_tiles, const float* d_swt, float* d_y, cudaStream_t st) {
  const int E = wd->N, F = wd->K;
  size_t smem = 0;
  const int spc = steps_per_chunk(wd->type, F, 8, &smem);
  dim3 grid((E + kWarps * kRows - 1) / (kWarps * kRows), max_tiles);
  const size_t mat_bytes = (size_t)E * wd->row_bytes;
  if (wd->type == IZB_Q4_K) {
    IZB_SMEM_OPTIN((moe_down_kernel<IZB_Q4_K>), kMaxSmem, wd->device);
    moe_down_kernel<IZB_Q4_K><<<grid, kWarps * 32, smem, st>>>(wd->raw, E, F, mat_bytes, d_hq, d_hsc, Sp, d_tiles, d_swt, d_y, spc);
  } else {
    IZB_SMEM_OPTIN((moe_down_kernel<IZB_Q8_0>), kMaxSmem, wd->device);
    moe_down_kernel<IZB_Q8_0><<<grid, kWarps * 32, smem, st>>>(wd->raw, E, F, mat_bytes, d_hq, d_hsc, Sp, d_tiles, d_swt, d_y, spc);
  }
  IZB_LAUNCHED();
  return IZB_OK;
}

extern "C" int izb_moe_combine_ex(float* d_x, const float* d_y, const int32_t* d_inv, int T, int NU, int E, const float* d_sh,
                                  const float* d_sgate, int partial, void* stream) {
  if (!d_x || !d_y || !d_inv) IZB_FAIL(IZB_ERR_ARG, "moe_combine: null pointer");
  if ((d_sh == nullptr) != (d_sgate == nullptr)) IZB_FAIL(IZB_ERR_ARG, "moe_combine: the shared expert's output and its gate come together");
  if (T < 1 || NU < 1 || E < 4 || E % 4) IZB_FAIL(IZB_ERR_SHAPE, "moe_combine: T=%d NU=%d E=%d (E %% 4 == 0)", T, NU, E);
  if (!izb_aligned(d_x, 16) || !izb_aligned(d_y, 16) || (d_sh && !izb_aligned(d_sh, 16))) IZB_FAIL(IZB_ERR_ALIGN, "moe_combine: x, y, sh must be 16-byte aligned");
  if ((E / 4 + 127) / 128 > 65535) IZB_FAIL(IZB_ERR_LIMIT, "moe_combine: E = %d too wide", E);
  dim3 grid(T, (E / 4 + 127) / 128);
  IZB_LAUNCH("moe_combine", (cudaStream_t)stream,
             moe_combine_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(d_x, d_y, d_inv, T, NU, E, d_sh, d_sgate, partial ? 1 : 0));
  return IZB_OK;
}

extern "C" int izb_moe_combine(float* d_x, const float* d_y, const int32_t* d_inv, int T, int NU, int E, void* stream) {
  return izb_moe_combine_ex(d_x, d_y, d_inv, T, NU, E, nullptr, nullptr, 0, stream);
}

// grouped tensor-core path (izb_gemm_tc.cu): tiles of up to 128 slots; +1 = shape not taken
int izb_moe_gateup_tc(const izb_weight* wg, const izb_weight* wu, const int8_t* d_aq, const float* d_asc, int Mp,
                      const int32_t* d_tiles, int max_tiles, const int32_t* d_stok, float* d_h, cudaStream_t st);
int izb_moe_down_tc(const izb_weight* wd, const int8_t* d_hq, const float* d_hsc, int Sp, const int32_t* d_tiles, int max_tiles,
                    const float* d_swt, float* d_y, cudaStream_t st);

int izb_moe_gateup_fused_tc(const izb_weight* wgu, const int8_t* d_aq, const float* d_asc, int Mp, const int32_t* d_tiles,
                            int max_tiles, const int32_t* d_stok, float* d_h, cudaStream_t st);

extern "C" int izb_moe_gateup(const izb_weight* wg, const izb_weight* wu, const int8_t* d_aq, const float* d_asc, int Mp,
                              const int32_t* d_tiles, int max_tiles, int TM, const int32_t* d_stok, float* d_h, void* stream) {
  if (wg && !wu && wg->gu32) {  // one interleaved gate | up stack: a single grouped GEMM with the SwiGLU product in its epilogue
    if (!d_aq || !d_asc || !d_tiles || !d_stok || !d_h) IZB_FAIL(IZB_ERR_ARG, "moe_gateup: null pointer");
    if (max_tiles < 1 || max_tiles > 65535) IZB_FAIL(IZB_ERR_LIMIT, "moe_gateup: max_tiles = %d (1..65535)", max_tiles);
    if (!izb_aligned(d_aq, 16)) IZB_FAIL(IZB_ERR_ALIGN, "moe_gateup: aq not 16-byte aligned");
    if (TM != 128) IZB_FAIL(IZB_ERR_SHAPE, "moe_gateup: an interleaved gate | up stack runs on the grouped tensor-core GEMM (TM = 128), not on tiles of %d", TM);
    if (int rc = izb_require_device(wg->device, "moe_gateup")) return rc;
    const int rc = izb_moe_gateup_fused_tc(wg, d_aq, d_asc, Mp, d_tiles, max_tiles, d_stok, d_h, (cudaStream_t)stream);
    if (rc <= 0) return rc;
    IZB_FAIL(IZB_ERR_SHAPE, "moe_gateup: the grouped tensor-core GEMM does not take this stack (2F = %d, K = %d)", wg->N, wg->K);
  }
  if (!wg || !wu || !d_aq || !d_asc || !d_tiles || !d_stok || !d_h) IZB_FAIL(IZB_ERR_ARG, "moe_gateup: null pointer");
  if (wg->type != wu->type || wg->N != wu->N || wg->K != wu->K || wg->n_mats != wu->n_mats)
    IZB_FAIL(IZB_ERR_SHAPE, "moe_gateup: gate and up stacks differ");
  if (max_tiles < 1 || max_tiles > 65535) IZB_FAIL(IZB_ERR_LIMIT, "moe_gateup: max_tiles = %d (1..65535)", max_tiles);
  if (!izb_aligned(d_aq, 16)) IZB_FAIL(IZB_ERR_ALIGN, "moe_gateup: aq not 16-byte aligned");
  if (wg->type == IZB_K16) IZB_FAIL(IZB_ERR_TYPE, "moe_gateup: expert stacks of ggml type %d are not taken (Q8_0, Q4_K, Q4_0)", wg->ggml_type);
  if (wu->device != wg->device) IZB_FAIL(IZB_ERR_ARG, "moe_gateup: gate and up stacks live on different devices");
  if (int rc = izb_require_device(wg->device, "moe_gateup")) return rc;
  if (TM >= 1 && TM <= 8) return izb_moe_gateup_tiles(wg, wu, d_aq, d_asc, Mp, d_tiles, max_tiles, d_stok, d_h, (cudaStream_t)stream);
  if (TM == 128) {
    const int rc = izb_moe_gateup_tc(wg, wu, d_aq, d_asc, Mp, d_tiles, max_tiles, d_stok, d_h, (cudaStream_t)stream);
    if (rc <= 0) return rc;
    IZB_FAIL(IZB_ERR_SHAPE, "moe_gateup: the grouped tensor-core GEMM needs F %% 128 == 0 and a weight with a tensor map (F = %d, K = %d); use TM <= 8", wg->N, wg->K);
  }
  IZB_FAIL(IZB_ERR_SHAPE, "moe_gateup: tiles of %d slots (1..8: per-tile GEMV kernels; 128: grouped tensor-core GEMM)", TM);
}

extern "C" int izb_moe_down(const izb_weight* wd, const int8_t* d_hq, const float* d_hsc, int Sp, const int32_t* d_tiles,
                            int max_tiles, int TM, const float* d_swt, float* d_y, void* stream) {
  if (!wd || !d_hq || !d_hsc || !d_tiles || !d_swt || !d_y) IZB_FAIL(IZB_ERR_ARG, "moe_down: null pointer");
  if (max_tiles < 1 || max_tiles > 65535) IZB_FAIL(IZB_ERR_LIMIT, "moe_down: max_tiles = %d (1..65535)", max_tiles);
  if (!izb_aligned(d_hq, 16)) IZB_FAIL(IZB_ERR_ALIGN, "moe_down: hq not 16-byte aligned");
  if (wd->type == IZB_K16) IZB_FAIL(IZB_ERR_TYPE, "moe_down: expert stacks of ggml type %d are not taken (Q8_0, Q4_K, Q4_0)", wd->ggml_type);
  if (int rc = izb_require_device(wd->device, "moe_down")) return rc;
  if (TM >= 1 && TM <= 8) return izb_moe_down_tiles(wd, d_hq, d_hsc, Sp, d_tiles, max_tiles, d_swt, d_y, (cudaStream_t)stream);
  if (TM == 128) {
    const int rc = izb_moe_down_tc(wd, d_hq, d_hsc, Sp, d_tiles, max_tiles, d_swt, d_y, (cudaStream_t)stream);
    if (rc <= 0) return rc;
    IZB_FAIL(IZB_ERR_SHAPE, "moe_down: the grouped tensor-core GEMM needs E %% 128 == 0 and a weight with a tensor map (E = %d, F = %d); use TM <= 8", wd->N, wd->K);
  }
  IZB_FAIL(IZB_ERR_SHAPE, "moe_down: tiles of %d slots (1..8: per-tile GEMV kernels; 128: grouped tensor-core GEMM)", TM);
}
