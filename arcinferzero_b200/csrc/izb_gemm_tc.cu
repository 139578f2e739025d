// Prefill GEMM on the 5th-generation tensor cores (tcgen05, TMEM accumulators), exact per-32-block semantics.
//
// Problem: C[m][n] = sum over 32-blocks b of asc[m][b] * wscale[n][b] * dot_b[m][n]  (- the Q4_K min term), where dot_b
// is an exact integer.  Both operands carry a scale per block, so a block's dot product must leave the tensor core
// before the next one is added: the f32 combine on the CUDA cores (M*N*K/32 fused multiply-adds), not the MMA, bounds
// the kernel.  The design therefore minimises CUDA-core work per (m, n, block) to ONE fma:
//   * operands are fed as fp16 holding exact integers: activations a in [-127,127]; Q4_K weights as sc*q in [0,945]
//     (the 6-bit sub-block scale folded in, exactly representable), Q8_0 weights q in [-128,127].  tcgen05.mma
//     kind::f16 then leaves (float)(sc*dot) in TMEM: every product and every partial sum is an integer below 2^24,
//     so the f32 accumulator holds it exactly (the verification mode reads these accumulators back and the tests
//     compare them bit for bit with the CPU's int32 dots).  A kind::i8 accumulator would need an int->float
//     conversion and a second multiply per element, which costs more than the slower fp16 MMA rate saves.
//   * Q4_K:  tq += asc[m][b] * D_b   per block;   res = fma(d[n], tq, res)   per superblock.
//     The min term  - sum_b (asc*asum)[m][b] * (dmin*mn)[n][b]  never touches the CUDA cores: it is one more GEMM on the
//     tensor cores, accumulated over the whole of K in a fourth TMEM accumulator and read once per tile.  Both factors
//     are f32 numbers, fed as bf16 triples (v = v1+v2+v3, u = u1+u2+u3, the six products that matter: v1u1, v1u2, v2u1,
//     v1u3, v2u2, v3u1; u = -dmin*mn has 17 significant bits, so its split is exact, v is exact to 2^-24).  Those 48
//     K-entries per superblock travel as a fifth "stage" through the same operand ring as the four fp16 stages.
//   * Q8_0:  res += (asc[m][b] * d[n][b]) * D_b.
//
// CTA = one 128 (tokens, TMEM lanes) x 128 (weight rows, TMEM columns) output tile, 16 warps:
//   warp 0      activation producer: cp.async.bulk of pre-swizzled operand tiles (made by act_prepare_kernel) into the
//               operand ring;
//   warp 3      weight producer: TMA (cp.async.bulk.tensor.2d) of the raw GGUF superblocks of 128 rows into a ring, and
//               the tile's activation scales;
//   warps 4-7   dequantisers: one thread per weight row, nibbles -> fp16 sc*q written in the 128-byte-swizzled K-major
//               operand layout, the min-term operand, block scales to shared memory;
//   warps 1-2   issue tcgen05.mma (one thread each, alternating stages) into a ring of three 128-column accumulators +
//               the min-term accumulator (always warp 2, so that one thread orders all updates of it);
//   warps 8-15  combine: tcgen05.ld of 64 columns at a time, one fma per element, final store with the reference's
//               store modes.
// All waits are bounded: a wait that gives up sets a CTA-wide abort flag and a device error word, the CTA drains and
// returns without storing (izb_device_status reports it).
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "izb_common.cuh"

void izb_set_tc_ok(int device, int ok);
void izb_note_noalloc_status(int device, uint32_t* status);
int izb_get_tc_ok(int device);
int izb_gemm_core_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int M, int Mp, float* C,
                         int ldc, int c_off, int acc, int32_t* dots, cudaStream_t st);

// Build-time experiment switches (defaults = the shipped kernel).

#ifndef IZB_TC_TRACE
#define IZB_TC_TRACE 0   // diagnostics build: CTA 0 stamps clock64() at the hand-overs of its first blocks into TcParams::trace
#endif
#if IZB_TC_TRACE
#define TRACE(ev, idx)                                                                                      \
  do {                                                                                                      \
    if (p.trace && blockIdx.x == 0 && lane == 0 && (idx) >= 0 && (idx) < 2048) p.trace[(ev) * 2048 + (idx)] = clock64(); \
  } while (0)
#else
#define TRACE(ev, idx) do { } while (0)
#endif

namespace {

constexpr int BM = 128, BN = 128, KS = 64;
constexpr int ND1 = 3;                    // accumulators of a 32-block in the ring
constexpr int STAGE_BYTES = BM * KS * 2;  // 16 KB: 128 rows x 128 B
constexpr int kThreads = 512;
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr int RAW_Q4 = 128 * 144, RAW_Q8 = 128 * 272;  // 18432, 34816: the raw superblocks of a tile's 128 weight rows
constexpr int NASC = 3;

// Ring depths.  The two operands of a stage travel through rings of their own: an activation image is a bulk copy from L2
// whose latency (not its bandwidth) is what has to be covered, so its ring is as deep as shared memory allows; a weight
// tile is written by the dequantiser warps from a raw tile that is already in shared memory.
#ifndef IZB_TC_NA4
#define IZB_TC_NA4 6
#endif
#ifndef IZB_TC_NB4
#define IZB_TC_NB4 4
#endif
#ifndef IZB_TC_NR4
#define IZB_TC_NR4 2
#endif
#ifndef IZB_TC_NA8
#define IZB_TC_NA8 4
#endif
#ifndef IZB_TC_NB8
#define IZB_TC_NB8 4
#endif

// shared memory map (bytes from a 1024-aligned base)
template <int QT>
struct Map {
  static constexpr bool q4 = QT == IZB_Q4_K;
  static constexpr int NA = q4 ? IZB_TC_NA4 : IZB_TC_NA8;  // activation stages
  static constexpr int NB = q4 ? IZB_TC_NB4 : IZB_TC_NB8;  // weight-operand stages
  static constexpr int NR = q4 ? IZB_TC_NR4 : 2;           // raw superblock tiles
  static constexpr int RAW = q4 ? RAW_Q4 : RAW_Q8;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + NA * STAGE_BYTES;
  static constexpr int OFF_RAW = OFF_B + NB * STAGE_BYTES;
  static constexpr int OFF_SCL = OFF_RAW + NR * RAW;              // Q4_K: 4 x [128] f32 superblock scales d; Q8_0: 4 x [8][128] f32 block scales
  static constexpr int OFF_ASC = OFF_SCL + (q4 ? 4 * 512 : 4 * 4096);  // NASC x [8 blocks][128 rows] f32 activation scales
  static constexpr int OFF_BAR = OFF_ASC + NASC * 4096;
  static constexpr int SMEM_BYTES = OFF_BAR + 1024 + 1024;        // barriers + alignment slack
  // 8-byte mbarriers
  static constexpr int A_FULL = 0, A_EMPTY = A_FULL + NA, B_FULL = A_EMPTY + NA, B_EMPTY = B_FULL + NB, RAW_FULL = B_EMPTY + NB,
                       RAW_EMPTY = RAW_FULL + NR, D1_FULL = RAW_EMPTY + NR, D1_EMPTY = D1_FULL + ND1, D2_FULL = D1_EMPTY + ND1,
                       D2_EMPTY = D2_FULL + 1, ASC_FULL = D2_EMPTY + 1, ASC_EMPTY = ASC_FULL + NASC, NUM_BARS = ASC_EMPTY + NASC;
  static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");
  static_assert(NUM_BARS * 8 + 16 <= 1024, "barrier area");
  static_assert(OFF_RAW % 1024 == 0 && OFF_SCL % 16 == 0, "alignment of the TMA destinations");
};

// error-word codes (which wait gave up)
enum : uint32_t { E_APROD = 1, E_WPROD = 2, E_DEQ = 4, E_MMA = 16, E_EPI = 32 };

struct TcParams {
  const uint16_t* aimg;   // [tiles][stages][128][64] 16-bit operand tiles, rows 128-byte swizzled; stages = K/64, and
                          // for the Q4_K GEMM one bf16 min-term tile after every four (5 per superblock)
  const float* ascimg;    // [tiles][K/32][128] f32: the tile rows' activation scales, gathered
  const int32_t* tiles;   // grouped: [1 + 3*max_tiles]; dense: null
  const int32_t* rowmap;  // grouped gather of activation rows (slot -> token) or null
  const float* rowscale;  // per output row factor or null
  int M;                  // dense: rows to store
  int n_mtiles;           // dense: row tiles (grouped: tiles[0], read on the device)
  int N, K;               // per matrix
  int mat;                // dense: matrix of the stack
  float* C;
  int ldc, c_off, acc;
  int32_t* dots;          // verification mode output or null
  uint32_t* err;
  uint32_t spin_limit;    // polls after which a wait gives up
  int skip_stage;         // diagnostics: the operand stage the activation producer leaves out (-1: none)
  unsigned long long* trace;  // diagnostics build only: [16][2048] clock stamps
};

// ---------------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// non-blocking look at a barrier's phase
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok;
}
// Bounded wait.  false = gave up (or another thread did): the caller leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* err,
                                          uint32_t limit, uint32_t code) {
  // (a satisfied wait is the common case: one non-blocking look costs less than the blocking form)
  if (mbar_test(bar, parity)) return true;
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicOr(err, code);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(tmap), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// tcgen05.ld of 64 columns + wait, delivered as 32 register pairs (columns 2i, 2i+1) for the f32x2 arithmetic.  The
// load, the wait and the moves are one asm block: nothing that uses the values can be scheduled before the wait.
__device__ __forceinline__ void tc_ld64_pairs(uint32_t taddr, unsigned long long (&r)[32]) {
  asm volatile(
      "{\n\t.reg .b32 t<64>;\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {t0,t1,t2,t3,t4,t5,t6,t7,t8,t9,t10,t11,t12,t13,t14,t15,t16,t17,t18,t19,t20,t21,t22,t23,t24,t25,t26,t27,t28,t29,t30,t31,t32,t33,t34,t35,t36,t37,t38,t39,t40,t41,t42,t43,t44,t45,t46,t47,t48,t49,t50,t51,t52,t53,t54,t55,t56,t57,t58,t59,t60,t61,t62,t63}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n\t"
      "mov.b64 %0, {t0,t1};\n\t"
      "mov.b64 %1, {t2,t3};\n\t"
      "mov.b64 %2, {t4,t5};\n\t"
      "mov.b64 %3, {t6,t7};\n\t"
      "mov.b64 %4, {t8,t9};\n\t"
      "mov.b64 %5, {t10,t11};\n\t"
      "mov.b64 %6, {t12,t13};\n\t"
      "mov.b64 %7, {t14,t15};\n\t"
      "mov.b64 %8, {t16,t17};\n\t"
      "mov.b64 %9, {t18,t19};\n\t"
      "mov.b64 %10, {t20,t21};\n\t"
      "mov.b64 %11, {t22,t23};\n\t"
      "mov.b64 %12, {t24,t25};\n\t"
      "mov.b64 %13, {t26,t27};\n\t"
      "mov.b64 %14, {t28,t29};\n\t"
      "mov.b64 %15, {t30,t31};\n\t"
      "mov.b64 %16, {t32,t33};\n\t"
      "mov.b64 %17, {t34,t35};\n\t"
      "mov.b64 %18, {t36,t37};\n\t"
      "mov.b64 %19, {t38,t39};\n\t"
      "mov.b64 %20, {t40,t41};\n\t"
      "mov.b64 %21, {t42,t43};\n\t"
      "mov.b64 %22, {t44,t45};\n\t"
      "mov.b64 %23, {t46,t47};\n\t"
      "mov.b64 %24, {t48,t49};\n\t"
      "mov.b64 %25, {t50,t51};\n\t"
      "mov.b64 %26, {t52,t53};\n\t"
      "mov.b64 %27, {t54,t55};\n\t"
      "mov.b64 %28, {t56,t57};\n\t"
      "mov.b64 %29, {t58,t59};\n\t"
      "mov.b64 %30, {t60,t61};\n\t"
      "mov.b64 %31, {t62,t63};\n\t"
      "}"
      : "=l"(r[0]), "=l"(r[1]), "=l"(r[2]), "=l"(r[3]), "=l"(r[4]), "=l"(r[5]), "=l"(r[6]), "=l"(r[7]), "=l"(r[8]), "=l"(r[9]), "=l"(r[10]), "=l"(r[11]), "=l"(r[12]), "=l"(r[13]), "=l"(r[14]), "=l"(r[15]), "=l"(r[16]), "=l"(r[17]), "=l"(r[18]), "=l"(r[19]), "=l"(r[20]), "=l"(r[21]), "=l"(r[22]), "=l"(r[23]), "=l"(r[24]), "=l"(r[25]), "=l"(r[26]), "=l"(r[27]), "=l"(r[28]), "=l"(r[29]), "=l"(r[30]), "=l"(r[31])
      : "r"(taddr)
      : "memory");
}
// the same for 32 columns (16 register pairs): for readers that are short of registers
__device__ __forceinline__ void tc_ld32_pairs(uint32_t taddr, unsigned long long (&r)[16]) {
  asm volatile(
      "{\n\t.reg .b32 t<32>;\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {t0,t1,t2,t3,t4,t5,t6,t7,t8,t9,t10,t11,t12,t13,t14,t15,t16,t17,t18,t19,t20,t21,t22,t23,t24,t25,t26,t27,t28,t29,t30,t31}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n\t"
      "mov.b64 %0, {t0,t1};\n\t"
      "mov.b64 %1, {t2,t3};\n\t"
      "mov.b64 %2, {t4,t5};\n\t"
      "mov.b64 %3, {t6,t7};\n\t"
      "mov.b64 %4, {t8,t9};\n\t"
      "mov.b64 %5, {t10,t11};\n\t"
      "mov.b64 %6, {t12,t13};\n\t"
      "mov.b64 %7, {t14,t15};\n\t"
      "mov.b64 %8, {t16,t17};\n\t"
      "mov.b64 %9, {t18,t19};\n\t"
      "mov.b64 %10, {t20,t21};\n\t"
      "mov.b64 %11, {t22,t23};\n\t"
      "mov.b64 %12, {t24,t25};\n\t"
      "mov.b64 %13, {t26,t27};\n\t"
      "mov.b64 %14, {t28,t29};\n\t"
      "mov.b64 %15, {t30,t31};\n\t"
      "}"
      : "=l"(r[0]), "=l"(r[1]), "=l"(r[2]), "=l"(r[3]), "=l"(r[4]), "=l"(r[5]), "=l"(r[6]), "=l"(r[7]), "=l"(r[8]), "=l"(r[9]), "=l"(r[10]), "=l"(r[11]), "=l"(r[12]), "=l"(r[13]), "=l"(r[14]), "=l"(r[15])
      : "r"(taddr)
      : "memory");
}
// packed f32x2 arithmetic (two IEEE round-to-nearest operations per instruction)
__device__ __forceinline__ void ffma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long fmul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long pack2(float x) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
  return r;
}
// up * silu(gate) (zero/kernels/gemm.cl:562-565).  Out of line on purpose: the epilogues call it 64 and 32 times per
// thread, and the role loops of the kernel compete for the instruction cache.
__device__ __noinline__ float swiglu_mul(float g, float u) { return __fmul_rn(u, __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)))); }
__device__ __forceinline__ unsigned long long pack_pair(float lo, float hi) {
  return (unsigned long long)__float_as_uint(lo) | ((unsigned long long)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ float lo_f(unsigned long long a) { return __uint_as_float((uint32_t)a); }
__device__ __forceinline__ float hi_f(unsigned long long a) { return __uint_as_float((uint32_t)(a >> 32)); }

// K-major operand tile of 128-byte rows, 128-byte swizzle: 8-row groups 1024 bytes apart (tcgen05 shared-memory
// descriptor: start address >> 4, stride byte offset >> 4 at bit 32, descriptor version 1 at bit 46, swizzle mode 2
// (128 B) at bit 61; the leading byte offset is not used when the MMA's K extent lies inside one swizzled row).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::f16: D = f32 (bit 4), A/B format at bits 7 / 10 (0 fp16, 1 bf16), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t kIdescF16 = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t kIdescBF16 = kIdescF16 | (1u << 7) | (1u << 10);

// position p (0..7) inside a 16-byte chunk of the Q4_K operand row holds element perm8[p] of that group of eight:
// the order in which the dequantiser's two-nibbles-per-word extraction delivers them
__device__ __forceinline__ int q4k_perm8(int p) { return (p & 4) | ((p & 1) << 1) | ((p >> 1) & 1); }

// ---------------------------------------------------------------------------------------------- activation pre-pass
// Per 128-row tile: fp16 operand images (one 16 KB swizzled stage per 64 elements of K), the tile's activation scales
// and, with sps == 5 (the Q4_K GEMM), after every four stages one more 16 KB image: the min-term factor
// v = asc * (float)asum of the superblock's eight blocks as three bf16 terms, laid out as the six 16-byte K-chunks
// (v1, v1, v2, v1, v2, v3) x eight blocks that meet the weight side's (u1, u2, u1, u3, u2, u1).
// One thread per (row, 16-byte output chunk).
template <int QT>
__global__ void __launch_bounds__(256) act_prepare_kernel(const int8_t* __restrict__ aq, const float* __restrict__ asc, int lda,
                                                          int K, int rows_total, const int32_t* __restrict__ tiles,
                                                          const int32_t* __restrict__ rowmap, uint16_t* __restrict__ aimg,
                                                          float* __restrict__ ascimg, int sps) {
  const int tile = blockIdx.y;
  int r0, nr;
  if (tiles) {
    if (tile >= tiles[0]) return;
    r0 = tiles[2 + 3 * tile];
    nr = tiles[3 + 3 * tile];
  } else {
    r0 = tile * BM;
    nr = min(BM, rows_total - r0);
  }
  const int nchunk = K / 8;                      // 16-byte output chunks per row
  const int idx = blockIdx.x * 256 + threadIdx.x;  // over 128 rows x nchunk, chunk fastest
  if (idx >= BM * nchunk) return;
  const int r = idx / nchunk, ch = idx % nchunk;
  const int stage = ch >> 3, c = ch & 7;
  int src = -1;
  if (r < nr) src = rowmap ? rowmap[r0 + r] : r0 + r;
  uint2 v = make_uint2(0, 0);
  if (src >= 0) v = *reinterpret_cast<const uint2*>(aq + (size_t)src * K + (size_t)ch * 8);
  int a[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a[i] = (int)(int8_t)(v.x >> (8 * i));
    a[4 + i] = (int)(int8_t)(v.y >> (8 * i));
  }
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e0 = QT == IZB_Q4_K ? q4k_perm8(2 * i) : 2 * i, e1 = QT == IZB_Q4_K ? q4k_perm8(2 * i + 1) : 2 * i + 1;
    const __half2 h = __floats2half2_rn((float)a[e0], (float)a[e1]);
    o[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  const size_t nstages = (size_t)(K / 256) * sps;
  uint8_t* tile_img = reinterpret_cast<uint8_t*>(aimg) + (size_t)tile * nstages * STAGE_BYTES;
  uint8_t* dst = tile_img + ((size_t)(stage >> 2) * sps + (stage & 3)) * STAGE_BYTES + r * 128 + ((c ^ (r & 7)) << 4);
  *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
  if (asc) {  // (null in the block-dot verification mode: no scales are used)
    int s = a[0] + a[1] + a[2] + a[3] + a[4] + a[5] + a[6] + a[7];
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);  // the four chunks of a 32-block are four consecutive threads of one row
    if ((ch & 3) == 0) {
      const int b = ch >> 2;
      const float sc = src >= 0 ? asc[(size_t)b * lda + src] : 0.0f;
      ascimg[((size_t)tile * (K / 32) + b) * BM + r] = sc;
      if (QT == IZB_Q4_K && sps == 5) {
        const float v = __fmul_rn(sc, (float)s);
        const __nv_bfloat16 h1 = __float2bfloat16_rn(v);
        const float r1 = __fsub_rn(v, __bfloat162float(h1));
        const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
        const __nv_bfloat16 h3 = __float2bfloat16_rn(__fsub_rn(r1, __bfloat162float(h2)));
        uint8_t* row = tile_img + ((size_t)(b >> 3) * 5 + 4) * STAGE_BYTES + r * 128 + 2 * (b & 7);
        const unsigned short t3[3] = {__bfloat16_as_ushort(h1), __bfloat16_as_ushort(h2), __bfloat16_as_ushort(h3)};
        constexpr int term[6] = {0, 0, 1, 0, 1, 2};
#pragma unroll
        for (int k = 0; k < 6; ++k) *reinterpret_cast<unsigned short*>(row + ((k ^ (r & 7)) << 4)) = t3[term[k]];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- quantiser + pre-pass in one
// izb_quantize_act (csrc/izb_quantize.cu, the arithmetic of quantize_act_cpu, src/quants.h:626-643, bit for bit) and
// act_prepare_kernel above in one pass over the f32 rows: a lane owns 8 consecutive values (= one 16-byte operand chunk),
// four lanes a 32-block.  Writes aq / asc exactly as the quantiser does (the caller's buffers stay valid for every other
// kernel) and, from the same registers, the operand images, the gathered scales and the min-term factors of the dense
// tensor-core GEMM: the int8 rows are not read back and the second launch is gone.  One CTA = 32 rows x one superblock.
template <int QT>
__global__ void __launch_bounds__(256) quant_prepare_kernel(const float* __restrict__ x, int ldx, int M, int Mp, int K,
                                                            int8_t* __restrict__ aq, float* __restrict__ asc,
                                                            uint16_t* __restrict__ aimg, float* __restrict__ ascimg, int sps, int n_tiles) {
  __shared__ float s_sc[8][33];
  const int sb = blockIdx.x, m0 = blockIdx.y * 32, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = sb * 256 + lane * 8;
  const size_t nstages = (size_t)(K / 256) * sps;
  float v[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + warp + 8 * i;
    if (m < M) {
      const float4* p = reinterpret_cast<const float4*>(x + (size_t)m * ldx + col);
      const float4 a = __ldcs(p), b = __ldcs(p + 1);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
      v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[i][k] = 0.0f;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = warp + 8 * i, m = m0 + rr;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[i][k]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int q[8], s = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float pr = __fmul_rn(v[i][k], inv);
      q[k] = fabsf(pr) <= 2147483520.0f ? __float2int_rn(pr) : 0;  // (see quantize_act_kernel: the overflow case)
      q[k] = (int)(int8_t)q[k];  // the stored byte is what the GEMM multiplies
      s += q[k];
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    const float sc = __fdiv_rn(amax, 127.0f);
    if (m < Mp) {
      uint2 pk;
      pk.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
      pk.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
      *reinterpret_cast<uint2*>(aq + (size_t)m * K + col) = pk;
    }
    if ((lane & 3) == 0) s_sc[lane >> 2][rr] = sc;
    // ---- the operand image of this chunk: tile m / 128, row m % 128, stage lane / 8 of the superblock, chunk lane % 8
    const int tile = m >> 7, r = m & 127;
    if (tile >= n_tiles) continue;  // (padding rows past the last tile the GEMM reads: aq / asc only)
    uint8_t* tile_img = reinterpret_cast<uint8_t*>(aimg) + (size_t)tile * nstages * STAGE_BYTES;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e0 = QT == IZB_Q4_K ? q4k_perm8(2 * j) : 2 * j, e1 = QT == IZB_Q4_K ? q4k_perm8(2 * j + 1) : 2 * j + 1;
      const __half2 h = __floats2half2_rn((float)q[e0], (float)q[e1]);
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(tile_img + ((size_t)sb * sps + (lane >> 3)) * STAGE_BYTES + r * 128 + (((lane & 7) ^ (r & 7)) << 4)) =
        make_uint4(o[0], o[1], o[2], o[3]);
    if ((lane & 3) == 0) {
      const int b = lane >> 2;  // block of the superblock
      ascimg[((size_t)tile * (K / 32) + sb * 8 + b) * BM + r] = sc;
      if (QT == IZB_Q4_K && sps == 5) {
        const float t = __fmul_rn(sc, (float)s);
        const __nv_bfloat16 h1 = __float2bfloat16_rn(t);
        const float r1 = __fsub_rn(t, __bfloat162float(h1));
        const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
        const __nv_bfloat16 h3 = __float2bfloat16_rn(__fsub_rn(r1, __bfloat162float(h2)));
        uint8_t* row = tile_img + ((size_t)sb * 5 + 4) * STAGE_BYTES + r * 128 + 2 * b;
        const unsigned short t3[3] = {__bfloat16_as_ushort(h1), __bfloat16_as_ushort(h2), __bfloat16_as_ushort(h3)};
        constexpr int term[6] = {0, 0, 1, 0, 1, 2};
#pragma unroll
        for (int k = 0; k < 6; ++k) *reinterpret_cast<unsigned short*>(row + ((k ^ (r & 7)) << 4)) = t3[term[k]];
      }
    }
  }
  __syncthreads();
  {
    const int b = threadIdx.x >> 5, r = threadIdx.x & 31;
    if (m0 + r < Mp) asc[(size_t)(sb * 8 + b) * Mp + m0 + r] = s_sc[b][r];
  }
}

// ---------------------------------------------------------------------------------------------- the GEMM kernel
template <int QT, bool kDots>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using MP = Map<QT>;
  constexpr int NA = MP::NA, NB = MP::NB, OFF_A = MP::OFF_A, OFF_B = MP::OFF_B, OFF_RAW = MP::OFF_RAW, OFF_DM = MP::OFF_SCL,
                OFF_D8 = MP::OFF_SCL, OFF_ASC = MP::OFF_ASC, OFF_BAR = MP::OFF_BAR, NUM_BARS = MP::NUM_BARS;
  constexpr int A_FULL = MP::A_FULL, A_EMPTY = MP::A_EMPTY, B_FULL = MP::B_FULL, B_EMPTY = MP::B_EMPTY, RAW_FULL = MP::RAW_FULL,
                RAW_EMPTY = MP::RAW_EMPTY, D1_FULL = MP::D1_FULL, D1_EMPTY = MP::D1_EMPTY, D2_FULL = MP::D2_FULL,
                D2_EMPTY = MP::D2_EMPTY, ASC_FULL = MP::ASC_FULL, ASC_EMPTY = MP::ASC_EMPTY;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NUM_BARS * 8);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + NUM_BARS * 8 + 4);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) -> uint32_t { return bar0 + 8u * (uint32_t)i; };

  // ---- the CTA's work: output tiles blockIdx.x, blockIdx.x + gridDim.x, ... of (row tiles) x (N / 128 column tiles), column
  // tile fastest.  Every role walks the same list; its ring positions and barrier parities run on from tile to tile, so
  // the producers, the dequantisers and the MMA issuers are already inside the next tile while the combine warps
  // store the current one.
  const int n_ntiles = p.N / BN;
  const int n_work = (p.tiles ? p.tiles[0] : p.n_mtiles) * n_ntiles;
  if ((int)blockIdx.x >= n_work) return;  // uniform over the CTA, before any barrier or TMEM use
  const int nsb = p.K >> 8, nb = p.K >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int SBB = QT == IZB_Q4_K ? 144 : 272;
  constexpr int RAW = MP::RAW, NR = MP::NR;
  constexpr bool kMins = QT == IZB_Q4_K && !kDots;
  constexpr int SPS = kMins ? 5 : 4;  // operand stages per superblock: four of 64 K-elements (+ the min-term stage)
  const int nstages = SPS * nsb;

  if (threadIdx.x == 0) {
    // Consumers release a buffer with one arrival per THREAD, not per warp: an elected lane costs a divergent branch and a
    // warp barrier per hand-over, which measured 10 % of the kernel (and one predicated arrival per warp measured no
    // better than 32).  A_FULL: the activation producer's expect_tx arrival; B_FULL: the 128 dequantiser threads;
    // A_EMPTY / B_EMPTY: one tcgen05.commit each
    constexpr int kDeqArr = 128, kCmbArr = 256;
    for (int i = 0; i < NA; ++i) { mbar_init(bar(A_FULL + i), 1); mbar_init(bar(A_EMPTY + i), 1); }
    for (int i = 0; i < NB; ++i) { mbar_init(bar(B_FULL + i), kDeqArr); mbar_init(bar(B_EMPTY + i), 1); }
    for (int i = 0; i < NR; ++i) { mbar_init(bar(RAW_FULL + i), 1); mbar_init(bar(RAW_EMPTY + i), kDeqArr); }
    for (int i = 0; i < ND1; ++i) { mbar_init(bar(D1_FULL + i), 1); mbar_init(bar(D1_EMPTY + i), kCmbArr); }
    mbar_init(bar(D2_FULL), 1);
    mbar_init(bar(D2_EMPTY), kCmbArr);
    for (int i = 0; i < NASC; ++i) { mbar_init(bar(ASC_FULL + i), 1); mbar_init(bar(ASC_EMPTY + i), kCmbArr); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    // Every role loop below is executed by its whole warp (uniform waits, lane 0 issues), so no lane of a role warp
    // sits at the final CTA barrier while another lane of the same warp is still working.
    if (warp == 0) {
      // ================= activation producer: the tile's stage images lie back to back in global memory
      int sa = 0, pa = 1;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const int tile = w / n_ntiles;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.aimg) + (size_t)tile * nstages * STAGE_BYTES;
        for (int g = 0; g < nstages; ++g) {
          if (!mbar_wait(bar(A_EMPTY + sa), pa, abort_flag, p.err, p.spin_limit, E_APROD)) { ok = false; break; }
          if (lane == 0 && g != p.skip_stage) {  // (skip_stage: diagnostics only, makes the waits of this stage run out)
            mbar_expect_tx(bar(A_FULL + sa), STAGE_BYTES);
            bulk_g2s(smem_u32(smem + OFF_A + sa * STAGE_BYTES), src + (size_t)g * STAGE_BYTES, STAGE_BYTES, bar(A_FULL + sa));
          }
          __syncwarp();
          if (++sa == NA) { sa = 0; pa ^= 1; }
        }
      }
    } else if (warp == 3) {
      // ================= weight producer: TMA of the raw superblocks of the tile's 128 weight rows, and per superblock the
      // 8 x 128 activation scales the combine warps need
      int rb = 0, pr = 1, sq = 0, pq = 1;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
      const int tile = w / n_ntiles;
      const int wrow = (p.tiles ? p.tiles[1 + 3 * tile] : p.mat) * p.N + (w % n_ntiles) * BN;
      for (int s = 0; s < nsb; ++s) {
        if (!mbar_wait(bar(RAW_EMPTY + rb), pr, abort_flag, p.err, p.spin_limit, E_WPROD)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(bar(RAW_FULL + rb), RAW);
          tma_2d(smem_u32(smem + OFF_RAW + rb * RAW), &tmW, s * (SBB / 4), wrow, bar(RAW_FULL + rb));
        }
        if (++rb == NR) { rb = 0; pr ^= 1; }
        if (!kDots) {
          if (!mbar_wait(bar(ASC_EMPTY + sq), pq, abort_flag, p.err, p.spin_limit, E_WPROD)) { ok = false; break; }
          if (lane == 0) {
            mbar_expect_tx(bar(ASC_FULL + sq), 4096);
            bulk_g2s(smem_u32(smem + OFF_ASC + sq * 4096), p.ascimg + ((size_t)tile * nb + 8 * s) * BM, 4096, bar(ASC_FULL + sq));
          }
          if (++sq == NASC) { sq = 0; pq ^= 1; }
        }
        __syncwarp();
      }
      }
    } else {
      // ================= MMA issuers.  Of a superblock's stages 0..3 (two 32-blocks each, every block into its own
      // accumulator buffer: two MMAs of K = 16 + one commit) warp 1 takes 0 and 2, warp 2 takes 1, 3 and the min-term stage 4
      // (three bf16 MMAs of K = 16 accumulated into the fourth TMEM buffer over the whole of K).  Two issuers because
      // what a thread pays per block -- barrier polls and commits between MMAs -- is longer than the 128 cycles the two
      // MMAs run; one issuer for the min term so that its accumulator is updated in program order.
      bool ok = true;
      int it = 0;  // tiles done: stage and block counts run on across tiles
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) {
      const int gs = it * nstages, jb = it * nb;
      for (int s = 0; s < nsb && ok; ++s) {
        for (int t = warp - 1; t < (warp == 1 ? 4 : SPS) && ok; t += (t == 3 ? 1 : 2)) {
          const int g = gs + SPS * s + t, sa = g % NA, sb = g % NB;
          TRACE(10, g);
          if (!mbar_wait(bar(B_FULL + sb), (g / NB) & 1, abort_flag, p.err, p.spin_limit, E_MMA)) { ok = false; break; }
          TRACE(11, g);
          if (!mbar_wait(bar(A_FULL + sa), (g / NA) & 1, abort_flag, p.err, p.spin_limit, E_MMA)) { ok = false; break; }
          TRACE(12, g);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + OFF_A + sa * STAGE_BYTES), b_addr = smem_u32(smem + OFF_B + sb * STAGE_BYTES);
          if (t < 4) {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              const int j = jb + 8 * s + 2 * t + blk, d = j % ND1;
              TRACE(0, j);
              if (!mbar_wait(bar(D1_EMPTY + d), ((j / ND1) & 1) ^ 1, abort_flag, p.err, p.spin_limit, E_MMA)) { ok = false; break; }
              TRACE(1, j);
              tc_fence_after();
              if (lane == 0) {
                const uint32_t dt = tmem_base + (uint32_t)(d * BN);
#pragma unroll
                for (int k16 = 0; k16 < 2; ++k16)
                  tc_mma_f16(dt, umma_desc(a_addr + blk * 64 + k16 * 32), umma_desc(b_addr + blk * 64 + k16 * 32), kIdescF16, k16);
                tc_commit(bar(D1_FULL + d));
              }
              TRACE(2, j);
              __syncwarp();
            }
            if (!ok) break;
          } else {
            // the min-term accumulator of the tile before must have been read before this tile's first MMA clears it
            if (s == 0 && it > 0 && !mbar_wait(bar(D2_EMPTY), (it - 1) & 1, abort_flag, p.err, p.spin_limit, E_MMA)) { ok = false; break; }
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
              for (int k16 = 0; k16 < 3; ++k16)
                tc_mma_f16(tmem_base + ND1 * BN, umma_desc(a_addr + k16 * 32), umma_desc(b_addr + k16 * 32), kIdescBF16, (s | k16) ? 1u : 0u);
            }
          }
          if (lane == 0) {
            tc_commit(bar(A_EMPTY + sa));
            tc_commit(bar(B_EMPTY + sb));
            if (kMins && t == 4 && s == nsb - 1) tc_commit(bar(D2_FULL));
          }
          __syncwarp();
        }
      }
      }
    }
  } else if (warp < 8) {
    // ================= dequantisers: thread t <-> weight row n0 + t
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    const int t = threadIdx.x - 128;
    bool ok = true;
    int sbq = 0, pbq = 1;  // operand ring position and wait parity
    int rb = 0, pr = 0;    // raw ring
    int sbc = 0;           // superblocks done (all tiles): position in the 4-deep ring of superblock scales
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x)
    for (int s = 0; s < nsb && ok; ++s, ++sbc) {
      if (!mbar_wait(bar(RAW_FULL + rb), pr, abort_flag, p.err, p.spin_limit, E_DEQ)) { ok = false; break; }
      const unsigned char* rrow = smem + OFF_RAW + rb * RAW + t * SBB;
      const uint4 hdr = *reinterpret_cast<const uint4*>(rrow);
      const uint32_t s3[3] = {hdr.y, hdr.z, hdr.w};
      if (QT == IZB_Q4_K) {
        if (kMins) reinterpret_cast<float*>(smem + OFF_DM + (sbc & 3) * 512)[t] = half_bits_to_float(hdr.x & 0xFFFFu);
      } else {
        float* d8 = reinterpret_cast<float*>(smem + OFF_D8 + (sbc & 3) * 4096);
        const uint32_t hw[4] = {hdr.x, hdr.y, hdr.z, hdr.w};
#pragma unroll
        for (int b = 0; b < 8; ++b) d8[b * 128 + t] = half_bits_to_float((b & 1) ? hw[b >> 1] >> 16 : hw[b >> 1] & 0xFFFFu);
      }
#pragma unroll 1  // (rolled on purpose: with the role loops resident at once, code size costs more than the loop)
      for (int c = 0; c < 4; ++c) {
        if (warp == 4) TRACE(7, sbc * SPS + c);
        if (!mbar_wait(bar(B_EMPTY + sbq), pbq, abort_flag, p.err, p.spin_limit, E_DEQ)) { ok = false; break; }
        if (warp == 4) TRACE(8, sbc * SPS + c);
        unsigned char* orow = smem + OFF_B + sbq * STAGE_BYTES + t * 128;
        if (QT == IZB_Q4_K) {
          const uint4 q0 = *reinterpret_cast<const uint4*>(rrow + 16 + 32 * c), q1 = *reinterpret_cast<const uint4*>(rrow + 32 + 32 * c);
          const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
          // the chunk's two 6-bit sub-block scales as half2 pairs (sc, sc) and (-1024 sc, -1024 sc): 0x6400 | sc is the
          // fp16 number 1024 + sc
          int sc_lo = 1, sc_hi = 1, mn_unused;
          if (!kDots) {
            q4k_scale_min(s3, 2 * c, sc_lo, mn_unused);
            q4k_scale_min(s3, 2 * c + 1, sc_hi, mn_unused);
          }
          const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400)), kneg = __half2half2(__ushort_as_half((unsigned short)0xE400));
          const uint32_t blo = 0x64006400u | (uint32_t)sc_lo | ((uint32_t)sc_lo << 16), bhi = 0x64006400u | (uint32_t)sc_hi | ((uint32_t)sc_hi << 16);
          const __half2 slo = __hsub2(*reinterpret_cast<const __half2*>(&blo), k1024), shi = __hsub2(*reinterpret_cast<const __half2*>(&bhi), k1024);
          const __half2 nlo = __hmul2(slo, kneg), nhi = __hmul2(shi, kneg);
          // High nibbles stay where they are: (word & 0x00F000F0) | 0x6400 is the fp16 number 1024 + 16 q, and
          // (1024 + 16 q) * (sc / 16) - 64 sc = sc * q exactly (one rounding, of an integer below 2^11).  One shift per
          // word (for its upper bytes) instead of three.
          const __half2 k16th = __half2half2(__ushort_as_half((unsigned short)0x2C00));  // 1 / 16
          const __half2 shi16 = __hmul2(shi, k16th), nhi16 = __hmul2(nhi, k16th);
          auto cv = [](uint32_t word, uint32_t mask, __half2 scale, __half2 neg) -> uint32_t {
            const uint32_t bitsv = (word & mask) | 0x64006400u;
            const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&bitsv), scale, neg);
            return *reinterpret_cast<const uint32_t*>(&r);
          };
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint32_t w0 = w[2 * jj], w1 = w[2 * jj + 1], x0 = w0 >> 8, x1 = w1 >> 8;
            *reinterpret_cast<uint4*>(orow + ((jj ^ (t & 7)) << 4)) =
                make_uint4(cv(w0, 0x000F000Fu, slo, nlo), cv(x0, 0x000F000Fu, slo, nlo), cv(w1, 0x000F000Fu, slo, nlo), cv(x1, 0x000F000Fu, slo, nlo));
            *reinterpret_cast<uint4*>(orow + (((4 + jj) ^ (t & 7)) << 4)) =
                make_uint4(cv(w0, 0x00F000F0u, shi16, nhi16), cv(x0, 0x00F000F0u, shi16, nhi16), cv(w1, 0x00F000F0u, shi16, nhi16), cv(x1, 0x00F000F0u, shi16, nhi16));
          }
        } else {
          const __half2 bias = __half2half2(__int2half_rn(1152));
          auto cvt = [&](uint32_t x, uint32_t sel) -> uint32_t {
            const uint32_t bitsv = __byte_perm(x, 0x64646464u, sel);  // (1024 + (q + 128)) in both halves
            const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&bitsv), bias);
            return *reinterpret_cast<const uint32_t*>(&r);
          };
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint4 q = *reinterpret_cast<const uint4*>(rrow + 16 + 64 * c + 16 * jj);
            const uint32_t x0 = q.x ^ 0x80808080u, x1 = q.y ^ 0x80808080u, x2 = q.z ^ 0x80808080u, x3 = q.w ^ 0x80808080u;
            *reinterpret_cast<uint4*>(orow + (((2 * jj) ^ (t & 7)) << 4)) =
                make_uint4(cvt(x0, 0x4140), cvt(x0, 0x4342), cvt(x1, 0x4140), cvt(x1, 0x4342));
            *reinterpret_cast<uint4*>(orow + (((2 * jj + 1) ^ (t & 7)) << 4)) =
                make_uint4(cvt(x2, 0x4140), cvt(x2, 0x4342), cvt(x3, 0x4140), cvt(x3, 0x4342));
          }
        }
        fence_proxy_async();
        mbar_arrive(bar(B_FULL + sbq));  // (every thread after its own stores and fence)
        if (warp == 4) TRACE(9, sbc * SPS + c);
        if (++sbq == NB) { sbq = 0; pbq ^= 1; }
      }
      if (!ok) break;
      if (kMins) {
        // the min-term stage: u[b] = -dmin * mn[b] (exact in f32: 11 x 6 bits) as three bf16 terms u1 + u2 + u3; the
        // stage's six 16-byte chunks hold (u1, u2, u1, u3, u2, u1) for the eight blocks, against the activation side's
        // (v1, v1, v2, v1, v2, v3)
        if (!mbar_wait(bar(B_EMPTY + sbq), pbq, abort_flag, p.err, p.spin_limit, E_DEQ)) { ok = false; break; }
        const float ndmin = -half_bits_to_float(hdr.x >> 16);
        uint32_t u1[4], u2[4], u3[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t h[2][3];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            int sc_unused, mn;
            q4k_scale_min(s3, 2 * k + e, sc_unused, mn);
            const float u = __fmul_rn(ndmin, (float)mn);
            const __nv_bfloat16 h1 = __float2bfloat16_rn(u);
            const float r1 = __fsub_rn(u, __bfloat162float(h1));
            const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
            const __nv_bfloat16 h3 = __float2bfloat16_rn(__fsub_rn(r1, __bfloat162float(h2)));
            h[e][0] = __bfloat16_as_ushort(h1);
            h[e][1] = __bfloat16_as_ushort(h2);
            h[e][2] = __bfloat16_as_ushort(h3);
          }
          u1[k] = h[0][0] | (h[1][0] << 16);
          u2[k] = h[0][1] | (h[1][1] << 16);
          u3[k] = h[0][2] | (h[1][2] << 16);
        }
        unsigned char* orow = smem + OFF_B + sbq * STAGE_BYTES + t * 128;
        const uint4 c1 = make_uint4(u1[0], u1[1], u1[2], u1[3]), c2 = make_uint4(u2[0], u2[1], u2[2], u2[3]), c3 = make_uint4(u3[0], u3[1], u3[2], u3[3]);
        *reinterpret_cast<uint4*>(orow + ((0 ^ (t & 7)) << 4)) = c1;
        *reinterpret_cast<uint4*>(orow + ((1 ^ (t & 7)) << 4)) = c2;
        *reinterpret_cast<uint4*>(orow + ((2 ^ (t & 7)) << 4)) = c1;
        *reinterpret_cast<uint4*>(orow + ((3 ^ (t & 7)) << 4)) = c3;
        *reinterpret_cast<uint4*>(orow + ((4 ^ (t & 7)) << 4)) = c2;
        *reinterpret_cast<uint4*>(orow + ((5 ^ (t & 7)) << 4)) = c1;
        fence_proxy_async();
        mbar_arrive(bar(B_FULL + sbq));  // (every thread after its own stores and fence)
        if (++sbq == NB) { sbq = 0; pbq ^= 1; }
      }
      mbar_arrive(bar(RAW_EMPTY + rb));
      if (++rb == NR) { rb = 0; pr ^= 1; }
    }
  } else {
    // ================= combine: thread <-> TMEM lane (token row) 32*(warp%4) + lane, 64 of the 128 columns.
    // All f32 arithmetic is done on register pairs (fma.rn.f32x2): half the instructions for the same IEEE results.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int q = warp & 3, half = (warp - 8) >> 2;
    const int r = 32 * q + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(half * 64);
    bool ok = true;
    int d = 0, pd = 0, sq = 0, pq = 0;  // accumulator ring / scale ring positions and wait parities
    int sbc = 0, it = 0;                // superblocks and tiles done
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) {
    const int tile = w / n_ntiles, n0 = (w % n_ntiles) * BN;
    const int r0 = p.tiles ? p.tiles[2 + 3 * tile] : tile * BM;
    const int nr = p.tiles ? p.tiles[3 + 3 * tile] : min(BM, p.M - r0);
    const bool row_ok = r < nr;
    const int out_row = r0 + r;
    unsigned long long res2[32], tq2[32];  // pairs of columns (2i, 2i+1)
#pragma unroll
    for (int c = 0; c < 32; ++c) res2[c] = tq2[c] = 0ull;
    for (int s = 0; s < nsb && ok; ++s, ++sbc) {
      const float* as = reinterpret_cast<const float*>(smem + OFF_ASC + sq * 4096) + r;  // this row's 8 block scales
      if (!kDots && !mbar_wait(bar(ASC_FULL + sq), pq, abort_flag, p.err, p.spin_limit, E_EPI)) { ok = false; break; }
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const unsigned long long a2 = pack2(kDots ? 0.0f : as[b * BM]);
        if (warp == 8) TRACE(3, sbc * 8 + b);
        if (!mbar_wait(bar(D1_FULL + d), pd, abort_flag, p.err, p.spin_limit, E_EPI)) { ok = false; break; }
        if (warp == 8) TRACE(4, sbc * 8 + b);
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // 32 columns at a time: the block loop's working set stays inside the register budget
          unsigned long long v[16];
          tc_ld32_pairs(t_lane + (uint32_t)(d * BN + 32 * h), v);
          if (h == 1) {
            tc_fence_before();
            if (warp == 8) TRACE(5, sbc * 8 + b);
            mbar_arrive(bar(D1_EMPTY + d));  // the accumulator buffer may be overwritten
          }
          if (kDots) {
            if (row_ok) {
              int32_t* o = p.dots + ((size_t)out_row * p.N + n0 + half * 64 + 32 * h) * nb + 8 * s + b;
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                o[(size_t)(2 * c) * nb] = __float2int_rn(lo_f(v[c]));
                o[(size_t)(2 * c + 1) * nb] = __float2int_rn(hi_f(v[c]));
              }
            }
          } else if (QT == IZB_Q4_K) {
            if (b == 0) {
#pragma unroll
              for (int c = 0; c < 16; ++c) tq2[16 * h + c] = fmul2(a2, v[c]);
            } else {
#pragma unroll
              for (int c = 0; c < 16; ++c) ffma2(tq2[16 * h + c], a2, v[c]);
            }
          } else {
            const ulonglong2* d8 = reinterpret_cast<const ulonglong2*>(smem + OFF_D8 + (sbc & 3) * 4096 + b * 512 + half * 256 + h * 128);
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              const ulonglong2 dd = d8[c4];  // four column scales
              ffma2(res2[16 * h + 2 * c4], fmul2(a2, dd.x), v[2 * c4]);
              ffma2(res2[16 * h + 2 * c4 + 1], fmul2(a2, dd.y), v[2 * c4 + 1]);
            }
          }
        }
        if (warp == 8) TRACE(6, sbc * 8 + b);
        if (++d == ND1) { d = 0; pd ^= 1; }
      }
      if (!ok) break;
      if (!kDots) {  // the superblock's scales are read: its ring slot may be refilled
        mbar_arrive(bar(ASC_EMPTY + sq));
        if (++sq == NASC) { sq = 0; pq ^= 1; }
      }
      if (kMins) {  // res += d * tq
        const ulonglong2* dv = reinterpret_cast<const ulonglong2*>(smem + OFF_DM + (sbc & 3) * 512 + half * 256);
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const ulonglong2 dd = dv[c4];
          ffma2(res2[2 * c4], dd.x, tq2[2 * c4]);
          ffma2(res2[2 * c4 + 1], dd.y, tq2[2 * c4 + 1]);
        }
      }
    }
    if (kMins && ok) {  // the min term of the whole row of K (already negative)
      ok = mbar_wait(bar(D2_FULL), it & 1, abort_flag, p.err, p.spin_limit, E_EPI);
      if (ok) {
        tc_fence_after();
        unsigned long long v[32];
        tc_ld64_pairs(t_lane + (uint32_t)(ND1 * BN), v);
        tc_fence_before();
        mbar_arrive(bar(D2_EMPTY));  // the next tile's min term may start
        const unsigned long long one2 = pack2(1.0f);
#pragma unroll
        for (int c = 0; c < 32; ++c) ffma2(res2[c], one2, v[c]);
      }
    }
    if (ok && !kDots && row_ok && !*abort_flag && p.acc == 3) {
      // Gate and up projections in one weight whose rows alternate in groups of 32 (izb_weight_create_gateup): this
      // thread's 64 columns are 32 gate outputs followed by the 32 up outputs of the same FFN rows, so the SwiGLU product
      // up * silu(gate) (zero/kernels/gemm.cl:562-565) is formed in registers and only the F-wide result is stored.
      float* cp = p.C + (size_t)out_row * p.ldc + p.c_off + (n0 >> 1) + half * 32;
      const bool wide = ((reinterpret_cast<uintptr_t>(cp) | ((size_t)p.ldc * 4)) & 31) == 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        unsigned long long o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned long long g2 = res2[4 * j + i], u2 = res2[16 + 4 * j + i];
          o[i] = pack_pair(swiglu_mul(lo_f(g2), lo_f(u2)), swiglu_mul(hi_f(g2), hi_f(u2)));
        }
        if (wide) {
          asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(cp + 8 * j), "l"(o[0]), "l"(o[1]), "l"(o[2]), "l"(o[3]) : "memory");
        } else {
          reinterpret_cast<float4*>(cp + 8 * j)[0] = make_float4(lo_f(o[0]), hi_f(o[0]), lo_f(o[1]), hi_f(o[1]));
          reinterpret_cast<float4*>(cp + 8 * j)[1] = make_float4(lo_f(o[2]), hi_f(o[2]), lo_f(o[3]), hi_f(o[3]));
        }
      }
    } else if (ok && !kDots && row_ok && !*abort_flag) {
      float* cp = p.C + (size_t)out_row * p.ldc + p.c_off + n0 + half * 64;
      const float rs = p.rowscale ? p.rowscale[out_row] : 1.0f;
      // plain store (with or without the row factor), 32-byte aligned rows: eight stores of one full 32-byte sector each
      // per thread
      if (p.acc == 0 && ((reinterpret_cast<uintptr_t>(cp) | ((size_t)p.ldc * 4)) & 31) == 0) {
        if (p.rowscale) {
          const unsigned long long rs2 = pack2(rs);
#pragma unroll
          for (int c = 0; c < 32; ++c) res2[c] = fmul2(rs2, res2[c]);
        }
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8)
          asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(cp + 8 * c8), "l"(res2[4 * c8]), "l"(res2[4 * c8 + 1]),
                       "l"(res2[4 * c8 + 2]), "l"(res2[4 * c8 + 3])
                       : "memory");
      } else
#pragma unroll
      for (int c4 = 0; c4 < 16; ++c4) {
        float4 v = make_float4(lo_f(res2[2 * c4]), hi_f(res2[2 * c4]), lo_f(res2[2 * c4 + 1]), hi_f(res2[2 * c4 + 1]));
        if (p.rowscale) { v.x = __fmul_rn(rs, v.x); v.y = __fmul_rn(rs, v.y); v.z = __fmul_rn(rs, v.z); v.w = __fmul_rn(rs, v.w); }
        float4* dst = reinterpret_cast<float4*>(cp) + c4;
        if (p.acc == 1) {
          const float4 o = *dst;
          v.x = __fadd_rn(v.x, o.x); v.y = __fadd_rn(v.y, o.y); v.z = __fadd_rn(v.z, o.z); v.w = __fadd_rn(v.w, o.w);
        } else if (p.acc == 2) {  // C holds the gate projection: C = v * silu(C)   (zero/kernels/gemm.cl:562-565)
          const float4 o = *dst;
          v.x = swiglu_mul(o.x, v.x);
          v.y = swiglu_mul(o.y, v.y);
          v.z = swiglu_mul(o.z, v.z);
          v.w = swiglu_mul(o.w, v.w);
        }
        *dst = v;
      }
    }
    }
  }
  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let copies and MMAs still in flight land before shared memory and TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Diagnostics hook (izb_debug_wait_test): the spin limit of the bounded waits and the operand stage the activation
// producer leaves out, for the NEXT launch only.
std::atomic<uint32_t> g_test_spin{0};
std::atomic<int> g_test_skip{-1};
std::atomic<unsigned long long*> g_test_trace{nullptr};

template <int QT, bool kDots>
int launch_tc(const izb_weight* w, TcParams& p, dim3 grid, cudaStream_t st) {
  constexpr int SMEM_BYTES = Map<QT>::SMEM_BYTES;
  IZB_SMEM_OPTIN((gemm_tc_kernel<QT, kDots>), SMEM_BYTES, w->device);
  const uint32_t spin = g_test_spin.exchange(0);
  p.spin_limit = spin ? spin : kSpinLimit;
  p.skip_stage = g_test_skip.exchange(-1);
  p.trace = g_test_trace.load();
  CUtensorMap tm;
  memcpy(&tm, w->tmap_raw, sizeof tm);
  IZB_LAUNCH("gemm_tc", st, gemm_tc_kernel<QT, kDots><<<grid, kThreads, SMEM_BYTES, st>>>(tm, p));
  return IZB_OK;
}

// persistent grid: one CTA per SM (shared memory allows no more), fewer when there are fewer tiles
int tc_grid(int device, int n_work) {
  const int sms = izb_sm_budget(device);
  return n_work < sms ? (n_work > 0 ? n_work : 1) : sms;
}

// scratch of one call: the operand images (sps stage images of 16 KB per superblock and tile) and the gathered scales
void tc_scratch_bytes(int n_tiles, int K, int sps, size_t* img_bytes, size_t* asc_bytes) {
  *img_bytes = (size_t)n_tiles * (K / 256) * sps * STAGE_BYTES;
  *asc_bytes = (size_t)n_tiles * (K / 32) * BM * 4;
}

// the activation pre-pass + the GEMM on scratch the caller owns (img_bytes + asc_bytes of tc_scratch_bytes)
int run_tc_on(const izb_weight* w, int mat, const int8_t* aq, const float* asc, int lda, int rows_total, const int32_t* tiles,
              int n_tiles_grid, const int32_t* rowmap, const float* rowscale, int M_store, float* C, int ldc, int c_off, int acc,
              int32_t* dots, void* ws, uint32_t* err, cudaStream_t st, bool reuse_images) {
  const int K = w->K;
  const int sps = (w->type == IZB_Q4_K && !dots) ? 5 : 4;
  size_t img_bytes, asc_bytes;
  tc_scratch_bytes(n_tiles_grid, K, sps, &img_bytes, &asc_bytes);
  uint16_t* aimg = (uint16_t*)ws;
  float* ascimg = (float*)((unsigned char*)ws + img_bytes);
  dim3 pg((BM * (K / 8) + 255) / 256, n_tiles_grid);
  if (reuse_images) {
  } else if (w->type == IZB_Q4_K)
    IZB_LAUNCH("act_prepare", st, act_prepare_kernel<IZB_Q4_K><<<pg, 256, 0, st>>>(aq, asc, lda, K, rows_total, tiles, rowmap, aimg, ascimg, sps));
  else
    IZB_LAUNCH("act_prepare", st, act_prepare_kernel<IZB_Q8_0><<<pg, 256, 0, st>>>(aq, asc, lda, K, rows_total, tiles, rowmap, aimg, ascimg, 4));
  TcParams p;
  p.aimg = aimg;
  p.ascimg = ascimg;
  p.tiles = tiles;
  p.rowmap = rowmap;
  p.rowscale = rowscale;
  p.M = M_store;
  p.N = w->N;
  p.K = K;
  p.mat = mat;
  p.C = C;
  p.ldc = ldc;
  p.c_off = c_off;
  p.acc = acc;
  p.dots = dots;
  p.err = err;
  p.n_mtiles = n_tiles_grid;
  dim3 grid(tc_grid(w->device, w->N / BN * n_tiles_grid));
  if (w->type == IZB_Q4_K) return dots ? launch_tc<IZB_Q4_K, true>(w, p, grid, st) : launch_tc<IZB_Q4_K, false>(w, p, grid, st);
  return dots ? launch_tc<IZB_Q8_0, true>(w, p, grid, st) : launch_tc<IZB_Q8_0, false>(w, p, grid, st);
}

// the activation pre-pass + the GEMM for one tile set
int run_tc(const izb_weight* w, int mat, const int8_t* aq, const float* asc, int lda, int rows_total, const int32_t* tiles,
           int n_tiles_grid, const int32_t* rowmap, const float* rowscale, int M_store, float* C, int ldc, int c_off, int acc,
           int32_t* dots, int ws_slot, cudaStream_t st, bool reuse_images = false) {
  // reuse_images: the call before this one, on the same stream and arena, prepared the same activation rows for a weight
  // of the same type and K (the up projection after the gate projection): its operand images are still there
  if (!w->has_tmap) return 1;
  if (w->N % BN || w->K % 256) return 1;
  const int sps = (w->type == IZB_Q4_K && !dots) ? 5 : 4;
  size_t img_bytes, asc_bytes;
  tc_scratch_bytes(n_tiles_grid, w->K, sps, &img_bytes, &asc_bytes);
  void* ws = nullptr;
  if (int rc = izb_workspace(w->device, ws_slot, img_bytes + asc_bytes, &ws)) return rc;
  uint32_t* err = izb_device_error_word(w->device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "gemm: no device error word");
  return run_tc_on(w, mat, aq, asc, lda, rows_total, tiles, n_tiles_grid, rowmap, rowscale, M_store, C, ldc, c_off, acc, dots, ws, err,
                   st, reuse_images);
}

}  // namespace

// scratch bytes of a dense tensor-core GEMM over `rows` activation rows (izb_reserve sizes the arenas with it)
size_t izb_gemm_tc_scratch_bytes(int type, int rows, int K) {
  size_t img_bytes, asc_bytes;
  tc_scratch_bytes((rows + BM - 1) / BM, K, type == IZB_Q4_K ? 5 : 4, &img_bytes, &asc_bytes);
  return img_bytes + asc_bytes;
}

// diagnostics builds (IZB_TC_TRACE): where CTA 0 of the following launches writes its clock stamps
extern "C" int izb_debug_set_trace(unsigned long long* d_trace) {
  g_test_trace.store(d_trace);
  return IZB_OK;
}

extern "C" int izb_debug_wait_test(uint32_t spin_limit, int skip_stage) {
  g_test_spin.store(spin_limit);
  g_test_skip.store(skip_stage);
  return IZB_OK;
}

int izb_make_raw_tensor_map(izb_weight* w) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return IZB_ERR_CUDA;
  const cuuint64_t rows = (cuuint64_t)w->n_mats * w->N;
  if (rows < 1 || w->row_bytes % 16) return IZB_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)(w->row_bytes / 4), rows};
  cuuint64_t strides[1] = {(cuuint64_t)w->row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(w->sb_bytes / 4), (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tm;
  const CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w->raw, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return IZB_ERR_CUDA;
  memcpy(w->tmap_raw, &tm, sizeof tm);
  return IZB_OK;
}

int izb_gemm_tc_launch(const izb_weight* w, int mat, const int8_t* aq, const float* asc, int M, int Mp, float* C, int ldc, int c_off,
                       int acc, int32_t* dots, cudaStream_t st) {
  const int n_tiles = (M + BM - 1) / BM;
  if (n_tiles > 65535) return 1;
  return run_tc(w, mat, aq, asc, Mp, Mp, nullptr, n_tiles, nullptr, nullptr, M, C, ldc, c_off, acc, dots, kWsGemm, st);
}

// quantise + multiply in one call (dense): the fused pre-pass over the M valid rows (rows up to Mp zeroed), then the GEMM on
// its images.  +1 = shape not taken.
int izb_gemm_tc_quant_launch(const izb_weight* w, int mat, const float* x, int ldx, int M, int Mp, int8_t* aq, float* asc, float* C,
                             int ldc, int c_off, int acc, cudaStream_t st) {
  const int n_tiles = (Mp + BM - 1) / BM;  // (the GEMM runs over the padded rows, as izb_matmul's does)
  if (n_tiles > 65535 || !w->has_tmap || w->N % BN || w->K % 256) return 1;
  const int K = w->K, sps = w->type == IZB_Q4_K ? 5 : 4;
  size_t img_bytes, asc_bytes;
  tc_scratch_bytes(n_tiles, K, sps, &img_bytes, &asc_bytes);
  void* ws = nullptr;
  if (int rc = izb_workspace(w->device, kWsGemm, img_bytes + asc_bytes, &ws)) return rc;
  uint32_t* err = izb_device_error_word(w->device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "gemm: no device error word");
  uint16_t* aimg = (uint16_t*)ws;
  float* ascimg = (float*)((unsigned char*)ws + img_bytes);
  const int rows_img = n_tiles * BM > Mp ? n_tiles * BM : Mp;  // every row of every tile is written (rows past M as zeros)
  dim3 grid(K / 256, (rows_img + 31) / 32);
  if (w->type == IZB_Q4_K)
    IZB_LAUNCH("quant_prepare", st, quant_prepare_kernel<IZB_Q4_K><<<grid, 256, 0, st>>>(x, ldx, M, Mp, K, aq, asc, aimg, ascimg, sps, n_tiles));
  else
    IZB_LAUNCH("quant_prepare", st, quant_prepare_kernel<IZB_Q8_0><<<grid, 256, 0, st>>>(x, ldx, M, Mp, K, aq, asc, aimg, ascimg, sps, n_tiles));
  return run_tc_on(w, mat, aq, asc, Mp, Mp, nullptr, n_tiles, nullptr, nullptr, Mp, C, ldc, c_off, acc, nullptr, ws, err, st, true);
}

// MoE on the tensor cores: the slots of each expert are tiles of up to 128 rows (izb_moe_sort with TM = 128); gate then up
// with the fused-SwiGLU store mode (h = up * silu(gate)), down with the routing weight as row scale.
int izb_moe_gateup_tc(const izb_weight* wg, const izb_weight* wu, const int8_t* d_aq, const float* d_asc, int Mp,
                      const int32_t* d_tiles, int max_tiles, const int32_t* d_stok, float* d_h, cudaStream_t st) {
  const int F = wg->N;
  int rc = run_tc(wg, 0, d_aq, d_asc, Mp, 0, d_tiles, max_tiles, d_stok, nullptr, 0, d_h, F, 0, 0, nullptr, kWsMoe, st);
  if (rc != 0) return rc;
  const bool same = wu->type == wg->type && wu->K == wg->K;
  return run_tc(wu, 0, d_aq, d_asc, Mp, 0, d_tiles, max_tiles, d_stok, nullptr, 0, d_h, F, 0, 2, nullptr, kWsMoe, st, same);
}

// gate and up of every expert in one interleaved stack (izb_weight_create_gateup): one grouped GEMM, SwiGLU in its epilogue
int izb_moe_gateup_fused_tc(const izb_weight* wgu, const int8_t* d_aq, const float* d_asc, int Mp, const int32_t* d_tiles,
                            int max_tiles, const int32_t* d_stok, float* d_h, cudaStream_t st) {
  return run_tc(wgu, 0, d_aq, d_asc, Mp, 0, d_tiles, max_tiles, d_stok, nullptr, 0, d_h, wgu->N / 2, 0, 3, nullptr, kWsMoe, st);
}

int izb_moe_down_tc(const izb_weight* wd, const int8_t* d_hq, const float* d_hsc, int Sp, const int32_t* d_tiles, int max_tiles,
                    const float* d_swt, float* d_y, cudaStream_t st) {
  return run_tc(wd, 0, d_hq, d_hsc, Sp, 0, d_tiles, max_tiles, nullptr, d_swt, 0, d_y, wd->N, 0, 0, nullptr, kWsMoe, st);
}

// ---------------------------------------------------------------------------------------------- start-up check
// Seeded data, both weight types, all store modes: tensor-core dots == CUDA-core dots bit for bit, outputs within 1e-5
// of max|ref| (Engine::xmx_check, zero/engine_setup.h:424-622, does the same for its XMX kernel against DP4a).
namespace {
__global__ void fill_kernel(uint8_t* p, size_t n, uint32_t seed, int mode) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t x = (uint32_t)i * 2654435761u + seed;
  x ^= x >> 15; x *= 2246822519u; x ^= x >> 13; x *= 3266489917u; x ^= x >> 16;
  p[i] = mode == 0 ? (uint8_t)x : (uint8_t)(int8_t)((int)(x % 255u) - 127);
}
__global__ void fix_q4k_headers(uint8_t* w, size_t n_sb, uint32_t seed) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_sb) return;
  uint32_t x = (uint32_t)i * 747796405u + seed;
  x ^= x >> 16; x *= 2246822519u; x ^= x >> 13;
  const __half d = __float2half(0.0001f + (float)(x & 0xFFFF) * (0.0099f / 65535.0f));
  const __half m = __float2half(0.0001f + (float)(x >> 16) * (0.0099f / 65535.0f));
  *reinterpret_cast<__half*>(w + i * 144) = d;
  *reinterpret_cast<__half*>(w + i * 144 + 2) = m;
}
__global__ void fix_q8_headers(uint8_t* w, size_t n_sb, uint32_t seed) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_sb * 8) return;
  uint32_t x = (uint32_t)i * 747796405u + seed;
  x ^= x >> 16; x *= 2246822519u; x ^= x >> 13;
  *reinterpret_cast<__half*>(w + (i / 8) * 272 + 2 * (i % 8)) = __float2half(0.001f + (float)(x & 0xFFFF) * (0.019f / 65535.0f));
}
__global__ void fill_scales(float* p, size_t n, uint32_t seed) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t x = (uint32_t)i * 2654435761u + seed;
  x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
  p[i] = 0.005f + (float)(x & 0xFFFF) * (0.03f / 65535.0f);
}
// out[0] = count of differing ints, out[1] = max|a-b| bits, out[2] = max|b| bits
__global__ void compare_kernel(const float* a, const float* b, size_t n, int as_int, unsigned int* out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (as_int) {
    if (reinterpret_cast<const int*>(a)[i] != reinterpret_cast<const int*>(b)[i]) atomicAdd(&out[0], 1u);
  } else {
    const float d = fabsf(a[i] - b[i]);
    if (!(d == d)) atomicAdd(&out[0], 1u);
    atomicMax(&out[1], __float_as_uint(d == d ? d : 0.0f));
    atomicMax(&out[2], __float_as_uint(fabsf(b[i])));
  }
}
}  // namespace

extern "C" int izb_selfcheck(int device) {
  if (izb_get_tc_ok(device) == 1) return IZB_OK;
  IZB_CUDA(cudaSetDevice(device));
  const int M = 200, Mp = 256, N = 256, K = 1024, nb = K / 32;
  int verdict = IZB_OK;
  for (int type : {IZB_Q4_K, IZB_Q8_0}) {
    izb_weight w;
    w.type = type; w.n_mats = 1; w.N = N; w.K = K; w.device = device;
    w.sb_bytes = type == IZB_Q4_K ? 144 : 272;
    w.row_bytes = (size_t)(K / 256) * w.sb_bytes;
    w.bytes = (size_t)N * w.row_bytes;
    const size_t n_out = (size_t)Mp * N, n_dots = (size_t)M * N * nb;
    void* ws = nullptr;
    const size_t need = w.bytes + kRawSlack + (size_t)Mp * K + (size_t)nb * Mp * 4 + 2 * n_out * 4 + 2 * n_dots * 4 + 4096;
    if (int rc = izb_workspace(device, kWsCheck, need, &ws)) return rc;
    uint8_t* base = (uint8_t*)ws;
    w.raw = base; base += (w.bytes + kRawSlack + 255) & ~size_t(255);
    int8_t* aq = (int8_t*)base; base += (size_t)Mp * K;
    float* asc = (float*)base; base += (size_t)nb * Mp * 4;
    float* c_tc = (float*)base; base += n_out * 4;
    float* c_core = (float*)base; base += n_out * 4;
    int32_t* d_tc = (int32_t*)base; base += n_dots * 4;
    int32_t* d_core = (int32_t*)base; base += n_dots * 4;
    unsigned int* cmp = (unsigned int*)base;
    fill_kernel<<<(unsigned)((w.bytes + 255) / 256), 256>>>(w.raw, w.bytes, 17u + type, type == IZB_Q4_K ? 0 : 1);
    if (type == IZB_Q4_K) fix_q4k_headers<<<(unsigned)((w.bytes / 144 + 255) / 256), 256>>>(w.raw, w.bytes / 144, 5u);
    else fix_q8_headers<<<(unsigned)((w.bytes / 272 * 8 + 255) / 256), 256>>>(w.raw, w.bytes / 272, 5u);
    fill_kernel<<<(unsigned)(((size_t)Mp * K + 255) / 256), 256>>>((uint8_t*)aq, (size_t)Mp * K, 99u, 1);
    fill_scales<<<(unsigned)(((size_t)nb * Mp + 255) / 256), 256>>>(asc, (size_t)nb * Mp, 7u);
    IZB_CUDA(cudaGetLastError());
    if (izb_make_raw_tensor_map(&w) != IZB_OK) { izb_set_tc_ok(device, 0); IZB_FAIL(IZB_ERR_SELFCHECK, "selfcheck: cannot encode a tensor map"); }
    w.has_tmap = true;
    unsigned int h[3];
    // dots
    int rc = izb_gemm_tc_launch(&w, 0, aq, nullptr, M, M, nullptr, 0, 0, 0, d_tc, 0);
    if (rc == 0) rc = izb_gemm_core_launch(&w, w.raw, aq, nullptr, M, M, nullptr, 0, 0, 0, d_core, 0);
    if (rc != 0) { izb_set_tc_ok(device, 0); return rc < 0 ? rc : IZB_ERR_SELFCHECK; }
    IZB_CUDA(cudaMemset(cmp, 0, 12));
    compare_kernel<<<(unsigned)((n_dots + 255) / 256), 256>>>((const float*)d_tc, (const float*)d_core, n_dots, 1, cmp);
    IZB_CUDA(cudaMemcpy(h, cmp, 12, cudaMemcpyDeviceToHost));
    if (h[0]) { verdict = IZB_ERR_SELFCHECK; izb_set_error("selfcheck: type %d: %u block dots differ between the tensor-core and CUDA-core kernels", type, h[0]); break; }
    for (int acc = 0; acc < 3 && verdict == IZB_OK; ++acc) {
      fill_scales<<<(unsigned)((n_out + 255) / 256), 256>>>(c_tc, n_out, 3u);
      fill_scales<<<(unsigned)((n_out + 255) / 256), 256>>>(c_core, n_out, 3u);
      rc = izb_gemm_tc_launch(&w, 0, aq, asc, M, Mp, c_tc, N, 0, acc, nullptr, 0);
      if (rc == 0) rc = izb_gemm_core_launch(&w, w.raw, aq, asc, M, Mp, c_core, N, 0, acc, nullptr, 0);
      if (rc != 0) { izb_set_tc_ok(device, 0); return rc < 0 ? rc : IZB_ERR_SELFCHECK; }
      IZB_CUDA(cudaMemset(cmp, 0, 12));
      compare_kernel<<<(unsigned)((n_out + 255) / 256), 256>>>(c_tc, c_core, n_out, 0, cmp);
      IZB_CUDA(cudaMemcpy(h, cmp, 12, cudaMemcpyDeviceToHost));
      float err, ref;
      memcpy(&err, &h[1], 4);
      memcpy(&ref, &h[2], 4);
      if (h[0] || !(err <= 1e-5f * ref)) {
        verdict = IZB_ERR_SELFCHECK;
        izb_set_error("selfcheck: type %d store mode %d: max|err| %g vs max|ref| %g (%u NaN)", type, acc, err, ref, h[0]);
      }
    }
    if (verdict != IZB_OK) break;
  }
  uint32_t word = 0;
  const int st = izb_device_status(device, &word);
  if (st != IZB_OK && verdict == IZB_OK) { verdict = st; }
  izb_set_tc_ok(device, verdict == IZB_OK ? 1 : 0);
  return verdict;
}

// ---------------------------------------------------------------------------------------------- GEMM without allocation
// izb_gemm_noalloc: the tensor-core GEMM for callers that must not allocate device memory while they run -- a serving
// loop that has handed the whole GPU to its own arena, or code that runs under an allocator it cannot re-enter.  izb_gemm keeps its activation images (the fp16 operand tiles,
// the min-term factors and the gathered scales that act_prepare_kernel writes) in an arena that grows with cudaMalloc;
// this entry point keeps them in a fixed array that is part of the library's device image instead.
//
// The array is a device symbol: in host code its name stands for the symbol, not for an address a kernel could use, so
// the address is looked up with cudaGetSymbolAddress -- once per device, with that device current -- and only that
// pointer is ever handed to a kernel.
namespace {
constexpr size_t kNoAllocBytes = IZB_NOALLOC_SCRATCH_BYTES;  // 24 MiB per GPU that loads the library, held until the process exits
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
static __device__ __align__(256) uint32_t g_noalloc_status[64];

struct NoAllocDev {
  unsigned char* scratch = nullptr;
  uint32_t* status = nullptr;
};
NoAllocDev g_noalloc_dev[16];
std::mutex g_noalloc_mu;

// Looks the two symbols up for `device` (which must be the current device) the first time it is called for it.
int noalloc_setup(int device, NoAllocDev** out) {
  if (device < 0 || device >= 16) IZB_FAIL(IZB_ERR_ARG, "gemm_noalloc: device %d out of range", device);
  int cur = -1;
  IZB_CUDA(cudaGetDevice(&cur));
  if (cur != device) IZB_FAIL(IZB_ERR_ARG, "gemm_noalloc: device %d must be current (current is %d)", device, cur);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  NoAllocDev& d = g_noalloc_dev[device];
  if (!d.scratch) {
    void* p = nullptr;
    void* s = nullptr;
    IZB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    IZB_CUDA(cudaGetSymbolAddress(&s, g_noalloc_status));
    d.status = (uint32_t*)s;
    d.scratch = (unsigned char*)p;
    izb_note_noalloc_status(device, d.status);  // izb_device_status reads (and clears) this word too
  }
  *out = &d;
  return IZB_OK;
}
}  // namespace

extern "C" int izb_gemm_noalloc(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, int M, int Mp, float* d_C,
                                int ldc, int c_off, int acc, uint32_t* d_status, void* stream) {
  if (!w || !d_aq || !d_asc || !d_C) IZB_FAIL(IZB_ERR_ARG, "gemm_noalloc: null pointer");
  if (mat < 0 || mat >= w->n_mats) IZB_FAIL(IZB_ERR_ARG, "gemm_noalloc: matrix %d of %d", mat, w->n_mats);
  if (acc < 0 || acc > 3 || (acc == 3 && !w->gu32)) IZB_FAIL(IZB_ERR_ARG, "gemm_noalloc: store mode %d", acc);
  if (Mp % 16 || w->N % BN || w->K % 256 || M < 1 || M > Mp)
    IZB_FAIL(IZB_ERR_SHAPE, "gemm_noalloc: M=%d Mp=%d N=%d K=%d (need Mp %% 16, N %% 128, K %% 256, 1 <= M <= Mp)", M, Mp, w->N, w->K);
  if (c_off < 0 || ldc < c_off + (acc == 3 ? w->N / 2 : w->N))
    IZB_FAIL(IZB_ERR_SHAPE, "gemm_noalloc: ldc = %d < c_off + output columns = %d", ldc, c_off + (acc == 3 ? w->N / 2 : w->N));
  if (!izb_aligned(d_aq, 16) || !izb_aligned(d_asc, 16) || !izb_aligned(d_C, 16) || ldc % 4 || c_off % 4 || (d_status && !izb_aligned(d_status, 4)))
    IZB_FAIL(IZB_ERR_ALIGN, "gemm_noalloc: aq, asc, C must be 16-byte aligned, ldc and c_off multiples of 4");
  if (w->type == IZB_K16) IZB_FAIL(IZB_ERR_TYPE, "gemm_noalloc: ggml type %d is not taken by the tensor-core kernel", w->ggml_type);
  if (!w->has_tmap) IZB_FAIL(IZB_ERR_CUDA, "gemm_noalloc: the weight has no tensor map (driver entry point missing at creation)");
  const int K = w->K;
  const int n_tiles = (M + BM - 1) / BM;
  const int sps = w->type == IZB_Q4_K ? 5 : 4;
  size_t img_bytes, asc_bytes;
  tc_scratch_bytes(n_tiles, K, sps, &img_bytes, &asc_bytes);
  if (img_bytes + asc_bytes > kNoAllocBytes || n_tiles > 65535)
    IZB_FAIL(IZB_ERR_LIMIT, "gemm_noalloc: M=%d K=%d needs %zu scratch bytes, the fixed array holds %zu (use izb_gemm, or fewer rows per call)",
             M, K, img_bytes + asc_bytes, kNoAllocBytes);
  NoAllocDev* dev = nullptr;
  if (int rc = noalloc_setup(w->device, &dev)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // Everything the GEMM reads from the array is rewritten by the pre-pass of the same call (all rows of all its tiles,
  // padding rows as zeros), so nothing stale from an earlier call is ever read; the status word is the one thing that
  // must start at zero.
  uint32_t* status = d_status ? d_status : dev->status;
  IZB_CUDA(cudaMemsetAsync(status, 0, 4, st));
  return run_tc_on(w, mat, d_aq, d_asc, Mp, Mp, nullptr, n_tiles, nullptr, nullptr, M, d_C, ldc, c_off, acc, nullptr, dev->scratch, status,
                   st, false);
}

