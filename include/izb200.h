/* izb200 -- B200 (sm_100a) implementation of inferzero's quantised matrix product, behind a C ABI.
 *
 * The path: int8 activations (one f32 scale per 32 values) x GGUF block-quantised weights (Q8_0, Q4_K), integer dot
 * products per 32-block, f32 combine.  Activation quantiser, prefill GEMM, decode GEMV (1..8 rows), MoE grouped
 * expert GEMM, tensor-parallel split + sum.  CUDA only: there is no CPU fallback; every entry point returns an error
 * when no sm_100 device is present.
 *
 * Conventions
 *   - every function returns an int status (IZB_OK = 0, errors < 0) and never throws; izb_last_error() gives the detail
 *     of the calling thread's last failure;
 *   - shapes and alignment are validated before anything is launched (the reference throws std::runtime_error at the
 *     same place, zero/engine.h:1233-1235);
 *   - pointers named d_* are device pointers owned by the caller; h_* are host pointers; izb_weight is library-owned and
 *     immutable after creation;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream); calls are asynchronous on it unless
 *     stated otherwise (the *_create calls and the *_host convenience calls synchronise);
 *   - devices and threads: the library keeps its state (scratch arenas, kernel attributes, error word) per device, so one
 *     process may drive several GPUs, one host thread per GPU, as the reference does (zero/mgpu/engine_tp.h:825).  A call
 *     that takes a handle (izb_weight, izb_tp) must be made with the handle's device current in the calling thread
 *     (cudaSetDevice), else it returns IZB_ERR_ARG; izb_weight_create* and izb_tp_create make their `device` current
 *     and leave it current;
 *   - per device the library is single-threaded, like one reference Engine (zero/runtime/clrt.h:143): the GEMM, MoE and
 *     tensor-parallel calls keep activation images in one scratch arena each per device, so two such calls of one
 *     device must be ordered (same stream, or events between streams); calls on different devices are independent.
 *     An arena grows when a call needs more than any call before it, which waits for the device and calls
 *     cudaFree / cudaMalloc: call izb_reserve once at start-up to keep that out of the hot path (and out of stream
 *     capture).
 *
 * Buffer layouts are the reference engine's (zero/engine_alloc.h:10,39,41):
 *   aq     int8  [Mp][K]      quantised activations, row-major
 *   asc    f32   [K/32][Mp]   one scale per 32-block, block-major / token-minor
 *   absum  int16 [K/16][Mp]   sums of 16 quantised values (optional everywhere: kernels recompute what they need)
 *   C      f32   [rows][ldc]  outputs, written at column offset c_off
 */
#ifndef IZB200_H
#define IZB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IZB_OK 0
#define IZB_ERR_ARG (-1)       /* null pointer, bad enum */
#define IZB_ERR_SHAPE (-2)     /* K not a multiple of 256, Mp not a multiple of 16, N out of range ... */
#define IZB_ERR_TYPE (-3)      /* a ggml type the library (or the called entry point) does not take */
#define IZB_ERR_ALIGN (-4)     /* pointer or leading dimension not aligned as documented */
#define IZB_ERR_CUDA (-5)      /* a CUDA runtime / driver call failed, or no sm_100 device */
#define IZB_ERR_NCCL (-6)
#define IZB_ERR_TIMEOUT (-7)   /* a bounded device-side wait gave up (see izb_device_status) */
#define IZB_ERR_NOMEM (-8)
#define IZB_ERR_SELFCHECK (-9) /* tensor-core kernel disagreed with the CUDA-core kernel at start-up */
#define IZB_ERR_LIMIT (-10)    /* a fixed capacity of the called entry point was exceeded */

#define IZB_Q8_0 8  /* ggml type ids, src/gguf.h:19-22 */
#define IZB_Q4_K 12
#define IZB_Q4_0 2    /* the further types: decoded once at load into a device form the kernels read (see izb_weight_create) */
#define IZB_Q5_K 13
#define IZB_Q6_K 14
#define IZB_IQ4_XS 23

/* izb_gemm `impl` */
#define IZB_GEMM_AUTO 0 /* tensor-core kernel when the shape allows it, else the CUDA-core kernel */
#define IZB_GEMM_CORE 1 /* CUDA-core dp4a kernel, f32 combine in the reference's order (zero/kernels/gemm.cl:441-487) */
#define IZB_GEMM_TC 2   /* tcgen05 kernel (TMEM accumulators), error if the shape is not taken */

typedef struct izb_weight izb_weight;
typedef struct izb_tp izb_tp;

const char* izb_status_string(int status);
const char* izb_last_error(void);
/* number of kernels this library has launched in the calling process (benchmark bookkeeping) */
uint64_t izb_launch_count(void);
/* Per-kernel timing, as Engine::profile / collect_profile (zero/engine.h:936-950): between start and stop every kernel
 * launch of the library is bracketed by two CUDA event records on its stream.  stop synchronises the device and writes
 * {"kernel": {"launches": n, "ms": total}, ...} as JSON text into `json`. */
int izb_profile_start(void);
int izb_profile_stop(char* json, size_t cap);
/* Reads and clears the device-side error word of `device`: non-zero when a kernel gave up on a bounded wait
 * (value = where).  Synchronises the device. */
int izb_device_status(int device, uint32_t* word);

/* Sizes the per-device scratch arenas of izb_gemm / izb_matmul, the grouped MoE calls and izb_tp_reduce_quant_gather for
 * calls of up to max_rows activation rows (token rows, or MoE slots) and K <= max_K, and creates the device error word,
 * so that none of those calls allocates or synchronises later (the arenas are what Engine::alloc_buffers sizes once in
 * the reference, zero/engine_alloc.h:10-41).  Synchronous; may be called again with larger sizes. */
int izb_reserve(int device, int max_rows, int max_K);
/* The tensor-core GEMM is a persistent kernel with one CTA per multiprocessor.  A host that wants another kernel to be
 * resident beside it -- the collective of the previous token chunk's tensor-parallel sum, as the reference overlaps its
 * sums with the next chunk's GEMMs (TpOverlap, zero/mgpu/engine_tp.h:126-151) -- caps the grid at `sms` multiprocessors
 * (0 = all).  Per device; takes effect from the next launch. */
int izb_set_sm_limit(int device, int sms);
/* Measured tensor-core rate of `device` (which must be current): `launches` back-to-back launches of a kernel that issues
 * iters x 4 tcgen05.mma of 128 x 256 x (16 | 32) per multiprocessor on operands resident in shared memory and accumulators
 * resident in TMEM, timed with CUDA events.  kind 0 = kind::f16 (f32 accumulation), 1 = kind::i8 (s32 accumulation).
 * *tops = 2*M*N*K operations per second / 1e12; *clk_per_mma (may be NULL) = SM clocks per instruction on one
 * multiprocessor.  The method of the reference's own peak probe (bench/gpu_bench.cpp:10-15).  Synchronous. */
int izb_tensor_peak(int device, int kind, int iters, int launches, double* tops, double* clk_per_mma);
/* Diagnostics: the NEXT tensor-core GEMM launch of this process gives up its bounded device-side waits after spin_limit
 * polls (0 = the default) and its activation producer leaves out operand stage `skip_stage` (-1 = none), so that the
 * waits for that stage run out: the kernel drains, stores nothing for the affected tiles and reports through
 * izb_device_status.  This is how the tests exercise the time-out path without a fault; never set it in production. */
int izb_debug_wait_test(uint32_t spin_limit, int skip_stage);

/* ------------------------------------------------------------------------------------------------ weights
 * Replaces Engine::make_weight / upload_padded (zero/engine_load.h:85-196) and the GpuWeight handle
 * (zero/engine.h:27-34).  h_gguf_rows: n_mats matrices of N rows of K values in GGUF block form (Q8_0: 34-byte blocks,
 * Q4_K: 144-byte superblocks), matrix-major, as in the file (MoE stacks are [NE][N][K], zero/engine_stream.h:285-306).
 * The device copy keeps Q4_K superblocks as they are and regroups Q8_0 per 256 values (8 fp16 scales, then 8 x 32
 * int8: the reference's gpu_raw_sb form, src/quants.h:728-751), followed by 1024 zero bytes of slack.  Synchronous.
 * Further types (the reference's table-driven block decoder, src/quants.h:89-315, zero/kernels/decode.cl:183-478):
 *   Q4_0 (2)                    rewritten as Q8_0 blocks (same scale, int8 quants q - 8: exact) -> every Q8_0 kernel;
 *   Q5_K (13), IQ4_XS (23)      decoded on the host into the reference's generic view, which is the device form: per 256
 *                               weights f32 d, f32 dmin, an int8 scale and a uint8 min per 16 elements, int8 quants with
 *                               their offset removed (304 bytes);
 *   Q6_K (14)                   kept packed: the file's 210-byte superblock (ql | qh | 16 scales | d) in 224 bytes, unpacked
 *                               by the kernels to the same int8 quants (the output head and part of the FFN of the common
 *                               Q4_K_M files are Q6_K: a decode step streams 0.875 instead of 1.19 bytes per weight).
 *                               These three: GEMV for 1..8 rows and a CUDA-core GEMM, both with exact integer dots per
 *                               16-element half (zero/kernels/decode.cl:992-1004); not taken by the tensor-core GEMM, the
 *                               MoE entry points or izb_gemm_noalloc (IZB_ERR_TYPE / IZB_ERR_SHAPE). */
int izb_weight_create(int ggml_type, const void* h_gguf_rows, int n_mats, int N, int K, int device, izb_weight** out);
/* Tensor-parallel shard of a matrix (Engine::tp_slice, zero/mgpu/engine_tp_shard.h:202-234): rows [n0, n1) and input
 * columns [k0, k1) of every matrix; k0, k1 multiples of 256. */
int izb_weight_create_slice(int ggml_type, const void* h_gguf_rows, int n_mats, int N, int K, int n0, int n1, int k0, int k1,
                            int device, izb_weight** out);
/* Several tensors of one type and one K uploaded as ONE matrix, their rows one after the other (load_w_stack,
 * zero/engine_load.h:315-339: the reference uploads Q | K | V and gate | up stacked and runs one GEMV launch over them,
 * gemv_gu, zero/engine.h:1128-1146).  The result is an ordinary weight of sum(n_rows) rows: a single izb_matmul / izb_gemv
 * over it writes the parts' outputs side by side, and a decode step pays one launch instead of n_parts. */
int izb_weight_create_stack(int ggml_type, const void* const* h_parts, const int* n_rows, int n_parts, int K, int device,
                            izb_weight** out);
/* The gate and the up projection of an FFN (or of every expert of a stack, n_mats > 1) as ONE weight of 2F rows per matrix
 * whose rows alternate in groups of 32: rows 64j .. 64j+31 are gate rows 32j .., rows 64j+32 .. 64j+63 the up rows of the
 * same FFN channels (F % 64 == 0; Q8_0, Q4_K, Q4_0).  With store mode 3 of izb_gemm (and izb_moe_gateup given this stack
 * and wu = NULL) one GEMM computes both projections and stores up * silu(gate) [rows][F]: the reference fuses the same
 * product into its up GEMM, which reads the gate GEMM's output back (store mode 2, zero/kernels/gemm.cl:562-565; the
 * `fused` flag of swiglu_quant, zero/kernels/ops.cl:277); here a thread of the GEMM's epilogue holds a gate column and its
 * up column side by side, so the gate projection never goes to memory.  Same operations, same roundings as mode 2. */
int izb_weight_create_gateup(int ggml_type, const void* h_gate_rows, const void* h_up_rows, int n_mats, int F, int K, int device,
                             izb_weight** out);
/* The row order izb_weight_create_gateup uploads, on the host alone (no device needed): h_dst receives n_mats matrices of
 * 2F GGUF rows, groups of 32 gate rows and 32 up rows alternating. */
int izb_gateup_interleave_host(int ggml_type, const void* h_gate_rows, const void* h_up_rows, int n_mats, int F, int K, void* h_dst,
                               size_t dst_bytes);
/* The loader's host-side decoder on its own (no device needed): n_superblocks superblocks (256 weights each) of a Q4_0,
 * Q5_K, Q6_K or IQ4_XS row -> the form izb_weight_create uploads: GGUF Q8_0 blocks (8 x 34 bytes) for Q4_0; 224 bytes for
 * Q6_K (the file's 210 + 14 zero bytes); else 304 bytes:
 * f32 d | f32 dmin | int8 scale[16] | uint8 min[16] | 8 zero bytes | int8 (quant - offset)[256]. */
int izb_weight_decode_host(int ggml_type, const void* h_src, size_t n_superblocks, void* h_dst, size_t dst_bytes);
void izb_weight_destroy(izb_weight* w);
int izb_weight_info(const izb_weight* w, int* ggml_type, int* n_mats, int* N, int* K, size_t* device_bytes);
/* Copies `bytes` of the device form back, from byte `offset` (rows of K/256 superblocks of 144 (Q4_K) or 272 (Q8_0) bytes,
 * matrix-major): lets a host check the layout against the reference's gpu_raw_sb (src/quants.h:728-751).  Synchronous. */
int izb_weight_download(const izb_weight* w, size_t offset, size_t bytes, void* h_out);

/* ------------------------------------------------------------------------------------------------ activations
 * Replaces Engine::quant_rows (zero/engine.h:1445) = ops.cl quant_store16 (zero/kernels/ops.cl:38-72); bit-exact with
 * quantize_act_cpu (src/quants.h:626-643).  d_x: [M_valid][ldx] f32; rows M_valid..Mp-1 of the outputs are written as
 * zeros with scale 0 (zero/kernels/ops.cl:132-135).  K % 256 == 0, Mp % 16 == 0, Mp >= M_valid.  d_absum may be NULL. */
int izb_quantize_act(const float* d_x, int ldx, int M_valid, int Mp, int K, int8_t* d_aq, float* d_asc, int16_t* d_absum,
                     void* stream);
/* SwiGLU then quantise (ops.cl swiglu_quant, zero/kernels/ops.cl:272-315): h = g/(1+exp(-g)) * u; d_gu: [M_valid][2F]
 * with gate in columns [0,F) and up in [F,2F) when `split` != 0, or d_gu = gate-times-up product already ([M][F],
 * split == 0: plain quantise).  d_h (may be NULL) receives h as f32 [M_valid][F]. */
int izb_swiglu_quant(const float* d_gu, int ldgu, int split, int M_valid, int Mp, int F, float* d_h, int8_t* d_aq,
                     float* d_asc, int16_t* d_absum, void* stream);
/* RMSNorm then quantise (ops.cl rmsnorm_quant, zero/kernels/ops.cl:104-141): y = (x * r) * w with
 * r = 1 / sqrt(sum(x^2) / K + eps) per row, quantised like izb_quantize_act; d_h (may be NULL) receives y as f32
 * [M_valid][K].  d_w: [K] f32.  The reference leaves the order of the sum of squares to the OpenCL work-group reduction;
 * here it is defined (256 fused-multiply-add chains over groups of 8 values, xor butterfly per 32, eight partial sums in order), so that
 * the int8 rows are reproducible bit for bit; the oracle repeats that order. */
int izb_rmsnorm_quant(const float* d_x, int ldx, const float* d_w, float eps, int M_valid, int Mp, int K, float* d_h,
                      int8_t* d_aq, float* d_asc, int16_t* d_absum, void* stream);
/* Residual add with a norm, then the next projection's quantised input (add_norm_quant, zero/kernels/ops_attn_g.cl:617-680;
 * the decode path's producer between two GEMVs): per row, in place,
 *   x = (x + (t * r) * w) * s,   r = 1 / sqrt(sum(t^2) / K + eps),
 * then y = (x * r2) * w2 with r2 from the new x (d_w2 != NULL), or y = x (d_w2 == NULL), quantised like
 * izb_quantize_act.  d_x, d_t: [M_valid][K] f32 (contiguous rows); d_w, d_w2: [K].  K % 256 == 0, K <= 16384 (the new row
 * stays in registers between the two steps, as in the reference).  The sums of squares are taken in a defined order as in
 * izb_rmsnorm_quant (here the 256 chains are strided by one element).  Rows M_valid..Mp-1 of the quantised outputs are zeros with scale 0. */
int izb_add_norm_quant(float* d_x, const float* d_t, const float* d_w, float eps, float s, const float* d_w2, int M_valid, int Mp,
                       int K, int8_t* d_aq, float* d_asc, int16_t* d_absum, void* stream);

/* Logit soft-cap of the output head (softcap_rows, zero/kernels/ops_attn_g.cl:724; the head GEMVs' HEAD_OUT epilogue,
 * zero/kernels/decode.cl:882-887; call site zero/engine.h:1102-1111): C[r][off + n] = cap * tanh(C[r][off + n] * (1 / cap))
 * for r < rows, n < N, in place; row stride ld in floats (the reference passes ld = 0 for one row: any ld is accepted when
 * rows == 1).  cap > 0.  Call it after izb_matmul / izb_gemv on the head's output rows. */
int izb_softcap_rows(float* d_C, int rows, int ld, int off, int N, float cap, void* stream);

/* ------------------------------------------------------------------------------------------------ matmul
 * Replaces Engine::matmul / matmul1 (zero/engine.h:1080,1147-1251): C[t][c_off + n] (op)= sum_k A[t][k] W[n][k] for
 * the T valid rows, dispatching on T as the reference does: T == 1 -> GEMV (decode.cl gemv, :913), 2..8 -> few-row
 * GEMV reading the weights once (gemv_mt, :1581), T > 8 -> GEMM over Mp padded rows (gemm.cl gemm, :163; needs
 * Mp % 16 == 0, N % 16 == 0).  acc: 0 store, 1 add to C, 2 C = result * silu(C) (fused SwiGLU, gemm.cl:562-565; GEMM
 * only, as in the reference), 3 (GEMM only, weights of izb_weight_create_gateup): C[t][c_off + f] = up_f * silu(gate_f),
 * N / 2 output columns.  `mat` selects the matrix of a stack (0 for a dense weight). */
int izb_matmul(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, const int16_t* d_absum, int T, int Mp,
               float* d_C, int ldc, int c_off, int acc, void* stream);
/* quant_rows + matmul in one call (Engine::quant_rows, zero/engine.h:1445, directly followed by Engine::matmul, :1080, as every
 * projection of a prompt chunk runs them): d_x [T][ldx] f32 -> d_aq [Mp][K], d_asc [K/32][Mp] exactly as izb_quantize_act
 * writes them (the buffers stay valid for further projections of the same activations), then C as izb_matmul.  For T > 8
 * on the tensor-core kernel the quantiser also writes that kernel's operand images, so the int8 rows are not read back
 * and the pre-pass launch of the GEMM is gone; results are bit for bit those of the two separate calls. */
int izb_quant_matmul(const izb_weight* w, int mat, const float* d_x, int ldx, int T, int Mp, int8_t* d_aq, float* d_asc, float* d_C,
                     int ldc, int c_off, int acc, void* stream);
/* The two kernels behind izb_matmul, callable directly (kernel ABIs of zero/kernels/decode.cl:913-915,1581-1583 and
 * zero/kernels/gemm.cl:163-166). */
int izb_gemv(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, int T, int Mp, float* d_C, int ldc,
             int c_off, int acc, void* stream);
int izb_gemm(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, int M_rows, int Mp, float* d_C, int ldc,
             int c_off, int acc, int impl, void* stream);
/* Verification mode (the reference's xmx_check idea, zero/engine_setup.h:424): the per-32-block integer dot products
 * themselves, d_dots int32 [M][N][K/32], from the CUDA-core kernel (impl = IZB_GEMM_CORE) or from the tensor-core
 * kernel's accumulators before any scaling (impl = IZB_GEMM_TC).  Both must equal the CPU values bit for bit. */
int izb_block_dots(const izb_weight* w, int mat, const int8_t* d_aq, int M, int32_t* d_dots, int impl, void* stream);
/* Start-up check in the manner of Engine::xmx_check: runs the tensor-core kernel and the CUDA-core kernel on seeded
 * data for both weight types and all store modes and compares (dots bit for bit, outputs within 1e-5 of max|ref|).
 * Synchronous.  IZB_ERR_SELFCHECK on disagreement; izb_matmul then keeps to the CUDA-core kernel on that device. */
int izb_selfcheck(int device);

/* izb_gemm for callers that cannot allocate device memory while they run.  It has no counterpart in the reference.
 * Who needs it: an inference server that gave the whole GPU to its own memory pool at start-up (a cudaMalloc inside a
 * request would fail or fragment it), and hosts that forbid allocator calls on their hot path (real-time loops,
 * processes whose device heap is locked down after initialisation).  izb_gemm keeps the tensor-core kernel's activation images in an arena
 * that it grows with cudaMalloc when a call is larger than any before; this call keeps them in a fixed array of
 * IZB_NOALLOC_SCRATCH_BYTES that lives in the library's device image: every GPU that loads the library holds those
 * bytes until the process exits, and the call itself calls no cudaMalloc, cudaFree or other allocating routine.
 *   - Same arguments and results as izb_gemm with impl = IZB_GEMM_TC (N % 128 == 0 is required here: there is no second
 *     kernel to fall back to), plus d_status.
 *   - Limit: ceil(M/128) * (K/256 * S * 16384 + K/32 * 512) bytes, S = 5 for Q4_K and 4 for Q8_0, must fit in the array (e.g. M = 1024 at K = 5120, or
 *     M = 512 at K = 10240); a larger call returns IZB_ERR_LIMIT and launches nothing.
 *   - d_status: a device uint32 of the caller's, or NULL to use a word inside the library's device image, which
 *     izb_device_status reports (and clears) together with the library's own error word.  It is cleared at the start of
 *     the call and is non-zero afterwards if a bounded device-side wait gave up (the output is then incomplete).
 *   - "Allocates nothing" is about the call itself.  The CUDA runtime loads a kernel's code onto the device the first
 *     time that kernel is launched, and that may reserve device memory: run one warm-up call per weight type before the
 *     phase in which nothing may be allocated.  While izb_profile_start is active the library brackets every launch with
 *     CUDA events and creates them on demand (cudaEventCreate): leave profiling off in that phase.
 *   - The first call on a device looks up the array's device address (the device must be current, as for every call):
 *     make that first call before any stream capture begins.
 *   - All calls share the one array and it keeps the last call's contents; each call rewrites everything it reads.  Two
 *     calls whose kernels can overlap on the GPU (different streams, no ordering between them) race on it: order them. */
#define IZB_NOALLOC_SCRATCH_BYTES (24u << 20)
int izb_gemm_noalloc(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, int M_rows, int Mp, float* d_C,
                     int ldc, int c_off, int acc, uint32_t* d_status, void* stream);

/* Host-buffer convenience call = what a caller without device code does per projection: copies h_x [M][K] to the
 * device, quantises, multiplies, copies C [M][N] back, synchronises.  Uses library-owned staging buffers per device.
 * Rows travel in chunks of 1024 through two staging buffers and three library-owned streams (copy in, compute, copy
 * out), ordered after the work already in `stream`, so that both directions of the host link and the GPU are busy at
 * once; pinned host buffers are needed for the copies to overlap.  Returns when h_C is complete. */
int izb_matmul_host(const izb_weight* w, int mat, const float* h_x, int M, float* h_C, void* stream);

/* ------------------------------------------------------------------------------------------------ mixture of experts
 * moe_route (zero/kernels/moe.cl:50-89): per token softmax numerators of the NU largest of NE logits (ties: lower
 * expert id), weights renormalised over the selection.  d_ids, d_wts: [T][NU]; d_counts: [NE] (overwritten). */
int izb_moe_route(const float* d_logits, int ldl, int T, int NE, int NU, int32_t* d_ids, float* d_wts, int32_t* d_counts,
                  void* stream);
/* The same with the shared expert's gate (SGATE, zero/kernels/moe.cl:44,88): d_sgate[t] = 1 / (1 + exp(-logits[t][NE])), the
 * sigmoid of the logit that follows the NE expert logits of a row (ldl >= NE + 1).  d_sgate == NULL: izb_moe_route. */
int izb_moe_route_ex(const float* d_logits, int ldl, int T, int NE, int NU, int32_t* d_ids, float* d_wts, int32_t* d_counts,
                     float* d_sgate, void* stream);
/* moe_scan + moe_scatter (zero/kernels/moe.cl:141-179), deterministic: slots of an expert in increasing (token, choice)
 * order.  d_offs [NE+1]; d_tiles [1 + 3*max_tiles] = count, then (expert, first slot, rows <= TM); d_stok, d_swt, d_inv
 * [T*NU]. */
int izb_moe_sort(const int32_t* d_ids, const float* d_wts, const int32_t* d_counts, int T, int NE, int NU, int TM,
                 int32_t* d_offs, int32_t* d_tiles, int max_tiles, int32_t* d_stok, float* d_swt, int32_t* d_inv,
                 void* stream);
/* Expert-parallel form (the reference's split of a MoE model by expert, zero/mgpu/engine_tp_shard.h:169-199,
 * zero/kernels/tp.cl:55-78): this rank holds the experts [e0, e1).  The other experts count as empty (no slots, no tiles),
 * their pairs get d_inv = -1, and a tile names its expert by its index in the rank's own weight stack (e - e0): pass the
 * stack of those e1 - e0 matrices to izb_moe_gateup / izb_moe_down.  d_ids / d_counts stay global, as routed. */
int izb_moe_sort_ex(const int32_t* d_ids, const float* d_wts, const int32_t* d_counts, int T, int NE, int NU, int TM, int e0,
                    int e1, int32_t* d_offs, int32_t* d_tiles, int max_tiles, int32_t* d_stok, float* d_swt, int32_t* d_inv,
                    void* stream);
/* moe_gateup_q (zero/kernels/decode_moe.cl:92-260): d_h[slot][F] = silu(x_tok Wg_e^T) * (x_tok Wu_e^T) for every tile
 * of d_tiles (made by izb_moe_sort with the same TM); wg, wu are stacks [NE][F][K]; the activations are token rows
 * (d_aq [Mp][K], d_asc [K/32][Mp]) gathered through d_stok.  TM 1..8: per-tile kernels on the raw rows, as the
 * reference; TM = 128: grouped tensor-core GEMM.  The grid is sized by max_tiles; tiles past d_tiles[0] return.
 * wu = NULL with wg a stack made by izb_weight_create_gateup (TM = 128): one grouped GEMM for both projections. */
int izb_moe_gateup(const izb_weight* wg, const izb_weight* wu, const int8_t* d_aq, const float* d_asc, int Mp,
                   const int32_t* d_tiles, int max_tiles, int TM, const int32_t* d_stok, float* d_h, void* stream);
/* moe_down_q (zero/kernels/decode_moe.cl:269-449): d_y[slot][E] = swt[slot] * (hq[slot] Wd_e^T); d_hq [Sp][F],
 * d_hsc [F/32][Sp] from izb_quantize_act over the slot rows of d_h. */
int izb_moe_down(const izb_weight* wd, const int8_t* d_hq, const float* d_hsc, int Sp, const int32_t* d_tiles, int max_tiles,
                 int TM, const float* d_swt, float* d_y, void* stream);
/* moe_combine (zero/kernels/moe.cl:344-352, no shared expert): x[t] += sum_k y[inv[t*NU+k]] in choice order. */
int izb_moe_combine(float* d_x, const float* d_y, const int32_t* d_inv, int T, int NU, int E, void* stream);
/* moe_combine in full (zero/kernels/moe.cl:344-352): v = sum_k y[inv[t*NU+k]] over the slots >= 0, in choice order,
 * + d_sgate[t] * d_sh[t] when a shared expert's output d_sh [T][E] and its gate are given (both or neither);
 * partial == 0: x[t] += v; partial != 0: x[t] = v, this rank's share of the sum in the expert-parallel split
 * (tp_moe_combine, zero/kernels/tp.cl:100-111; the shares are then summed over the ranks like any row-parallel output,
 * the shared expert added on one rank only). */
int izb_moe_combine_ex(float* d_x, const float* d_y, const int32_t* d_inv, int T, int NU, int E, const float* d_sh,
                       const float* d_sgate, int partial, void* stream);

/* ------------------------------------------------------------------------------------------------ tensor parallel
 * tp_range (zero/mgpu/engine_tp_shard.h:68-72): rank r's [begin, end) of `total` in whole `unit`s. */
int izb_tp_range(int64_t total, int64_t unit, int nranks, int rank, int64_t* begin, int64_t* end);
/* tp_add (zero/kernels/tp.cl:5-11): x[i] += part_0[i] + ... + part_{np-1}[i], rank order. */
int izb_tp_add(float* d_x, const float* d_parts, size_t n, int np, size_t stride, void* stream);
/* Communicator over NCCL (replaces TpComm, zero/mgpu/engine_tp.h:36-124).  id: 128 bytes from izb_tp_unique_id on rank
 * 0, distributed by the caller. */
int izb_tp_unique_id(void* id128);
int izb_tp_create(int nranks, int rank, const void* id128, int device, izb_tp** out);
/* The same with failure detection and a cap on the collectives' CTAs.  timeout_ms > 0 makes the communicator
 * non-blocking: creation and every collective call is followed by a wait of at most timeout_ms for NCCL's answer
 * (ncclCommGetAsyncError), after which the communicator is aborted and the call returns IZB_ERR_TIMEOUT (the reference
 * bounds every barrier and wait of its transport likewise, zero/mgpu/engine_tp.h:93-123).  max_ctas > 0 limits the CTAs a
 * collective may use (ncclConfig_t.maxCTAs), which leaves multiprocessors to a GEMM running beside it.  0, 0 = izb_tp_create. */
int izb_tp_create_ex(int nranks, int rank, const void* id128, int device, int timeout_ms, int max_ctas, izb_tp** out);
/* Bounded host wait for everything queued on `stream` (wait_done, zero/mgpu/engine_tp.h:1313-1372): returns IZB_OK when it
 * has finished; after timeout_ms, or when NCCL reports an asynchronous error, aborts the communicator -- which also ends
 * this rank's collectives that are waiting on the device for a missing peer -- and returns IZB_ERR_TIMEOUT / IZB_ERR_NCCL.
 * An aborted communicator refuses further collectives; destroy it and create a new one with the surviving ranks. */
int izb_tp_wait(izb_tp* tp, void* stream, int timeout_ms);
int izb_tp_abort(izb_tp* tp);
void izb_tp_destroy(izb_tp* tp);
/* tp_out's sum (zero/mgpu/engine_tp_shard.h:318-325, tp_reduce_at zero/mgpu/engine_tp.h:272): d_x[rows][E] += sum over
 * ranks of d_part (f32 all-reduce over NVLink; d_part is overwritten with the sum). */
int izb_tp_allreduce_rows(izb_tp* tp, float* d_x, float* d_part, int rows, int E, void* stream);
/* Same sum where the next step quantises anyway: reduce-scatter the f32 partials by token rows, add this rank's rows
 * of d_x, quantise them, all-gather int8 + scales.  Every element is summed on one rank only, so all ranks end with
 * identical int8 rows (the reference's bit-identical-residual property, zero/kernels/tp.cl:3-4).  rows % (16*nranks)
 * == 0.  d_xsum (may be NULL) receives this rank's summed f32 rows [rows/nranks][E]. */
int izb_tp_reduce_quant_gather(izb_tp* tp, const float* d_x, float* d_part, int rows, int E, float* d_xsum, int8_t* d_aq,
                               float* d_asc, void* stream);

/* The output head split by vocabulary rows in units of 16 (zero/mgpu/engine_tp_shard.h:68-72; the last rank also takes the
 * rows past the last whole unit) and its logits joined in rank order (the reference joins them on the host,
 * zero/mgpu/engine_tp.h:853-862): d_local [rows][ld_local] holds this rank's logits in its first end - begin columns,
 * d_full [rows][ld_full] receives the whole vocabulary on every rank.  rows <= 64 (decode rows). */
int izb_tp_gather_logits(izb_tp* tp, const float* d_local, int ld_local, int rows, int vocab, float* d_full, int ld_full,
                         void* stream);

/* ------------------------------------------------------------------------------------------------ peer transport without SMs
 * The sums of the row-parallel projections moved by the copy engines instead of a collective library: every rank copies
 * its partial rows into the owner's receive buffer and raises a flag there; the owner adds the parts in rank order
 * (izb_tp_add), quantises and copies the result into every rank's buffers the same way.  This is the shape of the
 * reference's own transport (TpComm: copy the rows to the owner, raise a counter, tp_add in rank order;
 * zero/mgpu/engine_tp.h:36-124,272-324) with NVLink copies in place of host-visible memory.  The pointers into other
 * ranks' memory are the host's to provide (CUDA IPC, cuMemMap, a symmetric-memory allocator); the library sees plain
 * device pointers.  Nothing here occupies a multiprocessor, so a GEMM that holds all of them runs beside the transfers.
 *
 * izb_p2p_push: n_copies device-to-device copies on `stream`, then `value` written to each of the n_flags flags (32-bit
 *   words, usually in the destination ranks' memory) in stream order: whoever sees the value sees the data.
 * izb_p2p_wait: `stream` waits until every flag (in this rank's own memory) is >= value.  Use a sequence number that only
 *   grows.  The flags must be written by OTHER devices: CUDA does not see the order between a wait and a write issued on
 *   two streams of one device and may serialise them the wrong way round (order what a rank hands to itself with events).
 * izb_p2p_wait_host: waits on the host until everything queued on `stream` has finished or timeout_ms has passed
 *   (IZB_ERR_TIMEOUT; the bounded barrier of the reference, engine_tp.h:93-123).  The stream wait itself cannot be
 *   released from this device: after a time-out the stream stays blocked until the peer writes or the context ends.
 * izb_tp_scales_from_ranks: the gathered block scales, pushed as [nranks][E/32][own], into the GEMM's [E/32][nranks*own]. */
int izb_p2p_push(int n_copies, void* const* d_dst, const void* const* d_src, const size_t* bytes, int n_flags,
                 uint32_t* const* d_flags, uint32_t value, void* stream);
int izb_p2p_wait(int n_flags, uint32_t* const* d_flags, uint32_t value, void* stream);
int izb_p2p_wait_host(void* stream, int timeout_ms);
int izb_tp_scales_from_ranks(float* d_asc, const float* d_stage, int nranks, int own, int E, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* IZB200_H */
