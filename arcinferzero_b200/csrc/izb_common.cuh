// Shared declarations of the izb200 library: the weight handle, error plumbing and small device helpers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/izb200.h"

// ---------------------------------------------------------------------------------------------- weight handle
// Device form of a weight (or of a stack of n_mats equal matrices): rows of K/256 superblocks.
//   Q4_K: the 144-byte GGUF superblock unchanged: fp16 d | fp16 dmin | 12 B packed 6-bit scales/mins | 128 B nibbles
//   Q8_0: 272 bytes per 256 values: fp16 d[8] | int8 q[8][32]
// Both are multiples of 16 bytes, so every superblock starts on a 16-byte boundary (128-bit loads, TMA boxes).
//   K16:  304 bytes per 256 values: f32 d | f32 dmin | int8 scale[16] | uint8 min[16] | 8 pad | int8 quant[256], the generic
//         view of Q5_K / Q6_K / IQ4_XS superblocks (izb_types.cu)
constexpr int IZB_K16 = 100;        // device form id (izb_weight::type holds the DEVICE form: IZB_Q8_0, IZB_Q4_K or IZB_K16)
constexpr int kK16SbBytes = 304;
// Q6_K stays packed on the device: the file's 210-byte superblock in 224 bytes (16-byte aligned sections):
//   ql[128] (low nibbles) | qh[64] (high 2 bits) | int8 scale[16] | fp16 d | 14 pad.  It is a K16 weight with `packed6` set:
//   the kernels of izb_types.cu unpack it to the same int8 quants and run the same arithmetic.
constexpr int kQ6pSbBytes = 224;
struct izb_weight {
  int type = 0, n_mats = 0, N = 0, K = 0, device = 0;
  int ggml_type = 0;     // the type of the file's tensor (Q4_0 is held as Q8_0, Q5_K / Q6_K / IQ4_XS as K16)
  bool has_min = false;  // K16: the type has mins (Q5_K)
  bool packed6 = false;  // K16 with Q6_K superblocks kept packed (kQ6pSbBytes each)
  bool gu32 = false;     // rows alternate in groups of 32 between a gate and an up projection (izb_weight_create_gateup)
  int sb_bytes = 0;      // 144, 272 or 304
  size_t row_bytes = 0;  // K/256 * sb_bytes
  size_t bytes = 0;      // n_mats * N * row_bytes (without the slack)
  uint8_t* raw = nullptr;
  alignas(64) unsigned char tmap_raw[128];  // CUtensorMap over raw: [n_mats*N rows][row_bytes/4 uint32]
  bool has_tmap = false;
};

static constexpr size_t kRawSlack = 1024;  // zero bytes after the last row (zero/engine_load.h:79-84)

// ---------------------------------------------------------------------------------------------- errors
void izb_set_error(const char* fmt, ...);
extern std::atomic<uint64_t> g_izb_launches;

#define IZB_FAIL(code, ...)     \
  do {                          \
    izb_set_error(__VA_ARGS__); \
    return (code);              \
  } while (0)

#define IZB_CUDA(call)                                                                              \
  do {                                                                                              \
    cudaError_t e__ = (call);                                                                       \
    if (e__ != cudaSuccess) {                                                                       \
      izb_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__);   \
      return IZB_ERR_CUDA;                                                                          \
    }                                                                                               \
  } while (0)

// after a kernel launch: count it and pick up launch-configuration errors
#define IZB_LAUNCHED()                                                                                    \
  do {                                                                                                    \
    g_izb_launches.fetch_add(1, std::memory_order_relaxed);                                               \
    cudaError_t e__ = cudaGetLastError();                                                                 \
    if (e__ != cudaSuccess) {                                                                             \
      izb_set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__), __FILE__, __LINE__);     \
      return IZB_ERR_CUDA;                                                                                \
    }                                                                                                     \
  } while (0)

// Optional per-kernel timing (izb_profile_start / izb_profile_stop): when on, every launch is bracketed by two event
// records on its stream; off by default (one relaxed atomic load per launch).
void izb_prof_begin(const char* name, cudaStream_t st);
void izb_prof_end(cudaStream_t st);
#define IZB_LAUNCH(name, st, ...) \
  do {                            \
    izb_prof_begin(name, st);     \
    __VA_ARGS__;                  \
    izb_prof_end(st);             \
    IZB_LAUNCHED();               \
  } while (0)

static inline bool izb_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---------------------------------------------------------------------------------------------- per-device state
// The reference drives N GPUs from N threads of ONE process (one Engine per GPU, zero/mgpu/engine_tp.h:825), so everything
// that belongs to a device's context -- a kernel's opt-in to more than 48 KB of dynamic shared memory, the SM count, the
// scratch arenas, the error word -- is kept per device here, never in a process-wide flag.
constexpr int kIzbMaxDev = 16;

// IZB_OK when `device` is the calling thread's current device.  Every entry point that takes a handle calls it: the
// caller's stream, the handle's memory and the kernel attributes below must all belong to one device.
int izb_require_device(int device, const char* what);
// multiprocessor count of `device` (looked up once per device)
int izb_sm_count(int device);
// the SMs a persistent GEMM grid may take: izb_sm_count, or less after izb_set_sm_limit
int izb_sm_budget(int device);

// Work that must run once per device at one call site (idempotent work only: two threads that race on the first call of
// a device may both run it).  One bit per device.
struct izb_device_once {
  std::atomic<uint32_t> done{0};
  template <class F>
  int run(int device, F&& f) {
    if (device < 0 || device >= kIzbMaxDev) IZB_FAIL(IZB_ERR_ARG, "device %d out of range", device);
    const uint32_t bit = 1u << device;
    if (done.load(std::memory_order_acquire) & bit) return IZB_OK;
    if (int rc = f()) return rc;
    done.fetch_or(bit, std::memory_order_release);
    return IZB_OK;
  }
};
// the usual case: let `kernel` use up to `bytes` of dynamic shared memory on `device` (which must be current)
#define IZB_SMEM_OPTIN(kernel, bytes, device)                                                                             \
  do {                                                                                                                    \
    static izb_device_once once__;                                                                                        \
    if (int rc__ = once__.run((device), [&]() -> int {                                                                    \
          IZB_CUDA(cudaFuncSetAttribute((kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes)));            \
          return IZB_OK;                                                                                                  \
        }))                                                                                                               \
      return rc__;                                                                                                        \
  } while (0)

// Device-side error word (one per device, in managed-free plain device memory): kernels that give up on a bounded
// wait OR a code into it; izb_device_status reads and clears it.
uint32_t* izb_device_error_word(int device);

// Per-device scratch arenas, one per user so that independent users never share bytes; each is grown on demand
// (cudaMalloc only when a call needs more than any call before it).  Calls that use the same arena must be ordered on
// one stream.
enum { kWsGemm = 0, kWsTp = 1, kWsMoe = 2, kWsCheck = 3, kWsNorm = 4 };
int izb_workspace(int device, int slot, size_t bytes, void** out);

// ---------------------------------------------------------------------------------------------- device helpers
#ifdef __CUDACC__
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float half_bits_to_float(uint32_t h16) { return __half2float(__ushort_as_half((unsigned short)h16)); }

// Q4_K: 6-bit scale and min of sub-block j (0..7) from the 12 packed bytes held as three little-endian words
// (get_scale_min_k4, src/quants.h:61-69)
__device__ __forceinline__ void q4k_scale_min(const uint32_t s[3], int j, int& sc, int& mn) {
  // shifts only, no indexing of s by a run-time value (that would put the three words in local memory)
  const int sh = 8 * (j & 3);
  const uint32_t a = s[0] >> sh, b = s[1] >> sh, c = s[2] >> sh;
  if (j < 4) {
    sc = a & 63;
    mn = b & 63;
  } else {
    sc = (c & 0xF) | (((a >> 6) & 3) << 4);
    mn = ((c >> 4) & 0xF) | (((b >> 6) & 3) << 4);
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
#endif
