// Measured tensor-core peaks of the device the library runs on: a loop of tcgen05.mma on operands that stay in shared
// memory and accumulators that stay in TMEM -- nothing is loaded or stored inside the timed loop.  The reference measures
// its GPUs' matrix-unit rate the same way (a register-resident DPAS loop, bench/gpu_bench.cpp:10-15); the benchmark
// reports the prefill GEMM against this figure for kind::i8 (the "% of int8 tensor peak" of its metric) and kind::f16
// (the MMA kind the GEMM kernel issues), beside the library-GEMM figure it is given from outside.
//
// One CTA per multiprocessor, 128 x 256 tiles (the largest single-CTA shape), K = 32 (int8) or 16 (fp16) per
// instruction, four instructions per pass over a 128-byte-swizzled K-major operand row, two accumulators of 256 TMEM
// columns used alternately.  One thread issues; the only wait is the commit after the last instruction (bounded).
#include "izb_common.cuh"

namespace {

constexpr int PM = 128, PN = 256;
constexpr int kPeakSmem = PM * 128 + PN * 128 + 1024 + 64;

__device__ __forceinline__ uint32_t p_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major operand rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart (same form as the GEMM's tiles)
__device__ __forceinline__ uint64_t p_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

template <bool I8>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters, uint32_t spin_limit, uint32_t* err, unsigned long long* clk) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PM * 128 + PN * 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  // operand bytes: small non-zero values (fp16 numbers of magnitude 2^-6 .. 2^-5 with mixed signs; any byte is a valid int8)
  for (int i = threadIdx.x; i < (PM * 128 + PN * 128) / 4; i += 128) {
    uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
    reinterpret_cast<uint32_t*>(smem)[i] = I8 ? x : ((x & 0x83FF83FFu) | 0x24002400u);
  }
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(p_smem_u32(bar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the generic-proxy stores above are read by the tensor core
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(p_smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // instruction descriptor: accumulator format at bit 4 (1 = f32, 2 = s32), A / B formats at bits 7 / 10 (kind::f16: 0 = fp16;
  // kind::i8: 1 = signed 8 bit), both operands K-major, N >> 3 at bit 17, M >> 4 at bit 24
  constexpr uint32_t idesc = (I8 ? (2u << 4) | (1u << 7) | (1u << 10) : (1u << 4)) | ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);
  const uint32_t a0 = p_smem_u32(smem), b0 = p_smem_u32(smem + PM * 128);
  bool ok = true;
  if (threadIdx.x == 0) {
    const unsigned long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tmem + (uint32_t)((it & 1) * PN);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint64_t ad = p_desc(a0 + k * 32), bd = p_desc(b0 + k * 32);
        const uint32_t accumulate = (it > 1 || k > 0) ? 1u : 0u;
        if (I8)
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                       "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate)
                       : "memory");
        else
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                       "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate)
                       : "memory");
      }
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(p_smem_u32(bar)) : "memory");
    ok = false;
    for (uint32_t i = 0; i < spin_limit; ++i) {
      uint32_t done;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(done)
                   : "r"(p_smem_u32(bar)), "r"(0u)
                   : "memory");
      if (done) { ok = true; break; }
    }
    if (!ok) atomicOr(err, 64u);
    if (clk) clk[blockIdx.x] = clock64() - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    if (!ok) {  // (lane 0 gave up: let what is still in flight land before TMEM is released)
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  }
}

}  // namespace

extern "C" int izb_tensor_peak(int device, int kind, int iters, int launches, double* tops, double* clk_per_mma) {
  if (!tops) IZB_FAIL(IZB_ERR_ARG, "tensor_peak: null pointer");
  if (kind != 0 && kind != 1) IZB_FAIL(IZB_ERR_ARG, "tensor_peak: kind %d (0 = kind::f16, 1 = kind::i8)", kind);
  if (iters < 1 || iters > (1 << 22) || launches < 1 || launches > 100000) IZB_FAIL(IZB_ERR_ARG, "tensor_peak: iters = %d, launches = %d", iters, launches);
  if (int rc = izb_require_device(device, "tensor_peak")) return rc;
  uint32_t* err = izb_device_error_word(device);
  if (!err) IZB_FAIL(IZB_ERR_NOMEM, "tensor_peak: no device error word");
  const int grid = izb_sm_count(device);
  unsigned long long* d_clk = nullptr;
  IZB_CUDA(cudaMalloc(&d_clk, (size_t)grid * 8));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaError_t e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  int rc = IZB_OK;
  auto launch = [&](int n_it) -> int {
    if (kind == 1) {
      IZB_SMEM_OPTIN((mma_peak_kernel<true>), kPeakSmem, device);
      IZB_LAUNCH("mma_peak", 0, mma_peak_kernel<true><<<grid, 128, kPeakSmem>>>(n_it, 1u << 24, err, d_clk));
    } else {
      IZB_SMEM_OPTIN((mma_peak_kernel<false>), kPeakSmem, device);
      IZB_LAUNCH("mma_peak", 0, mma_peak_kernel<false><<<grid, 128, kPeakSmem>>>(n_it, 1u << 24, err, d_clk));
    }
    return IZB_OK;
  };
  if (e == cudaSuccess) rc = launch(iters < 64 ? iters : 64);  // warm-up (loads the kernel's code)
  if (e == cudaSuccess && rc == IZB_OK) e = cudaDeviceSynchronize();
  if (e == cudaSuccess && rc == IZB_OK) {
    cudaEventRecord(e0, 0);
    for (int i = 0; i < launches && rc == IZB_OK; ++i) rc = launch(iters);
    cudaEventRecord(e1, 0);
    e = cudaEventSynchronize(e1);
  }
  float ms = 0.0f;
  if (e == cudaSuccess && rc == IZB_OK) e = cudaEventElapsedTime(&ms, e0, e1);
  unsigned long long c0 = 0;
  if (e == cudaSuccess && rc == IZB_OK) e = cudaMemcpy(&c0, d_clk, 8, cudaMemcpyDeviceToHost);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(d_clk);
  if (rc != IZB_OK) return rc;
  IZB_CUDA(e);
  const double ops = 2.0 * PM * PN * (kind == 1 ? 32 : 16) * 4.0 * iters * (double)launches * grid;
  *tops = ops / (ms * 1e-3) / 1e12;
  if (clk_per_mma) *clk_per_mma = (double)c0 / (4.0 * iters);
  return IZB_OK;
}
