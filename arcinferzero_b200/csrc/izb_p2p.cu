// Peer transport for the tensor-parallel sums that needs no multiprocessor: copies by the copy engines into buffers of the
// other ranks that the host has mapped into this process (CUDA IPC, virtual memory management or a symmetric-memory
// allocator: the library only sees plain device pointers), and 32-bit flags written behind the data and waited for with
// the driver's stream memory operations.  The reference moves its partial sums the same way -- every rank copies its
// rows to the owner and raises a counter, the owner adds them in rank order (TpComm / tp_reduce_at,
// zero/mgpu/engine_tp.h:36-124,272-324; tp_add, zero/kernels/tp.cl:5-11) -- through host-visible memory; here the copies
// cross NVLink and nothing on the host waits.
//
// No kernel of this file touches another GPU's memory, and no wait spins on a multiprocessor: a persistent GEMM that
// holds every SM runs beside the transfers.
//
// Two rules of the stream memory operations shape the interface.  (1) A stream may wait only for a value that ANOTHER
// device writes: CUDA does not see the order between a wait and a write issued on two streams of one device and may run
// them the wrong way round, for good.  What a rank hands to itself is ordered with events by the caller.  (2) A stream wait
// has no time limit and, by (1), this device cannot release it: izb_p2p_wait_host bounds the HOST's wait and reports
// IZB_ERR_TIMEOUT; the stream itself stays blocked until the peer writes or the process gives the context up.
#include <cuda.h>

#include <chrono>
#include <thread>

#include "izb_common.cuh"

namespace {

typedef CUresult (*StreamValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

StreamValueFn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return (StreamValueFn)p;
}
StreamValueFn write_value() {
  static StreamValueFn fn = driver_fn("cuStreamWriteValue32");
  return fn;
}
StreamValueFn wait_value() {
  static StreamValueFn fn = driver_fn("cuStreamWaitValue32");
  return fn;
}

}  // namespace

extern "C" int izb_p2p_push(int n_copies, void* const* d_dst, const void* const* d_src, const size_t* bytes, int n_flags,
                            uint32_t* const* d_flags, uint32_t value, void* stream) {
  if (n_copies < 0 || n_flags < 0 || n_copies > 4096 || n_flags > 4096) IZB_FAIL(IZB_ERR_ARG, "p2p_push: %d copies, %d flags", n_copies, n_flags);
  if ((n_copies && (!d_dst || !d_src || !bytes)) || (n_flags && !d_flags)) IZB_FAIL(IZB_ERR_ARG, "p2p_push: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  for (int i = 0; i < n_copies; ++i) {
    if (!d_dst[i] || !d_src[i]) IZB_FAIL(IZB_ERR_ARG, "p2p_push: copy %d has a null pointer", i);
    if (bytes[i]) IZB_CUDA(cudaMemcpyAsync(d_dst[i], d_src[i], bytes[i], cudaMemcpyDeviceToDevice, st));
  }
  if (n_flags) {
    StreamValueFn wr = write_value();
    if (!wr) IZB_FAIL(IZB_ERR_CUDA, "p2p_push: the driver has no cuStreamWriteValue32");
    for (int i = 0; i < n_flags; ++i) {
      if (!d_flags[i] || !izb_aligned(d_flags[i], 4)) IZB_FAIL(IZB_ERR_ALIGN, "p2p_push: flag %d is null or not 4-byte aligned", i);
      // (in stream order behind the copies above: a reader that sees the value sees the data)
      const CUresult r = wr((CUstream)st, (CUdeviceptr)(uintptr_t)d_flags[i], value, 0);
      if (r != CUDA_SUCCESS) IZB_FAIL(IZB_ERR_CUDA, "p2p_push: cuStreamWriteValue32 failed (%d)", (int)r);
    }
  }
  return IZB_OK;
}

extern "C" int izb_p2p_wait(int n_flags, uint32_t* const* d_flags, uint32_t value, void* stream) {
  if (n_flags < 0 || n_flags > 4096 || (n_flags && !d_flags)) IZB_FAIL(IZB_ERR_ARG, "p2p_wait: %d flags", n_flags);
  StreamValueFn wt = wait_value();
  if (!wt) IZB_FAIL(IZB_ERR_CUDA, "p2p_wait: the driver has no cuStreamWaitValue32");
  for (int i = 0; i < n_flags; ++i) {
    if (!d_flags[i] || !izb_aligned(d_flags[i], 4)) IZB_FAIL(IZB_ERR_ALIGN, "p2p_wait: flag %d is null or not 4-byte aligned", i);
    // flags only ever grow (a sequence number per sum), so "greater or equal" also holds for a waiter that comes late
    const CUresult r = wt((CUstream)stream, (CUdeviceptr)(uintptr_t)d_flags[i], value, CU_STREAM_WAIT_VALUE_GEQ);
    if (r != CUDA_SUCCESS) IZB_FAIL(IZB_ERR_CUDA, "p2p_wait: cuStreamWaitValue32 failed (%d)", (int)r);
  }
  return IZB_OK;
}

extern "C" int izb_p2p_wait_host(void* stream, int timeout_ms) {
  if (timeout_ms < 1) IZB_FAIL(IZB_ERR_ARG, "p2p_wait_host: timeout_ms = %d", timeout_ms);
  cudaEvent_t done = nullptr;
  IZB_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(done, (cudaStream_t)stream);
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  bool timed_out = false;
  while (e == cudaSuccess) {
    const cudaError_t q = cudaEventQuery(done);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) { e = q; break; }
    if (std::chrono::steady_clock::now() > t_end) { timed_out = true; break; }
    std::this_thread::sleep_for(std::chrono::microseconds(100));
  }
  cudaEventDestroy(done);  // (a pending event is released when it completes)
  IZB_CUDA(e);
  if (timed_out) IZB_FAIL(IZB_ERR_TIMEOUT, "p2p_wait_host: the stream did not drain within %d ms (a peer never raised its flag?)", timeout_ms);
  return IZB_OK;
}

// The block scales of the gathered rows: every rank's [E/32][own] block, rank after rank (the form in which the owners
// push them), into the GEMM's [E/32][rows] layout with rows = nranks * own.
extern "C" int izb_tp_scales_from_ranks(float* d_asc, const float* d_stage, int nranks, int own, int E, void* stream) {
  if (!d_asc || !d_stage) IZB_FAIL(IZB_ERR_ARG, "tp_scales_from_ranks: null pointer");
  if (nranks < 1 || own < 1 || E < 32 || E % 32) IZB_FAIL(IZB_ERR_SHAPE, "tp_scales_from_ranks: nranks=%d own=%d E=%d", nranks, own, E);
  const size_t rows = (size_t)nranks * own;
  for (int r = 0; r < nranks; ++r)
    IZB_CUDA(cudaMemcpy2DAsync(d_asc + (size_t)r * own, rows * 4, d_stage + (size_t)r * (E / 32) * own, (size_t)own * 4, (size_t)own * 4,
                               (size_t)(E / 32), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return IZB_OK;
}
