// Tensor-parallel sums.  The reference sums the partial outputs of its row-parallel projections (attention output,
// FFN down) with its own host barrier + copies (TpComm, zero/mgpu/engine_tp.h:36-124; tp_reduce_at :272-324; tp_add
// zero/kernels/tp.cl:5-11).  Here the exchange is NCCL over NVLink: one process per GPU, one communicator per process.
//
// NCCL is resolved at run time from the library the process already has loaded (the framework's bundled libnccl.so.2),
// so that no second copy of NCCL is linked in.  Only the stable C entry points below are used.
#include <dlfcn.h>
#include <limits.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <thread>

#include "izb_common.cuh"

namespace {

__global__ void tp_add_kernel(float* __restrict__ x, const float* __restrict__ p, size_t n, int np, size_t stride) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = x[i];
  for (int k = 0; k < np; ++k) s = __fadd_rn(s, p[(size_t)k * stride + i]);
  x[i] = s;
}

__global__ void tp_add1_v4_kernel(float4* __restrict__ x, const float4* __restrict__ p, size_t n4) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 a = x[i];
  const float4 b = p[i];
  a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
  x[i] = a;
}

extern "C" int izb_tp_range(int64_t total, int64_t unit, int nranks, int rank, int64_t* begin, int64_t* end);

// ---- the few NCCL entry points, by their public C signatures (nccl.h)
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclInt8 = 0, ncclFloat32 = 7 };
enum { ncclSum = 0 };
enum { ncclSuccess = 0, ncclInProgress = 7 };
// The leading fields of ncclConfig_t as nccl.h has declared them since 2.18 (later versions only append; the library reads
// `size` and `version` and gives every field past them its default).
struct ncclConfigPrefix {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;
  int cgaClusterSize;
  int minCTAs;
  int maxCTAs;
  const char* netName;
  int splitShare;
};
struct NcclApi {
  void* h = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfigPrefix*) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    g_nccl.h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.h) break;
  }
  if (!g_nccl.h) return;
#define SYM(f) *(void**)(&g_nccl.f) = dlsym(g_nccl.h, "nccl" #f)
  SYM(GetUniqueId); SYM(CommInitRank); SYM(CommDestroy); SYM(AllReduce); SYM(ReduceScatter); SYM(AllGather);
  SYM(GroupStart); SYM(GroupEnd); SYM(GetErrorString); SYM(CommInitRankConfig); SYM(CommGetAsyncError); SYM(CommAbort); SYM(Broadcast);
#undef SYM
  g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllReduce && g_nccl.ReduceScatter &&
              g_nccl.AllGather && g_nccl.GroupStart && g_nccl.GroupEnd;
}

int need_nccl() {
  std::call_once(g_nccl_once, load_nccl);
  if (!g_nccl.ok) {
    const char* why = dlerror();  // (a second call would return NULL: the message is consumed by the first)
    IZB_FAIL(IZB_ERR_NCCL, "libnccl.so.2 could not be loaded (%s)", why ? why : "symbols missing");
  }
  return IZB_OK;
}

#define IZB_NCCL(call)                                                                                            \
  do {                                                                                                            \
    int r__ = (call);                                                                                             \
    if (r__ != 0) {                                                                                               \
      izb_set_error("%s failed: %s", #call, g_nccl.GetErrorString ? g_nccl.GetErrorString(r__) : "nccl error");   \
      return IZB_ERR_NCCL;                                                                                        \
    }                                                                                                             \
  } while (0)

}  // namespace

struct izb_tp {
  int nranks = 1, rank = 0, device = 0;
  ncclComm_t comm = nullptr;
  int timeout_ms = 0;    // > 0: non-blocking communicator, every NCCL call is followed by a bounded wait for its result
  bool aborted = false;  // the communicator was aborted after a time-out or an asynchronous error: it takes no more calls
  cudaEvent_t done = nullptr;
};

namespace {
// Bounded wait for a call on a non-blocking communicator to leave the "in progress" state (the reference bounds every
// barrier and wait of its own transport the same way, zero/mgpu/engine_tp.h:93-123).  On a time-out or an error the
// communicator is aborted -- ncclCommAbort also ends collectives of this rank that are stuck on the device -- and marked.
int tp_settle(izb_tp* tp, int r, const char* what) {
  if (tp->timeout_ms <= 0 || !tp->comm) {
    if (r != ncclSuccess) {
      izb_set_error("%s failed: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error");
      return IZB_ERR_NCCL;
    }
    return IZB_OK;
  }
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(tp->timeout_ms);
  int state = r;
  while (state == ncclInProgress) {
    if (g_nccl.CommGetAsyncError(tp->comm, &state) != ncclSuccess) { state = -1; break; }
    if (state != ncclInProgress) break;
    if (std::chrono::steady_clock::now() > t_end) break;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  if (state == ncclSuccess) return IZB_OK;
  g_nccl.CommAbort(tp->comm);
  tp->comm = nullptr;
  tp->aborted = true;
  if (state == ncclInProgress) {
    izb_set_error("%s: no answer from the other ranks within %d ms; communicator aborted", what, tp->timeout_ms);
    return IZB_ERR_TIMEOUT;
  }
  izb_set_error("%s failed: %s; communicator aborted", what, state > 0 && g_nccl.GetErrorString ? g_nccl.GetErrorString(state) : "nccl error");
  return IZB_ERR_NCCL;
}
int tp_usable(izb_tp* tp, const char* what) {
  if (tp->aborted) IZB_FAIL(IZB_ERR_NCCL, "%s: the communicator was aborted after a time-out or an error; create a new one", what);
  return IZB_OK;
}
}  // namespace
#define IZB_TP_NCCL(tp, call, what)                      \
  do {                                                   \
    if (int rc__ = tp_settle((tp), (call), (what))) return rc__; \
  } while (0)

extern "C" int izb_tp_add(float* d_x, const float* d_parts, size_t n, int np, size_t stride, void* stream) {
  if (!d_x || !d_parts) IZB_FAIL(IZB_ERR_ARG, "tp_add: null pointer");
  if (np < 1 || n < 1) IZB_FAIL(IZB_ERR_SHAPE, "tp_add: n = %zu, np = %d", n, np);
  tp_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_x, d_parts, n, np, stride);
  IZB_LAUNCHED();
  return IZB_OK;
}

extern "C" int izb_tp_unique_id(void* id128) {
  if (!id128) IZB_FAIL(IZB_ERR_ARG, "tp_unique_id: null pointer");
  if (int rc = need_nccl()) return rc;
  ncclUniqueId id;
  IZB_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, 128);
  return IZB_OK;
}

extern "C" int izb_tp_create_ex(int nranks, int rank, const void* id128, int device, int timeout_ms, int max_ctas, izb_tp** out) {
  if (!out || (nranks > 1 && !id128)) IZB_FAIL(IZB_ERR_ARG, "tp_create: null pointer");
  *out = nullptr;
  if (nranks < 1 || rank < 0 || rank >= nranks) IZB_FAIL(IZB_ERR_ARG, "tp_create: rank %d of %d", rank, nranks);
  if (timeout_ms < 0 || max_ctas < 0) IZB_FAIL(IZB_ERR_ARG, "tp_create: timeout_ms = %d, max_ctas = %d", timeout_ms, max_ctas);
  IZB_CUDA(cudaSetDevice(device));
  izb_tp* tp = new izb_tp;
  tp->nranks = nranks;
  tp->rank = rank;
  tp->device = device;
  if (cudaEventCreateWithFlags(&tp->done, cudaEventDisableTiming) != cudaSuccess) {
    delete tp;
    IZB_FAIL(IZB_ERR_CUDA, "tp_create: cannot create an event");
  }
  if (nranks > 1) {
    if (int rc = need_nccl()) { cudaEventDestroy(tp->done); delete tp; return rc; }
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    int r;
    if (timeout_ms > 0 || max_ctas > 0) {
      if (!g_nccl.CommInitRankConfig || !g_nccl.CommGetAsyncError || !g_nccl.CommAbort) {
        cudaEventDestroy(tp->done);
        delete tp;
        IZB_FAIL(IZB_ERR_NCCL, "tp_create: this NCCL has no ncclCommInitRankConfig / ncclCommGetAsyncError / ncclCommAbort (2.18 or later needed)");
      }
      ncclConfigPrefix cfg;
      cfg.size = sizeof cfg;
      cfg.magic = 0xcafebeefu;
      cfg.version = 21800;  // NCCL_VERSION(2, 18, 0): the version whose ncclConfig_t ends with splitShare
      cfg.blocking = timeout_ms > 0 ? 0 : 1;
      cfg.cgaClusterSize = INT_MIN;  // NCCL_CONFIG_UNDEF_INT: the library's default
      cfg.minCTAs = INT_MIN;
      cfg.maxCTAs = max_ctas > 0 ? max_ctas : INT_MIN;
      cfg.netName = nullptr;
      cfg.splitShare = INT_MIN;
      tp->timeout_ms = timeout_ms;
      r = g_nccl.CommInitRankConfig(&tp->comm, nranks, id, rank, &cfg);
      if (timeout_ms > 0 && (r == ncclSuccess || r == ncclInProgress)) r = ncclInProgress;  // (the state is polled below)
    } else {
      r = g_nccl.CommInitRank(&tp->comm, nranks, id, rank);
    }
    if (int rc = tp_settle(tp, r, "ncclCommInitRank")) {
      if (tp->comm && !tp->aborted) g_nccl.CommAbort ? g_nccl.CommAbort(tp->comm) : g_nccl.CommDestroy(tp->comm);
      cudaEventDestroy(tp->done);
      delete tp;
      return rc;
    }
  }
  *out = tp;
  return IZB_OK;
}

extern "C" int izb_tp_create(int nranks, int rank, const void* id128, int device, izb_tp** out) {
  return izb_tp_create_ex(nranks, rank, id128, device, 0, 0, out);
}

extern "C" int izb_tp_abort(izb_tp* tp) {
  if (!tp) IZB_FAIL(IZB_ERR_ARG, "tp_abort: null handle");
  if (tp->comm && g_nccl.CommAbort) {
    g_nccl.CommAbort(tp->comm);
    tp->comm = nullptr;
  }
  tp->aborted = tp->nranks > 1;
  return IZB_OK;
}

extern "C" int izb_tp_wait(izb_tp* tp, void* stream, int timeout_ms) {
  if (!tp) IZB_FAIL(IZB_ERR_ARG, "tp_wait: null handle");
  if (timeout_ms < 1) IZB_FAIL(IZB_ERR_ARG, "tp_wait: timeout_ms = %d", timeout_ms);
  if (int rc = izb_require_device(tp->device, "tp_wait")) return rc;
  IZB_CUDA(cudaEventRecord(tp->done, (cudaStream_t)stream));
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    const cudaError_t q = cudaEventQuery(tp->done);
    if (q == cudaSuccess) return IZB_OK;
    if (q != cudaErrorNotReady) IZB_CUDA(q);
    int state = ncclSuccess;
    const bool async_ok = !tp->comm || !g_nccl.CommGetAsyncError || g_nccl.CommGetAsyncError(tp->comm, &state) == ncclSuccess;
    const bool failed = !async_ok || (state != ncclSuccess && state != ncclInProgress);
    if (failed || std::chrono::steady_clock::now() > t_end) {
      // ending the communicator also ends this rank's collectives that wait on the device for a peer
      if (tp->comm && g_nccl.CommAbort) {
        g_nccl.CommAbort(tp->comm);
        tp->comm = nullptr;
        tp->aborted = true;
      }
      if (failed) IZB_FAIL(IZB_ERR_NCCL, "tp_wait: NCCL reported %s; communicator aborted", state > 0 && g_nccl.GetErrorString ? g_nccl.GetErrorString(state) : "an error");
      IZB_FAIL(IZB_ERR_TIMEOUT, "tp_wait: the work queued on the stream did not finish within %d ms (a peer is missing?); communicator aborted", timeout_ms);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(100));
  }
}

extern "C" void izb_tp_destroy(izb_tp* tp) {
  if (!tp) return;
  if (tp->comm) g_nccl.CommDestroy(tp->comm);
  if (tp->done) cudaEventDestroy(tp->done);
  delete tp;
}

extern "C" int izb_tp_allreduce_rows(izb_tp* tp, float* d_x, float* d_part, int rows, int E, void* stream) {
  if (!tp || !d_x || !d_part) IZB_FAIL(IZB_ERR_ARG, "tp_allreduce_rows: null pointer");
  if (rows < 1 || E < 4 || E % 4) IZB_FAIL(IZB_ERR_SHAPE, "tp_allreduce_rows: rows=%d E=%d (E %% 4 == 0)", rows, E);
  if (!izb_aligned(d_x, 16) || !izb_aligned(d_part, 16)) IZB_FAIL(IZB_ERR_ALIGN, "tp_allreduce_rows: buffers must be 16-byte aligned");
  if (int rc = izb_require_device(tp->device, "tp_allreduce_rows")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = (size_t)rows * E;
  if (int rc = tp_usable(tp, "tp_allreduce_rows")) return rc;
  if (tp->nranks > 1) IZB_TP_NCCL(tp, g_nccl.AllReduce(d_part, d_part, n, ncclFloat32, ncclSum, tp->comm, st), "ncclAllReduce");
  tp_add1_v4_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>((float4*)d_x, (const float4*)d_part, n / 4);
  IZB_LAUNCHED();
  return IZB_OK;
}

extern "C" int izb_tp_reduce_quant_gather(izb_tp* tp, const float* d_x, float* d_part, int rows, int E, float* d_xsum,
                                          int8_t* d_aq, float* d_asc, void* stream) {
  if (!tp || !d_part || !d_aq || !d_asc) IZB_FAIL(IZB_ERR_ARG, "tp_reduce_quant_gather: null pointer");
  const int R = tp->nranks;
  if (rows < 1 || rows % (16 * R) || E % 256) IZB_FAIL(IZB_ERR_SHAPE, "tp_reduce_quant_gather: rows=%d (multiple of 16*%d) E=%d (multiple of 256)", rows, R, E);
  if (int rc = izb_require_device(tp->device, "tp_reduce_quant_gather")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int own = rows / R;
  const size_t n_own = (size_t)own * E;
  // 1. this rank's token rows of the sum of partials, in place at their position in d_part
  float* mine = d_part + (size_t)tp->rank * n_own;
  if (int rc = tp_usable(tp, "tp_reduce_quant_gather")) return rc;
  if (R > 1) IZB_TP_NCCL(tp, g_nccl.ReduceScatter(d_part, mine, n_own, ncclFloat32, ncclSum, tp->comm, st), "ncclReduceScatter");
  // 2. + this rank's rows of the residual stream
  if (d_x) {
    tp_add1_v4_kernel<<<(unsigned)((n_own / 4 + 255) / 256), 256, 0, st>>>((float4*)mine, (const float4*)(d_x + (size_t)tp->rank * n_own), n_own / 4);
    IZB_LAUNCHED();
  }
  if (d_xsum) IZB_CUDA(cudaMemcpyAsync(d_xsum, mine, n_own * 4, cudaMemcpyDeviceToDevice, st));
  // 3. quantise the own rows into rank-major staging: aq rows are contiguous per rank; the scales are [E/32][own] per
  //    rank and are re-laid to [E/32][rows] after the gather
  void* ws = nullptr;
  const size_t sc_bytes = (size_t)(E / 32) * rows * 4;
  if (int rc = izb_workspace(tp->device, kWsTp, sc_bytes, &ws)) return rc;
  float* sc_stage = (float*)ws;  // [R][E/32][own]
  if (int rc = izb_quantize_act(mine, E, own, own, E, d_aq + (size_t)tp->rank * n_own, sc_stage + (size_t)tp->rank * (E / 32) * own, nullptr, st)) return rc;
  if (R > 1) {
    // (inside a group a non-blocking communicator answers "in progress"; the group's end carries the result)
    IZB_NCCL(g_nccl.GroupStart());
    int r1 = g_nccl.AllGather(d_aq + (size_t)tp->rank * n_own, d_aq, n_own, ncclInt8, tp->comm, st);
    int r2 = g_nccl.AllGather(sc_stage + (size_t)tp->rank * (E / 32) * own, sc_stage, (size_t)(E / 32) * own, ncclFloat32, tp->comm, st);
    if (r1 == ncclInProgress) r1 = ncclSuccess;
    if (r2 == ncclInProgress) r2 = ncclSuccess;
    IZB_NCCL(r1);
    IZB_NCCL(r2);
    IZB_TP_NCCL(tp, g_nccl.GroupEnd(), "ncclAllGather");
  }
  // 4. [R][E/32][own] -> [E/32][R*own]
  IZB_CUDA(cudaMemcpy2DAsync(d_asc, (size_t)rows * 4, sc_stage, (size_t)own * 4, (size_t)own * 4, (size_t)(E / 32), cudaMemcpyDeviceToDevice, st));
  for (int r = 1; r < R; ++r)
    IZB_CUDA(cudaMemcpy2DAsync(d_asc + (size_t)r * own, (size_t)rows * 4, sc_stage + (size_t)r * (E / 32) * own, (size_t)own * 4,
                               (size_t)own * 4, (size_t)(E / 32), cudaMemcpyDeviceToDevice, st));
  return IZB_OK;
}

// The output head split by vocabulary rows (zero/mgpu/engine_tp_shard.h:68-72 with units of 16 rows; the reference joins the
// shards' logits on the host in rank order, zero/mgpu/engine_tp.h:853-862).  Every rank passes its own logits
// d_local [rows][ld_local] (its vocabulary rows [begin_r, end_r) of izb_tp_range(vocab, 16, nranks, rank) in the first
// end_r - begin_r columns) and receives all of them in d_full [rows][ld_full]: one broadcast per rank and token row, grouped.
extern "C" int izb_tp_gather_logits(izb_tp* tp, const float* d_local, int ld_local, int rows, int vocab, float* d_full, int ld_full,
                                    void* stream) {
  if (!tp || !d_local || !d_full) IZB_FAIL(IZB_ERR_ARG, "tp_gather_logits: null pointer");
  if (rows < 1 || rows > 64 || vocab < 1 || ld_full < vocab) IZB_FAIL(IZB_ERR_SHAPE, "tp_gather_logits: rows=%d (1..64) vocab=%d ld_full=%d", rows, vocab, ld_full);
  if (int rc = izb_require_device(tp->device, "tp_gather_logits")) return rc;
  if (int rc = tp_usable(tp, "tp_gather_logits")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int R = tp->nranks;
  int64_t b0 = 0, b1 = 0;
  izb_tp_range(vocab, 16, R, tp->rank, &b0, &b1);
  if (tp->rank == R - 1) b1 = vocab;  // (the rows past the last whole unit of 16 belong to the last rank)
  if (ld_local < (int)(b1 - b0)) IZB_FAIL(IZB_ERR_SHAPE, "tp_gather_logits: ld_local = %d < this rank's %lld rows", ld_local, (long long)(b1 - b0));
  if (R == 1) {
    IZB_CUDA(cudaMemcpy2DAsync(d_full, (size_t)ld_full * 4, d_local, (size_t)ld_local * 4, (size_t)vocab * 4, rows, cudaMemcpyDeviceToDevice, st));
    return IZB_OK;
  }
  if (!g_nccl.Broadcast) IZB_FAIL(IZB_ERR_NCCL, "tp_gather_logits: ncclBroadcast is missing");
  IZB_NCCL(g_nccl.GroupStart());
  int worst = ncclSuccess;
  for (int r = 0; r < R; ++r) {
    int64_t rb = 0, re = 0;
    izb_tp_range(vocab, 16, R, r, &rb, &re);
    if (r == R - 1) re = vocab;  // (rows past the last whole unit of 16 belong to the last rank)
    if (re <= rb) continue;
    for (int t = 0; t < rows; ++t) {
      const float* src = r == tp->rank ? d_local + (size_t)t * ld_local : d_full + (size_t)t * ld_full + rb;  // (ignored on non-roots)
      int rr = g_nccl.Broadcast(src, d_full + (size_t)t * ld_full + rb, (size_t)(re - rb), ncclFloat32, r, tp->comm, st);
      if (rr != ncclSuccess && rr != ncclInProgress) worst = rr;
    }
  }
  IZB_NCCL(worst);
  IZB_TP_NCCL(tp, g_nccl.GroupEnd(), "ncclBroadcast");
  return IZB_OK;
}
