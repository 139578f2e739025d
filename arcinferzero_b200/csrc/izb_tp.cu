// Tensor-parallel sums.  The reference sums the partial outputs of its row-parallel projections (attention output,
// FFN down) with its own host barrier + copies (TpComm, zero/mgpu/engine_tp.h:36-124; tp_reduce_at :272-324; tp_add
// zero/kernels/tp.cl:5-11).  Here the exchange is NCCL over NVLink: one process per GPU, one communicator per process.
//
// NCCL is resolved at run time from the library the process already has loaded (the framework's bundled libnccl.so.2),
// so that no second copy of NCCL is linked in.  Only the stable C entry points below are used.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

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

// ---- the few NCCL entry points, by their public C signatures (nccl.h)
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclInt8 = 0, ncclFloat32 = 7 };
enum { ncclSum = 0 };
struct NcclApi {
  void* h = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
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
  SYM(GroupStart); SYM(GroupEnd); SYM(GetErrorString);
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
};

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

extern "C" int izb_tp_create(int nranks, int rank, const void* id128, int device, izb_tp** out) {
  if (!out || (nranks > 1 && !id128)) IZB_FAIL(IZB_ERR_ARG, "tp_create: null pointer");
  *out = nullptr;
  if (nranks < 1 || rank < 0 || rank >= nranks) IZB_FAIL(IZB_ERR_ARG, "tp_create: rank %d of %d", rank, nranks);
  IZB_CUDA(cudaSetDevice(device));
  izb_tp* tp = new izb_tp;
  tp->nranks = nranks;
  tp->rank = rank;
  tp->device = device;
  if (nranks > 1) {
    if (int rc = need_nccl()) { delete tp; return rc; }
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    const int r = g_nccl.CommInitRank(&tp->comm, nranks, id, rank);
    if (r != 0) {
      delete tp;
      IZB_FAIL(IZB_ERR_NCCL, "ncclCommInitRank failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error");
    }
  }
  *out = tp;
  return IZB_OK;
}

extern "C" void izb_tp_destroy(izb_tp* tp) {
  if (!tp) return;
  if (tp->comm) g_nccl.CommDestroy(tp->comm);
  delete tp;
}

extern "C" int izb_tp_allreduce_rows(izb_tp* tp, float* d_x, float* d_part, int rows, int E, void* stream) {
  if (!tp || !d_x || !d_part) IZB_FAIL(IZB_ERR_ARG, "tp_allreduce_rows: null pointer");
  if (rows < 1 || E < 4 || E % 4) IZB_FAIL(IZB_ERR_SHAPE, "tp_allreduce_rows: rows=%d E=%d (E %% 4 == 0)", rows, E);
  if (!izb_aligned(d_x, 16) || !izb_aligned(d_part, 16)) IZB_FAIL(IZB_ERR_ALIGN, "tp_allreduce_rows: buffers must be 16-byte aligned");
  if (int rc = izb_require_device(tp->device, "tp_allreduce_rows")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = (size_t)rows * E;
  if (tp->nranks > 1) IZB_NCCL(g_nccl.AllReduce(d_part, d_part, n, ncclFloat32, ncclSum, tp->comm, st));
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
  if (R > 1) IZB_NCCL(g_nccl.ReduceScatter(d_part, mine, n_own, ncclFloat32, ncclSum, tp->comm, st));
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
    IZB_NCCL(g_nccl.GroupStart());
    IZB_NCCL(g_nccl.AllGather(d_aq + (size_t)tp->rank * n_own, d_aq, n_own, ncclInt8, tp->comm, st));
    IZB_NCCL(g_nccl.AllGather(sc_stage + (size_t)tp->rank * (E / 32) * own, sc_stage, (size_t)(E / 32) * own, ncclFloat32, tp->comm, st));
    IZB_NCCL(g_nccl.GroupEnd());
  }
  // 4. [R][E/32][own] -> [E/32][R*own]
  IZB_CUDA(cudaMemcpy2DAsync(d_asc, (size_t)rows * 4, sc_stage, (size_t)own * 4, (size_t)own * 4, (size_t)(E / 32), cudaMemcpyDeviceToDevice, st));
  for (int r = 1; r < R; ++r)
    IZB_CUDA(cudaMemcpy2DAsync(d_asc + (size_t)r * own, (size_t)rows * 4, sc_stage + (size_t)r * (E / 32) * own, (size_t)own * 4,
                               (size_t)own * 4, (size_t)(E / 32), cudaMemcpyDeviceToDevice, st));
  return IZB_OK;
}
