// C ABI of the library: weight handles, the row-count dispatch of Engine::matmul (zero/engine.h:1147-1251), the
// verification entry points and the host-buffer convenience call.
#include <cuda.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "izb_common.cuh"

std::atomic<uint64_t> g_izb_launches{0};

// kernels of the other translation units
int izb_gemm_core_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int M, int Mp, float* C,
                         int ldc, int c_off, int acc, int32_t* dots, cudaStream_t st);
// returns IZB_OK, an error, or +1 when the tensor-core kernel does not take this shape
int izb_gemm_tc_launch(const izb_weight* w, int mat, const int8_t* aq, const float* asc, int M, int Mp, float* C, int ldc,
                       int c_off, int acc, int32_t* dots, cudaStream_t st);
int izb_make_raw_tensor_map(izb_weight* w);
int izb_gemm_k16_launch(const izb_weight* w, const uint8_t* raw, const int8_t* aq, const float* asc, int M, int Mp, float* C, int ldc,
                        int c_off, int acc, int32_t* dots, cudaStream_t st);

int izb_gemm_tc_quant_launch(const izb_weight* w, int mat, const float* x, int ldx, int M, int Mp, int8_t* aq, float* asc, float* C,
                             int ldc, int c_off, int acc, cudaStream_t st);
int izb_swiglu_pairs_launch(const float* gu, int ldgu, int M, int F, float* C, int ldc, int c_off, cudaStream_t st);

// ---------------------------------------------------------------------------------------------- errors
static thread_local char t_err[512] = "";

void izb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof t_err, fmt, ap);
  va_end(ap);
}

extern "C" const char* izb_last_error(void) { return t_err; }
extern "C" uint64_t izb_launch_count(void) { return g_izb_launches.load(); }

extern "C" const char* izb_status_string(int s) {
  switch (s) {
    case IZB_OK: return "ok";
    case IZB_ERR_ARG: return "bad argument";
    case IZB_ERR_SHAPE: return "bad shape";
    case IZB_ERR_TYPE: return "unsupported weight type";
    case IZB_ERR_ALIGN: return "misaligned pointer or stride";
    case IZB_ERR_CUDA: return "CUDA error";
    case IZB_ERR_NCCL: return "NCCL error";
    case IZB_ERR_TIMEOUT: return "device-side wait timed out";
    case IZB_ERR_NOMEM: return "out of memory";
    case IZB_ERR_SELFCHECK: return "self-check failed";
    case IZB_ERR_LIMIT: return "capacity exceeded";
    default: return "unknown status";
  }
}

// ---------------------------------------------------------------------------------------------- per-kernel timing
namespace {
struct ProfRec { const char* name; cudaEvent_t a, b; };
std::atomic<int> g_prof_on{0};
std::mutex g_prof_mu;
std::vector<ProfRec> g_prof;
std::vector<cudaEvent_t> g_prof_pool;
cudaEvent_t prof_event() {
  if (!g_prof_pool.empty()) { cudaEvent_t e = g_prof_pool.back(); g_prof_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
}  // namespace

void izb_prof_begin(const char* name, cudaStream_t st) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  ProfRec r{name, prof_event(), prof_event()};
  cudaEventRecord(r.a, st);
  g_prof.push_back(r);
}
void izb_prof_end(cudaStream_t st) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (!g_prof.empty()) cudaEventRecord(g_prof.back().b, st);
}

extern "C" int izb_profile_start(void) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) { g_prof_pool.push_back(r.a); g_prof_pool.push_back(r.b); }
  g_prof.clear();
  g_prof_on.store(1);
  return IZB_OK;
}

extern "C" int izb_profile_stop(char* json, size_t cap) {
  g_prof_on.store(0);
  if (!json || cap < 64) IZB_FAIL(IZB_ERR_ARG, "profile_stop: buffer too small");
  IZB_CUDA(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lk(g_prof_mu);
  struct Agg { const char* name; int n; double ms; };
  std::vector<Agg> agg;
  for (auto& r : g_prof) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) != cudaSuccess) { cudaGetLastError(); ms = 0.0f; }
    size_t i = 0;
    for (; i < agg.size(); ++i)
      if (!strcmp(agg[i].name, r.name)) break;
    if (i == agg.size()) agg.push_back({r.name, 0, 0.0});
    agg[i].n++;
    agg[i].ms += ms;
    g_prof_pool.push_back(r.a);
    g_prof_pool.push_back(r.b);
  }
  g_prof.clear();
  size_t off = 0;
  off += snprintf(json + off, cap - off, "{");
  for (size_t i = 0; i < agg.size() && off + 96 < cap; ++i)
    off += snprintf(json + off, cap - off, "%s\"%s\": {\"launches\": %d, \"ms\": %.6f}", i ? ", " : "", agg[i].name, agg[i].n, agg[i].ms);
  snprintf(json + off, cap - off, "}");
  return IZB_OK;
}

// ---------------------------------------------------------------------------------------------- per-device state
namespace {
struct DevState {
  std::mutex mu;
  uint32_t* err_word = nullptr;
  void* ws[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};  // scratch arenas by user (izb_common.cuh: kWs*)
  size_t ws_bytes[5] = {0, 0, 0, 0, 0};
  void* stage = nullptr;  // staging of the host-buffer call
  size_t stage_bytes = 0;
  cudaStream_t hs[3] = {nullptr, nullptr, nullptr};  // host-buffer call: copy-in, compute, copy-out streams
  cudaEvent_t he[2][3] = {{nullptr, nullptr, nullptr}, {nullptr, nullptr, nullptr}};  // per staging buffer: in, computed, out
  cudaEvent_t hstart = nullptr;
  std::atomic<int> tc_ok{-1};  // -1 unknown, 0 self-check failed, 1 passed
  std::atomic<int> sms{0};
  std::atomic<int> sm_limit{0};  // izb_set_sm_limit: SMs the persistent GEMM may occupy (0 = all)
  uint32_t* noalloc_status = nullptr;  // status word of izb_gemm_noalloc (a device symbol's address), once looked up
};
DevState g_dev[kIzbMaxDev];

int check_device(int device) {
  if (device < 0 || device >= kIzbMaxDev) IZB_FAIL(IZB_ERR_ARG, "device %d out of range", device);
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device >= n) IZB_FAIL(IZB_ERR_CUDA, "no CUDA device %d (this library has no CPU path)", device);
  cudaDeviceProp p;
  IZB_CUDA(cudaGetDeviceProperties(&p, device));
  if (p.major != 10) IZB_FAIL(IZB_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, p.major, p.minor);
  return IZB_OK;
}

// Makes `device` current for the scope and puts the caller's device back: for the calls that name a device explicitly
// (status, reserve) and may come from a thread that drives another GPU.
struct DeviceScope {
  int prev = -1;
  bool switched = false;
  cudaError_t enter(int device) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev != device) {
      e = cudaSetDevice(device);
      switched = e == cudaSuccess;
    }
    return e;
  }
  ~DeviceScope() {
    if (switched) cudaSetDevice(prev);
  }
};
}  // namespace

int izb_require_device(int device, const char* what) {
  if (device < 0 || device >= kIzbMaxDev) IZB_FAIL(IZB_ERR_ARG, "%s: device %d out of range", what, device);
  int cur = -1;
  IZB_CUDA(cudaGetDevice(&cur));
  if (cur != device)
    IZB_FAIL(IZB_ERR_ARG, "%s: the handle lives on device %d but device %d is current in this thread (cudaSetDevice(%d) first)", what,
             device, cur, device);
  return IZB_OK;
}

int izb_sm_count(int device) {
  if (device < 0 || device >= kIzbMaxDev) return 148;
  int n = g_dev[device].sms.load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1) {
    cudaGetLastError();
    return 148;
  }
  g_dev[device].sms.store(n, std::memory_order_relaxed);
  return n;
}

int izb_sm_budget(int device) {
  const int n = izb_sm_count(device);
  const int lim = device >= 0 && device < kIzbMaxDev ? g_dev[device].sm_limit.load(std::memory_order_relaxed) : 0;
  return lim > 0 && lim < n ? lim : n;
}

extern "C" int izb_set_sm_limit(int device, int sms) {
  if (device < 0 || device >= kIzbMaxDev) IZB_FAIL(IZB_ERR_ARG, "set_sm_limit: device %d out of range", device);
  if (sms < 0) IZB_FAIL(IZB_ERR_ARG, "set_sm_limit: %d", sms);
  g_dev[device].sm_limit.store(sms);
  return IZB_OK;
}

// (called with `device` current: every caller has passed izb_require_device or holds a DeviceScope)
uint32_t* izb_device_error_word(int device) {
  DevState& d = g_dev[device];
  std::lock_guard<std::mutex> lk(d.mu);
  if (!d.err_word) {
    if (cudaMalloc(&d.err_word, 256) != cudaSuccess) return nullptr;
    cudaMemset(d.err_word, 0, 256);
  }
  return d.err_word;
}

void izb_note_noalloc_status(int device, uint32_t* status) {
  std::lock_guard<std::mutex> lk(g_dev[device].mu);
  g_dev[device].noalloc_status = status;
}

// An arena never shrinks and is only replaced when a call needs more than it holds.  Replacing waits for the device
// (work in flight may still read the old block) -- izb_reserve moves that wait out of the hot path.
static int grow_arena(DevState& d, int device, int slot, size_t bytes) {
  if (bytes <= d.ws_bytes[slot]) return IZB_OK;
  if (d.ws[slot]) {
    IZB_CUDA(cudaDeviceSynchronize());
    IZB_CUDA(cudaFree(d.ws[slot]));
    d.ws[slot] = nullptr;
    d.ws_bytes[slot] = 0;
  }
  const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  if (cudaMalloc(&d.ws[slot], want) != cudaSuccess) {
    cudaGetLastError();
    IZB_FAIL(IZB_ERR_NOMEM, "workspace of %zu bytes on device %d", want, device);
  }
  d.ws_bytes[slot] = want;
  return IZB_OK;
}

int izb_workspace(int device, int slot, size_t bytes, void** out) {
  DevState& d = g_dev[device];
  std::lock_guard<std::mutex> lk(d.mu);
  if (int rc = grow_arena(d, device, slot, bytes)) return rc;
  *out = d.ws[slot];
  return IZB_OK;
}

size_t izb_gemm_tc_scratch_bytes(int type, int rows, int K);

extern "C" int izb_reserve(int device, int max_rows, int max_K) {
  if (max_rows < 1 || max_K < 256 || max_K % 256) IZB_FAIL(IZB_ERR_SHAPE, "reserve: rows = %d, K = %d (K in whole superblocks)", max_rows, max_K);
  if (int rc = check_device(device)) return rc;
  DeviceScope scope;
  IZB_CUDA(scope.enter(device));
  DevState& d = g_dev[device];
  std::lock_guard<std::mutex> lk(d.mu);
  const size_t gemm = izb_gemm_tc_scratch_bytes(IZB_Q4_K, max_rows, max_K);
  if (int rc = grow_arena(d, device, kWsGemm, gemm)) return rc;
  if (int rc = grow_arena(d, device, kWsMoe, gemm)) return rc;
  if (int rc = grow_arena(d, device, kWsTp, (size_t)(max_K / 32) * max_rows * 4)) return rc;
  if (!d.err_word) {
    if (cudaMalloc(&d.err_word, 256) != cudaSuccess) { cudaGetLastError(); IZB_FAIL(IZB_ERR_NOMEM, "reserve: error word on device %d", device); }
    IZB_CUDA(cudaMemset(d.err_word, 0, 256));
  }
  return IZB_OK;
}

extern "C" int izb_device_status(int device, uint32_t* word) {
  if (!word) IZB_FAIL(IZB_ERR_ARG, "device_status: null pointer");
  if (int rc = check_device(device)) return rc;
  DeviceScope scope;
  IZB_CUDA(scope.enter(device));
  uint32_t* p = izb_device_error_word(device);
  if (!p) IZB_FAIL(IZB_ERR_NOMEM, "device_status: cannot allocate the error word");
  IZB_CUDA(cudaDeviceSynchronize());
  IZB_CUDA(cudaMemcpy(word, p, 4, cudaMemcpyDeviceToHost));
  IZB_CUDA(cudaMemset(p, 0, 4));
  // the word izb_gemm_noalloc uses when its caller passes no status pointer (no allocation: a device symbol's address)
  uint32_t* ns = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_dev[device].mu);
    ns = g_dev[device].noalloc_status;
  }
  if (ns) {
    uint32_t w2 = 0;
    IZB_CUDA(cudaMemcpy(&w2, ns, 4, cudaMemcpyDeviceToHost));
    IZB_CUDA(cudaMemset(ns, 0, 4));
    *word |= w2;
  }
  return *word ? IZB_ERR_TIMEOUT : IZB_OK;
}

// ---------------------------------------------------------------------------------------------- weights
namespace {
// GGUF Q8_0 (34-byte blocks: fp16 d, 32 int8) -> per 256 values: 8 fp16 scales then 8 x 32 int8 (272 bytes, the same
// count).  One thread per (superblock, 16-byte output piece); 17 pieces per superblock.
__global__ void regroup_q8_0_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t n_sb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_sb * 17) return;
  const size_t sb = i / 17;
  const int pc = (int)(i % 17);
  const uint8_t* s = src + sb * 272;
  uint8_t* d = dst + sb * 272 + pc * 16;
  if (pc == 0) {
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      d[2 * b] = s[34 * b];
      d[2 * b + 1] = s[34 * b + 1];
    }
  } else {
    const int b = (pc - 1) >> 1, h = (pc - 1) & 1;
#pragma unroll
    for (int k = 0; k < 16; ++k) d[k] = s[34 * b + 2 + 16 * h + k];
  }
}
}  // namespace

int izb_gguf_sb_bytes(int ggml_type);
void izb_transcode_sb(int ggml_type, const uint8_t* src, size_t n_sb, uint8_t* dst);

extern "C" int izb_weight_create_slice(int type, const void* h_rows, int n_mats, int N, int K, int n0, int n1, int k0, int k1,
                                       int device, izb_weight** out) {
  if (!h_rows || !out) IZB_FAIL(IZB_ERR_ARG, "weight_create: null pointer");
  *out = nullptr;
  const int src_sb = izb_gguf_sb_bytes(type);
  if (!src_sb) IZB_FAIL(IZB_ERR_TYPE, "weight_create: ggml type %d (taken: Q8_0 = 8, Q4_K = 12, Q4_0 = 2, Q5_K = 13, Q6_K = 14, IQ4_XS = 23)", type);
  if (n_mats < 1 || N < 1 || K < 256 || K % 256) IZB_FAIL(IZB_ERR_SHAPE, "weight_create: %d x [%d x %d] (K must be a multiple of 256)", n_mats, N, K);
  if (n0 < 0 || n1 > N || n0 >= n1 || k0 < 0 || k1 > K || k0 >= k1 || k0 % 256 || k1 % 256)
    IZB_FAIL(IZB_ERR_SHAPE, "weight_create: slice rows [%d,%d) cols [%d,%d) of %d x %d (columns in whole superblocks)", n0, n1, k0, k1, N, K);
  if (int rc = check_device(device)) return rc;
  IZB_CUDA(cudaSetDevice(device));
  const bool direct = type == IZB_Q8_0 || type == IZB_Q4_K;  // the file's bytes are what is uploaded
  izb_weight* w = new izb_weight;
  w->ggml_type = type;
  w->type = (type == IZB_Q8_0 || type == IZB_Q4_0) ? IZB_Q8_0 : type == IZB_Q4_K ? IZB_Q4_K : IZB_K16;
  w->has_min = type == IZB_Q5_K;
  w->n_mats = n_mats;
  w->N = n1 - n0;
  w->K = k1 - k0;
  w->device = device;
  w->packed6 = type == IZB_Q6_K;
  w->sb_bytes = w->type == IZB_Q4_K ? 144 : w->type == IZB_Q8_0 ? 272 : w->packed6 ? kQ6pSbBytes : kK16SbBytes;
  w->row_bytes = (size_t)(w->K / 256) * w->sb_bytes;
  w->bytes = (size_t)n_mats * w->N * w->row_bytes;
  const size_t src_row = (size_t)(K / 256) * src_sb;  // (the GGUF bytes of 256 values: 144 / 8*34 = 272 for the two direct types)
  if (cudaMalloc(&w->raw, w->bytes + kRawSlack) != cudaSuccess) {
    cudaGetLastError();
    const size_t want = w->bytes + kRawSlack;
    delete w;
    IZB_FAIL(IZB_ERR_NOMEM, "weight_create: %zu bytes on device %d", want, device);
  }
  cudaError_t e = cudaMemset(w->raw + w->bytes, 0, kRawSlack);
  uint8_t* upload = w->raw;
  uint8_t* tmp = nullptr;
  if (e == cudaSuccess && w->type == IZB_Q8_0) {  // (GGUF block order on the way in, regrouped on the device)
    e = cudaMalloc(&tmp, w->bytes);
    upload = tmp;
  }
  if (e == cudaSuccess && direct) {
    const uint8_t* src = (const uint8_t*)h_rows + (size_t)n0 * src_row + (size_t)(k0 / 256) * src_sb;
    if (n0 == 0 && n1 == N && k0 == 0 && k1 == K) {
      e = cudaMemcpy(upload, src, w->bytes, cudaMemcpyHostToDevice);
    } else {
      for (int m = 0; m < n_mats && e == cudaSuccess; ++m)
        e = cudaMemcpy2D(upload + (size_t)m * w->N * w->row_bytes, w->row_bytes, src + (size_t)m * N * src_row, src_row,
                         w->row_bytes, w->N, cudaMemcpyHostToDevice);
    }
  } else if (e == cudaSuccess) {
    // decode the rows of the slice on the host, a matrix at a time, into the form that is uploaded
    std::vector<uint8_t> stage;
    try {
      stage.resize((size_t)w->N * w->row_bytes);
    } catch (const std::exception&) {
      cudaFree(w->raw);
      if (tmp) cudaFree(tmp);
      delete w;
      IZB_FAIL(IZB_ERR_NOMEM, "weight_create: host staging for the decoded rows");
    }
    const size_t nsb_row = (size_t)w->K / 256;
    for (int m = 0; m < n_mats && e == cudaSuccess; ++m) {
      const uint8_t* src = (const uint8_t*)h_rows + ((size_t)m * N + n0) * src_row + (size_t)(k0 / 256) * src_sb;
#pragma omp parallel for schedule(static)
      for (int n = 0; n < w->N; ++n) izb_transcode_sb(type, src + (size_t)n * src_row, nsb_row, stage.data() + (size_t)n * w->row_bytes);
      e = cudaMemcpy(upload + (size_t)m * w->N * w->row_bytes, stage.data(), stage.size(), cudaMemcpyHostToDevice);
    }
  }
  if (e == cudaSuccess && w->type == IZB_Q8_0) {
    const size_t n_sb = w->bytes / 272, items = n_sb * 17;
    regroup_q8_0_kernel<<<(unsigned)((items + 255) / 256), 256>>>(tmp, w->raw, n_sb);
    g_izb_launches.fetch_add(1);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
  }
  if (tmp) cudaFree(tmp);
  if (e != cudaSuccess) {
    cudaFree(w->raw);
    delete w;
    IZB_FAIL(IZB_ERR_CUDA, "weight_create: upload failed: %s", cudaGetErrorString(e));
  }
  w->has_tmap = w->type != IZB_K16 && izb_make_raw_tensor_map(w) == IZB_OK;
  *out = w;
  return IZB_OK;
}

extern "C" int izb_weight_decode_host(int type, const void* h_src, size_t n_superblocks, void* h_dst, size_t dst_bytes) {
  if (!h_src || !h_dst) IZB_FAIL(IZB_ERR_ARG, "weight_decode_host: null pointer");
  if (type != IZB_Q4_0 && type != IZB_Q5_K && type != IZB_Q6_K && type != IZB_IQ4_XS)
    IZB_FAIL(IZB_ERR_TYPE, "weight_decode_host: ggml type %d is uploaded as it is (or is not taken at all)", type);
  const size_t per = type == IZB_Q4_0 ? 8 * 34 : type == IZB_Q6_K ? kQ6pSbBytes : kK16SbBytes;
  if (dst_bytes < n_superblocks * per) IZB_FAIL(IZB_ERR_SHAPE, "weight_decode_host: %zu bytes for %zu superblocks of %zu", dst_bytes, n_superblocks, per);
  izb_transcode_sb(type, (const uint8_t*)h_src, n_superblocks, (uint8_t*)h_dst);
  return IZB_OK;
}

extern "C" int izb_weight_create(int type, const void* h_rows, int n_mats, int N, int K, int device, izb_weight** out) {
  return izb_weight_create_slice(type, h_rows, n_mats, N, K, 0, N, 0, K, device, out);
}

extern "C" int izb_weight_create_stack(int type, const void* const* h_parts, const int* n_rows, int n_parts, int K, int device,
                                       izb_weight** out) {
  if (!h_parts || !n_rows || !out) IZB_FAIL(IZB_ERR_ARG, "weight_create_stack: null pointer");
  *out = nullptr;
  const int src_sb = izb_gguf_sb_bytes(type);
  if (!src_sb) IZB_FAIL(IZB_ERR_TYPE, "weight_create_stack: ggml type %d", type);
  if (n_parts < 1 || n_parts > 64 || K < 256 || K % 256) IZB_FAIL(IZB_ERR_SHAPE, "weight_create_stack: %d parts, K = %d", n_parts, K);
  const size_t src_row = (size_t)(K / 256) * src_sb;
  long long total = 0;
  for (int i = 0; i < n_parts; ++i) {
    if (!h_parts[i] || n_rows[i] < 1) IZB_FAIL(IZB_ERR_ARG, "weight_create_stack: part %d is empty", i);
    total += n_rows[i];
  }
  if (total > 0x7FFFFFFF) IZB_FAIL(IZB_ERR_SHAPE, "weight_create_stack: %lld rows", total);
  std::vector<uint8_t> rows;
  try {
    rows.resize((size_t)total * src_row);
  } catch (const std::exception&) {
    IZB_FAIL(IZB_ERR_NOMEM, "weight_create_stack: %lld rows of %zu bytes on the host", total, src_row);
  }
  size_t at = 0;
  for (int i = 0; i < n_parts; ++i) {
    memcpy(rows.data() + at, h_parts[i], (size_t)n_rows[i] * src_row);
    at += (size_t)n_rows[i] * src_row;
  }
  return izb_weight_create(type, rows.data(), 1, (int)total, K, device, out);
}

extern "C" int izb_gateup_interleave_host(int type, const void* h_gate, const void* h_up, int n_mats, int F, int K, void* h_dst,
                                         size_t dst_bytes) {
  if (!h_gate || !h_up || !h_dst) IZB_FAIL(IZB_ERR_ARG, "gateup_interleave: null pointer");
  const int src_sb = izb_gguf_sb_bytes(type);
  if (!src_sb) IZB_FAIL(IZB_ERR_TYPE, "gateup_interleave: ggml type %d", type);
  if (n_mats < 1 || F < 64 || F % 64 || K < 256 || K % 256 || (long long)n_mats * 2 * F > 0x7FFFFFFF)
    IZB_FAIL(IZB_ERR_SHAPE, "gateup_interleave: n_mats = %d, F = %d (multiple of 64), K = %d (multiple of 256)", n_mats, F, K);
  const size_t row = (size_t)(K / 256) * src_sb, grp = 32 * row;
  if (dst_bytes < (size_t)n_mats * 2 * F * row) IZB_FAIL(IZB_ERR_SHAPE, "gateup_interleave: %zu bytes for %d x %d rows of %zu", dst_bytes, n_mats, 2 * F, row);
  const uint8_t* g = (const uint8_t*)h_gate;
  const uint8_t* u = (const uint8_t*)h_up;
  uint8_t* dst = (uint8_t*)h_dst;
  const long long n_grp = (long long)n_mats * (F / 32);  // (F % 32 == 0: groups never straddle two matrices)
#pragma omp parallel for schedule(static)
  for (long long j = 0; j < n_grp; ++j) {
    memcpy(dst + (size_t)(2 * j) * grp, g + (size_t)j * grp, grp);
    memcpy(dst + (size_t)(2 * j + 1) * grp, u + (size_t)j * grp, grp);
  }
  return IZB_OK;
}

extern "C" int izb_weight_create_gateup(int type, const void* h_gate, const void* h_up, int n_mats, int F, int K, int device,
                                        izb_weight** out) {
  if (!h_gate || !h_up || !out) IZB_FAIL(IZB_ERR_ARG, "weight_create_gateup: null pointer");
  *out = nullptr;
  if (type != IZB_Q8_0 && type != IZB_Q4_K && type != IZB_Q4_0)
    IZB_FAIL(IZB_ERR_TYPE, "weight_create_gateup: ggml type %d does not run on the tensor-core GEMM (Q8_0, Q4_K, Q4_0 do)", type);
  if (n_mats < 1 || F < 64 || F % 64 || K < 256 || K % 256 || (long long)n_mats * 2 * F > 0x7FFFFFFF)
    IZB_FAIL(IZB_ERR_SHAPE, "weight_create_gateup: n_mats = %d, F = %d (multiple of 64), K = %d (multiple of 256)", n_mats, F, K);
  const size_t row = (size_t)(K / 256) * izb_gguf_sb_bytes(type);
  std::vector<uint8_t> rows;
  try {
    rows.resize((size_t)n_mats * 2 * F * row);
  } catch (const std::exception&) {
    IZB_FAIL(IZB_ERR_NOMEM, "weight_create_gateup: %d x %d rows of %zu bytes on the host", n_mats, 2 * F, row);
  }
  if (int rc = izb_gateup_interleave_host(type, h_gate, h_up, n_mats, F, K, rows.data(), rows.size())) return rc;
  const int rc = izb_weight_create(type, rows.data(), n_mats, 2 * F, K, device, out);
  if (rc == IZB_OK) (*out)->gu32 = true;
  return rc;
}

extern "C" void izb_weight_destroy(izb_weight* w) {
  if (!w) return;
  {
    DeviceScope scope;  // (the caller's current device is put back: a thread may free another GPU's handle)
    scope.enter(w->device);
    cudaFree(w->raw);
  }
  delete w;
}

extern "C" int izb_weight_download(const izb_weight* w, size_t offset, size_t bytes, void* h_out) {
  if (!w || !h_out) IZB_FAIL(IZB_ERR_ARG, "weight_download: null pointer");
  if (offset > w->bytes || bytes > w->bytes - offset) IZB_FAIL(IZB_ERR_SHAPE, "weight_download: [%zu, +%zu) of %zu bytes", offset, bytes, w->bytes);
  DeviceScope scope;
  IZB_CUDA(scope.enter(w->device));
  IZB_CUDA(cudaMemcpy(h_out, w->raw + offset, bytes, cudaMemcpyDeviceToHost));
  return IZB_OK;
}

extern "C" int izb_weight_info(const izb_weight* w, int* type, int* n_mats, int* N, int* K, size_t* bytes) {
  if (!w) IZB_FAIL(IZB_ERR_ARG, "weight_info: null handle");
  if (type) *type = w->ggml_type;
  if (n_mats) *n_mats = w->n_mats;
  if (N) *N = w->N;
  if (K) *K = w->K;
  if (bytes) *bytes = w->bytes + kRawSlack;
  return IZB_OK;
}

// ---------------------------------------------------------------------------------------------- matmul
static int check_gemm_args(const izb_weight* w, int mat, const int8_t* aq, const float* asc, int M, int Mp, const void* C,
                           int ldc, int c_off, int acc) {
  if (!w || !aq || !asc || !C) IZB_FAIL(IZB_ERR_ARG, "gemm: null pointer");
  if (mat < 0 || mat >= w->n_mats) IZB_FAIL(IZB_ERR_ARG, "gemm: matrix %d of %d", mat, w->n_mats);
  if (acc < 0 || acc > 3) IZB_FAIL(IZB_ERR_ARG, "gemm: store mode %d", acc);
  if (acc == 3 && !w->gu32) IZB_FAIL(IZB_ERR_ARG, "gemm: store mode 3 needs a weight made by izb_weight_create_gateup");
  // the reference's shape rule (zero/engine.h:1233): Mp % 16, N % 16, K % 256
  if (Mp % 16 || w->N % 16 || w->K % 256) IZB_FAIL(IZB_ERR_SHAPE, "gemm: bad shape Mp=%d N=%d K=%d (need Mp%%16, N%%16, K%%256)", Mp, w->N, w->K);
  if (M < 1 || M > Mp) IZB_FAIL(IZB_ERR_SHAPE, "gemm: %d rows of Mp = %d", M, Mp);
  const int n_out = acc == 3 ? w->N / 2 : w->N;
  if (c_off < 0 || ldc < c_off + n_out) IZB_FAIL(IZB_ERR_SHAPE, "gemm: ldc = %d < c_off + output columns = %d", ldc, c_off + n_out);
  if (!izb_aligned(aq, 16) || !izb_aligned(asc, 16) || !izb_aligned(C, 16) || ldc % 4 || c_off % 4)
    IZB_FAIL(IZB_ERR_ALIGN, "gemm: aq, asc, C must be 16-byte aligned, ldc and c_off multiples of 4");
  return IZB_OK;
}

extern "C" int izb_gemm(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, int M, int Mp, float* d_C, int ldc,
                        int c_off, int acc, int impl, void* stream) {
  if (int rc = check_gemm_args(w, mat, d_aq, d_asc, M, Mp, d_C, ldc, c_off, acc)) return rc;
  if (int rc = izb_require_device(w->device, "gemm")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (w->type == IZB_K16) {  // Q5_K / Q6_K / IQ4_XS: exact per-16 scales, CUDA cores (the reference requantises these for its GEMM)
    if (impl == IZB_GEMM_TC) IZB_FAIL(IZB_ERR_TYPE, "gemm: the tensor-core kernel does not take ggml type %d", w->ggml_type);
    if (impl != IZB_GEMM_AUTO && impl != IZB_GEMM_CORE) IZB_FAIL(IZB_ERR_ARG, "gemm: impl %d", impl);
    if (acc == 3) IZB_FAIL(IZB_ERR_TYPE, "gemm: store mode 3 is not built for ggml type %d", w->ggml_type);
    return izb_gemm_k16_launch(w, w->raw + (size_t)mat * w->N * w->row_bytes, d_aq, d_asc, M, Mp, d_C, ldc, c_off, acc, nullptr, st);
  }
  if (impl == IZB_GEMM_AUTO || impl == IZB_GEMM_TC) {
    const bool allowed = impl == IZB_GEMM_TC || g_dev[w->device].tc_ok.load() != 0;
    if (allowed) {
      const int rc = izb_gemm_tc_launch(w, mat, d_aq, d_asc, M, Mp, d_C, ldc, c_off, acc, nullptr, st);
      if (rc <= 0) return rc;
    }
    if (impl == IZB_GEMM_TC) IZB_FAIL(IZB_ERR_SHAPE, "gemm: the tensor-core kernel does not take M=%d Mp=%d N=%d K=%d", M, Mp, w->N, w->K);
  } else if (impl != IZB_GEMM_CORE) {
    IZB_FAIL(IZB_ERR_ARG, "gemm: impl %d", impl);
  }
  if (acc == 3) {  // both projections side by side into scratch, then the SwiGLU product of the column groups
    void* ws = nullptr;
    if (int rc = izb_workspace(w->device, kWsGemm, (size_t)Mp * w->N * 4, &ws)) return rc;
    if (int rc = izb_gemm_core_launch(w, w->raw + (size_t)mat * w->N * w->row_bytes, d_aq, d_asc, M, Mp, (float*)ws, w->N, 0, 0, nullptr, st)) return rc;
    return izb_swiglu_pairs_launch((const float*)ws, w->N, M, w->N / 2, d_C, ldc, c_off, st);
  }
  return izb_gemm_core_launch(w, w->raw + (size_t)mat * w->N * w->row_bytes, d_aq, d_asc, M, Mp, d_C, ldc, c_off, acc, nullptr, st);
}

extern "C" int izb_block_dots(const izb_weight* w, int mat, const int8_t* d_aq, int M, int32_t* d_dots, int impl, void* stream) {
  if (!w || !d_aq || !d_dots) IZB_FAIL(IZB_ERR_ARG, "block_dots: null pointer");
  if (mat < 0 || mat >= w->n_mats) IZB_FAIL(IZB_ERR_ARG, "block_dots: matrix %d of %d", mat, w->n_mats);
  if (M < 1) IZB_FAIL(IZB_ERR_SHAPE, "block_dots: M = %d", M);
  if (!izb_aligned(d_aq, 16)) IZB_FAIL(IZB_ERR_ALIGN, "block_dots: aq not 16-byte aligned");
  if (int rc = izb_require_device(w->device, "block_dots")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (w->type == IZB_K16) {
    if (impl != IZB_GEMM_CORE) IZB_FAIL(IZB_ERR_TYPE, "block_dots: the tensor-core kernel does not take ggml type %d", w->ggml_type);
    return izb_gemm_k16_launch(w, w->raw + (size_t)mat * w->N * w->row_bytes, d_aq, nullptr, M, M, nullptr, 0, 0, 0, d_dots, st);
  }
  if (impl == IZB_GEMM_TC) {
    const int rc = izb_gemm_tc_launch(w, mat, d_aq, nullptr, M, M, nullptr, 0, 0, 0, d_dots, st);
    if (rc > 0) IZB_FAIL(IZB_ERR_SHAPE, "block_dots: the tensor-core kernel does not take M=%d N=%d K=%d", M, w->N, w->K);
    return rc;
  }
  if (impl != IZB_GEMM_CORE) IZB_FAIL(IZB_ERR_ARG, "block_dots: impl %d", impl);
  // (dots mode: no scales are read; rows past M are not touched since Mp = M)
  return izb_gemm_core_launch(w, w->raw + (size_t)mat * w->N * w->row_bytes, d_aq, nullptr, M, M, nullptr, 0, 0, 0, d_dots, st);
}

extern "C" int izb_matmul(const izb_weight* w, int mat, const int8_t* d_aq, const float* d_asc, const int16_t* d_absum, int T,
                          int Mp, float* d_C, int ldc, int c_off, int acc, void* stream) {
  (void)d_absum;  // the kernels recompute the block sums they need from aq
  if (!w) IZB_FAIL(IZB_ERR_ARG, "matmul: null weight");
  if (T < 1) IZB_FAIL(IZB_ERR_SHAPE, "matmul: T = %d", T);
  if (T <= 8) {
    if (acc >= 2) IZB_FAIL(IZB_ERR_ARG, "matmul: store modes 2 and 3 (fused SwiGLU) exist for the GEMM only (T > 8)");
    return izb_gemv(w, mat, d_aq, d_asc, T, Mp, d_C, ldc, c_off, acc, stream);
  }
  return izb_gemm(w, mat, d_aq, d_asc, Mp, Mp, d_C, ldc, c_off, acc, IZB_GEMM_AUTO, stream);
}

extern "C" int izb_quant_matmul(const izb_weight* w, int mat, const float* d_x, int ldx, int T, int Mp, int8_t* d_aq, float* d_asc,
                                float* d_C, int ldc, int c_off, int acc, void* stream) {
  if (!w || !d_x || !d_aq || !d_asc || !d_C) IZB_FAIL(IZB_ERR_ARG, "quant_matmul: null pointer");
  if (T < 1 || T > Mp) IZB_FAIL(IZB_ERR_SHAPE, "quant_matmul: %d rows of Mp = %d", T, Mp);
  // the GEMM with the fused pre-pass: same checks as izb_gemm, then one launch writes aq / asc and the operand images
  if (T > 8 && (w->type == IZB_Q8_0 || w->type == IZB_Q4_K) && g_dev[w->device < 0 || w->device >= kIzbMaxDev ? 0 : w->device].tc_ok.load() != 0) {
    if (int rc = check_gemm_args(w, mat, d_aq, d_asc, Mp, Mp, d_C, ldc, c_off, acc)) return rc;
    if (ldx < w->K || ldx % 4 || !izb_aligned(d_x, 16)) IZB_FAIL(IZB_ERR_ALIGN, "quant_matmul: x must be 16-byte aligned with ldx >= K a multiple of 4");
    if (int rc = izb_require_device(w->device, "quant_matmul")) return rc;
    const int rc = izb_gemm_tc_quant_launch(w, mat, d_x, ldx, T, Mp, d_aq, d_asc, d_C, ldc, c_off, acc, (cudaStream_t)stream);
    if (rc <= 0) return rc;
  }
  if (int rc = izb_quantize_act(d_x, ldx, T, Mp, w->K, d_aq, d_asc, nullptr, stream)) return rc;
  return izb_matmul(w, mat, d_aq, d_asc, nullptr, T, Mp, d_C, ldc, c_off, acc, stream);
}

// records the verdict of the start-up check (izb_selfcheck lives with the tensor-core kernel)
void izb_set_tc_ok(int device, int ok) { g_dev[device].tc_ok.store(ok); }
int izb_get_tc_ok(int device) { return g_dev[device].tc_ok.load(); }

// ---------------------------------------------------------------------------------------------- host-buffer call
extern "C" int izb_matmul_host(const izb_weight* w, int mat, const float* h_x, int M, float* h_C, void* stream) {
  if (!w || !h_x || !h_C) IZB_FAIL(IZB_ERR_ARG, "matmul_host: null pointer");
  if (M < 1) IZB_FAIL(IZB_ERR_SHAPE, "matmul_host: M = %d", M);
  IZB_CUDA(cudaSetDevice(w->device));
  cudaStream_t st = (cudaStream_t)stream;
  const int K = w->K, N = w->N;
  // Rows travel in chunks through two staging buffers and three streams (copy in, quantise + multiply, copy out), so
  // that both directions of the host link and the GPU work at the same time; a call of up to kChunk rows is one chunk.
  constexpr int kChunk = 1024;
  const int rows_max = M < kChunk ? M : kChunk;
  auto pad = [](int m) { return m <= 8 ? 16 : (m >= 128 ? (m + 127) / 128 * 128 : (m + 15) / 16 * 16); };  // zero/engine.h:521-522
  const int Mp_max = pad(rows_max);
  const size_t bx = (size_t)rows_max * K * 4, baq = (size_t)Mp_max * K, basc = (size_t)(K / 32) * Mp_max * 4, bc = (size_t)Mp_max * N * 4;
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t per_buf = up(bx) + up(baq) + up(basc) + up(bc);
  const int nchunks = (M + kChunk - 1) / kChunk, nbuf = nchunks > 1 ? 2 : 1;
  const size_t total = per_buf * nbuf;
  DevState& d = g_dev[w->device];
  {
    std::lock_guard<std::mutex> lk(d.mu);
    if (total > d.stage_bytes) {
      if (d.stage) {
        IZB_CUDA(cudaDeviceSynchronize());
        IZB_CUDA(cudaFree(d.stage));
        d.stage = nullptr;
        d.stage_bytes = 0;
      }
      if (cudaMalloc(&d.stage, total) != cudaSuccess) {
        cudaGetLastError();
        IZB_FAIL(IZB_ERR_NOMEM, "matmul_host: %zu staging bytes", total);
      }
      d.stage_bytes = total;
    }
    if (!d.hstart) {
      for (int i = 0; i < 3; ++i) IZB_CUDA(cudaStreamCreateWithFlags(&d.hs[i], cudaStreamNonBlocking));
      for (int b = 0; b < 2; ++b)
        for (int i = 0; i < 3; ++i) IZB_CUDA(cudaEventCreateWithFlags(&d.he[b][i], cudaEventDisableTiming));
      IZB_CUDA(cudaEventCreateWithFlags(&d.hstart, cudaEventDisableTiming));
    }
  }
  // everything below is ordered after what the caller's stream holds
  IZB_CUDA(cudaEventRecord(d.hstart, st));
  for (int i = 0; i < 3; ++i) IZB_CUDA(cudaStreamWaitEvent(d.hs[i], d.hstart, 0));
  for (int c = 0; c < nchunks; ++c) {
    const int b = c & 1, m0 = c * kChunk, m = (M - m0) < kChunk ? (M - m0) : kChunk, Mp = pad(m);
    uint8_t* p = (uint8_t*)d.stage + (size_t)b * per_buf;
    float* dx = (float*)p;
    int8_t* daq = (int8_t*)(p + up(bx));
    float* dasc = (float*)(p + up(bx) + up(baq));
    float* dC = (float*)(p + up(bx) + up(baq) + up(basc));
    // copy in: the buffer's previous chunk must have been quantised
    if (c >= 2) IZB_CUDA(cudaStreamWaitEvent(d.hs[0], d.he[b][1], 0));
    IZB_CUDA(cudaMemcpyAsync(dx, h_x + (size_t)m0 * K, (size_t)m * K * 4, cudaMemcpyHostToDevice, d.hs[0]));
    IZB_CUDA(cudaEventRecord(d.he[b][0], d.hs[0]));
    // compute: after the copy in, and after the buffer's previous result has left
    IZB_CUDA(cudaStreamWaitEvent(d.hs[1], d.he[b][0], 0));
    if (c >= 2) IZB_CUDA(cudaStreamWaitEvent(d.hs[1], d.he[b][2], 0));
    if (int rc = izb_quant_matmul(w, mat, dx, K, m, Mp, daq, dasc, dC, N, 0, 0, d.hs[1])) return rc;
    IZB_CUDA(cudaEventRecord(d.he[b][1], d.hs[1]));
    // copy out
    IZB_CUDA(cudaStreamWaitEvent(d.hs[2], d.he[b][1], 0));
    IZB_CUDA(cudaMemcpyAsync(h_C + (size_t)m0 * N, dC, (size_t)m * N * 4, cudaMemcpyDeviceToHost, d.hs[2]));
    IZB_CUDA(cudaEventRecord(d.he[b][2], d.hs[2]));
  }
  // the caller's stream continues after the last copy out; the call itself returns when the result is in h_C
  IZB_CUDA(cudaStreamWaitEvent(st, d.he[(nchunks - 1) & 1][2], 0));
  IZB_CUDA(cudaStreamSynchronize(d.hs[2]));
  IZB_CUDA(cudaStreamSynchronize(st));
  return IZB_OK;
}

// ---------------------------------------------------------------------------------------------- tensor-parallel helpers
extern "C" int izb_tp_range(int64_t total, int64_t unit, int nranks, int rank, int64_t* begin, int64_t* end) {
  if (!begin || !end) IZB_FAIL(IZB_ERR_ARG, "tp_range: null pointer");
  if (unit < 1 || nranks < 1 || rank < 0 || rank >= nranks || total < 0) IZB_FAIL(IZB_ERR_ARG, "tp_range: total %lld unit %lld rank %d of %d", (long long)total, (long long)unit, rank, nranks);
  // zero/mgpu/engine_tp_shard.h:68-72: the first units % nranks ranks hold one unit more
  const int64_t units = total / unit, base = units / nranks, extra = units % nranks;
  const int64_t b = rank * base + (rank < extra ? rank : extra), e = b + base + (rank < extra ? 1 : 0);
  *begin = b * unit;
  *end = e * unit;
  return IZB_OK;
}
