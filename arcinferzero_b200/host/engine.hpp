// Host-side mirror of the reference engine's matmul interface over the izb200 C ABI.
//
// The reference's layer code (zero/engine_qwen.h, zero/engine_moe.h) talks to its GEMM back end through a handful of
// Engine members: quant_rows / rmsnorm_quant fill the engine-wide activation buffers aq_ / asc_ / absum_
// (zero/engine_alloc.h:10,39,41), matmul(name, w, Mp, C, ldc, c_off, acc, act32) multiplies them with a GpuWeight
// (zero/engine.h:1080), tp_out(name, w, Mp, act32) does the same for a row-parallel projection and sums the partial
// outputs over the GPUs (zero/mgpu/engine_tp_shard.h:318).  This header keeps those names, argument meanings and error
// behaviour (std::runtime_error before any launch on a bad shape, zero/engine.h:1233-1235), so the call sites of the
// reference read the same; underneath, every call is one C-ABI call of include/izb200.h.  There is no CPU fallback.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/izb200.h"

namespace izb {

inline void check(int rc, const char* what) {
  if (rc != IZB_OK) throw std::runtime_error(std::string(what) + ": " + izb_status_string(rc) + ": " + izb_last_error());
}

// GpuWeight of the reference (zero/engine.h:27-34): type, N, K and the device copy, owned here.
struct GpuWeight {
  int type = 0, N = 0, K = 0, n_mats = 1;
  izb_weight* h = nullptr;
  GpuWeight() = default;
  GpuWeight(const GpuWeight&) = delete;
  GpuWeight& operator=(const GpuWeight&) = delete;
  GpuWeight(GpuWeight&& o) noexcept { *this = std::move(o); }
  GpuWeight& operator=(GpuWeight&& o) noexcept {
    std::swap(type, o.type); std::swap(N, o.N); std::swap(K, o.K); std::swap(n_mats, o.n_mats); std::swap(h, o.h);
    return *this;
  }
  ~GpuWeight() { izb_weight_destroy(h); }
};

class Engine {
 public:
  explicit Engine(int device = 0, cudaStream_t stream = nullptr) : device_(device), stream_(stream) {}
  ~Engine() { release(); }
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  // make_weight (zero/engine_load.h:157): GGUF rows of one tensor -> device weight
  GpuWeight make_weight(int ggml_type, const void* gguf_rows, int N, int K, int n_mats = 1) const {
    GpuWeight w;
    check(izb_weight_create(ggml_type, gguf_rows, n_mats, N, K, device_, &w.h), "make_weight");
    w.type = ggml_type; w.N = N; w.K = K; w.n_mats = n_mats;
    return w;
  }
  // T(): this rank's slice of a tensor (zero/mgpu/engine_tp_shard.h:243-279): rows [n0, n1), input columns [k0, k1)
  GpuWeight make_weight_slice(int ggml_type, const void* gguf_rows, int N, int K, int n0, int n1, int k0, int k1) const {
    GpuWeight w;
    check(izb_weight_create_slice(ggml_type, gguf_rows, 1, N, K, n0, n1, k0, k1, device_, &w.h), "make_weight_slice");
    w.type = ggml_type; w.N = n1 - n0; w.K = k1 - k0;
    return w;
  }

  // load_w_stack (zero/engine_load.h:315-339): several tensors of one type and K as one weight (Q | K | V, gate | up), so
  // that one matmul writes their outputs side by side (gemv_gu, zero/engine.h:1128-1146)
  GpuWeight load_w_stack(int ggml_type, const void* const* parts, const int* n_rows, int n_parts, int K) const {
    GpuWeight w;
    check(izb_weight_create_stack(ggml_type, parts, n_rows, n_parts, K, device_, &w.h), "load_w_stack");
    w.type = ggml_type; w.K = K; w.N = 0;
    for (int i = 0; i < n_parts; ++i) w.N += n_rows[i];
    return w;
  }

  // gate and up of an FFN (or of every expert of a stack) as one weight with the rows interleaved in groups of 32: matmul
  // with store mode 3 then writes up * silu(gate) from ONE GEMM (the reference fuses the product into its up GEMM, store
  // mode 2, zero/kernels/gemm.cl:562-565, which reads the gate GEMM's output back)
  GpuWeight make_weight_gateup(int ggml_type, const void* gate_rows, const void* up_rows, int F, int K, int n_mats = 1) const {
    GpuWeight w;
    check(izb_weight_create_gateup(ggml_type, gate_rows, up_rows, n_mats, F, K, device_, &w.h), "make_weight_gateup");
    w.type = ggml_type; w.N = 2 * F; w.K = K; w.n_mats = n_mats;
    return w;
  }

  // alloc_buffers (zero/engine_alloc.h:4): activation buffers for up to max_rows rows of up to max_k values
  void alloc_buffers(int max_rows, int max_k) {
    release_buffers();
    max_rows_ = pad_rows(max_rows);
    max_k_ = max_k;
    if (cudaSetDevice(device_) != cudaSuccess || cudaMalloc(&aq_, (size_t)max_rows_ * max_k) != cudaSuccess ||
        cudaMalloc(&asc_, (size_t)max_rows_ * (max_k / 32) * sizeof(float)) != cudaSuccess)
      throw std::runtime_error("alloc_buffers: out of device memory");
    // the library's own scratch at its final size too: no call of up to max_rows x max_k allocates after this
    check(izb_reserve(device_, max_rows_, max_k), "alloc_buffers");
  }
  // row padding of a chunk (zero/engine.h:521-522)
  static int pad_rows(int T) { return T >= 128 ? (T + 127) / 128 * 128 : (T + 15) / 16 * 16; }
  void set_rows(int T) { cur_T_ = T; }
  int cur_T() const { return cur_T_; }

  // quant_rows (zero/engine.h:1445): f32 rows -> aq_ / asc_ (rows cur_T_..Mp-1 become zeros with scale 0)
  void quant_rows(const float* x, int ldx, int K, int Mp) {
    if (Mp > max_rows_ || K > max_k_) throw std::runtime_error("quant_rows: activation buffers too small");
    check(izb_quantize_act(x, ldx, cur_T_, Mp, K, aq_, asc_, nullptr, stream_), "quant_rows");
    cur_K_ = K; cur_Mp_ = Mp;
  }
  // swiglu_quant (zero/kernels/ops.cl:272): gu = [gate | up] rows of 2F -> quantised silu(gate) * up
  void swiglu_quant(const float* gu, int ldgu, int F, int Mp) {
    if (Mp > max_rows_ || F > max_k_) throw std::runtime_error("swiglu_quant: activation buffers too small");
    check(izb_swiglu_quant(gu, ldgu, 1, cur_T_, Mp, F, nullptr, aq_, asc_, nullptr, stream_), "swiglu_quant");
    cur_K_ = F; cur_Mp_ = Mp;
  }
  // rmsnorm_quant (zero/kernels/ops.cl:104): rows x -> quantised (x * r) * w, r = 1/sqrt(mean(x^2) + eps); hout (may be
  // null) receives the normalised rows as f32
  void rmsnorm_quant(const float* x, int ldx, const float* w, float eps, int K, int Mp, float* hout = nullptr) {
    if (Mp > max_rows_ || K > max_k_) throw std::runtime_error("rmsnorm_quant: activation buffers too small");
    check(izb_rmsnorm_quant(x, ldx, w, eps, cur_T_, Mp, K, hout, aq_, asc_, nullptr, stream_), "rmsnorm_quant");
    cur_K_ = K; cur_Mp_ = Mp;
  }
  // add_norm_quant (zero/kernels/ops_attn_g.cl:617): x = (x + rmsnorm(t) * w) * s in place, then the quantised
  // rmsnorm(x) * w2 (w2 null: x itself) for the next GEMV
  void add_norm_quant(float* x, const float* t, const float* w, float eps, float s, const float* w2, int K, int Mp) {
    if (Mp > max_rows_ || K > max_k_) throw std::runtime_error("add_norm_quant: activation buffers too small");
    check(izb_add_norm_quant(x, t, w, eps, s, w2, cur_T_, Mp, K, aq_, asc_, nullptr, stream_), "add_norm_quant");
    cur_K_ = K; cur_Mp_ = Mp;
  }
  // softcap_rows (zero/engine.h:1102-1111, zero/kernels/ops_attn_g.cl:724): the output head's logit soft-cap on the
  // current rows of C, columns c_off .. c_off + N - 1
  void softcap_rows(float* C, int ldc, int c_off, int N, float cap) {
    check(izb_softcap_rows(C, cur_T_, ldc, c_off, N, cap, stream_), "softcap_rows");
  }
  // matmul (zero/engine.h:1080): C[.][c_off + n] (op)= quantised rows x w; acc 0 store, 1 add, 2 fused SwiGLU.
  // `name` is the reference's profiling label; act32 is always on (per-32 scales, the reference's default).
  void matmul(const char* name, const GpuWeight& w, int Mp, float* C, int ldc, int c_off, int acc, bool act32 = true) {
    (void)name;
    if (!act32) throw std::runtime_error("matmul: only per-32 activation scales (act32) are implemented");
    if (w.K != cur_K_ || Mp != cur_Mp_) throw std::runtime_error("matmul: the quantised activations do not match this weight");
    check(izb_matmul(w.h, 0, aq_, asc_, nullptr, cur_T_, Mp, C, ldc, c_off, acc, stream_), "matmul");
  }

  // quant_rows + matmul in one call (zero/engine.h:1445 followed by :1080): for more than 8 rows the quantiser also writes
  // the tensor-core GEMM's operand images; aq_ / asc_ are left as quant_rows leaves them
  void quant_matmul(const char* name, const GpuWeight& w, const float* x, int ldx, int Mp, float* C, int ldc, int c_off, int acc) {
    (void)name;
    if (Mp > max_rows_ || w.K > max_k_) throw std::runtime_error("quant_matmul: more rows or columns than alloc_buffers reserved");
    check(izb_quant_matmul(w.h, 0, x, ldx, cur_T_, Mp, aq_, asc_, C, ldc, c_off, acc, stream_), "quant_matmul");
    cur_K_ = w.K; cur_Mp_ = Mp;
  }

  // tp_setup (zero/mgpu/engine_tp_shard.h:88): join the communicator; id128 from izb_tp_unique_id on rank 0
  void tp_setup(int nranks, int rank, const void* id128) {
    nranks_ = nranks; rank_ = rank;
    check(izb_tp_create(nranks, rank, id128, device_, &tp_), "tp_setup");
  }
  // the same with the reference's bounded barriers (zero/mgpu/engine_tp.h:93-123): collectives never block the host, and
  // tp_wait gives up after timeout_ms with the communicator aborted and the context usable
  void tp_setup(int nranks, int rank, const void* id128, int timeout_ms, int max_ctas = 0) {
    nranks_ = nranks; rank_ = rank;
    check(izb_tp_create_ex(nranks, rank, id128, device_, timeout_ms, max_ctas, &tp_), "tp_setup");
  }
  // wait_done (zero/mgpu/engine_tp.h:1313-1372): everything queued on the stream has finished, or a std::runtime_error
  void tp_wait(int timeout_ms) { check(izb_tp_wait(tp_, stream_, timeout_ms), "tp_wait"); }
  // tp_range (zero/mgpu/engine_tp_shard.h:68-72)
  void tp_range(int64_t total, int64_t unit, int64_t* b, int64_t* e) const { check(izb_tp_range(total, unit, nranks_, rank_, b, e), "tp_range"); }
  // tp_out (zero/mgpu/engine_tp_shard.h:318-325): row-parallel projection into `part`, summed over the ranks into x
  void tp_out(const char* name, const GpuWeight& w, int Mp, float* x, float* part, int E) {
    matmul(name, w, Mp, part, E, 0, 0);
    check(izb_tp_allreduce_rows(tp_, x, part, Mp, E, stream_), "tp_out");
  }

 private:
  void release_buffers() {
    if (aq_) cudaFree(aq_);
    if (asc_) cudaFree(asc_);
    aq_ = nullptr; asc_ = nullptr;
  }
  void release() {
    release_buffers();
    if (tp_) izb_tp_destroy(tp_);
    tp_ = nullptr;
  }
  int device_ = 0;
  cudaStream_t stream_ = nullptr;
  int8_t* aq_ = nullptr;
  float* asc_ = nullptr;
  int max_rows_ = 0, max_k_ = 0, cur_T_ = 0, cur_K_ = 0, cur_Mp_ = 0;
  int nranks_ = 1, rank_ = 0;
  izb_tp* tp_ = nullptr;
};

}  // namespace izb
