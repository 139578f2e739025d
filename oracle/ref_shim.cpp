// Builds the reference's own CPU code for the path into oracle/_ref/libizb_ref.so, from the sources where they lie
// (the REF_ROOT of oracle/Makefile): nothing of the reference is copied.  TEST INFRASTRUCTURE ONLY: used to pin the
// C restatement in izb_oracle.c, to generate tests/golden/, and as the "reference" CPU baseline of the benchmark.
//
// The translation unit includes tools/ref_forward.cpp whole (its main renamed), so its static matmul() -- dequant_row
// weights, activations fake-quantised per 32 (REF_Q=all REF_QB=32), double accumulation, OpenMP over weight rows --
// is the reference's code, not a restatement.  It reads its tensors from a GGUF file: the tests write a synthetic one.
#include <omp.h>
#include "src/log.h"
#define main izb_ref_forward_main
#include "tools/ref_forward.cpp"
#undef main

// the GGUF file the reference's global handle F is open on
static std::string g_open_path;
static void open_gguf(const char* path) {
  if (!F || g_open_path != path) {
    delete F;
    F = new GgufFile(path);
    g_open_path = path;
  }
}

extern "C" {

float ref_fp16_to_f32(uint16_t h) { return fp16_to_f32(h); }
uint16_t ref_f32_to_fp16(float x) { return f32_to_fp16(x); }

// src/quants.h:626 with act32 = true: asc [K/32][M], absum [K/16][M]
void ref_quantize_act(const float* x, int M, int K, int8_t* aq, float* asc, uint16_t* absum) {
  quantize_act_cpu(x, M, K, aq, asc, absum, true);
}

// tools/ref_forward.cpp:314: in-place y = x * r * w, r from a double-precision sum of squares
void ref_rmsnorm(float* x, int n, const float* w, float eps) { rmsnorm(x, n, w, eps); }

// src/quants.h:89: one 256-element superblock (type 12: 144 B; type 8: eight 34-byte blocks)
void ref_decode_sb(uint32_t type, const uint8_t* p, float* d, float* dmin, uint8_t* sc, uint8_t* mn, int16_t* q, float* d8) {
  DecodedSB o;
  decode_sb(type, p, o);
  *d = o.d;
  *dmin = o.dmin;
  for (int i = 0; i < 8; ++i) { sc[i] = o.sc[i]; mn[i] = o.mn[i]; d8[i] = o.d8[i]; }
  for (int i = 0; i < 256; ++i) q[i] = o.q[i];
}

// the generic view of the same decode (DecodedSB::wd .. has_min, src/quants.h:80-86), qoff subtracted from q
void ref_decode_generic_sb(uint32_t type, const uint8_t* p, float* wd, float* wdmin, int8_t* wsc, uint8_t* wmn, int* has_min, int16_t* q) {
  DecodedSB o;
  decode_sb(type, p, o);
  *wd = o.wd;
  *wdmin = o.wdmin;
  *has_min = o.has_min ? 1 : 0;
  for (int i = 0; i < 16; ++i) { wsc[i] = o.wsc[i]; wmn[i] = o.has_min ? o.wmn[i] : 0; }
  for (int i = 0; i < 256; ++i) q[i] = (int16_t)(o.q[i] - o.qoff);
}

void ref_dequant_row(uint32_t type, const uint8_t* row, int K, float* out) { dequant_row(type, row, K, out); }

// src/quants.h:728: the reference's GPU raw form of one superblock (Q8_0: scales first)
int ref_raw_padded_sb_bytes(uint32_t type) { return raw_padded_sb_bytes(type); }
void ref_gpu_raw_sb(uint32_t type, const uint8_t* src, uint8_t* dst) { gpu_raw_sb(type, src, dst); }

// tools/ref_forward.cpp:251 matmul() on tensor `name` of the GGUF file at `path`; X: [T][K] f32 (not yet rounded),
// Y: [T][N].  quant32 != 0 sets REF_Q=all REF_QB=32 (activations rounded to int8 per 32, tools/ref_forward.cpp:145).
int ref_forward_matmul(const char* path, const char* name, const float* X, int T, int quant32, float* Y, int threads) {
  try {
    if (quant32) { setenv("REF_Q", "all", 1); setenv("REF_QB", "32", 1); }
    else unsetenv("REF_Q");
    if (threads > 0) omp_set_num_threads(threads);
    open_gguf(path);
    const GgufTensor& t = F->get(name);
    const int K = (int)t.dims[0];
    std::vector<float> x(X, X + (size_t)T * K), y;
    matmul(name, x, T, y);
    memcpy(Y, y.data(), y.size() * sizeof(float));
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_forward_matmul: %s\n", e.what());
    return -1;
  }
}

// tools/ref_forward.cpp:333 expert_mv(): y[N] = W_e x for routed expert e of the stacked tensor `name`.weight
// ([n_expert][N][K], dequantised row by row, double accumulation); with quant32 the input is rounded to int8 per 32 first
// (REF_Q=all REF_QB=32), as the engine's moe_quant / quant_rows round it.
int ref_expert_mv(const char* path, const char* name, int e, int N, int K, const float* x, float* y, int quant32) {
  try {
    if (quant32) { setenv("REF_Q", "all", 1); setenv("REF_QB", "32", 1); }
    else unsetenv("REF_Q");
    open_gguf(path);
    expert_mv(name, e, N, K, x, y);
    return 0;
  } catch (const std::exception& ex) {
    fprintf(stderr, "ref_expert_mv: %s\n", ex.what());
    return -1;
  }
}

// tools/ref_forward.cpp:321
float ref_silu(float x) { return silu(x); }

int ref_max_threads() { return omp_get_max_threads(); }
}
