// Host-side declarations shared by the translation units of libxfold_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "../../include/xfold_b200.h"

namespace xf {

typedef __nv_bfloat16 bf16;

struct ProfRec {
  cudaEvent_t a, b;
  int tag;
};

struct Ctx {
  int device = 0;
  int sm_count = 148;
  int* d_status = nullptr;  // one word: first in-kernel error code (0 = ok)
  char last_error[256] = {0};
  long long launch_count = 0;  // kernels launched through this context
  int prof_on = 0;             // when set, every launch is bracketed by a pair of CUDA events
  int attn_tag = XFOLD_K_ATTENTION;  // kernel class the attention launchers account their launch to
  // While a stage's exchange kernels are meant to run beside its GEMMs (second stream), the persistent GEMMs leave some
  // SMs free and the exchange kernels are sized for them: a GEMM CTA fills its SM, so without free SMs the two serialise.
  int gemm_sms = 0;      // SMs a GEMM launch may take (0: all)
  int peer_cta_cap = 0;  // CTAs of a peer exchange kernel (0: its own default)
  std::vector<ProfRec> prof_recs, prof_pool;
};

// Brackets one kernel launch with events on its stream while profiling is enabled, and counts it.
struct ProfScope {
  Ctx* c;
  cudaStream_t st;
  ProfRec r;
  bool on;
  ProfScope(Ctx* c_, int tag, cudaStream_t st_) : c(c_), st(st_), on(c_->prof_on != 0) {
    c->launch_count++;
    if (!on) return;
    if (!c->prof_pool.empty()) {
      r = c->prof_pool.back();
      c->prof_pool.pop_back();
    } else {
      cudaEventCreate(&r.a);
      cudaEventCreate(&r.b);
    }
    r.tag = tag;
    cudaEventRecord(r.a, st);
  }
  ~ProfScope() {
    if (!on) return;
    cudaEventRecord(r.b, st);
    c->prof_recs.push_back(r);
  }
};

// returns XFOLD_OK or sets ctx->last_error and returns a status code
int fail(Ctx* c, int code, const char* fmt, ...);
int check_launch(Ctx* c, const char* what);

// ---- tensor maps --------------------------------------------------------------------------
// bf16 tensor of rank 3, innermost stride 1; s1/s2 are strides of dims 1/2 in ELEMENTS.
// 128-byte swizzle (or 64-byte, for boxes whose rows are 64 bytes), zero fill outside the extents.
bool make_tmap_bf16_3d(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                       uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, int swizzle_bytes = 128);

// ---- GEMM ---------------------------------------------------------------------------------
enum GemmEpi : int { EPI_PLAIN = 0, EPI_GATE_RESID = 1, EPI_SWIGLU = 2, EPI_TRIMUL_AB = 3 };

struct GemmArgs {
  int M = 0, N = 0, K = 0, batches = 1;
  int tiles_m = 0, tiles_n = 0;
  int a_row_mode = 0;  // 0: tile rows are consecutive rows of A; 1: tile rows step along dim 2, dim 1 fixed
  int a_dim1 = 1;      // row mode 1: extent of dim 1
  int b_batched = 0;
  int mn_major = 0;    // operands are stored [k][m] and [k][n] (tensor maps: inner dim = m / n, boxes of 64 x 64)
  // PLAIN / SWIGLU / GATE_RESID output
  bf16* out = nullptr;
  long long ldo = 0, out_batch_stride = 0;
  const float* col_bias = nullptr;
  const float* col_scale = nullptr;
  int f16_col0 = 0, f16_col1 = 0;  // PLAIN: output columns [f16_col0, f16_col1) are stored as fp16 (multiples of 32)
  const bf16* resid = nullptr;
  long long ldr = 0;
  const bf16* gate = nullptr;
  long long ldg = 0;
  const bf16* row_gate = nullptr;  // GATE_RESID: gate indexed by (m % row_gate_mod), for conditioning shared by samples
  int row_gate_mod = 0;
  // TRIMUL_AB
  bf16* out_a = nullptr;
  bf16* out_b = nullptr;
  bf16* out_g = nullptr;
  long long cm_chan_stride = 0;
  int cm_ld = 0;
  int ntok = 0;
  const float* mask = nullptr;
  int* status = nullptr;
};

// A is described by tmA (box 64 x 128 rows), B by tmB (box 64 x BN rows); BN is 128 or 256.
int launch_gemm(Ctx* c, int epi, int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a,
                cudaStream_t st);

}  // namespace xf
