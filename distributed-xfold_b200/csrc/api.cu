// extern "C" entry points of libxfold_b200.so: argument checking, tensor-map construction,
// workspace carving and the launch sequences of the module-level operators.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "internal.h"
#include "stages.h"

namespace xf {

int fail(Ctx* c, int code, const char* fmt, ...) {
  if (c) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->last_error, sizeof(c->last_error), fmt, ap);
    va_end(ap);
  }
  return code;
}

int check_launch(Ctx* c, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return XFOLD_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static bool load_encode() {
  if (g_encode) return true;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return false;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return true;
}

bool make_tmap_bf16_3d(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                       uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, int swizzle_bytes) {
  if (!g_encode) return false;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * 2, s2 * 2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t es[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (strides[0] & 15) || (strides[1] & 15)) return false;
  if ((swizzle_bytes != 64 && swizzle_bytes != 128) || b0 * 2 > (uint32_t)swizzle_bytes) return false;
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}


// ---------------------------------------------------------------------------------------------
// generic linear layers on top of the GEMM kernel
// ---------------------------------------------------------------------------------------------
static int gemm_rows(Ctx* c, int epi, const bf16* x, long long ldx, long long M, int K, const bf16* w, int wrows, int ldw,
                     GemmArgs a, int bn, cudaStream_t st) {
  if (M <= 0) return XFOLD_OK;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return fail(c, XFOLD_ERR_ARG, "linear: K and leading dimensions must be multiples of 8");
  CUtensorMap tA, tB;
  if (!make_tmap_bf16_3d(&tA, x, K, M, 1, ldx, (uint64_t)ldx * M, 64, 128, 1))
    return fail(c, XFOLD_ERR_ARG, "linear: cannot encode the activation tensor map (base 16 B aligned?)");
  if (!make_tmap_bf16_3d(&tB, w, K, wrows, 1, ldw, (uint64_t)ldw * wrows, 64, bn, 1))
    return fail(c, XFOLD_ERR_ARG, "linear: cannot encode the weight tensor map");
  a.M = (int)M;
  a.K = K;
  a.batches = 1;
  a.tiles_m = (int)((M + 127) / 128);
  a.status = c->d_status;
  return launch_gemm(c, epi, bn, tA, tB, a, st);
}

static int linear_plain(Ctx* c, const bf16* x, long long ldx, long long M, int K, const bf16* w, int N, const float* bias,
                        const float* scale, bf16* out, long long ldo, cudaStream_t st, int f16_col0 = 0, int f16_col1 = 0) {
  if (M >= (1ll << 31)) return fail(c, XFOLD_ERR_ARG, "linear: too many rows");
  GemmArgs a;
  const int bn = (N > 128) ? 256 : 128;
  a.N = N;
  a.tiles_n = (N + bn - 1) / bn;
  a.out = out;
  a.ldo = ldo;
  a.col_bias = bias;
  a.col_scale = scale;
  a.f16_col0 = f16_col0;
  a.f16_col1 = f16_col1;
  return gemm_rows(c, EPI_PLAIN, x, ldx, M, K, w, N, K, a, bn, st);
}

// for the translation units that compose operators out of plain projections
int linear_plain_fwd(Ctx* c, const bf16* x, long long ldx, long long M, int K, const bf16* w, int N, const float* bias,
                     const float* scale, bf16* out, long long ldo, cudaStream_t st) {
  return linear_plain(c, x, ldx, M, K, w, N, bias, scale, out, ldo, st);
}

static int linear_gate_resid(Ctx* c, const bf16* x, long long ldx, long long M, int K, const bf16* w, int N,
                             const bf16* gate, long long ldg, int row_gate_mod, const bf16* resid, long long ldr,
                             bf16* out, long long ldo, cudaStream_t st) {
  if (M >= (1ll << 31)) return fail(c, XFOLD_ERR_ARG, "linear: too many rows");
  GemmArgs a;
  const int bn = 128;
  a.N = N;
  a.tiles_n = (N + bn - 1) / bn;
  a.out = out;
  a.ldo = ldo;
  if (row_gate_mod > 0) { a.row_gate = gate; a.row_gate_mod = row_gate_mod; }
  else a.gate = gate;
  a.ldg = ldg;
  a.resid = resid;
  a.ldr = ldr;
  return gemm_rows(c, EPI_GATE_RESID, x, ldx, M, K, w, N, K, a, bn, st);
}

// The gated / residual projection in row chunks, with the caller's hook after each chunk's launch (see ChunkHook).
static int linear_gate_resid_chunked(Ctx* c, const bf16* x, long long ldx, long long M, int K, const bf16* w, int N,
                                     const bf16* resid, long long ldr, bf16* out, long long ldo, cudaStream_t st,
                                     const ChunkHook* hook) {
  if (!hook || !hook->after)
    return linear_gate_resid(c, x, ldx, M, K, w, N, nullptr, 0, 0, resid, ldr, out, ldo, st);
  if (hook->parts <= 1) {  // one chunk: the hook still runs, after the whole projection
    const int rc = linear_gate_resid(c, x, ldx, M, K, w, N, nullptr, 0, 0, resid, ldr, out, ldo, st);
    return rc ? rc : hook->after(0, M);
  }
  const long long unit = hook->unit > 0 ? hook->unit : 1;
  long long per = (M + hook->parts - 1) / hook->parts;
  per = (per + unit - 1) / unit * unit;
  const int sms0 = c->gemm_sms, cap0 = c->peer_cta_cap;
  if (hook->reserve_sms > 0 && hook->reserve_sms < c->sm_count) {
    c->gemm_sms = c->sm_count - hook->reserve_sms;
    c->peer_cta_cap = hook->reserve_sms * 8;
  }
  int rc = XFOLD_OK;
  for (long long m0 = 0; m0 < M && !rc; m0 += per) {
    const long long m = M - m0 < per ? M - m0 : per;
    rc = linear_gate_resid(c, x + m0 * ldx, ldx, m, K, w, N, nullptr, 0, 0, resid ? resid + m0 * ldr : nullptr, ldr,
                           out + m0 * ldo, ldo, st);
    if (!rc) rc = hook->after(m0, m);
  }
  c->gemm_sms = sms0;
  c->peer_cta_cap = cap0;
  return rc;
}

static int linear_swiglu(Ctx* c, const bf16* x, long long ldx, long long M, int K, const bf16* wp, int F, bf16* out,
                         long long ldo, cudaStream_t st) {
  if (F % 128) return fail(c, XFOLD_ERR_ARG, "linear_swiglu: F must be a multiple of 128");
  if (M >= (1ll << 31)) return fail(c, XFOLD_ERR_ARG, "linear: too many rows");
  GemmArgs a;
  a.N = 2 * F;
  a.tiles_n = F / 128;
  a.out = out;
  a.ldo = ldo;
  return gemm_rows(c, EPI_SWIGLU, x, ldx, M, K, wp, 2 * F, K, a, 256, st);
}

static int batched_contract(Ctx* c, const bf16* a_, const bf16* b_, bf16* out, int channels, int Mi, int Nj, int Kk,
                            long long ld, long long csa, long long csb, long long ldo, long long cso, cudaStream_t st) {
  if ((ld & 7) || (csa & 7) || (csb & 7) || (ldo & 7) || (cso & 7))
    return fail(c, XFOLD_ERR_ARG, "contract: strides must be multiples of 8 elements");
  CUtensorMap tA, tB;
  if (!make_tmap_bf16_3d(&tA, a_, Kk, Mi, channels, ld, csa, 64, 128, 1) ||
      !make_tmap_bf16_3d(&tB, b_, Kk, Nj, channels, ld, csb, 64, 256, 1))
    return fail(c, XFOLD_ERR_ARG, "contract: cannot encode tensor maps");
  GemmArgs a;
  a.M = Mi;
  a.N = Nj;
  a.K = Kk;
  a.batches = channels;
  a.b_batched = 1;
  a.tiles_m = (Mi + 127) / 128;
  a.tiles_n = (Nj + 255) / 256;
  a.out = out;
  a.ldo = ldo;
  a.out_batch_stride = cso;
  a.status = c->d_status;
  return launch_gemm(c, EPI_PLAIN, 256, tA, tB, a, st);
}

// ---------------------------------------------------------------------------------------------
// module-level operators
// ---------------------------------------------------------------------------------------------

// a / b are stored "row-interleaved channel-major": element (row i, channel c, k) at (i * 128 + c) * ld + k.
// A rank's rows are one contiguous block, so the all-gather of b over the row-shard group is a plain
// concatenation, and the per-channel operand of the contraction is a strided 2-D slice for TMA.
int trimul_project(Ctx* c, const bf16* z, const float* mask, int R, int N, int transposed_store,
                          const xfold_trimul_weights* w, bf16* x, bf16* a_out, bf16* b_out, bf16* g, long long chan_stride,
                          long long row_stride, cudaStream_t st) {
  const long long M = (long long)R * N;
  int rc = launch_ln_rows(c, z, 128, x, 128, M, 128, w->ln_in_gamma, w->ln_in_beta, 1e-5f, 0, nullptr, nullptr, 0,
                          nullptr, nullptr, 0, st);
  if (rc) return rc;
  CUtensorMap tA, tB;
  bool ok;
  GemmArgs a;
  if (!transposed_store) {
    ok = make_tmap_bf16_3d(&tA, x, 128, M, 1, 128, (uint64_t)128 * M, 64, 128, 1);
    a.a_row_mode = 0;
    a.tiles_m = (int)((M + 127) / 128);
  } else {  // tile rows step along the first token axis, second axis fixed: a[j][c][i] (needs R == N)
    ok = make_tmap_bf16_3d(&tA, x, 128, N, R, 128, (uint64_t)128 * N, 64, 1, 128);
    a.a_row_mode = 1;
    a.a_dim1 = N;
    a.tiles_m = N * ((R + 127) / 128);
  }
  ok = ok && make_tmap_bf16_3d(&tB, w->w_in, 128, 640, 1, 128, 128 * 640, 64, 256, 1);
  if (!ok) return fail(c, XFOLD_ERR_ARG, "trimul: cannot encode projection tensor maps");
  a.M = (int)M;
  a.N = 640;
  a.K = 128;
  a.tiles_n = 3;
  a.out_a = a_out;
  a.out_b = b_out;
  a.out_g = g;
  a.cm_chan_stride = chan_stride;
  a.cm_ld = row_stride;
  a.ntok = N;
  a.mask = mask;
  a.status = c->d_status;
  return launch_gemm(c, EPI_TRIMUL_AB, 256, tA, tB, a, st);
}

// o[i][c][j] = sum_k a[i][c][k] * b[j][c][k]   (a: Ri rows, b: Nj rows, both [.][128][ld]; o: [Ri][128][ldo])
// (chan, row) strides in elements: row-interleaved [rows][128][ld] has (ld, 128*ld); channel-major [128][rows][ld] has (rows*ld, ld)
int trimul_contract(Ctx* c, const bf16* a_, long long a_cs, long long a_rs, const bf16* b_, long long b_cs,
                           long long b_rs, int Ri, int Nj, int K, bf16* o, long long o_cs, long long o_rs, cudaStream_t st,
                           int channels) {
  if (((a_cs | a_rs | b_cs | b_rs | o_cs | o_rs) & 7)) return fail(c, XFOLD_ERR_ARG, "contract: strides must be multiples of 8");
  CUtensorMap tA, tB;
  if (!make_tmap_bf16_3d(&tA, a_, K, Ri, channels, a_rs, a_cs, 64, 128, 1) ||
      !make_tmap_bf16_3d(&tB, b_, K, Nj, channels, b_rs, b_cs, 64, 256, 1))
    return fail(c, XFOLD_ERR_ARG, "contract: cannot encode tensor maps");
  GemmArgs a;
  a.M = Ri;
  a.N = Nj;
  a.K = K;
  a.batches = channels;
  a.b_batched = 1;
  a.tiles_m = (Ri + 127) / 128;
  a.tiles_n = (Nj + 255) / 256;
  a.out = o;
  a.ldo = o_rs;
  a.out_batch_stride = o_cs;
  a.status = c->d_status;
  return launch_gemm(c, EPI_PLAIN, 256, tA, tB, a, st);
}

// The incoming-edges product on the SAME channel planes as the outgoing one ('ckj,cki->cij',
// nn/d_triangle_multiplication.py:122-124): o[c][i][j] = sum_k at[c][k][i] * bt[c][k][j], both operands read with the
// contraction index as their slow dimension (MN-major tensor-core operands), so no transposed copy of z, a or b is made.
int trimul_contract_mn(Ctx* c, const bf16* at, long long at_cs, long long at_rs, const bf16* bt, long long bt_cs,
                       long long bt_rs, int Mi, int Nj, int K, bf16* o, long long o_cs, long long o_rs, cudaStream_t st,
                       int channels) {
  if (((at_cs | at_rs | bt_cs | bt_rs | o_cs | o_rs) & 7)) return fail(c, XFOLD_ERR_ARG, "contract: strides must be multiples of 8");
  CUtensorMap tA, tB;
  if (!make_tmap_bf16_3d(&tA, at, Mi, K, channels, at_rs, at_cs, 64, 64, 1) ||
      !make_tmap_bf16_3d(&tB, bt, Nj, K, channels, bt_rs, bt_cs, 64, 64, 1))
    return fail(c, XFOLD_ERR_ARG, "contract: cannot encode tensor maps");
  GemmArgs a;
  a.M = Mi;
  a.N = Nj;
  a.K = K;
  a.batches = channels;
  a.b_batched = 1;
  a.mn_major = 1;
  a.tiles_m = (Mi + 127) / 128;
  a.tiles_n = (Nj + 255) / 256;
  a.out = o;
  a.ldo = o_rs;
  a.out_batch_stride = o_cs;
  a.status = c->d_status;
  return launch_gemm(c, EPI_PLAIN, 256, tA, tB, a, st);
}

// z (+)= Linear(LN_c(o)) * sigmoid(g); o: [R][128][ldo]; x: scratch [R*N][128]
int trimul_output(Ctx* c, const bf16* o, long long o_cs, long long o_rs, const bf16* g, int R, int N,
                         const xfold_trimul_weights* w, bf16* x, bf16* z, cudaStream_t st, bf16* upd) {
  int rc = launch_cm_ln(c, o, o_cs, o_rs, R, N, x, w->ln_c_gamma, w->ln_c_beta, 1e-5f, st);
  if (rc) return rc;
  // upd given: write the update alone there and leave z untouched; else z += update
  return linear_gate_resid(c, x, 128, (long long)R * N, 128, (const bf16*)w->w_out, 128, g, 128, 0, upd ? nullptr : z, 128,
                           upd ? upd : z, 128, st);
}

struct TriMulWs {
  bf16 *x, *a, *b, *g, *o;
  int ld;
  size_t bytes;
};
static TriMulWs carve_trimul(void* ws, size_t cap, int N) {
  TriMulWs w;
  Carver cv(ws, cap);
  w.ld = pad8(N);
  const size_t tok = (size_t)N * N * 128 * 2;
  const size_t cm = (size_t)128 * N * w.ld * 2;
  w.x = (bf16*)cv.take(tok);
  w.g = (bf16*)cv.take(tok);
  w.a = (bf16*)cv.take(cm);
  w.b = (bf16*)cv.take(cm);
  w.o = (bf16*)cv.take(cm);
  w.bytes = cv.off;
  return w;
}

static int trimul_fwd(Ctx* c, bf16* z, const float* mask, int N, int outgoing, const xfold_trimul_weights* w, void* ws,
                      size_t ws_bytes, cudaStream_t st, bf16* upd = nullptr) {
  if (!z || !w || !w->w_in || !w->w_out) return fail(c, XFOLD_ERR_ARG, "trimul: null argument");
  if (N <= 0) return XFOLD_OK;
  TriMulWs W = carve_trimul(ws, ws_bytes, N);
  if (!ws || W.bytes > ws_bytes) return fail(c, XFOLD_ERR_ARG, "trimul: workspace too small (%zu < %zu)", ws_bytes, W.bytes);
  // incoming: a and b are stored transposed, so that o[i][c][j] = sum_k bT[i][c][k] aT[j][c][k] is the same product
  // one GPU: plain channel-major planes [128][N][ld] (rows of a tile are 2 KB apart, best DRAM locality)
  const long long cs = (long long)N * W.ld, rs = W.ld;
  int rc = trimul_project(c, z, mask, N, N, outgoing ? 0 : 1, w, W.x, W.a, W.b, W.g, cs, rs, st);
  if (rc) return rc;
  rc = trimul_contract(c, outgoing ? W.a : W.b, cs, rs, outgoing ? W.b : W.a, cs, rs, N, N, N, W.o, cs, rs, st);
  if (rc) return rc;
  return trimul_output(c, W.o, cs, rs, W.g, N, N, w, W.x, z, st, upd);
}

struct TriAttnWs {
  bf16 *x, *qkvg, *nbT, *mext;
  int ldq;
  size_t bytes;
};
static TriAttnWs carve_triattn(void* ws, size_t cap, int R, int N) {
  TriAttnWs w;
  Carver cv(ws, cap);
  w.ldq = pad8(N);
  w.x = (bf16*)cv.take((size_t)R * N * 128 * 2);
  w.qkvg = (bf16*)cv.take((size_t)R * N * 512 * 2);
  w.nbT = (bf16*)cv.take((size_t)4 * N * w.ldq * 2);
  w.mext = (bf16*)cv.take((size_t)R * ((N + 127) / 128) * 4096);
  w.bytes = cv.off;
  return w;
}

// x = LN(z) for a block of R rows, plus the pair bias those rows contribute, bf16, query-major [h][q][k]:
//   rows_are_keys == 0: the rows are QUERY rows:  bias[h * plane + row_local * pitch + y]      (row-major walk)
//   rows_are_keys == 1: the rows are KEY rows x:  bias[h * plane + y * pitch + x_local]        (column-by-column walk)
int triattn_bias(Ctx* c, const bf16* z, int R, int N, const xfold_triattn_weights* w, bf16* x, bf16* bias,
                        int pitch, long long plane, int rows_are_keys, cudaStream_t st) {
  const long long M = (long long)R * N;
  if (!rows_are_keys)
    return launch_ln_rows(c, z, 128, x, 128, M, 128, w->ln_gamma, w->ln_beta, 1e-5f, 4, w->w_bias, nullptr, plane, nullptr,
                          nullptr, 0, st, bias, -N, 0, pitch);
  return launch_ln_rows(c, z, 128, x, 128, M, 128, w->ln_gamma, w->ln_beta, 1e-5f, 4, w->w_bias, nullptr, plane, nullptr,
                        nullptr, 0, st, bias, R, N, pitch);
}

// z (+)= out_proj(gated attention(x)) for R batch rows (sequence length N); biasT: bf16 [4][N][ldq], [h][query][key].
// transposed: the R x N token grid is stored [N][R] (sequence index outermost), used by the single-GPU ending node.
int triattn_core(Ctx* c, bf16* x, const bf16* biasT, int ldq, const float* mask, long long mask_ld, int R, int N,
                        int transposed, const xfold_triattn_weights* w, bf16* qkvg, bf16* mext, bf16* z, cudaStream_t st,
                        bf16* upd, const ChunkHook* hook) {
  const long long M = (long long)R * N;
  // the v columns are stored as fp16: the attention kernel's P V product runs with fp16 operands
  int rc = linear_plain(c, x, 128, M, 128, (const bf16*)w->w_qkvg, 512, nullptr, w->qkvg_scale, qkvg, 512, st, 256, 384);
  if (rc) return rc;
  if ((rc = launch_mext(c, mask, mask_ld, mext, R, N, st))) return rc;
  const long long seq_stride = transposed ? (long long)R * 128 : 128;
  const long long batch_stride = transposed ? 128 : (long long)N * 128;
  rc = launch_attention2(c, qkvg, 512, N, R, transposed, 0, 128, 256, 384, 4, biasT, ldq, mext, R, x, seq_stride,
                         batch_stride, st);
  if (rc) return rc;
  return linear_gate_resid_chunked(c, x, 128, M, 128, (const bf16*)w->w_out, 128, upd ? nullptr : z, 128, upd ? upd : z, 128,
                                   st, hook);
}

static int triattn_fwd(Ctx* c, bf16* z, const float* mask, int N, int transpose, const xfold_triattn_weights* w, void* ws,
                       size_t ws_bytes, cudaStream_t st, bf16* upd = nullptr) {
  if (!z || !w || !w->w_qkvg || !w->w_out || !w->w_bias) return fail(c, XFOLD_ERR_ARG, "triattn: null argument");
  if (N <= 0) return XFOLD_OK;
  TriAttnWs W = carve_triattn(ws, ws_bytes, N, N);
  if (!ws || W.bytes > ws_bytes) return fail(c, XFOLD_ERR_ARG, "triattn: workspace too small (%zu < %zu)", ws_bytes, W.bytes);
  // both nodes use bias(q, k) = projection of token (q, k), not transposed for the ending node
  int rc = triattn_bias(c, z, N, N, w, W.x, W.nbT, W.ldq, (long long)N * W.ldq, 0, st);
  if (rc) return rc;
  return triattn_core(c, W.x, W.nbT, W.ldq, mask, N, N, N, transpose, w, W.qkvg, W.mext, z, st, upd);
}

int transition_fwd(Ctx* c, bf16* x, long long rows, int C, int F, const xfold_transition_weights* w, void* ws,
                          size_t ws_bytes, cudaStream_t st, bf16* upd, const ChunkHook* hook) {
  if (!x || !w || !w->w1_packed || !w->w2) return fail(c, XFOLD_ERR_ARG, "transition: null argument");
  if (rows <= 0) return XFOLD_OK;
  // before any size arithmetic or launch: row counts the kernels cannot index, or whose byte sizes would wrap
  if (C <= 0 || F <= 0 || rows >= (1ll << 31)) return fail(c, XFOLD_ERR_ARG, "transition: bad shape (%lld rows, C=%d, F=%d)", rows, C, F);
  Carver cv(ws, ws_bytes);
  bf16* xn = (bf16*)cv.take((size_t)rows * C * 2);
  bf16* h = (bf16*)cv.take((size_t)rows * F * 2);
  if (!ws || !cv.ok()) return fail(c, XFOLD_ERR_ARG, "transition: workspace too small (%zu < %zu)", ws_bytes, cv.off);
  int rc = launch_ln_rows(c, x, C, xn, C, rows, C, w->ln_gamma, w->ln_beta, 1e-5f, 0, nullptr, nullptr, 0, nullptr,
                          nullptr, 0, st);
  if (rc) return rc;
  rc = linear_swiglu(c, xn, C, rows, C, (const bf16*)w->w1_packed, F, h, F, st);
  if (rc) return rc;
  return linear_gate_resid_chunked(c, h, F, rows, F, (const bf16*)w->w2, C, upd ? nullptr : x, C, upd ? upd : x, C, st, hook);
}

struct ApbWs {
  bf16 *qkvg, *biasT, *mext;
  int ldm, ldq;
};
static size_t apb_ws(int B, int S, int H, int Dp, Carver* cv, ApbWs* out) {
  Carver local(nullptr, 0);
  if (!cv) cv = &local;
  ApbWs w;
  w.ldm = (S + 127) / 128 * 128;
  w.ldq = pad8(S);
  w.qkvg = (bf16*)cv->take((size_t)B * S * 4 * H * Dp * 2);
  w.biasT = (bf16*)cv->take((size_t)H * S * w.ldq * 2);
  w.mext = (bf16*)cv->take((size_t)B * (w.ldm / 128) * 4096);  // room for one mask row per batch entry
  if (out) *out = w;
  return cv->off;
}

// pair_bias: float32 [H][S][S], or, when pair_biasT is given, the same as bf16 [H][S][pad8(S)] (both [h][query][key])
static int apb_core_fwd_(Ctx* c, const bf16* xn, int B, int S, int C, int H, int Dp, const bf16* w_qkvg,
                         const float* qkvg_bias, const float* qkvg_scale, const float* pair_bias, const bf16* pair_biasT,
                         const float* mask, bf16* out, void* ws, size_t ws_bytes, cudaStream_t st, long long mask_ld);
static int apb_core_fwd(Ctx* c, const bf16* xn, int B, int S, int C, int H, int Dp, const bf16* w_qkvg,
                        const float* qkvg_bias, const float* qkvg_scale, const float* pair_bias, const bf16* pair_biasT,
                        const float* mask, bf16* out, void* ws, size_t ws_bytes, cudaStream_t st, long long mask_ld = 0) {
  c->attn_tag = XFOLD_K_APB_ATTENTION;  // accounted separately from the TriangleAttention launches
  const int rc = apb_core_fwd_(c, xn, B, S, C, H, Dp, w_qkvg, qkvg_bias, qkvg_scale, pair_bias, pair_biasT, mask, out, ws,
                               ws_bytes, st, mask_ld);
  c->attn_tag = XFOLD_K_ATTENTION;
  return rc;
}
static int apb_core_fwd_(Ctx* c, const bf16* xn, int B, int S, int C, int H, int Dp, const bf16* w_qkvg,
                         const float* qkvg_bias, const float* qkvg_scale, const float* pair_bias, const bf16* pair_biasT,
                         const float* mask, bf16* out, void* ws, size_t ws_bytes, cudaStream_t st, long long mask_ld) {
  if (!xn || !w_qkvg || !out || (!pair_bias && !pair_biasT)) return fail(c, XFOLD_ERR_ARG, "apb: null argument");
  if ((Dp != 32 && Dp != 64) || (H * Dp) % 128) return fail(c, XFOLD_ERR_ARG, "apb: H x Dp must be a multiple of 128 with Dp 32 or 64");
  Carver cv(ws, ws_bytes);
  ApbWs W;
  apb_ws(B, S, H, Dp, &cv, &W);
  if (!ws || !cv.ok()) return fail(c, XFOLD_ERR_ARG, "apb: workspace too small (%zu < %zu)", ws_bytes, cv.off);
  const int Wd = H * Dp;
  // the v columns leave the projection as fp16: P and V are the fp16 operands of the P V product
  int rc = linear_plain(c, xn, C, (long long)B * S, C, w_qkvg, 4 * Wd, qkvg_bias, qkvg_scale, W.qkvg, 4 * Wd, st, 2 * Wd, 3 * Wd);
  if (rc) return rc;
  if (!pair_biasT) {
    if ((rc = launch_bias_transpose(c, pair_bias, W.biasT, H, S, W.ldq, st))) return rc;
    pair_biasT = W.biasT;
  }
  // mask_ld > 0: one mask row per batch entry (the TriangleAttention op); else one row shared by all
  const int mrows = (mask && mask_ld > 0) ? B : 1;
  if ((rc = launch_mext(c, mask, mask_ld, W.mext, mrows, S, st))) return rc;
  return launch_attention2(c, W.qkvg, 4 * Wd, S, B, 0, 0, Wd, 2 * Wd, 3 * Wd, H, pair_biasT, W.ldq, W.mext, mrows, out, Wd,
                           (long long)S * Wd, st, Dp);
}

size_t single_ws_bytes(int N) {
  return align_up((size_t)N * 384 * 2, 1024) + align_up((size_t)N * 512 * 2, 1024) + apb_ws(1, N, 16, 32, nullptr, nullptr) +
         align_up((size_t)N * 384 * 2, 1024) + align_up((size_t)N * 1536 * 2, 1024) + 16384;
}

// single += AttentionPairBias(single, pair logits) ; single += Transition(single)   (nn/d_pairformer.py:162-169)
// plT: bf16 [16][N][ldq] pair logits, [h][query][key].
int single_update(Ctx* c, bf16* s, const bf16* plT, int ldq, const float* seq_mask, int N,
                         const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, cudaStream_t st) {
  Carver cv(ws, ws_bytes);
  bf16* xn = (bf16*)cv.take((size_t)N * 384 * 2);
  bf16* o = (bf16*)cv.take((size_t)N * 512 * 2);
  const size_t apb_bytes = apb_ws(1, N, 16, 32, nullptr, nullptr);
  void* apb_scratch = cv.take(apb_bytes);
  const size_t tr_bytes = align_up((size_t)N * 384 * 2, 1024) + align_up((size_t)N * 1536 * 2, 1024) + 2048;
  void* tr_scratch = cv.take(tr_bytes);
  if (!ws || !cv.ok()) return fail(c, XFOLD_ERR_ARG, "single update: workspace too small (%zu < %zu)", ws_bytes, cv.off);
  int rc;
  if ((rc = launch_ln_rows(c, s, 384, xn, 384, N, 384, w->sa_ln_gamma, w->sa_ln_beta, 1e-5f, 0, nullptr, nullptr, 0,
                           nullptr, nullptr, 0, st))) return rc;
  if ((rc = apb_core_fwd(c, xn, 1, N, 384, 16, 32, (const bf16*)w->sa_w_qkvg, w->sa_qkvg_bias, w->sa_qkvg_scale, nullptr,
                         plT, seq_mask, o, apb_scratch, apb_bytes, st))) return rc;
  if ((rc = linear_gate_resid(c, o, 512, N, 512, (const bf16*)w->sa_w_out, 384, nullptr, 0, 0, s, 384, s, 384, st))) return rc;
  return transition_fwd(c, s, N, 384, 1536, &w->single_transition, tr_scratch, tr_bytes, st);
}

static size_t pairformer_ws_bytes(int N) {
  size_t a = carve_trimul(nullptr, 0, N).bytes;
  size_t b = carve_triattn(nullptr, 0, N, N).bytes;
  size_t t = align_up((size_t)N * N * 128 * 2, 1024) + align_up((size_t)N * N * 512 * 2, 1024) + 2048;
  size_t m = a > b ? a : b;
  if (t > m) m = t;
  size_t s = align_up((size_t)16 * N * pad8(N) * 2, 1024) + single_ws_bytes(N) + 4096;
  return (m > s ? m : s) + 4096;
}

static int pairformer_fwd(Ctx* c, bf16* z, bf16* s, const float* pair_mask, const float* seq_mask, int N,
                          const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!z || !w) return fail(c, XFOLD_ERR_ARG, "pairformer: null argument");
  if (ws_bytes < pairformer_ws_bytes(N)) return fail(c, XFOLD_ERR_ARG, "pairformer: workspace too small (%zu < %zu)", ws_bytes, pairformer_ws_bytes(N));
  int rc;
  if ((rc = trimul_fwd(c, z, pair_mask, N, 1, &w->tri_out, ws, ws_bytes, st))) return rc;
  if ((rc = trimul_fwd(c, z, pair_mask, N, 0, &w->tri_in, ws, ws_bytes, st))) return rc;
  if ((rc = triattn_fwd(c, z, pair_mask, N, 0, &w->att_start, ws, ws_bytes, st))) return rc;
  if ((rc = triattn_fwd(c, z, pair_mask, N, 1, &w->att_end, ws, ws_bytes, st))) return rc;
  if ((rc = transition_fwd(c, z, (long long)N * N, 128, 512, &w->pair_transition, ws, ws_bytes, st))) return rc;
  if (!s || !w->spl_w) return XFOLD_OK;
  Carver cv(ws, ws_bytes);
  const int ldq = pad8(N);
  bf16* pl = (bf16*)cv.take((size_t)16 * N * ldq * 2);
  void* rest = cv.take(single_ws_bytes(N));
  if (!cv.ok()) return fail(c, XFOLD_ERR_ARG, "pairformer: workspace too small for the single path");
  const long long M = (long long)N * N;
  if ((rc = launch_ln_rows(c, z, 128, nullptr, 128, M, 128, w->spl_ln_gamma, w->spl_ln_beta, 1e-5f, 16, w->spl_w, nullptr,
                           (long long)N * ldq, nullptr, nullptr, 0, st, pl, -N, 0, ldq))) return rc;
  return single_update(c, s, pl, ldq, seq_mask, N, w, rest, single_ws_bytes(N), st);
}

}  // namespace xf

using namespace xf;

struct xfold_ctx : public xf::Ctx {};

extern "C" {

const char* xfold_version(void) { return "xfold_b200 0.1 (sm_100a, tcgen05/TMA)"; }

int xfold_ctx_create(int device, xfold_ctx** out) {
  if (!out) return XFOLD_ERR_ARG;
  *out = nullptr;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) return XFOLD_ERR_DEVICE;
  if (cudaSetDevice(device) != cudaSuccess) return XFOLD_ERR_DEVICE;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return XFOLD_ERR_DEVICE;
  if (prop.major != 10) return XFOLD_ERR_DEVICE;  // sm_100a code only
  if (!load_encode()) return XFOLD_ERR_DEVICE;
  xfold_ctx* c = new xfold_ctx();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  if (cudaMalloc(&c->d_status, sizeof(int)) != cudaSuccess) { delete c; return XFOLD_ERR_DEVICE; }
  cudaMemset(c->d_status, 0, sizeof(int));
  *out = c;
  return XFOLD_OK;
}

void xfold_ctx_destroy(xfold_ctx* c) {
  if (!c) return;
  if (c->d_status) cudaFree(c->d_status);
  for (auto& r : c->prof_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  for (auto& r : c->prof_pool) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  delete c;
}

const char* xfold_last_error(xfold_ctx* c) { return c ? c->last_error : "null context"; }

long long xfold_launch_count(xfold_ctx* c) { return c ? c->launch_count : 0; }

int xfold_profile_enable(xfold_ctx* c, int on) {
  if (!c) return XFOLD_ERR_ARG;
  c->prof_on = on;
  return XFOLD_OK;
}

int xfold_profile_read(xfold_ctx* c, int kernel_class, float* ms_total, int* launches) {
  if (!c || !ms_total || !launches) return XFOLD_ERR_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "profile read: device error");
  float total = 0.f;
  int n = 0;
  std::vector<ProfRec> keep;
  for (auto& r : c->prof_recs) {
    if (r.tag != kernel_class) { keep.push_back(r); continue; }
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) { total += ms; ++n; }
    c->prof_pool.push_back(r);
  }
  c->prof_recs.swap(keep);
  *ms_total = total;
  *launches = n;
  return XFOLD_OK;
}

int xfold_check_status(xfold_ctx* c, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  int h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "status read: %s", cudaGetErrorString(e));
  if (h != 0) {
    cudaMemsetAsync(c->d_status, 0, sizeof(int), st);
    cudaStreamSynchronize(st);
    return fail(c, XFOLD_ERR_TIMEOUT, "in-kernel bounded wait ran out (code %d)", h);
  }
  return XFOLD_OK;
}

int xfold_layernorm_fwd(xfold_ctx* c, const void* x, long long ldx, void* y, long long ldy, long long rows, int C,
                        const float* gamma, const float* beta, float eps, int num_proj, const float* proj_w,
                        float* proj, long long proj_plane, const void* mod_scale, const void* mod_shift, int mod_rows,
                        void* stream) {
  if (!c || !x) return XFOLD_ERR_ARG;
  if (num_proj > 0 && (!proj_w || !proj)) return fail(c, XFOLD_ERR_ARG, "layernorm: projection requested without buffers");
  if ((mod_scale != nullptr) != (mod_shift != nullptr) || (mod_scale && mod_rows <= 0))
    return fail(c, XFOLD_ERR_ARG, "layernorm: modulation needs scale, shift and mod_rows");
  return launch_ln_rows(c, (const bf16*)x, ldx, (bf16*)y, ldy, rows, C, gamma, beta, eps, num_proj, proj_w, proj,
                        proj_plane, (const bf16*)mod_scale, (const bf16*)mod_shift, mod_rows, (cudaStream_t)stream);
}

int xfold_swiglu_fwd(xfold_ctx* c, const void* in, void* out, long long rows, int F, void* stream) {
  if (!c || !in || !out) return XFOLD_ERR_ARG;
  return launch_swiglu(c, (const bf16*)in, (bf16*)out, rows, F, (cudaStream_t)stream);
}

int xfold_linear_fwd(xfold_ctx* c, const void* x, long long ldx, long long M, int K, const void* w, int N,
                     const float* bias, const float* scale, void* out, long long ldo, void* stream) {
  if (!c || !x || !w || !out) return XFOLD_ERR_ARG;
  return linear_plain(c, (const bf16*)x, ldx, M, K, (const bf16*)w, N, bias, scale, (bf16*)out, ldo, (cudaStream_t)stream);
}

int xfold_linear_gate_residual_fwd(xfold_ctx* c, const void* x, long long ldx, long long M, int K, const void* w, int N,
                                   const void* gate, long long ldg, int row_gate_mod, const void* resid, long long ldr,
                                   void* out, long long ldo, void* stream) {
  if (!c || !x || !w || !out) return XFOLD_ERR_ARG;
  return linear_gate_resid(c, (const bf16*)x, ldx, M, K, (const bf16*)w, N, (const bf16*)gate, ldg, row_gate_mod,
                           (const bf16*)resid, ldr, (bf16*)out, ldo, (cudaStream_t)stream);
}

int xfold_linear_swiglu_fwd(xfold_ctx* c, const void* x, long long ldx, long long M, int K, const void* w_packed, int F,
                            void* out, long long ldo, void* stream) {
  if (!c || !x || !w_packed || !out) return XFOLD_ERR_ARG;
  return linear_swiglu(c, (const bf16*)x, ldx, M, K, (const bf16*)w_packed, F, (bf16*)out, ldo, (cudaStream_t)stream);
}

int xfold_batched_contract_fwd(xfold_ctx* c, const void* a, const void* b, void* out, int channels, int Mi, int Nj, int Kk,
                               long long ld, long long chan_stride_a, long long chan_stride_b, long long ldo,
                               long long chan_stride_o, void* stream) {
  if (!c || !a || !b || !out) return XFOLD_ERR_ARG;
  return batched_contract(c, (const bf16*)a, (const bf16*)b, (bf16*)out, channels, Mi, Nj, Kk, ld, chan_stride_a,
                          chan_stride_b, ldo, chan_stride_o, (cudaStream_t)stream);
}

size_t xfold_trimul_workspace_bytes(int N) { return carve_trimul(nullptr, 0, N).bytes; }
int xfold_triangle_multiplication_fwd(xfold_ctx* c, void* z, const float* mask, int N, int outgoing,
                                      const xfold_trimul_weights* w, void* ws, size_t ws_bytes, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return trimul_fwd(c, (bf16*)z, mask, N, outgoing, w, ws, ws_bytes, (cudaStream_t)stream);
}

size_t xfold_triattn_workspace_bytes(int N) { return carve_triattn(nullptr, 0, N, N).bytes; }
int xfold_triangle_attention_fwd(xfold_ctx* c, void* z, const float* mask, int N, int transpose,
                                 const xfold_triattn_weights* w, void* ws, size_t ws_bytes, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return triattn_fwd(c, (bf16*)z, mask, N, transpose, w, ws, ws_bytes, (cudaStream_t)stream);
}

size_t xfold_transition_workspace_bytes(long long rows, int C, int F) {
  return align_up((size_t)rows * C * 2, 1024) + align_up((size_t)rows * F * 2, 1024) + 2048;
}
int xfold_transition_fwd(xfold_ctx* c, void* x, long long rows, int C, int F, const xfold_transition_weights* w, void* ws,
                         size_t ws_bytes, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return transition_fwd(c, (bf16*)x, rows, C, F, w, ws, ws_bytes, (cudaStream_t)stream);
}

size_t xfold_apb_workspace_bytes(int B, int S, int H, int Dp) { return apb_ws(B, S, H, Dp, nullptr, nullptr) + 2048; }
int xfold_attention_pair_bias_core_fwd(xfold_ctx* c, const void* xn, int B, int S, int C, int H, int Dp,
                                       const void* w_qkvg, const float* qkvg_bias, const float* qkvg_scale,
                                       const float* pair_bias, const float* mask, void* out, void* ws, size_t ws_bytes,
                                       void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return apb_core_fwd(c, (const bf16*)xn, B, S, C, H, Dp, (const bf16*)w_qkvg, qkvg_bias, qkvg_scale, pair_bias, nullptr,
                      mask, (bf16*)out, ws, ws_bytes, (cudaStream_t)stream);
}

size_t xfold_pairformer_workspace_bytes(int N) { return pairformer_ws_bytes(N); }
int xfold_pairformer_block_fwd(xfold_ctx* c, void* z, void* s, const float* pair_mask, const float* seq_mask, int N,
                               const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return pairformer_fwd(c, (bf16*)z, (bf16*)s, pair_mask, seq_mask, N, w, ws, ws_bytes, (cudaStream_t)stream);
}

int xfold_pair_bias_prepare_fwd(xfold_ctx* c, const float* pair_bias, int H, int S, void* prepared, void* stream) {
  if (!c || !pair_bias || !prepared) return XFOLD_ERR_ARG;
  return launch_bias_transpose(c, pair_bias, (bf16*)prepared, H, S, pad8(S), (cudaStream_t)stream);
}

int xfold_attention_pair_bias_core_prepared_fwd(xfold_ctx* c, const void* xn, int B, int S, int C, int H, int Dp,
                                                const void* w_qkvg, const float* qkvg_bias, const float* qkvg_scale,
                                                const void* prepared_bias, const float* mask, void* out, void* ws,
                                                size_t ws_bytes, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return apb_core_fwd(c, (const bf16*)xn, B, S, C, H, Dp, (const bf16*)w_qkvg, qkvg_bias, qkvg_scale, nullptr,
                      (const bf16*)prepared_bias, mask, (bf16*)out, ws, ws_bytes, (cudaStream_t)stream);
}

int xfold_gated_attention_core_fwd(xfold_ctx* c, const void* xn, int B, int S, int C, int H, int Dp, const void* w_qkvg,
                                   const float* qkvg_bias, const float* qkvg_scale, const float* pair_bias,
                                   const float* mask, long long mask_ld, void* out, void* ws, size_t ws_bytes, void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  return apb_core_fwd(c, (const bf16*)xn, B, S, C, H, Dp, (const bf16*)w_qkvg, qkvg_bias, qkvg_scale, pair_bias, nullptr,
                      mask, (bf16*)out, ws, ws_bytes, (cudaStream_t)stream, mask_ld);
}

int xfold_pairformer_stack_fwd(xfold_ctx* c, void* z, void* s, const float* pair_mask, const float* seq_mask, int N,
                               const xfold_pairformer_weights* blocks, int num_blocks, void* ws, size_t ws_bytes,
                               void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  if (num_blocks < 0 || (num_blocks > 0 && !blocks)) return fail(c, XFOLD_ERR_ARG, "pairformer stack: no weights for %d blocks", num_blocks);
  for (int i = 0; i < num_blocks; ++i) {
    const int rc = pairformer_fwd(c, (bf16*)z, (bf16*)s, pair_mask, seq_mask, N, &blocks[i], ws, ws_bytes, (cudaStream_t)stream);
    if (rc) return rc;
  }
  return XFOLD_OK;
}

/* ---- row-shard stages ------------------------------------------------------------------------ */
int xfold_trimul_project_fwd(xfold_ctx* c, const void* z, const float* mask, int R, int N, const xfold_trimul_weights* w,
                             void* x_scratch, void* a, void* b, void* g, int ld, void* stream) {
  if (!c || !z || !w || !x_scratch || !a || !b || !g) return XFOLD_ERR_ARG;
  if (ld < N || (ld & 7)) return fail(c, XFOLD_ERR_ARG, "trimul project: ld must be >= N and a multiple of 8");
  return trimul_project(c, (const bf16*)z, mask, R, N, 0, w, (bf16*)x_scratch, (bf16*)a, (bf16*)b, (bf16*)g, ld,
                        (long long)128 * ld, (cudaStream_t)stream);
}
int xfold_trimul_contract_fwd(xfold_ctx* c, const void* a, const void* b_full, int R, int Nj, int K, int ld, void* o, int ldo,
                              void* stream) {
  if (!c || !a || !b_full || !o) return XFOLD_ERR_ARG;
  if ((ld & 7) || (ldo & 7)) return fail(c, XFOLD_ERR_ARG, "contract: leading dimensions must be multiples of 8");
  return trimul_contract(c, (const bf16*)a, ld, (long long)128 * ld, (const bf16*)b_full, ld, (long long)128 * ld, R, Nj, K,
                         (bf16*)o, ldo, (long long)128 * ldo, (cudaStream_t)stream);
}
int xfold_trimul_contract_planes_fwd(xfold_ctx* c, const void* a, const void* b, int channels, int Ni, int Nj, int K, int ld,
                                     void* o, int ldo, void* stream) {
  if (!c || !a || !b || !o) return XFOLD_ERR_ARG;
  if ((ld & 7) || (ldo & 7) || channels < 1) return fail(c, XFOLD_ERR_ARG, "contract: leading dimensions must be multiples of 8");
  return trimul_contract(c, (const bf16*)a, (long long)Ni * ld, ld, (const bf16*)b, (long long)Nj * ld, ld, Ni, Nj, K, (bf16*)o,
                         (long long)Ni * ldo, ldo, (cudaStream_t)stream, channels);
}
int xfold_trimul_output_fwd(xfold_ctx* c, const void* o, int ldo, const void* g, int R, int N, const xfold_trimul_weights* w,
                            void* x_scratch, void* z, void* stream) {
  if (!c || !o || !g || !w || !x_scratch || !z) return XFOLD_ERR_ARG;
  return trimul_output(c, (const bf16*)o, ldo, (long long)128 * ldo, (const bf16*)g, R, N, w, (bf16*)x_scratch, (bf16*)z,
                       (cudaStream_t)stream);
}
int xfold_triattn_bias_fwd(xfold_ctx* c, const void* z, int R, int N, const xfold_triattn_weights* w, void* x, void* biasT,
                           int pitch, long long plane, int rows_are_keys, void* stream) {
  if (!c || !z || !w || !x || !biasT) return XFOLD_ERR_ARG;
  return triattn_bias(c, (const bf16*)z, R, N, w, (bf16*)x, (bf16*)biasT, pitch, plane, rows_are_keys, (cudaStream_t)stream);
}
size_t xfold_triattn_core_scratch_bytes(int R, int N, size_t* mext_bytes) {
  if (mext_bytes) *mext_bytes = (size_t)R * ((N + 127) / 128) * 4096;
  return (size_t)R * N * 512 * 2;
}
int xfold_triattn_core_fwd(xfold_ctx* c, void* x, const void* biasT, int ldq, const float* mask, long long mask_ld, int R,
                           int N, const xfold_triattn_weights* w, void* qkvg_scratch, void* mext_scratch, void* z,
                           void* stream) {
  if (!c || !x || !biasT || !w || !qkvg_scratch || !mext_scratch || !z) return XFOLD_ERR_ARG;
  return triattn_core(c, (bf16*)x, (const bf16*)biasT, ldq, mask, mask_ld, R, N, 0, w, (bf16*)qkvg_scratch,
                      (bf16*)mext_scratch, (bf16*)z, (cudaStream_t)stream);
}
int xfold_pair_logits_fwd(xfold_ctx* c, const void* z, int R, int N, const float* ln_gamma, const float* ln_beta,
                          const float* w16, void* plT, int pitch, long long plane, int rows_are_keys, void* stream) {
  if (!c || !z || !w16 || !plT) return XFOLD_ERR_ARG;
  const long long M = (long long)R * N;
  return launch_ln_rows(c, (const bf16*)z, 128, nullptr, 128, M, 128, ln_gamma, ln_beta, 1e-5f, 16, w16, nullptr, plane,
                        nullptr, nullptr, 0, (cudaStream_t)stream, (bf16*)plT, rows_are_keys ? R : -N, rows_are_keys ? N : 0,
                        pitch);
}
size_t xfold_single_update_workspace_bytes(int N) { return single_ws_bytes(N); }
int xfold_single_update_fwd(xfold_ctx* c, void* s, const void* plT, int ldq, const float* seq_mask, int N,
                            const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, void* stream) {
  if (!c || !s || !plT || !w) return XFOLD_ERR_ARG;
  return single_update(c, (bf16*)s, (const bf16*)plT, ldq, seq_mask, N, w, ws, ws_bytes, (cudaStream_t)stream);
}

/* ---- update-only variants: the module forwards of the reference RETURN the update and leave the
 * residual add to the caller (e.g. nn/d_pairformer.py:122); these write it to `update` and do not touch z. */
int xfold_triangle_multiplication_update_fwd(xfold_ctx* c, const void* z, void* update, const float* mask, int N,
                                             int outgoing, const xfold_trimul_weights* w, void* ws, size_t ws_bytes,
                                             void* stream) {
  if (!c || !update) return XFOLD_ERR_ARG;
  return trimul_fwd(c, (bf16*)const_cast<void*>(z), mask, N, outgoing, w, ws, ws_bytes, (cudaStream_t)stream, (bf16*)update);
}
int xfold_triangle_attention_update_fwd(xfold_ctx* c, const void* z, void* update, const float* mask, int N, int transpose,
                                        const xfold_triattn_weights* w, void* ws, size_t ws_bytes, void* stream) {
  if (!c || !update) return XFOLD_ERR_ARG;
  return triattn_fwd(c, (bf16*)const_cast<void*>(z), mask, N, transpose, w, ws, ws_bytes, (cudaStream_t)stream, (bf16*)update);
}
int xfold_transition_update_fwd(xfold_ctx* c, const void* x, void* update, long long rows, int C, int F,
                                const xfold_transition_weights* w, void* ws, size_t ws_bytes, void* stream) {
  if (!c || !update) return XFOLD_ERR_ARG;
  return transition_fwd(c, (bf16*)const_cast<void*>(x), rows, C, F, w, ws, ws_bytes, (cudaStream_t)stream, (bf16*)update);
}

/* ---- Transition without caller-provided scratch -------------------------------------------------
 * Scratch for xfold_transition_static_fwd lives in the library image itself: one array per GPU that
 * loads the library, kept until the process exits.  XFOLD_STATIC_SCRATCH_BYTES is its (fixed) size. */
#define XFOLD_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[XFOLD_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[64] = {nullptr};  // device address of the array, per device ordinal

size_t xfold_transition_static_max_bytes(void) { return XFOLD_STATIC_SCRATCH_BYTES; }

int xfold_transition_static_fwd(xfold_ctx* c, void* x, long long rows, int C, int F, const xfold_transition_weights* w,
                                void* stream) {
  if (!c) return XFOLD_ERR_ARG;
  if (rows < 0 || C <= 0 || F <= 0 || rows >= (1ll << 31))
    return fail(c, XFOLD_ERR_ARG, "transition (static scratch): bad shape (%lld rows, C=%d, F=%d)", rows, C, F);
  const size_t need = xfold_transition_workspace_bytes(rows, C, F);
  if (need > XFOLD_STATIC_SCRATCH_BYTES)
    return fail(c, XFOLD_ERR_ARG,
                "transition (static scratch): %lld rows x (C=%d + F=%d) need %zu bytes of scratch, the built-in "
                "array holds %u; use xfold_transition_fwd with a caller-provided workspace",
                rows, C, F, need, (unsigned)XFOLD_STATIC_SCRATCH_BYTES);
  if (c->device < 0 || c->device >= 64) return fail(c, XFOLD_ERR_ARG, "transition (static scratch): device ordinal out of range");
  if (!g_static_scratch_addr[c->device]) {
    // first call on this device: resolve the device address of the array.  In host code the symbol
    // g_static_scratch is only a handle, so it is never passed to a kernel directly.
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != c->device)
      return fail(c, XFOLD_ERR_DEVICE, "transition (static scratch): device %d must be current (current: %d)", c->device, cur);
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return fail(c, XFOLD_ERR_DEVICE, "transition (static scratch): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_static_scratch_addr[c->device] = p;
  }
  const int prof = c->prof_on;  // event pairs are created on demand by the profiler: keep this path free of that
  c->prof_on = 0;
  const int rc = transition_fwd(c, (bf16*)x, rows, C, F, w, g_static_scratch_addr[c->device], XFOLD_STATIC_SCRATCH_BYTES,
                                (cudaStream_t)stream);
  c->prof_on = prof;
  return rc;
}

}  // extern "C"
