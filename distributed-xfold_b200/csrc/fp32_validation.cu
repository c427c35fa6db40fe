// fp32 validation build of the Pairformer block: float32 storage, float32 arithmetic on the CUDA cores (plain FMA
// products, exact exponentials, no fast-math), the reference's own weight layouts.  It is the counterpart of the
// reference's float32 kernel bodies, which it selects by dtype (csrc/Alpha_Attention.cpp:63-69, 85-91, 162-168;
// triangle_multiplication.h, grid_self_attention.h, transition.h), and exists to hold the path to the 1e-4 the
// float32 configuration is specified to; the bf16 tensor-core kernels are the product.  Nothing here is tuned: one
// generic strided GEMM, one warp per attention row.
#include "internal.h"
#include "stages.h"

namespace xf {
namespace v32 {

// ---------------------------------------------------------------------------------------------------------------
// LayerNorm over rows of C floats (one warp per row)
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ln_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int C,
                                                 const float* __restrict__ gamma, const float* __restrict__ beta, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * 8;
  for (long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += warps) {
    const float* xr = x + r * C;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += xr[c];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / C;
    float v = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float d = xr[c] - mean;
      v += d * d;
    }
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const float rstd = 1.f / sqrtf(v / C + eps);
    for (int c = lane; c < C; c += 32) {
      float t = (xr[c] - mean) * rstd;
      if (gamma) t *= gamma[c];
      if (beta) t += beta[c];
      y[r * C + c] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// out[b][m][n] = (sum_k A[b][m][k] * B[b][n][k] + bias[n]) * scale[n], every operand with explicit strides (elements)
// ---------------------------------------------------------------------------------------------------------------
struct GemmP {
  const float *A, *B;
  float* O;
  long long a_bs, a_rs, a_cs, b_bs, b_rs, b_cs, o_bs, o_rs, o_cs;
  int M, N, K;
  const float *bias, *scale;
};

__global__ void __launch_bounds__(256) gemm_kernel(GemmP p) {
  __shared__ float sa[16][65], sb[16][65];
  const int b = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float* A = p.A + (long long)b * p.a_bs;
  const float* B = p.B + (long long)b * p.b_bs;
  float acc[4][4] = {{0.f}};
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, k = e & 15;
      const bool kv = k0 + k < p.K;
      sa[k][r] = (kv && m0 + r < p.M) ? A[(long long)(m0 + r) * p.a_rs + (long long)(k0 + k) * p.a_cs] : 0.f;
      sb[k][r] = (kv && n0 + r < p.N) ? B[(long long)(n0 + r) * p.b_rs + (long long)(k0 + k) * p.b_cs] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = sa[k][ty * 4 + i];
        bv[i] = sb[k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < p.M && n < p.N) {
        float v = acc[i][j];
        if (p.bias) v += p.bias[n];
        if (p.scale) v *= p.scale[n];
        p.O[(long long)b * p.o_bs + (long long)m * p.o_rs + (long long)n * p.o_cs] = v;
      }
    }
}

static int gemm(Ctx* c, const GemmP& p, int batches, cudaStream_t st) {
  if (p.M <= 0 || p.N <= 0 || batches <= 0) return XFOLD_OK;
  dim3 grid((p.N + 63) / 64, (p.M + 63) / 64, batches);
  if (grid.y > 65535 || grid.z > 65535) return fail(c, XFOLD_ERR_ARG, "fp32 validation: problem too large for this simple kernel");
  c->launch_count++;
  gemm_kernel<<<grid, 256, 0, st>>>(p);
  return check_launch(c, "v32::gemm_kernel");
}

// y[M][N] = x[M][K] w[N][K]^T (+ bias) (* scale), row-major
static int linear(Ctx* c, const float* x, long long M, int K, const float* w, int N, float* y, const float* bias,
                  const float* scale, cudaStream_t st) {
  // grid.y is limited to 65535 tiles of 64 rows: split tall problems
  const long long chunk = 65535ll * 64;
  for (long long m0 = 0; m0 < M; m0 += chunk) {
    GemmP p{};
    p.A = x + m0 * K; p.B = w; p.O = y + m0 * N;
    p.a_rs = K; p.a_cs = 1; p.b_rs = K; p.b_cs = 1; p.o_rs = N; p.o_cs = 1;
    p.M = (int)((M - m0) < chunk ? (M - m0) : chunk); p.N = N; p.K = K;
    p.bias = bias; p.scale = scale;
    const int rc = gemm(c, p, 1, st);
    if (rc) return rc;
  }
  return XFOLD_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// element-wise pieces
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_(float v) { return 1.f / (1.f + expf(-v)); }

// p[m][n] = p[m][n] * mask[m] * sigmoid(g[m][n])     (nn/d_triangle_multiplication.py:155-160)
__global__ void gate_mask_kernel(float* p, const float* g, const float* mask, long long M, int N) {
  const long long n = M * N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / N;
    p[i] = p[i] * (mask ? mask[m] : 1.f) * sigmoid_(g[i]);
  }
}
// z[m][n] += u[m][n] * (gate ? sigmoid(gate[m][n]) : 1)
__global__ void gate_resid_kernel(float* z, const float* u, const float* gate, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    z[i] += u[i] * (gate ? sigmoid_(gate[i]) : 1.f);
}
// h[m][f] = silu(y[m][f]) * y[m][F + f]    (kernel_test/transition.py:40-42)
__global__ void swiglu_kernel(const float* y, float* h, long long M, int F) {
  const long long n = M * F;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / F;
    const int f = int(i - m * F);
    const float a = y[m * 2 * F + f];
    h[i] = a * sigmoid_(a) * y[m * 2 * F + F + f];
  }
}
static int blocks_for(long long n) { long long b = (n + 255) / 256; return (int)(b > 65535 * 4 ? 65535 * 4 : (b < 1 ? 1 : b)); }

// ---------------------------------------------------------------------------------------------------------------
// gated multi-head attention, one warp per (batch row, head, query):
//   out[b][q][h*D + d] = sigmoid(gate) * sum_k softmax_k(q.k + bias[h][q][k] + maskbias[b][k]) v[k][d]
// q is expected pre-scaled; q / k / v / gate are columns of one projection buffer with (batch, seq) strides.
// mask_mode 0: additive 1e9 * (mask - 1) (nn/d_attention.py:63); 1: masked_fill(-1e9) (test_utils/test_grid_attn.py:262-279)
// ---------------------------------------------------------------------------------------------------------------
struct AttnP {
  const float* qkvg;
  long long batch_stride, seq_stride;
  int q_col, k_col, v_col, g_col;
  const float* bias;
  long long bias_h, bias_q, bias_k;
  const float* mask;
  long long mask_ld;
  int mask_mode;
  float* out;
  long long out_batch_stride, out_seq_stride;
  int B, S, H;
};

template <int D>
__global__ void __launch_bounds__(256) attn_kernel(AttnP p) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)p.B * p.H * p.S;
  const long long warps = (long long)gridDim.x * 8;
  for (long long wi = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); wi < total; wi += warps) {
    const int q = int(wi % p.S);
    const int h = int((wi / p.S) % p.H);
    const int b = int(wi / ((long long)p.S * p.H));
    const float* base = p.qkvg + (long long)b * p.batch_stride;
    const float* qrow = base + (long long)q * p.seq_stride + p.q_col + h * D;
    float qv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) qv[d] = qrow[d];
    float m = -INFINITY, l = 0.f, acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int k0 = 0; k0 < p.S; k0 += 32) {
      const int k = k0 + lane;
      float s = -INFINITY;
      const float* vrow = nullptr;
      if (k < p.S) {
        const float* krow = base + (long long)k * p.seq_stride + p.k_col + h * D;
        vrow = base + (long long)k * p.seq_stride + p.v_col + h * D;
        float dot = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d) dot = fmaf(qv[d], krow[d], dot);
        s = dot;
        if (p.bias) s += p.bias[h * p.bias_h + q * p.bias_q + k * p.bias_k];
        if (p.mask) {
          const float mk = p.mask[(long long)b * p.mask_ld + k];
          if (p.mask_mode == 0) s += 1e9f * (mk - 1.f);
          else if (mk == 0.f) s = -1e9f;
        }
      }
      float cm = s;
      for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
      const float m_new = fmaxf(m, cm);
      const float corr = expf(m - m_new);
      const float pe = (k < p.S) ? expf(s - m_new) : 0.f;
      float ps = pe;
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l = l * corr + ps;
      m = m_new;
#pragma unroll
      for (int d = 0; d < D; ++d) acc[d] = acc[d] * corr + (vrow ? pe * vrow[d] : 0.f);
    }
#pragma unroll
    for (int d = 0; d < D; ++d)
      for (int o = 16; o > 0; o >>= 1) acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], o);
    if (lane == 0) {
      const float* grow = base + (long long)q * p.seq_stride + p.g_col + h * D;
      float* orow = p.out + (long long)b * p.out_batch_stride + (long long)q * p.out_seq_stride + h * D;
      for (int d = 0; d < D; ++d) orow[d] = acc[d] / l * sigmoid_(grow[d]);
    }
  }
}

static int attention(Ctx* c, const AttnP& p, int D, cudaStream_t st) {
  const long long total = (long long)p.B * p.H * p.S;
  if (total <= 0) return XFOLD_OK;
  long long blocks = (total + 7) / 8;
  if (blocks > 65535 * 8) blocks = 65535 * 8;
  c->launch_count++;
  if (D == 32) attn_kernel<32><<<(int)blocks, 256, 0, st>>>(p);
  else if (D == 24) attn_kernel<24><<<(int)blocks, 256, 0, st>>>(p);
  else if (D == 48) attn_kernel<48><<<(int)blocks, 256, 0, st>>>(p);
  else return fail(c, XFOLD_ERR_ARG, "fp32 validation: head dimension %d not instantiated", D);
  return check_launch(c, "v32::attn_kernel");
}

static int layernorm(Ctx* c, const float* x, float* y, long long rows, int C, const float* g, const float* b, cudaStream_t st) {
  if (rows <= 0) return XFOLD_OK;
  long long blocks = (rows + 7) / 8;
  if (blocks > 65535 * 4) blocks = 65535 * 4;
  c->launch_count++;
  ln_kernel<<<(int)blocks, 256, 0, st>>>(x, y, rows, C, g, b, 1e-5f);
  return check_launch(c, "v32::ln_kernel");
}

// ---------------------------------------------------------------------------------------------------------------
// operators (the statements of nn/d_triangle_multiplication.py:141-178, nn/d_attention.py:58-111, nn/d_primitives.py:31-38,
// nn/d_diffusion_transformer.py:221-265 and nn/d_pairformer.py:99-171 for world size 1)
// ---------------------------------------------------------------------------------------------------------------
struct Ws {
  float *x, *t0, *t1, *t2;  // x: [N*N][128]; t0, t1: [N*N][256]; t2: [N*N][1024]
};

static int trimul(Ctx* c, float* z, const float* mask, int N, int outgoing, const xfold_trimul_weights_f32* w, const Ws& W,
                  cudaStream_t st) {
  const int C = 128;
  const long long M = (long long)N * N;
  int rc;
  if ((rc = layernorm(c, z, W.x, M, C, w->ln_in_gamma, w->ln_in_beta, st))) return rc;
  if ((rc = linear(c, W.x, M, C, w->projection, 2 * C, W.t0, nullptr, nullptr, st))) return rc;
  if ((rc = linear(c, W.x, M, C, w->gate, 2 * C, W.t1, nullptr, nullptr, st))) return rc;
  c->launch_count++;
  gate_mask_kernel<<<blocks_for(M * 2 * C), 256, 0, st>>>(W.t0, W.t1, mask, M, 2 * C);
  if ((rc = check_launch(c, "v32::gate_mask_kernel"))) return rc;
  // a = even columns, b = odd columns of the gated projection (:162-165); per channel an N x N x N product
  float* o = W.t1;  // [N*N][128]
  GemmP p{};
  p.M = p.N = p.K = N;
  p.O = o; p.o_bs = 1; p.o_rs = (long long)N * C; p.o_cs = C;
  if (outgoing) {  // 'cik,cjk->cij'
    p.A = W.t0;     p.a_bs = 2; p.a_rs = (long long)N * 2 * C; p.a_cs = 2 * C;
    p.B = W.t0 + 1; p.b_bs = 2; p.b_rs = (long long)N * 2 * C; p.b_cs = 2 * C;
  } else {         // 'ckj,cki->cij': out[i][j] = sum_k a[k][j] * b[k][i]
    p.A = W.t0 + 1; p.a_bs = 2; p.a_rs = 2 * C; p.a_cs = (long long)N * 2 * C;
    p.B = W.t0;     p.b_bs = 2; p.b_rs = 2 * C; p.b_cs = (long long)N * 2 * C;
  }
  if ((rc = gemm(c, p, C, st))) return rc;
  float* on = W.t0;  // center_norm(o): [N*N][128]
  if ((rc = layernorm(c, o, on, M, C, w->ln_c_gamma, w->ln_c_beta, st))) return rc;
  float* u = W.t1;
  if ((rc = linear(c, on, M, C, w->output_projection, C, u, nullptr, nullptr, st))) return rc;
  float* gl = W.t0;
  if ((rc = linear(c, W.x, M, C, w->gating_linear, C, gl, nullptr, nullptr, st))) return rc;
  c->launch_count++;
  gate_resid_kernel<<<blocks_for(M * C), 256, 0, st>>>(z, u, gl, M * C);
  return check_launch(c, "v32::gate_resid_kernel");
}

static int triattn(Ctx* c, float* z, const float* mask, int N, int transpose, const xfold_triattn_weights_f32* w, const Ws& W,
                   float* scale512, cudaStream_t st) {
  const int C = 128, H = 4, D = 32;
  const long long M = (long long)N * N;
  int rc;
  if ((rc = layernorm(c, z, W.x, M, C, w->ln_gamma, w->ln_beta, st))) return rc;
  float* nb = W.t0;  // [N*N][4]: bias(h, q, k) = nb[(q*N + k)*4 + h], NOT transposed for the ending node (:62, :99)
  if ((rc = linear(c, W.x, M, C, w->pair_bias_projection, H, nb, nullptr, nullptr, st))) return rc;
  float* qkvg = W.t2;  // [N*N][512]: q (scaled by D^-0.5) | k | v | gate
  if ((rc = linear(c, W.x, M, C, w->qkvg, 4 * C, qkvg, nullptr, scale512, st))) return rc;
  AttnP a{};
  a.qkvg = qkvg;
  a.batch_stride = transpose ? 4 * C : (long long)N * 4 * C;   // transpose: batch index = second token axis (:65-66)
  a.seq_stride = transpose ? (long long)N * 4 * C : 4 * C;
  a.q_col = 0; a.k_col = C; a.v_col = 2 * C; a.g_col = 3 * C;
  a.bias = nb; a.bias_h = 1; a.bias_q = (long long)N * H; a.bias_k = H;
  a.mask = mask; a.mask_ld = N; a.mask_mode = 0;
  float* att = W.t1;  // token-major [N*N][128], written back in the untransposed order (:101-102)
  a.out = att;
  a.out_batch_stride = transpose ? C : (long long)N * C;
  a.out_seq_stride = transpose ? (long long)N * C : C;
  a.B = N; a.S = N; a.H = H;
  if ((rc = attention(c, a, D, st))) return rc;
  float* u = W.t0;
  if ((rc = linear(c, att, M, C, w->output_projection, C, u, nullptr, nullptr, st))) return rc;
  c->launch_count++;
  gate_resid_kernel<<<blocks_for(M * C), 256, 0, st>>>(z, u, nullptr, M * C);
  return check_launch(c, "v32::gate_resid_kernel");
}

// x[rows][C] += transition2(swiglu(transition1(LN(x))))
static int transition(Ctx* c, float* x, long long rows, int C, int F, const xfold_transition_weights_f32* w, float* xn, float* y,
                      float* h, float* u, cudaStream_t st) {
  int rc;
  if ((rc = layernorm(c, x, xn, rows, C, w->ln_gamma, w->ln_beta, st))) return rc;
  if ((rc = linear(c, xn, rows, C, w->transition1, 2 * F, y, nullptr, nullptr, st))) return rc;
  c->launch_count++;
  swiglu_kernel<<<blocks_for(rows * F), 256, 0, st>>>(y, h, rows, F);
  if ((rc = check_launch(c, "v32::swiglu_kernel"))) return rc;
  if ((rc = linear(c, h, rows, F, w->transition2, C, u, nullptr, nullptr, st))) return rc;
  c->launch_count++;
  gate_resid_kernel<<<blocks_for(rows * C), 256, 0, st>>>(x, u, nullptr, rows * C);
  return check_launch(c, "v32::gate_resid_kernel");
}

static size_t ws_floats(int N) {
  const size_t M = (size_t)N * N;
  return M * 128 + 2 * M * 256 + M * 1024 + 512 + 4096 + (size_t)N * (384 * 2 + 4 * 384 + 3072 + 1536 + 384) + 8192;
}

static int block(Ctx* c, float* z, float* s, const float* pair_mask, const float* seq_mask, int N,
                 const xfold_pairformer_weights_f32* w, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!z || !w) return fail(c, XFOLD_ERR_ARG, "fp32 validation: null argument");
  if (ws_bytes < ws_floats(N) * 4 || !ws) return fail(c, XFOLD_ERR_ARG, "fp32 validation: workspace too small (%zu < %zu)", ws_bytes, ws_floats(N) * 4);
  const size_t M = (size_t)N * N;
  float* f = static_cast<float*>(ws);
  Ws W;
  W.x = f; f += M * 128;
  W.t0 = f; f += M * 256;
  W.t1 = f; f += M * 256;
  W.t2 = f; f += M * 1024;
  float* scale512 = f; f += 512;
  // q columns carry D^-0.5 (kernel_test/grid_self_attenion_bf16.py:61-95)
  {
    float h[512];
    for (int i = 0; i < 512; ++i) h[i] = i < 128 ? 0.17677669529663687f : 1.f;
    if (cudaMemcpyAsync(scale512, h, sizeof(h), cudaMemcpyHostToDevice, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)
      return fail(c, XFOLD_ERR_LAUNCH, "fp32 validation: cannot stage the scale vector");
  }
  int rc;
  if ((rc = trimul(c, z, pair_mask, N, 1, &w->tri_out, W, st))) return rc;
  if ((rc = trimul(c, z, pair_mask, N, 0, &w->tri_in, W, st))) return rc;
  if ((rc = triattn(c, z, pair_mask, N, 0, &w->att_start, W, scale512, st))) return rc;
  if ((rc = triattn(c, z, pair_mask, N, 1, &w->att_end, W, scale512, st))) return rc;
  // h [N*N][512] spans t0 and t1 (adjacent); the update lands in x once the normalised rows are used up
  if ((rc = transition(c, z, (long long)M, 128, 512, &w->pair_transition, W.x, W.t2, W.t0, W.x, st))) return rc;
  if (!s || !w->spl_w) return XFOLD_OK;
  // single path (nn/d_pairformer.py:158-169): pair logits [16][N][N] from the updated pair representation
  const int CS = 384, H = 16, D = 24;
  if ((rc = layernorm(c, z, W.x, (long long)M, 128, w->spl_ln_gamma, w->spl_ln_beta, st))) return rc;
  float* pl = W.t0;  // [N*N][16]: logits(h, q, k) = pl[(q*N + k)*16 + h]
  if ((rc = linear(c, W.x, (long long)M, 128, w->spl_w, H, pl, nullptr, nullptr, st))) return rc;
  float* sn = f; f += (size_t)N * CS;
  float* qkvg = f; f += (size_t)N * 4 * CS;
  float* att = f; f += (size_t)N * CS;
  float* y = f; f += (size_t)N * 3072;
  float* hh = f; f += (size_t)N * 1536;
  float* u = f; f += (size_t)N * CS;
  float* sscale = f; f += 4 * CS;
  {
    static float h[4 * 384];
    for (int i = 0; i < 4 * CS; ++i) h[i] = i < CS ? 0.20412414523193148f : 1.f;  // 24^-0.5 on the q columns
    if (cudaMemcpyAsync(sscale, h, sizeof(float) * 4 * CS, cudaMemcpyHostToDevice, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)
      return fail(c, XFOLD_ERR_LAUNCH, "fp32 validation: cannot stage the scale vector");
  }
  if ((rc = layernorm(c, s, sn, N, CS, w->sa_ln_gamma, w->sa_ln_beta, st))) return rc;
  if ((rc = linear(c, sn, N, CS, w->sa_qkvg, 4 * CS, qkvg, w->sa_qkvg_bias, sscale, st))) return rc;
  AttnP a{};
  a.qkvg = qkvg; a.batch_stride = 0; a.seq_stride = 4 * CS;
  a.q_col = 0; a.k_col = CS; a.v_col = 2 * CS; a.g_col = 3 * CS;
  a.bias = pl; a.bias_h = 1; a.bias_q = (long long)N * H; a.bias_k = H;
  a.mask = seq_mask; a.mask_ld = 0; a.mask_mode = 1;
  a.out = att; a.out_batch_stride = 0; a.out_seq_stride = CS;
  a.B = 1; a.S = N; a.H = H;
  if ((rc = attention(c, a, D, st))) return rc;
  if ((rc = linear(c, att, N, CS, w->sa_out, CS, u, nullptr, nullptr, st))) return rc;
  c->launch_count++;
  gate_resid_kernel<<<blocks_for((long long)N * CS), 256, 0, st>>>(s, u, nullptr, (long long)N * CS);
  if ((rc = check_launch(c, "v32::gate_resid_kernel"))) return rc;
  return transition(c, s, N, CS, 1536, &w->single_transition, sn, y, hh, u, st);
}

}  // namespace v32
}  // namespace xf

using namespace xf;

extern "C" {

size_t xfold_pairformer_f32_workspace_bytes(int N) { return N > 0 ? v32::ws_floats(N) * 4 : 0; }

int xfold_pairformer_stack_f32_fwd(xfold_ctx* cx, float* z, float* s, const float* pair_mask, const float* seq_mask, int N,
                                   const xfold_pairformer_weights_f32* blocks, int num_blocks, void* ws, size_t ws_bytes,
                                   void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c) return XFOLD_ERR_ARG;
  if (num_blocks < 0 || (num_blocks > 0 && !blocks)) return fail(c, XFOLD_ERR_ARG, "fp32 validation: no weights for %d blocks", num_blocks);
  if (N <= 0 || N > 2048) return fail(c, XFOLD_ERR_ARG, "fp32 validation: 1 to 2048 tokens");
  for (int i = 0; i < num_blocks; ++i) {
    const int rc = v32::block(c, z, s, pair_mask, seq_mask, N, &blocks[i], ws, ws_bytes, (cudaStream_t)stream);
    if (rc) return rc;
  }
  return XFOLD_OK;
}

}  // extern "C"
