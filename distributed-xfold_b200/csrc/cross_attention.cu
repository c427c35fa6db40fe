// Gated cross attention with a per-batch-entry bias: the core of the atom cross-attention encoder / decoder
// (`_alpha_attention::batch_diffusion_cross_attention_forward`, csrc/Alpha_Attention.cpp:127-146, 201-204; spec class
// kernel_test/batch_diffusion_cross_attention.py:23-87).  Queries come from one token set (S per batch entry, 32 atoms
// in the model), keys and values from another (K, 128 atoms), and every batch entry has its own [H][S][K] bias.
//
// The four projections run on the tcgen05 GEMM (query bias and D^-0.5 in its epilogue).  What is left per batch entry is
// a few ten thousand multiply-adds -- at model size 0.5 GFLOP per call against 2 MB of bias to stream -- so the attention
// itself is a bandwidth-shaped CUDA-core kernel: one warp per (batch entry, head, query), lanes over keys, fp32 online
// softmax, the bias read once, coalesced along the key axis.
#include "internal.h"
#include "stages.h"
#include "umma.cuh"

namespace xf {

struct XAttnArgs {
  const bf16* qg;   // [B][S][2*H*D]: scaled queries | gate pre-activations
  const bf16* kv;   // [B][K][2*H*D]: keys | values
  const float* bias;  // [B][H][S][K]
  bf16* out;        // [B][S][H*D]
  int B, S, K, H;
};

template <int D>
__global__ void __launch_bounds__(256) xattn_kernel(XAttnArgs p) {
  const int lane = threadIdx.x & 31;
  const int W = p.H * D;
  const long long total = (long long)p.B * p.H * p.S;
  const long long warps = (long long)gridDim.x * 8;
  for (long long wi = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); wi < total; wi += warps) {
    const int q = int(wi % p.S);
    const int h = int((wi / p.S) % p.H);
    const int b = int(wi / ((long long)p.S * p.H));
    const bf16* qrow = p.qg + ((long long)b * p.S + q) * 2 * W + h * D;
    float qv[D];
#pragma unroll
    for (int d8 = 0; d8 < D / 8; ++d8) {
      const uint4 u = *reinterpret_cast<const uint4*>(qrow + d8 * 8);
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qv[d8 * 8 + 2 * e] = bf16_lo(w4[e]);
        qv[d8 * 8 + 2 * e + 1] = bf16_hi(w4[e]);
      }
    }
    const float* brow = p.bias + (((long long)b * p.H + h) * p.S + q) * p.K;
    float m = -INFINITY, l = 0.f, acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += 32) {
      const int k = k0 + lane;
      const bool kvalid = k < p.K;
      const bf16* krow = p.kv + ((long long)b * p.K + (kvalid ? k : 0)) * 2 * W + h * D;
      float s = -INFINITY;
      if (kvalid) {
        float dot = 0.f;
#pragma unroll
        for (int d8 = 0; d8 < D / 8; ++d8) {
          const uint4 u = *reinterpret_cast<const uint4*>(krow + d8 * 8);
          const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            dot = fmaf(qv[d8 * 8 + 2 * e], bf16_lo(w4[e]), dot);
            dot = fmaf(qv[d8 * 8 + 2 * e + 1], bf16_hi(w4[e]), dot);
          }
        }
        s = dot + brow[k];
      }
      float cm = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
      const float m_new = fmaxf(m, cm);
      const float corr = __expf(m - m_new);
      const float pe = kvalid ? __expf(s - m_new) : 0.f;
      float ps = pe;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l = l * corr + ps;
      m = m_new;
      const bf16* vrow = krow + W;
#pragma unroll
      for (int d8 = 0; d8 < D / 8; ++d8) {
        const uint4 u = *reinterpret_cast<const uint4*>(vrow + d8 * 8);
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[d8 * 8 + 2 * e] = fmaf(pe, bf16_lo(w4[e]), acc[d8 * 8 + 2 * e] * corr);
          acc[d8 * 8 + 2 * e + 1] = fmaf(pe, bf16_hi(w4[e]), acc[d8 * 8 + 2 * e + 1] * corr);
        }
      }
    }
    // sum the lanes' partial outputs (after the butterfly every lane holds the totals); lane i writes elements i and 32 + i
    float o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      float v = acc[d];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if ((d & 31) == lane) {
        if (d < 32) o0 = v;
        else o1 = v;
      }
    }
    const bf16* grow = qrow + W;
    bf16* orow = p.out + ((long long)b * p.S + q) * W + h * D;
    const float inv = 1.f / l;
    if (lane < D) orow[lane] = __float2bfloat16(o0 * inv * sigmoidf_fast(__bfloat162float(grow[lane])));
    if (D > 32) orow[32 + lane] = __float2bfloat16(o1 * inv * sigmoidf_fast(__bfloat162float(grow[32 + lane])));
  }
}

int linear_plain_fwd(Ctx* c, const bf16* x, long long ldx, long long M, int K, const bf16* w, int N, const float* bias,
                     const float* scale, bf16* out, long long ldo, cudaStream_t st);

}  // namespace xf

using namespace xf;

extern "C" {

size_t xfold_cross_attention_workspace_bytes(int B, int S, int K, int H, int D) {
  return align_up((size_t)B * S * 2 * H * D * 2, 1024) + align_up((size_t)B * K * 2 * H * D * 2, 1024) + 2048;
}

int xfold_cross_attention_fwd(xfold_ctx* cx, const void* q_data, const void* m_data, int B, int S, int K, int Ca, int Cm,
                              int H, int D, const void* w_qg, const float* qg_bias, const float* qg_scale, const void* w_kv,
                              const float* bias, void* out, void* ws, size_t ws_bytes, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !q_data || !m_data || !w_qg || !w_kv || !bias || !out) return XFOLD_ERR_ARG;
  if (D != 16 && D != 32 && D != 64) return fail(c, XFOLD_ERR_ARG, "cross attention: head dimension 16, 32 or 64");
  if (B <= 0 || S <= 0 || K <= 0) return XFOLD_OK;
  const int W = H * D;
  Carver cv(ws, ws_bytes);
  bf16* qg = (bf16*)cv.take((size_t)B * S * 2 * W * 2);
  bf16* kv = (bf16*)cv.take((size_t)B * K * 2 * W * 2);
  if (!ws || !cv.ok()) return fail(c, XFOLD_ERR_ARG, "cross attention: workspace too small (%zu < %zu)", ws_bytes, cv.off);
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if ((rc = linear_plain_fwd(c, (const bf16*)q_data, Ca, (long long)B * S, Ca, (const bf16*)w_qg, 2 * W, qg_bias, qg_scale, qg,
                             2 * W, st))) return rc;
  if ((rc = linear_plain_fwd(c, (const bf16*)m_data, Cm, (long long)B * K, Cm, (const bf16*)w_kv, 2 * W, nullptr, nullptr, kv,
                             2 * W, st))) return rc;
  XAttnArgs a{qg, kv, bias, (bf16*)out, B, S, K, H};
  const long long total = (long long)B * H * S;
  long long blocks = (total + 7) / 8;
  if (blocks > (long long)c->sm_count * 32) blocks = (long long)c->sm_count * 32;
  ProfScope ps(c, XFOLD_K_APB_ATTENTION, st);
  if (D == 16) xattn_kernel<16><<<(int)blocks, 256, 0, st>>>(a);
  else if (D == 32) xattn_kernel<32><<<(int)blocks, 256, 0, st>>>(a);
  else xattn_kernel<64><<<(int)blocks, 256, 0, st>>>(a);
  return check_launch(c, "xattn_kernel");
}

}  // extern "C"
