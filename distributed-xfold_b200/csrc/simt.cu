// Bandwidth-bound kernels: LayerNorm over rows (optionally with a small fused projection that
// produces the attention pair bias), LayerNorm of a channel-major tensor with a transposing
// write-back, and the element-wise pieces of the diffusion transformer (AdaLN modulation, gates).
// One warp per row, 8-byte vector accesses, fp32 statistics, warp-shuffle reductions.
#include "internal.h"
#include "umma.cuh"

namespace xf {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------------------
// y = LN(x) * gamma + beta  (gamma/beta may be null), rows of C bf16; optional
// proj[h][row] = sum_c y[c] * pw[h][c]  (fp32, computed from the un-rounded y)
// optional modulation: y = sigmoid(scale[row % mod_rows][c]) * y + shift[row % mod_rows][c]  (AdaLN)
// ---------------------------------------------------------------------------------------------
template <int C, int H>
__global__ void __launch_bounds__(256)
ln_rows_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ y, long long ldy, long long rows,
               const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
               const float* __restrict__ pw, float* __restrict__ proj, long long proj_plane,
               const bf16* __restrict__ mod_scale, const bf16* __restrict__ mod_shift, int mod_rows) {
  constexpr int V = C / 128;  // uint2 (4 x bf16) vectors per lane
  const int lane = threadIdx.x & 31;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long row = warp_global; row < rows; row += nwarps) {
    const uint2* xr = reinterpret_cast<const uint2*>(x + row * ldx);
    float v[V][4];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const uint2 u = xr[lane + 32 * k];
      v[k][0] = bf16_lo(u.x); v[k][1] = bf16_hi(u.x); v[k][2] = bf16_lo(u.y); v[k][3] = bf16_hi(u.y);
      s += v[k][0] + v[k][1] + v[k][2] + v[k][3];
    }
    const float mean = warp_sum(s) * (1.f / C);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < V; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[k][e] -= mean;
        ss += v[k][e] * v[k][e];
      }
    const float rstd = rsqrtf(warp_sum(ss) * (1.f / C) + eps);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int c0 = (lane + 32 * k) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float t = v[k][e] * rstd;
        if (gamma) t *= gamma[c0 + e];
        if (beta) t += beta[c0 + e];
        v[k][e] = t;
      }
    }
    if (mod_scale) {
      const long long mr = row % mod_rows;
      const uint2* sc = reinterpret_cast<const uint2*>(mod_scale + mr * C);
      const uint2* sh = reinterpret_cast<const uint2*>(mod_shift + mr * C);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const uint2 a = sc[lane + 32 * k], b = sh[lane + 32 * k];
        v[k][0] = sigmoidf_fast(bf16_lo(a.x)) * v[k][0] + bf16_lo(b.x);
        v[k][1] = sigmoidf_fast(bf16_hi(a.x)) * v[k][1] + bf16_hi(b.x);
        v[k][2] = sigmoidf_fast(bf16_lo(a.y)) * v[k][2] + bf16_lo(b.y);
        v[k][3] = sigmoidf_fast(bf16_hi(a.y)) * v[k][3] + bf16_hi(b.y);
      }
    }
    if (y) {
      uint2* yr = reinterpret_cast<uint2*>(y + row * ldy);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        uint2 u;
        u.x = pack_bf16x2(v[k][0], v[k][1]);
        u.y = pack_bf16x2(v[k][2], v[k][3]);
        yr[lane + 32 * k] = u;
      }
    }
    if constexpr (H > 0) {
      float acc[H];
#pragma unroll
      for (int h = 0; h < H; ++h) {
        float a = 0.f;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const float4 w = *reinterpret_cast<const float4*>(pw + h * C + (lane + 32 * k) * 4);
          a += v[k][0] * w.x + v[k][1] * w.y + v[k][2] * w.z + v[k][3] * w.w;
        }
        acc[h] = warp_sum(a);
      }
#pragma unroll
      for (int h = 0; h < H; ++h)
        if (lane == h) proj[(long long)h * proj_plane + row] = acc[h];
    }
  }
}

template <int C>
static int launch_ln_c(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, const float* g,
                       const float* b, float eps, int H, const float* pw, float* proj, long long plane,
                       const bf16* msc, const bf16* msh, int mod_rows, cudaStream_t st) {
  const int wpb = 8;
  long long blocks = (rows + wpb - 1) / wpb;
  const long long cap = (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks <= 0) return XFOLD_OK;
  ProfScope ps(c, XFOLD_K_LAYERNORM, st);
  switch (H) {
    case 0: ln_rows_kernel<C, 0><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows); break;
    case 4: ln_rows_kernel<C, 4><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows); break;
    case 16: ln_rows_kernel<C, 16><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows); break;
    case 64: ln_rows_kernel<C, 64><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows); break;
    default: return fail(c, XFOLD_ERR_ARG, "layernorm: fused projection supports 0, 4, 16 or 64 outputs, got %d", H);
  }
  return check_launch(c, "ln_rows_kernel");
}

int launch_ln_rows(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, int C, const float* g,
                   const float* b, float eps, int H, const float* pw, float* proj, long long plane, const bf16* msc,
                   const bf16* msh, int mod_rows, cudaStream_t st) {
  if ((ldx & 3) || (ldy & 3)) return fail(c, XFOLD_ERR_ARG, "layernorm: row strides must be multiples of 4 elements");
  switch (C) {
    case 128: return launch_ln_c<128>(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, st);
    case 384: return launch_ln_c<384>(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, st);
    case 768: return launch_ln_c<768>(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, st);
  }
  return fail(c, XFOLD_ERR_ARG, "layernorm: unsupported width %d (128, 384, 768)", C);
}

// ---------------------------------------------------------------------------------------------
// Channel-major -> token-major LayerNorm: in [128][R][ld] bf16, out [R*N][128] bf16.
// A block stages 128 channels x 64 tokens in shared memory (rows padded to 66 elements so that
// the per-token reads below are bank-conflict free), 4 threads share a token.
// ---------------------------------------------------------------------------------------------
constexpr int CMLN_TOK = 64;
__global__ void __launch_bounds__(256)
cm_ln_kernel(const bf16* __restrict__ in, long long chan_stride, int ld, int R, int N, bf16* __restrict__ out,
             const float* __restrict__ gamma, const float* __restrict__ beta, float eps) {
  __shared__ bf16 tile[128][CMLN_TOK + 2];
  const int tiles_j = (N + CMLN_TOK - 1) / CMLN_TOK;
  const long long ntiles = (long long)R * tiles_j;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int i = int(t / tiles_j);
    const int j0 = int(t % tiles_j) * CMLN_TOK;
    __syncthreads();
    // 128 rows of 64 tokens; a warp reads one channel row as 32 x 4-byte words
    for (int idx = threadIdx.x; idx < 128 * 32; idx += 256) {
      const int ch = idx >> 5, w = idx & 31;
      const int j = j0 + 2 * w;
      uint32_t u = 0;
      const bf16* src = in + ch * chan_stride + (long long)i * ld + j;
      if (j + 1 < N) u = *reinterpret_cast<const uint32_t*>(src);
      else if (j < N) u = uint32_t(*reinterpret_cast<const uint16_t*>(src));
      *reinterpret_cast<uint32_t*>(&tile[ch][2 * w]) = u;
    }
    __syncthreads();
    const int tk = threadIdx.x >> 2, part = threadIdx.x & 3;  // token in tile, quarter of the channels
    float v[32];
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      v[e] = __bfloat162float(tile[part * 32 + e][tk]);
      s += v[e];
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    const float mean = s * (1.f / 128);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      v[e] -= mean;
      ss += v[e] * v[e];
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const float rstd = rsqrtf(ss * (1.f / 128) + eps);
    const int j = j0 + tk;
    if (j < N) {
      bf16* orow = out + ((long long)i * N + j) * 128 + part * 32;
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int ch = part * 32 + g8 * 8 + e;
          float tv = v[g8 * 8 + e] * rstd;
          if (gamma) tv *= gamma[ch];
          if (beta) tv += beta[ch];
          o[e] = tv;
        }
        uint4 u;
        u.x = pack_bf16x2(o[0], o[1]); u.y = pack_bf16x2(o[2], o[3]);
        u.z = pack_bf16x2(o[4], o[5]); u.w = pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(orow + g8 * 8) = u;
      }
    }
  }
}

int launch_cm_ln(Ctx* c, const bf16* in, long long chan_stride, int ld, int R, int N, bf16* out, const float* gamma,
                 const float* beta, float eps, cudaStream_t st) {
  if (ld & 1) return fail(c, XFOLD_ERR_ARG, "cm_ln: leading dimension must be even");
  const long long ntiles = (long long)R * ((N + CMLN_TOK - 1) / CMLN_TOK);
  if (ntiles <= 0) return XFOLD_OK;
  long long blocks = ntiles;
  const long long cap = (long long)c->sm_count * 8;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_CHANNEL_LN, st);
  cm_ln_kernel<<<(int)blocks, 256, 0, st>>>(in, chan_stride, ld, R, N, out, gamma, beta, eps);
  return check_launch(c, "cm_ln_kernel");
}

// ---------------------------------------------------------------------------------------------
// SwiGLU over rows: in [rows][2F] -> out [rows][F] = silu(in[:, :F]) * in[:, F:]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
swiglu_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, long long rows, int F) {
  const long long n8 = rows * (F / 8);
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n8;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / (F / 8);
    const int c8 = int(idx % (F / 8)) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(in + r * 2 * F + c8);
    const uint4 b = *reinterpret_cast<const uint4*>(in + r * 2 * F + F + c8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a0 = bf16_lo(aw[e]), a1 = bf16_hi(aw[e]);
      o[e] = pack_bf16x2(a0 * sigmoidf_fast(a0) * bf16_lo(bw[e]), a1 * sigmoidf_fast(a1) * bf16_hi(bw[e]));
    }
    *reinterpret_cast<uint4*>(out + r * F + c8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int launch_swiglu(Ctx* c, const bf16* in, bf16* out, long long rows, int F, cudaStream_t st) {
  if (F & 7) return fail(c, XFOLD_ERR_ARG, "swiglu: F must be a multiple of 8");
  const long long n8 = rows * (F / 8);
  if (n8 <= 0) return XFOLD_OK;
  long long blocks = (n8 + 255) / 256;
  const long long cap = (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_SWIGLU, st);
  swiglu_kernel<<<(int)blocks, 256, 0, st>>>(in, out, rows, F);
  return check_launch(c, "swiglu_kernel");
}

}  // namespace xf
