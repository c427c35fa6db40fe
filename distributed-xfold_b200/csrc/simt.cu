// Bandwidth-bound kernels: LayerNorm over rows (optionally with a small fused projection that
// produces the attention pair bias), LayerNorm of a channel-major tensor with a transposing
// write-back, and the element-wise pieces of the diffusion transformer (AdaLN modulation, gates).
// One warp per row, 8-byte vector accesses, fp32 statistics, warp-shuffle reductions.
#include <cuda_fp16.h>

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
// proj_bf16 (instead of proj) is the attention kernel's pair-bias operand: 16-bit, holding FP16 values (the buffer
// is only typed bf16) multiplied by log2(e), because the head-dim-32 attention kernel exponentiates in base 2 and adds
// the bias tile, as it is, to fp16x2 exponent arguments.
// optional modulation: y = sigmoid(scale[row % mod_rows][c]) * y + shift[row % mod_rows][c]  (AdaLN)
// ---------------------------------------------------------------------------------------------
constexpr float kBiasLog2e = 1.4426950408889634f;
// fp16 bit pattern of v * log2(e) in a 16-bit slot of the bias buffer (clamped to the finite fp16 range)
__device__ __forceinline__ bf16 bias16(float v) {
  const __half h = __float2half_rn(fminf(fmaxf(v * kBiasLog2e, -60000.f), 60000.f));
  return *reinterpret_cast<const bf16*>(&h);
}

template <int C, int H>
__global__ void __launch_bounds__(256)
ln_rows_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ y, long long ldy, long long rows,
               const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
               const float* __restrict__ pw, float* __restrict__ proj, long long proj_plane,
               const bf16* __restrict__ mod_scale, const bf16* __restrict__ mod_shift, int mod_rows,
               bf16* __restrict__ proj_bf16, int trav_inner, int trav_outer, int proj_pitch) {
  constexpr int V = C / 128;  // uint2 (4 x bf16) vectors per lane
  // rows a warp keeps in flight at once: the loads of all of them are issued before any is reduced
  constexpr int RPW = (H == 0) ? (C == 128 ? 4 : 2) : (H == 4 ? 2 : 1);
  const int lane = threadIdx.x & 31;
  const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long base = warp_global; base < rows; base += nwarps * RPW) {
    uint2 raw[RPW][V];
    long long srow[RPW], pidx[RPW];
    bool valid[RPW];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
      const long long prow = base + (long long)j * nwarps;
      valid[j] = prow < rows;
      // transposed traversal: projection index (y, x) = (prow / inner, prow % inner) reads source row x * outer + y
      // trav_inner < 0: plain walk, but the projection rows (of -trav_inner entries) have pitch proj_pitch
      const long long inner = trav_inner > 0 ? trav_inner : -trav_inner;
      srow[j] = trav_inner > 0 ? (prow % inner) * trav_outer + prow / inner : prow;
      pidx[j] = trav_inner != 0 ? (prow / inner) * proj_pitch + prow % inner : prow;
      if (valid[j]) {
        const uint2* xr = reinterpret_cast<const uint2*>(x + srow[j] * ldx);
#pragma unroll
        for (int k = 0; k < V; ++k) raw[j][k] = xr[lane + 32 * k];
      }
    }
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
      if (!valid[j]) continue;
      const long long row = srow[j];
      float v[V][4];
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const uint2 u = raw[j][k];
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
          acc[h] = a;
        }
        if constexpr (H == 16) {
          // recursive halving over lane bits 4..1: a lane ends with the sum of head (lane >> 1) & 15 over the
          // 16 lanes that share its bit 0; one more exchange over bit 0 completes it
#pragma unroll
          for (int step = 0; step < 4; ++step) {
            const int off = 16 >> step, n = 8 >> step;
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < n; ++i) {
              const float send = upper ? acc[i] : acc[i + n];
              const float keep = upper ? acc[i + n] : acc[i];
              acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
          }
          const float tot = acc[0] + __shfl_xor_sync(0xffffffffu, acc[0], 1);
          const int h = (lane >> 1) & 15;
          if ((lane & 1) == 0) {
            if (proj_bf16) proj_bf16[(long long)h * proj_plane + pidx[j]] = bias16(tot);
            else proj[(long long)h * proj_plane + pidx[j]] = tot;
          }
        } else {
#pragma unroll
          for (int h = 0; h < H; ++h) acc[h] = warp_sum(acc[h]);
#pragma unroll
          for (int h = 0; h < H; ++h)
            if (lane == (h & 31)) {
              if (proj_bf16) proj_bf16[(long long)h * proj_plane + pidx[j]] = bias16(acc[h]);
              else proj[(long long)h * proj_plane + pidx[j]] = acc[h];
            }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Width-128 LayerNorm (the pair representation: ~1M rows per call at N = 1024).  Sixteen lanes share
// a row (one 16-byte load each, so a warp moves two rows per request), gamma / beta live in
// registers, the reductions take 4 shuffles, and SLOTS row pairs are in flight per warp.
// Same arguments and semantics as ln_rows_kernel.
// ---------------------------------------------------------------------------------------------
template <int H>
__global__ void __launch_bounds__(256, 3)
ln128_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ y, long long ldy, long long rows,
             const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
             const float* __restrict__ pw, float* __restrict__ proj, long long proj_plane,
             const bf16* __restrict__ mod_scale, const bf16* __restrict__ mod_shift, int mod_rows,
             bf16* __restrict__ proj_bf16, int trav_inner, int trav_outer, int proj_pitch) {
  // dynamic shared memory: H x 128 projection weights, then two tiles of 128 rows x 256 B.  The tile of the next
  // iteration is fetched with cp.async while the current one is processed, so loads stay in flight all the time.
  extern __shared__ __align__(16) float s_pw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>(s_pw + H * 128);
  if constexpr (H > 0) {
    // stored as [head][half][lane16][4] so that the 16 lanes of a row read consecutive 16-byte words
    for (int i = threadIdx.x; i < H * 128; i += blockDim.x) {
      const int h = i >> 7, c = i & 127;
      s_pw[((h * 2 + ((c >> 2) & 1)) * 16 + (c >> 3)) * 4 + (c & 3)] = pw[i];
    }
  }
  const int lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15, warp = threadIdx.x >> 5;
  const int c0 = l16 * 8;
  float gm[8], bt[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    gm[e] = gamma ? gamma[c0 + e] : 1.f;
    bt[e] = beta ? beta[c0 + e] : 0.f;
  }
  // transposed traversal: projection index (y, x) = (prow / inner, prow % inner) reads source row x * outer + y
  // trav_inner < 0: plain walk, but the projection rows (of -trav_inner entries) have pitch proj_pitch
  const long long inner = trav_inner > 0 ? trav_inner : -trav_inner;
  auto srow_of = [&](long long prow) { return trav_inner > 0 ? (prow % inner) * trav_outer + prow / inner : prow; };
  auto pidx_of = [&](long long prow) { return trav_inner != 0 ? (prow / inner) * proj_pitch + prow % inner : prow; };
  const long long ntiles = (rows + 127) / 128;
  auto fetch = [&](long long t, int buf) {
    for (int idx = threadIdx.x; idx < 128 * 16; idx += 256) {
      const long long prow = t * 128 + (idx >> 4);
      if (prow < rows)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                     ::"r"(smem_u32(tiles + buf * 32768 + idx * 16)), "l"(x + srow_of(prow) * ldx + (idx & 15) * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  int buf = 0;
  if ((long long)blockIdx.x < ntiles) fetch(blockIdx.x, 0);
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x, buf ^= 1) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // tile t is complete; every thread is done with the other buffer (and s_pw is filled)
    if (t + gridDim.x < ntiles) fetch(t + gridDim.x, buf ^ 1);
    constexpr int UNR = (H >= 16) ? 1 : 2;  // the wide projections hold 16 accumulators per row
#pragma unroll UNR
    for (int it = 0; it < 8; ++it) {
      const int r = warp * 16 + it * 2 + half;
      const long long prow_j = t * 128 + r;
      const bool valid_j = prow_j < rows;
      const long long srow_j = srow_of(prow_j);
      uint4 rawv = make_uint4(0, 0, 0, 0);
      if (valid_j) rawv = *reinterpret_cast<const uint4*>(tiles + buf * 32768 + r * 256 + l16 * 16);
      const uint32_t w4[4] = {rawv.x, rawv.y, rawv.z, rawv.w};
      // The kernel is bound by instruction issue, so the bf16 values are never unpacked: mixed-precision adds take the
      // packed halves as they are, once for the row sum and once to produce the centred fp32 values.
      float v[8];
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %1, hi, %1;\n\t}"
            : "+f"(s0), "+f"(s1) : "r"(w4[e]));
      float s = s0 + s1;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s * (1.f / 128);
      const float nmean = -mean;
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %3;\n\tadd.rn.f32.bf16 %1, hi, %3;\n\t}"
            : "=f"(v[2 * e]), "=f"(v[2 * e + 1]) : "r"(w4[e]), "f"(nmean));
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss * (1.f / 128) + eps);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = fmaf(v[e] * rstd, gm[e], bt[e]);
      if (mod_scale && valid_j) {
        const long long mr = srow_j % mod_rows;
        const uint4 a = *reinterpret_cast<const uint4*>(mod_scale + mr * 128 + c0);
        const uint4 b = *reinterpret_cast<const uint4*>(mod_shift + mr * 128 + c0);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] = sigmoidf_fast(bf16_lo(aw[e])) * v[2 * e] + bf16_lo(bw[e]);
          v[2 * e + 1] = sigmoidf_fast(bf16_hi(aw[e])) * v[2 * e + 1] + bf16_hi(bw[e]);
        }
      }
      if (y && valid_j) {
        uint4 u;
        u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
        u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(y + srow_j * ldy + c0) = u;
      }
      if constexpr (H > 0) {
#pragma unroll
        for (int hb = 0; hb < H; hb += 16) {
          constexpr int G = (H < 16) ? H : 16;  // heads reduced together over the 16 lanes of a row
          float acc[G];
#pragma unroll
          for (int h = 0; h < G; ++h) {
            const float4 w0 = *reinterpret_cast<const float4*>(s_pw + (((hb + h) * 2 + 0) * 16 + l16) * 4);
            const float4 w1 = *reinterpret_cast<const float4*>(s_pw + (((hb + h) * 2 + 1) * 16 + l16) * 4);
            acc[h] = v[0] * w0.x + v[1] * w0.y + v[2] * w0.z + v[3] * w0.w + v[4] * w1.x + v[5] * w1.y + v[6] * w1.z +
                     v[7] * w1.w;
          }
          // recursive halving over lane bits 3..0: the lane keeps the half of the heads its bit selects
          int nkeep = G;
#pragma unroll
          for (int off = 8; off > 0; off >>= 1) {
            if (nkeep > 1) {
              nkeep >>= 1;
              const bool upper = (l16 & off) != 0;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (i < nkeep) {
                  const float send = upper ? acc[i] : acc[i + nkeep];
                  const float keep = upper ? acc[i + nkeep] : acc[i];
                  acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
              }
            } else {
              acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], off);
            }
          }
          // G = 16: head = l16 (bits 3..0 each picked a half); G = 4: head = l16 >> 2, shared by 4 lanes
          const int hsel = (G == 16) ? (((l16 >> 3) & 1) * 8 + ((l16 >> 2) & 1) * 4 + ((l16 >> 1) & 1) * 2 + (l16 & 1))
                                     : (((l16 >> 3) & 1) * 2 + ((l16 >> 2) & 1));
          const bool writer = (G == 16) ? true : ((l16 & 3) == 0);
          if (writer && valid_j) {
            const long long o = (long long)(hb + hsel) * proj_plane + pidx_of(prow_j);
            if (proj_bf16) proj_bf16[o] = bias16(acc[0]);
            else proj[o] = acc[0];
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// LayerNorm of 128-wide rows with the 4- or 16-head pair-bias projection on the tensor core.
//
// The projection on the CUDA cores costs 32 (4 heads) or 128 (16 heads) FMAs per lane and row and made those launches
// 2x / 4.5x as long as the plain LayerNorm.  Here the tile of 128 RAW rows that cp.async stages in shared memory is
// laid out as the K-major, 128-byte-swizzled A operand of tcgen05.mma, and one 128 x 16 x 128 product per tile
//     D[row][h] = sum_c x[row][c] * w'[h][c],      w'[h][c] = bf16(w[h][c] * gamma[c])
// gives the un-normalised dot products; the LayerNorm enters through the row statistics the warps compute anyway:
//     proj[h][row] = rstd * (D - mean * colsum[h]) + colbias[h],  colsum[h] = sum_c w'[h][c],  colbias[h] = sum_c beta[c] w[h][c]
// (colsum from the rounded w', so a constant row cancels exactly).  The output is the attention kernel's bf16
// operand (times log2 e); y (the normalised rows) is written when asked for.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t LNTC_TILE = 32768;  // 128 rows x 256 B: two swizzled halves of 64 channels
constexpr uint32_t LNTC_OFF_W = 2 * LNTC_TILE, LNTC_OFF_MISC = LNTC_OFF_W + 4096;
constexpr uint32_t LNTC_SMEM = LNTC_OFF_MISC + 2048 + 1024;

template <int H>
__global__ void __launch_bounds__(256, 3)
ln128_tc_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ y, long long ldy, long long rows,
                const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                const float* __restrict__ pw, long long proj_plane, bf16* __restrict__ proj_bf16, int trav_inner,
                int trav_outer, int proj_pitch, int* status) {
  extern __shared__ uint8_t lntc_raw[];
  const uint32_t raw_addr = smem_u32(lntc_raw);
  uint8_t* smem = lntc_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sW = smem + LNTC_OFF_W;                                     // [2 halves][16 heads][128 B], swizzled
  float* colsum = reinterpret_cast<float*>(smem + LNTC_OFF_MISC);      // [16]
  float* colbias = colsum + 16;                                        // [16]
  float2* rstat = reinterpret_cast<float2*>(smem + LNTC_OFF_MISC + 128);  // [128] (mean, rstd) of the tile's rows
  uint64_t* mma_bar = reinterpret_cast<uint64_t*>(smem + LNTC_OFF_MISC + 128 + 1024);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 1);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15, warp = threadIdx.x >> 5;
  const AbortCtx ab{cta_abort, status};

  // folded weights: one head per half-warp pass
  for (int h = warp * 2 + half; h < 16; h += 16) {
    float s = 0.f, b = 0.f;
    uint32_t packed[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float w2[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = l16 * 8 + e * 2 + u;
        const float w = h < H ? pw[h * 128 + c] : 0.f;
        const bf16 wf = __float2bfloat16(w * (gamma ? gamma[c] : 1.f));
        w2[u] = __bfloat162float(wf);
        s += w2[u];
        b += (beta ? beta[c] : 0.f) * w;
      }
      packed[e] = pack_bf16x2(w2[0], w2[1]);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    // channels l16*8 .. +7 = 16-byte chunk (l16 & 7) of half (l16 >> 3) in row h
    *reinterpret_cast<uint4*>(sW + (l16 >> 3) * 2048 + h * 128 + ((uint32_t(l16 & 7) ^ uint32_t(h & 7)) << 4)) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
    if (l16 == 0) {
      colsum[h] = s;
      colbias[h] = b;
    }
  }
  if (threadIdx.x == 0) {
    mbar_init(mma_bar, 1);
    *cta_abort = 0;
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(tmem_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int c0 = l16 * 8;
  float gm[8], bt[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    gm[e] = gamma ? gamma[c0 + e] : 1.f;
    bt[e] = beta ? beta[c0 + e] : 0.f;
  }
  const long long inner = trav_inner > 0 ? trav_inner : -trav_inner;
  auto srow_of = [&](long long prow) { return trav_inner > 0 ? (prow % inner) * trav_outer + prow / inner : prow; };
  auto pidx_of = [&](long long prow) { return trav_inner != 0 ? (prow / inner) * proj_pitch + prow % inner : prow; };
  const long long ntiles = (rows + 127) / 128;
  // 16-byte piece w (0..15) of row r: half w >> 3, chunk (w & 7) ^ (r & 7) of the 128-byte swizzled row
  auto piece = [&](int buf, int r, int w) {
    return smem + buf * LNTC_TILE + (w >> 3) * 16384 + r * 128 + ((uint32_t(w & 7) ^ uint32_t(r & 7)) << 4);
  };
  auto fetch = [&](long long t, int buf) {
    for (int idx = threadIdx.x; idx < 128 * 16; idx += 256) {
      const int r = idx >> 4, w = idx & 15;
      const long long prow = t * 128 + r;
      if (prow < rows)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                     ::"r"(smem_u32(piece(buf, r, w))), "l"(x + srow_of(prow) * ldx + w * 8) : "memory");
      else
        *reinterpret_cast<uint4*>(piece(buf, r, w)) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  constexpr uint32_t idesc = make_idesc(128, 16);
  int buf = 0;
  uint32_t iter = 0;
  if ((long long)blockIdx.x < ntiles) fetch(blockIdx.x, 0);
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x, buf ^= 1, ++iter) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    fence_proxy_async_smem();  // the tile was written through the generic proxy; the tensor core reads it through the async one
    __syncthreads();           // tile t complete; all reads of the accumulator and of the other buffer are over
    if (threadIdx.x == 0) {
      tc_fence_after();
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const uint64_t ad = make_sdesc(smem_u32(smem + buf * LNTC_TILE + hf * 16384), 16, 1024);
        const uint64_t bd = make_sdesc(smem_u32(sW + hf * 2048), 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_ss(tmem_base, ad + 2 * k, bd + 2 * k, idesc, (hf | k) ? 1u : 0u);
      }
      umma_commit(mma_bar);
    }
    if (t + gridDim.x < ntiles) fetch(t + gridDim.x, buf ^ 1);
    // row statistics (and the normalised rows, when asked for) while the product runs
    constexpr int UNR = 2;
#pragma unroll UNR
    for (int it = 0; it < 8; ++it) {
      const int r = warp * 16 + it * 2 + half;
      const long long prow = t * 128 + r;
      const bool valid = prow < rows;
      const uint4 rawv = *reinterpret_cast<const uint4*>(piece(buf, r, l16));
      const uint32_t w4[4] = {rawv.x, rawv.y, rawv.z, rawv.w};
      float v[8];
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %1, hi, %1;\n\t}"
            : "+f"(s0), "+f"(s1) : "r"(w4[e]));
      float sm = s0 + s1;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
      const float mean = sm * (1.f / 128);
      const float nmean = -mean;
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %3;\n\tadd.rn.f32.bf16 %1, hi, %3;\n\t}"
            : "=f"(v[2 * e]), "=f"(v[2 * e + 1]) : "r"(w4[e]), "f"(nmean));
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss * (1.f / 128) + eps);
      if (l16 == 0) rstat[r] = make_float2(mean, rstd);
      if (y && valid) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = fmaf(v[e] * rstd, gm[e], bt[e]);
        uint4 u;
        u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
        u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(y + srow_of(prow) * ldy + c0) = u;
      }
    }
    __syncthreads();  // statistics of all 128 rows are in shared memory
    const bool okay = mbar_wait(mma_bar, iter & 1u, ab, XF_ERR_WAIT_TMEM_FULL);
    if (okay) {
      tc_fence_after();
      // warp w reads TMEM lanes 32 * (w & 3) ..: row = that lane; warps 0-3 take heads 0-7, warps 4-7 heads 8-15
      const int q = warp & 3, hsel = warp >> 2;
      if (hsel * 8 < H) {
        uint32_t d[8];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7])
                     : "r"(tmem_base + hsel * 8 + (uint32_t(q * 32) << 16))
                     : "memory");
        tmem_ld_wait();
        const int row = q * 32 + lane;
        const long long prow = t * 128 + row;
        if (prow < rows) {
          const float2 st = rstat[row];
          const long long o = pidx_of(prow);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int h = hsel * 8 + j;
            if (h < H) {
              const float val = fmaf(st.y, __uint_as_float(d[j]) - st.x * colsum[h], colbias[h]);
              proj_bf16[(long long)h * proj_plane + o] = bias16(val);
            }
          }
        }
      }
      tc_fence_before();
    }
    if (__syncthreads_or(!okay)) break;  // a bounded wait ran out: every thread leaves together
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

template <int H>
static int launch_ln128_tc(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, const float* g,
                           const float* b, float eps, const float* pw, long long plane, bf16* pbf, int tin, int tout,
                           int tpitch, cudaStream_t st) {
  long long blocks = (rows + 127) / 128;
  const long long cap = (long long)c->sm_count * 3;
  if (blocks > cap) blocks = cap;
  if (blocks <= 0) return XFOLD_OK;
  static bool attr_done[8] = {false};
  if (!attr_done[c->device & 7]) {
    cudaError_t e = cudaFuncSetAttribute(ln128_tc_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LNTC_SMEM);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "layernorm smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  ProfScope ps(c, XFOLD_K_LAYERNORM, st);
  ln128_tc_kernel<H><<<(int)blocks, 256, LNTC_SMEM, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, plane, pbf, tin, tout, tpitch,
                                                          c->d_status);
  return check_launch(c, "ln128_tc_kernel");
}

static int launch_ln128(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, const float* g,
                        const float* b, float eps, int H, const float* pw, float* proj, long long plane,
                        const bf16* msc, const bf16* msh, int mod_rows, bf16* pbf, int tin, int tout, int tpitch,
                        cudaStream_t st) {
  if ((ldx & 7) || (ldy & 7)) return fail(c, XFOLD_ERR_ARG, "layernorm(128): row strides must be multiples of 8 elements");
  if ((H == 4 || H == 16) && pbf && !proj && !msc) {  // the attention pair-bias operand: projection on the tensor core
    if (H == 4) return launch_ln128_tc<4>(c, x, ldx, y, ldy, rows, g, b, eps, pw, plane, pbf, tin, tout, tpitch, st);
    return launch_ln128_tc<16>(c, x, ldx, y, ldy, rows, g, b, eps, pw, plane, pbf, tin, tout, tpitch, st);
  }
  long long blocks = (rows + 127) / 128;  // tiles of 128 rows
  const long long cap = (long long)c->sm_count * (H <= 16 ? 3 : 2);  // one wave of resident CTAs: the loop is grid-strided
  if (blocks > cap) blocks = cap;
  if (blocks <= 0) return XFOLD_OK;
  const size_t sm = (size_t)H * 128 * sizeof(float) + 2 * 32768;
  {
    static bool attr_done[8][4] = {};
    const int hi = H == 0 ? 0 : H == 4 ? 1 : H == 16 ? 2 : 3;
    if (!attr_done[c->device & 7][hi]) {
      cudaError_t e = cudaSuccess;
      switch (H) {
        case 0: e = cudaFuncSetAttribute(ln128_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); break;
        case 4: e = cudaFuncSetAttribute(ln128_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); break;
        case 16: e = cudaFuncSetAttribute(ln128_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); break;
        case 64: e = cudaFuncSetAttribute(ln128_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); break;
        default: break;
      }
      if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "layernorm smem attribute: %s", cudaGetErrorString(e));
      attr_done[c->device & 7][hi] = true;
    }
  }
  ProfScope ps(c, XFOLD_K_LAYERNORM, st);
  switch (H) {
    case 0: ln128_kernel<0><<<(int)blocks, 256, sm, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    case 4: ln128_kernel<4><<<(int)blocks, 256, sm, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    case 16: ln128_kernel<16><<<(int)blocks, 256, sm, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    case 64: ln128_kernel<64><<<(int)blocks, 256, sm, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    default: return fail(c, XFOLD_ERR_ARG, "layernorm: fused projection supports 0, 4, 16 or 64 outputs, got %d", H);
  }
  return check_launch(c, "ln128_kernel");
}

template <int C>
static int launch_ln_c(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, const float* g,
                       const float* b, float eps, int H, const float* pw, float* proj, long long plane,
                       const bf16* msc, const bf16* msh, int mod_rows, bf16* pbf, int tin, int tout, int tpitch, cudaStream_t st) {
  const int wpb = 8;
  long long blocks = (rows + wpb - 1) / wpb;
  const long long cap = (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks <= 0) return XFOLD_OK;
  ProfScope ps(c, XFOLD_K_LAYERNORM, st);
  switch (H) {
    case 0: ln_rows_kernel<C, 0><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    case 4: ln_rows_kernel<C, 4><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    case 16: ln_rows_kernel<C, 16><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    case 64: ln_rows_kernel<C, 64><<<(int)blocks, 256, 0, st>>>(x, ldx, y, ldy, rows, g, b, eps, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch); break;
    default: return fail(c, XFOLD_ERR_ARG, "layernorm: fused projection supports 0, 4, 16 or 64 outputs, got %d", H);
  }
  return check_launch(c, "ln_rows_kernel");
}

int launch_ln_rows(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, int C, const float* g,
                   const float* b, float eps, int H, const float* pw, float* proj, long long plane, const bf16* msc,
                   const bf16* msh, int mod_rows, cudaStream_t st, bf16* pbf, int tin, int tout, int tpitch) {
  if ((ldx & 3) || (ldy & 3)) return fail(c, XFOLD_ERR_ARG, "layernorm: row strides must be multiples of 4 elements");
  switch (C) {
    case 128:
      if (((ldx | ldy) & 7) == 0)
        return launch_ln128(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch, st);
      return launch_ln_c<128>(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch, st);
    case 384: return launch_ln_c<384>(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch, st);
    case 768: return launch_ln_c<768>(c, x, ldx, y, ldy, rows, g, b, eps, H, pw, proj, plane, msc, msh, mod_rows, pbf, tin, tout, tpitch, st);
  }
  return fail(c, XFOLD_ERR_ARG, "layernorm: unsupported width %d (128, 384, 768)", C);
}

// ---------------------------------------------------------------------------------------------
// Channel-major -> token-major LayerNorm: in [128][R][ld] bf16, out [R*N][128] bf16.
// A block stages 128 channels x 64 tokens in shared memory (rows padded to 66 elements so that
// the per-token reads below are bank-conflict free), 4 threads share a token.
// ---------------------------------------------------------------------------------------------
constexpr int CMLN_TOK = 128;
constexpr int CMLN_PITCH = CMLN_TOK + 8;  // elements; keeps every row 16-byte aligned
constexpr size_t CMLN_TILE_BYTES = (size_t)128 * CMLN_PITCH * sizeof(bf16);
constexpr size_t CMLN_SMEM = 2 * CMLN_TILE_BYTES + 2 * 4 * CMLN_TOK * sizeof(float);

// The tile of the NEXT iteration is fetched with cp.async (global -> shared without passing through registers) while
// the current one is normalised and stored, so loads stay in flight through the compute and store phases.
__global__ void __launch_bounds__(256, 3)
cm_ln_kernel(const bf16* __restrict__ in, long long chan_stride, long long row_stride, int R, int N,
             bf16* __restrict__ out, const float* __restrict__ gamma, const float* __restrict__ beta, float eps) {
  extern __shared__ __align__(16) uint8_t cmln_smem[];
  bf16 (*tiles)[128][CMLN_PITCH] = reinterpret_cast<bf16 (*)[128][CMLN_PITCH]>(cmln_smem);
  float (*psum)[CMLN_TOK] = reinterpret_cast<float (*)[CMLN_TOK]>(cmln_smem + 2 * CMLN_TILE_BYTES);
  float (*psq)[CMLN_TOK] = psum + 4;
  const int tiles_j = (N + CMLN_TOK - 1) / CMLN_TOK;
  const long long ntiles = (long long)R * tiles_j;
  const bool vec_ok = ((chan_stride | row_stride) & 7) == 0;
  // 128 channel rows x 128 tokens: 16 x 16-byte pieces per row
  auto fetch = [&](long long t, int buf) {
    const int i = int(t / tiles_j);
    const int j0 = int(t % tiles_j) * CMLN_TOK;
    for (int idx = threadIdx.x; idx < 128 * 16; idx += 256) {
      const int ch = idx >> 4, w = idx & 15;
      const int j = j0 + 8 * w;
      const bf16* src = in + ch * chan_stride + (long long)i * row_stride + j;
      bf16* dst = &tiles[buf][ch][8 * w];
      if (vec_ok && j + 7 < N) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
      } else {
        bf16 tmp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = (j + e < N) ? src[e] : __float2bfloat16(0.f);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(tmp);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  int buf = 0;
  if ((long long)blockIdx.x < ntiles) fetch(blockIdx.x, 0);
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x, buf ^= 1) {
    const int i = int(t / tiles_j);
    const int j0 = int(t % tiles_j) * CMLN_TOK;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // tile t has landed for every thread; everybody is done with the other buffer and with psum
    if (t + gridDim.x < ntiles) fetch(t + gridDim.x, buf ^ 1);
    bf16 (*tile)[CMLN_PITCH] = tiles[buf];
    // thread = (token pair tp, quarter of the channels): a warp reads 32 consecutive 4-byte words per channel row
    const int tp = threadIdx.x & 63, part = threadIdx.x >> 6;
    float v0[32], v1[32];
    float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const uint32_t u = *reinterpret_cast<const uint32_t*>(&tile[part * 32 + e][2 * tp]);
      v0[e] = bf16_lo(u);
      v1[e] = bf16_hi(u);
      s0 += v0[e]; s1 += v1[e];
      q0 += v0[e] * v0[e]; q1 += v1[e] * v1[e];
    }
    psum[part][2 * tp] = s0; psum[part][2 * tp + 1] = s1;
    psq[part][2 * tp] = q0; psq[part][2 * tp + 1] = q1;
    __syncthreads();
    float mean[2], rstd[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int tk = 2 * tp + u;
      const float sm = psum[0][tk] + psum[1][tk] + psum[2][tk] + psum[3][tk];
      const float sq = psq[0][tk] + psq[1][tk] + psq[2][tk] + psq[3][tk];
      mean[u] = sm * (1.f / 128);
      rstd[u] = rsqrtf(fmaxf(sq * (1.f / 128) - mean[u] * mean[u], 0.f) + eps);
    }
    // Every thread holds its values in registers and the statistics are exchanged: the tile's buffer is free.  The
    // normalised tokens are staged there token-major, so that they leave as whole 256-byte rows (a thread's own 2 x 64
    // bytes written straight to global memory use half of every 128-byte line they touch).
    bf16 (*stage)[CMLN_PITCH] = tile;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      bf16* srow = &stage[2 * tp + u][part * 32];
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int ch = part * 32 + g8 * 8 + e;
          float tv = ((u ? v1[g8 * 8 + e] : v0[g8 * 8 + e]) - mean[u]) * rstd[u];
          if (gamma) tv *= gamma[ch];
          if (beta) tv += beta[ch];
          o[e] = tv;
        }
        uint4 w4;
        w4.x = pack_bf16x2(o[0], o[1]); w4.y = pack_bf16x2(o[2], o[3]);
        w4.z = pack_bf16x2(o[4], o[5]); w4.w = pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(srow + g8 * 8) = w4;
      }
    }
    __syncthreads();
    // 128 tokens x 16 pieces of 16 bytes: a warp writes two whole token rows per instruction
    for (int idx = threadIdx.x; idx < CMLN_TOK * 16; idx += 256) {
      const int tk = idx >> 4, piece = idx & 15;
      const int j = j0 + tk;
      if (j < N)
        *reinterpret_cast<uint4*>(out + ((long long)i * N + j) * 128 + piece * 8) =
            *reinterpret_cast<const uint4*>(&stage[tk][piece * 8]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

int launch_cm_ln(Ctx* c, const bf16* in, long long chan_stride, long long row_stride, int R, int N, bf16* out,
                 const float* gamma, const float* beta, float eps, cudaStream_t st) {
  const long long ntiles = (long long)R * ((N + CMLN_TOK - 1) / CMLN_TOK);
  if (ntiles <= 0) return XFOLD_OK;
  long long blocks = ntiles;
  const long long cap = (long long)c->sm_count * 3;  // one wave of resident CTAs (3 per SM): the loop is grid-strided
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_CHANNEL_LN, st);
  static bool attr_done[8] = {false};
  if (!attr_done[c->device & 7]) {
    cudaError_t e = cudaFuncSetAttribute(cm_ln_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CMLN_SMEM);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "channel LayerNorm smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  cm_ln_kernel<<<(int)blocks, 256, CMLN_SMEM, st>>>(in, chan_stride, row_stride, R, N, out, gamma, beta, eps);
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
