// Second-generation gated attention for head dim 32 (TriangleAttention; AttentionPairBias with the
// 24-wide heads padded to 32): the softmax warps never touch global memory.
//
// One CTA = 128 queries of one batch row x 2 heads (one head per softmax warpgroup).
//   warp 0      : TMA producer.  Q once; per 128-key block: K tile (+ the 4 KB mask-bias tile),
//                 one bf16 pair-bias tile per head, V tile.  Every buffer is single: a tile is
//                 re-filled as soon as the MMAs that read it have committed, which is long before
//                 it is needed again.
//   warp 1      : tcgen05.mma issuer.  For each head the logits accumulator is built from three
//                 products:  S  = Q K^T                      (K = 32)
//                            S += I  * Bias^T                (K = 128; I = identity, so the bias
//                                                             tile is ADDED on the tensor core)
//                            S += E1 * Mext^T                (K = 16; column 0 of E1 is all ones,
//                                                             column 0 of Mext is the additive
//                                                             mask bias of each key)
//                 then O_blk = P V once the warpgroup has published P.
//   warps 2..5 / 6..9 : softmax warpgroups, one thread per query row: row max straight from TMEM,
//                 ex2, row sum, P as bf16 into a swizzled K-major tile; running max/sum/output in
//                 registers.
//
// The pair bias arrives as bf16 [head][key][query] (query contiguous) so that a TMA tile
// [128 keys][128 queries] is directly the K-major B operand of the identity product.
#include "internal.h"
#include "umma.cuh"

namespace xf {

struct Attn2Args {
  int S, B;
  int q_col0, k_col0, v_col0, g_col0;
  int transposed;
  const bf16* qkvg;
  long long seq_stride, batch_stride;
  const bf16* mext;  // [B or 1][KB][2048] bf16: un-swizzled K-major [128 keys][16] tiles, column 0 = mask bias
  long long mext_batch_stride;  // elements; 0 when one mask row serves every batch row
  bf16* out;
  long long out_seq_stride, out_batch_stride;
  int* status;
};

constexpr int A2_THREADS = 320;
constexpr uint32_t A2_T = 16384;  // [128][64] bf16 tile
// Q, K, V, bias[2][2], P[2][2], I[2] tiles, then E1 and Mext (4 KB each), then barriers
constexpr uint32_t A2_OFF_Q = 0, A2_OFF_K = A2_T, A2_OFF_V = 2 * A2_T, A2_OFF_BIAS = 3 * A2_T, A2_OFF_P = 7 * A2_T,
                   A2_OFF_I = 11 * A2_T, A2_OFF_E1 = 13 * A2_T, A2_OFF_MEXT = 13 * A2_T + 4096,
                   A2_OFF_BAR = 13 * A2_T + 8192;
constexpr uint32_t A2_SMEM = A2_OFF_BAR + 256 + 1024;

__device__ __forceinline__ float ex2f_(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(A2_THREADS, 1)
attn2_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmb, const Attn2Args p) {
  constexpr int D = 32;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem + A2_OFF_Q;
  uint8_t* sK = smem + A2_OFF_K;
  uint8_t* sV = smem + A2_OFF_V;
  uint8_t* sBias = smem + A2_OFF_BIAS;  // warpgroup w: 2 tiles (queries 0..63, 64..127)
  uint8_t* sP = smem + A2_OFF_P;        // warpgroup w: 2 tiles (keys 0..63, 64..127)
  uint8_t* sI = smem + A2_OFF_I;        // 2 tiles
  uint8_t* sE1 = smem + A2_OFF_E1;
  uint8_t* sMext = smem + A2_OFF_MEXT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A2_OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* bias_full = bars + 5;   // [2]
  uint64_t* bias_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* pv_full = bars + 11;    // [2]
  uint64_t* p2done = bars + 13;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;  // query tile, head pair, batch row
  const AbortCtx ab{cta_abort, p.status};
  const int KB = (p.S + 127) / 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bias_full[s], 1);
      mbar_init(&bias_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&pv_full[s], 1);
      mbar_init(&p2done[s], 128);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm);
    tma_prefetch_desc(&tmb);
  }
  // constant operands: identity (two swizzled [128][64] tiles) and E1 (un-swizzled [128][16], column 0 = 1)
  for (uint32_t i = threadIdx.x; i < (2 * A2_T + 4096) / 16; i += A2_THREADS)
    reinterpret_cast<uint4*>(sI)[i] = make_uint4(0, 0, 0, 0);  // sI and sE1 are adjacent
  __syncthreads();
  if (threadIdx.x < 128) {
    const uint32_t m = threadIdx.x;
    const uint16_t one = 0x3F80;  // bf16 1.0
    *reinterpret_cast<uint16_t*>(sI + (m >> 6) * A2_T + sw128_offset(m, m & 63)) = one;
    *reinterpret_cast<uint16_t*>(sE1 + (m >> 3) * 256 + (m & 7) * 16) = one;
  }
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      auto load = [&](uint8_t* dst, uint64_t* bar, int col, int seq0) {
        if (p.transposed) tma_load_3d(dst, &tm, bar, col, b, seq0);
        else tma_load_3d(dst, &tm, bar, col, seq0, b);
      };
      mbar_arrive_expect_tx(q_full, A2_T);
      load(sQ, q_full, p.q_col0 + hp * 64, qt * 128);
      const bf16* mrow = p.mext + (long long)b * p.mext_batch_stride;
      for (int kb = 0; kb < KB; ++kb) {
        const uint32_t par = (kb & 1) ^ 1u;
        if (!mbar_wait(k_empty, par, ab, XF_ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(k_full, A2_T + 4096);
        load(sK, k_full, p.k_col0 + hp * 64, kb * 128);
        bulk_load(sMext, mrow + (long long)kb * 2048, 4096, k_full);
        bool okay = true;
        for (int w = 0; w < 2 && okay; ++w) {
          if (!mbar_wait(&bias_empty[w], par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&bias_full[w], 2 * A2_T);
          tma_load_3d(sBias + w * 2 * A2_T, &tmb, &bias_full[w], qt * 128, kb * 128, hp * 2 + w);
          tma_load_3d(sBias + w * 2 * A2_T + A2_T, &tmb, &bias_full[w], qt * 128 + 64, kb * 128, hp * 2 + w);
        }
        if (!okay) break;
        if (!mbar_wait(v_empty, par, ab, XF_ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(v_full, A2_T);
        load(sV, v_full, p.v_col0 + hp * 64, kb * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(128, 128);
      constexpr uint32_t idesc_pv = make_idesc(128, D, 0, 1);
      const uint64_t e1d = make_sdesc_noswizzle(smem_u32(sE1), 128, 256);
      const uint64_t mxd = make_sdesc_noswizzle(smem_u32(sMext), 128, 256);
      bool okay = mbar_wait(q_full, 0, ab, XF_ERR_WAIT_FULL);
      for (int n = 0; n <= KB && okay; ++n) {
        for (int w = 0; w < 2 && okay; ++w) {
          if (n > 0) {
            if (!mbar_wait(&p2done[w], (n - 1) & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
            tc_fence_after();
          }
          if (n < KB) {
            if (w == 0 && !mbar_wait(k_full, n & 1, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
            if (!mbar_wait(&bias_full[w], n & 1, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
            tc_fence_after();
            const uint32_t d = tmem_base + w * 128;
            const uint64_t qd = make_sdesc(smem_u32(sQ) + w * 64, 16, 1024);
            const uint64_t kd = make_sdesc(smem_u32(sK) + w * 64, 16, 1024);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) umma_ss(d, qd + 2 * k, kd + 2 * k, idesc_s, k ? 1u : 0u);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint32_t off = (ks >> 2) * A2_T + (ks & 3) * 32;
              umma_ss(d, make_sdesc(smem_u32(sI) + off, 16, 1024),
                      make_sdesc(smem_u32(sBias) + w * 2 * A2_T + off, 16, 1024), idesc_s, 1u);
            }
            umma_ss(d, e1d, mxd, idesc_s, 1u);
            umma_commit(&s_full[w]);
            umma_commit(&bias_empty[w]);
            if (w == 1) umma_commit(k_empty);
          }
          if (n > 0) {
            if (w == 0 && !mbar_wait(v_full, (n - 1) & 1, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
            tc_fence_after();
            const uint32_t pbase = smem_u32(sP + w * 2 * A2_T);
            const uint32_t vbase = smem_u32(sV) + w * 64;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t ad = make_sdesc(pbase + (ks >> 2) * A2_T + (ks & 3) * 32, 16, 1024);
              const uint64_t bd = make_sdesc(vbase + ks * 2048, A2_T, 1024);  // V is N-major: 16 keys = 2048 B
              umma_ss(tmem_base + 256 + w * 64, ad, bd, idesc_pv, ks ? 1u : 0u);
            }
            umma_commit(&pv_full[w]);
            if (w == 1) umma_commit(v_empty);
          }
        }
      }
    }
  } else {
    const int w = (warp - 2) >> 2;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const int qi = qt * 128 + row;
    const bool qvalid = qi < p.S;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + w * 128 + lane_addr;
    const uint32_t pv_addr = tmem_base + 256 + w * 64 + lane_addr;
    uint8_t* myP = sP + w * 2 * A2_T + row * 128;
    const uint32_t rsw = uint32_t(row & 7);

    float m_run = -3.0e38f, l_run = 0.f, O[D];
#pragma unroll
    for (int d = 0; d < D; ++d) O[d] = 0.f;
    bool okay = true;
    for (int kb = 0; kb < KB; ++kb) {
      if (!mbar_wait(&s_full[w], kb & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
      tc_fence_after();
      // ---- sweep 1: row maximum of the finished logits
      float mx = -3.0e38f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r0[32], r1[32];
        tmem_ld32(s_addr + half * 64, r0);
        tmem_ld32(s_addr + half * 64 + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          mx = fmaxf(mx, fmaxf(__uint_as_float(r0[e]), __uint_as_float(r0[e + 1])));
          mx = fmaxf(mx, fmaxf(__uint_as_float(r1[e]), __uint_as_float(r1[e + 1])));
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float alpha = ex2f_((m_run - m_new) * LOG2E);
      m_run = m_new;
      // ---- fold in the previous block's P V
      if (kb > 0) {
        if (!mbar_wait(&pv_full[w], (kb - 1) & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32(pv_addr, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) O[e] = (O[e] + __uint_as_float(r[e])) * alpha;
      }
      // ---- sweep 2: exponentiate, row sum, P -> shared memory
      const float mneg = -m_new * LOG2E;
      float lsum = 0.f;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        tmem_ld32(s_addr + cc * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float p0 = ex2f_(fmaf(__uint_as_float(r[2 * e]), LOG2E, mneg));
          const float p1 = ex2f_(fmaf(__uint_as_float(r[2 * e + 1]), LOG2E, mneg));
          lsum += p0 + p1;
          pk[e] = pack_bf16x2(p0, p1);
        }
        uint8_t* prow = myP + (cc >> 1) * A2_T;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t chunk = uint32_t((cc & 1) * 4 + g) ^ rsw;
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        }
      }
      l_run = l_run * alpha + lsum;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&p2done[w]);
    }
    if (okay && KB > 0) {
      if (mbar_wait(&pv_full[w], (KB - 1) & 1, ab, XF_ERR_WAIT_ATTN)) {
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32(pv_addr, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) O[e] += __uint_as_float(r[e]);
      } else okay = false;
    }
    if (okay && qvalid) {
      const int col = hp * 64 + w * D;
      const float inv = __fdividef(1.f, l_run);
      const bf16* grow = p.qkvg + (long long)b * p.batch_stride + (long long)qi * p.seq_stride + p.g_col0 + col;
      bf16* orow = p.out + (long long)b * p.out_batch_stride + (long long)qi * p.out_seq_stride + col;
#pragma unroll
      for (int g8 = 0; g8 < D / 8; ++g8) {
        const uint4 gu = *reinterpret_cast<const uint4*>(grow + g8 * 8);
        const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float o0 = O[g8 * 8 + 2 * e] * inv * sigmoidf_fast(bf16_lo(gw[e]));
          const float o1 = O[g8 * 8 + 2 * e + 1] * inv * sigmoidf_fast(bf16_hi(gw[e]));
          ow[e] = pack_bf16x2(o0, o1);
        }
        *reinterpret_cast<uint4*>(orow + g8 * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {}
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Mask-bias tiles: out[b][kb] is an un-swizzled K-major [128 keys][16] bf16 tile (core matrices of
// 8 keys x 8 columns, 128 B each; the two column halves 128 B apart, 8-key groups 256 B apart) whose
// column 0 holds 1e9 * (mask[b][k] - 1) for k < S and -1e30 for the padding of the last tile.
__global__ void mext_kernel(const float* __restrict__ mask, long long mask_ld, bf16* __restrict__ out, int B, int S,
                            int KB) {
  const long long n = (long long)B * KB * 128;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int r = int(idx & 127);
    const long long tile = idx >> 7;
    const int kb = int(tile % KB);
    const long long bb = tile / KB;
    const int k = kb * 128 + r;
    float v = -1.0e30f;
    if (k < S) v = mask ? 1.0e9f * (mask[bb * mask_ld + k] - 1.f) : 0.f;
    uint4 lo = make_uint4(uint32_t(__bfloat16_as_ushort(__float2bfloat16(v))), 0, 0, 0);
    uint8_t* t = reinterpret_cast<uint8_t*>(out) + tile * 4096 + (r >> 3) * 256 + (r & 7) * 16;
    *reinterpret_cast<uint4*>(t) = lo;
    *reinterpret_cast<uint4*>(t + 128) = make_uint4(0, 0, 0, 0);
  }
}

int launch_mext(Ctx* c, const float* mask, long long mask_ld, bf16* out, int B, int S, cudaStream_t st) {
  const int KB = (S + 127) / 128;
  const long long n = (long long)B * KB * 128;
  if (n <= 0) return XFOLD_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 8192) blocks = 8192;
  ProfScope ps(c, XFOLD_K_MASK_BIAS, st);
  mext_kernel<<<(int)blocks, 256, 0, st>>>(mask, mask_ld, out, B, S, KB);
  return check_launch(c, "mext_kernel");
}

// fp32 [H][S][S] (query-major) -> bf16 [H][S][ldq] (key-major, query contiguous): the layout the kernel's
// pair-bias tensor map expects.  32 x 32 tiles through shared memory.
__global__ void bias_transpose_kernel(const float* __restrict__ in, bf16* __restrict__ out, int S, int ldq) {
  __shared__ float t[32][33];
  const int h = blockIdx.z;
  const int q0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
  const float* src = in + (long long)h * S * S;
  bf16* dst = out + (long long)h * S * ldq;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int q = q0 + r, k = k0 + threadIdx.x;
    t[r][threadIdx.x] = (q < S && k < S) ? src[(long long)q * S + k] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, q = q0 + threadIdx.x;
    if (k < S && q < S) dst[(long long)k * ldq + q] = __float2bfloat16(t[threadIdx.x][r]);
  }
}

int launch_bias_transpose(Ctx* c, const float* in, bf16* out, int H, int S, int ldq, cudaStream_t st) {
  if (H <= 0 || S <= 0) return XFOLD_OK;
  dim3 grid((S + 31) / 32, (S + 31) / 32, H), block(32, 8);
  ProfScope ps(c, XFOLD_K_MASK_BIAS, st);
  bias_transpose_kernel<<<grid, block, 0, st>>>(in, out, S, ldq);
  return check_launch(c, "bias_transpose_kernel");
}

// qkvg: projection buffer ([B][S][width], or [S][B][width] when transposed); biasT: bf16 [heads][S][ldq];
// mext: tiles from launch_mext ([B][KB][2048] or one row shared by all batch rows when mext_rows == 1).
int launch_attention2(Ctx* c, const bf16* qkvg, int width, int S, int B, int transposed, int q_col0, int k_col0,
                      int v_col0, int g_col0, int heads, const bf16* biasT, int ldq, const bf16* mext, int mext_rows,
                      bf16* out, long long out_seq_stride, long long out_batch_stride, cudaStream_t st) {
  if ((width & 7) || (ldq & 7) || (heads & 1)) return fail(c, XFOLD_ERR_ARG, "attention: width and bias pitch must be multiples of 8, heads even");
  if (S <= 0 || B <= 0) return XFOLD_OK;
  if (B > 65535 || heads / 2 > 65535) return fail(c, XFOLD_ERR_ARG, "attention: batch %d exceeds the grid limit", B);
  CUtensorMap tm, tmb;
  bool ok;
  Attn2Args a;
  if (!transposed) {
    ok = make_tmap_bf16_3d(&tm, qkvg, width, S, B, width, (uint64_t)width * S, 64, 128, 1);
    a.seq_stride = width;
    a.batch_stride = (long long)S * width;
  } else {
    ok = make_tmap_bf16_3d(&tm, qkvg, width, B, S, width, (uint64_t)width * B, 64, 1, 128);
    a.seq_stride = (long long)B * width;
    a.batch_stride = width;
  }
  ok = ok && make_tmap_bf16_3d(&tmb, biasT, S, S, heads, ldq, (uint64_t)ldq * S, 64, 128, 1);
  if (!ok) return fail(c, XFOLD_ERR_ARG, "attention: cannot encode tensor maps");
  const int KB = (S + 127) / 128;
  a.S = S;
  a.B = B;
  a.q_col0 = q_col0;
  a.k_col0 = k_col0;
  a.v_col0 = v_col0;
  a.g_col0 = g_col0;
  a.transposed = transposed;
  a.qkvg = qkvg;
  a.mext = mext;
  a.mext_batch_stride = mext_rows == 1 ? 0 : (long long)KB * 2048;
  a.out = out;
  a.out_seq_stride = out_seq_stride;
  a.out_batch_stride = out_batch_stride;
  a.status = c->d_status;
  static bool attr_done[8] = {false};
  if (!attr_done[c->device & 7]) {
    cudaError_t e = cudaFuncSetAttribute(attn2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "attention smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  dim3 grid((S + 127) / 128, heads / 2, B);
  ProfScope ps(c, XFOLD_K_ATTENTION, st);
  attn2_kernel<<<grid, A2_THREADS, A2_SMEM, st>>>(tm, tmb, a);
  return check_launch(c, "attn2_kernel");
}

}  // namespace xf
