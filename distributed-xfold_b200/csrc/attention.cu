// Gated multi-head self-attention with an additive pair bias, flash style, for sm_100a.
//
// One CTA handles 128 queries of one batch row for a group of 128 projection columns
// (4 heads x 32 or 2 heads x 64).  q, k, v and the gate are columns of one fused projection
// buffer and are fetched by TMA straight into 128-byte-swizzled tiles, so the same kernel
// serves TriangleAttention (starting node: batch = pair row; ending node: the tensor-map
// coordinates are swapped, no transposed copy is made) and AttentionPairBias.
//
//   warp 0      : TMA producer (Q once, then double-buffered K/V tiles of 128 keys)
//   warp 1      : tcgen05.mma issuer.  S = Q K^T into TMEM, later O_blk = P V into TMEM
//   warps 2..5  : softmax warpgroup 0 (first half of the heads), one thread per query row
//   warps 6..9  : softmax warpgroup 1 (second half of the heads)
//
// Softmax is done in two sweeps over the 128-key tile: sweep 1 adds the pair bias and the
// mask bias to the logits, writes the sum back to TMEM and tracks the row maximum; sweep 2
// reads it back, exponentiates (ex2) and stores P as bf16 into a swizzled K-major tile that is
// the A operand of the P V MMA.  Running max / sum / output accumulator live in registers.
#include <type_traits>

#include "internal.h"
#include "umma.cuh"

namespace xf {

struct AttnArgs {
  int S, B;
  int q_col0, k_col0, v_col0, g_col0;
  int transposed;
  const bf16* qkvg;
  long long seq_stride, batch_stride;
  const float* bias;  // [heads][S][bias_ld]
  long long bias_head_stride;
  int bias_ld;
  int bias_vec;  // rows of the bias are 16-byte aligned, float4 loads allowed
  const float* maskb;  // [B][maskb_ld], additive, padded with -1e30 up to a multiple of 128 keys
  int maskb_ld;
  bf16* out;
  long long out_seq_stride, out_batch_stride;
  int* status;
};

constexpr int ATT_THREADS = 320;
constexpr uint32_t ATT_TILE = 16384;  // 128 rows x 64 bf16
constexpr uint32_t ATT_SMEM = 2 * ATT_TILE /*Q*/ + 2 * 4 * ATT_TILE /*K,V x 2 stages*/ + 2 * 2 * ATT_TILE /*P*/ + 1024 + 256;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_kernel(const __grid_constant__ CUtensorMap tm, const AttnArgs p) {
  constexpr int HPG = 128 / D;  // heads per CTA
  constexpr int HPW = HPG / 2;  // heads per softmax warpgroup
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + 2 * ATT_TILE;          // stage s: K chunks at s*4 tiles, V chunks 2 tiles later
  uint8_t* sP = smem + 10 * ATT_TILE;          // warpgroup w: 2 tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 14 * ATT_TILE);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* pv_full = bars + 7;    // [2]
  uint64_t* p2done = bars + 9;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
  const AbortCtx ab{cta_abort, p.status};
  const int KB = (p.S + 127) / 128;
  const int n_items = KB * HPW;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&pv_full[s], 1);
      mbar_init(&p2done[s], 128);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm);
  }
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
      mbar_arrive_expect_tx(q_full, 2 * ATT_TILE);
      load(sQ, q_full, p.q_col0 + hg * 128, qt * 128);
      load(sQ + ATT_TILE, q_full, p.q_col0 + hg * 128 + 64, qt * 128);
      for (int kb = 0; kb < KB; ++kb) {
        const int st = kb & 1;
        if (!mbar_wait(&kv_empty[st], ((kb >> 1) & 1) ^ 1u, ab, XF_ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(&kv_full[st], 4 * ATT_TILE);
        uint8_t* base = sKV + st * 4 * ATT_TILE;
        load(base, &kv_full[st], p.k_col0 + hg * 128, kb * 128);
        load(base + ATT_TILE, &kv_full[st], p.k_col0 + hg * 128 + 64, kb * 128);
        load(base + 2 * ATT_TILE, &kv_full[st], p.v_col0 + hg * 128, kb * 128);
        load(base + 3 * ATT_TILE, &kv_full[st], p.v_col0 + hg * 128 + 64, kb * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, 128);
      constexpr uint32_t idesc_pv = make_idesc(128, D, 0, 1);
      bool okay = mbar_wait(q_full, 0, ab, XF_ERR_WAIT_FULL);
      for (int n = 0; n <= n_items && okay; ++n) {
        for (int wg = 0; wg < 2 && okay; ++wg) {
          if (n > 0) {
            if (!mbar_wait(&p2done[wg], (n - 1) & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
            tc_fence_after();
          }
          if (n < n_items) {
            const int kb = n / HPW, hh = n % HPW, st = kb & 1;
            if (wg == 0 && hh == 0) {
              if (!mbar_wait(&kv_full[st], (kb >> 1) & 1, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
              tc_fence_after();
            }
            const int hl = wg * HPW + hh;
            const uint32_t coff = uint32_t((hl * D) / 64) * ATT_TILE + uint32_t((hl * D) % 64) * 2u;
            const uint64_t ad = make_sdesc(smem_u32(sQ) + coff, 16, 1024);
            const uint64_t bd = make_sdesc(smem_u32(sKV + st * 4 * ATT_TILE) + coff, 16, 1024);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) umma_ss(tmem_base + wg * 128, ad + 2 * k, bd + 2 * k, idesc_qk, k ? 1u : 0u);
            umma_commit(&s_full[wg]);
          }
          if (n > 0) {
            const int kbp = (n - 1) / HPW, hhp = (n - 1) % HPW, st = kbp & 1;
            const int hl = wg * HPW + hhp;
            const uint32_t voff = uint32_t((hl * D) / 64) * ATT_TILE + uint32_t((hl * D) % 64) * 2u;
            const uint32_t pbase = smem_u32(sP + wg * 2 * ATT_TILE);
            const uint32_t vbase = smem_u32(sKV + st * 4 * ATT_TILE + 2 * ATT_TILE) + voff;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t ad = make_sdesc(pbase + (ks >> 2) * ATT_TILE + (ks & 3) * 32, 16, 1024);
              const uint64_t bd = make_sdesc(vbase + ks * 2048, ATT_TILE, 1024);  // V is N-major: 16 keys = 2048 B
              umma_ss(tmem_base + 256 + wg * 64, ad, bd, idesc_pv, ks ? 1u : 0u);
            }
            umma_commit(&pv_full[wg]);
            if (wg == 1 && hhp == HPW - 1) umma_commit(&kv_empty[st]);
          }
        }
      }
    }
  } else {
    const int wg = (warp - 2) >> 2;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const int qi = qt * 128 + row;
    const bool qvalid = qi < p.S;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + wg * 128 + lane_addr;
    const uint32_t pv_addr = tmem_base + 256 + wg * 64 + lane_addr;
    uint8_t* myP = sP + wg * 2 * ATT_TILE;
    const float* mrow = p.maskb + (long long)b * p.maskb_ld;

    float m_run[HPW], l_run[HPW], O[HPW][D];
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
      m_run[h] = -3.0e38f;
      l_run[h] = 0.f;
#pragma unroll
      for (int d = 0; d < D; ++d) O[h][d] = 0.f;
    }
    bool okay = true;
    int n = 0;
    int kb = 0;
    // one (key block, head) item; HHc carries the compile-time head slot so that O[] stays in registers
    auto item = [&](auto HHc) -> bool {
      constexpr int hh = decltype(HHc)::value;
      const int hl = wg * HPW + hh;
      const float* brow = p.bias + (long long)(hg * HPG + hl) * p.bias_head_stride + (long long)qi * p.bias_ld +
                          kb * 128;
      if (!mbar_wait(&s_full[wg], n & 1, ab, XF_ERR_WAIT_ATTN)) return false;
      tc_fence_after();
      // ---- sweep 1: logits + pair bias + mask bias -> TMEM, row max
      float mx = -3.0e38f;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        tmem_ld32(s_addr + cc * 32, r);
        tmem_ld_wait();
        const int k0 = kb * 128 + cc * 32;
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4) {
          const float4 mb = *reinterpret_cast<const float4*>(mrow + k0 + g4 * 4);
          float4 nb = make_float4(0.f, 0.f, 0.f, 0.f);
          if (qvalid) {
            if (p.bias_vec && k0 + g4 * 4 + 3 < p.S) nb = *reinterpret_cast<const float4*>(brow + cc * 32 + g4 * 4);
            else {
              float t4[4] = {0.f, 0.f, 0.f, 0.f};
              for (int e = 0; e < 4; ++e)
                if (k0 + g4 * 4 + e < p.S) t4[e] = brow[cc * 32 + g4 * 4 + e];
              nb = make_float4(t4[0], t4[1], t4[2], t4[3]);
            }
          }
          const float t0 = __uint_as_float(r[g4 * 4 + 0]) + nb.x + mb.x;
          const float t1 = __uint_as_float(r[g4 * 4 + 1]) + nb.y + mb.y;
          const float t2 = __uint_as_float(r[g4 * 4 + 2]) + nb.z + mb.z;
          const float t3 = __uint_as_float(r[g4 * 4 + 3]) + nb.w + mb.w;
          mx = fmaxf(mx, fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)));
          r[g4 * 4 + 0] = __float_as_uint(t0);
          r[g4 * 4 + 1] = __float_as_uint(t1);
          r[g4 * 4 + 2] = __float_as_uint(t2);
          r[g4 * 4 + 3] = __float_as_uint(t3);
        }
        tmem_st32(s_addr + cc * 32, r);
      }
      tmem_st_wait();
      const float m_new = fmaxf(m_run[hh], mx);
      const float alpha = ex2f((m_run[hh] - m_new) * LOG2E);
      m_run[hh] = m_new;
      // ---- fold in the P V product of the previous item (it belongs to the other head when HPW == 2)
      if (n > 0) {
        if (!mbar_wait(&pv_full[wg], (n - 1) & 1, ab, XF_ERR_WAIT_ATTN)) return false;
        tc_fence_after();
        constexpr int hp = (HPW == 1) ? 0 : (1 - hh);
#pragma unroll
        for (int dc = 0; dc < D / 32; ++dc) {
          uint32_t r[32];
          tmem_ld32(pv_addr + dc * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) O[hp][dc * 32 + e] += __uint_as_float(r[e]);
        }
      }
#pragma unroll
      for (int d = 0; d < D; ++d) O[hh][d] *= alpha;
      // ---- sweep 2: exponentiate, row sum, P -> shared memory (bf16, swizzled K-major)
      const float mneg = -m_new * LOG2E;
      float lsum = 0.f;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        tmem_ld32(s_addr + cc * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float p0 = ex2f(fmaf(__uint_as_float(r[2 * e]), LOG2E, mneg));
          const float p1 = ex2f(fmaf(__uint_as_float(r[2 * e + 1]), LOG2E, mneg));
          lsum += p0 + p1;
          pk[e] = pack_bf16x2(p0, p1);
        }
        uint8_t* prow = myP + (cc >> 1) * ATT_TILE + row * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t chunk = uint32_t((cc & 1) * 4 + g) ^ uint32_t(row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        }
      }
      l_run[hh] = l_run[hh] * alpha + lsum;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&p2done[wg]);
      ++n;
      return true;
    };
    for (kb = 0; kb < KB && okay; ++kb) {
      okay = item(std::integral_constant<int, 0>{});
      if constexpr (HPW == 2) {
        if (okay) okay = item(std::integral_constant<int, 1>{});
      }
    }
    if (okay && n_items > 0) {
      if (mbar_wait(&pv_full[wg], (n_items - 1) & 1, ab, XF_ERR_WAIT_ATTN)) {
        tc_fence_after();
#pragma unroll
        for (int dc = 0; dc < D / 32; ++dc) {
          uint32_t r[32];
          tmem_ld32(pv_addr + dc * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) O[HPW - 1][dc * 32 + e] += __uint_as_float(r[e]);
        }
      } else okay = false;
    }
    if (okay && qvalid) {
#pragma unroll
      for (int hh = 0; hh < HPW; ++hh) {
        const int col = hg * 128 + (wg * HPW + hh) * D;
        const float inv = __fdividef(1.f, l_run[hh]);
        const bf16* grow = p.qkvg + (long long)b * p.batch_stride + (long long)qi * p.seq_stride + p.g_col0 + col;
        bf16* orow = p.out + (long long)b * p.out_batch_stride + (long long)qi * p.out_seq_stride + col;
#pragma unroll
        for (int g8 = 0; g8 < D / 8; ++g8) {
          const uint4 gu = *reinterpret_cast<const uint4*>(grow + g8 * 8);
          const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
          uint32_t ow[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float o0 = O[hh][g8 * 8 + 2 * e] * inv * sigmoidf_fast(bf16_lo(gw[e]));
            const float o1 = O[hh][g8 * 8 + 2 * e + 1] * inv * sigmoidf_fast(bf16_hi(gw[e]));
            ow[e] = pack_bf16x2(o0, o1);
          }
          *reinterpret_cast<uint4*>(orow + g8 * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
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

// maskb[b][k] = 1e9 * (mask[b][k] - 1) for k < S (0 when mask is null), -1e30 for the tile padding
__global__ void maskb_kernel(const float* __restrict__ mask, long long mask_ld, float* __restrict__ out, int B, int S,
                             int ld) {
  const long long n = (long long)B * ld;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long bb = idx / ld;
    const int k = int(idx % ld);
    float v = -1.0e30f;
    if (k < S) v = mask ? 1.0e9f * (mask[bb * mask_ld + k] - 1.f) : 0.f;
    out[idx] = v;
  }
}

int launch_maskb(Ctx* c, const float* mask, long long mask_ld, float* out, int B, int S, int ld, cudaStream_t st) {
  const long long n = (long long)B * ld;
  if (n <= 0) return XFOLD_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 4096) blocks = 4096;
  ProfScope ps(c, XFOLD_K_MASK_BIAS, st);
  maskb_kernel<<<(int)blocks, 256, 0, st>>>(mask, mask_ld, out, B, S, ld);
  return check_launch(c, "maskb_kernel");
}

int launch_attention(Ctx* c, int D, const CUtensorMap& tm, const AttnArgs& a, int head_groups, cudaStream_t st) {
  static bool attr_done[2][8] = {{false}};
  const int qt = (a.S + 127) / 128;
  if (qt <= 0 || a.B <= 0 || head_groups <= 0) return XFOLD_OK;
  if (a.B > 65535 || head_groups > 65535) return fail(c, XFOLD_ERR_ARG, "attention: batch %d / head groups %d exceed the grid limit", a.B, head_groups);
  dim3 grid(qt, head_groups, a.B);
  ProfScope ps(c, c->attn_tag, st);
  if (D == 32) {
    if (!attr_done[0][c->device & 7]) {
      cudaError_t e = cudaFuncSetAttribute(attn_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
      if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "attention smem attribute: %s", cudaGetErrorString(e));
      attr_done[0][c->device & 7] = true;
    }
    attn_kernel<32><<<grid, ATT_THREADS, ATT_SMEM, st>>>(tm, a);
  } else if (D == 64) {
    if (!attr_done[1][c->device & 7]) {
      cudaError_t e = cudaFuncSetAttribute(attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
      if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "attention smem attribute: %s", cudaGetErrorString(e));
      attr_done[1][c->device & 7] = true;
    }
    attn_kernel<64><<<grid, ATT_THREADS, ATT_SMEM, st>>>(tm, a);
  } else {
    return fail(c, XFOLD_ERR_ARG, "attention: head dim must be 32 or 64 (got %d)", D);
  }
  return check_launch(c, "attn_kernel");
}

int launch_attention_op(Ctx* c, int D, const bf16* qkvg, int width, int S, int B, int transposed, int q_col0,
                        int k_col0, int v_col0, int g_col0, int head_groups, const float* bias,
                        long long bias_head_stride, int bias_ld, const float* maskb, int maskb_ld, bf16* out,
                        long long out_seq_stride, long long out_batch_stride, cudaStream_t st) {
  if (width & 7) return fail(c, XFOLD_ERR_ARG, "attention: projection width must be a multiple of 8");
  CUtensorMap tm;
  bool ok;
  AttnArgs a;
  if (!transposed) {  // storage [B][S][width]
    ok = make_tmap_bf16_3d(&tm, qkvg, width, S, B, width, (uint64_t)width * S, 64, 128, 1);
    a.seq_stride = width;
    a.batch_stride = (long long)S * width;
  } else {  // storage [S][B][width]
    ok = make_tmap_bf16_3d(&tm, qkvg, width, B, S, width, (uint64_t)width * B, 64, 1, 128);
    a.seq_stride = (long long)B * width;
    a.batch_stride = width;
  }
  if (!ok) return fail(c, XFOLD_ERR_ARG, "attention: cannot encode the projection tensor map");
  a.S = S;
  a.B = B;
  a.q_col0 = q_col0;
  a.k_col0 = k_col0;
  a.v_col0 = v_col0;
  a.g_col0 = g_col0;
  a.transposed = transposed;
  a.qkvg = qkvg;
  a.bias = bias;
  a.bias_head_stride = bias_head_stride;
  a.bias_ld = bias_ld;
  a.bias_vec = ((bias_ld & 3) == 0) && ((bias_head_stride & 3) == 0) && ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
  a.maskb = maskb;
  a.maskb_ld = maskb_ld;
  a.out = out;
  a.out_seq_stride = out_seq_stride;
  a.out_batch_stride = out_batch_stride;
  a.status = c->d_status;
  return launch_attention(c, D, tm, a, head_groups, st);
}

}  // namespace xf
