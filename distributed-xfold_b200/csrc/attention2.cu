// Second-generation gated attention for head dim 32 (TriangleAttention; AttentionPairBias with the
// 24-wide heads padded to 32): the softmax warps never touch global memory.
//
// Work item = 128 queries of one batch row x 2 heads (one head per softmax warpgroup); CTAs are persistent
// (one per SM) and pipeline consecutive items into each other.
//   warp 0      : TMA producer.  Q once; per 128-key block: K tile (+ the 4 KB mask-bias tile),
//                 one bf16 pair-bias tile per head, V tile.  Every buffer is single: a tile is
//                 re-filled as soon as the MMAs that read it have committed, which is long before
//                 it is needed again.
//   warp 1      : tcgen05.mma issuer.  A softmax thread pulls its whole 128-wide logits row out of TMEM in
//                 one go, so the logits of block n+1 are produced while block n is being exponentiated;
//                 O accumulates in TMEM across key blocks and is rescaled lazily (only when a row maximum
//                 grows by more than 2^8).  For each head the logits accumulator is built from two
//                 products:  S  = Q K^T                      (K = 32)
//                            S += E1 * Mext^T                (K = 16; column 0 of E1 is all ones,
//                                                             column 0 of Mext is the additive
//                                                             mask bias of each key)
//                 then O += P V once the warpgroup has published P.  (tcgen05.mma costs ~65-85 cycles per
//                 instruction whatever its N, so the issuing thread is kept to 11 instructions per head
//                 and key block; adding the pair bias with an identity-matrix product, tried first, made
//                 that thread the bottleneck.)
//   warps 2..5 / 6..9 : softmax warpgroups, one thread per query row: pair bias added from the shared-memory
//                 tile, row max, ex2, row sum, P as bf16 into a swizzled K-major tile; running offset / sum in
//                 registers, output in TMEM.
//
// The pair bias arrives as bf16 [head][query][key] (key contiguous, row pitch a multiple of 8); TMA lays a
// [128 queries][64 keys] half tile out with the 128-byte swizzle, so the per-row 16-byte reads of the softmax
// threads are bank-conflict free.
#include <cstdlib>

#include <cuda_fp16.h>

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
  int heads;
  int* status;
};

constexpr int A2_THREADS = 320;
constexpr uint32_t A2_T = 16384;  // [128][64] bf16 tile
// Q, K, V, bias[2][2], P[2][2] tiles, then E1 and Mext (4 KB each), then barriers
constexpr uint32_t A2_OFF_Q = 0, A2_OFF_K = A2_T, A2_OFF_V = 2 * A2_T, A2_OFF_BIAS = 3 * A2_T, A2_OFF_P = 7 * A2_T,
                   A2_OFF_E1 = 11 * A2_T, A2_OFF_MEXT = 11 * A2_T + 4096, A2_OFF_BAR = 11 * A2_T + 8192;
constexpr uint32_t A2_SMEM = A2_OFF_BAR + 256 + 1024;

__device__ __forceinline__ float ex2f_(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st32_(uint32_t taddr, const uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_st_wait_() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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
  uint8_t* sBias = smem + A2_OFF_BIAS;  // warpgroup w: 2 tiles [128 queries][keys 0..63 | 64..127]
  uint8_t* sP = smem + A2_OFF_P;        // warpgroup w: 2 tiles (keys 0..63, 64..127)
  uint8_t* sE1 = smem + A2_OFF_E1;
  uint8_t* sMext = smem + A2_OFF_MEXT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A2_OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 4;
  uint64_t* v_empty = bars + 5;
  uint64_t* bias_full = bars + 6;   // [2]
  uint64_t* bias_empty = bars + 8;  // [2]
  uint64_t* s_full = bars + 10;     // [2] logits of a block are in TMEM
  uint64_t* pv_done = bars + 12;    // [2] P V product of a block complete
  uint64_t* p_ready = bars + 14;    // [2] P of a block is in shared memory
  uint64_t* s_read = bars + 16;     // [2] logits of a block are in registers
  uint64_t* turn = bars + 18;       // [2] warpgroup w may run its exponential phase
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const int KB = (p.S + 127) / 128;
  // Persistent CTA: work items (batch row, head pair, query tile), batch row slowest so that the K / V rows of
  // the ~gridDim.x items in flight stay in L2; every role walks the same item sequence and all barriers keep
  // counting across items, so the next item's loads and first logits overlap the current item's tail.
  const int QT = (p.S + 127) / 128, HP = p.heads / 2;
  const long long n_items = (long long)p.B * HP * QT;
  auto decode = [&](long long t, int& qt, int& hp, int& b) {
    qt = int(t % QT);
    hp = int((t / QT) % HP);
    b = int(t / ((long long)QT * HP));
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bias_full[s], 1);
      mbar_init(&bias_empty[s], 128);
      mbar_init(&s_full[s], 1);
      mbar_init(&pv_done[s], 1);
      mbar_init(&p_ready[s], 128);
      mbar_init(&s_read[s], 128);
      mbar_init(&turn[s], 128);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm);
    tma_prefetch_desc(&tmb);
  }
  // constant operand E1: un-swizzled [128][16] tile whose column 0 is all ones
  for (uint32_t i = threadIdx.x; i < 4096 / 16; i += A2_THREADS) reinterpret_cast<uint4*>(sE1)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (threadIdx.x < 128) {
    const uint32_t m = threadIdx.x;
    *reinterpret_cast<uint16_t*>(sE1 + (m >> 3) * 256 + (m & 7) * 16) = 0x3F80;  // bf16 1.0
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
      uint32_t it = 0;        // items started by this CTA
      uint32_t g = 0;         // key blocks started by this CTA (all items)
      bool okay = true;
      for (long long t = blockIdx.x; t < n_items && okay; t += gridDim.x, ++it) {
        int qt, hp, b;
        decode(t, qt, hp, b);
        auto load = [&](uint8_t* dst, uint64_t* bar, int col, int seq0) {
          if (p.transposed) tma_load_3d(dst, &tm, bar, col, b, seq0);
          else tma_load_3d(dst, &tm, bar, col, seq0, b);
        };
        if (!mbar_wait(q_empty, (it & 1) ^ 1u, ab, XF_ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(q_full, A2_T);
        load(sQ, q_full, p.q_col0 + hp * 64, qt * 128);
        const bf16* mrow = p.mext + (long long)b * p.mext_batch_stride;
        for (int kb = 0; kb < KB && okay; ++kb, ++g) {
          const uint32_t par = (g & 1) ^ 1u;
          if (!mbar_wait(k_empty, par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(k_full, A2_T + 4096);
          load(sK, k_full, p.k_col0 + hp * 64, kb * 128);
          bulk_load(sMext, mrow + (long long)kb * 2048, 4096, k_full);
          for (int w = 0; w < 2 && okay; ++w) {
            if (!mbar_wait(&bias_empty[w], par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
            mbar_arrive_expect_tx(&bias_full[w], 2 * A2_T);
            tma_load_3d(sBias + w * 2 * A2_T, &tmb, &bias_full[w], kb * 128, qt * 128, hp * 2 + w);
            tma_load_3d(sBias + w * 2 * A2_T + A2_T, &tmb, &bias_full[w], kb * 128 + 64, qt * 128, hp * 2 + w);
          }
          if (!okay) break;
          if (!mbar_wait(v_empty, par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(v_full, A2_T);
          load(sV, v_full, p.v_col0 + hp * 64, kb * 128);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(128, 128);
      constexpr uint32_t idesc_pv = make_idesc(128, D, 0, 1, 1);  // P and V are fp16 (V N-major): the v columns of the
                                                                  // projection buffer are written as fp16 by the GEMM
      const uint64_t e1d = make_sdesc_noswizzle(smem_u32(sE1), 128, 256);
      const uint64_t mxd = make_sdesc_noswizzle(smem_u32(sMext), 128, 256);
      const long long my_items = n_items > blockIdx.x ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      const long long G = my_items * KB;  // key blocks this CTA processes in total
      // TMEM per warpgroup w: logits S at columns w*128 .. +127, output accumulator O at 256 + w*32 .. +31.
      // A softmax thread pulls its whole logits row into registers at once, so S(g+1) is issued as soon as that
      // load has finished (s_read), i.e. while block g is still being exponentiated -- across item boundaries too.
      auto issue_s = [&](long long g, int w) -> bool {
        const int kb = int(g % KB);
        const uint32_t it = uint32_t(g / KB);
        if (w == 0 && kb == 0 && !mbar_wait(q_full, it & 1, ab, XF_ERR_WAIT_FULL)) return false;
        if (w == 0 && !mbar_wait(k_full, g & 1, ab, XF_ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + w * 128;
        const uint64_t qd = make_sdesc(smem_u32(sQ) + w * 64, 16, 1024);
        const uint64_t kd = make_sdesc(smem_u32(sK) + w * 64, 16, 1024);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_ss(d, qd + 2 * k, kd + 2 * k, idesc_s, k ? 1u : 0u);
        umma_ss(d, e1d, mxd, idesc_s, 1u);
        umma_commit(&s_full[w]);
        if (w == 1) {
          umma_commit(k_empty);
          if (kb == KB - 1) umma_commit(q_empty);  // last use of this item's Q tile
        }
        return true;
      };
      bool okay = G > 0;
      for (int w = 0; w < 2 && okay; ++w) okay = issue_s(0, w);
      for (long long g = 0; g < G && okay; ++g) {
        if (g + 1 < G) {
          for (int w = 0; w < 2 && okay; ++w) {
            if (!mbar_wait(&s_read[w], g & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
            okay = issue_s(g + 1, w);
          }
        }
        const int kb = int(g % KB);
        for (int w = 0; w < 2 && okay; ++w) {
          if (!mbar_wait(&p_ready[w], g & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
          if (w == 0 && !mbar_wait(v_full, g & 1, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
          tc_fence_after();
          const uint32_t pbase = smem_u32(sP + w * 2 * A2_T);
          const uint32_t vbase = smem_u32(sV) + w * 64;
          const uint32_t d = tmem_base + 256 + w * 32;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ad = make_sdesc(pbase + (ks >> 2) * A2_T + (ks & 3) * 32, 16, 1024);
            const uint64_t bd = make_sdesc(vbase + ks * 2048, A2_T, 1024);  // V is N-major: 16 keys = 2048 B
            umma_ss(d, ad, bd, idesc_pv, (kb | ks) ? 1u : 0u);              // O accumulates across the item's key blocks
          }
          umma_commit(&pv_done[w]);
          if (w == 1) umma_commit(v_empty);
        }
      }
    }
  } else {
    const int w = (warp - 2) >> 2;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + w * 128 + lane_addr;
    const uint32_t o_addr = tmem_base + 256 + w * 32 + lane_addr;
    uint8_t* myP = sP + w * 2 * A2_T + row * 128;
    const uint8_t* myBias = sBias + w * 2 * A2_T + row * 128;
    const uint32_t rsw = uint32_t(row & 7);
    uint32_t g = 0;  // key blocks processed by this CTA so far
    bool okay = true;
    // The two warpgroups share each scheduler's exponential unit (one warp of each per scheduler).  They take
    // turns in the ex2-heavy phase, so that one adds bias / takes maxima on the ALU while the other
    // exponentiates, instead of both queueing on the same unit at the same time.  Warpgroup 0 starts.
    if (w == 1) mbar_arrive(&turn[0]);
    for (long long t = blockIdx.x; t < n_items && okay; t += gridDim.x) {
      int qt, hp, b;
      decode(t, qt, hp, b);
      const int qi = qt * 128 + row;
      const bool qvalid = qi < p.S;
      // m_ref is the exponent offset in use (log2 units).  It follows the running maximum lazily: the output
      // accumulator in TMEM is rescaled only when some row of the warp saw its maximum grow by more than 2^8,
      // so most key blocks skip the TMEM round trip; until then P values up to 256 are harmless in bf16 / fp32.
      float m_ref = -3.0e38f, l_run = 0.f;
      for (int kb = 0; kb < KB; ++kb, ++g) {
        if (!mbar_wait(&s_full[w], g & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
        tc_fence_after();
        uint32_t r[128];
        tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[64]));
        tmem_ld32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&r[96]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_read[w]);  // the logits are in registers: the buffer may take the next block
        // add the pair bias (bf16 tile [128 queries][128 keys] in two swizzled halves, this thread's row) and
        // take the row maximum in the same pass
        if (!mbar_wait(&bias_full[w], g & 1, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
        float mx0 = -3.0e38f, mx1 = -3.0e38f, mx2 = -3.0e38f, mx3 = -3.0e38f;
#pragma unroll
        for (int c8 = 0; c8 < 16; ++c8) {
          const uint4 bq = *reinterpret_cast<const uint4*>(myBias + (c8 >> 3) * A2_T + ((uint32_t(c8 & 7) ^ rsw) << 4));
          const int e = c8 * 8;
          float t;
          t = __uint_as_float(r[e + 0]) + bf16_lo(bq.x); r[e + 0] = __float_as_uint(t); mx0 = fmaxf(mx0, t);
          t = __uint_as_float(r[e + 1]) + bf16_hi(bq.x); r[e + 1] = __float_as_uint(t); mx1 = fmaxf(mx1, t);
          t = __uint_as_float(r[e + 2]) + bf16_lo(bq.y); r[e + 2] = __float_as_uint(t); mx2 = fmaxf(mx2, t);
          t = __uint_as_float(r[e + 3]) + bf16_hi(bq.y); r[e + 3] = __float_as_uint(t); mx3 = fmaxf(mx3, t);
          t = __uint_as_float(r[e + 4]) + bf16_lo(bq.z); r[e + 4] = __float_as_uint(t); mx0 = fmaxf(mx0, t);
          t = __uint_as_float(r[e + 5]) + bf16_hi(bq.z); r[e + 5] = __float_as_uint(t); mx1 = fmaxf(mx1, t);
          t = __uint_as_float(r[e + 6]) + bf16_lo(bq.w); r[e + 6] = __float_as_uint(t); mx2 = fmaxf(mx2, t);
          t = __uint_as_float(r[e + 7]) + bf16_hi(bq.w); r[e + 7] = __float_as_uint(t); mx3 = fmaxf(mx3, t);
        }
        mbar_arrive(&bias_empty[w]);  // the bias tile may be refilled for the next block
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * LOG2E;
        // the previous P V product must be complete before P (shared memory) or O (TMEM) are touched
        if (kb > 0) {
          if (!mbar_wait(&pv_done[w], (g - 1) & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
          tc_fence_after();
        }
        const bool grow = mx > m_ref + 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? mx : m_ref;
          const float alpha = ex2f_(m_ref - m_new);
          m_ref = m_new;
          l_run *= alpha;
          if (kb > 0) {
            uint32_t o[32];
            tmem_ld32(o_addr, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st32_(o_addr, o);
            tmem_st_wait_();
          }
        }
        if (!mbar_wait(&turn[w], g & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
        // Exponentials two at a time: the exponents are packed to fp16x2 (x <= 8, so 2^x <= 256 fits; the fp16
        // spacing of x costs < 0.5 % relative error in P for every term that matters), one ex2.approx.f16x2
        // serves two keys, and P goes to shared memory as fp16 for the P V product.  Row sums accumulate in four
        // fp16x2 registers (16 terms each, <= 4096) and are combined in fp32.
        __half2 hs[4] = {__float2half2_rn(0.f), __float2half2_rn(0.f), __float2half2_rn(0.f), __float2half2_rn(0.f)};
#pragma unroll
        for (int c8 = 0; c8 < 16; ++c8) {  // 8 keys -> one 16-byte store
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x0 = fmaf(__uint_as_float(r[c8 * 8 + 2 * e]), LOG2E, -m_ref);
            const float x1 = fmaf(__uint_as_float(r[c8 * 8 + 2 * e + 1]), LOG2E, -m_ref);
            const __half2 xh = __floats2half2_rn(x0, x1);
            uint32_t ph;
            asm("ex2.approx.f16x2 %0, %1;" : "=r"(ph) : "r"(*reinterpret_cast<const uint32_t*>(&xh)));
            hs[e] = __hadd2(hs[e], *reinterpret_cast<const __half2*>(&ph));
            pk[e] = ph;
          }
          *reinterpret_cast<uint4*>(myP + (c8 >> 3) * A2_T + ((uint32_t(c8 & 7) ^ rsw) << 4)) =
              make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(hs[e]);
          ls0 += f.x;
          ls1 += f.y;
        }
        l_run += ls0 + ls1;
        mbar_arrive(&turn[w ^ 1]);
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&p_ready[w]);
      }
      if (!okay || KB == 0) break;
      // item epilogue: O / l, gate, store.  The next item's first logits are already being produced.
      if (!mbar_wait(&pv_done[w], (g - 1) & 1, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
      tc_fence_after();
      uint32_t o[32];
      tmem_ld32(o_addr, o);
      tmem_ld_wait();
      tc_fence_before();
      if (qvalid) {
        const int col = hp * 64 + w * D;
        const float inv = __fdividef(1.f, l_run);
        const bf16* grow_ = p.qkvg + (long long)b * p.batch_stride + (long long)qi * p.seq_stride + p.g_col0 + col;
        bf16* orow = p.out + (long long)b * p.out_batch_stride + (long long)qi * p.out_seq_stride + col;
#pragma unroll
        for (int g8 = 0; g8 < D / 8; ++g8) {
          const uint4 gu = *reinterpret_cast<const uint4*>(grow_ + g8 * 8);
          const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
          uint32_t ow[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float o0 = __uint_as_float(o[g8 * 8 + 2 * e]) * inv * sigmoidf_fast(bf16_lo(gw[e]));
            const float o1 = __uint_as_float(o[g8 * 8 + 2 * e + 1]) * inv * sigmoidf_fast(bf16_hi(gw[e]));
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
    // 1e9 * (mask - 1) as in the reference, floored at -60000: any such logit still exponentiates to exactly 0
    // next to an unmasked one, while a row whose keys are ALL masked keeps fp32-resolvable logits (at 1e9 the
    // fp32 spacing is 64, which would turn into exponents of +-128 and overflow the fp16 exponentials)
    if (k < S) v = mask ? fmaxf(1.0e9f * (mask[bb * mask_ld + k] - 1.f), -60000.f) : 0.f;
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

// fp32 [H][S][S] -> bf16 [H][S][ldq] (same query-major order, padded row pitch): the layout the kernel's
// pair-bias tensor map expects.
__global__ void bias_convert_kernel(const float* __restrict__ in, bf16* __restrict__ out, long long rows, int S, int ldq) {
  const long long n = rows * ldq;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / ldq;
    const int k = int(idx % ldq);
    out[idx] = __float2bfloat16(k < S ? in[r * S + k] : 0.f);
  }
}

int launch_bias_transpose(Ctx* c, const float* in, bf16* out, int H, int S, int ldq, cudaStream_t st) {
  if (H <= 0 || S <= 0) return XFOLD_OK;
  const long long rows = (long long)H * S;
  long long blocks = (rows * ldq + 255) / 256;
  if (blocks > 16384) blocks = 16384;
  ProfScope ps(c, XFOLD_K_MASK_BIAS, st);
  bias_convert_kernel<<<(int)blocks, 256, 0, st>>>(in, out, rows, S, ldq);
  return check_launch(c, "bias_convert_kernel");
}

// qkvg: projection buffer ([B][S][width], or [S][B][width] when transposed); biasT: bf16 [heads][query][ldq];
// mext: tiles from launch_mext ([B][KB][2048] or one row shared by all batch rows when mext_rows == 1).
int launch_attention2(Ctx* c, const bf16* qkvg, int width, int S, int B, int transposed, int q_col0, int k_col0,
                      int v_col0, int g_col0, int heads, const bf16* biasT, int ldq, const bf16* mext, int mext_rows,
                      bf16* out, long long out_seq_stride, long long out_batch_stride, cudaStream_t st) {
  if ((width & 7) || (ldq & 7) || (heads & 1)) return fail(c, XFOLD_ERR_ARG, "attention: width and bias pitch must be multiples of 8, heads even");
  if (S <= 0 || B <= 0) return XFOLD_OK;
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
  ok = ok && make_tmap_bf16_3d(&tmb, biasT, S, S, heads, ldq, (uint64_t)ldq * S, 64, 128, 1);  // dims: key, query, head
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
  a.heads = heads;
  static bool attr_done[8] = {false};
  if (!attr_done[c->device & 7]) {
    cudaError_t e = cudaFuncSetAttribute(attn2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "attention smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  const long long items = (long long)((S + 127) / 128) * (heads / 2) * B;
  const int grid = (int)(items < c->sm_count ? items : c->sm_count);
  ProfScope ps(c, XFOLD_K_ATTENTION, st);
  attn2_kernel<<<grid, A2_THREADS, A2_SMEM, st>>>(tm, tmb, a);
  return check_launch(c, "attn2_kernel");
}

}  // namespace xf
