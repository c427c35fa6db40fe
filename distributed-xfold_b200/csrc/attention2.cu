// Second-generation gated attention for head dim 32 (TriangleAttention; AttentionPairBias with the
// 24-wide heads padded to 32): the softmax warps never touch global memory.
//
// Work item = 128 queries of one batch row x 2 heads (one head per softmax warpgroup); CTAs are persistent
// (one per SM) and run their items' 64-key blocks as one continuous, double-buffered sequence.
//   warp 0      : TMA producer.  Q per item; per 64-key block the K tile (+ the 2 KB mask-bias tile) and the V
//                 tile; two stages each.
//   warps 1, 10 : tcgen05.mma issuers, one per warpgroup, so that the two heads never wait for each other.
//                 Per block:  S  = Q K^T                      (K = 32, N = 64)
//                             S += E1 * Mext^T                (K = 16; column 0 of E1 is all ones, column 0
//                                                              of Mext is the additive mask bias of each key)
//                             O += P V                        (K = 64, N = 32; O stays in TMEM for the item)
//                 S and P are double-buffered: S(n+2) is issued when the warpgroup publishes P(n), so logits
//                 are always waiting when a softmax pass starts.  The issuer also fetches its warpgroup's
//                 bf16 pair-bias tile two blocks ahead.
//   warps 2..5 / 6..9 : softmax warpgroups, one thread per query row.
//
// The exponential unit (16 lanes per SM) is the bound of this kernel: 2 x 128 x 64 exponentials per block are
// 2 x 512 cycles of it, and measurements show that it only overlaps with the other pipes when ONE warp's
// instruction stream interleaves both kinds of work -- a warp that takes maxima while another one
// exponentiates does not overlap with it.  The softmax pass is therefore a single sweep per block that
// exponentiates against the running reference exponent m_ref of the PREVIOUS blocks,
//     x = s * log2(e) + bias' - m_ref  (fp32; bias' = bias * log2(e) as delivered)  ->  fp16x2  ->  running max (fp16x2), ex2.approx.f16x2,
//     row sum (fp16x2 partial sums), P as fp16 into a swizzled K-major tile,
// and only looks at the block maximum afterwards: if some row of the warp saw x > 8 (P > 256; fp16 would
// overflow beyond 2^16), the warp takes the exact path -- fp32 row maximum from the logits still held in
// registers, O (TMEM) and the row sum rescaled, the sweep repeated.  The first block of an item always takes
// the exact path.  With trained or random weights the repeat is rare after the first block, so the common
// block costs one sweep.
//
// The pair bias arrives as bf16 [head][query][key], multiplied by log2(e) (key contiguous, row pitch a multiple of 8); TMA lays a
// [128 queries][64 keys] tile out with the 128-byte swizzle, so the per-row 16-byte reads of the softmax
// threads are bank-conflict free.
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

constexpr int A2_THREADS = 352;   // TMA warp, 2 MMA warps, 2 x 4 softmax warps
constexpr uint32_t A2_T = 16384;  // [128][64] 2-byte tile
constexpr uint32_t A2_H = 8192;   // [64][64] 2-byte tile
constexpr int A2_KV = 4;           // K / V stages: their rows come from DRAM (~1.3 us under load), three blocks of lead
// Q[2], K[4], V[4], bias[2 warpgroups][2], E1, Mext[4], barriers
constexpr uint32_t A2_OFF_Q = 0, A2_OFF_K = 2 * A2_T, A2_OFF_V = 4 * A2_T, A2_OFF_BIAS = 6 * A2_T,
                   A2_OFF_E1 = 10 * A2_T, A2_OFF_MEXT = 10 * A2_T + 4096, A2_OFF_BAR = 10 * A2_T + 4096 + 8192;
// TMEM columns: logits S of warpgroup w, buffer s at w*128 + s*64 (64 columns); output O of warpgroup w at
// 256 + w*32; probabilities P of warpgroup w, buffer s at 320 + w*64 + s*32 (64 keys as 32 fp16 pairs).
constexpr uint32_t A2_TM_O = 256, A2_TM_P = 320;
constexpr uint32_t A2_SMEM = A2_OFF_BAR + 512 + 1024;

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
attn2_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmkv,
             const __grid_constant__ CUtensorMap tmb, const Attn2Args p) {
  constexpr int D = 32;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem + A2_OFF_Q;        // [item & 1]
  uint8_t* sK = smem + A2_OFF_K;        // [block & 3], 8 KB each
  uint8_t* sV = smem + A2_OFF_V;        // [block & 3], 8 KB each
  uint8_t* sBias = smem + A2_OFF_BIAS;  // [warpgroup][block & 1]: [128 queries][64 keys] bf16
  uint8_t* sE1 = smem + A2_OFF_E1;
  uint8_t* sMext = smem + A2_OFF_MEXT;  // [block & 3], 2 KB each
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A2_OFF_BAR);
  uint64_t* q_full = bars;            // [2]
  uint64_t* q_empty = bars + 2;       // [2] both issuers have committed the item's last logits
  uint64_t* k_full = bars + 4;        // [4]
  uint64_t* k_empty = bars + 8;       // [4] both issuers have committed the block's logits
  uint64_t* v_full = bars + 12;       // [4]
  uint64_t* v_empty = bars + 16;      // [4] both issuers have committed the block's P V product
  uint64_t* sb_full = bars + 20;      // [warpgroup][2] logits of a block are in TMEM and its bias tile has landed
  uint64_t* pv_done = bars + 24;      // [warpgroup][2] P V product of a block complete
  uint64_t* p_ready = bars + 28;      // [warpgroup][2] P of a block is in TMEM (and its logits, bias consumed).  One
                                      // barrier per buffer: a warp may finish block g + 1 (its logits are waiting)
                                      // before a slower warp of the warpgroup has finished block g, and its arrival
                                      // must not be counted for block g.
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const int KB = (p.S + 63) / 64;
  // Persistent CTA: work items (batch row, head pair, query tile), batch row slowest so that the K / V rows of
  // the ~gridDim.x items in flight stay in L2.  Every role walks the same sequence of blocks; block numbers
  // (and with them buffer indices and barrier phases) keep counting across items.
  const int QT = (p.S + 127) / 128, HP = p.heads / 2;
  const long long n_items = (long long)p.B * HP * QT;
  const uint32_t my_items = n_items > blockIdx.x ? uint32_t((n_items - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0u;
  const uint32_t G = my_items * uint32_t(KB);  // blocks this CTA processes in total (the launcher bounds items * KB to 2^31)
  auto decode = [&](uint32_t it, int& qt, int& hp, int& b) {
    const uint32_t t = blockIdx.x + it * gridDim.x;
    qt = int(t % uint32_t(QT));
    hp = int((t / uint32_t(QT)) % uint32_t(HP));
    b = int(t / uint32_t(QT * HP));
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 2);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&p_ready[s], 128);
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 2);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 2);
      mbar_init(&sb_full[s], 2);  // the issuer's expect-tx arrival for the bias tile + the commit of the logits
      mbar_init(&pv_done[s], 1);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmq);
    tma_prefetch_desc(&tmkv);
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
      uint32_t j = 0;  // block number
      bool okay = true;
      for (uint32_t it = 0; it < my_items && okay; ++it) {
        int qt, hp, b;
        decode(it, qt, hp, b);
        const uint32_t qs = uint32_t(it & 1), qpar = uint32_t((it >> 1) & 1);
        if (!mbar_wait(&q_empty[qs], qpar ^ 1u, ab, XF_ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(&q_full[qs], A2_T);
        if (p.transposed) tma_load_3d(sQ + qs * A2_T, &tmq, &q_full[qs], p.q_col0 + hp * 64, b, qt * 128);
        else tma_load_3d(sQ + qs * A2_T, &tmq, &q_full[qs], p.q_col0 + hp * 64, qt * 128, b);
        const bf16* mrow = p.mext + (long long)b * p.mext_batch_stride;
        for (int kb = 0; kb < KB; ++kb, ++j) {
          const uint32_t st = uint32_t(j & (A2_KV - 1)), par = uint32_t((j / A2_KV) & 1) ^ 1u;
          if (!mbar_wait(&k_empty[st], par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&k_full[st], A2_H + 2048);
          if (p.transposed) tma_load_3d(sK + st * A2_H, &tmkv, &k_full[st], p.k_col0 + hp * 64, b, kb * 64);
          else tma_load_3d(sK + st * A2_H, &tmkv, &k_full[st], p.k_col0 + hp * 64, kb * 64, b);
          bulk_load(sMext + st * 2048, mrow + (long long)kb * 1024, 2048, &k_full[st]);
          if (!mbar_wait(&v_empty[st], par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&v_full[st], A2_H);
          if (p.transposed) tma_load_3d(sV + st * A2_H, &tmkv, &v_full[st], p.v_col0 + hp * 64, b, kb * 64);
          else tma_load_3d(sV + st * A2_H, &tmkv, &v_full[st], p.v_col0 + hp * 64, kb * 64, b);
        }
      }
    }
  } else if (warp == 1 || warp == 10) {
    if (lane == 0) {
      const int w = warp == 1 ? 0 : 1;
      constexpr uint32_t idesc_s = make_idesc(128, 64);
      constexpr uint32_t idesc_pv = make_idesc(128, D, 0, 1, 1);  // P and V are fp16 (V N-major): the v columns of the
                                                                  // projection buffer are written as fp16 by the GEMM
      const uint64_t e1d = make_sdesc_noswizzle(smem_u32(sE1), 128, 256);
      // The block whose logits and bias tile are issued next (two blocks ahead of the P V products), tracked
      // incrementally: this thread's instruction stream is the pacemaker of its warpgroup, so it carries no
      // divisions and probes the K / V barriers before it parks on p_ready.
      uint32_t aj = 0, ait = 0;
      int akb = 0, aqt, ahp, ab_;
      decode(0, aqt, ahp, ab_);
      auto issue_ahead = [&](bool k_ready) -> bool {
        const uint32_t s = aj & 1u, ks = aj & uint32_t(A2_KV - 1), kpar = (aj / A2_KV) & 1u;
        if (akb == 0 && !mbar_wait(&q_full[ait & 1], (ait >> 1) & 1u, ab, XF_ERR_WAIT_FULL)) return false;
        if (!k_ready && !mbar_wait(&k_full[ks], kpar, ab, XF_ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + w * 128 + s * 64;
        const uint64_t qd = make_sdesc(smem_u32(sQ) + (ait & 1u) * A2_T + w * 64, 16, 1024);
        const uint64_t kd = make_sdesc(smem_u32(sK) + ks * A2_H + w * 64, 16, 1024);
        const uint64_t mxd = make_sdesc_noswizzle(smem_u32(sMext) + ks * 2048, 128, 256);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_ss(d, qd + 2 * k, kd + 2 * k, idesc_s, k ? 1u : 0u);
        umma_ss(d, e1d, mxd, idesc_s, 1u);
        umma_commit(&sb_full[w * 2 + s]);
        umma_commit(&k_empty[ks]);
        if (akb == KB - 1) umma_commit(&q_empty[ait & 1]);  // last use of this item's Q tile
        mbar_arrive_expect_tx(&sb_full[w * 2 + s], A2_T);
        tma_load_3d(sBias + (w * 2 + s) * A2_T, &tmb, &sb_full[w * 2 + s], akb * 64, aqt * 128, ahp * 2 + w);
        ++aj;
        if (++akb == KB) {
          akb = 0;
          ++ait;
          decode(ait, aqt, ahp, ab_);
        }
        return true;
      };
      bool okay = true;
      while (aj < 2 && aj < G && okay) okay = issue_ahead(false);
      int kb = 0;  // key block of block g within its item
      for (uint32_t g = 0; g < G && okay; ++g) {
        const uint32_t s = g & 1u, vs = g & uint32_t(A2_KV - 1), vpar = (g / A2_KV) & 1u;
        // K and V tiles are fetched blocks ahead: probe their barriers now, so that the round trips overlap the wait below
        const bool v_ready = mbar_test_wait(&v_full[vs], vpar);
        const bool k_ready = aj < G && mbar_test_wait(&k_full[aj & uint32_t(A2_KV - 1)], (aj / A2_KV) & 1u);
        if (!mbar_wait(&p_ready[w * 2 + s], (g >> 1) & 1u, ab, XF_ERR_WAIT_ATTN)) break;
        // P(g) is published (and with it the logits buffer and bias tile of block g are free for block g + 2)
        if (!v_ready && !mbar_wait(&v_full[vs], vpar, ab, XF_ERR_WAIT_FULL)) break;
        tc_fence_after();
        const uint32_t pt = tmem_base + A2_TM_P + w * 64 + s * 32;
        const uint32_t vbase = smem_u32(sV) + vs * A2_H + w * 64;
        const uint32_t d = tmem_base + A2_TM_O + w * 32;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t bd = make_sdesc(vbase + ks * 2048, A2_T, 1024);  // V is N-major: 16 keys = 2048 B
          umma_ts(d, pt + ks * 8, bd, idesc_pv, (kb | ks) ? 1u : 0u);     // 16 keys = 8 columns of P; O accumulates
        }
        umma_commit(&pv_done[w * 2 + s]);
        umma_commit(&v_empty[vs]);
        if (++kb == KB) kb = 0;
        if (aj < G) okay = issue_ahead(k_ready);
      }
    }
  } else {
    const int w = (warp - 2) >> 2;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + w * 128 + lane_addr;
    const uint32_t o_addr = tmem_base + A2_TM_O + w * 32 + lane_addr;
    const uint32_t p_addr = tmem_base + A2_TM_P + w * 64 + lane_addr;
    const uint32_t rsw = uint32_t(row & 7);
    uint32_t g = 0;  // block number
    bool okay = true;
    bool ready = false;  // the probe of this block's barrier, made before the previous block's sweep, succeeded
    for (uint32_t it = 0; it < my_items && okay; ++it) {
      int qt, hp, b;
      decode(it, qt, hp, b);
      const int qi = qt * 128 + row;
      const bool qvalid = qi < p.S;
      // m_ref: exponent offset in use (log2 units); it follows the running maximum lazily (see the file header).
      float m_ref = -3.0e38f, l_run = 0.f;
      for (int kb = 0; kb < KB; ++kb, ++g) {
        const uint32_t s = uint32_t(g & 1), par = uint32_t((g >> 1) & 1);
        const uint8_t* myBias = sBias + (w * 2 + s) * A2_T + row * 128;
        // One barrier covers the logits and the bias tile.  It also covers the P buffer: the issuer queued
        // S(g) behind the P V product of block g - 2, so P buffer s has been consumed when S(g) is complete.
        if (!ready && !mbar_wait(&sb_full[w * 2 + s], par, ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
        tc_fence_after();
        uint32_t r[64];
        tmem_ld32(s_addr + s * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(s_addr + s * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        ready = mbar_test_wait(&sb_full[w * 2 + (s ^ 1u)], uint32_t(((g + 1) >> 1) & 1));  // probe block g + 1
        tmem_ld_wait();
        bool exact = kb == 0;
        __half2 hs[4];
        uint32_t pk[32];
        for (;;) {
          if (exact) {
            // fp32 row maximum of this block; move the reference if it grew by more than 2^8
            float mx0 = -3.0e38f, mx1 = -3.0e38f, mx2 = -3.0e38f, mx3 = -3.0e38f;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
              const uint4 bq = *reinterpret_cast<const uint4*>(myBias + ((uint32_t(c8) ^ rsw) << 4));
              const int e = c8 * 8;
              mx0 = fmaxf(mx0, fmaf(__uint_as_float(r[e + 0]), LOG2E, bf16_lo(bq.x)));
              mx1 = fmaxf(mx1, fmaf(__uint_as_float(r[e + 1]), LOG2E, bf16_hi(bq.x)));
              mx2 = fmaxf(mx2, fmaf(__uint_as_float(r[e + 2]), LOG2E, bf16_lo(bq.y)));
              mx3 = fmaxf(mx3, fmaf(__uint_as_float(r[e + 3]), LOG2E, bf16_hi(bq.y)));
              mx0 = fmaxf(mx0, fmaf(__uint_as_float(r[e + 4]), LOG2E, bf16_lo(bq.z)));
              mx1 = fmaxf(mx1, fmaf(__uint_as_float(r[e + 5]), LOG2E, bf16_hi(bq.z)));
              mx2 = fmaxf(mx2, fmaf(__uint_as_float(r[e + 6]), LOG2E, bf16_lo(bq.w)));
              mx3 = fmaxf(mx3, fmaf(__uint_as_float(r[e + 7]), LOG2E, bf16_hi(bq.w)));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            const bool grow = mx > m_ref + 8.f;
            if (__any_sync(0xffffffffu, grow)) {
              const float m_new = grow ? mx : m_ref;
              const float alpha = ex2f_(m_ref - m_new);
              m_ref = m_new;
              l_run *= alpha;
              if (kb > 0) {
                // every earlier P V product of the item must have landed before O is rescaled
                const uint32_t gp = g - 1;
                if (!mbar_wait(&pv_done[w * 2 + (gp & 1)], uint32_t((gp >> 1) & 1), ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
                tc_fence_after();
                uint32_t o[32];
                tmem_ld32(o_addr, o);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                tmem_st32_(o_addr, o);
                tmem_st_wait_();
              }
            }
          }
          // the sweep: exponent, fp16x2 pack, running max, exponential, row sum, P store (8 keys per 16-byte store)
          const float nm = -m_ref;
          __half2 hm = __float2half2_rn(-65504.f);
#pragma unroll
          for (int e = 0; e < 4; ++e) hs[e] = __float2half2_rn(0.f);
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const uint4 bq = *reinterpret_cast<const uint4*>(myBias + ((uint32_t(c8) ^ rsw) << 4));
            const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x0 = fmaf(__uint_as_float(r[c8 * 8 + 2 * e]), LOG2E, nm);
              float x1 = fmaf(__uint_as_float(r[c8 * 8 + 2 * e + 1]), LOG2E, nm);
              // the bias tile is in log2 units already: one mixed-precision add per key, straight from the packed pair
              asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %1, hi, %1;\n\t}"
                  : "+f"(x0), "+f"(x1) : "r"(bw[e]));
              const __half2 xh = __floats2half2_rn(x0, x1);
              hm = __hmax2(hm, xh);
              uint32_t ph;
              asm("ex2.approx.f16x2 %0, %1;" : "=r"(ph) : "r"(*reinterpret_cast<const uint32_t*>(&xh)));
              hs[e] = __hadd2(hs[e], *reinterpret_cast<const __half2*>(&ph));
              pk[c8 * 4 + e] = ph;
            }
          }
          if (exact) break;
          const float2 bm = __half22float2(hm);
          if (!__any_sync(0xffffffffu, fmaxf(bm.x, bm.y) > 8.f)) break;
          exact = true;  // some row outgrew the reference: exact maximum, rescale, sweep again
        }
        if (!okay) break;
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(hs[e]);
          ls0 += f.x;
          ls1 += f.y;
        }
        l_run += ls0 + ls1;
        tmem_st32_(p_addr + s * 32, pk);
        tmem_st_wait_();
        tc_fence_before();
        mbar_arrive(&p_ready[w * 2 + s]);
      }
      if (!okay || KB == 0) break;
      // item epilogue: O / l, gate, store (the next item's logits are already waiting)
      {
        const uint32_t gp = g - 1;
        if (!mbar_wait(&pv_done[w * 2 + (gp & 1)], uint32_t((gp >> 1) & 1), ab, XF_ERR_WAIT_ATTN)) { okay = false; break; }
      }
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
    // an aborted wait may have left copies in flight: give them time to land before the CTA's memory is released
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

// fp32 [H][S][S] -> bf16 [H][S][ldq] (same query-major order, padded row pitch) times log2(e): the operand the
// kernel's pair-bias tensor map expects (the kernel works in base 2 and adds the tile as it is).
__global__ void bias_convert_kernel(const float* __restrict__ in, bf16* __restrict__ out, long long rows, int S, int ldq) {
  const long long n = rows * ldq;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / ldq;
    const int k = int(idx % ldq);
    out[idx] = __float2bfloat16(k < S ? in[r * S + k] * 1.4426950408889634f : 0.f);
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
  CUtensorMap tmq, tmkv, tmb;
  bool ok;
  Attn2Args a;
  if (!transposed) {
    ok = make_tmap_bf16_3d(&tmq, qkvg, width, S, B, width, (uint64_t)width * S, 64, 128, 1) &&
         make_tmap_bf16_3d(&tmkv, qkvg, width, S, B, width, (uint64_t)width * S, 64, 64, 1);
    a.seq_stride = width;
    a.batch_stride = (long long)S * width;
  } else {
    ok = make_tmap_bf16_3d(&tmq, qkvg, width, B, S, width, (uint64_t)width * B, 64, 1, 128) &&
         make_tmap_bf16_3d(&tmkv, qkvg, width, B, S, width, (uint64_t)width * B, 64, 1, 64);
    a.seq_stride = (long long)B * width;
    a.batch_stride = width;
  }
  ok = ok && make_tmap_bf16_3d(&tmb, biasT, S, S, heads, ldq, (uint64_t)ldq * S, 64, 128, 1);  // dims: key, query, head
  if (!ok) return fail(c, XFOLD_ERR_ARG, "attention: cannot encode tensor maps");
  const int KB = (S + 127) / 128;  // 128-key mask tiles (two 64-key blocks each)
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
  if (items * ((S + 63) / 64) >= (1ll << 31)) return fail(c, XFOLD_ERR_ARG, "attention: batch x heads x sequence too large for one launch");
  const int grid = (int)(items < c->sm_count ? items : c->sm_count);
  ProfScope ps(c, c->attn_tag, st);
  attn2_kernel<<<grid, A2_THREADS, A2_SMEM, st>>>(tmq, tmkv, tmb, a);
  return check_launch(c, "attn2_kernel");
}

}  // namespace xf
