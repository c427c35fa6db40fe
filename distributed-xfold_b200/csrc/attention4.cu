// Gated attention for head dim 32 (TriangleAttention, 4 heads; AttentionPairBias with its 24-wide heads padded to
// 32, 16 heads): the softmax warps never touch global memory, and every wait of theirs hides behind a sweep.
//
// Work item = 128 queries of one batch row x 4 heads; CTAs are persistent (one per SM) and run their items' 64-key
// blocks as one continuous sequence.
//   warp 0        : TMA producer.  Q per item (128 rows x 4 heads x 32 = two 64-column boxes); per 64-key block the K
//                   tile (+ the 2 KB mask-bias tile) and the V tile, two stages each.
//   warps 1, 2    : tcgen05.mma issuers, one per PAIR of heads, warp-uniform code with an elected lane.  Per block and head:
//                       S  = Q K^T              (K = 32, N = 64)
//                       S += E1 * Mext^T        (K = 16; column 0 of E1 is all ones, column 0 of Mext is the
//                                                additive mask bias of each key)
//                       O += P V                (K = 64, N = 32; P read from tensor memory, O stays there for the item)
//                   and the fetch of the heads' pair-bias tiles (32-key halves, a ring of three per head).
//   warps 4..11   : softmax, one thread per query row; a warp serves TWO heads (warps 4-7: heads 0, 1; 8-11: heads 2, 3).
//
// Why this shape.  The exponential unit (16 results per clock and SM) bounds the kernel: 4 x 128 x 64 exponentials
// per block are 2048 clocks of it.  Around every sweep sit operations that cost a warp 250-450 clocks of latency each
// and almost no instructions: the tensor-memory load of the logits, the store of the probabilities and its
// completion, barrier round trips, the publication.  Warps of different heads do not fill these gaps for each other
// reliably (measured with two and with four softmax warps per scheduler: the unit idled half of the time either way).
// So each warp interleaves two heads itself: while it sweeps head A's block, head B's logits are already on their way
// into a second set of registers, and head A's probabilities are published a half-sweep later, when their store has
// long completed.  Two warps per scheduler at ~190 registers hold two 64-logit rows each.
//
// The sweep exponentiates against the running reference exponent m_ref of the PREVIOUS halves,
//     x = s * log2(e) - m_ref (fp32) -> fp16x2,  + bias' (fp16x2; bias' = bias * log2(e) as delivered),
//     ex2.approx.f16x2, row sum (fp16x2 partial sums of 8 terms), P as fp16,
// and only looks at the partial sums afterwards: if one of them exceeds 2^8 in some row of the warp (a P > 256, i.e.
// x > 8, shows there; fp16 would overflow beyond 2^16), the warp takes the exact path -- fp32 row maximum of the half
// still held in registers, O (tensor memory), the row sum and, in a block's second half, the stored first half of P
// rescaled, the sweep repeated.  The first half of an item always takes the exact path.  With trained or random weights
// the repeat is rare afterwards.
//
// The pair bias arrives as FP16 [head][query][key], multiplied by log2(e) (key contiguous, row pitch a multiple of
// 8); TMA lays a [128 queries][32 keys] tile out with the 64-byte swizzle, so the per-row 16-byte reads of the
// softmax threads are bank-conflict free.
#include <cuda_fp16.h>

#include "internal.h"
#include "umma.cuh"

namespace xf {

struct Attn3Args {
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

constexpr int A3_CTRL = 4;                       // control warpgroup: TMA producer, two MMA issuers, one idle warp
constexpr int A3_THREADS = (A3_CTRL + 8) * 32;   // + two softmax warpgroups
// registers per thread after the re-balancing at kernel start (launch: 168; 4 * 32 * (168 - 72) >= 8 * 32 * (216 - 168))
constexpr int A3_REGS_CTRL = 72, A3_REGS_SOFTMAX = 216;
constexpr uint32_t A3_Q = 32768;                 // [2 boxes][128 rows][64 columns]
constexpr uint32_t A3_KV = 16384;                // [2 boxes][64 rows][64 columns]
constexpr uint32_t A3_BT = 8192;                 // bias tile [128 queries][32 keys] fp16
constexpr int A3_BS = 3;                         // bias tiles in flight per head
constexpr uint32_t A3_OFF_Q = 0, A3_OFF_K = A3_Q, A3_OFF_V = A3_OFF_K + 2 * A3_KV, A3_OFF_BIAS = A3_OFF_V + 2 * A3_KV,
                   A3_OFF_E1 = A3_OFF_BIAS + 4 * A3_BS * A3_BT, A3_OFF_MEXT = A3_OFF_E1 + 4096,
                   A3_OFF_BAR = A3_OFF_MEXT + 2 * 2048;
constexpr uint32_t A3_SMEM = A3_OFF_BAR + 512 + 1024;
// TMEM columns: logits S of head w at w*64 (64 columns); output O of head w at 256 + w*32; probabilities P of head w at
// 384 + w*32 (64 keys as 32 fp16 pairs).
constexpr uint32_t A3_TM_O = 256, A3_TM_P = 384;

__device__ __forceinline__ float ex2f_(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_ld16_(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16_(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
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
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tmem_st_wait_() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// State of one head inside a softmax thread.
struct A3Head {
  uint32_t s_addr, o_addr, p_addr;  // TMEM addresses (with this warp's lane offset)
  uint64_t *sb, *s_free, *b_free, *p_ready, *pv_done;
  const uint8_t* bias;              // this row's 64 bytes inside bias slot 0
  float m_ref, l_run;               // exponent offset in use (log2 units, follows the running maximum lazily) and row sum
};

// One half (32 keys) of a block for one head: x, exponentials, row sum; pk receives the packed probabilities.
// r: the block's 64 logits of this thread's row.  Returns false when a bounded wait ran out.
template <int HALF>
__device__ __forceinline__ bool a3_sweep_half(A3Head& H, const uint32_t (&r)[64], uint32_t (&pk)[16], const uint8_t* bt,
                                              uint32_t bsw, int kb, uint32_t g, const AbortCtx& ab) {
  constexpr float LOG2E = 1.4426950408889634f;
  constexpr uint32_t FULL = 0xffffffffu;
  bool exact = (kb == 0 && HALF == 0);
  __half2 hs[4];
  for (;;) {
    if (exact) {
      // fp32 maximum of this half; move the reference if it grew by more than 2^8
      float mx0 = -3.0e38f, mx1 = -3.0e38f;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const uint4 bq = *reinterpret_cast<const uint4*>(bt + ((uint32_t(c4) ^ bsw) << 4));
        const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 bf = __half22float2(*reinterpret_cast<const __half2*>(&bw[e]));
          mx0 = fmaxf(mx0, fmaf(__uint_as_float(r[HALF * 32 + c4 * 8 + 2 * e]), LOG2E, bf.x));
          mx1 = fmaxf(mx1, fmaf(__uint_as_float(r[HALF * 32 + c4 * 8 + 2 * e + 1]), LOG2E, bf.y));
        }
      }
      const float mx = fmaxf(mx0, mx1);
      const bool grow = mx > H.m_ref + 8.f;
      if (__any_sync(FULL, grow)) {
        const float m_new = grow ? mx : H.m_ref;
        const float alpha = ex2f_(H.m_ref - m_new);
        H.m_ref = m_new;
        H.l_run *= alpha;
        if (kb > 0) {
          // every earlier P V product of the item must have landed before O is rescaled
          if (!__all_sync(FULL, mbar_wait(H.pv_done, (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN))) return false;
          tc_fence_after();
          uint32_t o[32];
          tmem_ld32(H.o_addr, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32_(H.o_addr, o);
          tmem_st_wait_();
        }
        if (HALF == 1) {  // the first half of this block's P is already stored: bring it to the new reference
          uint32_t q[16];
          tmem_st_wait_();
          tmem_ld16_(H.p_addr, q);
          tmem_ld_wait();
          const __half2 a2 = __float2half2_rn(alpha);
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&q[e]), a2);
            q[e] = *reinterpret_cast<const uint32_t*>(&v);
          }
          tmem_st16_(H.p_addr, q);
          tmem_st_wait_();
        }
      }
    }
    // the sweep: exponent, fp16x2 pack, bias, exponential, row sum (8 keys per 16-byte bias read)
    const float nm = -H.m_ref;
#pragma unroll
    for (int e = 0; e < 4; ++e) hs[e] = __float2half2_rn(0.f);
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const uint4 bq = *reinterpret_cast<const uint4*>(bt + ((uint32_t(c4) ^ bsw) << 4));
      const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x0 = fmaf(__uint_as_float(r[HALF * 32 + c4 * 8 + 2 * e]), LOG2E, nm);
        const float x1 = fmaf(__uint_as_float(r[HALF * 32 + c4 * 8 + 2 * e + 1]), LOG2E, nm);
        const __half2 xh = __hadd2(__floats2half2_rn(x0, x1), *reinterpret_cast<const __half2*>(&bw[e]));
        uint32_t ph;
        asm("ex2.approx.f16x2 %0, %1;" : "=r"(ph) : "r"(*reinterpret_cast<const uint32_t*>(&xh)));
        hs[e] = __hadd2(hs[e], *reinterpret_cast<const __half2*>(&ph));
        pk[c4 * 4 + e] = ph;
      }
    }
    if (exact) break;
    // a probability above 2^8 (x > 8) shows in the partial sum that holds it (8 terms each; an overflow reads inf)
    const float2 bm = __half22float2(__hmax2(__hmax2(hs[0], hs[1]), __hmax2(hs[2], hs[3])));
    if (!__any_sync(FULL, fmaxf(bm.x, bm.y) > 256.f)) break;
    exact = true;  // some row may have outgrown the reference: exact maximum, rescale if so, sweep again
  }
  float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __half22float2(hs[e]);
    ls0 += f.x;
    ls1 += f.y;
  }
  H.l_run += ls0 + ls1;
  return true;
}

__global__ void __launch_bounds__(A3_THREADS, 1)
attn3_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmkv,
             const __grid_constant__ CUtensorMap tmb, const Attn3Args p) {
  constexpr int D = 32;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem + A3_OFF_Q;
  uint8_t* sK = smem + A3_OFF_K;        // [block & 1]
  uint8_t* sV = smem + A3_OFF_V;        // [block & 1]
  uint8_t* sBias = smem + A3_OFF_BIAS;  // [head][half % 3]
  uint8_t* sE1 = smem + A3_OFF_E1;
  uint8_t* sMext = smem + A3_OFF_MEXT;  // [block & 1], 2 KB each
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A3_OFF_BAR);
  uint64_t* q_full = bars;         // [1]
  uint64_t* q_empty = bars + 1;    // [1] the logits of the item's last block are committed for all four heads
  uint64_t* k_full = bars + 2;     // [2]
  uint64_t* k_empty = bars + 4;    // [2] the block's logits are committed for all four heads
  uint64_t* v_full = bars + 6;     // [2]
  uint64_t* v_empty = bars + 8;    // [2] the block's P V product is committed for all four heads
  uint64_t* sb_full = bars + 10;   // [head][block & 1] the logits of a block are in TMEM AND both of its bias tiles have
                                   //        landed (three arrivals: the commit of the logits, the issuer's two expect-tx)
  uint64_t* s_free = bars + 18;    // [head] the softmax warps hold the block's logits in registers
  uint64_t* b_free = bars + 22;    // [head] the bias tile of a block's first half has been used up
  uint64_t* p_ready = bars + 26;   // [head] P of a block is in TMEM (and the bias tile of its second half is used up)
  uint64_t* pv_done = bars + 30;   // [head] P V product of a block complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 34);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // warp index and everything derived from it are the same in all lanes: the shuffle tells the compiler so, which keeps
  // the issuers' descriptors and counters out of per-thread registers
  const int warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const int KB = (p.S + 63) / 64;
  // Persistent CTA: work items (batch row, head group of 4, query tile), batch row slowest so that the K / V rows of
  // the ~gridDim.x items in flight stay in L2.  Every role walks the same sequence of blocks; block numbers (and with
  // them buffer indices and barrier phases) keep counting across items.
  const int QT = (p.S + 127) / 128, HG = p.heads / 4;
  const long long n_items = (long long)p.B * HG * QT;
  const uint32_t my_items = n_items > blockIdx.x ? uint32_t((n_items - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0u;
  const uint32_t G = my_items * uint32_t(KB);  // blocks this CTA processes in total (the launcher bounds items * KB to 2^30)
  auto decode = [&](uint32_t it, int& qt, int& hg, int& b) {
    const uint32_t t = blockIdx.x + it * gridDim.x;
    qt = int(t % uint32_t(QT));
    hg = int((t / uint32_t(QT)) % uint32_t(HG));
    b = int(t / uint32_t(QT * HG));
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 4);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 4);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 4);
    }
    for (int w = 0; w < 4; ++w) {
      mbar_init(&sb_full[w * 2], 3);
      mbar_init(&sb_full[w * 2 + 1], 3);
      mbar_init(&s_free[w], 4);   // one elected lane per softmax warp of the head
      mbar_init(&p_ready[w], 4);
      mbar_init(&b_free[w], 4);
      mbar_init(&pv_done[w], 1);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmq);
    tma_prefetch_desc(&tmkv);
    tma_prefetch_desc(&tmb);
  }
  // constant operand E1: un-swizzled [128][16] tile whose column 0 is all ones
  for (uint32_t i = threadIdx.x; i < 4096 / 16; i += A3_THREADS) reinterpret_cast<uint4*>(sE1)[i] = make_uint4(0, 0, 0, 0);
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
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);

  // Register re-balancing (whole warpgroups): the control warps run a handful of warp-uniform values, a softmax thread
  // holds two 64-logit rows and 16 packed probabilities.
  if (warp < A3_CTRL) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(A3_REGS_CTRL));
  else asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(A3_REGS_SOFTMAX));

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t j = 0;  // block number
      bool okay = true;
      for (uint32_t it = 0; it < my_items && okay; ++it) {
        int qt, hg, b;
        decode(it, qt, hg, b);
        if (!mbar_wait(q_empty, (it & 1u) ^ 1u, ab, XF_ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(q_full, A3_Q);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int col = p.q_col0 + hg * 128 + x * 64;
          if (p.transposed) tma_load_3d(sQ + x * (A3_Q / 2), &tmq, q_full, col, b, qt * 128);
          else tma_load_3d(sQ + x * (A3_Q / 2), &tmq, q_full, col, qt * 128, b);
        }
        const bf16* mrow = p.mext + (long long)b * p.mext_batch_stride;
        for (int kb = 0; kb < KB; ++kb, ++j) {
          const uint32_t st = j & 1u, par = ((j >> 1) & 1u) ^ 1u;
          if (!mbar_wait(&k_empty[st], par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&k_full[st], A3_KV + 2048);
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int col = p.k_col0 + hg * 128 + x * 64;
            if (p.transposed) tma_load_3d(sK + st * A3_KV + x * (A3_KV / 2), &tmkv, &k_full[st], col, b, kb * 64);
            else tma_load_3d(sK + st * A3_KV + x * (A3_KV / 2), &tmkv, &k_full[st], col, kb * 64, b);
          }
          bulk_load(sMext + st * 2048, mrow + (long long)kb * 1024, 2048, &k_full[st]);
          if (!mbar_wait(&v_empty[st], par, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&v_full[st], A3_KV);
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int col = p.v_col0 + hg * 128 + x * 64;
            if (p.transposed) tma_load_3d(sV + st * A3_KV + x * (A3_KV / 2), &tmkv, &v_full[st], col, b, kb * 64);
            else tma_load_3d(sV + st * A3_KV + x * (A3_KV / 2), &tmkv, &v_full[st], col, kb * 64, b);
          }
        }
      }
    }
  } else if (warp < 3) {
    // ------------------------------------------------------------------------------- MMA issuer of heads 2 * pair, 2 * pair + 1
    // The whole warp runs this code with identical values in every lane (waits included), and one elected lane issues
    // the tensor-core and TMA instructions.  It serves its two heads' events in the order in which the softmax warps
    // raise them (see the softmax role): per block  s_free(A), b_free(A), p_ready(B, previous block), s_free(B), b_free(B),
    // p_ready(A);  at the end of an item p_ready(B) follows p_ready(A) at once.
    const int pair = warp - 1;
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc(128, 64);
    constexpr uint32_t idesc_pv = make_idesc(128, D, 0, 1, 1);  // P and V are fp16 (V N-major): the v columns of the
                                                                // projection buffer are written as fp16 by the GEMM
    const uint64_t e1d = make_sdesc_noswizzle(smem_u32(sE1), 128, 256);
    const uint64_t mxd0 = make_sdesc_noswizzle(smem_u32(sMext), 128, 256);
    // heads 2 * pair + x live in 64-column box `pair`, in the lower (x = 0) or upper (x = 1) 64 bytes of its 128-byte rows
    const uint32_t box = uint32_t(pair) * (A3_KV / 2);
    const uint64_t qd0 = make_sdesc(smem_u32(sQ) + uint32_t(pair) * (A3_Q / 2), 16, 1024);
    const uint64_t kd0 = make_sdesc(smem_u32(sK) + box, 16, 1024);
    const uint64_t vd0 = make_sdesc(smem_u32(sV) + box, 16384, 1024);  // V is N-major: 16 keys = 2048 B
    bool okay = true;
    // per head x: next block whose logits are issued (one ahead of the softmax); next bias half to fetch
    uint32_t aj[2] = {0, 0}, ait[2] = {0, 0}, bi[2] = {0, 0};
    int akb[2] = {0, 0}, bkey[2] = {0, 0};
    uint32_t bslot[2] = {0, 0}, bit[2] = {0, 0};
    int bqt, bhg, bb_;
    decode(0, bqt, bhg, bb_);
    int bq_[2] = {bqt * 128, bqt * 128}, bh_[2] = {bhg * 4 + pair * 2, bhg * 4 + pair * 2 + 1};
    const int key_end = KB * 64;
    const uint32_t n_half = 2u * G;
    auto issue_s = [&](int x) -> bool {
      const int w = pair * 2 + x;
      const uint32_t ks = aj[x] & 1u;
      if (akb[x] == 0 && !mbar_wait(q_full, ait[x] & 1u, ab, XF_ERR_WAIT_FULL)) return false;
      if (!mbar_wait(&k_full[ks], (aj[x] >> 1) & 1u, ab, XF_ERR_WAIT_FULL)) return false;
      tc_fence_after();
      if (leader) {
        const uint32_t d_s = tmem_base + w * 64;
        const uint64_t qd = qd0 + uint64_t(x * 4);                              // + 64 bytes
        const uint64_t kd = kd0 + uint64_t(ks * (A3_KV >> 4) + x * 4);          // descriptor addresses count 16-byte units
        umma_ss(d_s, qd, kd, idesc_s, 0u);
        umma_ss(d_s, qd + 2, kd + 2, idesc_s, 1u);
        umma_ss(d_s, e1d, mxd0 + uint64_t(ks * (2048 >> 4)), idesc_s, 1u);
        umma_commit(&sb_full[w * 2 + ks]);  // ks = block & 1
        umma_commit(&k_empty[ks]);
        if (akb[x] == KB - 1) umma_commit(q_empty);  // last use of this item's Q tile
      }
      ++aj[x];
      if (++akb[x] == KB) {
        akb[x] = 0;
        ++ait[x];
      }
      return true;
    };
    auto issue_bias = [&](int x) {
      if (bi[x] >= n_half) return;
      const int w = pair * 2 + x;
      if (leader) {
        uint64_t* bar = &sb_full[w * 2 + ((bi[x] >> 1) & 1u)];  // the barrier of the block this half belongs to
        mbar_arrive_expect_tx(bar, A3_BT);
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(smem_u32(sBias) + (w * A3_BS + bslot[x]) * A3_BT), "l"(&tmb), "r"(smem_u32(bar)), "r"(bkey[x]), "r"(bq_[x]),
              "r"(bh_[x])
            : "memory");
      }
      ++bi[x];
      if (++bslot[x] == A3_BS) bslot[x] = 0;
      bkey[x] += 32;
      if (bkey[x] == key_end) {
        bkey[x] = 0;
        ++bit[x];
        int qt, hg, b;
        decode(bit[x], qt, hg, b);
        bq_[x] = qt * 128;
        bh_[x] = hg * 4 + pair * 2 + x;
      }
    };
    auto issue_pv = [&](int x, uint32_t g, int kb) -> bool {
      const int w = pair * 2 + x;
      const uint32_t vs = g & 1u, vpar = (g >> 1) & 1u;
      if (!mbar_wait(&p_ready[w], g & 1u, ab, XF_ERR_WAIT_ATTN)) return false;
      if (!mbar_wait(&v_full[vs], vpar, ab, XF_ERR_WAIT_FULL)) return false;
      tc_fence_after();
      if (leader) {
        const uint32_t d_o = tmem_base + A3_TM_O + w * 32, a_p = tmem_base + A3_TM_P + w * 32;
        const uint64_t vd = vd0 + uint64_t(vs * (A3_KV >> 4) + x * 4);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // 16 keys = 2048 B of V = 8 columns of P; O accumulates over the item
          umma_ts(d_o, a_p + ks * 8, vd + uint64_t(ks * (2048 >> 4)), idesc_pv, (kb | ks) ? 1u : 0u);
        umma_commit(&pv_done[w]);
        umma_commit(&v_empty[vs]);
      }
      issue_bias(x);
      return true;
    };
    for (int x = 0; x < 2; ++x)
      for (int i = 0; i < A3_BS; ++i) issue_bias(x);
    if (G > 0) okay = issue_s(0) && issue_s(1);
    int kb = 0;        // key block of block g within its item
    bool b_pending = false;  // head B's P V product of block g - 1 is still to be issued
    for (uint32_t g = 0; g < G && okay; ++g) {
      const uint32_t par = g & 1u;
      // head A: logits in registers -> next block's logits; first bias half used up -> next tile
      if (!mbar_wait(&s_free[pair * 2], par, ab, XF_ERR_WAIT_ATTN)) break;
      if (g + 1 < G && !issue_s(0)) break;
      if (!mbar_wait(&b_free[pair * 2], par, ab, XF_ERR_WAIT_ATTN)) break;
      issue_bias(0);
      // head B's probabilities of the previous block (published half a sweep late)
      if (b_pending) {
        if (!issue_pv(1, g - 1, kb == 0 ? KB - 1 : kb - 1)) break;
        b_pending = false;
      }
      if (!mbar_wait(&s_free[pair * 2 + 1], par, ab, XF_ERR_WAIT_ATTN)) break;
      if (g + 1 < G && !issue_s(1)) break;
      if (!mbar_wait(&b_free[pair * 2 + 1], par, ab, XF_ERR_WAIT_ATTN)) break;
      issue_bias(1);
      if (!issue_pv(0, g, kb)) break;
      if (kb == KB - 1) {  // end of an item: head B publishes at once
        if (!issue_pv(1, g, kb)) break;
      } else {
        b_pending = true;
      }
      if (++kb == KB) kb = 0;
    }
  } else if (warp >= A3_CTRL) {
    // ------------------------------------------------------------------------------------------- softmax warps
    // Program order per block g, heads A and B of this warp (every wait named here is either long satisfied or probed ahead):
    //   logits A in registers -> s_free(A);   fetch logits B (tensor-memory load in flight during A's sweeps)
    //   sweep A first half  -> store P(A) first half, b_free(A);   publish P(B, g - 1) (its store completed long ago)
    //   sweep A second half -> store P(A) second half
    //   logits B in registers -> s_free(B);   fetch logits A of block g + 1
    //   sweep B first half  -> store P(B) first half, b_free(B);   publish P(A, g)
    //   sweep B second half -> store P(B) second half              (published in block g + 1, or at once at an item's end)
    const int pair = (warp - A3_CTRL) >> 2;
    const int q4 = warp & 3;  // TMEM lane quarter this warp may access
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const uint32_t bsw = uint32_t(row >> 1) & 3u;  // 64-byte swizzle: 16-byte chunk index XOR (row / 2) % 4
    constexpr uint32_t FULL = 0xffffffffu;
    A3Head H[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int w = pair * 2 + x;
      H[x].s_addr = tmem_base + w * 64 + lane_addr;
      H[x].o_addr = tmem_base + A3_TM_O + w * 32 + lane_addr;
      H[x].p_addr = tmem_base + A3_TM_P + w * 32 + lane_addr;
      H[x].sb = sb_full + w * 2;
      H[x].s_free = s_free + w;
      H[x].b_free = b_free + w;
      H[x].p_ready = p_ready + w;
      H[x].pv_done = pv_done + w;
      H[x].bias = sBias + w * A3_BS * A3_BT + row * 64;
      H[x].m_ref = -3.0e38f;
      H[x].l_run = 0.f;
    }
    uint32_t g = 0, bslot = 0;  // block number; bias ring position (the same for both heads)
    bool okay = true;
    uint32_t rA[64], rB[64], pk[16];
    bool b_unpublished = false;  // P(B) of the previous block is stored but not yet published
    auto publish = [&](A3Head& h) {
      tmem_st_wait_();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(h.p_ready);
    };
    auto fetch = [&](A3Head& h, uint32_t blk, uint32_t (&r)[64]) -> bool {
      if (!__all_sync(FULL, mbar_wait(&h.sb[blk & 1u], (blk >> 1) & 1u, ab, XF_ERR_WAIT_ATTN))) return false;
      tc_fence_after();
      tmem_ld32(h.s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_ld32(h.s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
      return true;
    };
    auto arrive = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    // item epilogue of one head: O / l, gate, store
    auto finish = [&](A3Head& h, int x, int qt, int hg, int b) -> bool {
      if (!__all_sync(FULL, mbar_wait(h.pv_done, (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN))) return false;
      tc_fence_after();
      uint32_t o[32];
      tmem_ld32(h.o_addr, o);
      tmem_ld_wait();
      tc_fence_before();
      const int qi = qt * 128 + row;
      if (qi < p.S) {
        const int col = hg * 128 + (pair * 2 + x) * D;
        const float inv = __fdividef(1.f, h.l_run);
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
      h.m_ref = -3.0e38f;
      h.l_run = 0.f;
      return true;
    };
    if (G > 0) okay = fetch(H[0], 0, rA);
    for (uint32_t it = 0; it < my_items && okay; ++it) {
      int qt, hg, b;
      decode(it, qt, hg, b);
      for (int kb = 0; kb < KB && okay; ++kb, ++g) {
        // has the previous block's P V product read P?  (needed before this block's first P store; probed here, used later)
        bool pvA = (g == 0) || mbar_test_wait(H[0].pv_done, (g - 1) & 1u);
        // ---------------------------------------------------------------- head A
        tmem_ld_wait();  // logits A (fetched during the previous block's head-B sweeps)
        tc_fence_before();
        arrive(H[0].s_free);
        if (!(okay = fetch(H[1], g, rB))) break;
        const uint32_t slot0 = bslot, slot1 = bslot + 1 == A3_BS ? 0 : bslot + 1;
        if (!(okay = a3_sweep_half<0>(H[0], rA, pk, H[0].bias + slot0 * A3_BT, bsw, kb, g, ab))) break;
        if (!__all_sync(FULL, pvA)) pvA = mbar_test_wait(H[0].pv_done, (g - 1) & 1u);
        if (!__all_sync(FULL, pvA) && !(okay = __all_sync(FULL, mbar_wait(H[0].pv_done, (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN)))) break;
        tc_fence_after();
        tmem_st16_(H[0].p_addr, pk);
        arrive(H[0].b_free);
        if (b_unpublished) {  // P(B) of the previous block: stored a whole half-sweep ago
          publish(H[1]);
          b_unpublished = false;
        }
        bool pvB = (g == 0) || mbar_test_wait(H[1].pv_done, (g - 1) & 1u);
        if (!(okay = a3_sweep_half<1>(H[0], rA, pk, H[0].bias + slot1 * A3_BT, bsw, kb, g, ab))) break;
        tmem_st16_(H[0].p_addr + 16, pk);
        // ---------------------------------------------------------------- head B
        tmem_ld_wait();  // logits B
        tc_fence_before();
        arrive(H[1].s_free);
        if (g + 1 < G && !(okay = fetch(H[0], g + 1, rA))) break;
        if (!(okay = a3_sweep_half<0>(H[1], rB, pk, H[1].bias + slot0 * A3_BT, bsw, kb, g, ab))) break;
        if (!__all_sync(FULL, pvB)) pvB = mbar_test_wait(H[1].pv_done, (g - 1) & 1u);
        if (!__all_sync(FULL, pvB) && !(okay = __all_sync(FULL, mbar_wait(H[1].pv_done, (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN)))) break;
        tc_fence_after();
        tmem_st16_(H[1].p_addr, pk);
        arrive(H[1].b_free);
        publish(H[0]);  // P(A) of this block: its second half was stored a half-sweep ago
        if (!(okay = a3_sweep_half<1>(H[1], rB, pk, H[1].bias + slot1 * A3_BT, bsw, kb, g, ab))) break;
        tmem_st16_(H[1].p_addr + 16, pk);
        b_unpublished = true;
        bslot = slot1 + 1 == A3_BS ? 0 : slot1 + 1;
      }
      if (!okay || KB == 0) break;
      // end of the item: publish head B at once, then normalise, gate and store both heads' outputs
      publish(H[1]);
      b_unpublished = false;
      if (!(okay = finish(H[0], 0, qt, hg, b))) break;
      if (!(okay = finish(H[1], 1, qt, hg, b))) break;
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

// fp32 [H][S][S] -> 16-bit [H][S][ldq] (same query-major order, padded row pitch): FP16 values times log2(e), the operand
// the kernel's pair-bias tensor map expects (the kernel works in base 2 and adds the tile as it is).
__global__ void bias_convert_kernel(const float* __restrict__ in, __half* __restrict__ out, long long rows, int S, int ldq) {
  const long long n = rows * ldq;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / ldq;
    const int k = int(idx % ldq);
    out[idx] = __float2half_rn(k < S ? fminf(fmaxf(in[r * S + k] * 1.4426950408889634f, -60000.f), 60000.f) : 0.f);
  }
}

int launch_bias_transpose(Ctx* c, const float* in, bf16* out, int H, int S, int ldq, cudaStream_t st) {
  if (H <= 0 || S <= 0) return XFOLD_OK;
  const long long rows = (long long)H * S;
  long long blocks = (rows * ldq + 255) / 256;
  if (blocks > 16384) blocks = 16384;
  ProfScope ps(c, XFOLD_K_MASK_BIAS, st);
  bias_convert_kernel<<<(int)blocks, 256, 0, st>>>(in, reinterpret_cast<__half*>(out), rows, S, ldq);
  return check_launch(c, "bias_convert_kernel");
}

// qkvg: projection buffer ([B][S][width], or [S][B][width] when transposed); biasT: 16-bit [heads][query][ldq] holding FP16
// values; mext: tiles from launch_mext ([B][KB][2048] or one row shared by all batch rows when mext_rows == 1).
int launch_attention2(Ctx* c, const bf16* qkvg, int width, int S, int B, int transposed, int q_col0, int k_col0,
                      int v_col0, int g_col0, int heads, const bf16* biasT, int ldq, const bf16* mext, int mext_rows,
                      bf16* out, long long out_seq_stride, long long out_batch_stride, cudaStream_t st) {
  if ((width & 7) || (ldq & 7) || (heads & 3) || ((q_col0 | k_col0 | v_col0 | g_col0) & 7))
    return fail(c, XFOLD_ERR_ARG, "attention: width, column offsets and bias pitch must be multiples of 8, heads a multiple of 4");
  if (S <= 0 || B <= 0) return XFOLD_OK;
  CUtensorMap tmq, tmkv, tmb;
  bool ok;
  Attn3Args a;
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
  // dims: key, query, head; [128 queries][32 keys] tiles with 64-byte rows
  ok = ok && make_tmap_bf16_3d(&tmb, biasT, S, S, heads, ldq, (uint64_t)ldq * S, 32, 128, 1, 64);
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
    cudaError_t e = cudaFuncSetAttribute(attn3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A3_SMEM);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "attention smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  const long long items = (long long)((S + 127) / 128) * (heads / 4) * B;
  if (items * ((S + 63) / 64) >= (1ll << 30)) return fail(c, XFOLD_ERR_ARG, "attention: batch x heads x sequence too large for one launch");
  const int grid = (int)(items < c->sm_count ? items : c->sm_count);
  ProfScope ps(c, c->attn_tag, st);
  attn3_kernel<<<grid, A3_THREADS, A3_SMEM, st>>>(tmq, tmkv, tmb, a);
  return check_launch(c, "attn3_kernel");
}

}  // namespace xf
