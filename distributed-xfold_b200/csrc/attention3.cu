// Gated multi-head attention with an additive pair bias and a key mask (TriangleAttention: 4 heads x 32;
// AttentionPairBias: 16 heads x 24 padded to 32 in the trunk, 16 x 48 padded to 64 in the diffusion transformer).
// The softmax warps never touch global memory.
//
// Work item = 128 queries of one batch row x 128 projection columns: four heads of 32 (D = 32, 24 warps) or two heads of
// 64 (D = 64, 16 warps); CTAs are persistent (one per SM) and run their items' 64-key blocks as one continuous sequence.
//   warps 0 and 7   : TMA producers.  Warp 0: Q per item (two 64-column boxes) and per 64-key block the K tile (+ the 2 KB
//                     mask-bias tile); warp 7: the V tile per block; two stages each.  (One lane doing all of it was
//                     measured as a pacemaker of the kernel.)
//   warps 1..NH     : tcgen05.mma issuers, one per head, so that no head ever waits for another; warp-uniform code, one
//                     elected lane.  Per block:
//                         S  = Q K^T              (K = D, N = 64)
//                         S += E1 * Mext^T        (K = 16; column 0 of E1 is all ones, column 0 of Mext is the
//                                                  additive mask bias of each key)
//                         O += P V                (K = 64, N = D; P read from tensor memory, O stays there for the item)
//                     Each issuer also fetches its head's pair-bias tiles (32-key halves, a ring of three).
//   warps 8..8+4NH-1: one softmax warpgroup per head, one thread per query row.
//
// Why this shape.  The exponential unit (16 results per clock and SM) sets the floor: 4 x 128 x 64 exponentials per block
// are 2048 clocks of it.  Four warps per scheduler need a thread to fit in ~100 registers (setmaxnreg moves registers from
// the control warps to the softmax warps), so a thread loads the block's 64 logits, releases the logits buffer (the issuer
// already computes the next block's), and sweeps them in two halves of 32: exponent, exponential, 16 packed probabilities
// stored, then the other half, then P is published.  Tensor memory is exactly full with single buffers for D = 32:
// 4 x 64 columns of logits, 4 x 32 of output, 4 x 32 of probabilities.
//
// The sweep exponentiates against the running reference exponent m_ref of the PREVIOUS halves,
//     x = s * log2(e) - m_ref + bias'   (fp32; bias' = bias * log2(e) as delivered, FP16, added with the mixed-precision add),
//     ex2.approx (fp32), P packed to fp16 pairs, row sum as fp16x2 partial sums of 8 terms,
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

constexpr int A3_CTRL = 8;                       // two control warpgroups: TMA producer, four MMA issuers, three idle warps
constexpr int A3_REGS_CTRL = 32, A3_REGS_SOFTMAX = 104;  // registers per thread after the re-balancing at kernel start
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

// D = head dimension (32: four heads per work item, 64: two; either way an item's Q / K / V tiles are 128 columns wide)
template <int D>
__global__ void __launch_bounds__((A3_CTRL + 4 * (128 / D)) * 32, 1)
attn3_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmkv,
             const __grid_constant__ CUtensorMap tmb, const Attn3Args p) {
  static_assert(D == 32 || D == 64, "head dimension 32 or 64");
  constexpr int NH = 128 / D;                       // heads per work item = softmax warpgroups
  constexpr int THREADS = (A3_CTRL + 4 * NH) * 32;
  constexpr float LOG2E = 1.4426950408889634f;
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
  uint64_t* q_empty = bars + 1;    // [1] all four issuers have committed the item's last logits
  uint64_t* k_full = bars + 2;     // [2]
  uint64_t* k_empty = bars + 4;    // [2] all four issuers have committed the block's logits
  uint64_t* v_full = bars + 6;     // [2]
  uint64_t* v_empty = bars + 8;    // [2] all four issuers have committed the block's P V product
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
  const int QT = (p.S + 127) / 128, HG = p.heads / NH;
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
    mbar_init(q_empty, NH);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], NH);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], NH);
    }
    for (int w = 0; w < 4; ++w) {
      mbar_init(&sb_full[w * 2], 3);
      mbar_init(&sb_full[w * 2 + 1], 3);
      mbar_init(&s_free[w], 4);   // one elected lane per softmax warp
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
  for (uint32_t i = threadIdx.x; i < 4096 / 16; i += THREADS) reinterpret_cast<uint4*>(sE1)[i] = make_uint4(0, 0, 0, 0);
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

  // Register re-balancing (whole warpgroups): the control warps run single threads with a handful of values, the
  // softmax threads hold a block's 64 logits and 16 packed probabilities.
  // (With two heads per item the CTA has 512 threads and every thread 128 registers from the start.)
  if (warp < A3_CTRL) {
    if constexpr (NH == 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(A3_REGS_CTRL));
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
          }
        }
      }
    } else if (warp == 7) {
      // ------------------------------------------------------------------------------------------- TMA producer of V
      if (lane == 0) {
        uint32_t j = 0;
        bool okay = true;
        for (uint32_t it = 0; it < my_items && okay; ++it) {
          int qt, hg, b;
          decode(it, qt, hg, b);
          for (int kb = 0; kb < KB; ++kb, ++j) {
            const uint32_t st = j & 1u, par = ((j >> 1) & 1u) ^ 1u;
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
    } else if (warp <= NH) {
      // ------------------------------------------------------------------------------------------- MMA issuer of head w
      // The whole warp runs this code with identical values in every lane (waits included), and one elected lane issues
      // the tensor-core and TMA instructions: descriptors and counters are warp-uniform, built once outside the loop.
      {
        const int w = warp - 1;
        const bool leader = elect_one();
        constexpr uint32_t idesc_s = make_idesc(128, 64);
        constexpr uint32_t idesc_pv = make_idesc(128, D, 0, 1, 1);  // P and V are fp16 (V N-major): the v columns of the
                                                                    // projection buffer are written as fp16 by the GEMM
        // D = 32: head w lives in 64-column box w / 2, in the upper or lower 64 bytes of its 128-byte swizzled rows;
        // D = 64: head w is box w
        const uint32_t box = D == 32 ? uint32_t(w >> 1) : uint32_t(w), in_row = D == 32 ? uint32_t(w & 1) * 64u : 0u;
        const uint32_t k_off = box * (A3_KV / 2) + in_row;
        const uint64_t e1d = make_sdesc_noswizzle(smem_u32(sE1), 128, 256);
        const uint64_t qd = make_sdesc(smem_u32(sQ) + box * (A3_Q / 2) + in_row, 16, 1024);
        const uint64_t kd0 = make_sdesc(smem_u32(sK) + k_off, 16, 1024);
        const uint64_t mxd0 = make_sdesc_noswizzle(smem_u32(sMext), 128, 256);
        const uint64_t vd0 = make_sdesc(smem_u32(sV) + k_off, 16384, 1024);  // V is N-major: 16 keys = 2048 B
        const uint32_t d_s = tmem_base + w * 64, d_o = tmem_base + A3_TM_O + w * D, a_p = tmem_base + A3_TM_P + w * 32;
        uint64_t* my_sb = sb_full + w * 2;
        const uint32_t my_bias = smem_u32(sBias) + w * A3_BS * A3_BT;
        bool okay = true;
        // next block whose logits are issued (one ahead of the softmax), tracked without divisions
        uint32_t aj = 0, ait = 0;
        int akb = 0;
        auto issue_s = [&]() -> bool {
          const uint32_t ks = aj & 1u;
          if (akb == 0 && !mbar_wait(q_full, ait & 1u, ab, XF_ERR_WAIT_FULL)) return false;
          if (!mbar_wait(&k_full[ks], (aj >> 1) & 1u, ab, XF_ERR_WAIT_FULL)) return false;
          tc_fence_after();
          if (leader) {
            const uint64_t kd = kd0 + uint64_t(ks * (A3_KV >> 4));   // descriptor start address counts 16-byte units
#pragma unroll
            for (int j = 0; j < D / 16; ++j)  // 16 head-dimension columns = 32 B inside the swizzled row
              umma_ss(d_s, qd + uint64_t(2 * j), kd + uint64_t(2 * j), idesc_s, j ? 1u : 0u);
            umma_ss(d_s, e1d, mxd0 + uint64_t(ks * (2048 >> 4)), idesc_s, 1u);
            umma_commit(&my_sb[ks]);  // ks = block & 1
            umma_commit(&k_empty[ks]);
            if (akb == KB - 1) umma_commit(q_empty);  // last use of this item's Q tile
          }
          ++aj;
          if (++akb == KB) {
            akb = 0;
            ++ait;
          }
          return true;
        };
        // next bias tile to fetch: half bi of the CTA's block sequence = (item, key block, half)
        uint32_t bi = 0, bslot = 0, bit = 0;
        int bkey = 0, bqt, bhg, bb_;
        decode(0, bqt, bhg, bb_);
        const int key_end = KB * 64;
        auto issue_bias = [&]() {
          if (leader) {
            uint64_t* bar = &my_sb[(bi >> 1) & 1u];  // the barrier of the block this half belongs to
            mbar_arrive_expect_tx(bar, A3_BT);
            asm volatile(
                "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                ::"r"(my_bias + bslot * A3_BT), "l"(&tmb), "r"(smem_u32(bar)), "r"(bkey), "r"(bqt * 128), "r"(bhg * NH + w)
                : "memory");
          }
          ++bi;
          if (++bslot == A3_BS) bslot = 0;
          bkey += 32;
          if (bkey == key_end) {
            bkey = 0;
            ++bit;
            decode(bit, bqt, bhg, bb_);
          }
        };
        const uint32_t n_half = 2u * G;
        while (bi < uint32_t(A3_BS) && bi < n_half) issue_bias();
        if (G > 0) okay = issue_s();
        int kb = 0;  // key block of block g within its item
        for (uint32_t g = 0; g < G && okay; ++g) {
          const uint32_t par = g & 1u, vs = g & 1u, vpar = (g >> 1) & 1u;
          // the softmax warps hold S(g) in registers: the logits buffer is free for block g + 1
          if (!mbar_wait(&s_free[w], par, ab, XF_ERR_WAIT_ATTN)) break;
          if (g + 1 < G && !issue_s()) break;
          // the bias tile of the block's first half has been used up
          if (!mbar_wait(&b_free[w], par, ab, XF_ERR_WAIT_ATTN)) break;
          if (bi < n_half) issue_bias();
          const bool v_ready = mbar_test_wait(&v_full[vs], vpar);
          if (!mbar_wait(&p_ready[w], par, ab, XF_ERR_WAIT_ATTN)) break;
          if (!v_ready && !mbar_wait(&v_full[vs], vpar, ab, XF_ERR_WAIT_FULL)) break;
          tc_fence_after();
          if (leader) {
            const uint64_t vd = vd0 + uint64_t(vs * (A3_KV >> 4));
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)  // 16 keys = 2048 B of V = 8 columns of P; O accumulates over the item
              umma_ts(d_o, a_p + ks * 8, vd + uint64_t(ks * (2048 >> 4)), idesc_pv, (kb | ks) ? 1u : 0u);
            umma_commit(&pv_done[w]);
            umma_commit(&v_empty[vs]);
          }
          if (bi < n_half) issue_bias();
          if (++kb == KB) kb = 0;
        }
      }
    }
  } else {
    if constexpr (NH == 4) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(A3_REGS_SOFTMAX));
    // ------------------------------------------------------------------------------------------- softmax warps
    const int w = (warp - A3_CTRL) >> 2;
    const int q4 = warp & 3;  // TMEM lane quarter this warp may access
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + w * 64 + lane_addr;
    const uint32_t o_addr = tmem_base + A3_TM_O + w * D + lane_addr;
    const uint32_t p_addr = tmem_base + A3_TM_P + w * 32 + lane_addr;
    const uint32_t bsw = uint32_t(row >> 1) & 3u;  // 64-byte swizzle: 16-byte chunk index XOR (row / 2) % 4
    const uint8_t* my_bias = sBias + w * A3_BS * A3_BT + row * 64;
    uint64_t* my_sb = sb_full + w * 2;
    const uint32_t FULL = 0xffffffffu;
    uint32_t g = 0, bslot = 0;  // block number; bias ring position
    bool okay = true;
    for (uint32_t it = 0; it < my_items && okay; ++it) {
      int qt, hg, b;
      decode(it, qt, hg, b);
      const int qi = qt * 128 + row;
      const bool qvalid = qi < p.S;
      // m_ref: exponent offset in use (log2 units); it follows the running maximum lazily (see the file header).
      float m_ref = -3.0e38f, l_run = 0.f;
      bool next_ready = false;  // probe of this block's barrier, made before the previous block's second sweep
      for (int kb = 0; kb < KB && okay; ++kb, ++g) {
        // ONE wait per block: the logits and both bias tiles.  A barrier round trip costs a few hundred cycles even when
        // the phase is long complete, so it is probed a sweep ahead, and everything else is probed early and consumed late.
        // (Fetching the next block's logits before this block's probabilities are published was measured: slower, the
        // fence before the publication waits for the load.)
        if (!__all_sync(FULL, next_ready)) {
          okay = __all_sync(FULL, mbar_wait(&my_sb[g & 1u], (g >> 1) & 1u, ab, XF_ERR_WAIT_ATTN));
          if (!okay) break;
        }
        tc_fence_after();
        uint32_t r[64];
        tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        // While the logits are on their way, the previous block's P (its second store was issued a moment ago) completes:
        // it is published together with the release of the logits buffer, so that neither the completion of that store
        // nor the latency of this load is waited for on its own.  (An item's last block publishes itself.)
        if (kb > 0) tmem_st_wait_();
        tmem_ld_wait();
        // the whole block of logits is in registers: the issuer may overwrite the buffer with the next block's
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&s_free[w]);
          if (kb > 0) mbar_arrive(&p_ready[w]);
        }
        // has the previous block's P V product read P?  (needed before this block's first P store; it is issued about
        // now, so it is probed during the first sweep; an item's first block follows an awaited product)
        bool pv_ok = (kb == 0);
        next_ready = false;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint8_t* bt = my_bias + bslot * A3_BT;
          bool exact = (kb == 0 && h == 0);
          __half2 hs[4];
          uint32_t pk[16];
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
                  mx0 = fmaxf(mx0, fmaf(__uint_as_float(r[h * 32 + c4 * 8 + 2 * e]), LOG2E, bf.x));
                  mx1 = fmaxf(mx1, fmaf(__uint_as_float(r[h * 32 + c4 * 8 + 2 * e + 1]), LOG2E, bf.y));
                }
              }
              const float mx = fmaxf(mx0, mx1);
              const bool grow = mx > m_ref + 8.f;
              if (__any_sync(FULL, grow)) {
                const float m_new = grow ? mx : m_ref;
                const float alpha = ex2f_(m_ref - m_new);
                m_ref = m_new;
                l_run *= alpha;
                if (kb > 0) {
                  // every earlier P V product of the item must have landed before O is rescaled
                  okay = __all_sync(FULL, mbar_wait(&pv_done[w], (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN));
                  if (!okay) break;
                  tc_fence_after();
#pragma unroll 1
                  for (int oc = 0; oc < D; oc += 32) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + oc, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                    tmem_st32_(o_addr + oc, o);
                  }
                  tmem_st_wait_();
                }
                if (h == 1) {  // the first half of this block's P is already stored: bring it to the new reference
                  uint32_t q[16];
                  tmem_st_wait_();
                  tmem_ld16_(p_addr, q);
                  tmem_ld_wait();
                  const __half2 a2 = __float2half2_rn(alpha);
#pragma unroll
                  for (int e = 0; e < 16; ++e) {
                    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&q[e]), a2);
                    q[e] = *reinterpret_cast<const uint32_t*>(&v);
                  }
                  tmem_st16_(p_addr, q);
                  tmem_st_wait_();
                }
              }
            }
            // the sweep: exponent, fp16x2 pack, bias, running max, exponential, row sum (8 keys per 16-byte bias read)
            const float nm = -m_ref;
#pragma unroll
            for (int e = 0; e < 4; ++e) hs[e] = __float2half2_rn(0.f);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              // probes whose answers are wanted right after this sweep: issued before its last quarter, so that the
              // barrier's answer time passes behind arithmetic
              if (c4 == 3) {
                if (h == 0 && !pv_ok) pv_ok = mbar_test_wait(&pv_done[w], (g - 1) & 1u);
                if (h == 1 && !next_ready && kb + 1 < KB)
                  next_ready = mbar_test_wait(&my_sb[(g + 1) & 1u], ((g + 1) >> 1) & 1u);
              }
              const uint4 bq = *reinterpret_cast<const uint4*>(bt + ((uint32_t(c4) ^ bsw) << 4));
              const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float x0 = fmaf(__uint_as_float(r[h * 32 + c4 * 8 + 2 * e]), LOG2E, nm);
                float x1 = fmaf(__uint_as_float(r[h * 32 + c4 * 8 + 2 * e + 1]), LOG2E, nm);
                // bias in with the mixed-precision add, fp32 exponentials, one pack per pair: fewer instructions (and a more
                // accurate P) than packing first and exponentiating in fp16x2, which the hardware splits into halves anyway
                asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.f16 %0, lo, %0;\n\tadd.rn.f32.f16 %1, hi, %1;\n\t}"
                : "+f"(x0), "+f"(x1) : "r"(bw[e]));
                const __half2 ph2 = __floats2half2_rn(ex2f_(x0), ex2f_(x1));
                hs[e] = __hadd2(hs[e], ph2);
                pk[c4 * 4 + e] = *reinterpret_cast<const uint32_t*>(&ph2);
              }
            }
            if (exact) break;
            // a probability above 2^8 (x > 8) shows in the partial sum that holds it (8 terms each; an overflow reads inf)
            const float2 bm = __half22float2(__hmax2(__hmax2(hs[0], hs[1]), __hmax2(hs[2], hs[3])));
            if (!__any_sync(FULL, fmaxf(bm.x, bm.y) > 256.f)) break;
            exact = true;  // some row may have outgrown the reference: exact maximum, rescale if so, sweep again
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
          if (h == 0) {
            // the P V product of the previous block must have read P before it is overwritten (probed at the block's start)
            if (!__all_sync(FULL, pv_ok)) pv_ok = mbar_test_wait(&pv_done[w], (g - 1) & 1u);
            if (!__all_sync(FULL, pv_ok)) {
              okay = __all_sync(FULL, mbar_wait(&pv_done[w], (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN));
              if (!okay) break;
            }
            tc_fence_after();
            tmem_st16_(p_addr, pk);  // completes behind the second half's sweep
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_free[w]);  // this half's bias tile has been read by the whole warp
          } else {
            tmem_st16_(p_addr + 16, pk);  // completes behind the next block's load of the logits
          }
          if (++bslot == A3_BS) bslot = 0;
        }
        if (!okay) break;
        if (kb == KB - 1) {  // nothing of this item follows: publish now
          tmem_st_wait_();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_ready[w]);
        }
      }
      if (!okay || KB == 0) break;
      // item epilogue: O / l, gate, store
      okay = __all_sync(FULL, mbar_wait(&pv_done[w], (g - 1) & 1u, ab, XF_ERR_WAIT_ATTN));
      if (!okay) break;
      tc_fence_after();
      const float inv = __fdividef(1.f, l_run);
#pragma unroll 1
      for (int oc = 0; oc < D; oc += 32) {
      uint32_t o[32];
      tmem_ld32(o_addr + oc, o);
      tmem_ld_wait();
      if (oc + 32 == D) tc_fence_before();
      if (qvalid) {
        const int col = hg * 128 + w * D + oc;
        const bf16* grow_ = p.qkvg + (long long)b * p.batch_stride + (long long)qi * p.seq_stride + p.g_col0 + col;
        bf16* orow = p.out + (long long)b * p.out_batch_stride + (long long)qi * p.out_seq_stride + col;
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
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
template <int D>
static int launch_attn3(Ctx* c, int grid, const CUtensorMap& tmq, const CUtensorMap& tmkv, const CUtensorMap& tmb,
                        const Attn3Args& a, cudaStream_t st) {
  static bool attr_done[8] = {false};
  if (!attr_done[c->device & 7]) {
    cudaError_t e = cudaFuncSetAttribute(attn3_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, A3_SMEM);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "attention smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  ProfScope ps(c, c->attn_tag, st);
  attn3_kernel<D><<<grid, (A3_CTRL + 4 * (128 / D)) * 32, A3_SMEM, st>>>(tmq, tmkv, tmb, a);
  return check_launch(c, "attn3_kernel");
}

int launch_attention2(Ctx* c, const bf16* qkvg, int width, int S, int B, int transposed, int q_col0, int k_col0,
                      int v_col0, int g_col0, int heads, const bf16* biasT, int ldq, const bf16* mext, int mext_rows,
                      bf16* out, long long out_seq_stride, long long out_batch_stride, cudaStream_t st, int head_dim) {
  if (head_dim != 32 && head_dim != 64) return fail(c, XFOLD_ERR_ARG, "attention: head dimension must be 32 or 64");
  const int per_item = 128 / head_dim;
  if ((width & 7) || (ldq & 7) || (heads % per_item) || ((q_col0 | k_col0 | v_col0 | g_col0) & 7))
    return fail(c, XFOLD_ERR_ARG, "attention: width, column offsets and bias pitch must be multiples of 8, heads x head dimension a multiple of 128");
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
  const long long items = (long long)((S + 127) / 128) * (heads / per_item) * B;
  if (items * ((S + 63) / 64) >= (1ll << 30)) return fail(c, XFOLD_ERR_ARG, "attention: batch x heads x sequence too large for one launch");
  const int grid = (int)(items < c->sm_count ? items : c->sm_count);
  return head_dim == 32 ? launch_attn3<32>(c, grid, tmq, tmkv, tmb, a, st) : launch_attn3<64>(c, grid, tmq, tmkv, tmb, a, st);
}

}  // namespace xf
