// Persistent, warp-specialised bf16 GEMM  D[m][n] = sum_k A[m][k] * B[n][k]  for sm_100a.
//
//   warp 0      : TMA producer (one elected lane), 128-byte-swizzled K-major tiles, STAGES-deep ring
//   warp 1      : tcgen05.mma issuer (one elected lane); owns the TMEM allocation (2 accumulators)
//   warps 2..9  : epilogue; two warps share each 32-lane quarter of the 128-row accumulator (one per
//                 half of the columns) and drain it with tcgen05.ld while the MMA warp already fills
//                 the other buffer.  Row-major outputs leave through 128-byte-swizzled staging tiles
//                 and TMA stores; residual and gate tiles of the 128-wide configuration come in by TMA.
//
// Every projection of the Pairformer block, the SwiGLU transition and the per-channel N x N x N
// TriangleMultiplication contraction (batched over the 128 channels) run through this kernel; they
// differ only in the tensor maps and in the epilogue that is fused behind the accumulator.
#include <cuda_fp16.h>

#include "internal.h"
#include "umma.cuh"

namespace xf {

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps

constexpr uint32_t EPI_TILE = 128 * 64 * 2;  // one staged [128 rows][64 columns] bf16 chunk, 128-byte swizzled

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = 4;
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  // after the operand ring: 2 output chunks; with 128-wide tiles also 2 residual and 2 gate chunks
  static constexpr uint32_t OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr uint32_t OFF_RES = OFF_OUT + 2 * EPI_TILE;
  static constexpr uint32_t OFF_GATE = OFF_RES + 2 * EPI_TILE;
  static constexpr uint32_t OFF_BAR = (BN == 128) ? OFF_GATE + 2 * EPI_TILE : OFF_RES;
  static constexpr uint32_t SMEM_BYTES = OFF_BAR + 256 /*barriers*/ + 1024 /*align slack*/;
};

__device__ __forceinline__ void store8_bf16(bf16* dst, const float* v, int nvalid, bool vec_ok) {
  if (nvalid >= 8 && vec_ok) {
    uint4 u;
    u.x = pack_bf16x2(v[0], v[1]);
    u.y = pack_bf16x2(v[2], v[3]);
    u.z = pack_bf16x2(v[4], v[5]);
    u.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(dst) = u;
  } else {
    for (int e = 0; e < 8; ++e)
      if (e < nvalid) dst[e] = __float2bfloat16(v[e]);
  }
}
__device__ __forceinline__ void load8_bf16(const bf16* src, float* v, int nvalid, bool vec_ok) {
  if (nvalid >= 8 && vec_ok) {
    const uint4 u = *reinterpret_cast<const uint4*>(src);
    v[0] = bf16_lo(u.x); v[1] = bf16_hi(u.x); v[2] = bf16_lo(u.y); v[3] = bf16_hi(u.y);
    v[4] = bf16_lo(u.z); v[5] = bf16_hi(u.z); v[6] = bf16_lo(u.w); v[7] = bf16_hi(u.w);
  } else {
    for (int e = 0; e < 8; ++e) v[e] = (e < nvalid) ? __bfloat162float(src[e]) : 0.f;
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmR,
               const __grid_constant__ CUtensorMap tmG, const GemmArgs p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  // residual / gate chunks are prefetched by TMA only in the 128-wide gate/residual configuration
  constexpr bool EPI_LOADS = (EPI == EPI_GATE_RESID) && (BN == 128);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* efull = tempty + 2;   // [2] residual / gate chunk landed
  uint64_t* eempty = efull + 2;   // [2] residual / gate chunk consumed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(eempty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], 8);
      mbar_init(&efull[s], 1);
      mbar_init(&eempty[s], 8);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int KB = (p.K + BK - 1) / BK;
  const long long total = (long long)p.batches * p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, echunk = 0;
      bool okay = true;
      (void)echunk;
      for (long long t = blockIdx.x; t < total && okay; t += gridDim.x) {
        const int tn = int(t % p.tiles_n);
        const int tm = int((t / p.tiles_n) % p.tiles_m);
        const int b = int(t / ((long long)p.tiles_n * p.tiles_m));
        int a1, a2;
        if (p.a_row_mode == 0) { a1 = tm * BM; a2 = b; }
        else { a1 = tm % p.a_dim1; a2 = (tm / p.a_dim1) * BM; }
        const int bb = p.b_batched ? b : 0;
        if constexpr (EPI_LOADS) {
          const uint32_t nload = (p.resid ? 1u : 0u) + (p.gate ? 1u : 0u);
          if (nload) {
            for (int c = 0; c < BN / 64 && okay; ++c, ++echunk) {
              const uint32_t eb = echunk & 1u;
              if (!mbar_wait(&eempty[eb], ((echunk >> 1) & 1u) ^ 1u, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
              mbar_arrive_expect_tx(&efull[eb], nload * EPI_TILE);
              if (p.resid) tma_load_3d(smem + Cfg::OFF_RES + eb * EPI_TILE, &tmR, &efull[eb], tn * BN + c * 64, tm * BM, 0);
              if (p.gate) tma_load_3d(smem + Cfg::OFF_GATE + eb * EPI_TILE, &tmG, &efull[eb], tn * BN + c * 64, tm * BM, 0);
            }
            if (!okay) break;
          }
        }
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* sA = smem + stage * Cfg::STAGE_BYTES;
          if (!p.mn_major) {
            tma_load_3d(sA, &tmA, &full[stage], kb * BK, a1, a2);
            tma_load_3d(sA + Cfg::A_BYTES, &tmB, &full[stage], kb * BK, tn * BN, bb);
          } else {
            // operands stored [k][m] / [k][n]: one [64 k][64 m] box (8 KB, 128-byte rows) per 64 rows of the tile
#pragma unroll
            for (int x = 0; x < BM / 64; ++x) tma_load_3d(sA + x * 8192, &tmA, &full[stage], a1 + x * 64, kb * BK, a2);
#pragma unroll
            for (int x = 0; x < BN / 64; ++x)
              tma_load_3d(sA + Cfg::A_BYTES + x * 8192, &tmB, &full[stage], tn * BN + x * 64, kb * BK, bb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // MN-major operands (rows of the smem tile are K indices): 64-element chunks along M / N are 8 KB apart, a step of
      // 16 along K is 16 rows of 128 B
      const uint32_t idesc = p.mn_major ? make_idesc(BM, BN, 1, 1) : make_idesc(BM, BN);
      const uint32_t lbo = p.mn_major ? 8192u : 16u, kstep = p.mn_major ? 128u : 2u;
      uint32_t stage = 0, phase = 0, it = 0;
      bool okay = true;
      for (long long t = blockIdx.x; t < total && okay; t += gridDim.x, ++it) {
        const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
        if (!mbar_wait(&tempty[buf], aphase ^ 1u, ab, XF_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&full[stage], phase, ab, XF_ERR_WAIT_FULL)) { okay = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint64_t ad = make_sdesc(sA, lbo, 1024);
          const uint64_t bd = make_sdesc(sA + Cfg::A_BYTES, lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)  // K-major: 16 bf16 = 32 B along K inside the swizzled row
            umma_ss(d, ad + kstep * k, bd + kstep * k, idesc, (kb | k) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (okay) umma_commit(&tfull[buf]);
      }
    }
  } else {
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int ch = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    const int row = q * 32 + lane;
    uint32_t it = 0, ochunk = 0, echunk = 0;
    bool dead = false;
    (void)ochunk; (void)echunk; (void)dead;
    for (long long t = blockIdx.x; t < total; t += gridDim.x, ++it) {
      const int tn = int(t % p.tiles_n);
      const int tm = int((t / p.tiles_n) % p.tiles_m);
      const int b = int(t / ((long long)p.tiles_n * p.tiles_m));
      const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
      // TRIMUL_AB: where this thread's token goes, and its mask value, fetched BEFORE the wait for the accumulator so
      // that the load's latency hides behind the product instead of heading every tile's epilogue
      long long tok = 0, cm_off = 0;
      bool rvalid = false;
      float mk = 1.f;
      if constexpr (EPI == EPI_TRIMUL_AB) {
        if (p.a_row_mode == 0) {
          tok = (long long)tm * BM + row;
          rvalid = tok < p.M;
          const long long i = tok / p.ntok, j = tok - i * p.ntok;
          cm_off = i * p.cm_ld + j;
        } else {
          const long long jf = tm % p.a_dim1, i = (long long)(tm / p.a_dim1) * BM + row;
          rvalid = i * p.ntok < p.M;  // M = rows * ntok
          tok = i * p.ntok + jf;
          cm_off = jf * p.cm_ld + i;
        }
        if (tn < 2 && rvalid && p.mask) mk = p.mask[tok];
      }
      if (!mbar_wait(&tfull[buf], aphase, ab, XF_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(q * 32) << 16);

      if constexpr (EPI != EPI_TRIMUL_AB) {
        // Staged epilogue: the tile leaves in 64-column chunks.  Each of the 8 warps converts its 32 rows x 32
        // columns of the chunk into a 128-byte-swizzled shared-memory tile (conflict-free 16-byte stores), then
        // one thread hands the tile to TMA.  Residual / gate chunks arrive the same way in the other direction.
        constexpr int NCH = (EPI == EPI_SWIGLU) ? BN / 128 : BN / 64;  // output chunks per tile
        constexpr int WOUT = (EPI == EPI_SWIGLU) ? BN / 2 : BN;        // output columns per tile
        const int n_out = (EPI == EPI_SWIGLU) ? p.N / 2 : p.N;
        const long long m = (long long)tm * BM + row;
        const uint32_t rsw = uint32_t(row & 7);
        const bool elected = (warp == 2 && lane == 0);
#pragma unroll 1
        for (int c = 0; c < NCH; ++c, ++ochunk) {
          const int col0 = tn * WOUT + c * 64;          // first output column of the chunk
          const int colw = col0 + ch * 32;              // first output column of this warp
          uint8_t* so = smem + Cfg::OFF_OUT + (ochunk & 1u) * EPI_TILE + row * 128;
          float v[32];
          if constexpr (EPI == EPI_SWIGLU) {
            uint32_t ra[32], rb[32];
            tmem_ld32(taddr + c * 64 + ch * 32, ra);
            tmem_ld32(taddr + BN / 2 + c * 64 + ch * 32, rb);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float x = __uint_as_float(ra[e]);
              v[e] = x * sigmoidf_fast(x) * __uint_as_float(rb[e]);
            }
          } else {
            uint32_t r[32];
            tmem_ld32(taddr + c * 64 + ch * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
          }
          if constexpr (EPI == EPI_PLAIN) {
            if (p.col_bias) {
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] += (colw + e < n_out) ? p.col_bias[colw + e] : 0.f;
            }
            if (p.col_scale) {
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] *= (colw + e < n_out) ? p.col_scale[colw + e] : 0.f;
            }
          }
          if constexpr (EPI == EPI_GATE_RESID) {
            // order: v * sigmoid(gate) first, residual added last
            const bool rvalid = m < p.M;
            bool staged = false;
            uint32_t eb = 0;
            if constexpr (EPI_LOADS) {
              if (p.resid || p.gate) {
                staged = true;
                eb = echunk & 1u;
                if (!mbar_wait(&efull[eb], (echunk >> 1) & 1u, ab, XF_ERR_WAIT_FULL)) dead = true;
                ++echunk;
              }
            }
            if (p.gate) {
              if (staged) {
                const uint8_t* sg = smem + Cfg::OFF_GATE + eb * EPI_TILE + row * 128;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint4 u = *reinterpret_cast<const uint4*>(sg + ((uint32_t(ch * 4 + g) ^ rsw) << 4));
                  const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    v[g * 8 + 2 * e] *= sigmoidf_fast(bf16_lo(w4[e]));
                    v[g * 8 + 2 * e + 1] *= sigmoidf_fast(bf16_hi(w4[e]));
                  }
                }
              } else {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const int col = colw + g * 8, nvalid = rvalid ? n_out - col : 0;
                  if (nvalid <= 0) continue;
                  float t8[8];
                  load8_bf16(p.gate + m * p.ldg + col, t8, nvalid, (p.ldg & 7) == 0);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[g * 8 + e] *= sigmoidf_fast(t8[e]);
                }
              }
            }
            if (p.row_gate) {  // gate shared by rows with equal (row % mod): AdaLN-Zero conditioning of several samples
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int col = colw + g * 8, nvalid = rvalid ? n_out - col : 0;
                if (nvalid <= 0) continue;
                float t8[8];
                load8_bf16(p.row_gate + (m % p.row_gate_mod) * p.ldg + col, t8, nvalid, (p.ldg & 7) == 0);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[g * 8 + e] *= sigmoidf_fast(t8[e]);
              }
            }
            if (p.resid) {
              if (staged) {
                const uint8_t* sr = smem + Cfg::OFF_RES + eb * EPI_TILE + row * 128;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint4 u = *reinterpret_cast<const uint4*>(sr + ((uint32_t(ch * 4 + g) ^ rsw) << 4));
                  const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    v[g * 8 + 2 * e] += bf16_lo(w4[e]);
                    v[g * 8 + 2 * e + 1] += bf16_hi(w4[e]);
                  }
                }
              } else {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const int col = colw + g * 8, nvalid = rvalid ? n_out - col : 0;
                  if (nvalid <= 0) continue;
                  float t8[8];
                  load8_bf16(p.resid + m * p.ldr + col, t8, nvalid, (p.ldr & 7) == 0);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[g * 8 + e] += t8[e];
                }
              }
            }
            if (staged) {
              __syncwarp();
              if (lane == 0) mbar_arrive(&eempty[eb]);
            }
          }
          // the TMA store that last used this staging buffer (two chunks ago) must have read it out
          if (elected) tma_store_wait_read<1>();
          named_bar_sync(1, 256);
          bool as_f16 = false;
          if constexpr (EPI == EPI_PLAIN) as_f16 = colw >= p.f16_col0 && colw < p.f16_col1;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            if (as_f16) {
              u.x = pack_f16x2(v[g * 8 + 0], v[g * 8 + 1]);
              u.y = pack_f16x2(v[g * 8 + 2], v[g * 8 + 3]);
              u.z = pack_f16x2(v[g * 8 + 4], v[g * 8 + 5]);
              u.w = pack_f16x2(v[g * 8 + 6], v[g * 8 + 7]);
            } else {
              u.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
              u.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
              u.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
              u.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
            }
            *reinterpret_cast<uint4*>(so + ((uint32_t(ch * 4 + g) ^ rsw) << 4)) = u;
          }
          fence_proxy_async_smem();
          named_bar_sync(2, 256);
          if (elected && col0 < n_out) {
            tma_store_3d(&tmO, smem + Cfg::OFF_OUT + (ochunk & 1u) * EPI_TILE, col0, tm * BM, b);
            tma_store_commit();
          }
        }
      } else {  // EPI_TRIMUL_AB
        // tile_n 0: [projection | gate] rows of a; 1: the same for b; 2: gating_linear (first 128 columns)
        if (tn < 2) {
          bf16* dst = (tn == 0 ? p.out_a : p.out_b) + cm_off;
#pragma unroll 1
          for (int cc = ch * 2; cc < ch * 2 + 2; ++cc) {
            uint32_t rp[32], rg[32];
            tmem_ld32(taddr + cc * 32, rp);
            tmem_ld32(taddr + 128 + cc * 32, rg);
            tmem_ld_wait();
            if (rvalid) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const float v = __uint_as_float(rp[e]) * mk * sigmoidf_fast(__uint_as_float(rg[e]));
                dst[(long long)(cc * 32 + e) * p.cm_chan_stride] = __float2bfloat16(v);
              }
            }
          }
        } else {
          bf16* orow = p.out_g + tok * 128;
#pragma unroll 1
          for (int cc = ch * 2; cc < ch * 2 + 2; ++cc) {
            uint32_t r[32];
            tmem_ld32(taddr + cc * 32, r);
            tmem_ld_wait();
            if (rvalid) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g8 * 8 + e]);
                store8_bf16(orow + cc * 32 + g8 * 8, v, 8, true);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    if (warp == 2 && lane == 0) tma_store_wait_read<0>();  // staged tiles must be read out before the CTA exits
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    // give TMA copies that were already in flight time to land before the CTA's memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {}
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, int EPI>
static int launch_one(Ctx* c, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  static bool attr_done[8] = {false};
  auto kern = gemm_tn_kernel<BN, EPI>;
  if (!attr_done[c->device & 7]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return fail(c, XFOLD_ERR_LAUNCH, "gemm smem attribute: %s", cudaGetErrorString(e));
    attr_done[c->device & 7] = true;
  }
  const long long total = (long long)a.batches * a.tiles_m * a.tiles_n;
  if (total <= 0) return XFOLD_OK;
  CUtensorMap tmO = tmA, tmR = tmA, tmG = tmA;  // placeholders when unused
  if (EPI != EPI_TRIMUL_AB) {
    const int n_out = (EPI == EPI_SWIGLU) ? a.N / 2 : a.N;
    const uint64_t bstride = a.batches > 1 ? (uint64_t)a.out_batch_stride : (uint64_t)a.ldo * (uint64_t)a.M;
    if (!make_tmap_bf16_3d(&tmO, a.out, n_out, a.M, a.batches, a.ldo, bstride, 64, 128, 1))
      return fail(c, XFOLD_ERR_ARG, "gemm: cannot encode the output tensor map (16-byte aligned base, ld multiple of 8?)");
    if (EPI == EPI_GATE_RESID && BN == 128) {
      if (a.resid && !make_tmap_bf16_3d(&tmR, a.resid, a.N, a.M, 1, a.ldr, (uint64_t)a.ldr * a.M, 64, 128, 1))
        return fail(c, XFOLD_ERR_ARG, "gemm: cannot encode the residual tensor map");
      if (a.gate && !make_tmap_bf16_3d(&tmG, a.gate, a.N, a.M, 1, a.ldg, (uint64_t)a.ldg * a.M, 64, 128, 1))
        return fail(c, XFOLD_ERR_ARG, "gemm: cannot encode the gate tensor map");
    }
  }
  const int sms = c->gemm_sms > 0 && c->gemm_sms < c->sm_count ? c->gemm_sms : c->sm_count;
  const int grid = (int)(total < sms ? total : sms);
  const int tag = EPI == EPI_TRIMUL_AB ? XFOLD_K_TRIMUL_PROJ
                  : EPI == EPI_SWIGLU  ? XFOLD_K_LINEAR_SWIGLU
                  : EPI == EPI_GATE_RESID ? XFOLD_K_LINEAR_GATE_RESID
                  : (a.batches > 1 ? XFOLD_K_TRIMUL_CONTRACT : XFOLD_K_LINEAR);
  ProfScope ps(c, tag, st);
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(tmA, tmB, tmO, tmR, tmG, a);
  return check_launch(c, "gemm_tn_kernel");
}

int launch_gemm(Ctx* c, int epi, int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a,
                cudaStream_t st) {
  if (bn == 256) {
    switch (epi) {
      case EPI_PLAIN: return launch_one<256, EPI_PLAIN>(c, tmA, tmB, a, st);
      case EPI_GATE_RESID: return launch_one<256, EPI_GATE_RESID>(c, tmA, tmB, a, st);
      case EPI_SWIGLU: return launch_one<256, EPI_SWIGLU>(c, tmA, tmB, a, st);
      case EPI_TRIMUL_AB: return launch_one<256, EPI_TRIMUL_AB>(c, tmA, tmB, a, st);
    }
  } else if (bn == 128) {
    switch (epi) {
      case EPI_PLAIN: return launch_one<128, EPI_PLAIN>(c, tmA, tmB, a, st);
      case EPI_GATE_RESID: return launch_one<128, EPI_GATE_RESID>(c, tmA, tmB, a, st);
    }
  }
  return fail(c, XFOLD_ERR_ARG, "gemm: unsupported tile %d / epilogue %d", bn, epi);
}

}  // namespace xf
