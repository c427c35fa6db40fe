// Persistent, warp-specialised bf16 GEMM  D[m][n] = sum_k A[m][k] * B[n][k]  for sm_100a.
//
//   warp 0      : TMA producer (one elected lane), 128-byte-swizzled K-major tiles, STAGES-deep ring
//   warp 1      : tcgen05.mma issuer (one elected lane); owns the TMEM allocation (2 accumulators)
//   warps 2..9  : epilogue; two warps share each 32-lane quarter of the 128-row accumulator (one per
//                 half of the columns) and drain it with tcgen05.ld while the MMA warp already fills
//                 the other buffer
//
// Every projection of the Pairformer block, the SwiGLU transition and the per-channel N x N x N
// TriangleMultiplication contraction (batched over the 128 channels) run through this kernel; they
// differ only in the tensor maps and in the epilogue that is fused behind the accumulator.
#include "internal.h"
#include "umma.cuh"

namespace xf {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
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
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
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
      uint32_t stage = 0, phase = 0;
      bool okay = true;
      for (long long t = blockIdx.x; t < total && okay; t += gridDim.x) {
        const int tn = int(t % p.tiles_n);
        const int tm = int((t / p.tiles_n) % p.tiles_m);
        const int b = int(t / ((long long)p.tiles_n * p.tiles_m));
        int a1, a2;
        if (p.a_row_mode == 0) { a1 = tm * BM; a2 = b; }
        else { a1 = tm % p.a_dim1; a2 = (tm / p.a_dim1) * BM; }
        const int bb = p.b_batched ? b : 0;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, ab, XF_ERR_WAIT_EMPTY)) { okay = false; break; }
          mbar_arrive_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* sA = smem + stage * Cfg::STAGE_BYTES;
          tma_load_3d(sA, &tmA, &full[stage], kb * BK, a1, a2);
          tma_load_3d(sA + Cfg::A_BYTES, &tmB, &full[stage], kb * BK, tn * BN, bb);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
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
          const uint64_t ad = make_sdesc(sA, 16, 1024);
          const uint64_t bd = make_sdesc(sA + Cfg::A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 B along K inside the swizzled row
            umma_ss(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) ? 1u : 0u);
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
    uint32_t it = 0;
    for (long long t = blockIdx.x; t < total; t += gridDim.x, ++it) {
      const int tn = int(t % p.tiles_n);
      const int tm = int((t / p.tiles_n) % p.tiles_m);
      const int b = int(t / ((long long)p.tiles_n * p.tiles_m));
      const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
      if (!mbar_wait(&tfull[buf], aphase, ab, XF_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(q * 32) << 16);

      if constexpr (EPI == EPI_PLAIN || EPI == EPI_GATE_RESID) {
        const long long m = (long long)tm * BM + row;
        const bool rvalid = m < p.M;
        bf16* orow = p.out + (long long)b * p.out_batch_stride + m * p.ldo;
        const bool vec_ok = ((p.ldo & 7) == 0);
#pragma unroll 1
        for (int cc = ch * (BN / 64); cc < (ch + 1) * (BN / 64); ++cc) {
          uint32_t r[32];
          tmem_ld32(taddr + cc * 32, r);
          tmem_ld_wait();
          const int col0 = tn * BN + cc * 32;
          if (rvalid && col0 < p.N) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              const int col = col0 + g8 * 8;
              const int nvalid = p.N - col;
              if (nvalid <= 0) break;
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g8 * 8 + e]);
              if constexpr (EPI == EPI_PLAIN) {
                if (p.col_bias) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] += (e < nvalid) ? p.col_bias[col + e] : 0.f;
                }
                if (p.col_scale) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] *= (e < nvalid) ? p.col_scale[col + e] : 0.f;
                }
              } else {
                if (p.gate) {
                  float gv[8];
                  load8_bf16(p.gate + m * p.ldg + col, gv, nvalid, (p.ldg & 7) == 0);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] *= sigmoidf_fast(gv[e]);
                } else if (p.row_gate) {
                  float gv[8];
                  load8_bf16(p.row_gate + (m % p.row_gate_mod) * p.ldg + col, gv, nvalid, (p.ldg & 7) == 0);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] *= sigmoidf_fast(gv[e]);
                }
                if (p.resid) {
                  float rv[8];
                  load8_bf16(p.resid + m * p.ldr + col, rv, nvalid, (p.ldr & 7) == 0);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] += rv[e];
                }
              }
              store8_bf16(orow + col, v, nvalid, vec_ok);
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // columns [0,128) of the tile are the SiLU half, [128,256) the linear half of the same outputs
        const long long m = (long long)tm * BM + row;
        const bool rvalid = m < p.M;
        bf16* orow = p.out + m * p.ldo + tn * (BN / 2);
#pragma unroll 1
        for (int cc = ch * (BN / 128); cc < (ch + 1) * (BN / 128); ++cc) {
          uint32_t ra[32], rb[32];
          tmem_ld32(taddr + cc * 32, ra);
          tmem_ld32(taddr + BN / 2 + cc * 32, rb);
          tmem_ld_wait();
          if (rvalid) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float a = __uint_as_float(ra[g8 * 8 + e]);
                v[e] = a * sigmoidf_fast(a) * __uint_as_float(rb[g8 * 8 + e]);
              }
              store8_bf16(orow + cc * 32 + g8 * 8, v, 8, true);
            }
          }
        }
      } else {  // EPI_TRIMUL_AB
        // tile_n 0: [projection | gate] rows of a; 1: the same for b; 2: gating_linear (first 128 columns)
        long long tok, cm_off;
        bool rvalid;
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
        if (tn < 2) {
          const float mk = (rvalid && p.mask) ? p.mask[tok] : 1.f;
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
  const int grid = (int)(total < c->sm_count ? total : c->sm_count);
  const int tag = EPI == EPI_TRIMUL_AB ? XFOLD_K_TRIMUL_PROJ
                  : EPI == EPI_SWIGLU  ? XFOLD_K_LINEAR_SWIGLU
                  : EPI == EPI_GATE_RESID ? XFOLD_K_LINEAR_GATE_RESID
                  : (a.batches > 1 ? XFOLD_K_TRIMUL_CONTRACT : XFOLD_K_LINEAR);
  ProfScope ps(c, tag, st);
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(tmA, tmB, a);
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
