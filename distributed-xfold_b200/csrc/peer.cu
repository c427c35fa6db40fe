// Kernels that move data between GPUs through peer pointers over NVLink / NVSwitch (plain loads and
// stores; no multicast):
//   transpose_scatter : distributed transpose of the row-sharded pair representation.  Every rank writes
//                       each of its tokens z[i][j][:] (256 B) straight into the buffer of the rank that owns
//                       column j, at zT[j_local][i][:], so the whole exchange is one kernel per rank.
//   peer_barrier      : release / acquire flag barrier between the ranks.  The wait is bounded: when it runs
//                       out the kernel records XF_ERR_WAIT_PEER in the status word and returns.
#include "internal.h"
#include "umma.cuh"

namespace xf {

constexpr int MAX_PEERS = 8;

struct PeerTable {
  void* ptr[MAX_PEERS];      // base of every rank's destination buffer (peer-mapped addresses)
  int start[MAX_PEERS + 1];  // rank q owns columns [start[q], start[q+1])
  int world;
};

__global__ void __launch_bounds__(256)
transpose_scatter_kernel(const bf16* __restrict__ z, int R, int N, int row0, PeerTable pt) {
  // 16 threads move one token (128 bf16 = 16 x 16 B)
  const long long total = (long long)R * N * 16;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int part = int(idx & 15);
    const long long tok = idx >> 4;
    const int i = int(tok / N), j = int(tok % N);
    int q = 0;
#pragma unroll
    for (int r = 1; r < MAX_PEERS; ++r)
      if (r < pt.world && j >= pt.start[r]) q = r;
    const uint4 v = *reinterpret_cast<const uint4*>(z + tok * 128 + part * 8);
    bf16* dst = reinterpret_cast<bf16*>(pt.ptr[q]) + ((long long)(j - pt.start[q]) * N + (row0 + i)) * 128 + part * 8;
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

struct FlagTable {
  int* flags[MAX_PEERS];  // every rank's flag array (MAX_PEERS ints), peer-mapped
  int world, me;
};

__global__ void peer_barrier_kernel(FlagTable ft, int epoch, int* status) {
  const int q = threadIdx.x;
  if (q >= ft.world) return;
  __threadfence_system();  // everything this GPU wrote before the barrier is visible before the flag is
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ft.flags[q] + ft.me), "r"(epoch) : "memory");
  const int* mine = ft.flags[ft.me] + q;
  const long long t0 = clock64();
  int v;
  do {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if (clock64() - t0 > XF_WAIT_CYCLES) {
      atomicCAS(status, 0, XF_ERR_WAIT_PEER);
      break;
    }
  } while (true);
}

}  // namespace xf

using namespace xf;

extern "C" {

int xfold_transpose_scatter_fwd(xfold_ctx* cx, const void* z, int R, int N, int row0, void* const* peer_bufs,
                                const int* col_starts, int world, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !z || !peer_bufs || !col_starts) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS) return fail(c, XFOLD_ERR_ARG, "transpose: 1 to %d ranks supported, got %d", MAX_PEERS, world);
  if (R <= 0 || N <= 0) return XFOLD_OK;
  PeerTable pt;
  pt.world = world;
  for (int q = 0; q < MAX_PEERS; ++q) pt.ptr[q] = q < world ? peer_bufs[q] : nullptr;
  for (int q = 0; q <= MAX_PEERS; ++q) pt.start[q] = q <= world ? col_starts[q] : N;
  const long long total = (long long)R * N * 16;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, (cudaStream_t)stream);
  transpose_scatter_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)z, R, N, row0, pt);
  return check_launch(c, "transpose_scatter_kernel");
}

int xfold_peer_barrier(xfold_ctx* cx, void* const* peer_flags, int me, int world, int epoch, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !peer_flags) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS || me < 0 || me >= world) return fail(c, XFOLD_ERR_ARG, "peer barrier: bad rank %d / world %d", me, world);
  FlagTable ft;
  ft.world = world;
  ft.me = me;
  for (int q = 0; q < MAX_PEERS; ++q) ft.flags[q] = q < world ? (int*)peer_flags[q] : nullptr;
  ProfScope ps(c, XFOLD_K_PEER, (cudaStream_t)stream);
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ft, epoch, c->d_status);
  return check_launch(c, "peer_barrier_kernel");
}

}  // extern "C"
