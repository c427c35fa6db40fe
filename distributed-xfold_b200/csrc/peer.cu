// Kernels that move data between GPUs through peer pointers over NVLink / NVSwitch (plain loads and
// stores; no multicast):
//   transpose_scatter : distributed transpose of the row-sharded pair representation.  Every rank writes
//                       each of its tokens z[i][j][:] (256 B) straight into the buffer of the rank that owns
//                       column j, at zT[j_local][i][:], so the whole exchange is one kernel per rank.
//   channel_scatter   : row shard -> channel shard of the TriangleMultiplication operands.  Rank p holds a / b for its
//                       rows and all 128 channels; the contraction is independent per channel, so each rank takes
//                       128 / P channels for ALL rows: row (i, c) of 2 * ld bytes goes to rank c / (128 / P).  For
//                       P >= 4 this moves less than gathering b on every rank ((P-1)/P * 3 N^2 c / P elements per
//                       rank instead of (P-1)/P * N^2 c).
//   row_scatter       : the way back: the contraction output of a rank's channels, row i to the rank that owns i.
//   block_broadcast   : all-gather by peer stores: every rank copies its contiguous block to the same offset of every
//                       rank's destination buffer (the gather of the b rows at 2 ranks: ~2x the rate of the
//                       library all-gather it replaces, which was the largest part of the 2-GPU step's idle time).
//   peer_barrier      : release / acquire flag barrier between the ranks.  The wait is bounded: when it runs
//                       out the kernel records XF_ERR_WAIT_PEER in the status word and returns.
//
// Why two destination buffers are enough for the distributed transpose (the host alternates them, one per call):
// call t stores into buffer k(t) of every rank and ends with flag barrier t.  What it produced is read, on rank p,
// by the kernels between barrier t and p's own scatter kernel of call t + 1 (the pair representation lives in that
// buffer and is updated in place; the scatter of call t + 1 is its last reader, after which the live copy is in the
// other buffer).  Buffer k(t) is stored into again by call t + 2.  A rank q starts those stores only after it has
// passed barrier t + 1, and it passes barrier t + 1 only after every rank p has published epoch t + 1, which p does
// in stream order AFTER its scatter kernel of call t + 1.  Hence every read of buffer k(t) on every rank has
// finished before any store of call t + 2 into it starts.  (Each flag store is a release at system scope after a
// system-wide fence, each flag load an acquire, so the data stores of a call are visible before its flag.)  The same
// argument covers the plane buffers of the channel-sharded contraction, which are written once per
// TriangleMultiplication with a distributed transpose, i.e. a barrier, between two of them.
#include "internal.h"
#include "stages.h"
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

// One warp copies one row of ld elements (16-byte vectors).  src: [R][128][ld] (row i, channel c);
// dst on rank q = c / cq: planes [cq][N][ld], row (c % cq, row0 + i).
__global__ void __launch_bounds__(256)
channel_scatter_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, int R, int N, int ld, int row0, int cq,
                       PeerTable pa, PeerTable pb) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  const long long rows = (long long)R * 128 * 2;
  const int vecs = ld >> 3;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < rows; w += warps) {
    const int which = int(w & 1);
    const long long rc = w >> 1;
    const int c = int(rc & 127), i = int(rc >> 7);
    const int q = c / cq;
    const uint4* src = reinterpret_cast<const uint4*>((which ? b : a) + rc * ld);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(which ? pb.ptr[q] : pa.ptr[q]) +
                                          ((long long)(c - q * cq) * N + row0 + i) * ld);
    for (int v = lane; v < vecs; v += 32) dst[v] = src[v];
  }
}

// src: planes [cq][N][ldo] (local channel c, row i); dst on the rank p that owns row i: [R_p][128][ldo], row
// (i - start[p], chan0 + c).
__global__ void __launch_bounds__(256)
row_scatter_kernel(const bf16* __restrict__ o, int cq, int N, int ldo, int chan0, PeerTable pt) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  const long long rows = (long long)cq * N;
  const int vecs = ldo >> 3;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < rows; w += warps) {
    const int i = int(w % N), c = int(w / N);
    int p = 0;
#pragma unroll
    for (int r = 1; r < MAX_PEERS; ++r)
      if (r < pt.world && i >= pt.start[r]) p = r;
    const uint4* src = reinterpret_cast<const uint4*>(o + w * ldo);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(pt.ptr[p]) +
                                          ((long long)(i - pt.start[p]) * 128 + chan0 + c) * ldo);
    for (int v = lane; v < vecs; v += 32) dst[v] = src[v];
  }
}

__global__ void __launch_bounds__(256)
block_broadcast_kernel(const uint4* __restrict__ src, long long n16, long long off16, PeerTable pt) {
  const long long total = n16 * pt.world;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int q = int(idx / n16);
    const long long v = idx - (long long)q * n16;
    reinterpret_cast<uint4*>(pt.ptr[q])[off16 + v] = src[v];
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

// Strided block broadcast: block k (k < nblk) of `blk16` 16-byte vectors, read at src + k * src_stride16, is stored to
// every rank's buffer at dst_off16 + k * dst_stride16.  The all-gather of per-head bias planes whose local rows are
// QUERY rows: head h's rows [row0, row0 + R) are one contiguous block of the destination plane.
__global__ void __launch_bounds__(256)
block_broadcast2d_kernel(const uint4* __restrict__ src, int nblk, long long blk16, long long src_stride16,
                         long long dst_off16, long long dst_stride16, PeerTable pt) {
  const long long per_rank = (long long)nblk * blk16, total = per_rank * pt.world;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int q = int(idx / per_rank);
    const long long r = idx - (long long)q * per_rank;
    const int k = int(r / blk16);
    const long long v = r - (long long)k * blk16;
    reinterpret_cast<uint4*>(pt.ptr[q])[dst_off16 + k * dst_stride16 + v] = src[k * src_stride16 + v];
  }
}

// Column-block broadcast: `rows` rows of `cols` 16-bit elements (row pitch src_pitch) go to columns [col0, col0 + cols)
// of the same rows of every rank's buffer (row pitch dst_pitch).  The all-gather of bias planes whose local rows are
// KEY rows (they are columns of the [head][query][key] planes).  One warp per (row, rank); 16-byte stores when the
// alignment allows, element stores otherwise.
__global__ void __launch_bounds__(256)
cols_broadcast_kernel(const uint16_t* __restrict__ src, long long rows, int cols, int src_pitch, int col0, int dst_pitch,
                      PeerTable pt) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5), total = rows * pt.world;
  const bool vec = ((cols | src_pitch | col0 | dst_pitch) & 7) == 0;
  for (long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wi < total; wi += warps) {
    const int q = int(wi / rows);
    const long long r = wi - (long long)q * rows;
    const uint16_t* s = src + r * src_pitch;
    uint16_t* d = reinterpret_cast<uint16_t*>(pt.ptr[q]) + r * dst_pitch + col0;
    if (vec) {
      for (int v = lane; v < (cols >> 3); v += 32) reinterpret_cast<uint4*>(d)[v] = reinterpret_cast<const uint4*>(s)[v];
    } else {
      for (int e = lane; e < cols; e += 32) d[e] = s[e];
    }
  }
}

static PeerTable make_table(void* const* ptrs, const int* starts, int world, int fill) {
  PeerTable pt;
  pt.world = world;
  for (int q = 0; q < MAX_PEERS; ++q) pt.ptr[q] = q < world ? ptrs[q] : nullptr;
  for (int q = 0; q <= MAX_PEERS; ++q) pt.start[q] = starts ? (q <= world ? starts[q] : fill) : 0;
  return pt;
}

int launch_transpose_scatter(Ctx* c, const bf16* z, int R, int N, int row0, void* const* dst, const int* col_starts,
                             int world, cudaStream_t st) {
  if (R <= 0 || N <= 0) return XFOLD_OK;
  const PeerTable pt = make_table(dst, col_starts, world, N);
  const long long total = (long long)R * N * 16;
  long long blocks = (total + 255) / 256;
  const long long cap = c->peer_cta_cap > 0 ? c->peer_cta_cap : (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, st);
  transpose_scatter_kernel<<<(int)blocks, 256, 0, st>>>(z, R, N, row0, pt);
  return check_launch(c, "transpose_scatter_kernel");
}

int launch_channel_scatter(Ctx* c, const bf16* a, const bf16* b, int R, int N, int ld, int row0, void* const* peer_a,
                           void* const* peer_b, int world, cudaStream_t st) {
  if (R <= 0 || N <= 0) return XFOLD_OK;
  const PeerTable pa = make_table(peer_a, nullptr, world, 0), pb = make_table(peer_b, nullptr, world, 0);
  const long long rows = (long long)R * 128 * 2;
  long long blocks = (rows + 7) / 8;
  const long long cap = c->peer_cta_cap > 0 ? c->peer_cta_cap : (long long)c->sm_count * 8;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, st);
  channel_scatter_kernel<<<(int)blocks, 256, 0, st>>>(a, b, R, N, ld, row0, 128 / world, pa, pb);
  return check_launch(c, "channel_scatter_kernel");
}

int launch_row_scatter(Ctx* c, const bf16* o, int channels, int chan0, int N, int ldo, void* const* peer_o,
                       const int* row_starts, int world, cudaStream_t st) {
  if (channels <= 0 || N <= 0) return XFOLD_OK;
  const PeerTable pt = make_table(peer_o, row_starts, world, N);
  const long long rows = (long long)channels * N;
  long long blocks = (rows + 7) / 8;
  const long long cap = c->peer_cta_cap > 0 ? c->peer_cta_cap : (long long)c->sm_count * 8;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, st);
  row_scatter_kernel<<<(int)blocks, 256, 0, st>>>(o, channels, N, ldo, chan0, pt);
  return check_launch(c, "row_scatter_kernel");
}

int launch_block_broadcast2d(Ctx* c, const void* src, int nblk, long long blk_bytes, long long src_stride_bytes,
                             long long dst_off_bytes, long long dst_stride_bytes, void* const* dst, int world,
                             cudaStream_t st) {
  if (nblk <= 0 || blk_bytes <= 0) return XFOLD_OK;
  if ((blk_bytes | src_stride_bytes | dst_off_bytes | dst_stride_bytes | (long long)reinterpret_cast<uintptr_t>(src)) & 15)
    return fail(c, XFOLD_ERR_ARG, "peer broadcast: blocks, strides and offsets must be multiples of 16 bytes");
  const PeerTable pt = make_table(dst, nullptr, world, 0);
  const long long total = (long long)nblk * (blk_bytes >> 4) * world;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, st);
  block_broadcast2d_kernel<<<(int)blocks, 256, 0, st>>>((const uint4*)src, nblk, blk_bytes >> 4, src_stride_bytes >> 4,
                                                        dst_off_bytes >> 4, dst_stride_bytes >> 4, pt);
  return check_launch(c, "block_broadcast2d_kernel");
}

int launch_cols_broadcast(Ctx* c, const void* src, long long rows, int cols, int src_pitch, int col0, int dst_pitch,
                          void* const* dst, int world, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return XFOLD_OK;
  const PeerTable pt = make_table(dst, nullptr, world, 0);
  long long blocks = (rows * world + 7) / 8;
  const long long cap = (long long)c->sm_count * 8;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, st);
  cols_broadcast_kernel<<<(int)blocks, 256, 0, st>>>((const uint16_t*)src, rows, cols, src_pitch, col0, dst_pitch, pt);
  return check_launch(c, "cols_broadcast_kernel");
}

int launch_peer_barrier(Ctx* c, void* const* peer_flags, int me, int world, int epoch, cudaStream_t st) {
  FlagTable ft;
  ft.world = world;
  ft.me = me;
  for (int q = 0; q < MAX_PEERS; ++q) ft.flags[q] = q < world ? (int*)peer_flags[q] : nullptr;
  ProfScope ps(c, XFOLD_K_PEER, st);
  peer_barrier_kernel<<<1, 32, 0, st>>>(ft, epoch, c->d_status);
  return check_launch(c, "peer_barrier_kernel");
}

}  // namespace xf

using namespace xf;

extern "C" {

int xfold_transpose_scatter_fwd(xfold_ctx* cx, const void* z, int R, int N, int row0, void* const* peer_bufs,
                                const int* col_starts, int world, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !z || !peer_bufs || !col_starts) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS) return fail(c, XFOLD_ERR_ARG, "transpose: 1 to %d ranks supported, got %d", MAX_PEERS, world);
  return launch_transpose_scatter(c, (const bf16*)z, R, N, row0, peer_bufs, col_starts, world, (cudaStream_t)stream);
}

int xfold_trimul_scatter_channels_fwd(xfold_ctx* cx, const void* a, const void* b, int R, int N, int ld, int row0,
                                      void* const* peer_a, void* const* peer_b, int world, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !a || !b || !peer_a || !peer_b) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS || 128 % world) return fail(c, XFOLD_ERR_ARG, "channel scatter: the rank count must divide 128 (1, 2, 4, 8), got %d", world);
  if (ld & 7) return fail(c, XFOLD_ERR_ARG, "channel scatter: ld must be a multiple of 8");
  return launch_channel_scatter(c, (const bf16*)a, (const bf16*)b, R, N, ld, row0, peer_a, peer_b, world, (cudaStream_t)stream);
}

int xfold_trimul_scatter_rows_fwd(xfold_ctx* cx, const void* o, int channels, int chan0, int N, int ldo,
                                  void* const* peer_o, const int* row_starts, int world, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !o || !peer_o || !row_starts) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS) return fail(c, XFOLD_ERR_ARG, "row scatter: 1 to %d ranks supported, got %d", MAX_PEERS, world);
  if ((ldo & 7) || chan0 < 0 || chan0 + channels > 128) return fail(c, XFOLD_ERR_ARG, "row scatter: bad channel range or ldo");
  return launch_row_scatter(c, (const bf16*)o, channels, chan0, N, ldo, peer_o, row_starts, world, (cudaStream_t)stream);
}

int xfold_peer_allgather_fwd(xfold_ctx* cx, const void* src, long long bytes, long long offset_bytes, void* const* peer_dst,
                             int world, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !src || !peer_dst) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS) return fail(c, XFOLD_ERR_ARG, "peer all-gather: 1 to %d ranks supported, got %d", MAX_PEERS, world);
  if ((bytes & 15) || (offset_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15))
    return fail(c, XFOLD_ERR_ARG, "peer all-gather: block, offset and source must be multiples of 16 bytes");
  if (bytes <= 0) return XFOLD_OK;
  PeerTable pt;
  pt.world = world;
  for (int q = 0; q < MAX_PEERS; ++q) pt.ptr[q] = q < world ? peer_dst[q] : nullptr;
  for (int q = 0; q <= MAX_PEERS; ++q) pt.start[q] = 0;
  const long long n16 = bytes >> 4;
  long long blocks = (n16 * world + 255) / 256;
  const long long cap = (long long)c->sm_count * 16;
  if (blocks > cap) blocks = cap;
  ProfScope ps(c, XFOLD_K_PEER, (cudaStream_t)stream);
  block_broadcast_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, n16, offset_bytes >> 4, pt);
  return check_launch(c, "block_broadcast_kernel");
}

int xfold_peer_barrier(xfold_ctx* cx, void* const* peer_flags, int me, int world, int epoch, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !peer_flags) return XFOLD_ERR_ARG;
  if (world < 1 || world > MAX_PEERS || me < 0 || me >= world) return fail(c, XFOLD_ERR_ARG, "peer barrier: bad rank %d / world %d", me, world);
  return launch_peer_barrier(c, peer_flags, me, world, epoch, (cudaStream_t)stream);
}

}  // extern "C"
