// The Pairformer block on a pair representation partitioned by token rows over the GPUs of one node, with every
// exchange between its stages done by this library's own peer-memory kernels (plain stores over NVLink, bounded flag
// barriers) -- one C-ABI call runs a whole stack of blocks; the host does nothing between the stages.
//
// Layout.  Rank p holds rows [start[p], start[p+1]) of z (ShardInfo rule) in one of two peer-mapped buffers per rank;
// a distributed transpose writes the transposed shard into the OTHER buffer of every rank.  Per block:
//
//   z  : TriangleMultiplication outgoing   a, b rows -> channel planes on their owner (every rank takes 128 / P channels of
//   z  : TriangleMultiplication incoming   a and b for ALL rows), product per channel, output rows back to their owners.
//                                          The incoming product 'ckj,cki->cij' contracts over the ROW index of the same
//                                          planes: it runs with MN-major tensor-core operands, so z is not transposed
//                                          for it (the reference feeds it the column shard instead,
//                                          nn/d_triangle_multiplication.py:81).
//   z  : TriangleAttention starting node   the rows' pair bias is broadcast into every rank's [head][query][key] planes
//   zT : TriangleAttention ending node     (rows of zT are KEY rows of the bias: a column block of every plane), then
//   zT : pair Transition                   token-local
//   z  : pair logits of the single path, broadcast like the bias; the single path is replicated (< 1 % of the work)
//
// i.e. two distributed transposes per block in place of the reference's two all-gathers of the whole pair representation
// (nn/d_pairformer.py:134-155), and nine flag barriers.  Why the buffers need no more synchronisation than those barriers
// is argued in the header comment of peer.cu; the same reasoning covers the bias planes (their writers and their next
// readers are always separated by a barrier that every rank signals after its own last read, in stream order).
#include "internal.h"
#include "stages.h"

namespace xf {

constexpr int SH_MAX = 8;

struct ShardCtx {
  int world = 1, rank = 0, n = 0, ld = 0, rmax = 0, cq = 128;
  int start[SH_MAX + 1] = {0};
  void* z[2][SH_MAX] = {{nullptr}};
  void* pa[SH_MAX] = {nullptr};
  void* pb[SH_MAX] = {nullptr};
  void* po[SH_MAX] = {nullptr};
  void* bias[SH_MAX] = {nullptr};
  void* flags[SH_MAX] = {nullptr};
  int epoch = 0;  // flag barriers passed so far; every rank makes the same sequence of calls, so the counts agree
  // Exchange kernels run on a second stream, chunk by chunk, while the producing GEMM works on its next chunk.
  cudaStream_t side = nullptr;
  cudaEvent_t ev[8] = {nullptr};
  int ev_next = 0;
  // Chunks per producing stage.  One: every exchange follows its GEMM.  More were measured as no faster on 2-8 GPUs (a
  // persistent GEMM CTA fills its SM, so exchange kernels and GEMMs take turns) and, at N = 128 on two GPUs, gave
  // results that changed from run to run; with one chunk the sharded path reproduces the one-GPU path bit for bit.
  int parts = 1;
  int reserve = 0;  // SMs the chunked GEMMs leave free for the exchange kernels on the second stream
};

// For the lifetime of the object the context's GEMMs leave `reserve` SMs free and its exchange kernels are sized for them.
struct OverlapScope {
  Ctx* c;
  int sms0, cap0;
  OverlapScope(Ctx* c_, const ShardCtx* sc, bool chunked) : c(c_), sms0(c_->gemm_sms), cap0(c_->peer_cta_cap) {
    if (chunked && sc->reserve > 0 && sc->reserve < c->sm_count) {
      c->gemm_sms = c->sm_count - sc->reserve;
      c->peer_cta_cap = sc->reserve * 8;
    }
  }
  ~OverlapScope() {
    c->gemm_sms = sms0;
    c->peer_cta_cap = cap0;
  }
};

// side stream waits for what `main` has launched so far
static int fork_to_side(Ctx* c, ShardCtx* sc, cudaStream_t main) {
  cudaEvent_t e = sc->ev[sc->ev_next];
  sc->ev_next = (sc->ev_next + 1) & 7;
  if (cudaEventRecord(e, main) != cudaSuccess || cudaStreamWaitEvent(sc->side, e, 0) != cudaSuccess)
    return fail(c, XFOLD_ERR_LAUNCH, "sharded block: stream fork failed");
  return XFOLD_OK;
}
// `main` waits for everything launched on the side stream so far
static int join_side(Ctx* c, ShardCtx* sc, cudaStream_t main) {
  cudaEvent_t e = sc->ev[sc->ev_next];
  sc->ev_next = (sc->ev_next + 1) & 7;
  if (cudaEventRecord(e, sc->side) != cudaSuccess || cudaStreamWaitEvent(main, e, 0) != cudaSuccess)
    return fail(c, XFOLD_ERR_LAUNCH, "sharded block: stream join failed");
  return XFOLD_OK;
}

struct ShardWs {
  bf16 *x, *g, *a, *b, *op, *qkvg, *mext, *bias_loc;
  void *tr, *single;
  size_t tr_bytes, single_bytes, bytes;
};

static ShardWs carve_shard(void* ws, size_t cap, const ShardCtx& sc) {
  ShardWs W;
  const size_t R = sc.rmax, N = sc.n, ld = sc.ld;
  const size_t tok = R * N * 128 * 2;
  Carver cv(ws, cap);
  W.x = (bf16*)cv.take(tok);
  const size_t base = align_up(cv.off, 1024);
  // three users of the same region, never live together: TriangleMultiplication, attention, Transition
  Carver A(ws, cap), B(ws, cap);
  A.off = B.off = base;
  W.g = (bf16*)A.take(tok);
  W.a = (bf16*)A.take(R * 128 * ld * 2);
  W.b = (bf16*)A.take(R * 128 * ld * 2);
  W.op = (bf16*)A.take((size_t)sc.cq * N * ld * 2);
  W.qkvg = (bf16*)B.take(R * N * 512 * 2);
  W.mext = (bf16*)B.take(R * ((N + 127) / 128) * 4096);
  W.tr_bytes = align_up(tok, 1024) + align_up(R * N * 512 * 2, 1024) + 2048;
  size_t end = A.off > B.off ? A.off : B.off;
  if (base + W.tr_bytes > end) end = base + W.tr_bytes;
  W.tr = ws ? static_cast<uint8_t*>(ws) + base : nullptr;
  cv.off = end;
  const size_t rows_q = R * ld, rows_k = N * (size_t)pad8((int)R);
  W.bias_loc = (bf16*)cv.take(16 * (rows_q > rows_k ? rows_q : rows_k) * 2);
  W.single_bytes = single_ws_bytes((int)N);
  W.single = cv.take(W.single_bytes);
  W.bytes = cv.off + 1024;
  return W;
}

static int barrier(Ctx* c, ShardCtx* sc, cudaStream_t st) {
  return launch_peer_barrier(c, sc->flags, sc->rank, sc->world, ++sc->epoch, st);
}

// z[R][N][128] += TriangleMultiplication(z) on this rank's rows, both directions on the same layout
static int trimul_sharded(Ctx* c, ShardCtx* sc, bf16* z, const float* mask_rows, const xfold_trimul_weights* w, int outgoing,
                          const ShardWs& W, cudaStream_t st) {
  const int me = sc->rank, N = sc->n, ld = sc->ld, R = sc->start[me + 1] - sc->start[me], row0 = sc->start[me];
  // a, b for this rank's rows, all channels: [R][128][ld]; the rows of a finished chunk leave for their planes on the
  // second stream while the next chunk is projected
  const int parts = sc->parts > 1 && R >= 2 * sc->parts ? sc->parts : 1;
  const int rper = (R + parts - 1) / parts;
  const int cparts = sc->parts > 1 && sc->cq >= 2 * sc->parts ? sc->parts : 1;
  int rc;
  {
  OverlapScope ov(c, sc, parts > 1);
  for (int r0 = 0; r0 < R; r0 += rper) {
    const int rr = R - r0 < rper ? R - r0 : rper;
    const long long t0 = (long long)r0 * N;
    if ((rc = trimul_project(c, z + t0 * 128, mask_rows ? mask_rows + t0 : nullptr, rr, N, 0, w, W.x + t0 * 128,
                             W.a + (long long)r0 * 128 * ld, W.b + (long long)r0 * 128 * ld, W.g + t0 * 128, ld,
                             (long long)128 * ld, st))) return rc;
    if ((rc = fork_to_side(c, sc, st))) return rc;
    if ((rc = launch_channel_scatter(c, W.a + (long long)r0 * 128 * ld, W.b + (long long)r0 * 128 * ld, rr, N, ld, row0 + r0,
                                     sc->pa, sc->pb, sc->world, sc->side))) return rc;
  }
  }
  if ((rc = join_side(c, sc, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  // this rank's channels, all rows: planes [cq][N][ld]
  const bf16* pa = (const bf16*)sc->pa[me];
  const bf16* pb = (const bf16*)sc->pb[me];
  const long long cs = (long long)N * ld;
  // the product in groups of channels; a finished group's rows go back to their owners while the next group is computed
  const int cper = (sc->cq + cparts - 1) / cparts;
  {
  OverlapScope ov(c, sc, cparts > 1);
  for (int c0 = 0; c0 < sc->cq; c0 += cper) {
    const int cc = sc->cq - c0 < cper ? sc->cq - c0 : cper;
    const long long off = (long long)c0 * cs;
    if (outgoing) rc = trimul_contract(c, pa + off, cs, ld, pb + off, cs, ld, N, N, N, W.op + off, cs, ld, st, cc);   // sum_k a[i][k] b[j][k]
    else rc = trimul_contract_mn(c, pb + off, cs, ld, pa + off, cs, ld, N, N, N, W.op + off, cs, ld, st, cc);       // sum_k b[k][i] a[k][j]
    if (rc) return rc;
    if ((rc = fork_to_side(c, sc, st))) return rc;
    if ((rc = launch_row_scatter(c, W.op + off, cc, me * sc->cq + c0, N, ld, sc->po, sc->start, sc->world, sc->side))) return rc;
  }
  }
  if ((rc = join_side(c, sc, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  return trimul_output(c, (const bf16*)sc->po[me], ld, (long long)128 * ld, W.g, R, N, w, W.x, z, st);
}

static int block_sharded(Ctx* c, ShardCtx* sc, int* slot, bf16* s, const float* pair_mask, const float* seq_mask,
                         const xfold_pairformer_weights* w, const ShardWs& W, cudaStream_t st) {
  const int me = sc->rank, N = sc->n, ld = sc->ld, R = sc->start[me + 1] - sc->start[me], row0 = sc->start[me];
  const float* mask_rows = pair_mask ? pair_mask + (long long)row0 * N : nullptr;
  const bf16* bias = (const bf16*)sc->bias[me];
  bf16* z = (bf16*)sc->z[*slot][me];
  int rc;
  if ((rc = trimul_sharded(c, sc, z, mask_rows, &w->tri_out, 1, W, st))) return rc;
  if ((rc = trimul_sharded(c, sc, z, mask_rows, &w->tri_in, 0, W, st))) return rc;

  // TriangleAttention, starting node: this rank's rows are QUERY rows of the bias [head][query][key]
  if ((rc = triattn_bias(c, z, R, N, &w->att_start, W.x, W.bias_loc, ld, (long long)R * ld, 0, st))) return rc;
  if ((rc = launch_block_broadcast2d(c, W.bias_loc, 4, (long long)R * ld * 2, (long long)R * ld * 2, (long long)row0 * ld * 2,
                                     (long long)N * ld * 2, sc->bias, sc->world, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  // The attention's output projection runs in chunks of rows; the rows of a finished chunk are sent to the transposed
  // shard (zT[j][i] = z[i][j], in the OTHER buffer of the rank that owns column j) on the second stream meanwhile.
  ChunkHook to_t;
  to_t.parts = sc->parts;
  to_t.reserve_sms = sc->reserve;
  to_t.unit = N;
  bf16* src = z;
  int dst_slot = *slot ^ 1;
  to_t.after = [&](long long m0, long long m) -> int {
    int r = fork_to_side(c, sc, st);
    if (r) return r;
    return launch_transpose_scatter(c, src + m0 * 128, (int)(m / N), N, row0 + (int)(m0 / N), sc->z[dst_slot], sc->start,
                                    sc->world, sc->side);
  };
  if ((rc = triattn_core(c, W.x, bias, ld, mask_rows, N, R, N, 0, &w->att_start, W.qkvg, W.mext, z, st, nullptr, &to_t))) return rc;
  if ((rc = join_side(c, sc, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  *slot ^= 1;
  bf16* zt = (bf16*)sc->z[*slot][me];
  // ending node on zT: token zT[j][i] is pair (i, j), so this rank's rows are KEY rows of the bias (a column block of
  // every plane); the mask rows are the ones the reference passes, pair_mask[shard] (nn/d_pairformer.py:144)
  const int pitch_r = pad8(R);
  if ((rc = triattn_bias(c, zt, R, N, &w->att_end, W.x, W.bias_loc, pitch_r, (long long)N * pitch_r, 1, st))) return rc;
  if ((rc = launch_cols_broadcast(c, W.bias_loc, (long long)4 * N, R, pitch_r, row0, ld, sc->bias, sc->world, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  if ((rc = triattn_core(c, W.x, bias, ld, mask_rows, N, R, N, 0, &w->att_end, W.qkvg, W.mext, zt, st))) return rc;
  // and back, overlapped with the Transition's second projection in the same way
  src = zt;
  dst_slot = *slot ^ 1;
  if ((rc = transition_fwd(c, zt, (long long)R * N, 128, 512, &w->pair_transition, W.tr, W.tr_bytes, st, nullptr, &to_t))) return rc;
  if ((rc = join_side(c, sc, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  *slot ^= 1;
  if (!s || !w->spl_w) return XFOLD_OK;
  z = (bf16*)sc->z[*slot][me];
  // pair logits of the single path (nn/d_pairformer.py:158-160): 16 planes, this rank's rows are query rows
  if ((rc = launch_ln_rows(c, z, 128, nullptr, 128, (long long)R * N, 128, w->spl_ln_gamma, w->spl_ln_beta, 1e-5f, 16, w->spl_w,
                           nullptr, (long long)R * ld, nullptr, nullptr, 0, st, W.bias_loc, -N, 0, ld))) return rc;
  if ((rc = launch_block_broadcast2d(c, W.bias_loc, 16, (long long)R * ld * 2, (long long)R * ld * 2, (long long)row0 * ld * 2,
                                     (long long)N * ld * 2, sc->bias, sc->world, st))) return rc;
  if ((rc = barrier(c, sc, st))) return rc;
  return single_update(c, s, bias, ld, seq_mask, N, w, W.single, W.single_bytes, st);
}

}  // namespace xf

using namespace xf;

struct xfold_shard_ctx : public xf::ShardCtx {};

extern "C" {

void xfold_shard_ctx_destroy(xfold_shard_ctx* sc);

int xfold_shard_ctx_create(xfold_ctx* cx, const xfold_shard_desc* d, xfold_shard_ctx** out) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !d || !out) return XFOLD_ERR_ARG;
  *out = nullptr;
  if (d->world < 2 || d->world > SH_MAX || 128 % d->world || d->rank < 0 || d->rank >= d->world)
    return fail(c, XFOLD_ERR_ARG, "shard context: the rank count must be 2, 4 or 8 (it divides the 128 channels), got rank %d of %d",
                d->rank, d->world);
  if (d->n_tokens <= 0 || !d->row_starts || !d->zbuf0 || !d->zbuf1 || !d->plane_a || !d->plane_b || !d->plane_o || !d->bias ||
      !d->flags)
    return fail(c, XFOLD_ERR_ARG, "shard context: null argument");
  xfold_shard_ctx* sc = new xfold_shard_ctx();
  sc->world = d->world;
  sc->rank = d->rank;
  sc->n = d->n_tokens;
  sc->ld = pad8(d->n_tokens);
  sc->cq = 128 / d->world;
  for (int q = 0; q <= d->world; ++q) sc->start[q] = d->row_starts[q];
  bool ok = sc->start[0] == 0 && sc->start[d->world] == d->n_tokens;
  for (int q = 0; q < d->world; ++q) {
    const int r = sc->start[q + 1] - sc->start[q];
    ok = ok && r > 0;
    if (r > sc->rmax) sc->rmax = r;
    sc->z[0][q] = d->zbuf0[q];
    sc->z[1][q] = d->zbuf1[q];
    sc->pa[q] = d->plane_a[q];
    sc->pb[q] = d->plane_b[q];
    sc->po[q] = d->plane_o[q];
    sc->bias[q] = d->bias[q];
    sc->flags[q] = d->flags[q];
    ok = ok && sc->z[0][q] && sc->z[1][q] && sc->pa[q] && sc->pb[q] && sc->po[q] && sc->bias[q] && sc->flags[q];
  }
  if (!ok) {
    delete sc;
    return fail(c, XFOLD_ERR_ARG, "shard context: row offsets must rise from 0 to n_tokens and every peer pointer must be set");
  }
  if (cudaStreamCreateWithFlags(&sc->side, cudaStreamNonBlocking) != cudaSuccess) ok = false;
  for (int i = 0; i < 8 && ok; ++i) ok = cudaEventCreateWithFlags(&sc->ev[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    xfold_shard_ctx_destroy(sc);
    return fail(c, XFOLD_ERR_DEVICE, "shard context: cannot create the exchange stream");
  }
  *out = sc;
  return XFOLD_OK;
}

void xfold_shard_ctx_destroy(xfold_shard_ctx* sc) {
  if (!sc) return;
  for (int i = 0; i < 8; ++i)
    if (sc->ev[i]) cudaEventDestroy(sc->ev[i]);
  if (sc->side) cudaStreamDestroy(sc->side);
  delete sc;
}

size_t xfold_shard_workspace_bytes(const xfold_shard_ctx* sc) { return sc ? carve_shard(nullptr, 0, *sc).bytes : 0; }

int xfold_shard_ctx_set_overlap(xfold_shard_ctx* sc, int chunks, int reserved_sms) {
  if (!sc || chunks < 1 || chunks > 8 || reserved_sms < 0 || reserved_sms > 64) return XFOLD_ERR_ARG;
  sc->parts = chunks;
  sc->reserve = reserved_sms;
  return XFOLD_OK;
}

int xfold_pairformer_stack_sharded_fwd(xfold_ctx* cx, xfold_shard_ctx* sc, int z_slot, void* s, const float* pair_mask,
                                       const float* seq_mask, const xfold_pairformer_weights* blocks, int num_blocks,
                                       void* ws, size_t ws_bytes, void* stream, int* z_slot_out) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !sc || !z_slot_out || (num_blocks > 0 && !blocks)) return XFOLD_ERR_ARG;
  if (z_slot != 0 && z_slot != 1) return fail(c, XFOLD_ERR_ARG, "sharded stack: z_slot must be 0 or 1");
  const ShardWs W = carve_shard(ws, ws_bytes, *sc);
  if (!ws || W.bytes > ws_bytes) return fail(c, XFOLD_ERR_ARG, "sharded stack: workspace too small (%zu < %zu)", ws_bytes, W.bytes);
  int slot = z_slot;
  for (int i = 0; i < num_blocks; ++i) {
    const int rc = block_sharded(c, sc, &slot, (bf16*)s, pair_mask, seq_mask, &blocks[i], W, (cudaStream_t)stream);
    if (rc) return rc;
  }
  *z_slot_out = slot;
  return XFOLD_OK;
}

/* The incoming-edges product on channel planes without a transposed copy (MN-major operands). */
int xfold_trimul_contract_planes_incoming_fwd(xfold_ctx* cx, const void* a, const void* b, int channels, int Nk, int Ni, int Nj,
                                              int ld, void* o, int ldo, void* stream) {
  Ctx* c = reinterpret_cast<Ctx*>(cx);
  if (!c || !a || !b || !o) return XFOLD_ERR_ARG;
  if ((ld & 7) || (ldo & 7) || channels < 1) return fail(c, XFOLD_ERR_ARG, "contract: leading dimensions must be multiples of 8");
  return trimul_contract_mn(c, (const bf16*)b, (long long)Nk * ld, ld, (const bf16*)a, (long long)Nk * ld, ld, Ni, Nj, Nk,
                            (bf16*)o, (long long)Ni * ldo, ldo, (cudaStream_t)stream, channels);
}

}  // extern "C"
