// Declarations shared by the translation units that compose the operators out of kernel launches:
// api.cu (one GPU, and the row-shard stage entry points) and sharded.cu (the block on a row shard with the
// exchanges between its stages).
#pragma once
#include <functional>

#include "internal.h"

namespace xf {

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline int pad8(int n) { return (n + 7) & ~7; }

// Hands out 1 KB-aligned pieces of a caller-provided workspace; with a null base it only adds up sizes.
struct Carver {
  uint8_t* base;
  size_t off = 0, cap;
  Carver(void* p, size_t n) : base(static_cast<uint8_t*>(p)), cap(n) {}
  void* take(size_t bytes) {
    off = align_up(off, 1024);
    void* r = base ? base + off : nullptr;
    off += bytes;
    return r;
  }
  bool ok() const { return off <= cap; }
};

// Lets a caller overlap what follows an operator's LAST GEMM with that GEMM: the GEMM is issued in `parts` chunks of
// rows (chunk boundaries at multiples of `unit` rows) and `after(first_row, rows)` is called once a chunk is launched.
// The multi-GPU block uses it to send finished rows to their next owner on a second stream while the rest computes.
struct ChunkHook {
  int parts = 1;
  int reserve_sms = 0;  // SMs the chunks' GEMMs leave free for what the hook launches on another stream
  long long unit = 1;
  std::function<int(long long, long long)> after;
};

// ---- kernel launchers (simt.cu, attention*.cu) ----------------------------------------------------------
int launch_ln_rows(Ctx* c, const bf16* x, long long ldx, bf16* y, long long ldy, long long rows, int C, const float* g,
                   const float* b, float eps, int H, const float* pw, float* proj, long long plane, const bf16* msc,
                   const bf16* msh, int mod_rows, cudaStream_t st, bf16* proj_bf16 = nullptr, int trav_inner = 0,
                   int trav_outer = 0, int proj_pitch = 0);
int launch_mext(Ctx* c, const float* mask, long long mask_ld, bf16* out, int B, int S, cudaStream_t st);
int launch_bias_transpose(Ctx* c, const float* in, bf16* out, int H, int S, int ldq, cudaStream_t st);
int launch_attention2(Ctx* c, const bf16* qkvg, int width, int S, int B, int transposed, int q_col0, int k_col0,
                      int v_col0, int g_col0, int heads, const bf16* biasT, int ldq, const bf16* mext, int mext_rows,
                      bf16* out, long long out_seq_stride, long long out_batch_stride, cudaStream_t st, int head_dim = 32);
int launch_cm_ln(Ctx* c, const bf16* in, long long chan_stride, long long row_stride, int R, int N, bf16* out,
                 const float* gamma, const float* beta, float eps, cudaStream_t st);
int launch_swiglu(Ctx* c, const bf16* in, bf16* out, long long rows, int F, cudaStream_t st);
// ---- stages of the operators (api.cu); (chan, row) strides are in elements -------------------------------
int trimul_project(Ctx* c, const bf16* z, const float* mask, int R, int N, int transposed_store,
                   const xfold_trimul_weights* w, bf16* x, bf16* a_out, bf16* b_out, bf16* g, long long chan_stride,
                   long long row_stride, cudaStream_t st);
int trimul_contract(Ctx* c, const bf16* a_, long long a_cs, long long a_rs, const bf16* b_, long long b_cs,
                    long long b_rs, int Ri, int Nj, int K, bf16* o, long long o_cs, long long o_rs, cudaStream_t st,
                    int channels = 128);
int trimul_contract_mn(Ctx* c, const bf16* at, long long at_cs, long long at_rs, const bf16* bt, long long bt_cs,
                       long long bt_rs, int Mi, int Nj, int K, bf16* o, long long o_cs, long long o_rs, cudaStream_t st,
                       int channels = 128);
int trimul_output(Ctx* c, const bf16* o, long long o_cs, long long o_rs, const bf16* g, int R, int N,
                  const xfold_trimul_weights* w, bf16* x, bf16* z, cudaStream_t st, bf16* upd = nullptr);
int triattn_bias(Ctx* c, const bf16* z, int R, int N, const xfold_triattn_weights* w, bf16* x, bf16* bias, int pitch,
                 long long plane, int rows_are_keys, cudaStream_t st);
int triattn_core(Ctx* c, bf16* x, const bf16* biasT, int ldq, const float* mask, long long mask_ld, int R, int N,
                 int transposed, const xfold_triattn_weights* w, bf16* qkvg, bf16* mext, bf16* z, cudaStream_t st,
                 bf16* upd = nullptr, const ChunkHook* hook = nullptr);
int transition_fwd(Ctx* c, bf16* x, long long rows, int C, int F, const xfold_transition_weights* w, void* ws,
                   size_t ws_bytes, cudaStream_t st, bf16* upd = nullptr, const ChunkHook* hook = nullptr);
size_t single_ws_bytes(int N);
int single_update(Ctx* c, bf16* s, const bf16* plT, int ldq, const float* seq_mask, int N,
                  const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, cudaStream_t st);

// ---- peer-memory exchange launchers (peer.cu); pointer arrays are host arrays of `world` peer-mapped addresses ----
int launch_transpose_scatter(Ctx* c, const bf16* z, int R, int N, int row0, void* const* dst, const int* col_starts,
                             int world, cudaStream_t st);
int launch_channel_scatter(Ctx* c, const bf16* a, const bf16* b, int R, int N, int ld, int row0, void* const* peer_a,
                           void* const* peer_b, int world, cudaStream_t st);
int launch_row_scatter(Ctx* c, const bf16* o, int channels, int chan0, int N, int ldo, void* const* peer_o,
                       const int* row_starts, int world, cudaStream_t st);
int launch_block_broadcast2d(Ctx* c, const void* src, int nblk, long long blk_bytes, long long src_stride_bytes,
                             long long dst_off_bytes, long long dst_stride_bytes, void* const* dst, int world,
                             cudaStream_t st);
int launch_cols_broadcast(Ctx* c, const void* src, long long rows, int cols, int src_pitch, int col0, int dst_pitch,
                          void* const* dst, int world, cudaStream_t st);
int launch_peer_barrier(Ctx* c, void* const* peer_flags, int me, int world, int epoch, cudaStream_t st);

}  // namespace xf
