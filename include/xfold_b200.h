/* C ABI of libxfold_b200.so: the sm_100a replacement for the reference's fused CPU operator
 * library (the `_alpha_attention` ops of src/distributed_xfold/xsmm_kernels/csrc/Alpha_Attention.cpp)
 * and for the module forwards that sit directly on top of it.
 *
 * Conventions
 *  - every function returns XFOLD_OK (0) or a non-zero status; xfold_last_error() gives the text;
 *  - all tensor arguments are DEVICE pointers owned by the caller; activations and weights are
 *    bf16 (passed as void*), masks / LayerNorm parameters / biases are float32;
 *  - `stream` is a cudaStream_t passed as void*; calls are asynchronous on that stream;
 *  - the library allocates nothing except the context (one status word on the device); scratch
 *    memory is passed in by the caller (`ws`, size from the matching *_workspace_bytes function);
 *  - kernels never wait unboundedly: a wait that runs out records a code in the context's status
 *    word, the kernel drains and returns, and xfold_check_status() reports XFOLD_ERR_TIMEOUT.
 */
#ifndef XFOLD_B200_H_
#define XFOLD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  XFOLD_OK = 0,
  XFOLD_ERR_ARG = 1,     /* bad argument (shape, alignment, null pointer, workspace too small) */
  XFOLD_ERR_LAUNCH = 2,  /* CUDA reported an error at launch */
  XFOLD_ERR_DEVICE = 3,  /* no usable device / driver entry point missing */
  XFOLD_ERR_TIMEOUT = 4  /* an in-kernel bounded wait ran out (see xfold_check_status) */
};

typedef struct xfold_ctx xfold_ctx;

/* Context: replaces the implicit process-wide state of the reference extension module
 * (`tpp_pytorch_extension._C`, imported at prototypes/__init__.py:1). One per device. */
int xfold_ctx_create(int device, xfold_ctx** out);
void xfold_ctx_destroy(xfold_ctx* ctx);
const char* xfold_last_error(xfold_ctx* ctx);
/* Synchronises `stream`, reads and clears the device status word. */
int xfold_check_status(xfold_ctx* ctx, void* stream);
/* Version string with the build's gencode. */
const char* xfold_version(void);

/* Kernel accounting (the counterpart of the reference's RECORD_SCOPE / SCOPEIT timers,
 * csrc/Alpha_Attention.cpp:35-48).  xfold_launch_count: kernels launched through this context so
 * far.  With profiling enabled every launch is bracketed by CUDA events on its stream;
 * xfold_profile_read synchronises the device, returns the summed duration (ms) and the number of
 * launches recorded for one kernel class since the last read of that class, and clears them. */
enum {
  XFOLD_K_LAYERNORM = 0,
  XFOLD_K_TRIMUL_PROJ = 1,
  XFOLD_K_TRIMUL_CONTRACT = 2,
  XFOLD_K_CHANNEL_LN = 3,
  XFOLD_K_LINEAR_GATE_RESID = 4,
  XFOLD_K_LINEAR = 5,
  XFOLD_K_ATTENTION = 6,
  XFOLD_K_LINEAR_SWIGLU = 7,
  XFOLD_K_MASK_BIAS = 8,
  XFOLD_K_SWIGLU = 9,
  XFOLD_K_PEER = 10,
  XFOLD_K_APB_ATTENTION = 11, /* the attention kernel when launched for AttentionPairBias (XFOLD_K_ATTENTION: TriangleAttention) */
  XFOLD_K_COUNT = 12
};
long long xfold_launch_count(xfold_ctx* ctx);
int xfold_profile_enable(xfold_ctx* ctx, int on);
int xfold_profile_read(xfold_ctx* ctx, int kernel_class, float* ms_total, int* launches);

/* ---- primitives -------------------------------------------------------------------------- */

/* LayerNorm over rows of width C in {128, 384, 768}, eps as given (the reference uses 1e-5:
 * LayerNormFwdTPP at csrc/triangle_multiplication.h:51-52, csrc/transition.h:26).
 * gamma/beta may be NULL.  Optional fused projection: proj[h * proj_plane + row] =
 * sum_c y[row][c] * proj_w[h][c] for num_proj in {0, 4, 16, 64} (the pair-bias projections of
 * nn/d_attention.py:62 and nn/d_pairformer.py:158); y may then be NULL.  Optional AdaLN
 * modulation (nn/d_diffusion_transformer.py:67-72): y = sigmoid(mod_scale[row % mod_rows]) * y
 * + mod_shift[row % mod_rows], both bf16 [mod_rows][C], or NULL. */
int xfold_layernorm_fwd(xfold_ctx* ctx, const void* x, long long ldx, void* y, long long ldy, long long rows, int C,
                        const float* gamma, const float* beta, float eps, int num_proj, const float* proj_w,
                        float* proj, long long proj_plane, const void* mod_scale, const void* mod_shift,
                        int mod_rows, void* stream);

/* SwiGLU: out[r][f] = silu(in[r][f]) * in[r][F + f]   (xfold.fastnn.gated_linear_unit as pinned by
 * kernel_test/transition.py:37-43 and csrc/transition.h:65-88). */
int xfold_swiglu_fwd(xfold_ctx* ctx, const void* in, void* out, long long rows, int F, void* stream);

/* out[m][n] = (sum_k x[m][k] * w[n][k] + bias[n]) * scale[n]   (torch.nn.Linear; tcgen05 GEMM).
 * K multiple of 8, ldx/ldo multiples of 8; bias / scale may be NULL. */
int xfold_linear_fwd(xfold_ctx* ctx, const void* x, long long ldx, long long M, int K, const void* w, int N,
                     const float* bias, const float* scale, void* out, long long ldo, void* stream);

/* out[m][n] = resid[m][n] + (sum_k x[m][k] w[n][k]) * sigmoid(gate[m][n])   (gate and/or resid may be NULL;
 * out may alias resid).  row_gate: gate shared by rows with the same (m % row_gate_mod). */
int xfold_linear_gate_residual_fwd(xfold_ctx* ctx, const void* x, long long ldx, long long M, int K, const void* w,
                                   int N, const void* gate, long long ldg, int row_gate_mod, const void* resid,
                                   long long ldr, void* out, long long ldo, void* stream);

/* h[m][f] = silu(x w_a[f]) * (x w_b[f]) with w packed in 256-row tiles [128 rows of w_a | 128 rows of w_b]. */
int xfold_linear_swiglu_fwd(xfold_ctx* ctx, const void* x, long long ldx, long long M, int K, const void* w_packed,
                            int F, void* out, long long ldo, void* stream);

/* Batched contraction out[c][i][j] = sum_k a[c][i][k] * b[c][j][k] (the per-channel N x N x N product of
 * TriangleMultiplication: 'cik,cjk->cij' at nn/d_triangle_multiplication.py:122-124). */
int xfold_batched_contract_fwd(xfold_ctx* ctx, const void* a, const void* b, void* out, int channels, int Mi, int Nj,
                               int Kk, long long ld, long long chan_stride_a, long long chan_stride_b,
                               long long ldo, long long chan_stride_o, void* stream);

/* ---- TriangleMultiplication ------------------------------------------------------------------
 * Replaces `_alpha_attention::traingle_multiplication_forward` (csrc/Alpha_Attention.cpp:148-169,
 * 206-210) together with the residual add of nn/d_pairformer.py:122-123: z += TriMul(z, mask).
 * z: bf16 [N][N][128] updated in place; mask: float32 [N][N] or NULL. */
typedef struct {
  const float* ln_in_gamma;  /* left_norm_input  [128] */
  const float* ln_in_beta;
  const void* w_in;          /* bf16 [640][128]: rows 0..127 projection(a), 128..255 gate(a), 256..383 projection(b),
                                384..511 gate(b), 512..639 gating_linear  (a = even rows, b = odd rows of the
                                reference's interleaved weights, nn/d_triangle_multiplication.py:128-129) */
  const float* ln_c_gamma;   /* center_norm [128] */
  const float* ln_c_beta;
  const void* w_out;         /* bf16 [128][128] output_projection */
} xfold_trimul_weights;

size_t xfold_trimul_workspace_bytes(int N);
int xfold_triangle_multiplication_fwd(xfold_ctx* ctx, void* z, const float* mask, int N, int outgoing,
                                      const xfold_trimul_weights* w, void* ws, size_t ws_bytes, void* stream);

/* ---- TriangleAttention (GridSelfAttention) ---------------------------------------------------
 * Replaces `_alpha_attention::grid_self_attn_forward` (csrc/Alpha_Attention.cpp:50-70, 182-185) plus the
 * LayerNorm, pair-bias projection, optional transpose and residual add that the reference does in
 * Python (nn/d_attention.py:58-88, nn/d_pairformer.py:132, 144): z += Attn(LN(z)).
 * transpose = 0: starting node (attend along the second token axis); 1: ending node. */
typedef struct {
  const float* ln_gamma;   /* act_norm [128] */
  const float* ln_beta;
  const float* w_bias;     /* float32 [4][128] pair_bias_projection */
  const void* w_qkvg;      /* bf16 [512][128]: q, k, v, gating_query rows (head-major inside each) */
  const float* qkvg_scale; /* float32 [512]: D^-0.5 on the q columns, 1 elsewhere */
  const void* w_out;       /* bf16 [128][128] output_projection */
} xfold_triattn_weights;

size_t xfold_triattn_workspace_bytes(int N);
int xfold_triangle_attention_fwd(xfold_ctx* ctx, void* z, const float* mask, int N, int transpose,
                                 const xfold_triattn_weights* w, void* ws, size_t ws_bytes, void* stream);

/* ---- Transition ----------------------------------------------------------------------------------
 * Replaces `_alpha_attention::transition_forward` (csrc/Alpha_Attention.cpp:116-125, 187-189) and
 * DistributeTransition.forward (nn/d_primitives.py:31-38) plus the residual add: x += W2 swiglu(W1 LN(x)).
 * C in {128, 384}; F = factor * C. */
typedef struct {
  const float* ln_gamma;
  const float* ln_beta;
  const void* w1_packed; /* bf16 [2F][C] in 256-row tiles [128 SiLU rows | 128 linear rows] */
  const void* w2;        /* bf16 [C][F] */
} xfold_transition_weights;

size_t xfold_transition_workspace_bytes(long long rows, int C, int F);
int xfold_transition_fwd(xfold_ctx* ctx, void* x, long long rows, int C, int F, const xfold_transition_weights* w,
                         void* ws, size_t ws_bytes, void* stream);

/* ---- AttentionPairBias core ------------------------------------------------------------------
 * Replaces `_alpha_attention::batch_diffusion_self_attention_forward` (csrc/Alpha_Attention.cpp:72-92,
 * 191-194): gated multi-head attention with query bias and an additive [H][S][S] pair bias, no
 * output projection.  xn: bf16 [B][S][C] (already normalised); heads x head_dim = C; the head
 * dimension is padded to Dp in {32, 64} inside the packed weights:
 *   w_qkvg bf16 [4 * H * Dp][C], qkvg_bias / qkvg_scale float32 [4 * H * Dp];
 * out: bf16 [B][S][H * Dp] (pad columns are zero).  mask: float32 [S] or NULL. */
size_t xfold_apb_workspace_bytes(int B, int S, int H, int Dp);
int xfold_attention_pair_bias_core_fwd(xfold_ctx* ctx, const void* xn, int B, int S, int C, int H, int Dp,
                                       const void* w_qkvg, const float* qkvg_bias, const float* qkvg_scale,
                                       const float* pair_bias, const float* mask, void* out, void* ws,
                                       size_t ws_bytes, void* stream);

/* The pair bias as the attention kernel reads it: 16-bit [H][S][pad8(S)], FP16 values times log2(e) (the kernel works in
 * base 2).  A caller whose bias does not change between calls -- the diffusion transformer's pair logits are the same for
 * all 200 denoising steps (nn/d_diffusion_transformer.py:296-305 recomputes them per call) -- converts it once with
 * xfold_pair_bias_prepare_fwd (prepared: H * S * pad8(S) * 2 bytes) and passes it to the _prepared_ form of the core. */
int xfold_pair_bias_prepare_fwd(xfold_ctx* ctx, const float* pair_bias, int H, int S, void* prepared, void* stream);
int xfold_attention_pair_bias_core_prepared_fwd(xfold_ctx* ctx, const void* xn, int B, int S, int C, int H, int Dp,
                                                const void* w_qkvg, const float* qkvg_bias, const float* qkvg_scale,
                                                const void* prepared_bias, const float* mask, void* out, void* ws,
                                                size_t ws_bytes, void* stream);

/* The same core with one mask row per batch entry (mask float32, row b at mask + b * mask_ld; mask_ld = 0: one row for
 * all), which is what `_alpha_attention::grid_self_attn_forward` takes as its `bias` [B, 1, 1, S]
 * (csrc/Alpha_Attention.cpp:50-70). */
int xfold_gated_attention_core_fwd(xfold_ctx* ctx, const void* xn, int B, int S, int C, int H, int Dp, const void* w_qkvg,
                                   const float* qkvg_bias, const float* qkvg_scale, const float* pair_bias,
                                   const float* mask, long long mask_ld, void* out, void* ws, size_t ws_bytes,
                                   void* stream);

/* ---- gated cross attention (atom cross-attention core) ---------------------------------------------
 * Replaces `_alpha_attention::batch_diffusion_cross_attention_forward` (csrc/Alpha_Attention.cpp:127-146, 201-204; spec
 * class kernel_test/batch_diffusion_cross_attention.py:23-87): queries from q_data bf16 [B][S][Ca], keys and values from
 * m_data bf16 [B][K][Cm], a float32 bias per batch entry [B][H][S][K], gate sigmoid(q_data gating_w), no output projection.
 *   w_qg bf16 [2*H*D][Ca]: the query rows (head-major) then the gating rows; qg_bias / qg_scale float32 [2*H*D]
 *   (query bias and D^-0.5 on the query rows, 0 / 1 on the gating rows); w_kv bf16 [2*H*D][Cm]: key rows then value rows.
 * out: bf16 [B][S][H*D].  D in {16, 32, 64}. */
size_t xfold_cross_attention_workspace_bytes(int B, int S, int K, int H, int D);
int xfold_cross_attention_fwd(xfold_ctx* ctx, const void* q_data, const void* m_data, int B, int S, int K, int Ca, int Cm,
                              int H, int D, const void* w_qg, const float* qg_bias, const float* qg_scale,
                              const void* w_kv, const float* bias, void* out, void* ws, size_t ws_bytes, void* stream);

/* ---- PairformerBlock --------------------------------------------------------------------------
 * DistributePairformerBlock.forward (nn/d_pairformer.py:99-171) for world size 1: both TriMuls,
 * both TriAttns, pair Transition, then pair-logit projection, single AttentionPairBias (16 heads x 24,
 * padded to 32) and single Transition.  z [N][N][128] and s [N][384] are bf16, updated in place. */
typedef struct {
  xfold_trimul_weights tri_out, tri_in;
  xfold_triattn_weights att_start, att_end;
  xfold_transition_weights pair_transition;
  /* single path (all NULL when the block has no single representation) */
  const float* spl_ln_gamma;  /* single_pair_logits_norm [128] */
  const float* spl_ln_beta;
  const float* spl_w;         /* float32 [16][128] single_pair_logits_projection */
  const float* sa_ln_gamma;   /* single_attention_.adaptive_layernorm.layer_norm [384] */
  const float* sa_ln_beta;
  const void* sa_w_qkvg;      /* bf16 [2048][384] */
  const float* sa_qkvg_bias;  /* float32 [2048] */
  const float* sa_qkvg_scale; /* float32 [2048] */
  const void* sa_w_out;       /* bf16 [384][512] adaptive_zero_init.transition2 with padded head columns */
  xfold_transition_weights single_transition;
} xfold_pairformer_weights;

size_t xfold_pairformer_workspace_bytes(int N);
int xfold_pairformer_block_fwd(xfold_ctx* ctx, void* z, void* s, const float* pair_mask, const float* seq_mask,
                               int N, const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, void* stream);

/* The trunk loop `for pairformer_b in self.trunk_pairformer: pair, single = pairformer_b(...)`
 * (d_alphafold3.py:242-244; the confidence head runs the same loop over its 4 blocks, :450-458): `num_blocks`
 * blocks applied in order to the same z and s, `blocks` being an array of their weights. */
int xfold_pairformer_stack_fwd(xfold_ctx* ctx, void* z, void* s, const float* pair_mask, const float* seq_mask, int N,
                               const xfold_pairformer_weights* blocks, int num_blocks, void* ws, size_t ws_bytes,
                               void* stream);

/* ---- row-shard stages -------------------------------------------------------------------------
 * The pieces of TriangleMultiplication / TriangleAttention on a block of R pair rows, for the
 * multi-GPU block where the pair representation is partitioned by token rows
 * (nn/d_pairformer.py:119-156, distribute_utils.py:101-128) and a collective sits between stages.
 *
 * a, b: bf16 [rows][128][ld], element (row i, channel c, k) at (i * 128 + c) * ld + k, so a rank's rows
 * are one contiguous block and the all-gather of b (nn/d_triangle_multiplication.py:74-79) is a
 * concatenation.  g: bf16 [R * N][128].  o: bf16 [R][128][ldo]. */
int xfold_trimul_project_fwd(xfold_ctx* ctx, const void* z, const float* mask, int R, int N,
                             const xfold_trimul_weights* w, void* x_scratch, void* a, void* b, void* g, int ld,
                             void* stream);
/* o[i][c][j] = sum_k a[i][c][k] * b_full[j][c][k]  ('cik,cjk->cij' on the row shard of a against all rows of b) */
int xfold_trimul_contract_fwd(xfold_ctx* ctx, const void* a, const void* b_full, int R, int Nj, int K, int ld, void* o,
                              int ldo, void* stream);
/* The same product on channel-major planes: a [channels][Ni][ld], b [channels][Nj][ld] -> o [channels][Ni][ldo].
 * Used by the channel-sharded form of the multi-GPU contraction: the product is independent per channel
 * (the 'c' of 'cik,cjk->cij', nn/d_triangle_multiplication.py:122-124), so a rank may take a slice of the
 * channels for all rows instead of gathering b for its rows (nn/d_triangle_multiplication.py:74-79). */
int xfold_trimul_contract_planes_fwd(xfold_ctx* ctx, const void* a, const void* b, int channels, int Ni, int Nj, int K,
                                     int ld, void* o, int ldo, void* stream);
/* z[R][N][128] += output_projection(center_norm(o)) * sigmoid(g)   (nn/d_triangle_multiplication.py:92-99) */
int xfold_trimul_output_fwd(xfold_ctx* ctx, const void* o, int ldo, const void* g, int R, int N,
                            const xfold_trimul_weights* w, void* x_scratch, void* z, void* stream);
/* x = act_norm(z) for R rows and the pair bias these rows contribute (nn/d_attention.py:61-62), bf16, laid out
 * [head][query][key]:
 * rows_are_keys = 0: the rows are query rows,  bias[h * plane + row_local * pitch + y];
 * rows_are_keys = 1: the rows are key rows x,  bias[h * plane + y * pitch + x_local].
 * The bias buffer is an operand of the attention kernel, not a result to read: its entries are the projected
 * values times log2(e), because that kernel exponentiates in base 2 and adds the tile unchanged.  The same
 * holds for plT below. */
int xfold_triattn_bias_fwd(xfold_ctx* ctx, const void* z, int R, int N, const xfold_triattn_weights* w, void* x,
                           void* bias, int pitch, long long plane, int rows_are_keys, void* stream);
/* z[R][N][128] += output_projection(gated attention(x)) along the second axis; bias: bf16 [4][N][ldq],
 * [head][query][key], gathered from all ranks; mask: float32, row b at mask + b * mask_ld. */
size_t xfold_triattn_core_scratch_bytes(int R, int N, size_t* mext_bytes);
int xfold_triattn_core_fwd(xfold_ctx* ctx, void* x, const void* biasT, int ldq, const float* mask, long long mask_ld,
                           int R, int N, const xfold_triattn_weights* w, void* qkvg_scratch, void* mext_scratch, void* z,
                           void* stream);
/* Pair logits of the single path (nn/d_pairformer.py:158-160) for R rows, same layouts as the bias above (16 heads). */
int xfold_pair_logits_fwd(xfold_ctx* ctx, const void* z, int R, int N, const float* ln_gamma, const float* ln_beta,
                          const float* w16, void* plT, int pitch, long long plane, int rows_are_keys, void* stream);
/* single += AttentionPairBias(single, plT) ; single += Transition(single)   (nn/d_pairformer.py:162-169);
 * plT: bf16 [16][N][ldq] pair logits of the whole pair representation, [head][query][key]. */
size_t xfold_single_update_workspace_bytes(int N);
int xfold_single_update_fwd(xfold_ctx* ctx, void* s, const void* plT, int ldq, const float* seq_mask, int N,
                            const xfold_pairformer_weights* w, void* ws, size_t ws_bytes, void* stream);

/* ---- peer-memory exchange (multi-GPU) ------------------------------------------------------------
 * Replaces the reference's all-gather + re-slice of the whole pair representation between the
 * row-sharded and column-sharded halves of a block (nn/d_pairformer.py:134-156) by a distributed
 * transpose done in ONE kernel per rank: every token z[i][j][0..127] of this rank's R rows (global row
 * row0 + i) is stored into the buffer of the rank that owns column j, at zT[j - col_starts[q]][row0 + i][:].
 * peer_bufs: host array of `world` device pointers (each rank's destination buffer, mapped into this
 * process, e.g. CUDA IPC / symmetric memory); col_starts: host array of world + 1 column offsets
 * (ShardInfo rule, distribute_utils.py:101-128).  Plain stores over NVLink, no multicast. */
int xfold_transpose_scatter_fwd(xfold_ctx* ctx, const void* z, int R, int N, int row0, void* const* peer_bufs,
                                const int* col_starts, int world, void* stream);
/* Row shard -> channel shard of the TriangleMultiplication operands, in place of the all-gather of b
 * (nn/d_triangle_multiplication.py:74-79): a, b are this rank's [R][128][ld] operands (rows row0 ..); row (i, c)
 * goes to rank q = c / (128 / world), into its planes peer_a[q] / peer_b[q] = [128 / world][N][ld] at
 * (c % (128 / world), row0 + i).  world must divide 128.  Plain 16-byte stores over NVLink. */
int xfold_trimul_scatter_channels_fwd(xfold_ctx* ctx, const void* a, const void* b, int R, int N, int ld, int row0,
                                      void* const* peer_a, void* const* peer_b, int world, void* stream);
/* The way back: o = [channels][N][ldo] planes of this rank's channels chan0 .. chan0 + channels - 1; row (c, i) goes
 * to the rank p that owns pair row i (row_starts: world + 1 offsets), into peer_o[p] = [R_p][128][ldo] at
 * (i - row_starts[p], chan0 + c): the layout xfold_trimul_output_fwd reads. */
int xfold_trimul_scatter_rows_fwd(xfold_ctx* ctx, const void* o, int channels, int chan0, int N, int ldo,
                                  void* const* peer_o, const int* row_starts, int world, void* stream);
/* All-gather by peer stores (in place of distribute_utils.py:219-262 for a contiguous block per rank): this rank's
 * block of `bytes` bytes is copied to byte offset `offset_bytes` of every rank's destination buffer (peer_dst[q],
 * mapped into this process).  Sizes, offsets and the source are multiples of 16 bytes.  Follow with xfold_peer_barrier. */
int xfold_peer_allgather_fwd(xfold_ctx* ctx, const void* src, long long bytes, long long offset_bytes,
                             void* const* peer_dst, int world, void* stream);
/* Flag barrier between the ranks (the reference uses dist.barrier, run_inference.py:154-245): rank `me`
 * stores `epoch` into slot `me` of every rank's flag array (peer_flags[q], 8 ints, zero-initialised) and
 * waits until all slots of its own array reached `epoch`.  The wait is bounded; a time-out is reported by
 * xfold_check_status as XFOLD_ERR_TIMEOUT.  Epochs must increase by one per call. */
int xfold_peer_barrier(xfold_ctx* ctx, void* const* peer_flags, int me, int world, int epoch, void* stream);

/* ---- the block on a row shard, exchanges included ---------------------------------------------------
 * DistributePairformerBlock.forward for dp_size > 1 (nn/d_pairformer.py:119-156) and the trunk loop around it
 * (d_alphafold3.py:242-244) as ONE call per stack of blocks: the stages above plus every exchange between them
 * (operand planes and output rows of the TriangleMultiplication, the two distributed transposes, the broadcasts of
 * the pair bias and the pair logits), all as this library's peer-memory kernels and bounded flag barriers on the
 * caller's stream.  The pair representation stays sharded from the first block to the last; the incoming
 * TriangleMultiplication runs on the same channel planes as the outgoing one with MN-major tensor-core operands, so
 * a block needs two distributed transposes where the reference does two all-gathers of the whole pair representation.
 *
 * The context replaces the reference's process-group bookkeeping (init_dist_info, distribute_utils.py:83-99) for this
 * path: rank, world size, the row partition (ShardInfo rule, distribute_utils.py:101-128) and, per rank, the peer-mapped
 * addresses (CUDA IPC / symmetric memory, mapped into this process by the caller) of
 *   zbuf0, zbuf1 : two pair-shard buffers, rmax * N * 128 bf16 each (rmax = largest row count of a rank);
 *   plane_a, plane_b : (128 / world) * N * pad8(N) bf16, operand planes of the rank's channels;
 *   plane_o : rmax * 128 * pad8(N) bf16, contraction output rows;
 *   bias : 16 * N * pad8(N) 16-bit, pair bias / pair logits [head][query][key];
 *   flags : 8 ints, zero before the first call, used by nothing else.
 * world must be 2, 4 or 8.  Every rank makes the same sequence of calls.  On entry the rank's rows are in its own
 * zbuf<z_slot>; on return they are in zbuf<*z_slot_out>.  s (bf16 [N][384], replicated) may be NULL. */
typedef struct xfold_shard_ctx xfold_shard_ctx;
typedef struct {
  int world, rank, n_tokens;
  const int* row_starts; /* world + 1 offsets */
  void* const* zbuf0;
  void* const* zbuf1;
  void* const* plane_a;
  void* const* plane_b;
  void* const* plane_o;
  void* const* bias;
  void* const* flags;
} xfold_shard_desc;
int xfold_shard_ctx_create(xfold_ctx* ctx, const xfold_shard_desc* desc, xfold_shard_ctx** out);
void xfold_shard_ctx_destroy(xfold_shard_ctx* sc);
size_t xfold_shard_workspace_bytes(const xfold_shard_ctx* sc);
/* EXPERIMENTAL overlap of the exchanges with the GEMMs that produce their data: a producing stage is cut into `chunks`
 * (1..8, default 1 = off) so that a finished chunk's rows travel to their owners on the context's second stream while the
 * next chunk is computed; the chunked GEMMs leave `reserved_sms` SMs (0..64, default 0) free, for which the exchange
 * kernels are then sized -- a persistent GEMM CTA fills its SM, so with none reserved the two kinds of kernel take turns.
 * Measured as no faster on 2-8 GPUs, and with more than one chunk small problems (N = 128 on two GPUs) gave results that
 * varied between runs; the default reproduces the one-GPU path bit for bit. */
int xfold_shard_ctx_set_overlap(xfold_shard_ctx* sc, int chunks, int reserved_sms);
int xfold_pairformer_stack_sharded_fwd(xfold_ctx* ctx, xfold_shard_ctx* sc, int z_slot, void* s, const float* pair_mask,
                                       const float* seq_mask, const xfold_pairformer_weights* blocks, int num_blocks,
                                       void* ws, size_t ws_bytes, void* stream, int* z_slot_out);
/* The incoming-edges product of TriangleMultiplication ('ckj,cki->cij', nn/d_triangle_multiplication.py:122-124) on the
 * channel planes of xfold_trimul_contract_planes_fwd: a, b [channels][Nk][ld] -> o[c][i][j] = sum_k a[c][k][j] * b[c][k][i],
 * o [channels][Ni][ldo]; no transposed copy is made. */
int xfold_trimul_contract_planes_incoming_fwd(xfold_ctx* ctx, const void* a, const void* b, int channels, int Nk, int Ni,
                                              int Nj, int ld, void* o, int ldo, void* stream);

/* ---- update-only variants ----------------------------------------------------------------------
 * The reference's module forwards return the update and the caller adds it (`pair += module(pair, ...)`,
 * nn/d_pairformer.py:122-146).  These write the update to `update` (same shape as z) and leave z untouched. */
int xfold_triangle_multiplication_update_fwd(xfold_ctx* ctx, const void* z, void* update, const float* mask, int N,
                                             int outgoing, const xfold_trimul_weights* w, void* ws, size_t ws_bytes,
                                             void* stream);
int xfold_triangle_attention_update_fwd(xfold_ctx* ctx, const void* z, void* update, const float* mask, int N,
                                        int transpose, const xfold_triattn_weights* w, void* ws, size_t ws_bytes,
                                        void* stream);
int xfold_transition_update_fwd(xfold_ctx* ctx, const void* x, void* update, long long rows, int C, int F,
                                const xfold_transition_weights* w, void* ws, size_t ws_bytes, void* stream);

/* ---- fp32 validation build ------------------------------------------------------------------------
 * The same block with float32 storage and float32 arithmetic (plain FMA products on the CUDA cores, exact
 * exponentials), the counterpart of the float32 bodies the reference's ops dispatch to by dtype
 * (csrc/Alpha_Attention.cpp:63-69, 85-91, 162-168).  It exists to check the path against the reference's float32
 * results to 1e-4; it is not tuned.  Weights are float32 in the reference's OWN layouts (no packing):
 * torch.nn.Linear weights [out][in]; `projection` / `gate` [256][128] with a / b rows interleaved as in the
 * checkpoint (nn/d_triangle_multiplication.py:162-165); qkvg = q, k, v, gating_query weights stacked [4c][c]. */
typedef struct {
  const float *ln_in_gamma, *ln_in_beta, *projection, *gate, *ln_c_gamma, *ln_c_beta, *output_projection, *gating_linear;
} xfold_trimul_weights_f32;
typedef struct {
  const float *ln_gamma, *ln_beta, *pair_bias_projection, *qkvg, *output_projection;
} xfold_triattn_weights_f32;
typedef struct {
  const float *ln_gamma, *ln_beta, *transition1, *transition2;
} xfold_transition_weights_f32;
typedef struct {
  xfold_trimul_weights_f32 tri_out, tri_in;
  xfold_triattn_weights_f32 att_start, att_end;
  xfold_transition_weights_f32 pair_transition;
  const float *spl_ln_gamma, *spl_ln_beta, *spl_w; /* single path; spl_w NULL when the block has none */
  const float *sa_ln_gamma, *sa_ln_beta, *sa_qkvg /* [1536][384] */, *sa_qkvg_bias /* [1536], zero past the q rows */,
      *sa_out /* [384][384] adaptive_zero_init.transition2 */;
  xfold_transition_weights_f32 single_transition;
} xfold_pairformer_weights_f32;
size_t xfold_pairformer_f32_workspace_bytes(int N);
/* z float32 [N][N][128], s float32 [N][384] (or NULL), updated in place by `num_blocks` blocks. */
int xfold_pairformer_stack_f32_fwd(xfold_ctx* ctx, float* z, float* s, const float* pair_mask, const float* seq_mask,
                                   int N, const xfold_pairformer_weights_f32* blocks, int num_blocks, void* ws,
                                   size_t ws_bytes, void* stream);

/* ---- Transition for callers that cannot allocate device memory ------------------------------------
 * (This entry point has no counterpart in the reference.)
 * Same operation and result as xfold_transition_fwd, but the scratch (normalised input and SwiGLU
 * hidden activations) is a fixed array inside the library instead of a caller workspace.  It is meant
 * for hosts that are handed input/output buffers but may not call cudaMalloc themselves, e.g. a plugin
 * running inside another runtime's memory arena, or a latency path where allocation is forbidden.
 *  - Limit: xfold_transition_workspace_bytes(rows, C, F) must not exceed
 *    xfold_transition_static_max_bytes() (16 MiB: at most 4368 rows of the single representation, C 384 / F 1536,
 *    or 13105 pair tokens with C 128 / F 512); larger calls are rejected with XFOLD_ERR_ARG.
 *  - Every GPU that loads the library carries the array until the process exits.
 *  - The first call on a device looks up the array's device address (the context's device must be
 *    current); make that first call before starting any stream capture.
 *  - No cudaMalloc / cudaFree or other allocating call is made.  Nothing in the scratch has to start
 *    from zero: each call overwrites every element it later reads, so stale contents of an earlier call
 *    are harmless.  All calls share the one array: two calls that overlap on the GPU (different streams)
 *    race on it; serialise them. */
size_t xfold_transition_static_max_bytes(void);
int xfold_transition_static_fwd(xfold_ctx* ctx, void* x, long long rows, int C, int F,
                                const xfold_transition_weights* w, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XFOLD_B200_H_ */
