/*
 * b200seq.h -- C ABI of libb200seq.so: dense (bfloat16-weight) linear layers and the sequence operators of
 * layer-list models on B200 (sm_100a): multi-stream residual mixing with grouped RMS norm, short causal
 * convolutions with carried state, chunk/window-masked attention over a paged KV pool, the selective
 * state-space recurrence with per-slot state, gated feed-forward activations, the depth-averaged residual,
 * mixtures of experts (routed or chosen by a table), retention (fixed-decay linear attention), latent
 * attention (low-rank key / value cache, soft-max sink), per-head projections, token shift and the gated
 * post-norm residual, the residual with the norm on the sublayer's output and two-branch mixers, weighted
 * q / k norms, soft-capped scores, kept first positions, differential attention, minGRU and real-gated
 * linear recurrences, PolyNorm, soft-max routing with identity experts, a hashed bigram embedding,
 * arg-max sampling.
 *
 * It sits beside libb200q (include/b200q.h), which holds the quantized linear layer; the conventions are
 * the same:
 *   - every function returns 0 or a negative status; b200seq_last_error() gives the message;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - no allocation, no host synchronisation, no host scalar that changes from step to step: a step of
 *     fixed token count is CUDA-graph capturable;
 *   - no CPU fallback.
 *
 * A step is a flat batch of T tokens belonging to B entries (one entry = the next tokens of one request,
 * a prompt portion or a single decoded token).  The int32 device arrays every sequence operator reads:
 *   tok_ent[T]        entry of each token
 *   tok_pos[T]        position of each token in its sequence (from 0)
 *   ent_start[B + 1]  first token row of each entry (prefix sums of the portion lengths)
 *   ent_slot[B]       state slot of the entry's request
 *   ent_pos0[B]       position of the entry's first token (0 = a new sequence: carried state reads as zero)
 *   block_table[B][max_blocks]  KV pages of the entry's request
 * Activations that feed a linear layer are written in `act` dtype (B200SEQ_F32 or B200SEQ_BF16); everything
 * else (residual streams, norms, scores, recurrent state, KV pool) is float32.
 */
#ifndef B200SEQ_H
#define B200SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200SEQ_OK 0
#define B200SEQ_ERR_INVALID_ARG (-1)
#define B200SEQ_ERR_UNSUPPORTED (-2)
#define B200SEQ_ERR_CUDA (-3)

#define B200SEQ_F32 0
#define B200SEQ_BF16 2

/* b200seq_causal_conv modes */
#define B200SEQ_CONV_RESIDUAL 1 /* out = x + conv(x) */
#define B200SEQ_CONV_SILU 2     /* out = silu(conv(x) + bias) */

/* b200seq_linear paths */
#define B200SEQ_PATH_AUTO 0
#define B200SEQ_PATH_ROWS 1   /* weight-streaming warp-per-row kernel (few tokens) */
#define B200SEQ_PATH_TILED 2  /* float32 FMA tiles (any M, exact 32-bit arithmetic) */
#define B200SEQ_PATH_TC 3     /* tcgen05 tensor-core tiles (bf16 activations) */

typedef struct b200seq_step {
    const int32_t* tok_ent;
    const int32_t* tok_pos;
    const int32_t* ent_start;
    const int32_t* ent_slot;
    const int32_t* ent_pos0;
    const int32_t* block_table;
    int32_t T, B, max_blocks, block_size;
} b200seq_step;

const char* b200seq_last_error(void);
int b200seq_version(void);
int64_t b200seq_launch_count(void);
/* bit 0: a KV position fell outside its block table; bit 1: a bounded wait of the tensor-core GEMM ran out; bit 2: an expert table entry outside the experts */
int b200seq_error_flags(int* flags_out);

/* X[t][s][:] = table[ids[t]][:] * scale for every stream s.  table: bf16 [V, W]; X: f32 [T, S, W]. */
int b200seq_embed_streams(const void* table_bf16, const int32_t* ids, float scale, int T, int S, int W, float* X, void* stream);

/* Stream update and collapse around a sublayer, one block per row r (token t = rows ? rows[r] : r):
 *   if y:      X[t][j] <- sum_s post[S + s * S + j] * X[t][s] + post[j] * y[t]      (post = out[S] | mix[S][S], mix indexed [from][to])
 *   if norm_w: u = sum_s in_w[s] * X[t][s];  out[r] = group_rms(u, groups, eps) * norm_w
 * y: f32 [T, W] or null; out: [R, W] in out_dtype. */
int b200seq_hc_norm(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                    const int32_t* rows, int R, void* out, int out_dtype, void* stream);

/* The same followed by the sublayer's carried convolution (mode B200SEQ_CONV_RESIDUAL, no bias) in one kernel, for steps in which every
 * entry brings exactly one token (st->T == st->B, all rows): out[t] = h + conv(h), conv_state[slot][taps-1][W] read and shifted. */
int b200seq_hc_norm_conv(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                         const float* conv_w, float* conv_state, const b200seq_step* st, int taps, void* out, int out_dtype, void* stream);

/* Per-channel causal convolution over time with the last taps-1 inputs of every sequence carried in
 * state[slot][taps-1][C] (f32; read as zero when ent_pos0 == 0, rewritten for every entry of the step).
 * x: f32 rows of stride ldx; w: f32 [C, taps] (last column = current token); bias f32 [C] or null. */
int b200seq_causal_conv(const float* x, int64_t ldx, const float* w, const float* bias, float* state, const b200seq_step* st, int C, int taps, int mode,
                        void* out, int out_dtype, int64_t ldo, void* stream);

/* out[t] = group_rms(x[t], groups, eps) * w   (x f32 [T, D] stride ldx; out act dtype [T, D]) */
int b200seq_group_rmsnorm(const float* x, int64_t ldx, const float* w, int T, int D, int groups, float eps, void* out, int out_dtype, void* stream);

/* gu: f32 [T, 2F] = gate | up (interleaved = 0) or gate 0, up 0, gate 1, up 1, ... (interleaved = 1).
 * g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + up_shift) */
int b200seq_gated_act(const float* gu, int64_t ldg, int T, int F, float limit, float alpha, float up_shift, int interleaved, void* out, int out_dtype,
                      void* stream);

/* y[M, N] (f32, stride ldy) = x[M, K] (f32 or bf16, stride ldx) . w[N, K]^T (bf16, contiguous) */
int b200seq_linear(const void* x, int x_dtype, int64_t ldx, const void* w_bf16, int M, int N, int K, float* y, int64_t ldy, int path, void* stream);

/* Fused gate|up projection + gated activation: w_il is the stacked weight [2F, K] with rows alternating (gate 0, up 0, gate 1, up 1, ...);
 * out[M, F] (act dtype, stride ldo) = gated_act(x . w_il^T) with the formula of b200seq_gated_act.  The [M, 2F] product is never written.
 * M <= 8: weight-streaming rows (f32 or bf16 activations); more rows: the tensor-core path, which needs bf16 activations, K % 8 == 0 and
 * 16-byte aligned rows (B200SEQ_ERR_UNSUPPORTED otherwise). */
int b200seq_linear_gated(const void* x, int x_dtype, int64_t ldx, const void* w_il_bf16, int M, int F, int K, float limit, float alpha, float up_shift,
                         void* out, int out_dtype, int64_t ldo, void* stream);

/* Attention over a paged f32 KV pool (kpool [blocks][block_size][G][D], vpool [..][G][V]).
 * qkvg: f32 [T, ld] = q (H*D) | k (G*D) | v (G*V) | gate (H, only if gated).
 * prep: q and k are divided per head by their RMS over D when qk_eps >= 0 (q in place), k and v go to the pool.
 * attend: token at position i sees j <= i with floor(j / chunk) == floor(i / chunk) (chunk > 0) and i - j < window (window > 0);
 *         softmax in f32, output times sigmoid(gate) when gated, written in act dtype to out [T, H*V]. */
int b200seq_attn_prep(float* qkvg, int64_t ld, const b200seq_step* st, float* kpool, float* vpool, int H, int G, int D, int V, float qk_eps, void* stream);
size_t b200seq_attn_scratch_floats(int T, int B, int H, int G, int V, int max_keys);
/* scratch: f32 work area of b200seq_attn_scratch_floats(...) floats (max_keys = the most keys a token can see) or null: with it, steps of
 * few tokens split the keys of a row among several blocks and merge the partial soft-max results. */
int b200seq_attn(const float* qkvg, int64_t ld, const b200seq_step* st, const float* kpool, const float* vpool, int H, int G, int D, int V, float scale,
                 int chunk, int window, int gated, void* out, int out_dtype, float* scratch, size_t scratch_floats, void* stream);

/* Selective state-space recurrence, per head h (group g = h / (H / G)), state[slot][H][N][V] f32 carried per sequence:
 *   dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(A_log[h]) * dt) * S + dt * B x^T;  y = S^T C + D[h] * x;  out = y * silu(z)
 * proj: f32 rows (stride ldp) with z at column z0 (H*V) and dt_raw at column dt0 (H);
 * xbc:  f32 rows (stride ldx) = x (H*V) | B (G*N) | C (G*N), already convolved and activated.  out: f32 [T, H*V].
 * scratch: f32 work area of b200seq_ssm_scratch_floats(T, B, ...) floats or null.  With it, steps of many tokens cut every portion into
 * segments that run in parallel (local pass, in-order combine, final pass); without it (or for short steps) each portion is one
 * sequential walk.  Both give the same result up to rounding. */
size_t b200seq_ssm_scratch_floats(int T, int B, int H, int V, int N);
int b200seq_ssm_scan(const float* proj, int64_t ldp, int z0, int dt0, const float* xbc, int64_t ldx, const float* A_log, const float* Dp, const float* dt_bias,
                     float* state, const b200seq_step* st, int H, int V, int N, int G, float* out, float* scratch, size_t scratch_floats, void* stream);

/* ---- activations of a projection ------------------------------------------------------------------------------------------------
 * gated kinds take a stacked gate|up product whose rows alternate (gate j, up j) and give F = N / 2 outputs:
 *   B200SEQ_ACT_SWISH_CLAMP  g = min(gate, limit), u = clamp(up, -limit, limit): g * sigmoid(alpha * g) * (u + shift)
 *   B200SEQ_ACT_GELU_TANH    0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * up
 * plain kinds give N outputs:
 *   B200SEQ_ACT_RELU2        max(z, 0)^2 */
#define B200SEQ_ACT_SWISH_CLAMP 0
#define B200SEQ_ACT_GELU_TANH 1
#define B200SEQ_ACT_RELU2 2
#define B200SEQ_ACT_IDENT 3 /* plain kind: the product itself, written in out_dtype (a projection whose result feeds the next linear layer) */

/* out = act(x . w^T), the product itself never reaches memory.  w: bf16 [N, K]; out [M, N / 2] (gated kinds) or [M, N] (plain kinds) in
 * out_dtype, row stride ldo.  M <= 8: weight-streaming rows (f32 or bf16 activations); more rows: the tensor-core path, which needs bf16
 * activations, K % 8 == 0 and 16-byte aligned rows (B200SEQ_ERR_UNSUPPORTED otherwise).  b200seq_linear_gated is kind SWISH_CLAMP. */
int b200seq_linear_act(const void* x, int x_dtype, int64_t ldx, const void* w_bf16, int M, int N, int K, int act, float limit, float alpha, float shift,
                       void* out, int out_dtype, int64_t ldo, void* stream);
/* the same activation applied to a product that is in memory: z f32 [T, N] (stride ldz); gated kinds read interleaved pairs */
int b200seq_act(const float* z, int64_t ldz, int T, int N, int act, float limit, float alpha, float shift, void* out, int out_dtype, int64_t ldo, void* stream);

/* ---- depth-averaged residual + layer norm ---------------------------------------------------------------------------------------------
 * One residual stream whose layer inputs are learned averages over depth: with X_0 the embedding and X_(i+1) = x_i + y1 + y2 the result of
 * layer i (x_i = what layer i read), the next layer reads x_(i+1) = sum_(j <= i + 1) dwa[j] X_j.  One kernel, one block per row r
 * (token t = rows ? rows[r] : r), does what lies between two layers:
 *   if y1:   X_new = x_cur[t] + (y1[t] + y2[t])        (y2 may be null)
 *            hist_out[t] <- X_new                      (if hist_out: layer i stores X_(i+1) for the layers after it)
 *            x = dwa ? sum_(j < n_prev) dwa[j] * hist[j * hist_stride + t * W] + dwa[n_prev] * X_new : X_new;   x_out[t] <- x
 *   else     x = x_cur[t]
 *   out1[r] = layer_norm(x) * w1, out2[r] = layer_norm(x) * w2   (each optional; (x - mean) / sqrt(var + eps), biased variance, no bias)
 * Everything in f32; out1 / out2 in out_dtype.  x_out may be x_cur. */
int b200seq_depth_norm(const float* hist, int64_t hist_stride, int n_prev, const float* dwa, const float* x_cur, const float* y1, const float* y2,
                       float* hist_out, float* x_out, int W, float eps, const float* w1, const float* w2, const int32_t* rows, int R, void* out1, void* out2,
                       int out_dtype, void* stream);

/* ---- attention, general form ------------------------------------------------------------------------------------------------------------
 * Columns of the projection row: q at q_col (H*D), k at k_col (G*D), v at v_col (G*V; v_col == k_col: the values are the keys as projected,
 * before norm and rotation; needs V == D), one gate logit per query head at gate_col (< 0: no gate).
 * prep, in this order: unit-RMS q and k (qk_eps >= 0); rotation of the first rot_dims dimensions of every q and k head (rot_dims > 0):
 * the pair (2i, 2i+1) at position p turns by the angle p * rot_freq[i] and is multiplied by rot_scale (rot_freq: device f32 [rot_dims / 2]);
 * k and v go to the pool; when pool > 0 every block of `pool` positions that the step completes gets its mean key and mean value (of the
 * pool's rows, summed in position order) written to kpooled / vpooled: [blocks][pooled_per_page][G][D or V] with
 * pooled_per_page = ceil(block_size / pool), block b of a sequence lives in the page of its first position.
 * attend: as b200seq_attn; with pool > 0 (needs window > 0) position i also sees, in the same soft-max, the pooled key and value of every
 * block b with b * pool + pool - 1 <= i - window. */
typedef struct b200seq_attn_desc {
    int32_t H, G, D, V;
    int32_t q_col, k_col, v_col, gate_col;
    float scale;
    int32_t chunk, window, pool;
    float qk_eps;
    int32_t rot_dims;
    const float* rot_freq;
    float rot_scale;
    const float* sink;  /* attend: device f32 [H] or null; exp(sink[h]) is one more term of head h's soft-max denominator (no key, no value, not scaled) */
    int32_t latent_v;   /* attend: 1 = the values are the first V floats of the (single) key head's pool rows, vpool is not read (G == 1, V <= D) */
    const float* gate;  /* attend: when not null (and gate_col >= 0) the gate logit of (t, h) is gate[t * gate_ld + h] instead of the query row's */
    int64_t gate_ld;
    int32_t ctx_rows;   /* attend: 1 = kpool / vpool hold the step's gathered context instead of pages: the rows of entry 0's positions 0 .. pos0 + len - 1,
                           then entry 1's, ... (b200seq_latent_gather's order) */
    int32_t kd;         /* attend: 0 < kd < D: only the first kd floats of a key head lie in kpool (head g at g * kd); the other D - kd are one part
                           shared by all heads, read from krot's PAGED rows: krot[(page row) * krot_ld + (d - kd)] */
    int64_t kv_ld;      /* attend: > 0: floats per position row of kpool and of vpool (default G * D and G * V) */
    const float* krot;
    int64_t krot_ld;
    /* ---- fields below default to zero / null (older initialisers leave them so) ---- */
    const float* q_norm_w; /* prep: weighted RMS norm of q (needs qk_eps >= 0): [D] shared by all heads, or [H * D] when norm_full */
    const float* k_norm_w; /* prep: the same for k: [D] or [G * D] */
    int32_t norm_full;     /* prep: 1 = the RMS is taken over the whole q projection (all heads at once), and over the whole k projection */
    int32_t rot_half;      /* prep: 1 = rotated pairs are (i, i + rot_dims / 2) instead of (2i, 2i + 1) */
    const float* in_bias;  /* prep: f32 bias of the projection row (indexed by the row's columns), added to q, k and v before everything else */
    int32_t kv_shared;     /* prep: 1 = keys and values of this layer are another layer's pool rows: only the queries are prepared */
    int32_t vg;            /* > 0: number of value heads when it differs from G (G % vg == 0): key head g reads value head g / (G / vg) */
    float softcap;         /* attend: > 0: score <- softcap * tanh(score / softcap) after scaling */
    const float* head_scale; /* attend: device f32 [H] or null: the score of head h is also multiplied by head_scale[h] */
    int32_t keep_first;    /* attend (window > 0): positions j < keep_first stay visible to every later position, at their true positions */
    int32_t gate_elem;     /* attend (gate_col >= 0): 1 = one gate logit per output element, H * V of them at gate_col (or in `gate`), instead of one per head */
} b200seq_attn_desc;
int b200seq_attn_prep_ex(float* proj, int64_t ld, const b200seq_step* st, const b200seq_attn_desc* d, float* kpool, float* vpool, float* kpooled, float* vpooled,
                         void* stream);
int b200seq_attn_ex(const float* proj, int64_t ld, const b200seq_step* st, const b200seq_attn_desc* d, const float* kpool, const float* vpool,
                    const float* kpooled, const float* vpooled, void* out, int out_dtype, float* scratch, size_t scratch_floats, void* stream);

/* ---- latent attention: prep ---------------------------------------------------------------------------------------------------------------
 * The cache of a latent-attention layer holds per token one row [c (R) | kr (Rd)] of a pool [blocks][block_size][R + Rd]: the normed latent
 * c = rms_norm(kv[0 .. R), eps) * norm_w and the rotated key part kr = rot(kv[R .. R + Rd)) that all heads share, kv = proj[t][c_col ..).
 * Keys never leave the latent space: with k_h = [W_h c | kr] the score of head h is (W_h^T q_h[0 .. Dn)) . c + rot(q_h[Dn ..)) . kr, so the
 * attention runs as H query heads of size R + Rd over one key head whose values are its first R floats (b200seq_attn_desc.latent_v), and
 * the value projection is applied to the R-sized result.  This call, per token: writes the pool row; writes rot(q_h[Dn ..)) to
 * Qp[t][h * (R + Rd) + R ..) (the caller's projection fills the R columns before it); writes q_h[0 .. Dn) in qn_dtype to qn[(t * H + h)][Dn]
 * (the input of that projection); copies the H gate logits proj[t][gate_col ..) to Qp[t][H * (R + Rd) ..) when gate_col >= 0.
 * q: f32 [T, ldq] = H heads of [Dn | Rd].  Rotation: pairs (2i, 2i + 1), angle pos * rot_freq[i], cos and sin times rot_scale. */
int b200seq_latent_prep(const float* proj, int64_t ldp, int c_col, int gate_col, const float* q, int64_t ldq, const b200seq_step* st, int H, int Dn, int Rd, int R,
                        const float* norm_w, float eps, const float* rot_freq, float rot_scale, float* kpool, float* Qp, int64_t ldQ, void* qn, int qn_dtype,
                        void* stream);
/* Steps of prompt portions attend over per-head keys instead (fewer operations per key than in the latent space): Qp == qn == null makes
 * latent_prep turn the rotated part of every query head IN PLACE in q; b200seq_latent_gather then copies the latents of every position of
 * every entry's context (0 .. pos0 + len - 1, entry after entry: ctx_rows rows in all) out of the pages into out [ctx_rows, R] in out_dtype,
 * one projection of those rows gives per-head keys and values, and b200seq_attn_ex runs with ctx_rows = 1, kd = the unrotated key size and
 * krot = the pool's rotated part.  Both forms give the same result up to rounding. */
int b200seq_latent_gather(const float* kpool, int64_t kld, const b200seq_step* st, int R, int ctx_rows, void* out, int out_dtype, void* stream);

/* ---- per-head projections ------------------------------------------------------------------------------------------------------------------
 * out[t][h * ocol + n] = sum_k x[t][h * K + k] * w[h][n][k] for every token t < T and head h < H: x rows (f32 or bf16, stride ldx) hold the heads'
 * inputs side by side, w is bf16 [H][N][K], out rows (stride ldo) hold the heads' results at a pitch of ocol >= N columns.  act: -1 the f32
 * product; a plain kind (B200SEQ_ACT_IDENT: the product itself) written in out_dtype.  Few (token, head) pairs: the weights are streamed per
 * pair; many tokens: tcgen05 tiles per head (bf16 rows, K % 8 == 0, 16-byte aligned) or exact f32 fma tiles. */
int b200seq_head_linear(const void* x, int x_dtype, int64_t ldx, const void* w_bf16, int T, int H, int N, int K, int act, void* out, int out_dtype, int64_t ldo,
                        int64_t ocol, void* stream);

/* ---- rotary positions on head vectors inside projection rows -------------------------------------------------------------------------------
 * x[t][col + h * D + ..], h < nheads: the first rot_dims dimensions of every head turn by pos * freq[i]; pair (i, i + rot_dims / 2) when
 * half = 1, (2i, 2i + 1) when half = 0; cos and sin times rot_scale; then every element of the head times mult.  In place. */
int b200seq_rotary(float* x, int64_t ld, int col, int nheads, int D, const b200seq_step* st, int rot_dims, int half, const float* freq, float rot_scale, float mult,
                   void* stream);

/* ---- retention ---------------------------------------------------------------------------------------------------------------------------------
 * Linear attention with one fixed decay per head, no soft-max, no denominator.  Columns of the f32 projection row: q at q_col (H*D),
 * k at k_col (H*D), v at v_col (H*V), gate at g_col (H*V).  q and k get rotary positions (as b200seq_rotary; q and k are turned in place
 * in steps of portions), k is multiplied by k_scale; per head with state[slot][H][D][V] (f32, read as zero when ent_pos0 == 0):
 *   S_t = decay[h] * S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t;   out[t][h] = o_t / sqrt(mean(o_t^2) + eps) * silu(gate_t[h])   (act dtype [T, H*V])
 * decay: device f32 [2][H] = the decays, then their base-2 logarithms.  Steps in which every entry brings one token run one kernel and need
 * no work area; other steps cut the portions into chunks that run in parallel and need b200seq_retention_scratch_floats(...) floats. */
typedef struct b200seq_retention_desc {
    int32_t H, D, V;
    int32_t q_col, k_col, v_col, g_col;
    const float* decay;
    float eps;
    int32_t rot_dims, rot_half;
    const float* rot_freq;
    float rot_scale, k_scale;
} b200seq_retention_desc;
size_t b200seq_retention_scratch_floats(int T, int B, int H, int D, int V);
int b200seq_retention(float* proj, int64_t ld, const b200seq_step* st, const b200seq_retention_desc* d, float* state, void* out, int out_dtype, float* scratch,
                      size_t scratch_floats, void* stream);

/* ---- post-norm residual path with token shift and gated residual ------------------------------------------------------------------------
 * token_shift: out_shift[t] = x[t] + (prev - x[t]) * mu with prev = x[t - 1] inside a portion, state[slot] for a portion's first token
 * (zero when ent_pos0 == 0); out_plain[t] = x[t] (optional); both [T, W] in out_dtype.  The state is only read here.
 * post_norm, one block per row r (token t = rows ? rows[r] : r):
 *   v = y ? alpha * x[t] + (zg ? sigmoid(zg[t * ldz + i] + gate_b[i]) : 1) * y[t] : x[t]
 *   n = (v - mean) / sqrt(var + eps) * w + b          (biased variance; b may be null)
 *   x_out[t] <- n (f32, optional, may be x);  a_out[r] <- n in out_dtype (optional)
 *   state_out (optional, all rows): state_out[slot] <- x[t] for the last token of every entry (the shift state of the layer whose mixer read x)
 *   next_mu (optional, steps with one token per entry): a_shift_out[r] <- n + (prev - n) * next_mu, prev = next_state[slot] or zero: the
 *   token shift of the next mixer in the same pass. */
int b200seq_token_shift(const float* x, int W, const float* mu, const float* state, const b200seq_step* st, void* out_plain, void* out_shift, int out_dtype,
                        void* stream);
int b200seq_post_norm(const float* x, const float* y, const float* zg, int64_t ldz, const float* gate_b, float alpha, const float* w, const float* b, float eps, int W,
                      const int32_t* rows, int R, float* x_out, void* a_out, int out_dtype, float* state_out, const float* next_mu, const float* next_state,
                      void* a_shift_out, const b200seq_step* st, void* stream);

/* ---- mixture of experts -------------------------------------------------------------------------------------------------------------------
 * route: z f32 [T, >= E] (stride ldz) router logits; s = sigmoid(z).  Experts form `groups` equal groups of neighbours; a group's score is
 * the sum of its two largest s (of its one, when groups == E); only experts of the `keep` best groups can be chosen (groups <= 1: all).
 * The `top` largest s among those are chosen (ties: the lower index), ids[t][j] in falling order of s, wts[t][j] = s / (sum of the chosen s
 * + 1e-20).  counts[E] receives how many (token, choice) pairs every expert got.
 * sort: the pairs p = t * top + j ordered by expert (stable): offs[E + 1] prefix sums, sorted[slot] = p, slot_of[p] = slot. */
int b200seq_moe_route(const float* z, int64_t ldz, int T, int E, int groups, int keep, int top, int32_t* ids, float* wts, int32_t* counts, void* stream);
/* Router projection and choice of a step of at most 8 tokens in one kernel: z[t][n] = x[t] . w[n] for the NR >= E rows of the stacked router
 * weight (bf16 [NR, K]; rows behind the E experts' are projected and left in z for the caller), then the choice of b200seq_moe_route on z[t][0..E). */
int b200seq_moe_router(const void* x, int x_dtype, int64_t ldx, const void* w_bf16, int T, int NR, int K, int E, int groups, int keep, int top, float* z, int64_t ldz,
                       int32_t* ids, float* wts, void* stream);
/* Choice by table instead of a router: ids[t][j] = table[tok_ids[t]][j] (table int32 [vocab][top], the entries of a row differ),
 * wts[t][j] = 1 / top; counts as above (optional). */
int b200seq_moe_table_route(const int32_t* table, const int32_t* tok_ids, int T, int E, int top, int32_t* ids, float* wts, int32_t* counts, void* stream);
int b200seq_moe_sort(const int32_t* ids, int pairs, int E, const int32_t* counts, int32_t* offs, int32_t* sorted, int32_t* slot_of, void* stream);
/* One projection of every pair through its expert's weight: w bf16 [E][N][K].  Row r of the result belongs to pair p = sorted ? sorted[r] : r
 * (sorted + offs from b200seq_moe_sort: tiles of one expert's rows; null: one launch row per pair, weights streamed, for few pairs).
 * The input row of row r is x[(x_div > 0 ? p / x_div : r)] (x_div = top gathers the token's activations; 0: x is already laid out like the
 * result).  act: -1 none (out f32) or a plain activation kind (out in out_dtype).  out [pairs, N], stride ldo. */
int b200seq_moe_linear(const void* x, int x_dtype, int64_t ldx, int x_div, const void* w_bf16, const int32_t* ids, const int32_t* sorted, const int32_t* offs,
                       int pairs, int E, int N, int K, int act, void* out, int out_dtype, int64_t ldo, void* stream);
/* The same with any activation kind: gated kinds take expert weights [E][N][K] whose rows alternate (gate j, up j) and give out [pairs, N / 2]
 * in out_dtype (limit / alpha / shift as in B200SEQ_ACT_SWISH_CLAMP); the gate | up product never reaches memory. */
int b200seq_moe_linear_act(const void* x, int x_dtype, int64_t ldx, int x_div, const void* w_bf16, const int32_t* ids, const int32_t* sorted, const int32_t* offs,
                           int pairs, int E, int N, int K, int act, float limit, float alpha, float shift, void* out, int out_dtype, int64_t ldo, void* stream);
/* out[r] = x[sorted[r] / x_div] for every sorted pair r (bf16 rows of K): the tokens' activations in sorted order, so that the tensor-core
 * tiles of b200seq_moe_linear (sorted rows, x_div = 0, bf16, K % 8 == 0, 16-byte aligned rows, >= 32 pairs) can fetch them. */
int b200seq_moe_gather(const void* x_bf16, int64_t ldx, const int32_t* sorted, int x_div, int pairs, int K, void* out_bf16, int64_t ldo, void* stream);
/* y[t] = sum_j wts[t][j] * ys[slot_of ? slot_of[t * top + j] : t * top + j] (j ascending) + (shared ? sigmoid(gate_z[t * ldg]) * shared[t] : 0)
 * gate_z null with shared: the shared branch is added as it is.  ys, shared, y: f32 [., W]. */
int b200seq_moe_combine(const float* ys, const float* wts, const int32_t* slot_of, int T, int top, int W, const float* shared, const float* gate_z, int64_t ldg,
                        float* y, void* stream);

/* ---- the same choice with soft-max scores and a correction -------------------------------------------------------------------------------
 * kind 0: s = sigmoid(z) (b200seq_moe_route); kind 1: s = softmax(z[0 .. E)) in f32.  correction (f32 [E] or null) is added to s for the
 * CHOICE only; the weights are the chosen s / (their sum + 1e-20).  E counts every router output, identity experts included. */
int b200seq_moe_route_ex(const float* z, int64_t ldz, int T, int E, int groups, int keep, int top, int kind, const float* correction, int32_t* ids, float* wts,
                         int32_t* counts, void* stream);
/* b200seq_moe_router with the score kind and correction of b200seq_moe_route_ex */
int b200seq_moe_router_ex(const void* x, int x_dtype, int64_t ldx, const void* w_bf16, int T, int NR, int K, int E, int groups, int keep, int top, int kind,
                          const float* correction, float* z, int64_t ldz, int32_t* ids, float* wts, void* stream);
/* b200seq_moe_combine with identity experts: a pair whose expert id is >= E_real has no row in ys; its output is the token's own input
 * x_id[t] (f32 [T, W]) times the weight.  ids: [T * top]. */
int b200seq_moe_combine_ex(const float* ys, const float* wts, const int32_t* slot_of, const int32_t* ids, int E_real, const float* x_id, int T, int top, int W,
                           const float* shared, const float* gate_z, int64_t ldg, float* y, void* stream);

/* ---- b200seq_causal_conv with a bias on the INPUT (the convolution sees x + in_bias, zeros before the sequence's start; the carried state
 * holds the biased inputs) and an optional second copy of the result in out2_dtype (row stride ldo2). */
int b200seq_causal_conv_ex(const float* x, int64_t ldx, const float* in_bias, const float* w, const float* bias, float* state, const b200seq_step* st, int C, int taps,
                           int mode, void* out, int out_dtype, int64_t ldo, void* out2, int out2_dtype, int64_t ldo2, void* stream);

/* ---- embedding with a hashed bigram table ---------------------------------------------------------------------------------------------------
 * x[t] = table[ids[t]] * scale + bigram[row], row = (prev * mul_prev + ids[t] * mul_cur) mod buckets with prev the sequence's previous token:
 * ids[t - 1] inside a portion, ent_prev[e] for a portion's first token, and row = buckets (the table's last row) at position 0.
 * table bf16 [vocab, W]; bigram bf16 [buckets + 1, W] or null; ent_prev int32 [B].  x f32 [T, W]; a (optional) the same in a_dtype. */
int b200seq_embed_bigram(const void* table_bf16, const void* bigram_bf16, const int32_t* ids, const int32_t* ent_prev, const b200seq_step* st, float scale,
                         int buckets, int mul_prev, int mul_cur, int W, float* x, void* a, int a_dtype, void* stream);

/* ---- residual path with the norm on the sublayer's OUTPUT -----------------------------------------------------------------------------------
 * One block per row r (token t = rows ? rows[r] : r).  A sublayer's result is one branch y1 or the sum of two:
 *   b1 = y1[t] + bias1 (bias1 optional);  if w_b1: b1 <- rms_norm(b1, eps) * w_b1;   likewise b2 from y2 with w_b2 (y2 optional, no bias)
 *   v = s1 * b1 + s2 * b2;   x_new = x[t] + rms_norm(v, eps) * w
 *   x_out[t] <- x_new (optional, may be x);   a_out[r] <- fin_w ? rms_norm(x_new, eps) * fin_w : x_new, in out_dtype (optional)
 * rms_norm(u) = u / sqrt(mean(u^2) + eps).  Everything in f32. */
int b200seq_branch_norm(const float* x, const float* y1, const float* bias1, const float* w_b1, float s1, const float* y2, const float* w_b2, float s2,
                        const float* w, float eps, int W, const int32_t* rows, int R, float* x_out, void* a_out, int out_dtype, const float* fin_w, void* stream);

/* out[t] = c0 * N(z) + c1 * N(z^2) + c2 * N(z^3) + c3 with powers taken element by element and N(u) = u / sqrt(mean(u^2) + eps) over the
 * F values of the row; z f32 [T, F] (stride ldz), coef device f32 [4], out [T, F] in out_dtype (stride ldo). */
int b200seq_polynorm(const float* z, int64_t ldz, int T, int F, const float* coef, float eps, void* out, int out_dtype, int64_t ldo, void* stream);

/* x <- cap * tanh(x / cap) on n floats, in place */
int b200seq_softcap(float* x, int64_t n, float cap, void* stream);

/* Differential attention, second half: a f32 [T, 2 * H * V] holds the two maps' results per head in the order [g][map][r] (g < G key groups,
 * r < H / G heads of a group); out[t][h] = rms_norm(a1 - lambda * a2, eps) * out_scale over the V values of head h = g * (H / G) + r,
 * written in out_dtype as [T, H * V]. */
int b200seq_diff_combine(const float* a, int T, int H, int G, int V, float lambda, float out_scale, float eps, void* out, int out_dtype, void* stream);

/* ---- element-wise gated linear recurrences S_t = a_t * S_(t-1) + b_t with per-slot f32 state [slots][C] (zero when ent_pos0 == 0) -----------
 * min_gru:  z = sigmoid(proj[z_col + c] + bias[z_col + c]), u = proj[x_col + c] + bias[x_col + c], cand = u >= 0 ? u + 0.5 : sigmoid(u);
 *           a = 1 - z, b = z * cand;   out[t][c] = S_t * silu(proj[g_col + c])          (bias: f32 indexed by the projection row's columns, or null)
 * rg_lru:   r = sigmoid(gates[blk][c'] + gate_bias[..]), i = sigmoid(gates[blk][bw + c'] + ..) with gates rows laid out per block of bw = C / blocks
 *           channels as [r (bw) | i (bw)] and gate_bias the same layout; log a = -decay_c * r * sp_lam[c] (sp_lam = softplus(lam), precomputed),
 *           a = exp(log a), b = sqrt(1 - a^2) * i * u[t][c];   out[t][c] = S_t * gelu_tanh(proj[y_col + c] + bias[y_col + c])
 * proj, u, gates: f32 rows; out [T, C] in out_dtype. */
int b200seq_min_gru(const float* proj, int64_t ldp, int z_col, int x_col, int g_col, const float* bias, float* state, const b200seq_step* st, int C, void* out,
                    int out_dtype, void* stream);
int b200seq_rg_lru(const float* u, int64_t ldu, const float* gates, int64_t ldg, const float* gate_bias, const float* sp_lam, float decay_c, const float* proj,
                   int64_t ldp, int y_col, const float* bias, float* state, const b200seq_step* st, int C, int blocks, void* out, int out_dtype, void* stream);

/* ids[r] = argmax_v logits[r][v] (first maximum) */
int b200seq_argmax(const float* logits, int R, int V, int32_t* ids, void* stream);

#ifdef __cplusplus
}
#endif
#endif
