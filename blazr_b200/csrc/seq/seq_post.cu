// seq_post.cu -- the residual path of post-norm layers: sublayers read the residual x itself, a sublayer's result is multiplied by a
// learned sigmoid gate, and the layer norm (weight and bias) comes after the sum:
//     x <- LN(alpha * x + sigmoid(zg + gb) * y) * w + b
// plus the token shift in front of a mixer: the mixer reads x_t + (x_(t-1) - x_t) * mu, with the previous token's x carried per
// sequence in a state slot.  All arithmetic in f32; outputs that feed a linear layer are written in the activation type.
//
// Who writes the shift state: the post-norm kernel that closes the mixer's sublayer still reads the mixer's input x and stores the
// row of every entry's last token into the slot.  The shift itself only reads the slot (for an entry's first token), in an earlier
// launch, so no block reads a slot another block of the same launch writes.
#include "seq_common.cuh"

namespace b200seq {

// grid (T): out_plain[t] = x[t], out_shift[t] = x[t] + (prev - x[t]) * mu
__global__ void token_shift_kernel(const float* __restrict__ x, int W, const float* __restrict__ mu, const float* __restrict__ state, const b200seq_step st,
                                   void* __restrict__ out_plain, void* __restrict__ out_shift, int out_dtype) {
    const int t = blockIdx.x;
    const int e = st.tok_ent[t];
    const float* cur = x + (int64_t)t * W;
    const float* prev = nullptr;
    if (t > st.ent_start[e]) prev = cur - W;
    else if (st.ent_pos0[e] != 0) prev = state + (int64_t)st.ent_slot[e] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float c = cur[i], p = prev ? prev[i] : 0.f;
        if (out_plain) store_act(out_plain, out_dtype, (int64_t)t * W + i, c);
        store_act(out_shift, out_dtype, (int64_t)t * W + i, fmaf(p - c, mu[i], c));
    }
}

struct PostArgs {
    const float *x, *y, *zg;
    int64_t ldz;
    const float* gate_b;
    float alpha;
    const float *w, *b;
    float eps;
    int W;
    const int32_t* rows;
    float* x_out;
    void* a_out;
    int out_dtype;
    float* state_out;          // shift state of the layer whose mixer sublayer this closes (its input x is stored), or null
    const float* next_mu;      // single-token steps: the token shift of the NEXT mixer on the new x, from next_state
    const float* next_state;
    void* a_shift_out;
};

// grid (R), one block per row r (token t = rows ? rows[r] : r); dynamic shared memory: W floats + 40 of reduction scratch
__global__ void post_norm_kernel(const PostArgs a, const b200seq_step st) {
    extern __shared__ __align__(16) float sm[];
    float* u = sm;
    float* red = sm + a.W;
    const int r = blockIdx.x;
    const int64_t t = a.rows ? a.rows[r] : r;
    const int W = a.W;
    const float* xr = a.x + t * W;
    int e = -1;
    bool last = false;
    if (a.state_out || a.next_mu) {
        e = st.tok_ent[t];
        last = t + 1 == st.ent_start[e + 1];
    }
    float part = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float xv = xr[i];
        float v = xv;
        if (a.y) {
            const float g = a.zg ? sigmoidf_acc(a.zg[t * a.ldz + i] + (a.gate_b ? a.gate_b[i] : 0.f)) : 1.f;
            v = fmaf(a.alpha, xv, g * a.y[t * W + i]);
        }
        if (a.state_out && last) a.state_out[(int64_t)st.ent_slot[e] * W + i] = xv;
        u[i] = v;
        part += v;
    }
    const float mean = block_sum(part, red) / (float)W;    // block_sum's barriers also publish u
    float sq = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float d = u[i] - mean;
        sq = fmaf(d, d, sq);
    }
    const float rinv = 1.0f / sqrtf(block_sum(sq, red) / (float)W + a.eps);
    const float* prev = nullptr;
    if (a.next_mu && st.ent_pos0[e] != 0) prev = a.next_state + (int64_t)st.ent_slot[e] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float n = fmaf((u[i] - mean) * rinv, a.w[i], a.b ? a.b[i] : 0.f);
        if (a.x_out) a.x_out[t * W + i] = n;
        if (a.a_out) store_act(a.a_out, a.out_dtype, (int64_t)r * W + i, n);
        if (a.next_mu) store_act(a.a_shift_out, a.out_dtype, (int64_t)r * W + i, fmaf((prev ? prev[i] : 0.f) - n, a.next_mu[i], n));
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" int b200seq_token_shift(const float* x, int W, const float* mu, const float* state, const b200seq_step* st, void* out_plain, void* out_shift,
                                   int out_dtype, void* stream) {
    if (!x || !mu || !state || !st || !out_shift || W < 1) return fail(B200SEQ_ERR_INVALID_ARG, "token_shift: bad arguments");
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "token_shift: output dtype");
    if (st->T == 0) return 0;
    token_shift_kernel<<<st->T, W >= 1024 ? 256 : 128, 0, (cudaStream_t)stream>>>(x, W, mu, state, *st, out_plain, out_shift, out_dtype);
    SEQ_LAUNCH_CHECK("token_shift");
    return 0;
}

extern "C" int b200seq_post_norm(const float* x, const float* y, const float* zg, int64_t ldz, const float* gate_b, float alpha, const float* w, const float* b,
                                 float eps, int W, const int32_t* rows, int R, float* x_out, void* a_out, int out_dtype, float* state_out, const float* next_mu,
                                 const float* next_state, void* a_shift_out, const b200seq_step* st, void* stream) {
    if (!x || !w || W < 1 || R < 0 || (zg && (!y || ldz < W)) || (gate_b && !zg)) return fail(B200SEQ_ERR_INVALID_ARG, "post_norm: bad arguments");
    if ((state_out || next_mu) && (!st || rows)) return fail(B200SEQ_ERR_INVALID_ARG, "post_norm: the shift state needs the step and all rows");
    if (next_mu && (!next_state || !a_shift_out || st->T != st->B)) return fail(B200SEQ_ERR_INVALID_ARG, "post_norm: the fused shift is for single-token steps");
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "post_norm: output dtype");
    if (R == 0) return 0;
    const size_t smem = ((size_t)W + 40) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "post_norm: width %d too large", W);
    const PostArgs a{x, y, zg, ldz, gate_b, alpha, w, b, eps, W, rows, x_out, a_out, out_dtype, state_out, next_mu, next_state, a_shift_out};
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(post_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "post_norm attribute");
    }
    b200seq_step none{};
    post_norm_kernel<<<R, W >= 4096 ? 512 : (W >= 1024 ? 256 : 128), smem, (cudaStream_t)stream>>>(a, st ? *st : none);
    SEQ_LAUNCH_CHECK("post_norm");
    return 0;
}
