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

// The same with the row held in registers (W <= 4 * EPT * blockDim.x, W % 4 == 0, 16-byte accesses): a thread owns EPT pieces of four
// neighbouring elements.  PRE (steps of few rows, bound by latency): every input of the thread's pieces, the norm's weights and the next
// shift's operands included, is requested before the first is used, so a block pays one round trip to memory instead of one per pass.
// Without PRE (many rows, bound by bandwidth) only the sum is kept and the small per-column vectors are read where they are used.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void store_act4(void* out, int dtype, int64_t idx, const float4 v) {
    if (dtype == B200SEQ_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + idx) = v;
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo), u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + idx) = u;
    }
}
template <int EPT, bool PRE>
__global__ void post_norm_reg_kernel(const PostArgs a, const b200seq_step st) {
    __shared__ float red[40];
    const int r = blockIdx.x;
    const int64_t t = a.rows ? a.rows[r] : r;
    const int W = a.W, nt = blockDim.x;
    int e = -1;
    bool last = false;
    if (a.state_out || a.next_mu) {
        e = st.tok_ent[t];
        last = t + 1 == st.ent_start[e + 1];
    }
    const float* prev = nullptr;
    if (a.next_mu && st.ent_pos0[e] != 0) prev = a.next_state + (int64_t)st.ent_slot[e] * W;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 v[EPT], wv[PRE ? EPT : 1], bv[PRE ? EPT : 1], mu[PRE ? EPT : 1], pv[PRE ? EPT : 1];
    float4 xv[EPT], yv[EPT], zv[EPT], gv[EPT];
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int i = (threadIdx.x + k * nt) * 4;
        const bool in = i < W;
        xv[k] = in ? ld4(a.x + t * W + i) : zero;
        yv[k] = (in && a.y) ? ld4(a.y + t * W + i) : zero;
        zv[k] = (in && a.zg) ? ld4(a.zg + t * a.ldz + i) : zero;
        gv[k] = (in && a.gate_b) ? ld4(a.gate_b + i) : zero;
        if (PRE) {
            wv[k] = in ? ld4(a.w + i) : zero;
            bv[k] = (in && a.b) ? ld4(a.b + i) : zero;
            mu[k] = (in && a.next_mu) ? ld4(a.next_mu + i) : zero;
            pv[k] = (in && prev) ? ld4(prev + i) : zero;
        }
    }
    float part = 0.f;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int i = (threadIdx.x + k * nt) * 4;
        v[k] = xv[k];
        if (a.y) {
            const bool g = a.zg != nullptr;
            v[k].x = fmaf(a.alpha, xv[k].x, (g ? sigmoidf_acc(zv[k].x + gv[k].x) : 1.f) * yv[k].x);
            v[k].y = fmaf(a.alpha, xv[k].y, (g ? sigmoidf_acc(zv[k].y + gv[k].y) : 1.f) * yv[k].y);
            v[k].z = fmaf(a.alpha, xv[k].z, (g ? sigmoidf_acc(zv[k].z + gv[k].z) : 1.f) * yv[k].z);
            v[k].w = fmaf(a.alpha, xv[k].w, (g ? sigmoidf_acc(zv[k].w + gv[k].w) : 1.f) * yv[k].w);
        }
        if (i >= W) v[k] = zero;
        if (a.state_out && last && i < W) *reinterpret_cast<float4*>(a.state_out + (int64_t)st.ent_slot[e] * W + i) = xv[k];
        part += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    const float mean = block_sum(part, red) / (float)W;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        if ((threadIdx.x + k * nt) * 4 < W) {
            const float d0 = v[k].x - mean, d1 = v[k].y - mean, d2 = v[k].z - mean, d3 = v[k].w - mean;
            sq = fmaf(d0, d0, sq), sq = fmaf(d1, d1, sq), sq = fmaf(d2, d2, sq), sq = fmaf(d3, d3, sq);
        }
    }
    const float rinv = 1.0f / sqrtf(block_sum(sq, red) / (float)W + a.eps);
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int i = (threadIdx.x + k * nt) * 4;
        if (i >= W) continue;
        const float4 w4 = PRE ? wv[k] : ld4(a.w + i);
        const float4 b4 = PRE ? bv[k] : (a.b ? ld4(a.b + i) : zero);
        float4 n;
        n.x = fmaf((v[k].x - mean) * rinv, w4.x, b4.x), n.y = fmaf((v[k].y - mean) * rinv, w4.y, b4.y);
        n.z = fmaf((v[k].z - mean) * rinv, w4.z, b4.z), n.w = fmaf((v[k].w - mean) * rinv, w4.w, b4.w);
        if (a.x_out) *reinterpret_cast<float4*>(a.x_out + t * W + i) = n;
        if (a.a_out) store_act4(a.a_out, a.out_dtype, (int64_t)r * W + i, n);
        if (a.next_mu) {
            const float4 m4 = PRE ? mu[k] : ld4(a.next_mu + i);
            const float4 p4 = PRE ? pv[k] : (prev ? ld4(prev + i) : zero);
            store_act4(a.a_shift_out, a.out_dtype, (int64_t)r * W + i,
                       make_float4(fmaf(p4.x - n.x, m4.x, n.x), fmaf(p4.y - n.y, m4.y, n.y), fmaf(p4.z - n.z, m4.z, n.z), fmaf(p4.w - n.w, m4.w, n.w)));
        }
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
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (W <= 8192 && W % 4 == 0 && ldz % 4 == 0 && al(x) && al(y) && al(zg) && al(gate_b) && al(w) && al(b) && al(x_out) && al(a_out) && al(state_out) && al(next_mu) &&
        al(next_state) && al(a_shift_out)) {   // the row fits in registers, 16-byte accesses
        const int q = W / 4;
        const int nt = q <= 64 ? 64 : (q <= 128 ? 128 : (q <= 512 ? 256 : 512));
        const int ept = (q + nt - 1) / nt;
        const bool pre = R <= 64;
        cudaStream_t cs = (cudaStream_t)stream;
        const b200seq_step sd = st ? *st : none;
#define POST_LAUNCH(E_)                                                            \
    do {                                                                           \
        if (pre) post_norm_reg_kernel<E_, true><<<R, nt, 0, cs>>>(a, sd);          \
        else post_norm_reg_kernel<E_, false><<<R, nt, 0, cs>>>(a, sd);             \
    } while (0)
        if (ept <= 1) POST_LAUNCH(1);
        else if (ept <= 2) POST_LAUNCH(2);
        else POST_LAUNCH(4);
#undef POST_LAUNCH
        SEQ_LAUNCH_CHECK("post_norm");
        return 0;
    }
    post_norm_kernel<<<R, 512, smem, (cudaStream_t)stream>>>(a, st ? *st : none);
    SEQ_LAUNCH_CHECK("post_norm");
    return 0;
}
