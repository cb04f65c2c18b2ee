// seq_branch.cu -- operators of layers whose norm sits on the sublayer's OUTPUT and whose mixer may be two branches side by side
// (an attention beside an element-wise gated recurrence): embedding with a hashed bigram table, the branch sum + output norm +
// residual sum in one kernel, the PolyNorm activation, soft caps, the second half of differential attention, and the two gated
// linear recurrences (minGRU, real-gated LRU).  All arithmetic in f32.
#include "seq_common.cuh"

namespace b200seq {

// ---- embedding + hashed bigram ------------------------------------------------------------------------------------------------------------
// grid (T)
__global__ void embed_bigram_kernel(const __nv_bfloat16* __restrict__ table, const __nv_bfloat16* __restrict__ bigram, const int32_t* __restrict__ ids,
                                    const int32_t* __restrict__ ent_prev, const b200seq_step st, float scale, int buckets, int mul_prev, int mul_cur, int W,
                                    float* __restrict__ x, void* __restrict__ a, int a_dtype) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const __nv_bfloat16* row = table + (int64_t)id * W;
    const __nv_bfloat16* brow = nullptr;
    if (bigram) {
        const int e = st.tok_ent[t];
        int64_t r;
        if (st.tok_pos[t] == 0) {
            r = buckets;
        } else {
            const int prev = (t == st.ent_start[e]) ? ent_prev[e] : ids[t - 1];
            r = ((int64_t)prev * mul_prev + (int64_t)id * mul_cur) % buckets;
            if (r < 0) r += buckets;
        }
        brow = bigram + r * W;
    }
    if ((W & 7) == 0) {   // rows start on 16-byte boundaries: eight elements per thread and pass
        for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
            const uint4 rv = *reinterpret_cast<const uint4*>(row + i);
            const uint4 bv = brow ? *reinterpret_cast<const uint4*>(brow + i) : make_uint4(0u, 0u, 0u, 0u);
            const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w}, bu[4] = {bv.x, bv.y, bv.z, bv.w};
            float v[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[2 * j] = __uint_as_float(ru[j] << 16) * scale + __uint_as_float(bu[j] << 16);
                v[2 * j + 1] = __uint_as_float(ru[j] & 0xffff0000u) * scale + __uint_as_float(bu[j] & 0xffff0000u);
            }
            float4* xo = reinterpret_cast<float4*>(x + (int64_t)t * W + i);
            xo[0] = make_float4(v[0], v[1], v[2], v[3]), xo[1] = make_float4(v[4], v[5], v[6], v[7]);
            if (a && a_dtype == B200SEQ_F32) {
                float4* ao = reinterpret_cast<float4*>(reinterpret_cast<float*>(a) + (int64_t)t * W + i);
                ao[0] = xo[0], ao[1] = xo[1];
            } else if (a) {
                uint4 pk;
                uint32_t* pu = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                    pu[j] = *reinterpret_cast<const uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a) + (int64_t)t * W + i) = pk;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = __bfloat162float(row[i]) * scale;
        if (brow) v += __bfloat162float(brow[i]);
        x[(int64_t)t * W + i] = v;
        if (a) store_act(a, a_dtype, (int64_t)t * W + i, v);
    }
}

// ---- branch sum + output norm + residual ------------------------------------------------------------------------------------------------------
struct BranchArgs {
    const float *x, *y1, *bias1, *w_b1, *y2, *w_b2, *w, *fin_w;
    float s1, s2, eps;
    int W;
    const int32_t* rows;
    float* x_out;
    void* a_out;
    int out_dtype;
};

// one block per row; dynamic shared memory: W floats (the branch sum) + 40 of reduction scratch
__global__ void branch_norm_kernel(const BranchArgs a) {
    extern __shared__ float bsm[];
    float* v = bsm;
    float* red = bsm + a.W;
    const int r = blockIdx.x;
    const int64_t t = a.rows ? a.rows[r] : r;
    const int W = a.W;
    const float invW = 1.0f / (float)W;
    const float* y1 = a.y1 + t * W;
    const float* y2 = a.y2 ? a.y2 + t * W : nullptr;
    float ss1 = 0.f, ss2 = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float b1 = y1[i] + (a.bias1 ? a.bias1[i] : 0.f);
        v[i] = b1;
        ss1 = fmaf(b1, b1, ss1);
        if (y2) ss2 = fmaf(y2[i], y2[i], ss2);
    }
    float r1 = 1.f, r2 = 1.f;
    if (a.w_b1) r1 = 1.0f / sqrtf(block_sum(ss1, red) * invW + a.eps);
    if (y2 && a.w_b2) r2 = 1.0f / sqrtf(block_sum(ss2, red) * invW + a.eps);
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {   // every thread reads back only what it wrote
        float b1 = v[i] * r1;
        if (a.w_b1) b1 *= a.w_b1[i];
        float s = a.s1 * b1;
        if (y2) {
            float b2 = y2[i] * r2;
            if (a.w_b2) b2 *= a.w_b2[i];
            s = fmaf(a.s2, b2, s);
        }
        v[i] = s;
        ss = fmaf(s, s, ss);
    }
    const float rn = 1.0f / sqrtf(block_sum(ss, red) * invW + a.eps);
    const float* xr = a.x + t * W;
    float sf = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float xn = xr[i] + v[i] * rn * a.w[i];
        v[i] = xn;
        sf = fmaf(xn, xn, sf);
        if (a.x_out) a.x_out[t * W + i] = xn;
    }
    if (!a.a_out) return;
    float rf = 1.f;
    if (a.fin_w) rf = 1.0f / sqrtf(block_sum(sf, red) * invW + a.eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) store_act(a.a_out, a.out_dtype, (int64_t)r * W + i, a.fin_w ? v[i] * rf * a.fin_w[i] : v[i]);
}

// ---- PolyNorm ------------------------------------------------------------------------------------------------------------------------------
// grid (T): three sums of even powers, then the polynomial of the three normalised powers
__global__ void polynorm_kernel(const float* __restrict__ z, int64_t ldz, int F, const float* __restrict__ coef, float eps, void* __restrict__ out, int out_dtype,
                                int64_t ldo) {
    __shared__ float red[40];
    const int64_t t = blockIdx.x;
    const float* zr = z + t * ldz;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float u = zr[i], u2 = u * u, u3 = u2 * u;
        s2 = fmaf(u, u, s2), s4 = fmaf(u2, u2, s4), s6 = fmaf(u3, u3, s6);
    }
    const float invF = 1.0f / (float)F;
    const float n1 = 1.0f / sqrtf(block_sum(s2, red) * invF + eps);
    const float n2 = 1.0f / sqrtf(block_sum(s4, red) * invF + eps);
    const float n3 = 1.0f / sqrtf(block_sum(s6, red) * invF + eps);
    const float c0 = coef[0] * n1, c1 = coef[1] * n2, c2 = coef[2] * n3, c3 = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float u = zr[i], u2 = u * u;
        store_act(out, out_dtype, t * ldo + i, fmaf(c0, u, fmaf(c1, u2, fmaf(c2, u2 * u, c3))));
    }
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t n, float cap) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// ---- differential attention: o = a1 - lambda a2, unit RMS per head, times out_scale ----------------------------------------------------------
// grid (T, H), one warp per (token, head)
__global__ void diff_combine_kernel(const float* __restrict__ a, int H, int G, int V, float lambda, float out_scale, float eps, void* __restrict__ out, int out_dtype) {
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y, lane = threadIdx.x;
    const int R = H / G, g = h / R, r = h - g * R;
    const float* a1 = a + (t * 2 * H + (int64_t)(2 * g) * R + r) * V;
    const float* a2 = a1 + (int64_t)R * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) {
        const float o = fmaf(-lambda, a2[i], a1[i]);
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)V + eps);
    for (int i = lane; i < V; i += 32) store_act(out, out_dtype, (t * H + h) * V + i, fmaf(-lambda, a2[i], a1[i]) * f);
}

// ---- gated linear recurrences ------------------------------------------------------------------------------------------------------------------
// S_t = a_t S_(t-1) + b_t per channel, out_t = S_t * o_t; (a_t, b_t, o_t) depend on the token's own inputs only.
// Two forms with the same result up to rounding:
//   steps of single tokens: one thread per (entry, channel) (neighbouring threads = neighbouring channels: coalesced);
//   steps with portions:    a block = 8 channels x 16 warps x 4 lanes per channel; every lane takes 16 consecutive tokens of every group of 1024,
//                           keeps their (a, b, o) in registers and reduces them to (A, B) = (product of a, local end state from 0); the lanes'
//                           (A, B) are chained by shuffles inside a warp and through shared memory between warps to every lane's entry state,
//                           and the tokens are replayed from the registers.
//                           Every input is read once and every output written once.
struct GruArgs {
    const float* proj;
    int64_t ldp;
    int z_col, x_col, g_col;
    const float* bias;
    float* state;
    int C;
    void* out;
    int out_dtype;
};
struct GruCoef {
    float bz, bx;
    __device__ __forceinline__ void init(const GruArgs& a, int c) {
        bz = a.bias ? a.bias[a.z_col + c] : 0.f, bx = a.bias ? a.bias[a.x_col + c] : 0.f;
    }
    static constexpr int NIN = 3;
    // raw inputs of (t, c) first, arithmetic later: the chunked form issues the loads of all its tokens before it needs any of them
    __device__ __forceinline__ void load(const GruArgs& a, int t, int c, float* r) const {
        const float* p = a.proj + (int64_t)t * a.ldp;
        r[0] = p[a.z_col + c], r[1] = p[a.x_col + c], r[2] = p[a.g_col + c];
    }
    __device__ __forceinline__ void coef(const float* r, float& av, float& bv, float& ov) const {
        const float z = sigmoidf_acc(r[0] + bz);
        const float u = r[1] + bx;
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_acc(u);
        av = 1.f - z, bv = z * cand, ov = siluf_acc(r[2]);
    }
};

struct LruArgs {
    const float* u;
    int64_t ldu;
    const float* gates;
    int64_t ldg;
    const float *gate_bias, *sp_lam;
    float decay_c;
    const float* proj;
    int64_t ldp;
    int y_col;
    const float* bias;
    float* state;
    int C, bw;
    void* out;
    int out_dtype;
};
struct LruCoef {
    int rc, ic;
    float br, bi, by, k;
    __device__ __forceinline__ void init(const LruArgs& a, int c) {
        const int blk = c / a.bw, cc = c - blk * a.bw;
        rc = blk * 2 * a.bw + cc, ic = rc + a.bw;
        br = a.gate_bias ? a.gate_bias[rc] : 0.f, bi = a.gate_bias ? a.gate_bias[ic] : 0.f;
        by = a.bias ? a.bias[a.y_col + c] : 0.f;
        k = -a.decay_c * a.sp_lam[c];
    }
    static constexpr int NIN = 4;
    __device__ __forceinline__ void load(const LruArgs& a, int t, int c, float* r) const {
        const float* gp = a.gates + (int64_t)t * a.ldg;
        r[0] = gp[rc], r[1] = gp[ic], r[2] = a.u[(int64_t)t * a.ldu + c], r[3] = a.proj[(int64_t)t * a.ldp + a.y_col + c];
    }
    __device__ __forceinline__ void coef(const float* r, float& av, float& bv, float& ov) const {
        const float rg = sigmoidf_acc(r[0] + br), ig = sigmoidf_acc(r[1] + bi);
        const float la = k * rg;
        av = expf(la);
        bv = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * ig * r[2];   // sqrt(1 - a^2) without cancellation near a = 1
        ov = gelu_tanhf_acc(r[3] + by);
    }
};

template <typename Args, typename Coef>
__global__ void scan_step_kernel(const Args a, const b200seq_step st) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int e = blockIdx.y;
    if (c >= a.C) return;
    const int t0 = st.ent_start[e], t1 = st.ent_start[e + 1];
    if (t1 <= t0) return;
    float* sp = a.state + (int64_t)st.ent_slot[e] * a.C + c;
    float S = st.ent_pos0[e] == 0 ? 0.f : *sp;
    Coef k;
    k.init(a, c);
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float r[Coef::NIN], av, bv, ov;
        k.load(a, t, c, r);
        k.coef(r, av, bv, ov);
        S = fmaf(av, S, bv);
        store_act(a.out, a.out_dtype, (int64_t)t * a.C + c, S * ov);
    }
    *sp = S;
}

constexpr int SC_L = 16, SC_NW = 16, SC_CH = 8, SC_SUB = 32 / SC_CH;   // tokens per lane, warps, channels per block, lanes per channel in a warp
template <typename Args, typename Coef>
__global__ void __launch_bounds__(SC_NW * 32, 1) scan_chunk_kernel(const Args a, const b200seq_step st) {
    __shared__ float sA[SC_NW][SC_CH], sB[SC_NW][SC_CH];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int ch = lane & (SC_CH - 1), sub = lane / SC_CH;
    const int c = blockIdx.x * SC_CH + ch;
    const int e = blockIdx.y;
    const bool valid = c < a.C;
    const int cc = valid ? c : a.C - 1;
    const int t0 = st.ent_start[e], t1 = st.ent_start[e + 1];
    if (t1 <= t0) return;
    float* sp = a.state + (int64_t)st.ent_slot[e] * a.C + cc;
    float S = st.ent_pos0[e] == 0 ? 0.f : *sp;
    Coef k;
    k.init(a, cc);
    for (int g0 = t0; g0 < t1; g0 += SC_NW * SC_SUB * SC_L) {
        const int base = g0 + (wid * SC_SUB + sub) * SC_L;
        float raw[SC_L][Coef::NIN], av[SC_L], bv[SC_L], ov[SC_L];
#pragma unroll
        for (int i = 0; i < SC_L; ++i) {   // all loads of the lane's tokens are in flight before the first is used
#pragma unroll
            for (int j = 0; j < Coef::NIN; ++j) raw[i][j] = 0.f;
            if (base + i < t1) k.load(a, base + i, cc, raw[i]);
        }
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int i = 0; i < SC_L; ++i) {
            av[i] = 1.f, bv[i] = 0.f, ov[i] = 0.f;
            if (base + i < t1) k.coef(raw[i], av[i], bv[i], ov[i]);
            B = fmaf(av[i], B, bv[i]);
            A *= av[i];
        }
        // the lanes of one channel inside the warp, in token order; then the warps through shared memory
        float As[SC_SUB], Bs[SC_SUB], WA = 1.f, WB = 0.f;
#pragma unroll
        for (int j = 0; j < SC_SUB; ++j) {
            As[j] = __shfl_sync(0xffffffffu, A, ch + SC_CH * j), Bs[j] = __shfl_sync(0xffffffffu, B, ch + SC_CH * j);
            WB = fmaf(As[j], WB, Bs[j]);
            WA *= As[j];
        }
        if (sub == 0) sA[wid][ch] = WA, sB[wid][ch] = WB;
        __syncthreads();
        float s = S;
        for (int w = 0; w < wid; ++w) s = fmaf(sA[w][ch], s, sB[w][ch]);
        float send = s;
        for (int w = wid; w < SC_NW; ++w) send = fmaf(sA[w][ch], send, sB[w][ch]);
#pragma unroll
        for (int j = 0; j < SC_SUB; ++j)
            if (j < sub) s = fmaf(As[j], s, Bs[j]);
#pragma unroll
        for (int i = 0; i < SC_L; ++i) {
            s = fmaf(av[i], s, bv[i]);
            if (base + i < t1 && valid) store_act(a.out, a.out_dtype, (int64_t)(base + i) * a.C + c, s * ov[i]);
        }
        S = send;
        __syncthreads();   // sA / sB are rewritten by the next group
    }
    if (wid == 0 && sub == 0 && valid) *sp = S;
}

template <typename Args, typename Coef>
static int launch_scan(const Args& a, const b200seq_step* st, cudaStream_t cs) {
    if (st->T == st->B) {   // one token per entry
        const int nt = a.C >= 4096 ? 128 : (a.C >= 1024 ? 64 : 32);
        scan_step_kernel<Args, Coef><<<dim3((a.C + nt - 1) / nt, st->B), nt, 0, cs>>>(a, *st);
    } else {
        scan_chunk_kernel<Args, Coef><<<dim3((a.C + SC_CH - 1) / SC_CH, st->B), SC_NW * 32, 0, cs>>>(a, *st);
    }
    return 0;
}

}  // namespace b200seq

using namespace b200seq;

static bool act_dtype_ok(int d) { return d == B200SEQ_F32 || d == B200SEQ_BF16; }

extern "C" {

int b200seq_embed_bigram(const void* table, const void* bigram, const int32_t* ids, const int32_t* ent_prev, const b200seq_step* st, float scale, int buckets,
                         int mul_prev, int mul_cur, int W, float* x, void* a, int a_dtype, void* stream) {
    if (!table || !ids || !st || !x || W < 1 || (bigram && (!ent_prev || buckets < 1)) || (a && !act_dtype_ok(a_dtype)))
        return fail(B200SEQ_ERR_INVALID_ARG, "embed_bigram: bad arguments");
    if (st->T == 0) return 0;
    embed_bigram_kernel<<<st->T, W >= 2048 ? 256 : 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, ids, ent_prev, *st, scale,
                                                                                   buckets, mul_prev, mul_cur, W, x, a, a_dtype);
    SEQ_LAUNCH_CHECK("embed_bigram");
    return 0;
}

int b200seq_branch_norm(const float* x, const float* y1, const float* bias1, const float* w_b1, float s1, const float* y2, const float* w_b2, float s2, const float* w,
                        float eps, int W, const int32_t* rows, int R, float* x_out, void* a_out, int out_dtype, const float* fin_w, void* stream) {
    if (!x || !y1 || !w || W < 1 || R < 0 || (a_out && !act_dtype_ok(out_dtype)) || (w_b2 && !y2)) return fail(B200SEQ_ERR_INVALID_ARG, "branch_norm: bad arguments");
    if (R == 0) return 0;
    const size_t smem = (size_t)(W + 40) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "branch_norm: width too large");
    static size_t set_ = 0;
    if (smem > 48 * 1024 && smem > set_) {
        cudaError_t e = cudaFuncSetAttribute(branch_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "branch_norm attribute");
        set_ = smem;
    }
    const BranchArgs a{x, y1, bias1, w_b1, y2, w_b2, w, fin_w, s1, s2, eps, W, rows, x_out, a_out, out_dtype};
    branch_norm_kernel<<<R, W >= 2048 ? 512 : (W >= 512 ? 256 : 128), smem, (cudaStream_t)stream>>>(a);
    SEQ_LAUNCH_CHECK("branch_norm");
    return 0;
}

int b200seq_polynorm(const float* z, int64_t ldz, int T, int F, const float* coef, float eps, void* out, int out_dtype, int64_t ldo, void* stream) {
    if (!z || !coef || !out || T < 0 || F < 1 || ldz < F || ldo < F || !act_dtype_ok(out_dtype)) return fail(B200SEQ_ERR_INVALID_ARG, "polynorm: bad arguments");
    if (T == 0) return 0;
    polynorm_kernel<<<T, F >= 2048 ? 512 : (F >= 512 ? 256 : 128), 0, (cudaStream_t)stream>>>(z, ldz, F, coef, eps, out, out_dtype, ldo);
    SEQ_LAUNCH_CHECK("polynorm");
    return 0;
}

int b200seq_softcap(float* x, int64_t n, float cap, void* stream) {
    if (!x || n < 0 || !(cap > 0.f)) return fail(B200SEQ_ERR_INVALID_ARG, "softcap: bad arguments");
    if (n == 0) return 0;
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, cap);
    SEQ_LAUNCH_CHECK("softcap");
    return 0;
}

int b200seq_diff_combine(const float* a, int T, int H, int G, int V, float lambda, float out_scale, float eps, void* out, int out_dtype, void* stream) {
    if (!a || !out || T < 0 || H < 1 || G < 1 || H % G || V < 1 || H > 65535 || !act_dtype_ok(out_dtype)) return fail(B200SEQ_ERR_INVALID_ARG, "diff_combine: bad arguments");
    if (T == 0) return 0;
    diff_combine_kernel<<<dim3(T, H), 32, 0, (cudaStream_t)stream>>>(a, H, G, V, lambda, out_scale, eps, out, out_dtype);
    SEQ_LAUNCH_CHECK("diff_combine");
    return 0;
}

int b200seq_min_gru(const float* proj, int64_t ldp, int z_col, int x_col, int g_col, const float* bias, float* state, const b200seq_step* st, int C, void* out,
                    int out_dtype, void* stream) {
    if (!proj || !state || !st || !out || C < 1 || z_col < 0 || x_col < 0 || g_col < 0 || !act_dtype_ok(out_dtype)) return fail(B200SEQ_ERR_INVALID_ARG, "min_gru: bad arguments");
    if (st->T == 0 || st->B == 0) return 0;
    if (st->B > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "min_gru: too many entries");
    const GruArgs a{proj, ldp, z_col, x_col, g_col, bias, state, C, out, out_dtype};
    launch_scan<GruArgs, GruCoef>(a, st, (cudaStream_t)stream);
    SEQ_LAUNCH_CHECK("min_gru");
    return 0;
}

int b200seq_rg_lru(const float* u, int64_t ldu, const float* gates, int64_t ldg, const float* gate_bias, const float* sp_lam, float decay_c, const float* proj,
                   int64_t ldp, int y_col, const float* bias, float* state, const b200seq_step* st, int C, int blocks, void* out, int out_dtype, void* stream) {
    if (!u || !gates || !sp_lam || !proj || !state || !st || !out || C < 1 || blocks < 1 || C % blocks || y_col < 0 || !act_dtype_ok(out_dtype))
        return fail(B200SEQ_ERR_INVALID_ARG, "rg_lru: bad arguments");
    if (st->T == 0 || st->B == 0) return 0;
    if (st->B > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "rg_lru: too many entries");
    const LruArgs a{u, ldu, gates, ldg, gate_bias, sp_lam, decay_c, proj, ldp, y_col, bias, state, C, C / blocks, out, out_dtype};
    launch_scan<LruArgs, LruCoef>(a, st, (cudaStream_t)stream);
    SEQ_LAUNCH_CHECK("rg_lru");
    return 0;
}

}  // extern "C"
