// seq_glue.cu -- element-wise / per-row operators of layer-list models: embedding into residual streams, stream mixing fused
// with the grouped RMS norm, short causal convolutions with carried state, gated activations, arg-max.  All arithmetic in f32.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "seq_common.cuh"

namespace b200seq {

static std::atomic<int64_t> g_launches{0};
static thread_local char g_err[512] = "";
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_status(cudaError_t e, const char* what) { return fail(B200SEQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e)); }

__device__ int g_error_flags = 0;
int* error_flag_dev() {
    int* p = nullptr;
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_error_flags);
    return p;
}

constexpr int MAX_STREAMS = 8;
constexpr int MAX_TAPS = 8;

__global__ void embed_streams_kernel(const __nv_bfloat16* __restrict__ table, const int32_t* __restrict__ ids, float scale, int S, int W,
                                     float* __restrict__ X) {
    const int t = blockIdx.x;
    const __nv_bfloat16* row = table + (int64_t)ids[t] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = __bfloat162float(row[i]) * scale;
        for (int s = 0; s < S; ++s) X[((int64_t)t * S + s) * W + i] = v;
    }
}

// one block per row; dynamic shared memory: W floats (the collapsed vector) + 40 floats of reduction scratch.
// S is a compile-time constant so that the mixing weights stay in registers; VW = 4: 16-byte accesses (W % 4 == 0).
// With conv_w (steps in which every entry brings ONE token, rows == null): the carried convolution of the sublayer's input follows in
// the same kernel, out = h + conv(h) with the taps-1 earlier h of the sequence read from and shifted in conv_state[slot][taps-1][W].
struct HcConv {
    const float* w;      // [W, taps] or null
    float* state;
    const int32_t *ent_slot, *ent_pos0;
    int taps;
};
template <int S, int VW>
__global__ void hc_norm_kernel(float* __restrict__ X, const float* __restrict__ y, const float* __restrict__ post, const float* __restrict__ in_w,
                               const float* __restrict__ norm_w, int W, int groups, float eps, const int32_t* __restrict__ rows,
                               void* __restrict__ out, int out_dtype, const HcConv cv) {
    extern __shared__ __align__(16) float sm[];
    float* u = sm;
    float* red = sm + W;
    float* rs = red + 40;        // [groups]: 1 / rms of every group (convolution variant)
    const int r = blockIdx.x;
    const int64_t t = rows ? rows[r] : r;
    float mixr[S * S], outr[S], inr[S];
    if (y) {
#pragma unroll
        for (int s = 0; s < S; ++s) outr[s] = post[s];
#pragma unroll
        for (int s = 0; s < S * S; ++s) mixr[s] = post[S + s];
    }
    if (norm_w) {
#pragma unroll
        for (int s = 0; s < S; ++s) inr[s] = in_w[s];
    }
    float* Xt = X + t * S * W;
    for (int i = threadIdx.x * VW; i < W; i += blockDim.x * VW) {
        float xs[S][VW];
#pragma unroll
        for (int s = 0; s < S; ++s) {
            if (VW == 4) {
                const float4 v = *reinterpret_cast<const float4*>(Xt + (int64_t)s * W + i);
                xs[s][0] = v.x, xs[s][1 % VW] = v.y, xs[s][2 % VW] = v.z, xs[s][3 % VW] = v.w;
            } else {
                xs[s][0] = Xt[(int64_t)s * W + i];
            }
        }
        if (y) {
            float yv[VW];
            if (VW == 4) {
                const float4 v = *reinterpret_cast<const float4*>(y + t * W + i);
                yv[0] = v.x, yv[1 % VW] = v.y, yv[2 % VW] = v.z, yv[3 % VW] = v.w;
            } else {
                yv[0] = y[t * W + i];
            }
            float xn[S][VW];
#pragma unroll
            for (int j = 0; j < S; ++j)
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int s2 = 0; s2 < S; ++s2) a = fmaf(mixr[s2 * S + j], xs[s2][e], a);
                    xn[j][e] = fmaf(outr[j], yv[e], a);
                }
#pragma unroll
            for (int j = 0; j < S; ++j) {
#pragma unroll
                for (int e = 0; e < VW; ++e) xs[j][e] = xn[j][e];
                if (VW == 4) *reinterpret_cast<float4*>(Xt + (int64_t)j * W + i) = make_float4(xn[j][0], xn[j][1 % VW], xn[j][2 % VW], xn[j][3 % VW]);
                else Xt[(int64_t)j * W + i] = xn[j][0];
            }
        }
        if (norm_w) {
#pragma unroll
            for (int e = 0; e < VW; ++e) {
                float a = 0.f;
#pragma unroll
                for (int s2 = 0; s2 < S; ++s2) a = fmaf(inr[s2], xs[s2][e], a);
                u[i + e] = a;
            }
        }
    }
    if (!norm_w) return;
    __syncthreads();
    const int Wg = W / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < Wg; i += blockDim.x) {
            const float v = u[g * Wg + i];
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, red);
        const float rinv = 1.0f / sqrtf(ss / (float)Wg + eps);
        if (!cv.w) {
            for (int i = threadIdx.x; i < Wg; i += blockDim.x) store_act(out, out_dtype, (int64_t)r * W + g * Wg + i, u[g * Wg + i] * rinv * norm_w[g * Wg + i]);
        } else if (threadIdx.x == 0) {
            rs[g] = rinv;
        }
    }
    if (!cv.w) return;
    __syncthreads();
    // convolution.  All old state rows and taps of a batch of the thread's channels are fetched before any of them is stored: the
    // stores would otherwise order every later load behind them (one memory round trip per channel).
    constexpr int HC_U = 8, HC_T = 4;
    const int hist = cv.taps - 1;
    const bool fresh = cv.ent_pos0[r] == 0;
    float* sp = cv.state + (int64_t)cv.ent_slot[r] * hist * W;
    if (cv.taps <= HC_T) {
        for (int base = 0; base < W; base += HC_U * blockDim.x) {
            float cold[HC_U][HC_T - 1], cw[HC_U][HC_T];
#pragma unroll
            for (int k = 0; k < HC_U; ++k) {
                const int c = base + threadIdx.x + k * blockDim.x;
#pragma unroll
                for (int j = 0; j < HC_T; ++j) cw[k][j] = (c < W && j < cv.taps) ? cv.w[(int64_t)c * cv.taps + j] : 0.f;
#pragma unroll
                for (int j = 0; j < HC_T - 1; ++j) cold[k][j] = (c < W && j < hist && !fresh) ? sp[(int64_t)j * W + c] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < HC_U; ++k) {
                const int c = base + threadIdx.x + k * blockDim.x;
                if (c < W) {
                    const float hv = u[c] * rs[c / Wg] * norm_w[c];
                    float acc = 0.f;
#pragma unroll
                    for (int j = 0; j < HC_T; ++j) acc = fmaf(cw[k][j], j == hist ? hv : (j < hist ? cold[k][j < HC_T - 1 ? j : 0] : 0.f), acc);
#pragma unroll
                    for (int j = 0; j < HC_T - 1; ++j)       // row j receives the old row j + 1, the last row the new h
                        if (j < hist) sp[(int64_t)j * W + c] = j == hist - 1 ? hv : cold[k][j + 1 < HC_T - 1 ? j + 1 : 0];
                    store_act(out, out_dtype, (int64_t)r * W + c, hv + acc);
                }
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float hv = u[c] * rs[c / Wg] * norm_w[c];
        const float* wc = cv.w + (int64_t)c * cv.taps;
        float acc = wc[hist] * hv;
        float next = hv;                           // what row j receives: the old row j + 1 (the new h for the last row)
        for (int j = hist - 1; j >= 0; --j) {
            const float old = fresh ? 0.f : sp[(int64_t)j * W + c];
            acc = fmaf(wc[j], old, acc);
            sp[(int64_t)j * W + c] = next;
            next = old;
        }
        store_act(out, out_dtype, (int64_t)r * W + c, hv + acc);
    }
}

// thread = VW neighbouring channels (VW = 4: 16-byte accesses), blockIdx.y = a tile of CONV_TILE consecutive token rows.  The first
// taps-1 tokens of an entry read the carried state; they and the state's rewrite belong to the thread that meets the entry's first
// token, so no other thread touches that state.
constexpr int CONV_TILE = 16;
template <int VW>
__global__ void causal_conv_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ in_bias, const float* __restrict__ w,
                                   const float* __restrict__ bias, float* __restrict__ state, b200seq_step st, int C, int taps, int mode,
                                   void* __restrict__ out, int out_dtype, int64_t ldo, void* __restrict__ out2, int out2_dtype, int64_t ldo2) {
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VW;
    if (c0 >= C) return;
    float wr[VW][MAX_TAPS], b[VW], ib[VW];   // ib: bias of the input (the convolution sees x + ib; the carried state holds biased inputs)
#pragma unroll
    for (int e = 0; e < VW; ++e) {
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) wr[e][j] = j < taps ? w[(int64_t)(c0 + e) * taps + j] : 0.f;
        b[e] = bias ? bias[c0 + e] : 0.f;
        ib[e] = in_bias ? in_bias[c0 + e] : 0.f;
    }
    const int hist = taps - 1;
    auto finish = [&](float acc, float bb, float xin) {
        float v = acc + bb;
        if (mode & B200SEQ_CONV_SILU) v = siluf_acc(v);
        if (mode & B200SEQ_CONV_RESIDUAL) v = xin + v;
        return v;
    };
    const int t0 = blockIdx.y * CONV_TILE, t1 = min(t0 + CONV_TILE, st.T);
    for (int t = t0; t < t1; ++t) {
        const int en = st.tok_ent[t];
        const int s0 = st.ent_start[en];
        const int i = t - s0;
        if (i < hist) {
            if (i != 0) continue;
            const int len = st.ent_start[en + 1] - s0;
            const bool fresh = st.ent_pos0[en] == 0;
            const int n_own = min(hist, len);
#pragma unroll
            for (int e = 0; e < VW; ++e) {
                const int c = c0 + e;
                const int64_t sbase = (int64_t)st.ent_slot[en] * hist * C + c;
                float old[MAX_TAPS];
#pragma unroll
                for (int j = 0; j < MAX_TAPS; ++j) old[j] = (j < hist && !fresh) ? state[sbase + (int64_t)j * C] : 0.f;
                // input at entry-relative index idx (negative = carried)
                auto src = [&](int idx) -> float {
                    if (idx >= 0) return x[(int64_t)(s0 + idx) * ldx + c] + ib[e];
                    float v = 0.f;
#pragma unroll
                    for (int j = 0; j < MAX_TAPS; ++j)
                        if (j == hist + idx) v = old[j];
                    return v;
                };
                for (int ii = 0; ii < n_own; ++ii) {
                    float acc = 0.f;
#pragma unroll
                    for (int j = 0; j < MAX_TAPS; ++j)
                        if (j < taps) acc = fmaf(wr[e][j], src(ii - hist + j), acc);
                    const float r = finish(acc, b[e], x[(int64_t)(s0 + ii) * ldx + c] + ib[e]);
                    store_act(out, out_dtype, (int64_t)(s0 + ii) * ldo + c, r);
                    if (out2) store_act(out2, out2_dtype, (int64_t)(s0 + ii) * ldo2 + c, r);
                }
                float nv[MAX_TAPS];
#pragma unroll
                for (int j = 0; j < MAX_TAPS; ++j) nv[j] = j < hist ? src(len - hist + j) : 0.f;
#pragma unroll
                for (int j = 0; j < MAX_TAPS; ++j)
                    if (j < hist) state[sbase + (int64_t)j * C] = nv[j];
            }
            continue;
        }
        float acc[VW], cur[VW];
#pragma unroll
        for (int e = 0; e < VW; ++e) acc[e] = 0.f, cur[e] = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            if (j < taps) {
                const float* xp = x + (int64_t)(t - hist + j) * ldx + c0;
                if (VW == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(xp);
                    cur[0] = v.x + ib[0], cur[1 % VW] = v.y + ib[1 % VW], cur[2 % VW] = v.z + ib[2 % VW], cur[3 % VW] = v.w + ib[3 % VW];
                } else {
                    cur[0] = xp[0] + ib[0];
                }
#pragma unroll
                for (int e = 0; e < VW; ++e) acc[e] = fmaf(wr[e][j], cur[e], acc[e]);
            }
        }
        // cur holds the row's own input (the last tap)
        float v[VW];
#pragma unroll
        for (int e = 0; e < VW; ++e) v[e] = finish(acc[e], b[e], cur[e]);
        if (VW == 4) {
            if (out_dtype == B200SEQ_F32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (int64_t)t * ldo + c0) = make_float4(v[0], v[1 % VW], v[2 % VW], v[3 % VW]);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1 % VW]), hi = __floats2bfloat162_rn(v[2 % VW], v[3 % VW]);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo), pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + (int64_t)t * ldo + c0) = pk;
            }
        } else {
            store_act(out, out_dtype, (int64_t)t * ldo + c0, v[0]);
        }
        if (out2) {
#pragma unroll
            for (int e = 0; e < VW; ++e) store_act(out2, out2_dtype, (int64_t)t * ldo2 + c0 + e, v[e]);
        }
    }
}

// grid (T, groups): one block per norm group of a row
__global__ void group_rmsnorm_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ w, int D, int groups, float eps,
                                     void* __restrict__ out, int out_dtype) {
    __shared__ float red[40];
    const int64_t t = blockIdx.x;
    const int g = blockIdx.y;
    const int Dg = D / groups;
    const float* xr = x + t * ldx + (int64_t)g * Dg;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Dg; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)Dg + eps);
    for (int i = threadIdx.x; i < Dg; i += blockDim.x) {
        const int k = g * Dg + i;
        store_act(out, out_dtype, t * D + k, xr[i] * rinv * (w ? w[k] : 1.f));
    }
}

// F outputs per row; gated kinds read the pair (gate f, up f) from columns (2f, 2f + 1) (interleaved) or (f, F + f)
__global__ void gated_act_kernel(const float* __restrict__ gu, int64_t ldg, int T, int F, const ActParams act, int interleaved, void* __restrict__ out,
                                 int out_dtype, int64_t ldo) {
    const int64_t n = (int64_t)T * F;
    const bool gated = act_is_gated(act.kind);
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / F;
        const int f = (int)(idx - t * F);
        float v;
        if (gated) v = act_gated(act, gu[t * ldg + (interleaved ? 2 * f : f)], gu[t * ldg + (interleaved ? 2 * f + 1 : F + f)]);
        else v = act_plain(act.kind, gu[t * ldg + f]);
        store_act(out, out_dtype, t * ldo + f, v);
    }
}

__global__ void argmax_kernel(const float* __restrict__ logits, int V, int32_t* __restrict__ ids) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (int64_t)blockIdx.x * V;
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < arg)) best = v, arg = i;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ov > best || (ov == best && oi < arg)) best = ov, arg = oi;
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) bv[wid] = best, bi[wid] = arg;
    __syncthreads();
    if (wid == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        arg = lane < nw ? bi[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oi < arg)) best = ov, arg = oi;
        }
        if (lane == 0) ids[blockIdx.x] = arg == 0x7fffffff ? 0 : arg;
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" {

const char* b200seq_last_error(void) { return g_err; }
int b200seq_version(void) { return 1; }
int64_t b200seq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200seq_error_flags(int* flags_out) {
    if (!flags_out) return fail(B200SEQ_ERR_INVALID_ARG, "flags_out is null");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_status(e, "synchronize");
    int zero = 0;
    e = cudaMemcpyFromSymbol(flags_out, g_error_flags, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "read error flags");
    e = cudaMemcpyToSymbol(g_error_flags, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "clear error flags");
    return 0;
}

int b200seq_embed_streams(const void* table, const int32_t* ids, float scale, int T, int S, int W, float* X, void* stream) {
    if (!table || !ids || !X || T < 0 || S < 1 || S > MAX_STREAMS || W < 1) return fail(B200SEQ_ERR_INVALID_ARG, "embed_streams: bad arguments");
    if (T == 0) return 0;
    embed_streams_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)table, ids, scale, S, W, X);
    SEQ_LAUNCH_CHECK("embed_streams");
    return 0;
}

static int hc_norm_launch(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                          const int32_t* rows, int R, void* out, int out_dtype, const HcConv cv, void* stream);

int b200seq_hc_norm(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                    const int32_t* rows, int R, void* out, int out_dtype, void* stream) {
    return hc_norm_launch(X, y, post, in_w, norm_w, S, W, groups, eps, rows, R, out, out_dtype, HcConv{nullptr, nullptr, nullptr, nullptr, 1}, stream);
}

int b200seq_hc_norm_conv(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                         const float* conv_w, float* conv_state, const b200seq_step* st, int taps, void* out, int out_dtype, void* stream) {
    if (!conv_w || !st || !norm_w || taps < 1 || taps > MAX_TAPS || (taps > 1 && !conv_state)) return fail(B200SEQ_ERR_INVALID_ARG, "hc_norm_conv: bad arguments");
    if (st->T != st->B) return fail(B200SEQ_ERR_INVALID_ARG, "hc_norm_conv: every entry of the step must bring exactly one token");
    return hc_norm_launch(X, y, post, in_w, norm_w, S, W, groups, eps, nullptr, st->T, out, out_dtype, HcConv{conv_w, conv_state, st->ent_slot, st->ent_pos0, taps}, stream);
}

static int hc_norm_launch(float* X, const float* y, const float* post, const float* in_w, const float* norm_w, int S, int W, int groups, float eps,
                          const int32_t* rows, int R, void* out, int out_dtype, const HcConv cv, void* stream) {
    if (!X || S < 1 || S > MAX_STREAMS || W < 1 || R < 0) return fail(B200SEQ_ERR_INVALID_ARG, "hc_norm: bad arguments");
    if ((y && !post) || (norm_w && (!in_w || !out || groups < 1 || W % groups))) return fail(B200SEQ_ERR_INVALID_ARG, "hc_norm: missing parameters or width not divisible by groups");
    if (R == 0) return 0;
    const size_t smem = ((size_t)W + 40 + (cv.w ? groups : 0)) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "hc_norm: width %d too large", W);
    const bool vec = W % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0 && (!y || (reinterpret_cast<uintptr_t>(y) & 15) == 0);
    const int nt_want = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
    cudaError_t e = cudaSuccess;
#define HC_LAUNCH(S_, VW_)                                                                                                                   \
    do {                                                                                                                                     \
        static int max_threads = 0;   /* what the instantiation's register use allows */                                                    \
        if (!max_threads) {                                                                                                                  \
            cudaFuncAttributes fa;                                                                                                           \
            e = cudaFuncGetAttributes(&fa, hc_norm_kernel<S_, VW_>);                                                                         \
            if (e == cudaSuccess) max_threads = fa.maxThreadsPerBlock;                                                                       \
        }                                                                                                                                    \
        int nt = nt_want;                                                                                                                    \
        while (e == cudaSuccess && nt > max_threads && nt > 32) nt >>= 1;                                                                    \
        if (e == cudaSuccess && smem > 48 * 1024)                                                                                            \
            e = cudaFuncSetAttribute(hc_norm_kernel<S_, VW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
        if (e == cudaSuccess)                                                                                                                \
            hc_norm_kernel<S_, VW_><<<R, nt, smem, (cudaStream_t)stream>>>(X, y, post, in_w, norm_w, W, groups, eps, rows, out, out_dtype, cv);  \
    } while (0)
#define HC_CASE(S_)                  \
    case S_:                         \
        if (vec) HC_LAUNCH(S_, 4);   \
        else HC_LAUNCH(S_, 1);       \
        break
    switch (S) {
        HC_CASE(1);
        HC_CASE(2);
        HC_CASE(3);
        HC_CASE(4);
        HC_CASE(5);
        HC_CASE(6);
        HC_CASE(7);
        HC_CASE(8);
    }
#undef HC_CASE
#undef HC_LAUNCH
    if (e != cudaSuccess) return cuda_status(e, "hc_norm attribute");
    SEQ_LAUNCH_CHECK("hc_norm");
    return 0;
}

int b200seq_causal_conv(const float* x, int64_t ldx, const float* w, const float* bias, float* state, const b200seq_step* st, int C, int taps, int mode,
                        void* out, int out_dtype, int64_t ldo, void* stream) {
    return b200seq_causal_conv_ex(x, ldx, nullptr, w, bias, state, st, C, taps, mode, out, out_dtype, ldo, nullptr, B200SEQ_F32, 0, stream);
}

int b200seq_causal_conv_ex(const float* x, int64_t ldx, const float* in_bias, const float* w, const float* bias, float* state, const b200seq_step* st, int C, int taps,
                           int mode, void* out, int out_dtype, int64_t ldo, void* out2, int out2_dtype, int64_t ldo2, void* stream) {
    if (!x || !w || !st || !out || C < 1 || taps < 1 || taps > MAX_TAPS || (taps > 1 && !state)) return fail(B200SEQ_ERR_INVALID_ARG, "causal_conv: bad arguments (1 <= taps <= %d)", MAX_TAPS);
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "causal_conv: output dtype");
    if (out2 && ((out2_dtype != B200SEQ_F32 && out2_dtype != B200SEQ_BF16) || ldo2 < C)) return fail(B200SEQ_ERR_INVALID_ARG, "causal_conv: second output");
    if (st->T == 0) return 0;
    const bool vec = C % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (vec) {
        dim3 grid((C / 4 + 127) / 128, (st->T + CONV_TILE - 1) / CONV_TILE);
        causal_conv_kernel<4><<<grid, 128, 0, (cudaStream_t)stream>>>(x, ldx, in_bias, w, bias, state, *st, C, taps, mode, out, out_dtype, ldo, out2, out2_dtype, ldo2);
    } else {
        dim3 grid((C + 127) / 128, (st->T + CONV_TILE - 1) / CONV_TILE);
        causal_conv_kernel<1><<<grid, 128, 0, (cudaStream_t)stream>>>(x, ldx, in_bias, w, bias, state, *st, C, taps, mode, out, out_dtype, ldo, out2, out2_dtype, ldo2);
    }
    SEQ_LAUNCH_CHECK("causal_conv");
    return 0;
}

int b200seq_group_rmsnorm(const float* x, int64_t ldx, const float* w, int T, int D, int groups, float eps, void* out, int out_dtype, void* stream) {
    if (!x || !out || T < 0 || D < 1 || groups < 1 || D % groups) return fail(B200SEQ_ERR_INVALID_ARG, "group_rmsnorm: bad arguments");
    if (T == 0) return 0;
    group_rmsnorm_kernel<<<dim3(T, groups), D / groups >= 512 ? 256 : 128, 0, (cudaStream_t)stream>>>(x, ldx, w, D, groups, eps, out, out_dtype);
    SEQ_LAUNCH_CHECK("group_rmsnorm");
    return 0;
}

int b200seq_gated_act(const float* gu, int64_t ldg, int T, int F, float limit, float alpha, float up_shift, int interleaved, void* out, int out_dtype,
                      void* stream) {
    if (!gu || !out || T < 0 || F < 1) return fail(B200SEQ_ERR_INVALID_ARG, "gated_act: bad arguments");
    if (T == 0) return 0;
    const int64_t n = (int64_t)T * F;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    gated_act_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(gu, ldg, T, F, ActParams{B200SEQ_ACT_SWISH_CLAMP, limit, alpha, up_shift}, interleaved, out, out_dtype, F);
    SEQ_LAUNCH_CHECK("gated_act");
    return 0;
}

int b200seq_act(const float* z, int64_t ldz, int T, int N, int act, float limit, float alpha, float shift, void* out, int out_dtype, int64_t ldo, void* stream) {
    if (!z || !out || T < 0 || N < 1 || !act_kind_known(act) || (act_kind_gated(act) && (N & 1))) return fail(B200SEQ_ERR_INVALID_ARG, "act: bad arguments");
    if (T == 0) return 0;
    const int F = act_kind_gated(act) ? N / 2 : N;
    const int64_t n = (int64_t)T * F;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    gated_act_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(z, ldz, T, F, ActParams{act, limit, alpha, shift}, 1, out, out_dtype, ldo);
    SEQ_LAUNCH_CHECK("act");
    return 0;
}

int b200seq_argmax(const float* logits, int R, int V, int32_t* ids, void* stream) {
    if (!logits || !ids || R < 0 || V < 1) return fail(B200SEQ_ERR_INVALID_ARG, "argmax: bad arguments");
    if (R == 0) return 0;
    argmax_kernel<<<R, V >= 4096 ? 1024 : 256, 0, (cudaStream_t)stream>>>(logits, V, ids);
    SEQ_LAUNCH_CHECK("argmax");
    return 0;
}

}  // extern "C"
