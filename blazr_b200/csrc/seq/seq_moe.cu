// seq_moe.cu -- mixture-of-experts feed-forward of layer-list models (bfloat16 expert weights [E][N][K], f32 accumulation).
//   route   : sigmoid scores, group-limited choice of the `top` experts per token, weights normalised over the chosen ones (all f32).
//   sort    : (token, choice) pairs ordered by expert, stable, so that one expert's rows form tiles.
//   linear  : one projection of every pair through its expert's weight.  Few pairs (decode): one launch row per pair, the expert's
//             weight rows streamed by warps with 16-byte loads.  Many pairs: tiles over each expert's sorted rows -- tcgen05 tiles
//             (the grouped form of seq_linear_tc.cu) for bfloat16 rows that lie in sorted order (gather puts the tokens' rows there),
//             64 x 64 f32 fma tiles otherwise (exact 32-bit arithmetic; rows are gathered through the sort on load).
//   combine : weighted sum of a token's expert outputs in choice order, plus an optional shared branch times a sigmoid token gate.
// A pair's result depends on its token and expert only; which other tokens are in the step changes at most the kernel variant.
#include "seq_common.cuh"

namespace b200seq {

constexpr int MOE_MAX_E = 1024;

bool linear_tc_usable(int x_dtype, int64_t ldx, int M, int N, int K, const void* x, const void* w);
int launch_linear_tc_grouped(const void* x, int64_t ldx, const void* w, const int32_t* offs, int E, int rows, int N, int K, int act_kind, void* out, int out_dtype,
                             int64_t ldo, cudaStream_t st);
int launch_linear_tc_heads(const void* x, int64_t ldx, const void* w, int T, int H, int N, int K, int act_kind, void* out, int out_dtype, int64_t ldo, int64_t ocol,
                           cudaStream_t st);
int launch_linear_tc_grouped_act(const void* x, int64_t ldx, const void* w, const int32_t* offs, int E, int rows, int N, int K, const ActParams act, void* out,
                                 int out_dtype, int64_t ldo, cudaStream_t st);

// grid (pairs): row r of the result = the activation row of the token behind the r-th sorted pair (contiguous rows for the tensor-core tiles)
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const int32_t* __restrict__ sorted, int x_div, int K,
                                  __nv_bfloat16* __restrict__ out, int64_t ldo) {
    const int r = blockIdx.x;
    const __nv_bfloat16* src = x + (int64_t)(sorted[r] / x_div) * ldx;
    __nv_bfloat16* dst = out + (int64_t)r * ldo;
    if ((K & 7) == 0 && (ldx & 7) == 0 && (ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<const uint4*>(src + k);
    } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = src[k];
    }
}

// choice of one token by one warp: zr = its E router logits; sm = 2 * E + groups floats of shared memory
// kind 0: sigmoid scores; kind 1: soft-max over the E logits.  corr (or null) is added to the scores for the choice only.
__device__ __forceinline__ void route_token(const float* zr, float* sm, int t, int lane, int E, int groups, int keep, int top, int32_t* __restrict__ ids,
                                            float* __restrict__ wts, int32_t* __restrict__ counts, int kind = 0, const float* __restrict__ corr = nullptr) {
    float* s = sm;            // [E] scores
    float* avail = sm + E;    // [E] choice scores; a chosen or excluded expert is marked by -inf
    float* gsc = avail + E;   // [groups]
    if (kind == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
        mx = warp_max(mx);
        float den = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(zr[e] - mx);
            s[e] = v;
            den += v;
        }
        den = warp_sum(den);
        for (int e = lane; e < E; e += 32) {
            const float v = s[e] / den;
            s[e] = v, avail[e] = v + (corr ? corr[e] : 0.f);
        }
    } else {
        for (int e = lane; e < E; e += 32) {
            const float v = sigmoidf_acc(zr[e]);
            s[e] = v, avail[e] = v + (corr ? corr[e] : 0.f);
        }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int gs = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -1.f, b = -1.f;   // two largest
            for (int i = 0; i < gs; ++i) {
                const float v = s[g * gs + i];
                if (v > a) b = a, a = v;
                else if (v > b) b = v;
            }
            gsc[g] = gs > 1 ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups stay: mark them by a negative score, then exclude the experts of every other group
        for (int k = 0; k < keep; ++k) {
            float best = -1.f;
            int arg = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gsc[g] > best) best = gsc[g], arg = g;
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ov > best || (ov == best && oi < arg)) best = ov, arg = oi;
            }
            if (lane == 0 && arg != 0x7fffffff) gsc[arg] = -2.f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gsc[e / gs] != -2.f) avail[e] = -INFINITY;
        __syncwarp();
    }
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (avail[e] > best) best = avail[e], arg = e;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oi < arg)) best = ov, arg = oi;
        }
        if (arg == 0x7fffffff) arg = 0;   // fewer allowed experts than `top`: cannot happen with a valid configuration
        best = s[arg];                    // the weight is the score itself, without the correction
        __syncwarp();
        if (lane == 0) {
            ids[(int64_t)t * top + k] = arg;
            wts[(int64_t)t * top + k] = best;
            avail[arg] = -INFINITY;
            if (counts) atomicAdd(&counts[arg], 1);
        }
        sum += best;
        __syncwarp();
    }
    const float inv = 1.0f / (sum + 1e-20f);
    __syncwarp();
    for (int k = lane; k < top; k += 32) wts[(int64_t)t * top + k] *= inv;
}

// grid (T), one warp per token
__global__ void moe_route_kernel(const float* __restrict__ z, int64_t ldz, int E, int groups, int keep, int top, int32_t* __restrict__ ids,
                                 float* __restrict__ wts, int32_t* __restrict__ counts, int kind, const float* __restrict__ corr) {
    extern __shared__ float sm[];
    route_token(z + (int64_t)blockIdx.x * ldz, sm, blockIdx.x, threadIdx.x, E, groups, keep, top, ids, wts, counts, kind, corr);
}

// choice by table: one thread per (token, choice)
__global__ void moe_table_route_kernel(const int32_t* __restrict__ table, const int32_t* __restrict__ tok_ids, int T, int E, int top, int32_t* __restrict__ ids,
                                       float* __restrict__ wts, int32_t* __restrict__ counts, int* err) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= T * top) return;
    const int t = p / top, j = p - t * top;
    int e = table[(int64_t)tok_ids[t] * top + j];
    if (e < 0 || e >= E) {   // a table entry outside the experts: flagged, and kept inside the weights
        atomicOr(err, 4);
        e = 0;
    }
    ids[p] = e;
    wts[p] = 1.0f / (float)top;
    if (counts) atomicAdd(&counts[e], 1);
}

__device__ __forceinline__ void bf16x8_f32(const uint4 v, float* f);
template <typename XT>
__device__ __forceinline__ float ldx(const XT* p);

// Router of a step of few tokens in one kernel: grid (T), 8 warps.  The warps share out the NR rows of the router weight (the E experts'
// rows and any rows stacked behind them), z[t][n] = x[t] . w[n] goes to memory and to shared memory, then warp 0 makes the token's choice.
template <typename XT, bool VEC>
__global__ void __launch_bounds__(256) moe_router_rows_kernel(const XT* __restrict__ x, int64_t ldx_, const __nv_bfloat16* __restrict__ w, int NR, int K,
                                                              float* __restrict__ z, int64_t ldz, int E, int groups, int keep, int top,
                                                              int32_t* __restrict__ ids, float* __restrict__ wts, int kind, const float* __restrict__ corr) {
    extern __shared__ float sm[];   // NR logits, then the choice's 2 * E + groups floats
    const int t = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const XT* xr = x + (int64_t)t * ldx_;
    for (int n = wid; n < NR; n += 8) {
        const __nv_bfloat16* wr = w + (int64_t)n * K;
        float acc = 0.f;
        if (VEC) {
#pragma unroll 4
            for (int k = lane * 8; k < K; k += 256) {
                float wv[8], xv[8];
                bf16x8_f32(__ldg(reinterpret_cast<const uint4*>(wr + k)), wv);
                if (sizeof(XT) == 4) {
                    const float4 q0 = __ldg(reinterpret_cast<const float4*>(xr + k)), q1 = __ldg(reinterpret_cast<const float4*>(xr + k) + 1);
                    xv[0] = q0.x, xv[1] = q0.y, xv[2] = q0.z, xv[3] = q0.w, xv[4] = q1.x, xv[5] = q1.y, xv[6] = q1.z, xv[7] = q1.w;
                } else {
                    bf16x8_f32(__ldg(reinterpret_cast<const uint4*>(xr + k)), xv);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) acc = fmaf(wv[i], xv[i], acc);
            }
        } else {
            for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(wr[k]), ldx<XT>(xr + k), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            sm[n] = acc;
            z[(int64_t)t * ldz + n] = acc;
        }
    }
    __syncthreads();
    if (wid == 0) route_token(sm, sm + NR, t, lane, E, groups, keep, top, ids, wts, nullptr, kind, corr);
}

// grid (E), 256 threads: block e places the pairs of expert e behind those of the experts before it, in pair order
__global__ void moe_sort_kernel(const int32_t* __restrict__ ids, int pairs, int E, const int32_t* __restrict__ counts, int32_t* __restrict__ offs,
                                int32_t* __restrict__ sorted, int32_t* __restrict__ slot_of) {
    __shared__ int seg[9];
    __shared__ int red[8];
    const int e = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int before = 0;
    for (int i = threadIdx.x; i < e; i += blockDim.x) before += counts[i];
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    if (lane == 0) red[wid] = before;
    __syncthreads();
    int off = 0;
    for (int w = 0; w < 8; ++w) off += red[w];
    if (threadIdx.x == 0) {
        offs[e] = off;
        if (e == E - 1) offs[E] = off + counts[e];
    }
    const int per = ((pairs + 7) / 8 + 31) & ~31;   // a warp's contiguous share of the pairs
    const int lo = wid * per, hi = min(pairs, lo + per);
    int n = 0;
    for (int p0 = lo; p0 < hi; p0 += 32) {
        const int p = p0 + lane;
        n += __popc(__ballot_sync(0xffffffffu, p < hi && ids[p] == e));
    }
    if (lane == 0) seg[wid + 1] = n;
    __syncthreads();
    if (threadIdx.x == 0) {
        seg[0] = 0;
        for (int w = 1; w <= 8; ++w) seg[w] += seg[w - 1];
    }
    __syncthreads();
    int at = off + seg[wid];
    for (int p0 = lo; p0 < hi; p0 += 32) {
        const int p = p0 + lane;
        const bool mine = p < hi && ids[p] == e;
        const uint32_t bal = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            const int slot = at + __popc(bal & ((1u << lane) - 1));
            sorted[slot] = p;
            slot_of[p] = slot;
        }
        at += __popc(bal);
    }
}

__device__ __forceinline__ void bf16x8_f32(const uint4 v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
template <typename XT>
__device__ __forceinline__ float ldx(const XT* p);
template <>
__device__ __forceinline__ float ldx<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename XT, bool VEC>
__device__ __forceinline__ float moe_row_dot(const __nv_bfloat16* __restrict__ wr, const XT* __restrict__ xr, int K, int lane) {
    float acc = 0.f;
    if (VEC) {
#pragma unroll 4
        for (int k = lane * 8; k < K; k += 256) {
            float wv[8], xv[8];
            bf16x8_f32(__ldg(reinterpret_cast<const uint4*>(wr + k)), wv);
            if (sizeof(XT) == 4) {
                const float4 q0 = __ldg(reinterpret_cast<const float4*>(xr + k)), q1 = __ldg(reinterpret_cast<const float4*>(xr + k) + 1);
                xv[0] = q0.x, xv[1] = q0.y, xv[2] = q0.z, xv[3] = q0.w, xv[4] = q1.x, xv[5] = q1.y, xv[6] = q1.z, xv[7] = q1.w;
            } else {
                bf16x8_f32(__ldg(reinterpret_cast<const uint4*>(xr + k)), xv);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(wv[i], xv[i], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(wr[k]), ldx<XT>(xr + k), acc);
    }
    return acc;
}

struct MoeLin {
    const void* x;
    int64_t ldx;
    int x_div;
    const __nv_bfloat16* w;
    const int32_t *ids, *sorted, *offs;
    int pairs, E, N, K, act;
    void* out;
    int out_dtype;
    int64_t ldo;
    ActParams gate;   // gated kinds (act = the kind): weight rows alternate (gate j, up j), the result has N / 2 columns
};

template <typename XT, bool VEC>
__device__ __forceinline__ float moe_row_dot(const __nv_bfloat16* __restrict__ wr, const XT* __restrict__ xr, int K, int lane);

// gated form of the per-pair rows: grid (blocks of 8 warps over N / 2, pairs): a warp = one (gate, up) pair of rows = one output of one pair
template <typename XT, bool VEC>
__global__ void __launch_bounds__(256) moe_rows_gated_kernel(const MoeLin a) {
    const int lane = threadIdx.x & 31;
    const int f = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int p = blockIdx.y;
    if (2 * f + 1 >= a.N) return;
    const int e = a.ids[p];
    if (e >= a.E) return;   // an expert without weights (identity): the pair has no row here
    const __nv_bfloat16* wr = a.w + ((int64_t)e * a.N + 2 * f) * a.K;
    const XT* xr = reinterpret_cast<const XT*>(a.x) + (int64_t)(a.x_div > 0 ? p / a.x_div : p) * a.ldx;
    const float g = warp_sum(moe_row_dot<XT, VEC>(wr, xr, a.K, lane));
    const float u = warp_sum(moe_row_dot<XT, VEC>(wr + a.K, xr, a.K, lane));
    if (lane == 0) store_act(a.out, a.out_dtype, (int64_t)p * a.ldo + f, act_gated(a.gate, g, u));
}

// grid (blocks of 8 warps over N, pairs): a warp = one output of one pair
template <typename XT, bool VEC>
__global__ void __launch_bounds__(256) moe_rows_kernel(const MoeLin a) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int p = blockIdx.y;
    if (n >= a.N) return;
    const int e = a.ids[p];
    if (e >= a.E) return;
    const __nv_bfloat16* wr = a.w + ((int64_t)e * a.N + n) * a.K;
    const XT* xr = reinterpret_cast<const XT*>(a.x) + (int64_t)(a.x_div > 0 ? p / a.x_div : p) * a.ldx;
    float acc = 0.f;
    if (VEC) {
#pragma unroll 4
        for (int k = lane * 8; k < a.K; k += 256) {
            float wv[8], xv[8];
            bf16x8_f32(__ldg(reinterpret_cast<const uint4*>(wr + k)), wv);
            if (sizeof(XT) == 4) {
                const float4 q0 = __ldg(reinterpret_cast<const float4*>(xr + k)), q1 = __ldg(reinterpret_cast<const float4*>(xr + k) + 1);
                xv[0] = q0.x, xv[1] = q0.y, xv[2] = q0.z, xv[3] = q0.w, xv[4] = q1.x, xv[5] = q1.y, xv[6] = q1.z, xv[7] = q1.w;
            } else {
                bf16x8_f32(__ldg(reinterpret_cast<const uint4*>(xr + k)), xv);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(wv[i], xv[i], acc);
        }
    } else {
        for (int k = lane; k < a.K; k += 32) acc = fmaf(__bfloat162float(wr[k]), ldx<XT>(xr + k), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        if (a.act < 0) reinterpret_cast<float*>(a.out)[(int64_t)p * a.ldo + n] = acc;
        else store_act(a.out, a.out_dtype, (int64_t)p * a.ldo + n, act_plain(a.act, acc));
    }
}

// 64 x 64 tiles over the sorted rows of one expert; grid (N tiles, upper bound of the row tiles of all experts)
constexpr int MT = 64, MTK = 16;
template <typename XT>
__global__ void __launch_bounds__(256) moe_tiled_kernel(const MoeLin a) {
    __shared__ float xs[MTK][MT + 4];
    __shared__ float ws[MTK][MT + 4];
    __shared__ int rowsrc[MT];
    int e = 0, r0 = 0, rend = 0;
    {   // which expert and which of its row tiles this block has
        int acc = 0, idx = blockIdx.y;
        bool found = false;
        for (e = 0; e < a.E; ++e) {
            const int b = a.offs[e], c = a.offs[e + 1] - b;
            const int nt = (c + MT - 1) / MT;
            if (idx < acc + nt) {
                r0 = b + (idx - acc) * MT, rend = b + c;
                found = true;
                break;
            }
            acc += nt;
        }
        if (!found) return;
    }
    const int n0 = blockIdx.x * MT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    if (threadIdx.x < MT) {
        const int r = r0 + threadIdx.x;
        rowsrc[threadIdx.x] = r < rend ? (a.x_div > 0 ? a.sorted[r] / a.x_div : r) : -1;
    }
    __syncthreads();
    const XT* x = reinterpret_cast<const XT*>(a.x);
    const __nv_bfloat16* w = a.w + (int64_t)e * a.N * a.K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += MTK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            const int src = rowsrc[r];
            xs[kk][r] = (src >= 0 && k < a.K) ? ldx<XT>(x + (int64_t)src * a.ldx + k) : 0.f;
            ws[kk][r] = (n0 + r < a.N && k < a.K) ? __bfloat162float(w[(int64_t)(n0 + r) * a.K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MTK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = xs[kk][ty * 4 + i], bv[i] = ws[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    if (a.act >= 0 && act_is_gated(a.act)) {   // a thread's four columns are two (gate, up) pairs
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + ty * 4 + i;
            if (r >= rend) continue;
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < a.N) store_act(a.out, a.out_dtype, (int64_t)r * a.ldo + (n >> 1), act_gated(a.gate, acc[i][j], acc[i][j + 1]));
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty * 4 + i;
        if (r >= rend) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            if (a.act < 0) reinterpret_cast<float*>(a.out)[(int64_t)r * a.ldo + n] = acc[i][j];
            else store_act(a.out, a.out_dtype, (int64_t)r * a.ldo + n, act_plain(a.act, acc[i][j]));
        }
    }
}

// ---- per-head projections: out[t][h * ocol + n] = sum_k x[t][h * K + k] * w[h][n][k] ---------------------------------------------------------
struct HeadLin {
    const void* x;
    int64_t ldx;
    const __nv_bfloat16* w;
    int T, H, N, K, act;
    void* out;
    int out_dtype;
    int64_t ldo, ocol;
};
__device__ __forceinline__ void head_store(const HeadLin& a, int64_t idx, float v) {
    if (a.act < 0) reinterpret_cast<float*>(a.out)[idx] = v;
    else store_act(a.out, a.out_dtype, idx, act_plain(a.act, v));
}
// few (token, head) pairs: grid (blocks of 8 warps over N, T * H), a warp = one output of one pair, the head's weight rows streamed
template <typename XT, bool VEC>
__global__ void __launch_bounds__(256) head_rows_kernel(const HeadLin a) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= a.N) return;
    const int t = blockIdx.y / a.H, h = blockIdx.y - t * a.H;
    const float acc = warp_sum(moe_row_dot<XT, VEC>(a.w + ((int64_t)h * a.N + n) * a.K, reinterpret_cast<const XT*>(a.x) + (int64_t)t * a.ldx + (int64_t)h * a.K, a.K, lane));
    if (lane == 0) head_store(a, (int64_t)t * a.ldo + (int64_t)h * a.ocol + n, acc);
}
// 64 x 64 f32 fma tiles: grid (N tiles, token tiles, H)
template <typename XT>
__global__ void __launch_bounds__(256) head_tiled_kernel(const HeadLin a) {
    __shared__ float xs[MTK][MT + 4];
    __shared__ float ws[MTK][MT + 4];
    const int n0 = blockIdx.x * MT, t0 = blockIdx.y * MT, h = blockIdx.z;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const XT* x = reinterpret_cast<const XT*>(a.x) + (int64_t)h * a.K;
    const __nv_bfloat16* w = a.w + (int64_t)h * a.N * a.K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += MTK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            xs[kk][r] = (t0 + r < a.T && k < a.K) ? ldx<XT>(x + (int64_t)(t0 + r) * a.ldx + k) : 0.f;
            ws[kk][r] = (n0 + r < a.N && k < a.K) ? __bfloat162float(w[(int64_t)(n0 + r) * a.K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MTK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = xs[kk][ty * 4 + i], bv[i] = ws[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= a.T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < a.N) head_store(a, (int64_t)t * a.ldo + (int64_t)h * a.ocol + n, acc[i][j]);
        }
    }
}

// grid (T)
__global__ void moe_combine_kernel(const float* __restrict__ ys, const float* __restrict__ wts, const int32_t* __restrict__ slot_of, int top, int W,
                                   const float* __restrict__ shared, const float* __restrict__ gate_z, int64_t ldg, float* __restrict__ y,
                                   const int32_t* __restrict__ ids, int E_real, const float* __restrict__ x_id) {
    const int64_t t = blockIdx.x;
    float gate = 1.f;
    if (shared && gate_z) gate = sigmoidf_acc(gate_z[t * ldg]);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int64_t p = t * top + j;
            const int64_t slot = slot_of ? slot_of[p] : p;
            acc = fmaf(wts[p], (ids && ids[p] >= E_real) ? x_id[t * W + c] : ys[slot * W + c], acc);
        }
        if (shared) acc = fmaf(gate, shared[t * W + c], acc);
        y[t * W + c] = acc;
    }
}

}  // namespace b200seq

using namespace b200seq;

extern "C" {

int b200seq_moe_route(const float* z, int64_t ldz, int T, int E, int groups, int keep, int top, int32_t* ids, float* wts, int32_t* counts, void* stream) {
    return b200seq_moe_route_ex(z, ldz, T, E, groups, keep, top, 0, nullptr, ids, wts, counts, stream);
}

int b200seq_moe_route_ex(const float* z, int64_t ldz, int T, int E, int groups, int keep, int top, int kind, const float* correction, int32_t* ids, float* wts,
                         int32_t* counts, void* stream) {
    if (kind != 0 && kind != 1) return fail(B200SEQ_ERR_INVALID_ARG, "moe_route: score kind 0 (sigmoid) or 1 (soft-max)");
    if (!z || !ids || !wts || T < 0 || E < 1 || E > MOE_MAX_E || top < 1 || top > E || ldz < E) return fail(B200SEQ_ERR_INVALID_ARG, "moe_route: bad arguments (experts <= %d)", MOE_MAX_E);
    if (groups > 1 && (E % groups || keep < 1 || keep > groups || (int64_t)keep * (E / groups) < top))
        return fail(B200SEQ_ERR_INVALID_ARG, "moe_route: groups must divide the experts and the kept groups must hold `top` experts");
    cudaStream_t cs = (cudaStream_t)stream;
    if (counts) {
        cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int32_t), cs);
        if (e != cudaSuccess) return cuda_status(e, "moe_route memset");
    }
    if (T == 0) return 0;
    const int g = groups > 1 ? groups : 1;
    moe_route_kernel<<<T, 32, (size_t)(2 * E + g) * sizeof(float), cs>>>(z, ldz, E, g, groups > 1 ? keep : 1, top, ids, wts, counts, kind, correction);
    SEQ_LAUNCH_CHECK("moe_route");
    return 0;
}

int b200seq_moe_table_route(const int32_t* table, const int32_t* tok_ids, int T, int E, int top, int32_t* ids, float* wts, int32_t* counts, void* stream) {
    if (!table || !tok_ids || !ids || !wts || T < 0 || E < 1 || top < 1 || top > E) return fail(B200SEQ_ERR_INVALID_ARG, "moe_table_route: bad arguments");
    cudaStream_t cs = (cudaStream_t)stream;
    if (counts) {
        cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int32_t), cs);
        if (e != cudaSuccess) return cuda_status(e, "moe_table_route memset");
    }
    if (T == 0) return 0;
    moe_table_route_kernel<<<(T * top + 127) / 128, 128, 0, cs>>>(table, tok_ids, T, E, top, ids, wts, counts, error_flag_dev());
    SEQ_LAUNCH_CHECK("moe_table_route");
    return 0;
}

int b200seq_moe_router(const void* x, int x_dtype, int64_t ldx_, const void* w, int T, int NR, int K, int E, int groups, int keep, int top, float* z, int64_t ldz,
                       int32_t* ids, float* wts, void* stream) {
    return b200seq_moe_router_ex(x, x_dtype, ldx_, w, T, NR, K, E, groups, keep, top, 0, nullptr, z, ldz, ids, wts, stream);
}

int b200seq_moe_router_ex(const void* x, int x_dtype, int64_t ldx_, const void* w, int T, int NR, int K, int E, int groups, int keep, int top, int kind,
                          const float* correction, float* z, int64_t ldz, int32_t* ids, float* wts, void* stream) {
    if (kind != 0 && kind != 1) return fail(B200SEQ_ERR_INVALID_ARG, "moe_router: score kind 0 (sigmoid) or 1 (soft-max)");
    if (!x || !w || !z || !ids || !wts || T < 0 || T > 8 || E < 1 || E > MOE_MAX_E || NR < E || K < 1 || ldx_ < K || ldz < NR || top < 1 || top > E)
        return fail(B200SEQ_ERR_INVALID_ARG, "moe_router: bad arguments (at most 8 tokens, experts <= %d)", MOE_MAX_E);
    if (groups > 1 && (E % groups || keep < 1 || keep > groups || (int64_t)keep * (E / groups) < top))
        return fail(B200SEQ_ERR_INVALID_ARG, "moe_router: groups must divide the experts and the kept groups must hold `top` experts");
    if (x_dtype != B200SEQ_F32 && x_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "moe_router: activation dtype");
    if (T == 0) return 0;
    const int g = groups > 1 ? groups : 1, kp = groups > 1 ? keep : 1;
    const size_t smem = (size_t)(NR + 2 * E + g) * sizeof(float);
    const size_t es = x_dtype == B200SEQ_F32 ? 4 : 2;
    const bool vec = K % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx_ * es) % 16 == 0;
    cudaStream_t cs = (cudaStream_t)stream;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    if (x_dtype == B200SEQ_F32) {
        if (vec) moe_router_rows_kernel<float, true><<<T, 256, smem, cs>>>((const float*)x, ldx_, wb, NR, K, z, ldz, E, g, kp, top, ids, wts, kind, correction);
        else moe_router_rows_kernel<float, false><<<T, 256, smem, cs>>>((const float*)x, ldx_, wb, NR, K, z, ldz, E, g, kp, top, ids, wts, kind, correction);
    } else {
        if (vec) moe_router_rows_kernel<__nv_bfloat16, true><<<T, 256, smem, cs>>>((const __nv_bfloat16*)x, ldx_, wb, NR, K, z, ldz, E, g, kp, top, ids, wts, kind, correction);
        else moe_router_rows_kernel<__nv_bfloat16, false><<<T, 256, smem, cs>>>((const __nv_bfloat16*)x, ldx_, wb, NR, K, z, ldz, E, g, kp, top, ids, wts, kind, correction);
    }
    SEQ_LAUNCH_CHECK("moe_router");
    return 0;
}

int b200seq_moe_sort(const int32_t* ids, int pairs, int E, const int32_t* counts, int32_t* offs, int32_t* sorted, int32_t* slot_of, void* stream) {
    if (!ids || !counts || !offs || !sorted || !slot_of || pairs < 0 || E < 1) return fail(B200SEQ_ERR_INVALID_ARG, "moe_sort: bad arguments");
    moe_sort_kernel<<<E, 256, 0, (cudaStream_t)stream>>>(ids, pairs, E, counts, offs, sorted, slot_of);
    SEQ_LAUNCH_CHECK("moe_sort");
    return 0;
}

int b200seq_moe_linear(const void* x, int x_dtype, int64_t ldx_, int x_div, const void* w, const int32_t* ids, const int32_t* sorted, const int32_t* offs, int pairs,
                       int E, int N, int K, int act, void* out, int out_dtype, int64_t ldo, void* stream) {
    if (act >= 0 && act_kind_gated(act)) return fail(B200SEQ_ERR_INVALID_ARG, "moe_linear: only plain activation kinds (gated kinds: b200seq_moe_linear_act)");
    return b200seq_moe_linear_act(x, x_dtype, ldx_, x_div, w, ids, sorted, offs, pairs, E, N, K, act, 0.f, 0.f, 0.f, out, out_dtype, ldo, stream);
}

int b200seq_moe_linear_act(const void* x, int x_dtype, int64_t ldx_, int x_div, const void* w, const int32_t* ids, const int32_t* sorted, const int32_t* offs, int pairs,
                           int E, int N, int K, int act, float limit, float alpha, float shift, void* out, int out_dtype, int64_t ldo, void* stream) {
    const bool gated = act >= 0 && act_kind_gated(act);
    if (!x || !w || !out || pairs < 0 || E < 1 || N < 1 || K < 1 || ldx_ < K || ldo < (gated ? N / 2 : N) || x_div < 0 || (gated && (N & 1)))
        return fail(B200SEQ_ERR_INVALID_ARG, "moe_linear: bad arguments");
    if (x_dtype != B200SEQ_F32 && x_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "moe_linear: activation dtype");
    if (act >= 0 && !act_kind_known(act)) return fail(B200SEQ_ERR_INVALID_ARG, "moe_linear: unknown activation kind");
    if (act >= 0 && out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "moe_linear: output dtype");
    if ((sorted == nullptr) != (offs == nullptr) || (!sorted && !ids)) return fail(B200SEQ_ERR_INVALID_ARG, "moe_linear: ids, or sorted with offs");
    if (pairs == 0) return 0;
    const ActParams ap{act, limit, alpha, shift};
    const MoeLin a{x, ldx_, x_div, (const __nv_bfloat16*)w, ids, sorted, offs, pairs, E, N, K, act, out, out_dtype, ldo, ap};
    cudaStream_t cs = (cudaStream_t)stream;
    if (!sorted && gated) {
        const size_t es = x_dtype == B200SEQ_F32 ? 4 : 2;
        const bool vec = K % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx_ * es) % 16 == 0;
        if (pairs > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "moe_linear: too many pairs for the row form");
        dim3 grid((N / 2 + 7) / 8, pairs);
        if (x_dtype == B200SEQ_F32) {
            if (vec) moe_rows_gated_kernel<float, true><<<grid, 256, 0, cs>>>(a);
            else moe_rows_gated_kernel<float, false><<<grid, 256, 0, cs>>>(a);
        } else {
            if (vec) moe_rows_gated_kernel<__nv_bfloat16, true><<<grid, 256, 0, cs>>>(a);
            else moe_rows_gated_kernel<__nv_bfloat16, false><<<grid, 256, 0, cs>>>(a);
        }
        SEQ_LAUNCH_CHECK("moe_linear gated rows");
        return 0;
    }
    if (!sorted) {
        const size_t es = x_dtype == B200SEQ_F32 ? 4 : 2;
        const bool vec = K % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx_ * es) % 16 == 0;
        if (pairs > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "moe_linear: too many pairs for the row form");
        dim3 grid((N + 7) / 8, pairs);
        if (x_dtype == B200SEQ_F32) {
            if (vec) moe_rows_kernel<float, true><<<grid, 256, 0, cs>>>(a);
            else moe_rows_kernel<float, false><<<grid, 256, 0, cs>>>(a);
        } else {
            if (vec) moe_rows_kernel<__nv_bfloat16, true><<<grid, 256, 0, cs>>>(a);
            else moe_rows_kernel<__nv_bfloat16, false><<<grid, 256, 0, cs>>>(a);
        }
        SEQ_LAUNCH_CHECK("moe_linear rows");
        return 0;
    }
    if (x_div == 0 && pairs >= 32 && linear_tc_usable(x_dtype, ldx_, pairs, N, K, x, w)) {   // rows laid out like the result: tcgen05 tiles per expert
        if (gated) return launch_linear_tc_grouped_act(x, ldx_, w, offs, E, pairs, N, K, ap, out, out_dtype, ldo, cs);
        return launch_linear_tc_grouped(x, ldx_, w, offs, E, pairs, N, K, act, out, out_dtype, ldo, cs);
    }
    const int tiles = (pairs + MT - 1) / MT + E;
    if (tiles > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "moe_linear: too many row tiles");
    dim3 grid((N + MT - 1) / MT, tiles);
    if (x_dtype == B200SEQ_F32) moe_tiled_kernel<float><<<grid, 256, 0, cs>>>(a);
    else moe_tiled_kernel<__nv_bfloat16><<<grid, 256, 0, cs>>>(a);
    SEQ_LAUNCH_CHECK("moe_linear tiles");
    return 0;
}

int b200seq_head_linear(const void* x, int x_dtype, int64_t ldx_, const void* w, int T, int H, int N, int K, int act, void* out, int out_dtype, int64_t ldo, int64_t ocol,
                        void* stream) {
    if (!x || !w || !out || T < 0 || H < 1 || N < 1 || K < 1 || ldx_ < (int64_t)H * K || ocol < N || ldo < (int64_t)(H - 1) * ocol + N)
        return fail(B200SEQ_ERR_INVALID_ARG, "head_linear: bad arguments");
    if (x_dtype != B200SEQ_F32 && x_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "head_linear: activation dtype");
    if (act >= 0 && (!act_kind_known(act) || act_kind_gated(act) || (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16)))
        return fail(B200SEQ_ERR_INVALID_ARG, "head_linear: a plain activation kind and an output dtype");
    if (T == 0) return 0;
    if (H > 65535 || (int64_t)T * H > 65535 * 64) return fail(B200SEQ_ERR_UNSUPPORTED, "head_linear: too many heads or tokens in one step");
    const HeadLin a{x, ldx_, (const __nv_bfloat16*)w, T, H, N, K, act, out, out_dtype, ldo, ocol};
    cudaStream_t cs = (cudaStream_t)stream;
    const size_t es = x_dtype == B200SEQ_F32 ? 4 : 2;
    if ((int64_t)T * H <= 64) {
        const bool vec = K % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx_ * es) % 16 == 0;
        dim3 grid((N + 7) / 8, T * H);
        if (x_dtype == B200SEQ_F32) {
            if (vec) head_rows_kernel<float, true><<<grid, 256, 0, cs>>>(a);
            else head_rows_kernel<float, false><<<grid, 256, 0, cs>>>(a);
        } else {
            if (vec) head_rows_kernel<__nv_bfloat16, true><<<grid, 256, 0, cs>>>(a);
            else head_rows_kernel<__nv_bfloat16, false><<<grid, 256, 0, cs>>>(a);
        }
        SEQ_LAUNCH_CHECK("head_linear rows");
        return 0;
    }
    if (T >= 32 && linear_tc_usable(x_dtype, ldx_, T, N, K, x, w)) return launch_linear_tc_heads(x, ldx_, w, T, H, N, K, act, out, out_dtype, ldo, ocol, cs);
    dim3 grid((N + MT - 1) / MT, (T + MT - 1) / MT, H);
    if (x_dtype == B200SEQ_F32) head_tiled_kernel<float><<<grid, 256, 0, cs>>>(a);
    else head_tiled_kernel<__nv_bfloat16><<<grid, 256, 0, cs>>>(a);
    SEQ_LAUNCH_CHECK("head_linear tiles");
    return 0;
}

int b200seq_moe_gather(const void* x_bf16, int64_t ldx_, const int32_t* sorted, int x_div, int pairs, int K, void* out_bf16, int64_t ldo, void* stream) {
    if (!x_bf16 || !sorted || !out_bf16 || x_div < 1 || pairs < 0 || K < 1 || ldx_ < K || ldo < K) return fail(B200SEQ_ERR_INVALID_ARG, "moe_gather: bad arguments");
    if (pairs == 0) return 0;
    moe_gather_kernel<<<pairs, K >= 2048 ? 256 : 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x_bf16, ldx_, sorted, x_div, K, (__nv_bfloat16*)out_bf16, ldo);
    SEQ_LAUNCH_CHECK("moe_gather");
    return 0;
}

int b200seq_moe_combine(const float* ys, const float* wts, const int32_t* slot_of, int T, int top, int W, const float* shared, const float* gate_z, int64_t ldg,
                        float* y, void* stream) {
    return b200seq_moe_combine_ex(ys, wts, slot_of, nullptr, 0, nullptr, T, top, W, shared, gate_z, ldg, y, stream);
}

int b200seq_moe_combine_ex(const float* ys, const float* wts, const int32_t* slot_of, const int32_t* ids, int E_real, const float* x_id, int T, int top, int W,
                           const float* shared, const float* gate_z, int64_t ldg, float* y, void* stream) {
    if (!ys || !wts || !y || T < 0 || top < 1 || W < 1 || (ids && !x_id)) return fail(B200SEQ_ERR_INVALID_ARG, "moe_combine: bad arguments");
    if (T == 0) return 0;
    moe_combine_kernel<<<T, W >= 1024 ? 256 : 128, 0, (cudaStream_t)stream>>>(ys, wts, slot_of, top, W, shared, gate_z, ldg, y, ids, E_real, x_id);
    SEQ_LAUNCH_CHECK("moe_combine");
    return 0;
}

}  // extern "C"
