// seq_retention.cu -- retention: linear attention with one fixed decay per head, no soft-max and no denominator, over a flat mixed
// batch.  Per head (decay d, key size D, value size V), with the state S [D][V] carried per sequence in f32:
//     S_t = d * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
// followed by the division of every head's o_t by its root mean square and the multiplication by silu(gate).
// Everything here is f32: rotation angles, the keys' scale, the decay powers, scores, state, the unit norm and the gate.
//
// Steps in which every entry brings ONE token (decode): one kernel per (entry, head) -- rotation of q and k, state update, output,
// unit norm and gate.
// Other steps: the portions are cut into chunks of RET_C tokens (from the portion's first token; chunk borders have nothing to do
// with positions, pages or earlier portions) that run in parallel:
//   rotate   q and k turn in place (b200seq_rotary), k times its scale
//   A        U_c = sum_i d^(L-1-i) k_i v_i^T                           per chunk, from its L tokens alone
//   B        start_c = S;  S = d^L S + U_c   in chunk order per entry; the last S goes to the sequence's slot
//   C        o_i = d^(i+1) start_c^T q_i + sum_(j<=i) d^(i-j) (q_i . k_j) v_j
//   finish   unit norm over V and gate, written in the activation type
// Powers of the decay are exp2(n * log2 d) with log2 d handed in (computed in double by the caller).
#include "seq_common.cuh"

namespace b200seq {

constexpr int RET_C = 64;    // tokens per chunk
constexpr int RET_DS = 32;   // key dimensions per staged slab
constexpr int RET_NT = 256;

// ---- rotary positions on head vectors inside projection rows ------------------------------------------------------------------------
// grid (T), any block size: heads [nheads][D] at column `col` of row t; the first rot_dims dimensions of every head turn by
// pos * freq[i], pair (i, i + rot_dims / 2) (half = 1) or (2i, 2i + 1) (half = 0); cos and sin times rot_scale; every element of
// the head (rotated or not) times mult.
__global__ void rotary_kernel(float* __restrict__ x, int64_t ld, int col, int nheads, int D, const int32_t* __restrict__ tok_pos, int rot_dims, int half,
                              const float* __restrict__ freq, float rot_scale, float mult) {
    extern __shared__ float cs_sm[];   // [rot_dims]: cos | sin of every pair at this position
    const int t = blockIdx.x;
    const int np = rot_dims >> 1;
    const float pos = (float)tok_pos[t];
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        cs_sm[i] = cs * rot_scale, cs_sm[np + i] = sn * rot_scale;
    }
    __syncthreads();
    float* row = x + (int64_t)t * ld + col;
    const int per = np + (D - rot_dims);   // work items of a head: its pairs, then its unrotated elements
    for (int idx = threadIdx.x; idx < nheads * per; idx += blockDim.x) {
        const int h = idx / per, i = idx - h * per;
        float* p = row + (int64_t)h * D;
        if (i < np) {
            const int iu = half ? i : 2 * i, iv = half ? i + np : 2 * i + 1;
            const float u = p[iu], v = p[iv], c = cs_sm[i], s = cs_sm[np + i];
            p[iu] = (u * c - v * s) * mult;
            p[iv] = (v * c + u * s) * mult;
        } else if (mult != 1.f) {
            p[rot_dims + (i - np)] *= mult;
        }
    }
}

struct RetArgs {
    float* proj;
    int64_t ld;
    int q_col, k_col, v_col, g_col;
    int H, D, V;
    const float* decay;   // [2][H]: decay, log2(decay)
    float eps;
    int rot_dims, rot_half;
    const float* rot_freq;
    float rot_scale, k_scale;
    float* state;       // [slots][H][D][V]
    float* seg_state;   // [chunks][H][D][V]
    float* o_raw;       // [T][H * V]
    void* out;
    int out_dtype;
};

// ---- decode: grid (B, H), RET_NT threads ------------------------------------------------------------------------------------------------
// dynamic shared memory: q [D] | k [D] | partial o [4][V] | 40 floats of reduction scratch
__global__ void __launch_bounds__(RET_NT) retention_step_kernel(const RetArgs a, const b200seq_step st) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, V = a.V, H = a.H;
    float* qs = sm;
    float* ks = qs + D;
    float* part = ks + D;        // [4][V]
    float* red = part + 4 * V;
    const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int t = st.ent_start[e];
    const float pos = (float)st.tok_pos[t];
    const float* row = a.proj + (int64_t)t * a.ld;
    const float* qg = row + a.q_col + (int64_t)h * D;
    const float* kg = row + a.k_col + (int64_t)h * D;
    const int np = a.rot_dims >> 1;
    for (int i = tid; i < D; i += RET_NT) {
        float q = qg[i], k = kg[i];
        if (i < a.rot_dims) {
            const int pi = a.rot_half ? (i < np ? i : i - np) : (i >> 1);
            const bool first = a.rot_half ? i < np : !(i & 1);
            const int other = a.rot_half ? (first ? i + np : i - np) : (i ^ 1);
            float sn, cs;
            sincosf(pos * a.rot_freq[pi], &sn, &cs);
            cs *= a.rot_scale, sn *= a.rot_scale;
            const float qo = qg[other], ko = kg[other];
            q = first ? q * cs - qo * sn : q * cs + qo * sn;
            k = first ? k * cs - ko * sn : k * cs + ko * sn;
        }
        qs[i] = q, ks[i] = k * a.k_scale;
    }
    __syncthreads();
    const float dec = a.decay[h];
    float* S = a.state + ((int64_t)st.ent_slot[e] * H + h) * D * V;
    const bool fresh = st.ent_pos0[e] == 0;
    const float* vg = row + a.v_col + (int64_t)h * V;
    // thread = (value column of a tile of 64, one of 4 groups of key dimensions)
    const int vt = tid & 63, dg = tid >> 6;
    for (int v0 = 0; v0 < V; v0 += 64) {
        const int v = v0 + vt;
        float o = 0.f;
        if (v < V) {
            const float vv = vg[v];
            for (int d = dg; d < D; d += 4) {
                float* sp = S + (int64_t)d * V + v;
                const float s = fmaf(dec, fresh ? 0.f : *sp, ks[d] * vv);
                *sp = s;
                o = fmaf(s, qs[d], o);
            }
            part[dg * V + v] = o;
        }
    }
    __syncthreads();
    float ss = 0.f;
    for (int v = tid; v < V; v += RET_NT) {
        const float o = (part[v] + part[V + v]) + (part[2 * V + v] + part[3 * V + v]);
        part[v] = o;
        ss = fmaf(o, o, ss);
    }
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)V + a.eps);
    const float* gg = row + a.g_col + (int64_t)h * V;
    for (int v = tid; v < V; v += RET_NT) store_act(a.out, a.out_dtype, ((int64_t)t * H + h) * V + v, part[v] * rinv * siluf_acc(gg[v]));
}

// ---- chunked form -------------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool ret_find_chunk(const b200seq_step& st, int idx, int& e, int& row0, int& len) {
    int acc = 0;
    for (e = 0; e < st.B; ++e) {
        const int s0 = st.ent_start[e], n = st.ent_start[e + 1] - s0;
        const int nc = (n + RET_C - 1) / RET_C;
        if (idx < acc + nc) {
            const int local = idx - acc;
            row0 = s0 + local * RET_C;
            len = min(RET_C, n - local * RET_C);
            return true;
        }
        acc += nc;
    }
    return false;
}

// pass A: grid (V tiles of 64, D tiles of 64, chunks * H).  U[d][v] = sum_i d^(L-1-i) k_i[d] v_i[v]; thread (ty, tx): d = ty * 4 + i, v = tx * 4 + u
__global__ void __launch_bounds__(RET_NT) retention_local_kernel(const RetArgs a, const b200seq_step st) {
    __shared__ __align__(16) float Ks[RET_C][68];
    __shared__ __align__(16) float Vs[RET_C][68];
    const int c = blockIdx.z / a.H, h = blockIdx.z - c * a.H;
    int e, row0, len;
    if (!ret_find_chunk(st, c, e, row0, len)) return;
    const int D = a.D, V = a.V;
    const int v0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float l2 = a.decay[a.H + h];
    for (int idx = tid; idx < RET_C * 64; idx += RET_NT) {
        const int i = idx >> 6, cc = idx & 63;
        const bool in = i < len;
        const float* row = a.proj + (int64_t)(row0 + i) * a.ld;
        Ks[i][cc] = (in && d0 + cc < D) ? row[a.k_col + (int64_t)h * D + d0 + cc] * exp2f((float)(len - 1 - i) * l2) : 0.f;
        Vs[i][cc] = (in && v0 + cc < V) ? row[a.v_col + (int64_t)h * V + v0 + cc] : 0.f;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[i][u] = 0.f;
    for (int i = 0; i < len; ++i) {
        const float4 k = *reinterpret_cast<const float4*>(&Ks[i][ty * 4]);
        const float4 v = *reinterpret_cast<const float4*>(&Vs[i][tx * 4]);
        const float kk[4] = {k.x, k.y, k.z, k.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[ii][u] = fmaf(kk[ii], vv[u], acc[ii][u]);
    }
    float* U = a.seg_state + ((int64_t)c * a.H + h) * D * V;
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
        const int d = d0 + ty * 4 + ii;
        if (d >= D) continue;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + tx * 4 + u;
            if (v < V) U[(int64_t)d * V + v] = acc[ii][u];
        }
    }
}

// pass B: one thread per (entry, head, d, v); walks the entry's chunks in order
__global__ void retention_combine_kernel(const RetArgs a, const b200seq_step st) {
    const int64_t per = (int64_t)a.H * a.D * a.V;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int e = blockIdx.y;
    if (idx >= per) return;
    const int h = (int)(idx / ((int64_t)a.D * a.V));
    int c0 = 0;
    for (int i = 0; i < e; ++i) c0 += (st.ent_start[i + 1] - st.ent_start[i] + RET_C - 1) / RET_C;
    const int n = st.ent_start[e + 1] - st.ent_start[e];
    const int nc = (n + RET_C - 1) / RET_C;
    const float l2 = a.decay[a.H + h];
    const float full = exp2f((float)RET_C * l2);
    float* slot = a.state + (int64_t)st.ent_slot[e] * per + idx;
    float S = st.ent_pos0[e] == 0 ? 0.f : *slot;
    constexpr int AHEAD = 8;   // the chunks' local states do not depend on the walk: fetch a batch of them before the dependent chain uses them
    for (int c0b = 0; c0b < nc; c0b += AHEAD) {
        float U[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) U[j] = c0b + j < nc ? a.seg_state[(int64_t)(c0 + c0b + j) * per + idx] : 0.f;
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            const int c = c0b + j;
            if (c >= nc) break;
            a.seg_state[(int64_t)(c0 + c) * per + idx] = S;
            const int len = min(RET_C, n - c * RET_C);
            S = fmaf(len == RET_C ? full : exp2f((float)len * l2), S, U[j]);
        }
    }
    *slot = S;
}

// pass C: grid (V tiles of 64, chunks, H).  Thread (ty, tx): tokens ty * 4 + i; keys tx + 16 j of the score tile, value columns tx * 4 + u.
__global__ void __launch_bounds__(RET_NT) retention_out_kernel(const RetArgs a, const b200seq_step st) {
    __shared__ __align__(16) float A[RET_C][RET_DS + 4];     // q slab
    __shared__ __align__(16) float Bm[RET_C][68];            // k slab [key][RET_DS + 4], then the value tile [key][64], then state slabs [RET_DS][64]
    __shared__ __align__(16) float Ps[RET_C][RET_C + 4];
    __shared__ float pw[RET_C + 1];
    const int c = blockIdx.y, h = blockIdx.z;
    int e, row0, len;
    if (!ret_find_chunk(st, c, e, row0, len)) return;
    const int D = a.D, V = a.V, H = a.H;
    const int v0 = blockIdx.x * 64;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float l2 = a.decay[H + h];
    if (tid <= RET_C) pw[tid] = exp2f((float)tid * l2);
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int d0 = 0; d0 < D; d0 += RET_DS) {
        __syncthreads();
        for (int idx = tid; idx < RET_C * RET_DS; idx += RET_NT) {
            const int i = idx / RET_DS, dd = idx - i * RET_DS;
            const bool in = i < len && d0 + dd < D;
            const float* row = a.proj + (int64_t)(row0 + i) * a.ld + (int64_t)h * D + d0 + dd;
            A[i][dd] = in ? row[a.q_col] : 0.f;
            Bm[i][dd] = in ? row[a.k_col] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int dd = 0; dd < RET_DS; dd += 4) {
            float4 q[4], k[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = *reinterpret_cast<const float4*>(&A[ty * 4 + i][dd]);
#pragma unroll
            for (int j = 0; j < 4; ++j) k[j] = *reinterpret_cast<const float4*>(&Bm[tx + 16 * j][dd]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(q[i].x, k[j].x, s[i][j]), s[i][j] = fmaf(q[i].y, k[j].y, s[i][j]);
                    s[i][j] = fmaf(q[i].z, k[j].z, s[i][j]), s[i][j] = fmaf(q[i].w, k[j].w, s[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int qi = ty * 4 + i, kj = tx + 16 * j;
            Ps[qi][kj] = (kj <= qi && qi < len) ? s[i][j] * pw[qi - kj] : 0.f;
        }
    __syncthreads();   // every thread is done with the k slab; Ps is complete after the next barrier
    for (int idx = tid; idx < RET_C * 64; idx += RET_NT) {
        const int i = idx >> 6, cc = idx & 63;
        Bm[i][cc] = (i < len && v0 + cc < V) ? a.proj[(int64_t)(row0 + i) * a.ld + a.v_col + (int64_t)h * V + v0 + cc] : 0.f;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[i][u] = 0.f;
    for (int k = 0; k < RET_C; k += 4) {
        float4 p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = *reinterpret_cast<const float4*>(&Ps[ty * 4 + i][k]);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const float4 v = *reinterpret_cast<const float4*>(&Bm[k + kk][tx * 4]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float pv = kk == 0 ? p[i].x : kk == 1 ? p[i].y : kk == 2 ? p[i].z : p[i].w;
                acc[i][0] = fmaf(pv, v.x, acc[i][0]), acc[i][1] = fmaf(pv, v.y, acc[i][1]);
                acc[i][2] = fmaf(pv, v.z, acc[i][2]), acc[i][3] = fmaf(pv, v.w, acc[i][3]);
            }
        }
    }
    // the state the chunk starts from: o_i += d^(i+1) * sum_d q_i[d] start[d][v]
    const float* S0 = a.seg_state + ((int64_t)c * H + h) * D * V;
    float acs[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) acs[i][u] = 0.f;
    for (int d0 = 0; d0 < D; d0 += RET_DS) {
        __syncthreads();
        for (int idx = tid; idx < RET_C * RET_DS; idx += RET_NT) {
            const int i = idx / RET_DS, dd = idx - i * RET_DS;
            A[i][dd] = (i < len && d0 + dd < D) ? a.proj[(int64_t)(row0 + i) * a.ld + a.q_col + (int64_t)h * D + d0 + dd] : 0.f;
        }
        for (int idx = tid; idx < RET_DS * 64; idx += RET_NT) {
            const int dd = idx >> 6, cc = idx & 63;
            Bm[dd][cc] = (d0 + dd < D && v0 + cc < V) ? S0[(int64_t)(d0 + dd) * V + v0 + cc] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int dd = 0; dd < RET_DS; ++dd) {
            const float4 sv = *reinterpret_cast<const float4*>(&Bm[dd][tx * 4]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float q = A[ty * 4 + i][dd];
                acs[i][0] = fmaf(q, sv.x, acs[i][0]), acs[i][1] = fmaf(q, sv.y, acs[i][1]);
                acs[i][2] = fmaf(q, sv.z, acs[i][2]), acs[i][3] = fmaf(q, sv.w, acs[i][3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = ty * 4 + i;
        if (qi >= len) continue;
        const float w = pw[qi + 1];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + tx * 4 + u;
            if (v < V) a.o_raw[((int64_t)(row0 + qi) * H + h) * V + v] = fmaf(w, acs[i][u], acc[i][u]);
        }
    }
}

// finish: grid (T, H), 64 or 128 threads: unit norm over V, gate
__global__ void retention_finish_kernel(const RetArgs a) {
    __shared__ float red[40];
    const int t = blockIdx.x, h = blockIdx.y, V = a.V;
    const float* o = a.o_raw + ((int64_t)t * a.H + h) * V;
    float ss = 0.f;
    for (int v = threadIdx.x; v < V; v += blockDim.x) ss = fmaf(o[v], o[v], ss);
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)V + a.eps);
    const float* gg = a.proj + (int64_t)t * a.ld + a.g_col + (int64_t)h * V;
    for (int v = threadIdx.x; v < V; v += blockDim.x) store_act(a.out, a.out_dtype, ((int64_t)t * a.H + h) * V + v, o[v] * rinv * siluf_acc(gg[v]));
}

}  // namespace b200seq

using namespace b200seq;

extern "C" int b200seq_rotary(float* x, int64_t ld, int col, int nheads, int D, const b200seq_step* st, int rot_dims, int half, const float* freq, float rot_scale,
                              float mult, void* stream) {
    if (!x || !st || col < 0 || nheads < 1 || D < 1 || rot_dims < 0 || rot_dims > D || (rot_dims & 1) || (rot_dims > 0 && !freq))
        return fail(B200SEQ_ERR_INVALID_ARG, "rotary: rotary dimensions must be even, at most the head size, with a frequency table");
    if (st->T == 0 || (rot_dims == 0 && mult == 1.f)) return 0;
    rotary_kernel<<<st->T, 256, (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float), (cudaStream_t)stream>>>(x, ld, col, nheads, D, st->tok_pos, rot_dims, half, freq,
                                                                                                                 rot_scale, mult);
    SEQ_LAUNCH_CHECK("rotary");
    return 0;
}

extern "C" size_t b200seq_retention_scratch_floats(int T, int B, int H, int D, int V) {
    if (T < 1 || B < 1 || T == B) return 0;
    const size_t chunks = (size_t)(T + RET_C - 1) / RET_C + (size_t)B;
    return chunks * H * D * V + (size_t)T * H * V;
}

extern "C" int b200seq_retention(float* proj, int64_t ld, const b200seq_step* st, const b200seq_retention_desc* d, float* state, void* out, int out_dtype,
                                 float* scratch, size_t scratch_floats, void* stream) {
    if (!proj || !st || !d || !state || !out || d->H < 1 || d->D < 1 || d->V < 1 || !d->decay || d->q_col < 0 || d->k_col < 0 || d->v_col < 0 || d->g_col < 0)
        return fail(B200SEQ_ERR_INVALID_ARG, "retention: bad arguments");
    if (d->rot_dims < 0 || d->rot_dims > d->D || (d->rot_dims & 1) || (d->rot_dims > 0 && !d->rot_freq))
        return fail(B200SEQ_ERR_INVALID_ARG, "retention: rotary dimensions must be even, at most the key size, with a frequency table");
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "retention: output dtype");
    if (st->T == 0 || st->B == 0) return 0;
    cudaStream_t cs = (cudaStream_t)stream;
    RetArgs a{proj, ld, d->q_col, d->k_col, d->v_col, d->g_col, d->H, d->D, d->V, d->decay, d->eps, d->rot_dims, d->rot_half, d->rot_freq, d->rot_scale, d->k_scale,
              state, nullptr, nullptr, out, out_dtype};
    if (st->T == st->B) {
        const size_t smem = ((size_t)2 * d->D + 4 * d->V + 40) * sizeof(float);
        if (smem > 48 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "retention: head sizes too large");
        if (st->B > 65535 || d->H > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "retention: too many entries or heads");
        retention_step_kernel<<<dim3(st->B, d->H), RET_NT, smem, cs>>>(a, *st);
        SEQ_LAUNCH_CHECK("retention step");
        return 0;
    }
    const size_t need = b200seq_retention_scratch_floats(st->T, st->B, d->H, d->D, d->V);
    if (!scratch || scratch_floats < need) return fail(B200SEQ_ERR_INVALID_ARG, "retention: a step of portions needs %zu floats of work area", need);
    const int chunks = (st->T + RET_C - 1) / RET_C + st->B;   // upper bound of the step's chunk count
    const int64_t per = (int64_t)d->H * d->D * d->V;
    a.seg_state = scratch;
    a.o_raw = scratch + (size_t)chunks * per;
    if ((int64_t)chunks * d->H > 65535 || d->H > 65535) return fail(B200SEQ_ERR_UNSUPPORTED, "retention: too many chunks x heads in one step");
    if (int rc = b200seq_rotary(proj, ld, d->q_col, d->H, d->D, st, d->rot_dims, d->rot_half, d->rot_freq, d->rot_scale, 1.f, stream)) return rc;
    if (int rc = b200seq_rotary(proj, ld, d->k_col, d->H, d->D, st, d->rot_dims, d->rot_half, d->rot_freq, d->rot_scale, d->k_scale, stream)) return rc;
    const int vt = (d->V + 63) / 64, dt = (d->D + 63) / 64;
    retention_local_kernel<<<dim3(vt, dt, chunks * d->H), RET_NT, 0, cs>>>(a, *st);
    SEQ_LAUNCH_CHECK("retention local pass");
    retention_combine_kernel<<<dim3((unsigned)((per + 255) / 256), st->B), 256, 0, cs>>>(a, *st);
    SEQ_LAUNCH_CHECK("retention combine pass");
    retention_out_kernel<<<dim3(vt, chunks, d->H), RET_NT, 0, cs>>>(a, *st);
    SEQ_LAUNCH_CHECK("retention output pass");
    retention_finish_kernel<<<dim3(st->T, d->H), d->V <= 64 ? 64 : 128, 0, cs>>>(a);
    SEQ_LAUNCH_CHECK("retention finish");
    return 0;
}
