// seq_attn.cu -- attention of a flat mixed batch (prompt portions beside single decoded tokens) over a paged f32 KV pool.
//   prep  : per-head unit-RMS q and k (no weight) and / or rotary positions (interleaved pairs, per-pair frequencies from a table, so
//           that any frequency scaling is the caller's), k and v rows stored at the token's page slot; the values may be the keys
//           as projected.  With pooling, a second kernel writes the mean key and mean value of every block of positions the step
//           completes (from the pool's rows, in position order: the result does not depend on how the prompt was cut).
//   attend: tiles of (token, query head) rows against tiles of the keys they can see (the token's own chunk and / or window, read
//           through the entry's block table, and with pooling the pooled entries of the blocks that lie wholly before the window,
//           in the same soft-max); scores, soft-max and the weighted sum in f32; optional per-head sigmoid gate.
// A row's result depends on the token's position and on its sequence's pages only; the rest of the batch changes at most how the
// keys are split among blocks (rounding).
#include "seq_common.cuh"

namespace b200seq {

__device__ __forceinline__ int64_t kv_row(const b200seq_step& st, int e, int pos, int* err) {
    const int b = pos / st.block_size;
    if (b >= st.max_blocks || pos < 0) {
        atomicOr(err, 1);
        return -1;
    }
    return (int64_t)st.block_table[(int64_t)e * st.max_blocks + b] * st.block_size + pos % st.block_size;
}

// pooled entry of block b (positions b * P .. b * P + P - 1) of a sequence: it lives in the page of the block's first position, at
// the block's rank among the blocks that start in that page
__device__ __forceinline__ int64_t pooled_row(const int32_t* bt, int bs, int P, int ppp, int b) {
    const int pg = (b * P) / bs;
    const int first = (pg * bs + P - 1) / P;
    return (int64_t)bt[pg] * ppp + (b - first);
}

// mean key and mean value of block b (positions b * P .. b * P + P - 1) from the pool's rows, summed in position order
// (columns c0, c0 + cstep, ... of the G * D key columns followed by the G * V value columns)
__device__ __forceinline__ void pool_block(const b200seq_step& st, const int32_t* bt, int b, int G, int D, int V, int P, int ppp, const float* __restrict__ kpool,
                                           const float* __restrict__ vpool, float* __restrict__ kpp, float* __restrict__ vpp, int c0, int cstep) {
    const int bs = st.block_size;
    const int64_t prow = pooled_row(bt, bs, P, ppp, b);
    const int nk = G * D, nv = G * V;
    const float inv = 1.0f / (float)P;
    for (int c = c0; c < nk + nv; c += cstep) {
        const bool isk = c < nk;
        const float* src = isk ? kpool : vpool;
        const int cc = isk ? c : c - nk, wdt = isk ? nk : nv;
        float acc = 0.f;
#pragma unroll 4
        for (int j = 0; j < P; ++j) {   // the loads do not depend on one another; the sum keeps position order
            const int pj = b * P + j;
            acc += src[((int64_t)bt[pj / bs] * bs + pj % bs) * wdt + cc];
        }
        (isk ? kpp : vpp)[prow * wdt + cc] = acc * inv;
    }
}

// grid (T), one warp per head unit: H query heads, G key heads, G value heads.  Dynamic shared memory: rot_dims floats, the (cos, sin)
// of every pair at this token's position, computed once for all heads.  fuse_pool (steps in which every entry brings one token): the
// block that stores the last position of a pooled block also writes the block's mean -- the other rows are in the pool already.
__global__ void attn_prep_kernel(float* __restrict__ proj, int64_t ld, b200seq_step st, const b200seq_attn_desc a, float* __restrict__ kpool,
                                 float* __restrict__ vpool, float* __restrict__ kpp, float* __restrict__ vpp, int fuse_pool, int* err) {
    extern __shared__ float rot_sm[];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int e = st.tok_ent[t];
    const int pos = st.tok_pos[t];
    const int64_t row = kv_row(st, e, pos, err);
    float* base = proj + (int64_t)t * ld;
    const int H = a.H, G = a.G, D = a.D, V = a.V;
    if (a.rot_dims > 0) {
        for (int i = threadIdx.x; i < (a.rot_dims >> 1); i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * a.rot_freq[i], &sn, &cs);
            rot_sm[2 * i] = cs * a.rot_scale, rot_sm[2 * i + 1] = sn * a.rot_scale;
        }
        __syncthreads();
    }
    // 16-byte form: a lane holds two whole pairs, so the rotation needs no neighbour and q turns in place without a barrier
    const bool vec4 = ((D | V | a.q_col | a.k_col | a.v_col) & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
    for (int u = wid; u < H + 2 * G; u += nw) {
        if (u < H + G) {   // q or k head: normalise, rotate
            float* p = u < H ? base + a.q_col + (int64_t)u * D : base + a.k_col + (int64_t)(u - H) * D;
            float rinv = 1.f;
            if (a.qk_eps >= 0.f) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) ss = fmaf(p[d], p[d], ss);
                ss = warp_sum(ss);
                rinv = 1.0f / sqrtf(ss / (float)D + a.qk_eps);
            }
            float* dst = u < H ? p : (row >= 0 ? kpool + (row * G + (u - H)) * D : nullptr);
            if (vec4) {
                if (dst) {
                    for (int i = lane; i < (D >> 2); i += 32) {
                        float4 v = reinterpret_cast<const float4*>(p)[i];
                        v.x *= rinv, v.y *= rinv, v.z *= rinv, v.w *= rinv;
                        const int d = 4 * i;
                        if (d < a.rot_dims) {
                            const float cs = rot_sm[d], sn = rot_sm[d + 1], x = v.x, y = v.y;
                            v.x = fmaf(x, cs, -y * sn), v.y = fmaf(y, cs, x * sn);
                        }
                        if (d + 2 < a.rot_dims) {
                            const float cs = rot_sm[d + 2], sn = rot_sm[d + 3], x = v.z, y = v.w;
                            v.z = fmaf(x, cs, -y * sn), v.w = fmaf(y, cs, x * sn);
                        }
                        reinterpret_cast<float4*>(dst)[i] = v;
                    }
                }
                continue;
            }
            for (int d0 = 0; d0 < D; d0 += 32) {   // a pair (2i, 2i + 1) lies in one pass: both are read before either is written
                const int d = d0 + lane;
                float v = 0.f;
                if (d < D) {
                    v = p[d] * rinv;
                    if (d < a.rot_dims) {
                        const float other = p[d ^ 1] * rinv;
                        const float cs = rot_sm[d & ~1], sn = rot_sm[d | 1];
                        v = (d & 1) ? fmaf(v, cs, other * sn) : fmaf(v, cs, -other * sn);
                    }
                }
                __syncwarp();
                if (d < D && dst) dst[d] = v;
            }
        } else if (row >= 0) {
            const int g = u - H - G;
            const float* p = base + a.v_col + (int64_t)g * V;
            float* dst = vpool + (row * G + g) * V;
            if (vec4) {
                for (int i = lane; i < (V >> 2); i += 32) reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(p)[i];
            } else {
                for (int d = lane; d < V; d += 32) dst[d] = p[d];
            }
        }
    }
    if (fuse_pool && a.pool > 0 && row >= 0 && (pos + 1) % a.pool == 0) {
        __syncthreads();   // this block's own k and v rows are in the pool
        const int ppp = (st.block_size + a.pool - 1) / a.pool;
        pool_block(st, st.block_table + (int64_t)e * st.max_blocks, pos / a.pool, G, D, V, a.pool, ppp, kpool, vpool, kpp, vpp, threadIdx.x, blockDim.x);
    }
}

// General form of the prep step, for layers that use what the kernel above leaves out: a bias of the projection row, an RMS norm WITH weights
// (per head, weight [D] shared by the heads, or over the whole q / k projection at once, weights [H * D] / [G * D]), rotation of halves
// (pairs (i, i + rot_dims / 2)), fewer value heads than key heads, keys and values that belong to another layer (only q is prepared).
// grid (T), 256 threads, a warp per head unit; the unit's normalised values are staged in the warp's slice of shared memory so that the
// rotation can read any partner.  Dynamic shared memory: rot_dims floats (cos, sin per pair) + 8 * Dmax (Dmax = max(D, V)) + 40.
__global__ void attn_prep_gen_kernel(float* __restrict__ proj, int64_t ld, b200seq_step st, const b200seq_attn_desc a, float* __restrict__ kpool,
                                     float* __restrict__ vpool, int Dmax, int* err) {
    extern __shared__ float gsm[];
    float* rot_sm = gsm;                       // [rot_dims / 2] cos | [rot_dims / 2] sin
    float* stage = gsm + a.rot_dims;           // [8][Dmax]
    float* red = stage + 8 * Dmax;
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int e = st.tok_ent[t], pos = st.tok_pos[t];
    const int H = a.H, G = a.G, D = a.D, V = a.V;
    const int Gv = a.vg > 0 ? a.vg : G;
    const int np = a.rot_dims >> 1;
    const int64_t row = a.kv_shared ? -1 : kv_row(st, e, pos, err);
    float* base = proj + (int64_t)t * ld;
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * a.rot_freq[i], &sn, &cs);
        rot_sm[i] = cs * a.rot_scale, rot_sm[np + i] = sn * a.rot_scale;
    }
    float rq = 1.f, rk = 1.f;
    if (a.norm_full && a.qk_eps >= 0.f) {   // one RMS over all heads of q, one over all heads of k
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
            const float v = base[a.q_col + i] + (a.in_bias ? a.in_bias[a.q_col + i] : 0.f);
            sq = fmaf(v, v, sq);
        }
        rq = 1.0f / sqrtf(block_sum(sq, red) / (float)(H * D) + a.qk_eps);
        if (!a.kv_shared) {
            for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
                const float v = base[a.k_col + i] + (a.in_bias ? a.in_bias[a.k_col + i] : 0.f);
                sk = fmaf(v, v, sk);
            }
            rk = 1.0f / sqrtf(block_sum(sk, red) / (float)(G * D) + a.qk_eps);
        }
    }
    __syncthreads();   // rot_sm
    float* hs = stage + wid * Dmax;
    const int nu = a.kv_shared ? H : H + G + Gv;
    for (int u = wid; u < nu; u += nw) {
        if (u < H + G) {
            const bool isq = u < H;
            const int hh = isq ? u : u - H;
            const int col = (isq ? a.q_col : a.k_col) + hh * D;
            const float* nw_ = isq ? a.q_norm_w : a.k_norm_w;
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) {
                const float v = base[col + d] + (a.in_bias ? a.in_bias[col + d] : 0.f);
                hs[d] = v;
                ss = fmaf(v, v, ss);
            }
            float rinv = 1.f;
            if (a.qk_eps >= 0.f) rinv = a.norm_full ? (isq ? rq : rk) : 1.0f / sqrtf(warp_sum(ss) / (float)D + a.qk_eps);
            for (int d = lane; d < D; d += 32) hs[d] = hs[d] * rinv * (nw_ ? nw_[a.norm_full ? hh * D + d : d] : 1.f);
            __syncwarp();
            float* dst = isq ? base + col : (row >= 0 ? kpool + (row * G + hh) * D : nullptr);
            if (dst) {
                for (int d = lane; d < D; d += 32) {
                    float v = hs[d];
                    if (d < a.rot_dims) {
                        int i, pd;
                        bool first;
                        if (a.rot_half) first = d < np, i = first ? d : d - np, pd = first ? d + np : d - np;
                        else first = !(d & 1), i = d >> 1, pd = d ^ 1;
                        const float cs = rot_sm[i], sn = rot_sm[np + i], o = hs[pd];
                        v = first ? fmaf(v, cs, -o * sn) : fmaf(v, cs, o * sn);
                    }
                    dst[d] = v;
                }
            }
            __syncwarp();   // hs is reused by the warp's next unit
        } else if (row >= 0) {
            const int g = u - H - G;
            const int col = a.v_col + g * V;
            float* dst = vpool + (row * Gv + g) * V;
            for (int d = lane; d < V; d += 32) dst[d] = base[col + d] + (a.in_bias ? a.in_bias[col + d] : 0.f);
        }
    }
}

// grid (T, column slices): the token that completes a block of P positions writes the block's mean key and mean value, one column per thread
__global__ void attn_pool_kernel(b200seq_step st, int G, int D, int V, int P, int ppp, const float* __restrict__ kpool, const float* __restrict__ vpool,
                                 float* __restrict__ kpp, float* __restrict__ vpp, int* err) {
    const int t = blockIdx.x;
    const int pos = st.tok_pos[t];
    if ((pos + 1) % P != 0) return;
    const int e = st.tok_ent[t];
    if (pos / st.block_size >= st.max_blocks || pos < 0) {
        if (threadIdx.x == 0) atomicOr(err, 1);
        return;
    }
    pool_block(st, st.block_table + (int64_t)e * st.max_blocks, pos / P, G, D, V, P, ppp, kpool, vpool, kpp, vpp, blockIdx.y * blockDim.x + threadIdx.x,
               gridDim.y * blockDim.x);
}

// ---- latent attention: what is cached is one low-rank latent per token plus one rotated key part shared by all heads ---------------------
// grid (T), 256 threads.  Per token: the latent c = rms_norm(kv[0 .. R)) * w and the rotated shared key part kr = rot(kv[R .. R + Rd))
// go to the token's pool row [c | kr]; every query head's rotated part goes to its place behind the (still empty) R latent-space
// columns of the attention's query row, its unrotated part leaves in the activation type for the projection into the latent space
// (scores are q_nope . (W c) = (W^T q_nope) . c: the keys never leave the latent space), and the gate logits are copied behind the heads.
// Rotation: interleaved pairs (2i, 2i + 1) over the whole rotated part, angle pos * freq[i], cos and sin times rot_scale.
// Dynamic shared memory: Rd floats (cos | sin) + 40 of reduction scratch.
struct LatentPrep {
    const float* proj;
    int64_t ldp;
    int c_col, gate_col;
    const float* q;
    int64_t ldq;
    int H, Dn, Rd, R;
    const float* norm_w;
    float eps;
    const float* freq;
    float rot_scale;
    float* kpool;
    float* Qp;
    int64_t ldQ;
    void* qn;
    int qn_dtype;
};
__global__ void latent_prep_kernel(const LatentPrep a, const b200seq_step st, int* err) {
    extern __shared__ float lsm[];
    float* cs = lsm;                 // [Rd / 2] cos, [Rd / 2] sin
    float* red = lsm + a.Rd;
    const int t = blockIdx.x, tid = threadIdx.x;
    const int e = st.tok_ent[t], pos = st.tok_pos[t];
    const int np = a.Rd >> 1, R = a.R, H = a.H, Dn = a.Dn, Rd = a.Rd;
    for (int i = tid; i < np; i += blockDim.x) {
        float sn, c;
        sincosf((float)pos * a.freq[i], &sn, &c);
        cs[i] = c * a.rot_scale, cs[np + i] = sn * a.rot_scale;
    }
    const float* kv = a.proj + (int64_t)t * a.ldp + a.c_col;
    float ss = 0.f;
    for (int i = tid; i < R; i += blockDim.x) ss = fmaf(kv[i], kv[i], ss);
    ss = block_sum(ss, red);         // its barriers also publish cs
    const float rinv = 1.0f / sqrtf(ss / (float)R + a.eps);
    const int64_t row = kv_row(st, e, pos, err);
    if (row >= 0) {
        float* dst = a.kpool + row * (R + Rd);
        for (int i = tid; i < R; i += blockDim.x) dst[i] = kv[i] * rinv * a.norm_w[i];
        for (int i = tid; i < np; i += blockDim.x) {
            const float u = kv[R + 2 * i], v = kv[R + 2 * i + 1];
            dst[R + 2 * i] = u * cs[i] - v * cs[np + i];
            dst[R + 2 * i + 1] = v * cs[i] + u * cs[np + i];
        }
    }
    const float* qr = a.q + (int64_t)t * a.ldq;
    if (!a.Qp) {   // the step attends over per-head keys: the rotated part of every query head turns in place, nothing else is needed
        float* qw = const_cast<float*>(qr);
        for (int idx = tid; idx < H * np; idx += blockDim.x) {
            const int h = idx / np, i = idx - h * np;
            float* p = qw + (int64_t)h * (Dn + Rd) + Dn + 2 * i;
            const float u = p[0], v = p[1];
            p[0] = u * cs[i] - v * cs[np + i];
            p[1] = v * cs[i] + u * cs[np + i];
        }
        return;
    }
    float* Qt = a.Qp + (int64_t)t * a.ldQ;
    for (int idx = tid; idx < H * np; idx += blockDim.x) {
        const int h = idx / np, i = idx - h * np;
        const float u = qr[(int64_t)h * (Dn + Rd) + Dn + 2 * i], v = qr[(int64_t)h * (Dn + Rd) + Dn + 2 * i + 1];
        Qt[(int64_t)h * (R + Rd) + R + 2 * i] = u * cs[i] - v * cs[np + i];
        Qt[(int64_t)h * (R + Rd) + R + 2 * i + 1] = v * cs[i] + u * cs[np + i];
    }
    for (int idx = tid; idx < H * Dn; idx += blockDim.x) {
        const int h = idx / Dn, i = idx - h * Dn;
        store_act(a.qn, a.qn_dtype, ((int64_t)t * H + h) * Dn + i, qr[(int64_t)h * (Dn + Rd) + i]);
    }
    if (a.gate_col >= 0)
        for (int h = tid; h < H; h += blockDim.x) Qt[(int64_t)H * (R + Rd) + h] = a.proj[(int64_t)t * a.ldp + a.gate_col + h];
}

// grid (rows of the gathered context): row r = the r-th (entry, position) pair, entries in order, positions 0 .. pos0 + len - 1 of each;
// copies the first R floats of the position's pool row (the latent) in the activation type
__global__ void latent_gather_kernel(const float* __restrict__ kpool, int64_t kld, const b200seq_step st, int R, void* __restrict__ out, int out_dtype, int* err) {
    int64_t r = blockIdx.x;
    int e = 0;
    for (; e < st.B; ++e) {
        const int n = st.ent_pos0[e] + st.ent_start[e + 1] - st.ent_start[e];
        if (r < n) break;
        r -= n;
    }
    if (e == st.B) return;
    const int pos = (int)r;
    const int64_t row = kv_row(st, e, pos, err);
    if (row < 0) return;
    const float* src = kpool + row * kld;
    for (int i = threadIdx.x; i < R; i += blockDim.x) store_act(out, out_dtype, (int64_t)blockIdx.x * R + i, src[i]);
}

// ---- attend -----------------------------------------------------------------------------------------------------------------------
// One block of 256 threads per (tile of consecutive tokens of one entry, kv head, block of its query heads, split of the keys).
// Its rows are (token, query head) pairs, RQ = 16 * RT of them (RT = 4: prompt portions; RT = 1: steps of few tokens); the keys the
// rows can see are walked in tiles of 64: K and V rows come through the block table into shared memory with coalesced loads, the
// scores of the tile are an f32 register-tiled product (thread (ty, tx): rows ty * RT + i, keys tx + 16 j), the soft-max is kept
// online per row (maximum and sum in f32, reduced over the 16 lanes of a row), the weights go through shared memory into the second
// product (value columns 4 tx + u + 64 j).  Key tiles are dealt round-robin to `nsplit` blocks when there are too few rows to fill
// the GPU (decode); the partial (maximum, sum, weighted values) of each split is merged by attn_merge_kernel.
constexpr int AT_KT = 64;
constexpr int AT_NT = 256;

struct AttnArgs {
    const float* qkvg;
    int64_t ld;
    const float *kpool, *vpool;
    const float *kpp, *vpp;   // pooled keys / values, pool > 0
    int pool, ppp;            // positions per pooled block; pooled entries per page
    int q_col, gate_col;
    int H, G, D, V, Rb, HB, QT, nsplit, share_kv;   // share_kv: V tiles reuse the K tile's shared memory (large heads: more blocks per SM)
    float scale;
    int chunk, window, gated;
    void* out;
    int out_dtype;
    float* part;   // [T][H][nsplit][V + 2] when nsplit > 1
    int* err;
    const float* sink;   // [H] or null: exp(sink[h]) joins the soft-max denominator of head h once; it has no key and no value
    const float* gate;   // gate logits [T][gld] (+ h)
    int64_t gld;
    int64_t kld, vld;    // floats per position in kpool / vpool (G * D and G * V, or the key row's width when the values lie inside the key rows)
    int ctx_rows;        // 1: kpool / vpool rows are the step's gathered context, entry after entry, position after position (no pages)
    int kd;              // floats of a key head that lie in kpool (at g * kd); the remaining D - kd come from krot, one part for all heads
    const float* krot;   // paged rows of krld floats (pointer already at the part's first column), or null
    int64_t krld;
    const float* head_scale;   // [H] or null: one more factor of head h's scores
    float softcap;             // > 0: score <- softcap * tanh(score / softcap)
    int keep_first;            // with a window: positions below this stay visible to all later positions
    int vdiv;                  // key head g reads value head g / vdiv
    int gate_elem;             // the gate has one logit per output element: gate[t * gld + h * V + c]
};

__device__ __forceinline__ bool attn_find_tile(const b200seq_step& st, int idx, int QT, int& e, int& t0, int& nq) {
    int acc = 0;
    for (e = 0; e < st.B; ++e) {
        const int s0 = st.ent_start[e], n = st.ent_start[e + 1] - s0;
        const int nt = (n + QT - 1) / QT;
        if (idx < acc + nt) {
            const int local = idx - acc;
            t0 = s0 + local * QT;
            nq = min(QT, n - local * QT);
            return true;
        }
        acc += nt;
    }
    return false;
}

__device__ __forceinline__ float dot4(const float4 a, const float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc), acc = fmaf(a.y, b.y, acc), acc = fmaf(a.z, b.z, acc), acc = fmaf(a.w, b.w, acc);
    return acc;
}

template <int RT, int VPT>
__global__ void __launch_bounds__(AT_NT, (VPT == 4) ? 3 : (VPT == 8 ? 2 : 1)) attn_tile_kernel(const AttnArgs a, const b200seq_step st) {
    extern __shared__ __align__(16) float sm[];
    constexpr int RQ = 16 * RT, VS = 16 * VPT, PS = AT_KT + 4;
    const int D = a.D, V = a.V, H = a.H, G = a.G;
    const int Dp = (D + 3) & ~3, QS = Dp + 4;
    float* Qs = sm;                     // [RQ][QS]
    float* Ks = Qs + RQ * QS;           // [AT_KT][QS]
    const int kv_floats = a.share_kv ? max(AT_KT * QS, AT_KT * VS) : AT_KT * QS;
    float* Vs = a.share_kv ? Ks : Ks + AT_KT * QS;   // [AT_KT][VS]
    float* Ps = a.share_kv ? Ks + kv_floats : Vs + AT_KT * VS;   // [RQ][PS]
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    int e, t0, nq;
    if (!attn_find_tile(st, blockIdx.x, a.QT, e, t0, nq)) return;
    const int g = blockIdx.y / a.HB, hb = blockIdx.y - g * a.HB;
    const int R = H / G;
    const int h0 = g * R + hb * a.Rb, nh = min(a.Rb, R - hb * a.Rb);
    const int split = blockIdx.z;
    const int p0 = st.tok_pos[t0], hi = p0 + nq - 1;
    const int bs = st.block_size;
    const int32_t* bt = st.block_table + (int64_t)e * st.max_blocks;
    if (hi / bs >= st.max_blocks || p0 < 0) {
        if (tid == 0) atomicOr(a.err, 1);
        return;
    }
    int kbeg = a.chunk > 0 ? (p0 / a.chunk) * a.chunk : 0;
    if (a.window > 0) kbeg = max(kbeg, p0 - a.window + 1);
    int64_t cstart = 0;   // first row of this entry's context in the gathered form: the contexts of the entries before it
    if (a.ctx_rows)
        for (int i = 0; i < e; ++i) cstart += st.ent_pos0[i] + st.ent_start[i + 1] - st.ent_start[i];
    // queries (zero rows where the tile has no token or the block no head)
    for (int idx = tid; idx < RQ * Dp; idx += AT_NT) {
        const int r = idx / Dp, d = idx - r * Dp;
        const int tq = r / a.Rb, hr = r - tq * a.Rb;
        Qs[r * QS + d] = (tq < nq && hr < nh && d < D) ? a.qkvg[(int64_t)(t0 + tq) * a.ld + a.q_col + (int64_t)(h0 + hr) * D + d] : 0.f;
    }
    // per-row limits of the visible keys
    int rlo[RT], rhi[RT], rnb[RT];   // visible positions [rlo, rhi]; visible pooled blocks [0, rnb)
    float m[RT], l[RT], acc[RT][VPT], rsc[RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) {
        const int r = ty * RT + i;
        const int tq = r / a.Rb, hr = r - tq * a.Rb;
        if (tq < nq && hr < nh) {
            const int p = p0 + tq;
            int lo = a.chunk > 0 ? (p / a.chunk) * a.chunk : 0;
            if (a.window > 0) lo = max(lo, p - a.window + 1);
            rlo[i] = lo, rhi[i] = p;
            rnb[i] = (a.pool > 0 && p - a.window + 1 > 0) ? (p - a.window + 1) / a.pool : 0;
            rsc[i] = a.head_scale ? a.scale * a.head_scale[h0 + hr] : a.scale;
        } else {
            rlo[i] = 1, rhi[i] = 0, rnb[i] = 0;   // sees nothing
            rsc[i] = a.scale;
        }
        m[i] = -INFINITY, l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) acc[i][j] = 0.f;
    }
    const bool vecD = ((D | a.kld | a.kd | a.krld) & 3) == 0 && (reinterpret_cast<uintptr_t>(a.krot) & 15) == 0, vecV = ((V | a.vld) & 3) == 0;
    // pooled blocks every row of the tile may see (the tile's last row sees the most), then the positions from kbeg to hi
    const int nbmax = (a.pool > 0 && hi - a.window + 1 > 0) ? (hi - a.window + 1) / a.pool : 0;
    const int npt = (nbmax + AT_KT - 1) / AT_KT;
    // kept first positions that lie before the window of the tile's first row: tiles of their own, seen by every row of the tile; those
    // inside [kbeg, hi] come with the window tiles (a later row's window may have left them behind: the row test below keeps them)
    const int keep = (a.window > 0 && a.keep_first > 0) ? a.keep_first : 0;
    const int nfirst = min(keep, kbeg);
    const int nft = (nfirst + AT_KT - 1) / AT_KT;
    const int ntiles = npt + nft + (hi - kbeg) / AT_KT + 1;
    auto load_v = [&](int k0, bool pooled, int klim) {
        const int k = tid >> 2, sub = tid & 3;
        const int kp = k0 + k;
        const bool in = pooled ? kp < nbmax : kp <= klim;
        const float* src = !in ? nullptr
                           : pooled ? a.vpp + (pooled_row(bt, bs, a.pool, a.ppp, kp) * G + g) * V
                                    : a.vpool + (a.ctx_rows ? cstart + kp : (int64_t)bt[kp / bs] * bs + kp % bs) * a.vld + (int64_t)(g / a.vdiv) * V;
        if (vecV) {
            for (int c4 = sub; c4 < (VS >> 2); c4 += 4)
                *reinterpret_cast<float4*>(Vs + k * VS + 4 * c4) = (in && 4 * c4 < V) ? *reinterpret_cast<const float4*>(src + 4 * c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int c = sub; c < VS; c += 4) Vs[k * VS + c] = (in && c < V) ? src[c] : 0.f;
        }
    };
    for (int tile = 0; tile < ntiles; ++tile) {
        if (tile % a.nsplit != split) continue;
        const bool pooled = tile < npt;
        const bool first = !pooled && tile < npt + nft;
        const int k0 = pooled ? tile * AT_KT : (first ? (tile - npt) * AT_KT : kbeg + (tile - npt - nft) * AT_KT);
        const int klim = first ? nfirst - 1 : hi;   // last position this tile may load
        __syncthreads();   // the previous tile's products are done with Ks, Vs, Ps (and Qs is written before the first)
        {   // four threads per key: the page lookup happens once per thread and tile
            const int k = tid >> 2, sub = tid & 3;
            const int kp = k0 + k;
            const bool in = pooled ? kp < nbmax : kp <= klim;
            const int64_t prow = (in && !pooled) ? (int64_t)bt[kp / bs] * bs + kp % bs : 0;
            const float* src = !in ? nullptr
                               : pooled ? a.kpp + (pooled_row(bt, bs, a.pool, a.ppp, kp) * G + g) * D
                                        : a.kpool + (a.ctx_rows ? cstart + kp : prow) * a.kld + (int64_t)g * a.kd;
            const float* src2 = (in && a.krot) ? a.krot + prow * a.krld - a.kd : src;   // dimensions kd .. D - 1 of the key, indexed by d
            const int kd = pooled ? D : a.kd;
            if (vecD) {
                for (int d4 = sub; d4 < (D >> 2); d4 += 4)
                    *reinterpret_cast<float4*>(Ks + k * QS + 4 * d4) = in ? *reinterpret_cast<const float4*>((4 * d4 < kd ? src : src2) + 4 * d4) : make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                for (int d = sub; d < Dp; d += 4) Ks[k * QS + d] = (in && d < D) ? (d < kd ? src[d] : src2[d]) : 0.f;
            }
        }
        if (!a.share_kv) load_v(k0, pooled, klim);
        __syncthreads();
        float s[RT][4];
#pragma unroll
        for (int i = 0; i < RT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        for (int d = 0; d < Dp; d += 4) {
            float4 q[RT], k[4];
#pragma unroll
            for (int i = 0; i < RT; ++i) q[i] = *reinterpret_cast<const float4*>(Qs + (ty * RT + i) * QS + d);
#pragma unroll
            for (int j = 0; j < 4; ++j) k[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * QS + d);
#pragma unroll
            for (int i = 0; i < RT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = dot4(q[i], k[j], s[i][j]);
        }
#pragma unroll
        for (int i = 0; i < RT; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kp = k0 + tx + 16 * j;
                const bool seen = pooled ? kp < rnb[i] : (first ? (kp < nfirst && rhi[i] >= rlo[i]) : ((kp >= rlo[i] || kp < keep) && kp <= rhi[i]));
                float sv = s[i][j] * rsc[i];
                if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
                s[i][j] = seen ? sv : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mn = fmaxf(m[i], mx);
            float corr = 1.f, sum = 0.f;
            if (mn != -INFINITY) {
                corr = expf(m[i] - mn);   // m = -inf before the first visible key: 0
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = s[i][j] == -INFINITY ? 0.f : expf(s[i][j] - mn);
                    sum += s[i][j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            l[i] = l[i] * corr + sum;
            m[i] = mn;
#pragma unroll
            for (int j = 0; j < VPT; ++j) acc[i][j] *= corr;
#pragma unroll
            for (int j = 0; j < 4; ++j) Ps[(ty * RT + i) * PS + tx + 16 * j] = s[i][j];
        }
        __syncthreads();
        if (a.share_kv) {   // every thread is done with the K tile: the V tile takes its place
            load_v(k0, pooled, klim);
            __syncthreads();
        }
        for (int k = 0; k < AT_KT; k += 4) {
            float4 p[RT];
#pragma unroll
            for (int i = 0; i < RT; ++i) p[i] = *reinterpret_cast<const float4*>(Ps + (ty * RT + i) * PS + k);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int jv = 0; jv < VPT / 4; ++jv) {
                    const float4 v = *reinterpret_cast<const float4*>(Vs + (k + kk) * VS + jv * 64 + tx * 4);
#pragma unroll
                    for (int i = 0; i < RT; ++i) {
                        const float pv = kk == 0 ? p[i].x : kk == 1 ? p[i].y : kk == 2 ? p[i].z : p[i].w;
                        acc[i][4 * jv] = fmaf(pv, v.x, acc[i][4 * jv]);
                        acc[i][4 * jv + 1] = fmaf(pv, v.y, acc[i][4 * jv + 1]);
                        acc[i][4 * jv + 2] = fmaf(pv, v.z, acc[i][4 * jv + 2]);
                        acc[i][4 * jv + 3] = fmaf(pv, v.w, acc[i][4 * jv + 3]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < RT; ++i) {
        const int r = ty * RT + i;
        const int tq = r / a.Rb, hr = r - tq * a.Rb;
        if (tq >= nq || hr >= nh) continue;
        const int t = t0 + tq, h = h0 + hr;
        if (a.nsplit == 1) {
            float gate = 1.f;
            if (a.gated && !a.gate_elem) gate = sigmoidf_acc(a.gate[(int64_t)t * a.gld + h]);
            float den = l[i], resc = 1.f;
            if (a.sink) {   // the sink's term, under the larger of the two maxima
                const float sk = a.sink[h], mn = fmaxf(m[i], sk);
                resc = expf(m[i] - mn);
                den = fmaf(l[i], resc, expf(sk - mn));
            }
            const float f = gate * resc / den;
#pragma unroll
            for (int jv = 0; jv < VPT / 4; ++jv)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = jv * 64 + tx * 4 + u;
                    if (c < V) {
                        const float ge = a.gate_elem ? sigmoidf_acc(a.gate[(int64_t)t * a.gld + (int64_t)h * V + c]) : 1.f;
                        store_act(a.out, a.out_dtype, ((int64_t)t * H + h) * V + c, acc[i][4 * jv + u] * f * ge);
                    }
                }
        } else {
            float* pp = a.part + (((int64_t)t * H + h) * a.nsplit + split) * (V + 2);
            if (tx == 0) pp[0] = m[i], pp[1] = l[i];
#pragma unroll
            for (int jv = 0; jv < VPT / 4; ++jv)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = jv * 64 + tx * 4 + u;
                    if (c < V) pp[2 + c] = acc[i][4 * jv + u];
                }
        }
    }
}

// grid (T, H): merges the splits of one (token, head) in split order
__global__ void attn_merge_kernel(const AttnArgs a) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int V = a.V, ns = a.nsplit;
    const float* pp = a.part + ((int64_t)t * a.H + h) * ns * (V + 2);
    float M = a.sink ? a.sink[h] : -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, pp[s * (V + 2)]);
    float L = a.sink ? expf(a.sink[h] - M) : 0.f;
    for (int s = 0; s < ns; ++s) {
        const float ms = pp[s * (V + 2)];
        if (ms != -INFINITY) L = fmaf(pp[s * (V + 2) + 1], expf(ms - M), L);
    }
    float gate = 1.f;
    if (a.gated && !a.gate_elem) gate = sigmoidf_acc(a.gate[(int64_t)t * a.gld + h]);
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        if (a.gate_elem) gate = sigmoidf_acc(a.gate[(int64_t)t * a.gld + (int64_t)h * V + c]);
        float o = 0.f;
        for (int s = 0; s < ns; ++s) {
            const float ms = pp[s * (V + 2)];
            if (ms != -INFINITY) o = fmaf(pp[s * (V + 2) + 2 + c], expf(ms - M), o);
        }
        store_act(a.out, a.out_dtype, ((int64_t)t * a.H + h) * V + c, o / L * gate);
    }
}

struct AttnPlan {
    int RT, Rb, HB, QT, tiles, nsplit;
};

// how a step of T tokens in B entries is cut; max_keys bounds the keys one token can see
static AttnPlan attn_plan(int T, int B, int H, int G, int max_keys) {
    AttnPlan p;
    const int R = H / G;
    p.RT = T > 16 ? 4 : 1;
    const int RQ = 16 * p.RT;
    p.Rb = R < RQ ? R : RQ;
    p.HB = (R + p.Rb - 1) / p.Rb;
    p.QT = RQ / p.Rb;
    p.tiles = (T + p.QT - 1) / p.QT + B;   // upper bound of the step's query tiles
    const int real = (T + p.QT - 1) / p.QT * G * p.HB;
    int ns = (2 * 148 + real - 1) / real;
    const int kt = (max_keys + AT_KT - 1) / AT_KT;
    ns = ns < kt ? ns : kt;
    p.nsplit = ns < 1 ? 1 : (ns > 32 ? 32 : ns);
    return p;
}

}  // namespace b200seq

using namespace b200seq;

static int desc_check(const b200seq_attn_desc* d, const char* what) {
    if (!d || d->H < 1 || d->G < 1 || d->H % d->G || d->D < 1 || d->V < 1 || d->q_col < 0 || d->k_col < 0 || d->v_col < 0)
        return fail(B200SEQ_ERR_INVALID_ARG, "%s: bad head counts, sizes or columns", what);
    if (!d->latent_v && d->v_col == d->k_col && d->V != d->D) return fail(B200SEQ_ERR_INVALID_ARG, "%s: values taken from the keys need V == D", what);
    if (d->latent_v && (d->G != 1 || d->V > d->D)) return fail(B200SEQ_ERR_INVALID_ARG, "%s: values inside the key rows need one key head and V <= D", what);
    if (d->kd < 0 || d->kd > d->D || ((d->kd > 0 && d->kd < d->D) != (d->krot != nullptr)) || (d->krot && (d->pool > 0 || d->krot_ld < d->D - d->kd)))
        return fail(B200SEQ_ERR_INVALID_ARG, "%s: a key part shared by all heads needs its rows, 0 < kd < D and no pooled blocks", what);
    if (d->ctx_rows && (d->pool > 0 || d->latent_v)) return fail(B200SEQ_ERR_INVALID_ARG, "%s: gathered context rows go with plain key / value rows", what);
    if (d->rot_dims < 0 || d->rot_dims > d->D || (d->rot_dims & 1) || (d->rot_dims > 0 && !d->rot_freq))
        return fail(B200SEQ_ERR_INVALID_ARG, "%s: rotary dimensions must be even, at most D, with a frequency table", what);
    if (d->pool < 0 || (d->pool > 0 && d->window < 1)) return fail(B200SEQ_ERR_INVALID_ARG, "%s: pooled blocks need a window", what);
    if (d->vg < 0 || (d->vg > 0 && (d->G % d->vg || d->pool > 0 || d->latent_v || d->v_col == d->k_col)))
        return fail(B200SEQ_ERR_INVALID_ARG, "%s: the value heads must divide the key heads (no pooled blocks, own value columns)", what);
    if (d->keep_first < 0 || (d->keep_first > 0 && (d->window < 1 || d->chunk > 0 || d->pool > 0)))
        return fail(B200SEQ_ERR_INVALID_ARG, "%s: kept first positions go with a window (no chunks, no pooled blocks)", what);
    if ((d->q_norm_w || d->k_norm_w || d->norm_full) && d->qk_eps < 0.f) return fail(B200SEQ_ERR_INVALID_ARG, "%s: norm weights need qk_eps >= 0", what);
    if (d->kv_shared && (d->pool > 0 || d->v_col == d->k_col)) return fail(B200SEQ_ERR_INVALID_ARG, "%s: shared keys / values go with plain pools", what);
    return 0;
}

extern "C" {

int b200seq_attn_prep_ex(float* proj, int64_t ld, const b200seq_step* st, const b200seq_attn_desc* d, float* kpool, float* vpool, float* kpooled, float* vpooled,
                         void* stream) {
    if (!proj || !st || !d || ((!kpool || !vpool) && !d->kv_shared)) return fail(B200SEQ_ERR_INVALID_ARG, "attn_prep: bad arguments");
    if (int rc = desc_check(d, "attn_prep")) return rc;
    if (d->pool > 0 && (!kpooled || !vpooled)) return fail(B200SEQ_ERR_INVALID_ARG, "attn_prep: pooled blocks need their pools");
    if (st->T == 0) return 0;
    if (d->q_norm_w || d->k_norm_w || d->norm_full || d->rot_half || d->in_bias || d->kv_shared || d->vg > 0) {
        if (d->pool > 0 || d->v_col == d->k_col) return fail(B200SEQ_ERR_UNSUPPORTED, "attn_prep: the general form has no pooled blocks and own value columns");
        const int Dmax = d->D > d->V ? d->D : d->V;
        const size_t smem = (size_t)(d->rot_dims + 8 * Dmax + 40) * sizeof(float);
        if (smem > 48 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "attn_prep: head size too large");
        attn_prep_gen_kernel<<<st->T, 256, smem, (cudaStream_t)stream>>>(proj, ld, *st, *d, kpool, vpool, Dmax, error_flag_dev());
        SEQ_LAUNCH_CHECK("attn_prep");
        return 0;
    }
    const int fuse_pool = d->pool > 0 && st->T == st->B;   // one token per entry: no other block of this step writes a row the mean reads
    attn_prep_kernel<<<st->T, 256, (size_t)d->rot_dims * sizeof(float), (cudaStream_t)stream>>>(proj, ld, *st, *d, kpool, vpool, kpooled, vpooled, fuse_pool,
                                                                                                 error_flag_dev());
    SEQ_LAUNCH_CHECK("attn_prep");
    if (d->pool > 0 && !fuse_pool) {
        const int ppp = (st->block_size + d->pool - 1) / d->pool;
        const int cols = d->G * (d->D + d->V);
        attn_pool_kernel<<<dim3(st->T, (cols + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*st, d->G, d->D, d->V, d->pool, ppp, kpool, vpool, kpooled, vpooled, error_flag_dev());
        SEQ_LAUNCH_CHECK("attn_pool");
    }
    return 0;
}

int b200seq_attn_prep(float* qkvg, int64_t ld, const b200seq_step* st, float* kpool, float* vpool, int H, int G, int D, int V, float qk_eps, void* stream) {
    const b200seq_attn_desc d{H, G, D, V, 0, H * D, (H + G) * D, -1, 1.f, 0, 0, 0, qk_eps, 0, nullptr, 1.f, nullptr, 0, nullptr, 0, 0, 0, 0, nullptr, 0};
    return b200seq_attn_prep_ex(qkvg, ld, st, &d, kpool, vpool, nullptr, nullptr, stream);
}

int b200seq_latent_prep(const float* proj, int64_t ldp, int c_col, int gate_col, const float* q, int64_t ldq, const b200seq_step* st, int H, int Dn, int Rd, int R,
                        const float* norm_w, float eps, const float* rot_freq, float rot_scale, float* kpool, float* Qp, int64_t ldQ, void* qn, int qn_dtype,
                        void* stream) {
    if (!proj || !q || !st || !norm_w || !kpool || ((Qp == nullptr) != (qn == nullptr)) || H < 1 || Dn < 1 || Rd < 0 || (Rd & 1) || R < 1 || c_col < 0 || (Rd > 0 && !rot_freq))
        return fail(B200SEQ_ERR_INVALID_ARG, "latent_prep: bad arguments (the rotated part has an even size)");
    if (ldq < (int64_t)H * (Dn + Rd) || (Qp && ldQ < (int64_t)H * (R + Rd) + (gate_col >= 0 ? H : 0))) return fail(B200SEQ_ERR_INVALID_ARG, "latent_prep: rows too short");
    if (Qp && qn_dtype != B200SEQ_F32 && qn_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "latent_prep: activation dtype");
    if (st->T == 0) return 0;
    const LatentPrep a{proj, ldp, c_col, gate_col, q, ldq, H, Dn, Rd, R, norm_w, eps, rot_freq, rot_scale, kpool, Qp, ldQ, qn, qn_dtype};
    latent_prep_kernel<<<st->T, 256, (size_t)(Rd + 40) * sizeof(float), (cudaStream_t)stream>>>(a, *st, error_flag_dev());
    SEQ_LAUNCH_CHECK("latent_prep");
    return 0;
}

int b200seq_latent_gather(const float* kpool, int64_t kld, const b200seq_step* st, int R, int ctx_rows, void* out, int out_dtype, void* stream) {
    if (!kpool || !st || !out || R < 1 || kld < R || ctx_rows < 0) return fail(B200SEQ_ERR_INVALID_ARG, "latent_gather: bad arguments");
    if (out_dtype != B200SEQ_F32 && out_dtype != B200SEQ_BF16) return fail(B200SEQ_ERR_INVALID_ARG, "latent_gather: output dtype");
    if (ctx_rows == 0) return 0;
    latent_gather_kernel<<<ctx_rows, R >= 256 ? 128 : 64, 0, (cudaStream_t)stream>>>(kpool, kld, *st, R, out, out_dtype, error_flag_dev());
    SEQ_LAUNCH_CHECK("latent_gather");
    return 0;
}

static int attn_max_keys(const b200seq_step* st, int chunk, int window, int pool, int keep_first = 0) {
    const int ctx = st->max_blocks * st->block_size;
    int max_keys = ctx;
    if (chunk > 0 && chunk < max_keys) max_keys = chunk;
    if (window > 0 && window < max_keys) max_keys = window;
    if (pool > 0) max_keys += ctx / pool;
    if (window > 0 && keep_first > 0) max_keys = max_keys + keep_first < ctx ? max_keys + keep_first : ctx;
    return max_keys;
}
size_t b200seq_attn_scratch_floats(int T, int B, int H, int G, int V, int max_keys) {
    if (T < 1 || B < 1 || H < 1 || G < 1 || H % G) return 0;
    const AttnPlan p = attn_plan(T, B, H, G, max_keys);
    return p.nsplit > 1 ? (size_t)T * H * p.nsplit * (V + 2) : 0;
}

int b200seq_attn_ex(const float* qkvg, int64_t ld, const b200seq_step* st, const b200seq_attn_desc* d, const float* kpool, const float* vpool,
                    const float* kpooled, const float* vpooled, void* out, int out_dtype, float* scratch, size_t scratch_floats, void* stream) {
    if (!qkvg || !st || !kpool || !out || !d || (!vpool && !d->latent_v)) return fail(B200SEQ_ERR_INVALID_ARG, "attn: bad arguments");
    if (int rc = desc_check(d, "attn")) return rc;
    if (d->V > 512) return fail(B200SEQ_ERR_INVALID_ARG, "attn: value size <= 512");
    if (d->pool > 0 && (!kpooled || !vpooled)) return fail(B200SEQ_ERR_INVALID_ARG, "attn: pooled blocks need their pools");
    if (st->T == 0) return 0;
    const int H = d->H, G = d->G, D = d->D, V = d->V, gated = d->gate_col >= 0;
    const int max_keys = attn_max_keys(st, d->chunk, d->window, d->pool, d->keep_first);
    AttnPlan p = attn_plan(st->T, st->B, H, G, max_keys);
    if (p.nsplit > 1 && (!scratch || scratch_floats < (size_t)st->T * H * p.nsplit * (V + 2))) p.nsplit = 1;
    const int ppp = d->pool > 0 ? (st->block_size + d->pool - 1) / d->pool : 0;
    AttnArgs a{qkvg, ld, kpool, vpool, kpooled, vpooled, d->pool, ppp, d->q_col, d->gate_col, H, G, D, V, p.Rb, p.HB, p.QT, p.nsplit, 0, d->scale, d->chunk, d->window,
               gated, out, out_dtype, scratch, error_flag_dev(), d->sink, d->gate ? d->gate : qkvg + (gated ? d->gate_col : 0), d->gate ? d->gate_ld : ld, d->kv_ld > 0 ? d->kv_ld : (int64_t)G * D,
               d->kv_ld > 0 ? d->kv_ld : (d->latent_v ? (int64_t)G * D : (int64_t)(d->vg > 0 ? d->vg : G) * V), d->ctx_rows, (d->kd > 0 && d->kd < D) ? d->kd : D, d->krot, d->krot_ld,
               d->head_scale, d->softcap, d->keep_first, d->vg > 0 ? G / d->vg : 1, (gated && d->gate_elem) ? 1 : 0};
    if (d->latent_v) a.vpool = kpool;
    const int VPT = V <= 64 ? 4 : (V <= 128 ? 8 : (V <= 256 ? 16 : 32));
    if (VPT == 32 && p.RT != 1) return fail(B200SEQ_ERR_UNSUPPORTED, "attn: value sizes above 256 only in steps of few tokens (one query row per thread)");
    const int RQ = 16 * p.RT, QS = ((D + 3) & ~3) + 4;
    size_t smem = ((size_t)(RQ + AT_KT) * QS + (size_t)AT_KT * 16 * VPT + (size_t)RQ * (AT_KT + 4)) * sizeof(float);
    if (smem > 72 * 1024) {   // fewer than three blocks per SM would fit: let V reuse the K tile
        a.share_kv = 1;
        const size_t kv = (size_t)AT_KT * (QS > 16 * VPT ? QS : 16 * VPT);
        smem = ((size_t)RQ * QS + kv + (size_t)RQ * (AT_KT + 4)) * sizeof(float);
    }
    if (smem > 220 * 1024) return fail(B200SEQ_ERR_UNSUPPORTED, "attn: head size too large");
    dim3 grid(p.tiles, G * p.HB, p.nsplit);
    cudaStream_t cs = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
#define ATT_LAUNCH(RT_, VPT_)                                                                                                   \
    do {                                                                                                                        \
        static size_t set_ = 0;                                                                                                 \
        if (smem > 48 * 1024 && smem > set_) {                                                                                  \
            e = cudaFuncSetAttribute(attn_tile_kernel<RT_, VPT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
            set_ = smem;                                                                                                        \
        }                                                                                                                       \
        if (e == cudaSuccess) attn_tile_kernel<RT_, VPT_><<<grid, AT_NT, smem, cs>>>(a, *st);                                   \
    } while (0)
    if (p.RT == 4) {
        if (VPT == 4) ATT_LAUNCH(4, 4);
        else if (VPT == 8) ATT_LAUNCH(4, 8);
        else ATT_LAUNCH(4, 16);
    } else {
        if (VPT == 4) ATT_LAUNCH(1, 4);
        else if (VPT == 8) ATT_LAUNCH(1, 8);
        else if (VPT == 16) ATT_LAUNCH(1, 16);
        else ATT_LAUNCH(1, 32);
    }
#undef ATT_LAUNCH
    if (e != cudaSuccess) return cuda_status(e, "attn attribute");
    SEQ_LAUNCH_CHECK("attn");
    if (p.nsplit > 1) {
        attn_merge_kernel<<<dim3(st->T, H), V <= 64 ? 64 : 128, 0, cs>>>(a);
        SEQ_LAUNCH_CHECK("attn merge");
    }
    return 0;
}

int b200seq_attn(const float* qkvg, int64_t ld, const b200seq_step* st, const float* kpool, const float* vpool, int H, int G, int D, int V, float scale,
                 int chunk, int window, int gated, void* out, int out_dtype, float* scratch, size_t scratch_floats, void* stream) {
    const b200seq_attn_desc d{H, G, D, V, 0, H * D, (H + G) * D, gated ? (H + G) * D + G * V : -1, scale, chunk, window, 0, -1.f, 0, nullptr, 1.f, nullptr, 0, nullptr, 0, 0, 0, 0, nullptr, 0};
    return b200seq_attn_ex(qkvg, ld, st, &d, kpool, vpool, nullptr, nullptr, out, out_dtype, scratch, scratch_floats, stream);
}

}  // extern "C"
