// seq_linear_tc.cu -- tensor-core path of the dense linear layer: y[M,N] (f32) = x[M,K] (bf16) . w[N,K]^T (bf16), f32 accumulation
// on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// One CTA per 128 (n) x 128 (m) output tile.  The weight tile is the MMA's A operand (TMEM lane = n), the activation tile its B
// operand (TMEM column = m), so that in the epilogue the 32 threads of a warp hold 32 consecutive n of one token: coalesced stores.
// Both operands are K-major bf16 rows in global memory; TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) brings 64-k slabs of both
// into a ring of shared-memory stages, rows and k beyond the matrices read as zero.  Warp 0 / lane 0 issues the copies, warp 1 /
// lane 0 the MMAs (4 per slab, K = 16 each); tcgen05.commit releases a stage and, after the last slab, publishes the accumulator
// to all 4 warps, which read it with tcgen05.ld.  The ring is 3 stages of 32 KB so that two CTAs share an SM and one's epilogue
// runs under the other's main loop.  The k order of every output element is fixed (ascending slabs), whatever M is.
//
// Optional epilogue EPI_GATED for a stacked gate|up weight whose rows alternate (gate j, up j): neighbouring lanes hold the pair,
// out[m][j] = act(gate, up) (clamped swish or tanh-gelu gate, seq_common.cuh) is written in the activation type and the [M, 2F]
// product never reaches memory.  EPI_PLAIN_ACT applies an activation of one argument (squared relu) to every output.
//
// Every wait is bounded: a wait that runs out sets bit 1 of the library's error flags and the CTA leaves through the common
// exit (its copies in flight are waited for, again bounded, and its tensor memory is freed).
#include <cuda.h>

#include "seq_common.cuh"

namespace b200seq {

namespace {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3;
constexpr int STAGE_BYTES = (BM + BN) * BK * 2;            // 32 KB: weight slab then activation slab
constexpr uint32_t WAIT_LIMIT = 1u << 24;                  // try_wait polls (each blocks for a while in hardware): seconds at most

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// false: the wait ran out (the caller leaves; nothing it waited for may be touched)
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
                 "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                   "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

struct TcParams {
    float* y;
    void* act_out;
    int64_t ldy, ldo;
    int M, N, K, epi, out_dtype;
    ActParams act;
    int* err;
    const int32_t* offs;   // grouped form: [E + 1] first row of every group; rows of group e use the weight rows e * N .. e * N + N - 1
    int E;
    int heads;             // per-head form (blockIdx.z = head e): every row goes through every head's weight rows e * N .., reading the columns
    int64_t ocol;          // e * K .. of its x row and writing the columns e * ocol .. of its output row
};
constexpr int EPI_NONE = 0, EPI_GATED = 1, EPI_PLAIN_ACT = 2;

__global__ void __launch_bounds__(128) linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full[STAGES], empty[STAGES], acc_full;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // token tiles vary fastest: the CTAs that run together share a few weight tiles and all activation tiles, which L2 holds, so the
    // weights cross HBM once instead of once per token tile
    const int n0 = blockIdx.y * BN;
    int m0 = blockIdx.x * BM, m_end = p.M, wrow0 = n0, xk0 = 0;
    int64_t oc0 = 0;
    if (p.heads) wrow0 = (int)blockIdx.z * p.N + n0, xk0 = (int)blockIdx.z * p.K, oc0 = (int64_t)blockIdx.z * p.ocol;
    if (p.offs) {   // grouped: blockIdx.x counts the row tiles of all groups in group order; a tile never crosses into the next group's rows
        __shared__ int grp[3];
        if (threadIdx.x == 0) {
            int acc = 0, e = 0;
            grp[2] = -1;
            for (; e < p.E; ++e) {
                const int b = p.offs[e], c = p.offs[e + 1] - b;
                const int nt = (c + BM - 1) / BM;
                if ((int)blockIdx.x < acc + nt) {
                    grp[0] = b + ((int)blockIdx.x - acc) * BM, grp[1] = b + c, grp[2] = e;
                    break;
                }
                acc += nt;
            }
        }
        __syncthreads();
        if (grp[2] < 0) return;   // more tiles were launched than the groups have (the bound does not know the group sizes)
        m0 = grp[0], m_end = grp[1], wrow0 = grp[2] * p.N + n0;
    }
    const int nk = (p.K + BK - 1) / BK;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], 1);
        mbar_init(&acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(&tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base;
    volatile int* ab = &abort_flag;

    if (warp == 0 && lane == 0) {
        int issued = 0;
        for (int kb = 0; kb < nk; ++kb, ++issued) {
            const int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait_bounded(&empty[s], ((kb / STAGES) - 1) & 1, ab)) break;
            mbar_expect_tx(&full[s], STAGE_BYTES);
            uint8_t* st = smem + (size_t)s * STAGE_BYTES;
            tma_load_2d(st, &map_w, kb * BK, wrow0, &full[s]);
            tma_load_2d(st + BN * BK * 2, &map_x, xk0 + kb * BK, m0, &full[s]);
        }
        if (*ab) {   // leave only when the copies already issued have landed (or the bounded wait gives up on them too)
            for (int kb = max(0, issued - STAGES); kb < issued; ++kb) {
                uint32_t i = 0;
                while (!mbar_try_wait(&full[kb % STAGES], (kb / STAGES) & 1) && ++i < WAIT_LIMIT) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);   // bf16 x bf16 -> f32
        bool ok = true;
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % STAGES;
            ok = mbar_wait_bounded(&full[s], (kb / STAGES) & 1, ab);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
            const uint64_t da = make_desc(sa), db = make_desc(sa + BN * BK * 2);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) tc_mma_ss(tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0 ? 1u : 0u);
            tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&acc_full);
    }
    __syncwarp();
    const bool have = mbar_wait_bounded(&acc_full, 0, ab);
    tc_fence_after();
    if (have) {
        const int n = n0 + warp * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BM; c += 16) {
            if (m0 + c >= m_end) break;          // uniform across the CTA
            uint32_t r[16];
            tc_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, r);
            tc_wait_ld();
            if (p.epi == EPI_NONE) {
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (m0 + c + j < m_end) p.y[(int64_t)(m0 + c + j) * p.ldy + oc0 + n] = __uint_as_float(r[j]);
                }
            } else if (p.epi == EPI_PLAIN_ACT) {
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (m0 + c + j < m_end) store_act(p.act_out, p.out_dtype, (int64_t)(m0 + c + j) * p.ldo + oc0 + n, act_plain(p.act.kind, __uint_as_float(r[j])));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float mine = __uint_as_float(r[j]);
                    const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                    if ((lane & 1) == 0 && n + 1 < p.N && m0 + c + j < m_end)
                        store_act(p.act_out, p.out_dtype, (int64_t)(m0 + c + j) * p.ldo + oc0 + (n >> 1), act_gated(p.act, mine, other));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) atomicOr(p.err, 2);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmem) : "memory");
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeFn>(f);
    }();
    return fn;
}

// rows x K bf16 matrix with row stride ld elements; box = 64 k x 128 rows, 128-byte swizzle, zero fill outside
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {BK, 128};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch(const void* x, int64_t ldx, const void* w, TcParams p, cudaStream_t st) {
    CUtensorMap mw, mx;
    const int64_t wrows = p.offs ? (int64_t)p.E * p.N : (p.heads ? (int64_t)p.heads * p.N : p.N);
    if (!make_map(&mw, w, wrows, p.K, p.K) || !make_map(&mx, x, p.M, p.heads ? (int64_t)p.heads * p.K : p.K, ldx))
        return fail(B200SEQ_ERR_CUDA, "linear: tensor map encoding failed");
    static bool attr_set = false;
    const int smem = STAGES * STAGE_BYTES + 1024;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_status(e, "linear tc attribute");
        attr_set = true;
    }
    p.err = error_flag_dev();
    dim3 grid((p.M + BM - 1) / BM + (p.offs ? p.E : 0), (p.N + BN - 1) / BN, p.heads ? p.heads : 1);
    linear_tc_kernel<<<grid, 128, smem, st>>>(mw, mx, p);
    SEQ_LAUNCH_CHECK("linear tc");
    return 0;
}

}  // namespace

bool linear_tc_usable(int x_dtype, int64_t ldx, int M, int N, int K, const void* x, const void* w) {
    (void)M, (void)N;
    return x_dtype == B200SEQ_BF16 && K % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           encode_fn() != nullptr;
}

int launch_linear_tc(const void* x, int64_t ldx, const void* w, int M, int N, int K, float* y, int64_t ldy, cudaStream_t st) {
    TcParams p{};
    p.y = y, p.ldy = ldy, p.M = M, p.N = N, p.K = K, p.epi = EPI_NONE;
    return launch(x, ldx, w, p, st);
}

// grouped form: rows [offs[e], offs[e + 1]) of x go through the weight w[e] ([E][N][K]); act_kind < 0: f32 product to out, else a plain activation
int launch_linear_tc_grouped(const void* x, int64_t ldx, const void* w, const int32_t* offs, int E, int rows, int N, int K, int act_kind, void* out, int out_dtype,
                             int64_t ldo, cudaStream_t st) {
    TcParams p{};
    p.M = rows, p.N = N, p.K = K, p.offs = offs, p.E = E;
    if (act_kind < 0) p.y = reinterpret_cast<float*>(out), p.ldy = ldo, p.epi = EPI_NONE;
    else p.act_out = out, p.ldo = ldo, p.out_dtype = out_dtype, p.epi = EPI_PLAIN_ACT, p.act = ActParams{act_kind, 0.f, 0.f, 0.f};
    return launch(x, ldx, w, p, st);
}

// per-head form: out[t][h * ocol + n] = sum_k x[t][h * K + k] * w[h][n][k]; act_kind < 0: f32 product, else a plain kind written in out_dtype
int launch_linear_tc_heads(const void* x, int64_t ldx, const void* w, int T, int H, int N, int K, int act_kind, void* out, int out_dtype, int64_t ldo, int64_t ocol,
                           cudaStream_t st) {
    TcParams p{};
    p.M = T, p.N = N, p.K = K, p.heads = H, p.ocol = ocol;
    if (act_kind < 0) p.y = reinterpret_cast<float*>(out), p.ldy = ldo, p.epi = EPI_NONE;
    else p.act_out = out, p.ldo = ldo, p.out_dtype = out_dtype, p.epi = EPI_PLAIN_ACT, p.act = ActParams{act_kind, 0.f, 0.f, 0.f};
    return launch(x, ldx, w, p, st);
}

// grouped form with any activation kind (gated kinds: the group's weight rows alternate gate / up, out has N / 2 columns)
int launch_linear_tc_grouped_act(const void* x, int64_t ldx, const void* w, const int32_t* offs, int E, int rows, int N, int K, const ActParams act, void* out,
                                 int out_dtype, int64_t ldo, cudaStream_t st) {
    TcParams p{};
    p.M = rows, p.N = N, p.K = K, p.offs = offs, p.E = E;
    p.act_out = out, p.ldo = ldo, p.out_dtype = out_dtype, p.epi = act_kind_gated(act.kind) ? EPI_GATED : EPI_PLAIN_ACT, p.act = act;
    return launch(x, ldx, w, p, st);
}

int launch_linear_tc_act(const void* x, int64_t ldx, const void* w, int M, int N, int K, const ActParams act, void* out, int out_dtype, int64_t ldo,
                         cudaStream_t st) {
    TcParams p{};
    p.act_out = out, p.ldo = ldo, p.out_dtype = out_dtype, p.M = M, p.N = N, p.K = K, p.epi = act_kind_gated(act.kind) ? EPI_GATED : EPI_PLAIN_ACT, p.act = act;
    return launch(x, ldx, w, p, st);
}

}  // namespace b200seq
