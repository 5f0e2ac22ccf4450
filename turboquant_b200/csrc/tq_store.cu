// Store path, fp32 kernel: compress a chunk of key/value vectors into pool
// block records.  One CTA handles 32 tokens of one kv head and follows the
// reference's order of operations exactly (quantizer.py:129-149,231-257,
// kv_cache.py:45-98), with the three DxD products done in fp32 FMAs with a
// fixed summation order.  This is the bit-faithful path; the tensor-core
// kernel in tq_store_tc.cu is the fast one.
#include "tq_common.cuh"

namespace {

constexpr int TM = 32;        // tokens per CTA
constexpr int LDT = TM + 4;   // row stride of the transposed [k][token] tiles
constexpr int NTHREADS = 256;

struct StoreParams {
    const void* key;
    const void* value;
    int64_t n_tokens;
    int64_t stride_token, stride_head;
    const int64_t* slot_mapping;
    const int32_t* block_table;
    int64_t start_pos;
    uint8_t* pool;
    int64_t num_blocks;
    int H;
    const float* pi;
    const float* pi_t;
    const float* s_t;
    TqCodebook cb;
    int key_bits, val_bits;
};

// C[t][c] += sum_k A[k][t] * B[k][c] for NTQ tokens x 4 columns per thread.
template <int D, int NTQ>
__device__ __forceinline__ void gemm_tile(const float* __restrict__ a_t, const float* __restrict__ b, int t_base,
                                          int col, float (&acc)[NTQ][4]) {
#pragma unroll
    for (int t = 0; t < NTQ; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[t][c] = 0.f;
    // rows of B come from L2: eight are requested before the first is used, so the loop is not
    // a chain of dependent memory latencies; the summation order over k is unchanged
    constexpr int KB = 8;
#pragma unroll 1
    for (int k0 = 0; k0 < D; k0 += KB) {
        float4 bv[KB];
#pragma unroll
        for (int kk = 0; kk < KB; ++kk) bv[kk] = __ldg(reinterpret_cast<const float4*>(b + (size_t)(k0 + kk) * D + col));
#pragma unroll
        for (int kk = 0; kk < KB; ++kk) {
            const int k = k0 + kk;
            float av[NTQ];
#pragma unroll
            for (int t4 = 0; t4 < NTQ / 4; ++t4) {
                const float4 a4 = *reinterpret_cast<const float4*>(a_t + k * LDT + t_base + 4 * t4);
                av[4 * t4 + 0] = a4.x;
                av[4 * t4 + 1] = a4.y;
                av[4 * t4 + 2] = a4.z;
                av[4 * t4 + 3] = a4.w;
            }
#pragma unroll
            for (int t = 0; t < NTQ; ++t) {
                acc[t][0] = fmaf(av[t], bv[kk].x, acc[t][0]);
                acc[t][1] = fmaf(av[t], bv[kk].y, acc[t][1]);
                acc[t][2] = fmaf(av[t], bv[kk].z, acc[t][2]);
                acc[t][3] = fmaf(av[t], bv[kk].w, acc[t][3]);
            }
        }
    }
}

// sum over k of tile[k][t]^2, fixed order: 8 partial sums of D/8 terms each.
template <int D>
__device__ __forceinline__ void column_sumsq(const float* tile, float* part, float* out, int tid) {
    const int t = tid & 31, pr = tid >> 5;
    float s = 0.f;
    for (int k = pr * (D / 8); k < (pr + 1) * (D / 8); ++k) {
        const float v = tile[k * LDT + t];
        s = fmaf(v, v, s);
    }
    part[pr * TM + t] = s;
    __syncthreads();
    if (tid < TM) {
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot += part[i * TM + tid];
        out[tid] = tot;
    }
    __syncthreads();
}

template <int D, int DT>
__global__ void __launch_bounds__(NTHREADS) tq_store_f32_kernel(const StoreParams p) {
    using E = TqElem<DT>;
    const TqLayout L = tq_make_layout(D, p.key_bits, p.val_bits);
    const int mse_bits = p.key_bits - 1;
    const int n_cent = 1 << mse_bits;
    constexpr int NTQ = TM * D / (NTHREADS * 4);  // tokens per thread in the GEMMs
    constexpr int NG = D / 32;

    extern __shared__ __align__(16) float smem[];
    float* xo = smem;                 // [D][LDT] original x (fp32), first used as value scratch
    float* xa = xo + D * LDT;         // [D][LDT] GEMM A operand: x_unit, later the residual
    float* ya = xa + D * LDT;         // [D][LDT] centroid values y_hat
    float* part = ya + D * LDT;       // [8][TM]
    float* sumsq = part + 8 * TM;     // [TM]
    float* norm_d = sumsq + TM;       // [TM] norm rounded to the input dtype
    float* den = norm_d + TM;         // [TM]
    float* rnorm = den + TM;          // [TM]
    int64_t* slot = reinterpret_cast<int64_t*>(rnorm + TM);  // [TM]

    const int tid = threadIdx.x;
    const int h = blockIdx.y;
    const int64_t t0 = (int64_t)blockIdx.x * TM;
    const int n_here = (int)min((int64_t)TM, p.n_tokens - t0);

    if (tid < TM) {
        int64_t s = -1;
        if (tid < n_here) {
            if (p.slot_mapping) {
                s = p.slot_mapping[t0 + tid];
            } else {
                const int64_t pos = p.start_pos + t0 + tid;
                s = (int64_t)p.block_table[pos >> 4] * TQ_BLOCK_TOKENS + (pos & 15);
            }
            if (s >= 0 && (s >> 4) >= p.num_blocks) s = -1;
        }
        slot[tid] = s;
    }

    // ---------------- values: per-group min/max quantisation ----------------
    {
        float* vb = xo;  // [TM][D+1]
        for (int i = tid; i < TM * D; i += NTHREADS) {
            const int t = i / D, j = i % D;
            float v = 0.f;
            if (t < n_here) v = E::load(p.value, (t0 + t) * p.stride_token + (int64_t)h * p.stride_head + j);
            vb[t * (D + 1) + j] = v;
        }
        __syncthreads();
        const float n_levels = (float)((1 << p.val_bits) - 1);
        const float min_scale = E::round(1e-10f);
        for (int item = tid; item < TM * NG; item += NTHREADS) {
            const int t = item % TM, grp = item / TM;
            const int64_t s = slot[t];
            if (s < 0) continue;
            const float* row = vb + t * (D + 1) + grp * 32;
            float vmin = row[0], vmax = row[0];
#pragma unroll 8
            for (int i = 1; i < 32; ++i) {
                vmin = fminf(vmin, row[i]);
                vmax = fmaxf(vmax, row[i]);
            }
            float scale = E::round(__fdiv_rn(E::round(vmax - vmin), n_levels));
            scale = fmaxf(scale, min_scale);
            uint8_t* rec = p.pool + ((s >> 4) * p.H + h) * (int64_t)L.block_bytes;
            const int tl = (int)(s & 15);
            reinterpret_cast<__half*>(rec + L.off_vscale)[grp * TQ_BLOCK_TOKENS + tl] = __float2half_rn(scale);
            reinterpret_cast<__half*>(rec + L.off_vzero)[grp * TQ_BLOCK_TOKENS + tl] = __float2half_rn(vmin);
            uint32_t q[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float r = rintf(E::round(__fdiv_rn(E::round(row[i] - vmin), scale)));
                q[i] = (uint32_t)fminf(fmaxf(r, 0.f), n_levels);
            }
            if (p.val_bits == 2) {
#pragma unroll
                for (int bt = 0; bt < 8; ++bt) {
                    const uint32_t byte = q[4 * bt] | (q[4 * bt + 1] << 2) | (q[4 * bt + 2] << 4) | (q[4 * bt + 3] << 6);
                    rec[L.off_vcodes + tq_vcode_native(D, 2, tl, grp * 8 + bt)] = (uint8_t)byte;
                }
            } else {
#pragma unroll
                for (int bt = 0; bt < 16; ++bt) {
                    const uint32_t byte = q[2 * bt] | (q[2 * bt + 1] << 4);
                    rec[L.off_vcodes + tq_vcode_native(D, 4, tl, grp * 16 + bt)] = (uint8_t)byte;
                }
            }
        }
        __syncthreads();
    }

    // ---------------- keys ----------------
    for (int i = tid; i < TM * D; i += NTHREADS) {
        const int t = i / D, j = i % D;
        float v = 0.f;
        if (t < n_here) v = E::load(p.key, (t0 + t) * p.stride_token + (int64_t)h * p.stride_head + j);
        xo[j * LDT + t] = v;
    }
    __syncthreads();
    column_sumsq<D>(xo, part, sumsq, tid);
    if (tid < TM) {
        const float nd = E::round(__fsqrt_rn(sumsq[tid]));  // norm in the input dtype (quantizer.py:136)
        norm_d[tid] = nd;
        den[tid] = E::round(nd + 1e-10f);                   // quantizer.py:138
    }
    __syncthreads();
    for (int i = tid; i < TM * D; i += NTHREADS) {
        const int j = i / TM, t = i % TM;
        xa[j * LDT + t] = E::round(__fdiv_rn(xo[j * LDT + t], den[t]));
    }
    __syncthreads();

    const int cq = tid % (D / 4), tg = tid / (D / 4);
    const int col = 4 * cq, t_base = tg * NTQ;
    float acc[NTQ][4];

    // y = x_unit @ Pi^T, bucket search, pack (quantizer.py:141-147)
    gemm_tile<D, NTQ>(xa, p.pi_t, t_base, col, acc);
#pragma unroll
    for (int t = 0; t < NTQ; ++t) {
        uint32_t idx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float y = acc[t][c];
            uint32_t k = 0;
            for (int bnd = 0; bnd < n_cent - 1; ++bnd) k += (p.cb.boundaries[bnd] < y) ? 1u : 0u;
            if (y != y) k = n_cent - 1;  // searchsorted orders NaN after every number
            idx[c] = k;
            ya[(col + c) * LDT + t_base + t] = p.cb.centroids[k];
        }
        const int64_t s = slot[t_base + t];
        if (s >= 0) {
            uint8_t* rec = p.pool + ((s >> 4) * p.H + h) * (int64_t)L.block_bytes;
            uint8_t* row = rec + L.off_kcodes + (int)(s & 15) * L.kcode_row;
            if (mse_bits == 2) {
                row[cq] = (uint8_t)(idx[0] | (idx[1] << 2) | (idx[2] << 4) | (idx[3] << 6));
            } else {
                row[2 * cq] = (uint8_t)(idx[0] | (idx[1] << 4));
                row[2 * cq + 1] = (uint8_t)(idx[2] | (idx[3] << 4));
            }
        }
    }
    __syncthreads();

    // x_hat = (y_hat @ Pi) * norm ; r = x - x_hat (quantizer.py:157-163,241-244)
    gemm_tile<D, NTQ>(ya, p.pi, t_base, col, acc);
#pragma unroll
    for (int t = 0; t < NTQ; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float xh = acc[t][c] * norm_d[t_base + t];
            xa[(col + c) * LDT + t_base + t] = xo[(col + c) * LDT + t_base + t] - xh;
        }
    __syncthreads();
    column_sumsq<D>(xa, part, sumsq, tid);
    if (tid < TM) rnorm[tid] = __fsqrt_rn(sumsq[tid]);

    // p = r @ S^T, sign bits (quantizer.py:248-249,214-222)
    gemm_tile<D, NTQ>(xa, p.s_t, t_base, col, acc);
#pragma unroll
    for (int t = 0; t < NTQ; ++t) {
        uint32_t nib = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) nib |= (acc[t][c] > 0.f ? 1u : 0u) << c;
        const uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 1);
        const int64_t s = slot[t_base + t];
        if (s >= 0 && (cq & 1) == 0) {
            uint8_t* rec = p.pool + ((s >> 4) * p.H + h) * (int64_t)L.block_bytes;
            rec[L.off_ksigns + (int)(s & 15) * L.ksign_row + (cq >> 1)] = (uint8_t)(nib | (other << 4));
        }
    }
    __syncthreads();
    if (tid < TM) {
        const int64_t s = slot[tid];
        if (s >= 0) {
            uint8_t* rec = p.pool + ((s >> 4) * p.H + h) * (int64_t)L.block_bytes;
            reinterpret_cast<__half*>(rec + L.off_knorm)[s & 15] = __float2half_rn(norm_d[tid]);
            reinterpret_cast<__half*>(rec + L.off_krnorm)[s & 15] = __float2half_rn(rnorm[tid]);
        }
    }
}

template <int D, int DT>
int launch_f32(const StoreParams& p, int64_t n_tokens, int n_heads, cudaStream_t st) {
    const size_t smem = (size_t)(3 * D * LDT + 8 * TM + 4 * TM) * sizeof(float) + TM * sizeof(int64_t);
    static TqSmemOptIn opt_in;
    if (tq_opt_in_smem(tq_store_f32_kernel<D, DT>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
    dim3 grid((unsigned)((n_tokens + TM - 1) / TM), (unsigned)n_heads);
    tq_store_f32_kernel<D, DT><<<grid, NTHREADS, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

}  // namespace

int tq_store_tc_launch(const tq_consts* consts, const void* key, const void* value, tq_dtype dtype, int64_t n_tokens,
                       int32_t n_heads, int64_t stride_token, int64_t stride_head, const int64_t* slot_mapping,
                       const int32_t* block_table, int64_t start_pos, const tq_pool* pool, cudaStream_t st,
                       int* handled, const TqPagedSource* paged);

extern "C" int tq_store(const tq_consts* consts, const void* key, const void* value, tq_dtype dtype, int64_t n_tokens,
                        int32_t n_heads, int64_t stride_token, int64_t stride_head, const int64_t* slot_mapping,
                        const int32_t* block_table, int64_t start_pos, const tq_pool* pool, void* stream) {
    if (!consts || !key || !value || !pool || !pool->base) return TQ_ERR_NULL;
    if (!slot_mapping && !block_table) return TQ_ERR_NULL;
    if (!consts->pi || !consts->pi_t || !consts->s_t) return TQ_ERR_NULL;
    int rc = tq_check_config(&consts->cfg);
    if (rc != TQ_OK) return rc;
    if (n_tokens < 0 || n_heads <= 0 || start_pos < 0) return TQ_ERR_SHAPE;
    if (n_heads != pool->num_kv_heads || pool->num_blocks <= 0) return TQ_ERR_SHAPE;
    if (stride_token < consts->cfg.head_dim && n_tokens > 1) return TQ_ERR_SHAPE;
    if (dtype != TQ_F32 && dtype != TQ_BF16 && dtype != TQ_F16) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)pool->base & 15) != 0) return TQ_ERR_ALIGN;
    if (n_tokens == 0) return TQ_OK;
    cudaStream_t st = (cudaStream_t)stream;

    int handled = 0;
    rc = tq_store_tc_launch(consts, key, value, dtype, n_tokens, n_heads, stride_token, stride_head, slot_mapping,
                            block_table, start_pos, pool, st, &handled, nullptr);
    if (rc != TQ_OK || handled) return rc;
    tq_note_launch(st, TQ_LAUNCH_NEUTRAL);

    StoreParams p;
    p.key = key;
    p.value = value;
    p.n_tokens = n_tokens;
    p.stride_token = stride_token;
    p.stride_head = stride_head;
    p.slot_mapping = slot_mapping;
    p.block_table = block_table;
    p.start_pos = start_pos;
    p.pool = (uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = n_heads;
    p.pi = consts->pi;
    p.pi_t = consts->pi_t;
    p.s_t = consts->s_t;
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        p.cb.centroids[i] = consts->centroids[i];
        p.cb.boundaries[i] = consts->boundaries[i];
    }
    p.key_bits = consts->cfg.key_bits;
    p.val_bits = consts->cfg.value_bits;

    const int D = consts->cfg.head_dim;
#define TQ_LAUNCH(DD, TT) return launch_f32<DD, TT>(p, n_tokens, n_heads, st)
    if (D == 128) {
        if (dtype == TQ_F32) TQ_LAUNCH(128, TQ_F32);
        if (dtype == TQ_BF16) TQ_LAUNCH(128, TQ_BF16);
        TQ_LAUNCH(128, TQ_F16);
    } else {
        if (dtype == TQ_F32) TQ_LAUNCH(256, TQ_F32);
        if (dtype == TQ_BF16) TQ_LAUNCH(256, TQ_BF16);
        TQ_LAUNCH(256, TQ_F16);
    }
#undef TQ_LAUNCH
}

extern "C" int tq_store_paged(const tq_consts* consts, const void* key_cache, const void* value_cache, tq_dtype dtype,
                              int64_t src_num_blocks, int32_t src_block_size, int32_t n_heads, int64_t stride_block,
                              int64_t stride_token, int64_t stride_head, const int32_t* src_block_table,
                              int64_t n_tokens, const int32_t* block_table, int64_t start_pos, const tq_pool* pool,
                              void* stream) {
    if (!consts || !key_cache || !value_cache || !src_block_table || !block_table || !pool || !pool->base)
        return TQ_ERR_NULL;
    int rc = tq_check_config(&consts->cfg);
    if (rc != TQ_OK) return rc;
    if (n_tokens < 0 || n_heads <= 0 || start_pos < 0 || src_num_blocks <= 0 || src_block_size <= 0) return TQ_ERR_SHAPE;
    if (n_heads != pool->num_kv_heads || pool->num_blocks <= 0) return TQ_ERR_SHAPE;
    if (stride_token < consts->cfg.head_dim || stride_block < consts->cfg.head_dim) return TQ_ERR_SHAPE;
    if (((uintptr_t)pool->base & 15) != 0) return TQ_ERR_ALIGN;
    if (n_tokens == 0) return TQ_OK;
    TqPagedSource src;
    src.table = src_block_table;
    src.num_blocks = src_num_blocks;
    src.block_size = src_block_size;
    src.stride_block = stride_block;
    int handled = 0;
    rc = tq_store_tc_launch(consts, key_cache, value_cache, dtype, n_tokens, n_heads, stride_token, stride_head, nullptr,
                            block_table, start_pos, pool, (cudaStream_t)stream, &handled, &src);
    if (rc != TQ_OK) return rc;
    return handled ? TQ_OK : TQ_ERR_UNSUPPORTED;
}
