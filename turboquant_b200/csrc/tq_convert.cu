// Format conversion between pool block records and the reference's flat
// planes, and the dequantisation entry points (API completeness; the decode
// kernel never dequantises to memory).
#include "tq_common.cuh"

namespace {

struct ConvParams {
    uint8_t* pool;
    int64_t num_blocks;
    int H;
    const int32_t* block_table;
    int64_t n_tokens, start_pos;
    tq_planes planes;
    int D, key_bits, val_bits;
};

// One CTA per (logical block, head).  to_pool = false: gather; true: scatter.
template <bool TO_POOL>
__global__ void tq_convert_kernel(const ConvParams p) {
    const TqLayout L = tq_make_layout(p.D, p.key_bits, p.val_bits);
    const int h = blockIdx.y;
    const int64_t first_pos = p.start_pos - (p.start_pos & 15);
    const int64_t pos0 = first_pos + (int64_t)blockIdx.x * TQ_BLOCK_TOKENS;  // sequence position of token 0 of the block
    const int64_t phys = p.block_table[pos0 >> 4];
    if (phys < 0 || phys >= p.num_blocks) return;
    uint8_t* rec = p.pool + (phys * p.H + h) * (int64_t)L.block_bytes;
    const int64_t cap = p.planes.capacity;
    const int ng = L.ngroups;

    for (int tl = 0; tl < TQ_BLOCK_TOKENS; ++tl) {
        const int64_t pos = pos0 + tl;
        const int64_t n = pos - p.start_pos;  // plane row
        if (n < 0 || n >= p.n_tokens) continue;
        const int64_t row = (int64_t)h * cap + n;
        for (int i = threadIdx.x; i < L.kcode_row; i += blockDim.x) {
            uint8_t* a = rec + L.off_kcodes + tl * L.kcode_row + i;
            uint8_t* b = p.planes.mse_indices + row * L.kcode_row + i;
            if (TO_POOL) *a = *b; else *b = *a;
        }
        for (int i = threadIdx.x; i < L.ksign_row; i += blockDim.x) {
            uint8_t* a = rec + L.off_ksigns + tl * L.ksign_row + i;
            uint8_t* b = p.planes.qjl_signs + row * L.ksign_row + i;
            if (TO_POOL) *a = *b; else *b = *a;
        }
        for (int i = threadIdx.x; i < L.vcode_row; i += blockDim.x) {
            uint8_t* a = rec + L.off_vcodes + tq_vcode_native(p.D, p.val_bits, tl, i);
            uint8_t* b = p.planes.v_data + row * L.vcode_row + i;
            if (TO_POOL) *a = *b; else *b = *a;
        }
        for (int i = threadIdx.x; i < ng; i += blockDim.x) {
            uint16_t* a = reinterpret_cast<uint16_t*>(rec + L.off_vscale) + i * TQ_BLOCK_TOKENS + tl;
            uint16_t* b = p.planes.v_scales + row * ng + i;
            uint16_t* c = reinterpret_cast<uint16_t*>(rec + L.off_vzero) + i * TQ_BLOCK_TOKENS + tl;
            uint16_t* d = p.planes.v_zeros + row * ng + i;
            if (TO_POOL) { *a = *b; *c = *d; } else { *b = *a; *d = *c; }
        }
        if (threadIdx.x == 0) {
            uint16_t* a = reinterpret_cast<uint16_t*>(rec + L.off_knorm) + tl;
            uint16_t* b = p.planes.norms + row;
            uint16_t* c = reinterpret_cast<uint16_t*>(rec + L.off_krnorm) + tl;
            uint16_t* d = p.planes.residual_norms + row;
            if (TO_POOL) { *a = *b; *c = *d; } else { *b = *a; *d = *c; }
        }
    }
}

struct DequantParams {
    const uint8_t* pool;
    int64_t num_blocks;
    int H;
    const int32_t* block_table;
    int64_t n_tokens;
    const float* pi;
    const float* s;
    TqCodebook cb;
    float qjl_scale;
    int D, key_bits, val_bits, with_qjl;
    float* out;
};

// One CTA (D threads) per (block, head): k_hat = (c[idx] @ Pi) * norm + qjl_scale*rnorm*(signs @ S).
__global__ void tq_dequant_keys_kernel(const DequantParams p) {
    const TqLayout L = tq_make_layout(p.D, p.key_bits, p.val_bits);
    extern __shared__ float sm[];
    float* yh = sm;                              // [16][D]
    float* sg = sm + TQ_BLOCK_TOKENS * p.D;      // [16][D]
    const int h = blockIdx.y, j = threadIdx.x, D = p.D;
    const int64_t phys = p.block_table[blockIdx.x];
    if (phys < 0 || phys >= p.num_blocks) return;
    const uint8_t* rec = p.pool + (phys * p.H + h) * (int64_t)L.block_bytes;
    const int mse_bits = p.key_bits - 1;
    const int width = mse_bits == 2 ? 2 : 4, vpb = 8 / width;
    for (int tl = 0; tl < TQ_BLOCK_TOKENS; ++tl) {
        const uint8_t byte = rec[L.off_kcodes + tl * L.kcode_row + j / vpb];
        yh[tl * D + j] = p.cb.centroids[(byte >> ((j % vpb) * width)) & ((1 << width) - 1)];
        const uint8_t sb = rec[L.off_ksigns + tl * L.ksign_row + (j >> 3)];
        sg[tl * D + j] = ((sb >> (j & 7)) & 1) ? 1.f : -1.f;
    }
    __syncthreads();
    float am[TQ_BLOCK_TOKENS], aq[TQ_BLOCK_TOKENS];
#pragma unroll
    for (int t = 0; t < TQ_BLOCK_TOKENS; ++t) am[t] = aq[t] = 0.f;
    for (int k = 0; k < D; ++k) {
        const float pv = __ldg(p.pi + (size_t)k * D + j);
        const float sv = p.with_qjl ? __ldg(p.s + (size_t)k * D + j) : 0.f;
#pragma unroll
        for (int t = 0; t < TQ_BLOCK_TOKENS; ++t) {
            am[t] = fmaf(yh[t * D + k], pv, am[t]);
            aq[t] = fmaf(sg[t * D + k], sv, aq[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < TQ_BLOCK_TOKENS; ++t) {
        const int64_t n = (int64_t)blockIdx.x * TQ_BLOCK_TOKENS + t;
        if (n >= p.n_tokens) break;
        const float norm = __half2float(reinterpret_cast<const __half*>(rec + L.off_knorm)[t]);
        const float rn = __half2float(reinterpret_cast<const __half*>(rec + L.off_krnorm)[t]);
        float v = am[t] * norm;
        if (p.with_qjl) v += aq[t] * (p.qjl_scale * rn);
        p.out[((int64_t)h * p.n_tokens + n) * D + j] = v;
    }
}

__global__ void tq_dequant_values_kernel(const DequantParams p) {
    const TqLayout L = tq_make_layout(p.D, p.key_bits, p.val_bits);
    const int h = blockIdx.y, d = threadIdx.x, D = p.D;
    const int64_t phys = p.block_table[blockIdx.x];
    if (phys < 0 || phys >= p.num_blocks) return;
    const uint8_t* rec = p.pool + (phys * p.H + h) * (int64_t)L.block_bytes;
    const int grp = d >> 5;
    for (int tl = 0; tl < TQ_BLOCK_TOKENS; ++tl) {
        const int64_t n = (int64_t)blockIdx.x * TQ_BLOCK_TOKENS + tl;
        if (n >= p.n_tokens) break;
        uint32_t code;
        if (p.val_bits == 2) {
            code = (rec[L.off_vcodes + tq_vcode_native(D, 2, tl, d >> 2)] >> (2 * (d & 3))) & 3u;
        } else {
            code = (rec[L.off_vcodes + tq_vcode_native(D, 4, tl, d >> 1)] >> (4 * (d & 1))) & 15u;
        }
        const float sc = __half2float(reinterpret_cast<const __half*>(rec + L.off_vscale)[grp * 16 + tl]);
        const float zr = __half2float(reinterpret_cast<const __half*>(rec + L.off_vzero)[grp * 16 + tl]);
        p.out[((int64_t)h * p.n_tokens + n) * D + d] = (float)code * sc + zr;  // kv_cache.py:115
    }
}

// Bucket search + code packing of rotated vectors and sign packing of QJL
// projections, the integer stages of the store path on their own.
__global__ void tq_pack_stage_kernel(const float* __restrict__ y, const float* __restrict__ proj, int64_t n, int D,
                                     int mse_bits, TqCodebook cb, uint8_t* __restrict__ codes,
                                     uint8_t* __restrict__ signs) {
    const int64_t row = blockIdx.x;
    const int n_cent = 1 << mse_bits;
    const int width = mse_bits == 2 ? 2 : 4, vpb = 8 / width;
    const int kcode_row = D / vpb;
    for (int b = threadIdx.x; b < kcode_row; b += blockDim.x) {
        uint32_t byte = 0;
        for (int e = 0; e < vpb; ++e) {
            const float v = y[row * D + b * vpb + e];
            uint32_t k = 0;
            for (int i = 0; i < n_cent - 1; ++i) k += (cb.boundaries[i] < v) ? 1u : 0u;
            if (v != v) k = n_cent - 1;
            byte |= k << (e * width);
        }
        codes[row * kcode_row + b] = (uint8_t)byte;
    }
    for (int b = threadIdx.x; b < D / 8; b += blockDim.x) {
        uint32_t byte = 0;
        for (int e = 0; e < 8; ++e) byte |= (proj[row * D + b * 8 + e] > 0.f ? 1u : 0u) << e;
        signs[row * (D / 8) + b] = (uint8_t)byte;
    }
}

int check_planes(const tq_planes* pl) {
    if (!pl) return TQ_ERR_NULL;
    if (!pl->mse_indices || !pl->qjl_signs || !pl->norms || !pl->residual_norms || !pl->v_data || !pl->v_scales ||
        !pl->v_zeros)
        return TQ_ERR_NULL;
    if (pl->capacity <= 0) return TQ_ERR_SHAPE;
    return TQ_OK;
}

template <bool TO_POOL>
int convert(const tq_config* cfg, const tq_pool* pool, const int32_t* block_table, int64_t n_tokens,
            int64_t start_pos, const tq_planes* planes, void* stream) {
    if (!cfg || !pool || !pool->base || !block_table) return TQ_ERR_NULL;
    int rc = tq_check_config(cfg);
    if (rc != TQ_OK) return rc;
    rc = check_planes(planes);
    if (rc != TQ_OK) return rc;
    if (n_tokens < 0 || start_pos < 0 || n_tokens > planes->capacity || pool->num_kv_heads <= 0) return TQ_ERR_SHAPE;
    if (n_tokens == 0) return TQ_OK;
    ConvParams p;
    p.pool = (uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = pool->num_kv_heads;
    p.block_table = block_table;
    p.n_tokens = n_tokens;
    p.start_pos = start_pos;
    p.planes = *planes;
    p.D = cfg->head_dim;
    p.key_bits = cfg->key_bits;
    p.val_bits = cfg->value_bits;
    const int64_t first = start_pos >> 4, last = (start_pos + n_tokens - 1) >> 4;
    dim3 grid((unsigned)(last - first + 1), (unsigned)pool->num_kv_heads);
    tq_convert_kernel<TO_POOL><<<grid, 128, 0, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

}  // namespace

extern "C" int tq_pool_to_planes(const tq_config* cfg, const tq_pool* pool, const int32_t* block_table,
                                 int64_t n_tokens, const tq_planes* planes, void* stream) {
    return convert<false>(cfg, pool, block_table, n_tokens, 0, planes, stream);
}

extern "C" int tq_planes_to_pool(const tq_config* cfg, const tq_planes* planes, int64_t n_tokens,
                                 const int32_t* block_table, int64_t start_pos, const tq_pool* pool, void* stream) {
    return convert<true>(cfg, pool, block_table, n_tokens, start_pos, planes, stream);
}

extern "C" int tq_dequant_keys(const tq_consts* consts, const tq_pool* pool, const int32_t* block_table,
                               int64_t n_tokens, int32_t with_qjl, float* out, void* stream) {
    if (!consts || !pool || !pool->base || !block_table || !out || !consts->pi || !consts->s) return TQ_ERR_NULL;
    int rc = tq_check_config(&consts->cfg);
    if (rc != TQ_OK) return rc;
    if (n_tokens < 0 || pool->num_kv_heads <= 0) return TQ_ERR_SHAPE;
    if (n_tokens == 0) return TQ_OK;
    DequantParams p;
    p.pool = (const uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = pool->num_kv_heads;
    p.block_table = block_table;
    p.n_tokens = n_tokens;
    p.pi = consts->pi;
    p.s = consts->s;
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        p.cb.centroids[i] = consts->centroids[i];
        p.cb.boundaries[i] = consts->boundaries[i];
    }
    p.qjl_scale = consts->qjl_scale;
    p.D = consts->cfg.head_dim;
    p.key_bits = consts->cfg.key_bits;
    p.val_bits = consts->cfg.value_bits;
    p.with_qjl = with_qjl;
    p.out = out;
    dim3 grid((unsigned)((n_tokens + 15) / 16), (unsigned)pool->num_kv_heads);
    const size_t smem = 2 * TQ_BLOCK_TOKENS * p.D * sizeof(float);
    tq_dequant_keys_kernel<<<grid, p.D, smem, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

extern "C" int tq_dequant_values(const tq_config* cfg, const tq_pool* pool, const int32_t* block_table,
                                 int64_t n_tokens, float* out, void* stream) {
    if (!cfg || !pool || !pool->base || !block_table || !out) return TQ_ERR_NULL;
    int rc = tq_check_config(cfg);
    if (rc != TQ_OK) return rc;
    if (n_tokens < 0 || pool->num_kv_heads <= 0) return TQ_ERR_SHAPE;
    if (n_tokens == 0) return TQ_OK;
    DequantParams p = {};
    p.pool = (const uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = pool->num_kv_heads;
    p.block_table = block_table;
    p.n_tokens = n_tokens;
    p.D = cfg->head_dim;
    p.key_bits = cfg->key_bits;
    p.val_bits = cfg->value_bits;
    p.out = out;
    dim3 grid((unsigned)((n_tokens + 15) / 16), (unsigned)pool->num_kv_heads);
    tq_dequant_values_kernel<<<grid, p.D, 0, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

extern "C" int tq_pack_stage(const tq_consts* consts, const float* y, const float* projected, int64_t n_rows,
                             uint8_t* codes, uint8_t* signs, void* stream) {
    if (!consts || !y || !projected || !codes || !signs) return TQ_ERR_NULL;
    int rc = tq_check_config(&consts->cfg);
    if (rc != TQ_OK) return rc;
    if (n_rows < 0) return TQ_ERR_SHAPE;
    if (n_rows == 0) return TQ_OK;
    TqCodebook cb;
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        cb.centroids[i] = consts->centroids[i];
        cb.boundaries[i] = consts->boundaries[i];
    }
    tq_pack_stage_kernel<<<(unsigned)n_rows, 64, 0, (cudaStream_t)stream>>>(
        y, projected, n_rows, consts->cfg.head_dim, consts->cfg.key_bits - 1, cb, codes, signs);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}
