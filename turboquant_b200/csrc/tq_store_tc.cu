// Store path on the 5th-generation tensor cores (tcgen05 + TMEM), head_dim 128,
// bf16 input.  One persistent 512-thread CTA per SM; a tile is 128 tokens of one
// kv head; four threads share a token row, each owning 32 channels from load to
// packed output:
//
//   load row -> norm, normalise (bf16, as torch does) -> operand tiles in shared memory
//   MMA 1 : Y = x_unit * Pi^T   (Pi as two bf16 limbs: exact-enough fp32 rotation)
//           E = e * Pi_hi^T     (e = x - norm*x_unit, the normalisation's rounding error)
//   read Y, E from TMEM -> bucket search + code packing; residual IN ROTATED SPACE
//           r = norm*(Y - centroid[code]) + E   (the reference's x - x_hat, rotated: no
//           un-rotation product); |r| is the residual norm; r as bf16 hi + lo limbs
//   MMA 2 : P = r * M^T, M = S * Pi^T as two bf16 limbs (hi*hi + hi*lo + lo*hi)
//   read P from TMEM -> sign bits
//   values: per-group min/max quantisation by the same thread while MMA 1 runs
//   the tile's eight 16-token block records are assembled in shared memory and
//   leave with one bulk (TMA) store each.
//
// Reference arithmetic: quantizer.py:129-149,231-257 and kv_cache.py:45-98.
// Operand tiles use the no-swizzle K-major core-matrix layout (8 rows x 16 bytes
// contiguous; LBO between the two K halves of an MMA step, SBO between 8-row
// groups).  All waits on the MMA-completion mbarriers are bounded.
#include "tq_common.cuh"

namespace {

constexpr int TC_D = 128;
constexpr int TC_TOK = 128;
constexpr int TC_THREADS = 512;
constexpr int TILE_BYTES = TC_TOK * TC_D * 2;   // one bf16 operand tile
constexpr int LBO = 128;                        // bytes between core matrices along K
constexpr int SBO = (TC_D / 8) * 128;           // bytes between 8-row groups
constexpr int TMEM_COLS = 512;
constexpr int REC_MAX = 2624;                   // largest block record at head_dim 128 (4-bit keys and values)

struct TcParams {
    const __nv_bfloat16* key;
    const __nv_bfloat16* value;
    int64_t n_tokens, stride_token, stride_head;
    const int32_t* block_table;
    int64_t start_block;   // start_pos / 16
    uint8_t* pool;
    int64_t num_blocks;
    int H;
    const __nv_bfloat16* b_mat[4];   // Pi_hi, Pi_lo, M_hi, M_lo, each (128,128) row-major [n][k]
    TqCodebook cb;
    int key_bits, val_bits;
    int64_t n_tiles;
    int* status;
};

__device__ int g_tq_store_status;   // 0 or a tq_status left by a bounded wait that ran out


__device__ __forceinline__ int core_off(int row, int k8) { return (row >> 3) * SBO + k8 * LBO + (row & 7) * 16; }

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    // start address, leading/stride byte offsets in 16-byte units, descriptor version 1, no swizzle
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(LBO >> 4) << 16) | ((uint64_t)(SBO >> 4) << 32) |
           (1ull << 46);
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N = 128, M = 128
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(IDESC), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tq_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// a / b for a caller that rounds the result to bf16 next: the product with the
// reciprocal is within 2 ulp of the quotient, which can change the bf16 rounding
// only next to a rounding tie (low half-word 0x8000); only there the exact
// division runs.  Bit-identical to rounding __fdiv_rn(a, b), at a tenth of the cost.
__device__ __forceinline__ float div_then_bf16(float a, float b, float rb) {
    float q = a * rb;
    if (((__float_as_uint(q) + 0x8004u) & 0xFFFFu) < 9u) q = __fdiv_rn(a, b);
    return q;
}
// round two floats to bf16 with one conversion; returns the packed pair and the rounded values
__device__ __forceinline__ uint32_t round_pair(float a, float b, float& ra, float& rb) {
    const uint32_t pk = pack_bf16(a, b);
    ra = __uint_as_float(pk << 16);
    rb = __uint_as_float(pk & 0xffff0000u);
    return pk;
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float (&f)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

}  // namespace

namespace {

// Asymmetric min/max quantisation of ONE 32-channel group of one value row in
// bf16 arithmetic (kv_cache.py:64-90), from the four preloaded 16-byte pieces;
// codes go to the record image in the decode kernel's byte order, scale / zero
// point group-major.
template <int VAL_BITS>
__device__ __forceinline__ void quantize_value_group(const uint4 (&raw)[4], uint8_t* rec, const TqLayout& L, int tl,
                                                     int grp) {
    constexpr uint32_t N_LEVELS = (1u << VAL_BITS) - 1u;
    const float min_scale = bf16r(1e-10f);
    float v[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float f[8];
        unpack_bf16x8(raw[c], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c * 8 + i] = f[i];
    }
    float vmin = v[0], vmax = v[0];
#pragma unroll
    for (int i = 1; i < 32; ++i) {
        vmin = fminf(vmin, v[i]);
        vmax = fmaxf(vmax, v[i]);
    }
    float scale = bf16r(__fdiv_rn(bf16r(vmax - vmin), (float)N_LEVELS));
    scale = fmaxf(scale, min_scale);
    const float rscale = __frcp_rn(scale);
    reinterpret_cast<__half*>(rec + L.off_vscale)[grp * TQ_BLOCK_TOKENS + tl] = __float2half_rn(scale);
    reinterpret_cast<__half*>(rec + L.off_vzero)[grp * TQ_BLOCK_TOKENS + tl] = __float2half_rn(vmin);
    constexpr int PER_BYTE = 8 / VAL_BITS;
#pragma unroll
    for (int bt = 0; bt < 32 / PER_BYTE; ++bt) {
        uint32_t byte = 0;
#pragma unroll
        for (int e = 0; e < PER_BYTE; e += 2) {
            float d0, d1, t0, t1;
            round_pair(v[bt * PER_BYTE + e] - vmin, v[bt * PER_BYTE + e + 1] - vmin, d0, d1);   // (v - zero) in bf16
            round_pair(div_then_bf16(d0, scale, rscale), div_then_bf16(d1, scale, rscale), t0, t1);   // / scale in bf16
            // round half to even, clamp to [0, levels]; t >= 0 because zero = min
            byte |= min(__float2uint_rn(t0), N_LEVELS) << (e * VAL_BITS);
            byte |= min(__float2uint_rn(t1), N_LEVELS) << ((e + 1) * VAL_BITS);
        }
        rec[L.off_vcodes + tq_vcode_native(TC_D, VAL_BITS, tl, grp * (32 / PER_BYTE) + bt)] = (uint8_t)byte;
    }
}

// 512 threads: thread (row = tid % 128, q = tid / 128) owns channels [32q, 32q+32) of
// token row `row` - one TMEM chunk, one value group.  Warp w reads TMEM lanes of
// quarter w % 4 = row / 32, as the hardware requires.
template <int MSE_BITS, int VAL_BITS>
__global__ void __launch_bounds__(TC_THREADS, 1) tq_store_tc_kernel(const TcParams p) {
    const TqLayout L = tq_make_layout(TC_D, MSE_BITS + 1, VAL_BITS);
    const int BB = L.block_bytes;
    constexpr int N_CENT = 1 << MSE_BITS;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sB = smem;                               // Pi_hi, Pi_lo, M_hi, M_lo operand tiles
    uint8_t* sA0 = smem + 4 * TILE_BYTES;             // x_unit, later r_hi
    uint8_t* sA1 = sA0 + TILE_BYTES;                  // e, later r_lo
    uint8_t* sRec = sA1 + TILE_BYTES;                 // image of the tile's 8 block records
    float* s_part = reinterpret_cast<float*>(sRec + 8 * REC_MAX);   // [4][128] partial sums of squares
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_part + 4 * TC_TOK);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int row = tid & (TC_TOK - 1), q = tid >> 7;

    // constant operands, once per CTA, into the core-matrix layout
#pragma unroll 1
    for (int m = 0; m < 4; ++m)
        for (int c = tid; c < TC_D * TC_D / 8; c += TC_THREADS) {
            const int n = c >> 4, k8 = c & 15;
            *reinterpret_cast<uint4*>(sB + m * TILE_BYTES + core_off(n, k8)) =
                __ldg(reinterpret_cast<const uint4*>(p.b_mat[m] + n * TC_D + k8 * 8));
        }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tq_smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        tq_mbar_init(bars + 0, 1);
        tq_mbar_init(bars + 1, 1);
        tq_mbar_fence_init();
    }
    tq_fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_y = tmem, tmem_e = tmem + 128, tmem_p = tmem + 256;
    const uint32_t lane_base = (uint32_t)(row & ~31) << 16;   // this warp's quarter of the 128 TMEM lanes
    const uint32_t aA0 = tq_smem_u32(sA0), aA1 = tq_smem_u32(sA1), aB = tq_smem_u32(sB);

    uint32_t ph0 = 0, ph1 = 0;
    bool failed = false;
    const int blk_l = row >> 4, tl = row & 15;
    uint8_t* rec = sRec + blk_l * BB;

    // this thread's 32 key channels of the NEXT tile, fetched while the current tile finishes
    uint4 knext[4];
    auto fetch_keys = [&](int64_t tile_idx) {
        const int hh = (int)(tile_idx % p.H);
        const int64_t tk = (tile_idx / p.H) * TC_TOK + row;
        const bool ok = tile_idx < p.n_tiles && tk < p.n_tokens;
        const __nv_bfloat16* src = p.key + tk * p.stride_token + (int64_t)hh * p.stride_head + q * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            knext[c] = ok ? __ldg(reinterpret_cast<const uint4*>(src + c * 8)) : make_uint4(0u, 0u, 0u, 0u);
    };
    fetch_keys(blockIdx.x);

    int tile_no = -1;
#pragma unroll 1
    for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
        ++tile_no;
        const int h = (int)(tile % p.H);
        const int64_t t0 = (tile / p.H) * TC_TOK;
        const int64_t tok = t0 + row;
        const bool valid = tok < p.n_tokens;

        // value channels of this tile: in flight while the keys are normalised
        uint4 vraw[4];
        {
            const __nv_bfloat16* vseg = p.value + tok * p.stride_token + (int64_t)h * p.stride_head + q * 32;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                vraw[c] = valid ? __ldg(reinterpret_cast<const uint4*>(vseg + c * 8)) : make_uint4(0u, 0u, 0u, 0u);
        }

        // ---------------- key row: norm, normalise, operand tiles ----------------
        float nd;
        {
            float ss = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float f[8];
                unpack_bf16x8(knext[c], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
            }
            s_part[q * TC_TOK + row] = ss;
            __syncthreads();
            ss = (s_part[row] + s_part[TC_TOK + row]) + (s_part[2 * TC_TOK + row] + s_part[3 * TC_TOK + row]);
            nd = bf16r(__fsqrt_rn(ss));              // quantizer.py:136, in the input dtype
            const float den = bf16r(nd + 1e-10f);    // quantizer.py:138
            const float rden = __frcp_rn(den);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float f[8];
                unpack_bf16x8(knext[c], f);
                uint32_t up[4], ep[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float u0, u1;
                    up[i] = round_pair(div_then_bf16(f[2 * i], den, rden), div_then_bf16(f[2 * i + 1], den, rden), u0, u1);
                    // what the bf16 normalisation lost, exact in fp32
                    ep[i] = pack_bf16(fmaf(-nd, u0, f[2 * i]), fmaf(-nd, u1, f[2 * i + 1]));
                }
                *reinterpret_cast<uint4*>(sA0 + core_off(row, q * 4 + c)) = make_uint4(up[0], up[1], up[2], up[3]);
                *reinterpret_cast<uint4*>(sA1 + core_off(row, q * 4 + c)) = make_uint4(ep[0], ep[1], ep[2], ep[3]);
            }
        }
        tq_fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks)
                umma(tmem_y, smem_desc(aA0 + ks * 2 * LBO), smem_desc(aB + 0 * TILE_BYTES + ks * 2 * LBO), ks > 0);
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks)
                umma(tmem_y, smem_desc(aA0 + ks * 2 * LBO), smem_desc(aB + 1 * TILE_BYTES + ks * 2 * LBO), 1);
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks)
                umma(tmem_e, smem_desc(aA1 + ks * 2 * LBO), smem_desc(aB + 0 * TILE_BYTES + ks * 2 * LBO), ks > 0);
            umma_commit(bars + 0);
        }

        // ---------------- values (group q of the row), while the tensor core works ----------------
        quantize_value_group<VAL_BITS>(vraw, rec, L, tl, q);

        {
            const bool ok = tq_mbar_wait_bounded(bars + 0, ph0);
            ph0 ^= 1;
            if (__syncthreads_or(!ok)) {
                failed = true;
                break;
            }
        }
        tc_fence_after();

        // ---------------- codes and rotated-space residual of channels [32q, 32q+32) ----------------
        {
            float y[32], er[32];
            tmem_ld32(tmem_y + lane_base + q * 32, y);
            tmem_ld32(tmem_e + lane_base + q * 32, er);
            uint32_t* kc = reinterpret_cast<uint32_t*>(rec + L.off_kcodes + tl * L.kcode_row);
            constexpr int WIDTH = MSE_BITS == 2 ? 2 : 4, PER_WORD = 32 / WIDTH;
            float rn2 = 0.f;
#pragma unroll
            for (int w = 0; w < 32 / PER_WORD; ++w) {
                uint32_t word = 0;
#pragma unroll
                for (int jj = 0; jj < PER_WORD; ++jj) {
                    const int j = w * PER_WORD + jj;
                    uint32_t k = 0;
#pragma unroll
                    for (int bnd = 0; bnd < N_CENT - 1; ++bnd) k += (p.cb.boundaries[bnd] < y[j]) ? 1u : 0u;
                    if (y[j] != y[j]) k = N_CENT - 1;
                    word |= k << (WIDTH * jj);       // quantizer.py:50-68
                    const float r = fmaf(nd, y[j] - p.cb.centroids[k], er[j]);
                    rn2 = fmaf(r, r, rn2);
                    y[j] = r;
                }
                kc[q * (32 / PER_WORD) + w] = word;
            }
            s_part[q * TC_TOK + row] = rn2;
            // residual as bf16 hi + lo limbs -> operand tiles of the QJL product
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float a = y[c * 8 + 2 * i], b = y[c * 8 + 2 * i + 1];
                    float ah, bh;
                    hi[i] = round_pair(a, b, ah, bh);
                    lo[i] = pack_bf16(a - ah, b - bh);
                }
                *reinterpret_cast<uint4*>(sA0 + core_off(row, q * 4 + c)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(sA1 + core_off(row, q * 4 + c)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
        tq_fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks)
                umma(tmem_p, smem_desc(aA0 + ks * 2 * LBO), smem_desc(aB + 2 * TILE_BYTES + ks * 2 * LBO), ks > 0);
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks)
                umma(tmem_p, smem_desc(aA0 + ks * 2 * LBO), smem_desc(aB + 3 * TILE_BYTES + ks * 2 * LBO), 1);
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks)
                umma(tmem_p, smem_desc(aA1 + ks * 2 * LBO), smem_desc(aB + 2 * TILE_BYTES + ks * 2 * LBO), 1);
            umma_commit(bars + 1);
        }
        fetch_keys(tile + gridDim.x);
        if (q == 0) {   // norms of the row (partials were published before the barrier above)
            const float rn2 = (s_part[row] + s_part[TC_TOK + row]) + (s_part[2 * TC_TOK + row] + s_part[3 * TC_TOK + row]);
            reinterpret_cast<__half*>(rec + L.off_knorm)[tl] = __float2half_rn(nd);
            reinterpret_cast<__half*>(rec + L.off_krnorm)[tl] = __float2half_rn(__fsqrt_rn(rn2));
        }
        {
            const bool ok = tq_mbar_wait_bounded(bars + 1, ph1);
            ph1 ^= 1;
            if (__syncthreads_or(!ok)) {
                failed = true;
                break;
            }
        }
        tc_fence_after();

        // ---------------- sign bits of channels [32q, 32q+32) (quantizer.py:214-222) ----------------
        {
            float pr[32];
            tmem_ld32(tmem_p + lane_base + q * 32, pr);
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) w |= (pr[j] > 0.f ? 1u : 0u) << j;
            reinterpret_cast<uint32_t*>(rec + L.off_ksigns + tl * L.ksign_row)[q] = w;
        }
        tq_fence_proxy_async();
        tc_fence_before();
        __syncthreads();

        // ---------------- the tile's block records leave with one bulk store each ----------------
        if (tid < 8 && t0 + tid * TQ_BLOCK_TOKENS < p.n_tokens) {
            const int64_t phys = p.block_table[p.start_block + (t0 >> 4) + tid];
            if (phys >= 0 && phys < p.num_blocks) {
                tq_bulk_s2g(p.pool + (phys * p.H + h) * (int64_t)BB, sRec + tid * BB, (uint32_t)BB);
                tq_bulk_commit();
                tq_bulk_wait_all_read();
            } else {
                atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_RANGE);
            }
        }
        __syncthreads();
        tc_fence_after();
    }
    if (failed && tid == 0) atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_TIMEOUT);
    if (tid < 8) tq_bulk_wait_all();   // the records must have landed before the CTA retires

    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

}  // namespace

// Launches the tensor-core kernel when the call fits it: head_dim 128, bf16,
// destination given as (block table, start position) with the start on a block
// boundary, 16-byte aligned rows, and the split operands present.  Otherwise
// *handled stays 0 and tq_store runs its fp32 kernel.
int tq_store_tc_launch(const tq_consts* consts, const void* key, const void* value, tq_dtype dtype, int64_t n_tokens,
                       int32_t n_heads, int64_t stride_token, int64_t stride_head, const int64_t* slot_mapping,
                       const int32_t* block_table, int64_t start_pos, const tq_pool* pool, cudaStream_t st,
                       int* handled) {
    *handled = 0;
    const tq_config& cfg = consts->cfg;
    if (cfg.head_dim != TC_D || dtype != TQ_BF16 || slot_mapping != nullptr || block_table == nullptr) return TQ_OK;
    if ((start_pos & 15) != 0) return TQ_OK;
    if (!consts->pi_limbs[0] || !consts->pi_limbs[1] || !consts->m_limbs[0] || !consts->m_limbs[1]) return TQ_OK;
    if (((uintptr_t)key & 15) || ((uintptr_t)value & 15) || (stride_token & 7) || (stride_head & 7)) return TQ_OK;
    *handled = 1;

    TcParams p;
    p.key = (const __nv_bfloat16*)key;
    p.value = (const __nv_bfloat16*)value;
    p.n_tokens = n_tokens;
    p.stride_token = stride_token;
    p.stride_head = stride_head;
    p.block_table = block_table;
    p.start_block = start_pos >> 4;
    p.pool = (uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = n_heads;
    p.b_mat[0] = (const __nv_bfloat16*)consts->pi_limbs[0];
    p.b_mat[1] = (const __nv_bfloat16*)consts->pi_limbs[1];
    p.b_mat[2] = (const __nv_bfloat16*)consts->m_limbs[0];
    p.b_mat[3] = (const __nv_bfloat16*)consts->m_limbs[1];
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        p.cb.centroids[i] = consts->centroids[i];
        p.cb.boundaries[i] = consts->boundaries[i];
    }
    p.key_bits = cfg.key_bits;
    p.val_bits = cfg.value_bits;
    p.n_tiles = ((n_tokens + TC_TOK - 1) / TC_TOK) * n_heads;
    p.status = nullptr;

    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const size_t smem = (size_t)6 * TILE_BYTES + 8 * REC_MAX + 4 * TC_TOK * sizeof(float) + 2 * sizeof(uint64_t) + 16;
    const unsigned grid = (unsigned)(p.n_tiles < sms ? p.n_tiles : sms);
    const int mse_bits = cfg.key_bits - 1;
#define TQ_TC(MB, VB)                                                                                            \
    do {                                                                                                         \
        static bool attr_set = false;                                                                            \
        if (!attr_set) {                                                                                         \
            if (cudaFuncSetAttribute(tq_store_tc_kernel<MB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                     (int)smem) != cudaSuccess)                                                  \
                return TQ_ERR_CUDA;                                                                              \
            attr_set = true;                                                                                     \
        }                                                                                                        \
        tq_store_tc_kernel<MB, VB><<<grid, TC_THREADS, smem, st>>>(p);                                           \
    } while (0)
    if (mse_bits == 2 && cfg.value_bits == 2) TQ_TC(2, 2);
    else if (mse_bits == 2) TQ_TC(2, 4);
    else if (cfg.value_bits == 2) TQ_TC(3, 2);
    else TQ_TC(3, 4);
#undef TQ_TC
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}


// Status left by the tensor-core store kernel (0, or a tq_status if a bounded
// wait ran out or a block index was out of range).  Synchronises the device.
extern "C" int tq_store_read_status(int32_t* out) {
    if (!out) return TQ_ERR_NULL;
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tq_store_status, sizeof(int)) != cudaSuccess) return TQ_ERR_CUDA;
    *out = v;
    return TQ_OK;
}
