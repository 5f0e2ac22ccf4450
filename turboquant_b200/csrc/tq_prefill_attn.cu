// Causal prefill attention over a layer's own (uncompressed) K/V on the 5th-generation tensor cores:
// what the reference's no-alloc mode computes with F.scaled_dot_product_attention after repeating
// the kv heads (integration/vllm.py:150-180), for one sequence of n tokens with grouped query heads.
//
// One CTA = 128 query tokens of one query head.  It walks the key/value tiles (128 tokens) up to its
// own diagonal:
//   TMA   : Q once, K and V tiles (128-byte-swizzled boxes of 64 channels) -> shared memory
//   MMA 1 : S = Q K^T            (tcgen05, operands from shared memory, fp32 in tensor memory)
//   soft  : four threads per query row read their share of the row of S, exchange the row maximum,
//           exponentiate against a running maximum that is only moved when the true one has grown by
//           more than 2^8 (the accumulator is then rescaled in tensor memory - rare), and write the
//           probabilities back to tensor memory as a 16-bit A operand
//   MMA 2 : O += P V             (A from tensor memory; V is used as it lies, its channel dimension
//                                 contiguous: the MN-major operand form)
// and finally divides by the row sums.  K/V are read from L2 / HBM once per query head and tile; no
// score matrix ever leaves the SM.  Tensor memory: S 128 columns | P 64 | O head_dim; at head_dim 128
// S and P are doubled and Q K^T of the next tile runs under the softmax of this one.
//
// One warp issues every TMA load and MMA (one elected lane); the compute threads hand over through
// mbarriers.  Every wait is bounded; a timeout frees tensor memory and leaves a status.
#include <cuda.h>

#include "tq_common.cuh"
#include "tq_tcgen05.cuh"

using namespace tqtc;

namespace {

constexpr int PA_TOK = 128;                   // query rows and key rows per tile
constexpr int PA_BOX = PA_TOK * 128;          // one swizzled box: 128 rows x 64 channels of 16 bits
// Kernel variants.
//   AHEAD (head_dim 128): two S and two P buffers, two key/value stages: Q K^T of tile t+1 runs under the softmax
//         of tile t.
//   WIDE  (head_dim 256): O takes 256 tensor-memory columns, leaving one S and one P buffer; one key/value stage,
//         the key tile refilled as soon as S has been computed, the value tile once P V has completed.
// (Two CTAs per SM with P written over S - 256 columns and 97 KB each, serial chains covering one another - were
// measured at head_dim 128: 8 % slower than AHEAD.)
enum PaVariant { PA_AHEAD = 1, PA_WIDE = 2 };
template <int V> struct PaCols;
template <> struct PaCols<PA_AHEAD> { static constexpr uint32_t S = 0, S_STEP = 128, P = 256, P_STEP = 64, O = 384; };
template <> struct PaCols<PA_WIDE> { static constexpr uint32_t S = 0, S_STEP = 0, P = 128, P_STEP = 0, O = 256; };
constexpr int PA_TPR = 4;                          // compute threads per query row
constexpr int PA_THREADS = PA_TOK * PA_TPR + 32;   // plus the issuing warp
constexpr float PA_RESCALE_STEP = 8.f;        // log2 of the factor the running maximum may lag behind

struct PrefillParams {
    int64_t n_tokens;
    int num_q_heads, group;                   // query heads per kv head
    int n_tiles;                              // query tiles
    float scale_log2;                         // softmax scale * log2(e)
    int is_bf16;
    void* out;
    int64_t out_stride_token, out_stride_head;   // elements
};

__device__ int g_tq_prefill_status;

__device__ __forceinline__ void pa_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tq_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float pa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float pa_max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
__device__ __forceinline__ uint32_t pa_pack(float lo, float hi, bool bf16) {
    if (bf16) return pack_bf16(lo, hi);
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D, int VAR>
__global__ void __launch_bounds__(PA_THREADS, 1)
tq_prefill_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    constexpr int TPR = PA_TPR;                   // compute threads per query row
    constexpr int OC = D / TPR;               // accumulator columns per thread
    constexpr int NCOMP = PA_TOK * TPR;       // compute threads
    constexpr int SC = PA_TOK / TPR;          // columns of S per thread
    constexpr int NBOX = D / 64;              // boxes per tile
    constexpr int NST = VAR == PA_AHEAD ? 2 : 1;  // key/value stages
    constexpr bool AHEAD = VAR == PA_AHEAD;       // S of tile t+1 is issued before P V of tile t
    using Col = PaCols<VAR>;
    static_assert((VAR == PA_WIDE) == (D == 256), "head_dim 256 runs the wide variant, head_dim 128 the other");
    constexpr int TILE_BYTES = NBOX * PA_BOX;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tq_smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + TILE_BYTES;            // [NST]
    uint8_t* sV = sK + NST * TILE_BYTES;      // [NST]
    float* s_red = reinterpret_cast<float*>(sV + NST * TILE_BYTES);   // [2][TPR][128], by tile parity
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_red + 2 * TPR * PA_TOK);
    uint64_t *bar_q = bars, *bar_k = bars + 1, *bar_v = bars + 3, *bar_s = bars + 5, *bar_p = bars + 7, *bar_o = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* s_fail = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // A launch that follows in the stream (the store of the same keys and values) may begin as SMs free up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tq_smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 9; ++i) tq_mbar_init(bars + i, i == 7 ? NCOMP : 1);
        *s_fail = 0;
        tq_mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int qt = p.n_tiles - 1 - (int)blockIdx.x;      // long rows of tiles first
    const int qh = blockIdx.y, kvh = qh / p.group;
    const int q0 = qt * PA_TOK;
    const int n_kv_tiles = qt + 1;
    const uint32_t idesc_s = umma_idesc_bf16(128, false, !p.is_bf16);
    const uint32_t idesc_o = umma_idesc_bf16(D, true, !p.is_bf16);

    if (warp == NCOMP / 32) {
        // =============================== issuing warp ===============================
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
        auto wait1 = [&](uint64_t* bar, uint32_t parity) -> bool {
            uint32_t ok = 0;
            for (int i = 0; i < (1 << 20); ++i) {
                if (tq_mbar_try_wait(bar, parity)) {
                    ok = 1;
                    break;
                }
                __nanosleep(32);
                if ((i & 255) == 255 && *s_fail) break;
            }
            ok = __all_sync(0xffffffffu, ok != 0);
            if (!ok) *s_fail = 1;
            return ok != 0;
        };
        auto elected = [&]() -> bool {
            uint32_t pred;
            asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
            return pred != 0;
        };
        auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int tok0, int head) {
            if (elected()) {
                tq_mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
                for (int b = 0; b < NBOX; ++b) tma_load_3d(dst + b * PA_BOX, tm, 64 * b, head, tok0, bar);
            }
            __syncwarp();
        };
        load_tile(sQ, &tm_q, bar_q, q0, qh);
        load_tile(sK, &tm_k, bar_k, 0, kvh);
        load_tile(sV, &tm_v, bar_v, 0, kvh);
        if (AHEAD && n_kv_tiles > 1) {
            load_tile(sK + TILE_BYTES, &tm_k, bar_k + 1, PA_TOK, kvh);
            load_tile(sV + TILE_BYTES, &tm_v, bar_v + 1, PA_TOK, kvh);
        }
        bool ok = wait1(bar_q, 0);
        const uint32_t aQ = tq_smem_u32(sQ), aK = tq_smem_u32(sK), aV = tq_smem_u32(sV);
        auto issue_s = [&](int t) -> bool {   // S_t = Q K_t^T into S buffer t % 2 (head_dim 128) or the only one
            const int st = t % NST;
            if (!wait1(bar_k + st, (uint32_t)(t / NST) & 1u)) return false;
            tc_fence_after();
            if (elected()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * PA_BOX + (ks & 3) * 32;
                    umma_ss(tmem_u + Col::S + (t & 1) * Col::S_STEP, smem_desc_sw128(aQ + off),
                            smem_desc_sw128(aK + st * TILE_BYTES + off), idesc_s, ks ? 1u : 0u);
                }
                umma_commit(bar_s + (AHEAD ? (t & 1) : 0));
            }
            __syncwarp();
            return true;
        };
        auto issue_pv = [&](int t) -> bool {  // O += P_t V_t, sixteen key tokens per step
            const int st = t % NST;
            if (!wait1(bar_v + st, (uint32_t)(t / NST) & 1u)) return false;
            tc_fence_after();
            if (elected()) {
#pragma unroll
                for (int ks = 0; ks < PA_TOK / 16; ++ks)
                    umma_ts(tmem_u + Col::O, tmem_u + Col::P + (t & 1) * Col::P_STEP + ks * 8,
                            smem_desc_sw128_mn(aV + st * TILE_BYTES + ks * 2048, PA_BOX), idesc_o, (t | ks) ? 1u : 0u);
                umma_commit(bar_o);
            }
            __syncwarp();
            return true;
        };
        if (AHEAD) {
            // S_0 | S_1, PV_0 | S_2, PV_1 | ...: the tensor pipe works on S_{t+1} while the threads turn S_t
            // into P_t.  S buffer (t+1) % 2 is free because the threads passed bar_p of tile t-1; the key stage
            // of tile t is free once S_t has been computed, the value stage once P_t V_t has completed.
            ok = ok && issue_s(0);
#pragma unroll 1
            for (int t = 0; t < n_kv_tiles && ok; ++t) {
                if (t + 1 < n_kv_tiles && !(ok = issue_s(t + 1))) break;
                if (t + 2 < n_kv_tiles) {   // S_t has been computed (long ago, as a rule): its key stage is free
                    if (!(ok = wait1(bar_s + (t & 1), (uint32_t)(t >> 1) & 1u))) break;
                    load_tile(sK + (t % NST) * TILE_BYTES, &tm_k, bar_k + t % NST, (t + 2) * PA_TOK, kvh);
                }
                if (!(ok = wait1(bar_p, (uint32_t)t & 1u))) break;
                if (!(ok = issue_pv(t))) break;
                if (t + 2 < n_kv_tiles) {
                    if (!(ok = wait1(bar_o, (uint32_t)t & 1u))) break;
                    load_tile(sV + (t % NST) * TILE_BYTES, &tm_v, bar_v + t % NST, (t + 2) * PA_TOK, kvh);
                }
            }
        } else {
            // one S buffer: S_t, P_t V_t, S_{t+1} ... in tile order.  The key stage is refilled as soon as S_t has
            // been computed, the value stage once P_t V_t has completed; both loads run under the softmax.
#pragma unroll 1
            for (int t = 0; t < n_kv_tiles && ok; ++t) {
                if (!(ok = issue_s(t))) break;          // P_{t-1} V_{t-1} has completed: S (and P over it) is free
                if (t + 1 < n_kv_tiles) {
                    if (!(ok = wait1(bar_s, (uint32_t)t & 1u))) break;
                    load_tile(sK, &tm_k, bar_k, (t + 1) * PA_TOK, kvh);
                }
                if (!(ok = wait1(bar_p, (uint32_t)t & 1u))) break;
                if (!(ok = issue_pv(t))) break;
                if (t + 1 < n_kv_tiles) {
                    if (!(ok = wait1(bar_o, (uint32_t)t & 1u))) break;
                    load_tile(sV, &tm_v, bar_v, (t + 1) * PA_TOK, kvh);
                }
            }
        }
    } else {
        // =============================== compute threads ===============================
        const int row = tid & (PA_TOK - 1), part = tid >> 7;
        const uint32_t lane_base = (uint32_t)(row & ~31) << 16;
        const bool bf16 = p.is_bf16 != 0;
        auto wait_warp = [&](uint64_t* bar, uint32_t parity) -> bool {
            uint32_t ok = 1;
            if (lane == 0) {
                ok = 0;
                for (int i = 0; i < (1 << 21); ++i) {
                    if (tq_mbar_try_wait(bar, parity)) {
                        ok = 1;
                        break;
                    }
                    if (i >= 4) __nanosleep(20);
                    if ((i & 255) == 255 && *s_fail) break;
                }
                if (!ok) *s_fail = 1;
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            return ok != 0;
        };
        auto barrier_or = [&](bool flag) -> bool {   // the compute threads only
            uint32_t out;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
                "bar.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(out)
                : "r"((uint32_t)flag), "r"(NCOMP)
                : "memory");
            return out != 0;
        };
        float m_run = -INFINITY;   // the maximum the probabilities are expressed against
        float l_run = 0.f;         // this thread's share of the row sum, against m_run
        bool ok = true;
#pragma unroll 1
        for (int t = 0; t < n_kv_tiles; ++t) {
            bool bad = !wait_warp(bar_s + (AHEAD ? (t & 1) : 0), (uint32_t)(AHEAD ? t >> 1 : t) & 1u);
            tc_fence_after();
            const uint32_t col_s = Col::S + (t & 1) * Col::S_STEP, col_p = Col::P + (t & 1) * Col::P_STEP;
            // raw logits; the softmax scale (> 0, times log2 e) is applied inside the exponent's multiply-add
            float s[SC];
#pragma unroll
            for (int c = 0; c < SC / 32; ++c) {
                float v[32];
                tmem_ld32(tmem + lane_base + col_s + part * SC + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) s[c * 32 + i] = v[i];
            }
            if (t == qt) {   // the diagonal tile: a key after the query is masked
#pragma unroll
                for (int i = 0; i < SC; ++i)
                    if (part * SC + i > row) s[i] = -INFINITY;
            }
            float mx = pa_max3(s[0], s[1], s[2]);
#pragma unroll
            for (int i = 3; i + 1 < SC; i += 2) mx = pa_max3(mx, s[i], s[i + 1]);
            if ((SC & 1) == 0) mx = fmaxf(mx, s[SC - 1]);
            // two exchange buffers: with S issued a tile ahead, a fast thread may start the next tile while a
            // slow one still reads this tile's maxima; it cannot get two tiles ahead of the barrier below
            float* red = s_red + (t & 1) * TPR * PA_TOK;
            red[part * PA_TOK + row] = mx;
            if (barrier_or(bad)) {
                ok = false;
                break;
            }
#pragma unroll
            for (int q = 0; q < TPR; ++q) mx = fmaxf(mx, red[q * PA_TOK + row]);
            mx *= p.scale_log2;
            // every tile holds at least key 0 <= row unmasked, so mx is finite
            float alpha = 1.f;
            const bool move = mx > m_run + PA_RESCALE_STEP;   // also the first tile (m_run = -inf)
            if (move) {
                alpha = pa_ex2(m_run - mx);
                m_run = mx;
            }
            float sum = 0.f;
            uint32_t pk[SC / 2];
            const float neg_m = -m_run;
#pragma unroll
            for (int i = 0; i < SC / 2; ++i) {
                const float a = pa_ex2(fmaf(s[2 * i], p.scale_log2, neg_m)), b = pa_ex2(fmaf(s[2 * i + 1], p.scale_log2, neg_m));
                sum += a + b;
                pk[i] = pa_pack(a, b, bf16);
            }
            l_run = l_run * alpha + sum;
#pragma unroll
            for (int c = 0; c < SC / 32; ++c) {
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) w[i] = pk[c * 16 + i];
                tmem_st16(tmem + lane_base + col_p + part * (SC / 2) + c * 16, w);
            }
            // The accumulator may be rescaled in place once the product of the tile before has completed:
            // implied by this tile's S when the products are issued in tile order; waited for otherwise -
            // by every thread at every tile, so that each sees every phase of bar_o and a later wait on
            // its parity cannot be satisfied by an older phase.
            if (AHEAD && t > 0) {
                if (!wait_warp(bar_o, (uint32_t)(t - 1) & 1u)) *s_fail = 1;
                tc_fence_after();
            }
            if (t > 0 && __any_sync(0xffffffffu, move)) {
#pragma unroll
                for (int c = 0; c < OC / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem + lane_base + Col::O + part * OC + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= alpha;
                    tmem_st32(tmem + lane_base + Col::O + part * OC + c * 32, o);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            pa_arrive(bar_p);
        }
        if (ok) {
            bool bad = !wait_warp(bar_o, (uint32_t)(n_kv_tiles - 1) & 1u);
            tc_fence_after();
            float* red = s_red + (n_kv_tiles & 1) * TPR * PA_TOK;
            red[part * PA_TOK + row] = l_run;
            if (barrier_or(bad)) ok = false;
            if (ok) {
                float l = 0.f;
#pragma unroll
                for (int q = 0; q < TPR; ++q) l += red[q * PA_TOK + row];
                const float inv = 1.f / l;
                const int64_t tok = (int64_t)q0 + row;
#pragma unroll
                for (int c = 0; c < OC / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem + lane_base + Col::O + part * OC + c * 32, o);
                    if (tok < p.n_tokens) {
                        uint16_t* dst = static_cast<uint16_t*>(p.out) + tok * p.out_stride_token +
                                        (int64_t)qh * p.out_stride_head + part * OC + c * 32;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 w;
                            w.x = pa_pack(o[8 * i] * inv, o[8 * i + 1] * inv, bf16);
                            w.y = pa_pack(o[8 * i + 2] * inv, o[8 * i + 3] * inv, bf16);
                            w.z = pa_pack(o[8 * i + 4] * inv, o[8 * i + 5] * inv, bf16);
                            w.w = pa_pack(o[8 * i + 6] * inv, o[8 * i + 7] * inv, bf16);
                            reinterpret_cast<uint4*>(dst)[i] = w;
                        }
                    }
                }
            }
        }
        if (!ok && tid == 0) atomicCAS(&g_tq_prefill_status, 0, (int)TQ_ERR_TIMEOUT);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn pa_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// (tokens, heads, D) 16-bit elements, strides in elements, token stride >= head stride: boxes of 64
// channels x 128 tokens of one head
bool pa_rows_map(CUtensorMap* tm, const void* base, bool bf16, int D, int64_t n_tokens, int n_heads, int64_t stride_token,
                 int64_t stride_head) {
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_heads, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_token * 2};
    const cuuint32_t box[3] = {64, 1, PA_TOK};
    const cuuint32_t estr[3] = {1, 1, 1};
    return pa_encode_fn()(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                          const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int tq_prefill_attention(const void* query, const void* key, const void* value, void* out, tq_dtype dtype,
                                    int64_t n_tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                    int64_t q_stride_token, int64_t q_stride_head, int64_t kv_stride_token,
                                    int64_t kv_stride_head, int64_t out_stride_token, int64_t out_stride_head,
                                    float scale, void* stream) {
    if (!query || !key || !value || !out) return TQ_ERR_NULL;
    if (n_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return TQ_ERR_SHAPE;
    if (head_dim != 128 && head_dim != 256) return TQ_ERR_UNSUPPORTED;
    if (dtype != TQ_BF16 && dtype != TQ_F16) return TQ_ERR_UNSUPPORTED;
    if (n_tokens >= ((int64_t)1 << 31) - 256 || num_q_heads > 65535) return TQ_ERR_SHAPE;
    const int D = head_dim;
    if (((uintptr_t)query & 15) || ((uintptr_t)key & 15) || ((uintptr_t)value & 15) || ((uintptr_t)out & 15) ||
        (q_stride_token & 7) || (q_stride_head & 7) || (kv_stride_token & 7) || (kv_stride_head & 7) ||
        (out_stride_token & 7) || (out_stride_head & 7))
        return TQ_ERR_ALIGN;
    if (q_stride_head < D || kv_stride_head < D || out_stride_head < D || q_stride_token < q_stride_head ||
        kv_stride_token < kv_stride_head)
        return TQ_ERR_SHAPE;
    if (n_tokens == 0) return TQ_OK;
    if (pa_encode_fn() == nullptr) return TQ_ERR_CUDA;
    const bool bf16 = dtype == TQ_BF16;
    CUtensorMap tm_q, tm_k, tm_v;
    if (!pa_rows_map(&tm_q, query, bf16, D, n_tokens, num_q_heads, q_stride_token, q_stride_head) ||
        !pa_rows_map(&tm_k, key, bf16, D, n_tokens, num_kv_heads, kv_stride_token, kv_stride_head) ||
        !pa_rows_map(&tm_v, value, bf16, D, n_tokens, num_kv_heads, kv_stride_token, kv_stride_head))
        return TQ_ERR_SHAPE;
    PrefillParams p;
    p.n_tokens = n_tokens;
    p.num_q_heads = num_q_heads;
    p.group = num_q_heads / num_kv_heads;
    p.n_tiles = (int)((n_tokens + PA_TOK - 1) / PA_TOK);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.is_bf16 = bf16 ? 1 : 0;
    p.out = out;
    p.out_stride_token = out_stride_token;
    p.out_stride_head = out_stride_head;
    const dim3 grid((unsigned)p.n_tiles, (unsigned)num_q_heads);
    cudaStream_t st = (cudaStream_t)stream;
    tq_note_launch(st, TQ_LAUNCH_NEUTRAL);   // plain stream order for this launch; it writes neither rows nor pool
    auto smem_of = [&](int nst, int tpr) {
        return (size_t)(1 + 2 * nst) * (D / 64) * PA_BOX + (size_t)2 * tpr * PA_TOK * sizeof(float) + 11 * sizeof(uint64_t) +
               16 + 1024;
    };
    if (D == 128) {
        const size_t smem = smem_of(2, PA_TPR);
        static TqSmemOptIn opt_in;
        if (tq_opt_in_smem(tq_prefill_attn_kernel<128, PA_AHEAD>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
        tq_prefill_attn_kernel<128, PA_AHEAD><<<grid, PA_THREADS, smem, st>>>(tm_q, tm_k, tm_v, p);
    } else {
        const size_t smem = smem_of(1, PA_TPR);
        static TqSmemOptIn opt_in;
        if (tq_opt_in_smem(tq_prefill_attn_kernel<256, PA_WIDE>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
        tq_prefill_attn_kernel<256, PA_WIDE><<<grid, PA_THREADS, smem, st>>>(tm_q, tm_k, tm_v, p);
    }
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

// Status left by the prefill attention kernel since the last call (0, or TQ_ERR_TIMEOUT if a bounded wait ran
// out); reading it clears it.  Synchronises the device.
extern "C" int tq_prefill_attention_read_status(int32_t* out) {
    if (!out) return TQ_ERR_NULL;
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tq_prefill_status, sizeof(int)) != cudaSuccess) return TQ_ERR_CUDA;
    if (v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_tq_prefill_status, &zero, sizeof(int)) != cudaSuccess) return TQ_ERR_CUDA;
    }
    *out = v;
    return TQ_OK;
}
