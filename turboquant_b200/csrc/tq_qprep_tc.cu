// Query preparation for large batches on the tensor cores (head_dim 128, bf16 queries): the rotated query
// q Pi^T and the sketched query q S^T (quantizer.py:274-302 computes both per call) for 128 query vectors
// per CTA as ONE 128 x 256 x 128 product - B operand rows 0-127 are Pi, rows 128-255 are S, each as two
// bf16 limbs (the query is exact in bf16, so the product carries ~2^-17 relative error, far inside what
// the fp16 MMA fragments of the decode kernel keep).  tcgen05.mma with both operands in shared memory,
// fp32 accumulators in 256 tensor-memory columns; two threads per vector (one per half of the columns)
// write the fp32 results and the fragment words.  The fp32 FMA kernels do the same work at 1/3 of the
// CUDA cores' peak: 44 us for the 16384 queries of a 256-sequence x 64-head step.
#include <cuda.h>

#include "tq_decode_common.cuh"
#include "tq_tcgen05.cuh"

using namespace tqtc;
using namespace tqdec;

namespace {

constexpr int QT_D = 128;
constexpr int QT_VEC = 128;                       // vectors per CTA
constexpr int QT_BOX = QT_VEC * 128;              // [128 rows][64 x 16 bit], swizzled
constexpr int QT_THREADS = 2 * QT_VEC + 32;       // (vector, half of the columns) + the issuing warp
constexpr int QT_BBOX = 256 * 128;                // B operand box: 256 rows (Pi | S) x 64 channels
constexpr uint32_t QT_IDESC = umma_idesc_bf16(256);

struct QtParams {
    int64_t nvec;
    float* out;
    uint32_t* frag;
    int G, Qh, mse_bits;
    int* status;
};

__global__ void __launch_bounds__(QT_THREADS, 1)
tq_qprep_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_p0,
                   const __grid_constant__ CUtensorMap tm_p1, const __grid_constant__ CUtensorMap tm_s0,
                   const __grid_constant__ CUtensorMap tm_s1, const QtParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tq_smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = smem;                           // 2 boxes
    uint8_t* sB = sQ + 2 * QT_BOX;                // [2 limbs][2 channel boxes][256 rows]
    float* s_tr = reinterpret_cast<float*>(sB + 4 * QT_BBOX);   // [8 warps][32][33] transposition buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_tr + 8 * 32 * 33);
    uint64_t *bar_q = bars, *bar_b = bars + 1, *bar_d = bars + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile int* s_fail = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tq_smem_u32(tmem_slot)),
                     "r"(256)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        tq_mbar_init(bar_q, 1);
        tq_mbar_init(bar_b, 1);
        tq_mbar_init(bar_d, 1);
        *s_fail = 0;
        tq_mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int64_t v0 = (int64_t)blockIdx.x * QT_VEC;

    auto wait_warp = [&](uint64_t* bar) -> bool {
        uint32_t ok = 1;
        if (lane == 0) {
            ok = 0;
            for (int i = 0; i < (1 << 20); ++i) {
                if (tq_mbar_try_wait(bar, 0)) {
                    ok = 1;
                    break;
                }
                if (i >= 4) __nanosleep(32);
                if ((i & 255) == 255 && *s_fail) break;
            }
            if (!ok) *s_fail = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        __syncwarp();
        return ok != 0;
    };

    if (warp == 2 * QT_VEC / 32) {
        // ---- issuing warp: the constant operands at once, the queries after the launch ahead has completed ----
        uint32_t leader;
        asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
        if (leader) {
            tq_mbar_expect_tx(bar_b, 4 * QT_BBOX);
            const CUtensorMap* tp[2] = {&tm_p0, &tm_p1};
            const CUtensorMap* ts[2] = {&tm_s0, &tm_s1};
#pragma unroll
            for (int l = 0; l < 2; ++l)
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
                    uint8_t* dst = sB + (l * 2 + kb) * QT_BBOX;
                    tma_load_2d(dst, tp[l], 64 * kb, 0, bar_b);                 // rows 0-127: Pi
                    tma_load_2d(dst + QT_BBOX / 2, ts[l], 64 * kb, 0, bar_b);   // rows 128-255: S
                }
        }
        __syncwarp();
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the queries may come from the kernel ahead
        if (leader) {
            tq_mbar_expect_tx(bar_q, 2 * QT_BOX);
            tma_load_2d(sQ, &tm_q, 0, (int)v0, bar_q);
            tma_load_2d(sQ + QT_BOX, &tm_q, 64, (int)v0, bar_q);
        }
        __syncwarp();
        bool ok = wait_warp(bar_b) && wait_warp(bar_q);
        tc_fence_after();
        if (ok && leader) {
            const uint32_t aQ = tq_smem_u32(sQ), aB = tq_smem_u32(sB);
#pragma unroll
            for (int l = 0; l < 2; ++l)
#pragma unroll
                for (int ks = 0; ks < QT_D / 16; ++ks) {
                    const uint32_t koff = (ks & 3) * 32;
                    umma_ss(tmem, smem_desc_sw128(aQ + (ks >> 2) * QT_BOX + koff),
                            smem_desc_sw128(aB + (l * 2 + (ks >> 2)) * QT_BBOX + koff), QT_IDESC, (l | ks) ? 1u : 0u);
                }
            umma_commit(bar_d);
        }
        __syncwarp();
    } else {
        // ---- thread (vector row, which): columns [128 * which, +128) of [q Pi^T | q S^T] ----
        const int row = tid & (QT_VEC - 1), which = tid >> 7;
        const uint32_t lane_base = (uint32_t)(row & ~31) << 16;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // results and fragments are read by the launch ahead
        bool ok = wait_warp(bar_q);
        // squared norm of the vector: the fragments' power-of-two scale is derived from it alone
        float qn2 = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint4 w = lds_sw128(sQ + (c >> 3) * QT_BOX, row, c & 7);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = bf_lo(ww[i]), b = bf_hi(ww[i]);
                qn2 = fmaf(a, a, qn2);
                qn2 = fmaf(b, b, qn2);
            }
        }
        ok = wait_warp(bar_d) && ok;
        tc_fence_after();
        const int64_t vec = v0 + row;
        const bool live = vec < p.nvec;          // tensor-memory loads are warp-wide: only the stores are guarded
        if (ok) {
            // all 128 columns of this thread's half row; a chunk of 32 is one quarter of the head dimension
            // (fragment index tig)
            float v[4][32];
#pragma unroll
            for (int tig = 0; tig < 4; ++tig) tmem_ld32(tmem + lane_base + which * QT_D + tig * 32, v[tig]);
            if (live && p.frag != nullptr) {
                const int qh = (int)(vec % p.Qh), g = qh % p.G;
                const int64_t pair = (vec / p.Qh) * (p.Qh / p.G) + qh / p.G;     // (sequence, kv head)
                const bool split = p.G > 4 || p.mse_bits == 3;                   // separate rotated / sketched fragment sets
                uint32_t* base = p.frag + pair * qf_words(QT_D, split ? 8 : 4);
                const float bound = sqrtf(qn2) * (which ? 2.f * sqrtf((float)QT_D) : 1.f);
                int e = 0;
                if (bound > 0.f && bound < 3.0e38f) e = max(-100, min(100, 14 - ilogbf(bound)));
                reinterpret_cast<float*>(base)[which * 8 + g] = (float)e;
                const bool nibble = p.mse_bits == 3 && which == 0;
                const int gid = split ? g : g + 4 * which;
                const int set = split ? which : 0;
                // one 16-byte store per fragment row: the four quarters' words of this (vector, position) are
                // adjacent, and the eight query heads of a kv head fill the 128-byte row
#pragma unroll
                for (int r = 0; r < 16; ++r) {   // element layout as in tq_qprep_kernel
                    const int wi = r >> 3, jf = r & 7;
                    const int c0 = nibble ? 2 * r : wi * 16 + jf, c1 = nibble ? 2 * r + 1 : wi * 16 + 8 + jf;
                    const int sh = nibble ? 0 : (which ? sign_pos(sign_bit(wi, jf)) : 2 * code_pos(jf));
                    const float scale = __int_as_float((127 + e - sh) << 23);
                    uint32_t w[4];
#pragma unroll
                    for (int tig = 0; tig < 4; ++tig) {
                        const __half2 h2 = __floats2half2_rn(v[tig][c0] * scale, v[tig][c1] * scale);
                        w[tig] = *reinterpret_cast<const uint32_t*>(&h2);
                    }
                    *reinterpret_cast<uint4*>(base + QF_HDR + (set * (QT_D / 8) + r) * 32 + gid * 4) =
                        make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            // fp32 results: transposed through shared memory, a warp's 32 rows one after the other, so that
            // every store instruction writes 128 consecutive bytes of one row (rows past the end are skipped)
            float* tbuf = s_tr + warp * (32 * 33);
            const int64_t row0 = v0 + (row & ~31);
#pragma unroll
            for (int tig = 0; tig < 4; ++tig) {
#pragma unroll
                for (int i = 0; i < 32; ++i) tbuf[lane * 33 + i] = v[tig][i];
                __syncwarp();
#pragma unroll 4
                for (int r = 0; r < 32; ++r)
                    if (row0 + r < p.nvec) p.out[((row0 + r) * 2 + which) * QT_D + tig * 32 + lane] = tbuf[r * 33 + lane];
                __syncwarp();
            }
        }
        if (!ok && lane == 0) atomicCAS(p.status, 0, (int)TQ_ERR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn qt_encode_fn() {
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

// (rows, 128) bf16 row-major: boxes of 64 columns x 128 rows, 128-byte swizzle
bool qt_map(CUtensorMap* tm, const void* base, int64_t rows) {
    const cuuint64_t dims[2] = {QT_D, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {QT_D * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t estr[2] = {1, 1};
    return qt_encode_fn()(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Runs the tensor-core query preparation when the call fits it (head_dim 128, contiguous bf16 queries,
// the split operands present); otherwise *handled stays 0 and the caller takes its fp32 kernels.
int tq_qprep_tc_launch(const tq_consts* consts, const void* q, int dt, int64_t nvec, float* out, uint32_t* frag, int G,
                       int Qh, int mse_bits, int* status, cudaStream_t st, int* handled) {
    *handled = 0;
    if (consts->cfg.head_dim != QT_D || dt != TQ_BF16 || nvec < 1024 || nvec >= ((int64_t)1 << 31) - 256) return TQ_OK;
    if (!consts->pi_limbs[0] || !consts->pi_limbs[1] || !consts->s_limbs[0] || !consts->s_limbs[1]) return TQ_OK;
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 15) || qt_encode_fn() == nullptr) return TQ_OK;
    CUtensorMap tm_q, tm_p[2], tm_s[2];
    if (!qt_map(&tm_q, q, nvec)) return TQ_OK;
    for (int l = 0; l < 2; ++l)
        if (((uintptr_t)consts->pi_limbs[l] & 15) || ((uintptr_t)consts->s_limbs[l] & 15) ||
            !qt_map(&tm_p[l], consts->pi_limbs[l], QT_D) || !qt_map(&tm_s[l], consts->s_limbs[l], QT_D))
            return TQ_OK;
    QtParams p;
    p.nvec = nvec;
    p.out = out;
    p.frag = frag;
    p.G = G;
    p.Qh = Qh;
    p.mse_bits = mse_bits;
    p.status = status;
    const size_t smem = 2 * (size_t)QT_BOX + 4 * (size_t)QT_BBOX + 8 * 32 * 33 * sizeof(float) + 3 * sizeof(uint64_t) + 16 + 1024;
    static TqSmemOptIn opt_in;
    if (tq_opt_in_smem(tq_qprep_tc_kernel, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // operand loads run under the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tq_pdl_for_decode(st);   // behind a store that is still writing the pool: plain stream order
    tq_note_launch(st, TQ_LAUNCH_DECODE);
    cfg.stream = st;
    cfg.gridDim = dim3((unsigned)((nvec + QT_VEC - 1) / QT_VEC));
    cfg.blockDim = dim3(QT_THREADS);
    cfg.dynamicSmemBytes = smem;
    *handled = 1;
    return cudaLaunchKernelEx(&cfg, tq_qprep_tc_kernel, tm_q, tm_p[0], tm_p[1], tm_s[0], tm_s[1], p) == cudaSuccess
               ? TQ_OK
               : TQ_ERR_CUDA;
}
