// Read path: query preparation, split-sequence decode attention over pool
// block records plus the exact ring, and the unscaled score kernel.
//
// Algebra (reference triton_kernels.py:49-53,138 and quantizer.py:274-302):
//   <q, k_hat> = norm * <q Pi^T, centroid[idx]> + qjl_scale * rnorm * <q S^T, signs>
// so the query is rotated once and the keys are never dequantised.
//
// One CTA owns one (sequence, kv head, split): it streams its share of the
// sequence's block records through shared memory with bulk (TMA) copies on a
// 3-stage mbarrier ring, keeps an online softmax for all G query heads of the
// kv head and accumulates the dequantised values.  Extra CTAs do the same for
// the exact ring tokens.  Every CTA writes a partial (m, l, acc); the last one
// to finish for a (sequence, kv head) - found with an atomic ticket, no
// waiting - merges the partials and writes the output.
#include <mutex>

#include "tq_decode_common.cuh"

using namespace tqdec;

namespace {

// q_rot = q @ Pi^T and q_sketch = q @ S^T.  One CTA = 32 output columns of one
// matrix for up to 4 query vectors; 8 warps split the contraction.  Besides the
// fp32 result it can emit the fp16 MMA fragments of the tensor-core decode
// kernel directly: every entry is scaled by a power of two derived from the
// query's norm alone (|q Pi^T|_inf <= |q|_2 and |q S^T|_inf <= 2 sqrt(D) |q|_2
// for a Gaussian S), so no CTA needs another CTA's columns.
// Optional extra job of the query-prep launch: append one new exact token per
// sequence to the ring (capture.py:219-228 does this with tensor slicing).
struct RingAppend {
    const void* new_k;     // (B, H, D) in the ring's dtype; nullptr = nothing to append
    const void* new_v;
    void* ring_k;
    void* ring_v;
    int32_t* ring_lens;    // position of the new token; incremented
    int elem_bytes, B, H, capacity;
    int64_t stride_seq, stride_token;   // in elements
    int early_inputs;   // query and new token come from host memory that no earlier kernel writes:
                        // read them before waiting for the kernel ahead (their latency hides under it)
};

// VPC = query vectors per CTA; OCC = CTAs per SM the registers are budgeted for (2 for a grid that is resident
// all at once - fewer CTAs share an SM for the latency-critical part after the wait - 3 for throughput).
template <int D, int VPC, int OCC>
__global__ void __launch_bounds__(256, OCC) tq_qprep_kernel(const void* __restrict__ q, int dt, int64_t nvec,
                                                       const float* __restrict__ pi_t,
                                                       const float* __restrict__ s_t, float* __restrict__ out,
                                                       uint32_t* __restrict__ frag, int G, int Qh, int mse_bits,
                                                       const RingAppend ap, int groups) {
    // the decode kernel may start its set-up now; it waits for this grid before it reads our output
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float qsm[VPC * D];          // queries
    __shared__ float red[8 * VPC * 32];     // partial sums
    __shared__ float qn2[VPC];              // squared norms
    // A CTA takes `groups` consecutive groups of VPC vectors against the matrix slice it holds in
    // registers (large batches: the slice is fetched once per CTA, not once per four vectors).
    int64_t v0 = (int64_t)blockIdx.y * groups * VPC;
    int nv = (int)min((int64_t)VPC, nvec - v0);
    constexpr int chunks = D / 32;
    const int which = blockIdx.x / chunks;            // 0: Pi^T, 1: S^T
    const int chunk = blockIdx.x % chunks;
    const int lane = threadIdx.x & 31, ks = threadIdx.x >> 5;
    const int col = chunk * 32 + lane;
    const float* __restrict__ m = which ? s_t : pi_t;
    // the matrix slice does not depend on the query: request it first, the query arrives meanwhile
    const int k0 = ks * (D / 8);
    float mv[D / 8];
#pragma unroll
    for (int k = 0; k < D / 8; ++k) mv[k] = __ldg(m + (size_t)(k0 + k) * D + col);
    // This grid may itself have been started before the kernel ahead of it in the stream finished
    // (programmatic dependent launch): the query and the ring belong to that kernel until the wait -
    // unless they are host buffers nobody on the device writes, which are then fetched first.
    const bool do_append = ap.new_k != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    const int row_bytes = D * ap.elem_bytes, chunks_per_row = row_bytes / 16;
    const int n_app = do_append ? ap.B * ap.H * chunks_per_row : 0;
    uint4 ak = make_uint4(0u, 0u, 0u, 0u), av = ak;   // first append chunk of this thread, when fetched early
    float qv[VPC * D / 256];
    if (ap.early_inputs) {
#pragma unroll
        for (int u = 0; u < VPC * D / 256; ++u) {
            const int i = threadIdx.x + u * 256, v = i / D;
            qv[u] = v < nv ? tq_load_any(q, (v0 + v) * D + (i % D), dt) : 0.f;
        }
        if ((int)threadIdx.x < n_app) {
            const int i = threadIdx.x;
            const int c = i % chunks_per_row, h = (i / chunks_per_row) % ap.H, b = i / (chunks_per_row * ap.H);
            const int64_t src = ((int64_t)(b * ap.H + h) * D) * ap.elem_bytes;
            ak = *reinterpret_cast<const uint4*>((const char*)ap.new_k + src + c * 16);
            av = *reinterpret_cast<const uint4*>((const char*)ap.new_v + src + c * 16);
        }
    }
    // Two passes over the same instructions.  The first is a rehearsal that runs while this grid would
    // otherwise sit waiting for the kernel ahead of it: it computes on whatever the query buffer holds
    // and stores nothing outside shared memory, but it pulls the code of the second pass - which is on
    // the critical path of every decode step - into the instruction cache.
    // (only a grid small enough to be resident all at once rehearses: a larger one has no idle wait to fill)
#pragma unroll 1
    for (int pass = (gridDim.x * gridDim.y <= 256u) ? 0 : 1; pass < 2; ++pass) {
    const bool live = pass == 1;
    if (live) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    if (do_append && live) {
        for (int i = threadIdx.x; i < n_app; i += 256) {
            const int c = i % chunks_per_row, h = (i / chunks_per_row) % ap.H, b = i / (chunks_per_row * ap.H);
            const int pos = ap.ring_lens[b];
            if (pos < 0 || pos >= ap.capacity) continue;
            const int64_t dst = ((int64_t)b * ap.stride_seq + (int64_t)pos * ap.stride_token + (int64_t)h * D) * ap.elem_bytes;
            const int64_t src = ((int64_t)(b * ap.H + h) * D) * ap.elem_bytes;
            const bool early = ap.early_inputs && i == (int)threadIdx.x;
            *reinterpret_cast<uint4*>((char*)ap.ring_k + dst + c * 16) =
                early ? ak : *reinterpret_cast<const uint4*>((const char*)ap.new_k + src + c * 16);
            *reinterpret_cast<uint4*>((char*)ap.ring_v + dst + c * 16) =
                early ? av : *reinterpret_cast<const uint4*>((const char*)ap.new_v + src + c * 16);
        }
        __syncthreads();
        for (int b = threadIdx.x; b < ap.B; b += 256)
            if (ap.ring_lens[b] >= 0 && ap.ring_lens[b] < ap.capacity) ap.ring_lens[b] += 1;
    }
#pragma unroll 1
    for (int gi = 0; gi < groups && v0 < nvec; ++gi, v0 += VPC, nv = (int)min((int64_t)VPC, nvec - v0)) {
    if (ap.early_inputs) {
#pragma unroll
        for (int u = 0; u < VPC * D / 256; ++u) qsm[threadIdx.x + u * 256] = qv[u];
    } else {
        // before the wait the query still belongs to the kernel ahead: the rehearsal computes on zeros
        for (int i = threadIdx.x; i < VPC * D; i += 256) {
            const int v = i / D;
            qsm[i] = (live && v < nv) ? tq_load_any(q, (v0 + v) * D + (i % D), dt) : 0.f;
        }
    }
    __syncthreads();
    if (ks < VPC) {
        float s2 = 0.f;
        for (int j = lane; j < D; j += 32) s2 = fmaf(qsm[ks * D + j], qsm[ks * D + j], s2);
        s2 = tq_warp_sum(s2);
        if (lane == 0) qn2[ks] = s2;
    }
    float a[VPC];
#pragma unroll
    for (int v = 0; v < VPC; ++v) a[v] = 0.f;
#pragma unroll
    for (int k = 0; k < D / 8; ++k) {
#pragma unroll
        for (int v = 0; v < VPC; ++v) a[v] = fmaf(qsm[v * D + k0 + k], mv[k], a[v]);
    }
#pragma unroll
    for (int v = 0; v < VPC; ++v) red[(ks * VPC + v) * 32 + lane] = a[v];
    __syncthreads();
    if (threadIdx.x < VPC * 32) {
        const int v = threadIdx.x >> 5;
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[(i * VPC + v) * 32 + lane];
        if (v < nv) {
            if (live) out[((v0 + v) * 2 + which) * D + col] = t;
            if (frag != nullptr) {
                const int64_t vec = v0 + v;
                const int qh = (int)(vec % Qh), g = qh % G;
                const int64_t pair = (vec / Qh) * (Qh / G) + qh / G;   // (sequence, kv head)
                const bool split = G > 4 || mse_bits == 3;   // separate rotated / sketched fragment sets
                uint32_t* base = frag + pair * qf_words(D, split ? 8 : 4);
                const float bound = sqrtf(qn2[v]) * (which ? 2.f * sqrtf((float)D) : 1.f);
                int e = 0;
                if (bound > 0.f && bound < 3.0e38f) e = max(-100, min(100, 14 - ilogbf(bound)));
                if (live && chunk == 0 && lane == 0) reinterpret_cast<float*>(base)[which * 8 + g] = (float)e;
                const int tig = col / (D / 4), rem = col % (D / 4);
                int wi = rem >> 4, half = (rem >> 3) & 1, jf = rem & 7;
                int r = wi * 8 + jf;
                int sh = which ? sign_pos(sign_bit(wi, jf)) : 2 * code_pos(jf);
                if (mse_bits == 3 && which == 0) {
                    // nibble codes: registers pair adjacent dims, k-step = 4 dims, true centroid values (no scaling)
                    r = rem >> 1;
                    half = rem & 1;
                    sh = 0;
                }
                const int gid = split ? g : g + 4 * which;
                const int set = split ? which : 0;
                __half* dst = reinterpret_cast<__half*>(base + QF_HDR + ((set * (D / 8) + r) * 32 + gid * 4 + tig));
                if (live) dst[half] = __float2half_rn(t * __int_as_float((127 + e - sh) << 23));
            }
        }
    }
    __syncthreads();   // shared memory is reused by the next group / the second pass
    }
    v0 = (int64_t)blockIdx.y * groups * VPC;
    nv = (int)min((int64_t)VPC, nvec - v0);
    }
}

// Query preparation for large batches: a plain tiled fp32 product (64 vectors x 64 columns per CTA,
// 4 x 4 outputs per thread) instead of the latency-oriented kernel above, whose CTAs re-read their
// matrix slice and the queries from shared memory once per multiply-add.  A CTA's 64 columns are four
// strips of 16 - one in each quarter of the head dimension - because that is what fills whole rows of
// the fp16 MMA fragments (a fragment row holds, for eight query heads, the four quarters' elements of
// one position): the results are staged in shared memory and leave as full 128-byte rows.
constexpr int QB_V = 64, QB_C = 64, QB_K = 32;
template <int D>
__global__ void __launch_bounds__(256) tq_qprep_batched_kernel(const void* __restrict__ q, int dt, int64_t nvec,
                                                               const float* __restrict__ pi_t,
                                                               const float* __restrict__ s_t, float* __restrict__ out,
                                                               uint32_t* __restrict__ frag, int G, int Qh, int mse_bits) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) float qb_smem[];
    float* qT = qb_smem;                    // [D][QB_V] queries, transposed; later the [QB_V][QB_C + 1] results
    float* mt = qT + D * QB_V;              // [QB_K][QB_C] matrix rows of the current k chunk
    float* part = mt + QB_K * QB_C;         // [4][QB_V] partial squared norms
    const int tid = threadIdx.x;
    const int64_t v0 = (int64_t)blockIdx.y * QB_V;
    const int which = blockIdx.x / (D / 64), strip = blockIdx.x % (D / 64);
    // local column lc: quarter lc / 16 of the head dimension, position 16 * strip + lc % 16 inside it
    auto column = [&](int lc) { return (lc >> 4) * (D / 4) + 16 * strip + (lc & 15); };
    const float* __restrict__ m = which ? s_t : pi_t;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the queries may come from the kernel ahead
    {   // queries: 16-byte chunks, lanes walking the vectors so that the transposed stores spread over the banks
        const int esz = dt == TQ_F32 ? 4 : 2, per = 16 / esz, chunks = D / per;
        for (int i = tid; i < QB_V * chunks; i += 256) {
            const int v = i & (QB_V - 1), c = i / QB_V;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (v0 + v < nvec)
                raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const char*>(q) + ((v0 + v) * D + (int64_t)c * per) * esz));
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            float* dst = qT + (c * per) * QB_V + v;
            if (dt == TQ_F32) {
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j * QB_V] = __uint_as_float(w[j]);
            } else if (dt == TQ_BF16) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dst[(2 * j) * QB_V] = __uint_as_float(w[j] << 16);
                    dst[(2 * j + 1) * QB_V] = __uint_as_float(w[j] & 0xffff0000u);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                    dst[(2 * j) * QB_V] = f2.x;
                    dst[(2 * j + 1) * QB_V] = f2.y;
                }
            }
        }
        __syncthreads();
        const int v = tid & (QB_V - 1), qtr = tid >> 6;   // squared norm of vector v, a quarter of the channels each
        float s2 = 0.f;
        for (int k = qtr * (D / 4); k < (qtr + 1) * (D / 4); ++k) {
            const float x = qT[k * QB_V + v];
            s2 = fmaf(x, x, s2);
        }
        part[qtr * QB_V + v] = s2;
    }
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 1
    for (int k0 = 0; k0 < D; k0 += QB_K) {
        __syncthreads();   // queries stored (first round) / previous matrix chunk consumed
        for (int i = tid; i < QB_K * QB_C / 4; i += 256) {
            const int kk = i / (QB_C / 4), c4 = i % (QB_C / 4);
            reinterpret_cast<float4*>(mt)[i] = __ldg(reinterpret_cast<const float4*>(m + (size_t)(k0 + kk) * D + column(4 * c4)));
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < QB_K; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(qT + (k0 + kk) * QB_V + 4 * ty);
            const float4 b = *reinterpret_cast<const float4*>(mt + kk * QB_C + 4 * tx);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    __syncthreads();   // the queries are consumed: their space takes the results
    constexpr int RP = QB_C + 1;
    float* res = qT;   // [QB_V][RP]
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) res[(4 * ty + i) * RP + 4 * tx + j] = acc[i][j];
    __syncthreads();
    // fp32 results: 64-byte runs (one strip of one quarter)
    for (int i = tid; i < QB_V * QB_C; i += 256) {
        const int v = i / QB_C, lc = i % QB_C;
        if (v0 + v < nvec) out[((v0 + v) * 2 + which) * D + column(lc)] = res[v * RP + lc];
    }
    if (frag == nullptr) return;
    // fragment words: thread = (quarter, vector); lanes (quarter, vector % 8) write one 128-byte fragment row
    // when eight query heads share a kv head.  Element layout as in tq_qprep_kernel.
    const int tig = tid & 3, v = tid >> 2;
    if (v0 + v >= nvec) return;
    const int64_t vec = v0 + v;
    const int qh = (int)(vec % Qh), g = qh % G;
    const int64_t pair = (vec / Qh) * (Qh / G) + qh / G;   // (sequence, kv head)
    const bool split = G > 4 || mse_bits == 3;             // separate rotated / sketched fragment sets
    uint32_t* base = frag + pair * qf_words(D, split ? 8 : 4);
    const float qn2 = (part[v] + part[QB_V + v]) + (part[2 * QB_V + v] + part[3 * QB_V + v]);
    const float bound = sqrtf(qn2) * (which ? 2.f * sqrtf((float)D) : 1.f);
    int e = 0;
    if (bound > 0.f && bound < 3.0e38f) e = max(-100, min(100, 14 - ilogbf(bound)));
    if (strip == 0 && tig == 0) reinterpret_cast<float*>(base)[which * 8 + g] = (float)e;
    const bool nibble = mse_bits == 3 && which == 0;       // two adjacent positions per word instead of j, j + 8
    const int gid = split ? g : g + 4 * which;
    const int set = split ? which : 0;
#pragma unroll
    for (int rl = 0; rl < 8; ++rl) {
        const int lc0 = tig * 16 + (nibble ? 2 * rl : rl), lc1 = tig * 16 + (nibble ? 2 * rl + 1 : rl + 8);
        const int sh = nibble ? 0 : (which ? sign_pos(sign_bit(strip, rl)) : 2 * code_pos(rl));
        const float scale = __int_as_float((127 + e - sh) << 23);
        const __half2 h2 = __floats2half2_rn(res[v * RP + lc0] * scale, res[v * RP + lc1] * scale);
        base[QF_HDR + (set * (D / 8) + 8 * strip + rl) * 32 + gid * 4 + tig] = *reinterpret_cast<const uint32_t*>(&h2);
    }
}

int launch_qprep(const void* q, int dt, int64_t nvec, int D, const float* pi_t, const float* s_t, float* out,
                 uint32_t* frag, int G, int Qh, int mse_bits, const RingAppend& ap, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // its matrix loads may run under the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tq_pdl_for_decode(st);   // behind a store that is still writing the pool: plain stream order
    tq_note_launch(st, TQ_LAUNCH_DECODE);
    cfg.stream = st;
    cfg.blockDim = dim3(256);
    if (nvec >= 4096 && ap.new_k == nullptr && !ap.early_inputs && ((uintptr_t)q & 15) == 0) {   // throughput kernel
        const size_t smem = sizeof(float) * ((size_t)D * QB_V + QB_K * QB_C + 4 * QB_V);
        cfg.gridDim = dim3((unsigned)(2 * D / QB_C), (unsigned)((nvec + QB_V - 1) / QB_V));
        cfg.dynamicSmemBytes = smem;
        const int dtb = dt;
        cudaError_t eb;
        if (D == 128) {
            static TqSmemOptIn opt_in;
            if (tq_opt_in_smem(tq_qprep_batched_kernel<128>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
            eb = cudaLaunchKernelEx(&cfg, tq_qprep_batched_kernel<128>, q, dtb, nvec, pi_t, s_t, out, frag, G, Qh, mse_bits);
        } else {
            static TqSmemOptIn opt_in;
            if (tq_opt_in_smem(tq_qprep_batched_kernel<256>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
            eb = cudaLaunchKernelEx(&cfg, tq_qprep_batched_kernel<256>, q, dtb, nvec, pi_t, s_t, out, frag, G, Qh, mse_bits);
        }
        return eb == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
    }
    // four vectors per CTA: with eight the grid packs four CTAs onto each of the few SMs that free up first
    // under a running decode kernel, and they then share one SM for the part after the wait (measured: slower)
    constexpr int vpc = 4;
    // large batches: about three waves of CTAs, each working through several groups of four vectors
    const int64_t n_groups = (nvec + vpc - 1) / vpc;
    const int64_t ctas_y_wanted = (3 * (int64_t)tq_sm_count() * 2) / (2 * D / 32) + 1;
    int groups = (int)((n_groups + ctas_y_wanted - 1) / ctas_y_wanted);
    if (groups < 1 || ap.early_inputs) groups = 1;
    if (groups > 64) groups = 64;
    cfg.gridDim = dim3((unsigned)(2 * D / 32), (unsigned)((n_groups + groups - 1) / groups));
    cfg.dynamicSmemBytes = 0;
    const int dti = dt;
    cudaError_t e;
    const bool small = cfg.gridDim.x * cfg.gridDim.y <= 256u;
    if (D == 128 && small)
        e = cudaLaunchKernelEx(&cfg, tq_qprep_kernel<128, vpc, 2>, q, dti, nvec, pi_t, s_t, out, frag, G, Qh, mse_bits, ap, groups);
    else if (D == 128)
        e = cudaLaunchKernelEx(&cfg, tq_qprep_kernel<128, vpc, 3>, q, dti, nvec, pi_t, s_t, out, frag, G, Qh, mse_bits, ap, groups);
    else if (small)
        e = cudaLaunchKernelEx(&cfg, tq_qprep_kernel<256, vpc, 2>, q, dti, nvec, pi_t, s_t, out, frag, G, Qh, mse_bits, ap, groups);
    else
        e = cudaLaunchKernelEx(&cfg, tq_qprep_kernel<256, vpc, 3>, q, dti, nvec, pi_t, s_t, out, frag, G, Qh, mse_bits, ap, groups);
    return e == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

template <int D, int MSE_BITS, int VAL_BITS, int GP>
__global__ void __launch_bounds__(DEC_THREADS) tq_decode_kernel(const DecodeParams p) {
    constexpr int DPT = D / DEC_THREADS;
    const TqLayout L = tq_make_layout(D, MSE_BITS + 1, VAL_BITS);
    const int BB = L.block_bytes;

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;                                                        // [NSTAGE][4*BB]; ring CTAs: K/V rows
    const int stage_bytes = max(NSTAGE * TILE_BLOCKS * BB, 2 * RING_TOK * D * 4);  // same rule as the launcher
    float* qr = reinterpret_cast<float*>(smem + stage_bytes);                      // [D][GP]
    float* qs = qr + D * GP;                                                       // [D][GP]
    float* sp = qs + D * GP;                                                       // [2][GP][64]
    float* pp = sp + 2 * GP * TILE_TOK;                                            // [64][GP]
    float* m_run = pp + TILE_TOK * GP;                                             // [GP]
    float* l_run = m_run + GP;                                                     // [GP]
    float* alpha = l_run + GP;                                                     // [GP]
    float* cent = alpha + GP;                                                      // [16]
    uint64_t* bars = reinterpret_cast<uint64_t*>(cent + TQ_MAX_CENTROIDS);         // [NSTAGE]
    float* wsm = reinterpret_cast<float*>(bars + NSTAGE);                          // merge scratch

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, h = blockIdx.y, x = blockIdx.x;

    float acc[GP][DPT];
#pragma unroll
    for (int g = 0; g < GP; ++g)
#pragma unroll
        for (int i = 0; i < DPT; ++i) acc[g][i] = 0.f;
    if (tid < GP) {
        m_run[tid] = -INFINITY;
        l_run[tid] = 0.f;
    }
    if (tid < TQ_MAX_CENTROIDS) cent[tid] = p.cb.centroids[tid];

    if (x < p.num_splits) {
        // ------------------------- compressed history -------------------------
        int n = p.seq_lens[b];
        if (n > p.max_seq_len) {   // the host bound sized the grid and the block-table check
            if (tid == 0) atomicCAS(p.status, 0, (int)TQ_ERR_RANGE);
            n = p.max_seq_len;
        }
        if (n < p.min_history) n = 0;
        const int nblk = (n + TQ_BLOCK_TOKENS - 1) / TQ_BLOCK_TOKENS;
        const int ntile = (nblk + TILE_BLOCKS - 1) / TILE_BLOCKS;
        const int tps = (ntile + p.num_splits - 1) / p.num_splits;
        const int tile0 = x * tps;
        const int tile1 = min(ntile, tile0 + tps);
        const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;

        if (tile0 < tile1) {
            for (int i = tid; i < D * GP; i += DEC_THREADS) {
                const int j = i / GP, g = i % GP;
                float a = 0.f, c = 0.f;
                if (g < p.G) {
                    const float* src = p.qprep + ((int64_t)(b * p.Qh + h * p.G + g) * 2) * D;
                    a = src[j];
                    c = src[D + j];
                }
                qr[i] = a;
                qs[i] = c;
            }
            if (tid == 0) {
                for (int s = 0; s < NSTAGE; ++s) tq_mbar_init(bars + s, 1);
                tq_mbar_fence_init();
            }
            __syncthreads();
            if (tid == 0) {
                for (int s = 0; s < NSTAGE - 1 && tile0 + s < tile1; ++s)
                    issue_tile(stages + s * TILE_BLOCKS * BB, bars + s, p.pool, p.num_blocks, bt,
                               (tile0 + s) * TILE_BLOCKS, nblk, p.H, h, BB, p.status);
            }
            for (int tile = tile0; tile < tile1; ++tile) {
                const int it = tile - tile0, st = it % NSTAGE;
                if (tid == 0 && tile + NSTAGE - 1 < tile1) {
                    const int s2 = (it + NSTAGE - 1) % NSTAGE;
                    issue_tile(stages + s2 * TILE_BLOCKS * BB, bars + s2, p.pool, p.num_blocks, bt,
                               (tile + NSTAGE - 1) * TILE_BLOCKS, nblk, p.H, h, BB, p.status);
                }
                const bool ok = tq_mbar_wait_bounded(bars + st, (uint32_t)((it / NSTAGE) & 1));
                if (__syncthreads_or(!ok)) {
                    if (tid == 0) atomicCAS(p.status, 0, (int)TQ_ERR_TIMEOUT);
                    break;
                }
                const uint8_t* stage = stages + st * TILE_BLOCKS * BB;
                const int tok_base = tile * TILE_TOK;
                const int valid = min(TILE_TOK, n - tok_base);

                // scores: 2 threads per token, one per half of the head dimension
                {
                    const int tk = tid & (TILE_TOK - 1), half = tid >> 6;
                    float part[GP];
                    if (tk < valid) {
                        token_half_scores<D, MSE_BITS, GP>(stage + (tk >> 4) * BB, L, tk & 15, half, qr, qs, cent,
                                                           p.qjl_scale, part);
                    } else {
#pragma unroll
                        for (int g = 0; g < GP; ++g) part[g] = 0.f;
                    }
#pragma unroll
                    for (int g = 0; g < GP; ++g) sp[(half * GP + g) * TILE_TOK + tk] = part[g];
                }
                __syncthreads();
                // online softmax, one warp per query head
                for (int g = warp; g < GP; g += DEC_THREADS / 32) {
                    float s0 = -INFINITY, s1 = -INFINITY;
                    if (lane < valid) s0 = (sp[g * TILE_TOK + lane] + sp[(GP + g) * TILE_TOK + lane]) * p.scale;
                    if (lane + 32 < valid)
                        s1 = (sp[g * TILE_TOK + lane + 32] + sp[(GP + g) * TILE_TOK + lane + 32]) * p.scale;
                    const float m_old = m_run[g];
                    const float m_new = fmaxf(m_old, tq_warp_max(fmaxf(s0, s1)));
                    const float p0 = (s0 == -INFINITY) ? 0.f : __expf(s0 - m_new);
                    const float p1 = (s1 == -INFINITY) ? 0.f : __expf(s1 - m_new);
                    const float a = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
                    const float sum = tq_warp_sum(p0 + p1);
                    pp[lane * GP + g] = p0;
                    pp[(lane + 32) * GP + g] = p1;
                    if (lane == 0) {
                        m_run[g] = m_new;
                        l_run[g] = l_run[g] * a + sum;
                        alpha[g] = a;
                    }
                }
                __syncthreads();
                // values: each thread owns DPT channels for all query heads
                {
#pragma unroll
                    for (int g = 0; g < GP; ++g) {
                        const float a = alpha[g];
#pragma unroll
                        for (int i = 0; i < DPT; ++i) acc[g][i] *= a;
                    }
                    const int d0 = tid * DPT, grp = d0 >> 5;
                    for (int t = 0; t < valid; ++t) {
                        const uint8_t* rec = stage + (t >> 4) * BB;
                        const int tl = t & 15;
                        const float sc = __half2float(reinterpret_cast<const __half*>(rec + L.off_vscale)[grp * 16 + tl]);
                        const float zr = __half2float(reinterpret_cast<const __half*>(rec + L.off_vzero)[grp * 16 + tl]);
                        float v[DPT];
                        if (VAL_BITS == 2) {
                            const uint32_t byte = rec[L.off_vcodes + tq_vcode_native(D, 2, tl, d0 >> 2)];
#pragma unroll
                            for (int i = 0; i < DPT; ++i) v[i] = fmaf((float)((byte >> (2 * ((d0 + i) & 3))) & 3u), sc, zr);
                        } else {
                            const uint32_t byte = rec[L.off_vcodes + tq_vcode_native(D, 4, tl, d0 >> 1)];
#pragma unroll
                            for (int i = 0; i < DPT; ++i) v[i] = fmaf((float)((byte >> (4 * ((d0 + i) & 1))) & 15u), sc, zr);
                        }
                        const float* pt = pp + t * GP;
#pragma unroll
                        for (int g = 0; g < GP; ++g)
#pragma unroll
                            for (int i = 0; i < DPT; ++i) acc[g][i] = fmaf(pt[g], v[i], acc[g][i]);
                    }
                }
                __syncthreads();
            }
        }
        __syncthreads();
        write_partial_regs<D, GP>(p, b, h, x, acc, m_run, l_run);
        ticket_and_merge<D, GP>(p, b, h, wsm);
        return;
    }

    // ------------------------------ exact ring ------------------------------
    __syncthreads();
    // m_run, l_run are adjacent: [2*GP]; the stage region (sized for it by the launcher) holds the ring rows
    ring_part<D, GP>(p, b, h, x, qr, sp, pp, m_run, stages, stages + RING_TOK * D * 4);
    ticket_and_merge<D, GP>(p, b, h, wsm);
}

// Unscaled logits of up to 8 query vectors per CTA against one 64-token tile.
template <int D, int MSE_BITS>
__global__ void __launch_bounds__(DEC_THREADS) tq_scores_kernel(const ScoreParams p, int key_bits, int val_bits) {
    constexpr int GP = 8;
    const TqLayout L = tq_make_layout(D, key_bits, val_bits);
    const int BB = L.block_bytes;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stage = smem;
    float* qr = reinterpret_cast<float*>(smem + TILE_BLOCKS * BB);
    float* qs = qr + D * GP;
    float* sp = qs + D * GP;  // [2][GP][64]
    float* cent = sp + 2 * GP * TILE_TOK;
    uint64_t* bar = reinterpret_cast<uint64_t*>(cent + TQ_MAX_CENTROIDS);

    const int tid = threadIdx.x;
    const int tile = blockIdx.x, h = blockIdx.y, q0 = blockIdx.z * GP;
    const int nq = min(GP, p.n_q - q0);
    const int nblk = (int)((p.n_tokens + TQ_BLOCK_TOKENS - 1) / TQ_BLOCK_TOKENS);
    if (tid < TQ_MAX_CENTROIDS) cent[tid] = p.cb.centroids[tid];
    for (int i = tid; i < D * GP; i += DEC_THREADS) {
        const int j = i / GP, g = i % GP;
        float a = 0.f, c = 0.f;
        if (g < nq) {
            const float* src = p.qprep + ((int64_t)(h * p.n_q + q0 + g) * 2) * D;
            a = src[j];
            c = src[D + j];
        }
        qr[i] = a;
        qs[i] = c;
    }
    if (tid == 0) {
        tq_mbar_init(bar, 1);
        tq_mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0)
        issue_tile(stage, bar, p.pool, p.num_blocks, p.block_table, tile * TILE_BLOCKS, nblk, p.H, h, BB, p.status);
    const bool ok = tq_mbar_wait_bounded(bar, 0);
    if (__syncthreads_or(!ok)) {
        if (tid == 0) atomicCAS(p.status, 0, (int)TQ_ERR_TIMEOUT);
        return;
    }
    const int valid = (int)min((int64_t)TILE_TOK, p.n_tokens - (int64_t)tile * TILE_TOK);
    const int tk = tid & (TILE_TOK - 1), half = tid >> 6;
    float part[GP];
    if (tk < valid) {
        token_half_scores<D, MSE_BITS, GP>(stage + (tk >> 4) * BB, L, tk & 15, half, qr, qs, cent, p.qjl_scale, part);
    } else {
#pragma unroll
        for (int g = 0; g < GP; ++g) part[g] = 0.f;
    }
#pragma unroll
    for (int g = 0; g < GP; ++g) sp[(half * GP + g) * TILE_TOK + tk] = part[g];
    __syncthreads();
    for (int i = tid; i < nq * TILE_TOK; i += DEC_THREADS) {
        const int g = i / TILE_TOK, t = i % TILE_TOK;
        if (t < valid)
            p.logits[((int64_t)h * p.n_q + q0 + g) * p.n_tokens + (int64_t)tile * TILE_TOK + t] =
                sp[g * TILE_TOK + t] + sp[(GP + g) * TILE_TOK + t];
    }
}

template <int D, int GP>
size_t decode_smem_bytes(int block_bytes, int nslot) {
    size_t s = (size_t)NSTAGE * TILE_BLOCKS * block_bytes;
    if (s < (size_t)2 * RING_TOK * D * 4) s = (size_t)2 * RING_TOK * D * 4;   // ring CTAs stage their K/V rows here
    s += sizeof(float) * (2 * D * GP + 2 * GP * TILE_TOK + TILE_TOK * GP + 3 * GP + TQ_MAX_CENTROIDS);
    s += sizeof(uint64_t) * NSTAGE;
    // merge scratch sized for at least 128 partials so that the launch size
    // (and with it the kernel's shared-memory attribute) rarely changes
    s += sizeof(float) * ((size_t)(nslot > 128 ? nslot : 128) * GP + 2 * GP);
    return s;
}

template <int D, int MSE_BITS, int VAL_BITS, int GP>
int launch_decode(const DecodeParams& p, int B, int block_bytes, cudaStream_t st) {
    const int nslot = p.num_splits + p.ring_splits;
    const size_t smem = decode_smem_bytes<D, GP>(block_bytes, nslot);
    auto kern = tq_decode_kernel<D, MSE_BITS, VAL_BITS, GP>;
    static TqSmemOptIn opt_in;
    if (tq_opt_in_smem(kern, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
    dim3 grid((unsigned)nslot, (unsigned)p.H, (unsigned)B);
    kern<<<grid, DEC_THREADS, smem, st>>>(p);
    tq_note_launch(st, TQ_LAUNCH_DECODE);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

template <int D, int MSE_BITS, int VAL_BITS>
int launch_decode_g(const DecodeParams& p, int B, int block_bytes, cudaStream_t st) {
    if (p.G <= 4) return launch_decode<D, MSE_BITS, VAL_BITS, 4>(p, B, block_bytes, st);
    return launch_decode<D, MSE_BITS, VAL_BITS, 8>(p, B, block_bytes, st);
}

struct WsLayout {
    size_t off_tickets, off_qprep, off_qfrag, off_partials, total;
};

// Partial results are GP x (D + 2) floats per slot.  The tensor-core kernel pads the query heads of a
// kv head to 8 whenever it keeps separate rotated / sketched fragment sets (more than four heads, or
// 3-bit codes), the CUDA-core kernel only with more than four heads: size for the larger of the two.
WsLayout decode_ws_layout(int D, int B, int Qh, int H, int max_slots, int mse_bits) {
    WsLayout w;
    const int G = Qh / H;
    const int GP = (G <= 4 && mse_bits != 3) ? 4 : 8;
    w.off_tickets = TQ_WS_HEADER_BYTES;
    w.off_qprep = w.off_tickets + (((size_t)B * H * sizeof(int32_t) + 255) / 256) * 256;
    w.off_qfrag = w.off_qprep + (((size_t)B * Qh * 2 * D * sizeof(float) + 255) / 256) * 256;
    w.off_partials = w.off_qfrag + (((size_t)B * H * qf_words(D, 8) * sizeof(uint32_t) + 255) / 256) * 256;
    w.total = w.off_partials + (size_t)B * H * max_slots * GP * (D + 2) * sizeof(float);
    return w;
}

int ring_splits_for(int max_ring_len, int ring_tok) { return (max_ring_len + ring_tok - 1) / ring_tok; }

// Ring tokens per ring CTA: 64 when the whole launch then fits one wave (fewer ring CTAs leave more
// SMs to the history), else 32.  A pure function of the launch shape, so that callers can plan with it.
int ring_tok_for(int max_ring_len, int64_t pairs, int splits) {
    if (max_ring_len <= RING_TOK) return RING_TOK;
    const int r64 = (max_ring_len + 2 * RING_TOK - 1) / (2 * RING_TOK);
    return pairs * (splits + r64) <= tq_sm_count() ? 2 * RING_TOK : RING_TOK;
}

}  // namespace

extern "C" int tq_decode_workspace_bytes(const tq_config* cfg, int32_t batch, int32_t num_q_heads,
                                         int32_t num_kv_heads, int32_t max_splits, size_t* out) {
    if (!cfg || !out) return TQ_ERR_NULL;
    int rc = tq_check_config(cfg);
    if (rc != TQ_OK) return rc;
    if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_splits <= 0) return TQ_ERR_SHAPE;
    if (num_q_heads % num_kv_heads != 0 || num_q_heads / num_kv_heads > TQ_MAX_GROUP_HEADS) return TQ_ERR_UNSUPPORTED;
    // ring CTAs need partial slots too: reserve for a ring of up to 256 tokens
    *out = decode_ws_layout(cfg->head_dim, batch, num_q_heads, num_kv_heads, max_splits + 8, cfg->key_bits - 1).total;
    return TQ_OK;
}

extern "C" int tq_scores_workspace_bytes(const tq_config* cfg, int64_t n_vectors, size_t* out) {
    if (!cfg || !out) return TQ_ERR_NULL;
    int rc = tq_check_config(cfg);
    if (rc != TQ_OK) return rc;
    if (n_vectors <= 0) return TQ_ERR_SHAPE;
    *out = TQ_WS_HEADER_BYTES + (size_t)n_vectors * 2 * cfg->head_dim * sizeof(float);
    return TQ_OK;
}

static int decode_impl(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* a, void* stream,
                       int early_inputs, int validate_only = 0) {
    if (!consts || !pool || !a) return TQ_ERR_NULL;
    if (!pool->base || !a->query || !a->out || !a->workspace || !a->block_table || !a->seq_lens) return TQ_ERR_NULL;
    if (!consts->pi_t || !consts->s_t) return TQ_ERR_NULL;
    int rc = tq_check_config(&consts->cfg);
    if (rc != TQ_OK) return rc;
    const int D = consts->cfg.head_dim, H = pool->num_kv_heads;
    if (a->batch <= 0 || a->num_q_heads <= 0 || H <= 0 || a->max_seq_len < 0 || a->block_table_stride < 0)
        return TQ_ERR_SHAPE;
    if (a->num_q_heads % H != 0) return TQ_ERR_SHAPE;
    const int G = a->num_q_heads / H;
    if (G > TQ_MAX_GROUP_HEADS) return TQ_ERR_UNSUPPORTED;
    if ((int64_t)a->block_table_stride * TQ_BLOCK_TOKENS < a->max_seq_len) return TQ_ERR_SHAPE;
    const bool has_ring = a->ring_k != nullptr && a->max_ring_len > 0;
    if (has_ring && (!a->ring_v || !a->ring_lens)) return TQ_ERR_NULL;
    if (has_ring && a->max_ring_len > 256) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)pool->base & 15) || ((uintptr_t)a->workspace & 255) || ((uintptr_t)a->out & 15)) return TQ_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;

    const TqLayout L = tq_make_layout(D, consts->cfg.key_bits, consts->cfg.value_bits);
    const int ntile = (a->max_seq_len + TILE_TOK - 1) / TILE_TOK;
    int splits = a->num_splits;
    if (splits <= 0) {
        // about two CTAs per SM over the whole launch, at least 2 tiles per split
        const int sms = tq_sm_count();
        const int want = (2 * sms + a->batch * H - 1) / (a->batch * H);
        splits = want < 1 ? 1 : want;
        const int cap = (ntile + 1) / 2;
        if (splits > cap) splits = cap;
        // at most 512 block records per split: the tensor-core kernel keeps a split's block-table slice in
        // shared memory, and long and short sequences of a batch balance better
        const int nblk = (a->max_seq_len + TQ_BLOCK_TOKENS - 1) / TQ_BLOCK_TOKENS;
        if (splits < (nblk + 511) / 512) splits = (nblk + 511) / 512;
    }
    if (splits < 1) splits = 1;
    if (splits > ntile && ntile > 0) splits = ntile;
    const int ring_tok = has_ring ? ring_tok_for(a->max_ring_len, (int64_t)a->batch * H, splits) : RING_TOK;
    const int rsplits = has_ring ? ring_splits_for(a->max_ring_len, ring_tok) : 0;
    const WsLayout w = decode_ws_layout(D, a->batch, a->num_q_heads, H, splits + rsplits, consts->cfg.key_bits - 1);
    if (w.total > a->workspace_bytes) return TQ_ERR_WORKSPACE;

    uint8_t* ws = (uint8_t*)a->workspace;
    float* qprep = (float*)(ws + w.off_qprep);
    uint32_t* qfrag = (uint32_t*)(ws + w.off_qfrag);
    RingAppend ap = {};
    ap.early_inputs = early_inputs;
    if (a->append_k != nullptr) {
        if (!has_ring || !a->append_v || a->query_prepared) return TQ_ERR_NULL;
        if (a->ring_capacity < a->max_ring_len) return TQ_ERR_SHAPE;
        const int eb = (int)tq_dtype_size(a->ring_dtype);
        if (((uintptr_t)a->append_k | (uintptr_t)a->append_v | (uintptr_t)a->ring_k | (uintptr_t)a->ring_v) & 15)
            return TQ_ERR_ALIGN;
        if ((a->ring_stride_seq * eb) % 16 || (a->ring_stride_token * eb) % 16) return TQ_ERR_ALIGN;
        ap.new_k = a->append_k;
        ap.new_v = a->append_v;
        ap.ring_k = const_cast<void*>(a->ring_k);
        ap.ring_v = const_cast<void*>(a->ring_v);
        ap.ring_lens = const_cast<int32_t*>(a->ring_lens);
        ap.elem_bytes = eb;
        ap.B = a->batch;
        ap.H = H;
        ap.capacity = a->ring_capacity;
        ap.stride_seq = a->ring_stride_seq;
        ap.stride_token = a->ring_stride_token;
    }
    if (validate_only) return TQ_OK;   // every host-side check has passed; nothing was enqueued
    if (!a->query_prepared) {
        const int64_t nvec = (int64_t)a->batch * a->num_q_heads;
        int on_tensor_cores = 0;
        if (ap.new_k == nullptr && !early_inputs &&
            tq_qprep_tc_launch(consts, a->query, a->q_dtype, nvec, qprep, qfrag, G, a->num_q_heads,
                               consts->cfg.key_bits - 1, (int*)ws, st, &on_tensor_cores) != TQ_OK)
            return TQ_ERR_CUDA;
        if (!on_tensor_cores &&
            launch_qprep(a->query, a->q_dtype, nvec, D, consts->pi_t, consts->s_t, qprep, qfrag, G, a->num_q_heads,
                         consts->cfg.key_bits - 1, ap, st) != TQ_OK)
            return TQ_ERR_CUDA;
    }

    DecodeParams p;
    p.pool = (const uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = H;
    p.Qh = a->num_q_heads;
    p.G = G;
    p.block_table = a->block_table;
    p.bt_stride = a->block_table_stride;
    p.seq_lens = a->seq_lens;
    p.max_seq_len = a->max_seq_len;
    p.min_history = a->min_history;
    p.qprep = qprep;
    p.qfrag = qfrag;
    p.query = a->query;
    p.q_dtype = a->q_dtype;
    p.ring_k = has_ring ? a->ring_k : nullptr;
    p.ring_v = has_ring ? a->ring_v : nullptr;
    p.ring_dtype = a->ring_dtype;
    p.ring_lens = has_ring ? a->ring_lens : nullptr;
    p.max_ring_len = has_ring ? a->max_ring_len : 0;
    p.ring_stride_seq = a->ring_stride_seq;
    p.ring_stride_token = a->ring_stride_token;
    p.scale = a->scale;
    p.qjl_scale = consts->qjl_scale;
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        p.cb.centroids[i] = consts->centroids[i];
        p.cb.boundaries[i] = consts->boundaries[i];
    }
    p.out = a->out;
    p.partials = (float*)(ws + w.off_partials);
    p.tickets = (int32_t*)(ws + w.off_tickets);
    p.status = (int32_t*)ws;
    p.num_splits = splits;
    p.ring_splits = rsplits;
    p.ring_tok = ring_tok;
    p.land_bytes = 0;

    const int mse_bits = consts->cfg.key_bits - 1, vb = consts->cfg.value_bits;
    if (a->kernel != 1) {   // tensor-core kernel where it applies
        int handled = 0;
        rc = tq_decode_mma_launch(p, D, mse_bits, vb, a->batch, a->max_seq_len, st, &handled);
        if (rc != TQ_OK || handled) return rc;
    }
#define TQ_DEC(DD, MB, VB) return launch_decode_g<DD, MB, VB>(p, a->batch, L.block_bytes, st)
    if (D == 128) {
        if (mse_bits == 2 && vb == 2) TQ_DEC(128, 2, 2);
        if (mse_bits == 2 && vb == 4) TQ_DEC(128, 2, 4);
        if (mse_bits == 3 && vb == 2) TQ_DEC(128, 3, 2);
        TQ_DEC(128, 3, 4);
    } else {
        if (mse_bits == 2 && vb == 2) TQ_DEC(256, 2, 2);
        if (mse_bits == 2 && vb == 4) TQ_DEC(256, 2, 4);
        if (mse_bits == 3 && vb == 2) TQ_DEC(256, 3, 2);
        TQ_DEC(256, 3, 4);
    }
#undef TQ_DEC
}

extern "C" int tq_decode(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* a, void* stream) {
    return decode_impl(consts, pool, a, stream, 0);
}

extern "C" int tq_scores(const tq_consts* consts, const tq_pool* pool, const int32_t* block_table, int64_t n_tokens,
                         const void* query, tq_dtype q_dtype, int32_t n_q, float* logits, void* workspace,
                         size_t workspace_bytes, void* stream) {
    if (!consts || !pool || !pool->base || !block_table || !query || !logits || !workspace) return TQ_ERR_NULL;
    if (!consts->pi_t || !consts->s_t) return TQ_ERR_NULL;
    int rc = tq_check_config(&consts->cfg);
    if (rc != TQ_OK) return rc;
    if (n_tokens < 0 || n_q <= 0 || pool->num_kv_heads <= 0) return TQ_ERR_SHAPE;
    if (n_tokens == 0) return TQ_OK;
    const int D = consts->cfg.head_dim, H = pool->num_kv_heads;
    size_t need = 0;
    tq_scores_workspace_bytes(&consts->cfg, (int64_t)H * n_q, &need);
    if (need > workspace_bytes) return TQ_ERR_WORKSPACE;
    if ((uintptr_t)workspace & 255) return TQ_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    float* qprep = (float*)((uint8_t*)workspace + TQ_WS_HEADER_BYTES);
    const int64_t nvec = (int64_t)H * n_q;
    if (launch_qprep(query, q_dtype, nvec, D, consts->pi_t, consts->s_t, qprep, nullptr, 1, 1, 2, RingAppend{}, st) != TQ_OK)
        return TQ_ERR_CUDA;

    const TqLayout L = tq_make_layout(D, consts->cfg.key_bits, consts->cfg.value_bits);
    ScoreParams p;
    p.pool = (const uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = H;
    p.block_table = block_table;
    p.n_tokens = n_tokens;
    p.qprep = qprep;
    p.n_q = n_q;
    p.qjl_scale = consts->qjl_scale;
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        p.cb.centroids[i] = consts->centroids[i];
        p.cb.boundaries[i] = consts->boundaries[i];
    }
    p.logits = logits;
    p.status = (int32_t*)workspace;
    const size_t smem = (size_t)TILE_BLOCKS * L.block_bytes +
                        sizeof(float) * (2 * D * 8 + 2 * 8 * TILE_TOK + TQ_MAX_CENTROIDS) + sizeof(uint64_t);
    dim3 grid((unsigned)((n_tokens + TILE_TOK - 1) / TILE_TOK), (unsigned)H, (unsigned)((n_q + 7) / 8));
    const int mse_bits = consts->cfg.key_bits - 1;
#define TQ_SC(DD, MB)                                                                                          \
    do {                                                                                                       \
        static TqSmemOptIn opt_in;                                                                             \
        if (tq_opt_in_smem(tq_scores_kernel<DD, MB>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;               \
        tq_scores_kernel<DD, MB><<<grid, DEC_THREADS, smem, st>>>(p, consts->cfg.key_bits, consts->cfg.value_bits); \
    } while (0)
    if (D == 128 && mse_bits == 2) TQ_SC(128, 2);
    else if (D == 128) TQ_SC(128, 3);
    else if (mse_bits == 2) TQ_SC(256, 2);
    else TQ_SC(256, 3);
#undef TQ_SC
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Decode for callers that cannot hand over scratch memory
// ---------------------------------------------------------------------------
// Some hosts of this library never get to call cudaMalloc themselves: a plugin
// running inside an engine that has claimed all device memory for its own KV
// pool up front, or code entered while the engine's allocator is locked (for
// instance between the engine's warm-up and its CUDA-graph replay).  For them
// the scratch of tq_decode lives in this fixed array inside the library image.
// Every GPU that loads the library carries these bytes until the process ends,
// which is why the size is kept modest.
#define TQ_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_tq_static_scratch[TQ_STATIC_SCRATCH_BYTES];

namespace {
void* g_static_scratch_ptr[TQ_MAX_DEVICES];   // device address of the array, per device ordinal
}  // namespace

extern "C" size_t tq_decode_static_scratch_bytes(void) { return (size_t)TQ_STATIC_SCRATCH_BYTES; }

namespace {

// Small step inputs are pulled from mapped host memory by a one-CTA kernel: a copy-engine
// transfer between two kernels of a stream costs several microseconds of switching.  Launched
// with programmatic stream serialisation, it reads the host buffer into registers while the
// kernel ahead of it is still running and writes the device buffer (which that kernel may be
// reading) only after it has completed.
__global__ void __launch_bounds__(1024) tq_stage_in_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int n16) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint4 v[4];   // n16 <= 4096
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = threadIdx.x + u * 1024;
        if (i < n16) v[u] = src[i];
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = threadIdx.x + u * 1024;
        if (i < n16) dst[i] = v[u];
    }
}

constexpr size_t HOST_IO_DIRECT_MAX = 64 * 1024;

// true when the GPU may dereference `ptr` itself: page-locked (pinned or registered) host memory
// under unified addressing.  Step buffers are reused, so the last few answers are remembered per
// device; tq_host_buffer_forget drops them when a buffer is unregistered or freed.
struct HostPtrCache {
    const void* ptr[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t bytes[4] = {0, 0, 0, 0};
    int next = 0;
};
HostPtrCache g_host_ptr_cache[TQ_MAX_DEVICES];
std::mutex g_host_ptr_mu;   // callers may come from several host threads

bool host_ptr_is_mapped(const void* ptr, size_t bytes) {
    const int dev = tq_current_device();
    if (dev < 0 || dev >= TQ_MAX_DEVICES) return false;
    std::lock_guard<std::mutex> lock(g_host_ptr_mu);
    HostPtrCache& c = g_host_ptr_cache[dev];
    for (int i = 0; i < 4; ++i)
        if (c.ptr[i] == ptr && c.bytes[i] >= bytes) return true;
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (at.type != cudaMemoryTypeHost || at.devicePointer != ptr) return false;
    cudaPointerAttributes at2;   // the end of the range must belong to the same registration
    if (cudaPointerGetAttributes(&at2, (const char*)ptr + bytes - 1) != cudaSuccess || at2.type != cudaMemoryTypeHost) {
        cudaGetLastError();
        return false;
    }
    c.ptr[c.next] = ptr;
    c.bytes[c.next] = bytes;
    c.next = (c.next + 1) & 3;
    return true;
}

}  // namespace

extern "C" int tq_host_buffer_forget(const void* host_ptr) {
    std::lock_guard<std::mutex> lock(g_host_ptr_mu);
    for (int d = 0; d < TQ_MAX_DEVICES; ++d)
        for (int i = 0; i < 4; ++i)
            if (host_ptr == nullptr || g_host_ptr_cache[d].ptr[i] == host_ptr) {
                g_host_ptr_cache[d].ptr[i] = nullptr;
                g_host_ptr_cache[d].bytes[i] = 0;
            }
    return TQ_OK;
}

extern "C" int tq_decode_host_io(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* a,
                                 const void* host_in, void* dev_in, size_t in_bytes, void* host_out, size_t out_bytes,
                                 void* stream) {
    if (!a) return TQ_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    tq_decode_args b = *a;
    int early_inputs = 0;
    if (host_in != nullptr && in_bytes > 0) {
        if (!dev_in) return TQ_ERR_NULL;
        const bool direct = in_bytes <= HOST_IO_DIRECT_MAX && (in_bytes & 15) == 0 &&
                            (((uintptr_t)host_in | (uintptr_t)dev_in) & 15) == 0 && host_ptr_is_mapped(host_in, in_bytes);
        // Arguments that point into dev_in can be redirected into the mapped host buffer: the query
        // preparation then reads them itself, before it waits for the kernel ahead of it, and no
        // transfer of its own sits on the stream.  (The ring CTAs read the raw query from there too.)
        auto inside = [&](const void* p) {
            return p != nullptr && (const char*)p >= (const char*)dev_in && (const char*)p < (const char*)dev_in + in_bytes;
        };
        auto redirect = [&](const void* p) { return (const void*)((const char*)host_in + ((const char*)p - (const char*)dev_in)); };
        const bool all_inside = inside(a->query) && (a->append_k == nullptr || (inside(a->append_k) && inside(a->append_v)));
        if (direct && all_inside && !a->query_prepared) {
            b.query = redirect(a->query);
            if (a->append_k != nullptr) {
                b.append_k = redirect(a->append_k);
                b.append_v = redirect(a->append_v);
            }
            early_inputs = 1;
        } else if (direct) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1);
            cfg.blockDim = dim3(1024);
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = tq_pdl_for_decode(st);
            tq_note_launch(st, TQ_LAUNCH_DECODE);
            if (cudaLaunchKernelEx(&cfg, tq_stage_in_kernel, (const uint4*)host_in, (uint4*)dev_in, (int)(in_bytes / 16)) !=
                cudaSuccess)
                return TQ_ERR_CUDA;
        } else if (cudaMemcpyAsync(dev_in, host_in, in_bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) {
            return TQ_ERR_CUDA;
        }
    }
    // a small result is written to mapped host memory by the merge itself
    const bool out_direct = host_out != nullptr && out_bytes > 0 && out_bytes <= HOST_IO_DIRECT_MAX &&
                            ((uintptr_t)host_out & 15) == 0 && host_ptr_is_mapped(host_out, out_bytes);
    if (out_direct) b.out = host_out;
    const int rc = decode_impl(consts, pool, &b, stream, early_inputs);
    if (rc != TQ_OK) return rc;
    if (host_out != nullptr && out_bytes > 0 && !out_direct) {
        if (cudaMemcpyAsync(host_out, a->out, out_bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess) return TQ_ERR_CUDA;
    }
    return TQ_OK;
}


// Device address of the built-in array on the current device, looked up on first use.
static int static_scratch_address(void** out) {
    const int dev = tq_current_device();
    if (dev < 0 || dev >= TQ_MAX_DEVICES) return TQ_ERR_CUDA;
    if (g_static_scratch_ptr[dev] == nullptr) {
        // In host code the array's name is only a handle; the kernels need the
        // address the symbol has on THIS device.  Looked up once per device, on
        // the first call made with that device current.
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_tq_static_scratch) != cudaSuccess || ptr == nullptr) return TQ_ERR_CUDA;
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return TQ_OK;
}

extern "C" int tq_decode_static(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* a, void* stream) {
    if (!consts || !pool || !a) return TQ_ERR_NULL;
    if (a->batch <= 0 || pool->num_kv_heads <= 0) return TQ_ERR_SHAPE;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != TQ_OK) return rc;
    tq_decode_args b = *a;
    b.workspace = scratch;
    b.workspace_bytes = TQ_STATIC_SCRATCH_BYTES;
    b.query_prepared = 0;   // the prepared query of an earlier call may have been overwritten by another caller
    // Everything the host can check is checked before anything is enqueued (a refused call leaves the
    // array as it was); TQ_ERR_WORKSPACE when the launch needs more than the array.
    rc = decode_impl(consts, pool, &b, stream, 0, /*validate_only=*/1);
    if (rc != TQ_OK) return rc;
    // The array keeps whatever the previous call left.  The per-(sequence, head) tickets must start at
    // zero: a call that was cut short (or overlapped another one) may have left them counting.  The
    // status word in front of them is NOT cleared: an error stays until tq_decode_static_read_status
    // has reported it.
    const size_t tickets = (((size_t)a->batch * pool->num_kv_heads * sizeof(int32_t) + 255) / 256) * 256;
    if (cudaMemsetAsync((char*)scratch + TQ_WS_HEADER_BYTES, 0, tickets, (cudaStream_t)stream) != cudaSuccess)
        return TQ_ERR_CUDA;
    return decode_impl(consts, pool, &b, stream, 0, 0);
}

extern "C" int tq_decode_static_read_status(void* stream, int32_t* out) {
    if (!out) return TQ_ERR_NULL;
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != TQ_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t v = 0;
    if (cudaMemcpyAsync(&v, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess) return TQ_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return TQ_ERR_CUDA;
    if (v != 0 && cudaMemsetAsync(scratch, 0, sizeof(int32_t), st) != cudaSuccess) return TQ_ERR_CUDA;   // reported: clear
    *out = v;
    return TQ_OK;
}
