// Pieces shared by the two decode kernels (CUDA-core and tensor-core): launch
// parameters, tile loading, the exact-ring part, and the ticketed merge of the
// per-CTA partial results.
#pragma once
#include "tq_common.cuh"

namespace tqdec {

constexpr int DEC_THREADS = 128;
constexpr int TILE_BLOCKS = 4;
constexpr int TILE_TOK = TILE_BLOCKS * TQ_BLOCK_TOKENS;  // 64
constexpr int NSTAGE = 3;
constexpr int RING_TOK = 32;  // ring tokens a ring CTA stages at a time


struct DecodeParams {
    const uint8_t* pool;
    int64_t num_blocks;
    int H, Qh, G;
    const int32_t* block_table;
    int bt_stride;
    const int32_t* seq_lens;
    int max_seq_len;     // host upper bound of seq_lens
    int min_history;
    const float* qprep;  // [B][Qh][2][D] rotated / sketched query
    const uint32_t* qfrag;   // per (sequence, kv head): the same query as fp16 MMA fragments (see QF_*)
    const void* query;
    int q_dtype;
    const void* ring_k;
    const void* ring_v;
    int ring_dtype;
    const int32_t* ring_lens;
    int max_ring_len;    // host upper bound of ring_lens (sizes the ring CTAs)
    int64_t ring_stride_seq, ring_stride_token;
    float scale, qjl_scale;
    TqCodebook cb;
    void* out;
    float* partials;
    int32_t* tickets;
    int32_t* status;
    int num_splits, ring_splits;
    int ring_tok;          // ring tokens per ring CTA, a multiple of RING_TOK
    uint32_t land_bytes;   // tensor-core kernel: shared memory in front of its barriers, reusable by the merge
};

// ---- operand geometry of the tensor-core kernel, shared with the query preparation ----
// Thread (gid = lane/4, tig = lane%4).  Score MMA k-step s uses B/A register pair
// r = 2s, 2s+1; register r covers dims d_lo = (D/4)*tig + 16*(r/8) + r%8 (low half)
// and d_lo + 8 (high half): the two 16-bit halves of code word r/8, field j = r%8.
__host__ __device__ constexpr int code_pos(int j) { return j <= 4 ? j : j - 3; }            // 2-bit field index after the optional >>6
__host__ __device__ constexpr int sign_bit(int wi, int j) { return j + 8 * (wi & 1); }      // bit in the byte-swapped sign word
__host__ __device__ constexpr int sign_pos(int b) { return b <= 9 ? b : b - 6; }

// Query fragments of one (sequence, kv head): QF_HDR floats (exponent of the
// rotated query per head [8], of the sketched query per head [8]) followed by
// `sets` x (D/8) registers x 32 lanes of packed fp16 pairs.  With G <= 4 there
// is one set: B-fragment columns 0-3 hold the rotated query of heads 0-3
// scaled by 2^(e - 2*code_pos), columns 4-7 the sketched query scaled by
// 2^(e - sign_pos); with G > 4 set 0 is the rotated, set 1 the sketched query.
constexpr int QF_HDR = 16;
__host__ __device__ constexpr int qf_words(int D, int G) { return QF_HDR + (G > 4 ? 2 : 1) * (D / 8) * 32; }

struct ScoreParams {
    const uint8_t* pool;
    int64_t num_blocks;
    int H;
    const int32_t* block_table;
    int64_t n_tokens;
    const float* qprep;  // [H][n_q][2][D]
    int n_q;
    float qjl_scale;
    TqCodebook cb;
    float* logits;  // [H][n_q][n_tokens]
    int32_t* status;
};

// Partial logits of one token over dims [dim0, dim0 + D/2) for GP query heads.
template <int D, int MSE_BITS, int GP>
__device__ __forceinline__ void token_half_scores(const uint8_t* rec, const TqLayout& L, int tl, int half,
                                                  const float* __restrict__ qr, const float* __restrict__ qs,
                                                  const float* __restrict__ cent, float qjl_scale, float (&out)[GP]) {
    constexpr int WIDTH = MSE_BITS == 2 ? 2 : 4;
    constexpr int DIMS_PER_CW = 32 / WIDTH;       // dims per 32-bit code word
    constexpr int CW_PER_SW = 32 / DIMS_PER_CW;   // code words per 32-bit sign word
    constexpr uint32_t MASK = (1u << WIDTH) - 1u;
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(rec + L.off_kcodes + tl * L.kcode_row) + half * (D / 2) / DIMS_PER_CW;
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(rec + L.off_ksigns + tl * L.ksign_row) + half * (D / 64);
    float am[GP], aq[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) am[g] = aq[g] = 0.f;
    int j = half * (D / 2);
#pragma unroll 1
    for (int s = 0; s < D / 64; ++s) {
        uint32_t sg = sw[s];
#pragma unroll
        for (int c = 0; c < CW_PER_SW; ++c) {
            uint32_t w = cw[s * CW_PER_SW + c];
#pragma unroll 4
            for (int i = 0; i < DIMS_PER_CW; ++i, ++j) {
                const float cv = cent[w & MASK];
                w >>= WIDTH;
                const float sv = (sg & 1u) ? 1.f : -1.f;
                sg >>= 1;
                const float* qrj = qr + j * GP;
                const float* qsj = qs + j * GP;
#pragma unroll
                for (int g4 = 0; g4 < GP / 4; ++g4) {
                    const float4 a = *reinterpret_cast<const float4*>(qrj + 4 * g4);
                    const float4 b = *reinterpret_cast<const float4*>(qsj + 4 * g4);
                    am[4 * g4 + 0] = fmaf(a.x, cv, am[4 * g4 + 0]);
                    am[4 * g4 + 1] = fmaf(a.y, cv, am[4 * g4 + 1]);
                    am[4 * g4 + 2] = fmaf(a.z, cv, am[4 * g4 + 2]);
                    am[4 * g4 + 3] = fmaf(a.w, cv, am[4 * g4 + 3]);
                    aq[4 * g4 + 0] = fmaf(b.x, sv, aq[4 * g4 + 0]);
                    aq[4 * g4 + 1] = fmaf(b.y, sv, aq[4 * g4 + 1]);
                    aq[4 * g4 + 2] = fmaf(b.z, sv, aq[4 * g4 + 2]);
                    aq[4 * g4 + 3] = fmaf(b.w, sv, aq[4 * g4 + 3]);
                }
            }
        }
    }
    const float norm = __half2float(reinterpret_cast<const __half*>(rec + L.off_knorm)[tl]);
    const float rn = __half2float(reinterpret_cast<const __half*>(rec + L.off_krnorm)[tl]) * qjl_scale;
#pragma unroll
    for (int g = 0; g < GP; ++g) out[g] = norm * am[g] + rn * aq[g];
}

// Issue the bulk copies of one tile (up to 4 block records) into a stage.
static __device__ __forceinline__ void issue_tile(uint8_t* stage, uint64_t* bar, const uint8_t* pool, int64_t num_blocks,
                                           const int32_t* bt, int first_blk, int nblk_total, int H, int h,
                                           int block_bytes, int32_t* status) {
    const int nb = min(TILE_BLOCKS, nblk_total - first_blk);
    tq_mbar_expect_tx(bar, (uint32_t)(nb * block_bytes));
    for (int i = 0; i < nb; ++i) {
        int64_t phys = bt[first_blk + i];
        if (phys < 0 || phys >= num_blocks) {
            if (status) atomicCAS(status, 0, (int)TQ_ERR_RANGE);
            phys = 0;
        }
        tq_bulk_g2s(stage + i * block_bytes, pool + (phys * H + h) * (int64_t)block_bytes, (uint32_t)block_bytes, bar);
    }
}

// Partial result of one CTA: m[GP] (natural-log domain), l[GP], acc[GP][D].
template <int D, int GP>
__device__ __forceinline__ float* partial_ptr(const DecodeParams& p, int b, int h, int slot_idx) {
    const int nslot = p.num_splits + p.ring_splits;
    return p.partials + ((int64_t)(b * p.H + h) * nslot + slot_idx) * (GP * (D + 2));
}

// Each thread owns D/128 consecutive channels of every query head.
template <int D, int GP>
__device__ __forceinline__ void write_partial_regs(const DecodeParams& p, int b, int h, int slot_idx,
                                                   const float (&acc)[GP][D / DEC_THREADS], const float* m_run,
                                                   const float* l_run) {
    constexpr int DPT = D / DEC_THREADS;
    const int tid = threadIdx.x;
    float* mine = partial_ptr<D, GP>(p, b, h, slot_idx);
    if (tid < GP) {
        mine[tid] = m_run[tid];
        mine[GP + tid] = l_run[tid];
    }
#pragma unroll
    for (int g = 0; g < GP; ++g)
#pragma unroll
        for (int i = 0; i < DPT; ++i) mine[2 * GP + g * D + tid * DPT + i] = acc[g][i];
}

// After a CTA has written its partial: take a ticket; the last CTA of this
// (sequence, kv head) merges all partials and writes the output.  Nobody waits.
// Every partial is always fully written with finite numbers, so the merge is
// branch free: a float4 of one head per thread, slots unrolled.
//
// `land` / `land_bytes`: shared memory the CTA no longer needs.  When all the
// partials of the pair fit there, the last CTA fetches them with bulk copies
// (one trip to L2 instead of a chain of dependent loads) and merges out of
// shared memory; otherwise it reads them from global memory.
template <int D, int GP>
__device__ __forceinline__ void ticket_and_merge(const DecodeParams& p, int b, int h,
                                                 float* wsm /* [max(nslot,128)*GP + 2*GP] */,
                                                 uint8_t* land = nullptr, uint32_t land_bytes = 0) {
    constexpr int PS = GP * (D + 2);
    const int tid = threadIdx.x, nt = blockDim.x;
    const int nslot = p.num_splits + p.ring_splits;
    __shared__ int s_last;
    __shared__ __align__(8) uint64_t s_bar;
    __syncthreads();          // every thread's part of the partial is written ...
    if (tid == 0) {
        // ... and, release being cumulative, visible device-wide before the ticket; the acquire half orders
        // the last CTA's reads of the other partials behind it
        int t;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.tickets + b * p.H + h) : "memory");
        s_last = (t == nslot - 1);
    }
    __syncthreads();
    if (!s_last) return;

    const float* base = p.partials + (int64_t)(b * p.H + h) * nslot * PS;
    const uint32_t total = (uint32_t)nslot * PS * 4u;
    const bool staged = land != nullptr && total <= land_bytes && total < (1u << 20);
    if (staged) {
        if (tid == 0) {
            tq_mbar_init(&s_bar, 1);
            tq_mbar_fence_init();
            asm volatile("fence.proxy.async;" ::: "memory");   // other CTAs' generic writes -> this bulk read
            tq_mbar_expect_tx(&s_bar, total);
            for (uint32_t off = 0; off < total; off += 32768u)
                tq_bulk_g2s(land + off, reinterpret_cast<const uint8_t*>(base) + off, min(32768u, total - off), &s_bar);
        }
        __syncthreads();
        bool ok = tq_mbar_wait_bounded(&s_bar, 0u);
        if (!__syncthreads_and(ok)) {   // never arrived: report; the kernel must not touch `land` again
            if (tid == 0) {
                atomicCAS(p.status, 0, (int)TQ_ERR_TIMEOUT);
                p.tickets[b * p.H + h] = 0;   // the output of this launch is lost, the workspace stays usable
            }
            return;
        }
        // Out of shared memory: a thread owns four channels of one head; the head is the same for a whole
        // warp, so the warp works out the slots' weights once into its own row of `wsm` (padded with
        // zeros to a multiple of eight) and then takes the slots eight at a time, all loads first.
        const float* sb = reinterpret_cast<const float*>(land);
        const int lane = tid & 31;
        const int items = p.G * (D / 4);
        const int wstride = (nslot + 7) & ~7;
        float* ww = wsm + (tid >> 5) * wstride;   // tensor-core kernel: wsm holds one row of max(nslot,128) + 8 floats per warp
        for (int i0 = (tid >> 5) * 32; i0 < items; i0 += nt) {   // D/4 is a multiple of 32: one head per warp pass
            const int i = i0 + lane;
            const int g = i0 / (D / 4), d = (i % (D / 4)) * 4;
            float mx = -INFINITY;
            for (int s = lane; s < nslot; s += 32) mx = fmaxf(mx, sb[s * PS + g]);
            mx = tq_warp_max(mx);
            float l = 0.f;
            for (int s = lane; s < wstride; s += 32) {
                float wm = 0.f;
                if (s < nslot) {
                    const float ms = sb[s * PS + g];
                    wm = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
                    l = fmaf(wm, sb[s * PS + GP + g], l);
                }
                ww[s] = wm;
            }
            l = tq_warp_sum(l);
            __syncwarp();
            const float4* src = reinterpret_cast<const float4*>(sb + 2 * GP + g * D + d);
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < nslot; s += 8) {
                float4 v[8];
                float w8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    v[u] = src[min(s + u, nslot - 1) * (PS / 4)];   // past the end: a valid slot, weight 0
                    w8[u] = ww[s + u];
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    o.x = fmaf(w8[u], v[u].x, o.x);
                    o.y = fmaf(w8[u], v[u].y, o.y);
                    o.z = fmaf(w8[u], v[u].z, o.z);
                    o.w = fmaf(w8[u], v[u].w, o.w);
                }
            }
            __syncwarp();   // the row of weights is rewritten by the warp's next pass
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const int64_t dst = ((int64_t)b * p.Qh + h * p.G + g) * D + d;
            tq_store4_any(p.out, dst, o.x * inv, o.y * inv, o.z * inv, o.w * inv, p.q_dtype);
        }
        if (tid == 0) p.tickets[b * p.H + h] = 0;  // ready for the next launch
        return;
    }

    float* wL = wsm;             // [GP] global sum
    float* w = wsm + 2 * GP;     // [nslot][GP] weight of each partial
    const int warp = tid >> 5, lane = tid & 31;
    for (int g = warp; g < GP; g += nt / 32) {
        float mx = -INFINITY;
        for (int s = lane; s < nslot; s += 32) mx = fmaxf(mx, __ldcg(base + (int64_t)s * PS + g));
        mx = tq_warp_max(mx);
        float sum = 0.f;
        for (int s = lane; s < nslot; s += 32) {
            const float ms = __ldcg(base + (int64_t)s * PS + g);
            const float ls = __ldcg(base + (int64_t)s * PS + GP + g);
            const float ws = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
            w[s * GP + g] = ws;
            sum += ws * ls;
        }
        sum = tq_warp_sum(sum);
        if (lane == 0) wL[g] = sum;
    }
    __syncthreads();
    for (int i = tid; i < p.G * (D / 4); i += nt) {
        const int g = i / (D / 4), d = (i % (D / 4)) * 4;
        const float4* src = reinterpret_cast<const float4*>(base + 2 * GP + g * D + d);   // PS*4 and (2GP+gD+d)*4 are multiples of 16
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        int s = 0;
        for (; s + 8 <= nslot; s += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(src + (int64_t)(s + u) * (PS / 4));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float ws = w[(s + u) * GP + g];
                o.x = fmaf(ws, v[u].x, o.x);
                o.y = fmaf(ws, v[u].y, o.y);
                o.z = fmaf(ws, v[u].z, o.z);
                o.w = fmaf(ws, v[u].w, o.w);
            }
        }
        for (; s < nslot; ++s) {
            const float4 v = __ldcg(src + (int64_t)s * (PS / 4));
            const float ws = w[s * GP + g];
            o.x = fmaf(ws, v.x, o.x);
            o.y = fmaf(ws, v.y, o.y);
            o.z = fmaf(ws, v.z, o.z);
            o.w = fmaf(ws, v.w, o.w);
        }
        const float l = wL[g];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int64_t dst = ((int64_t)b * p.Qh + h * p.G + g) * D + d;
        tq_store4_any(p.out, dst, o.x * inv, o.y * inv, o.z * inv, o.w * inv, p.q_dtype);
    }
    if (tid == 0) p.tickets[b * p.H + h] = 0;  // ready for the next launch
}

// Exact attention over this CTA's slice of the ring: p.ring_tok tokens, taken RING_TOK (32) at a
// time, fp32 like the reference's matmul path (score.py:154-170); works for any block size.  The
// sub-slice's key and value rows are first staged in shared memory with 16-byte loads that are all
// in flight at once; everything after that runs out of shared memory.  Sub-slices are merged with
// the usual running max / sum; the CTA writes its partial itself.
// scratch: qf [D][GP], sc [GP][RING_TOK], pp [RING_TOK][GP] floats, ml [2*GP],
//          kst / vst: RING_TOK * D * element size bytes each, 16-byte aligned.
template <int D, int GP>
__device__ __forceinline__ void ring_part(const DecodeParams& p, int b, int h, int slot_idx, float* qf, float* sc,
                                          float* pp, float* ml, uint8_t* kst, uint8_t* vst) {
    constexpr int MAX_OWN = (GP * D + 127) / 128;   // outputs per thread with at least 128 threads
    const int tid = threadIdx.x, nt = blockDim.x, warp = tid >> 5, lane = tid & 31;
    const int rs = slot_idx - p.num_splits;
    int R = p.ring_lens ? p.ring_lens[b] : 0;
    if (R > p.max_ring_len) {   // more than the host promised: the ring CTAs only cover max_ring_len tokens
        if (tid == 0) atomicCAS(p.status, 0, (int)TQ_ERR_RANGE);
        R = p.max_ring_len;
    }
    float* mine = partial_ptr<D, GP>(p, b, h, slot_idx);
    // running state: ml[0..GP) max, ml[GP..2GP) sum (shared), acc of this thread's outputs (registers)
    float acc[MAX_OWN];
#pragma unroll
    for (int u = 0; u < MAX_OWN; ++u) acc[u] = 0.f;
    if (tid < GP) {
        ml[tid] = -INFINITY;
        ml[GP + tid] = 0.f;
    }
    const int eb = p.ring_dtype == TQ_F32 ? 4 : 2;
    const int row_chunks = D * eb / 16;
    bool have_q = false;
    for (int sub = 0; sub < p.ring_tok / RING_TOK; ++sub) {
        const int r0 = rs * p.ring_tok + sub * RING_TOK;
        const int nr = max(0, min(RING_TOK, R - r0));
        if (nr <= 0) break;   // uniform over the CTA
        __syncthreads();      // the previous sub-slice is consumed
        for (int i = tid; i < nr * row_chunks; i += nt) {
            const int t = i / row_chunks, c = i % row_chunks;
            const int64_t off = ((int64_t)b * p.ring_stride_seq + (int64_t)(r0 + t) * p.ring_stride_token +
                                 (int64_t)h * D) * eb + c * 16;
            reinterpret_cast<uint4*>(kst)[i] = *reinterpret_cast<const uint4*>((const char*)p.ring_k + off);
            reinterpret_cast<uint4*>(vst)[i] = *reinterpret_cast<const uint4*>((const char*)p.ring_v + off);
        }
        if (!have_q) {
            for (int i = tid; i < D * GP; i += nt) {
                const int j = i / GP, g = i % GP;
                qf[i] = g < p.G ? tq_load_any(p.query, ((int64_t)b * p.Qh + h * p.G + g) * D + j, p.q_dtype) : 0.f;
            }
            have_q = true;
        }
        __syncthreads();
        for (int t = warp; t < nr; t += nt / 32) {
            float a[GP];
#pragma unroll
            for (int g = 0; g < GP; ++g) a[g] = 0.f;
            for (int j = lane; j < D; j += 32) {
                const float kx = tq_load_any(kst, t * D + j, p.ring_dtype);
#pragma unroll
                for (int g = 0; g < GP; ++g) a[g] = fmaf(qf[j * GP + g], kx, a[g]);
            }
#pragma unroll
            for (int g = 0; g < GP; ++g) {
                const float s = tq_warp_sum(a[g]);
                if (lane == 0) sc[g * RING_TOK + t] = s * p.scale;
            }
        }
        __syncthreads();
        // per head: new running max, probabilities of this sub-slice, factor for what came before
        for (int g = warp; g < GP; g += nt / 32) {
            const float s0 = lane < nr ? sc[g * RING_TOK + lane] : -INFINITY;
            const float m_old = ml[g];
            const float m_new = fmaxf(m_old, tq_warp_max(s0));
            const float p0 = (s0 == -INFINITY) ? 0.f : __expf(s0 - m_new);
            const float sum = tq_warp_sum(p0);
            pp[lane * GP + g] = p0;
            if (lane == 0) {
                const float alpha = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
                sc[g * RING_TOK] = alpha;        // the scores of this head are consumed: reuse slot 0
                ml[g] = m_new;
                ml[GP + g] = ml[GP + g] * alpha + sum;
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < MAX_OWN; ++u) {
            const int i = tid + u * nt;
            if (i < GP * D) {
                const int g = i / D, d = i % D;
                float a = acc[u] * sc[g * RING_TOK];
                for (int t = 0; t < nr; ++t) a = fmaf(pp[t * GP + g], tq_load_any(vst, t * D + d, p.ring_dtype), a);
                acc[u] = a;
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < MAX_OWN; ++u) {
        const int i = tid + u * nt;
        if (i < GP * D) mine[2 * GP + i] = acc[u];
    }
    if (tid < 2 * GP) mine[tid] = ml[tid];
}

// Launcher of the tensor-core kernel (tq_decode_mma.cu); *handled = 0 when the
// configuration is outside what it covers and the CUDA-core kernel must run.
int tq_decode_mma_launch(const DecodeParams& p, int D, int mse_bits, int val_bits, int batch, int max_seq_len,
                         cudaStream_t st, int* handled);

}  // namespace tqdec

// Tensor-core query preparation (tq_qprep_tc.cu): *handled = 0 when the call does not fit it.
int tq_qprep_tc_launch(const tq_consts* consts, const void* q, int dt, int64_t nvec, float* out, uint32_t* frag, int G,
                       int Qh, int mse_bits, int* status, cudaStream_t st, int* handled);
