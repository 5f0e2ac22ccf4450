// Tensor-core decode attention over compressed block records.
//
// Decode is HBM-bound only if the arithmetic is almost free: a record of
// 100-196 bytes carries 3*D*G multiply-adds, far beyond what CUDA cores can do
// at HBM speed.  So every contraction runs on the tensor cores (mma.sync
// m16n8k16, fp16 in / fp32 accumulate) with operands expanded from the packed
// codes IN REGISTERS, one logic instruction per pair of elements:
//
//  * A 16-token block record is exactly one MMA row tile.  A warp owns whole
//    records, streams them through a private 4-stage ring of bulk (TMA) copies
//    and keeps its own online-softmax state; warps never synchronise in the
//    main loop.
//  * A single bit kept in place inside a 16-bit lane IS an fp16 number
//    (bit b <= 9 is the subnormal 2^(b-24)); a 2/4-bit field is the subnormal
//    code * 2^(pos-24).  So `word & mask` yields an A-operand register holding
//    two elements.  The per-position power of two is folded into the B operand
//    (scores) or into a per-row factor applied once at the end (values).
//  * Scores: the 2-bit MSE code is used as two bit planes because the code book
//    is affine in the bits (c = c0 + (c1-c0) b0 + (c2-c0) b1 for a symmetric
//    4-level book), the QJL signs are a third bit plane.  With G <= 4 query
//    heads per kv head, columns 0-3 of the B fragment hold the rotated query
//    and columns 4-7 the sketched query, so one B fragment serves all planes.
//  * Values: out[d][g] = sum_n code[n][d] * (p[n][g] * scale[n][grp(d)])
//                        + sum_n p[n][g] * zero[n][grp(d)];
//    the 16 rows of an MMA tile are 16 channels of one group, the contraction
//    runs over the 16 tokens, the group scale rides on the probabilities and
//    the zero-point term is one more small MMA.
#include "tq_decode_common.cuh"

using namespace tqdec;

namespace {

constexpr int NSTW = 4;    // bulk-copy stages per warp, one block record each
// Warps per CTA.  A launch that fits one wave runs 12-warp CTAs, one per SM (all of an SM's warps
// share one set of query fragments and one merge).  A launch of several waves runs 8-warp CTAs, two
// per SM, so that the set-up and the merge of one CTA overlap the main loop of the other.
constexpr int NW_WAVE = 12;
constexpr int NW_MULTI = 8;
constexpr int BT_MAX = 1024;   // block-table entries a CTA keeps in shared memory


// 2^x for x <= 0 (softmax terms): the bare approximation instruction, results below 2^-126 flush to 0
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((127 + e) << 23); }   // 2^e, -126 <= e <= 127

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Same with a zero accumulator coming in (the first k-step of a record: no register clearing).
__device__ __forceinline__ void mma16816_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t hmul2_sat(uint32_t a, uint32_t b) {
    const __half2 r = __hmin2(__hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b)),
                              __floats2half2_rn(65504.f, 65504.f));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// MSE_BITS == 2: bit-plane scores as described above.  MSE_BITS == 3 (codes in nibbles, 8 centroids): the
// nibbles are byte-table selectors - two PRMTs look up the low and high bytes of four fp16 centroids, two more
// interleave them into two A registers - so the A operand holds true centroid values, one plane, and the
// rotated query needs no per-position scaling; it always uses separate rotated / sketched fragment sets.
template <int D, int MSE_BITS, int VAL_BITS, bool SPLITB, int NW>
__global__ void __launch_bounds__(NW * 32, NW == NW_MULTI ? 2 : 1) tq_decode_mma_kernel(const DecodeParams p) {
    static_assert(MSE_BITS == 2 || SPLITB, "3-bit codes use separate rotated / sketched fragment sets");
    constexpr int NT = NW * 32;
    constexpr int GP = SPLITB ? 8 : 4;
    constexpr int KS = D / 16;    // score k-steps
    constexpr int NWK = D / 64;   // 32-bit words of 2-bit codes per thread per token; twice the sign words
    constexpr int NMB = D / 16;   // value M-blocks
    constexpr int NG = D / 32;
    const TqLayout L = tq_make_layout(D, MSE_BITS + 1, VAL_BITS);
    const int BB = L.block_bytes;

    extern __shared__ __align__(128) uint8_t smem[];
    // [0, land_bytes): stages, ml, bt_s (+ padding) - all dead once the CTA's partial is written, so the
    // merge may land every partial of the pair there
    uint8_t* stages = smem;                                              // [NW warps][NSTW][BB]; reused after the loop
    float* ml = reinterpret_cast<float*>(smem + NW * NSTW * BB);         // [NW warps][2][GP]
    int* bt_s = reinterpret_cast<int*>(ml + 2 * NW * GP);                // [BT_MAX] physical blocks of this CTA
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.land_bytes);   // [NW][NSTW] + 1 for the query fragments
    uint32_t* qf_s = reinterpret_cast<uint32_t*>(bars + NW * NSTW + 2);  // query fragments of this (sequence, kv head)
    float* wsm = reinterpret_cast<float*>(qf_s + qf_words(D, SPLITB ? 8 : 4));   // merge scratch

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;
    // kv head fastest, slot next: the ring slots (x >= num_splits) are the last CTAs of a sequence in launch
    // order.  When this grid starts under the tail of the previous kernels, the CTAs that find their SM still
    // taken by the query preparation are then ring CTAs, which are off the critical path.
    const int b = blockIdx.z, h = blockIdx.x, x = blockIdx.y;
    // a kernel launched behind this one with programmatic stream serialisation may be scheduled as soon
    // as every CTA of this grid is running; whatever it reads of ours it reads after its own wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (x >= p.num_splits) {
        // exact ring tokens: CUDA-core fp32 path shared with the generic kernel.  The ring and its
        // length may have been written by the query-prep grid this launch overlaps with.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        float* scratch = reinterpret_cast<float*>(stages);
        uint8_t* kst = reinterpret_cast<uint8_t*>(scratch + D * GP + 2 * GP * RING_TOK);   // 16-byte aligned
        ring_part<D, GP>(p, b, h, x, scratch, scratch + D * GP, scratch + D * GP + GP * RING_TOK, ml, kst,
                         kst + RING_TOK * D * 4);
        ticket_and_merge<D, GP>(p, b, h, wsm, smem, p.land_bytes);
        return;
    }

    // ------------------------------ this CTA's share of the history ------------------------------
    constexpr uint32_t QF_BYTES = qf_words(D, SPLITB ? 8 : 4) * 4u;
    int n = p.seq_lens[b];
    if (n > p.max_seq_len) {   // the host bound sized the grid, the block table and this CTA's table slice
        if (tid == 0) atomicCAS(p.status, 0, (int)TQ_ERR_RANGE);
        n = p.max_seq_len;
    }
    if (n < p.min_history) n = 0;
    const uint32_t nblk = (uint32_t)(n + TQ_BLOCK_TOKENS - 1) / TQ_BLOCK_TOKENS;
    // 32-bit arithmetic: the launcher keeps num_splits * nblk below 2^31
    const int blk0 = (int)((uint32_t)x * nblk / (uint32_t)p.num_splits);
    const int blk1 = (int)((uint32_t)(x + 1) * nblk / (uint32_t)p.num_splits);
    const int nmine = min(blk1 - blk0, BT_MAX);   // the launcher guarantees <= BT_MAX blocks per split
    const int cnt = nmine > warp ? (nmine - warp + NW - 1) / NW : 0;   // records of this warp

    // block table slice and barriers first, so the copies overlap the query set-up
    const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
    for (int i = tid; i < nmine; i += NT) {
        int phys = bt[blk0 + i];
        if (phys < 0 || phys >= p.num_blocks) {
            atomicCAS(p.status, 0, (int)TQ_ERR_RANGE);
            phys = 0;
        }
        bt_s[i] = phys;
    }
    if (tid < NW * NSTW + 1) {   // one barrier per thread
        tq_mbar_init(bars + tid, 1);
        tq_mbar_fence_init();
    }
    __syncthreads();
    uint8_t* my_stage = stages + warp * NSTW * BB;
    uint64_t* my_bar = bars + warp * NSTW;
    // The query fragments belong to the kernels ahead of this launch until they have completed: the
    // query-prep grid of this call, or - when the caller says the query is already prepared - whatever
    // earlier call prepared it, which may still be running when this grid starts (every kernel of the
    // library lets its dependents start early).  Thread 0 waits for them and asks for the fragments
    // before its own warp's records, so that they queue behind as few record copies as possible; the
    // other warps start their copies at once.
    if (tid == 0) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        tq_mbar_expect_tx(bars + NW * NSTW, QF_BYTES);
        tq_bulk_g2s(qf_s, p.qfrag + (int64_t)(b * p.H + h) * qf_words(D, SPLITB ? 8 : 4), QF_BYTES, bars + NW * NSTW);
    }
    __syncwarp();
    if (lane < NSTW && lane < cnt) {   // one stage per lane
        tq_mbar_expect_tx(my_bar + lane, (uint32_t)BB);
        tq_bulk_g2s(my_stage + lane * BB, p.pool + ((int64_t)bt_s[warp + NW * lane] * p.H + h) * BB, (uint32_t)BB,
                    my_bar + lane);
    }

    // ---- query fragments, prepared once per (sequence, kv head) by the query-prep kernel ----
    // (launched with programmatic stream serialisation: everything above overlapped that kernel)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool failed = !__all_sync(0xffffffffu, tq_mbar_wait_bounded(bars + NW * NSTW, 0u));   // then no record is processed
    // Head_dim 256 with separate rotated / sketched sets: two sets of 32 fragment registers do not fit beside
    // the 64 value accumulators, so the fragments stay in shared memory and are read where they are used.
    constexpr bool BSM = (D == 256) && SPLITB;
    uint32_t bq[BSM ? 1 : 2 * KS];
    uint32_t bsk[(SPLITB && !BSM) ? 2 * KS : 1];
#define BQ(r) (BSM ? qf_s[QF_HDR + (r) * 32 + lane] : bq[BSM ? 0 : (r)])
#define BSK(r) (BSM ? qf_s[QF_HDR + (2 * KS + (r)) * 32 + lane] : bsk[(SPLITB && !BSM) ? (r) : 0])
    float k0[2], k1[2], kb0[2], ksg[2], kq[2];
    {
        const uint32_t* qf = qf_s;
        const float* hdr = reinterpret_cast<const float*>(qf);
        const int g_col = SPLITB ? gid : (gid & 3);             // head of this thread's B-fragment column
        const bool col_live = g_col < p.G;
        if (BSM) {
            if (!col_live)   // columns without a head: nobody wrote their fragments - clear this lane's words
                for (int r = 0; r < 4 * KS; ++r) qf_s[QF_HDR + r * 32 + lane] = 0u;
            __syncwarp();
        } else {
#pragma unroll
            for (int r = 0; r < 2 * KS; ++r) {
                bq[BSM ? 0 : r] = col_live ? qf[QF_HDR + r * 32 + lane] : 0u;
                if (SPLITB) bsk[(SPLITB && !BSM) ? r : 0] = col_live ? qf[QF_HDR + (2 * KS + r) * 32 + lane] : 0u;
            }
        }
        // Sums of the fp16-rounded query over all dims (the constant terms of the bit-plane form), taken
        // with the score MMAs themselves: an A operand with every code (sign) bit set multiplies each
        // fragment entry by the power of two its position stands for, so the accumulator of column g is
        // 2^(e-24) * sum_d q[g][d], in the lanes that hold column g's scores later.
        float one_c[4] = {0.f, 0.f, 0.f, 0.f}, one_s[4] = {0.f, 0.f, 0.f, 0.f};
        float one_c2[4] = {0.f, 0.f, 0.f, 0.f}, one_s2[4] = {0.f, 0.f, 0.f, 0.f};   // odd k-steps: shorter chains
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            const int wi = s >> 2, jj = s & 3;
            if (MSE_BITS == 2) {
                const uint32_t m0 = 0x00010001u << (2 * code_pos(2 * jj)), m1 = 0x00010001u << (2 * code_pos(2 * jj + 1));
                mma16816((s & 1) ? one_c2 : one_c, m0, m0, m1, m1, BQ(2 * s), BQ(2 * s + 1));
            }
            const uint32_t n0 = 0x00010001u << sign_pos(sign_bit(wi, 2 * jj));
            const uint32_t n1 = 0x00010001u << sign_pos(sign_bit(wi, 2 * jj + 1));
            mma16816((s & 1) ? one_s2 : one_s, n0, n0, n1, n1, SPLITB ? BSK(2 * s) : BQ(2 * s),
                     SPLITB ? BSK(2 * s + 1) : BQ(2 * s + 1));
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            one_c[c] += one_c2[c];
            one_s[c] += one_s2[c];
        }
        if (!SPLITB) {   // sketched-query columns 4..7 live two lanes to the right
            one_s[0] = __shfl_xor_sync(0xffffffffu, one_s[0], 2);
            one_s[1] = __shfl_xor_sync(0xffffffffu, one_s[1], 2);
        }
        // constants of this thread's two score columns g = 2*tig, 2*tig+1:
        // logit*log2e*scale = nk * (k0 + k1*acc1 + kb0*acc0) + rk * (ks*accs - kq)
        const float c0 = p.cb.centroids[0], c1 = p.cb.centroids[1], c2 = p.cb.centroids[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int g = (2 * tig + i) & (GP - 1);
            const int e_rot = (int)hdr[g], e_sk = (int)hdr[8 + g];
            const float s_rot = one_c[i] * pow2i(24 - e_rot), s_sk = one_s[i] * pow2i(24 - e_sk);
            if (MSE_BITS == 2) {
                k0[i] = c0 * s_rot;
                k1[i] = (c2 - c0) * pow2i(23 - e_rot);
                kb0[i] = (c1 - c0) * pow2i(24 - e_rot);
            } else {   // acc0 = sum centroid * (q * 2^e): undo the scale, no constant term, no second plane
                k0[i] = 0.f;
                k1[i] = 0.f;
                kb0[i] = pow2i(-e_rot);
            }
            ksg[i] = pow2i(25 - e_sk);
            kq[i] = s_sk;
        }
    }
    const float sm_scale = p.scale * 1.4426950408889634f;   // softmax in base 2
    const float qjl = p.qjl_scale;
    const bool col_ok = SPLITB || tig < 2;                   // this thread's score columns are real heads

    float o[NMB][4];
#pragma unroll
    for (int mb = 0; mb < NMB; ++mb)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[mb][c] = 0.f;
    float zacc[4] = {0.f, 0.f, 0.f, 0.f};
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    const int tokA = 4 * (gid >> 1) + (gid & 1), tokB = tokA + 2;   // tokens of score rows gid, gid+8
    // 3-bit codes: low / high bytes of the eight fp16 centroids, selectable by PRMT
    uint32_t t_lo0 = 0, t_lo1 = 0, t_hi0 = 0, t_hi1 = 0;
    if (MSE_BITS == 3) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t a = __half_as_ushort(__float2half_rn(p.cb.centroids[i]));
            const uint32_t c = __half_as_ushort(__float2half_rn(p.cb.centroids[4 + i]));
            t_lo0 |= (a & 0xffu) << (8 * i);
            t_hi0 |= (a >> 8) << (8 * i);
            t_lo1 |= (c & 0xffu) << (8 * i);
            t_hi1 |= (c >> 8) << (8 * i);
        }
    }

    for (int it = 0; it < cnt && !failed; ++it) {
        const int st = it % NSTW;
        bool ok = tq_mbar_wait_bounded(my_bar + st, (uint32_t)((it / NSTW) & 1));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            failed = true;
            break;
        }
        uint8_t* rec = my_stage + st * BB;
        const int blk = blk0 + warp + NW * it;
        const int valid = min(TQ_BLOCK_TOKENS, n - blk * TQ_BLOCK_TOKENS);
        if (valid < TQ_BLOCK_TOKENS) {
            // the sequence's last, partly filled record: unused slots may hold anything.  Their scores are
            // masked below; their value scales and zero points ([grp][16 tok] fp16, contiguous) are cleared
            // here, so that probability 0 times a stale Inf/NaN cannot reach the value MMAs.
            __half* sz = reinterpret_cast<__half*>(rec + L.off_vscale);
            for (int i = lane; i < 2 * NG * TQ_BLOCK_TOKENS; i += 32)
                if ((i & (TQ_BLOCK_TOKENS - 1)) >= valid) sz[i] = __float2half(0.f);
            tq_fence_proxy_async();   // generic writes to a stage that a later bulk copy may refill
            __syncwarp();
        }

        // ------------------------------ scores ------------------------------
        float acc1[4], acc0[4], accs[4];   // written by the first k-step's MMAs
        if (MSE_BITS == 3) acc1[0] = acc1[1] = acc1[2] = acc1[3] = 0.f;
        if (MSE_BITS == 2) {
            const uint32_t* cwA = reinterpret_cast<const uint32_t*>(rec + L.off_kcodes + tokA * L.kcode_row) + tig * NWK;
            const uint32_t* cwB = reinterpret_cast<const uint32_t*>(rec + L.off_kcodes + tokB * L.kcode_row) + tig * NWK;
            const uint32_t* swA = reinterpret_cast<const uint32_t*>(rec + L.off_ksigns + tokA * L.ksign_row) + tig * (NWK / 2);
            const uint32_t* swB = reinterpret_cast<const uint32_t*>(rec + L.off_ksigns + tokB * L.ksign_row) + tig * (NWK / 2);
            uint32_t wA[NWK], wB[NWK], sA[NWK / 2], sB[NWK / 2];
            if (NWK == 4) {
                const uint4 a = *reinterpret_cast<const uint4*>(cwA), bb = *reinterpret_cast<const uint4*>(cwB);
                wA[0] = a.x; wA[1] = a.y; wA[NWK - 2] = a.z; wA[NWK - 1] = a.w;
                wB[0] = bb.x; wB[1] = bb.y; wB[NWK - 2] = bb.z; wB[NWK - 1] = bb.w;
                const uint2 c = *reinterpret_cast<const uint2*>(swA), d = *reinterpret_cast<const uint2*>(swB);
                sA[0] = c.x; sA[NWK / 2 - 1] = c.y;
                sB[0] = d.x; sB[NWK / 2 - 1] = d.y;
            } else {
                const uint2 a = *reinterpret_cast<const uint2*>(cwA), bb = *reinterpret_cast<const uint2*>(cwB);
                wA[0] = a.x; wA[1] = a.y;
                wB[0] = bb.x; wB[1] = bb.y;
                sA[0] = swA[0];
                sB[0] = swB[0];
            }
#pragma unroll
            for (int wi = 0; wi < NWK; ++wi) {
                const uint32_t a_lo = wA[wi], b_lo = wB[wi];
                const uint32_t a_hi = a_lo >> 6, b_hi = b_lo >> 6;
                // sign word with bytes 1 and 2 swapped: halves then pair the same dims as the code word
                const uint32_t sa_lo = __byte_perm(sA[wi >> 1], 0, 0x3120), sb_lo = __byte_perm(sB[wi >> 1], 0, 0x3120);
                const uint32_t sa_hi = sa_lo >> 6, sb_hi = sb_lo >> 6;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int s = wi * 4 + jj;
                    const int j0 = 2 * jj, j1 = j0 + 1;
                    const uint32_t m0 = 0x00010001u << (2 * code_pos(j0)), m1 = 0x00010001u << (2 * code_pos(j1));
                    const uint32_t xa0 = j0 <= 4 ? a_lo : a_hi, xb0 = j0 <= 4 ? b_lo : b_hi;
                    const uint32_t xa1 = j1 <= 4 ? a_lo : a_hi, xb1 = j1 <= 4 ? b_lo : b_hi;
                    if (s == 0) {
                        mma16816_z(acc0, xa0 & m0, xb0 & m0, xa1 & m1, xb1 & m1, BQ(2 * s), BQ(2 * s + 1));
                        mma16816_z(acc1, xa0 & (m0 << 1), xb0 & (m0 << 1), xa1 & (m1 << 1), xb1 & (m1 << 1), BQ(2 * s),
                                   BQ(2 * s + 1));
                    } else {
                        mma16816(acc0, xa0 & m0, xb0 & m0, xa1 & m1, xb1 & m1, BQ(2 * s), BQ(2 * s + 1));
                        mma16816(acc1, xa0 & (m0 << 1), xb0 & (m0 << 1), xa1 & (m1 << 1), xb1 & (m1 << 1), BQ(2 * s),
                                 BQ(2 * s + 1));
                    }
                    const int sb0 = sign_bit(wi, j0), sb1 = sign_bit(wi, j1);
                    const uint32_t n0 = 0x00010001u << sign_pos(sb0), n1 = 0x00010001u << sign_pos(sb1);
                    const uint32_t ya0 = sb0 <= 9 ? sa_lo : sa_hi, yb0 = sb0 <= 9 ? sb_lo : sb_hi;
                    const uint32_t ya1 = sb1 <= 9 ? sa_lo : sa_hi, yb1 = sb1 <= 9 ? sb_lo : sb_hi;
                    if (s == 0)
                        mma16816_z(accs, ya0 & n0, yb0 & n0, ya1 & n1, yb1 & n1, SPLITB ? BSK(0) : BQ(0),
                                   SPLITB ? BSK(1) : BQ(1));
                    else if (SPLITB)
                        mma16816(accs, ya0 & n0, yb0 & n0, ya1 & n1, yb1 & n1, BSK(2 * s), BSK(2 * s + 1));
                    else
                        mma16816(accs, ya0 & n0, yb0 & n0, ya1 & n1, yb1 & n1, BQ(2 * s), BQ(2 * s + 1));
                }
            }
        }
        if (MSE_BITS == 3) {
            constexpr int NWC = D / 32;    // words of nibble codes per thread per token (8 codes each)
            constexpr int NWS = D / 128;   // sign words per thread per token
            const uint4* cwA = reinterpret_cast<const uint4*>(rec + L.off_kcodes + tokA * L.kcode_row) + tig * (NWC / 4);
            const uint4* cwB = reinterpret_cast<const uint4*>(rec + L.off_kcodes + tokB * L.kcode_row) + tig * (NWC / 4);
            const uint32_t* swA = reinterpret_cast<const uint32_t*>(rec + L.off_ksigns + tokA * L.ksign_row) + tig * NWS;
            const uint32_t* swB = reinterpret_cast<const uint32_t*>(rec + L.off_ksigns + tokB * L.ksign_row) + tig * NWS;
#pragma unroll
            for (int q4 = 0; q4 < NWC / 4; ++q4) {
                const uint4 a4 = cwA[q4], b4 = cwB[q4];
                const uint32_t wa[4] = {a4.x, a4.y, a4.z, a4.w}, wb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        // k-step s covers dims 8*(4*q4+wi) + 4*hf + {0,1 | 2,3} of this thread's slice
                        const int s = (q4 * 4 + wi) * 2 + hf;
                        const uint32_t sa = hf ? wa[wi] >> 16 : wa[wi], sb = hf ? wb[wi] >> 16 : wb[wi];
                        const uint32_t la = __byte_perm(t_lo0, t_lo1, sa), ha = __byte_perm(t_hi0, t_hi1, sa);
                        const uint32_t lb = __byte_perm(t_lo0, t_lo1, sb), hb = __byte_perm(t_hi0, t_hi1, sb);
                        if (s == 0)
                            mma16816_z(acc0, __byte_perm(la, ha, 0x5140), __byte_perm(lb, hb, 0x5140),
                                       __byte_perm(la, ha, 0x7362), __byte_perm(lb, hb, 0x7362), BQ(0), BQ(1));
                        else
                            mma16816(acc0, __byte_perm(la, ha, 0x5140), __byte_perm(lb, hb, 0x5140),
                                     __byte_perm(la, ha, 0x7362), __byte_perm(lb, hb, 0x7362), BQ(2 * s), BQ(2 * s + 1));
                    }
                }
            }
#pragma unroll
            for (int sw = 0; sw < NWS; ++sw) {
                const uint32_t sa_lo = __byte_perm(swA[sw], 0, 0x3120), sb_lo = __byte_perm(swB[sw], 0, 0x3120);
                const uint32_t sa_hi = sa_lo >> 6, sb_hi = sb_lo >> 6;
#pragma unroll
                for (int wi = 2 * sw; wi < 2 * sw + 2; ++wi) {
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int s = wi * 4 + jj;
                        const int sb0 = sign_bit(wi, 2 * jj), sb1 = sign_bit(wi, 2 * jj + 1);
                        const uint32_t n0 = 0x00010001u << sign_pos(sb0), n1 = 0x00010001u << sign_pos(sb1);
                        const uint32_t ya0 = sb0 <= 9 ? sa_lo : sa_hi, yb0 = sb0 <= 9 ? sb_lo : sb_hi;
                        const uint32_t ya1 = sb1 <= 9 ? sa_lo : sa_hi, yb1 = sb1 <= 9 ? sb_lo : sb_hi;
                        if (s == 0)
                            mma16816_z(accs, ya0 & n0, yb0 & n0, ya1 & n1, yb1 & n1, BSK(0), BSK(1));
                        else
                            mma16816(accs, ya0 & n0, yb0 & n0, ya1 & n1, yb1 & n1, BSK(2 * s),
                                     BSK(2 * s + 1));
                    }
                }
            }
        }
        if (!SPLITB) {   // sketched-query columns 4..7 live two lanes to the right
#pragma unroll
            for (int c = 0; c < 4; ++c) accs[c] = __shfl_xor_sync(0xffffffffu, accs[c], 2);
        }

        // ------------------------------ online softmax ------------------------------
        const __half* nrm = reinterpret_cast<const __half*>(rec + L.off_knorm);
        const __half* rnm = reinterpret_cast<const __half*>(rec + L.off_krnorm);
        const float nA = __half2float(nrm[tokA]) * sm_scale, nB = __half2float(nrm[tokB]) * sm_scale;
        const float rA = __half2float(rnm[tokA]) * (qjl * sm_scale), rB = __half2float(rnm[tokB]) * (qjl * sm_scale);
        float sA[2], sB[2], pA[2], pB[2];
        bool rescale = false;
        float alpha[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sA[i] = nA * (k0[i] + k1[i] * acc1[i] + kb0[i] * acc0[i]) + rA * (ksg[i] * accs[i] - kq[i]);
            sB[i] = nB * (k0[i] + k1[i] * acc1[2 + i] + kb0[i] * acc0[2 + i]) + rB * (ksg[i] * accs[2 + i] - kq[i]);
            if (valid < TQ_BLOCK_TOKENS) {   // warp-uniform: only the sequence's last record
                if (tokA >= valid) sA[i] = -INFINITY;
                if (tokB >= valid) sB[i] = -INFINITY;
            }
            float mx = fmaxf(sA[i], sB[i]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[i], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[i] = ex2_fast(m_run[i] - m_use);
            pA[i] = ex2_fast(sA[i] - m_use);
            pB[i] = ex2_fast(sB[i] - m_use);
            l_run[i] = l_run[i] * alpha[i] + pA[i] + pB[i];
            rescale |= (m_new != m_run[i]);
            m_run[i] = m_new;
        }
        if (__any_sync(0xffffffffu, rescale && col_ok)) {
#pragma unroll
            for (int mb = 0; mb < NMB; ++mb) {
                o[mb][0] *= alpha[0];
                o[mb][1] *= alpha[1];
                o[mb][2] *= alpha[0];
                o[mb][3] *= alpha[1];
            }
            zacc[0] *= alpha[0];
            zacc[1] *= alpha[1];
            zacc[2] *= alpha[0];
            zacc[3] *= alpha[1];
        }
        // probabilities (x16, clear of fp16 underflow) -> B fragment of the value MMA
        const uint32_t t0 = movmatrix_trans(col_ok ? pack_half2(pA[0] * 16.f, pA[1] * 16.f) : 0u);
        const uint32_t t1 = movmatrix_trans(col_ok ? pack_half2(pB[0] * 16.f, pB[1] * 16.f) : 0u);

        // ------------------------------ values ------------------------------
        {
            // tokens of this thread's contraction slots: 4*tig .. 4*tig+3
            const uint2* vsc = reinterpret_cast<const uint2*>(rec + L.off_vscale) + tig;   // [grp][16 tok] fp16: 4 uint2 per group
            const uint2* vzr = reinterpret_cast<const uint2*>(rec + L.off_vzero) + tig;
            // zero-point term: rows = groups
            {
                uint2 z = make_uint2(0u, 0u);
                if (gid < NG) z = vzr[gid * 4];
                mma16816(zacc, z.x, 0u, z.y, 0u, t0, t1);
            }
            const uint4* vcw = reinterpret_cast<const uint4*>(rec + L.off_vcodes) + lane;   // [chunk][lane] 16 B
            if (VAL_BITS == 2) {
                // word (p, gp): [tokA grp 2gp, tokA grp 2gp+1, tokB grp 2gp, tokB grp 2gp+1]
                constexpr int NGP = NG / 2;
                uint32_t w[2 * NGP];
                if (NGP == 4) {
                    const uint4 a = vcw[0], c = vcw[32];
                    w[0] = a.x; w[1] = a.y; w[NGP - 2] = a.z; w[NGP - 1] = a.w;
                    w[NGP] = c.x; w[NGP + 1] = c.y; w[2 * NGP - 2] = c.z; w[2 * NGP - 1] = c.w;
                } else {
                    const uint4 a = vcw[0];
                    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
                }
#pragma unroll
                for (int gp = 0; gp < NGP; ++gp) {
                    const uint32_t w0 = w[gp], w1 = w[NGP + gp];
                    const uint32_t w0h = w0 >> 6, w1h = w1 >> 6;
#pragma unroll
                    for (int odd = 0; odd < 2; ++odd) {
                        const int grp = 2 * gp + odd;
                        const uint2 sc = vsc[grp * 4];
                        const uint32_t bp0 = hmul2_sat(t0, sc.x), bp1 = hmul2_sat(t1, sc.y);
#pragma unroll
                        for (int hb = 0; hb < 2; ++hb) {   // the two M-blocks of the group
                            const int i_lo = 2 * hb, i_hi = i_lo + 1;
                            // even group: field i at bits 2i; odd group: i=0 at bits 8-9, i>=1 after >>6 at 2(i+1)
                            const int p_lo = odd ? (i_lo == 0 ? 4 : i_lo + 1) : i_lo;
                            const int p_hi = odd ? i_hi + 1 : i_hi;
                            const bool sh_lo = odd && i_lo != 0, sh_hi = odd;
                            const uint32_t mk_lo = 0x00030003u << (2 * p_lo), mk_hi = 0x00030003u << (2 * p_hi);
                            mma16816(o[2 * grp + hb], (sh_lo ? w0h : w0) & mk_lo, (sh_hi ? w0h : w0) & mk_hi,
                                     (sh_lo ? w1h : w1) & mk_lo, (sh_hi ? w1h : w1) & mk_hi, bp0, bp1);
                        }
                    }
                }
            } else {
                // word (p, grp): [tokA byte0, tokA byte1, tokB byte0, tokB byte1]; byte0 = codes 0,1, byte1 = codes 2,3
                uint32_t w[2 * NG];
#pragma unroll
                for (int c = 0; c < 2 * NG / 4; ++c) {
                    const uint4 a = vcw[32 * c];
                    w[4 * c] = a.x; w[4 * c + 1] = a.y; w[4 * c + 2] = a.z; w[4 * c + 3] = a.w;
                }
#pragma unroll
                for (int grp = 0; grp < NG; ++grp) {
                    const uint32_t w0 = w[grp], w1 = w[NG + grp];
                    const uint32_t w0h = w0 >> 8, w1h = w1 >> 8;
                    const uint2 sc = vsc[grp * 4];
                    const uint32_t bp0 = hmul2_sat(t0, sc.x), bp1 = hmul2_sat(t1, sc.y);
                    mma16816(o[2 * grp], w0 & 0x000f000fu, w0 & 0x00f000f0u, w1 & 0x000f000fu, w1 & 0x00f000f0u, bp0, bp1);
                    mma16816(o[2 * grp + 1], w0h & 0x000f000fu, w0h & 0x00f000f0u, w1h & 0x000f000fu,
                             w1h & 0x00f000f0u, bp0, bp1);
                }
            }
        }

        __syncwarp();
        if (lane == 0 && it + NSTW < cnt) {   // refill the stage just consumed
            tq_mbar_expect_tx(my_bar + st, (uint32_t)BB);
            tq_bulk_g2s(my_stage + st * BB, p.pool + ((int64_t)bt_s[warp + NW * (it + NSTW)] * p.H + h) * BB,
                        (uint32_t)BB, my_bar + st);
        }
    }
    if (failed && lane == 0) atomicCAS(p.status, 0, (int)TQ_ERR_TIMEOUT);

    // ------------------------------ combine the warps of the CTA ------------------------------
#pragma unroll
    for (int i = 0; i < 2; ++i) {   // row sums over the eight row groups
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 4);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 8);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 16);
    }
    // zero-point sums Z[grp][g] sit in lane (grp, tig); fetch the ones of this thread's rows
    float zrow[NG][2];
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {
        zrow[grp][0] = __shfl_sync(0xffffffffu, zacc[0], grp * 4 + tig);
        zrow[grp][1] = __shfl_sync(0xffffffffu, zacc[1], grp * 4 + tig);
    }
    __syncthreads();   // every warp is done with its stages: reuse them
    // [NW warps][GP][D + 4]: the padding spreads the four lanes that share a channel quad (one per
    // pair of heads) over different banks; a thread stores the quad of a head with one 16-byte store
    constexpr int DP = D + 4;
    float* osm = reinterpret_cast<float*>(stages);
    if (col_ok) {
#pragma unroll
        for (int grp = 0; grp < NG; ++grp) {
            const int odd = grp & 1;
            float f[4];   // A value = code * 2^(sh - 24); probabilities carried x16
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int sh;
                if (VAL_BITS == 2) sh = 2 * (odd ? (i == 0 ? 4 : i + 1) : i);
                else sh = 4 * (i & 1);
                f[i] = pow2i(24 - sh - 4);
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int g = 2 * tig + c;
                const float z = zrow[grp][c] * 0.0625f;
                // channels 4*gid + i of the group: i = 2*hb + half sits in M-block 2*grp + hb, register 2*half + c
                const float4 v = make_float4(fmaf(o[2 * grp][c], f[0], z), fmaf(o[2 * grp][2 + c], f[1], z),
                                             fmaf(o[2 * grp + 1][c], f[2], z), fmaf(o[2 * grp + 1][2 + c], f[3], z));
                *reinterpret_cast<float4*>(osm + (warp * GP + g) * DP + 32 * grp + 4 * gid) = v;
            }
        }
        if (gid == 0) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                ml[(warp * 2 + 0) * GP + 2 * tig + c] = m_run[c];
                ml[(warp * 2 + 1) * GP + 2 * tig + c] = l_run[c];
            }
        }
    }
    __syncthreads();
    // Every thread owns four channels of one head: it weighs the warps' partials itself (NW exp2f)
    // instead of waiting for a serial pass over the heads.
    {
        const bool single = p.num_splits + p.ring_splits == 1;   // then this CTA writes the output itself
        float* mine = partial_ptr<D, GP>(p, b, h, x);
        for (int i = tid; i < GP * (D / 4); i += NT) {
            const int g = i / (D / 4), d = (i % (D / 4)) * 4;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < NW; ++w) mx = fmaxf(mx, ml[(w * 2) * GP + g]);
            float lsum = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float mw = ml[(w * 2) * GP + g];
                const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mx);
                lsum = fmaf(f, ml[(w * 2 + 1) * GP + g], lsum);
                const float4 v = *reinterpret_cast<const float4*>(osm + (w * GP + g) * DP + d);
                acc.x = fmaf(f, v.x, acc.x);
                acc.y = fmaf(f, v.y, acc.y);
                acc.z = fmaf(f, v.z, acc.z);
                acc.w = fmaf(f, v.w, acc.w);
            }
            if (single) {
                if (g < p.G) {
                    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
                    const int64_t dst = ((int64_t)b * p.Qh + h * p.G + g) * D + d;
                    tq_store4_any(p.out, dst, acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv, p.q_dtype);
                }
            } else {
                *reinterpret_cast<float4*>(mine + 2 * GP + g * D + d) = acc;
                if (d == 0) {
                    mine[g] = mx * 0.6931471805599453f;   // back to the natural-log domain of the merge
                    mine[GP + g] = lsum;
                }
            }
        }
        if (single) {
            return;
        }
    }
    __syncthreads();   // wsm is reused by the merge
    ticket_and_merge<D, GP>(p, b, h, wsm, smem, p.land_bytes);
}

// Bytes in front of the barriers: stages, ml, bt_s, grown (one CTA per SM only) until the merge
// can land all `nslot` partials of a (sequence, kv head) there.
template <int D, bool SPLITB, int NW>
size_t mma_land_bytes(int block_bytes, int nslot) {
    constexpr int GP = SPLITB ? 8 : 4;
    size_t s = (size_t)NW * NSTW * block_bytes + sizeof(float) * (2 * NW * GP) + sizeof(int) * BT_MAX;
    const size_t want = (size_t)nslot * GP * (D + 2) * sizeof(float);
    if (NW == NW_WAVE && want > s && want <= 200 * 1024) s = want;
    return (s + 127) / 128 * 128;
}
template <int D, bool SPLITB, int NW>
size_t mma_smem_bytes(int block_bytes, int nslot) {
    constexpr int GP = SPLITB ? 8 : 4;
    size_t s = mma_land_bytes<D, SPLITB, NW>(block_bytes, nslot);
    s += sizeof(uint64_t) * (NW * NSTW + 2) + sizeof(uint32_t) * qf_words(D, SPLITB ? 8 : 4);
    // merge scratch: one row of slot weights per warp of the merging CTA
    s += sizeof(float) * ((size_t)((nslot > 128 ? nslot : 128) + 8) * NW + 2 * GP);
    return s;
}

template <int D, int MSE_BITS, int VAL_BITS, bool SPLITB, int NW>
int launch_mma_nw(const DecodeParams& p_in, int batch, cudaStream_t st) {
    DecodeParams p = p_in;
    constexpr int NT = NW * 32;
    const TqLayout L = tq_make_layout(D, MSE_BITS + 1, VAL_BITS);
    const int nslot = p.num_splits + p.ring_splits;
    const size_t smem = mma_smem_bytes<D, SPLITB, NW>(L.block_bytes, nslot);
    p.land_bytes = (uint32_t)mma_land_bytes<D, SPLITB, NW>(L.block_bytes, nslot);
    auto kern = tq_decode_mma_kernel<D, MSE_BITS, VAL_BITS, SPLITB, NW>;
    static TqSmemOptIn opt_in;
    if (tq_opt_in_smem(kern, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.H, (unsigned)nslot, (unsigned)batch);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // start while the previous kernel drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tq_pdl_for_decode(st);   // behind a store that is still writing the pool: plain stream order
    tq_note_launch(st, TQ_LAUNCH_DECODE);
    return cudaLaunchKernelEx(&cfg, kern, p) == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

constexpr size_t SMEM_PER_CTA_MAX = 227 * 1024;

// *handled = 0 when not even the 8-warp CTA's stages fit shared memory (the caller then runs the CUDA-core kernel)
template <int D, int MSE_BITS, int VAL_BITS, bool SPLITB>
int launch_mma(const DecodeParams& p, int batch, cudaStream_t st, int* handled) {
    const TqLayout L = tq_make_layout(D, MSE_BITS + 1, VAL_BITS);
    const int nslot = p.num_splits + p.ring_splits;
    const int64_t ctas = (int64_t)nslot * p.H * batch;
    const bool fits_wave = mma_smem_bytes<D, SPLITB, NW_WAVE>(L.block_bytes, nslot) <= SMEM_PER_CTA_MAX;
    const bool fits_multi = mma_smem_bytes<D, SPLITB, NW_MULTI>(L.block_bytes, nslot) <= SMEM_PER_CTA_MAX;
    *handled = 1;
    // two 8-warp CTAs per SM need two merge scratch areas in shared memory: only with few slots
    if (fits_multi && ((ctas > tq_sm_count() && nslot <= 128) || !fits_wave))
        return launch_mma_nw<D, MSE_BITS, VAL_BITS, SPLITB, NW_MULTI>(p, batch, st);
    if (fits_wave) return launch_mma_nw<D, MSE_BITS, VAL_BITS, SPLITB, NW_WAVE>(p, batch, st);
    *handled = 0;
    return TQ_OK;
}

}  // namespace


namespace tqdec {

int tq_decode_mma_launch(const DecodeParams& p, int D, int mse_bits, int val_bits, int batch, int max_seq_len,
                         cudaStream_t st, int* handled) {
    *handled = 0;
    const int nblk = (max_seq_len + TQ_BLOCK_TOKENS - 1) / TQ_BLOCK_TOKENS;
    if ((nblk + p.num_splits - 1) / p.num_splits + 1 > BT_MAX) return TQ_OK;   // block-table slice kept in shared memory
    if ((int64_t)(p.num_splits + 1) * nblk >= (int64_t)1 << 31) return TQ_OK;   // 32-bit split arithmetic in the kernel
    if (mse_bits == 3) {
        if (D == 128)
            return val_bits == 2 ? launch_mma<128, 3, 2, true>(p, batch, st, handled) : launch_mma<128, 3, 4, true>(p, batch, st, handled);
        return val_bits == 2 ? launch_mma<256, 3, 2, true>(p, batch, st, handled) : launch_mma<256, 3, 4, true>(p, batch, st, handled);
    }
    if (mse_bits != 2) return TQ_OK;
    // the bit-plane form needs a code book that is affine in the two code bits
    const float* c = p.cb.centroids;
    if (fabsf(c[3] - c[2] - c[1] + c[0]) > 1e-6f * fabsf(c[3] - c[0])) return TQ_OK;
    const bool split = p.G > 4;
    if (D == 128) {
        if (val_bits == 2)
            return split ? launch_mma<128, 2, 2, true>(p, batch, st, handled) : launch_mma<128, 2, 2, false>(p, batch, st, handled);
        return split ? launch_mma<128, 2, 4, true>(p, batch, st, handled) : launch_mma<128, 2, 4, false>(p, batch, st, handled);
    }
    if (val_bits == 2)
        return split ? launch_mma<256, 2, 2, true>(p, batch, st, handled) : launch_mma<256, 2, 2, false>(p, batch, st, handled);
    return split ? launch_mma<256, 2, 4, true>(p, batch, st, handled) : launch_mma<256, 2, 4, false>(p, batch, st, handled);
}

}  // namespace tqdec
