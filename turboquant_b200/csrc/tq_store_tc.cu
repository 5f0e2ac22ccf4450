// Store path on the 5th-generation tensor cores (tcgen05 + TMEM), head_dim 128,
// bf16 input.  One persistent CTA per SM: 16 compute warps plus one warp whose
// single elected thread issues every TMA load and every MMA.  A tile is 128
// token positions of one kv head; four compute threads share a token row, each
// owning 32 channels from load to packed output.
//
//   TMA (2 swizzled boxes)   : key rows and value rows of the tile -> shared memory
//   N  norm, normalise       : u = bf16(x / |x|) exactly as torch does, e' = x/|x| - u (what the bf16
//                              rounding lost); both written to TENSOR MEMORY as MMA A operands
//   MMA 1 (A from TMEM)      : Y = u * Pi^T (Pi as two bf16 limbs), E = e' * Pi_hi^T
//   V  values                : per-group min/max quantisation in packed bf16 arithmetic (under MMA 1)
//   C  codes                 : bucket search on Y, code packing; residual IN ROTATED SPACE
//                              r' = (Y - centroid[code]) + E  (the reference's x - x_hat, rotated and
//                              divided by |x|: no un-rotation product); r' as bf16 hi + lo limbs -> TMEM
//   MMA 2 (A from TMEM)      : P = r' * M^T, M = S * Pi^T as two bf16 limbs (hi*hi + hi*lo + lo*hi)
//   S  sign bits of P; the tile's eight 16-token block records, assembled in shared memory, leave
//      with one bulk (TMA) store each.
//
// Two tiles are in flight: MMA 2 of tile t runs under the normalisation of tile t+1, MMA 1 of tile
// t+1 under its value quantisation; the key / value boxes of the tile after that are already on
// their way.  The compute warps hand work to the issuing thread through mbarriers they only arrive
// on, and meet one another at two CTA barriers per tile (norm exchange, record image complete), so
// they drift apart and fill each other's stalls.  The constant operands (Pi_hi, Pi_lo, M_hi, M_lo: 128 KB) stay in shared memory; no A
// operand ever touches it.  Tensor memory (512 columns): Y 128 | E, later P 128 | u 64 | e' 64 |
// r'_hi 64 | r'_lo 64.
//
// Destinations: a block table with any start position (tiles are laid on the 16-token block grid;
// a first block that already holds earlier tokens is read, completed and written back) or a slot
// mapping (whole records where sixteen rows fill one block in order, byte scatter otherwise).
//
// Reference arithmetic: quantizer.py:129-149,231-257 and kv_cache.py:45-98.  Every wait on an
// mbarrier is bounded; a timeout frees tensor memory and returns with a status.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "tq_common.cuh"
#include "tq_tcgen05.cuh"

using namespace tqtc;

namespace {

constexpr int TC_D = 128;
constexpr int TC_TOK = 128;
constexpr int TC_THREADS = 512;                 // compute threads
constexpr int TC_LAUNCH = TC_THREADS + 32;      // plus the issuing warp
constexpr int BOX_BYTES = TC_TOK * 128;          // one swizzled box: 128 rows x 128 bytes (64 bf16)
constexpr int MAT_BYTES = 2 * BOX_BYTES;         // a 128 x 128 bf16 operand: two boxes (k 0-63, 64-127)
constexpr int TMEM_COLS = 512;
constexpr size_t SMEM_LIMIT = 227 * 1024;

// tensor-memory columns
constexpr uint32_t COL_Y = 0, COL_E = 128, COL_U = 256, COL_EP = 320, COL_RH = 384, COL_RL = 448;

struct TcParams {
    int64_t n_tokens;
    const int64_t* slot_mapping;   // destination of token i when given (negative: skip) ...
    const int32_t* block_table;    // ... else position start_pos + i of this sequence
    int64_t start_pos;
    int lead;                      // start_pos & 15: rows of the first tile that precede token 0
    uint8_t* pool;
    int64_t num_blocks;
    int H;
    TqCodebook cb;
    int n_tiles;                   // token tiles x heads (the launcher keeps it below 2^31)
    int n_rec_buf;                 // record images in shared memory (2 when they fit)
    int tok_outer;                 // tensor-map dimension order: 1 = (channel, head, token), 0 = (channel, token, head)
    // paged source (a cache of fixed-size token blocks addressed through a table) instead of flat rows:
    const int32_t* src_table;      // logical source block -> physical block; nullptr: flat rows
    int32_t src_num_blocks;        // physical blocks of the source cache
    int src_bs_log2;               // log2 of its block size in tokens (>= 4)
    int64_t src_tail_block;        // logical block that holds fewer than a block's tokens (-1: none)
};

__device__ int g_tq_store_status;   // 0 or a tq_status left by a bounded wait that ran out

// ---------------------------------------------------------------------------
// MMA shapes of this file
// ---------------------------------------------------------------------------
constexpr uint32_t IDESC = umma_idesc_bf16(128);        // N = 128
constexpr uint32_t IDESC_N256 = umma_idesc_bf16(256);   // N = 256
__device__ __forceinline__ void umma_ss_n256(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    umma_ss(tmem_d, a_desc, b_desc, IDESC_N256, accumulate);
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t accumulate) {
    tqtc::umma_ts(tmem_d, tmem_a, b_desc, IDESC, accumulate);
}

// Offset inside a block record of byte `cb` of token `tl`'s share (a token owns bytes_per_token bytes:
// codes, signs, norm, residual norm, value codes, group scales, group zero points - in that order).
__device__ __forceinline__ int rec_byte_offset(const TqLayout& L, int tl, int cb) {
    if (cb < L.kcode_row) return L.off_kcodes + tl * L.kcode_row + cb;
    cb -= L.kcode_row;
    if (cb < L.ksign_row) return L.off_ksigns + tl * L.ksign_row + cb;
    cb -= L.ksign_row;
    if (cb < 2) return L.off_knorm + tl * 2 + cb;
    cb -= 2;
    if (cb < 2) return L.off_krnorm + tl * 2 + cb;
    cb -= 2;
    if (cb < L.vcode_row) return L.off_vcodes + tq_vcode_native(L.D, L.val_bits, tl, cb);
    cb -= L.vcode_row;
    if (cb < 2 * L.ngroups) return L.off_vscale + ((cb >> 1) * TQ_BLOCK_TOKENS + tl) * 2 + (cb & 1);
    cb -= 2 * L.ngroups;
    return L.off_vzero + ((cb >> 1) * TQ_BLOCK_TOKENS + tl) * 2 + (cb & 1);
}

// ---------------------------------------------------------------------------
// Values: asymmetric min/max quantisation of ONE 32-channel group of one row in
// bf16 arithmetic (kv_cache.py:64-90), on packed pairs.
//   v - zero        : one packed bf16 subtraction per pair (a single rounding, as torch's)
//   (.) / scale     : both operands are bf16 numbers, so the quotient is either exactly representable
//                     or at least 2^-17 (relative) away from every bf16 rounding boundary: the
//                     product with the fp32 reciprocal rounds to the same bf16 as the division
//   round, clamp    : adding 128 in bf16 (unit in the last place: 1) IS round-half-to-even of a value
//                     in [0, 128); the code sits in the low mantissa bits
// Codes go to the record image in the decode kernel's byte order, scale / zero point group-major.
// ---------------------------------------------------------------------------
template <int VAL_BITS, int D = TC_D>
__device__ __forceinline__ void quantize_value_group(const uint4 (&raw)[4], uint8_t* rec, const TqLayout& L, int tl,
                                                     int grp, bool wr) {
    constexpr uint32_t N_LEVELS = (1u << VAL_BITS) - 1u;
    constexpr uint32_t FIELD = VAL_BITS == 2 ? 0x00030003u : 0x000f000fu;
    const uint32_t w[16] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w,
                            raw[2].x, raw[2].y, raw[2].z, raw[2].w, raw[3].x, raw[3].y, raw[3].z, raw[3].w};
    __nv_bfloat162 mn = as_bf162(w[0]), mx = mn;
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        mn = __hmin2(mn, as_bf162(w[i]));
        mx = __hmax2(mx, as_bf162(w[i]));
    }
    const float vmin = fminf(bf_lo(as_u32(mn)), bf_hi(as_u32(mn)));
    const float vmax = fmaxf(bf_lo(as_u32(mx)), bf_hi(as_u32(mx)));
    float scale = bf16r(__fdiv_rn(bf16r(vmax - vmin), (float)N_LEVELS));
    scale = fmaxf(scale, bf16r(1e-10f));
    const float rscale = __frcp_rn(scale);
    const __nv_bfloat162 zero2 = __floats2bfloat162_rn(vmin, vmin);
    const __nv_bfloat162 magic = __floats2bfloat162_rn(128.f, 128.f);
    uint32_t code[16];   // code of the pair's elements in bits 0.. and 16..
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t d = as_u32(__hsub2(as_bf162(w[i]), zero2));
        // z <= levels * (1 + 2^-7) < levels + 1/2: the rounding below cannot leave the field
        const __nv_bfloat162 z = as_bf162(pack_bf16(bf_lo(d) * rscale, bf_hi(d) * rscale));
        code[i] = as_u32(__hadd2(z, magic)) & FIELD;
    }
    if (!wr) return;
    reinterpret_cast<__half*>(rec + L.off_vscale)[grp * TQ_BLOCK_TOKENS + tl] = __float2half_rn(scale);
    reinterpret_cast<__half*>(rec + L.off_vzero)[grp * TQ_BLOCK_TOKENS + tl] = __float2half_rn(vmin);
    uint8_t* vc = rec + L.off_vcodes;
    if (VAL_BITS == 2) {
#pragma unroll
        for (int bt = 0; bt < 8; ++bt) {   // byte = four codes, LSB first (kv_cache.py:80-84)
            const uint32_t t = code[2 * bt] | (code[2 * bt + 1] << 4);
            vc[tq_vcode_native(D, 2, tl, grp * 8 + bt)] = (uint8_t)(t | (t >> 14));
        }
    } else {
#pragma unroll
        for (int bt = 0; bt < 16; ++bt) {  // byte = two codes (kv_cache.py:86-90)
            const uint32_t t = code[bt];
            vc[tq_vcode_native(D, 4, tl, grp * 16 + bt)] = (uint8_t)(t | (t >> 12));
        }
    }
}

// Comparisons as arithmetic.  The fp32 pipes are the only full-rate ones of an SM; compares, selects and
// bit logic run at half rate and would bound this kernel.  For finite a:
//     step_gt(a, BIG, -b * BIG) = saturate((a - b) * 2^126)  is exactly 1 when a > b and exactly 0 when
// a <= b, as long as |a - b| is either 0 or at least 2^-126 - true for every boundary that is not itself
// tiny; the second saturating multiply of step_gt2 extends that to every float (2^-149 * 2^252 >= 1).
// NaN saturates to 0.
constexpr float BIG = 8.507059173023462e37f;   // 2^126
__device__ __forceinline__ float fma_sat(float a, float b, float c) {
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float mul_sat(float a, float b) {
    float d;
    asm("mul.rn.sat.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

// The code book prepared for that arithmetic (registers): nb[i] = -boundary[i] * 2^126, c0 = centroid[0],
// step[i] = centroid[i+1] - centroid[i].
template <int MSE_BITS>
struct BookRegs {
    float nb[(1 << MSE_BITS) - 1], step[(1 << MSE_BITS) - 1], c0;
};

// Bucket search of one rotated coordinate y (torch.searchsorted on the interior boundaries, left: the
// code is the number of boundaries below y) and y minus its centroid.  `code` comes back as a float.
template <int MSE_BITS>
__device__ __forceinline__ void bucket(const BookRegs<MSE_BITS>& bk, float y, float& code, float& y_minus_c) {
    constexpr int NB = (1 << MSE_BITS) - 1, MID = NB / 2;   // the middle boundary is (next to) zero
    float k = 0.f, r = y - bk.c0;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        float t = fma_sat(y, BIG, bk.nb[i]);
        if (i == MID) t = mul_sat(t, BIG);
        k += t;
        r = fmaf(-t, bk.step[i], r);
    }
    code = k;
    y_minus_c = r;
}

// Destination of one image block (16 rows) of a tile: asked for early, looked at when the records leave
// (the loaded words are not touched before that - not even widened - so nobody waits for them).
struct RecordDest {
    int32_t blk = -1;     // block-table mode, lane 0: physical block
    int64_t slot = -1;    // slot mode: slot of row `lane & 15`
    bool asked = false;
};
__device__ __forceinline__ void ask_destination(const TcParams& p, int64_t tok0, int warp, int lane, RecordDest& d) {
    if (warp >= 8) return;
    if (p.slot_mapping == nullptr) {
        const int64_t first = tok0 + warp * TQ_BLOCK_TOKENS;      // token index of the block's first row
        d.asked = lane == 0 && first < p.n_tokens && first + TQ_BLOCK_TOKENS > 0;
        if (d.asked) d.blk = __ldg(p.block_table + ((p.start_pos + first) >> 4));
    } else {
        const int64_t i = tok0 + warp * TQ_BLOCK_TOKENS + (lane & 15);
        if (i >= 0 && i < p.n_tokens) d.slot = __ldg(p.slot_mapping + i);
    }
}
// Warp j < 8 sends image block j on its way: one bulk (TMA) store when the block is a whole record of
// the pool, a byte scatter to each token's own slot otherwise.
__device__ __forceinline__ void leave_records(const TcParams& p, const TqLayout& L, const uint8_t* img, int h, int j,
                                              int lane, const RecordDest& d) {
    const int BB = L.block_bytes;
    if (p.slot_mapping == nullptr) {
        if (d.asked) {
            if (d.blk >= 0 && d.blk < p.num_blocks) {
                tq_bulk_s2g(p.pool + ((int64_t)d.blk * p.H + h) * (int64_t)BB, img + j * BB, (uint32_t)BB);
                tq_bulk_commit();
            } else {
                atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_RANGE);
            }
        }
        return;
    }
    // slot mapping: sixteen rows that fill one block in order leave as a whole record, anything else is
    // scattered byte by byte
    int64_t slot = d.slot;
    if (slot >= 0 && (slot >> 4) >= p.num_blocks) {
        atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_RANGE);
        slot = -1;
    }
    const int64_t slot0 = __shfl_sync(0xffffffffu, slot, 0);
    const bool whole = __all_sync(0xffffffffu, slot0 >= 0 && (slot0 & 15) == 0 && slot == slot0 + (lane & 15));
    if (whole) {
        if (lane == 0) {
            tq_bulk_s2g(p.pool + ((slot0 >> 4) * p.H + h) * (int64_t)BB, img + j * BB, (uint32_t)BB);
            tq_bulk_commit();
        }
        return;
    }
    const int per_tok = BB / TQ_BLOCK_TOKENS;
    const uint8_t* src = img + j * BB;
    for (int t = 0; t < TQ_BLOCK_TOKENS; ++t) {
        const int64_t s = __shfl_sync(0xffffffffu, slot, t);
        if (s < 0) continue;
        uint8_t* dst = p.pool + ((s >> 4) * p.H + h) * (int64_t)BB;
        for (int cb = lane; cb < per_tok; cb += 32)
            dst[rec_byte_offset(L, (int)(s & 15), cb)] = src[rec_byte_offset(L, t, cb)];
    }
}

// Rows of one tile (128 tokens of one head, n_cbox boxes of 64 channels) from a PAGED source: the tile
// is covered by 128 / block_size source blocks (or lies inside one), each looked up in the source table
// and fetched by its own lane of the issuing warp - the swizzle pattern depends on the shared-memory
// address alone, so boxes of 16+ rows stacked 1024-byte aligned form the same image as one 128-row box.
// Blocks past the end are requested out of range (zero fill); the block that is only partly valid goes
// through `tm_tail`, the same cache with its token dimension cut to the valid rows, so that rows past
// the last token read as zeros exactly as they do from flat rows.
__device__ __forceinline__ void issue_paged_rows(uint8_t* dst, const CUtensorMap* tm, const CUtensorMap* tm_tail,
                                                 uint64_t* bar, const TcParams& p, int64_t tok0, int head, int n_cbox,
                                                 int lane, bool is_elected) {
    const int lg = p.src_bs_log2;
    const int rows = lg >= 7 ? TC_TOK : (1 << lg);          // token rows per box
    const int per_tile = TC_TOK / rows;
    if (is_elected) tq_mbar_expect_tx(bar, (uint32_t)(n_cbox * BOX_BYTES));
    __syncwarp();
    if (lane < per_tile * n_cbox) {
        const int jj = lane / n_cbox, cb = lane - jj * n_cbox;
        const int64_t tok = tok0 + (int64_t)jj * rows;
        const int64_t sb = tok >> lg;
        int32_t phys = p.src_num_blocks;                     // out of range: zeros
        if (tok < p.n_tokens) {
            phys = __ldg(p.src_table + sb);
            if (phys < 0 || phys >= p.src_num_blocks) {
                atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_RANGE);
                phys = p.src_num_blocks;
            }
        }
        const int in_blk = (int)(tok & (((int64_t)1 << lg) - 1));
        tma_load_4d(dst + cb * BOX_BYTES + jj * rows * 128, sb == p.src_tail_block ? tm_tail : tm, 64 * cb,
                    p.tok_outer ? head : in_blk, p.tok_outer ? in_blk : head, phys, bar);
    }
    __syncwarp();
}

// This launch may have started while the launch ahead of it in the stream still runs (programmatic
// dependent launch; only when that launch is one of the library's that cannot be writing key / value
// rows, see TqLaunchKind): the rows may be fetched at once, but the pool - which that launch
// may write, and whose stream order of writes the caller relies on - is touched only after this wait.
__device__ __forceinline__ void pool_writes_may_begin() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tq_smem_u32(bar)) : "memory");
}
// Barrier of the 512 compute threads (the issuing warp is not part of it); true if any thread passes true.
__device__ __forceinline__ bool compute_barrier_or(bool flag) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, 512, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"((uint32_t)flag)
        : "memory");
    return out != 0;
}

// Compute thread (row = tid % 128, q = tid / 128), tid < 512, owns channels [32q, 32q+32) of token row
// `row` - one value group, 16 packed columns of an A operand, 32 accumulator columns.  Warp w reads
// and writes TMEM lanes of quarter w % 4 = row / 32, as the hardware requires.  Warp 16 only issues.
template <int MSE_BITS, int VAL_BITS>
__global__ void __launch_bounds__(TC_LAUNCH, 1)
tq_store_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_vt,
                   const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
                   const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_b3,
                   const TcParams p) {
    const TqLayout L = tq_make_layout(TC_D, MSE_BITS + 1, VAL_BITS);
    const int BB = L.block_bytes;
    const int IMG = 8 * BB;                           // one record image: the tile's 8 block records

    extern __shared__ uint8_t smem_raw[];
    // swizzled boxes need a 1024-byte aligned base in the shared window
    uint8_t* smem = smem_raw + ((1024u - (tq_smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sB = smem;                               // Pi_hi, Pi_lo, M_hi, M_lo: 4 x (2 boxes)
    uint8_t* sX = sB + 4 * MAT_BYTES;                 // key rows of the tile (2 boxes)
    uint8_t* sV = sX + MAT_BYTES;                     // value rows of the tile (2 boxes)
    uint8_t* sRec = sV + MAT_BYTES;                   // n_rec_buf record images
    float* s_ss = reinterpret_cast<float*>(sRec + p.n_rec_buf * IMG);   // [4][128] partial sums of squares of x
    float* s_rn = s_ss + 4 * TC_TOK;                                    // [4][128] ... of r'
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_rn + 4 * TC_TOK);
    // completed by TMA bytes / MMA commits (count 1) ...
    uint64_t *bar_b = bars, *bar_k = bars + 1, *bar_v = bars + 2, *bar_y = bars + 3, *bar_e = bars + 4,
             *bar_p = bars + 5, *bar_r = bars + 6;
    // ... and by the 512 compute threads, waited for by the issuing thread:
    uint64_t* bar_n = bars + 7;    // u / e' of a tile written (Y was read before), its key rows consumed
    uint64_t* bar_a = bars + 8;    // P of the tile before read: E's columns are free
    uint64_t* bar_c = bars + 9;    // r' limbs written, Y and E read
    uint64_t* bar_vf = bars + 10;  // value rows consumed
    uint64_t* bar_m = bars + 11;   // (TMA bytes, count 1) M_hi, M_lo landed; bar_b: Pi_hi, Pi_lo
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* s_fail = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool slot_mode = p.slot_mapping != nullptr;
    // The launch that follows in the stream may take over each SM as soon as this CTA leaves it; whatever
    // it reads or writes in the pool comes after its own wait for this grid (see pool_writes_may_begin).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tq_smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 7; ++i) tq_mbar_init(bars + i, 1);
#pragma unroll
        for (int i = 7; i < 11; ++i) tq_mbar_init(bars + i, TC_THREADS);
        tq_mbar_init(bar_m, 1);
        *s_fail = 0;
        tq_mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // tile -> (kv head, first row's token index).  Tiles lie on the block grid of the destination
    // sequence: row r of token tile tt is token i = 128 * tt + r - lead (lead > 0: the first block already
    // holds `lead` earlier tokens); the boxes of rows outside [0, n_tokens) arrive as zeros.
    // (32-bit unsigned arithmetic: 64-bit division is a long instruction sequence)
    auto tile_head = [&](int tile) { return (int)((uint32_t)tile % (uint32_t)p.H); };
    auto tile_tok0 = [&](int tile) { return (int64_t)((uint32_t)tile / (uint32_t)p.H) * TC_TOK - p.lead; };
    const int tile0 = blockIdx.x;   // the grid never exceeds the tile count
    const bool rmw = !slot_mode && p.lead != 0 && tile0 < p.H;   // this CTA's first tile completes a begun block

    // One poller per warp; gives up after `limit` polls or as soon as somebody has flagged a failure.
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
        __syncwarp();   // the poller's acquire covers the whole warp
        return ok != 0;
    };

    if (warp == TC_THREADS / 32) {
        // =============================== issuing warp ===============================
        // The whole warp runs this code with identical values, so that addresses and descriptors stay
        // in the uniform datapath the MMA and TMA instructions take their operands from; one elected
        // lane issues.
        {
            const uint32_t aB = tq_smem_u32(sB);
            const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
            auto wait1 = [&](uint64_t* bar, uint32_t parity) -> bool {
                uint32_t ok = 0;
                for (int i = 0; i < (1 << 20); ++i) {
                    if (tq_mbar_try_wait(bar, parity)) {
                        ok = 1;
                        break;
                    }
                    __nanosleep(40);   // a spinning warp takes issue slots from the compute warps of its scheduler
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
            auto issue_kv = [&](uint8_t* dst, const CUtensorMap* tm, const CUtensorMap* tm_tail, uint64_t* bar, int tile) {
                const int hh = tile_head(tile), t0 = (int)tile_tok0(tile);
                if (p.src_table != nullptr) {
                    issue_paged_rows(dst, tm, tm_tail, bar, p, tile_tok0(tile), hh, 2, lane, elected());
                    return;
                }
                if (elected()) {
                    tq_mbar_expect_tx(bar, 2 * BOX_BYTES);
                    tma_load_3d(dst, tm, 0, p.tok_outer ? hh : t0, p.tok_outer ? t0 : hh, bar);
                    tma_load_3d(dst + BOX_BYTES, tm, 64, p.tok_outer ? hh : t0, p.tok_outer ? t0 : hh, bar);
                }
                __syncwarp();
            };
            // operand descriptors: the upper word is a constant, the lower one the address in 16-byte units
            const uint32_t desc_lo = (uint32_t)(smem_desc_sw128(aB) & 0xffffffffu);
            const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(aB) >> 32);
            auto b_desc = [&](int mat, int ks) {
                const uint32_t lo = desc_lo + (uint32_t)((mat * MAT_BYTES + (ks >> 2) * BOX_BYTES + (ks & 3) * 32) >> 4);
                return ((uint64_t)desc_hi << 32) | lo;
            };
            auto issue_mma_y = [&]() {   // Y = u Pi_hi^T + u Pi_lo^T
                tc_fence_after();
                if (elected()) {
#pragma unroll
                    for (int m = 0; m < 2; ++m)
#pragma unroll
                        for (int ks = 0; ks < TC_D / 16; ++ks)
                            umma_ts(tmem + COL_Y, tmem + COL_U + ks * 8, b_desc(m, ks), (m | ks) != 0);
                    umma_commit(bar_y);
                }
                __syncwarp();
            };
            auto issue_mma_e = [&]() {   // E = e' Pi_hi^T
                tc_fence_after();
                if (elected()) {
#pragma unroll
                    for (int ks = 0; ks < TC_D / 16; ++ks)
                        umma_ts(tmem + COL_E, tmem + COL_EP + ks * 8, b_desc(0, ks), ks != 0);
                    umma_commit(bar_e);
                }
                __syncwarp();
            };
            auto issue_mma_p = [&]() {   // P = r_hi M_hi^T + r_hi M_lo^T + r_lo M_hi^T, over E's columns
                tc_fence_after();
                if (elected()) {
#pragma unroll
                    for (int m = 0; m < 3; ++m)
#pragma unroll
                        for (int ks = 0; ks < TC_D / 16; ++ks)
                            umma_ts(tmem + COL_E, tmem + (m == 2 ? COL_RL : COL_RH) + ks * 8, b_desc(m == 1 ? 3 : 2, ks),
                                    (m | ks) != 0);
                    umma_commit(bar_p);
                }
                __syncwarp();
            };

            // in the order they are needed: key rows (normalisation), Pi (Y and E products), value rows, M (P product)
            issue_kv(sX, &tm_k, &tm_kt, bar_k, tile0);
            const CUtensorMap* tb[4] = {&tm_b0, &tm_b1, &tm_b2, &tm_b3};
            auto load_pair = [&](int m0, uint64_t* bar) {
                if (elected()) {
                    tq_mbar_expect_tx(bar, 2 * MAT_BYTES);
#pragma unroll
                    for (int m = m0; m < m0 + 2; ++m) {
                        tma_load_2d(sB + m * MAT_BYTES, tb[m], 0, 0, bar);
                        tma_load_2d(sB + m * MAT_BYTES + BOX_BYTES, tb[m], 64, 0, bar);
                    }
                }
                __syncwarp();
            };
            load_pair(0, bar_b);
            issue_kv(sV, &tm_v, &tm_vt, bar_v, tile0);
            load_pair(2, bar_m);
            if (rmw) {   // the block this append continues, into block 0 of the first record image
                pool_writes_may_begin();
                if (elected()) {
                    const int64_t phys = p.block_table[p.start_pos >> 4];
                    if (phys >= 0 && phys < p.num_blocks) {
                        tq_mbar_expect_tx(bar_r, (uint32_t)BB);
                        tq_bulk_g2s(sRec, p.pool + (phys * p.H + tile_head(tile0)) * (int64_t)BB, (uint32_t)BB, bar_r);
                    } else {
                        atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_RANGE);
                        tq_mbar_expect_tx(bar_r, 0);   // completes the phase: nobody waits for bytes
                    }
                }
                __syncwarp();
            }
            bool ok = wait1(bar_b, 0);
            // per tile, in the order the compute threads arrive: [n] Y product, next key rows; [vf] next value
            // rows; [a] E product; [c] P product
            auto feed = [&](int i, int tile) -> bool {
                const int next = tile + (int)gridDim.x;
                if (!wait1(bar_n, i & 1)) return false;
                issue_mma_y();
                if (next < p.n_tiles) issue_kv(sX, &tm_k, &tm_kt, bar_k, next);
                if (p.n_rec_buf == 2) {
                    if (!wait1(bar_vf, i & 1)) return false;
                    if (next < p.n_tiles) issue_kv(sV, &tm_v, &tm_vt, bar_v, next);
                }
                if (!wait1(bar_a, i & 1)) return false;
                issue_mma_e();
                if (p.n_rec_buf != 2) {   // with one record image the values follow the record store
                    if (!wait1(bar_vf, i & 1)) return false;
                    if (next < p.n_tiles) issue_kv(sV, &tm_v, &tm_vt, bar_v, next);
                }
                return true;
            };
            int i = 0;
            ok = ok && feed(0, tile0);
            ok = ok && wait1(bar_m, 0);
#pragma unroll 1
            for (int tile = tile0; tile < p.n_tiles && ok; tile += (int)gridDim.x, ++i) {
                if (!(ok = wait1(bar_c, i & 1))) break;
                issue_mma_p();
                if (tile + (int)gridDim.x < p.n_tiles) ok = feed(i + 1, tile + (int)gridDim.x);
            }
        }
    } else {
        // =============================== compute warps ===============================
        const int row = tid & (TC_TOK - 1), q = tid >> 7;
        const int blk_l = row >> 4, tl = row & 15;
        const uint32_t lane_base = (uint32_t)(row & ~31) << 16;   // this warp's quarter of the 128 TMEM lanes
        BookRegs<MSE_BITS> bk;   // the code book, in registers
        bk.c0 = p.cb.centroids[0];
#pragma unroll
        for (int i = 0; i < (1 << MSE_BITS) - 1; ++i) {
            bk.nb[i] = -p.cb.boundaries[i] * BIG;
            bk.step[i] = p.cb.centroids[i + 1] - p.cb.centroids[i];
        }
        bool bad = false;      // one of this warp's waits ran out; reported at the next compute barrier
        float nd = 0.f;        // |x| of this thread's row in the input dtype, from N to S of the same tile
        float nd_next = 0.f;

        // N: key rows of a tile -> norm, u and e' in tensor memory; false (uniform) = a wait ran out
        auto phase_n = [&](uint32_t parity, float& nd_out) -> bool {
            bad |= !wait_warp(bar_k, parity);
            uint32_t xw[16];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 v = lds_sw128(sX + (q >> 1) * BOX_BYTES, row, (q & 1) * 4 + c);
                xw[4 * c] = v.x; xw[4 * c + 1] = v.y; xw[4 * c + 2] = v.z; xw[4 * c + 3] = v.w;
            }
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float a = bf_lo(xw[i]), b = bf_hi(xw[i]);
                ss = fmaf(a, a, ss);
                ss = fmaf(b, b, ss);
            }
            s_ss[q * TC_TOK + row] = ss;
            if (compute_barrier_or(bad)) return false;    // partial sums (of x, and of the r' before) published
            ss = (s_ss[row] + s_ss[TC_TOK + row]) + (s_ss[2 * TC_TOK + row] + s_ss[3 * TC_TOK + row]);
            const float n_d = bf16r(__fsqrt_rn(ss));               // quantizer.py:136, in the input dtype
            const float den = bf16r(n_d + 1e-10f);                 // quantizer.py:138
            const float rden = __frcp_rn(den);
            uint32_t up[16], ep[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                // numerator and denominator are bf16 numbers: the product with the reciprocal rounds to
                // the same bf16 as the division (see quantize_value_group)
                const float q0 = bf_lo(xw[i]) * rden, q1 = bf_hi(xw[i]) * rden;
                const uint32_t u = pack_bf16(q0, q1);
                up[i] = u;
                ep[i] = pack_bf16(q0 - bf_lo(u), q1 - bf_hi(u));   // what the bf16 normalisation lost
            }
            tmem_st16(tmem + lane_base + COL_U + q * 16, up);
            tmem_st16(tmem + lane_base + COL_EP + q * 16, ep);
            tmem_st_wait();
            nd_out = n_d;
            return true;
        };
        // V: value rows in shared memory -> codes, scales, zero points of one tile's record image
        auto phase_v = [&](uint32_t parity, uint8_t* image, int64_t tok_first) {
            bad |= !wait_warp(bar_v, parity);
            uint4 vraw[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) vraw[c] = lds_sw128(sV + (q >> 1) * BOX_BYTES, row, (q & 1) * 4 + c);
            mbar_arrive(bar_vf);                          // this thread's value row is in registers
            quantize_value_group<VAL_BITS>(vraw, image + blk_l * BB, L, tl, q, tok_first + row >= 0);
        };

        // N of a tile, then the hand-over to the issuing thread: its Y product may start (every thread
        // passed the C phase of the tile before, so Y has been read), the key rows are consumed
        auto phase_n_and_arrive = [&](uint32_t parity, float& nd_out) -> bool {
            if (!phase_n(parity, nd_out)) return false;
            tc_fence_before();
            mbar_arrive(bar_n);
            return true;
        };

        // ---- first tile: keys normalised, the begun block fetched, values quantised ----
        bool ok = phase_n_and_arrive(0, nd);
        if (ok) {
            mbar_arrive(bar_a);                           // nothing occupies E's columns yet
            if (rmw) bad |= !wait_warp(bar_r, 0);
            phase_v(0, sRec, tile_tok0(tile0));
        }

        int tile_no = 0;
#pragma unroll 1
        for (int tile = tile0; tile < p.n_tiles && ok; tile += (int)gridDim.x, ++tile_no) {
            const int next = tile + (int)gridDim.x;
            const bool has_next = next < p.n_tiles;
            const uint32_t par = tile_no & 1;
            const int h = tile_head(tile);
            const int64_t tok0 = tile_tok0(tile);
            const bool wr = tok0 + row >= 0;                 // rows before token 0 belong to an earlier append
            uint8_t* img = sRec + (p.n_rec_buf == 2 ? (tile_no & 1) : 0) * IMG;
            uint8_t* nimg = sRec + (p.n_rec_buf == 2 ? ((tile_no + 1) & 1) : 0) * IMG;
            uint8_t* rec = img + blk_l * BB;

            RecordDest dest;
            ask_destination(p, tok0, warp, lane, dest);

            // ---------------- C: codes and rotated-space residual of channels [32q, 32q+32) ----------------
            bad |= !wait_warp(bar_y, par);
            tc_fence_after();
            {
                float y[32];
                tmem_ld32(tmem + lane_base + COL_Y + q * 32, y);
                // codes of 16 bits' worth of coordinates are summed in one float (exact), LSB first
                // (quantizer.py:50-68), and converted once
                constexpr int WIDTH = MSE_BITS == 2 ? 2 : 4, PER_HALF = 16 / WIDTH;
                uint32_t halves[32 / PER_HALF];
#pragma unroll
                for (int w = 0; w < 32 / PER_HALF; ++w) {
                    float wf = 0.f;
#pragma unroll
                    for (int jj = 0; jj < PER_HALF; ++jj) {
                        float code;
                        bucket<MSE_BITS>(bk, y[w * PER_HALF + jj], code, y[w * PER_HALF + jj]);   // quantizer.py:144
                        wf = fmaf(code, (float)(1u << (WIDTH * jj)), wf);
                    }
                    halves[w] = __float_as_uint(wf + 8388608.f) & 0xffffu;   // 2^23 + integer: the integer sits in the mantissa
                }
                if (wr) {
                    uint32_t* kc = reinterpret_cast<uint32_t*>(rec + L.off_kcodes + tl * L.kcode_row) + q * (16 / PER_HALF);
#pragma unroll
                    for (int w = 0; w < 16 / PER_HALF; ++w) kc[w] = halves[2 * w] | (halves[2 * w + 1] << 16);
                }
                bad |= !wait_warp(bar_e, par);            // the E product was issued last: it lands under the search above
                tc_fence_after();
                float er[32];
                tmem_ld32(tmem + lane_base + COL_E + q * 32, er);
                float rn2 = 0.f;
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float a = y[2 * i] + er[2 * i], b = y[2 * i + 1] + er[2 * i + 1];   // r' = (Y - c) + E
                    rn2 = fmaf(a, a, rn2);
                    rn2 = fmaf(b, b, rn2);
                    const uint32_t hh = pack_bf16(a, b);
                    hi[i] = hh;
                    lo[i] = pack_bf16(a - bf_lo(hh), b - bf_hi(hh));
                }
                tmem_st16(tmem + lane_base + COL_RH + q * 16, hi);
                tmem_st16(tmem + lane_base + COL_RL + q * 16, lo);
                s_rn[q * TC_TOK + row] = rn2;
                tmem_st_wait();
            }
            tc_fence_before();
            mbar_arrive(bar_c);                           // the P product may start once every thread is here

            // the other record image is written next (values of the following tile): what it held must have left
            if (lane == 0 && warp < 8) tq_bulk_wait_all_read();

            // ---------------- N of the next tile, under the P product ----------------
            if (has_next) {
                if (!phase_n_and_arrive(par ^ 1, nd_next)) {
                    ok = false;
                    break;
                }
            } else if (compute_barrier_or(bad)) {         // same barrier: publishes the r' partial sums
                ok = false;
                break;
            }

            // ---------------- V of the next tile (two record images: before this tile's records are complete) ----------------
            if (has_next && p.n_rec_buf == 2) phase_v(par ^ 1, nimg, tile_tok0(next));

            // ---------------- S: sign bits of channels [32q, 32q+32) (quantizer.py:214-222) ----------------
            bad |= !wait_warp(bar_p, par);
            tc_fence_after();
            {
                float pr[32];
                tmem_ld32(tmem + lane_base + COL_E + q * 32, pr);
                tc_fence_before();
                if (has_next) mbar_arrive(bar_a);         // P is read: the next E product may use its columns
                float w_lo = 0.f, w_hi = 0.f;   // bit j = (P_j > 0), sixteen bits per float
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    w_lo = fmaf(mul_sat(mul_sat(pr[j], BIG), BIG), (float)(1u << j), w_lo);
                    w_hi = fmaf(mul_sat(mul_sat(pr[16 + j], BIG), BIG), (float)(1u << j), w_hi);
                }
                uint32_t w = (__float_as_uint(w_lo + 8388608.f) & 0xffffu) | (__float_as_uint(w_hi + 8388608.f) << 16);
                if (nd == 0.f) w = 0;   // x = 0: the reference's residual is exactly 0, r' is not
                if (wr) reinterpret_cast<uint32_t*>(rec + L.off_ksigns + tl * L.ksign_row)[q] = w;
            }
            if (q == 0 && wr) {   // norms of the row
                const float rn2 = (s_rn[row] + s_rn[TC_TOK + row]) + (s_rn[2 * TC_TOK + row] + s_rn[3 * TC_TOK + row]);
                reinterpret_cast<__half*>(rec + L.off_knorm)[tl] = __float2half_rn(nd);
                // |r| = |x| * |r'| (the reference's residual x - x_hat, quantizer.py:244-245)
                reinterpret_cast<__half*>(rec + L.off_krnorm)[tl] = __float2half_rn(nd * __fsqrt_rn(rn2));
            }
            tq_fence_proxy_async();
            if (compute_barrier_or(bad)) {                // record image complete
                ok = false;
                break;
            }

            // ---------------- the tile's block records leave ----------------
            if (warp < 8) {
                if (tile_no == 0) pool_writes_may_begin();
                leave_records(p, L, img, h, warp, lane, dest);
                if (lane == 0 && p.n_rec_buf == 1) tq_bulk_wait_all_read();
            }
            if (p.n_rec_buf == 1) {
                compute_barrier_or(false);                // the single image is rewritten by the values below
                if (has_next) phase_v(par ^ 1, nimg, tile_tok0(next));
            }
            nd = nd_next;
        }
        if (!ok && tid == 0) atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_TIMEOUT);
        if (lane == 0 && warp < 8) tq_bulk_wait_all();   // the records must have landed before the CTA retires
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ---------------------------------------------------------------------------
// head_dim 256
// ---------------------------------------------------------------------------
// Same arithmetic, different residency: four 256 x 256 operand matrices (512 KB) cannot stay in shared
// memory, and a 128-row A operand of 256 packed channels takes 128 tensor-memory columns, so that u, e',
// r'_hi and r'_lo alone would fill it.  Here the A operands live in SHARED memory - the key rows land by
// TMA, are normalised in place, e' takes the place of the value rows once they are quantised, and r'_hi /
// r'_lo overwrite both after the first products - tensor memory holds Y (256 columns) and E (256), later P
// over Y, and the constant operands stream through a two-slot ring of 32 KB boxes (256 rows x 64
// channels), each box used for every product that needs it while it is resident: Pi_hi for Y and E, Pi_lo
// for Y, M_hi for r'_hi and r'_lo, M_lo for r'_hi - 512 KB from L2 per tile.  One tile in flight.
// A compute thread (row, q) owns channels [64q, 64q+64): two value groups, one 128-byte row of a box.
constexpr int D2 = 256;
constexpr int D2_TILE_BYTES = 4 * BOX_BYTES;      // 128 rows x 256 bf16: four boxes
constexpr int D2_CHUNK_BYTES = 2 * BOX_BYTES;     // 256 rows x 64 bf16 of a constant operand

template <int MSE_BITS, int VAL_BITS>
__global__ void __launch_bounds__(TC_LAUNCH, 1)
tq_store_tc256_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_vt,
                      const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
                      const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_b3,
                      const TcParams p) {
    const TqLayout L = tq_make_layout(D2, MSE_BITS + 1, VAL_BITS);
    const int BB = L.block_bytes;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tq_smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sA0 = smem;                              // key rows -> u -> r'_hi
    uint8_t* sA1 = sA0 + D2_TILE_BYTES;               // value rows -> e' -> r'_lo
    uint8_t* sBr = sA1 + D2_TILE_BYTES;               // two slots of the constant-operand ring
    uint8_t* sRec = sBr + 2 * D2_CHUNK_BYTES;         // image of the tile's 8 block records
    float* s_ss = reinterpret_cast<float*>(sRec + 8 * BB);   // [4][128] partial sums of squares (x, then r')
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_ss + 4 * TC_TOK);
    uint64_t *bar_k = bars, *bar_v = bars + 1, *bar_m1 = bars + 2, *bar_m2 = bars + 3, *bar_r = bars + 4;
    uint64_t *bar_full = bars + 5, *bar_empty = bars + 7;     // [2] each: ring slot filled / its products done
    uint64_t *bar_n = bars + 9, *bar_c = bars + 10;           // 512 arrivals: u, e' written / r' written
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* s_fail = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool slot_mode = p.slot_mapping != nullptr;
    // The launch that follows in the stream may take over each SM as soon as this CTA leaves it; whatever
    // it reads or writes in the pool comes after its own wait for this grid (see pool_writes_may_begin).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tq_smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 9; ++i) tq_mbar_init(bars + i, 1);
        tq_mbar_init(bar_n, TC_THREADS);
        tq_mbar_init(bar_c, TC_THREADS);
        *s_fail = 0;
        tq_mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr uint32_t C_Y = 0, C_E = 256;

    auto tile_head = [&](int tile) { return (int)((uint32_t)tile % (uint32_t)p.H); };
    auto tile_tok0 = [&](int tile) { return (int64_t)((uint32_t)tile / (uint32_t)p.H) * TC_TOK - p.lead; };
    const int tile0 = blockIdx.x;
    const bool rmw = !slot_mode && p.lead != 0 && tile0 < p.H;

    if (warp == TC_THREADS / 32) {
        // =============================== issuing warp (uniform, one elected lane issues) ===============================
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
        auto wait1 = [&](uint64_t* bar, uint32_t parity) -> bool {
            uint32_t ok = 0;
            for (int i = 0; i < (1 << 20); ++i) {
                if (tq_mbar_try_wait(bar, parity)) {
                    ok = 1;
                    break;
                }
                __nanosleep(40);
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
        auto issue_rows = [&](uint8_t* dst, const CUtensorMap* tm, const CUtensorMap* tm_tail, uint64_t* bar, int tile) {
            const int hh = tile_head(tile), t0 = (int)tile_tok0(tile);
            if (p.src_table != nullptr) {
                issue_paged_rows(dst, tm, tm_tail, bar, p, tile_tok0(tile), hh, 4, lane, elected());
                return;
            }
            if (elected()) {
                tq_mbar_expect_tx(bar, D2_TILE_BYTES);
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    tma_load_3d(dst + b * BOX_BYTES, tm, 64 * b, p.tok_outer ? hh : t0, p.tok_outer ? t0 : hh, bar);
            }
            __syncwarp();
        };
        const CUtensorMap* tb[4] = {&tm_b0, &tm_b1, &tm_b2, &tm_b3};
        const uint32_t a0 = tq_smem_u32(sA0), a1 = tq_smem_u32(sA1), ar = tq_smem_u32(sBr);
        // chunk c of a tile: constant operand c / 4 (Pi_hi, Pi_lo, M_hi, M_lo), channels [64 (c % 4), +64)
        int g_loaded = 0;       // chunks requested so far, over all tiles of this CTA
        auto load_chunk = [&](int c) -> bool {
            const int slot = g_loaded & 1;
            if (g_loaded >= 2 && !wait1(bar_empty + slot, ((g_loaded - 2) >> 1) & 1)) return false;
            if (elected()) {
                tq_mbar_expect_tx(bar_full + slot, D2_CHUNK_BYTES);
                tma_load_2d(sBr + slot * D2_CHUNK_BYTES, tb[c >> 2], 64 * (c & 3), 0, bar_full + slot);
            }
            __syncwarp();
            ++g_loaded;
            return true;
        };
        int g_used = 0;
        auto use_chunk = [&](int c) -> bool {   // issue every product that reads chunk c, then release its slot
            const int slot = g_used & 1, kc = c & 3, mat = c >> 2;
            if (!wait1(bar_full + slot, (g_used >> 1) & 1)) return false;
            tc_fence_after();
            if (elected()) {
                const uint32_t b_addr = ar + slot * D2_CHUNK_BYTES;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t bd = smem_desc_sw128(b_addr + ks * 32);
                    const uint64_t d0 = smem_desc_sw128(a0 + kc * BOX_BYTES + ks * 32);
                    const uint64_t d1 = smem_desc_sw128(a1 + kc * BOX_BYTES + ks * 32);
                    const uint32_t first = (kc | ks) == 0 ? 0u : 1u;
                    if (mat == 0) {            // Pi_hi: Y (u) and E (e')
                        umma_ss_n256(tmem_u + C_Y, d0, bd, first);
                        umma_ss_n256(tmem_u + C_E, d1, bd, first);
                    } else if (mat == 1) {     // Pi_lo: Y (u)
                        umma_ss_n256(tmem_u + C_Y, d0, bd, 1u);
                    } else if (mat == 2) {     // M_hi: P (r'_hi) and P (r'_lo), over Y's columns
                        umma_ss_n256(tmem_u + C_Y, d0, bd, first);
                        umma_ss_n256(tmem_u + C_Y, d1, bd, 1u);
                    } else {                   // M_lo: P (r'_hi)
                        umma_ss_n256(tmem_u + C_Y, d0, bd, 1u);
                    }
                }
                umma_commit(bar_empty + slot);
                if (c == 7) umma_commit(bar_m1);
                if (c == 15) umma_commit(bar_m2);
            }
            __syncwarp();
            ++g_used;
            return true;
        };

        issue_rows(sA0, &tm_k, &tm_kt, bar_k, tile0);
        issue_rows(sA1, &tm_v, &tm_vt, bar_v, tile0);
        if (rmw) {
            pool_writes_may_begin();
            if (elected()) {
                const int64_t phys = p.block_table[p.start_pos >> 4];
                if (phys >= 0 && phys < p.num_blocks) {
                    tq_mbar_expect_tx(bar_r, (uint32_t)BB);
                    tq_bulk_g2s(sRec, p.pool + (phys * p.H + tile_head(tile0)) * (int64_t)BB, (uint32_t)BB, bar_r);
                } else {
                    atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_RANGE);
                    tq_mbar_expect_tx(bar_r, 0);
                }
            }
            __syncwarp();
        }
        bool ok = load_chunk(0) && load_chunk(1);
        int i = 0;
#pragma unroll 1
        for (int tile = tile0; tile < p.n_tiles && ok; tile += (int)gridDim.x, ++i) {
            const int next = tile + (int)gridDim.x;
            if (!(ok = wait1(bar_n, i & 1))) break;              // u, e' in shared memory
#pragma unroll 1
            for (int c = 0; c < 16 && ok; ++c) {
                if (c == 8 && !(ok = wait1(bar_c, i & 1))) break;   // r' limbs in shared memory
                ok = use_chunk(c);
                // keep the ring full: the chunk two ahead (of this tile, or the first ones of the next tile)
                const int ahead = c + 2;
                if (ok && (ahead < 16 || next < p.n_tiles)) ok = load_chunk(ahead & 15);
            }
            if (!ok) break;
            if (next < p.n_tiles) {
                if (!(ok = wait1(bar_m2, i & 1))) break;         // the A tiles are free again
                issue_rows(sA0, &tm_k, &tm_kt, bar_k, next);
                issue_rows(sA1, &tm_v, &tm_vt, bar_v, next);
            }
        }
    } else {
        // =============================== compute warps ===============================
        const int row = tid & (TC_TOK - 1), q = tid >> 7;
        const int blk_l = row >> 4, tl = row & 15;
        const uint32_t lane_base = (uint32_t)(row & ~31) << 16;
        BookRegs<MSE_BITS> bk;
        bk.c0 = p.cb.centroids[0];
#pragma unroll
        for (int i = 0; i < (1 << MSE_BITS) - 1; ++i) {
            bk.nb[i] = -p.cb.boundaries[i] * BIG;
            bk.step[i] = p.cb.centroids[i + 1] - p.cb.centroids[i];
        }
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
        // this thread's 128 bytes (64 channels) of row `row` in box q of an A tile
        auto row_chunk = [&](uint8_t* tile, int c) { return reinterpret_cast<uint4*>(tile + q * BOX_BYTES + row * 128 + ((c ^ (row & 7)) << 4)); };
        bool bad = false, ok = true;
        int tile_no = 0;
#pragma unroll 1
        for (int tile = tile0; tile < p.n_tiles; tile += (int)gridDim.x, ++tile_no) {
            const uint32_t par = tile_no & 1;
            const int h = tile_head(tile);
            const int64_t tok0 = tile_tok0(tile);
            const bool wr = tok0 + row >= 0;
            uint8_t* rec = sRec + blk_l * BB;
            RecordDest dest;
            ask_destination(p, tok0, warp, lane, dest);

            // ---------------- V: the two value groups of channels [64q, 64q+64) ----------------
            if (tile_no == 0 && rmw) bad |= !wait_warp(bar_r, 0);
            bad |= !wait_warp(bar_v, par);
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {
                uint4 vraw[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) vraw[c] = *row_chunk(sA1, 4 * g2 + c);
                quantize_value_group<VAL_BITS, D2>(vraw, rec, L, tl, 2 * q + g2, wr);
            }
            // ---------------- N: norm, u in place of the key row, e' in place of the value row ----------------
            bad |= !wait_warp(bar_k, par);
            float nd;
            {
                uint32_t xw[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *row_chunk(sA0, c);
                    xw[4 * c] = v.x; xw[4 * c + 1] = v.y; xw[4 * c + 2] = v.z; xw[4 * c + 3] = v.w;
                }
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float a = bf_lo(xw[i]), b = bf_hi(xw[i]);
                    ss = fmaf(a, a, ss);
                    ss = fmaf(b, b, ss);
                }
                s_ss[q * TC_TOK + row] = ss;
                if (compute_barrier_or(bad)) {   // partial sums published; every thread has read its value row
                    ok = false;
                    break;
                }
                ss = (s_ss[row] + s_ss[TC_TOK + row]) + (s_ss[2 * TC_TOK + row] + s_ss[3 * TC_TOK + row]);
                nd = bf16r(__fsqrt_rn(ss));
                const float rden = __frcp_rn(bf16r(nd + 1e-10f));
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t up[4], ep[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float q0 = bf_lo(xw[4 * c + i]) * rden, q1 = bf_hi(xw[4 * c + i]) * rden;
                        up[i] = pack_bf16(q0, q1);
                        ep[i] = pack_bf16(q0 - bf_lo(up[i]), q1 - bf_hi(up[i]));
                    }
                    *row_chunk(sA0, c) = make_uint4(up[0], up[1], up[2], up[3]);
                    *row_chunk(sA1, c) = make_uint4(ep[0], ep[1], ep[2], ep[3]);
                }
            }
            tq_fence_proxy_async();   // generic writes -> the MMA's reads
            mbar_arrive(bar_n);

            // ---------------- C: codes, r' limbs over u / e' ----------------
            bad |= !wait_warp(bar_m1, par);
            tc_fence_after();
            float rn2 = 0.f;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                float y[32];
                tmem_ld32(tmem + lane_base + C_Y + q * 64 + hf * 32, y);
                constexpr int WIDTH = MSE_BITS == 2 ? 2 : 4, PER_HALF = 16 / WIDTH;
                uint32_t halves[32 / PER_HALF];
#pragma unroll
                for (int w = 0; w < 32 / PER_HALF; ++w) {
                    float wf = 0.f;
#pragma unroll
                    for (int jj = 0; jj < PER_HALF; ++jj) {
                        float code;
                        bucket<MSE_BITS>(bk, y[w * PER_HALF + jj], code, y[w * PER_HALF + jj]);
                        wf = fmaf(code, (float)(1u << (WIDTH * jj)), wf);
                    }
                    halves[w] = __float_as_uint(wf + 8388608.f) & 0xffffu;
                }
                if (wr) {
                    uint32_t* kc = reinterpret_cast<uint32_t*>(rec + L.off_kcodes + tl * L.kcode_row) +
                                   (2 * q + hf) * (16 / PER_HALF);
#pragma unroll
                    for (int w = 0; w < 16 / PER_HALF; ++w) kc[w] = halves[2 * w] | (halves[2 * w + 1] << 16);
                }
                float er[32];
                tmem_ld32(tmem + lane_base + C_E + q * 64 + hf * 32, er);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float a = y[8 * c + 2 * i] + er[8 * c + 2 * i], b = y[8 * c + 2 * i + 1] + er[8 * c + 2 * i + 1];
                        rn2 = fmaf(a, a, rn2);
                        rn2 = fmaf(b, b, rn2);
                        hi[i] = pack_bf16(a, b);
                        lo[i] = pack_bf16(a - bf_lo(hi[i]), b - bf_hi(hi[i]));
                    }
                    *row_chunk(sA0, 4 * hf + c) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *row_chunk(sA1, 4 * hf + c) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            s_ss[q * TC_TOK + row] = rn2;
            tc_fence_before();
            tq_fence_proxy_async();
            mbar_arrive(bar_c);

            // ---------------- S: sign bits, norms ----------------
            bad |= !wait_warp(bar_m2, par);
            tc_fence_after();
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                float pr[32];
                tmem_ld32(tmem + lane_base + C_Y + q * 64 + hf * 32, pr);
                float w_lo = 0.f, w_hi = 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    w_lo = fmaf(mul_sat(mul_sat(pr[j], BIG), BIG), (float)(1u << j), w_lo);
                    w_hi = fmaf(mul_sat(mul_sat(pr[16 + j], BIG), BIG), (float)(1u << j), w_hi);
                }
                uint32_t w = (__float_as_uint(w_lo + 8388608.f) & 0xffffu) | (__float_as_uint(w_hi + 8388608.f) << 16);
                if (nd == 0.f) w = 0;
                if (wr) reinterpret_cast<uint32_t*>(rec + L.off_ksigns + tl * L.ksign_row)[2 * q + hf] = w;
            }
            tc_fence_before();
            if (compute_barrier_or(bad)) {   // the r' partial sums are published
                ok = false;
                break;
            }
            if (q == 0 && wr) {
                const float r2 = (s_ss[row] + s_ss[TC_TOK + row]) + (s_ss[2 * TC_TOK + row] + s_ss[3 * TC_TOK + row]);
                reinterpret_cast<__half*>(rec + L.off_knorm)[tl] = __float2half_rn(nd);
                reinterpret_cast<__half*>(rec + L.off_krnorm)[tl] = __float2half_rn(nd * __fsqrt_rn(r2));
            }
            tq_fence_proxy_async();
            compute_barrier_or(false);       // record image complete
            if (warp < 8) {
                if (tile_no == 0) pool_writes_may_begin();
                leave_records(p, L, sRec, h, warp, lane, dest);
                if (lane == 0) tq_bulk_wait_all_read();
            }
            compute_barrier_or(false);       // the image and s_ss are free for the next tile
        }
        if (!ok && tid == 0) atomicCAS(&g_tq_store_status, 0, (int)TQ_ERR_TIMEOUT);
        if (lane == 0 && warp < 8) tq_bulk_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

// (D x D) bf16 matrix, row-major: boxes of 64 columns x D rows (128 or 256), 128-byte swizzle
bool make_matrix_map(CUtensorMap* tm, const void* base, int D) {
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)D};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)D};
    const cuuint32_t estr[2] = {1, 1};
    return encode_tiled_fn()(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// (tokens, heads, D) bf16 with element strides: boxes of 64 channels x 128 tokens of one head; the
// dimension with the larger stride goes last
bool make_rows_map(CUtensorMap* tm, const void* base, int D, int64_t n_tokens, int n_heads, int64_t stride_token,
                   int64_t stride_head, bool tok_outer) {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_heads, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_token * 2};
    cuuint32_t box[3] = {64, 1, TC_TOK};
    if (!tok_outer) {
        dims[1] = (cuuint64_t)n_tokens; dims[2] = (cuuint64_t)n_heads;
        strides[0] = (cuuint64_t)stride_token * 2; strides[1] = (cuuint64_t)stride_head * 2;
        box[1] = TC_TOK; box[2] = 1;
    }
    const cuuint32_t estr[3] = {1, 1, 1};
    return encode_tiled_fn()(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The four constant operands' maps are the same for every call of a layer: the last few sets are kept
// (a map holds only the address and the geometry, never the matrix).
struct OperandMapSet {
    const void* ptr[4];
    int D;
    CUtensorMap tm[4];
};
bool operand_maps(CUtensorMap (&out)[4], const tq_consts* consts, int D) {
    constexpr int SETS = 16;
    static std::mutex mu;
    static OperandMapSet sets[SETS];
    static int n_sets = 0, next = 0;
    const void* want[4] = {consts->pi_limbs[0], consts->pi_limbs[1], consts->m_limbs[0], consts->m_limbs[1]};
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < n_sets; ++i)
        if (sets[i].D == D && memcmp(sets[i].ptr, want, sizeof(want)) == 0) {
            memcpy(out, sets[i].tm, sizeof(sets[i].tm));
            return true;
        }
    OperandMapSet fresh;
    memcpy(fresh.ptr, want, sizeof(want));
    fresh.D = D;
    for (int i = 0; i < 4; ++i)
        if (!make_matrix_map(&fresh.tm[i], want[i], D)) return false;
    sets[next] = fresh;
    next = (next + 1) % SETS;
    if (n_sets < SETS) ++n_sets;
    memcpy(out, fresh.tm, sizeof(fresh.tm));
    return true;
}

// Paged cache (blocks, block_size tokens, heads, D) bf16 with element strides: boxes of 64 channels x
// `box_rows` tokens of one head of one block.  `rows` is the extent of the token dimension - the block
// size, or fewer for the view whose rows past the sequence's last token must read as zeros.
bool make_paged_map(CUtensorMap* tm, const void* base, int D, int64_t num_blocks, int rows, int box_rows, int n_heads,
                    int64_t stride_block, int64_t stride_token, int64_t stride_head, bool tok_outer) {
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)n_heads, (cuuint64_t)rows, (cuuint64_t)num_blocks};
    cuuint64_t strides[3] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_token * 2, (cuuint64_t)stride_block * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    if (!tok_outer) {
        dims[1] = (cuuint64_t)rows; dims[2] = (cuuint64_t)n_heads;
        strides[0] = (cuuint64_t)stride_token * 2; strides[1] = (cuuint64_t)stride_head * 2;
        box[1] = (cuuint32_t)box_rows; box[2] = 1;
    }
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return encode_tiled_fn()(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Launches a tensor-core kernel when the call fits one: head_dim 128 (any bit widths) or 256 (3-bit keys
// with 2-bit values, the combination whose record image fits beside the operands), bf16, 16-byte aligned
// rows, the split operands present.  Otherwise *handled stays 0 and tq_store runs its fp32 kernel.
//
// `paged` (may be null) makes key / value the two planes of a paged cache: rows are then addressed as
// (source block from paged->table, token in block) instead of by stride_token from one base.
int tq_store_tc_launch(const tq_consts* consts, const void* key, const void* value, tq_dtype dtype, int64_t n_tokens,
                       int32_t n_heads, int64_t stride_token, int64_t stride_head, const int64_t* slot_mapping,
                       const int32_t* block_table, int64_t start_pos, const tq_pool* pool, cudaStream_t st,
                       int* handled, const TqPagedSource* paged) {
    *handled = 0;
    const tq_config& cfg = consts->cfg;
    const int D = cfg.head_dim;
    if ((D != TC_D && D != D2) || dtype != TQ_BF16) return TQ_OK;
    const TqLayout L = tq_make_layout(D, cfg.key_bits, cfg.value_bits);
    const size_t img = (size_t)8 * L.block_bytes;
    const size_t smem256 = 2 * (size_t)D2_TILE_BYTES + 2 * (size_t)D2_CHUNK_BYTES + img + 4 * TC_TOK * sizeof(float) +
                           11 * sizeof(uint64_t) + 16 + 1024;
    if (D == D2 && smem256 > SMEM_LIMIT) return TQ_OK;
    if (!consts->pi_limbs[0] || !consts->pi_limbs[1] || !consts->m_limbs[0] || !consts->m_limbs[1]) return TQ_OK;
    if (((uintptr_t)key & 15) || ((uintptr_t)value & 15) || (stride_token & 7) || (stride_head & 7)) return TQ_OK;
    if (stride_token < D || (n_heads > 1 && stride_head < D)) return TQ_OK;
    if (n_heads == 1) stride_head = stride_token > D ? D : stride_token;
    int bs_log2 = 0;
    if (paged) {   // block sizes the box stacking can express: 16, 32, 64 and multiples of 128 that are powers of two
        while ((1 << bs_log2) < paged->block_size && bs_log2 < 30) ++bs_log2;
        if ((1 << bs_log2) != paged->block_size || bs_log2 < 4) return TQ_OK;
        if ((start_pos & 15) || slot_mapping || (paged->stride_block & 7) || paged->num_blocks >= ((int64_t)1 << 31))
            return TQ_OK;
    }   // never dereferenced; keep the map well formed
    for (int i = 0; i < 2; ++i)
        if (((uintptr_t)consts->pi_limbs[i] & 15) || ((uintptr_t)consts->m_limbs[i] & 15)) return TQ_OK;
    if (n_tokens >= ((int64_t)1 << 31) - 256) return TQ_OK;   // 32-bit box coordinates
    if (encode_tiled_fn() == nullptr) return TQ_OK;
    {   // the kernel's comparison arithmetic treats only the middle boundary as possibly (next to) zero
        const int nb = (1 << (cfg.key_bits - 1)) - 1;
        for (int i = 0; i < nb; ++i)
            if (i != nb / 2 && !(fabsf(consts->boundaries[i]) >= 1e-30f && fabsf(consts->boundaries[i]) < 2.f)) return TQ_OK;
        if (!(fabsf(consts->boundaries[nb / 2]) < 2.f)) return TQ_OK;
    }

    TcParams p;
    p.n_tokens = n_tokens;
    p.slot_mapping = slot_mapping;
    p.block_table = block_table;
    p.start_pos = slot_mapping ? 0 : start_pos;
    p.lead = slot_mapping ? 0 : (int)(start_pos & 15);
    p.pool = (uint8_t*)pool->base;
    p.num_blocks = pool->num_blocks;
    p.H = n_heads;
    p.tok_outer = stride_token >= stride_head ? 1 : 0;
    p.src_table = paged ? paged->table : nullptr;
    p.src_num_blocks = paged ? (int32_t)paged->num_blocks : 0;
    p.src_bs_log2 = bs_log2;
    p.src_tail_block = paged && (n_tokens & (paged->block_size - 1)) ? n_tokens >> bs_log2 : -1;
    for (int i = 0; i < TQ_MAX_CENTROIDS; ++i) {
        p.cb.centroids[i] = consts->centroids[i];
        p.cb.boundaries[i] = consts->boundaries[i];
    }
    const int64_t n_tiles = ((p.lead + n_tokens + TC_TOK - 1) / TC_TOK) * n_heads;
    if (n_tiles >= ((int64_t)1 << 30)) return TQ_OK;
    p.n_tiles = (int)n_tiles;

    CUtensorMap tm_k, tm_v, tm_kt, tm_vt, tm_b[4];
    bool maps_ok;
    if (paged) {
        const int bs = paged->block_size, box_rows = bs < TC_TOK ? bs : TC_TOK;
        const int tail = (int)(n_tokens & (bs - 1));
        const bool to = p.tok_outer != 0;
        maps_ok = make_paged_map(&tm_k, key, D, paged->num_blocks, bs, box_rows, n_heads, paged->stride_block, stride_token, stride_head, to) &&
                  make_paged_map(&tm_v, value, D, paged->num_blocks, bs, box_rows, n_heads, paged->stride_block, stride_token, stride_head, to) &&
                  make_paged_map(&tm_kt, key, D, paged->num_blocks, tail ? tail : bs, box_rows, n_heads, paged->stride_block, stride_token, stride_head, to) &&
                  make_paged_map(&tm_vt, value, D, paged->num_blocks, tail ? tail : bs, box_rows, n_heads, paged->stride_block, stride_token, stride_head, to);
    } else {
        maps_ok = make_rows_map(&tm_k, key, D, n_tokens, n_heads, stride_token, stride_head, p.tok_outer != 0) &&
                  make_rows_map(&tm_v, value, D, n_tokens, n_heads, stride_token, stride_head, p.tok_outer != 0);
        tm_kt = tm_k;
        tm_vt = tm_v;
    }
    if (!maps_ok || !operand_maps(tm_b, consts, D))
        return TQ_OK;   // a stride pattern the tensor map cannot express: the fp32 kernel takes the call
    *handled = 1;

    const int mse_bits = cfg.key_bits - 1;
    const int sms = tq_sm_count();
    const unsigned grid = (unsigned)(p.n_tiles < sms ? p.n_tiles : sms);
    // programmatic dependent launch: this grid may begin under the tail of the launch ahead of it
    cudaLaunchConfig_t lc = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = tq_pdl_for_store(st);   // behind a decode launch (ring append): plain stream order
    tq_note_launch(st, TQ_LAUNCH_STORE_EARLY);
    lc.stream = st;
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(TC_LAUNCH);
    if (D == D2) {
        p.n_rec_buf = 1;
        if (mse_bits != 2 || cfg.value_bits != 2) {   // unreachable: no other image passed the size check above
            *handled = 0;
            return TQ_OK;
        }
        static TqSmemOptIn opt_in;
        if (tq_opt_in_smem(tq_store_tc256_kernel<2, 2>, smem256, opt_in) != TQ_OK) return TQ_ERR_CUDA;
        lc.dynamicSmemBytes = smem256;
        return cudaLaunchKernelEx(&lc, tq_store_tc256_kernel<2, 2>, tm_k, tm_v, tm_kt, tm_vt, tm_b[0], tm_b[1], tm_b[2],
                                  tm_b[3], p) == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
    }
    const size_t fixed = (size_t)6 * MAT_BYTES + 8 * TC_TOK * sizeof(float) + 12 * sizeof(uint64_t) + 16 + 1024;
    p.n_rec_buf = fixed + 2 * img <= SMEM_LIMIT ? 2 : 1;
    const size_t smem = fixed + (size_t)p.n_rec_buf * img;
    cudaError_t launched = cudaSuccess;
#define TQ_TC(MB, VB)                                                                                            \
    do {                                                                                                         \
        static TqSmemOptIn opt_in;                                                                               \
        if (tq_opt_in_smem(tq_store_tc_kernel<MB, VB>, smem, opt_in) != TQ_OK) return TQ_ERR_CUDA;               \
        lc.dynamicSmemBytes = smem;                                                                              \
        launched = cudaLaunchKernelEx(&lc, tq_store_tc_kernel<MB, VB>, tm_k, tm_v, tm_kt, tm_vt, tm_b[0], tm_b[1],   \
                                      tm_b[2], tm_b[3], p);                                                      \
    } while (0)
    if (mse_bits == 2 && cfg.value_bits == 2) TQ_TC(2, 2);
    else if (mse_bits == 2) TQ_TC(2, 4);
    else if (cfg.value_bits == 2) TQ_TC(3, 2);
    else TQ_TC(3, 4);
#undef TQ_TC
    return launched == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

// Status left by the tensor-core store kernels since the last call (0, or a tq_status if a bounded wait ran
// out or a block index was out of range); reading it clears it.  Synchronises the device.
extern "C" int tq_store_read_status(int32_t* out) {
    if (!out) return TQ_ERR_NULL;
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tq_store_status, sizeof(int)) != cudaSuccess) return TQ_ERR_CUDA;
    if (v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_tq_store_status, &zero, sizeof(int)) != cudaSuccess) return TQ_ERR_CUDA;
    }
    *out = v;
    return TQ_OK;
}
