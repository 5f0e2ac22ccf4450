// Shared device/host helpers: block-record layout, dtype rounding, bulk-copy
// (TMA) and mbarrier wrappers with bounded waits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "turboquant_b200.h"

#define TQ_HD __host__ __device__ __forceinline__

// ---------------------------------------------------------------------------
// block-record layout
// ---------------------------------------------------------------------------

struct TqLayout {
    int D, mse_bits, val_bits;
    int kcode_row, ksign_row, vcode_row, ngroups;
    int off_kcodes, off_ksigns, off_knorm, off_krnorm, off_vcodes, off_vscale, off_vzero;
    int block_bytes;
};

// Bytes of packed MSE codes per token: the reference packs 1-bit codes 8 per
// byte, 2-bit 4 per byte and 3/4-bit codes 2 per byte (quantizer.py:50-59).
TQ_HD int tq_kcode_row(int D, int mse_bits) {
    return mse_bits == 1 ? D / 8 : (mse_bits == 2 ? D / 4 : D / 2);
}

TQ_HD TqLayout tq_make_layout(int D, int key_bits, int val_bits) {
    TqLayout L;
    L.D = D;
    L.mse_bits = key_bits - 1;
    L.val_bits = val_bits;
    L.kcode_row = tq_kcode_row(D, L.mse_bits);
    L.ksign_row = D / 8;
    L.vcode_row = val_bits == 2 ? D / 4 : D / 2;
    L.ngroups = D / 32;
    L.off_kcodes = 0;
    L.off_ksigns = L.off_kcodes + TQ_BLOCK_TOKENS * L.kcode_row;
    L.off_knorm = L.off_ksigns + TQ_BLOCK_TOKENS * L.ksign_row;
    L.off_krnorm = L.off_knorm + TQ_BLOCK_TOKENS * 2;
    L.off_vcodes = L.off_krnorm + TQ_BLOCK_TOKENS * 2;
    L.off_vscale = L.off_vcodes + TQ_BLOCK_TOKENS * L.vcode_row;
    L.off_vzero = L.off_vscale + L.ngroups * TQ_BLOCK_TOKENS * 2;
    L.block_bytes = L.off_vzero + L.ngroups * TQ_BLOCK_TOKENS * 2;
    return L;
}

// Value codes keep the reference's code values and its packing inside a byte
// (kv_cache.py:80-90) but the BYTES of a 16-token block are ordered for the
// tensor-core decode kernel.  In its P*V product the 16 rows of one MMA tile
// are 16 channels of one quantisation group and the contraction runs over
// tokens, so lane (j, q) of a warp (j = lane/4, q = lane%4) needs, for tokens
// 4q..4q+3 and every group, the byte(s) that hold channels 4j..4j+3 of the
// group.  Those bytes are stored as 32-bit words
//     [tokA byte0, tokA byte1, tokB byte0, tokB byte1]   (tokA even, tokB = tokA+1)
// so that masking one word yields fp16 pairs (code of tokA, code of tokB);
// for 2-bit codes byte0/byte1 belong to two adjacent groups, for 4-bit codes
// to the two bytes of one group.  Words are laid out [chunk][lane][4 words]:
// one 128-bit shared-memory load per lane per chunk, conflict free.
TQ_HD int tq_vcode_native(int D, int val_bits, int tok, int cbyte) {
    const int ng = D / 32;
    const int q = tok >> 2, p = (tok >> 1) & 1, ab = tok & 1;
    int wi, byte, j;
    if (val_bits == 2) {
        const int grp = cbyte >> 3;
        j = cbyte & 7;
        wi = p * (ng / 2) + (grp >> 1);
        byte = (grp & 1) + 2 * ab;
    } else {
        const int grp = cbyte >> 4;
        const int bp = cbyte & 15;
        j = bp >> 1;
        wi = p * ng + grp;
        byte = (bp & 1) + 2 * ab;
    }
    const int lane = j * 4 + q;
    return (wi >> 2) * 512 + lane * 16 + (wi & 3) * 4 + byte;
}

// ---------------------------------------------------------------------------
// dtype helpers: torch CPU computes bf16/fp16 elementwise ops in fp32 and
// rounds the result to the tensor dtype after every op.
// ---------------------------------------------------------------------------

template <int DT> struct TqElem;
template <> struct TqElem<TQ_F32> {
    using type = float;
    static __device__ __forceinline__ float load(const void* p, int64_t i) { return ((const float*)p)[i]; }
    static __device__ __forceinline__ float round(float x) { return x; }
    static __device__ __forceinline__ void store(void* p, int64_t i, float x) { ((float*)p)[i] = x; }
};
template <> struct TqElem<TQ_BF16> {
    using type = __nv_bfloat16;
    static __device__ __forceinline__ float load(const void* p, int64_t i) {
        return __bfloat162float(((const __nv_bfloat16*)p)[i]);
    }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ void store(void* p, int64_t i, float x) {
        ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(x);
    }
};
template <> struct TqElem<TQ_F16> {
    using type = __half;
    static __device__ __forceinline__ float load(const void* p, int64_t i) {
        return __half2float(((const __half*)p)[i]);
    }
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ void store(void* p, int64_t i, float x) { ((__half*)p)[i] = __float2half_rn(x); }
};

__device__ __forceinline__ float tq_load_any(const void* p, int64_t i, int dt) {
    if (dt == TQ_F32) return ((const float*)p)[i];
    if (dt == TQ_BF16) return __bfloat162float(((const __nv_bfloat16*)p)[i]);
    return __half2float(((const __half*)p)[i]);
}
__device__ __forceinline__ void tq_store_any(void* p, int64_t i, float x, int dt) {
    if (dt == TQ_F32) ((float*)p)[i] = x;
    else if (dt == TQ_BF16) ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(x);
    else ((__half*)p)[i] = __float2half_rn(x);
}

// four consecutive elements starting at an index that is a multiple of 4, one store
__device__ __forceinline__ void tq_store4_any(void* p, int64_t i, float a, float b, float c, float d, int dt) {
    if (dt == TQ_F32) {
        *reinterpret_cast<float4*>((float*)p + i) = make_float4(a, b, c, d);
    } else if (dt == TQ_BF16) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        *reinterpret_cast<uint2*>((__nv_bfloat16*)p + i) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        const __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
        *reinterpret_cast<uint2*>((__half*)p + i) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

static inline size_t tq_dtype_size(int dt) { return dt == TQ_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------
// bulk copies (TMA, untiled) completing on an mbarrier; every wait is bounded
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t tq_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void tq_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tq_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tq_mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tq_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tq_smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool tq_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tq_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Spin at most `limit` polls; false means the copy never arrived.
__device__ __forceinline__ bool tq_mbar_wait_bounded(uint64_t* bar, uint32_t parity, int limit = (1 << 22)) {
    for (int i = 0; i < limit; ++i)
        if (tq_mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared; dst, src and bytes must all be multiples of 16.
__device__ __forceinline__ void tq_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     tq_smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(tq_smem_u32(bar))
                 : "memory");
}
// shared -> global bulk store (bulk async-group completion).
__device__ __forceinline__ void tq_bulk_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(tq_smem_u32(src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tq_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tq_bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tq_bulk_wait_all_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tq_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float tq_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float tq_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Centroids / boundaries travel as kernel parameters (constant bank).
struct TqCodebook {
    float centroids[TQ_MAX_CENTROIDS];
    float boundaries[TQ_MAX_CENTROIDS];
};

// Workspace header: word 0 = device status, then per-(sequence, kv head) tickets.
#define TQ_WS_HEADER_BYTES 256

int tq_check_config(const tq_config* cfg);

// ---------------------------------------------------------------------------
// per-device host bookkeeping: kernel attributes and SM counts belong to a
// device, not to the process
// ---------------------------------------------------------------------------
constexpr int TQ_MAX_DEVICES = 64;
int tq_current_device();   // ordinal of the calling thread's current device, -1 on error
int tq_sm_count();         // multiprocessors of the current device (148 when the query fails)

// Which of the library's kernels was launched last on a stream.  Several kernels let the launch behind them
// begin before they have finished (programmatic dependent launch) and do part of their work before they wait
// for the launch ahead; that is only safe when the launch still in flight cannot be writing what is read early:
//   * the tensor-core store kernels fetch their key / value rows before the wait.  The decode family appends
//     the new token to the ring - rows a flush then reads - so a store behind a decode launch is launched in
//     plain stream order;
//   * the decode family reads sequence lengths, block tables and the first pool records before the wait.
//     The tensor-core store kernels write the pool and let their dependents begin at once, so the first
//     kernel of a decode call behind such a store is launched in plain stream order.
// Kernels of other libraries between two of ours never start early and only make the order stricter; a
// stream the library has not seen counts as unknown.
enum TqLaunchKind { TQ_LAUNCH_UNKNOWN = 0, TQ_LAUNCH_DECODE = 1, TQ_LAUNCH_STORE_EARLY = 2, TQ_LAUNCH_NEUTRAL = 3 };
void tq_note_launch(cudaStream_t st, int kind);
int tq_last_launch(cudaStream_t st);
// programmatic-launch attribute count (0 or 1) for a kernel of the decode family / of the early-starting stores
inline int tq_pdl_for_decode(cudaStream_t st) { return tq_last_launch(st) == TQ_LAUNCH_STORE_EARLY ? 0 : 1; }
inline int tq_pdl_for_store(cudaStream_t st) {
    const int k = tq_last_launch(st);
    return (k == TQ_LAUNCH_STORE_EARLY || k == TQ_LAUNCH_NEUTRAL) ? 1 : 0;
}

// Largest dynamic shared-memory size a kernel has been opted in for, per device.
// A paged bf16 cache as the source of a store call (see tq_store_paged).
struct TqPagedSource {
    const int32_t* table;    // device: logical block of the sequence -> physical block
    int64_t num_blocks;      // physical blocks in the cache
    int32_t block_size;      // tokens per block
    int64_t stride_block;    // elements between blocks
};

struct TqSmemOptIn {
    size_t bytes[TQ_MAX_DEVICES] = {};
};
// Raises the kernel's dynamic shared-memory limit on the current device when `smem`
// exceeds what was set there before; steady-state calls issue nothing but the launch.
template <class Kern>
inline int tq_opt_in_smem(Kern kern, size_t smem, TqSmemOptIn& state) {
    const int dev = tq_current_device();
    if (dev < 0 || dev >= TQ_MAX_DEVICES) return TQ_ERR_CUDA;
    if (smem > state.bytes[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return TQ_ERR_CUDA;
        state.bytes[dev] = smem;
    }
    return TQ_OK;
}
