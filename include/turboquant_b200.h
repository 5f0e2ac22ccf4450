/*
 * turboquant_b200 - C ABI of the B200 (sm_100a) TurboQuant KV-cache hot path.
 *
 * The reference implementation (0xSero/turboquant) has no FFI: its hot path is
 * Python calling torch ops.  Each entry point below replaces the torch
 * arithmetic of one reference function; the Python host classes of this
 * package keep the reference's names and call these through ctypes.
 *
 * Conventions
 *   - plain pointers and sizes only; every data pointer is a DEVICE pointer
 *     owned by the caller unless its comment says "host";
 *   - every call returns 0 (TQ_OK) or a negative tq_status, never throws;
 *   - no entry point allocates, frees or synchronises: scratch memory is the
 *     caller's `workspace`, work is enqueued on the caller's `stream`
 *     (a cudaStream_t passed as void*), so calls can be captured in CUDA graphs;
 *   - arguments are validated on the host before anything is launched.
 *
 * Storage: compressed K/V lives in a pool of fixed-size BLOCK RECORDS.  One
 * record holds TQ_BLOCK_TOKENS (16) consecutive tokens of ONE kv head:
 *
 *     pool[(block * num_kv_heads + head) * layout.block_bytes + ...]
 *       off_kcodes : [16][kcode_row] key MSE codes, byte order of the reference's
 *                    _pack_indices (LSB first, 3-bit codes in nibbles)
 *       off_ksigns : [16][D/8]      QJL sign bits (bit j of byte i = coordinate 8i+j)
 *       off_knorm  : [16] fp16      key norms
 *       off_krnorm : [16] fp16      residual norms
 *       off_vcodes : 16*vcode_row   value codes; code VALUES as the reference packs
 *                    them, byte ORDER permuted for the decode kernel's tensor-core
 *                    fragments (tq_vcode_native_offset)
 *       off_vscale : [D/32][16] fp16 group scales, group-major
 *       off_vzero  : [D/32][16] fp16 group zero points, group-major
 *
 * A sequence is a list of blocks (block table), as in a paged KV cache; a
 * "flat" store is a pool with the identity block table.  tq_pool_to_planes
 * returns the reference's flat plane format (store.py:19-23) for API users.
 */
#ifndef TURBOQUANT_B200_H
#define TURBOQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_BLOCK_TOKENS 16
#define TQ_MAX_CENTROIDS 16
#define TQ_MAX_GROUP_HEADS 8   /* query heads per kv head handled by one decode CTA */

typedef enum tq_status {
    TQ_OK = 0,
    TQ_ERR_NULL = -1,        /* a required pointer is NULL */
    TQ_ERR_SHAPE = -2,       /* a size is zero, negative or inconsistent */
    TQ_ERR_ALIGN = -3,       /* a pointer or stride breaks the 16-byte rule */
    TQ_ERR_UNSUPPORTED = -4, /* head_dim / bits / dtype outside the compiled set */
    TQ_ERR_CUDA = -5,        /* the CUDA runtime refused the launch */
    TQ_ERR_WORKSPACE = -6,   /* workspace too small */
    TQ_ERR_RANGE = -7,       /* an index (block, slot, split) is out of range */
    TQ_ERR_TIMEOUT = -8      /* a bounded device-side wait ran out (see tq_read_status) */
} tq_status;

typedef enum tq_dtype { TQ_F32 = 0, TQ_BF16 = 1, TQ_F16 = 2 } tq_dtype;

/* Quantiser shape.  Reference: CompressedKVStore.__init__ (store.py:34-57). */
typedef struct tq_config {
    int32_t head_dim;    /* 128 or 256 */
    int32_t key_bits;    /* 3 or 4 total key bits; the MSE stage uses key_bits-1 */
    int32_t value_bits;  /* 2 or 4 */
    int32_t group_size;  /* 32 (score.py:94 hard-codes it on the read path) */
} tq_config;

/* Per-layer constants.  Reference: TurboQuantMSE/Prod.__init__
 * (quantizer.py:102-127,187-212), rotation.py:17-56, codebook.py:176-181. */
typedef struct tq_consts {
    tq_config cfg;
    const float* pi;    /* (D,D) row-major rotation Pi            */
    const float* pi_t;  /* (D,D) Pi transposed                    */
    const float* s;     /* (D,D) row-major QJL matrix S           */
    const float* s_t;   /* (D,D) S transposed                     */
    float centroids[TQ_MAX_CENTROIDS];   /* host copy, 2^(key_bits-1) used */
    float boundaries[TQ_MAX_CENTROIDS];  /* host copy, interior decision boundaries, 2^(key_bits-1)-1 used */
    float qjl_scale;    /* sqrt(pi/2)/D (quantizer.py:212) */
    /* Optional operands of the tensor-core store kernel, all device, all (D,D)
     * bf16 row-major [n][k]: Pi split into three bf16 limbs, and M = S * Pi^T
     * split into two.  With any of them NULL the store runs its fp32 kernel. */
    const void* pi_limbs[3];
    const void* m_limbs[2];
    /* Optional operands of the tensor-core query preparation (large decode
     * batches at head_dim 128): S split into two bf16 limbs, (D,D) row-major.
     * With either NULL (or pi_limbs missing) the fp32 kernels prepare the queries. */
    const void* s_limbs[2];
} tq_consts;

/* Byte offsets inside one block record. */
typedef struct tq_layout {
    int32_t block_tokens;
    int32_t kcode_row, ksign_row, vcode_row, n_groups;
    int32_t off_kcodes, off_ksigns, off_knorm, off_krnorm, off_vcodes, off_vscale, off_vzero;
    int32_t block_bytes;
    int32_t bytes_per_token;   /* block_bytes / 16: 100 (D128 k3v2), 196 (D256 k3v2), 164 (D128 k4v4) */
} tq_layout;

typedef struct tq_pool {
    void* base;            /* num_blocks * num_kv_heads * block_bytes bytes, 256-byte aligned */
    int64_t num_blocks;
    int32_t num_kv_heads;
} tq_pool;

/* The reference's flat planes (store.py:19-23, quantizer.py:29-35, kv_cache.py:20-25),
 * row `capacity` tokens long per head; norms/scales/zeros as fp16. */
typedef struct tq_planes {
    uint8_t* mse_indices;     /* (H, capacity, kcode_row) */
    uint8_t* qjl_signs;       /* (H, capacity, D/8)       */
    uint16_t* norms;          /* (H, capacity) fp16       */
    uint16_t* residual_norms; /* (H, capacity) fp16       */
    uint8_t* v_data;          /* (H, capacity, vcode_row) */
    uint16_t* v_scales;       /* (H, capacity, D/32) fp16 */
    uint16_t* v_zeros;        /* (H, capacity, D/32) fp16 */
    int64_t capacity;
} tq_planes;

/* ---- host-only queries -------------------------------------------------- */

/* Layout of a block record for a configuration.  Replaces the byte accounting
 * of CompressedKVStore.memory_bytes (store.py:116-128). */
int tq_get_layout(const tq_config* cfg, tq_layout* out);

/* Position of canonical value-code byte `canonical_byte` of token-in-block
 * `token` inside the record's value-code area (see header comment). */
int tq_vcode_native_offset(const tq_config* cfg, int32_t token, int32_t canonical_byte);

/* Scratch bytes tq_decode needs for `batch` sequences, `num_q_heads` query
 * heads and at most `max_splits` sequence splits per (sequence, kv head). */
int tq_decode_workspace_bytes(const tq_config* cfg, int32_t batch, int32_t num_q_heads,
                              int32_t num_kv_heads, int32_t max_splits, size_t* out);

/* Scratch bytes tq_scores needs for n_vectors query vectors. */
int tq_scores_workspace_bytes(const tq_config* cfg, int64_t n_vectors, size_t* out);

const char* tq_strerror(int status);
const char* tq_version(void);

/* ---- prefill attention (no paged cache) ----------------------------------- */

/* Causal attention of one sequence's n_tokens query tokens over its own keys
 * and values, grouped query heads (query head q reads kv head
 * q / (num_q_heads / num_kv_heads)).  Replaces _no_alloc_prefill_attention
 * (integration/vllm.py:150-180: repeat_interleave of the kv heads +
 * F.scaled_dot_product_attention(is_causal=True)).  Element (t, h, :) of a
 * tensor is at base + t*stride_token + h*stride_head (in elements), head_dim
 * contiguous; bf16 or fp16, head_dim 128 or 256 (else TQ_ERR_UNSUPPORTED);
 * bases 16-byte aligned, strides multiples of 8 elements, token stride >=
 * head stride.  `out` in the input dtype.  Runs on the tensor cores
 * (tcgen05); the launch lets the next launch of the stream - normally
 * tq_store of the same keys and values - begin under its tail. */
int tq_prefill_attention(const void* query, const void* key, const void* value, void* out, tq_dtype dtype,
                         int64_t n_tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                         int64_t q_stride_token, int64_t q_stride_head, int64_t kv_stride_token,
                         int64_t kv_stride_head, int64_t out_stride_token, int64_t out_stride_head,
                         float scale, void* stream);

/* Status left by the prefill attention kernel since the last call (0, or
 * TQ_ERR_TIMEOUT if one of its bounded device-side waits ran out); reading
 * clears it.  Synchronises the device. */
int tq_prefill_attention_read_status(int32_t* out);

/* ---- store path ---------------------------------------------------------- */

/* Compress `n_tokens` key/value vectors of `n_heads` kv heads and write them
 * into the pool.  Replaces CompressedKVStore.append_chunk (store.py:73-90) =
 * TurboQuantProd.quantize (quantizer.py:231-257) + quantize_values
 * (kv_cache.py:45-98).  Element (t, h, :) of key/value is at
 * base + t*stride_token + h*stride_head (in elements), D contiguous.
 * Destination of token t: slot_mapping[t] (= block*16 + offset, negative =
 * skip) when slot_mapping is given, else position start_pos+t of the
 * sequence whose blocks are block_table[0..].
 * bf16 input with 16-byte aligned rows runs on the tensor cores (head_dim 128;
 * head_dim 256 with 3-bit keys and 2-bit values); those kernels are launched
 * as programmatic dependents: one that follows another store or
 * tq_prefill_attention on the stream may fetch its key / value rows while
 * that launch is still running, and touches the pool only after it has
 * completed.  A store that follows one of the tq_decode* calls on the stream
 * (whose ring append may still be writing rows the store is about to read)
 * is launched in plain stream order; likewise the first kernel of a tq_decode*
 * call that follows one of these stores (the decode kernels fetch lengths,
 * block tables and their first records before they wait for the launch ahead).
 * Device-side status: tq_store_read_status. */
int tq_store(const tq_consts* consts, const void* key, const void* value, tq_dtype dtype,
             int64_t n_tokens, int32_t n_heads, int64_t stride_token, int64_t stride_head,
             const int64_t* slot_mapping, const int32_t* block_table, int64_t start_pos,
             const tq_pool* pool, void* stream);

/* Compress the first `n_tokens` tokens of a sequence that lives in a PAGED
 * bf16 cache - blocks of `src_block_size` tokens, element (b, t, h, :) of the
 * key plane at key_cache + b*stride_block + t*stride_token + h*stride_head
 * (in elements; the value plane likewise from value_cache), logical block j
 * of the sequence at physical block src_block_table[j] (device memory) - and
 * write them into the pool at positions start_pos.. of block_table, in one
 * launch whose tile loader walks the table (nothing is gathered first).
 * Replaces the gather loop of KVCaptureEngine.ingest_prefill_from_paged_cache
 * (capture.py:187-217) followed by append_chunk; for vLLM's
 * (2, num_blocks, block_size, H, D) tensor pass the two planes' bases.
 * Needs the tensor-core store (bf16; head_dim 128, or 256 with 3-bit keys and
 * 2-bit values; split operands in `consts`), a power-of-two src_block_size
 * >= 16, start_pos a multiple of 16 and 16-byte aligned planes and strides:
 * anything else returns TQ_ERR_UNSUPPORTED and nothing is launched.  Records
 * are byte-identical to tq_store on the gathered rows. */
int tq_store_paged(const tq_consts* consts, const void* key_cache, const void* value_cache, tq_dtype dtype,
                   int64_t src_num_blocks, int32_t src_block_size, int32_t n_heads, int64_t stride_block,
                   int64_t stride_token, int64_t stride_head, const int32_t* src_block_table, int64_t n_tokens,
                   const int32_t* block_table, int64_t start_pos, const tq_pool* pool, void* stream);

/* Status left by the tensor-core store kernels since the last call: 0, or
 * TQ_ERR_TIMEOUT / TQ_ERR_RANGE if one of their bounded waits ran out or a
 * block index (destination or paged source) was out of range - such a
 * record is skipped, nothing outside the pool is touched.  Reading clears
 * the word.  Synchronises the device. */
int tq_store_read_status(int32_t* out);

/* ---- read path ------------------------------------------------------------ */

typedef struct tq_decode_args {
    const void* query;          /* (batch, num_q_heads, D), contiguous */
    tq_dtype q_dtype;           /* also the dtype of `out` */
    int32_t batch;
    int32_t num_q_heads;        /* multiple of pool.num_kv_heads, ratio <= 8 */
    const int32_t* block_table; /* (batch, block_table_stride) physical block ids */
    int32_t block_table_stride;
    const int32_t* seq_lens;    /* (batch) compressed tokens per sequence, device */
    int32_t max_seq_len;        /* host upper bound of seq_lens, sizes the grid */
    int32_t min_history;        /* compressed history shorter than this is ignored (score.py:26: 16) */
    const void* ring_k;         /* exact recent tokens, element (b, r, h, :) at        */
    const void* ring_v;         /*   b*ring_stride_seq + r*ring_stride_token + h*D; or NULL */
    tq_dtype ring_dtype;
    const int32_t* ring_lens;   /* (batch) valid ring tokens, device; NULL with ring_k NULL */
    int32_t max_ring_len;       /* host upper bound of ring_lens */
    int64_t ring_stride_seq, ring_stride_token;
    float scale;                /* softmax scale, 1/sqrt(D) by default in the reference */
    void* out;                  /* (batch, num_q_heads, D) in q_dtype, 16-byte aligned */
    void* workspace;
    size_t workspace_bytes;
    int32_t num_splits;         /* sequence splits per (sequence, kv head); 0 = choose */
    int32_t query_prepared;     /* nonzero: the workspace already holds this query's rotated /
                                   sketched form from an earlier tq_decode with the same workspace */
    int32_t kernel;             /* 0: tensor-core kernel where it applies; 1: always the CUDA-core kernel */
    /* Optional: append one new exact token per sequence to the ring before attending (the
     * reference's KVCaptureEngine.ingest_decode, capture.py:219-228, fused into this call).
     * append_k / append_v: (batch, num_kv_heads, D) in ring_dtype, 16-byte aligned; the token of
     * sequence b lands at ring position ring_lens[b], which is then incremented on the device.
     * max_ring_len must already count the new token; ring_capacity is the ring's row count. */
    const void* append_k;
    const void* append_v;
    int32_t ring_capacity;
} tq_decode_args;

/* One decode-attention step over compressed history plus the exact ring:
 * softmax over [history || ring] jointly, no K/V materialised.  Replaces
 * compute_hybrid_attention (score.py:29-173) and the fused Triton decode
 * (triton_kernels.py:209-356,505-607). */
int tq_decode(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* args, void* stream);

/* tq_decode for a caller whose step inputs and result live in HOST memory (pinned for the
 * copies to be asynchronous): on `stream`, copies `in_bytes` from `host_in` to the device
 * buffer `dev_in`, runs tq_decode(args), and copies `out_bytes` from args->out to `host_out`.
 * args->query / append_k / append_v normally point into `dev_in`.  Nothing is synchronised; either
 * copy is skipped when its host pointer is NULL.  Transfers of at most 64 KiB to or from
 * page-locked host memory that the GPU can address (cudaHostAlloc / cudaHostRegister; checked
 * with cudaPointerGetAttributes) do not use the copy engines: when query / append_k / append_v
 * all point into `dev_in`, the query-preparation kernel reads them straight from `host_in`
 * (before it waits for the kernel ahead of it on the stream) and `dev_in` is not written at
 * all; otherwise a one-CTA kernel pulls `host_in` into `dev_in`.  The decode kernel writes the
 * result into `host_out` itself (args->out is then left untouched).  Anything else goes through
 * cudaMemcpyAsync.  `host_in` must stay unchanged until the step has completed.  The answer of the
 * page-locked check is remembered per device and pointer: a buffer must stay registered for as
 * long as the library may be given it, and tq_host_buffer_forget must be called before it is
 * unregistered or freed (a stale "mapped" answer would let a kernel touch unmapped memory). */
int tq_decode_host_io(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* args, const void* host_in,
                      void* dev_in, size_t in_bytes, void* host_out, size_t out_bytes, void* stream);

/* Drop what tq_decode_host_io remembers about `host_ptr` (NULL: about every buffer, on every
 * device).  Host-only; call it before cudaHostUnregister / cudaFreeHost of a step buffer. */
int tq_host_buffer_forget(const void* host_ptr);

/* tq_decode without caller-provided scratch: `workspace` / `workspace_bytes` of
 * the arguments are ignored and a fixed array inside the library, resident on
 * every GPU that loads it, is used instead.  No counterpart in the reference:
 * it exists for hosts that cannot allocate device memory at the point of the
 * call (a plugin inside an engine that has already claimed the whole GPU for
 * its KV pool, or code running while that engine's allocator is locked).
 * Limits and rules:
 *   - the launch must fit tq_decode_static_scratch_bytes() (8 MiB); a larger
 *     batch x heads x splits is refused with TQ_ERR_WORKSPACE (lower num_splits
 *     or use tq_decode);
 *   - the first call on a device (of this function or of
 *     tq_decode_static_read_status) looks up the array's device address: make it
 *     with that device current, before any stream capture, and BEFORE the host
 *     application claims the rest of the device memory - the CUDA runtime loads
 *     the library's device code lazily, and the array's 8 MiB are taken from the
 *     device at that first use, not when the shared library is opened;
 *   - all calls on a device share the one array: calls that overlap on the GPU
 *     (different streams) race - serialise them;
 *   - `query_prepared` is ignored (the query is always prepared again);
 *   - arguments are checked before anything is enqueued; every call clears the
 *     array's tickets but not its status word, which keeps the first device-side
 *     error until tq_decode_static_read_status has returned it.
 * It calls no cudaMalloc / cudaFree or any other allocating routine. */
int tq_decode_static(const tq_consts* consts, const tq_pool* pool, const tq_decode_args* args, void* stream);
size_t tq_decode_static_scratch_bytes(void);

/* Device status word of the built-in array on the current device: 0, or the
 * tq_status (TQ_ERR_TIMEOUT, TQ_ERR_RANGE) a tq_decode_static kernel left there.
 * Synchronises `stream`, then clears a non-zero status.  No counterpart in the
 * reference, like tq_decode_static itself; allocates nothing. */
int tq_decode_static_read_status(void* stream, int32_t* out);

/* Unscaled logits <q, k_hat> of every query vector against the first n_tokens
 * of one sequence: query (H, n_q, D) -> logits (H, n_q, n_tokens) fp32.
 * Replaces TurboQuantProd.attention_score (quantizer.py:274-302) and the two
 * Triton score kernels (triton_kernels.py:55-196). */
int tq_scores(const tq_consts* consts, const tq_pool* pool, const int32_t* block_table,
              int64_t n_tokens, const void* query, tq_dtype q_dtype, int32_t n_q,
              float* logits, void* workspace, size_t workspace_bytes, void* stream);

/* ---- format conversion / dequantisation ----------------------------------- */

/* Gather tokens [0, n_tokens) of a sequence into the reference's flat planes
 * (CompressedKVStore.get_flat_cache, store.py:92-114). */
int tq_pool_to_planes(const tq_config* cfg, const tq_pool* pool, const int32_t* block_table,
                      int64_t n_tokens, const tq_planes* planes, void* stream);

/* Scatter flat planes (e.g. produced by the reference) into pool blocks. */
int tq_planes_to_pool(const tq_config* cfg, const tq_planes* planes, int64_t n_tokens,
                      const int32_t* block_table, int64_t start_pos, const tq_pool* pool, void* stream);

/* k_hat (H, n_tokens, D) fp32 = centroids[idx] @ Pi * norm + qjl_scale * rnorm * signs @ S.
 * Replaces TurboQuantProd.dequantize (quantizer.py:259-272); with_qjl = 0 gives
 * TurboQuantMSE.dequantize (quantizer.py:151-165). */
int tq_dequant_keys(const tq_consts* consts, const tq_pool* pool, const int32_t* block_table,
                    int64_t n_tokens, int32_t with_qjl, float* out, void* stream);

/* v (H, n_tokens, D) fp32 = code * scale + zero.  Replaces dequantize_values
 * (kv_cache.py:101-116). */
int tq_dequant_values(const tq_config* cfg, const tq_pool* pool, const int32_t* block_table,
                      int64_t n_tokens, float* out, void* stream);

/* The integer stages of the store path alone: bucket search + LSB-first code
 * packing of already rotated unit vectors y (n_rows, D) fp32, and sign packing
 * of QJL projections (n_rows, D) fp32.  codes (n_rows, kcode_row), signs
 * (n_rows, D/8).  Replaces torch.searchsorted + _pack_indices (quantizer.py:
 * 144-147,38-69) and _pack_qjl_signs (quantizer.py:214-222). */
int tq_pack_stage(const tq_consts* consts, const float* y, const float* projected, int64_t n_rows,
                  uint8_t* codes, uint8_t* signs, void* stream);

/* Zero a workspace (status word and tickets must start at zero; kernels leave
 * them zero again).  Call once after allocating it. */
int tq_workspace_init(void* workspace, size_t bytes, void* stream);

/* Device status word of a workspace: 0, or a tq_status written by a kernel:
 * TQ_ERR_TIMEOUT when a bounded wait ran out (the output of that launch is then
 * undefined; the workspace stays usable, its tickets are reset), TQ_ERR_RANGE
 * when a block index was outside the pool or a device-side length exceeded the
 * host bound (max_seq_len / max_ring_len; the length is clamped to the bound).
 * Synchronises the stream. */
int tq_read_status(const void* workspace, void* stream, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif /* TURBOQUANT_B200_H */
