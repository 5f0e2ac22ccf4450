// Host-only entry points: configuration checks, layout queries, messages.
#include <mutex>

#include "tq_common.cuh"

int tq_check_config(const tq_config* cfg) {
    if (!cfg) return TQ_ERR_NULL;
    if (cfg->head_dim != 128 && cfg->head_dim != 256) return TQ_ERR_UNSUPPORTED;
    if (cfg->key_bits != 3 && cfg->key_bits != 4) return TQ_ERR_UNSUPPORTED;
    if (cfg->value_bits != 2 && cfg->value_bits != 4) return TQ_ERR_UNSUPPORTED;
    if (cfg->group_size != 32) return TQ_ERR_UNSUPPORTED;
    return TQ_OK;
}

int tq_current_device() {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

int tq_sm_count() {
    static int sms[TQ_MAX_DEVICES] = {};
    const int dev = tq_current_device();
    if (dev < 0 || dev >= TQ_MAX_DEVICES) return 148;
    if (sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

namespace {
struct StreamNote {
    cudaStream_t st;
    int kind;
};
std::mutex g_note_mu;
StreamNote g_notes[TQ_MAX_DEVICES][8];
int g_note_count[TQ_MAX_DEVICES], g_note_next[TQ_MAX_DEVICES];
}  // namespace

void tq_note_launch(cudaStream_t st, int kind) {
    const int dev = tq_current_device();
    if (dev < 0 || dev >= TQ_MAX_DEVICES) return;
    std::lock_guard<std::mutex> lock(g_note_mu);
    for (int i = 0; i < g_note_count[dev]; ++i)
        if (g_notes[dev][i].st == st) {
            g_notes[dev][i].kind = kind;
            return;
        }
    const int slot = g_note_next[dev];
    g_notes[dev][slot] = StreamNote{st, kind};
    g_note_next[dev] = (slot + 1) % 8;
    if (g_note_count[dev] < 8) ++g_note_count[dev];
}

// Kind of the library's latest launch on the stream (a stream never noted, or whose note was displaced: unknown).
int tq_last_launch(cudaStream_t st) {
    const int dev = tq_current_device();
    if (dev < 0 || dev >= TQ_MAX_DEVICES) return TQ_LAUNCH_UNKNOWN;
    std::lock_guard<std::mutex> lock(g_note_mu);
    for (int i = 0; i < g_note_count[dev]; ++i)
        if (g_notes[dev][i].st == st) return g_notes[dev][i].kind;
    return TQ_LAUNCH_UNKNOWN;
}

extern "C" int tq_get_layout(const tq_config* cfg, tq_layout* out) {
    if (!cfg || !out) return TQ_ERR_NULL;
    int rc = tq_check_config(cfg);
    if (rc != TQ_OK) return rc;
    const TqLayout L = tq_make_layout(cfg->head_dim, cfg->key_bits, cfg->value_bits);
    out->block_tokens = TQ_BLOCK_TOKENS;
    out->kcode_row = L.kcode_row;
    out->ksign_row = L.ksign_row;
    out->vcode_row = L.vcode_row;
    out->n_groups = L.ngroups;
    out->off_kcodes = L.off_kcodes;
    out->off_ksigns = L.off_ksigns;
    out->off_knorm = L.off_knorm;
    out->off_krnorm = L.off_krnorm;
    out->off_vcodes = L.off_vcodes;
    out->off_vscale = L.off_vscale;
    out->off_vzero = L.off_vzero;
    out->block_bytes = L.block_bytes;
    out->bytes_per_token = L.block_bytes / TQ_BLOCK_TOKENS;
    return TQ_OK;
}

extern "C" int tq_vcode_native_offset(const tq_config* cfg, int32_t token, int32_t canonical_byte) {
    int rc = tq_check_config(cfg);
    if (rc != TQ_OK) return rc;
    const TqLayout L = tq_make_layout(cfg->head_dim, cfg->key_bits, cfg->value_bits);
    if (token < 0 || token >= TQ_BLOCK_TOKENS || canonical_byte < 0 || canonical_byte >= L.vcode_row)
        return TQ_ERR_RANGE;
    return tq_vcode_native(cfg->head_dim, cfg->value_bits, token, canonical_byte);
}

extern "C" const char* tq_strerror(int status) {
    switch (status) {
        case TQ_OK: return "ok";
        case TQ_ERR_NULL: return "a required pointer is NULL";
        case TQ_ERR_SHAPE: return "a size is zero, negative or inconsistent";
        case TQ_ERR_ALIGN: return "a pointer or stride is not aligned as required";
        case TQ_ERR_UNSUPPORTED: return "head_dim, bit width, group size or dtype outside the compiled set";
        case TQ_ERR_CUDA: return "the CUDA runtime refused the launch";
        case TQ_ERR_WORKSPACE: return "workspace too small";
        case TQ_ERR_RANGE: return "index out of range";
        case TQ_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        default: return "unknown status";
    }
}

extern "C" const char* tq_version(void) { return "turboquant_b200 0.1 (sm_100a)"; }

extern "C" int tq_workspace_init(void* workspace, size_t bytes, void* stream) {
    if (!workspace) return TQ_ERR_NULL;
    if (bytes < TQ_WS_HEADER_BYTES) return TQ_ERR_WORKSPACE;
    return cudaMemsetAsync(workspace, 0, bytes, (cudaStream_t)stream) == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}

extern "C" int tq_read_status(const void* workspace, void* stream, int32_t* out) {
    if (!workspace || !out) return TQ_ERR_NULL;
    if (cudaMemcpyAsync(out, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess)
        return TQ_ERR_CUDA;
    return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? TQ_OK : TQ_ERR_CUDA;
}
