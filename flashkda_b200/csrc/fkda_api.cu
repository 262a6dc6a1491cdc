// C ABI of the library: argument validation and dispatch to the device implementations.
// Replaces the reference's host binding (csrc/flash_kda.cpp:28-217) below its tensor checks.
#include "fkda_internal.h"

namespace {
thread_local int g_last_launches = 0;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}  // namespace

extern "C" {

int fkda_version(void) { return 1001; }

size_t fkda_params_size(void) { return sizeof(fkda_fwd_params); }

const char* fkda_status_string(int status) {
    switch (status) {
        case FKDA_OK: return "ok";
        case FKDA_ERR_NULL_POINTER: return "a required pointer is NULL";
        case FKDA_ERR_BAD_SHAPE: return "B, T, H, N or a stride is out of range";
        case FKDA_ERR_BAD_STATE_DTYPE: return "state_dtype must be FKDA_STATE_BF16 or FKDA_STATE_FP32";
        case FKDA_ERR_VARLEN_BATCH: return "B must be 1 when cu_seqlens is provided";
        case FKDA_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case FKDA_ERR_BAD_ALGO: return "unknown algo";
        case FKDA_ERR_LAUNCH: return "a kernel launch or CUDA runtime call failed";
        case FKDA_ERR_ALIGNMENT: return "tensor base addresses and token strides must be 16-byte aligned";
        case FKDA_ERR_DEVICE_STATUS: return "a kernel reported an internal time-out";
        case FKDA_ERR_NOALLOC_TOO_LARGE:
            return "problem too large for the built-in scratch of fkda_fwd_noalloc (use fkda_fwd with a workspace)";
        default: return "unknown status";
    }
}

static int resolve_algo(int32_t algo) {
    if (algo == FKDA_ALGO_AUTO) return FKDA_ALGO_TC;
    return algo;
}

size_t fkda_workspace_bytes(int64_t T_total, int64_t H, int64_t N, int32_t algo) {
    if (T_total < 0 || H <= 0 || N < 0) return 0;
    switch (resolve_algo(algo)) {
        case FKDA_ALGO_TWOPASS: return fkda::twopass_workspace_bytes(T_total, H, N);
        case FKDA_ALGO_TC: return fkda::tc_workspace_bytes(T_total, H, N);
        default: return 0;
    }
}

// Scratch bytes this particular call needs: never more than fkda_workspace_bytes() for the same totals, and much
// less where the call takes a path that keeps no per-chunk records (a decode step needs the status word only).
size_t fkda_workspace_bytes_for(const fkda_fwd_params* p) {
    if (p == nullptr || p->B <= 0 || p->T < 0 || p->H <= 0 || p->N <= 0) return 0;
    switch (resolve_algo(p->algo)) {
        case FKDA_ALGO_TWOPASS: return fkda::twopass_workspace_bytes(p->B * p->T, p->H, p->N);
        case FKDA_ALGO_TC: return fkda::tc_workspace_bytes_for(*p);
        default: return 0;
    }
}

int fkda_last_launch_count(void) { return g_last_launches; }

int fkda_device_status(const void* workspace, void* stream_v) {
    if (workspace == nullptr) workspace = fkda::noalloc_scratch_or_null();  // the built-in scratch of fkda_fwd_noalloc
    if (workspace == nullptr) return FKDA_ERR_NULL_POINTER;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
    int32_t hdr[2] = {0, 0};
    if (cudaMemcpyAsync(hdr, workspace, sizeof(hdr), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return FKDA_ERR_LAUNCH;
    return hdr[1] == 0 ? FKDA_OK : FKDA_ERR_DEVICE_STATUS;
}

int fkda_fwd(const fkda_fwd_params* p, void* stream_v) {
    g_last_launches = 0;
    if (p == nullptr) return FKDA_ERR_NULL_POINTER;
    if (p->B <= 0 || p->T < 0 || p->H <= 0 || p->H > 65535 || p->N <= 0) return FKDA_ERR_BAD_SHAPE;
    if (p->cu_seqlens != nullptr && p->B != 1) return FKDA_ERR_VARLEN_BATCH;
    if (p->cu_seqlens == nullptr && p->N != p->B) return FKDA_ERR_BAD_SHAPE;
    if (p->token_stride < p->H * FKDA_HEAD_DIM || p->beta_token_stride < p->H) return FKDA_ERR_BAD_SHAPE;
    if (p->state_dtype != FKDA_STATE_BF16 && p->state_dtype != FKDA_STATE_FP32) return FKDA_ERR_BAD_STATE_DTYPE;
    if (p->chunk_states != nullptr && (p->chunk_states_every < 1 || !aligned16(p->chunk_states))) return FKDA_ERR_BAD_SHAPE;
    if (!p->A_log || !p->dt_bias) return FKDA_ERR_NULL_POINTER;
    const int64_t T_total = p->B * p->T;
    if (T_total > 0 && (!p->q || !p->k || !p->v || !p->g || !p->beta || !p->out)) return FKDA_ERR_NULL_POINTER;
    if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->g) || !aligned16(p->out) ||
        !aligned16(p->dt_bias) || (p->token_stride % 8) != 0 || !aligned16(p->initial_state) ||
        !aligned16(p->final_state))
        return FKDA_ERR_ALIGNMENT;
    const int algo = resolve_algo(p->algo);
    if (algo != FKDA_ALGO_TWOPASS && algo != FKDA_ALGO_TC) return FKDA_ERR_BAD_ALGO;
    const size_t need = fkda_workspace_bytes_for(p);
    if (need > 0 && (p->workspace == nullptr || p->workspace_bytes < need ||
                     (reinterpret_cast<uintptr_t>(p->workspace) & 255u) != 0))
        return FKDA_ERR_WORKSPACE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
    int launches = 0;
    int rc;
    if (algo == FKDA_ALGO_TC && fkda::decode_eligible(*p) && !(p->flags & FKDA_FLAG_NO_DECODE) && p->chunk_states == nullptr)
        rc = fkda::launch_decode(*p, stream, &launches);  // one token per sequence: state read-modify-write
    else if (algo == FKDA_ALGO_TC && fkda::short_eligible(*p) && !(p->flags & FKDA_FLAG_NO_SHORT))
        rc = fkda::launch_short(*p, stream, &launches);   // at most one chunk per sequence: one fused kernel
    else if (algo == FKDA_ALGO_TC)
        rc = fkda::launch_tc(*p, stream, &launches);
    else
        rc = fkda::launch_twopass(*p, stream, &launches);
    if (rc == FKDA_OK) g_last_launches = launches;
    return rc;
}

}  // extern "C"
