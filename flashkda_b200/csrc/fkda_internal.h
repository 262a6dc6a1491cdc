// Internal host/device declarations shared by the translation units of the library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/flashkda_b200.h"

namespace fkda {

// Kernel arguments of the two-pass implementation (passed by value).
struct TwoPassArgs {
    const __nv_bfloat16 *q, *k, *v, *g, *beta;
    __nv_bfloat16* out;
    const float *A_log, *dt_bias;
    const void* initial_state;
    void* final_state;
    const int64_t* cu_seqlens;
    int32_t* tile_prefix;  // [N + 1] chunk-count prefix (varlen only)
    const int32_t* seq_order;  // [N] sequences by decreasing length (varlen with N <= kSeqOrderMaxN, else nullptr)
    uint8_t* workspace;    // [H][total_tiles] per-chunk records
    int32_t* queue;        // header word 0: tail / queue ticket counter of the persistent recurrence (zeroed per call)
    int32_t* status;       // header word 1: device status, 0 ok, else the code of a bounded wait that gave up
    int32_t* short_flag;   // header word 8, or null: written by the prefix kernel of a ragged batch that MAY consist of
                           // one-chunk sequences; the kernels that can serve the call are all enqueued and all but one
                           // return at once: 2 = every sequence has exactly one token (decode kernel), 1 = no sequence is
                           // longer than one chunk (fused short-sequence kernel), 0 = the general kernels
                           // (header words 2, 3: push counter and finished-chain counter of the segment queue;
                           //  words 4..6: claim counters of the three layers of first segments)
    int32_t* qslots;       // segment queue: slot i receives the i-th pushed item (-1 = not yet pushed)
    uint32_t* seg_state;   // [chain][16][128] uint4: bf16 state handed from one segment of a chain to the next
    int32_t seg_chunks;    // chunks per scheduling segment (0 = whole chains)
    int32_t slab_c0, slab_chunks;  // fixed batches only: this launch covers chunks [slab_c0, slab_c0 + slab_chunks) of
                                   // every sequence (slab_chunks == 0: all chunks); a chain's state travels from one
                                   // slab to the next through seg_state
    int64_t T, H, N, total_tiles;
    int64_t token_stride, beta_token_stride;
    float scale, gate_scale;
    __nv_bfloat16* chunk_states;   // optional export of the state before every cs_every-th chunk (see fkda_fwd_params)
    const int32_t* cs_prefix;      // [N] first export slot of every sequence (varlen; fixed batches compute it)
    int32_t cs_every;
    uint64_t wait_ns;      // limit of every bounded device-side wait (mbarrier, queue slot)
    bool state_fp32;
    bool test_drop_push;   // test hook (FKDA_FLAG_TEST_DROP_PUSH): finished segments do not queue their follow-up
};

// Workspace layout of both two-pass implementations:
//   [0, 256)  header: int32 ticket counter, device status, push counter, finished-chain counter, 3 layer counters
//   [256, ..) tile prefix (N + 1 int32, padded to 256 B)
//   then      H * total_tiles records
constexpr size_t kWsHeaderBytes = 256;
// (N + 1) chunk-prefix entries, N entries of the length order, N + 1 entries of the state-export prefix
inline size_t ws_prefix_bytes(int64_t N) { return (size_t)(((3 * N + 2) * 4 + 255) / 256 * 256); }
constexpr int64_t kSeqOrderMaxN = 512;  // beyond this the quadratic ranking in the prefix kernel is not worth its time
inline int64_t ws_tiles_upper_bound(int64_t T_total, int64_t N) { return (T_total + 15) / 16 + N; }

size_t twopass_workspace_bytes(int64_t T_total, int64_t H, int64_t N);
int launch_twopass(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches);
size_t tc_workspace_bytes(int64_t T_total, int64_t H, int64_t N);   // upper bound for these totals
size_t tc_workspace_bytes_for(const fkda_fwd_params& p);            // what this particular call needs
int device_sm_count();
// Device address of the built-in scratch of fkda_fwd_noalloc on the current device, or nullptr before that
// entry point's first call there.
void* noalloc_scratch_or_null();
int launch_tc(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches);
// Decode step (fixed batch, T == 1): one read-modify-write kernel over the states, no workspace records.
bool decode_eligible(const fkda_fwd_params& p);
int launch_decode(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches);
// Short sequences (fixed batch, 2 <= T <= 16): one fused kernel per (sequence, head), no workspace records.
bool short_eligible(const fkda_fwd_params& p);
int launch_short(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches);
// Ragged batches: whether the call MAY consist of sequences of at most one chunk each (the host knows only the totals;
// the prefix kernel decides on the device), and the launch of the fused kernel behind that decision.
bool short_ragged_candidate(const fkda_fwd_params& p);
int launch_short_ragged(const TwoPassArgs& a, cudaStream_t stream);
int launch_decode_ragged(const TwoPassArgs& a, cudaStream_t stream);   // as many tokens as sequences: maybe one each

// Fills the kernel arguments common to both implementations (pointers, strides, gate scale,
// workspace carving).
void fill_args(const fkda_fwd_params& p, TwoPassArgs* a);
void launch_tile_prefix(const int64_t* cu_seqlens, int64_t N, int32_t* prefix, int32_t* seq_order, int32_t* cs_prefix,
                        int cs_tokens, int32_t* short_flag, bool decode_enqueued, int32_t* critical_chunks, int64_t heads,
                        int chain_slots, cudaStream_t stream);
// First state-export slot of sequence n.
__device__ __forceinline__ int64_t cs_first_slot(const TwoPassArgs& a, int64_t n) {
    if (a.cu_seqlens != nullptr) return a.cs_prefix[n];
    const int64_t group = 16 * (int64_t)a.cs_every;
    return n * ((a.T + group - 1) / group);
}

}  // namespace fkda
