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
    uint8_t* workspace;    // [H][total_tiles] records of kWsRecord bytes
    int64_t T, H, N, total_tiles;
    int64_t token_stride, beta_token_stride;
    float scale, gate_scale;
    bool state_fp32;
};

size_t twopass_workspace_bytes(int64_t T_total, int64_t H, int64_t N);
int launch_twopass(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches);

}  // namespace fkda
