// Context parallelism, the fold of a state through a shard's affine map: out = S . M + N per (piece, head), all
// [128,128] fp32 row-major (S and N as [V,K], M as [K,K]).  A shard of chunks maps the state it receives to the state it
// leaves as S_out = S_in . M + N; a rank composes the maps of the shards before its own into its initial state with a
// handful of these products (at most world_size - 1 of them, 4 MFLOP each per head), so this is a plain fp32 FMA
// kernel: fixed summation order k = 0 .. 127, no tensor cores, no library call on the context-parallel path.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/flashkda_b200.h"

namespace fkda {

constexpr int kFoldD = 128;
constexpr int kFoldRows = 32;   // rows of out per CTA

// grid (count, 128 / kFoldRows), 256 threads: thread t owns column t % 128 of 16 rows
__global__ void __launch_bounds__(256) cp_fold_kernel(const float* __restrict__ S, const float* __restrict__ M,
                                                      const float* __restrict__ N, float* __restrict__ out) {
    __shared__ float s_tile[kFoldRows][kFoldD];
    const int64_t mat = blockIdx.x;
    const int row0 = blockIdx.y * kFoldRows;
    const float* Sm = S + mat * kFoldD * kFoldD + (int64_t)row0 * kFoldD;
    const float* Mm = M + mat * kFoldD * kFoldD;
    for (int i = threadIdx.x; i < kFoldRows * kFoldD; i += 256) s_tile[i / kFoldD][i % kFoldD] = Sm[i];
    __syncthreads();
    const int col = threadIdx.x & 127, rg = threadIdx.x >> 7;   // rows rg * 16 .. rg * 16 + 15 of the tile
    float acc[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) acc[r] = 0.0f;
#pragma unroll 16   // sixteen rows of M in flight per thread: the loop is bound by their latency
    for (int k = 0; k < kFoldD; ++k) {
        const float m = __ldg(Mm + k * kFoldD + col);
#pragma unroll
        for (int r = 0; r < 16; ++r) acc[r] = __fmaf_rn(s_tile[rg * 16 + r][k], m, acc[r]);
    }
    const int64_t base = mat * kFoldD * kFoldD + (int64_t)(row0 + rg * 16) * kFoldD + col;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const float n = N != nullptr ? N[base + r * kFoldD] : 0.0f;
        out[base + r * kFoldD] = __fadd_rn(acc[r], n);
    }
}

}  // namespace fkda

extern "C" int fkda_cp_fold(const float* S, const float* M, const float* N, float* out, int64_t count, void* stream) {
    if (S == nullptr || M == nullptr || out == nullptr) return FKDA_ERR_NULL_POINTER;
    if (count < 0 || count > 0x7fffffff) return FKDA_ERR_BAD_SHAPE;
    if (out == S || out == M) return FKDA_ERR_BAD_SHAPE;   // every CTA reads whole rows of S and all of M
    if (count == 0) return FKDA_OK;
    fkda::cp_fold_kernel<<<dim3((unsigned)count, fkda::kFoldD / fkda::kFoldRows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        S, M, N, out);
    return cudaGetLastError() == cudaSuccess ? FKDA_OK : FKDA_ERR_LAUNCH;
}
