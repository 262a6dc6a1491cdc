// Short sequences: a fixed batch whose sequences hold 2 .. 16 tokens each, or a ragged batch in which no sequence
// holds more than 16 (ONE chunk per sequence), the step between a decode step (one token, fkda_decode.cu) and
// prefill -- e.g. the verification pass of speculative decoding.  Such a batch is bound by HBM traffic on the [128,128] states (read once, written once), so the whole
// forward of a (sequence, head) chain runs in ONE kernel with nothing staged in HBM: no chunk records, no second
// launch, 256 bytes of workspace.
//
// One 128-thread CTA per FOUR chains, three CTAs per SM:
//   * first every warp runs the prepare stage of one of the four chunks (the same warp-per-chunk routine as the
//     prefill path), record left in shared memory: the prepare stage is a long serial instruction stream, so four
//     of them run side by side instead of three warps waiting for one;
//   * after one block barrier the four chains are walked one after the other by all four warps: every warp brings
//     its 32 state rows into mma.sync A-fragment registers (thread g = lane / 4, tq = lane % 4 of warp w holds rows
//     32 w + 16 mt + {g, g + 8}, columns 16 j + {2tq, 2tq+1, 2tq+8, 2tq+9} for the row tiles mt = 0, 1 and the K steps
//     j = 0 .. 7): whole rows from global memory (512 contiguous bytes per warp instruction) into a 4 KB staging tile
//     per warp, from there with ldmatrix; then it runs the chunk step on mma.sync, state in registers throughout:
//       D1[V,32] = S . [kd; qd]^T   (8 K steps in order: the reference's accumulation order)
//       u' = (v (-) bf(u0)) (*) bf(beta),  U = bf(u' INV^T),  out = bf(o0) (+) bf(U Mqk^T)
//       DST[V,K] = U^T . kr,  S[v,k] = bf(fma(S[v,k], E_tot[k], DST[v,k]))  (accumulator and A fragments of a
//       16 x 16 block hold the same elements, so the update runs fragment on fragment)
//     and the refreshed rows leave the same way, fragments into the staging tile, whole rows out.
// Numerics and results: those of the chunked kernels on the same inputs (tests/torch_ref.py:153-251 of the
// reference; the reference itself runs such batches through its two general kernels,
// csrc/smxx/fwd_kernel1.cuh / fwd_kernel2.cuh).
#include "fkda_common.cuh"
#include "fkda_internal.h"
#include "fkda_prepare_warp.cuh"

namespace fkda {

// B operand fragments of mma.sync m16n8k16 for n-tile rows r = 8 nt + g of a K-major [rows, K] tile in the record's
// B1 layout (byte = (k/8)*528 + (r/8)*128 + (r%8)*16 + (k%8)*2): b0 = (k 16j + 2tq, +1), b1 = (k 16j + 8 + 2tq, +1)
__device__ __forceinline__ void short_b1_frag(const uint8_t* b1, int r, int j, int tq, uint32_t& b0, uint32_t& b1r) {
    const uint8_t* p = b1 + (2 * j) * kTcB1Lbo + (r >> 3) * 128 + (r & 7) * 16 + tq * 4;
    b0 = *reinterpret_cast<const uint32_t*>(p);
    b1r = *reinterpret_cast<const uint32_t*>(p + kTcB1Lbo);
}
// Four 8x8 b16 matrices, transposed on the way: lane 8m + r gives the address of row r (16 bytes) of matrix m; thread
// (g, tq) receives elements (rows 2tq, 2tq+1; column g) of each, i.e. mma.sync B fragments of row-major [K, N] tiles.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* row_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

constexpr int kShortChainsPerCta = 4;
// Per warp, a staging tile of 16 state rows as bf16 (256 bytes a row): the states travel between global memory and the
// fragment registers through it, so that global memory sees whole rows (512 contiguous bytes per warp instruction)
// instead of 4-byte pieces.  The 16-byte piece c of row r sits at r * 256 + ((c ^ (r & 7)) * 16): rows 8 apart in
// banks, so the 8-row reads of ldmatrix and the fragment stores do not collide.
constexpr int kShortStageBytes = 16 * 256;
constexpr int kShortSmemBytes = kShortChainsPerCta * kTcRecord + 4 * kShortStageBytes + 16;
__device__ __forceinline__ int short_stage_off(int r, int piece) { return r * 256 + ((piece ^ (r & 7)) << 4); }

__global__ void __launch_bounds__(128, 3) short_kernel(const __grid_constant__ TwoPassArgs a) {
    extern __shared__ uint8_t short_smem[];
    uint8_t* recs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(short_smem) + 15) & ~(uintptr_t)15);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    // a ragged batch that the prefix kernel has given to other kernels (a longer sequence: the general ones; one token
    // each: the decode kernel)
    if (a.short_flag != nullptr && *a.short_flag != 1) return;
    const int64_t n_chains = a.N * a.H;
    const int64_t chain0 = (int64_t)blockIdx.x * kShortChainsPerCta;
    const int row0 = warp * 32 + g;           // my rows: row0 + 16 mt + 8 hi
    uint8_t* stage = recs + kShortChainsPerCta * kTcRecord + warp * kShortStageBytes;   // my warp's staging tile
    // The state of the chain that comes next is asked into L2 one chain ahead (the first before the prepare stage), so
    // that its loads find it there: one chain ahead only, more than that competes with the loads that are needed now.
    auto prefetch_state = [&](int64_t chain) {
        if (a.initial_state == nullptr || chain >= n_chains) return;
        const int64_t bytes = (int64_t)kD * kD * (a.state_fp32 ? 4 : 2);
        const char* base = reinterpret_cast<const char*>(a.initial_state) + chain * bytes;
        for (int64_t off = (int64_t)threadIdx.x * 128; off < bytes; off += 128 * 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
    };
    prefetch_state(chain0);
    // first token and length (0 .. 16 tokens: at most one chunk) of sequence n
    auto locate = [&](int64_t n, int64_t* t0, int* len) {
        if (a.cu_seqlens != nullptr) {
            const int64_t b = a.cu_seqlens[n], e = a.cu_seqlens[n + 1];
            *t0 = b;
            *len = e > b ? (int)(e - b) : 0;
        } else {
            *t0 = n * a.T;
            *len = (int)a.T;
        }
    };

    // ---- the operands of the four chunks: warp w runs the prepare stage of chain chain0 + w, record left in
    //      shared memory (layout of fkda_common.cuh) ----
    if (chain0 + warp < n_chains) {
        const int64_t n = (chain0 + warp) / a.H;
        const int h = (int)(chain0 + warp - n * a.H);
        uint8_t* rec = recs + warp * kTcRecord;
        int64_t t0;
        int len;
        locate(n, &t0, &len);
        if (len > 0) {
            PrepPrefetch pf;
            prep_prefetch(a, t0, len, h, lane, pf);
            prepare_chunk_warp<true, true>(a, t0, len, h, rec, *reinterpret_cast<PrepWarpSmem*>(rec), lane, pf, false, 0, 0, 0);
        }
    }
    __syncthreads();   // the four records are complete

#pragma unroll 1
    for (int ci = 0; ci < kShortChainsPerCta; ++ci) {
    const int64_t chain = chain0 + ci;
    if (chain >= n_chains) break;
    const int64_t n = chain / a.H;
    const int h = (int)(chain - n * a.H);
    int64_t t0;
    int len;
    locate(n, &t0, &len);
    const uint8_t* rec = recs + ci * kTcRecord;
    if (ci + 1 < kShortChainsPerCta) prefetch_state(chain + 1);

    // ---- state rows into A-fragment registers: sreg[mt][j][e], e = {row g: cols 2tq | row g+8 | row g: cols 2tq+8 | row g+8},
    //      16 rows (one row tile mt) at a time through the warp's staging tile ----
    uint32_t sreg[2][8][4];
    const int64_t st_chain = chain * (int64_t)(kD * kD);
    if (a.initial_state != nullptr) {
        if (a.state_fp32) {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                // 16 rows x 512 bytes: piece p = 32 i + lane is 4 floats, row p / 32, columns 4 (p % 32) ..
                const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.initial_state) + st_chain +
                                                                    (int64_t)(warp * 32 + 16 * mt) * kD);
                float4 x[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) x[i] = __ldg(src + 32 * i + lane);
#pragma unroll
                for (int i = 0; i < 16; ++i)   // row i, columns 4 lane .. 4 lane + 3: half (lane & 1) of piece lane / 2
                    *reinterpret_cast<uint2*>(stage + short_stage_off(i, lane >> 1) + 8 * (lane & 1)) =
                        make_uint2(pack_bf2(x[i].x, x[i].y), pack_bf2(x[i].z, x[i].w));
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    ldmatrix_x4(sreg[mt][j][0], sreg[mt][j][1], sreg[mt][j][2], sreg[mt][j][3],
                                stage + short_stage_off((lane & 7) + 8 * ((lane >> 3) & 1), 2 * j + (lane >> 4)));
                __syncwarp();
            }
        } else {
            // 32 rows x 256 bytes: piece p = 32 i + lane is 8 bf16, row p / 16, columns 8 (p % 16) ..; both row tiles are
            // fetched before the first is staged
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(a.initial_state) + st_chain +
                                                              (int64_t)(warp * 32) * kD);
            uint4 x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = __ldg(src + 32 * i + lane);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                for (int i = 0; i < 8; ++i)   // row 2 i + lane / 16 of the tile, piece lane % 16
                    *reinterpret_cast<uint4*>(stage + short_stage_off(2 * i + (lane >> 4), lane & 15)) = x[8 * mt + i];
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    ldmatrix_x4(sreg[mt][j][0], sreg[mt][j][1], sreg[mt][j][2], sreg[mt][j][3],
                                stage + short_stage_off((lane & 7) + 8 * ((lane >> 3) & 1), 2 * j + (lane >> 4)));
                __syncwarp();
            }
        }
    } else {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sreg[mt][j][e] = 0u;
    }
    // A row tile of the refreshed state leaves through the staging tile: fragments in, whole rows out.
    auto stage_frag = [&](int j, const uint32_t (&y)[4]) {   // fragment j of the tile: (row g | g+8) x (piece 2j | 2j+1)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            *reinterpret_cast<uint32_t*>(stage + short_stage_off(g + 8 * (e & 1), 2 * j + (e >> 1)) + 4 * tq) = y[e];
    };
    auto flush_tile = [&](int mt) {
        __syncwarp();
        if (a.state_fp32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.final_state) + st_chain + (int64_t)(warp * 32 + 16 * mt) * kD);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint2 y = *reinterpret_cast<const uint2*>(stage + short_stage_off(i, lane >> 1) + 8 * (lane & 1));
                dst[32 * i + lane] = make_float4(bf_lo(y.x), bf_hi(y.x), bf_lo(y.y), bf_hi(y.y));
            }
        } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.final_state) + st_chain + (int64_t)(warp * 32 + 16 * mt) * kD);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                dst[32 * i + lane] = *reinterpret_cast<const uint4*>(stage + short_stage_off(2 * i + (lane >> 4), lane & 15));
        }
        __syncwarp();
    };
    if (len == 0) {   // an empty sequence of a ragged batch: its state passes through (rounded to bf16, as everywhere)
        if (a.final_state != nullptr) {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                for (int j = 0; j < 8; ++j) stage_frag(j, sreg[mt][j]);
                flush_tile(mt);
            }
        }
        continue;
    }
    // value tile in A-fragment layout (zero past the sequence end), straight from global memory
    uint32_t vfr[2][4];
    {
        const unsigned short* vp = reinterpret_cast<const unsigned short*>(a.v) + t0 * a.token_stride + (int64_t)h * kD;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = row0 + 16 * mt + 8 * (e & 1), tok = 2 * tq + 8 * (e >> 1);
                const uint32_t lo = tok < len ? vp[(int64_t)tok * a.token_stride + row] : 0u;
                const uint32_t hi = tok + 1 < len ? vp[(int64_t)(tok + 1) * a.token_stride + row] : 0u;
                vfr[mt][e] = lo | (hi << 16);
            }
        }
    }

    // ---- D1[V,32] = S . [kd; qd]^T: rows 0-15 of B1 are kd (-> u0), rows 16-31 qd (-> o0) ----
    float d1[2][4][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) d1[mt][nt][i] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            uint32_t b0, b1;
            short_b1_frag(rec + kTcB1, 8 * nt + g, j, tq, b0, b1);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
                mma_bf16_f32acc(d1[mt][nt], sreg[mt][j][0], sreg[mt][j][1], sreg[mt][j][2], sreg[mt][j][3], b0, b1);
        }
    }
    // ---- u' = (v (-) bf(u0)) (*) bf(beta);  U = bf(u' INV^T);  out = bf(o0) (+) bf(U Mqk^T) ----
    const uint32_t* beta32 = reinterpret_cast<const uint32_t*>(rec + kTcBeta);
    const uint32_t bp0 = beta32[tq], bp1 = beta32[tq + 4];
    uint32_t invb[2][2], mqkb[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
        invb[nt][0] = *reinterpret_cast<const uint32_t*>(rec + kTcInv + tc_sq_off(8 * nt + g, 2 * tq));
        invb[nt][1] = *reinterpret_cast<const uint32_t*>(rec + kTcInv + tc_sq_off(8 * nt + g, 2 * tq + 8));
        mqkb[nt][0] = *reinterpret_cast<const uint32_t*>(rec + kTcMqk + tc_sq_off(8 * nt + g, 2 * tq));
        mqkb[nt][1] = *reinterpret_cast<const uint32_t*>(rec + kTcMqk + tc_sq_off(8 * nt + g, 2 * tq + 8));
    }
    uint32_t ufr[2][4];
    unsigned short* og = reinterpret_cast<unsigned short*>(a.out) + t0 * a.token_stride + (int64_t)h * kD;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        uint32_t up[4];   // accumulator tiles nt = 0, 1 of D1 are u0 for tokens 0-7, 8-15: {c0,c1 | c2,c3} = {row g | row g+8}
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t u0 = pack_bf2(d1[mt][e >> 1][2 * (e & 1)], d1[mt][e >> 1][2 * (e & 1) + 1]);
            up[e] = bf2_mul(bf2_sub(vfr[mt][e], u0), (e >> 1) ? bp1 : bp0);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            mma_bf16_f32acc(c, up[0], up[1], up[2], up[3], invb[nt][0], invb[nt][1]);
            ufr[mt][2 * nt] = pack_bf2(c[0], c[1]);
            ufr[mt][2 * nt + 1] = pack_bf2(c[2], c[3]);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            mma_bf16_f32acc(c, ufr[mt][0], ufr[mt][1], ufr[mt][2], ufr[mt][3], mqkb[nt][0], mqkb[nt][1]);
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                const uint32_t o = bf2_add(pack_bf2(d1[mt][2 + nt][2 * hi], d1[mt][2 + nt][2 * hi + 1]), pack_bf2(c[2 * hi], c[2 * hi + 1]));
                const int row = row0 + 16 * mt + 8 * hi, tok = 8 * nt + 2 * tq;
                if (tok < len) og[(int64_t)tok * a.token_stride + row] = (unsigned short)(o & 0xffffu);
                if (tok + 1 < len) og[(int64_t)(tok + 1) * a.token_stride + row] = (unsigned short)(o >> 16);
            }
        }
    }
    if (a.final_state == nullptr) continue;

    // ---- DST[V,K] = U^T . kr and S[v,k] = bf(fma(S[v,k], E_tot[k], DST[v,k])), 16 state columns (K step j) at a time;
    //      the refreshed fragments go straight to the final state ----
    const float* et = reinterpret_cast<const float*>(rec + kTcEt);
    // KR tile: kr[token i][column k] at (i/8)*2304 + (k/8)*144 + (i%8)*16 + (k%8)*2: 8x8 blocks with tokens as rows.
    // ldmatrix lane 8m + r: matrix m = (token group m & 1, column block 2j + (m >> 1)), row r = token
    const uint8_t* kr_row = rec + kTcKr + ((lane >> 3) & 1) * kTcKrLbo + (lane >> 4) * kTcKrSbo + (lane & 7) * 16;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t b00, b01, b10, b11;   // column block 2j: tokens 0-7, 8-15; column block 2j+1: tokens 0-7, 8-15
            ldmatrix_x4_trans(b00, b01, b10, b11, kr_row + (2 * j) * kTcKrSbo);
            const float2 e0 = *reinterpret_cast<const float2*>(et + 16 * j + 2 * tq);        // E_tot of columns 16j + 2tq, +1
            const float2 e1 = *reinterpret_cast<const float2*>(et + 16 * j + 8 + 2 * tq);    // 16j + 8 + 2tq, +1
            float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
            mma_bf16_f32acc(c0, ufr[mt][0], ufr[mt][1], ufr[mt][2], ufr[mt][3], b00, b01);   // columns 16j + 0..7
            mma_bf16_f32acc(c1, ufr[mt][0], ufr[mt][1], ufr[mt][2], ufr[mt][3], b10, b11);   // columns 16j + 8..15
            const uint32_t s0 = sreg[mt][j][0], s1 = sreg[mt][j][1], s2 = sreg[mt][j][2], s3 = sreg[mt][j][3];
            const uint32_t y[4] = {
                pack_bf2(__fmaf_rn(bf_lo(s0), e0.x, c0[0]), __fmaf_rn(bf_hi(s0), e0.y, c0[1])),    // row g
                pack_bf2(__fmaf_rn(bf_lo(s1), e0.x, c0[2]), __fmaf_rn(bf_hi(s1), e0.y, c0[3])),    // row g+8
                pack_bf2(__fmaf_rn(bf_lo(s2), e1.x, c1[0]), __fmaf_rn(bf_hi(s2), e1.y, c1[1])),
                pack_bf2(__fmaf_rn(bf_lo(s3), e1.x, c1[2]), __fmaf_rn(bf_hi(s3), e1.y, c1[3]))};
            stage_frag(j, y);
        }
        flush_tile(mt);
    }
    }   // chains of this CTA
}

bool short_eligible(const fkda_fwd_params& p) {
    return p.cu_seqlens == nullptr && p.T >= 2 && p.T <= kChunk && p.chunk_states == nullptr &&
           (p.phase_mask == 0 || p.phase_mask == (FKDA_PHASE_PREPARE | FKDA_PHASE_RECURRENCE));
}

bool short_ragged_candidate(const fkda_fwd_params& p) {
    // tokens <= 16 per sequence on average is necessary for "no sequence longer than a chunk"; a handful of chains is
    // not worth two extra launches
    return p.cu_seqlens != nullptr && p.N > 0 && p.B * p.T <= kChunk * p.N && p.N * p.H >= 64 &&
           p.chunk_states == nullptr && (p.phase_mask == 0 || p.phase_mask == (FKDA_PHASE_PREPARE | FKDA_PHASE_RECURRENCE));
}

int launch_short_ragged(const TwoPassArgs& a, cudaStream_t stream) {
    const int64_t chains = a.N * a.H;
    if (chains > 0x7fffffff) return FKDA_ERR_BAD_SHAPE;
    if (cudaFuncSetAttribute(short_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kShortSmemBytes) != cudaSuccess)
        return FKDA_ERR_LAUNCH;
    const int64_t ctas = (chains + kShortChainsPerCta - 1) / kShortChainsPerCta;
    short_kernel<<<(unsigned)ctas, 128, kShortSmemBytes, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? FKDA_OK : FKDA_ERR_LAUNCH;
}

int launch_short(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches) {
    TwoPassArgs a;
    fill_args(p, &a);
    if (cudaMemsetAsync(p.workspace, 0, 16, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;  // header: device status
    const int64_t chains = p.N * p.H;
    if (chains > 0x7fffffff) return FKDA_ERR_BAD_SHAPE;
    if (cudaFuncSetAttribute(short_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kShortSmemBytes) != cudaSuccess)
        return FKDA_ERR_LAUNCH;
    const int64_t ctas = (chains + kShortChainsPerCta - 1) / kShortChainsPerCta;
    short_kernel<<<(unsigned)ctas, 128, kShortSmemBytes, stream>>>(a);
    if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
    *n_launches = 1;
    return FKDA_OK;
}

}  // namespace fkda
