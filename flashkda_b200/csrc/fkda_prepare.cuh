// The token-parallel "prepare" kernel shared by the two-pass implementations: per (chunk, head)
// it produces the chunk operands kd, qd, kr, E_tot, INV, Mqk (and the activated beta) in an HBM
// workspace record.  Numerics: tests/torch_ref.py:153-229 of the reference; structure is this
// repository's own (one CTA per chunk, 16 lanes of 8 elements per token row).
#pragma once

#include "fkda_common.cuh"
#include "fkda_internal.h"

namespace fkda {

// ---------------------------------------------------------------------------------
// prepare: one CTA per (chunk, head), 256 threads = 16 rows x 16 lanes of 8 elements
// ---------------------------------------------------------------------------------
constexpr int kPitch = kD + 8;  // bf16 row pitch in shared memory (272 B: conflict-free 16 B reads)
constexpr int kLd16 = 24;       // fp16 row pitch of the 16x16 matrices

struct PrepSmem {
    float G[kChunk][kD];               // gate, then its in-chunk cumulative sum
    __nv_bfloat16 kd[kChunk][kPitch];  // k * 2^G
    __nv_bfloat16 qd[kChunk][kPitch];  // q * 2^G * scale
    __nv_bfloat16 ki[kChunk][kPitch];  // k * 2^-G
    float etot[kD];
    __half L[kChunk][kLd16];
    __half W[kChunk][kLd16];
    float beta_act[kChunk];
};

// kTc = false: row-major record for the CUDA-core recurrence (kWs* offsets).
// kTc = true : record whose operand tiles are already in the no-swizzle UMMA canonical layouts
//              (kTc* offsets), so the tensor-core recurrence fetches it with one bulk copy.
template <bool kTc>
__global__ void __launch_bounds__(256) prepare_kernel(TwoPassArgs a) {
    __shared__ __align__(16) PrepSmem sm;
    const int tid = threadIdx.x;
    const int h = blockIdx.y;
    const int64_t tile = blockIdx.x;

    // ---- which sequence / which chunk of it ----
    int64_t n, local_t, bos, seq_len;
    if (a.cu_seqlens != nullptr) {
        const int32_t* pre = a.tile_prefix;
        if (tile >= pre[a.N]) return;
        int64_t lo = 0, hi = a.N;  // find n with pre[n] <= tile < pre[n+1]
        while (hi - lo > 1) {
            int64_t mid = (lo + hi) >> 1;
            if (pre[mid] <= tile) lo = mid; else hi = mid;
        }
        n = lo;
        local_t = tile - pre[n];
        bos = a.cu_seqlens[n];
        seq_len = a.cu_seqlens[n + 1] - bos;
    } else {
        const int64_t tps = (a.T + kChunk - 1) / kChunk;
        n = tile / tps;
        local_t = tile - n * tps;
        bos = n * a.T;
        seq_len = a.T;
    }
    const int64_t t0 = bos + local_t * kChunk;
    const int len = (int)min((int64_t)kChunk, seq_len - local_t * kChunk);

    const int row = tid >> 4;       // token within the chunk
    const int c8 = (tid & 15) * 8;  // first of this thread's 8 columns
    const bool valid = row < len;
    const int64_t tok_off = (t0 + row) * a.token_stride + (int64_t)h * kD + c8;

    // ---- load q, k, g (8 bf16 each); rows past the sequence end are zero ----
    uint4 qraw = make_uint4(0, 0, 0, 0), kraw = qraw, graw = qraw;
    if (valid) {
        qraw = *reinterpret_cast<const uint4*>(a.q + tok_off);
        kraw = *reinterpret_cast<const uint4*>(a.k + tok_off);
        graw = *reinterpret_cast<const uint4*>(a.g + tok_off);
    }
    float qv[8], kv[8], gv[8];
    {
        const uint32_t* qp = &qraw.x; const uint32_t* kp = &kraw.x; const uint32_t* gp = &graw.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qv[2 * i] = bf_lo(qp[i]); qv[2 * i + 1] = bf_hi(qp[i]);
            kv[2 * i] = bf_lo(kp[i]); kv[2 * i + 1] = bf_hi(kp[i]);
            gv[2 * i] = bf_lo(gp[i]); gv[2 * i + 1] = bf_hi(gp[i]);
        }
    }
    // ---- q/k L2 normalisation: per-lane FMA chain, xor butterfly over the 16 lanes of the row ----
    float qs = 0.f, ks = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { qs = __fmaf_rn(qv[i], qv[i], qs); ks = __fmaf_rn(kv[i], kv[i], ks); }
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) {
        qs = __fadd_rn(qs, __shfl_xor_sync(0xffffffffu, qs, d));
        ks = __fadd_rn(ks, __shfl_xor_sync(0xffffffffu, ks, d));
    }
    const float qinv = rsqrt_approx(__fadd_rn(qs, 1e-6f));
    const float kinv = rsqrt_approx(__fadd_rn(ks, 1e-6f));
    uint32_t qn[4], kn[4];  // normalised q, k as bf16x2 pairs
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qn[i] = pack_bf2(__fmul_rn(qv[2 * i], qinv), __fmul_rn(qv[2 * i + 1], qinv));
        kn[i] = pack_bf2(__fmul_rn(kv[2 * i], kinv), __fmul_rn(kv[2 * i + 1], kinv));
    }

    // ---- gate activation: gate_scale * sigmoid(exp(A_log) * (g + dt_bias)); 0 past the end ----
    const float a_exp = ex2_approx(__fmul_rn(a.A_log[h], 1.4426950408889634f));
    {
        const float4 dt0 = *reinterpret_cast<const float4*>(a.dt_bias + (int64_t)h * kD + c8);
        const float4 dt1 = *reinterpret_cast<const float4*>(a.dt_bias + (int64_t)h * kD + c8 + 4);
        const float dt[8] = {dt0.x, dt0.y, dt0.z, dt0.w, dt1.x, dt1.y, dt1.z, dt1.w};
        float gt[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x = __fmul_rn(a_exp, __fadd_rn(gv[i], dt[i]));
            gt[i] = valid ? __fmul_rn(a.gate_scale, sigmoid_tanh(x)) : 0.0f;
        }
        *reinterpret_cast<float4*>(&sm.G[row][c8]) = make_float4(gt[0], gt[1], gt[2], gt[3]);
        *reinterpret_cast<float4*>(&sm.G[row][c8 + 4]) = make_float4(gt[4], gt[5], gt[6], gt[7]);
    }
    if (tid < kChunk) {
        float b = 0.0f;
        if (tid < len) b = bf2f(a.beta[(t0 + tid) * a.beta_token_stride + h]);
        sm.beta_act[tid] = sigmoid_tanh(b);
    }
    __syncthreads();
    // ---- in-chunk cumulative sum down the rows, one column per thread, in row order ----
    if (tid < kD) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < kChunk; ++r) { s = __fadd_rn(s, sm.G[r][tid]); sm.G[r][tid] = s; }
        sm.etot[tid] = ex2_approx(s);
    }
    __syncthreads();

    // ---- decay application; kd, qd, kr go straight to the workspace ----
    const int64_t rec = ((int64_t)h * a.total_tiles + tile) * (int64_t)(kTc ? kTcRecord : kWsRecord);
    uint8_t* ws = a.workspace + rec;
    {
        const uint32_t sc2 = pack_bf2(a.scale, a.scale);
        const float4 g0 = *reinterpret_cast<const float4*>(&sm.G[row][c8]);
        const float4 g1 = *reinterpret_cast<const float4*>(&sm.G[row][c8 + 4]);
        const float4 t0v = *reinterpret_cast<const float4*>(&sm.etot[c8]);
        const float4 t1v = *reinterpret_cast<const float4*>(&sm.etot[c8 + 4]);
        const float G[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float Et[8] = {t0v.x, t0v.y, t0v.z, t0v.w, t1v.x, t1v.y, t1v.z, t1v.w};
        uint32_t kd_p[4], qd_p[4], ki_p[4], kr_p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // bf16x2 arithmetic: one rounding per element and operation
            const uint32_t ep = pack_bf2(ex2_approx(G[2 * i]), ex2_approx(G[2 * i + 1]));
            const uint32_t em = pack_bf2(ex2_approx(-G[2 * i]), ex2_approx(-G[2 * i + 1]));
            const uint32_t et = pack_bf2(Et[2 * i], Et[2 * i + 1]);
            kd_p[i] = bf2_mul(kn[i], ep);
            qd_p[i] = bf2_mul(bf2_mul(qn[i], ep), sc2);
            ki_p[i] = bf2_mul(kn[i], em);
            kr_p[i] = bf2_mul(ki_p[i], et);
        }
        const uint4 kd4 = make_uint4(kd_p[0], kd_p[1], kd_p[2], kd_p[3]);
        const uint4 qd4 = make_uint4(qd_p[0], qd_p[1], qd_p[2], qd_p[3]);
        const uint4 ki4 = make_uint4(ki_p[0], ki_p[1], ki_p[2], ki_p[3]);
        const uint4 kr4 = make_uint4(kr_p[0], kr_p[1], kr_p[2], kr_p[3]);
        *reinterpret_cast<uint4*>(&sm.kd[row][c8]) = kd4;
        *reinterpret_cast<uint4*>(&sm.qd[row][c8]) = qd4;
        *reinterpret_cast<uint4*>(&sm.ki[row][c8]) = ki4;
        if constexpr (kTc) {
            const int kc = c8 >> 3;
            *reinterpret_cast<uint4*>(ws + kTcB1 + tc_b1_off(row, kc)) = kd4;
            *reinterpret_cast<uint4*>(ws + kTcB1 + tc_b1_off(kChunk + row, kc)) = qd4;
            *reinterpret_cast<uint4*>(ws + kTcKr + tc_kr_off(row, kc)) = kr4;
        } else {
            const int eoff = (row * kD + c8) * 2;
            *reinterpret_cast<uint4*>(ws + kWsKd + eoff) = kd4;
            *reinterpret_cast<uint4*>(ws + kWsQd + eoff) = qd4;
            *reinterpret_cast<uint4*>(ws + kWsKr + eoff) = kr4;
        }
    }
    if (tid < kD) reinterpret_cast<float*>(ws + (kTc ? kTcEt : kWsEt))[tid] = sm.etot[tid];
    if (kTc && tid < kChunk) reinterpret_cast<float*>(ws + kTcBeta)[tid] = bf2f(f2bf(sm.beta_act[tid]));
    __syncthreads();

    // ---- L = fp16(kd ki^T) masked * fp16(beta) (warp 0), Mqk = bf16(qd ki^T) masked (warp 1):
    //      mma.sync m16n8k16 bf16 -> fp32, operand fragments fetched with conflict-free 32-bit loads ----
    if (tid < 64) {
        const int w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
        const __nv_bfloat16(*A)[kPitch] = (w == 0) ? sm.kd : sm.qd;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < kD / 16; ++j) {
            const int col = 16 * j + 2 * t;
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&A[g][col]);
            const uint32_t a1 = *reinterpret_cast<const uint32_t*>(&A[g + 8][col]);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&A[g][col + 8]);
            const uint32_t a3 = *reinterpret_cast<const uint32_t*>(&A[g + 8][col + 8]);
            const uint32_t b00 = *reinterpret_cast<const uint32_t*>(&sm.ki[g][col]);
            const uint32_t b01 = *reinterpret_cast<const uint32_t*>(&sm.ki[g][col + 8]);
            const uint32_t b10 = *reinterpret_cast<const uint32_t*>(&sm.ki[g + 8][col]);
            const uint32_t b11 = *reinterpret_cast<const uint32_t*>(&sm.ki[g + 8][col + 8]);
            mma_bf16_f32acc(c0, a0, a1, a2, a3, b00, b01);  // columns 0-7
            mma_bf16_f32acc(c1, a0, a1, a2, a3, b10, b11);  // columns 8-15
        }
        // fragment element e of n-tile nt: row = g + 8*(e>>1), column = 8*nt + 2*t + (e&1)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int i = g + 8 * hr, j = 8 * nt + 2 * t;
                const float x0 = nt ? c1[2 * hr] : c0[2 * hr], x1 = nt ? c1[2 * hr + 1] : c0[2 * hr + 1];
                if (w == 0) {
                    const __half bh = __float2half_rn(sm.beta_act[i]);
                    const __half l0 = (i > j) ? __hmul(__float2half_rn(x0), bh) : __float2half_rn(0.0f);
                    const __half l1 = (i > j + 1) ? __hmul(__float2half_rn(x1), bh) : __float2half_rn(0.0f);
                    *reinterpret_cast<__half2*>(&sm.L[i][j]) = __halves2half2(l0, l1);
                } else {
                    const uint32_t m = pack_bf2((i >= j) ? x0 : 0.0f, (i >= j + 1) ? x1 : 0.0f);
                    if constexpr (kTc)
                        *reinterpret_cast<uint32_t*>(ws + kTcMqk + tc_sq_off(i, j)) = m;
                    else
                        *reinterpret_cast<uint32_t*>(ws + kWsMqk + (i * kChunk + j) * 2) = m;
                }
            }
        }
    }
    __syncwarp();
    if (tid < 32)
        neumann_inverse_warp<kTc>(&sm.L[0][0], &sm.W[0][0], kLd16, ws + (kTc ? kTcInv : kWsInv), tid);
}


}  // namespace fkda
