// Decode step: every sequence of the batch has exactly ONE token (fixed batch, T == 1).
//
// With a single valid row the chunk algebra of the forward collapses (the in-chunk triangular system is
// the identity, Mqk is one number), and the step is a read-modify-write of the [128,128] state per
// (sequence, head): it is bound by HBM traffic on the states (2 x 32 KB in bf16, 2 x 64 KB in fp32),
// not by the tensor cores.  One 128-thread CTA per (sequence, head); warp w owns state rows 32w..32w+31,
// lane l columns 4l..4l+3 of each, so every state row is read and written once as one coalesced
// 256-byte (bf16) or 512-byte (fp32) warp access, and stays in registers in between.
//
// Numerics: the same rounding steps as the chunked kernels on a chunk with one valid row
// (tests/torch_ref.py:153-251 of the reference): bf16 after every element-wise operation, fp32
// accumulation in the dot products, tanh.approx / ex2.approx / rsqrt.approx, state rounded to bf16.
#include "fkda_common.cuh"
#include "fkda_internal.h"
#include "fkda_prepare_warp.cuh"

namespace fkda {

// x[i] holds this lane's partial sum of row i (32 rows).  Returns the warp total of row `lane`:
// at each halving step a lane keeps the half of the rows whose index bit matches its lane bit and
// hands the other half to its partner (31 shuffles instead of 32 x 5).
__device__ __forceinline__ float warp_rows_reduce(float (&x)[32], int lane) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float send = up ? x[i] : x[i + off];
            const float keep = up ? x[i + off] : x[i];
            x[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, off));
        }
    }
    return x[0];
}

__global__ void __launch_bounds__(128, 3) decode_kernel(const __grid_constant__ TwoPassArgs a) {
    // a ragged batch with as many tokens as sequences: mine only if the prefix kernel found one token in each (then
    // sequence n is token n, as in a fixed batch)
    if (a.short_flag != nullptr && *a.short_flag != 2) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t chain = blockIdx.x;
    const int64_t n = chain / a.H;          // sequence = token index (T == 1)
    const int h = (int)(chain - n * a.H);
    const int c4 = lane * 4;                // my 4 columns
    const int row0 = warp * 32;             // my warp's 32 state rows

    // ---- the token's q, k, g columns, beta, and my row's v ----
    const int64_t tok = n * a.token_stride + (int64_t)h * kD;
    const uint2 qraw = __ldg(reinterpret_cast<const uint2*>(a.q + tok + c4));
    const uint2 kraw = __ldg(reinterpret_cast<const uint2*>(a.k + tok + c4));
    const uint2 graw = __ldg(reinterpret_cast<const uint2*>(a.g + tok + c4));
    const __nv_bfloat16 v_mine = a.v[tok + row0 + lane];
    const float beta_logit = bf2f(a.beta[n * a.beta_token_stride + h]);
    const float4 dtv = *reinterpret_cast<const float4*>(a.dt_bias + (int64_t)h * kD + c4);
    const float a_exp = ex2_approx(__fmul_rn(a.A_log[h], 1.4426950408889634f));

    // ---- state rows into registers (bf16 pairs; an fp32 state is rounded on load) ----
    const int64_t st_base = (chain * kD + row0) * (int64_t)kD + c4;  // + r * kD
    uint32_t sreg[64];
    if (a.initial_state != nullptr) {
        if (a.state_fp32) {
            const float* src = reinterpret_cast<const float*>(a.initial_state) + st_base;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const float4 x = *reinterpret_cast<const float4*>(src + r * kD);
                sreg[2 * r] = pack_bf2(x.x, x.y);
                sreg[2 * r + 1] = pack_bf2(x.z, x.w);
            }
        } else {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.initial_state) + st_base;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const uint2 x = *reinterpret_cast<const uint2*>(src + r * kD);
                sreg[2 * r] = x.x;
                sreg[2 * r + 1] = x.y;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) sreg[i] = 0u;
    }

    // ---- chunk operands of a one-row chunk (every warp computes them for its lanes' columns) ----
    const float qv[4] = {bf_lo(qraw.x), bf_hi(qraw.x), bf_lo(qraw.y), bf_hi(qraw.y)};
    const float kv[4] = {bf_lo(kraw.x), bf_hi(kraw.x), bf_lo(kraw.y), bf_hi(kraw.y)};
    const float gv[4] = {bf_lo(graw.x), bf_hi(graw.x), bf_lo(graw.y), bf_hi(graw.y)};
    const float dt[4] = {dtv.x, dtv.y, dtv.z, dtv.w};
    const float qinv = rsqrt_approx(__fadd_rn(row_sumsq(qv, lane), 1e-6f));
    const float kinv = rsqrt_approx(__fadd_rn(row_sumsq(kv, lane), 1e-6f));
    const uint32_t qn0 = pack_bf2(__fmul_rn(qv[0], qinv), __fmul_rn(qv[1], qinv));
    const uint32_t qn1 = pack_bf2(__fmul_rn(qv[2], qinv), __fmul_rn(qv[3], qinv));
    const uint32_t kn0 = pack_bf2(__fmul_rn(kv[0], kinv), __fmul_rn(kv[1], kinv));
    const uint32_t kn1 = pack_bf2(__fmul_rn(kv[2], kinv), __fmul_rn(kv[3], kinv));
    float gsum[4], et[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float x = __fmul_rn(a_exp, __fadd_rn(gv[i], dt[i]));
        gsum[i] = __fadd_rn(0.0f, __fmul_rn(a.gate_scale, sigmoid_tanh(x)));  // in-chunk cumulative gate, one row
        et[i] = ex2_approx(gsum[i]);                                            // fp32 decay of the state
    }
    const uint32_t sc2 = pack_bf2(a.scale, a.scale);
    const uint32_t ep0 = pack_bf2(et[0], et[1]), ep1 = pack_bf2(et[2], et[3]);
    const uint32_t em0 = pack_bf2(ex2_approx(-gsum[0]), ex2_approx(-gsum[1]));
    const uint32_t em1 = pack_bf2(ex2_approx(-gsum[2]), ex2_approx(-gsum[3]));
    const uint32_t kd0 = bf2_mul(kn0, ep0), kd1 = bf2_mul(kn1, ep1);
    const uint32_t qd0 = bf2_mul(bf2_mul(qn0, ep0), sc2), qd1 = bf2_mul(bf2_mul(qn1, ep1), sc2);
    const uint32_t ki0 = bf2_mul(kn0, em0), ki1 = bf2_mul(kn1, em1);
    const uint32_t kr0 = bf2_mul(ki0, ep0), kr1 = bf2_mul(ki1, ep1);  // ki (*) bf(E_tot); bf(E_tot) = e+ for one row
    const float kdf[4] = {bf_lo(kd0), bf_hi(kd0), bf_lo(kd1), bf_hi(kd1)};
    const float qdf[4] = {bf_lo(qd0), bf_hi(qd0), bf_lo(qd1), bf_hi(qd1)};
    const float krf[4] = {bf_lo(kr0), bf_hi(kr0), bf_lo(kr1), bf_hi(kr1)};
    // Mqk[0,0] = bf(qd . ki): the only entry of the masked in-chunk product; INV is the identity
    float mq = 0.0f;
    mq = __fmaf_rn(qdf[0], bf_lo(ki0), mq);
    mq = __fmaf_rn(qdf[1], bf_hi(ki0), mq);
    mq = __fmaf_rn(qdf[2], bf_lo(ki1), mq);
    mq = __fmaf_rn(qdf[3], bf_hi(ki1), mq);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mq = __fadd_rn(mq, __shfl_xor_sync(0xffffffffu, mq, off));
    const float mqk = bf2f(f2bf(mq));
    const __nv_bfloat16 beta_b = f2bf(sigmoid_tanh(beta_logit));

    // ---- u0 = bf(kd . S[v,:]), o0 = bf(qd . S[v,:]) for my warp's rows ----
    float pu[32], po[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        const float s0 = bf_lo(sreg[2 * r]), s1 = bf_hi(sreg[2 * r]), s2 = bf_lo(sreg[2 * r + 1]), s3 = bf_hi(sreg[2 * r + 1]);
        pu[r] = __fmaf_rn(kdf[3], s3, __fmaf_rn(kdf[2], s2, __fmaf_rn(kdf[1], s1, __fmul_rn(kdf[0], s0))));
        po[r] = __fmaf_rn(qdf[3], s3, __fmaf_rn(qdf[2], s2, __fmaf_rn(qdf[1], s1, __fmul_rn(qdf[0], s0))));
    }
    const __nv_bfloat16 u0 = f2bf(warp_rows_reduce(pu, lane));  // row row0 + lane
    const __nv_bfloat16 o0 = f2bf(warp_rows_reduce(po, lane));

    // ---- u' = (v (-) u0) (*) beta;  U = u' (identity inverse);  out = o0 (+) bf(Mqk U) ----
    const __nv_bfloat16 u_new = bfmul(bfsub(v_mine, u0), beta_b);
    const float u_f = bf2f(u_new);
    a.out[tok + row0 + lane] = bfadd(o0, f2bf(__fmul_rn(mqk, u_f)));

    // ---- S[v,k] = bf(fma(S[v,k], E_tot[k], kr[k] U[v])) and out to the final state ----
    if (a.final_state == nullptr) return;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        const float ur = __shfl_sync(0xffffffffu, u_f, r);
        const uint32_t x0 = sreg[2 * r], x1 = sreg[2 * r + 1];
        const float n0 = __fmaf_rn(bf_lo(x0), et[0], __fmul_rn(krf[0], ur));
        const float n1 = __fmaf_rn(bf_hi(x0), et[1], __fmul_rn(krf[1], ur));
        const float n2 = __fmaf_rn(bf_lo(x1), et[2], __fmul_rn(krf[2], ur));
        const float n3 = __fmaf_rn(bf_hi(x1), et[3], __fmul_rn(krf[3], ur));
        const uint32_t y0 = pack_bf2(n0, n1), y1 = pack_bf2(n2, n3);
        if (a.state_fp32) {
            float* dst = reinterpret_cast<float*>(a.final_state) + st_base + r * kD;
            *reinterpret_cast<float4*>(dst) = make_float4(bf_lo(y0), bf_hi(y0), bf_lo(y1), bf_hi(y1));
        } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.final_state) + st_base + r * kD;
            *reinterpret_cast<uint2*>(dst) = make_uint2(y0, y1);
        }
    }
}

bool decode_eligible(const fkda_fwd_params& p) {
    return p.cu_seqlens == nullptr && p.T == 1 && (p.phase_mask == 0 || p.phase_mask == (FKDA_PHASE_PREPARE | FKDA_PHASE_RECURRENCE));
}

int launch_decode_ragged(const TwoPassArgs& a, cudaStream_t stream) {
    const int64_t chains = a.N * a.H;
    if (chains > 0x7fffffff) return FKDA_ERR_BAD_SHAPE;
    decode_kernel<<<(unsigned)chains, 128, 0, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? FKDA_OK : FKDA_ERR_LAUNCH;
}

int launch_decode(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches) {
    TwoPassArgs a;
    fill_args(p, &a);
    if (cudaMemsetAsync(p.workspace, 0, 16, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;  // header: device status
    const int64_t chains = p.N * p.H;
    if (chains > 0x7fffffff) return FKDA_ERR_BAD_SHAPE;
    decode_kernel<<<(unsigned)chains, 128, 0, stream>>>(a);
    if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
    *n_launches = 1;
    return FKDA_OK;
}

}  // namespace fkda
