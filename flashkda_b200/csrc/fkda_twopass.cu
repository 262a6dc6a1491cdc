// Two-pass KDA forward on CUDA cores: a token-parallel "prepare" kernel writes the
// per-chunk operands to an HBM workspace, a per-(sequence, head) "recurrence" kernel
// walks the chunks serially with the [128,128] state in shared memory.
//
// This is the plain, easy-to-audit implementation of the numerics contract
// (tests/torch_ref.py:124-251 in the reference); it shares the kernel split of the
// reference (csrc/smxx/fwd_kernel1.cuh:105-588 prepare, csrc/smxx/fwd_kernel2.cuh:133-839
// recurrence) but none of its code: no CuTe, one thread per state row, scalar fp32 FMAs.
// The fused tensor-core kernel is checked against it on the device.
#include "fkda_common.cuh"
#include "fkda_internal.h"

namespace fkda {

// ---------------------------------------------------------------------------------
// varlen: chunk-count prefix over the sequences, tile_prefix[n] = sum_{m<n} ceil(len_m/16)
// (replaces the reference's single-thread loop, csrc/smxx/fwd_kernel1.cuh:88-103)
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) tile_prefix_kernel(const int64_t* __restrict__ cu, int64_t N,
                                                           int32_t* __restrict__ prefix) {
    __shared__ int64_t part[1024];
    const int tid = threadIdx.x;
    const int64_t per = (N + 1023) / 1024;
    const int64_t lo = tid * per, hi = (lo + per < N) ? lo + per : N;
    int64_t s = 0;
    for (int64_t n = lo; n < hi; ++n) {
        int64_t len = cu[n + 1] - cu[n];
        if (len < 0) len = 0;
        s += (len + kChunk - 1) / kChunk;
    }
    part[tid] = s;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
        int64_t add = (tid >= off) ? part[tid - off] : 0;
        __syncthreads();
        part[tid] += add;
        __syncthreads();
    }
    int64_t run = (tid == 0) ? 0 : part[tid - 1];
    for (int64_t n = lo; n < hi; ++n) {
        prefix[n] = (int32_t)run;
        int64_t len = cu[n + 1] - cu[n];
        if (len < 0) len = 0;
        run += (len + kChunk - 1) / kChunk;
    }
    if (tid == 1023) prefix[N] = (int32_t)part[1023];
}

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
    __nv_bfloat16 qn[8], kn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { qn[i] = f2bf(__fmul_rn(qv[i], qinv)); kn[i] = f2bf(__fmul_rn(kv[i], kinv)); }

    // ---- gate activation: gate_scale * sigmoid(exp(A_log) * (g + dt_bias)); 0 past the end ----
    const float a_exp = ex2_approx(__fmul_rn(a.A_log[h], 1.4426950408889634f));
    {
        const float4 dt0 = *reinterpret_cast<const float4*>(a.dt_bias + (int64_t)h * kD + c8);
        const float4 dt1 = *reinterpret_cast<const float4*>(a.dt_bias + (int64_t)h * kD + c8 + 4);
        const float dt[8] = {dt0.x, dt0.y, dt0.z, dt0.w, dt1.x, dt1.y, dt1.z, dt1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x = __fmul_rn(a_exp, __fadd_rn(gv[i], dt[i]));
            sm.G[row][c8 + i] = valid ? __fmul_rn(a.gate_scale, sigmoid_tanh(x)) : 0.0f;
        }
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
    const int64_t rec = ((int64_t)h * a.total_tiles + tile) * (int64_t)kWsRecord;
    uint8_t* ws = a.workspace + rec;
    {
        const __nv_bfloat16 sc = f2bf(a.scale);
        uint32_t kd_p[4], qd_p[4], ki_p[4], kr_p[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            __nv_bfloat16 r[4][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float G = sm.G[row][c8 + i + j];
                const __nv_bfloat16 ep = f2bf(ex2_approx(G));
                const __nv_bfloat16 em = f2bf(ex2_approx(-G));
                const __nv_bfloat16 et = f2bf(sm.etot[c8 + i + j]);
                r[0][j] = bfmul(kn[i + j], ep);
                r[1][j] = bfmul(bfmul(qn[i + j], ep), sc);
                r[2][j] = bfmul(kn[i + j], em);
                r[3][j] = bfmul(r[2][j], et);
            }
            auto pk = [](__nv_bfloat16 lo, __nv_bfloat16 hi) {
                __nv_bfloat162 v(lo, hi);
                return *reinterpret_cast<uint32_t*>(&v);
            };
            kd_p[i / 2] = pk(r[0][0], r[0][1]);
            qd_p[i / 2] = pk(r[1][0], r[1][1]);
            ki_p[i / 2] = pk(r[2][0], r[2][1]);
            kr_p[i / 2] = pk(r[3][0], r[3][1]);
        }
        const uint4 kd4 = make_uint4(kd_p[0], kd_p[1], kd_p[2], kd_p[3]);
        const uint4 qd4 = make_uint4(qd_p[0], qd_p[1], qd_p[2], qd_p[3]);
        const uint4 ki4 = make_uint4(ki_p[0], ki_p[1], ki_p[2], ki_p[3]);
        const uint4 kr4 = make_uint4(kr_p[0], kr_p[1], kr_p[2], kr_p[3]);
        *reinterpret_cast<uint4*>(&sm.kd[row][c8]) = kd4;
        *reinterpret_cast<uint4*>(&sm.qd[row][c8]) = qd4;
        *reinterpret_cast<uint4*>(&sm.ki[row][c8]) = ki4;
        const int eoff = (row * kD + c8) * 2;
        *reinterpret_cast<uint4*>(ws + kWsKd + eoff) = kd4;
        *reinterpret_cast<uint4*>(ws + kWsQd + eoff) = qd4;
        *reinterpret_cast<uint4*>(ws + kWsKr + eoff) = kr4;
    }
    if (tid < kD) reinterpret_cast<float*>(ws + kWsEt)[tid] = sm.etot[tid];
    __syncthreads();

    // ---- L = fp16(kd ki^T) masked * fp16(beta), Mqk = bf16(qd ki^T) masked; thread (i, j) ----
    {
        const int i = tid >> 4, j = tid & 15;
        float sl = 0.f, sq = 0.f;
#pragma unroll 4
        for (int c = 0; c < kD; c += 8) {
            const uint4 A = *reinterpret_cast<const uint4*>(&sm.kd[i][c]);
            const uint4 Q = *reinterpret_cast<const uint4*>(&sm.qd[i][c]);
            const uint4 Bv = *reinterpret_cast<const uint4*>(&sm.ki[j][c]);
            const uint32_t* ap = &A.x; const uint32_t* qp = &Q.x; const uint32_t* bp = &Bv.x;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sl = __fmaf_rn(bf_lo(ap[e]), bf_lo(bp[e]), sl);
                sq = __fmaf_rn(bf_lo(qp[e]), bf_lo(bp[e]), sq);
                sl = __fmaf_rn(bf_hi(ap[e]), bf_hi(bp[e]), sl);
                sq = __fmaf_rn(bf_hi(qp[e]), bf_hi(bp[e]), sq);
            }
        }
        __half l = __float2half_rn(0.0f);
        if (i > j) l = __hmul(__float2half_rn(sl), __float2half_rn(sm.beta_act[i]));
        sm.L[i][j] = l;
        reinterpret_cast<__nv_bfloat16*>(ws + kWsMqk)[i * kChunk + j] = (i >= j) ? f2bf(sq) : f2bf(0.0f);
    }
    __syncthreads();
    if (tid < 32)
        neumann_inverse_warp(&sm.L[0][0], &sm.W[0][0], kLd16, reinterpret_cast<__nv_bfloat16*>(ws + kWsInv), tid);
}

// ---------------------------------------------------------------------------------
// recurrence: one CTA per (sequence, head), 128 threads, thread v owns state row S[v][:]
// ---------------------------------------------------------------------------------
constexpr int kSPitch = kD + 2;  // bf16 pitch 260 B = 65 words: conflict-free row-per-thread access

struct RecSmem {
    __nv_bfloat16 S[kD][kSPitch];
    float kd[kChunk][kD];
    float qd[kChunk][kD];
    float krT[kD][kChunk];
    float etot[kD];
    float inv[kChunk][kChunk];
    float mqk[kChunk][kChunk];
    float beta_bf[kChunk];  // bf16-rounded sigmoid(beta), widened
};

__global__ void __launch_bounds__(128) recurrence_kernel(TwoPassArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    RecSmem& sm = *reinterpret_cast<RecSmem*>(smem_raw);
    const int v = threadIdx.x;
    const int h = blockIdx.y;
    const int64_t n = blockIdx.x;

    int64_t bos, seq_len, tile_base;
    if (a.cu_seqlens != nullptr) {
        bos = a.cu_seqlens[n];
        seq_len = a.cu_seqlens[n + 1] - bos;
        if (seq_len < 0) seq_len = 0;
        tile_base = a.tile_prefix[n];
    } else {
        bos = n * a.T;
        seq_len = a.T;
        tile_base = n * ((a.T + kChunk - 1) / kChunk);
    }
    const int64_t n_chunks = (seq_len + kChunk - 1) / kChunk;
    const int64_t st_off = (n * a.H + h) * (int64_t)(kD * kD) + (int64_t)v * kD;

    // ---- initial state: bf16 as is, fp32 rounded to bf16, or zero ----
    if (a.initial_state != nullptr) {
        if (a.state_fp32) {
            const float* src = reinterpret_cast<const float*>(a.initial_state) + st_off;
            for (int c = 0; c < kD; ++c) sm.S[v][c] = f2bf(src[c]);
        } else {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.initial_state) + st_off;
            for (int c = 0; c < kD; ++c) sm.S[v][c] = src[c];
        }
    } else {
        for (int c = 0; c < kD; ++c) sm.S[v][c] = f2bf(0.0f);
    }

    for (int64_t t = 0; t < n_chunks; ++t) {
        const int64_t t0 = bos + t * kChunk;
        const int len = (int)min((int64_t)kChunk, seq_len - t * kChunk);
        const uint8_t* ws = a.workspace + ((int64_t)h * a.total_tiles + tile_base + t) * (int64_t)kWsRecord;
        __syncthreads();  // previous chunk's readers are done with the operand tiles
        // ---- stage the chunk operands as fp32 ----
        for (int e = v; e < kChunk * kD; e += 128) {
            const int r = e >> 7, c = e & 127;
            sm.kd[r][c] = bf2f(reinterpret_cast<const __nv_bfloat16*>(ws + kWsKd)[e]);
            sm.qd[r][c] = bf2f(reinterpret_cast<const __nv_bfloat16*>(ws + kWsQd)[e]);
            sm.krT[c][r] = bf2f(reinterpret_cast<const __nv_bfloat16*>(ws + kWsKr)[e]);
        }
        sm.etot[v] = reinterpret_cast<const float*>(ws + kWsEt)[v];
        for (int e = v; e < kChunk * kChunk; e += 128) {
            sm.inv[e >> 4][e & 15] = bf2f(reinterpret_cast<const __nv_bfloat16*>(ws + kWsInv)[e]);
            sm.mqk[e >> 4][e & 15] = bf2f(reinterpret_cast<const __nv_bfloat16*>(ws + kWsMqk)[e]);
        }
        if (v < kChunk) {
            float b = 0.0f;
            if (v < len) b = bf2f(a.beta[(t0 + v) * a.beta_token_stride + h]);
            sm.beta_bf[v] = bf2f(f2bf(sigmoid_tanh(b)));
        }
        __syncthreads();

        // ---- u0[i] = kd[i,:] . S[v,:],  o0[i] = qd[i,:] . S[v,:]  (fp32, k ascending) ----
        float u[kChunk], o[kChunk];
#pragma unroll
        for (int i = 0; i < kChunk; ++i) { u[i] = 0.f; o[i] = 0.f; }
        const uint32_t* Srow = reinterpret_cast<const uint32_t*>(&sm.S[v][0]);
#pragma unroll 2
        for (int c = 0; c < kD; c += 4) {
            const uint32_t s01 = Srow[c >> 1], s23 = Srow[(c >> 1) + 1];
            const float s0 = bf_lo(s01), s1 = bf_hi(s01), s2 = bf_lo(s23), s3 = bf_hi(s23);
#pragma unroll
            for (int i = 0; i < kChunk; ++i) {
                const float4 kk = *reinterpret_cast<const float4*>(&sm.kd[i][c]);
                const float4 qq = *reinterpret_cast<const float4*>(&sm.qd[i][c]);
                u[i] = __fmaf_rn(kk.x, s0, u[i]); o[i] = __fmaf_rn(qq.x, s0, o[i]);
                u[i] = __fmaf_rn(kk.y, s1, u[i]); o[i] = __fmaf_rn(qq.y, s1, o[i]);
                u[i] = __fmaf_rn(kk.z, s2, u[i]); o[i] = __fmaf_rn(qq.z, s2, o[i]);
                u[i] = __fmaf_rn(kk.w, s3, u[i]); o[i] = __fmaf_rn(qq.w, s3, o[i]);
            }
        }
        // ---- u' = (v - bf(u0)) * bf(beta), bf16 after each op; rows past the end use v = 0 ----
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
            float vv = 0.0f;
            if (i < len) vv = bf2f(a.v[(t0 + i) * a.token_stride + (int64_t)h * kD + v]);
            const float d = bf2f(f2bf(__fsub_rn(vv, bf2f(f2bf(u[i])))));
            u[i] = bf2f(f2bf(__fmul_rn(d, sm.beta_bf[i])));
        }
        // ---- U = bf(INV u') ----
        float U[kChunk];
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < kChunk; ++j) s = __fmaf_rn(sm.inv[i][j], u[j], s);
            U[i] = bf2f(f2bf(s));
        }
        // ---- out = bf(o0) (+) bf(Mqk U), valid rows only ----
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < kChunk; ++j) s = __fmaf_rn(sm.mqk[i][j], U[j], s);
            if (i < len)
                a.out[(t0 + i) * a.token_stride + (int64_t)h * kD + v] =
                    f2bf(__fadd_rn(bf2f(f2bf(o[i])), bf2f(f2bf(s))));
        }
        // ---- S[v][k] = bf(fma(S[v][k], E_tot[k], sum_i kr[i][k] U[i])) ----
        uint32_t* Sw = reinterpret_cast<uint32_t*>(&sm.S[v][0]);
#pragma unroll 2
        for (int c = 0; c < kD; c += 2) {
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int i = 0; i < kChunk; i += 4) {
                const float4 k0 = *reinterpret_cast<const float4*>(&sm.krT[c][i]);
                const float4 k1 = *reinterpret_cast<const float4*>(&sm.krT[c + 1][i]);
                d0 = __fmaf_rn(k0.x, U[i], d0); d1 = __fmaf_rn(k1.x, U[i], d1);
                d0 = __fmaf_rn(k0.y, U[i + 1], d0); d1 = __fmaf_rn(k1.y, U[i + 1], d1);
                d0 = __fmaf_rn(k0.z, U[i + 2], d0); d1 = __fmaf_rn(k1.z, U[i + 2], d1);
                d0 = __fmaf_rn(k0.w, U[i + 3], d0); d1 = __fmaf_rn(k1.w, U[i + 3], d1);
            }
            const uint32_t s01 = Sw[c >> 1];
            Sw[c >> 1] = pack_bf2(__fmaf_rn(bf_lo(s01), sm.etot[c], d0), __fmaf_rn(bf_hi(s01), sm.etot[c + 1], d1));
        }
    }

    // ---- final state: bf16, or the bf16 state widened to fp32 ----
    if (a.final_state != nullptr) {
        if (a.state_fp32) {
            float* dst = reinterpret_cast<float*>(a.final_state) + st_off;
            for (int c = 0; c < kD; ++c) dst[c] = bf2f(sm.S[v][c]);
        } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.final_state) + st_off;
            for (int c = 0; c < kD; ++c) dst[c] = sm.S[v][c];
        }
    }
}

// ---------------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------------
size_t twopass_workspace_bytes(int64_t T_total, int64_t H, int64_t N) {
    const int64_t tiles = (T_total + kChunk - 1) / kChunk + N;  // upper bound with ragged tails
    const size_t prefix = (size_t)(((N + 1) * 4 + 255) / 256 * 256);
    return prefix + (size_t)H * (size_t)tiles * (size_t)kWsRecord;
}

int launch_twopass(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches) {
    TwoPassArgs a;
    a.q = reinterpret_cast<const __nv_bfloat16*>(p.q);
    a.k = reinterpret_cast<const __nv_bfloat16*>(p.k);
    a.v = reinterpret_cast<const __nv_bfloat16*>(p.v);
    a.g = reinterpret_cast<const __nv_bfloat16*>(p.g);
    a.beta = reinterpret_cast<const __nv_bfloat16*>(p.beta);
    a.out = reinterpret_cast<__nv_bfloat16*>(p.out);
    a.A_log = p.A_log;
    a.dt_bias = p.dt_bias;
    a.initial_state = p.initial_state;
    a.final_state = p.final_state;
    a.state_fp32 = (p.state_dtype == FKDA_STATE_FP32);
    a.cu_seqlens = p.cu_seqlens;
    a.T = p.T;
    a.H = p.H;
    a.N = p.N;
    a.token_stride = p.token_stride;
    a.beta_token_stride = p.beta_token_stride;
    a.scale = p.scale;
    a.gate_scale = (float)(p.lower_bound * 1.4426950408889634);  // log2-domain gate (csrc/flash_kda.cpp:128)
    const int64_t T_total = p.B * p.T;
    const bool varlen = p.cu_seqlens != nullptr;
    a.total_tiles = varlen ? (T_total + kChunk - 1) / kChunk + p.N : p.N * ((p.T + kChunk - 1) / kChunk);
    const size_t prefix_bytes = (size_t)(((p.N + 1) * 4 + 255) / 256 * 256);
    a.tile_prefix = reinterpret_cast<int32_t*>(p.workspace);
    a.workspace = reinterpret_cast<uint8_t*>(p.workspace) + prefix_bytes;

    int launches = 0;
    const bool do_prep = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_PREPARE);
    const bool do_rec = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_RECURRENCE);
    if (varlen && do_prep) {
        tile_prefix_kernel<<<1, 1024, 0, stream>>>(p.cu_seqlens, p.N, a.tile_prefix);
        ++launches;
    }
    if (a.total_tiles > 0 && do_prep) {
        dim3 grid1((unsigned)a.total_tiles, (unsigned)p.H);
        prepare_kernel<<<grid1, 256, 0, stream>>>(a);
        ++launches;
    }
    // per device and cheap, so set on every call rather than cached per process
    if (cudaFuncSetAttribute(recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)sizeof(RecSmem)) != cudaSuccess)
        return FKDA_ERR_LAUNCH;
    if (do_rec) {
        dim3 grid2((unsigned)p.N, (unsigned)p.H);
        recurrence_kernel<<<grid2, 128, sizeof(RecSmem), stream>>>(a);
        ++launches;
    }
    if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
    *n_launches = launches;
    return FKDA_OK;
}

}  // namespace fkda
