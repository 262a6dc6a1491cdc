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
#include "fkda_prepare_warp.cuh"

namespace fkda {

// ---------------------------------------------------------------------------------
// varlen: chunk-count prefix over the sequences, tile_prefix[n] = sum_{m<n} ceil(len_m/16)
// (replaces the reference's single-thread loop, csrc/smxx/fwd_kernel1.cuh:88-103)
// ---------------------------------------------------------------------------------
// Also ranks the sequences by decreasing length (order[rank] = sequence; ties by index) when the batch is small
// enough for the quadratic count: the recurrence starts the longest chains first and keeps them apart.
__global__ void __launch_bounds__(1024) tile_prefix_kernel(const int64_t* __restrict__ cu, int64_t N,
                                                           int32_t* __restrict__ prefix, int32_t* __restrict__ order,
                                                           int32_t* __restrict__ cs_prefix, int cs_tokens,
                                                           int32_t* __restrict__ short_flag, int decode_enqueued,
                                                           int32_t* __restrict__ critical_chunks, int64_t heads, int chain_slots) {
    __shared__ int64_t part[1024];
    const int tid = threadIdx.x;
    const int64_t per = (N + 1023) / 1024;
    const int64_t lo = tid * per, hi = (lo + per < N) ? lo + per : N;
    // exclusive prefix over the sequences of ceil(len / unit): chunks (unit 16), or state-export groups
    auto scan = [&](int64_t unit, int32_t* out) {
        int64_t s = 0;
        for (int64_t n = lo; n < hi; ++n) {
            int64_t len = cu[n + 1] - cu[n];
            if (len < 0) len = 0;
            s += (len + unit - 1) / unit;
        }
        __syncthreads();
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
            out[n] = (int32_t)run;
            int64_t len = cu[n + 1] - cu[n];
            if (len < 0) len = 0;
            run += (len + unit - 1) / unit;
        }
        if (tid == 1023) out[N] = (int32_t)part[1023];
    };
    scan(kChunk, prefix);
    // A chain at least as long as a chain slot's even share of the whole work is on the critical path from its first
    // chunk: the recurrence walks it in one piece instead of in queued segments.
    if (critical_chunks != nullptr && tid == 1023)
        *critical_chunks = (int32_t)((heads * part[1023] + chain_slots - 1) / chain_slots);
    if (cs_prefix != nullptr) scan(cs_tokens, cs_prefix);
    if (short_flag != nullptr) {   // who serves the call (see TwoPassArgs::short_flag)
        int longer = 0, not_one = 0;
        for (int64_t n = lo; n < hi; ++n) {
            const int64_t len = cu[n + 1] - cu[n];
            longer |= (len > kChunk) ? 1 : 0;
            not_one |= (len != 1) ? 1 : 0;
        }
        longer = __syncthreads_or(longer);
        not_one = __syncthreads_or(not_one);
        if (tid == 0) *short_flag = longer ? 0 : ((decode_enqueued && !not_one) ? 2 : 1);
    }
    if (order != nullptr) {
        for (int64_t n = tid; n < N; n += 1024) {
            const int64_t len_n = cu[n + 1] - cu[n];
            int rank = 0;
            for (int64_t m = 0; m < N; ++m) {
                const int64_t len_m = cu[m + 1] - cu[m];
                rank += (len_m > len_n || (len_m == len_n && m < n)) ? 1 : 0;
            }
            order[rank] = (int32_t)n;
        }
    }
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
        if (a.chunk_states != nullptr && t % a.cs_every == 0) {   // export the state before this group of chunks
            __nv_bfloat16* dst = a.chunk_states + ((cs_first_slot(a, n) + t / a.cs_every) * a.H + h) * (int64_t)(kD * kD) + (int64_t)v * kD;
            for (int c = 0; c < kD; ++c) dst[c] = sm.S[v][c];
        }
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
void launch_tile_prefix(const int64_t* cu_seqlens, int64_t N, int32_t* prefix, int32_t* seq_order, int32_t* cs_prefix,
                        int cs_tokens, int32_t* short_flag, bool decode_enqueued, int32_t* critical_chunks, int64_t heads,
                        int chain_slots, cudaStream_t stream) {
    tile_prefix_kernel<<<1, 1024, 0, stream>>>(cu_seqlens, N, prefix, seq_order, cs_prefix, cs_tokens, short_flag,
                                               decode_enqueued ? 1 : 0, critical_chunks, heads, chain_slots);
}

size_t twopass_workspace_bytes(int64_t T_total, int64_t H, int64_t N) {
    return kWsHeaderBytes + ws_prefix_bytes(N) +
           (size_t)H * (size_t)ws_tiles_upper_bound(T_total, N) * (size_t)kWsRecord;
}

void fill_args(const fkda_fwd_params& p, TwoPassArgs* out) {
    TwoPassArgs& a = *out;
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
    const uint64_t wait_ms = (uint64_t)((p.flags >> 16) & 0x3fff);
    a.wait_ns = (wait_ms ? wait_ms : 2000u) * 1000000ull;
    a.chunk_states = reinterpret_cast<__nv_bfloat16*>(p.chunk_states);
    a.cs_every = p.chunk_states != nullptr ? p.chunk_states_every : 1;
    a.test_drop_push = (p.flags & FKDA_FLAG_TEST_DROP_PUSH) != 0;
    const int64_t T_total = p.B * p.T;
    const bool varlen = p.cu_seqlens != nullptr;
    a.total_tiles = varlen ? ws_tiles_upper_bound(T_total, p.N) : p.N * ((p.T + kChunk - 1) / kChunk);
    uint8_t* base = reinterpret_cast<uint8_t*>(p.workspace);
    a.queue = reinterpret_cast<int32_t*>(base);
    a.status = reinterpret_cast<int32_t*>(base) + 1;
    a.short_flag = nullptr;
    a.qslots = nullptr;
    a.seg_state = nullptr;
    a.seg_chunks = 0;
    a.slab_c0 = 0;
    a.slab_chunks = 0;
    a.tile_prefix = reinterpret_cast<int32_t*>(base + kWsHeaderBytes);
    a.seq_order = (varlen && p.N <= kSeqOrderMaxN) ? a.tile_prefix + (p.N + 1) : nullptr;
    a.cs_prefix = a.tile_prefix + (2 * p.N + 1);
    a.workspace = base + kWsHeaderBytes + ws_prefix_bytes(p.N);
}

int launch_twopass(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches) {
    TwoPassArgs a;
    fill_args(p, &a);
    const bool varlen = p.cu_seqlens != nullptr;
    int launches = 0;
    if (cudaMemsetAsync(p.workspace, 0, 16, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;  // queue + status
    const bool do_prep = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_PREPARE);
    const bool do_rec = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_RECURRENCE);
    if (varlen && do_prep) {
        launch_tile_prefix(p.cu_seqlens, p.N, a.tile_prefix, const_cast<int32_t*>(a.seq_order),
                           a.chunk_states != nullptr ? const_cast<int32_t*>(a.cs_prefix) : nullptr, 16 * a.cs_every, nullptr, false, nullptr, 0, 1, stream);
        ++launches;
    }
    if (a.total_tiles > 0 && do_prep) {
        if (launch_prepare_warp<false>(a, stream) != FKDA_OK) return FKDA_ERR_LAUNCH;
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
