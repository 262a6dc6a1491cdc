// Tensor-core two-pass KDA forward for sm_100a: the token-parallel prepare kernel writes per-chunk
// operand records already laid out as tcgen05 (UMMA) shared-memory operands; a persistent
// recurrence kernel walks the chunks of each (sequence, head) chain with
//   * one bulk asynchronous copy (TMA engine) per chunk record, double buffered on mbarriers; value
//     columns prefetched into registers one chunk ahead, out rows stored from registers,
//   * the [128,128] bf16 state resident in shared memory as the A operand of the state contraction,
//   * all contractions on tcgen05.mma with fp32 accumulators in tensor memory, in the transposed
//     formulation that makes V = 128 the MMA M dimension:
//        D1[V,32]  = S[V,K] . [kd; qd]^T          (8 x M128 N32 K16)
//        D2[V,16]  = u'^T[V,16] . INV^T           (M128 N16 K16)
//        D3[V,16]  = U^T[V,16] . Mqk^T            (M128 N16 K16)
//        DS[V,K]   = U^T[V,16] . kr[16,K]         (M128 N128 K16, MN-major B)
//   * element-wise steps (bf16 roundings, beta, gate decay) by 128 threads, one per V row, reading the
//     accumulators with tcgen05.ld.
// Three independent chains run per CTA (one warpgroup each) so that the tensor-core / barrier latency
// of one chain is covered by the element-wise work of the others.
//
// Numerics: steps B1-B7 of the reference's contract (tests/torch_ref.py:231-251; the reference's own
// recurrence is csrc/smxx/fwd_kernel2.cuh:434-742, built on mma.sync with register transposes).
#include "fkda_common.cuh"
#include "fkda_internal.h"
#include "fkda_prepare.cuh"
#include "fkda_sm100.cuh"

namespace fkda {

using namespace sm100;

// Profiling aid (off by default): with -DFKDA_TC_TIMING thread 0 of CTA 0 stores clock64() deltas of
// the stages of its 64th chunk into the workspace header (ints 16..31).
#ifdef FKDA_TC_TIMING
#define TC_STAMP(i) do { if (blockIdx.x == 0 && threadIdx.x == 0 && t == 64) stamps[i] = clock64(); } while (0)
#else
#define TC_STAMP(i) do { } while (0)
#endif

constexpr int kTcChains = 3;    // chains (warpgroups) per CTA
constexpr int kTcStages = 2;    // chunk records in flight per chain
constexpr int kTcTmemCols = 512;
constexpr uint32_t kTcWaitNs = 2000000000u;

// byte offsets inside one chain's shared-memory block
constexpr int kSmS = 0;                                    // state, canonical K-major A operand [128, 128]
constexpr int kSmStage = 32768;                            // kTcStages x (record + value tile)
constexpr int kSmStageBytes = kTcRecord;                   // 13888
constexpr int kSmA23 = kSmStage + kTcStages * kSmStageBytes;  // A operand of the 16-deep products [128, 16]
constexpr int kSmChainBytes = kSmA23 + 4096;               // 64640
static_assert(kSmChainBytes % 128 == 0, "chain blocks stay 128-byte aligned");

struct TcCtrl {
    uint64_t full[kTcChains][kTcStages];
    uint64_t mma[kTcChains];
    uint32_t tmem_base;
    int32_t next_chain[kTcChains];
    int32_t abort_flag;
};
constexpr int kTcSmemBytes = kTcChains * kSmChainBytes + (int)sizeof(TcCtrl) + 128;
static_assert(kTcSmemBytes <= 232448, "exceeds the 227 KB shared-memory limit of a CTA");

// state element (v, k..k+7) lives at kc*2048 + (v/8)*128 + (v%8)*16   (kc = k/8)
__device__ __forceinline__ int s_off(int v, int kc) { return kc * 2048 + (v >> 3) * 128 + (v & 7) * 16; }

__global__ void __launch_bounds__(kTcChains * 128, 1) recurrence_tc_kernel(TwoPassArgs a) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 127) & ~(uintptr_t)127);
    TcCtrl& ctl = *reinterpret_cast<TcCtrl*>(smem + kTcChains * kSmChainBytes);

    // warp-uniform role indices (the shuffle makes the uniformity visible to the compiler, so the
    // single-thread tcgen05 issue below sits in warp-uniform control flow)
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int wg = warp >> 2;          // chain slot
    const int wiw = warp & 3;          // warp within the warpgroup
    const int v = threadIdx.x & 127;   // state row = TMEM lane
    uint8_t* cs = smem + wg * kSmChainBytes;
    volatile int* abort_flag = &ctl.abort_flag;

    if (threadIdx.x == 0) {
        for (int c = 0; c < kTcChains; ++c) {
            for (int s = 0; s < kTcStages; ++s) mbar_init(&ctl.full[c][s], 1);
            mbar_init(&ctl.mma[c], 1);
        }
        ctl.abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(&ctl.tmem_base, kTcTmemCols);
        tmem_relinquish_alloc_permit();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl.tmem_base;
    // columns: DS of chain c at 128*c (128 wide), D1 of chain c at 384 + 32*c (32 wide; D2 reuses
    // its first 16 columns and D3 its last 16 once D1 has been read)
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_ds = tmem_base + 128u * wg;
    const uint32_t t_d1 = tmem_base + 384u + 32u * wg;

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, false, false);
    constexpr uint32_t idesc_n16 = make_idesc_bf16_f32(128, 16, false, false);
    constexpr uint32_t idesc_ds = make_idesc_bf16_f32(128, 128, false, true);

    const uint32_t s_addr = smem_u32(cs + kSmS);
    const uint32_t a23_addr = smem_u32(cs + kSmA23);
    const uint64_t s_desc0 = make_smem_desc(s_addr, 2048, 128);      // + 256 per K step of 16 (4096 B >> 4)
    const uint64_t a23_desc = make_smem_desc(a23_addr, 2048, 128);
    const int bar_id = 1 + wg;
    const int64_t n_chains = a.N * a.H;
    uint32_t full_phase[kTcStages] = {0, 0};
    uint32_t mma_phase = 0;
    bool failed = false;
#ifdef FKDA_TC_TIMING
    long long stamps[24] = {0};
#endif

    while (!failed) {
        // ---- next chain from the work queue ----
        if (v == 0) ctl.next_chain[wg] = atomicAdd(a.queue, 1);
        named_barrier_sync(bar_id, 128);
        const int64_t chain = ctl.next_chain[wg];
        if (chain >= n_chains) break;
        const int64_t n = chain / a.H;
        const int h = (int)(chain - n * a.H);
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
        const uint8_t* rec_base = a.workspace + ((int64_t)h * a.total_tiles + tile_base) * (int64_t)kTcRecord;
        const int64_t st_off = (n * a.H + h) * (int64_t)(kD * kD) + (int64_t)v * kD;

        auto issue_load = [&](int64_t t) {  // one thread: the record of chunk t into stage t % kTcStages
            const int s = (int)(t % kTcStages);
            mbar_arrive_expect_tx(&ctl.full[wg][s], (uint32_t)kTcRecord);
            bulk_g2s(cs + kSmStage + s * kSmStageBytes, rec_base + t * (int64_t)kTcRecord, kTcRecord,
                     &ctl.full[wg][s]);
        };
        if (v == 0) {
            for (int64_t t = 0; t < kTcStages && t < n_chunks; ++t) issue_load(t);
        }
        // value column of this thread for chunk t: rows (2i, 2i+1) packed as bf16x2, zero past the end;
        // fetched straight from global memory one chunk ahead (64 contiguous bytes per warp and row)
        const unsigned short* vcol = reinterpret_cast<const unsigned short*>(a.v) + bos * a.token_stride +
                                     (int64_t)h * kD + v;
        // (the raw 16-bit values are kept apart until they are used, so the loads stay in flight)
        auto load_v = [&](int64_t t, unsigned short (&dst)[kChunk]) {
            const int len = (int)min((int64_t)kChunk, seq_len - t * kChunk);
            const unsigned short* p = vcol + t * kChunk * a.token_stride;
#pragma unroll
            for (int i = 0; i < kChunk; ++i) {
                dst[i] = (i < len) ? __ldg(p) : (unsigned short)0;
                p += a.token_stride;
            }
        };
        unsigned short v_cur[kChunk], v_nxt[kChunk];
        if (n_chunks > 0) load_v(0, v_cur);

        // ---- initial state into the canonical A-operand layout (fp32 rounded to bf16) ----
        if (a.initial_state != nullptr) {
            if (a.state_fp32) {
                const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.initial_state) + st_off);
#pragma unroll 4
                for (int kc = 0; kc < 16; ++kc) {
                    const float4 x = src[2 * kc], y = src[2 * kc + 1];
                    *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, kc)) =
                        make_uint4(pack_bf2(x.x, x.y), pack_bf2(x.z, x.w), pack_bf2(y.x, y.y), pack_bf2(y.z, y.w));
                }
            } else {
                const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.initial_state) + st_off);
#pragma unroll 4
                for (int kc = 0; kc < 16; ++kc) *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, kc)) = src[kc];
            }
        } else {
#pragma unroll 4
            for (int kc = 0; kc < 16; ++kc) *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, kc)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        named_barrier_sync(bar_id, 128);

        // out rows of the previous chunk, finished while the next chunk's first MMA runs
        uint32_t o_pend[8];
        int64_t o_pend_t = -1;
        auto flush_out = [&]() {
            if (o_pend_t < 0) return;
            const int len = (int)min((int64_t)kChunk, seq_len - o_pend_t * kChunk);
            unsigned short* dst = reinterpret_cast<unsigned short*>(a.out) +
                                  (bos + o_pend_t * kChunk) * a.token_stride + (int64_t)h * kD + v;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (2 * i < len) *dst = (unsigned short)(o_pend[i] & 0xffffu);
                dst += a.token_stride;
                if (2 * i + 1 < len) *dst = (unsigned short)(o_pend[i] >> 16);
                dst += a.token_stride;
            }
            o_pend_t = -1;
        };

        for (int64_t t = 0; t < n_chunks; ++t) {
            const int s = (int)(t % kTcStages);
            uint8_t* st = cs + kSmStage + s * kSmStageBytes;
            const uint32_t st_addr = smem_u32(st);

            TC_STAMP(8);
            // ---- operands of chunk t have landed ----
            if (!mbar_wait_bounded(&ctl.full[wg][s], full_phase[s], abort_flag, kTcWaitNs)) { failed = true; break; }
            full_phase[s] ^= 1u;
            TC_STAMP(0);
#ifdef FKDA_TC_TIMING
            if (blockIdx.x == 0 && threadIdx.x == 0 && t == 65) stamps[12] = clock64();
#endif

            // ---- MMA1: D1[V,32] = S . [kd; qd]^T ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, 512, 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        umma_ss(t_d1, s_desc0 + (uint64_t)(j * 256), bd0 + (uint64_t)(j * 64), idesc_n32, j > 0 ? 1u : 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            TC_STAMP(1);
            // work off the critical path while the MMA runs
            flush_out();
            TC_STAMP(13);
            if (t + 1 < n_chunks) load_v(t + 1, v_nxt);
            TC_STAMP(14);
            const float4* bp = reinterpret_cast<const float4*>(st + kTcBeta);
            uint32_t bpk[8];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                const float4 b = bp[i4];
                bpk[2 * i4] = pack_bf2(b.x, b.y);  // exact: the record holds bf16-rounded values
                bpk[2 * i4 + 1] = pack_bf2(b.z, b.w);
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(2);

            // ---- u' = (v (-) bf(u0)) (*) bf(beta) -> A operand; keep bf(o0) ----
            uint32_t ob[8];
            {
                uint32_t r[32];
                tmem_ld32(t_d1 + lane_sel, r);
                tmem_wait_ld();
                uint32_t up[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t u0 = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    const uint32_t vp = (uint32_t)v_cur[2 * i] | ((uint32_t)v_cur[2 * i + 1] << 16);
                    up[i] = bf2_mul(bf2_sub(vp, u0), bpk[i]);
                    ob[i] = pack_bf2(__uint_as_float(r[16 + 2 * i]), __uint_as_float(r[16 + 2 * i + 1]));
                }
                uint8_t* ap = cs + kSmA23 + (v >> 3) * 128 + (v & 7) * 16;
                *reinterpret_cast<uint4*>(ap) = make_uint4(up[0], up[1], up[2], up[3]);
                *reinterpret_cast<uint4*>(ap + 2048) = make_uint4(up[4], up[5], up[6], up[7]);
            }
            TC_STAMP(3);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);
            TC_STAMP(4);

            // ---- MMA2: D2[V,16] = u'^T . INV^T ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ss(t_d1, a23_desc, make_smem_desc(st_addr + kTcInv, 256, 128), idesc_n16, 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(5);
            {
                uint32_t r[16];
                tmem_ld16(t_d1 + lane_sel, r);
                tmem_wait_ld();
                uint8_t* ap = cs + kSmA23 + (v >> 3) * 128 + (v & 7) * 16;
                uint32_t p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) p[i] = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                *reinterpret_cast<uint4*>(ap) = make_uint4(p[0], p[1], p[2], p[3]);
                *reinterpret_cast<uint4*>(ap + 2048) = make_uint4(p[4], p[5], p[6], p[7]);
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);
            TC_STAMP(6);

            // ---- MMA3: D3[V,16] = U^T . Mqk^T ;  DS[V,K] = U^T . kr ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ss(t_d1 + 16, a23_desc, make_smem_desc(st_addr + kTcMqk, 256, 128), idesc_n16, 0u);
                    umma_ss(t_ds, a23_desc, make_smem_desc(st_addr + kTcKr, 2048, 128), idesc_ds, 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(7);

            // ---- S[v][k] = bf(fma(S[v][k], E_tot[k], DS[v][k])), TMEM loads one batch ahead;
            //      out = bf(o0) (+) bf(Mqk U) is only formed here, its stores wait for the next MMA1 ----
            auto update_cols = [&](int cb, const uint32_t (&r)[32]) {
                // all loads of the batch first: the stores below may alias them as far as the compiler knows
                const float4* ep = reinterpret_cast<const float4*>(st + kTcEt) + cb * 8;
                uint4 sv[4];
                float4 e[8];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) sv[q4] = *reinterpret_cast<const uint4*>(cs + kSmS + s_off(v, cb * 4 + q4));
#pragma unroll
                for (int q = 0; q < 8; ++q) e[q] = ep[q];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float4 e0 = e[2 * q4], e1 = e[2 * q4 + 1];
                    const uint32_t* rr = r + q4 * 8;
                    uint4 nv;
                    nv.x = pack_bf2(__fmaf_rn(bf_lo(sv[q4].x), e0.x, __uint_as_float(rr[0])),
                                    __fmaf_rn(bf_hi(sv[q4].x), e0.y, __uint_as_float(rr[1])));
                    nv.y = pack_bf2(__fmaf_rn(bf_lo(sv[q4].y), e0.z, __uint_as_float(rr[2])),
                                    __fmaf_rn(bf_hi(sv[q4].y), e0.w, __uint_as_float(rr[3])));
                    nv.z = pack_bf2(__fmaf_rn(bf_lo(sv[q4].z), e1.x, __uint_as_float(rr[4])),
                                    __fmaf_rn(bf_hi(sv[q4].z), e1.y, __uint_as_float(rr[5])));
                    nv.w = pack_bf2(__fmaf_rn(bf_lo(sv[q4].w), e1.z, __uint_as_float(rr[6])),
                                    __fmaf_rn(bf_hi(sv[q4].w), e1.w, __uint_as_float(rr[7])));
                    *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, cb * 4 + q4)) = nv;
                }
            };
            {
                uint32_t r3[16], ra[32], rb[32];
                tmem_ld32(t_ds + lane_sel, ra);
                tmem_ld16(t_d1 + 16 + lane_sel, r3);
                TC_STAMP(16);
                tmem_wait_ld();
                TC_STAMP(17);
                tmem_ld32(t_ds + 32 + lane_sel, rb);
                TC_STAMP(18);
                update_cols(0, ra);
                TC_STAMP(19);
                tmem_wait_ld();
                TC_STAMP(20);
                tmem_ld32(t_ds + 64 + lane_sel, ra);
                update_cols(1, rb);
                TC_STAMP(21);
                tmem_wait_ld();
                TC_STAMP(22);
                tmem_ld32(t_ds + 96 + lane_sel, rb);
                update_cols(2, ra);
                tmem_wait_ld();
                update_cols(3, rb);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    o_pend[i] = bf2_add(ob[i], pack_bf2(__uint_as_float(r3[2 * i]), __uint_as_float(r3[2 * i + 1])));
                o_pend_t = t;
            }
            TC_STAMP(9);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);
            TC_STAMP(10);

            // ---- refill the stage just consumed ----
            if (v == 0 && t + kTcStages < n_chunks) issue_load(t + kTcStages);
#pragma unroll
            for (int i = 0; i < kChunk; ++i) v_cur[i] = v_nxt[i];
            TC_STAMP(11);
#ifdef FKDA_TC_TIMING
            if (blockIdx.x == 0 && threadIdx.x == 0 && t == 65) {
                for (int i = 0; i < 23; ++i) a.status[15 + i] = (int)(stamps[i] - stamps[0]);
            }
#endif
        }
        if (failed) break;
        flush_out();

        // ---- final state: bf16, or the bf16 state widened to fp32 ----
        if (a.final_state != nullptr) {
            if (a.state_fp32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.final_state) + st_off);
#pragma unroll 4
                for (int kc = 0; kc < 16; ++kc) {
                    const uint4 sv = *reinterpret_cast<const uint4*>(cs + kSmS + s_off(v, kc));
                    dst[2 * kc] = make_float4(bf_lo(sv.x), bf_hi(sv.x), bf_lo(sv.y), bf_hi(sv.y));
                    dst[2 * kc + 1] = make_float4(bf_lo(sv.z), bf_hi(sv.z), bf_lo(sv.w), bf_hi(sv.w));
                }
            } else {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.final_state) + st_off);
#pragma unroll 4
                for (int kc = 0; kc < 16; ++kc) dst[kc] = *reinterpret_cast<const uint4*>(cs + kSmS + s_off(v, kc));
            }
        }
        // all rows exported and all operand reads done before the next chain overwrites S / the stages
        named_barrier_sync(bar_id, 128);
    }

    if (failed) {
        ctl.abort_flag = 1;
        atomicExch(a.status, FKDA_ERR_DEVICE_STATUS);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

// ---------------------------------------------------------------------------------
size_t tc_workspace_bytes(int64_t T_total, int64_t H, int64_t N) {
    return kWsHeaderBytes + ws_prefix_bytes(N) +
           (size_t)H * (size_t)ws_tiles_upper_bound(T_total, N) * (size_t)kTcRecord;
}

int launch_tc(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches) {
    TwoPassArgs a;
    fill_args(p, &a);
    const bool varlen = p.cu_seqlens != nullptr;
    const bool do_prep = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_PREPARE);
    const bool do_rec = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_RECURRENCE);
    int launches = 0;
    if (cudaMemsetAsync(p.workspace, 0, 8, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;  // queue + status
    if (varlen && do_prep) {
        launch_tile_prefix(p.cu_seqlens, p.N, a.tile_prefix, stream);
        ++launches;
    }
    if (a.total_tiles > 0 && do_prep) {
        dim3 grid1((unsigned)a.total_tiles, (unsigned)p.H);
        prepare_kernel<true><<<grid1, 256, 0, stream>>>(a);
        ++launches;
    }
    if (do_rec) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return FKDA_ERR_LAUNCH;
        if (cudaFuncSetAttribute(recurrence_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) !=
            cudaSuccess)
            return FKDA_ERR_LAUNCH;
        const int64_t chains = p.N * p.H;
        int64_t ctas = (chains + kTcChains - 1) / kTcChains;
        if (ctas > sms) ctas = sms;
        if (ctas < 1) ctas = 1;
        recurrence_tc_kernel<<<(unsigned)ctas, kTcChains * 128, kTcSmemBytes, stream>>>(a);
        ++launches;
    }
    if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
    *n_launches = launches;
    return FKDA_OK;
}

}  // namespace fkda
