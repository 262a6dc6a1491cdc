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
//   * element-wise steps (bf16 roundings, beta, gate decay) by 256 threads per chain: two threads per
//     V row (= TMEM lane), each owning half of the tokens / half of the state columns, reading the
//     accumulators with tcgen05.ld.
// Three independent chains run per CTA (eight warps each) so that the tensor-core / barrier latency
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
// the stages of its 64th chunk into the workspace header (ints 16..).
#ifdef FKDA_TC_TIMING
#define TC_STAMP(i) do { if (stamp_on && t == 64) stamps[i] = clock64(); } while (0)
#else
#define TC_STAMP(i) do { } while (0)
#endif

constexpr int kTcChains = 3;          // chains per CTA
constexpr int kTcChainThreads = 256;  // threads per chain: 2 per V row
constexpr int kTcStages = 2;          // chunk records in flight per chain
constexpr int kTcTmemCols = 512;
constexpr uint32_t kTcWaitNs = 2000000000u;

// byte offsets inside one chain's shared-memory block
constexpr int kSmS = 0;                                       // state, canonical K-major A operand [128, 128]
constexpr int kSmStage = 32768;                               // kTcStages chunk records
constexpr int kSmStageBytes = kTcRecord;                      // 13888
constexpr int kSmA23 = kSmStage + kTcStages * kSmStageBytes;  // A operand of the 16-deep products [128, 16]
constexpr int kSmChainBytes = kSmA23 + 4096;                  // 64640
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

__global__ void __launch_bounds__(kTcChains * kTcChainThreads, 1) recurrence_tc_kernel(TwoPassArgs a) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 127) & ~(uintptr_t)127);
    TcCtrl& ctl = *reinterpret_cast<TcCtrl*>(smem + kTcChains * kSmChainBytes);

    // warp-uniform role indices (the shuffle makes the uniformity visible to the compiler, so the
    // single-thread tcgen05 issue below sits in warp-uniform control flow)
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int c = warp >> 3;           // chain slot
    const int wic = warp & 7;          // warp within the chain
    const int half = wic >> 2;         // which half of the tokens / state columns this thread owns
    const int v = threadIdx.x & 127;   // state row = TMEM lane
    uint8_t* cs = smem + c * kSmChainBytes;
    volatile int* abort_flag = &ctl.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kTcChains; ++i) {
            for (int s = 0; s < kTcStages; ++s) mbar_init(&ctl.full[i][s], 1);
            mbar_init(&ctl.mma[i], 1);
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
    // TMEM columns of chain c: DS at 128*c (128 wide; its first 16 columns also receive D2, which is
    // consumed before DS is written), D1 at 384 + 32*c (u0 in 0-15, o0 in 16-31; D3 later replaces u0)
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_ds = tmem_base + 128u * c;
    const uint32_t t_d1 = tmem_base + 384u + 32u * c;

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, false, false);
    constexpr uint32_t idesc_n16 = make_idesc_bf16_f32(128, 16, false, false);
    constexpr uint32_t idesc_ds = make_idesc_bf16_f32(128, 128, false, true);

    const uint32_t s_addr = smem_u32(cs + kSmS);
    const uint32_t a23_addr = smem_u32(cs + kSmA23);
    const uint64_t s_desc0 = make_smem_desc(s_addr, 2048, 128);  // + 256 per K step of 16 (4096 B >> 4)
    const uint64_t a23_desc = make_smem_desc(a23_addr, 2048, 128);
    uint8_t* const a23_mine = cs + kSmA23 + half * 2048 + (v >> 3) * 128 + (v & 7) * 16;
    const int bar_id = 1 + c;
    const int64_t n_chains = a.N * a.H;
    uint32_t full_phase[kTcStages] = {0, 0};
    uint32_t mma_phase = 0;
    bool failed = false;
#ifdef FKDA_TC_TIMING
    long long stamps[24] = {0};
#endif

    while (!failed) {
        // ---- next chain from the work queue ----
        if ((threadIdx.x & 255) == 0) ctl.next_chain[c] = atomicAdd(a.queue, 1);
        named_barrier_sync(bar_id, kTcChainThreads);
        const int64_t chain = ctl.next_chain[c];
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
        const int n_chunks = (int)((seq_len + kChunk - 1) / kChunk);
        const uint8_t* rec_base = a.workspace + ((int64_t)h * a.total_tiles + tile_base) * (int64_t)kTcRecord;
        // this thread's half row of the state: columns 64*half .. 64*half+63 of row v
        const int64_t st_off = (n * a.H + h) * (int64_t)(kD * kD) + (int64_t)v * kD + half * 64;

#ifdef FKDA_TC_TIMING
        const bool stamp_on = (chain == 0) && (threadIdx.x & 255) == 0;
#endif
        auto issue_load = [&](int t) {  // one thread: the record of chunk t into stage t % kTcStages
            const int s = t % kTcStages;
            mbar_arrive_expect_tx(&ctl.full[c][s], (uint32_t)kTcRecord);
            bulk_g2s(cs + kSmStage + s * kSmStageBytes, rec_base + (int64_t)t * kTcRecord, kTcRecord, &ctl.full[c][s]);
        };
        if ((threadIdx.x & 255) == 0) {
            for (int t = 0; t < kTcStages && t < n_chunks; ++t) issue_load(t);
        }
        // value column v of this thread's 8 tokens (8*half ..) of chunk t, fetched straight from global
        // memory one chunk ahead (64 contiguous bytes per warp and row); the raw 16-bit values are kept
        // apart until they are used, so the loads stay in flight
        const int64_t tstride = a.token_stride;
        const unsigned short* vcol = reinterpret_cast<const unsigned short*>(a.v) + (bos + 8 * half) * tstride +
                                     (int64_t)h * kD + v;
        unsigned short* ocol = reinterpret_cast<unsigned short*>(a.out) + (bos + 8 * half) * tstride +
                               (int64_t)h * kD + v;
        auto load_v = [&](int t, unsigned short (&dst)[8]) {
            const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)t * kChunk) - 8 * half;  // my valid rows
            const unsigned short* p = vcol + (int64_t)t * kChunk * tstride;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dst[i] = (i < len) ? __ldg(p) : (unsigned short)0;
                p += tstride;
            }
        };
        unsigned short v_cur[8], v_nxt[8];
        if (n_chunks > 0) load_v(0, v_cur);

        // ---- initial state into the canonical A-operand layout (fp32 rounded to bf16) ----
        if (a.initial_state != nullptr) {
            if (a.state_fp32) {
                const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.initial_state) + st_off);
#pragma unroll 4
                for (int q = 0; q < 8; ++q) {
                    const float4 x = src[2 * q], y = src[2 * q + 1];
                    *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, 8 * half + q)) =
                        make_uint4(pack_bf2(x.x, x.y), pack_bf2(x.z, x.w), pack_bf2(y.x, y.y), pack_bf2(y.z, y.w));
                }
            } else {
                const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.initial_state) + st_off);
#pragma unroll 4
                for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, 8 * half + q)) = src[q];
            }
        } else {
#pragma unroll 4
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, 8 * half + q)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        named_barrier_sync(bar_id, kTcChainThreads);

        // out rows of the previous chunk (this thread's 8 tokens), stored while the next chunk's first
        // MMA runs
        uint32_t o_pend[4];
        int o_pend_t = -1;
        auto flush_out = [&]() {
            if (o_pend_t < 0) return;
            const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)o_pend_t * kChunk) - 8 * half;
            unsigned short* dst = ocol + (int64_t)o_pend_t * kChunk * tstride;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (2 * i < len) *dst = (unsigned short)(o_pend[i] & 0xffffu);
                dst += tstride;
                if (2 * i + 1 < len) *dst = (unsigned short)(o_pend[i] >> 16);
                dst += tstride;
            }
            o_pend_t = -1;
        };

        for (int t = 0; t < n_chunks; ++t) {
            const int s = t % kTcStages;
            uint8_t* st = cs + kSmStage + s * kSmStageBytes;
            const uint32_t st_addr = smem_u32(st);

            TC_STAMP(8);
            // ---- operands of chunk t have landed ----
            if (!mbar_wait_bounded(&ctl.full[c][s], full_phase[s], abort_flag, kTcWaitNs)) { failed = true; break; }
            full_phase[s] ^= 1u;
            TC_STAMP(0);

            // ---- MMA1: D1[V,32] = S . [kd; qd]^T ----
            if (wic == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, 512, 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        umma_ss(t_d1, s_desc0 + (uint64_t)(j * 256), bd0 + (uint64_t)(j * 64), idesc_n32, j > 0 ? 1u : 0u);
                    umma_commit(&ctl.mma[c]);
                }
                __syncwarp();
            }
            TC_STAMP(1);
            // work off the critical path while the MMA runs
            flush_out();
            if (t + 1 < n_chunks) load_v(t + 1, v_nxt);
            uint32_t bpk[4];  // bf16x2 pairs of sigmoid(beta) for my 8 tokens (the record holds bf16-rounded values)
            {
                const float4* bp = reinterpret_cast<const float4*>(st + kTcBeta) + 2 * half;
                const float4 b0 = bp[0], b1 = bp[1];
                bpk[0] = pack_bf2(b0.x, b0.y); bpk[1] = pack_bf2(b0.z, b0.w);
                bpk[2] = pack_bf2(b1.x, b1.y); bpk[3] = pack_bf2(b1.z, b1.w);
            }
            if (!mbar_wait_bounded(&ctl.mma[c], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(2);

            // ---- u' = (v (-) bf(u0)) (*) bf(beta) for my 8 tokens -> my half of the A operand ----
            {
                uint32_t r[8];
                tmem_ld8(t_d1 + 8 * half + lane_sel, r);
                tmem_wait_ld();
                uint32_t up[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t u0 = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    const uint32_t vp = (uint32_t)v_cur[2 * i] | ((uint32_t)v_cur[2 * i + 1] << 16);
                    up[i] = bf2_mul(bf2_sub(vp, u0), bpk[i]);
                }
                *reinterpret_cast<uint4*>(a23_mine) = make_uint4(up[0], up[1], up[2], up[3]);
            }
            TC_STAMP(3);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, kTcChainThreads);
            TC_STAMP(4);

            // ---- MMA2: D2[V,16] = u'^T . INV^T  (into the first 16 DS columns) ----
            if (wic == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ss(t_ds, a23_desc, make_smem_desc(st_addr + kTcInv, 256, 128), idesc_n16, 0u);
                    umma_commit(&ctl.mma[c]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[c], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(5);
            {
                uint32_t r[8];
                tmem_ld8(t_ds + 8 * half + lane_sel, r);
                tmem_wait_ld();
                *reinterpret_cast<uint4*>(a23_mine) =
                    make_uint4(pack_bf2(__uint_as_float(r[0]), __uint_as_float(r[1])),
                               pack_bf2(__uint_as_float(r[2]), __uint_as_float(r[3])),
                               pack_bf2(__uint_as_float(r[4]), __uint_as_float(r[5])),
                               pack_bf2(__uint_as_float(r[6]), __uint_as_float(r[7])));
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, kTcChainThreads);
            TC_STAMP(6);

            // ---- MMA3: D3[V,16] = U^T . Mqk^T (over the dead u0 columns);  DS[V,K] = U^T . kr ----
            if (wic == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ss(t_d1, a23_desc, make_smem_desc(st_addr + kTcMqk, 256, 128), idesc_n16, 0u);
                    umma_ss(t_ds, a23_desc, make_smem_desc(st_addr + kTcKr, 2048, 128), idesc_ds, 0u);
                    umma_commit(&ctl.mma[c]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[c], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(7);

            // ---- my 64 state columns: S[v][k] = bf(fma(S[v][k], E_tot[k], DS[v][k])), TMEM loads one
            //      batch of 16 columns ahead; out = bf(o0) (+) bf(Mqk U) for my 8 tokens is formed here and
            //      stored while the next chunk's first MMA runs ----
            auto update_cols = [&](int b, const uint32_t (&r)[16]) {
                // all loads of the batch first: the stores below may alias them as far as the compiler knows
                const int kc0 = 8 * half + 2 * b;
                const float4* ep = reinterpret_cast<const float4*>(st + kTcEt) + 2 * kc0;
                uint4 sv[2];
                float4 e[4];
#pragma unroll
                for (int q = 0; q < 2; ++q) sv[q] = *reinterpret_cast<const uint4*>(cs + kSmS + s_off(v, kc0 + q));
#pragma unroll
                for (int q = 0; q < 4; ++q) e[q] = ep[q];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const float4 e0 = e[2 * q], e1 = e[2 * q + 1];
                    const uint32_t* rr = r + q * 8;
                    uint4 nv;
                    nv.x = pack_bf2(__fmaf_rn(bf_lo(sv[q].x), e0.x, __uint_as_float(rr[0])),
                                    __fmaf_rn(bf_hi(sv[q].x), e0.y, __uint_as_float(rr[1])));
                    nv.y = pack_bf2(__fmaf_rn(bf_lo(sv[q].y), e0.z, __uint_as_float(rr[2])),
                                    __fmaf_rn(bf_hi(sv[q].y), e0.w, __uint_as_float(rr[3])));
                    nv.z = pack_bf2(__fmaf_rn(bf_lo(sv[q].z), e1.x, __uint_as_float(rr[4])),
                                    __fmaf_rn(bf_hi(sv[q].z), e1.y, __uint_as_float(rr[5])));
                    nv.w = pack_bf2(__fmaf_rn(bf_lo(sv[q].w), e1.z, __uint_as_float(rr[6])),
                                    __fmaf_rn(bf_hi(sv[q].w), e1.w, __uint_as_float(rr[7])));
                    *reinterpret_cast<uint4*>(cs + kSmS + s_off(v, kc0 + q)) = nv;
                }
            };
            {
                uint32_t ra[16], rb[16], r3[8], ro[8];
                const uint32_t ds_mine = t_ds + 64 * half + lane_sel;
                tmem_ld16(ds_mine, ra);
                tmem_ld8(t_d1 + 8 * half + lane_sel, r3);
                tmem_ld8(t_d1 + 16 + 8 * half + lane_sel, ro);
                tmem_wait_ld();
                tmem_ld16(ds_mine + 16, rb);
                update_cols(0, ra);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    o_pend[i] = bf2_add(pack_bf2(__uint_as_float(ro[2 * i]), __uint_as_float(ro[2 * i + 1])),
                                        pack_bf2(__uint_as_float(r3[2 * i]), __uint_as_float(r3[2 * i + 1])));
                o_pend_t = t;
                tmem_wait_ld();
                tmem_ld16(ds_mine + 32, ra);
                update_cols(1, rb);
                tmem_wait_ld();
                tmem_ld16(ds_mine + 48, rb);
                update_cols(2, ra);
                tmem_wait_ld();
                update_cols(3, rb);
            }
            TC_STAMP(9);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, kTcChainThreads);
            TC_STAMP(10);

            // ---- refill the stage just consumed ----
            if ((threadIdx.x & 255) == 0 && t + kTcStages < n_chunks) issue_load(t + kTcStages);
#pragma unroll
            for (int i = 0; i < 8; ++i) v_cur[i] = v_nxt[i];
            TC_STAMP(11);
#ifdef FKDA_TC_TIMING
            if (stamp_on && t == 65) {
                stamps[12] = clock64();
                for (int i = 0; i < 13; ++i) a.status[15 + i] = (int)(stamps[i] - stamps[0]);
            }
#endif
        }
        if (failed) break;
        flush_out();

        // ---- final state (my 64 columns): bf16, or the bf16 state widened to fp32 ----
        if (a.final_state != nullptr) {
            if (a.state_fp32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.final_state) + st_off);
#pragma unroll 4
                for (int q = 0; q < 8; ++q) {
                    const uint4 sv = *reinterpret_cast<const uint4*>(cs + kSmS + s_off(v, 8 * half + q));
                    dst[2 * q] = make_float4(bf_lo(sv.x), bf_hi(sv.x), bf_lo(sv.y), bf_hi(sv.y));
                    dst[2 * q + 1] = make_float4(bf_lo(sv.z), bf_hi(sv.z), bf_lo(sv.w), bf_hi(sv.w));
                }
            } else {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.final_state) + st_off);
#pragma unroll 4
                for (int q = 0; q < 8; ++q) dst[q] = *reinterpret_cast<const uint4*>(cs + kSmS + s_off(v, 8 * half + q));
            }
        }
        // all rows exported and all operand reads done before the next chain overwrites S / the stages
        named_barrier_sync(bar_id, kTcChainThreads);
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
        recurrence_tc_kernel<<<(unsigned)ctas, kTcChains * kTcChainThreads, kTcSmemBytes, stream>>>(a);
        ++launches;
    }
    if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
    *n_launches = launches;
    return FKDA_OK;
}

}  // namespace fkda
