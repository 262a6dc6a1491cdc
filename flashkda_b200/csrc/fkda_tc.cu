// Tensor-core two-pass KDA forward for sm_100a: the token-parallel prepare kernel writes per-chunk
// operand records already laid out as tcgen05 (UMMA) shared-memory operands; a persistent
// recurrence kernel walks the chunks of each (sequence, head) chain with
//   * per chunk one bulk asynchronous copy of the record plus one tiled TMA load (tensor map) of the
//     [16,128] value tile, double buffered on mbarriers; out tiles leave through a tiled TMA store,
//   * all contractions on tcgen05.mma with fp32 accumulators in tensor memory (M = 128 always):
//        D1[V,32]   = S[V,K] . [kd; qd]^T         (8 x M128 N32 K16; A = S^T tile read MN-major)
//        D2[V,16]   = u'^T[V,16] . INV^T          (M128 N16 K16)
//        D3[V,16]   = U^T[V,16] . Mqk^T           (M128 N16 K16)
//        DST[K,V]   = kr^T[K,16] . U[16,V]        (M128 N128 K16; the state update, TRANSPOSED: lane = k)
//   * the bf16 state held twice: in the registers of its owner threads (thread k owns S[:,k], 64 packed
//     registers) for the element-wise update S[v,k] = bf(fma(S[v,k], E_tot[k], DST[k,v])) -- one gate
//     scalar per thread, no shared-memory reads -- and as the S^T tile in shared memory (written once
//     per chunk) that the next chunk's first MMA reads as its A operand,
//   * the other element-wise steps (bf16 roundings, beta) by the same 128 threads in the other
//     orientation (thread v = TMEM lane v of D1/D2/D3), reading accumulators with tcgen05.ld.
// Three independent chains run per CTA (one warpgroup each) so that the tensor-core / barrier latency
// of one chain is covered by the element-wise work of the others.
// The kernel of THIS file keeps the state copy and the 16-deep operands in shared memory; it is the
// FKDA_TC_SS=1 variant.  The default kernels live in their own files and share the helpers below:
// fkda_tc_ts.cuh (the same walk with every A operand in tensor memory: default for more chains than SMs) and
// fkda_tc_wide.cuh (one chain per CTA, for no more chains than SMs).
//
// Numerics: steps B1-B7 of the reference's contract (tests/torch_ref.py:231-251; the reference's own
// recurrence is csrc/smxx/fwd_kernel2.cuh:434-742, built on mma.sync with register transposes).
#include <cuda.h>
#include <stdlib.h>

#include <mutex>

#include "fkda_common.cuh"
#include "fkda_internal.h"
#include "fkda_prepare_warp.cuh"
#include "fkda_sm100.cuh"

namespace fkda {

using namespace sm100;

// Profiling aid (off by default): with -DFKDA_TC_TIMING thread 0 of CTA 0 stores clock64() deltas of
// the stages of its 64th chunk into the workspace header (ints 16..31).
#ifdef FKDA_TC_TIMING
#define TC_STAMP(i) do { if (stamp_on && t == 64) stamps[i] = clock64(); } while (0)
#else
#define TC_STAMP(i) do { } while (0)
#endif

constexpr int kTcChains = 3;    // chains (warpgroups) per CTA
constexpr int kTcStages = 2;    // chunk records in flight per chain
constexpr int kTcTmemCols = 512;
constexpr uint32_t kTcWaitNs = 2000000000u;

// byte offsets inside one chain's shared-memory block
constexpr int kSmS = 0;                                    // S^T tile: the state as MN-major A operand [v, k]
constexpr int kSmStage = 32768;                            // kTcStages chunk records
constexpr int kSmStageBytes = kTcRecord;                   // 14656
constexpr int kSmV = kSmStage + kTcStages * kSmStageBytes;    // kTcStages value tiles [16][128] bf16 (60544)
constexpr int kSmA23 = kSmV + kTcStages * 4096;               // A operand of the 16-deep products [128, 16]
constexpr int kSmOut = kSmA23;                                // out tile [16][128] bf16: reuses the A23 tile, which
                                                              // is dead between the chunk's last MMA and the next E1
constexpr int kSmChainBytes = kSmA23 + 4096;
static_assert(kSmV % 128 == 0 && kSmOut % 128 == 0, "TMA tiles are 128-byte aligned");
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

// S^T tile, MN-major canonical A operand [M = v, K = k]: elements (v..v+7, k) are the 16 bytes at
// (k/8)*2048 + (v/8)*128 + (k%8)*16
__device__ __forceinline__ int sT_off(int k, int vg) { return (k >> 3) * 2048 + vg * 128 + (k & 7) * 16; }

// Tensor maps over v and out viewed as [token][head][128] bf16 (box = 16 tokens x 1 head x 128).
struct alignas(64) TcMaps {
    CUtensorMap v, out;
};

// ---------------------------------------------------------------------------------
// Pieces shared by the recurrence kernels of this file and of fkda_tc_wide.cuh / fkda_tc_ts.cuh.

// Where the tokens and records of one (sequence, head) chain live.
struct TcChain {
    int64_t n;        // sequence
    int h;            // head
    int64_t bos;      // first token
    int64_t seq_len;
    int n_chunks;
    const uint8_t* rec_base;  // record of the chain's chunk 0
};
__device__ __forceinline__ TcChain tc_locate_chain(const TwoPassArgs& a, int64_t chain) {
    TcChain c;
    const int64_t s = chain / a.H;  // position in the order the chains are started in
    c.h = (int)(chain - s * a.H);
    c.n = a.seq_order != nullptr ? a.seq_order[s] : s;
    int64_t tile_base;
    if (a.cu_seqlens != nullptr) {
        c.bos = a.cu_seqlens[c.n];
        c.seq_len = a.cu_seqlens[c.n + 1] - c.bos;
        if (c.seq_len < 0) c.seq_len = 0;
        tile_base = a.tile_prefix[c.n];
    } else {
        c.bos = c.n * a.T;
        c.seq_len = a.T;
        tile_base = c.n * ((a.T + kChunk - 1) / kChunk);
    }
    c.n_chunks = (int)((c.seq_len + kChunk - 1) / kChunk);
    c.rec_base = a.workspace + ((int64_t)c.h * a.total_tiles + tile_base) * (int64_t)kTcRecord;
    return c;
}

// Next work item of a chain slot (called by ONE thread).  An item is one segment (seg_chunks chunks) of one
// chain; item id = seg * n_chains + chain.  Tickets below n_chains are the first segments; every later ticket
// reads the slot that the finisher of some segment fills with the follow-up segment, so chains take turns on
// the chain slots (first come, first served) and more chains than slots still share the machine evenly.
// The first ticket of a chain slot is static, the chain slots of all CTAs filled one layer at a time (so that
// few chains spread over the SMs instead of crowding the first CTAs); later tickets are first come.
// Returns the item, -2 when all chains are finished, -3 when the bounded wait gave up.
__device__ __forceinline__ int tc_next_item(const TwoPassArgs& a, bool first_ticket, int wg, int64_t n_chains,
                                            volatile int* abort_flag) {
    // (odd layers run backwards over the CTAs: with chains ordered by decreasing length the longest chains of one
    //  layer meet the shortest of the next)
    const int cta = (wg & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const int ticket = first_ticket ? wg * (int)gridDim.x + cta
                                    : kTcChains * (int)gridDim.x + atomicAdd(a.queue, 1);
    if (ticket < n_chains) return ticket;
    int item = -2;
    if (a.seg_chunks > 0) {
        volatile int32_t* slot = a.qslots + (ticket - (int)n_chains);
        volatile int32_t* finished = a.queue + 3;
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        for (;;) {
            const int x = *slot;
            if (x >= 0) { item = x; break; }
            if (*finished >= (int)n_chains) break;
            if ((++spins & 63u) == 0 && (*abort_flag != 0 || global_timer_ns() - t0 > kTcWaitNs)) { item = -3; break; }
            __nanosleep(200);
        }
        __threadfence();  // the pusher's state stores are visible before we read them
    }
    return item;
}
// The finisher of a non-final segment queues the follow-up segment (ONE thread, after the state hand-over
// stores of all threads have been fenced and a barrier has passed).
__device__ __forceinline__ void tc_push_followup(const TwoPassArgs& a, int item, int64_t n_chains) {
    const int pos = atomicAdd(a.queue + 2, 1);
    __threadfence();
    *reinterpret_cast<volatile int32_t*>(a.qslots + pos) = item + (int)n_chains;
}

// sigmoid(beta) of the 16 rows as bf16x2 pairs (the record holds them as 16 bf16 values)
__device__ __forceinline__ void tc_load_beta(const uint8_t* rec, uint32_t (&bpk)[8]) {
    const uint4* bp = reinterpret_cast<const uint4*>(rec + kTcBeta);
    const uint4 x = bp[0], y = bp[1];
    bpk[0] = x.x; bpk[1] = x.y; bpk[2] = x.z; bpk[3] = x.w;
    bpk[4] = y.x; bpk[5] = y.y; bpk[6] = y.z; bpk[7] = y.w;
}
// value column v of the chunk from the [16][128] tile (zero past the sequence end)
__device__ __forceinline__ void tc_load_v_column(const uint8_t* v_tile, int v, int len, unsigned short (&v_cur)[kChunk]) {
    const unsigned short* vt = reinterpret_cast<const unsigned short*>(v_tile) + v;
    if (len == kChunk) {  // the common case without per-row masks
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v_cur[i] = vt[i * kD];
    } else {
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v_cur[i] = (i < len) ? vt[i * kD] : (unsigned short)0;
    }
}
// Row v of a [128, 16] K-major operand tile (the A operand of the 16-deep products): two 16-byte pieces.
__device__ __forceinline__ void tc_store_a23_row(uint8_t* a23, int v, const uint32_t (&p)[8]) {
    uint8_t* ap = a23 + (v >> 3) * 128 + (v & 7) * 16;
    *reinterpret_cast<uint4*>(ap) = make_uint4(p[0], p[1], p[2], p[3]);
    *reinterpret_cast<uint4*>(ap + 2048) = make_uint4(p[4], p[5], p[6], p[7]);
}
// u' = (v (-) bf(u0)) (*) bf(beta) for V row v, from the u0 accumulators in tensor memory, into the A tile
__device__ __forceinline__ void tc_form_u_prime(uint32_t t_u0_lane, uint8_t* a23, int v,
                                                const unsigned short (&v_cur)[kChunk], const uint32_t (&bpk)[8]) {
    uint32_t r[16];
    tmem_ld16(t_u0_lane, r);
    tmem_wait_ld();
    uint32_t up[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t u0 = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        const uint32_t vp = (uint32_t)v_cur[2 * i] | ((uint32_t)v_cur[2 * i + 1] << 16);
        up[i] = bf2_mul(bf2_sub(vp, u0), bpk[i]);
    }
    tc_store_a23_row(a23, v, up);
}
// U = bf(D2) for V row v into the A tile
__device__ __forceinline__ void tc_form_u(uint32_t t_d2_lane, uint8_t* a23, int v) {
    uint32_t r[16];
    tmem_ld16(t_d2_lane, r);
    tmem_wait_ld();
    uint32_t p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    tc_store_a23_row(a23, v, p);
}
// out = bf(o0) (+) bf(Mqk U) for V row v; r holds D3 in 0-15 and o0 in 16-31.  Full chunks go through the out
// tile (one TMA store later), ragged tails straight to global memory, valid rows only.
__device__ __forceinline__ void tc_store_out(const uint32_t (&r)[32], unsigned short* out_tile, unsigned short* out_global,
                                             int64_t tstride, int v, int len) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t o = bf2_add(pack_bf2(__uint_as_float(r[16 + 2 * i]), __uint_as_float(r[16 + 2 * i + 1])),
                                   pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
        if (len == kChunk) {
            out_tile[(2 * i) * kD + v] = (unsigned short)(o & 0xffffu);
            out_tile[(2 * i + 1) * kD + v] = (unsigned short)(o >> 16);
        } else {
            unsigned short* dst = out_global + (int64_t)(2 * i) * tstride;
            if (2 * i < len) dst[0] = (unsigned short)(o & 0xffffu);
            if (2 * i + 1 < len) dst[tstride] = (unsigned short)(o >> 16);
        }
    }
}

__global__ void __launch_bounds__(kTcChains * 128, 1)
recurrence_tc_kernel(const __grid_constant__ TwoPassArgs a, const __grid_constant__ TcMaps maps) {
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
    // columns: DST of chain c at 128*c (128 wide; its first 16 columns also receive D2, which is consumed
    // before DST is written), D1 at 384 + 32*c (u0 in 0-15, o0 in 16-31; D3 later replaces u0)
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_ds = tmem_base + 128u * wg;
    const uint32_t t_d1 = tmem_base + 384u + 32u * wg;

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, true, false);    // A = S^T tile, MN-major
    constexpr uint32_t idesc_n16 = make_idesc_bf16_f32(128, 16, false, false);
    constexpr uint32_t idesc_dst = make_idesc_bf16_f32(128, 128, true, false);   // A = kr tile, MN-major

    const uint32_t s_addr = smem_u32(cs + kSmS);
    const uint32_t a23_addr = smem_u32(cs + kSmA23);
    const uint64_t s_desc0 = make_smem_desc(s_addr, 2048, 128);      // LBO: k groups, SBO: v groups; + 256 per K step
    const uint64_t a23_desc = make_smem_desc(a23_addr, 2048, 128);
    const int bar_id = 1 + wg;
    const int64_t n_chains = a.N * a.H;
    uint32_t full_phase[kTcStages] = {0, 0};
    uint32_t mma_phase = 0;
    bool failed = false;
    bool first_ticket = true;
#ifdef FKDA_TC_TIMING
    long long stamps[24] = {0};
#endif

    while (!failed) {
        // ---- next work item (a segment of a chain) ----
        if (v == 0) ctl.next_chain[wg] = tc_next_item(a, first_ticket, wg, n_chains, abort_flag);
        first_ticket = false;
        named_barrier_sync(bar_id, 128);
        const int item = ctl.next_chain[wg];
        if (item == -3) { failed = true; break; }
        if (item < 0) break;
        const int seg = item / (int)n_chains;
        const int64_t chain = item - (int64_t)seg * n_chains;
        const TcChain ch = tc_locate_chain(a, chain);
        const int64_t n = ch.n, bos = ch.bos, seq_len = ch.seq_len;
        const int h = ch.h, n_chunks = ch.n_chunks;
        const int c0 = seg * a.seg_chunks;                                             // my chunk range
        const int c1 = (a.seg_chunks > 0 && c0 + a.seg_chunks < n_chunks) ? c0 + a.seg_chunks : n_chunks;
        const uint8_t* rec_base = ch.rec_base;
        // thread k = v owns state column k: element S[vv][k] of this chain sits at st_base + vv * 128
        const int64_t st_base = (n * a.H + h) * (int64_t)(kD * kD) + v;
#ifdef FKDA_TC_TIMING
        const bool stamp_on = (chain == 0) && v == 0;
#endif

        auto issue_load = [&](int t) {  // one thread: the record of chunk t into stage t % kTcStages
            const int s = t % kTcStages;
            mbar_arrive_expect_tx(&ctl.full[wg][s], (uint32_t)(kTcRecord + kChunk * kD * 2));
            bulk_g2s(cs + kSmStage + s * kSmStageBytes, rec_base + (int64_t)t * kTcRecord, kTcRecord, &ctl.full[wg][s]);
            // rows past the end of the tensor arrive as zeros; rows of the next sequence are never used
            tma_load_3d(cs + kSmV + s * 4096, &maps.v, 0, h, (int)(bos + (int64_t)t * kChunk), &ctl.full[wg][s]);
        };
        if (v == 0) {
            for (int t = c0; t < c0 + kTcStages && t < c1; ++t) issue_load(t);
        }
        const int64_t tstride = a.token_stride;
        unsigned short* ocol = reinterpret_cast<unsigned short*>(a.out) + bos * tstride + (int64_t)h * kD + v;

        // ---- initial state: column k of S into registers (pairs over v) and into the S^T tile ----
        uint32_t sreg[64];
        uint4* const seg_mine = reinterpret_cast<uint4*>(a.seg_state) + (chain * 16) * 128 + v;  // + i * 128
        if (seg > 0) {  // handed over by the previous segment (another SM wrote it: bypass L1)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint4 x = __ldcg(seg_mine + i * 128);
                sreg[4 * i] = x.x; sreg[4 * i + 1] = x.y; sreg[4 * i + 2] = x.z; sreg[4 * i + 3] = x.w;
            }
        } else if (a.initial_state != nullptr) {
            if (a.state_fp32) {
                const float* src = reinterpret_cast<const float*>(a.initial_state) + st_base;
#pragma unroll
                for (int i = 0; i < 64; ++i) sreg[i] = pack_bf2(src[(2 * i) * kD], src[(2 * i + 1) * kD]);
            } else {
                const unsigned short* src = reinterpret_cast<const unsigned short*>(a.initial_state) + st_base;
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    sreg[i] = (uint32_t)src[(2 * i) * kD] | ((uint32_t)src[(2 * i + 1) * kD] << 16);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) sreg[i] = 0u;
        }
#pragma unroll
        for (int vg = 0; vg < 16; ++vg)
            *reinterpret_cast<uint4*>(cs + kSmS + sT_off(v, vg)) =
                make_uint4(sreg[4 * vg], sreg[4 * vg + 1], sreg[4 * vg + 2], sreg[4 * vg + 3]);
        fence_proxy_async_smem();
        named_barrier_sync(bar_id, 128);

        __nv_bfloat16* out_tile = reinterpret_cast<__nv_bfloat16*>(cs + kSmOut);

        for (int t = c0; t < c1; ++t) {
            const int s = t % kTcStages;
            uint8_t* st = cs + kSmStage + s * kSmStageBytes;
            const uint32_t st_addr = smem_u32(st);

            TC_STAMP(8);
            // ---- operands of chunk t have landed ----
            if (!mbar_wait_bounded(&ctl.full[wg][s], full_phase[s], abort_flag, kTcWaitNs)) { failed = true; break; }
            full_phase[s] ^= 1u;
            TC_STAMP(0);

            // ---- MMA1: D1[V,32] = S . [kd; qd]^T ----
            if (wiw == 0) {
                if (elect_one()) {
                    // the previous out tile shares the A23 tile: its TMA store must have read it before anybody
                    // (released by this MMA's completion) writes u' there
                    bulk_wait_group_read<0>();
                    tc_fence_after_sync();
                    const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, kTcB1Lbo, 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        umma_ss(t_d1, s_desc0 + (uint64_t)(j * 256), bd0 + (uint64_t)(j * (2 * kTcB1Lbo / 16)), idesc_n32, j > 0 ? 1u : 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            TC_STAMP(1);
            // work off the critical path while the MMA runs
            const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)t * kChunk);
            unsigned short v_cur[kChunk];  // value column v of this chunk (zero past the sequence end)
            tc_load_v_column(cs + kSmV + s * 4096, v, len, v_cur);
            const float e_mine = reinterpret_cast<const float*>(st + kTcEt)[v];  // gate decay of my state column
            uint32_t bpk[8];  // bf16x2 pairs of sigmoid(beta)
            tc_load_beta(st, bpk);
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(2);

            // ---- u' = (v (-) bf(u0)) (*) bf(beta) -> A operand (thread = V row) ----
            tc_form_u_prime(t_d1 + lane_sel, cs + kSmA23, v, v_cur, bpk);
            TC_STAMP(3);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);
            TC_STAMP(4);

            // ---- MMA2: D2[V,16] = u'^T . INV^T  (into the first 16 DST columns) ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ss(t_ds, a23_desc, make_smem_desc(st_addr + kTcInv, 256, 128), idesc_n16, 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(5);
            tc_form_u(t_ds + lane_sel, cs + kSmA23, v);  // U = bf(D2)
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);
            TC_STAMP(6);

            // ---- MMA3: D3[V,16] = U^T . Mqk^T (over the dead u0 columns);  DST[K,V] = kr^T . U ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ss(t_d1, a23_desc, make_smem_desc(st_addr + kTcMqk, 256, 128), idesc_n16, 0u);
                    umma_ss(t_ds, make_smem_desc(st_addr + kTcKr, kTcKrLbo, kTcKrSbo), a23_desc, idesc_dst, 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();
            TC_STAMP(7);

            // ---- out = bf(o0) (+) bf(Mqk U) (thread = V row); the TMEM loads of the state update that
            //      follows are kept one batch of 16 columns ahead of the arithmetic ----
            uint32_t ra[16], rb[16];
            {
                uint32_t r[32];
                tmem_ld32(t_d1 + lane_sel, r);  // D3 in 0-15, o0 in 16-31
                tmem_ld16(t_ds + lane_sel, ra);
                tmem_wait_ld();
                tmem_ld16(t_ds + 16 + lane_sel, rb);
                tc_store_out(r, reinterpret_cast<unsigned short*>(out_tile), ocol + (int64_t)t * kChunk * tstride, tstride, v, len);
            }
            // ---- state column k (thread = TMEM lane k of DST): S[vv][k] = bf(fma(S[vv][k], E_tot[k], DST[k][vv])),
            //      registers only; the refreshed column also goes to the S^T tile for the next chunk's MMA1 ----
            auto update16 = [&](int b, const uint32_t (&r)[16]) {  // rows vv = 16b .. 16b+15
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t sv = sreg[8 * b + i];
                    sreg[8 * b + i] = pack_bf2(__fmaf_rn(bf_lo(sv), e_mine, __uint_as_float(r[2 * i])),
                                               __fmaf_rn(bf_hi(sv), e_mine, __uint_as_float(r[2 * i + 1])));
                }
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    *reinterpret_cast<uint4*>(cs + kSmS + sT_off(v, 2 * b + q)) =
                        make_uint4(sreg[8 * b + 4 * q], sreg[8 * b + 4 * q + 1], sreg[8 * b + 4 * q + 2],
                                   sreg[8 * b + 4 * q + 3]);
            };
#pragma unroll
            for (int b = 0; b < 8; b += 2) {
                update16(b, ra);
                tmem_wait_ld();
                if (b + 2 < 8) tmem_ld16(t_ds + 16 * (b + 2) + lane_sel, ra);
                update16(b + 1, rb);
                if (b + 2 < 8) {
                    tmem_wait_ld();
                    tmem_ld16(t_ds + 16 * (b + 3) + lane_sel, rb);
                }
            }
            TC_STAMP(9);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);
            TC_STAMP(10);

            // ---- store the out tile, refill the stage just consumed ----
            if (wiw == 0) {
                if (elect_one()) {
                    if (len == kChunk) {
                        tma_store_3d(&maps.out, 0, h, (int)(bos + (int64_t)t * kChunk), out_tile);
                        bulk_commit_group();
                    }
                    if (t + kTcStages < c1) issue_load(t + kTcStages);
                }
                __syncwarp();
            }
            TC_STAMP(11);
#ifdef FKDA_TC_TIMING
            if (stamp_on && t == 65) {
                stamps[12] = clock64();
                for (int i = 0; i < 13; ++i) a.status[15 + i] = (int)(stamps[i] - stamps[0]);
            }
#endif
        }
        if (failed) break;

        if (c1 < n_chunks) {
            // ---- not the last segment: hand the state over and queue the follow-up segment ----
#pragma unroll
            for (int i = 0; i < 16; ++i)
                seg_mine[i * 128] = make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
            __threadfence();
            named_barrier_sync(bar_id, 128);
            if (v == 0) tc_push_followup(a, item, n_chains);
            continue;
        }
        if (v == 0) atomicAdd(a.queue + 3, 1);  // this chain is finished
        // ---- final state: my column, bf16 or widened to fp32 ----
        if (a.final_state != nullptr) {
            if (a.state_fp32) {
                float* dst = reinterpret_cast<float*>(a.final_state) + st_base;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    dst[(2 * i) * kD] = bf_lo(sreg[i]);
                    dst[(2 * i + 1) * kD] = bf_hi(sreg[i]);
                }
            } else {
                unsigned short* dst = reinterpret_cast<unsigned short*>(a.final_state) + st_base;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    dst[(2 * i) * kD] = (unsigned short)(sreg[i] & 0xffffu);
                    dst[(2 * i + 1) * kD] = (unsigned short)(sreg[i] >> 16);
                }
            }
        }
        // all operand reads done before the next chain overwrites the S^T tile / the stages
        named_barrier_sync(bar_id, 128);
    }

    if (failed) {
        ctl.abort_flag = 1;
        atomicExch(a.status, FKDA_ERR_DEVICE_STATUS);
    }
    bulk_wait_group<0>();  // (the store-issuing lanes) out tiles fully written
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

}  // namespace fkda

#include "fkda_tc_ts.cuh"
#include "fkda_tc_wide.cuh"

namespace fkda {

// ---------------------------------------------------------------------------------
// Segment scheduling is used when there are more chains than a B200 can hold at once (3 per SM);
// with fewer chains every chain has its own slot and whole chains are the work items.
constexpr int64_t kSegThresholdChains = 148 * kTcChains;  // every chain has its own chain slot up to here
constexpr int kSegChunksMax = 64, kSegChunksMin = 16;
// Segment length: 64 chunks when there is plenty of work (the hand-over of a 32 KB state costs about one chunk
// step), shorter when the whole problem is only a few segments per chain slot, so that 512 chains of 64 chunks
// do not run as one full round plus a nearly empty one.  Even, so that the double-buffer parity of a segment's
// first chunk is fixed.  A function of (T_total, H, N) only: the workspace is sized with the same value.
// Tuning aid: $FKDA_SEG_CHUNKS overrides it (read once per process).
static int seg_chunks_for(int64_t T_total, int64_t H, int64_t N) {
    static int forced = -1;
    if (forced < 0) {
        forced = 0;
        if (const char* e = getenv("FKDA_SEG_CHUNKS")) {
            const int x = atoi(e) / 2 * 2;
            if (x >= 2) forced = x;
        }
    }
    if (forced > 0) return forced;
    const int64_t chain_slots = 148 * kTcChains;
    int64_t seg = H * ws_tiles_upper_bound(T_total, N) / (4 * chain_slots);  // aim at >= 4 segments per chain slot
    seg = seg / 2 * 2;
    if (seg > kSegChunksMax) seg = kSegChunksMax;
    if (seg < kSegChunksMin) seg = kSegChunksMin;
    return (int)seg;
}
static bool use_segments(int64_t H, int64_t N) { return H * N > kSegThresholdChains; }
static size_t seg_slot_count(int64_t T_total, int64_t H, int64_t N) {
    // one push per segment after the first of each chain, plus one ticket per resident warpgroup at the end
    return (size_t)(H * (ws_tiles_upper_bound(T_total, N) / seg_chunks_for(T_total, H, N) + N) + 4096);
}
static size_t seg_slots_bytes(int64_t T_total, int64_t H, int64_t N) {
    return use_segments(H, N) ? (seg_slot_count(T_total, H, N) * 4 + 255) / 256 * 256 : 0;
}
// hand-over states (32 KB per chain): between the segments of the work queue, or between the slabs of a
// pipelined forward
static size_t seg_state_bytes(int64_t H, int64_t N) { return (size_t)(H * N) * 32768; }

// Side stream and events of the slab pipeline, one set per device, created on first use.
constexpr int kMaxSlabs = 4;
struct SlabStreams {
    std::mutex launch_mu;  // one slab pipeline at a time is ENQUEUED per device (event record / wait pairs stay paired)
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, done[kMaxSlabs] = {nullptr, nullptr, nullptr, nullptr};
    bool ready = false;
};
static SlabStreams* slab_streams(int dev) {
    static std::mutex mu;
    static SlabStreams table[64];
    if (dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    SlabStreams& t = table[dev];
    if (!t.ready) {
        if (cudaStreamCreateWithFlags(&t.side, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        for (int i = 0; i < kMaxSlabs; ++i)
            if (cudaEventCreateWithFlags(&t.done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
        t.ready = true;
    }
    return &t;
}

size_t tc_workspace_bytes(int64_t T_total, int64_t H, int64_t N) {
    return kWsHeaderBytes + ws_prefix_bytes(N) + seg_slots_bytes(T_total, H, N) + seg_state_bytes(H, N) +
           (size_t)H * (size_t)ws_tiles_upper_bound(T_total, N) * (size_t)kTcRecord;
}

// The driver entry point is looked up through the runtime (no link-time dependency on libcuda, so
// the library also loads on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

static bool encode_token_map(CUtensorMap* m, const void* base, int64_t T_total, int64_t H, int64_t token_stride) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)H, (cuuint64_t)(T_total > 0 ? T_total : 1)};
    const cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)token_stride * 2};  // bytes, dims 1 and 2
    const cuuint32_t box[3] = {(cuuint32_t)kD, 1u, (cuuint32_t)kChunk};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_tc(const fkda_fwd_params& p, cudaStream_t stream, int* n_launches) {
    TwoPassArgs a;
    fill_args(p, &a);
    const bool varlen = p.cu_seqlens != nullptr;
    const bool do_prep = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_PREPARE);
    const bool do_rec = p.phase_mask == 0 || (p.phase_mask & FKDA_PHASE_RECURRENCE);
    int launches = 0;
    if (cudaMemsetAsync(p.workspace, 0, 16, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;  // header counters
    {   // carve the segment queue and the hand-over states in front of the records
        const int64_t T_total = p.B * p.T;
        uint8_t* base = reinterpret_cast<uint8_t*>(p.workspace) + kWsHeaderBytes + ws_prefix_bytes(p.N);
        const size_t slots = seg_slots_bytes(T_total, p.H, p.N), states = seg_state_bytes(p.H, p.N);
        if (use_segments(p.H, p.N)) {
            a.qslots = reinterpret_cast<int32_t*>(base);
            a.seg_state = reinterpret_cast<uint32_t*>(base + slots);
            a.seg_chunks = seg_chunks_for(T_total, p.H, p.N);
            if (do_rec && cudaMemsetAsync(a.qslots, 0xff, slots, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;
        }
        a.seg_state = reinterpret_cast<uint32_t*>(base + slots);
        a.workspace = base + slots + states;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return FKDA_ERR_LAUNCH;
    const int64_t chains = p.N * p.H;
    const bool wide = chains <= sms && getenv("FKDA_TC_NO_WIDE") == nullptr;  // (the switch is a tuning aid)
    TcMaps maps;
    if (do_rec && (!encode_token_map(&maps.v, p.v, p.B * p.T, p.H, p.token_stride) ||
                   !encode_token_map(&maps.out, p.out, p.B * p.T, p.H, p.token_stride)))
        return FKDA_ERR_LAUNCH;
    const int wide_smem = kWideCtrlOff + (int)sizeof(TcWideCtrl) + 128;
    if (do_rec && wide &&
        cudaFuncSetAttribute(recurrence_tc_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide_smem) != cudaSuccess)
        return FKDA_ERR_LAUNCH;

    // ---- few chains on a fixed batch: the recurrence is a serial walk on `chains` SMs and leaves the others
    //      idle, so the forward is cut into slabs of chunks and the prepare stage of slab i+1 runs on the idle SMs
    //      (side stream) while the recurrence walks slab i; the state of a chain travels through seg_state.
    //      Only stream order and events connect the launches: no kernel waits for another one. ----
    const int64_t tps = (p.T + kChunk - 1) / kChunk;
    const int idle_sms = sms - (int)chains;
    if (wide && !varlen && p.phase_mask == 0 && idle_sms >= 32 && tps >= 64 && getenv("FKDA_TC_NO_SLABS") == nullptr) {
        SlabStreams* ss = slab_streams(dev);
        if (ss == nullptr) return FKDA_ERR_LAUNCH;
        // host threads that call concurrently on one device share the side stream and its events
        std::lock_guard<std::mutex> enqueue_lock(ss->launch_mu);
        // Slab boundaries.  The prepare of slab i+1 (on idle_sms SMs, about 5.2 ns per (chunk, head) on the whole
        // GPU) must be done when the recurrence (about 1.18 us per chunk) has walked slab i.  When prepare is at
        // least twice as fast (x <= 0.5) the slabs grow, 1/8, 1/4, 5/16, 5/16 of the chunks (1/3, 2/3 for two), so
        // that little prepare work goes first, unhidden; otherwise they are equal.
        const int n_slabs = tps >= 256 ? kMaxSlabs : 2;
        const double x = (double)chains * (double)sms / ((double)idle_sms * 227.0);
        static const double grow4[kMaxSlabs + 1] = {0.0, 0.125, 0.375, 0.6875, 1.0}, grow2[3] = {0.0, 1.0 / 3.0, 1.0};
        int bounds[kMaxSlabs + 1];
        for (int i = 0; i <= n_slabs; ++i) {
            const double frac = x <= 0.5 ? (n_slabs == 2 ? grow2[i] : grow4[i]) : (double)i / n_slabs;
            bounds[i] = (int)((int64_t)(frac * (double)tps + 1.0) / 2 * 2);  // even
        }
        bounds[0] = 0;
        bounds[n_slabs] = (int)tps;
        auto slab_args = [&](int i) {
            TwoPassArgs x = a;
            x.slab_c0 = bounds[i];
            x.slab_chunks = bounds[i + 1] - bounds[i];
            return x;
        };
        if (launch_prepare_warp<true>(slab_args(0), stream) != FKDA_OK) return FKDA_ERR_LAUNCH;
        ++launches;
        if (cudaEventRecord(ss->fork, stream) != cudaSuccess || cudaStreamWaitEvent(ss->side, ss->fork, 0) != cudaSuccess)
            return FKDA_ERR_LAUNCH;
        for (int i = 1; i < n_slabs; ++i) {
            if (bounds[i + 1] <= bounds[i]) continue;
            if (launch_prepare_warp<true>(slab_args(i), ss->side, idle_sms) != FKDA_OK) return FKDA_ERR_LAUNCH;
            ++launches;
            if (cudaEventRecord(ss->done[i], ss->side) != cudaSuccess) return FKDA_ERR_LAUNCH;
        }
        for (int i = 0; i < n_slabs; ++i) {
            if (bounds[i + 1] <= bounds[i]) continue;
            if (i > 0 && cudaStreamWaitEvent(stream, ss->done[i], 0) != cudaSuccess) return FKDA_ERR_LAUNCH;
            recurrence_tc_wide_kernel<<<(unsigned)chains, 384, wide_smem, stream>>>(slab_args(i), maps);
            ++launches;
        }
        if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
        *n_launches = launches;
        return FKDA_OK;
    }

    if (varlen && do_prep) {
        launch_tile_prefix(p.cu_seqlens, p.N, a.tile_prefix, const_cast<int32_t*>(a.seq_order), stream);
        ++launches;
    }
    if (a.total_tiles > 0 && do_prep) {
        if (launch_prepare_warp<true>(a, stream) != FKDA_OK) return FKDA_ERR_LAUNCH;
        ++launches;
    }
    if (do_rec) {
        int64_t ctas = chains;  // one chain per SM while they last, then two, then three
        if (ctas > sms) ctas = sms;
        if (ctas < 1) ctas = 1;
        if (wide) {
            // few chains: one per CTA, the idle warpgroups help with the state update
            recurrence_tc_wide_kernel<<<(unsigned)ctas, 384, wide_smem, stream>>>(a, maps);
        } else if (getenv("FKDA_TC_SS") != nullptr) {
            // the variant that keeps the state's MMA copy and the 16-deep operands in shared memory
            if (cudaFuncSetAttribute(recurrence_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) !=
                cudaSuccess)
                return FKDA_ERR_LAUNCH;
            recurrence_tc_kernel<<<(unsigned)ctas, kTcChains * 128, kTcSmemBytes, stream>>>(a, maps);
        } else {
            // default: state copy and 16-deep A operands in tensor memory
            if (cudaFuncSetAttribute(recurrence_tc_ts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTsSmemBytes) !=
                cudaSuccess)
                return FKDA_ERR_LAUNCH;
            recurrence_tc_ts_kernel<<<(unsigned)ctas, kTcChains * 128, kTsSmemBytes, stream>>>(a, maps);
        }
        ++launches;
    }
    if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
    *n_launches = launches;
    return FKDA_OK;
}

}  // namespace fkda
