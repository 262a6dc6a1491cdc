// "Wide" variant of the tensor-core recurrence for the few-chains regime (no more chains than SMs): ONE chain per
// CTA, laid out for the shortest possible chunk step, because here the forward is a serial walk and its time is
// (number of chunks) x (latency of one step).
//
// Roles (13 warps):
//   * warpgroup 0 (warps 0-3) runs the element-wise part of a chunk (u', U, out) and owns no state;
//   * warpgroups 1, 2 (warps 4-11) own the state: thread v of warpgroup 1 keeps S[v, 0..63] in registers, thread v
//     of warpgroup 2 S[v, 64..127] (four batches of 16 columns each), apply the update
//     S[v,k] = bf(fma(S[v,k], E_tot[k], DST[v,k])) and write the refreshed bf16 pairs to the tensor-memory copy
//     that the next chunk's first product reads;
//   * warp 12, the control warp: one thread issues every tcgen05.mma, the TMA loads of the operand stages and the
//     TMA stores of the out tiles.  The other warps tell it what is ready through mbarriers, so no warpgroup ever
//     stops at a CTA barrier inside a chunk.
//
// What keeps the step short (cycle stamps on a B200: about 1 600 cycles from one chunk's D1 to the next's):
//   * the two 16-deep products, U = bf(u' INV^T) on the chain and the out term U Mqk^T beside it, run on mma.sync
//     inside warpgroup 0: the accumulators of D1 are read from tensor memory in the 16x256b shape, which IS the
//     mma.sync fragment layout, and U goes back to tensor memory with a 16x128b store as the A operand of the
//     update product.  That is one tcgen05 round trip and one barrier less per chunk than three tcgen05 products
//     in a row; the out term is computed while U's tensor-memory store is in flight;
//   * a tensor-memory store takes about 180 cycles to complete, so the state owners store their four batches
//     back to back and wait once; each half of the state is then announced on its own mbarrier and the control
//     thread issues the K steps of the next chunk's first product, D1 = S . [kd; qd]^T, half by half;
//   * warpgroup 0 holds no state columns, so nothing on the chain waits for the out tile;
//   * five operand stages, refilled by the control warp as soon as a chunk's last reader is done: the records
//     come from HBM, about a chunk step away, so the look-ahead has to be several chunks deep.
//
// Tensor memory (256 columns): DST [0,128), D1 = u0 | o0 [128,160), bf16 state copy [160,224), U^T [224,232).
// Same numerics, record format and results as recurrence_tc_ts_kernel.  Included by fkda_tc.cu.
#pragma once

namespace fkda {

constexpr int kWideStages = 5;   // operands come from HBM (about a microsecond away): four chunks of look-ahead
constexpr int kWideThreads = 13 * 32;
constexpr int kWideStageOff = 0;                                                       // kWideStages chunk records
constexpr int kWideV = (kWideStages * kTcStageBytes + 127) / 128 * 128;                // kWideStages value tiles
constexpr int kWideOut = kWideV + kWideStages * 4096;                                  // 2 out tiles [16][128] bf16
constexpr int kWideCtrlOff = kWideOut + 2 * 4096;
struct TcWideCtrl {
    uint64_t full[kWideStages];  // operands of a chunk have landed (transaction bytes)
    uint64_t mma1;               // D1 of the current chunk complete
    uint64_t mma3;               // DST of the current chunk complete
    uint64_t upd[2];             // half h of the tensor-memory state copy refreshed (one arrival per owner warp)
    uint64_t u_ready;            // U^T of the current chunk is in tensor memory (one arrival per warp of warpgroup 0)
    uint64_t out_ready;          // the out tile of the current chunk is written
    uint32_t tmem_base;
    int32_t abort_flag;
};
constexpr int kWideSmemBytes = kWideCtrlOff + (int)sizeof(TcWideCtrl) + 128;

// A state owner keeps 64 columns of row v: half 0 = columns 0..63 (warpgroup 1), half 1 = 64..127 (warpgroup 2), as
// 32 registers of bf16 pairs = 8 groups of 8 columns; local group i is global group 8 * half + i.
// Initial values: handed over by the previous slab, from initial_state, or zero.
__device__ __forceinline__ void wide_load_state(uint32_t (&sreg)[32], const TwoPassArgs& a, const uint4* seg_mine,
                                                int64_t st_base, bool from_handover, int half) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gi = 8 * half + i;   // global group: state columns 8 gi .. 8 gi + 7
        if (from_handover) {
            const uint4 x = __ldcg(seg_mine + gi * 128);
            sreg[4 * i] = x.x; sreg[4 * i + 1] = x.y; sreg[4 * i + 2] = x.z; sreg[4 * i + 3] = x.w;
        } else if (a.initial_state != nullptr) {
            if (a.state_fp32) {
                const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.initial_state) + st_base) + 2 * gi;
                const float4 x = src[0], y = src[1];
                sreg[4 * i] = pack_bf2(x.x, x.y); sreg[4 * i + 1] = pack_bf2(x.z, x.w);
                sreg[4 * i + 2] = pack_bf2(y.x, y.y); sreg[4 * i + 3] = pack_bf2(y.z, y.w);
            } else {
                const uint4 x = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(a.initial_state) + st_base)[gi];
                sreg[4 * i] = x.x; sreg[4 * i + 1] = x.y; sreg[4 * i + 2] = x.z; sreg[4 * i + 3] = x.w;
            }
        } else {
            sreg[4 * i] = sreg[4 * i + 1] = sreg[4 * i + 2] = sreg[4 * i + 3] = 0u;
        }
    }
}
// Export of my half of row v as bf16 (the state before a group of chunks).
__device__ __forceinline__ void wide_export_state(const uint32_t (&sreg)[32], uint4* row, int half) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
        row[8 * half + i] = make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
}
// My half of row v leaves: to the hand-over buffer (not the last slab) or to final_state (bf16, or widened to fp32).
__device__ __forceinline__ void wide_store_state(const uint32_t (&sreg)[32], const TwoPassArgs& a, uint4* seg_mine,
                                                 int64_t st_base, bool to_handover, int half) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gi = 8 * half + i;
        if (to_handover) {
            seg_mine[gi * 128] = make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
        } else if (a.final_state != nullptr) {
            if (a.state_fp32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.final_state) + st_base) + 2 * gi;
                dst[0] = make_float4(bf_lo(sreg[4 * i]), bf_hi(sreg[4 * i]), bf_lo(sreg[4 * i + 1]), bf_hi(sreg[4 * i + 1]));
                dst[1] = make_float4(bf_lo(sreg[4 * i + 2]), bf_hi(sreg[4 * i + 2]), bf_lo(sreg[4 * i + 3]), bf_hi(sreg[4 * i + 3]));
            } else {
                reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.final_state) + st_base)[gi] =
                    make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
            }
        }
    }
}

__global__ void __launch_bounds__(kWideThreads, 1)
recurrence_tc_wide_kernel(const __grid_constant__ TwoPassArgs a, const __grid_constant__ TcMaps maps) {
    // (a ragged batch that the fused short-sequence kernel has served: nothing to do)
    if (a.short_flag != nullptr && *a.short_flag != 0) return;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* cs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 127) & ~(uintptr_t)127);
    TcWideCtrl& ctl = *reinterpret_cast<TcWideCtrl*>(cs + kWideCtrlOff);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int wg = warp >> 2;          // 0: chunk math + batch 0; 1, 2: state-update helpers; 3: control warp
    const int v = threadIdx.x & 127;   // TMEM lane = V row = state row (warpgroups 0-2)
    volatile int* abort_flag = &ctl.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWideStages; ++s) mbar_init(&ctl.full[s], 1);
        mbar_init(&ctl.mma1, 1);
        mbar_init(&ctl.mma3, 1);
        for (int b = 0; b < 2; ++b) mbar_init(&ctl.upd[b], 4);
        mbar_init(&ctl.u_ready, 4);
        mbar_init(&ctl.out_ready, 4);
        ctl.abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(&ctl.tmem_base, 256);
        tmem_relinquish_alloc_permit();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl.tmem_base;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_ds = tmem_base;          // DST (128 columns)
    const uint32_t t_d1 = tmem_base + 128u;   // u0 | o0
    const uint32_t t_s = tmem_base + 160u;    // bf16 state copy, 64 columns of k pairs (A operand of the first product)
    const uint32_t t_a = tmem_base + 224u;    // U^T: 8 columns of token pairs (A operand of the update product)

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, false, false);
    constexpr uint32_t idesc_dst = make_idesc_bf16_f32(128, 128, false, true);   // B = kr tile, N-major
    const int64_t n_chains = a.N * a.H;
    // mbarrier phases (every barrier completes exactly once per chunk; upd also once when the initial state is loaded)
    uint32_t full_bits = 0;   // bit s = phase of full[s]
    uint32_t mma1_phase = 0, mma3_phase = 0, upd_phase = 0, u_phase = 0, out_phase = 0;
    bool failed = false;
    // a wait of a whole warp: if it runs out for one lane, the warp gives up together (its lanes meet in
    // __syncwarp afterwards)
    auto warp_wait = [&](uint64_t* bar, uint32_t phase) {
        return __all_sync(0xffffffffu, mbar_wait_bounded(bar, phase, abort_flag, a.wait_ns)) != 0;
    };

    for (int64_t chain = blockIdx.x; chain < n_chains && !failed; chain += gridDim.x) {
        const TcChain ch = tc_locate_chain(a, chain);
        const int64_t n = ch.n, bos = ch.bos, seq_len = ch.seq_len;
        const int h = ch.h, n_chunks = ch.n_chunks;
        const uint8_t* rec_base = ch.rec_base;
        const int64_t st_base = ((n * a.H + h) * (int64_t)kD + v) * (int64_t)kD;  // S[v][k] at st_base + k
        // chunk range of this launch: all chunks, or one slab of a pipelined forward (fixed batches)
        const int c0 = a.slab_chunks > 0 ? a.slab_c0 : 0;
        const int c1 = (a.slab_chunks > 0 && c0 + a.slab_chunks < n_chunks) ? c0 + a.slab_chunks : n_chunks;
        const int64_t tstride = a.token_stride;

        if (wg == 3) {
            // =========================== control warp ===========================
            if (elect_one()) {
                auto issue_load = [&](int t) {
                    const int s = t % kWideStages;
                    mbar_arrive_expect_tx(&ctl.full[s], (uint32_t)(kTcRecord + kChunk * kD * 2));
                    bulk_g2s(cs + kWideStageOff + s * kTcStageBytes, rec_base + (int64_t)t * kTcRecord, kTcRecord, &ctl.full[s]);
                    // rows past the end of the tensor arrive as zeros; rows of the next sequence are never used
                    tma_load_3d(cs + kWideV + s * 4096, &maps.v, 0, h, (int)(bos + (int64_t)t * kChunk), &ctl.full[s]);
                };
                for (int t = c0; t < c0 + kWideStages && t < c1; ++t) issue_load(t);
                // The thread's work per chunk is ordered by what the chain waits for: the first product of chunk t goes
                // out the moment the state is refreshed, so everything else (operands of chunk t landed, the previous out
                // tile stored, a stage refilled) is done in the slack before that moment.
                auto store_out = [&](int t) {   // out tile of chunk t leaves through TMA once warpgroup 0 has written it
                    if (!mbar_wait_bounded(&ctl.out_ready, out_phase, abort_flag, a.wait_ns)) { failed = true; return; }
                    out_phase ^= 1u;
                    if (seq_len - (int64_t)t * kChunk >= kChunk) {   // (ragged tails were stored row by row by their owners)
                        tma_store_3d(&maps.out, 0, h, (int)(bos + (int64_t)t * kChunk), cs + kWideOut + (t & 1) * 4096);
                        bulk_commit_group();
                    }
                };
                if (c0 < c1) {   // operands of the first chunk
                    if (!mbar_wait_bounded(&ctl.full[c0 % kWideStages], (full_bits >> (c0 % kWideStages)) & 1u, abort_flag, a.wait_ns)) failed = true;
                    full_bits ^= 1u << (c0 % kWideStages);
                }
                for (int t = c0; t < c1 && !failed; ++t) {
                    const int s = t % kWideStages;
                    const uint32_t st_addr = smem_u32(cs + kWideStageOff + s * kTcStageBytes);
                    // ---- D1[V,32] = S . [kd; qd]^T: four K steps per refreshed half of the state ----
                    const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, kTcB1Lbo, 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if ((j & 3) == 0 && !failed && !mbar_wait_bounded(&ctl.upd[j >> 2], upd_phase, abort_flag, a.wait_ns))
                            failed = true;
                        if (!failed) {
                            tc_fence_after_sync();
                            umma_ts(t_d1, t_s + 8u * j, bd0 + (uint64_t)(j * (2 * kTcB1Lbo / 16)), idesc_n32, j > 0 ? 1u : 0u);
                        }
                    }
                    if (failed) break;
                    upd_phase ^= 1u;
                    umma_commit(&ctl.mma1);
                    // ---- slack while D1 runs and warpgroup 0 forms U: the previous chunk's out tile and stage ----
                    if (t > c0) {
                        store_out(t - 1);
                        if (failed) break;
                        // every reader of the previous chunk's stage is done (its last readers were the state updates
                        // observed above): refill it
                        if (t - 1 + kWideStages < c1) issue_load(t - 1 + kWideStages);
                    }
                    // ---- DST[V,K] = U^T . kr, as soon as warpgroup 0 has U in tensor memory ----
                    if (!mbar_wait_bounded(&ctl.u_ready, u_phase, abort_flag, a.wait_ns)) { failed = true; break; }
                    u_phase ^= 1u;
                    tc_fence_after_sync();
                    umma_ts(t_ds, t_a, make_smem_desc(st_addr + kTcKr, kTcKrLbo, kTcKrSbo), idesc_dst, 0u);
                    umma_commit(&ctl.mma3);
                    // ---- slack while DST runs and the state is updated: be ready for the next chunk ----
                    if (t + 1 < c1) {
                        const int s1 = (t + 1) % kWideStages;
                        if (!mbar_wait_bounded(&ctl.full[s1], (full_bits >> s1) & 1u, abort_flag, a.wait_ns)) { failed = true; break; }
                        full_bits ^= 1u << s1;
                    }
                    // the out-tile stores issued so far have read their tiles: warpgroup 0 rewrites the tile of chunk t-1
                    // for chunk t+1 only after that chunk's first product, issued at the top of the next round, completes
                    bulk_wait_group_read<0>();
                }
                if (!failed) {
                    if (c0 < c1) store_out(c1 - 1);
                    // the updates of the last chunk (or the loading of the initial state, for an empty range):
                    // consumed here so that the phases stay in step for the next chain
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        if (!failed && !mbar_wait_bounded(&ctl.upd[j], upd_phase, abort_flag, a.wait_ns)) failed = true;
                    upd_phase ^= 1u;
                }
            }
            failed = __any_sync(0xffffffffu, failed) != 0;
        } else {
            // =========================== warpgroups 0-2 ===========================
            uint4* const seg_mine = reinterpret_cast<uint4*>(a.seg_state) + (chain * 16) * 128 + v;  // + i * 128
            unsigned short* ocol = reinterpret_cast<unsigned short*>(a.out) + bos * tstride + (int64_t)h * kD;

            // ---- initial state: my half of row v into registers (pairs over k) and into the tensor-memory copy ----
            const int half = wg - 1;   // state owners: 0 or 1 (warpgroup 0: unused)
            uint32_t sreg[32];         // my 64 state columns of row v as bf16 pairs (state owners only)
            const uint32_t t_s_mine = t_s + lane_sel + 32u * half;    // my 32 columns of the tensor-memory copy
            const uint32_t t_ds_mine = t_ds + lane_sel + 64u * half;  // my 64 columns of DST
            auto publish_half = [&]() {   // my four batches are in the tensor-memory copy: tell the control warp
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl.upd[half]);
            };
            auto store_copy = [&](int lb) {   // local batch lb = 16 columns = 8 pairs
                tmem_st8(t_s_mine + 8 * lb, sreg[8 * lb], sreg[8 * lb + 1], sreg[8 * lb + 2], sreg[8 * lb + 3],
                         sreg[8 * lb + 4], sreg[8 * lb + 5], sreg[8 * lb + 6], sreg[8 * lb + 7]);
            };
            if (wg != 0) {
                wide_load_state(sreg, a, seg_mine, st_base, c0 > 0, half);
#pragma unroll
                for (int lb = 0; lb < 4; ++lb) store_copy(lb);
                publish_half();
            }

            // My four batches of my state row: S[v][k] = bf(fma(S[v][k], E_tot[k], DST[v][k])), 16 columns per batch.
            // The DST columns of the next batch are fetched while a batch is computed; the refreshed pairs of all four
            // batches are stored back to back and their completion is awaited once (a tensor-memory store takes far
            // longer than the arithmetic of a batch).
            auto update_half = [&](const float4* et4) {   // et4: E_tot of my 64 columns
                uint32_t r[2][16];
                tmem_ld16(t_ds_mine, r[0]);
#pragma unroll
                for (int lb = 0; lb < 4; ++lb) {
                    const int cur = lb & 1;
                    tmem_wait_ld();
                    if (lb + 1 < 4) tmem_ld16(t_ds_mine + 16 * (lb + 1), r[cur ^ 1]);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 e = et4[4 * lb + q];  // same address in every lane: one broadcast read
                        const uint32_t s0 = sreg[8 * lb + 2 * q], s1 = sreg[8 * lb + 2 * q + 1];
                        sreg[8 * lb + 2 * q] = pack_bf2(__fmaf_rn(bf_lo(s0), e.x, __uint_as_float(r[cur][4 * q])),
                                                        __fmaf_rn(bf_hi(s0), e.y, __uint_as_float(r[cur][4 * q + 1])));
                        sreg[8 * lb + 2 * q + 1] = pack_bf2(__fmaf_rn(bf_lo(s1), e.z, __uint_as_float(r[cur][4 * q + 2])),
                                                            __fmaf_rn(bf_hi(s1), e.w, __uint_as_float(r[cur][4 * q + 3])));
                    }
                    store_copy(lb);
                }
                publish_half();
            };

            for (int t = c0; t < c1; ++t) {
                const int s = t % kWideStages;
                const uint8_t* st = cs + kWideStageOff + s * kTcStageBytes;
                const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)t * kChunk);
                // ---- optional export: the state before this group of chunks (my half of my row, bf16) ----
                if (a.chunk_states != nullptr && wg != 0 && t % a.cs_every == 0) {
                    uint4* row = reinterpret_cast<uint4*>(a.chunk_states + ((ch.cs_slot0 + t / a.cs_every) * a.H + h) * (int64_t)(kD * kD) +
                                                          (int64_t)v * kD);
                    wide_export_state(sreg, row, half);
                }
                // ---- operands of chunk t have landed ----
                if (!warp_wait(&ctl.full[s], (full_bits >> s) & 1u)) { failed = true; break; }
                full_bits ^= 1u << s;

                if (wg == 0) {
                    // Fragment coordinates of this thread: g = lane / 4, tq = lane % 4; its warp covers V rows
                    // 32 (warp) + 16 mt + {g, g + 8} for the two row tiles mt, tokens {2tq, 2tq+1, 2tq+8, 2tq+9}.
                    const int g = lane >> 2, tq = lane & 3;
                    const int row0 = warp * 32 + g;   // + 16 mt + 8 hi
                    // -- operands that do not depend on the state, fetched while the first product runs --
                    const unsigned short* vt = reinterpret_cast<const unsigned short*>(cs + kWideV + s * 4096);
                    uint32_t vfr[2][4];   // value tile as A fragments: {row g: tokens 2tq,+1 | row g+8 | row g: tokens 2tq+8,+9 | row g+8}
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int row = row0 + 16 * mt + 8 * (e & 1), tok = 2 * tq + 8 * (e >> 1);
                            const uint32_t lo = tok < len ? vt[tok * kD + row] : 0u;
                            const uint32_t hi = tok + 1 < len ? vt[(tok + 1) * kD + row] : 0u;
                            vfr[mt][e] = lo | (hi << 16);
                        }
                    }
                    const uint32_t* beta32 = reinterpret_cast<const uint32_t*>(st + kTcBeta);
                    const uint32_t bp0 = beta32[tq], bp1 = beta32[tq + 4];   // sigmoid(beta) of tokens (2tq, 2tq+1), (2tq+8, 2tq+9)
                    uint32_t invb[2][2], mqkb[2][2];   // B fragments of INV^T and Mqk^T for the token tiles nt = 0, 1
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        invb[nt][0] = *reinterpret_cast<const uint32_t*>(st + kTcInv + tc_sq_off(8 * nt + g, 2 * tq));
                        invb[nt][1] = *reinterpret_cast<const uint32_t*>(st + kTcInv + tc_sq_off(8 * nt + g, 2 * tq + 8));
                        mqkb[nt][0] = *reinterpret_cast<const uint32_t*>(st + kTcMqk + tc_sq_off(8 * nt + g, 2 * tq));
                        mqkb[nt][1] = *reinterpret_cast<const uint32_t*>(st + kTcMqk + tc_sq_off(8 * nt + g, 2 * tq + 8));
                    }
                    if (!warp_wait(&ctl.mma1, mma1_phase)) { failed = true; break; }
                    mma1_phase ^= 1u;
                    tc_fence_after_sync();
                    // -- D1 as mma.sync accumulator fragments: u0 (columns 0-15) and o0 (16-31), read together: the
                    //    control thread may overwrite D1 with the next chunk's product as soon as the state is refreshed --
                    uint32_t u0f[2][8], o0f[2][8];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
                        tmem_ld_16x256b_x2(t_d1 + lane_sel + ((uint32_t)(16 * mt) << 16), u0f[mt]);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
                        tmem_ld_16x256b_x2(t_d1 + lane_sel + ((uint32_t)(16 * mt) << 16) + 16, o0f[mt]);
                    tmem_wait_ld();
                    // -- u' = (v (-) bf(u0)) (*) bf(beta);  U = bf(u' INV^T): on the chain --
                    uint32_t ufr[2][4];   // U as A fragments
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        uint32_t up[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t u0 = pack_bf2(__uint_as_float(u0f[mt][2 * e]), __uint_as_float(u0f[mt][2 * e + 1]));
                            up[e] = bf2_mul(bf2_sub(vfr[mt][e], u0), (e >> 1) ? bp1 : bp0);
                        }
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt) {
                            float c[4] = {0.f, 0.f, 0.f, 0.f};
                            mma_bf16_f32acc(c, up[0], up[1], up[2], up[3], invb[nt][0], invb[nt][1]);
                            ufr[mt][2 * nt] = pack_bf2(c[0], c[1]);       // row g,   tokens 8nt + 2tq, +1
                            ufr[mt][2 * nt + 1] = pack_bf2(c[2], c[3]);   // row g+8
                        }
                        tmem_st_16x128b_x2(t_a + lane_sel + ((uint32_t)(16 * mt) << 16), ufr[mt][0], ufr[mt][1], ufr[mt][2], ufr[mt][3]);
                    }
                    // -- while that store is in flight: the out term bf(U Mqk^T) --
                    uint32_t d3[2][2][2];   // [mt][nt][row g | row g+8], token pairs
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt) {
                            float c[4] = {0.f, 0.f, 0.f, 0.f};
                            mma_bf16_f32acc(c, ufr[mt][0], ufr[mt][1], ufr[mt][2], ufr[mt][3], mqkb[nt][0], mqkb[nt][1]);
                            d3[mt][nt][0] = pack_bf2(c[0], c[1]);
                            d3[mt][nt][1] = pack_bf2(c[2], c[3]);
                        }
                    }
                    tmem_wait_st();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl.u_ready);
                    // -- out = bf(o0) (+) bf(U Mqk^T): off the chain, beside the update product and the state update --
                    unsigned short* out_tile = reinterpret_cast<unsigned short*>(cs + kWideOut + (t & 1) * 4096);
                    unsigned short* og = ocol + (int64_t)t * kChunk * tstride;
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                            for (int hi = 0; hi < 2; ++hi) {
                                const uint32_t o = bf2_add(pack_bf2(__uint_as_float(o0f[mt][4 * nt + 2 * hi]),
                                                                    __uint_as_float(o0f[mt][4 * nt + 2 * hi + 1])),
                                                           d3[mt][nt][hi]);
                                const int row = row0 + 16 * mt + 8 * hi, tok = 8 * nt + 2 * tq;
                                if (len == kChunk) {
                                    out_tile[tok * kD + row] = (unsigned short)(o & 0xffffu);
                                    out_tile[(tok + 1) * kD + row] = (unsigned short)(o >> 16);
                                } else {
                                    if (tok < len) og[(int64_t)tok * tstride + row] = (unsigned short)(o & 0xffffu);
                                    if (tok + 1 < len) og[(int64_t)(tok + 1) * tstride + row] = (unsigned short)(o >> 16);
                                }
                            }
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl.out_ready);
                } else {
                    // ---- state owners: the update product of this chunk is complete; my half of my state row ----
                    const float4* et4 = reinterpret_cast<const float4*>(st + kTcEt) + 16 * half;  // gate decay of my 64 columns
                    if (!warp_wait(&ctl.mma3, mma3_phase)) { failed = true; break; }
                    mma3_phase ^= 1u;
                    tc_fence_after_sync();
                    update_half(et4);
                }
            }
            if (!failed && wg != 0) {
                const bool handover = c1 < n_chunks;   // not the last slab: the state goes to the hand-over buffer
                wide_store_state(sreg, a, seg_mine, st_base, handover, half);
            }
        }
        if (failed) ctl.abort_flag = 1;   // the other roles leave their waits
        // one chain is done with the stages, the tiles and the tensor memory before the next one starts
        named_barrier_sync(1, kWideThreads);
        failed = failed || ctl.abort_flag != 0;
    }

    if (failed) {
        ctl.abort_flag = 1;
        atomicExch(a.status, FKDA_ERR_DEVICE_STATUS);
    }
    bulk_wait_group<0>();   // (the control thread) out tiles fully written
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 256);
    }
}

}  // namespace fkda
