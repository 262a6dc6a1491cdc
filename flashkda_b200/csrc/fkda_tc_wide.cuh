// "Wide" variant of the tensor-core recurrence for the few-chains regime (no more chains than SMs):
// ONE chain per CTA, and the two warpgroups that would otherwise idle help with the largest
// element-wise step of a chunk, the state update.  Warpgroup 0 runs the chunk exactly as in
// recurrence_tc_kernel (MMA issue, u', U, out); the 128 rows v of the transposed state update
// DST[k, v] are split in three ranges, one per warpgroup (thread k of warpgroup j owns S[v, k] for v
// in its range, in registers).  Same numerics, same record format, same TMEM / shared-memory layout
// (chain block 0 only).  Included by fkda_tc.cu.
#pragma once

namespace fkda {

// rows v = 16*b .. 16*b+15 of the state are "batch" b; batches [lo, hi) per warpgroup
// (warpgroup 0 also forms the out tile, so it gets the smallest share)
__device__ __forceinline__ int wide_batch_lo(int wg) { return wg == 0 ? 0 : (wg == 1 ? 2 : 5); }
__device__ __forceinline__ int wide_batch_hi(int wg) { return wg == 0 ? 2 : (wg == 1 ? 5 : 8); }

// State update of batches [kLo, kHi) of column k: S[vv][k] = bf(fma(S[vv][k], E_tot[k], DST[k][vv])) in
// registers, and the refreshed rows into the S^T tile.
template <int kLo, int kHi>
__device__ __forceinline__ void wide_update(uint32_t (&sreg)[64], uint32_t t_ds_lane, float e_mine, uint8_t* s_tile,
                                            int k) {
#pragma unroll
    for (int b = kLo; b < kHi; ++b) {
        uint32_t r[16];
        sm100::tmem_ld16(t_ds_lane + 16 * b, r);
        sm100::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t sv = sreg[8 * b + i];
            sreg[8 * b + i] = pack_bf2(__fmaf_rn(bf_lo(sv), e_mine, __uint_as_float(r[2 * i])),
                                       __fmaf_rn(bf_hi(sv), e_mine, __uint_as_float(r[2 * i + 1])));
        }
#pragma unroll
        for (int q = 0; q < 2; ++q)
            *reinterpret_cast<uint4*>(s_tile + sT_off(k, 2 * b + q)) =
                make_uint4(sreg[8 * b + 4 * q], sreg[8 * b + 4 * q + 1], sreg[8 * b + 4 * q + 2],
                           sreg[8 * b + 4 * q + 3]);
    }
}

constexpr int kWideOut = kSmChainBytes;            // 2 x [16][128] bf16
constexpr int kWideCtrlOff = kWideOut + 2 * 4096;
struct TcWideCtrl {
    uint64_t full[kTcStages];
    uint64_t mma;    // completion of MMA1 and MMA2 (warpgroup 0 only)
    uint64_t mma3;   // completion of the chunk's last MMAs (all warpgroups)
    uint32_t tmem_base;
    int32_t abort_flag;
};

__global__ void __launch_bounds__(384, 1)
recurrence_tc_wide_kernel(const __grid_constant__ TwoPassArgs a, const __grid_constant__ TcMaps maps) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* cs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 127) & ~(uintptr_t)127);
    // after the chain block: two out tiles (a TMA store reads one while the next chunk's is formed), then the
    // control block
    TcWideCtrl& ctl = *reinterpret_cast<TcWideCtrl*>(cs + kWideCtrlOff);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int wg = warp >> 2;          // 0: runs the chunk; 1, 2: state-update helpers
    const int wiw = warp & 3;
    const int v = threadIdx.x & 127;   // TMEM lane: V row (D1..D3) / state column k (DST)
    const int b_lo = wide_batch_lo(wg), b_hi = wide_batch_hi(wg);
    volatile int* abort_flag = &ctl.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) mbar_init(&ctl.full[s], 1);
        mbar_init(&ctl.mma, 1);
        mbar_init(&ctl.mma3, 1);
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
    const uint32_t t_ds = tmem_base;          // DST (128 columns; D2 in its first 16)
    const uint32_t t_d1 = tmem_base + 128u;   // u0 | o0, later D3 | o0

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, true, false);
    constexpr uint32_t idesc_n16 = make_idesc_bf16_f32(128, 16, false, false);
    constexpr uint32_t idesc_dst = make_idesc_bf16_f32(128, 128, true, false);
    const uint64_t s_desc0 = make_smem_desc(smem_u32(cs + kSmS), 2048, 128);
    const uint64_t a23_desc = make_smem_desc(smem_u32(cs + kSmA23), 2048, 128);
    constexpr int kBarMain = 1, kBarAll = 2;
    const int64_t n_chains = a.N * a.H;
    uint32_t full_phase[kTcStages] = {0, 0};
    uint32_t mma_phase = 0, mma3_phase = 0;
    bool failed = false;

    for (int64_t chain = blockIdx.x; chain < n_chains && !failed; chain += gridDim.x) {
        const TcChain ch = tc_locate_chain(a, chain);
        const int64_t n = ch.n, bos = ch.bos, seq_len = ch.seq_len;
        const int h = ch.h, n_chunks = ch.n_chunks;
        const uint8_t* rec_base = ch.rec_base;
        const int64_t st_base = (n * a.H + h) * (int64_t)(kD * kD) + v;  // S[vv][k = v] at st_base + vv * 128
        // chunk range of this launch: all chunks, or one slab of a pipelined forward (fixed batches)
        const int c0 = a.slab_chunks > 0 ? a.slab_c0 : 0;
        const int c1 = (a.slab_chunks > 0 && c0 + a.slab_chunks < n_chunks) ? c0 + a.slab_chunks : n_chunks;
        uint4* const seg_mine = reinterpret_cast<uint4*>(a.seg_state) + (chain * 16) * 128 + v;  // + i * 128

        auto issue_load = [&](int t) {
            const int s = t % kTcStages;
            mbar_arrive_expect_tx(&ctl.full[s], (uint32_t)(kTcRecord + kChunk * kD * 2));
            bulk_g2s(cs + kSmStage + s * kSmStageBytes, rec_base + (int64_t)t * kTcRecord, kTcRecord, &ctl.full[s]);
            tma_load_3d(cs + kSmV + s * 4096, &maps.v, 0, h, (int)(bos + (int64_t)t * kChunk), &ctl.full[s]);
        };
        if (threadIdx.x == 0) {
            for (int t = c0; t < c0 + kTcStages && t < c1; ++t) issue_load(t);
        }
        const int64_t tstride = a.token_stride;
        unsigned short* ocol = reinterpret_cast<unsigned short*>(a.out) + bos * tstride + (int64_t)h * kD + v;

        // ---- initial state: my rows of column k into registers (pairs over v) and into the S^T tile ----
        uint32_t sreg[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) sreg[i] = 0u;
        if (c0 > 0) {  // handed over by the launch that ran the previous slab
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if ((i >> 1) >= b_lo && (i >> 1) < b_hi) {
                    const uint4 x = __ldcg(seg_mine + i * 128);
                    sreg[4 * i] = x.x; sreg[4 * i + 1] = x.y; sreg[4 * i + 2] = x.z; sreg[4 * i + 3] = x.w;
                }
            }
        } else if (a.initial_state != nullptr) {
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                if ((i >> 3) >= b_lo && (i >> 3) < b_hi) {
                    if (a.state_fp32) {
                        const float* src = reinterpret_cast<const float*>(a.initial_state) + st_base;
                        sreg[i] = pack_bf2(src[(2 * i) * kD], src[(2 * i + 1) * kD]);
                    } else {
                        const unsigned short* src = reinterpret_cast<const unsigned short*>(a.initial_state) + st_base;
                        sreg[i] = (uint32_t)src[(2 * i) * kD] | ((uint32_t)src[(2 * i + 1) * kD] << 16);
                    }
                }
            }
        }
#pragma unroll
        for (int vg = 0; vg < 16; ++vg)
            if ((vg >> 1) >= b_lo && (vg >> 1) < b_hi)
                *reinterpret_cast<uint4*>(cs + kSmS + sT_off(v, vg)) =
                    make_uint4(sreg[4 * vg], sreg[4 * vg + 1], sreg[4 * vg + 2], sreg[4 * vg + 3]);
        fence_proxy_async_smem();
        named_barrier_sync(kBarAll, 384);

        for (int t = c0; t < c1; ++t) {
            const int s = t % kTcStages;
            uint8_t* st = cs + kSmStage + s * kSmStageBytes;
            const uint32_t st_addr = smem_u32(st);
            const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)t * kChunk);
            __nv_bfloat16* out_tile = reinterpret_cast<__nv_bfloat16*>(cs + kWideOut + (t & 1) * 4096);

            // ---- operands of chunk t have landed (every warpgroup observes it: the helpers read E_tot) ----
            if (!mbar_wait_bounded(&ctl.full[s], full_phase[s], abort_flag, kTcWaitNs)) { failed = true; break; }
            full_phase[s] ^= 1u;
            if (wg == 0) {
                // ---- MMA1: D1[V,32] = S . [kd; qd]^T ----
                if (wiw == 0) {
                    if (elect_one()) {
                        tc_fence_after_sync();
                        const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, kTcB1Lbo, 128);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            umma_ss(t_d1, s_desc0 + (uint64_t)(j * 256), bd0 + (uint64_t)(j * (2 * kTcB1Lbo / 16)),
                                    idesc_n32, j > 0 ? 1u : 0u);
                        umma_commit(&ctl.mma);
                    }
                    __syncwarp();
                }
                unsigned short v_cur[kChunk];  // value column v of this chunk (zero past the sequence end)
                tc_load_v_column(cs + kSmV + s * 4096, v, len, v_cur);
                uint32_t bpk[8];  // bf16x2 pairs of sigmoid(beta)
                tc_load_beta(st, bpk);
                if (!mbar_wait_bounded(&ctl.mma, mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
                mma_phase ^= 1u;
                tc_fence_after_sync();
                // ---- u' = (v (-) bf(u0)) (*) bf(beta) -> A operand (thread = V row) ----
                tc_form_u_prime(t_d1 + lane_sel, cs + kSmA23, v, v_cur, bpk);
                fence_proxy_async_smem();
                tc_fence_before_sync();
                named_barrier_sync(kBarMain, 128);
                // ---- MMA2: D2[V,16] = u'^T . INV^T  (into the first 16 DST columns) ----
                if (wiw == 0) {
                    if (elect_one()) {
                        tc_fence_after_sync();
                        umma_ss(t_ds, a23_desc, make_smem_desc(st_addr + kTcInv, 256, 128), idesc_n16, 0u);
                        umma_commit(&ctl.mma);
                    }
                    __syncwarp();
                }
                if (!mbar_wait_bounded(&ctl.mma, mma_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
                mma_phase ^= 1u;
                tc_fence_after_sync();
                tc_form_u(t_ds + lane_sel, cs + kSmA23, v);  // U = bf(D2)
                fence_proxy_async_smem();
                tc_fence_before_sync();
                named_barrier_sync(kBarMain, 128);
                // ---- MMA3: D3[V,16] = U^T . Mqk^T (over the dead u0 columns);  DST[K,V] = kr^T . U ----
                if (wiw == 0) {
                    if (elect_one()) {
                        tc_fence_after_sync();
                        umma_ss(t_d1, a23_desc, make_smem_desc(st_addr + kTcMqk, 256, 128), idesc_n16, 0u);
                        umma_ss(t_ds, make_smem_desc(st_addr + kTcKr, kTcKrLbo, kTcKrSbo), a23_desc, idesc_dst, 0u);
                        umma_commit(&ctl.mma3);
                    }
                    __syncwarp();
                }
            }
            // ---- every warpgroup: the chunk's last MMAs are done ----
            if (!mbar_wait_bounded(&ctl.mma3, mma3_phase, abort_flag, kTcWaitNs)) { failed = true; break; }
            mma3_phase ^= 1u;
            tc_fence_after_sync();
            const float e_mine = reinterpret_cast<const float*>(st + kTcEt)[v];  // gate decay of my state column

            if (wg == 0) {
                // ---- out = bf(o0) (+) bf(Mqk U) (thread = V row) ----
                uint32_t r[32];
                tmem_ld32(t_d1 + lane_sel, r);  // D3 in 0-15, o0 in 16-31
                tmem_wait_ld();
                tc_store_out(r, reinterpret_cast<unsigned short*>(out_tile), ocol + (int64_t)t * kChunk * tstride, tstride, v, len);
            }
            // ---- my rows of state column k ----
            if (wg == 0) wide_update<0, 2>(sreg, t_ds + lane_sel, e_mine, cs + kSmS, v);
            else if (wg == 1) wide_update<2, 5>(sreg, t_ds + lane_sel, e_mine, cs + kSmS, v);
            else wide_update<5, 8>(sreg, t_ds + lane_sel, e_mine, cs + kSmS, v);
            // warp 4 issues the TMA store and the refill, so that warpgroup 0 can go straight to the next chunk's MMA;
            // before the barrier it makes sure the store of the previous chunk has read its out tile (the one the
            // next chunk will overwrite)
            if (warp == 4) {
                if (elect_one()) bulk_wait_group_read<0>();
                __syncwarp();
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(kBarAll, 384);
            // ---- store the out tile, refill the stage just consumed ----
            if (warp == 4) {
                if (elect_one()) {
                    if (len == kChunk) {
                        tma_store_3d(&maps.out, 0, h, (int)(bos + (int64_t)t * kChunk), out_tile);
                        bulk_commit_group();
                    }
                    if (t + kTcStages < c1) issue_load(t + kTcStages);
                }
                __syncwarp();
            }
        }
        if (failed) break;
        if (c1 < n_chunks) {  // not the last slab: my rows of the state to the hand-over buffer
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if ((i >> 1) >= b_lo && (i >> 1) < b_hi)
                    seg_mine[i * 128] = make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
        } else if (a.final_state != nullptr) {
            // ---- final state: my rows of my column, bf16 or widened to fp32 ----
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                if ((i >> 3) >= b_lo && (i >> 3) < b_hi) {
                    if (a.state_fp32) {
                        float* dst = reinterpret_cast<float*>(a.final_state) + st_base;
                        dst[(2 * i) * kD] = bf_lo(sreg[i]);
                        dst[(2 * i + 1) * kD] = bf_hi(sreg[i]);
                    } else {
                        unsigned short* dst = reinterpret_cast<unsigned short*>(a.final_state) + st_base;
                        dst[(2 * i) * kD] = (unsigned short)(sreg[i] & 0xffffu);
                        dst[(2 * i + 1) * kD] = (unsigned short)(sreg[i] >> 16);
                    }
                }
            }
        }
        named_barrier_sync(kBarAll, 384);
    }

    if (failed) {
        ctl.abort_flag = 1;
        atomicExch(a.status, FKDA_ERR_DEVICE_STATUS);
    }
    bulk_wait_group<0>();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 256);
    }
}

}  // namespace fkda
