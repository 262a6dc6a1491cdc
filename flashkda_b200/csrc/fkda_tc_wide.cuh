// "Wide" variant of the tensor-core recurrence for the few-chains regime (no more chains than SMs):
// ONE chain per CTA, and the two warpgroups that would otherwise idle help with the largest
// element-wise step of a chunk, the state update.  Warpgroup 0 runs the chunk as in
// recurrence_tc_ts_kernel (MMA issue, u', U, out; every A operand in tensor memory); the 128 columns k of
// the state update DST[v, k] are split in three ranges, one per warpgroup (thread v of warpgroup j owns
// S[v, k] for k in its range, in registers, and writes the refreshed pairs to the tensor-memory copy that the
// next chunk's first MMA reads).  Same numerics and record format.  Included by fkda_tc.cu.
#pragma once

namespace fkda {

// columns k = 16*b .. 16*b+15 of the state are "batch" b; batches [lo, hi) per warpgroup
// (warpgroup 0 also forms the out tile, so it gets the smallest share)
__device__ __forceinline__ int wide_batch_lo(int wg) { return wg == 0 ? 0 : (wg == 1 ? 1 : 4); }
__device__ __forceinline__ int wide_batch_hi(int wg) { return wg == 0 ? 1 : (wg == 1 ? 4 : 8); }

// State update of batches [kLo, kHi) of row v: S[v][k] = bf(fma(S[v][k], E_tot[k], DST[v][k])) in registers,
// and the refreshed pairs into the tensor-memory state copy.
template <int kLo, int kHi>
__device__ __forceinline__ void wide_update(uint32_t (&sreg)[64], uint32_t t_ds_lane, uint32_t t_s_lane, const float4* et4) {
#pragma unroll
    for (int b = kLo; b < kHi; ++b) {
        uint32_t r[16];
        sm100::tmem_ld16(t_ds_lane + 16 * b, r);
        sm100::tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 e = et4[4 * b + q];  // same address in every lane: one broadcast read
            const uint32_t s0 = sreg[8 * b + 2 * q], s1 = sreg[8 * b + 2 * q + 1];
            sreg[8 * b + 2 * q] = pack_bf2(__fmaf_rn(bf_lo(s0), e.x, __uint_as_float(r[4 * q])),
                                           __fmaf_rn(bf_hi(s0), e.y, __uint_as_float(r[4 * q + 1])));
            sreg[8 * b + 2 * q + 1] = pack_bf2(__fmaf_rn(bf_lo(s1), e.z, __uint_as_float(r[4 * q + 2])),
                                               __fmaf_rn(bf_hi(s1), e.w, __uint_as_float(r[4 * q + 3])));
        }
        sm100::tmem_st8(t_s_lane + 8 * b, sreg[8 * b], sreg[8 * b + 1], sreg[8 * b + 2], sreg[8 * b + 3],
                        sreg[8 * b + 4], sreg[8 * b + 5], sreg[8 * b + 6], sreg[8 * b + 7]);
    }
}

// shared memory of the one chain: record stages and value tiles as in fkda_tc_ts.cuh, then two out tiles (a TMA
// store reads one while the next chunk's is formed), then the control block
constexpr int kWideOut = kTsOut;                   // 2 x [16][128] bf16
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
    TcWideCtrl& ctl = *reinterpret_cast<TcWideCtrl*>(cs + kWideCtrlOff);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int wg = warp >> 2;          // 0: runs the chunk; 1, 2: state-update helpers
    const int wiw = warp & 3;
    const int v = threadIdx.x & 127;   // TMEM lane = V row = state row
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
    const uint32_t t_s = tmem_base + 160u;    // bf16 state copy, 64 columns of k pairs (A operand of MMA1)
    const uint32_t t_a = tmem_base + 224u;    // u'^T, then U^T: 8 columns of token pairs (A operand of MMA2, MMA3)

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, false, false);
    constexpr uint32_t idesc_n16 = make_idesc_bf16_f32(128, 16, false, false);
    constexpr uint32_t idesc_dst = make_idesc_bf16_f32(128, 128, false, true);   // B = kr tile, N-major
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
        const int64_t st_base = ((n * a.H + h) * (int64_t)kD + v) * (int64_t)kD;  // S[v][k] at st_base + k
        // chunk range of this launch: all chunks, or one slab of a pipelined forward (fixed batches)
        const int c0 = a.slab_chunks > 0 ? a.slab_c0 : 0;
        const int c1 = (a.slab_chunks > 0 && c0 + a.slab_chunks < n_chunks) ? c0 + a.slab_chunks : n_chunks;
        uint4* const seg_mine = reinterpret_cast<uint4*>(a.seg_state) + (chain * 16) * 128 + v;  // + i * 128

        auto issue_load = [&](int t) {
            const int s = t % kTcStages;
            mbar_arrive_expect_tx(&ctl.full[s], (uint32_t)(kTcRecord + kChunk * kD * 2));
            bulk_g2s(cs + kTsStage + s * kTcStageBytes, rec_base + (int64_t)t * kTcRecord, kTcRecord, &ctl.full[s]);
            tma_load_3d(cs + kTsV + s * 4096, &maps.v, 0, h, (int)(bos + (int64_t)t * kChunk), &ctl.full[s]);
        };
        if (threadIdx.x == 0) {
            for (int t = c0; t < c0 + kTcStages && t < c1; ++t) issue_load(t);
        }
        const int64_t tstride = a.token_stride;
        unsigned short* ocol = reinterpret_cast<unsigned short*>(a.out) + bos * tstride + (int64_t)h * kD + v;

        // ---- initial state: my columns of row v into registers (pairs over k) and into the tensor-memory copy ----
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
            for (int i = 0; i < 16; ++i) {   // group i = state columns 8i .. 8i+7 = registers 4i .. 4i+3
                if ((i >> 1) >= b_lo && (i >> 1) < b_hi) {
                    if (a.state_fp32) {
                        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.initial_state) + st_base) + 2 * i;
                        const float4 x = src[0], y = src[1];
                        sreg[4 * i] = pack_bf2(x.x, x.y); sreg[4 * i + 1] = pack_bf2(x.z, x.w);
                        sreg[4 * i + 2] = pack_bf2(y.x, y.y); sreg[4 * i + 3] = pack_bf2(y.z, y.w);
                    } else {
                        const uint4 x = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(a.initial_state) + st_base)[i];
                        sreg[4 * i] = x.x; sreg[4 * i + 1] = x.y; sreg[4 * i + 2] = x.z; sreg[4 * i + 3] = x.w;
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 8; ++b)
            if (b >= b_lo && b < b_hi)
                tmem_st8(t_s + 8 * b + lane_sel, sreg[8 * b], sreg[8 * b + 1], sreg[8 * b + 2], sreg[8 * b + 3],
                         sreg[8 * b + 4], sreg[8 * b + 5], sreg[8 * b + 6], sreg[8 * b + 7]);
        tmem_wait_st();
        tc_fence_before_sync();
        named_barrier_sync(kBarAll, 384);

        for (int t = c0; t < c1; ++t) {
            const int s = t % kTcStages;
            uint8_t* st = cs + kTsStage + s * kTcStageBytes;
            const uint32_t st_addr = smem_u32(st);
            const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)t * kChunk);
            __nv_bfloat16* out_tile = reinterpret_cast<__nv_bfloat16*>(cs + kWideOut + (t & 1) * 4096);

            // ---- operands of chunk t have landed (every warpgroup observes it: the helpers read E_tot) ----
            if (!mbar_wait_bounded(&ctl.full[s], full_phase[s], abort_flag, a.wait_ns)) { failed = true; break; }
            full_phase[s] ^= 1u;
            if (wg == 0) {
                // ---- MMA1: D1[V,32] = S . [kd; qd]^T ----
                if (wiw == 0) {
                    if (elect_one()) {
                        tc_fence_after_sync();
                        const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, kTcB1Lbo, 128);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            umma_ts(t_d1, t_s + 8u * j, bd0 + (uint64_t)(j * (2 * kTcB1Lbo / 16)), idesc_n32, j > 0 ? 1u : 0u);
                        umma_commit(&ctl.mma);
                    }
                    __syncwarp();
                }
                unsigned short v_cur[kChunk];  // value column v of this chunk (zero past the sequence end)
                tc_load_v_column(cs + kTsV + s * 4096, v, len, v_cur);
                uint32_t bpk[8];  // bf16x2 pairs of sigmoid(beta)
                tc_load_beta(st, bpk);
                if (!mbar_wait_bounded(&ctl.mma, mma_phase, abort_flag, a.wait_ns)) { failed = true; break; }
                mma_phase ^= 1u;
                tc_fence_after_sync();
                // ---- u' = (v (-) bf(u0)) (*) bf(beta) -> A operand (thread = V row) ----
                {
                    uint32_t r[16];
                    tmem_ld16(t_d1 + lane_sel, r);
                    tmem_wait_ld();
                    uint32_t up[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t u0 = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                        const uint32_t vp = (uint32_t)v_cur[2 * i] | ((uint32_t)v_cur[2 * i + 1] << 16);
                        up[i] = bf2_mul(bf2_sub(vp, u0), bpk[i]);
                    }
                    tmem_st8(t_a + lane_sel, up[0], up[1], up[2], up[3], up[4], up[5], up[6], up[7]);
                    tmem_wait_st();
                }
                tc_fence_before_sync();
                named_barrier_sync(kBarMain, 128);
                // ---- MMA2: D2[V,16] = u'^T . INV^T  (into the first 16 DST columns) ----
                if (wiw == 0) {
                    if (elect_one()) {
                        tc_fence_after_sync();
                        umma_ts(t_ds, t_a, make_smem_desc(st_addr + kTcInv, 256, 128), idesc_n16, 0u);
                        umma_commit(&ctl.mma);
                    }
                    __syncwarp();
                }
                if (!mbar_wait_bounded(&ctl.mma, mma_phase, abort_flag, a.wait_ns)) { failed = true; break; }
                mma_phase ^= 1u;
                tc_fence_after_sync();
                {   // U = bf(D2) replaces u' as the A operand
                    uint32_t r[16];
                    tmem_ld16(t_ds + lane_sel, r);
                    tmem_wait_ld();
                    uint32_t p[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) p[i] = pack_bf2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    tmem_st8(t_a + lane_sel, p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7]);
                    tmem_wait_st();
                }
                tc_fence_before_sync();
                named_barrier_sync(kBarMain, 128);
                // ---- MMA3: D3[V,16] = U^T . Mqk^T (over the dead u0 columns);  DST[V,K] = U^T . kr ----
                if (wiw == 0) {
                    if (elect_one()) {
                        tc_fence_after_sync();
                        umma_ts(t_d1, t_a, make_smem_desc(st_addr + kTcMqk, 256, 128), idesc_n16, 0u);
                        umma_ts(t_ds, t_a, make_smem_desc(st_addr + kTcKr, kTcKrLbo, kTcKrSbo), idesc_dst, 0u);
                        umma_commit(&ctl.mma3);
                    }
                    __syncwarp();
                }
            }
            // ---- every warpgroup: the chunk's last MMAs are done ----
            if (!mbar_wait_bounded(&ctl.mma3, mma3_phase, abort_flag, a.wait_ns)) { failed = true; break; }
            mma3_phase ^= 1u;
            tc_fence_after_sync();
            const float4* et4 = reinterpret_cast<const float4*>(st + kTcEt);  // gate decay of the 128 state columns

            if (wg == 0) {
                // ---- out = bf(o0) (+) bf(Mqk U) (thread = V row) ----
                uint32_t r[32];
                tmem_ld32(t_d1 + lane_sel, r);  // D3 in 0-15, o0 in 16-31
                tmem_wait_ld();
                tc_store_out(r, reinterpret_cast<unsigned short*>(out_tile), ocol + (int64_t)t * kChunk * tstride, tstride, v, len);
            }
            // ---- my columns of state row v ----
            if (wg == 0) wide_update<0, 1>(sreg, t_ds + lane_sel, t_s + lane_sel, et4);
            else if (wg == 1) wide_update<1, 4>(sreg, t_ds + lane_sel, t_s + lane_sel, et4);
            else wide_update<4, 8>(sreg, t_ds + lane_sel, t_s + lane_sel, et4);
            tmem_wait_st();
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
            // ---- final state: my columns of my row, bf16 or widened to fp32 ----
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if ((i >> 1) >= b_lo && (i >> 1) < b_hi) {
                    if (a.state_fp32) {
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.final_state) + st_base) + 2 * i;
                        dst[0] = make_float4(bf_lo(sreg[4 * i]), bf_hi(sreg[4 * i]), bf_lo(sreg[4 * i + 1]), bf_hi(sreg[4 * i + 1]));
                        dst[1] = make_float4(bf_lo(sreg[4 * i + 2]), bf_hi(sreg[4 * i + 2]), bf_lo(sreg[4 * i + 3]), bf_hi(sreg[4 * i + 3]));
                    } else {
                        reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.final_state) + st_base)[i] =
                            make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
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
