// Tensor-core recurrence with every tcgen05.mma A operand in TENSOR MEMORY (the default kernel when there are
// more chains than SMs).
//
// Same chunk walk, records, numerics and scheduling as recurrence_tc_kernel (fkda_tc.cu); what changes is where
// the operands live and the orientation of the state update:
//   * thread v (= TMEM lane v) owns state ROW v, S[v, 0..127], in 64 packed registers (k pairs);
//   * the copy that the first product of a chunk reads, D1[V,32] = S[V,K] . [kd; qd]^T, is the A operand
//     of tcgen05.mma in tensor memory (lane = v, 64 columns of bf16 pairs), written with tcgen05.st by
//     the owner threads: no 32 KB shared-memory tile is written and re-read per chunk;
//   * the A operands of the 16-deep products, u'^T and U^T ([V, 16 tokens] = 8 columns of bf16 pairs), are
//     written to tensor memory by the threads that form them as well: no shared-memory operand tile and no
//     generic-to-async proxy fence between the element-wise steps and the next MMA;
//   * the update product is DST[V,K] = U^T[V,16] . kr[16,K] (B = the kr tile read N-major), so thread v reads
//     DST[v, :] from its own lane and applies S[v,k] = bf(fma(S[v,k], E_tot[k], DST[v,k])) with E_tot
//     broadcast from the record in shared memory;
//   * the state copy aliases the first 64 of the 128 DST columns: it is dead once D1 is complete, and
//     the update writes pairs 8b..8b+7 only after DST columns 16b..16b+15 have been read.
// Tensor memory per chain: DST 128 + D1 32 + A 8 columns; 504 of 512 with three chains.  Shared memory holds only
// what TMA moves: two record stages, two value tiles, one out tile per chain.
// Included by fkda_tc.cu.
#pragma once

namespace fkda {

// byte offsets inside one chain's shared-memory block (no state tile)
constexpr int kTsStage = 0;                                   // kTcStages chunk records
constexpr int kTsV = (kTsStage + kTcStages * kTcStageBytes + 127) / 128 * 128;   // kTcStages value tiles [16][128] bf16
constexpr int kTsOut = kTsV + kTcStages * 4096;               // out tile [16][128] bf16
constexpr int kTsChainBytes = kTsOut + 4096;
static_assert(kTsV % 128 == 0 && kTsChainBytes % 128 == 0, "TMA tiles are 128-byte aligned");
constexpr int kTsSmemBytes = kTcChains * kTsChainBytes + (int)sizeof(TcCtrl) + 128;

__global__ void __launch_bounds__(kTcChains * 128, 1)
recurrence_tc_ts_kernel(const __grid_constant__ TwoPassArgs a, const __grid_constant__ TcMaps maps) {
    // (a ragged batch that the fused short-sequence kernel has served: nothing to do)
    if (a.short_flag != nullptr && *a.short_flag != 0) return;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 127) & ~(uintptr_t)127);
    TcCtrl& ctl = *reinterpret_cast<TcCtrl*>(smem + kTcChains * kTsChainBytes);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int wg = warp >> 2;          // chain slot
    const int wiw = warp & 3;          // warp within the warpgroup
    const int v = threadIdx.x & 127;   // state row = TMEM lane
    uint8_t* cs = smem + wg * kTsChainBytes;
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
    // columns: DST of chain c at 128*c (its first 64 columns hold the bf16 state copy between chunks, and its
    // first 16 receive D2 in between), D1 at 384 + 32*c (u0 in 0-15, o0 in 16-31; D3 later replaces u0)
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_ds = tmem_base + 128u * wg;
    const uint32_t t_d1 = tmem_base + 384u + 32u * wg;
    // the A operands of the 16-deep products (u', then U: [V = 128 lanes, 16 tokens] bf16 = 8 columns) also live
    // in tensor memory, written by their owner threads: no shared-memory operand tile, no proxy fences
    const uint32_t t_a = tmem_base + 480u + 8u * wg;

    constexpr uint32_t idesc_n32 = make_idesc_bf16_f32(128, 32, false, false);   // A = state copy in TMEM
    constexpr uint32_t idesc_n16 = make_idesc_bf16_f32(128, 16, false, false);
    constexpr uint32_t idesc_dst = make_idesc_bf16_f32(128, 128, false, true);   // B = kr tile, N-major

    const int bar_id = 1 + wg;
    const int64_t n_chains = a.N * a.H;
    uint32_t full_bits = 0;   // bit s = phase of full[wg][s]
    uint32_t mma_phase = 0;
    bool failed = false;
    bool first_claim = true;

    while (!failed) {
        // ---- next work item (a segment of a chain) ----
        if (v == 0) ctl.next_chain[wg] = tc_next_item(a, first_claim, wg, n_chains, abort_flag);
        first_claim = false;
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
        // (header word 9: the length from which a chain of a ragged batch is on the critical path and walked in one piece;
        //  0 for fixed batches, whose chains are all alike)
        const int critical = a.queue[9];
        const int c1 = (a.seg_chunks > 0 && !(critical > 0 && n_chunks >= critical) && c0 + a.seg_chunks < n_chunks) ? c0 + a.seg_chunks : n_chunks;
        const uint8_t* rec_base = ch.rec_base;
        // thread v owns state row v: element S[v][k] of this chain sits at st_base + k
        const int64_t st_base = ((n * a.H + h) * (int64_t)kD + v) * (int64_t)kD;

        auto issue_load = [&](int t) {  // one thread: the record of chunk t into stage t % kTcStages
            const int s = t % kTcStages;
            mbar_arrive_expect_tx(&ctl.full[wg][s], (uint32_t)(kTcRecord + kChunk * kD * 2));
            bulk_g2s(cs + kTsStage + s * kTcStageBytes, rec_base + (int64_t)t * kTcRecord, kTcRecord, &ctl.full[wg][s]);
            // rows past the end of the tensor arrive as zeros; rows of the next sequence are never used
            tma_load_3d(cs + kTsV + s * 4096, &maps.v, 0, h, (int)(bos + (int64_t)t * kChunk), &ctl.full[wg][s]);
        };
        if (v == 0) {
            for (int t = c0; t < c0 + kTcStages && t < c1; ++t) issue_load(t);
        }
        const int64_t tstride = a.token_stride;
        unsigned short* ocol = reinterpret_cast<unsigned short*>(a.out) + bos * tstride + (int64_t)h * kD + v;

        // ---- initial state: row v of S into registers (pairs over k) and into the tensor-memory copy ----
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
                const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.initial_state) + st_base);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float4 x = src[i];
                    sreg[2 * i] = pack_bf2(x.x, x.y);
                    sreg[2 * i + 1] = pack_bf2(x.z, x.w);
                }
            } else {
                const uint4* src =
                    reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(a.initial_state) + st_base);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint4 x = src[i];
                    sreg[4 * i] = x.x; sreg[4 * i + 1] = x.y; sreg[4 * i + 2] = x.z; sreg[4 * i + 3] = x.w;
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) sreg[i] = 0u;
        }
#pragma unroll
        for (int b = 0; b < 8; ++b)
            tmem_st8(t_ds + 8 * b + lane_sel, sreg[8 * b], sreg[8 * b + 1], sreg[8 * b + 2], sreg[8 * b + 3],
                     sreg[8 * b + 4], sreg[8 * b + 5], sreg[8 * b + 6], sreg[8 * b + 7]);
        tmem_wait_st();
        tc_fence_before_sync();
        named_barrier_sync(bar_id, 128);

        __nv_bfloat16* out_tile = reinterpret_cast<__nv_bfloat16*>(cs + kTsOut);

        for (int t = c0; t < c1; ++t) {
            const int s = t % kTcStages;
            uint8_t* st = cs + kTsStage + s * kTcStageBytes;
            const uint32_t st_addr = smem_u32(st);

            // ---- optional export: the state before this group of chunks (my row, bf16) ----
            if (a.chunk_states != nullptr && t % a.cs_every == 0) {
                uint4* dst = reinterpret_cast<uint4*>(a.chunk_states + ((ch.cs_slot0 + t / a.cs_every) * a.H + h) * (int64_t)(kD * kD) +
                                                      (int64_t)v * kD);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    dst[i] = make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
            }
            // ---- operands of chunk t have landed ----
            if (!mbar_wait_bounded(&ctl.full[wg][s], (full_bits >> s) & 1u, abort_flag, a.wait_ns)) { failed = true; break; }
            full_bits ^= 1u << s;

            // ---- MMA1: D1[V,32] = S . [kd; qd]^T, A = the state copy in tensor memory (8 columns per K step) ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    const uint64_t bd0 = make_smem_desc(st_addr + kTcB1, kTcB1Lbo, 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        umma_ts(t_d1, t_ds + 8u * j, bd0 + (uint64_t)(j * (2 * kTcB1Lbo / 16)), idesc_n32, j > 0 ? 1u : 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            // work off the critical path while the MMA runs
            const int len = (int)min((int64_t)kChunk, seq_len - (int64_t)t * kChunk);
            unsigned short v_cur[kChunk];  // value column v of this chunk (zero past the sequence end)
            tc_load_v_column(cs + kTsV + s * 4096, v, len, v_cur);
            uint32_t bpk[8];  // bf16x2 pairs of sigmoid(beta)
            tc_load_beta(st, bpk);
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, a.wait_ns)) { failed = true; break; }
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
            named_barrier_sync(bar_id, 128);

            // ---- MMA2: D2[V,16] = u'^T . INV^T  (into the first 16 DST columns; the state copy there is dead) ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    umma_ts(t_ds, t_a, make_smem_desc(st_addr + kTcInv, 256, 128), idesc_n16, 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, a.wait_ns)) { failed = true; break; }
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
            named_barrier_sync(bar_id, 128);

            // ---- MMA3: D3[V,16] = U^T . Mqk^T (over the dead u0 columns);  DST[V,K] = U^T . kr ----
            if (wiw == 0) {
                if (elect_one()) {
                    tc_fence_after_sync();
                    // the previous out tile must have been read by its TMA store before this chunk's is formed
                    // (by all threads, once this commit has released them)
                    bulk_wait_group_read<0>();
                    umma_ts(t_d1, t_a, make_smem_desc(st_addr + kTcMqk, 256, 128), idesc_n16, 0u);
                    umma_ts(t_ds, t_a, make_smem_desc(st_addr + kTcKr, kTcKrLbo, kTcKrSbo), idesc_dst, 0u);
                    umma_commit(&ctl.mma[wg]);
                }
                __syncwarp();
            }
            if (!mbar_wait_bounded(&ctl.mma[wg], mma_phase, abort_flag, a.wait_ns)) { failed = true; break; }
            mma_phase ^= 1u;
            tc_fence_after_sync();

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
            // ---- state row v (thread = TMEM lane v of DST): S[v][k] = bf(fma(S[v][k], E_tot[k], DST[v][k])) in
            //      registers; the refreshed pairs go back to tensor memory for the next chunk's MMA1 ----
            const float4* et4 = reinterpret_cast<const float4*>(st + kTcEt);
            auto update16 = [&](int b, const uint32_t (&r)[16]) {  // columns k = 16b .. 16b+15
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 e = et4[4 * b + q];  // same address in every lane: one broadcast read
                    const uint32_t s0 = sreg[8 * b + 2 * q], s1 = sreg[8 * b + 2 * q + 1];
                    sreg[8 * b + 2 * q] = pack_bf2(__fmaf_rn(bf_lo(s0), e.x, __uint_as_float(r[4 * q])),
                                                   __fmaf_rn(bf_hi(s0), e.y, __uint_as_float(r[4 * q + 1])));
                    sreg[8 * b + 2 * q + 1] = pack_bf2(__fmaf_rn(bf_lo(s1), e.z, __uint_as_float(r[4 * q + 2])),
                                                       __fmaf_rn(bf_hi(s1), e.w, __uint_as_float(r[4 * q + 3])));
                }
                tmem_st8(t_ds + 8 * b + lane_sel, sreg[8 * b], sreg[8 * b + 1], sreg[8 * b + 2], sreg[8 * b + 3],
                         sreg[8 * b + 4], sreg[8 * b + 5], sreg[8 * b + 6], sreg[8 * b + 7]);
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
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_barrier_sync(bar_id, 128);

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
        // ---- final state: my row, bf16 or widened to fp32 ----
        if (a.final_state != nullptr) {
            if (a.state_fp32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.final_state) + st_base);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    dst[i] = make_float4(bf_lo(sreg[2 * i]), bf_hi(sreg[2 * i]), bf_lo(sreg[2 * i + 1]), bf_hi(sreg[2 * i + 1]));
            } else {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.final_state) + st_base);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    dst[i] = make_uint4(sreg[4 * i], sreg[4 * i + 1], sreg[4 * i + 2], sreg[4 * i + 3]);
            }
        }
        // all operand reads done before the next chain overwrites the stages
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
