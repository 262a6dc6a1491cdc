// Warp-per-chunk "prepare" stage: one warp turns one (chunk, head) of q, k, g, beta into the chunk
// operands kd, qd, kr, E_tot, INV, Mqk (workspace record), with no block-level synchronisation:
// lane l owns columns 4l..4l+3 of all 16 token rows, so the in-chunk gate cumsum runs in registers,
// the q/k row norms use warp shuffles (in the exact summation order of the contract: an FMA chain
// over each group of 8 columns, then a butterfly over the 16 groups), and only the two small
// 16x16x128 products (mma.sync bf16) and the 16x16 inverse (mma.sync f16) go through a few KB of
// per-warp shared memory.  Warps are independent, so the same routine serves as a producer inside
// a persistent kernel.  Numerics: tests/torch_ref.py:153-229 of the reference.
#pragma once

#include <stddef.h>

#include "fkda_common.cuh"
#include "fkda_internal.h"
#include "fkda_sm100.cuh"

namespace fkda {

constexpr int kPwKiLbo = 272;  // ki tile: K-major core matrices, 16-byte K chunks 272 bytes apart (256 + 16 padding)

// Per-warp shared memory.  b1 is the B1 part of the record ([kd; qd] in its final UMMA layout, see
// fkda_common.cuh); kikr first holds ki (K-major core matrices: byte = (k/8)*272 + (r/8)*128 + (r%8)*16 +
// (k%8)*2) for the in-chunk products and then kr in the record's KR layout.  Both are shipped to the
// workspace with bulk copies; the padded strides keep the column-owning lanes free of bank conflicts.
struct alignas(16) PrepWarpSmem {
    uint8_t b1[kTcB1Bytes];
    uint8_t kikr[kTcKrBytes];
    float beta_act[kChunk];
};
static_assert(16 * kPwKiLbo <= kTcKrBytes, "the ki tile fits the KR buffer");
static_assert(offsetof(PrepWarpSmem, b1) == kTcB1 && offsetof(PrepWarpSmem, kikr) == kTcKr &&
              offsetof(PrepWarpSmem, beta_act) == kTcInv && sizeof(float) * kChunk <= 512,
              "the per-warp tiles coincide with the B1 and KR parts of a record (kRecordInSmem)");

// Where chunk `tile` of the (possibly ragged) batch lives: first token and number of valid rows.
// Returns false for a tile index past the last chunk (ragged upper bound).
__device__ __forceinline__ bool locate_tile(const TwoPassArgs& a, int64_t tile, int64_t* t0, int* len) {
    int64_t n, local_t, bos, seq_len;
    if (a.cu_seqlens != nullptr) {
        const int32_t* pre = a.tile_prefix;
        if (tile >= pre[a.N]) return false;
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
    *t0 = bos + local_t * kChunk;
    *len = (int)min((int64_t)kChunk, seq_len - local_t * kChunk);
    return true;
}

// Sum of squares of one 128-wide row held 4 columns per lane, in the contract's order: FMA chain
// over columns 8m..8m+7 (lanes 2m then 2m+1), then xor-butterfly with offsets 8,4,2,1 over the 16
// groups.  All lanes return the row total.
__device__ __forceinline__ float row_sumsq(const float (&x)[4], int lane) {
    float p = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) p = __fmaf_rn(x[i], x[i], p);
    const float first = __shfl_sync(0xffffffffu, p, lane & ~1);  // partial of the even lane of my pair
    float c = first;
#pragma unroll
    for (int i = 0; i < 4; ++i) c = __fmaf_rn(x[i], x[i], c);     // odd lanes: chain continued over their 4
#pragma unroll
    for (int off = 16; off >= 2; off >>= 1) c = __fadd_rn(c, __shfl_xor_sync(0xffffffffu, c, off));
    return __shfl_sync(0xffffffffu, c, lane | 1);                 // the odd lanes hold the group sums
}

// Sums of squares of TWO rows (q and k of one token) at once, each in the order of row_sumsq: after the pair
// chains, the first butterfly step (groups 8 apart = lanes 16 apart) also splits the work, the lower half-warp
// continuing with the q sums and the upper one with the k sums (a butterfly value is the same in both halves),
// so the remaining three steps move one value per lane instead of two; 8 shuffles instead of 12.
__device__ __forceinline__ void row_sumsq2(const float (&x)[4], const float (&y)[4], int lane, float* sx, float* sy) {
    float px = 0.f, py = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        px = __fmaf_rn(x[i], x[i], px);
        py = __fmaf_rn(y[i], y[i], py);
    }
    float cx = __shfl_sync(0xffffffffu, px, lane & ~1);  // partial of the even lane of my pair
    float cy = __shfl_sync(0xffffffffu, py, lane & ~1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {                         // odd lanes: chain continued over their 4 columns
        cx = __fmaf_rn(x[i], x[i], cx);
        cy = __fmaf_rn(y[i], y[i], cy);
    }
    const bool upper = (lane & 16) != 0;
    const float keep = upper ? cy : cx, send = upper ? cx : cy;
    float c = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 16));
#pragma unroll
    for (int off = 8; off >= 2; off >>= 1) c = __fadd_rn(c, __shfl_xor_sync(0xffffffffu, c, off));
    *sx = __shfl_sync(0xffffffffu, c, (lane & 15) | 1);        // odd lanes of the lower half hold the q total
    *sy = __shfl_sync(0xffffffffu, c, (lane & 15) | 17);       // odd lanes of the upper half hold the k total
}

// What a warp fetches ahead of a chunk: the first kPf rows of q, k, g (my 4 columns), and the per-chunk
// scalars.  Filled for the NEXT unit while the current one is in its last (memory-free) stage, so that a
// chunk does not start with an exposed DRAM round trip.
constexpr int kPf = 4;  // rows fetched ahead of their use
struct PrepPrefetch {
    uint2 q[kPf], k[kPf], g[kPf];
    float4 dtv;
    float a_log, beta_logit;  // beta of row `lane` (lanes below 16; 0 past the end, as zero padding does)
};
__device__ __forceinline__ void prep_prefetch(const TwoPassArgs& a, int64_t t0, int len, int h, int lane,
                                              PrepPrefetch& p) {
    const int c4 = lane * 4;
    const int64_t base = t0 * a.token_stride + (int64_t)h * kD + c4;
#pragma unroll
    for (int r = 0; r < kPf; ++r) {
        p.q[r] = p.k[r] = p.g[r] = make_uint2(0, 0);
        if (r < len) {
            p.q[r] = __ldg(reinterpret_cast<const uint2*>(a.q + base + (int64_t)r * a.token_stride));
            p.k[r] = __ldg(reinterpret_cast<const uint2*>(a.k + base + (int64_t)r * a.token_stride));
            p.g[r] = __ldg(reinterpret_cast<const uint2*>(a.g + base + (int64_t)r * a.token_stride));
        }
    }
    p.dtv = __ldg(reinterpret_cast<const float4*>(a.dt_bias + (int64_t)h * kD + c4));
    p.a_log = __ldg(a.A_log + h);
    p.beta_logit = 0.0f;
    if (lane < len) p.beta_logit = bf2f(a.beta[(t0 + lane) * a.beta_token_stride + h]);  // len <= 16
}

// One warp, one (chunk, head).  `ws` is the record to fill; kTc selects its layout (see fkda_common.cuh).
// `pf` holds the prefetched head of this chunk and leaves holding that of the next unit (if `next_valid`).
// kRecordInSmem (tensor-core layout only): `ws` and `sm` are the SAME 14 656 bytes of shared memory; the record
// stays there for a consumer in the same CTA (B1 and KR are built in place, nothing is copied; the sigmoid(beta)
// scratch at the start of the INV tile is consumed before the inverse is written).
template <bool kTc, bool kRecordInSmem = false>
__device__ __forceinline__ void prepare_chunk_warp(const TwoPassArgs& a, int64_t t0, int len, int h, uint8_t* ws,
                                                   PrepWarpSmem& sm, int lane, PrepPrefetch& pf, bool next_valid,
                                                   int64_t next_t0, int next_len, int next_h) {
    const int c4 = lane * 4;  // my 4 columns
    const float a_exp_half = __fmul_rn(ex2_approx(__fmul_rn(pf.a_log, 1.4426950408889634f)), 0.5f);
    const float dt[4] = {pf.dtv.x, pf.dtv.y, pf.dtv.z, pf.dtv.w};
    const uint32_t sc2 = pack_bf2(a.scale, a.scale);
    const __nv_bfloat16* qp = a.q + t0 * a.token_stride + (int64_t)h * kD + c4;
    const __nv_bfloat16* kp = a.k + t0 * a.token_stride + (int64_t)h * kD + c4;
    const __nv_bfloat16* gp = a.g + t0 * a.token_stride + (int64_t)h * kD + c4;

    // sigmoid(beta) of row `lane` (rows past the end use logit 0, as zero padding does)
    if (lane < kChunk) {
        const float sb = sigmoid_tanh(pf.beta_logit);
        sm.beta_act[lane] = sb;
        if constexpr (kTc) reinterpret_cast<__nv_bfloat16*>(ws + kTcBeta)[lane] = f2bf(sb);
    }

    float csum[4] = {0.f, 0.f, 0.f, 0.f};  // running in-chunk gate sum of my columns
    // rows are fetched kPf rows ahead of their use so that several DRAM round trips overlap
    uint2 (&ring_q)[kPf] = pf.q, (&ring_k)[kPf] = pf.k, (&ring_g)[kPf] = pf.g;
    auto fetch = [&](int r, int slot) {
        ring_q[slot] = ring_k[slot] = ring_g[slot] = make_uint2(0, 0);
        if (r < len) {
            ring_q[slot] = __ldg(reinterpret_cast<const uint2*>(qp + (int64_t)r * a.token_stride));
            ring_k[slot] = __ldg(reinterpret_cast<const uint2*>(kp + (int64_t)r * a.token_stride));
            ring_g[slot] = __ldg(reinterpret_cast<const uint2*>(gp + (int64_t)r * a.token_stride));
        }
    };
#pragma unroll 1
    for (int rb = 0; rb < kChunk; rb += kPf) {
#pragma unroll
    for (int rr = 0; rr < kPf; ++rr) {
        const int r = rb + rr;
        const bool valid = r < len;
        if (!valid) {
            // a row past the sequence end (warp-uniform): q = k = 0 and no gate contribution, so its rows of the
            // tiles are zeros (qd keeps the sign that the multiplication by bf(scale) gives a zero)
            const uint32_t qz = bf2_mul(0u, sc2);
            const int off = tc_b1_off(r, lane >> 1) + (lane & 1) * 8;
            *reinterpret_cast<uint2*>(sm.b1 + off) = make_uint2(0u, 0u);
            *reinterpret_cast<uint2*>(sm.b1 + off + 2 * 128) = make_uint2(qz, qz);
            *reinterpret_cast<uint2*>(sm.kikr + (lane >> 1) * kPwKiLbo + (r >> 3) * 128 + (r & 7) * 16 + (lane & 1) * 8) = make_uint2(0u, 0u);
            if constexpr (!kTc) {
                *reinterpret_cast<uint2*>(ws + kWsKd + (r * kD + c4) * 2) = make_uint2(0u, 0u);
                *reinterpret_cast<uint2*>(ws + kWsQd + (r * kD + c4) * 2) = make_uint2(qz, qz);
            }
            continue;
        }
        const uint2 qraw = ring_q[rr], kraw = ring_k[rr], graw = ring_g[rr];
        if (r + kPf < kChunk) fetch(r + kPf, rr);
        const float qv[4] = {bf_lo(qraw.x), bf_hi(qraw.x), bf_lo(qraw.y), bf_hi(qraw.y)};
        const float kv[4] = {bf_lo(kraw.x), bf_hi(kraw.x), bf_lo(kraw.y), bf_hi(kraw.y)};
        const float gv[4] = {bf_lo(graw.x), bf_hi(graw.x), bf_lo(graw.y), bf_hi(graw.y)};
        // q/k L2 normalisation
        float qss, kss;
        row_sumsq2(qv, kv, lane, &qss, &kss);
        const float qinv = rsqrt_approx(__fadd_rn(qss, 1e-6f));
        const float kinv = rsqrt_approx(__fadd_rn(kss, 1e-6f));
        const uint32_t qn0 = pack_bf2(__fmul_rn(qv[0], qinv), __fmul_rn(qv[1], qinv));
        const uint32_t qn1 = pack_bf2(__fmul_rn(qv[2], qinv), __fmul_rn(qv[3], qinv));
        const uint32_t kn0 = pack_bf2(__fmul_rn(kv[0], kinv), __fmul_rn(kv[1], kinv));
        const uint32_t kn1 = pack_bf2(__fmul_rn(kv[2], kinv), __fmul_rn(kv[3], kinv));
        // gate = gate_scale * sigmoid(exp(A_log) * (g + dt_bias)), 0 past the end; cumulative over rows
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // sigmoid(x) = tanh(x/2)/2 + 1/2 with x = a_exp (g + dt): the halving is exact, so it is folded into a_exp
            const float th = tanh_approx(__fmul_rn(a_exp_half, __fadd_rn(gv[i], dt[i])));
            const float gt = valid ? __fmul_rn(a.gate_scale, __fmaf_rn(th, 0.5f, 0.5f)) : 0.0f;
            csum[i] = __fadd_rn(csum[i], gt);
        }
        // decay application in bf16x2: one rounding per element and operation
        const uint32_t ep0 = pack_bf2(ex2_approx(csum[0]), ex2_approx(csum[1]));
        const uint32_t ep1 = pack_bf2(ex2_approx(csum[2]), ex2_approx(csum[3]));
        const uint32_t em0 = pack_bf2(ex2_approx(-csum[0]), ex2_approx(-csum[1]));
        const uint32_t em1 = pack_bf2(ex2_approx(-csum[2]), ex2_approx(-csum[3]));
        const uint2 kd = make_uint2(bf2_mul(kn0, ep0), bf2_mul(kn1, ep1));
        const uint2 qd = make_uint2(bf2_mul(bf2_mul(qn0, ep0), sc2), bf2_mul(bf2_mul(qn1, ep1), sc2));
        {
            const int off = tc_b1_off(r, lane >> 1) + (lane & 1) * 8;
            *reinterpret_cast<uint2*>(sm.b1 + off) = kd;
            *reinterpret_cast<uint2*>(sm.b1 + off + 2 * 128) = qd;  // rows 16..31 = two row groups further
            *reinterpret_cast<uint2*>(sm.kikr + (lane >> 1) * kPwKiLbo + (r >> 3) * 128 + (r & 7) * 16 + (lane & 1) * 8) =
                make_uint2(bf2_mul(kn0, em0), bf2_mul(kn1, em1));
        }
        if constexpr (!kTc) {
            *reinterpret_cast<uint2*>(ws + kWsKd + (r * kD + c4) * 2) = kd;
            *reinterpret_cast<uint2*>(ws + kWsQd + (r * kD + c4) * 2) = qd;
        }
    }
    }
    // E_tot now; kr = ki (*) bf(E_tot) is formed after the products have consumed the ki tile
    float et[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) et[i] = ex2_approx(csum[i]);
    *reinterpret_cast<float4*>(ws + (kTc ? kTcEt : kWsEt) + c4 * 4) = make_float4(et[0], et[1], et[2], et[3]);
    __syncwarp();
    // the head of the next unit travels while the in-chunk products and the inverse (no global loads) run
    if (next_valid) prep_prefetch(a, next_t0, next_len, next_h, lane, pf);

    // ---- L = fp16(kd ki^T) masked * fp16(beta), Mqk = bf16(qd ki^T) masked: mma.sync m16n8k16
    //      bf16 -> fp32, operand fragments fetched with conflict-free 32-bit loads ----
    Frag16 lfrag;  // L as the A / C fragment the inverse starts from
    {
        const int g = lane >> 2, t = lane & 3;
        float l0[4] = {0.f, 0.f, 0.f, 0.f}, l1[4] = {0.f, 0.f, 0.f, 0.f};
        float m0[4] = {0.f, 0.f, 0.f, 0.f}, m1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        // lane 8m + r addresses row r of the m-th 8x8 matrix of a fragment: matrix m of an A fragment is (row group
        // m & 1, K chunk m >> 1), matrix m of the B pair is (K chunk m & 1, row group m >> 1); rows are 16 bytes
        const int lr = lane & 7, lm = lane >> 3;
        const uint8_t* a_row = sm.b1 + (lm >> 1) * kTcB1Lbo + (lm & 1) * 128 + lr * 16;
        const uint8_t* b_row = sm.kikr + (lm & 1) * kPwKiLbo + (lm >> 1) * 128 + lr * 16;
#pragma unroll
        for (int j = 0; j < kD / 16; ++j) {
            uint32_t b00, b01, b10, b11;
            ldmatrix_x4(b00, b01, b10, b11, b_row + 2 * j * kPwKiLbo);
            {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(a0, a1, a2, a3, a_row + 2 * j * kTcB1Lbo);
                mma_bf16_f32acc(l0, a0, a1, a2, a3, b00, b01);  // columns 0-7
                mma_bf16_f32acc(l1, a0, a1, a2, a3, b10, b11);  // columns 8-15
            }
            {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(a0, a1, a2, a3, a_row + 2 * j * kTcB1Lbo + 256);  // qd = rows 16..31
                mma_bf16_f32acc(m0, a0, a1, a2, a3, b00, b01);
                mma_bf16_f32acc(m1, a0, a1, a2, a3, b10, b11);
            }
        }
        // fragment element e of n-tile nt: row = g + 8*(e>>1), column = 8*nt + 2*t + (e&1)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int i = g + 8 * hr, j = 8 * nt + 2 * t;
                const float x0 = nt ? l1[2 * hr] : l0[2 * hr], x1 = nt ? l1[2 * hr + 1] : l0[2 * hr + 1];
                const float y0 = nt ? m1[2 * hr] : m0[2 * hr], y1 = nt ? m1[2 * hr + 1] : m0[2 * hr + 1];
                const __half bh = __float2half_rn(sm.beta_act[i]);
                const __half h0 = (i > j) ? __hmul(__float2half_rn(x0), bh) : __float2half_rn(0.0f);
                const __half h1 = (i > j + 1) ? __hmul(__float2half_rn(x1), bh) : __float2half_rn(0.0f);
                const __half2 lh = __halves2half2(h0, h1);
                lfrag.r[hr + 2 * nt] = *reinterpret_cast<const uint32_t*>(&lh);
                const uint32_t m = pack_bf2((i >= j) ? y0 : 0.0f, (i >= j + 1) ? y1 : 0.0f);
                if constexpr (kTc)
                    *reinterpret_cast<uint32_t*>(ws + kTcMqk + tc_sq_off(i, j)) = m;
                else
                    *reinterpret_cast<uint32_t*>(ws + kWsMqk + (i * kChunk + j) * 2) = m;
            }
        }
    }
    __syncwarp();
    // ---- kr = ki (*) bf(E_tot): read my ki columns back, then overwrite the buffer in the KR layout ----
    {
        const uint32_t et0 = pack_bf2(et[0], et[1]), et1 = pack_bf2(et[2], et[3]);
        uint2 kr[kChunk];
#pragma unroll
        for (int r = 0; r < kChunk; ++r) {
            const uint2 ki = *reinterpret_cast<const uint2*>(sm.kikr + (lane >> 1) * kPwKiLbo + (r >> 3) * 128 +
                                                             (r & 7) * 16 + (lane & 1) * 8);
            kr[r] = make_uint2(bf2_mul(ki.x, et0), bf2_mul(ki.y, et1));
        }
        __syncwarp();
#pragma unroll
        for (int r = 0; r < kChunk; ++r) {
            if constexpr (kTc)
                *reinterpret_cast<uint2*>(sm.kikr + tc_kr_off(r, lane >> 1) + (lane & 1) * 8) = kr[r];
            else
                *reinterpret_cast<uint2*>(ws + kWsKr + (r * kD + c4) * 2) = kr[r];
        }
    }
    if constexpr (kTc && !kRecordInSmem) {  // ship [kd; qd] and kr: two bulk copies shared memory -> workspace record
        sm100::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            sm100::bulk_s2g(ws + kTcB1, sm.b1, kTcB1Bytes);
            sm100::bulk_s2g(ws + kTcKr, sm.kikr, kTcKrBytes);
            sm100::bulk_commit_group();
        }
    }
    neumann_inverse_warp<kTc>(lfrag, ws + (kTc ? kTcInv : kWsInv), lane);
    if constexpr (kTc && !kRecordInSmem) {  // the tiles are rewritten by the next chunk: the copies must have read them
        if (lane == 0) sm100::bulk_wait_group_read<0>();
    }
    __syncwarp();
}

// Grid-stride kernel: warp w of the grid takes (chunk, head) pairs w, w + W, ... with the head index
// fastest, so that neighbouring warps read neighbouring 256-byte rows.
constexpr int kPwWarpsPerCta = 16;
template <bool kTc>
__global__ void __launch_bounds__(kPwWarpsPerCta * 32, 1) prepare_warp_kernel(const __grid_constant__ TwoPassArgs a) {
    // (a ragged batch that the fused short-sequence kernel has served: nothing to do)
    if (a.short_flag != nullptr && *a.short_flag != 0) return;
    extern __shared__ __align__(16) uint8_t pw_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    PrepWarpSmem& sm = reinterpret_cast<PrepWarpSmem*>(pw_smem)[warp];
    // units = (chunk, head) pairs, head fastest; with a slab (fixed batches) only chunks [slab_c0, slab_c0 +
    // slab_chunks) of every sequence, enumerated densely
    const int64_t tps = (a.T + kChunk - 1) / kChunk;  // chunks per sequence of a fixed batch
    const int64_t n_units = (a.slab_chunks > 0 ? a.N * (int64_t)a.slab_chunks : a.total_tiles) * a.H;
    const int64_t stride = (int64_t)gridDim.x * kPwWarpsPerCta;
    // units past the last chunk of a ragged batch (upper-bound tile count) all sit at the end of the range
    auto locate = [&](int64_t u, int64_t* tile, int64_t* t0, int* len, int* h) {
        if (u >= n_units) return false;
        int64_t t = u / a.H;
        *h = (int)(u - t * a.H);
        if (a.slab_chunks > 0) {
            const int64_t n = t / a.slab_chunks;
            t = n * tps + a.slab_c0 + (t - n * a.slab_chunks);
        }
        *tile = t;
        return locate_tile(a, t, t0, len);
    };
    int64_t u = (int64_t)blockIdx.x * kPwWarpsPerCta + warp;
    int64_t tile = 0, tile_n = 0, t0 = 0, t0n = 0;
    int len = 0, h = 0, lenn = 0, hn = 0;
    bool valid = locate(u, &tile, &t0, &len, &h);
    PrepPrefetch pf;
    if (valid) prep_prefetch(a, t0, len, h, lane, pf);
    while (valid) {
        const bool next_valid = locate(u + stride, &tile_n, &t0n, &lenn, &hn);
        uint8_t* ws = a.workspace + ((int64_t)h * a.total_tiles + tile) * (int64_t)(kTc ? kTcRecord : kWsRecord);
        prepare_chunk_warp<kTc>(a, t0, len, h, ws, sm, lane, pf, next_valid, t0n, lenn, hn);
        u += stride;
        valid = next_valid;
        tile = tile_n; t0 = t0n; len = lenn; h = hn;
    }
    sm100::bulk_wait_group<0>();  // (lane 0) the last records have landed
}

// max_ctas > 0 caps the grid (a launch that shares the GPU with a concurrent recurrence kernel)
template <bool kTc>
inline int launch_prepare_warp(const TwoPassArgs& a, cudaStream_t stream, int max_ctas = 0) {
    const int smem = (int)sizeof(PrepWarpSmem) * kPwWarpsPerCta;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaFuncSetAttribute(prepare_warp_kernel<kTc>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return FKDA_ERR_LAUNCH;
    const int64_t n_units = (a.slab_chunks > 0 ? a.N * (int64_t)a.slab_chunks : a.total_tiles) * a.H;
    int64_t ctas = (n_units + kPwWarpsPerCta - 1) / kPwWarpsPerCta;
    if (ctas > sms) ctas = sms;
    if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;
    prepare_warp_kernel<kTc><<<(unsigned)ctas, kPwWarpsPerCta * 32, smem, stream>>>(a);
    return FKDA_OK;
}

}  // namespace fkda
