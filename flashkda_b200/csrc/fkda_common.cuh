// Shared device helpers for the KDA forward kernels (sm_100a).
//
// The numerics follow the reference's executable contract (tests/torch_ref.py:124-251
// and the device helpers csrc/smxx/utils.cuh:38-59): the same approximate PTX
// transcendentals, one bf16 rounding after every element-wise bf16 operation, fp32
// accumulation in contractions, fp16 in the 16x16 inverse.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fkda {

constexpr int kD = 128;     // K = V
constexpr int kChunk = 16;  // tokens per recurrence step

// Bytes of one (head, chunk) record in the two-pass workspace:
// kd, qd, kr [16,128] bf16; E_tot [128] f32; INV, Mqk [16,16] bf16.
constexpr int kWsKd = 0;
constexpr int kWsQd = kWsKd + kChunk * kD * 2;
constexpr int kWsKr = kWsQd + kChunk * kD * 2;
constexpr int kWsEt = kWsKr + kChunk * kD * 2;
constexpr int kWsInv = kWsEt + kD * 4;
constexpr int kWsMqk = kWsInv + kChunk * kChunk * 2;
constexpr int kWsRecord = kWsMqk + kChunk * kChunk * 2;  // 13824
static_assert(kWsRecord == 13824, "workspace record size");

// Record of the tensor-core two-pass workspace: operand tiles in the no-swizzle UMMA canonical
// layouts (8 x 16-byte "core matrices" of 128 contiguous bytes).  The strides between core matrices are
// padded by 16 bytes so that the prepare stage, whose lanes own columns, fills the same tiles in shared
// memory without bank conflicts and ships them with bulk copies:
//   B1  [kd; qd] as the K-major B operand [32 rows, K=128]: byte = (k/8)*528 + (r/8)*128 + (r%8)*16 + (k%8)*2
//   KR  kr as the MN-major operand [128 k, 16 tokens]:      byte = (i/8)*2304 + (n/8)*144 + (i%8)*16 + (n%8)*2
//   INV, MQK as K-major B operands [16, 16]:                byte = (j/8)*256 + (i/8)*128 + (i%8)*16 + (j%8)*2
//   ET  E_tot [128] f32;  BETA sigmoid(beta) [16] bf16 (in a 64-byte slot)
constexpr int kTcB1Lbo = 528;                   // between the 16-byte K chunks of B1
constexpr int kTcB1Bytes = 16 * kTcB1Lbo;       // 8448
constexpr int kTcKrSbo = 144;                   // between 8-column groups of KR
constexpr int kTcKrLbo = 16 * kTcKrSbo;         // 2304, between the two 8-token groups
constexpr int kTcKrBytes = 2 * kTcKrLbo;        // 4608
constexpr int kTcB1 = 0;
constexpr int kTcKr = kTcB1 + kTcB1Bytes;       // 8448
constexpr int kTcInv = kTcKr + kTcKrBytes;      // 13056
constexpr int kTcMqk = kTcInv + 512;            // 13568
constexpr int kTcEt = kTcMqk + 512;             // 14080
constexpr int kTcBeta = kTcEt + 512;            // 14592
constexpr int kTcRecord = kTcBeta + 64;         // 14656
static_assert(kTcRecord % 16 == 0, "bulk copies move multiples of 16 bytes");
__host__ __device__ constexpr int tc_b1_off(int r, int kc) { return kc * kTcB1Lbo + (r >> 3) * 128 + (r & 7) * 16; }
__host__ __device__ constexpr int tc_kr_off(int i, int nc) { return (i >> 3) * kTcKrLbo + nc * kTcKrSbo + (i & 7) * 16; }
__host__ __device__ constexpr int tc_sq_off(int i, int j) {
    return (j >> 3) * 256 + (i >> 3) * 128 + (i & 7) * 16 + (j & 7) * 2;
}

// ---- approximate transcendentals: the instructions are part of the contract ----
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float tanh_approx(float x) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
    float r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// sigmoid(x) = tanh(x/2)/2 + 1/2  (csrc/smxx/utils.cuh:50-53)
__device__ __forceinline__ float sigmoid_tanh(float x) {
    float th = tanh_approx(x * 0.5f);
    return __fmaf_rn(th, 0.5f, 0.5f);
}

// Two independent fp32 fused multiply-adds in one instruction (sm_100 packed fp32 pipe): d = a * b + c per half,
// each rounded to nearest-even exactly like fma.rn.f32.
__device__ __forceinline__ void fma2_rn(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n.reg .b64 ra, rb, rc, rd;\nmov.b64 ra, {%2,%3};\nmov.b64 rb, {%4,%5};\nmov.b64 rc, {%6,%7};\n"
        "fma.rn.ftz.f32x2 rd, ra, rb, rc;\nmov.b64 {%0,%1}, rd;\n}\n"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}

// ---- bf16 helpers: every op rounds to nearest-even once ----
__device__ __forceinline__ float bf2f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float x) { return __float2bfloat16_rn(x); }
__device__ __forceinline__ __nv_bfloat16 bfmul(__nv_bfloat16 a, __nv_bfloat16 b) { return f2bf(bf2f(a) * bf2f(b)); }
__device__ __forceinline__ __nv_bfloat16 bfadd(__nv_bfloat16 a, __nv_bfloat16 b) { return f2bf(bf2f(a) + bf2f(b)); }
__device__ __forceinline__ __nv_bfloat16 bfsub(__nv_bfloat16 a, __nv_bfloat16 b) { return f2bf(bf2f(a) - bf2f(b)); }

__device__ __forceinline__ float bfbits2f(uint32_t hi16) { return __uint_as_float(hi16 << 16); }
__device__ __forceinline__ float bf_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// packed bf16x2 arithmetic: one round-to-nearest-even per element, as the scalar helpers above
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// ---- warp-level mma.sync m16n8k16, fp16 operands AND fp16 accumulators ----
// (the instruction the reference's inverse uses: csrc/smxx/utils.cuh:199-260)
__device__ __forceinline__ void mma_f16_f16acc(uint32_t& d0, uint32_t& d1, uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1, uint32_t c0, uint32_t c1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%9};\n"
        : "=r"(d0), "=r"(d1)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}
// bf16 operands, fp32 accumulators
// Four 8x8 b16 matrices from shared memory into mma.sync fragment registers: lane 8m + r gives the address of
// row r (16 bytes) of matrix m; thread (g = lane / 4, t = lane % 4) receives elements (g, 2t), (g, 2t + 1) of each.
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* row_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_f32acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
    __half2 x = *reinterpret_cast<__half2*>(&a), y = *reinterpret_cast<__half2*>(&b);
    __half2 z = __hadd2(x, y);
    return *reinterpret_cast<uint32_t*>(&z);
}

// 16x16 fp16 matrices held by one warp as mma.sync fragments.  A / C fragment of a row-major X:
// regs {X[g][2t..], X[g+8][2t..], X[g][2t+8..], X[g+8][2t+8..]} with g = lane / 4, t = lane % 4.
struct Frag16 {
    uint32_t r[4];
};
// Transposes each 8x8 tile of a fragment in registers: turns the C (= A) fragment of a 16x16 row-major matrix
// into its B fragment (tile (rows 8i.., cols 8j..) of register i + 2j becomes the pair column of the same register).
__device__ __forceinline__ Frag16 c_to_b_frag_h(const Frag16& c) {
    Frag16 b;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(b.r[i]) : "r"(c.r[i]));
    return b;
}
__device__ __forceinline__ Frag16 mma16x16_h(const Frag16& a, const Frag16& b) {
    Frag16 c;
    mma_f16_f16acc(c.r[0], c.r[1], a.r[0], a.r[1], a.r[2], a.r[3], b.r[0], b.r[1], 0u, 0u);
    mma_f16_f16acc(c.r[2], c.r[3], a.r[0], a.r[1], a.r[2], a.r[3], b.r[2], b.r[3], 0u, 0u);
    return c;
}

// Inverse of the unit lower-triangular (I + L), L strictly lower 16x16 fp16, by one warp:
//   (I + L)^-1 = (I - L)(I + L^2)(I + L^4)(I + L^8)
// with fp16 products/accumulators and fp16 additions, result rounded to bf16
// (csrc/smxx/utils.cuh:262-311; tests/torch_ref.py:221-229).
// L: the matrix as an mma.sync A / C fragment (what the product that forms it leaves in registers); inv_out:
// bf16 [16][16], dense row-major (kCanonical = false) or in the UMMA canonical K-major layout (tc_sq_off).
// All 32 lanes of the warp must call.
template <bool kCanonical>
__device__ __forceinline__ void neumann_inverse_warp(const Frag16& L, uint8_t* inv_out, int lane) {
    const int g = lane >> 2, t = lane & 3;
    // INV0 = I - L in C-fragment coordinates (register i: row g + 8 (i & 1), columns 2t + 8 (i >> 1), + 1)
    Frag16 inv_c;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = g + 8 * (i & 1), c = 2 * t + 8 * (i >> 1);
        const __half2 x = *reinterpret_cast<const __half2*>(&L.r[i]);
        const __half one = __float2half_rn(1.0f);
        const __half e0 = (r == c) ? __hsub(one, __low2half(x)) : __hneg(__low2half(x));
        const __half e1 = (r == c + 1) ? __hsub(one, __high2half(x)) : __hneg(__high2half(x));
        const __half2 v = __halves2half2(e0, e1);
        inv_c.r[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
    // A-fragment and C-fragment register layouts coincide for a 16x16 row-major matrix
    // (regs: [g][2t], [g+8][2t], [g][2t+8], [g+8][2t+8]), so L and INV can be used as A directly.
    Frag16 pow_a = L;
    Frag16 pow_b = c_to_b_frag_h(pow_a);         // the powers stay in registers: B fragments by register transposes
#pragma unroll
    for (int step = 0; step < 3; ++step) {
        Frag16 p2 = mma16x16_h(pow_a, pow_b);  // L^(2^(step+1))
        pow_b = c_to_b_frag_h(p2);
        pow_a = p2;
        Frag16 m = mma16x16_h(inv_c, pow_b);  // INV * L^(2^(step+1))
#pragma unroll
        for (int i = 0; i < 4; ++i) inv_c.r[i] = hadd2_u32(inv_c.r[i], m.r[i]);
    }
    auto st = [&](int r, int c, uint32_t packed) {
        __half2 h = *reinterpret_cast<__half2*>(&packed);
        float2 f = __half22float2(h);
        const int off = kCanonical ? tc_sq_off(r, c) : (r * kChunk + c) * 2;
        *reinterpret_cast<uint32_t*>(inv_out + off) = pack_bf2(f.x, f.y);
    };
    st(g, 2 * t, inv_c.r[0]);
    st(g + 8, 2 * t, inv_c.r[1]);
    st(g, 2 * t + 8, inv_c.r[2]);
    st(g + 8, 2 * t + 8, inv_c.r[3]);
}

}  // namespace fkda
