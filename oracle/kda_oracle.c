/*
 * CPU oracle for the Kimi Delta Attention forward pass (K = V = 128, chunk 16).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is
 * compared with; nothing in the shipped library links, loads or calls it.
 *
 * It restates, in plain C, the algorithm of the reference's executable
 * numerics contract tests/torch_ref.py (function torch_ref, lines 124-251) with
 * every rounding point kept: bf16 after each element-wise op, fp32
 * accumulation in the contractions, fp16 operands and results in the 16x16
 * inverse, and a bf16 state that is re-rounded after every 16-token chunk.
 *
 * Deliberate substitutions (the reference computes these on a GPU):
 *   - sigmoid(x) = tanh.approx.f32(x/2)/2 + 1/2   -> tanhf(x/2)/2 + 1/2
 *     (tests/torch_ref.py:12-21)
 *   - the fp16-accumulate cuBLAS GEMM of the inverse -> fp32 accumulate, one
 *     rounding to fp16 per product matrix (tests/torch_ref.py:57-76)
 *   - rsqrt -> 1/sqrtf, exp2 -> exp2f with flush-to-zero
 * Because of the exact-vs-approximate transcendental difference the oracle is
 * compared with GPU results under a tolerance, not bit for bit.
 *
 * Parity pin: checked against fixtures produced by executing the reference's
 * own torch_ref text on the CPU (tests/golden/make_golden.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define D 128
#define CHUNK 16
#define LOG2E 1.4426950408889634

typedef uint16_t bf16_t;
typedef _Float16 fp16_t;

/* ---- scalar format helpers ------------------------------------------------ */

static inline float bf2f(bf16_t x) {
    uint32_t u = (uint32_t)x << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16 (the conversion torch's .to(bfloat16) does) */
static inline bf16_t f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x40); /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (bf16_t)(u >> 16);
}

/* bf16 (x) bf16 -> bf16, computed in fp32 then rounded once (torch bf16 mul) */
static inline bf16_t bfmul(bf16_t a, bf16_t b) { return f2bf(bf2f(a) * bf2f(b)); }
static inline bf16_t bfadd(bf16_t a, bf16_t b) { return f2bf(bf2f(a) + bf2f(b)); }
static inline bf16_t bfsub(bf16_t a, bf16_t b) { return f2bf(bf2f(a) - bf2f(b)); }

/* tests/torch_ref.py:86-91 fp32_ex2_ftz: exp2 with subnormal results flushed */
static inline float ex2_ftz(float x) {
    float r = exp2f(x);
    if (fabsf(r) < 1.17549435e-38f) r = 0.0f;
    return r;
}

/* tests/torch_ref.py:12-21 sigmoid through tanh (exact tanh here) */
static inline float sigmoid_tanh(float x) {
    float th = tanhf(x * 0.5f);
    return th * 0.5f + 0.5f;
}

/* ---- tests/torch_ref.py:101-117 l2_normalize_kernel_match ----------------- */
/* 16 lanes x 8 elements: per-lane FMA chain, xor butterfly 8,4,2,1, rsqrt(s+1e-6),
 * fp32 multiply, one rounding to bf16. */
static void l2_normalize_row(const bf16_t* x, bf16_t* y) {
    float xf[D], part[16], tmp[16];
    for (int i = 0; i < D; ++i) xf[i] = bf2f(x[i]);
    for (int l = 0; l < 16; ++l) {
        float s = 0.0f;
        for (int i = 0; i < 8; ++i) s = fmaf(xf[l * 8 + i], xf[l * 8 + i], s);
        part[l] = s;
    }
    for (int off = 8; off >= 1; off >>= 1) {
        for (int l = 0; l < 16; ++l) tmp[l] = part[l] + part[l ^ off];
        memcpy(part, tmp, sizeof(part));
    }
    float inv = 1.0f / sqrtf(part[0] + 1e-6f);
    for (int i = 0; i < D; ++i) y[i] = f2bf(xf[i] * inv);
}

/* C[16x16] = A[16x16] * B[16x16], fp16 operands, fp32 accumulate, fp16 result
 * (stand-in for tests/torch_ref.py:57-76 matmul_fp16acc) */
static void mm16_h(const fp16_t* A, const fp16_t* B, fp16_t* C) {
    for (int i = 0; i < CHUNK; ++i)
        for (int j = 0; j < CHUNK; ++j) {
            float s = 0.0f;
            for (int k = 0; k < CHUNK; ++k) s += (float)A[i * CHUNK + k] * (float)B[k * CHUNK + j];
            C[i * CHUNK + j] = (fp16_t)s;
        }
}

/* ---- one (sequence, head) chain: tests/torch_ref.py:179-245 ---------------- */
typedef struct {
    const bf16_t *q, *k, *v, *g, *beta;
    bf16_t* out;
    const float *A_log, *dt_bias;
    float gate_scale; /* float(lower_bound * log2(e)), csrc/flash_kda.cpp:128 */
    bf16_t scale_bf16;
    int64_t H;
} chain_args_t;

static void run_chain(const chain_args_t* a, int64_t bos, int64_t eos, int64_t h, bf16_t* S /* [V][K] */) {
    const int64_t H = a->H;
    /* tests/torch_ref.py:163 a_log_exp = exp2(A_log * log2e) in fp32 */
    const float a_log_exp = ex2_ftz(a->A_log[h] * (float)LOG2E);
    const float* dtb = a->dt_bias + h * D;
    const int64_t seq_len = eos - bos;
    const int64_t n_chunks = (seq_len + CHUNK - 1) / CHUNK;

    bf16_t(*qn)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*kn)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*vc)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*kd)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*qd)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*ki)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*kr)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*U)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    bf16_t(*o0)[D] = malloc(sizeof(bf16_t) * CHUNK * D);
    float(*G)[D] = malloc(sizeof(float) * CHUNK * D);
    float* delta = malloc(sizeof(float) * D * D); /* [K][V] */

    for (int64_t c = 0; c < n_chunks; ++c) {
        const int64_t t0 = bos + c * CHUNK;
        const int len = (int)((eos - t0) < CHUNK ? (eos - t0) : CHUNK);
        float beta_act[CHUNK];

        /* zero-padded chunk tiles (tests/torch_ref.py:191-201), q/k normalised
         * (:153-154), gate activation (:160-164) */
        for (int i = 0; i < CHUNK; ++i) {
            if (i < len) {
                const int64_t off = ((t0 + i) * H + h) * D;
                l2_normalize_row(a->q + off, qn[i]);
                l2_normalize_row(a->k + off, kn[i]);
                memcpy(vc[i], a->v + off, sizeof(bf16_t) * D);
                for (int d = 0; d < D; ++d) {
                    float x = bf2f(a->g[off + d]) + dtb[d];
                    G[i][d] = a->gate_scale * sigmoid_tanh(a_log_exp * x);
                }
                beta_act[i] = sigmoid_tanh(bf2f(a->beta[(t0 + i) * H + h]));
            } else {
                memset(qn[i], 0, sizeof(bf16_t) * D);
                memset(kn[i], 0, sizeof(bf16_t) * D);
                memset(vc[i], 0, sizeof(bf16_t) * D);
                for (int d = 0; d < D; ++d) G[i][d] = 0.0f;
                beta_act[i] = sigmoid_tanh(0.0f);
            }
        }
        /* in-chunk cumulative sum over the 16 rows (:203) */
        for (int i = 1; i < CHUNK; ++i)
            for (int d = 0; d < D; ++d) G[i][d] = G[i - 1][d] + G[i][d];

        /* decay application (:204-210) */
        float e_tot[D];
        bf16_t e_tot_bf[D];
        const bf16_t sc = a->scale_bf16;
        for (int d = 0; d < D; ++d) {
            e_tot[d] = ex2_ftz(G[CHUNK - 1][d]);
            e_tot_bf[d] = f2bf(e_tot[d]);
        }
        for (int i = 0; i < CHUNK; ++i)
            for (int d = 0; d < D; ++d) {
                bf16_t ep = f2bf(ex2_ftz(G[i][d]));
                bf16_t em = f2bf(ex2_ftz(-G[i][d]));
                kd[i][d] = bfmul(kn[i][d], ep);
                qd[i][d] = bfmul(bfmul(qn[i][d], ep), sc);
                ki[i][d] = bfmul(kn[i][d], em);
                kr[i][d] = bfmul(ki[i][d], e_tot_bf[d]);
            }

        /* L = fp16(kd ki^T), Mqk = bf16(qd ki^T), fp32 accumulation (:211-212) */
        fp16_t L[CHUNK * CHUNK], INV[CHUNK * CHUNK], L2[CHUNK * CHUNK], L4[CHUNK * CHUNK], L8[CHUNK * CHUNK],
            P[CHUNK * CHUNK];
        bf16_t Mqk[CHUNK][CHUNK], INVb[CHUNK][CHUNK];
        for (int i = 0; i < CHUNK; ++i)
            for (int j = 0; j < CHUNK; ++j) {
                float sl = 0.0f, sm = 0.0f;
                for (int d = 0; d < D; ++d) {
                    float kj = bf2f(ki[j][d]);
                    sl += bf2f(kd[i][d]) * kj;
                    sm += bf2f(qd[i][d]) * kj;
                }
                /* strict lower triangle times fp16(beta_i); Mqk lower incl. diagonal (:215-219) */
                L[i * CHUNK + j] = (i > j) ? (fp16_t)((float)(fp16_t)sl * (float)(fp16_t)beta_act[i]) : (fp16_t)0.0f;
                Mqk[i][j] = (i >= j) ? f2bf(sm) : (bf16_t)0;
            }
        /* (I + L)^-1 = (I - L)(I + L^2)(I + L^4)(I + L^8) in fp16 (:221-227) */
        for (int i = 0; i < CHUNK; ++i)
            for (int j = 0; j < CHUNK; ++j)
                INV[i * CHUNK + j] = (fp16_t)((i == j ? 1.0f : 0.0f) - (float)L[i * CHUNK + j]);
        mm16_h(L, L, L2);
        mm16_h(INV, L2, P);
        for (int x = 0; x < CHUNK * CHUNK; ++x) INV[x] = (fp16_t)((float)INV[x] + (float)P[x]);
        mm16_h(L2, L2, L4);
        mm16_h(INV, L4, P);
        for (int x = 0; x < CHUNK * CHUNK; ++x) INV[x] = (fp16_t)((float)INV[x] + (float)P[x]);
        mm16_h(L4, L4, L8);
        mm16_h(INV, L8, P);
        for (int x = 0; x < CHUNK * CHUNK; ++x) INV[x] = (fp16_t)((float)INV[x] + (float)P[x]);
        for (int i = 0; i < CHUNK; ++i)
            for (int j = 0; j < CHUNK; ++j) INVb[i][j] = f2bf((float)INV[i * CHUNK + j]); /* :229 */

        /* u' = (v - bf16(kd S^T)) * bf16(beta); o0 = bf16(qd S^T) (:231-237) */
        for (int i = 0; i < CHUNK; ++i) {
            const bf16_t bb = f2bf(beta_act[i]);
            for (int vv = 0; vv < D; ++vv) {
                float su = 0.0f, so = 0.0f;
                const bf16_t* Srow = S + vv * D;
                for (int d = 0; d < D; ++d) {
                    float s = bf2f(Srow[d]);
                    su += bf2f(kd[i][d]) * s;
                    so += bf2f(qd[i][d]) * s;
                }
                vc[i][vv] = bfmul(bfsub(vc[i][vv], f2bf(su)), bb);
                o0[i][vv] = f2bf(so);
            }
        }
        /* U = bf16(INV u') (:236) */
        for (int i = 0; i < CHUNK; ++i)
            for (int vv = 0; vv < D; ++vv) {
                float s = 0.0f;
                for (int j = 0; j < CHUNK; ++j) s += bf2f(INVb[i][j]) * bf2f(vc[j][vv]);
                U[i][vv] = f2bf(s);
            }
        /* out = o0 (+) bf16(Mqk U), valid rows only (:237-238, :245) */
        for (int i = 0; i < len; ++i) {
            const int64_t off = ((t0 + i) * H + h) * D;
            for (int vv = 0; vv < D; ++vv) {
                float s = 0.0f;
                for (int j = 0; j < CHUNK; ++j) s += bf2f(Mqk[i][j]) * bf2f(U[j][vv]);
                a->out[off + vv] = bfadd(o0[i][vv], f2bf(s));
            }
        }
        /* state: S[v][k] = bf16(fma(S[v][k], E_tot[k], sum_i kr[i][k] U[i][v])) (:239-243) */
        for (int d = 0; d < D; ++d)
            for (int vv = 0; vv < D; ++vv) {
                float s = 0.0f;
                for (int i = 0; i < CHUNK; ++i) s += bf2f(kr[i][d]) * bf2f(U[i][vv]);
                delta[d * D + vv] = s;
            }
        for (int vv = 0; vv < D; ++vv)
            for (int d = 0; d < D; ++d) S[vv * D + d] = f2bf(fmaf(bf2f(S[vv * D + d]), e_tot[d], delta[d * D + vv]));
    }
    free(qn); free(kn); free(vc); free(kd); free(qd); free(ki); free(kr); free(U); free(o0); free(G); free(delta);
}

/*
 * Whole forward, same argument meaning as flash_kda.fwd (flash_kda/__init__.py:5-41).
 * Tensors are row-major [B, T, H, 128] bf16 bit patterns (beta [B, T, H]);
 * states are [N, H, V, K]; state_dtype 0 = bf16, 1 = fp32.  cu_seqlens may be
 * NULL (then N = B sequences of length T).  Returns 0, or a negative value for
 * a bad argument.
 */
int kda_oracle_fwd(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* g, const uint16_t* beta,
                   float scale, uint16_t* out, const float* A_log, const float* dt_bias, double lower_bound,
                   const void* initial_state, void* final_state, int state_dtype, const int64_t* cu_seqlens,
                   int64_t B, int64_t T, int64_t H, int64_t N, int n_threads) {
    if (!q || !k || !v || !g || !beta || !out || !A_log || !dt_bias) return -1;
    if (cu_seqlens && B != 1) return -2;
    if (!cu_seqlens && N != B) return -3;
    chain_args_t a = {q, k, v, g, beta, out, A_log, dt_bias, (float)(lower_bound * LOG2E), f2bf(scale), H};
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
    const int64_t n_chains = N * H;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t c = 0; c < n_chains; ++c) {
        const int64_t n = c / H, h = c % H;
        const int64_t bos = cu_seqlens ? cu_seqlens[n] : n * T;
        const int64_t eos = cu_seqlens ? cu_seqlens[n + 1] : (n + 1) * T;
        bf16_t* S = malloc(sizeof(bf16_t) * D * D);
        const int64_t soff = (n * H + h) * D * D;
        /* tests/torch_ref.py:174-177: fp32 initial state is rounded to bf16 on entry */
        if (initial_state) {
            if (state_dtype == 1)
                for (int x = 0; x < D * D; ++x) S[x] = f2bf(((const float*)initial_state)[soff + x]);
            else
                memcpy(S, (const bf16_t*)initial_state + soff, sizeof(bf16_t) * D * D);
        } else {
            memset(S, 0, sizeof(bf16_t) * D * D);
        }
        run_chain(&a, bos, eos, h, S);
        /* tests/torch_ref.py:247-251: fp32 final state is the bf16 state widened */
        if (final_state) {
            if (state_dtype == 1)
                for (int x = 0; x < D * D; ++x) ((float*)final_state)[soff + x] = bf2f(S[x]);
            else
                memcpy((bf16_t*)final_state + soff, S, sizeof(bf16_t) * D * D);
        }
        free(S);
    }
    return 0;
}

int kda_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
