/*
 * flashkda_b200 — C ABI of the B200 (sm_100a) Kimi Delta Attention forward.
 *
 * Plain pointers and sizes only; every pointer is DEVICE memory unless stated
 * otherwise.  All entry points enqueue work on the CUDA stream they are given
 * and return without synchronising (the contract of the reference operator,
 * csrc/flash_kda.cpp:136).  A return value of 0 means success; any other value
 * is one of the FKDA_ERR_* codes (fkda_status_string() names them).
 *
 * Reference interfaces replaced (paths within the reference project):
 *   fkda_fwd              <- fwd(...)               csrc/flash_kda.cpp:28-217
 *                            launch_fwd<...>(...)   csrc/fwd.h:6-27
 *   fkda_workspace_bytes  <- get_workspace_size()   csrc/flash_kda.cpp:5-26
 */
#ifndef FLASHKDA_B200_H_
#define FLASHKDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FKDA_HEAD_DIM 128 /* K = V = 128 (csrc/flash_kda.cpp:110) */
#define FKDA_CHUNK 16     /* tokens per recurrence step (csrc/flash_kda.cpp:138) */

enum {
    FKDA_OK = 0,
    FKDA_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
    FKDA_ERR_BAD_SHAPE = 2,      /* B, T, H, N or a stride is out of range */
    FKDA_ERR_BAD_STATE_DTYPE = 3,
    FKDA_ERR_VARLEN_BATCH = 4,   /* cu_seqlens given but B != 1 */
    FKDA_ERR_WORKSPACE = 5,      /* workspace missing or too small */
    FKDA_ERR_BAD_ALGO = 6,
    FKDA_ERR_LAUNCH = 7,         /* a kernel launch or CUDA runtime call failed */
    FKDA_ERR_ALIGNMENT = 8,      /* a tensor base address or stride is not 16-byte aligned */
    FKDA_ERR_DEVICE_STATUS = 9,  /* a kernel gave up on a bounded internal wait */
    FKDA_ERR_NOALLOC_TOO_LARGE = 10 /* problem needs more scratch than fkda_fwd_noalloc has built in */
};

enum { FKDA_STATE_BF16 = 0, FKDA_STATE_FP32 = 1 };

enum { FKDA_PHASE_PREPARE = 1, FKDA_PHASE_RECURRENCE = 2 };

/* Which device implementation runs. */
enum {
    FKDA_ALGO_AUTO = 0,
    FKDA_ALGO_TWOPASS = 1, /* prepare kernel -> HBM workspace -> recurrence kernel (CUDA cores) */
    FKDA_ALGO_TC = 2       /* prepare kernel -> HBM workspace -> persistent tcgen05/TMEM recurrence; a fixed batch
                              with T == 1 (decode step) runs one state read-modify-write kernel instead, one with
                              2 <= T <= 16 one fused kernel per (sequence, head) */
};

/*
 * Arguments of one forward call; mirrors flash_kda.fwd (flash_kda/__init__.py:5).
 * Token-major tensors are addressed as
 *     x[token][head][d]  at  x + token * token_stride + head * 128 + d     (bf16 elements)
 *     beta[token][head]  at  beta + token * beta_token_stride + head
 * with token = b * T + t.  Dense tensors use token_stride = H * 128 and
 * beta_token_stride = H; a larger stride addresses a head-slice of a wider tensor
 * without a copy.  States are dense [N, H, 128 (V), 128 (K)].
 */
typedef struct fkda_fwd_params {
    const void* q;             /* bf16 */
    const void* k;             /* bf16 */
    const void* v;             /* bf16 */
    const void* g;             /* bf16, gate before activation */
    const void* beta;          /* bf16, beta logits */
    void* out;                 /* bf16, written in place */
    const float* A_log;        /* [H] */
    const float* dt_bias;      /* [H, 128] */
    const void* initial_state; /* NULL = start from zero */
    void* final_state;         /* NULL = not exported */
    int32_t state_dtype;       /* FKDA_STATE_*: dtype of whichever states are given */
    int32_t algo;              /* FKDA_ALGO_* */
    const int64_t* cu_seqlens; /* [N + 1] device int64, or NULL for B sequences of length T */
    int64_t B, T, H, N;        /* N = number of sequences (= B when cu_seqlens is NULL) */
    int64_t token_stride;      /* elements between consecutive tokens of q/k/v/g/out */
    int64_t beta_token_stride; /* elements between consecutive tokens of beta */
    float scale;
    double lower_bound;        /* gate lower bound, -5 <= lower_bound <= 0 */
    void* workspace;           /* >= fkda_workspace_bytes(B*T, H, N, algo) bytes, 256-byte aligned */
    size_t workspace_bytes;
    int32_t phase_mask;        /* measurement aid for multi-kernel algos: 0 = whole forward; otherwise a
                                  bit set of FKDA_PHASE_* to launch (the workspace must then already hold
                                  what the skipped phases produce) */
    int32_t flags;             /* 0 for normal use; FKDA_FLAG_* bits select kernel variants for tests and tuning */
    void* chunk_states;        /* optional bf16 [slots, H, 128 (V), 128 (K)]: the state of every sequence BEFORE each group
                                  of `chunk_states_every` chunks (16 * every tokens), i.e. before tokens 0, 16*every,
                                  2*16*every, ... of the sequence; a sequence of L tokens fills ceil(L / (16*every))
                                  consecutive slots, sequences follow each other in order (fixed batches: every
                                  sequence ceil(T / (16*every)) slots).  NULL = not exported.  This is what FLA's
                                  chunk_kda returns as `h` with return_intermediate_states (chunk size 64: every = 4);
                                  the reference operator has no such output. */
    int32_t chunk_states_every; /* >= 1 when chunk_states is given */
    int32_t reserved;
} fkda_fwd_params;

/* fkda_fwd_params.flags.  All zero is the production setting. */
enum {
    FKDA_FLAG_NO_DECODE = 1,       /* run a T == 1 batch through the chunked kernels instead of the decode kernel */
    FKDA_FLAG_NO_WIDE = 2,         /* never pick the one-chain-per-CTA recurrence */
    FKDA_FLAG_NO_SLABS = 4,        /* no slab pipeline (prepare of the next slab beside the recurrence) */
    FKDA_FLAG_NO_SHORT = 8,        /* run a batch of sequences of at most 16 tokens each through the general kernels */
    FKDA_FLAG_TEST_DROP_PUSH = 16  /* TEST ONLY: finished segments do not queue their follow-up, so that the
                                      work queue starves and its bounded waits give up */
};
/* bits 8..15: segment length of the work queue in chunks (0 = automatic; tuning aid)
 * bits 16..29: limit of every bounded device-side wait in milliseconds (0 = the default of 2000) */
#define FKDA_FLAGS_SEG_CHUNKS(x) (((x) & 0xff) << 8)
#define FKDA_FLAGS_WAIT_MS(x) (((x) & 0x3fff) << 16)

/* Scratch bytes one call needs (0 is a valid answer).  Replaces get_workspace_size
 * (csrc/flash_kda.cpp:5-26): same arguments plus the implementation selector. */
size_t fkda_workspace_bytes(int64_t T_total, int64_t H, int64_t N, int32_t algo);

/* Scratch bytes THIS call needs (<= fkda_workspace_bytes for the same totals): a fixed batch with at most 16 tokens
 * per sequence (a decode step, T == 1, or a short step, T <= 16) needs only the 256-byte header, other calls their
 * records and queue.  No counterpart in the reference. */
size_t fkda_workspace_bytes_for(const fkda_fwd_params* p);

/* Enqueues the forward pass on `stream` (a cudaStream_t passed as void*).
 * Paths: a fixed batch with T == 1 is one state read-modify-write kernel, with 2 <= T <= 16 one fused kernel, anything
 * else the prepare kernel plus the tensor-core recurrence.  For a ragged batch (cu_seqlens) the host knows only the
 * totals: when there are at most 16 tokens per sequence on average (and at least 64 (sequence, head) pairs), a prefix
 * kernel decides on the device whether every sequence has one token, or at most 16, and the kernels of the paths that
 * may apply are all enqueued; those that are not needed return at once.  Results do not depend on the path
 * (the one-token kernel: to the summation order of its dot products). */
int fkda_fwd(const fkda_fwd_params* p, void* stream);

/* Synchronises `stream`, then reads the device status word that the kernels of the last call
 * using `workspace` left there: FKDA_OK, or FKDA_ERR_DEVICE_STATUS when a kernel gave up on one of
 * its bounded internal waits (its outputs are then invalid).  Other failures: FKDA_ERR_LAUNCH.
 * workspace == NULL reads the built-in scratch of fkda_fwd_noalloc on the current device.
 * fkda_fwd itself never synchronises, so it cannot report this condition: a caller that shares the GPU
 * with other long-running kernels should poll this after synchronising. */
int fkda_device_status(const void* workspace, void* stream);

/*
 * fkda_fwd_noalloc: fkda_fwd for callers that cannot allocate device memory (no counterpart in the
 * reference, whose wrapper allocates a workspace tensor on every call).
 *
 * Some callers cannot call cudaMalloc or a framework allocator at the point where they need the
 * forward pass: a serving loop whose device memory is wholly owned by a pool, a plugin called from
 * another library's callback, a latency-critical thread that must not take allocator locks.  They
 * pass inputs and outputs as usual and leave `workspace` / `workspace_bytes` unset (both are
 * ignored); the per-chunk scratch comes from a fixed array of FKDA_NOALLOC_SCRATCH_BYTES bytes that
 * every GPU loading this library holds until the process exits.
 *
 * Limit: fkda_workspace_bytes_for(p) must not exceed FKDA_NOALLOC_SCRATCH_BYTES.  With the default
 * algorithm a chunk record takes 14 656 bytes and a (sequence, head) chain 32 KB of hand-over state when
 * the call may be pipelined or queued, so about H * (B*T/16) <= 2 250 chunk records minus 2.2 records per
 * chain (algo = twopass: 13 824-byte records, about 2 400); a decode step (T == 1) needs 256 bytes whatever
 * its batch size.  Larger problems return FKDA_ERR_NOALLOC_TOO_LARGE and launch nothing.
 * The call itself performs no cudaMalloc/cudaFree and allocates no device memory through any library.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); the first
 * call on a device that takes the slab pipeline (fixed batch, few long sequences) also creates a side
 * stream and five events, driver objects that hold no device memory.  Make those first calls outside of
 * any stream capture.
 * fkda_device_status(NULL, stream) reports whether a bounded wait gave up in the last such call.
 * All calls on a device share the one array: calls whose kernels may overlap on the GPU race with
 * each other, so serialise them (one stream, or explicit ordering).  The array is not cleared
 * between calls; the header words that must start at zero are reset by each call.
 */
#define FKDA_NOALLOC_SCRATCH_BYTES (32u * 1024u * 1024u)
int fkda_fwd_noalloc(const fkda_fwd_params* p, void* stream);

/* Size of the built-in scratch of fkda_fwd_noalloc, as compiled into the loaded library. */
size_t fkda_noalloc_scratch_bytes(void);

/* Library ABI version (major * 1000 + minor). */
int fkda_version(void);   /* 1001: fkda_fwd_params gained chunk_states, chunk_states_every */

/* sizeof(fkda_fwd_params) as compiled into the loaded library: a binding checks its own struct against it. */
size_t fkda_params_size(void);

/* Static, human-readable name of a status code. */
const char* fkda_status_string(int status);

/* Number of kernels the last successful fkda_fwd call on this thread launched. */
int fkda_last_launch_count(void);

/* Context parallelism (no counterpart in the reference, which has no multi-GPU path): a shard of chunks maps the state
 * it receives to the state it leaves as S_out = S_in . M + N (S, N as [V,K], M as [K,K]).  This folds `count`
 * independent [128,128] fp32 row-major matrices: out[i] = S[i] . M[i] + N[i] (N == NULL: no offset), plain fp32 FMAs in
 * the order k = 0 .. 127.  `out` must not alias S or M.  Enqueued on `stream`. */
int fkda_cp_fold(const float* S, const float* M, const float* N, float* out, int64_t count, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHKDA_B200_H_ */
