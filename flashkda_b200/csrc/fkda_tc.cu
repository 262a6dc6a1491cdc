// Tensor-core two-pass KDA forward for sm_100a: the token-parallel prepare kernel writes per-chunk
// operand records already laid out as tcgen05 (UMMA) shared-memory operands; a persistent
// recurrence kernel walks the chunks of each (sequence, head) chain with
//   * per chunk one bulk asynchronous copy of the record plus one tiled TMA load (tensor map) of the
//     [16,128] value tile, multi-buffered on mbarriers; out tiles leave through a tiled TMA store,
//   * all contractions on tcgen05.mma with fp32 accumulators in tensor memory (M = 128 always):
//        D1[V,32]   = S[V,K] . [kd; qd]^T         (8 x M128 N32 K16; A = the bf16 state copy in tensor memory)
//        D2[V,16]   = u'^T[V,16] . INV^T          (M128 N16 K16)
//        D3[V,16]   = U^T[V,16] . Mqk^T           (M128 N16 K16)
//        DST[V,K]   = U^T[V,16] . kr[16,K]        (M128 N128 K16; the state update)
//   * the bf16 state held twice: in the registers of its owner threads (thread v owns S[v,:]) for the
//     element-wise update S[v,k] = bf(fma(S[v,k], E_tot[k], DST[v,k])), and as the tensor-memory copy that the
//     next chunk's first MMA reads as its A operand,
//   * the other element-wise steps (bf16 roundings, beta) by the same threads (thread v = TMEM lane v of
//     D1/D2/D3), reading accumulators with tcgen05.ld.
// The kernels live in their own files and share the helpers below: fkda_tc_ts.cuh (three chains per CTA: the
// default for more chains than SMs) and fkda_tc_wide.cuh (one chain per CTA, for no more chains than SMs).
//
// Numerics: steps B1-B7 of the reference's contract (tests/torch_ref.py:231-251; the reference's own
// recurrence is csrc/smxx/fwd_kernel2.cuh:434-742, built on mma.sync with register transposes).
#include <cuda.h>
#include <string.h>

#include <mutex>

#include "fkda_common.cuh"
#include "fkda_internal.h"
#include "fkda_prepare_warp.cuh"
#include "fkda_sm100.cuh"

namespace fkda {

using namespace sm100;

constexpr int kTcChains = 3;    // chains (warpgroups) per CTA
constexpr int kTcStages = 3;    // chunk records in flight per chain
constexpr int kTcTmemCols = 512;
constexpr int kTcStageBytes = kTcRecord;   // one chunk record per stage

struct TcCtrl {
    uint64_t full[kTcChains][kTcStages];
    uint64_t mma[kTcChains];
    uint32_t tmem_base;
    int32_t next_chain[kTcChains];
    int32_t abort_flag;
};

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
    int64_t cs_slot0;         // first state-export slot of the sequence (valid when chunk_states is given)
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
    c.cs_slot0 = a.chunk_states != nullptr ? cs_first_slot(a, c.n) : 0;
    return c;
}

// Next work item of a chain slot (called by ONE thread of the slot's warpgroup).  An item is one segment
// (seg_chunks chunks) of one chain; item id = seg * n_chains + chain.
//
// First segments are CLAIMED, never assigned: nothing waits for a CTA that is not resident (SMs held by another
// kernel, or a second persistent launch on another stream), so the kernel makes progress with whatever CTAs run.
//   * The first kTcChains * gridDim chains form kTcChains layers of gridDim entries.  Warpgroup j's first claim
//     comes from layer j (an atomic counter per layer), so few chains spread one per SM before any SM takes a
//     second; odd layers are handed out backwards, so with chains ordered by decreasing length the longest of one
//     layer meet the shortest of the next on an SM.
//   * Every later claim first looks for entries that are still unclaimed in any layer (left by CTAs that have not
//     started), then takes the chains beyond the layers in order (the tail counter).
//   * When all first segments are taken, the tail counter hands out queue tickets: ticket q reads slot q, which
//     the finisher of some segment fills with the follow-up segment, so chains take turns on the chain slots
//     (first come, first served) and more chains than slots still share the machine evenly.  Only warpgroups that
//     run hold tickets, and every unfinished chain is either being walked by a running warpgroup or sits in a
//     slot, so a waiter never depends on a CTA that has not started.
// Returns the item, -2 when nothing is left to do, -3 when the bounded wait gave up.
__device__ __forceinline__ int tc_layer_item(int j, int x, int cnt) {
    return j * (int)gridDim.x + ((j & 1) ? cnt - 1 - x : x);
}
__device__ __forceinline__ int tc_next_item(const TwoPassArgs& a, bool first_claim, int wg, int64_t n_chains,
                                            volatile int* abort_flag) {
    const int G = (int)gridDim.x;
    int32_t* layer = a.queue + 4;   // header words 4 .. 4 + kTcChains - 1
    auto layer_count = [&](int j) {
        const int64_t c = n_chains - (int64_t)j * G;
        return (int)(c < 0 ? 0 : (c > G ? G : c));
    };
    if (first_claim) {
        const int cnt = layer_count(wg);
        if (cnt > 0) {
            const int x = atomicAdd(layer + wg, 1);
            if (x < cnt) return tc_layer_item(wg, x, cnt);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kTcChains; ++j) {
            const int cnt = layer_count(j);
            if (*reinterpret_cast<volatile int32_t*>(layer + j) < cnt) {
                const int x = atomicAdd(layer + j, 1);
                if (x < cnt) return tc_layer_item(j, x, cnt);
            }
        }
    }
    const int64_t n_tail = n_chains > (int64_t)kTcChains * G ? n_chains - (int64_t)kTcChains * G : 0;
    const int t = atomicAdd(a.queue, 1);
    if (t < n_tail) return kTcChains * G + t;
    int item = -2;
    if (a.seg_chunks > 0) {
        volatile int32_t* slot = a.qslots + (t - (int)n_tail);
        volatile int32_t* finished = a.queue + 3;
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        for (;;) {
            const int x = *slot;
            if (x >= 0) { item = x; break; }
            if (*finished >= (int)n_chains) break;
            if ((++spins & 63u) == 0 && (*abort_flag != 0 || global_timer_ns() - t0 > a.wait_ns)) { item = -3; break; }
            __nanosleep(200);
        }
        __threadfence();  // the pusher's state stores are visible before we read them
    }
    return item;
}
// The finisher of a non-final segment queues the follow-up segment (ONE thread, after the state hand-over
// stores of all threads have been fenced and a barrier has passed).
__device__ __forceinline__ void tc_push_followup(const TwoPassArgs& a, int item, int64_t n_chains) {
    if (a.test_drop_push) return;  // test hook: starve the queue so that its bounded waits give up
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

}  // namespace fkda

#include "fkda_tc_ts.cuh"
#include "fkda_tc_wide.cuh"

namespace fkda {

// ---------------------------------------------------------------------------------
// SM count of the current device (B200: 148), cached per device; 148 when no device can be asked (sizing calls
// on a machine without a GPU).
int device_sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cache[dev] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
        cache[dev] = sms;
    }
    return cache[dev];
}

// Segment scheduling is used when there are more chains than the GPU can hold at once (3 per SM);
// with fewer chains every chain has its own slot and whole chains are the work items.
constexpr int kSegChunksMax = 64, kSegChunksMin = 16;
// Segment length: 64 chunks when there is plenty of work (the hand-over of a 32 KB state costs about one chunk
// step), shorter when the whole problem is only a few segments per chain slot, so that 512 chains of 64 chunks
// do not run as one full round plus a nearly empty one.  Even, so that the stage parity of a segment's
// first chunk is fixed.  A function of (T_total, H, N) only: the workspace is sized with the same value.
static int seg_chunks_for(int64_t T_total, int64_t H, int64_t N, int sms) {
    const int64_t chain_slots = (int64_t)sms * kTcChains;
    int64_t seg = H * ws_tiles_upper_bound(T_total, N) / (4 * chain_slots);  // aim at >= 4 segments per chain slot
    seg = seg / 2 * 2;
    if (seg > kSegChunksMax) seg = kSegChunksMax;
    if (seg < kSegChunksMin) seg = kSegChunksMin;
    return (int)seg;
}
static bool use_segments(int64_t H, int64_t N, int sms) { return H * N > (int64_t)sms * kTcChains; }
// slots of the segment queue: sized for the shortest segment length a call may ask for (8 chunks), plus one
// ticket per resident warpgroup at the end
static size_t seg_slots_bytes(int64_t T_total, int64_t H, int64_t N, int sms) {
    if (!use_segments(H, N, sms)) return 0;
    const size_t count = (size_t)(H * (ws_tiles_upper_bound(T_total, N) / 8 + N) + 4096);
    return (count * 4 + 255) / 256 * 256;
}
// Few chains on a fixed batch may run as a slab pipeline (see launch_tc); its chain states travel through the
// same hand-over buffer as the segments of the work queue (32 KB per chain).
static bool slabs_possible(int64_t chains, int sms) { return chains <= sms - 32; }
static size_t seg_state_bytes(int64_t H, int64_t N, bool needed) { return needed ? (size_t)(H * N) * 32768 : 0; }

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

// Upper bound over every call with these totals (the caller may not know yet whether the batch is ragged).
size_t tc_workspace_bytes(int64_t T_total, int64_t H, int64_t N) {
    const int sms = device_sm_count();
    const bool states = use_segments(H, N, sms) || slabs_possible(H * N, sms);
    return kWsHeaderBytes + ws_prefix_bytes(N) + seg_slots_bytes(T_total, H, N, sms) + seg_state_bytes(H, N, states) +
           (size_t)H * (size_t)ws_tiles_upper_bound(T_total, N) * (size_t)kTcRecord;
}

// What one particular call needs: the same carving as launch_tc (a function of the shapes only, not of
// phase_mask or flags, so that calls which share a workspace find the records in the same place).
struct TcCarve {
    size_t slots, states, records;
    bool segments;
};
static TcCarve tc_carve(const fkda_fwd_params& p, int sms) {
    const int64_t T_total = p.B * p.T, chains = p.N * p.H;
    const bool varlen = p.cu_seqlens != nullptr;
    TcCarve c;
    c.segments = use_segments(p.H, p.N, sms);
    c.slots = seg_slots_bytes(T_total, p.H, p.N, sms);
    c.states = seg_state_bytes(p.H, p.N, c.segments || (!varlen && slabs_possible(chains, sms)));
    const int64_t tiles = varlen ? ws_tiles_upper_bound(T_total, p.N) : p.N * ((p.T + kChunk - 1) / kChunk);
    c.records = (size_t)p.H * (size_t)tiles * (size_t)kTcRecord;
    return c;
}
size_t tc_workspace_bytes_for(const fkda_fwd_params& p) {
    if (decode_eligible(p) && !(p.flags & FKDA_FLAG_NO_DECODE) && p.chunk_states == nullptr) return kWsHeaderBytes;  // status word only
    if (short_eligible(p) && !(p.flags & FKDA_FLAG_NO_SHORT)) return kWsHeaderBytes;
    const TcCarve c = tc_carve(p, device_sm_count());
    return kWsHeaderBytes + ws_prefix_bytes(p.N) + c.slots + c.states + c.records;
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
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return FKDA_ERR_LAUNCH;
    const int sms = device_sm_count();
    const int64_t T_total = p.B * p.T;
    if (cudaMemsetAsync(p.workspace, 0, 64, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;  // header counters
    {   // carve the segment queue and the hand-over states in front of the records
        uint8_t* base = reinterpret_cast<uint8_t*>(p.workspace) + kWsHeaderBytes + ws_prefix_bytes(p.N);
        const TcCarve c = tc_carve(p, sms);
        if (c.segments) {
            a.qslots = reinterpret_cast<int32_t*>(base);
            const int forced = ((p.flags >> 8) & 0xff) / 2 * 2;
            a.seg_chunks = forced >= 8 ? forced : seg_chunks_for(T_total, p.H, p.N, sms);
            if (do_rec && cudaMemsetAsync(a.qslots, 0xff, c.slots, stream) != cudaSuccess) return FKDA_ERR_LAUNCH;
        }
        a.seg_state = reinterpret_cast<uint32_t*>(base + c.slots);
        a.workspace = base + c.slots + c.states;
    }
    const int64_t chains = p.N * p.H;
    const bool wide = chains <= sms && !(p.flags & FKDA_FLAG_NO_WIDE);
    TcMaps maps;
    memset(&maps, 0, sizeof(maps));
    // (an empty batch has no tiles to move: its chains only pass their state through)
    if (do_rec && T_total > 0 &&
        (!encode_token_map(&maps.v, p.v, T_total, p.H, p.token_stride) ||
         !encode_token_map(&maps.out, p.out, T_total, p.H, p.token_stride)))
        return FKDA_ERR_LAUNCH;
    const int wide_smem = kWideSmemBytes;
    if (do_rec && wide &&
        cudaFuncSetAttribute(recurrence_tc_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide_smem) != cudaSuccess)
        return FKDA_ERR_LAUNCH;

    // ---- few chains on a fixed batch: the recurrence is a serial walk on `chains` SMs and leaves the others
    //      idle, so the forward is cut into slabs of chunks and the prepare stage of slab i+1 runs on the idle SMs
    //      (side stream) while the recurrence walks slab i; the state of a chain travels through seg_state.
    //      Only stream order and events connect the launches: no kernel waits for another one. ----
    const int64_t tps = (p.T + kChunk - 1) / kChunk;
    const int idle_sms = sms - (int)chains;
    if (wide && !varlen && p.phase_mask == 0 && slabs_possible(chains, sms) && tps >= 64 && !(p.flags & FKDA_FLAG_NO_SLABS)) {
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
            recurrence_tc_wide_kernel<<<(unsigned)chains, kWideThreads, wide_smem, stream>>>(slab_args(i), maps);
            ++launches;
        }
        if (cudaGetLastError() != cudaSuccess) return FKDA_ERR_LAUNCH;
        *n_launches = launches;
        return FKDA_OK;
    }

    // A ragged batch whose sequences MAY all fit one chunk (the host sees only the totals): the prefix kernel decides,
    // the fused short-sequence kernel and the general kernels are both enqueued and one side returns at once.
    if (short_ragged_candidate(p) && !(p.flags & FKDA_FLAG_NO_SHORT)) a.short_flag = a.queue + 8;
    // as many tokens as sequences: they may have one token each, the decode kernel's case
    const bool try_decode = a.short_flag != nullptr && T_total == p.N && !(p.flags & FKDA_FLAG_NO_DECODE);
    if (varlen && do_prep) {
        launch_tile_prefix(p.cu_seqlens, p.N, a.tile_prefix, const_cast<int32_t*>(a.seq_order),
                           a.chunk_states != nullptr ? const_cast<int32_t*>(a.cs_prefix) : nullptr, 16 * a.cs_every,
                           a.short_flag, try_decode, a.qslots != nullptr ? a.queue + 9 : nullptr, p.H, sms * kTcChains, stream);
        ++launches;
    }
    if (try_decode) {
        if (launch_decode_ragged(a, stream) != FKDA_OK) return FKDA_ERR_LAUNCH;
        ++launches;
    }
    if (a.short_flag != nullptr) {
        if (launch_short_ragged(a, stream) != FKDA_OK) return FKDA_ERR_LAUNCH;
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
            recurrence_tc_wide_kernel<<<(unsigned)ctas, kWideThreads, wide_smem, stream>>>(a, maps);
        } else {
            // three chains per CTA, state copy and 16-deep A operands in tensor memory
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
