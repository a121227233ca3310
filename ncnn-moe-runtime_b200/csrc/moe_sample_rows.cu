// Streaming sampler kernel: one pass over each logit row.
//
// A row is cut into `splits` contiguous slices, one CTA each (one slice per row
// once there are about as many rows as resident CTAs).  A CTA streams its slice
// through a shared-memory ring that the copy engine fills with bulk
// asynchronous copies (cp.async.bulk + mbarrier, no cluster forms), reads it
// back with 128-bit shared loads and keeps only the records that can still
// matter:
//   greedy rows      the best finite logit                     (session.cpp:404-424)
//   Top-K rows       the logits at or above a threshold sampled from the first
//                    chunks, at least k of them                (session.cpp:80-87)
//   full-vocab rows  the records whose softmax numerator could be >= 2^-26
//                    relative to the running maximum ("live" records)
// A chunk is filtered with one packed maximum per 16-byte vector, one compare
// and one warp vote; vectors that reach the threshold are queued per warp and
// unpacked one per lane.  After the stream the survivors are ordered (shuffle
// network per warp + rank by binary search), and one warp replays the
// reference's sequential softmax / Min-P / Top-P / renormalise / inverse-CDF
// arithmetic on them (moe_epilogue.cuh) after all threads have computed the
// softmax numerators.  When rows are sliced, a CTA publishes its survivors to a
// small global scratch slot and counts itself in; nobody waits, and the CTA that
// arrives last for a row gathers the row's slots and finishes it.
//
// Rows whose live set does not fit on chip, and draws that fall through to a
// numerically dead candidate, are appended to a list that the exact kernel
// (moe_sample_exact.cu) finishes.

#include <cstdlib>

#include "moe_common.cuh"
#include "moe_epilogue.cuh"
#include "moe_internal.h"
#include "moe_select.cuh"

#ifdef MOE_PHASE_TIMERS
// Debug builds only: cycles spent per kernel phase, summed over CTAs.
__device__ unsigned long long g_phase_cycles[24];
extern "C" void moe_debug_phase_cycles(unsigned long long* out, int reset)
{
    cudaMemcpyFromSymbol(out, g_phase_cycles, sizeof(unsigned long long) * 24);
    if (reset)
    {
        unsigned long long zeros[24] = {};
        cudaMemcpyToSymbol(g_phase_cycles, zeros, sizeof(zeros));
    }
}
#define MOE_PHASE_MARK(slot)                                                      \
    do                                                                            \
    {                                                                             \
        if (threadIdx.x == 0)                                                     \
        {                                                                         \
            const long long moe_now = clock64();                                  \
            atomicAdd(&g_phase_cycles[slot], static_cast<unsigned long long>(moe_now - moe_phase_start)); \
            moe_phase_start = moe_now;                                            \
        }                                                                         \
    } while (0)
#define MOE_PHASE_BEGIN() long long moe_phase_start = clock64()
// per-CTA wall-clock trace: SM id, start, end of stream, end (globaltimer ns)
__device__ unsigned long long g_cta_trace[4 * 16384];
extern "C" void moe_debug_cta_trace(unsigned long long* out, int entries)
{
    cudaMemcpyFromSymbol(out, g_cta_trace, sizeof(unsigned long long) * 4 * entries);
}
__device__ __forceinline__ unsigned long long moe_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define MOE_TRACE(slot)                                                                  \
    do                                                                                   \
    {                                                                                    \
        if (threadIdx.x == 0 && blockIdx.x < 16384)                                      \
        {                                                                                \
            if ((slot) == 0)                                                             \
            {                                                                            \
                unsigned smid;                                                           \
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));                        \
                g_cta_trace[4 * blockIdx.x + 0] = smid;                                  \
                g_cta_trace[4 * blockIdx.x + 1] = moe_globaltimer();                     \
            }                                                                            \
            else                                                                         \
                g_cta_trace[4 * blockIdx.x + (slot) + 1] = moe_globaltimer();            \
        }                                                                                \
    } while (0)
#else
#define MOE_TRACE(slot) do {} while (0)
#define MOE_PHASE_MARK(slot) do {} while (0)
#define MOE_PHASE_BEGIN() do {} while (0)
#endif
#ifdef MOE_PHASE_TIMERS
#define MOE_SUB_BEGIN() long long moe_sub_start = clock64()
#define MOE_SUB(slot) do { if (threadIdx.x == 0) { const long long moe_sub_now = clock64(); atomicAdd(&g_phase_cycles[slot], static_cast<unsigned long long>(moe_sub_now - moe_sub_start)); moe_sub_start = moe_sub_now; } } while (0)
#else
#define MOE_SUB_BEGIN() do {} while (0)
#define MOE_SUB(slot) do {} while (0)
#endif
#ifdef MOE_PHASE_TIMERS
// per-warp stopwatches inside the streaming loop (lane 0 adds them up at the end)
#define MOE_LAP_DECLARE() long long moe_lap_start = clock64(); long long moe_lap[4] = {0, 0, 0, 0}
#define MOE_LAP(slot) do { const long long moe_lap_now = clock64(); moe_lap[slot] += moe_lap_now - moe_lap_start; moe_lap_start = moe_lap_now; } while (0)
#define MOE_LAP_FLUSH() do { if ((threadIdx.x & 31) == 0) for (int moe_l = 0; moe_l < 4; ++moe_l) atomicAdd(&g_phase_cycles[11 + moe_l], static_cast<unsigned long long>(moe_lap[moe_l])); } while (0)
#else
#define MOE_LAP_DECLARE() do {} while (0)
#define MOE_LAP(slot) do {} while (0)
#define MOE_LAP_FLUSH() do {} while (0)
#endif

namespace moe {

namespace {

// Programmatic dependent launch (sm_90+).  `wait` blocks until every kernel this
// launch depends on has completed and its memory is visible; `launch_dependents`
// lets the next kernel of the stream begin once all CTAs have issued it or exited.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_release()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

#ifndef MOE_ROW_MIN_CTAS
#define MOE_ROW_MIN_CTAS 2 // CTAs per SM the register allocation leaves room for
#endif
#ifndef MOE_ROW_THREADS
#define MOE_ROW_THREADS 256
#endif
constexpr int kThreads = MOE_ROW_THREADS;
constexpr int kWarps = kThreads / 32;
constexpr int kCapSmall = 2048;           // records a CTA can hold: batches whose Top-K sizes are small
constexpr int kCapLarge = 4096;           // ... and batches with top_k up to MOE_SAMPLER_TOPK_FAST_MAX
constexpr int kItems = kCapLarge / kThreads; // most records per thread in block-wide passes
constexpr int kMaxStages = 8;             // ring slots per warp, at most
constexpr uint32_t kHitQueue = 64;        // queued hit vectors per warp
// A Top-K slice lets about 200 logits through its sampled threshold, spread
// like a Gamma variate, and ordering more than kThreads survivors costs two
// sorts instead of one.  When the buffer holds kTightenAt records, the k-th
// best of them is a lower bound of the slice's k-th best: raising the
// threshold to it leaves only a handful of later arrivals.
constexpr uint32_t kTightenAt = 176;
constexpr uint32_t kTightenWindow = 256;  // records looked at (zeroed at kernel start, so an unwritten slot reads as absent)
constexpr uint32_t kTightenTopKMax = 128;
constexpr int kGroupsPerTile = 2;         // careful loop: 128-bit loads in flight per thread
// live mode: the buffer is re-tested against the running maximum at half fill;
// more survivors than live_abort(cap) send the row to the exact kernel
__host__ __device__ constexpr uint32_t live_abort(uint32_t cap)
{
    return cap / 2u - 256u < 1024u ? cap / 2u - 256u : 1024u;
}
constexpr uint32_t kSliceCap = MOE_SLICE_SLOT_RECORDS; // records a slice may publish
// A candidate whose (logit/T - peak) is below this has exp() < 2^-26 and is
// absorbed by every running fp32 sum that starts at the head candidate.
constexpr float kDeadOffset = -18.1f;

enum Mode : int
{
    kGreedy = 0,
    kTopK = 1,
    kLive = 2
};

// Fixed part of a CTA's shared memory; `cap` records and `cap` floats follow it.
struct __align__(16) RowShared
{
    SelectShared<kThreads> sel;
    uint32_t count;
    uint32_t maxkey;
    uint32_t abort_flag;
    uint32_t overflow;
    // completion barriers of the streaming ring: one per warp and slot
    uint64_t ring_full[kWarps][kMaxStages];
    // per warp, the 16-byte vectors whose maximum reached the threshold and the
    // index of their first logit: queued by the streaming loop with no
    // divergence, unpacked one vector per lane when the queue runs full
    uint4 hit_vector[kWarps][kHitQueue];
    uint32_t hit_index[kWarps][kHitQueue];
    float uniform; // the row's Philox uniform, computed off the critical path
    uint32_t sample_keys[kThreads]; // per-thread maxima of the threshold sample, one sorted run per warp
    // Top-K streams: once enough records are in the buffer, one warp finds their
    // k-th best key and every warp raises its threshold to it
    uint32_t tighten_claimed;
    uint32_t tighten_key;
};

struct Ctx
{
    RowShared& s;
    uint64_t* rec;  // cap records
    float* work;    // cap floats (epilogue scratch)
    uint32_t cap;
    Mode mode;
    uint32_t k;
    uint32_t flush_level;
    float temperature;
    float tau;
    bool primed;
    bool aborted;
    bool sorted; // the buffer is already in rank order
};

// The out-of-line helpers of the careful paths take the context by reference,
// which would pin it to local memory — reached through L2 once the shared-memory
// carve-out has left no L1 — for the whole kernel.  The hot path therefore keeps
// its context in registers and hands those helpers a copy.
__device__ __forceinline__ void copy_back_context(Ctx& to, const Ctx& from)
{
    to.mode = from.mode;
    to.k = from.k;
    to.flush_level = from.flush_level;
    to.tau = from.tau;
    to.primed = from.primed;
    to.aborted = from.aborted;
    to.sorted = from.sorted;
}

__device__ __forceinline__ float live_threshold(uint32_t maxkey, float temperature)
{
    if (maxkey == 0)
        return -INFINITY;
    const float peak_logit = key_to_float(maxkey);
    // Lower than every logit whose (logit/T - peak/T), evaluated in fp32 as
    // the reference does, can reach kDeadOffset: 0.1*T of slack plus 2^-20 of
    // the peak's magnitude covers the three roundings involved.
    return __fsub_rn(__fsub_rn(peak_logit, __fmul_rn(18.2f, temperature)), __fmul_rn(9.5367431640625e-07f, fabsf(peak_logit)));
}

// max of two packed bf16 pairs; a NaN operand is ignored, exactly like fmaxf
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

template<typename T>
struct Unpack;

template<>
struct Unpack<float>
{
    static constexpr int kWidth = 4;
    __device__ static __forceinline__ void values(const uint4& v, float (&x)[4])
    {
        x[0] = __uint_as_float(v.x);
        x[1] = __uint_as_float(v.y);
        x[2] = __uint_as_float(v.z);
        x[3] = __uint_as_float(v.w);
    }
    __device__ static __forceinline__ float maximum(const uint4& v)
    {
        return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)), fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
    }
    // maxima are combined in the logits' own format and widened once
    using Packed = float;
    __device__ static __forceinline__ Packed packed_maximum(const uint4& v)
    {
        return maximum(v);
    }
    __device__ static __forceinline__ Packed combine(Packed a, Packed b)
    {
        return fmaxf(a, b);
    }
    __device__ static __forceinline__ float widen(Packed p)
    {
        return p;
    }
    __device__ static __forceinline__ uint4 nan_vector()
    {
        return make_uint4(0x7FC00000u, 0x7FC00000u, 0x7FC00000u, 0x7FC00000u);
    }
};

template<>
struct Unpack<__nv_bfloat16>
{
    static constexpr int kWidth = 8;
    __device__ static __forceinline__ void values(const uint4& v, float (&x)[8])
    {
        x[0] = __uint_as_float(v.x << 16);
        x[1] = __uint_as_float(v.x & 0xFFFF0000u);
        x[2] = __uint_as_float(v.y << 16);
        x[3] = __uint_as_float(v.y & 0xFFFF0000u);
        x[4] = __uint_as_float(v.z << 16);
        x[5] = __uint_as_float(v.z & 0xFFFF0000u);
        x[6] = __uint_as_float(v.w << 16);
        x[7] = __uint_as_float(v.w & 0xFFFF0000u);
    }
    __device__ static __forceinline__ float maximum(const uint4& v)
    {
        return widen(packed_maximum(v));
    }
    // maxima are combined as bf16 pairs (a NaN operand is ignored, like fmaxf) and widened once
    using Packed = uint32_t;
    __device__ static __forceinline__ Packed packed_maximum(const uint4& v)
    {
        return max_bf16x2(max_bf16x2(v.x, v.y), max_bf16x2(v.z, v.w));
    }
    __device__ static __forceinline__ Packed combine(Packed a, Packed b)
    {
        return max_bf16x2(a, b);
    }
    __device__ static __forceinline__ float widen(Packed p)
    {
        return fmaxf(__uint_as_float(p << 16), __uint_as_float(p & 0xFFFF0000u));
    }
    __device__ static __forceinline__ uint4 nan_vector()
    {
        return make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u);
    }
};

// Tests `kWidth` consecutive logits of every lane against the threshold and
// appends the passing ones to the record buffer.  Called by whole warps.
// Returns true when the buffer needs a flush (fill level reached, enough
// records to establish a first threshold, or overflow).
template<int kWidth>
__device__ __forceinline__ bool push_values(Ctx& c, const float (&x)[kWidth], uint32_t first_index, bool retry, uint32_t& stored, int bit_base)
{
    RowShared& s = c.s;
    const int lane = threadIdx.x & 31;
    bool want_flush = false;
#pragma unroll
    for (int e = 0; e < kWidth; ++e)
    {
        const float v = x[e];
        bool pass;
        if (c.mode == kLive)
        {
            pass = v > c.tau;
        }
        else
        {
            pass = c.primed ? (retry ? (v >= c.tau) : (v > c.tau)) : (v >= -INFINITY);
            if (c.mode == kGreedy)
                pass = pass && (fabsf(v) < INFINITY);
        }
        pass = pass && (((stored >> (bit_base + e)) & 1u) == 0u);
        const unsigned voters = __ballot_sync(kFullMask, pass);
        if (voters == 0)
            continue;
        const int leader = __ffs(voters) - 1;
        const uint32_t votes = __popc(voters);
        const uint32_t key = pass ? ordered_key(v) : 0u;
        uint32_t base = 0;
        if (lane == leader)
            base = atomicAdd(&s.count, votes);
        base = __shfl_sync(kFullMask, base, leader);
        const uint32_t slot = base + __popc(voters & ((1u << lane) - 1u));
        if (pass && slot < c.cap)
        {
            c.rec[slot] = make_record(key, first_index + e);
            stored |= 1u << (bit_base + e);
        }
        if (c.mode == kLive)
        {
            const uint32_t best = __reduce_max_sync(kFullMask, key);
            if (lane == leader)
                atomicMax(&s.maxkey, best);
        }
        const uint32_t filled = base + votes;
        if (filled >= c.flush_level || (!c.primed && filled >= c.k))
            want_flush = true;
    }
    return want_flush;
}

// Tightens the buffer: Top-K keeps the k best records and sets the threshold
// to the k-th logit; live mode drops records that fell out of the live window
// of the (larger) running maximum.  Returns true when records had been dropped
// for lack of space, i.e. the current tile must be offered again.
__device__ __noinline__ bool flush_buffer(Ctx& c)
{
    RowShared& s = c.s;
    const uint32_t raw = s.count;
    const bool overflowed = raw > c.cap;
    uint32_t n = overflowed ? static_cast<uint32_t>(c.cap) : raw;
    __syncthreads();
    if (c.mode == kLive)
    {
        const uint32_t maxkey = s.maxkey;
        const float temperature = c.temperature;
        const float peak = __fdiv_rn(key_to_float(maxkey), temperature);
        n = block_compact<kThreads, kItems>(c.rec, n, s.sel, [=](uint64_t record) {
            const float offset = scaled_offset(key_to_float(record_key(record)), temperature, peak);
            return !(offset < kDeadOffset); // keeps NaN offsets: the epilogue reports them
        });
        c.tau = live_threshold(maxkey, temperature);
        if (n > live_abort(c.cap))
            c.aborted = true;
    }
    else if (n > c.k)
    {
        const uint64_t smallest = block_radix_select<kThreads, kItems>(c.rec, n, c.k, s.sel);
        n = c.k;
        c.tau = key_to_float(record_key(smallest));
        c.primed = true;
    }
    else if (n == c.k)
    {
        const uint64_t smallest = block_min_record<kThreads>(c.rec, n, s.sel);
        c.tau = key_to_float(record_key(smallest));
        c.primed = true;
    }
    if (threadIdx.x == 0)
        s.count = n;
    __syncthreads();
    return overflowed;
}

template<typename T, int kGroups>
__device__ __forceinline__ bool emit_tile(Ctx& c, const uint4 (&v)[kGroups], uint32_t first_group, uint32_t head, bool retry, uint32_t& stored)
{
    using U = Unpack<T>;
    bool want_flush = false;
#pragma unroll
    for (int g = 0; g < kGroups; ++g)
    {
        const float top = U::maximum(v[g]);
        bool interesting;
        if (c.mode == kLive)
            interesting = top > c.tau;
        else
            interesting = c.primed ? (retry ? (top >= c.tau) : (top > c.tau)) : (top >= -INFINITY);
        if (__any_sync(kFullMask, interesting))
        {
            float x[U::kWidth];
            U::values(v[g], x);
            const uint32_t first_index = head + ((first_group + g) * kThreads + threadIdx.x) * U::kWidth;
            want_flush |= push_values<U::kWidth>(c, x, first_index, retry, stored, g * U::kWidth);
        }
    }
    return want_flush;
}

// Offers one tile, then resolves fills and overflows until every record of
// the tile has either been stored or beaten.
template<typename T, int kGroups>
__device__ __forceinline__ void run_tile(Ctx& c, const uint4 (&v)[kGroups], uint32_t first_group, uint32_t head)
{
    uint32_t stored = 0;
    bool want = emit_tile<T, kGroups>(c, v, first_group, head, false, stored);
    bool flush = __syncthreads_or(want) != 0;
    while (flush)
    {
        const bool overflowed = flush_buffer(c);
        if (!overflowed || c.aborted)
            break;
        want = emit_tile<T, kGroups>(c, v, first_group, head, true, stored);
        flush = __syncthreads_or(want) != 0;
    }
    if (c.mode == kLive)
        c.tau = fmaxf(c.tau, live_threshold(c.s.maxkey, c.temperature));
}

// The careful streaming loop: a block barrier after every tile, exact radix
// selects whenever the buffer fills, and a retry of the tile when records had to
// be dropped.  It makes no assumption about the order of the logits (ascending
// rows, constant rows and plateaus all work) and is what a slice falls back to
// when the barrier-free loop below could not finish it.
template<typename T>
__device__ __noinline__ void stream_slice_safe(Ctx& c, const T* row_pointer, uint32_t vocab, uint32_t head, uint32_t vectors, uint32_t tail_begin,
                                               uint32_t group_begin, uint32_t group_end, uint32_t rank, uint32_t splits)
{
    using U = Unpack<T>;
    const int tid = threadIdx.x;
    const uint4* vector_base = reinterpret_cast<const uint4*>(row_pointer + head);
    // unaligned leading logits (lowest indices: first, by the first CTA)
    if (rank == 0 && head > 0)
    {
        float x[1] = {tid < static_cast<int>(head) ? LogitTraits<T>::widen(row_pointer, tid) : __uint_as_float(0x7FC00000u)};
        uint32_t stored = 0;
        const bool want = push_values<1>(c, x, static_cast<uint32_t>(tid), false, stored, 0);
        if (__syncthreads_or(want))
            flush_buffer(c);
    }

    uint32_t g = group_begin;
    // a short first tile establishes the threshold cheaply
    if (g < group_end && !c.aborted)
    {
        uint4 v[1];
        const uint32_t vi = g * kThreads + tid;
        v[0] = (vi < vectors) ? load_stream_16(vector_base + vi) : U::nan_vector();
        run_tile<T, 1>(c, v, g, head);
        g += 1;
    }
    // full tiles, next tile's loads in flight while this one is filtered
    const uint32_t full_groups = vectors / kThreads; // groups with all kThreads vectors present
    const uint32_t full_end = min(group_end, full_groups);
    if (g + kGroupsPerTile <= full_end && !c.aborted)
    {
        uint4 current[kGroupsPerTile];
#pragma unroll
        for (int j = 0; j < kGroupsPerTile; ++j)
            current[j] = load_stream_16(vector_base + (g + j) * kThreads + tid);
        while (true)
        {
            const bool has_next = (g + 2 * kGroupsPerTile <= full_end);
            uint4 next[kGroupsPerTile];
            if (has_next)
            {
#pragma unroll
                for (int j = 0; j < kGroupsPerTile; ++j)
                    next[j] = load_stream_16(vector_base + (g + kGroupsPerTile + j) * kThreads + tid);
            }
            run_tile<T, kGroupsPerTile>(c, current, g, head);
            g += kGroupsPerTile;
            if (!has_next || c.aborted)
                break;
#pragma unroll
            for (int j = 0; j < kGroupsPerTile; ++j)
                current[j] = next[j];
        }
    }
    // leftover groups (fewer than a tile, or the ragged last group)
    while (g < group_end && !c.aborted)
    {
        uint4 v[1];
        const uint32_t vi = g * kThreads + tid;
        v[0] = (vi < vectors) ? load_stream_16(vector_base + vi) : U::nan_vector();
        run_tile<T, 1>(c, v, g, head);
        g += 1;
    }
    // unaligned trailing logits (highest indices: last, by the last CTA)
    if (rank == splits - 1 && tail_begin < vocab && !c.aborted)
    {
        const uint32_t index = tail_begin + tid;
        float x[1] = {index < vocab ? LogitTraits<T>::widen(row_pointer, index) : __uint_as_float(0x7FC00000u)};
        uint32_t stored = 0;
        const bool want = push_values<1>(c, x, index, false, stored, 0);
        if (__syncthreads_or(want))
            flush_buffer(c);
    }
    __syncthreads();
    if (!c.aborted)
        flush_buffer(c); // exact k best / exact live set of this slice
}

// Appends the logits of one lane that reach the threshold.  Runs divergently:
// only lanes whose vector maximum reached the threshold get here.
template<int kWidth>
__device__ __forceinline__ void offer_values(RowShared& s, uint64_t* rec, uint32_t cap, Mode mode, float tau, const float (&x)[kWidth],
                                             uint32_t first_index)
{
#pragma unroll
    for (int e = 0; e < kWidth; ++e)
    {
        const float v = x[e];
        bool pass = v >= tau; // false for NaN
        if (mode == kGreedy)
            pass = pass && (fabsf(v) < INFINITY);
        if (pass)
        {
            const uint32_t key = ordered_key(v);
            const uint32_t slot = atomic_add_shared(shared_address(&s.count), 1u);
            if (slot < cap)
                store_shared_64(shared_address(rec + slot), make_record(key, first_index + e));
            else
                store_shared_32(shared_address(&s.overflow), 1u);
            if (mode == kLive)
                atomic_max_shared(shared_address(&s.maxkey), key);
        }
    }
}

// ---- shared-memory ring fed by bulk asynchronous copies -------------------------
// Bytes in flight are what a bandwidth-bound stream needs, and registers are the
// wrong place to hold them: every warp owns `stages` ring slots of kChunkBytes
// in shared memory, lane 0 asks the copy engine for the warp's next chunks
// (cp.async.bulk, global -> shared, completion counted in bytes on one mbarrier
// per slot) and the warp filters a chunk as soon as it has landed.  A warp only
// ever waits for its own slots, so the stream has no block barrier, and the
// copies of the next chunks proceed while hits are unpacked.

#ifndef MOE_RING_VECTORS
#define MOE_RING_VECTORS 8
#endif
constexpr int kVectorsPerLane = MOE_RING_VECTORS;            // 16-byte vectors a lane takes from one chunk
constexpr uint32_t kChunkVectors = 32u * kVectorsPerLane;    // 16-byte vectors per chunk
constexpr uint32_t kChunkBytes = kChunkVectors * 16u;
constexpr uint32_t kSpinLimit = 1u << 20;                    // polls of one slot before the stream gives up on the ring

// barriers and ring slots are named by their shared-window addresses
__device__ __forceinline__ void barrier_init(uint32_t barrier, uint32_t arrivals)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(barrier), "r"(arrivals) : "memory");
}

// one arrival that also announces `bytes` of copy traffic for the current phase
__device__ __forceinline__ void barrier_expect_bytes(uint32_t barrier, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barrier), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool barrier_test(uint32_t barrier, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(barrier), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded: a slot that never completes makes the caller fall back to plain loads.
__device__ __forceinline__ bool barrier_wait(uint32_t barrier, uint32_t parity)
{
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (barrier_test(barrier, parity))
            return true;
    return false;
}

__device__ __forceinline__ uint64_t evict_first_policy()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// `bytes` (a multiple of 16) from 16-byte aligned global memory into this CTA's shared memory
__device__ __forceinline__ void bulk_copy_to_shared(uint32_t destination, const void* source, uint32_t bytes, uint32_t barrier, uint64_t policy)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(destination),
                 "l"(__cvta_generic_to_global(source)), "r"(bytes), "r"(barrier), "l"(policy)
                 : "memory");
}

// A warp's view of its ring.  All fields are warp-uniform.
struct Ring
{
    uint32_t data;         // shared-window address of this warp's slots: stages * kChunkBytes
    uint32_t full;         // ... and of its barriers, one per slot
    uint32_t stages;
    uint32_t issue_slot;   // slot the next request goes to
    uint32_t wait_slot;    // slot of the oldest outstanding request
    uint32_t wait_parity;  // phase parity that request completes
    uint32_t outstanding;  // requests not yet consumed
    uint64_t policy;
};

// lane 0 only; the other lanes call ring_count_request to keep their cursors equal
__device__ __forceinline__ void ring_issue(const Ring& ring, const void* source, uint32_t bytes)
{
    const uint32_t barrier = ring.full + 8u * ring.issue_slot;
    barrier_expect_bytes(barrier, bytes);
    bulk_copy_to_shared(ring.data + ring.issue_slot * kChunkBytes, source, bytes, barrier, ring.policy);
}
__device__ __forceinline__ void ring_count_request(Ring& ring)
{
    ring.issue_slot = (ring.issue_slot + 1u == ring.stages) ? 0u : ring.issue_slot + 1u;
    ++ring.outstanding;
}
// whole warps only; the answer is the same for every lane
__device__ __forceinline__ bool ring_acquire(const Ring& ring)
{
    return __all_sync(kFullMask, barrier_wait(ring.full + 8u * ring.wait_slot, ring.wait_parity)) != 0;
}
// the q-th outstanding request (q < stages), without consuming anything
__device__ __forceinline__ bool ring_acquire_ahead(const Ring& ring, uint32_t q)
{
    uint32_t slot = ring.wait_slot + q;
    uint32_t parity = ring.wait_parity;
    if (slot >= ring.stages)
    {
        slot -= ring.stages;
        parity ^= 1u;
    }
    return __all_sync(kFullMask, barrier_wait(ring.full + 8u * slot, parity)) != 0;
}
// shared-window address of the q-th outstanding chunk / of the oldest one
__device__ __forceinline__ uint32_t ring_ahead(const Ring& ring, uint32_t q)
{
    uint32_t slot = ring.wait_slot + q;
    if (slot >= ring.stages)
        slot -= ring.stages;
    return ring.data + slot * kChunkBytes;
}
__device__ __forceinline__ uint32_t ring_front(const Ring& ring)
{
    return ring.data + ring.wait_slot * kChunkBytes;
}
__device__ __forceinline__ void ring_release(Ring& ring)
{
    if (ring.wait_slot + 1u == ring.stages)
    {
        ring.wait_slot = 0u;
        ring.wait_parity ^= 1u;
    }
    else
    {
        ++ring.wait_slot;
    }
    --ring.outstanding;
}
// Waits (bounded) for every copy still in flight: shared memory must not be
// written after the CTA has moved on.
__device__ __forceinline__ bool ring_drain(Ring& ring)
{
    bool ok = true;
    while (ring.outstanding != 0u)
    {
        ok = ring_acquire(ring) && ok;
        ring_release(ring);
    }
    return ok;
}

// Unpacks a warp's queued hit vectors, one per lane and round, and appends the
// logits that reach the threshold.  Called by whole warps.
template<typename T>
__device__ __forceinline__ void drain_hit_queue(RowShared& s, uint64_t* rec, uint32_t cap, Mode mode, float tau, uint32_t queued)
{
    using U = Unpack<T>;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = threadIdx.x >> 5;
    __syncwarp();
    const uint32_t vectors = shared_address(&s.hit_vector[warp][0]);
    const uint32_t indices = shared_address(&s.hit_index[warp][0]);
    for (uint32_t i = lane; i < queued; i += 32)
    {
        float x[U::kWidth];
        U::values(load_shared_16(vectors + 16u * i), x);
        offer_values<U::kWidth>(s, rec, cap, mode, tau, x, load_shared_32(indices + 4u * i));
    }
    __syncwarp();
}

// The chunks one warp streams: chunk_begin + warp, + kWarps, ... of the row body.
struct SliceFeed
{
    const unsigned char* body; // first 16-byte vector of the row body
    uint32_t vectors;          // 16-byte vectors in the row body
    uint32_t chunk_begin;      // the slice: [chunk_begin, chunk_end)
    uint32_t chunk_end;
    uint32_t my_chunks;        // chunks of the slice that are this warp's

    __device__ __forceinline__ uint32_t chunk_of(uint32_t i) const
    {
        return chunk_begin + (threadIdx.x >> 5) + kWarps * i;
    }
    // asks for this warp's i-th chunk (whole warps call it; lane 0 issues)
    __device__ __forceinline__ void request(Ring& ring, uint32_t i) const
    {
        const uint32_t chunk = chunk_of(i);
        const uint32_t count = min(kChunkVectors, vectors - chunk * kChunkVectors);
        if ((threadIdx.x & 31u) == 0u)
            ring_issue(ring, body + static_cast<size_t>(chunk) * kChunkBytes, count * 16u);
        ring_count_request(ring);
    }
    // fills the ring before anything else is known about the row
    __device__ __forceinline__ void prefetch(Ring& ring) const
    {
        const uint32_t ahead = min(ring.stages, my_chunks);
        for (uint32_t i = 0; i < ahead; ++i)
            request(ring, i);
    }
};

enum StreamResult : int
{
    kStreamCareful = 0, // not finished here: the careful loop must take the slice
    kStreamDone = 1,    // every logit >= threshold is in the buffer and there are enough of them
    kStreamTooLarge = 2 // live row whose live set cannot fit on chip: the exact kernel takes the row
};

// One warp: the largest key K such that at least k of records[0..m) (m <=
// kTightenWindow) have a key >= K, by binary search over the 32 key bits; 0 when
// fewer than k records are present.  Slots still being written read as 0.
__device__ __forceinline__ uint32_t warp_kth_key(const uint64_t* rec, uint32_t m, uint32_t k)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t base = shared_address(rec);
    uint32_t keys[kTightenWindow / 32];
#pragma unroll
    for (uint32_t j = 0; j < kTightenWindow / 32; ++j)
    {
        const uint32_t i = lane + 32u * j;
        keys[j] = i < m ? static_cast<uint32_t>(load_shared_64(base + 8u * i) >> 32) : 0u;
    }
    uint32_t result = 0;
    for (int bit = 31; bit >= 0; --bit)
    {
        const uint32_t candidate = result | (1u << bit);
        uint32_t reached = 0;
#pragma unroll
        for (uint32_t j = 0; j < kTightenWindow / 32; ++j)
            reached += keys[j] >= candidate ? 1u : 0u;
        if (__reduce_add_sync(kFullMask, reached) >= k)
            result = candidate;
    }
    return result;
}

// Rank (1 = largest) of the thread maximum of the sample that becomes the
// threshold of a Top-K slice.  The sample holds `sample_elements` of the
// slice's `slice_elements` logits, so the number of the slice's k best that
// fall into it is Poisson with mean lambda = k * sample / slice; taking the
// r-th largest sampled value with r = lambda + 4.3 sqrt(lambda) + 3 leaves
// fewer than k logits of the slice above the threshold with probability below
// 1e-5 (lambda 1: r = 9, tail 1e-6; lambda 4: r = 16, 5e-6; lambda 8: r = 24,
// 5e-6; lambda 50: r = 84, 1e-6), and lets about r * slice / sample through.
__device__ __forceinline__ uint32_t threshold_rank(uint32_t k, float slice_elements, float sample_elements)
{
    const float lambda = static_cast<float>(k) * fminf(1.0f, sample_elements / slice_elements);
    return static_cast<uint32_t>(ceilf(lambda + 4.3f * sqrtf(lambda) + 3.0f));
}

// The barrier-free streaming loop.  The chunks that fill the ring first (one
// "sample" of the slice) estimate a threshold from the per-thread maxima —
// their r-th largest, see threshold_rank; live mode uses the sample maximum —
// then every chunk is filtered against that threshold: one packed max per
// vector, one compare and one warp vote per chunk.  A lane whose maximum
// reached the threshold copies the vectors concerned to its warp's queue (slot
// from a shared counter); the queue is unpacked one vector per lane when it is
// half full and at the end.
// All logits >= threshold end up in the buffer, so if at least k were found the
// slice's k best are among them regardless of the order of the logits.
template<typename T>
__device__ __forceinline__ int stream_slice_ring(RowShared& s, Ring& ring, const SliceFeed& feed, uint64_t* rec, uint32_t cap, Mode mode, uint32_t k,
                                                 float temperature, const T* row_pointer, uint32_t vocab, uint32_t head, uint32_t tail_begin,
                                                 bool first_rank, bool last_rank)
{
    using U = Unpack<T>;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t vectors = feed.vectors;
    const uint32_t chunk_begin = feed.chunk_begin;
    const uint32_t chunk_end = feed.chunk_end;
    const uint32_t my_chunks = feed.my_chunks;
    // the sample: the chunks every warp has on request when the stream starts, all of them complete
    const uint32_t rounds_available = (chunk_end - chunk_begin) / kWarps;
    const uint32_t complete_chunks = vectors / kChunkVectors;
    // (all but one of the ring's slots: the last one keeps bytes arriving while the threshold is worked out)
    uint32_t sample_rounds = min(max(ring.stages, 2u) - 1u, rounds_available);
    if (chunk_begin + kWarps * sample_rounds > complete_chunks)
        sample_rounds = (complete_chunks > chunk_begin) ? (complete_chunks - chunk_begin) / kWarps : 0u;
    if (sample_rounds == 0u)
    {
        ring_drain(ring);
        return kStreamCareful;
    }

    // rank r of the thread maximum that becomes the threshold
    uint32_t r = 1;
    if (mode == kTopK)
    {
        const float slice_elements = static_cast<float>(chunk_end - chunk_begin) * (kChunkVectors * U::kWidth);
        const float sample_elements = static_cast<float>(sample_rounds) * (kWarps * kChunkVectors * U::kWidth);
        r = threshold_rank(k, slice_elements, sample_elements);
        if (r > (3u * kThreads) / 4u)
        {
            ring_drain(ring);
            return kStreamCareful; // the threshold would pass nearly everything
        }
    }

    MOE_LAP_DECLARE();
    uint32_t* lists = s.sample_keys;
    const uint32_t hit_vectors = shared_address(&s.hit_vector[warp][0]);
    const uint32_t hit_indices = shared_address(&s.hit_index[warp][0]);
    const uint32_t overflow_flag = shared_address(&s.overflow);
    const uint32_t maximum_key = shared_address(&s.maxkey);
    const uint32_t record_count = shared_address(&s.count);
    const uint32_t tighten_claimed = shared_address(&s.tighten_claimed);
    const uint32_t tighten_key = shared_address(&s.tighten_key);
    uint32_t sorted_key = 0;
    uint32_t live_maximum = 0; // live mode, second attempt: the slice maximum found by the first
    bool fault = false;
    for (int attempt = 0;; ++attempt)
    {
        if (ring.outstanding == 0u)
            feed.prefetch(ring); // the first attempt finds the ring filled by the kernel's first instructions

        if (attempt == 0)
        {
            // Each warp sorts its 32 thread maxima with a shuffle network; the block-wide
            // rank of a maximum is its warp rank plus, for every other warp, the number
            // of larger maxima in that warp's sorted list.
            float top = __uint_as_float(0x7FC00000u);
            for (uint32_t q = 0; q < sample_rounds; ++q)
            {
                if (!ring_acquire_ahead(ring, q))
                {
                    fault = true;
                    break;
                }
                const uint32_t sample = ring_ahead(ring, q) + 16u * lane;
#pragma unroll
                for (int j = 0; j < kVectorsPerLane; ++j)
                    top = fmaxf(top, U::maximum(load_shared_16(sample + 512u * j)));
            }
            sorted_key = (top == top) ? ordered_key(top) : 0u; // descending by lane after the network
#pragma unroll
            for (int size = 2; size <= 32; size <<= 1)
            {
#pragma unroll
                for (int stride = size >> 1; stride > 0; stride >>= 1)
                {
                    const uint32_t other = __shfl_xor_sync(kFullMask, sorted_key, stride);
                    const bool descending = (lane & size) == 0;
                    const bool lower_lane = (lane & stride) == 0;
                    sorted_key = (descending == lower_lane) ? max(sorted_key, other) : min(sorted_key, other);
                }
            }
            lists[tid] = sorted_key;
        }

        // Threshold = the r-th largest thread maximum: at least r logits of the sample reach it.
        if (tid == 0)
            s.sel.bucket = 0;
        __syncthreads();
        if (static_cast<uint32_t>(lane) < r)
        {
            uint32_t rank_in_block = lane; // keys strictly greater, plus equal keys of earlier warps, precede this one
            if (r <= 32u)
            {
                // Only rank r - 1 is looked for: a list cannot hold more than r - 1 keys ahead of
                // that one, so its first r entries decide (independent loads, no search).
#pragma unroll
                for (int w = 0; w < kWarps; ++w)
                {
                    if (w == warp)
                        continue;
                    const uint32_t* list = lists + w * 32;
                    for (uint32_t q = 0; q < r; ++q)
                    {
                        const uint32_t value = list[q];
                        rank_in_block += ((value > sorted_key) || (value == sorted_key && w < warp)) ? 1u : 0u;
                    }
                }
            }
            else
            {
                for (int w = 0; w < kWarps; ++w)
                {
                    if (w == warp)
                        continue;
                    const uint32_t* list = lists + w * 32;
                    uint32_t lo = 0, hi = 32;
                    while (lo < hi)
                    {
                        const uint32_t mid = (lo + hi) >> 1;
                        const uint32_t value = list[mid];
                        if ((value > sorted_key) || (value == sorted_key && w < warp))
                            lo = mid + 1;
                        else
                            hi = mid;
                    }
                    rank_in_block += lo;
                }
            }
            if (rank_in_block == r - 1)
                s.sel.bucket = sorted_key;
        }
        __syncthreads();
        // a live row whose first attempt overflowed knows its true maximum now: use it
        const uint32_t threshold_key = (live_maximum != 0u) ? live_maximum : s.sel.bucket;
        bool usable = threshold_key > kKeyNegInf; // else the sample holds (almost) nothing finite
        float tau = 0.0f;
        if (usable)
        {
            if (mode == kLive)
            {
                if (tid == 0)
                    atomicMax(&s.maxkey, threshold_key);
                tau = live_threshold(threshold_key, temperature);
            }
            else
            {
                tau = key_to_float(threshold_key);
            }
        }

        MOE_LAP(0); // threshold estimate
        uint32_t seen_max = threshold_key; // live mode: the largest key this warp knows of
        // live mode, first attempt, buffer already overflowed: only the maximum is still of interest
        bool maximum_only = false;
        // only the first attempt finds the record buffer zeroed beyond what has been written
        const bool tightening = mode == kTopK && attempt == 0 && k <= kTightenTopKMax;
        uint32_t queued = 0; // hit vectors on this warp's queue
        const unsigned lanes_below = (1u << lane) - 1u;
        // Unpacks the queue; true when the stream of this warp is over (the buffer overflowed).
        const auto flush_queue = [&]() -> bool {
            if (mode == kLive)
                tau = fmaxf(tau, live_threshold(load_shared_32_volatile(maximum_key), temperature));
            drain_hit_queue<T>(s, rec, cap, mode, tau, queued);
            queued = 0;
            if (tightening)
            {
                // the first warp to see kTightenAt records in the buffer raises everybody's threshold
                uint32_t present = 0;
                if (lane == 0)
                {
                    present = load_shared_32_volatile(record_count);
                    if (present < kTightenAt || atomic_add_shared(tighten_claimed, 1u) != 0u)
                        present = 0;
                }
                present = __shfl_sync(kFullMask, present, 0);
                if (present != 0u)
                {
                    const uint32_t kth = warp_kth_key(rec, min(present, kTightenWindow), k);
                    if (kth > kKeyNegInf && lane == 0)
                        store_shared_32(tighten_key, kth);
                }
            }
            if (load_shared_32_volatile(overflow_flag) != 0u)
            {
                if (mode == kLive && live_maximum == 0u)
                    maximum_only = true; // keep looking for the row's maximum
                else
                    return true;
            }
            return false;
        };
        for (uint32_t i = 0; usable && !fault && i < my_chunks; ++i)
        {
            if (!ring_acquire(ring))
            {
                fault = true;
                break;
            }
            MOE_LAP(1); // waiting for the copy engine
            if (tightening)
            {
                const uint32_t tighter = load_shared_32_volatile(tighten_key);
                if (tighter != 0u)
                    tau = fmaxf(tau, key_to_float(tighter));
            }
            const uint32_t front = ring_front(ring) + 16u * lane;
            uint4 v[kVectorsPerLane];
#pragma unroll
            for (int j = 0; j < kVectorsPerLane; ++j)
                v[j] = load_shared_16(front + 512u * j);
            const uint32_t first_vector = feed.chunk_of(i) * kChunkVectors;
            if (first_vector + kChunkVectors > vectors)
            {
                // the ragged last chunk of the row: slots beyond it hold stale bytes
#pragma unroll
                for (int j = 0; j < kVectorsPerLane; ++j)
                    if (first_vector + j * 32 + lane >= vectors)
                        v[j] = U::nan_vector();
            }
            typename U::Packed top[kVectorsPerLane];
#pragma unroll
            for (int j = 0; j < kVectorsPerLane; ++j)
                top[j] = U::packed_maximum(v[j]);
            typename U::Packed best_packed = top[0];
#pragma unroll
            for (int j = 1; j < kVectorsPerLane; ++j)
                best_packed = U::combine(best_packed, top[j]);
            const float best = U::widen(best_packed);
            const bool hit = best >= tau;
            // the vote needs every lane's values, so all reads of the slot are complete behind it
            const unsigned voters = __ballot_sync(kFullMask, hit);
            ring_release(ring);
            if (i + ring.stages < my_chunks)
                feed.request(ring, i + ring.stages);
            MOE_LAP(2); // filter + refill request
            if (voters != 0)
            {
                if (maximum_only)
                {
                    if (hit && ordered_key(best) > seen_max)
                        atomic_max_shared(maximum_key, ordered_key(best));
                }
                else
                {
                    // Queue the vectors that reached the threshold.  A lane's first slot is the queue
                    // length plus the vectors of the lanes below it: a popcount of the vote when no lane
                    // has more than one (nearly always), a prefix sum over the lanes otherwise.
                    uint32_t mine = 0;
#pragma unroll
                    for (int j = 0; j < kVectorsPerLane; ++j)
                        mine |= (U::widen(top[j]) >= tau ? 1u : 0u) << j;
                    const uint32_t count = __popc(mine);
                    uint32_t before = __popc(voters & lanes_below);
                    uint32_t total = __popc(voters);
                    if (__ballot_sync(kFullMask, count > 1u) != 0u)
                    {
                        uint32_t inclusive = count;
#pragma unroll
                        for (int offset = 1; offset < 32; offset <<= 1)
                        {
                            const uint32_t other = __shfl_up_sync(kFullMask, inclusive, offset);
                            if (lane >= offset)
                                inclusive += other;
                        }
                        before = inclusive - count;
                        total = __shfl_sync(kFullMask, inclusive, 31);
                    }
                    if (queued + total > kHitQueue && flush_queue())
                        break;
                    if (total > kHitQueue)
                    {
                        // nearly everything in this chunk passes: the sampled threshold is useless for this slice
                        if (lane == 0)
                            store_shared_32(overflow_flag, 1u);
                        break;
                    }
                    uint32_t slot = queued + before;
#pragma unroll
                    for (int j = 0; j < kVectorsPerLane; ++j)
                    {
                        if ((mine >> j) & 1u)
                        {
                            store_shared_16(hit_vectors + 16u * slot, v[j]);
                            store_shared_32(hit_indices + 4u * slot, head + (first_vector + j * 32 + lane) * U::kWidth);
                            ++slot;
                        }
                    }
                    if (mode == kLive && hit && ordered_key(best) > seen_max)
                        atomic_max_shared(maximum_key, ordered_key(best));
                    queued += total;
                    if (queued >= kHitQueue / 2u && flush_queue())
                        break;
                }
            }
            if (mode == kLive)
            {
                seen_max = load_shared_32_volatile(maximum_key);
                tau = fmaxf(tau, live_threshold(seen_max, temperature));
            }
            MOE_LAP(3); // hits
        }
        if (mode == kLive)
            tau = fmaxf(tau, live_threshold(load_shared_32_volatile(maximum_key), temperature));
        if (tightening)
        {
            const uint32_t tighter = load_shared_32_volatile(tighten_key);
            if (tighter != 0u)
                tau = fmaxf(tau, key_to_float(tighter));
        }
        __syncwarp();
        drain_hit_queue<T>(s, rec, cap, mode, tau, queued);
        MOE_LAP(3);
        MOE_LAP_FLUSH();
        if (!ring_drain(ring))
            fault = true;
        if (usable && !fault)
        {
            // logits before / after the 16-byte aligned body of the row
            if (first_rank && tid < static_cast<int>(head))
            {
                const float x[1] = {LogitTraits<T>::widen(row_pointer, tid)};
                offer_values<1>(s, rec, cap, mode, tau, x, static_cast<uint32_t>(tid));
            }
            if (last_rank && tail_begin + tid < vocab)
            {
                const float x[1] = {LogitTraits<T>::widen(row_pointer, tail_begin + tid)};
                offer_values<1>(s, rec, cap, mode, tau, x, tail_begin + tid);
            }
        }
        const bool any_fault = __syncthreads_or(fault ? 1 : 0) != 0;
        const uint32_t found = s.count;
        const bool overflow = s.overflow != 0;
        const uint32_t seen_maximum = s.maxkey;
        __syncthreads();
        if (usable && !any_fault && !overflow && (mode == kLive || found >= k))
            return kStreamDone;
        // Too few logits reached the sampled threshold (or far too many): forget
        // them.  A short count is retried once or twice with a lower threshold —
        // the slice is in L2 now — before the careful loop takes over.  A live
        // row that overflowed (its maximum came late, so the threshold of the
        // sample let too much through) has seen its true maximum by now and
        // is streamed once more against it; if it overflows again its live set
        // really is too large for the chip.
        if (tid == 0)
        {
            s.count = 0;
            s.maxkey = 0;
            s.overflow = 0;
        }
        __syncthreads();
        if (!usable || any_fault)
            return kStreamCareful;
        if (mode == kLive)
        {
            if (live_maximum != 0u)
                return kStreamTooLarge;
            if (seen_maximum == 0u)
                return kStreamCareful;
            live_maximum = seen_maximum;
            continue;
        }
        const uint32_t limit = (3u * kThreads) / 4u;
        if (overflow || r >= limit || attempt >= 2)
            return kStreamCareful;
        r = min(limit, 4u * r + 16u);
    }
}

// Brings the buffer down to what the row can still need: the k best records
// (Top-K, greedy) or the records live against the buffer's maximum.  A Top-K
// buffer of at most one block's worth is simply sorted (the k best are then
// its front); larger ones go through the radix select first.  With `sort` the
// result is left in rank order whenever it fits the block-wide sort.
__device__ __forceinline__ void reduce_buffer(Ctx& c, bool sort)
{
    RowShared& s = c.s;
    MOE_SUB_BEGIN();
    c.sorted = false;
    if (c.aborted)
        return;
    const uint32_t n = load_shared_32(shared_address(&s.count));
    if (n <= 2u * kThreads)
    {
        // At most two records per thread.  Live mode first blanks the records that
        // fell out of the live window of the final maximum (0 sorts last and is
        // not counted); then one sort puts the survivors in rank order, and the
        // k best of a Top-K buffer are its front.
        uint32_t kept = n;
        if (c.mode == kLive)
        {
            const uint32_t tid = threadIdx.x;
            const float peak = __fdiv_rn(key_to_float(s.maxkey), c.temperature);
            uint32_t keeps = 0;
            for (uint32_t i = tid; i < n; i += kThreads)
            {
                const float offset = scaled_offset(key_to_float(record_key(c.rec[i])), c.temperature, peak);
                if (offset < kDeadOffset) // keeps NaN offsets: the epilogue reports them
                    c.rec[i] = 0ull;
                else
                    ++keeps;
            }
            keeps = __reduce_add_sync(kFullMask, keeps);
            if (tid == 0)
                s.sel.out_count = 0;
            __syncthreads();
            if ((tid & 31u) == 0u && keeps != 0u)
                atomicAdd(&s.sel.out_count, keeps);
            __syncthreads();
            kept = s.sel.out_count;
        }
        MOE_SUB(16);
        if (n <= kThreads)
        {
            block_rank_sort_descending<kThreads>(c.rec, n);
        }
        else if (c.mode != kLive && c.k <= kThreads / 2u)
        {
            // A little over one record per thread: the k-th best key of the first kThreads records
            // is a lower bound of the row's k-th best, so everything below it can go before the sort.
            static_assert(kTightenWindow == kThreads, "warp_kth_key looks at one record per thread of the block");
            if (threadIdx.x < 32)
            {
                const uint32_t kth = warp_kth_key(c.rec, kThreads, c.k);
                if (threadIdx.x == 0)
                    s.tighten_key = kth;
            }
            __syncthreads();
            const uint32_t kth = s.tighten_key;
            const uint32_t survivors = block_compact<kThreads, kItems>(c.rec, n, s.sel, [=](uint64_t record) { return record_key(record) >= kth; });
            if (threadIdx.x == 0)
                s.count = survivors;
            __syncthreads();
            if (survivors <= kThreads)
                block_rank_sort_descending<kThreads>(c.rec, survivors);
            else
                block_rank_sort_descending2<kThreads>(c.rec, survivors);
            MOE_SUB(3);
            kept = min(survivors, c.k);
            if (kept != survivors)
            {
                if (threadIdx.x == 0)
                    s.count = kept;
                __syncthreads();
            }
            c.sorted = true;
            return;
        }
        else
        {
            block_rank_sort_descending2<kThreads>(c.rec, n);
        }
        MOE_SUB(3);
        if (c.mode != kLive)
            kept = min(n, c.k);
        if (kept != n)
        {
            if (threadIdx.x == 0)
                s.count = kept;
            __syncthreads();
        }
        c.sorted = true;
        MOE_SUB(17);
        return;
    }
    {
        Ctx careful = c;
        flush_buffer(careful);
        copy_back_context(c, careful);
    }
    if (sort && !c.aborted && s.count <= 2u * kThreads)
    {
        if (s.count <= kThreads)
            block_rank_sort_descending<kThreads>(c.rec, s.count);
        else
            block_rank_sort_descending2<kThreads>(c.rec, s.count);
        c.sorted = true;
    }
}

// Sorts the surviving records into rank order and finishes the row: writes the
// Top-K index list, runs the sequential arithmetic on one warp, flags stop
// tokens, or hands the row to the exact kernel.  Called by the whole block.
__device__ __forceinline__ void finish_row_block(const SampleArgs& a, RowShared& s, Ctx& c, const moe_row_params& p, uint32_t row,
                                                 uint32_t* exact_count, uint32_t* exact_rows)
{
    const int tid = threadIdx.x;
    const bool candidates_only = a.candidates_out != nullptr;
    if (c.aborted)
    {
        if (tid == 0)
            exact_rows[atomicAdd(exact_count, 1u)] = row;
        return;
    }
    const uint32_t n = load_shared_32(shared_address(&s.count));
    const uint32_t record_base = shared_address(c.rec);
    const uint32_t work_base = shared_address(c.work);
    if (!c.sorted)
    {
        if (n <= kThreads)
        {
            block_rank_sort_descending<kThreads>(c.rec, n);
        }
        else if (n <= 2u * kThreads)
        {
            block_rank_sort_descending2<kThreads>(c.rec, n);
        }
        else
        {
            const uint32_t padded = next_pow2(n);
            for (uint32_t i = n + tid; i < padded; i += kThreads)
                c.rec[i] = 0ull;
            __syncthreads();
            block_sort_descending<kThreads>(c.rec, padded);
        }
    }

    if (candidates_only)
    {
        for (uint32_t i = tid; i < a.candidates_k; i += kThreads)
        {
            uint64_t record = 0ull;
            if (i < n)
                record = make_record(record_key(c.rec[i]), record_index(c.rec[i]) + a.vocab_begin);
            a.candidates_out[static_cast<size_t>(row) * a.candidates_k + i] = record;
        }
        return;
    }

    MOE_SUB_BEGIN();
    if (a.topk_index != nullptr)
    {
        const uint32_t listed = (c.mode == kTopK) ? min(n, c.k) : 0u;
        for (uint32_t i = tid; i < a.topk_stride; i += kThreads)
            a.topk_index[static_cast<size_t>(row) * a.topk_stride + i] = (i < listed) ? static_cast<int32_t>(record_index(load_shared_64(record_base + 8u * i))) : -1;
    }
    MOE_SUB(4);

    // The expensive, order-independent part of the epilogue runs on all warps:
    // one softmax numerator per thread (session.cpp:94-100; a double-precision
    // exp each), and the row's uniform on a warp of its own.  What is left for
    // the first warp are the sums that have to be replayed in rank order.
    bool numerators_ready = false;
    if (c.mode != kGreedy && n > 0)
    {
        const uint32_t head_key = record_key(load_shared_64(record_base));
        if (head_key < kKeyPosInf && head_key > kKeyNegInf)
        {
            const uint32_t considered = (p.top_k > 0 && p.top_k <= n) ? p.top_k : n;
            const float peak = __fdiv_rn(key_to_float(head_key), p.temperature);
            for (uint32_t i = tid; i < considered; i += kThreads)
            {
                const uint32_t key = record_key(load_shared_64(record_base + 8u * i));
                if (key > kKeyNegInf)
                    store_shared_32(work_base + 4u * i, __float_as_uint(exact_expf(scaled_offset(key_to_float(key), p.temperature, peak))));
            }
            numerators_ready = true;
        }
        if (tid == kThreads - 32)
            s.uniform = philox_uniform(p.seed, p.row_id, p.step + a.step_offset);
        __syncthreads();
    }
    MOE_SUB(5);

    if (tid < 32)
    {
        RowOutcome out{MOE_ROW_OK, -1, 0.0f, 0u, false};
        const KeptList kept_list = kept_list_of_row(a.kept_token, a.kept_probability, a.kept_count, a.kept_stride, row);
        if (c.mode == kGreedy)
        {
            if (n == 0)
            {
                out.status = MOE_ROW_NO_FINITE_LOGIT;
            }
            else
            {
                out.token = static_cast<int32_t>(record_index(c.rec[0]));
                out.probability = 1.0f;
            }
            if (kept_list.count != nullptr && tid == 0)
            {
                // greedy builds no distribution (session.cpp:404-424): the chosen token stands alone
                *kept_list.count = n == 0 ? 0u : 1u;
                if (n != 0 && kept_list.stride > 0)
                {
                    if (kept_list.token != nullptr)
                        kept_list.token[0] = out.token;
                    if (kept_list.probability != nullptr)
                        kept_list.probability[0] = 1.0f;
                }
            }
        }
        else
        {
            const float uniform = n > 0 ? s.uniform : 0.0f;
            out = finish_row_warp(c.rec, n, c.work, numerators_ready, p.temperature, p.top_k, p.top_p, p.min_p, uniform, c.mode == kLive, kept_list);
            MOE_SUB(8);
        }
        if (tid == 0)
        {
            if (out.defer)
            {
                exact_rows[atomicAdd(exact_count, 1u)] = row;
            }
            else
            {
                if (out.status == MOE_ROW_OK && is_stop_token(a.stop_offsets, a.stop_tokens, row, out.token))
                    out.flags |= MOE_ROW_FLAG_STOP_TOKEN;
                a.token_id[row] = out.token;
                a.probability[row] = out.probability;
                if (a.row_flags != nullptr)
                    a.row_flags[row] = out.flags;
                if (a.row_status != nullptr)
                    a.row_status[row] = out.status;
            }
        }
    }
}

// Shared memory of a CTA: ring | RowShared | cap records | cap floats.
__host__ __device__ constexpr size_t ring_bytes_for(uint32_t stages)
{
    return static_cast<size_t>(stages) * kWarps * kChunkBytes;
}
__host__ __device__ constexpr size_t shared_bytes_for(uint32_t cap, uint32_t stages = 0)
{
    return ring_bytes_for(stages) + sizeof(RowShared) + static_cast<size_t>(cap) * (sizeof(uint64_t) + sizeof(float));
}

template<typename T, bool kLargeBuffer>
__global__ void __launch_bounds__(kThreads, MOE_ROW_MIN_CTAS) sample_rows_kernel(const SampleArgs a, const Workspace ws, const uint32_t splits, const uint32_t stages)
{
    extern __shared__ __align__(128) unsigned char shared_raw[];
    constexpr uint32_t kCapacity = kLargeBuffer ? kCapLarge : kCapSmall;
    unsigned char* const ring_base = shared_raw;
    RowShared& s = *reinterpret_cast<RowShared*>(shared_raw + ring_bytes_for(stages));
    uint64_t* const records = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(&s) + sizeof(RowShared));
    float* const scratch = reinterpret_cast<float*>(records + kCapacity);
    const uint32_t row = blockIdx.x / splits;
    const uint32_t rank = blockIdx.x - row * splits;
    const int tid = threadIdx.x;
    const bool candidates_only = a.candidates_out != nullptr;

    // Overlapped launches: the next launch on the stream may start as soon as
    // every CTA of this one has started (all of them are then resident, so a
    // dependent CTA that waits for this grid can never keep one of its CTAs
    // off an SM).  Its CTAs fill the SM slots this grid leaves free and stream
    // their own logits while this grid finishes.
    if (a.overlap_previous)
        grid_dependency_release();

    // ---- the slice of this CTA, and its first bytes on request at once -----------
    const T* row_pointer = static_cast<const T*>(a.logits) + static_cast<size_t>(row) * a.row_stride;
    const uint32_t vocab = a.vocab;
    // the row body is walked in 16-byte vectors from the first 32-byte boundary;
    // `groups` of kThreads vectors (or of one ring chunk of every lane's size if
    // that is more) are dealt to the row's CTAs in contiguous runs
    const uint32_t misaligned = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(row_pointer) & 31u);
    uint32_t head = ((32u - misaligned) & 31u) / static_cast<uint32_t>(sizeof(T));
    head = min(head, vocab);
    const uint32_t vectors = (vocab - head) / Unpack<T>::kWidth;
    const uint32_t tail_begin = head + vectors * Unpack<T>::kWidth;
    constexpr uint32_t kGroupVectors = (kChunkVectors > kThreads) ? kChunkVectors : static_cast<uint32_t>(kThreads);
    const uint32_t groups = (vectors + kGroupVectors - 1) / kGroupVectors;
    const uint32_t group_begin = static_cast<uint32_t>(static_cast<uint64_t>(rank) * groups / splits);
    const uint32_t group_end = static_cast<uint32_t>(static_cast<uint64_t>(rank + 1) * groups / splits);
    const uint32_t chunks = (vectors + kChunkVectors - 1) / kChunkVectors;
    SliceFeed feed;
    feed.body = reinterpret_cast<const unsigned char*>(row_pointer + head);
    feed.vectors = vectors;
    feed.chunk_begin = group_begin * (kGroupVectors / kChunkVectors);
    feed.chunk_end = min(group_end * (kGroupVectors / kChunkVectors), chunks);
    const uint32_t slice_chunks = feed.chunk_end - feed.chunk_begin;
    feed.my_chunks = (slice_chunks + kWarps - 1u - static_cast<uint32_t>(tid >> 5)) / kWarps;
    if (slice_chunks <= static_cast<uint32_t>(tid >> 5))
        feed.my_chunks = 0;

    Ring ring;
    ring.data = shared_address(ring_base) + static_cast<uint32_t>(tid >> 5) * stages * kChunkBytes;
    ring.full = shared_address(&s.ring_full[tid >> 5][0]);
    ring.stages = stages;
    ring.issue_slot = ring.wait_slot = ring.wait_parity = ring.outstanding = 0u;
    ring.policy = evict_first_policy();
    if ((tid & 31) == 0)
    {
        for (uint32_t slot = 0; slot < stages; ++slot)
            barrier_init(ring.full + 8u * slot, 1u);
        // make the initialised barriers visible to the copy engine
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    feed.prefetch(ring); // a warp only ever uses its own barriers: no block barrier needed first

    moe_row_params p;
    if (candidates_only)
    {
        p.temperature = 1.0f;
        p.top_k = a.candidates_k;
        p.top_p = 1.0f;
        p.min_p = 0.0f;
        p.seed = p.row_id = p.step = 0;
    }
    else
    {
        p = a.params[row];
    }
    MOE_PHASE_BEGIN();
    MOE_TRACE(0);
    const int invalid = validate_row(p);
    if (invalid != MOE_ROW_OK)
    {
        ring_drain(ring);
        // every CTA of the row takes this branch, so the arrival counter stays untouched
        if (a.overlap_previous)
            grid_dependency_wait();
        if (rank == 0)
        {
            if (tid == 0)
            {
                a.token_id[row] = -1;
                a.probability[row] = 0.0f;
                if (a.row_flags != nullptr)
                    a.row_flags[row] = 0;
                if (a.row_status != nullptr)
                    a.row_status[row] = invalid;
                if (a.kept_count != nullptr)
                    a.kept_count[row] = 0;
            }
            if (a.topk_index != nullptr)
                for (uint32_t i = tid; i < a.topk_stride; i += kThreads)
                    a.topk_index[static_cast<size_t>(row) * a.topk_stride + i] = -1;
        }
        return;
    }

    Ctx c{s, records, scratch, kCapacity, kLive, 0xFFFFFFFFu, kCapacity / 2u, p.temperature, -INFINITY, true, false, false};
    if (p.temperature == 0.0f)
    {
        c.mode = kGreedy;
        c.k = 1;
    }
    else if (p.top_k > 0 && p.top_k <= MOE_SAMPLER_TOPK_FAST_MAX)
    {
        c.mode = kTopK;
        c.k = p.top_k;
    }
    if (c.mode != kLive)
    {
        c.primed = false;
        const uint32_t level = max(2u * c.k, c.k + 512u);
        c.flush_level = min(level, c.cap - 1024u);
    }

    if (tid == 0)
    {
        s.count = 0;
        s.maxkey = 0;
        s.abort_flag = 0;
        s.overflow = 0;
        s.tighten_claimed = 0;
        s.tighten_key = 0;
    }
    for (uint32_t i = tid; i < kTightenWindow; i += kThreads)
        records[i] = 0ull; // an unwritten slot must read as "no record" to the threshold tightening
    __syncthreads();

    MOE_PHASE_MARK(0);
    const int streamed = stream_slice_ring<T>(s, ring, feed, c.rec, c.cap, c.mode, c.k, p.temperature, row_pointer, vocab, head, tail_begin, rank == 0,
                                              rank == splits - 1);
    MOE_PHASE_MARK(1);
    MOE_TRACE(1);
#ifdef MOE_PHASE_TIMERS
    if (tid == 0)
    {
        atomicAdd(&g_phase_cycles[10], static_cast<unsigned long long>(streamed == kStreamDone ? s.count : 0u));
        atomicAdd(&g_phase_cycles[9], streamed == kStreamDone ? 0ull : 1ull);
    }
#endif
    if (streamed == kStreamTooLarge)
        c.aborted = true;
    else if (streamed == kStreamCareful)
    {
        Ctx careful = c;
        stream_slice_safe<T>(careful, row_pointer, vocab, head, vectors, tail_begin, group_begin * (kGroupVectors / kThreads),
                             min(group_end * (kGroupVectors / kThreads), (vectors + kThreads - 1) / kThreads), rank, splits);
        copy_back_context(c, careful);
    }
    MOE_PHASE_MARK(2);
    if (a.overlap_previous)
    {
        // Everything up to here only read the logits and the row parameters.  The
        // slots, counters and outputs below may still be in use by the previous
        // launch: wait until it has completed.
        grid_dependency_wait();
    }

    if (splits > 1)
    {
        // ---- publish this slice, count in, and leave unless last -------------------
        reduce_buffer(c, false); // Top-K: the slice's k best; live: re-tested against the slice maximum
        const uint32_t mine = s.count;
        const bool publishable = !c.aborted && mine <= kSliceCap;
        uint64_t* slot_records = ws.slice_records + static_cast<size_t>(blockIdx.x) * kSliceCap;
        uint32_t* slot_header = ws.slice_header + static_cast<size_t>(blockIdx.x) * 4u;
        if (publishable)
            for (uint32_t i = tid; i < mine; i += kThreads)
                slot_records[i] = c.rec[i];
        if (tid == 0)
        {
            slot_header[0] = publishable ? mine : 0u;
            slot_header[1] = publishable ? 0u : 1u; // the row needs the exact kernel
            slot_header[2] = s.maxkey;
        }
        // one release for the whole CTA: the barrier orders every thread's stores
        // before thread 0's fence, which makes them visible before the arrival count
        __syncthreads();
        if (tid == 0)
        {
            __threadfence();
            s.sel.bucket = (atomicAdd(&ws.row_arrivals[row], 1u) == splits - 1) ? 1u : 0u;
        }
        __syncthreads();
        const bool last = s.sel.bucket != 0;
        MOE_PHASE_MARK(3);
        MOE_TRACE(2);
        if (!last)
            return;
        __threadfence();
        if (tid == 0)
            ws.row_arrivals[row] = 0; // ready for the next launch
        if (!publishable)
            c.aborted = true;
        // ---- gather the other slices of the row -------------------------------------
        for (uint32_t peer = 0; peer < splits; ++peer)
        {
            if (peer == rank)
                continue;
            const uint32_t peer_block = row * splits + peer;
            const uint32_t* peer_header = ws.slice_header + static_cast<size_t>(peer_block) * 4u;
            const uint32_t remote_count = __ldcg(peer_header + 0);
            const uint32_t remote_abort = __ldcg(peer_header + 1);
            const uint32_t remote_max = __ldcg(peer_header + 2);
            if (remote_abort != 0)
                c.aborted = true;
            if (c.aborted)
                continue;
            if (s.count + remote_count > c.cap)
            {
                {
                    Ctx careful = c;
                    flush_buffer(careful);
                    copy_back_context(c, careful);
                }
                if (c.aborted || s.count + remote_count > c.cap)
                {
                    c.aborted = true;
                    continue;
                }
            }
            const uint32_t local_count = s.count;
            const uint64_t* remote_records = ws.slice_records + static_cast<size_t>(peer_block) * kSliceCap;
            for (uint32_t i = tid; i < remote_count; i += kThreads)
                c.rec[local_count + i] = __ldcg(reinterpret_cast<const unsigned long long*>(remote_records + i));
            __syncthreads();
            if (tid == 0)
            {
                s.count = local_count + remote_count;
                s.maxkey = max(s.maxkey, remote_max);
            }
            __syncthreads();
        }
        MOE_PHASE_MARK(5);
    }
    reduce_buffer(c, true); // the row's exact k best / exact live set, in rank order
    MOE_PHASE_MARK(6);
    finish_row_block(a, s, c, p, row, ws.exact_count, ws.exact_rows);
    MOE_PHASE_MARK(7);
    MOE_TRACE(2);
}

// Vocabulary-sharded sampling, second step: after the caller's all-gather each
// row has shards * top_k records (one rank-ordered list per GPU, global token
// ids).  The k best of their union are the row's global Top-K
// (session.cpp:80-87); the reference normalises over exactly those, so no
// partial softmax sums cross GPUs.  One CTA per row.
__global__ void __launch_bounds__(kThreads, 2) merge_candidates_kernel(const uint64_t* gathered, uint32_t shards, uint32_t rows, uint32_t top_k,
                                                                        const SampleArgs a)
{
    extern __shared__ __align__(128) unsigned char shared_raw[];
    RowShared& s = *reinterpret_cast<RowShared*>(shared_raw);
    uint64_t* const records = reinterpret_cast<uint64_t*>(shared_raw + sizeof(RowShared));
    float* const scratch = reinterpret_cast<float*>(records + kCapLarge);
    const uint32_t row = blockIdx.x;
    const int tid = threadIdx.x;
    const moe_row_params p = a.params[row];
    int invalid = validate_row(p);
    if (invalid == MOE_ROW_OK && p.temperature != 0.0f && p.top_k != top_k)
        invalid = MOE_ROW_WORKSPACE_EXHAUSTED; // the gathered lists were built for another k
    if (invalid != MOE_ROW_OK)
    {
        if (tid == 0)
        {
            a.token_id[row] = -1;
            a.probability[row] = 0.0f;
            if (a.row_flags != nullptr)
                a.row_flags[row] = 0;
            if (a.row_status != nullptr)
                a.row_status[row] = invalid;
        }
        if (a.topk_index != nullptr)
            for (uint32_t i = tid; i < a.topk_stride; i += kThreads)
                a.topk_index[static_cast<size_t>(row) * a.topk_stride + i] = -1;
        return;
    }
    Ctx c{s, records, scratch, kCapLarge, kTopK, top_k, 0xFFFFFFFFu, p.temperature, -INFINITY, false, false, false};
    if (tid == 0)
    {
        s.count = 0;
        s.maxkey = 0;
        s.abort_flag = 0;
    }
    __syncthreads();
    for (uint32_t shard = 0; shard < shards; ++shard)
    {
        if (s.count + top_k > c.cap)
        {
            Ctx careful = c;
            flush_buffer(careful);
            copy_back_context(c, careful);
        }
        const uint32_t local_count = s.count;
        const uint64_t* list = gathered + (static_cast<size_t>(shard) * rows + row) * top_k;
        // a shard's list is dense from the front; empty slots hold 0
        uint32_t mine = 0;
        for (uint32_t i = tid; i < top_k; i += kThreads)
        {
            const uint64_t record = list[i];
            if (record != 0ull)
            {
                c.rec[local_count + i] = record;
                ++mine;
            }
        }
        // number of non-empty records of this shard (block reduction through the selector's counter)
        if (tid == 0)
            s.sel.out_count = 0;
        __syncthreads();
        mine = __reduce_add_sync(kFullMask, mine);
        if ((tid & 31) == 0 && mine != 0)
            atomicAdd(&s.sel.out_count, mine);
        __syncthreads();
        if (tid == 0)
            s.count = local_count + s.sel.out_count;
        __syncthreads();
    }
    if (p.temperature == 0.0f)
    {
        // greedy over the merged candidates: best finite record (session.cpp:404-424)
        const uint32_t n = s.count;
        const uint32_t kept = block_compact<kThreads, kItems>(c.rec, n, s.sel, [](uint64_t record) {
            const uint32_t key = record_key(record);
            return key > kKeyNegInf && key < kKeyPosInf;
        });
        if (tid == 0)
            s.count = kept;
        __syncthreads();
        c.mode = kGreedy;
        c.k = 1;
    }
    reduce_buffer(c, true); // the k best of the union, in rank order (one block-wide sort for up to 512 candidates)
    finish_row_block(a, s, c, p, row, nullptr, nullptr);
}

template<typename T, bool kLargeBuffer>
cudaError_t launch_typed(const SampleArgs& args, const Workspace& ws, uint32_t splits, uint32_t stages, cudaStream_t stream)
{
    static SharedOptIn opt_in;
    const size_t shared_bytes = shared_bytes_for(kLargeBuffer ? kCapLarge : kCapSmall, stages);
    cudaError_t status = opt_in_shared(opt_in, sample_rows_kernel<T, kLargeBuffer>, shared_bytes);
    if (status != cudaSuccess)
        return status;
    if (!args.overlap_previous)
    {
        sample_rows_kernel<T, kLargeBuffer><<<args.rows * splits, kThreads, shared_bytes, stream>>>(args, ws, splits, stages);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(args.rows * splits, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, sample_rows_kernel<T, kLargeBuffer>, args, ws, splits, stages);
}

// Ring slots per warp and CTAs per SM that go with them.  Two CTAs per SM with
// two slots of kChunkBytes (4 KiB) per warp keep 128 KiB per SM on request.
uint32_t ring_stages(bool large_top_k)
{
    static const uint32_t forced = [] {
        const char* text = std::getenv("MOE_B200_RING_STAGES");
        const long value = text != nullptr ? std::strtol(text, nullptr, 10) : 0;
        return (value >= 1 && value <= kMaxStages) ? static_cast<uint32_t>(value) : 0u;
    }();
    if (forced != 0u)
        return forced;
    return large_top_k ? 1u : 2u;
}

uint32_t resident_per_sm(bool large_top_k, uint32_t stages)
{
    // 227 KiB per SM, 1 KiB reserved per CTA
    const size_t per_cta = shared_bytes_for(large_top_k ? kCapLarge : kCapSmall, stages) + 1024u;
    const uint32_t fit = static_cast<uint32_t>((227u * 1024u) / per_cta);
    const uint32_t by_registers = MOE_ROW_MIN_CTAS; // the launch bounds promise registers for this many
    return fit < 1u ? 1u : (fit > by_registers ? by_registers : fit);
}

} // namespace

cudaError_t launch_sample_rows(const SampleArgs& args, const Workspace& ws, uint32_t splits, cudaStream_t stream)
{
    if (args.rows == 0)
        return cudaSuccess;
    const uint32_t stages = ring_stages(args.large_top_k);
    if (args.large_top_k)
    {
        if (args.dtype == MOE_DTYPE_F32)
            return launch_typed<float, true>(args, ws, splits, stages, stream);
        return launch_typed<__nv_bfloat16, true>(args, ws, splits, stages, stream);
    }
    if (args.dtype == MOE_DTYPE_F32)
        return launch_typed<float, false>(args, ws, splits, stages, stream);
    return launch_typed<__nv_bfloat16, false>(args, ws, splits, stages, stream);
}

namespace {
__global__ void pack_sampled_rows_kernel(const int32_t* token_id, const float* probability, const uint32_t* row_flags, const int32_t* row_status,
                                         uint32_t rows, moe_sampled_row* packed)
{
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row < rows)
        packed[row] = moe_sampled_row{token_id[row], probability[row], row_flags[row], row_status[row]};
}
} // namespace

cudaError_t launch_pack_sampled_rows(const int32_t* token_id, const float* probability, const uint32_t* row_flags, const int32_t* row_status,
                                     uint32_t rows, moe_sampled_row* packed, cudaStream_t stream)
{
    if (rows == 0)
        return cudaSuccess;
    pack_sampled_rows_kernel<<<(rows + 255u) / 256u, 256, 0, stream>>>(token_id, probability, row_flags, row_status, rows, packed);
    return cudaGetLastError();
}

cudaError_t launch_merge_candidates(const uint64_t* gathered, uint32_t shards, uint32_t rows, uint32_t top_k, const moe_row_params* params,
                                    uint64_t step_offset, int32_t* token_id, float* probability, uint32_t* row_flags, int32_t* row_status,
                                    int32_t* topk_index, uint32_t topk_stride, cudaStream_t stream)
{
    if (rows == 0)
        return cudaSuccess;
    static SharedOptIn opt_in;
    const size_t shared_bytes = shared_bytes_for(kCapLarge);
    if (cudaError_t status = opt_in_shared(opt_in, merge_candidates_kernel, shared_bytes))
        return status;
    SampleArgs a = {};
    a.rows = rows;
    a.params = params;
    a.step_offset = step_offset;
    a.token_id = token_id;
    a.probability = probability;
    a.row_flags = row_flags;
    a.row_status = row_status;
    a.topk_index = topk_index;
    a.topk_stride = topk_stride;
    merge_candidates_kernel<<<rows, kThreads, shared_bytes, stream>>>(gathered, shards, rows, top_k, a);
    return cudaGetLastError();
}

uint32_t choose_splits(uint32_t rows, uint32_t vocab, int dtype, int sm_count, uint32_t slice_slots, bool large_top_k, bool overlapped)
{
    // A row is cut into slices only while all CTAs of the launch stay resident
    // at once: a single wave has no ragged second wave, and the fixed per-slice
    // work (threshold estimate, select, publication) stays small next to a
    // slice of at least 128 KiB.  The ring decouples the bytes on request from
    // the number of CTAs, so one CTA per row is enough once there are about as
    // many rows as resident CTAs.
    (void)overlapped;
    const uint64_t row_bytes = static_cast<uint64_t>(vocab) * (dtype == MOE_DTYPE_F32 ? 4u : 2u);
    const uint64_t by_size = row_bytes / (128u * 1024u);
    const uint64_t resident = static_cast<uint64_t>(sm_count) * resident_per_sm(large_top_k, ring_stages(large_top_k));
    uint64_t splits = rows > 0 ? resident / rows : 1u;
    splits = splits < by_size ? splits : by_size;
    splits = splits < 32u ? splits : 32u;
    if (rows > 0 && splits * rows > slice_slots)
        splits = slice_slots / rows;
    return splits < 1u ? 1u : static_cast<uint32_t>(splits);
}

} // namespace moe
