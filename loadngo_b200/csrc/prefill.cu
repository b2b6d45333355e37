// Prefill (prompt-pass) attention for gpt-oss on sm_100a: tcgen05 tensor cores with TMEM
// accumulators, operands staged by TMA, causal and sliding-window tile skipping.
//
// Replaces loadngo's `attention_grouped_tiled` (metal-compute/src/kernels.metal:588-720, host
// entry metal-compute/src/apple.rs:1311-1401): for t new positions of a sequence starting at
// `start`, every query attends the cache rows its causal / window rule allows
// (gpt-oss/src/model.rs:434-438), with the head's sink logit in the softmax maximum and
// denominator only (model.rs:449-455).  The new positions' keys and values are already in
// the paged cache (the fused RoPE + append kernel ran first).
//
// At head_dim 64 the exponentials bound this kernel, not the products: a 128 x 128 score tile
// needs 16 384 exp2 (1 024 cycles of the SM's 16-lane special-function unit) against about 820
// cycles of tensor pipe (measured: 8 score instructions of ~56 cycles, 8 product instructions of
// ~46).  Measured too, and shaping what follows: a tcgen05.commit is seen by a waiting thread
// about 440 cycles after the last instruction it covers was issued, so every hand-over through
// the tensor pipe is expensive; four softmax warps per scheduler are needed to keep the exp2
// unit near its rate (one warp alone reaches half); and the softmax warps' loops have to stay
// small and rolled (fully unrolled sweeps ran 1.4x slower, out of the instruction cache).
//
// A work item = 256 consecutive queries of one head = two query tiles, A and B, of 128 rows.
// CTAs are persistent (one per SM) and walk a fixed sequence of items, heaviest first, the 8
// heads of a KV group next to each other so that they share K and V through L2.  Every 128-key
// tile of K and V that an item needs is loaded once and used by both query tiles, which halves
// the traffic from L2 into shared memory.  The unit of work inside the CTA is a job = (query
// tile, key tile); all roles enumerate the same job sequence n = 0, 1, 2, ... (per key tile: A's
// job, then B's, where the tile is in that query tile's range).  Nineteen warps, four roles:
//   warp 0   producer: TMA loads of the query tiles (hi and lo planes) into a ring of three
//            slots, and per key tile sixteen 16-key pages (eight of K, eight of V, found through
//            the block table, one per lane) into a ring of three stages;
//   warp 1   one thread issues the scores of job n, S = Qhi K^T + Qlo K^T (tcgen05.mma
//            M128 N128 K64 twice), into score buffer n mod 3 in tensor memory.  That buffer held
//            the P of job n - 3: the scores wait only until that job's product has been ISSUED
//            (the pipe runs what it is given in order), not until it has finished;
//   warp 18  one thread issues the products O_A or O_B += P V (M128 N64 K128, P read from
//            tensor memory) as soon as a job's P is published;
//   warps 2-9 (tile A) and 10-17 (tile B)  softmax, two threads per query row, 64 keys each: a
//            first sweep over the thread's scores in tensor memory finds their maximum, the two
//            threads of a row compare through shared memory, a second sweep computes
//            P = exp2(s - m), sums the rounded weights and writes them as bf16 over the first
//            half of the scores they came from.  The two tiles' warps drift half a job apart, so
//            one tile's waits, first sweep and publishing run under the other's exponentials.
//            O is rescaled only when a row maximum moved by more than 2^8 (rare after the first
//            tiles); at the end of an item the two halves of the row sum meet, the sink is folded
//            in and each thread normalises and stores its 64 bytes of the bf16 output row.
// Tiles entirely outside a query tile's causal / window range are never visited (the loop
// bounds exclude them, as kernels.metal:631-634 does); only edge tiles are masked per element.
//
// Every wait is bounded; one that runs out raises the status word and the CTA drains, frees its
// TMEM and returns.  A wait on an mbarrier names a phase by its parity, so no role may wait more
// than one phase ahead of a barrier: where one query tile has no rows for a while (ragged
// sequences), its warps hold back until the other tile's warps have caught up (`seen`).
#include "kernels.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace cc {
namespace {

constexpr int kTileQ = 128, kTileK = 128;
constexpr int kQSlots = 3;                                  // ring of query tiles (hi plane + lo plane each)
constexpr int kStagesKV = 3;                                // K tile + V tile per stage
constexpr int kSBufs = 3;                                   // score / P buffers in tensor memory
constexpr int kPvRing = 8;                                  // "product done" barriers, by job index mod 8
constexpr int kThreadsPrefill = 608;                        // producer, score issuer, 16 softmax warps, product issuer
constexpr int kPvWarp = 18;
constexpr int kPlaneBytes = kTileQ * kHeadDim * 2;          // 16 KiB: 128 rows of 128 bytes
constexpr int kOffQ = 0;
constexpr int kOffKV = kQSlots * 2 * kPlaneBytes;
constexpr int kOffXchg = kOffKV + kStagesKV * 2 * kPlaneBytes;   // [2 query tiles][2 parities][2 halves][128 rows] f32
constexpr int kOffBars = kOffXchg + 2 * 2 * 2 * 128 * 4;
constexpr int kSeqCache = 512;                              // sequences whose offsets are kept in shared memory
constexpr int kOffSeq = kOffBars + 512;                     // q_offsets[0..n] then starts[0..n-1]
constexpr int kPrefillSmem = kOffSeq + (2 * kSeqCache + 1) * 4 + 1024;
static_assert(kPrefillSmem <= 232448, "shared memory per CTA");
// TMEM columns: score buffers 0-127, 128-255, 256-383 (each softmax thread writes its 32 columns
// of packed bf16 P over the first half of the 64 score columns it owns, behind its own reads);
// O of query tile A 384-447, of tile B 448-511.
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 384;
constexpr float kRescaleThreshold = 8.0f;                   // log2 domain

struct Bars {
    uint64_t q_full[kQSlots], q_empty[kQSlots];
    uint64_t kv_full[kStagesKV];
    uint64_t s_full[kSBufs], p_full[kSBufs];
    uint64_t pv_issued[kPvRing]; // job n's product is in the tensor pipe's queue: the scores of job n + 3 may follow it
    uint64_t pv_done[kPvRing];   // job n's product: frees its P columns, maybe its K/V stage, and O for a rescale
    uint64_t o_free[2];          // per query tile: the item's O rows are in registers
    uint64_t pair[2][4];         // per query tile and lane quarter: both threads of every row have written the exchange buffer
    uint32_t seen[2];            // per query tile: jobs whose scores its softmax warps have seen arrive
    uint32_t tmem_base;
    uint32_t pad;
};
static_assert(sizeof(Bars) <= 512, "barrier block");

// Optional cycle accounting of where each role waits (built only with -DCC_PREFILL_PROF).
#ifdef CC_PREFILL_PROF
__device__ unsigned long long g_prefill_prof[16];
__device__ long long g_prefill_trace[4 * 48 * 6];   // CTA 0, the four softmax warps of lane quarter 2: per job, six timestamps
__device__ long long g_prefill_trace2[3 * 96];   // CTA 0: per job, when its scores were issued, when its product was issued, when the score issuer saw the product of n-3 done
#define TRACE2(k, n) do { if (blockIdx.x == 0 && (n) < 96) g_prefill_trace2[(k) * 96 + (n)] = clock64(); } while (0)
#define TRACE(k) do { if (blockIdx.x == 0 && lane == 0 && quarter == 2 && own_jobs <= 48) g_prefill_trace[((grp * 2 + half) * 48 + (own_jobs - 1)) * 6 + (k)] = clock64(); } while (0)
#define PROF_ON (threadIdx.x == 64 || threadIdx.x == 0 || threadIdx.x == 32 || threadIdx.x == 576)
#define PROF_DECL unsigned long long prof_acc[16] = {}
#define PROF_PARAM , unsigned long long (&prof_acc)[16]
#define PROF_ARG , prof_acc
#define PROF_BEGIN(name) const long long name = clock64()
#define PROF_END(slot, name) prof_acc[slot] += static_cast<unsigned long long>(clock64() - name)
#define PROF_COUNT(slot) prof_acc[slot] += 1ull
#define PROF_FAIL(cond, site, num) do { if (!(cond)) { atomicOr(&g_prefill_prof[9], 1ull << (site)); if (atomicCAS(&g_prefill_prof[10], 0ull, static_cast<unsigned long long>(site)) == 0ull) { g_prefill_prof[11] = static_cast<unsigned long long>(num) * 1000ull + blockIdx.x; } } } while (0)
#define PROF_FLUSH() do { if (PROF_ON) { _Pragma("unroll") for (int i_ = 0; i_ < 16; ++i_) if (prof_acc[i_]) atomicAdd(&g_prefill_prof[i_], prof_acc[i_]); } } while (0)
#else
#define PROF_DECL
#define PROF_PARAM
#define PROF_ARG
#define PROF_BEGIN(name)
#define PROF_END(slot, name)
#define PROF_COUNT(slot)
#define TRACE(k)
#define TRACE2(k, n)
#define PROF_FAIL(cond, site, num)
#define PROF_FLUSH()
#endif

__device__ __forceinline__ float neg_inf_f() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// One work item: 256 queries (fewer at a sequence's end) of one head, as query tiles 0 (A) and 1 (B).
struct Item {
    bool valid;
    int head, kv_head, seq;
    int row0;            // first row of the sequence in q / out
    int t;               // new positions of the sequence
    int q0;              // first query of tile A within them
    int end;             // start + t: keys beyond are not there
    int first_pos[2], last_pos[2];
    int lo[2], hi[2];    // key tiles of each query tile (hi < lo: the tile has no rows)
    int t_lo, t_hi;      // key tiles of the item
};

// `q_offsets` and `starts` point at the shared-memory copies when the sequences fit there: item
// boundaries sit on the tensor-core threads' critical path and must not wait on global loads.
__device__ __forceinline__ Item make_item(const PrefillParams &p, const int32_t *q_offsets, const int32_t *starts,
                                          int id, int n_qt) {
    Item it;
    it.head = id % static_cast<int>(p.heads);
    const int r = id / static_cast<int>(p.heads);
    it.seq = r % static_cast<int>(p.seqs);
    const int q_tile = n_qt - 1 - r / static_cast<int>(p.seqs);   // long items first
    it.kv_head = it.head / kGroup;
    it.row0 = q_offsets[it.seq];
    it.t = q_offsets[it.seq + 1] - it.row0;
    it.q0 = q_tile * 2 * kTileQ;
    it.valid = it.q0 < it.t;
    const int start = starts[it.seq];
    it.end = start + it.t;
    const int W = static_cast<int>(p.window);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const int q_first = it.q0 + g * kTileQ;
        it.first_pos[g] = start + q_first;
        it.last_pos[g] = start + min(q_first + kTileQ, it.t) - 1;
        const int key_lo = (W != 0 && it.first_pos[g] + 1 > W) ? it.first_pos[g] + 1 - W : 0;
        const bool rows = q_first < it.t;
        it.lo[g] = rows ? key_lo / kTileK : 1;
        it.hi[g] = rows ? it.last_pos[g] / kTileK : 0;
    }
    it.t_lo = it.lo[0];
    it.t_hi = it.hi[1] >= it.lo[1] ? it.hi[1] : it.hi[0];
    return it;
}

// The softmax of one job for one query row (one thread): scores in `s_addr` (128 columns of this
// thread's TMEM lane), P written over their first 64 columns.  `lo_col..hi_col` are the visible
// columns of the row in this key tile (used on edge tiles only).
// A softmax thread owns 64 of a job's 128 score columns of its query row.  Both sweeps are
// loops of 32-column chunks, rolled on purpose: with the sweeps fully unrolled the straight-line
// code of the softmax warps no longer fitted the instruction cache and ran 1.4x slower.
constexpr int kColsPerThread = 64;

// First sweep: the maximum of this thread's scores.  `col0` is the tile column of the first one;
// `lo_col..hi_col` are the visible columns of the row in this key tile (used on edge tiles only).
template <bool kEdge>
__device__ __forceinline__ void max16(const uint32_t (&s)[16], int col, int lo_col, int hi_col, float &mx0, float &mx1,
                                      float &mx2, float &mx3) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        v[i] = (kEdge && (col + i > hi_col || col + i < lo_col)) ? neg_inf_f() : __uint_as_float(s[i]);
    mx0 = fmax3(mx0, v[0], v[1]);
    mx1 = fmax3(mx1, v[2], v[3]);
    mx2 = fmax3(mx2, v[4], v[5]);
    mx3 = fmax3(mx3, v[6], v[7]);
    mx0 = fmax3(mx0, v[8], v[9]);
    mx1 = fmax3(mx1, v[10], v[11]);
    mx2 = fmax3(mx2, v[12], v[13]);
    mx3 = fmax3(mx3, v[14], v[15]);
}

// Edge tiles of a window layer: minus infinity over the scores of this thread's 64 columns outside
// lo_col..hi_col.  Tensor-memory loads and stores are warp-wide instructions: only what every row of
// the warp sees whole is skipped.
__device__ __forceinline__ void mask_scores(uint32_t s_addr, int col0, int lo_col, int hi_col) {
#pragma unroll 1
    for (int c = 0; c < kColsPerThread / 16; ++c) {
        const int col = col0 + c * 16;
        if (__all_sync(0xffffffffu, col >= lo_col && col + 15 <= hi_col)) continue;
        uint32_t s[16];
        tmem_ld_x16(s_addr + c * 16, s);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (col + i > hi_col || col + i < lo_col) s[i] = 0xff800000u;
        tmem_st_x16(s_addr + c * 16, s);
    }
    tmem_wait_st();
}

// First sweep: the row maximum of this thread's 64 score columns.  The scores come from tensor memory
// in pieces of 16 columns, the next piece on its way while the current one is used; the loop stays
// rolled (two trips of 32 columns): unrolled, the kernel is bound by instruction fetch.
template <bool kEdge>
__device__ __forceinline__ float row_max_sweep(uint32_t s_addr, int col0, int lo_col, int hi_col) {
    float mx0 = neg_inf_f(), mx1 = neg_inf_f(), mx2 = neg_inf_f(), mx3 = neg_inf_f();
    uint32_t a[16], b[16];
    tmem_ld_x16(s_addr, a);
    tmem_wait_ld();
#pragma unroll 1
    for (int c = 0; c < kColsPerThread / 32; ++c) {
        tmem_ld_x16(s_addr + c * 32 + 16, b);
        max16<kEdge>(a, col0 + c * 32, lo_col, hi_col, mx0, mx1, mx2, mx3);
        tmem_wait_ld();
        if (c + 1 < kColsPerThread / 32) tmem_ld_x16(s_addr + c * 32 + 32, a);
        max16<kEdge>(b, col0 + c * 32 + 16, lo_col, hi_col, mx0, mx1, mx2, mx3);
        if (c + 1 < kColsPerThread / 32) tmem_wait_ld();
    }
    return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

template <bool kEdge>
__device__ __forceinline__ void exp16(const uint32_t (&s)[16], uint32_t p_addr, int col, int lo_col, int hi_col,
                                      float2 scale2, float2 neg_m2, float2 &l_acc) {
    uint32_t w[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        uint32_t s0 = s[2 * e], s1 = s[2 * e + 1];
        if (kEdge) {
            if (col + 2 * e > hi_col || col + 2 * e < lo_col) s0 = 0xff800000u;
            if (col + 2 * e + 1 > hi_col || col + 2 * e + 1 < lo_col) s1 = 0xff800000u;
        }
        const float2 x = ffma2(make_float2(__uint_as_float(s0), __uint_as_float(s1)), scale2, neg_m2);
        const uint32_t pair = pack_bf16x2_fast(ex2(x.x), ex2(x.y));
        w[e] = pair;
        l_acc = fadd2(l_acc, make_float2(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u)));
    }
    tmem_st_x8(p_addr, w);
}

// Second sweep: P = exp2(s * scale - m) as packed bf16 pairs, written to `p_addr` (32 columns,
// behind the scores already read); returns the sum of the rounded weights, the ones the product uses.
// Pieces of 16 columns, the next one on its way while the current one is used, as in the first sweep.
template <bool kEdge>
__device__ __forceinline__ float exp_sweep(uint32_t s_addr, uint32_t p_addr, int col0, int lo_col, int hi_col, float scale,
                                           float m_use) {
    const float2 scale2 = make_float2(scale, scale), neg_m2 = make_float2(-m_use, -m_use);
    float2 l_acc = make_float2(0.f, 0.f);
    uint32_t a[16], b[16];
    tmem_ld_x16(s_addr, a);
    tmem_wait_ld();
#pragma unroll 1
    for (int c = 0; c < kColsPerThread / 32; ++c) {
        tmem_ld_x16(s_addr + c * 32 + 16, b);
        exp16<kEdge>(a, p_addr + c * 16, col0 + c * 32, lo_col, hi_col, scale2, neg_m2, l_acc);
        tmem_wait_ld();
        if (c + 1 < kColsPerThread / 32) tmem_ld_x16(s_addr + c * 32 + 32, a);
        exp16<kEdge>(b, p_addr + c * 16 + 8, col0 + c * 32 + 16, lo_col, hi_col, scale2, neg_m2, l_acc);
        if (c + 1 < kColsPerThread / 32) tmem_wait_ld();
    }
    return l_acc.x + l_acc.y;
}

// Two instances.  kWindow false, launched for causal layers: the one edge tile per row of tiles takes
// the masked sweeps.  kWindow true, launched for window layers, where every tile is an edge tile:
// minus infinity is written over the unseen scores in a pass of its own and the sweeps exist unmasked
// only, 11 % faster there.  In one kernel the two ways cost each other time: the softmax warps are
// bound by instruction fetch, and every variant that made their code larger ran slower.
template <bool kWindow>
__global__ void __launch_bounds__(kThreadsPrefill, 1) prefill_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_qt = (static_cast<int>(p.max_t) + 2 * kTileQ - 1) / (2 * kTileQ);
    const int n_items = static_cast<int>(p.seqs) * n_qt * static_cast<int>(p.heads);
    const int W = static_cast<int>(p.window);

    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    Bars *bars = reinterpret_cast<Bars *>(smem + kOffBars);
    const uint32_t smem_base = smem_u32(smem);

    if (warp == 0 && lane == 0) {
        for (int b = 0; b < kQSlots; ++b) {
            mbar_init(&bars->q_full[b], 1);
            mbar_init(&bars->q_empty[b], 1);
        }
        for (int b = 0; b < kSBufs; ++b) {
            mbar_init(&bars->s_full[b], 1);
            mbar_init(&bars->p_full[b], 8);
        }
        for (int s = 0; s < kStagesKV; ++s) mbar_init(&bars->kv_full[s], 1);
        for (int s = 0; s < kPvRing; ++s) {
            mbar_init(&bars->pv_done[s], 1);
            mbar_init(&bars->pv_issued[s], 1);
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(&bars->o_free[g], 8);
            for (int q = 0; q < 4; ++q) mbar_init(&bars->pair[g][q], 2);
            bars->seen[g] = 0;
        }
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    const int32_t *q_offsets = p.q_offsets, *starts = p.starts;
    if (p.seqs <= kSeqCache) {
        int32_t *cache = reinterpret_cast<int32_t *>(smem + kOffSeq);
        for (int i = tid; i <= static_cast<int>(p.seqs); i += kThreadsPrefill) cache[i] = p.q_offsets[i];
        for (int i = tid; i < static_cast<int>(p.seqs); i += kThreadsPrefill) cache[p.seqs + 1 + i] = p.starts[i];
        q_offsets = cache;
        starts = cache + p.seqs + 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    PROF_DECL;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        const int pg = lane & 7;
        const bool is_v = lane >= 8;
        bool ok = true;
        int qs = 0, gt = 0, n = 0;
        int last_job[kStagesKV];   // last job that reads the tile held by each stage
#pragma unroll
        for (int s = 0; s < kStagesKV; ++s) last_job[s] = -1;
        for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
            const Item it = make_item(p, q_offsets, starts, id, n_qt);
            if (!it.valid) continue;
            if (lane == 0) {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if (it.hi[g] < it.lo[g] || !ok) continue;
                    const int slot = qs % kQSlots;
                    if (qs >= kQSlots) ok = mbar_wait(&bars->q_empty[slot], (qs / kQSlots - 1) & 1);
                    PROF_FAIL(ok, 1, qs);
                    if (ok) {
                        uint8_t *q_dst = smem + kOffQ + slot * 2 * kPlaneBytes;
                        const int row = it.row0 + it.q0 + g * kTileQ;
                        mbar_expect_tx(&bars->q_full[slot], 2 * kPlaneBytes);
                        tma_load_3d(q_dst, &p.q_hi_map, 0, it.head, row, &bars->q_full[slot]);
                        tma_load_3d(q_dst + kPlaneBytes, &p.q_lo_map, 0, it.head, row, &bars->q_full[slot]);
                    }
                    ++qs;
                }
            }
            const int32_t *table_row = p.block_table + static_cast<size_t>(it.seq) * p.max_pages;
            // row of this lane's page in the pool (a row past the end of the tensor = TMA writes zeros)
            auto lookup = [&](int kt) -> int {
                const int lp = kt * 8 + pg;
                int y = static_cast<int>(p.pool_rows);
                if (lane < 16 && lp * kPageTokens < it.end) {
                    uint32_t idx = static_cast<uint32_t>(lp);
                    if (p.ring_pages) idx %= p.ring_pages;
                    const int32_t page = idx < p.max_pages ? table_row[idx] : -1;
                    if (page < 0 || static_cast<uint32_t>(page) >= p.pool_pages)
                        raise_status(p.status, kStatusBadPage);
                    else
                        y = (page * static_cast<int>(p.kv_heads) + it.kv_head) * kTileRows + (is_v ? kPageTokens : 0);
                }
                return y;
            };
            int y_next = lookup(it.t_lo);
            for (int kt = it.t_lo; kt <= it.t_hi; ++kt, ++gt) {
                const int stage = gt % kStagesKV;
                const int y = y_next;
                if (kt < it.t_hi) y_next = lookup(kt + 1);   // in flight while this tile is issued
                int prev = -1;
#pragma unroll
                for (int s = 0; s < kStagesKV; ++s)
                    if (s == stage) prev = last_job[s];
                if (lane == 0) {
                    // the stage is free once the last product that read its previous tile is done
                    PROF_BEGIN(t_st);
                    if (prev >= 0) ok = mbar_wait(&bars->pv_done[prev % kPvRing], (prev / kPvRing) & 1);
                    PROF_END(15, t_st);
                    PROF_FAIL(ok, 2, gt);
                    if (ok) mbar_expect_tx(&bars->kv_full[stage], 2 * kPlaneBytes);
                }
                ok = __all_sync(0xffffffffu, ok);   // also orders the expect_tx before the loads below
                if (!ok) break;
                if (lane < 16)
                    tma_load_2d(smem + kOffKV + stage * 2 * kPlaneBytes + (is_v ? kPlaneBytes : 0) + pg * 2048, &p.pool_map,
                                0, y, &bars->kv_full[stage]);
#pragma unroll
                for (int g = 0; g < 2; ++g)
                    if (kt >= it.lo[g] && kt <= it.hi[g]) ++n;
#pragma unroll
                for (int s = 0; s < kStagesKV; ++s)
                    if (s == stage) last_job[s] = n - 1;
            }
        }
        if (!ok && lane == 0) raise_status(p.status, kStatusWaitTimeout);
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ score issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(kTileQ, kTileK, false);
            bool ok = true;
            int qs = 0, gt = 0, n = 0;
            for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
                const Item it = make_item(p, q_offsets, starts, id, n_qt);
                if (!it.valid) continue;
                int slot[2];
                bool q_ready[2] = {false, false};
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    slot[g] = qs;
                    if (it.hi[g] >= it.lo[g]) ++qs;
                }
                for (int kt = it.t_lo; kt <= it.t_hi && ok; ++kt, ++gt) {
                    const int stage = gt % kStagesKV;
                    PROF_BEGIN(t_kv);
                    ok = mbar_wait(&bars->kv_full[stage], (gt / kStagesKV) & 1);
                    PROF_END(12, t_kv);
                    PROF_FAIL(ok, 3, gt);
                    const uint64_t k_desc = smem_desc_sw128(smem_base + kOffKV + stage * 2 * kPlaneBytes, 16, 1024);
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        if (kt < it.lo[g] || kt > it.hi[g] || !ok) continue;
                        const int sl = slot[g] % kQSlots;
                        if (!q_ready[g]) {
                            ok = mbar_wait(&bars->q_full[sl], (slot[g] / kQSlots) & 1);
                            PROF_FAIL(ok, 4, n);
                            q_ready[g] = true;
                        }
                        const uint64_t qhi_desc = smem_desc_sw128(smem_base + kOffQ + sl * 2 * kPlaneBytes, 16, 1024);
                        const uint64_t qlo_desc = qhi_desc + (kPlaneBytes >> 4);
                        const uint32_t d = tmem + static_cast<uint32_t>(n % kSBufs) * kTileK;
                        uint64_t *full_bar = &bars->s_full[n % kSBufs];
                        // S(n) goes where P(n - 3) was.  The tensor pipe runs what it is given in order,
                        // so that product only has to have been issued (not finished) before these scores
                        // are: the fences on both sides of the barrier order the two threads' instructions.
                        PROF_BEGIN(t_sf);
                        if (ok && n >= kSBufs)
                            ok = mbar_wait(&bars->pv_issued[(n - kSBufs) % kPvRing], ((n - kSBufs) / kPvRing) & 1);
                        PROF_END(13, t_sf);
                        PROF_FAIL(ok, 5, n);
                        if (!ok) break;
                        tc_fence_after();
                        TRACE2(2, n);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) umma_bf16(d, qhi_desc + ks * 2, k_desc + ks * 2, idesc_qk, ks > 0);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) umma_bf16(d, qlo_desc + ks * 2, k_desc + ks * 2, idesc_qk, true);
                        TRACE2(0, n);
                        umma_commit(full_bar);
                        if (kt == it.hi[g]) umma_commit(&bars->q_empty[sl]);   // all scores of this query tile are issued
                        ++n;
                    }
                }
            }
            if (!ok) raise_status(p.status, kStatusWaitTimeout);
        }
        __syncwarp();
    } else if (warp == kPvWarp) {
        // ---------------------------------------------------------- product issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc_pv = umma_idesc_bf16(kTileQ, kHeadDim, true);
            bool ok = true;
            int gt = 0, n = 0;
            int items_of[2] = {0, 0};   // items in which each query tile had rows
            for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
                const Item it = make_item(p, q_offsets, starts, id, n_qt);
                if (!it.valid) continue;
                bool first[2] = {true, true};
                for (int kt = it.t_lo; kt <= it.t_hi && ok; ++kt, ++gt) {
                    const int stage = gt % kStagesKV;
                    const uint64_t v_desc =
                        smem_desc_sw128(smem_base + kOffKV + stage * 2 * kPlaneBytes + kPlaneBytes, 1024, 1024);
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        if (kt < it.lo[g] || kt > it.hi[g] || !ok) continue;
                        // the first product of an item overwrites O: the previous item's rows must be out
                        if (first[g] && items_of[g] > 0) ok = mbar_wait(&bars->o_free[g], (items_of[g] - 1) & 1);
                        PROF_FAIL(ok, 6, n);
                        // everything that does not need P first: what follows the wait for P is on
                        // the critical path of the job after next
                        if (ok) ok = mbar_wait(&bars->kv_full[stage], (gt / kStagesKV) & 1);   // long since there
                        // P comes from tensor memory: 16 keys of a k-step are 8 columns of packed bf16 pairs;
                        // keys 0-63 sit in columns 0-31 of the buffer, keys 64-127 in columns 64-95
                        const uint32_t p_tmem = tmem + static_cast<uint32_t>(n % kSBufs) * kTileK;
                        const uint32_t o_tmem = tmem + kColO + static_cast<uint32_t>(g) * kHeadDim;
                        uint64_t *done_bar = &bars->pv_done[n % kPvRing], *issued_bar = &bars->pv_issued[n % kPvRing];
                        const bool fresh = first[g];
                        PROF_BEGIN(t_pf);
                        if (ok) ok = mbar_wait(&bars->p_full[n % kSBufs], (n / kSBufs) & 1);
                        PROF_END(14, t_pf);
                        PROF_FAIL(ok, 7, n);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            umma_bf16_ts(o_tmem, p_tmem + (ks >> 2) * 64 + (ks & 3) * 8, v_desc + ks * (2048 >> 4), idesc_pv, !fresh || ks > 0);
                        umma_commit(done_bar);
                        tc_fence_before();
                        mbar_arrive(issued_bar);
                        TRACE2(1, n);
                        first[g] = false;
                        ++n;
                    }
                }
#pragma unroll
                for (int g = 0; g < 2; ++g)
                    if (it.hi[g] >= it.lo[g]) ++items_of[g];
            }
            if (!ok) raise_status(p.status, kStatusWaitTimeout);
        }
        __syncwarp();
    } else {
        // ------------------------------------- softmax, two threads per query row (64 keys each)
        const int sw = warp - 2;                      // 0..15
        const int quarter = warp & 3;                 // the TMEM lanes this warp can reach
        const int grp = sw >> 3;                      // query tile A or B
        const int half = (sw >> 2) & 1;               // which 64 of a tile's 128 keys, which 32 of O's 64 columns
        const int row = quarter * 32 + lane;          // row of the query tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t o_addr = tmem + lane_addr + kColO + static_cast<uint32_t>(grp * kHeadDim + half * 32);
        float *xchg = reinterpret_cast<float *>(smem + kOffXchg) + grp * (2 * 2 * 128);
        uint64_t *pair_bar = &bars->pair[grp][quarter];
        const float scale = p.scale_log2e;
        bool ok = true;
        int n = 0;
        uint32_t meets = 0;    // exchanges with the row's other thread so far
        uint32_t own_jobs = 0, other_jobs = 0;
        volatile uint32_t *seen_own = &bars->seen[grp], *seen_other = &bars->seen[grp ^ 1];
        PROF_BEGIN(t_soft);
        // Both threads of a row leave their value in the exchange buffer and pick up the other's.
        auto exchange = [&](float mine, float &theirs) -> bool {
            const uint32_t par = meets & 1;
            xchg[(par * 2 + half) * 128 + row] = mine;
            __syncwarp();
            if (lane == 0) mbar_arrive(pair_bar);
            const bool met = __all_sync(0xffffffffu, mbar_wait(pair_bar, par));
            theirs = xchg[(par * 2 + (half ^ 1)) * 128 + row];
            ++meets;
            return met;
        };
        for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
            const Item it = make_item(p, q_offsets, starts, id, n_qt);
            if (!it.valid) continue;
            const int my_first = grp ? it.first_pos[1] : it.first_pos[0];
            const int my_last = grp ? it.last_pos[1] : it.last_pos[0];
            const int pos = my_first + row;                // absolute position of this query
            const int vis_lo = (W != 0 && pos + 1 > W) ? pos + 1 - W : 0;
            float m = neg_inf_f(), l = 0.f;   // l: this thread's half of the row sum
            int prev_own = -1;
            for (int kt = it.t_lo; kt <= it.t_hi && ok; ++kt) {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if (kt < it.lo[g] || kt > it.hi[g] || !ok) continue;
                    if (g != grp) {
                        ++other_jobs;
                        ++n;
                        continue;
                    }
                    const int b = n % kSBufs;
                    PROF_BEGIN(t_s);
                    // A wait on an mbarrier names a phase by its parity only, so it must not be
                    // made more than one phase early: the other query tile's softmax has to have
                    // seen the scores of all its earlier jobs (the last users of this buffer among
                    // them) before this one's are waited for.  Matters when one tile has no rows
                    // for a while and its warps run ahead.
                    if (*seen_other < other_jobs) {
                        const long long began = clock64();
                        while (*seen_other < other_jobs && ok) {
                            __nanosleep(64);
                            if (clock64() - began > kWaitCycles) ok = false;
                        }
                        ok = __all_sync(0xffffffffu, ok);
                        PROF_FAIL(ok, 8, n);
                        if (!ok) break;
                    }
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[b], (n / kSBufs) & 1));
                    ++own_jobs;
                    if ((sw & 7) == 0 && lane == 0) *seen_own = own_jobs;
                    TRACE(0);
                    PROF_END(0, t_s);
                    PROF_FAIL(ok, 9, n);
                    if (!ok) break;
                    tc_fence_after();
                    PROF_BEGIN(t_p1);
                    const uint32_t s_addr = tmem + lane_addr + static_cast<uint32_t>(b * kTileK + half * kColsPerThread);
                    const uint32_t p_addr = s_addr;   // P goes over this thread's own scores, behind the reads
                    const int col0 = half * kColsPerThread;
                    const int lo_col = vis_lo - kt * kTileK, hi_col = pos - kt * kTileK;
                    const bool edge = (kt * kTileK + kTileK - 1 > my_first) || (W != 0 && kt * kTileK + W <= my_last);
                    float mx;
                    if constexpr (kWindow) {
                        if (edge) mask_scores(s_addr, col0, lo_col, hi_col);
                        mx = row_max_sweep<false>(s_addr, col0, lo_col, hi_col);
                    } else {
                        mx = edge ? row_max_sweep<true>(s_addr, col0, lo_col, hi_col)
                                  : row_max_sweep<false>(s_addr, col0, lo_col, hi_col);
                    }
                    PROF_END(1, t_p1);
                    TRACE(1);
                    PROF_BEGIN(t_x);
                    float mx_other;
                    ok = exchange(mx, mx_other);
                    PROF_END(2, t_x);
                    TRACE(2);
                    PROF_FAIL(ok, 10, n);
                    if (!ok) break;
                    mx = fmaxf(mx, mx_other);
                    const float m_cand = fmaxf(m, mx * scale);
                    // keep the old maximum unless it moved by more than 2^8: fewer trips through TMEM
                    const bool move = (m_cand > m + kRescaleThreshold) || (m == neg_inf_f() && m_cand > m);
                    const float m_new = move ? m_cand : m;
                    const float m_use = m_new == neg_inf_f() ? 0.f : m_new;
                    const float alpha = move ? ex2(m - m_use) : 1.0f;
                    m = m_new;
                    l *= alpha;
                    // Only a rescale has to wait for this query tile's previous product.
                    if (prev_own >= 0 && __any_sync(0xffffffffu, move)) {
                        PROF_BEGIN(t_rs);
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done[prev_own % kPvRing], (prev_own / kPvRing) & 1));
                        if (!ok) break;
                        tc_fence_after();
                        uint32_t o[32];
                        tmem_ld_x32(o_addr, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_x32(o_addr, o);
                        tmem_wait_st();

                    }
                    TRACE(3);
                    PROF_BEGIN(t_ex);
                    if constexpr (kWindow) {
                        l += exp_sweep<false>(s_addr, p_addr, col0, lo_col, hi_col, scale, m_use);
                    } else {
                        l += edge ? exp_sweep<true>(s_addr, p_addr, col0, lo_col, hi_col, scale, m_use)
                                  : exp_sweep<false>(s_addr, p_addr, col0, lo_col, hi_col, scale, m_use);
                    }
                    PROF_END(4, t_ex);
                    TRACE(4);
                    PROF_BEGIN(t_pub);
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->p_full[b]);
                    PROF_END(5, t_pub);
                    TRACE(5);
                    PROF_COUNT(8);
                    prev_own = n;
                    ++n;
                }
            }
            if (!ok) break;
            if (prev_own < 0) continue;   // this query tile has no rows in this item
            // ---- the item's rows: wait for the last product, read O, hand the accumulator back, store
            PROF_BEGIN(t_epi);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done[prev_own % kPvRing], (prev_own / kPvRing) & 1));
            PROF_FAIL(ok, 12, n);
            if (!ok) break;
            tc_fence_after();
            uint32_t o[32];
            tmem_ld_x32(o_addr, o);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->o_free[grp]);    // the next item's first product may overwrite O now
            float l_other;
            ok = exchange(l, l_other);
            PROF_FAIL(ok, 13, n);
            if (!ok) break;
            l += l_other;
            const float sink2 = p.sinks ? p.sinks[it.head] * 1.4426950408889634f : neg_inf_f();
            const float Mt = fmaxf(m, sink2);
            const float e = m == neg_inf_f() ? 0.f : ex2(m - Mt);
            const float total = l * e + (p.sinks ? ex2(sink2 - Mt) : 0.f);
            const float inv = total > 0.f ? e / total : 0.f;
            const int q_row = it.q0 + grp * kTileQ + row;
            if (q_row < it.t) {
                uint16_t *out_row = p.out + (static_cast<size_t>(it.row0 + q_row) * p.heads + it.head) * kHeadDim + half * 32;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v = make_uint4(pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                                         pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                                         pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                                         pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
                    *reinterpret_cast<uint4 *>(out_row + i) = v;
                }
            }
            PROF_END(6, t_epi);
        }
        PROF_END(7, t_soft);
        if (!ok && lane == 0) raise_status(p.status, kStatusWaitTimeout);
    }
    PROF_FLUSH();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

#ifdef CC_PREFILL_PROF
extern "C" void cc_debug_prefill_trace(long long *out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_prefill_trace, sizeof(long long) * 4 * 48 * 6);
    cudaMemcpyFromSymbol(out + 4 * 48 * 6, g_prefill_trace2, sizeof(long long) * 3 * 96);
}
extern "C" void cc_debug_prefill_prof(unsigned long long *out, int reset) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_prefill_prof, sizeof(unsigned long long) * 16);
    if (reset) {
        unsigned long long zero[16] = {};
        cudaMemcpyToSymbol(g_prefill_prof, zero, sizeof zero);
    }
}
#endif

void launch_prefill(const PrefillParams &p, cudaStream_t stream) {
    cudaFuncSetAttribute(prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem);
    cudaFuncSetAttribute(prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem);
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long items = static_cast<long long>(p.seqs) * ((p.max_t + 2 * kTileQ - 1) / (2 * kTileQ)) * p.heads;
    const unsigned grid = static_cast<unsigned>(items < sms ? items : sms);   // one persistent CTA per SM
    if (p.window != 0)
        prefill_kernel<true><<<grid, kThreadsPrefill, kPrefillSmem, stream>>>(p);
    else
        prefill_kernel<false><<<grid, kThreadsPrefill, kPrefillSmem, stream>>>(p);
}

}  // namespace cc
