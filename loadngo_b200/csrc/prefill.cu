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
// A work item = 128 queries of one head.  CTAs are persistent (one per SM): each walks its own
// fixed sequence of items (heaviest first, the 8 heads of a KV group next to each other so that
// they share K and V through L2), and its pipelines run on across item boundaries: while the
// softmax warps finish one item, the producer is already loading the next item's Q, K and V and
// the tensor core is already computing its first scores.  Eleven warps, four roles:
//   warp 0  producer: TMA loads of the Q tile (hi and lo planes, double-buffered) and, per
//           128-key tile, eight 16-key pages of K and of V, found through the block table, into
//           rings (sixteen lanes look up and issue one page each);
//   warp 1  one thread issues the score products S = Qhi K^T + Qlo K^T (tcgen05.mma M128 N128 K64
//           twice) into one of two S buffers in TMEM, up to two tiles ahead of the products;
//   warp 10 one thread issues O += P V (M128 N64 K128, P read from TMEM) into the O accumulator
//           in TMEM.  Every tcgen05.mma costs about 60 cycles of tensor pipe however narrow it is
//           (measured), so nothing small rides on the tensor core (the row sums stay with the
//           softmax threads), and the two streams have an issuer each so that one thread's
//           barrier traffic never leaves the pipe empty;
//   warps 2-9  softmax: two threads per query row, each owning 64 of the tile's 128 keys.  A
//           thread reads its half of the S row from TMEM, masks edge tiles, shares the row
//           maximum with its partner through shared memory, writes P = exp2(s - m) as bf16
//           back into tensor memory over the scores it came from (the products read their A
//           operand from TMEM, so P never touches shared memory, whose bandwidth the Q K^T
//           operands already use), and rescales its half of the O row (and the L column) in TMEM when the maximum moved
//           by more than 2^8; at the end of an item it folds the sink in, normalises and stores
//           64 bytes of bf16 output.
// Tiles entirely outside a query tile's causal / window range are never visited (the loop
// bounds exclude them, as kernels.metal:631-634 does); only edge tiles are masked per element.
//
// Every mbarrier wait is bounded; a wait that runs out raises the status word and the CTA
// drains, frees its TMEM and returns.
#include "kernels.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace cc {
namespace {

constexpr int kTileQ = 128, kTileK = 128;
constexpr int kStagesKV = 3;                               // K tile + V tile per stage
constexpr int kPvRing = 6;                                  // "product done" barriers, by tile index mod 6
constexpr int kThreadsPrefill = 352;
constexpr int kSoftmaxThreads = 256;
constexpr int kPlaneBytes = kTileQ * kHeadDim * 2;          // 16 KiB: 128 rows of 128 bytes
constexpr int kOffQ = 0;                                    // 2 buffers of (hi plane, lo plane)
constexpr int kOffKV = 2 * 2 * kPlaneBytes;                 // per stage: K tile then V tile
constexpr int kOffXchg = kOffKV + kStagesKV * 2 * kPlaneBytes;    // [2 tiles in flight + 1 for row sums][2 halves][128 rows] f32
constexpr int kOffBars = kOffXchg + 3 * 2 * 128 * 4;
constexpr int kSeqCache = 512;                              // sequences whose offsets are kept in shared memory
constexpr int kOffSeq = kOffBars + 256;                     // q_offsets[0..n] then starts[0..n-1]
constexpr int kPrefillSmem = kOffSeq + (2 * kSeqCache + 1) * 4 + 1024;
// TMEM columns: S0 0-127, S1 128-255 (P(g) overwrites the first 64 columns of S(g)'s buffer as
// packed bf16 pairs once both threads of every row hold their scores in registers), O 256-319.
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 256;
constexpr float kRescaleThreshold = 8.0f;                   // log2 domain

struct Bars {
    uint64_t q_full[2], q_empty[2];
    uint64_t kv_full[kStagesKV];
    uint64_t s_full[2], p_full[2];
    uint64_t pv_done[kPvRing];   // tile g's product: frees its K/V stage, its P columns, and O for a rescale
    uint64_t o_free;
    uint32_t tmem_base;
    uint32_t pad;
};
static_assert(sizeof(Bars) <= 256, "barrier block");

__device__ __forceinline__ float neg_inf_f() { return __int_as_float(0xff800000); }

// Optional cycle accounting of where each role waits (built only with -DCC_PREFILL_PROF).
#ifdef CC_PREFILL_PROF
__device__ unsigned long long g_prefill_prof[16];
#define PROF_T0() const long long prof_t0_ = clock64()
#define PROF_ADD(slot) atomicAdd(&g_prefill_prof[slot], static_cast<unsigned long long>(clock64() - prof_t0_))
#define PROF_WAIT(slot, expr) [&] { const long long t_ = clock64(); const bool r_ = (expr); \
    atomicAdd(&g_prefill_prof[slot], static_cast<unsigned long long>(clock64() - t_)); return r_; }()
#define PROF_BEGIN(name) const long long name = clock64()
#define PROF_END(slot, name) atomicAdd(&g_prefill_prof[slot], static_cast<unsigned long long>(clock64() - name))
#else
#define PROF_BEGIN(name)
#define PROF_END(slot, name)
#define PROF_T0()
#define PROF_ADD(slot)
#define PROF_WAIT(slot, expr) (expr)
#endif

// One work item: 128 queries (fewer at a sequence's end) of one head.
struct Item {
    bool valid;
    int head, kv_head, seq;
    int row0;        // first row of the sequence in q / out
    int t;           // new positions of the sequence
    int q0;          // first query of this tile within them
    int end;         // start + t: keys beyond are not there
    int first_pos, last_pos;
    int kt_lo, n_tiles;
};

// `q_offsets` and `starts` point at the shared-memory copies when the sequences fit there: item
// boundaries sit on the tensor-core thread's critical path and must not wait on global loads.
__device__ __forceinline__ Item make_item(const PrefillParams &p, const int32_t *q_offsets, const int32_t *starts,
                                          int id, int n_qt) {
    Item it;
    it.head = id % static_cast<int>(p.heads);
    const int r = id / static_cast<int>(p.heads);
    const int q_tile = n_qt - 1 - (r % n_qt);   // long tiles first
    it.seq = r / n_qt;
    it.kv_head = it.head / kGroup;
    it.row0 = q_offsets[it.seq];
    it.t = q_offsets[it.seq + 1] - it.row0;
    it.q0 = q_tile * kTileQ;
    it.valid = it.q0 < it.t;
    const int start = starts[it.seq];
    it.end = start + it.t;
    it.first_pos = start + it.q0;
    it.last_pos = start + min(it.q0 + kTileQ, it.t) - 1;
    const int W = static_cast<int>(p.window);
    const int key_lo = (W != 0 && it.first_pos + 1 > W) ? it.first_pos + 1 - W : 0;
    it.kt_lo = key_lo / kTileK;
    it.n_tiles = it.valid ? it.last_pos / kTileK - it.kt_lo + 1 : 0;
    return it;
}

__global__ void __launch_bounds__(kThreadsPrefill, 1) prefill_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_qt = (static_cast<int>(p.max_t) + kTileQ - 1) / kTileQ;
    const int n_items = static_cast<int>(p.seqs) * n_qt * static_cast<int>(p.heads);
    const int W = static_cast<int>(p.window);

    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    Bars *bars = reinterpret_cast<Bars *>(smem + kOffBars);
    const uint32_t smem_base = smem_u32(smem);

    if (warp == 0 && lane == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->q_full[b], 1);
            mbar_init(&bars->q_empty[b], 1);
            mbar_init(&bars->s_full[b], 1);
            mbar_init(&bars->p_full[b], kSoftmaxThreads);
        }
        for (int s = 0; s < kStagesKV; ++s) mbar_init(&bars->kv_full[s], 1);
        for (int s = 0; s < kPvRing; ++s) mbar_init(&bars->pv_done[s], 1);
        mbar_init(&bars->o_free, kSoftmaxThreads);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        const int pg = lane & 7;
        const bool is_v = lane >= 8;
        bool ok = true;
        int n_it = 0, g = 0;
        for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
            const Item it = make_item(p, q_offsets, starts, id, n_qt);
            if (!it.valid) continue;
            const int qb = n_it & 1;
            if (lane == 0) {
                if (n_it >= 2) ok = mbar_wait(&bars->q_empty[qb], ((n_it >> 1) - 1) & 1);
                if (ok) {
                    uint8_t *q_dst = smem + kOffQ + qb * 2 * kPlaneBytes;
                    mbar_expect_tx(&bars->q_full[qb], 2 * kPlaneBytes);
                    tma_load_3d(q_dst, &p.q_hi_map, 0, it.head, it.row0 + it.q0, &bars->q_full[qb]);
                    tma_load_3d(q_dst + kPlaneBytes, &p.q_lo_map, 0, it.head, it.row0 + it.q0, &bars->q_full[qb]);
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
            int y_next = lookup(it.kt_lo);
            for (int j = 0; j < it.n_tiles; ++j, ++g) {
                const int stage = g % kStagesKV;
                const int y = y_next;
                if (j + 1 < it.n_tiles) y_next = lookup(it.kt_lo + j + 1);   // in flight while this tile is issued
                if (lane == 0) {
                    // the stage is free once the product of the tile that used it (g - 3) is done
                    if (g >= kStagesKV)
                        ok = PROF_WAIT(10, mbar_wait(&bars->pv_done[(g - kStagesKV) % kPvRing], ((g - kStagesKV) / kPvRing) & 1));
                    if (ok) mbar_expect_tx(&bars->kv_full[stage], 2 * kPlaneBytes);
                }
                ok = __all_sync(0xffffffffu, ok);   // also orders the expect_tx before the loads below
                if (!ok) break;
                if (lane < 16)
                    tma_load_2d(smem + kOffKV + stage * 2 * kPlaneBytes + (is_v ? kPlaneBytes : 0) + pg * 2048, &p.pool_map,
                                0, y, &bars->kv_full[stage]);
            }
            ++n_it;
        }
        if (!ok && lane == 0) raise_status(p.status, kStatusWaitTimeout);
        __syncwarp();
    } else if (warp == 1 || warp == 10) {
        // ------------------------------------------- two MMA issuers: warp 1 scores, warp 10 products
        // Each walks the CTA's item sequence on its own.  One thread issuing everything spent more
        // time on barrier waits and commits between its instructions than the tensor pipe needs
        // to run them; with two issuers the pipe always has the other stream's work queued.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(kTileQ, kTileK, false);
            constexpr uint32_t idesc_pv = umma_idesc_bf16(kTileQ, kHeadDim, true);
            const bool scores = warp == 1;
            bool ok = true;
            int n_it = 0, g = 0;
            PROF_T0();
            for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
                const Item it = make_item(p, q_offsets, starts, id, n_qt);
                if (!it.valid) continue;
                const int qb = n_it & 1;
                if (scores) {
                    ok = PROF_WAIT(0, mbar_wait(&bars->q_full[qb], (n_it >> 1) & 1));
                    const uint64_t qhi_desc = smem_desc_sw128(smem_base + kOffQ + qb * 2 * kPlaneBytes, 16, 1024);
                    const uint64_t qlo_desc = qhi_desc + (kPlaneBytes >> 4);
                    for (int j = 0; j < it.n_tiles && ok; ++j, ++g) {
                        const int stage = g % kStagesKV;
                        ok = PROF_WAIT(1, mbar_wait(&bars->kv_full[stage], (g / kStagesKV) & 1));
                        // S(g) goes where P(g - 2) was: that product must have read it
                        if (ok && g >= 2) ok = PROF_WAIT(2, mbar_wait(&bars->pv_done[(g - 2) % kPvRing], ((g - 2) / kPvRing) & 1));
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t k_desc = smem_desc_sw128(smem_base + kOffKV + stage * 2 * kPlaneBytes, 16, 1024);
                        const uint32_t d = tmem + static_cast<uint32_t>(g & 1) * kTileK;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) umma_bf16(d, qhi_desc + ks * 2, k_desc + ks * 2, idesc_qk, ks > 0);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) umma_bf16(d, qlo_desc + ks * 2, k_desc + ks * 2, idesc_qk, true);
                        umma_commit(&bars->s_full[g & 1]);
                    }
                    if (ok) umma_commit(&bars->q_empty[qb]);   // all scores of this item are issued
                } else {
                    // the first product of an item overwrites O: the previous item's rows must be out
                    if (n_it > 0) ok = PROF_WAIT(3, mbar_wait(&bars->o_free, (n_it - 1) & 1));
                    for (int j = 0; j < it.n_tiles && ok; ++j, ++g) {
                        const int stage = g % kStagesKV, b = g & 1;
                        ok = PROF_WAIT(4, mbar_wait(&bars->p_full[b], (g >> 1) & 1));
                        if (ok) ok = mbar_wait(&bars->kv_full[stage], (g / kStagesKV) & 1);   // long since there
                        if (!ok) break;
                        tc_fence_after();
                        // P comes from tensor memory: 16 keys of a k-step are 8 columns of packed bf16 pairs
                        const uint32_t p_tmem = tmem + static_cast<uint32_t>(b) * kTileK;
                        const uint64_t v_desc =
                            smem_desc_sw128(smem_base + kOffKV + stage * 2 * kPlaneBytes + kPlaneBytes, 1024, 1024);
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            umma_bf16_ts(tmem + kColO, p_tmem + ks * 8, v_desc + ks * (2048 >> 4), idesc_pv, j > 0 || ks > 0);
                        umma_commit(&bars->pv_done[g % kPvRing]);
                    }
                }
                ++n_it;
            }
            if (!ok) raise_status(p.status, kStatusWaitTimeout);
            PROF_ADD(5);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------- softmax, two threads per row (64 keys each)
        const int quarter = warp & 3;                 // the TMEM lanes this warp can reach
        const int half = (warp - 2) >> 2;             // which 64 of the tile's 128 keys, which 32 of O's 64 columns
        const int row = quarter * 32 + lane;          // row of the query tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        float *xchg = reinterpret_cast<float *>(smem + kOffXchg);
        const float scale = p.scale_log2e;
        bool ok = true;
        int n_it = 0, g = 0;
#ifdef CC_PREFILL_PROF
        const long long soft_t0 = clock64();
#endif
        for (int id = blockIdx.x; id < n_items && ok; id += gridDim.x) {
            const Item it = make_item(p, q_offsets, starts, id, n_qt);
            if (!it.valid) continue;
            const int pos = it.first_pos + row;       // absolute position of this query
            const int vis_lo = (W != 0 && pos + 1 > W) ? pos + 1 - W : 0;
            float m = neg_inf_f(), l = 0.f;   // l: this thread's half of the row sum
            for (int j = 0; j < it.n_tiles; ++j, ++g) {
                const int b = g & 1;
#ifdef CC_PREFILL_PROF
                if (tid == 64) ok = PROF_WAIT(6, mbar_wait(&bars->s_full[b], (g >> 1) & 1));
                else
#endif
                ok = mbar_wait(&bars->s_full[b], (g >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                uint32_t s[2][32];
#pragma unroll
                for (int c = 0; c < 2; ++c) tmem_ld_x32(tmem + lane_addr + b * kTileK + half * 64 + c * 32, s[c]);
                tmem_wait_ld();
                const int kt = it.kt_lo + j;
                const int key0 = kt * kTileK + half * 64;
                const bool edge = (kt * kTileK + kTileK - 1 > it.first_pos) || (W != 0 && kt * kTileK + W <= it.last_pos);
                if (edge) {
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int key = key0 + c * 32 + i;
                            if (key > pos || key < vis_lo) s[c][i] = 0xff800000u;
                        }
                }
                float mx = neg_inf_f();
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx = fmaxf(mx, fmaxf(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])));
                // the row maximum over both halves: through shared memory, one named barrier per tile
                xchg[(b * 2 + half) * 128 + row] = mx;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                mx = fmaxf(mx, xchg[(b * 2 + (half ^ 1)) * 128 + row]);
                const float m_cand = fmaxf(m, mx * scale);
                // keep the old maximum unless it moved by more than 2^8: fewer trips through TMEM
                const bool move = (m_cand > m + kRescaleThreshold) || (m == neg_inf_f() && m_cand > m);
                const float m_new = move ? m_cand : m;
                const float m_use = m_new == neg_inf_f() ? 0.f : m_new;
                const float alpha = move ? ex2(m - m_use) : 1.0f;
                m = m_new;
                l *= alpha;
                // Only a rescale has to wait for the previous tile's P V product; the common case
                // goes straight on to its exponentials while that product is still running.
                if (j > 0 && __any_sync(0xffffffffu, move)) {
                    ok = mbar_wait(&bars->pv_done[(g - 1) % kPvRing], ((g - 1) / kPvRing) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t o[32];
                    tmem_ld_x32(tmem + lane_addr + kColO + half * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_x32(tmem + lane_addr + kColO + half * 32, o);
                    tmem_wait_st();
                }
                // P = exp2(s * scale - m) as packed bf16 pairs, written over this row's scores in
                // tensor memory (every thread of the CTA holds its scores in registers since the
                // barrier above; the tensor core reads P before it overwrites the buffer again).
                const float2 scale2 = make_float2(scale, scale), neg_m2 = make_float2(-m_use, -m_use);
                uint32_t w[32];
                float l_acc[2] = {0.f, 0.f};
#pragma unroll
                for (int c = 0; c < 2; ++c) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const float2 x = ffma2(make_float2(__uint_as_float(s[c][2 * e]), __uint_as_float(s[c][2 * e + 1])),
                                               scale2, neg_m2);
                        const uint32_t pair = pack_bf16x2_fast(ex2(x.x), ex2(x.y));
                        w[c * 16 + e] = pair;
                        // the denominator sums the rounded weights, the ones the product uses
                        l_acc[e & 1] += __uint_as_float(pair << 16) + __uint_as_float(pair & 0xffff0000u);
                    }
                }
                l += l_acc[0] + l_acc[1];
                tmem_st_x32(tmem + lane_addr + b * kTileK + half * 32, w);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars->p_full[b]);
            }
            if (!ok) break;
            // ---- the item's rows: wait for its last product, read O and L, hand them back, store
#ifdef CC_PREFILL_PROF
            if (tid == 64) ok = PROF_WAIT(7, mbar_wait(&bars->pv_done[(g - 1) % kPvRing], ((g - 1) / kPvRing) & 1));
            else
#endif
            ok = mbar_wait(&bars->pv_done[(g - 1) % kPvRing], ((g - 1) / kPvRing) & 1);
            if (!ok) break;
            tc_fence_after();
            uint32_t o[32];
            tmem_ld_x32(tmem + lane_addr + kColO + half * 32, o);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&bars->o_free);    // the next item's first product may overwrite O now
            // the two halves of the row sum meet through their own slots of the exchange buffer
            xchg[(4 + half) * 128 + row] = l;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            l += xchg[(4 + (half ^ 1)) * 128 + row];
            const float sink2 = p.sinks ? p.sinks[it.head] * 1.4426950408889634f : neg_inf_f();
            const float Mt = fmaxf(m, sink2);
            const float e = m == neg_inf_f() ? 0.f : ex2(m - Mt);
            const float total = l * e + (p.sinks ? ex2(sink2 - Mt) : 0.f);
            const float inv = total > 0.f ? e / total : 0.f;
            if (it.q0 + row < it.t) {
                uint16_t *out_row =
                    p.out + (static_cast<size_t>(it.row0 + it.q0 + row) * p.heads + it.head) * kHeadDim + half * 32;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v = make_uint4(pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                                         pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                                         pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                                         pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
                    *reinterpret_cast<uint4 *>(out_row + i) = v;
                }
            }
            ++n_it;
        }
        if (!ok && lane == 0) raise_status(p.status, kStatusWaitTimeout);
#ifdef CC_PREFILL_PROF
        if (tid == 64) {
            atomicAdd(&g_prefill_prof[8], static_cast<unsigned long long>(clock64() - soft_t0));
            atomicAdd(&g_prefill_prof[9], static_cast<unsigned long long>(g));
        }
#endif
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

#ifdef CC_PREFILL_PROF
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
    cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem);
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long items = static_cast<long long>(p.seqs) * ((p.max_t + kTileQ - 1) / kTileQ) * p.heads;
    const unsigned grid = static_cast<unsigned>(items < sms ? items : sms);   // one persistent CTA per SM
    prefill_kernel<<<grid, kThreadsPrefill, kPrefillSmem, stream>>>(p);
}

}  // namespace cc
