// Tensor-core candidate pass of the exact kNN: a persistent, warp-specialised sm_100a
// kernel.  Per work item (one tile of 128 queries x one contiguous range of database
// tiles) it keeps the bf16 query tile resident in shared memory, streams bf16 database
// tiles of 256 rows through a TMA ring, multiplies them with tcgen05.mma into two
// 128 x 256 fp32 accumulators in tensor memory (so the next tile's MMAs overlap the
// current tile's epilogue).  The operand planes carry 16 extra columns (ones on the query
// side, -||x||^2/2 split into three bf16 terms on the database side), so one extra K=16 MMA
// step makes every accumulator element the score
//     s = <q, x> - ||x||^2 / 2          (larger = closer)
// and the epilogue only compares: scores above a row's threshold feed that query's
// candidate pool in shared memory.  Nothing of the 128 x 256 score tile ever reaches global
// memory; per query and range only the two warpgroups' pools (32 entries each, 12 kept at a
// compaction; deeper or global-memory pools in the modes described below) and their final
// thresholds are written, unsorted.
//
// Warp roles (320 threads): warps 0-7 epilogue in two warpgroups (group g takes columns
// 128g..128g+127 of every accumulator; warp w reads TMEM lanes 32(w%4)..32(w%4)+31, one query
// row per thread, and keeps a pool per row), warp 8 TMA producer, warp 9 MMA issuer and TMEM
// owner.
// Every wait is bounded; a wait that gives up raises a CTA-wide abort flag, records where
// it happened in the status words and every role falls through to the common exit.
#include "knn_internal.h"
#include "pool.cuh"
#include "tc_ptx.cuh"
#include <stdlib.h>

namespace fl {

using namespace tc;

constexpr int TC_BM = 128;            // queries per tile (MMA M)
constexpr int TC_BN = 256;            // database rows per tile (MMA N)
constexpr int TC_BK = 64;             // bf16 features per shared-memory chunk (128 bytes)
constexpr int TC_NWG = 2;             // epilogue warpgroups; group g owns columns 128g.. of every tile
constexpr int TC_K1 = 12;             // entries a (query, warpgroup) pool keeps at compaction
constexpr int TC_CAP = 32;            // pool capacity before compaction
constexpr int TC_PSTR = TC_CAP + 1;   // padded pool row stride (bank spread); the extra slot is scratch
constexpr int TC_BIG_K1 = 128;        // large-k mode (16 < k <= 128): pools live in global memory,
constexpr int TC_BIG_CAP = 256;       // directly in the published-pool buffers
constexpr int TC_MID_K1 = 24;         // deep-pool mode: a query has few pools (inverted-file scan: two per
constexpr int TC_MID_CAP = 48;        // probed list), so each must reach further below the k-th neighbour
constexpr int TC_MID_PUB = 64;        // published entries per pool in that mode (padded)
constexpr int TC_THREADS = (4 * TC_NWG + 2) * 32;
constexpr int TC_A_CHUNK = TC_BM * 128;   // bytes of one K-chunk of the query tile
constexpr int TC_A_AUG = TC_BM * 32;      // bytes of the query tile's 16 norm columns
constexpr int TC_B_CHUNK = TC_BN * 128;   // bytes of one K-chunk of a database tile
constexpr int TC_B_AUG = TC_BN * 32;      // bytes of a database tile's 16 norm columns
constexpr int TC_B_STAGE = TC_B_CHUNK + TC_B_AUG;   // ring slot: a K-chunk, plus the norm
                                                    // columns when it is the tile's last chunk
constexpr int TC_MAX_STAGES = 6;
constexpr uint64_t TC_WAIT_DEFAULT_NS = 2000000000ull;   // 2 s per wait unless the launch says otherwise

struct TcSmemPlan {
    int nkc, nstage;
    int off_a, off_b, off_pool_sc, off_pool_id, off_hbuf, off_bar, bytes;
};

// nabuf: query-tile buffers (2: the next item's tile is loaded while the current item is scored).
static TcSmemPlan tc_smem_plan(int d_pad, int smem_limit, int pool_stride = TC_PSTR, int slot_bytes = TC_B_STAGE, int nabuf = 1) {
    TcSmemPlan s{};
    s.nkc = d_pad / TC_BK;
    int cur = 0;
    s.off_a = cur; cur += nabuf * (s.nkc * TC_A_CHUNK + TC_A_AUG);
    const int pool = TC_NWG * TC_BM * pool_stride * 4;   // 0: no pools in shared memory
    const int fixed = cur + 2 * pool + 256 + 1024 /* alignment slack */;
    int ns = (smem_limit - fixed) / slot_bytes;
    if (ns > TC_MAX_STAGES) ns = TC_MAX_STAGES;
    s.nstage = ns;
    s.off_b = cur; cur += (ns > 0 ? ns : 0) * slot_bytes;
    s.off_pool_sc = cur; cur += pool;
    s.off_pool_id = cur; cur += pool;
    s.off_hbuf = cur;
    s.off_bar = cur; cur += 256;
    s.bytes = cur + 1024;
    return s;
}

// Per-CTA cycle counters of the last launch (debug aid, read by fl_debug_tc_prof_read):
// [0] producer waiting for a free slot, [1] MMA waiting for operands, [2] MMA waiting for a
// free accumulator, [3] epilogue waiting for an accumulator, [4] cycles in the epilogue's
// second pass, [5] column groups revisited there, [6] pool compactions, [7] scores appended
// (warp 0 / lane 0 views), [8] kernel cycles, [9] tiles.
// The counters cost registers in the epilogue warps, so they are compiled in only with -DFL_TC_PROF
// (FLASHLIB_B200_NVCC_FLAGS=-DFL_TC_PROF python -m flashlib_b200._build --force); otherwise
// fl_debug_tc_prof_read returns zeros.
constexpr int TC_PROF_WORDS = 16;
__device__ unsigned long long g_tc_prof[160 * TC_PROF_WORDS];
#ifdef FL_TC_PROF
#define TC_PROF(...) __VA_ARGS__
#else
#define TC_PROF(...)
#endif

struct TcKernelParams {
    int n_qtiles, n_tiles, nsplit, tiles_per_split, nkc, nstage;
    int nabuf;               // query-tile buffers in shared memory (1 or 2)
    int off_b, off_pool_sc, off_pool_id, off_bar;
    int64_t nq_pad;
    float* part_sc; uint32_t* part_id;
    float* tau;
    float* part_tau;
    int* part_cnt;           // large-k mode: entries of every published pool
    const int* nq_dev;       // optional: live query rows, counted on the device by an earlier kernel
    const int* row_query;    // optional: query of every (gathered) query row, -1 for rows without one, and
    float* tau_q;            //   a running threshold per query shared by all rows of that query
    const int* item_t0;      // optional (one range per query tile): first / one-past-last database
    const int* item_t1;      //   tile of query tile `it`, instead of the uniform ranges
    int item_tile_cap;       // > 0: at most this many tiles of every table range (seeding over item tables)
    const int* item_order;   // optional, with item tables: the CTAs walk item item_order[i] in place of item i
                             //   (longest ranges first, so that the round-robin deal comes out even)
    float* seed_cls;         // seeding output: [nq_pad][TC_NWG][16] class maxima
    float2* gpool;           // global-pool mode: (score, row) pairs, [nq_pad][nsplit][TC_NWG][TC_GP_CAP]
    float* asg_sc; uint32_t* asg_id;   // assignment mode outputs: [rows][TC_NWG] x (best, second) / centroid
    int32_t* status;
    uint32_t wait_hint_ns;   // suspend-time hint of the barrier waits
    uint64_t wait_ns;        // limit of the MMA lane's barrier waits; a wait that runs out aborts the CTA
                             // (FL_ETIMEOUT).  The producer and the epilogue warps, which can only starve
                             // after the MMA lane has, wait twice as long, so the status names the wait
                             // nearest to the cause.
    int tile_stride;         // database tile actually read for loop index t is t * tile_stride (1 outside seeding)
    int dbg_flags;           // timing experiments (results invalid): 1 skip pass 2, 2 skip the
                             // reductions of pass 1, 4 skip the tensor-memory loads too, 8 skip the
                             // norm-column MMA step, 16 issue no MMA at all (operand streaming only);
                             // 32 the producer leaves out its fourth operand load, so the MMA lane's
                             // wait for it runs out (host-visible test of the bounded-wait exit)
    float* dbg_scores;       // optional: [128][n_tiles*256] scores of query tile 0
    int64_t dbg_ld;
};

// Database tiles [t0, t1) of work item `it`: a uniform range of the whole plane, or the item's own
// range from the tables (cut to item_tile_cap tiles when that is set).
__device__ __forceinline__ void tc_item_range(const TcKernelParams& p, int it, int split, int& t0, int& t1) {
    if (p.item_t0 != nullptr) {
        t0 = __ldg(p.item_t0 + it);
        t1 = __ldg(p.item_t1 + it);
        if (p.item_tile_cap > 0) t1 = min(t1, t0 + p.item_tile_cap);
    } else {
        t0 = split * p.tiles_per_split;
        t1 = min(p.n_tiles, t0 + p.tiles_per_split);
    }
}

__device__ __forceinline__ void tc_report_timeout(int32_t* status, int role, int which) {
    if (status) {
        if (atomicCAS(status + FL_STATUS_ERROR, 0, FL_ETIMEOUT) == 0) status[FL_STATUS_WHERE] = (role << 16) | which;
    }
}

// Compacts the pools of the rows named in `need` (one bit per lane = row of this warp).
// Kept out of line: compaction is rare and the sorting network is large.
// `stride` = elements between the pools of consecutive rows.
template <int CAP, int K1>
static __device__ __noinline__ float2 tc_compact_rows(unsigned need, float* warp_sc, uint32_t* warp_id, int64_t stride,
                                                      int cnt, float tau) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    while (need) {
        const int src = __ffs(need) - 1;
        need &= need - 1;
        const int n = __shfl_sync(FULL_MASK, cnt, src);
        const float thr = warp_pool_compact<(CAP + 31) / 32>(warp_sc + src * stride, warp_id + src * stride, n, K1);
        if (lane == src) { cnt = min(n, K1); tau = fmaxf(tau, thr); }
    }
    return make_float2(__int_as_float(cnt), tau);
}

// Same for pools stored as (score, row) pairs of 8 bytes (the deep-pool mode), `stride` pairs apart.
template <int CAP, int K1>
static __device__ __noinline__ float2 tc_compact_rows_pairs(unsigned need, float2* warp_pool, int stride, int cnt, float tau) {
    constexpr int NPL = (CAP + 31) / 32;
    const int lane = threadIdx.x & 31;
    __syncwarp();
    while (need) {
        const int src = __ffs(need) - 1;
        need &= need - 1;
        const int n = __shfl_sync(FULL_MASK, cnt, src);
        float2* pool = warp_pool + src * stride;
        float key[NPL];
        uint32_t id[NPL];
#pragma unroll
        for (int r = 0; r < NPL; ++r) {
            const int e = (r << 5) | lane;
            const float2 v = e < n ? pool[e] : make_float2(neg_inf(), __uint_as_float(INVALID_ID));
            key[r] = v.x;
            id[r] = __float_as_uint(v.y);
        }
        warp_sort_desc<NPL, false>(key, id);
        float thr = neg_inf();
#pragma unroll
        for (int r = 0; r < NPL; ++r) {
            const int e = (r << 5) | lane;
            if (e < K1) pool[e] = make_float2(key[r], __uint_as_float(id[r]));
            if (((K1 - 1) >> 5) == r) thr = __shfl_sync(FULL_MASK, key[r], (K1 - 1) & 31);
        }
        __syncwarp();
        if (lane == src) { cnt = min(n, K1); tau = fmaxf(tau, n >= K1 ? thr : neg_inf()); }
    }
    return make_float2(__int_as_float(cnt), tau);
}

// MODE 1 (TC_MODE_SEED) turns the kernel into the threshold-seeding pass: it scans a strided sample of
// the database tiles and, instead of pools, keeps 16 running maxima per query row over
// disjoint column classes; their minimum is a score that 16 distinct rows reach, i.e. a valid
// starting threshold that spares the main pass most of its cold-start appends.
//
// MODE 2 (TC_MODE_ASSIGN) is the k-means assignment: the "database" is the (small) centroid
// set, every row only needs its best centroid, so each thread keeps the best and second-best
// score of its row in registers (the column index rides in the low 7 mantissa bits of the
// score) and no pool is touched.
//
// MODE 3 (TC_MODE_KNN_BIG) is MODE 0 for 16 < k <= 128: pools of 256 entries (128 kept) that do not
// fit shared memory; they live in global memory, in place in the published-pool buffers (appends
// are predicated stores, compaction reads them back through the L2), and each pool's entry
// count is published with it.
//
// MODE 4 (TC_MODE_KNN_MID) is MODE 0 with deeper pools in shared memory (24 of 48 kept, 64
// published): for callers whose queries have only a few pools each (a small database scored as
// one range; the inverted-file scan, where a query row meets only the tiles of one list).  There a
// row has a candidate in most tiles, which the screen-then-revisit epilogue of MODE 0 handles
// badly (every group of columns ends up revisited, one latency-bound step each); this mode
// compares every score against the row's threshold and appends the passing ones with predicated
// 8-byte stores -- three instructions per score, no branch, no second pass.
//
// MODE 5 (TC_MODE_KNN_GPOOL) is MODE 4 with the pools in global memory, as (score, row) pairs in
// the buffer the finalisation reads (64 slots per (query row, warpgroup), 24 kept at a
// compaction, entry counts published): no pool takes shared memory, so the TMA ring is four
// slots deep -- two whole tiles, where MODE 4 has room for one and stalls on every load -- and
// nothing is copied out when an item ends.  The inverted-file scan runs in this mode.
//
// MODE 6 (TC_MODE_KNN_GS) is MODE 0 with its small pools (32 slots, 12 kept) in global memory, in
// place in the published-pool buffers like MODE 3: appends are rare in MODE 0 (about a hundred per
// query row and launch), so their stores and the compactions' reads can afford the L2, and the
// 67 KB of shared memory the pools took go to the TMA ring (four slots instead of three at 128
// features, four instead of two at 256).
constexpr int TC_MODE_KNN = 0, TC_MODE_SEED = 1, TC_MODE_ASSIGN = 2, TC_MODE_KNN_BIG = 3, TC_MODE_KNN_MID = 4,
              TC_MODE_KNN_GPOOL = 5, TC_MODE_KNN_GS = 6;
constexpr int TC_GP_K1 = 24, TC_GP_CAP = 64;
//
// PAIR: two CTAs of a cluster work as one (tcgen05 cta_group::2).  CTA r of the pair owns query
// tile 2 i + r of pair-item i, loads its own query tile and rows 128 r .. 128 r + 127 of every
// 256-row database tile (half the L2 and shared-memory traffic per CTA), the leader (r = 0)
// issues one M = 256 MMA per step that reads both halves and writes each CTA's 128 x 256
// accumulator into that CTA's tensor memory; both CTAs run the epilogue on their own rows.
// Operand and accumulator barriers live in the leader; "slot free", "query tile free" and
// "accumulator full" are committed to both CTAs.
template <bool DBG, int MODE, bool PAIR = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
knn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_q_aug,
              const __grid_constant__ CUtensorMap map_db, const __grid_constant__ CUtensorMap map_db_aug,
              const TcKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    // the swizzled operand tiles need 1024-byte aligned shared memory
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t a_addr = sbase;                                // nkc chunks of 16 KB
    const uint32_t a_aug_addr = sbase + p.nkc * TC_A_CHUNK;       // 4 KB: the query tile's norm columns
    const uint32_t b_addr = sbase + p.off_b;                      // nstage slots of 40 KB
    float* pool_sc = reinterpret_cast<float*>(smem + p.off_pool_sc);
    uint32_t* pool_id = reinterpret_cast<uint32_t*>(smem + p.off_pool_id);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);
    // barrier slots: [0, 6) full, [6, 12) empty, 12 a_full, 13 a_empty, 14-15 tmem_full, 16-17 tmem_empty,
    // 18 a_full / 19 a_empty of the second query-tile buffer
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * i; };
    constexpr int B_FULL = 0, B_EMPTY = 6, B_AFULL = 12, B_AEMPTY = 13, B_TFULL = 14, B_TEMPTY = 16;
    // Query-tile buffer of item number i of this CTA: buffer i % nabuf, used for the (i / nabuf)-th time.
    const uint32_t a_stride = (uint32_t)(p.nkc * TC_A_CHUNK + TC_A_AUG);
    const bool two_a = !PAIR && p.nabuf == 2;
    auto a_buf = [&](uint32_t item) { return two_a ? (item & 1u) : 0u; };
    auto a_phase = [&](uint32_t item) { return two_a ? ((item >> 1) & 1u) : (item & 1u); };
    auto a_full_bar = [&](uint32_t buf) { return BAR(buf ? 18 : B_AFULL); };
    auto a_empty_bar = [&](uint32_t buf) { return BAR(buf ? 19 : B_AEMPTY); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 20);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    // a timing experiment leaves work out: whoever reads the status words learns that the
    // neighbours of this launch are not to be used
    if (DBG && (p.dbg_flags & 31) && blockIdx.x == 0 && tid == 0 && p.status != nullptr) {
        if (atomicCAS(p.status + FL_STATUS_ERROR, 0, FL_EUNSUPPORTED) == 0) p.status[FL_STATUS_WHERE] = 0xDB600 | p.dbg_flags;
    }
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = cta_rank == 0;
    // geometry of one ring slot and of the work split
    constexpr int B_ROWS = PAIR ? TC_BN / 2 : TC_BN;          // database rows this CTA loads per tile
    constexpr int SLOT_CHUNK = B_ROWS * 128, SLOT_BYTES = B_ROWS * 128 + B_ROWS * 32;
    constexpr uint32_t OPERAND_CTAS = PAIR ? 2u : 1u;         // CTAs whose loads one operand barrier counts

    if (tid == 0) {
        for (int i = 0; i < TC_MAX_STAGES; ++i) { mbar_init(BAR(B_FULL + i), 1); mbar_init(BAR(B_EMPTY + i), 1); }
        mbar_init(BAR(B_AFULL), 1);
        mbar_init(BAR(B_AEMPTY), 1);
        mbar_init(BAR(18), 1);
        mbar_init(BAR(19), 1);
        for (int i = 0; i < 2; ++i) { mbar_init(BAR(B_TFULL + i), 1); mbar_init(BAR(B_TEMPTY + i), 4 * TC_NWG * OPERAND_CTAS); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    constexpr int W_PRODUCER = 4 * TC_NWG, W_MMA = 4 * TC_NWG + 1;
    if (warp == W_PRODUCER && lane == 0) {
        prefetch_tensormap(&map_q); prefetch_tensormap(&map_q_aug);
        prefetch_tensormap(&map_db); prefetch_tensormap(&map_db_aug);
    }
    if (warp == W_MMA) {
        if (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), 512); tmem_relinquish_pair(); }
        else { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) cluster_sync_all();      // the peer's barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // query tiles: fixed by the launch, or (nq_dev) cut down to the live rows counted on the device
    int n_qtiles = p.n_qtiles;
    if (p.nq_dev != nullptr) {
        const int live = (__ldcg(p.nq_dev) + TC_BM - 1) / TC_BM;
        n_qtiles = live < n_qtiles ? live : n_qtiles;
    }
    // item = (range, query tile) or, for CTA pairs, (range, pair of query tiles); a pair walks the
    // items together
    const int n_units = PAIR ? n_qtiles / 2 : n_qtiles;
    const int n_items = n_units * p.nsplit;
    const int it_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int it_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int d_pad = p.nkc * TC_BK;

    if (warp == W_PRODUCER) {
        // ------------------------------ TMA producer --------------------------------------
        if (lane == 0) {
            uint32_t fill = 0;     // database chunks issued so far
            uint32_t item_no = 0;
            bool ok = true;
            TC_PROF(long long prof_a = 0;)
            // loads of a pair are credited to the leader's barrier, which expects both CTAs' bytes
            auto load = [&](uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
                if (PAIR) tma_load_2d_pair(dst, map, c0, c1, bar); else tma_load_2d(dst, map, c0, c1, bar);
            };
            for (int it = it_first; it < n_items && ok; it += it_step, ++item_no) {
                const int itp = p.item_order != nullptr ? __ldg(p.item_order + it) : it;
                const int split = itp / n_units, unit = itp - split * n_units;
                const int qt = PAIR ? 2 * unit + (int)cta_rank : unit;
                int t0, t1;
                tc_item_range(p, itp, split, t0, t1);
                const uint32_t ab = a_buf(item_no), a_off = ab * a_stride;
                if (!mbar_wait(a_empty_bar(ab), a_phase(item_no) ^ 1u, abort_flag, 2 * p.wait_ns, p.wait_hint_ns)) {
                    tc_report_timeout(p.status, 4, ab ? 19 : B_AEMPTY); ok = false; break;
                }
                if (leader) mbar_expect_tx(a_full_bar(ab), (p.nkc * TC_A_CHUNK + TC_A_AUG) * OPERAND_CTAS);
                for (int kc = 0; kc < p.nkc; ++kc)
                    load(a_addr + a_off + kc * TC_A_CHUNK, &map_q, kc * TC_BK, qt * TC_BM, a_full_bar(ab));
                load(a_aug_addr + a_off, &map_q_aug, d_pad, qt * TC_BM, a_full_bar(ab));
                const int nt = t1 - t0;
                const int rot = (int)(((int64_t)unit * nt) / n_units);
                for (int i = 0; i < nt && ok; ++i) {
                    // Query tiles walk their range from different starting tiles, so the CTAs of a
                    // wave do not all ask the L2 for the same lines at the same moment.
                    const int t = t0 + (i + rot < nt ? i + rot : i + rot - nt);
                    for (int kc = 0; kc < p.nkc; ++kc, ++fill) {
                        const int s = fill % p.nstage;
                        const uint32_t ph = (fill / p.nstage) & 1;
                        TC_PROF(const long long c0 = clock64();)
                        if (!mbar_wait(BAR(B_EMPTY + s), ph ^ 1, abort_flag, 2 * p.wait_ns, p.wait_hint_ns)) {
                            tc_report_timeout(p.status, 4, B_EMPTY + s); ok = false; break;
                        }
                        TC_PROF(prof_a += clock64() - c0;)
                        const bool last = (kc == p.nkc - 1);
                        const int row0 = t * p.tile_stride * TC_BN + (int)cta_rank * B_ROWS;
                        if (DBG && (p.dbg_flags & 32) && fill == 3) continue;   // this slot never fills
                        if (leader) mbar_expect_tx(BAR(B_FULL + s), (last ? SLOT_BYTES : SLOT_CHUNK) * OPERAND_CTAS);
                        load(b_addr + s * SLOT_BYTES, &map_db, kc * TC_BK, row0, BAR(B_FULL + s));
                        if (last) load(b_addr + s * SLOT_BYTES + SLOT_CHUNK, &map_db_aug, d_pad, row0, BAR(B_FULL + s));
                    }
                }
            }
            TC_PROF(if (blockIdx.x < 160) g_tc_prof[blockIdx.x * TC_PROF_WORDS + 0] = prof_a;)
            if (!ok) {
                // give copies already in flight a bounded time to land before the CTA exits
                const uint64_t t_start = globaltimer_ns();
                while (globaltimer_ns() - t_start < 2000000ull) { }
            }
        }
    } else if (warp == W_MMA) {
        // ------------------------------ MMA issuer -----------------------------------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(PAIR ? 2 * TC_BM : TC_BM, TC_BN);
            auto mma = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t acc) {
                if (DBG && (p.dbg_flags & 16)) return;     // timing experiment: operand streaming only
                if (PAIR) umma_bf16_pair(d, a, b, idesc, acc); else umma_bf16(d, a, b, idesc, acc);
            };
            auto commit = [&](uint32_t bar) { if (PAIR) umma_commit_pair(bar); else umma_commit(bar); };
            uint32_t use = 0;      // database chunks consumed so far
            uint32_t tile_no = 0;  // tiles issued so far (accumulator ring position)
            uint32_t item_no = 0;
            bool ok = true;
            TC_PROF(long long prof_full = 0; long long prof_tempty = 0;)
            for (int it = it_first; it < n_items && ok; it += it_step, ++item_no) {
                const int itp = p.item_order != nullptr ? __ldg(p.item_order + it) : it;
                const int split = itp / n_units;
                int t0, t1;
                tc_item_range(p, itp, split, t0, t1);
                const uint32_t ab = a_buf(item_no), a_off = ab * a_stride;
                if (!mbar_wait(a_full_bar(ab), a_phase(item_no), abort_flag, p.wait_ns, p.wait_hint_ns)) {
                    tc_report_timeout(p.status, 5, ab ? 18 : B_AFULL); ok = false; break;
                }
                for (int t = t0; t < t1 && ok; ++t, ++tile_no) {
                    const int b = tile_no & 1;
                    TC_PROF(const long long c0 = clock64();)
                    if (!mbar_wait(BAR(B_TEMPTY + b), ((tile_no >> 1) & 1) ^ 1, abort_flag, p.wait_ns, p.wait_hint_ns)) {
                        tc_report_timeout(p.status, 5, B_TEMPTY + b); ok = false; break;
                    }
                    TC_PROF(prof_tempty += clock64() - c0;)
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + b * TC_BN;
                    for (int kc = 0; kc < p.nkc; ++kc, ++use) {
                        const int s = use % p.nstage;
                        const uint32_t ph = (use / p.nstage) & 1;
                        TC_PROF(const long long c1 = clock64();)
                        if (!mbar_wait(BAR(B_FULL + s), ph, abort_flag, p.wait_ns, p.wait_hint_ns)) {
                            tc_report_timeout(p.status, 5, B_FULL + s); ok = false; break;
                        }
                        TC_PROF(prof_full += clock64() - c1;)
                        tc_fence_after_sync();
                        const uint64_t da = umma_desc(a_addr + a_off + kc * TC_A_CHUNK);
                        const uint64_t db = umma_desc(b_addr + s * SLOT_BYTES);
#pragma unroll
                        for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                            // +32 bytes per 16-feature step inside the 128-byte swizzled row
                            mma(d_tmem, da + 2 * k4, db + 2 * k4, (kc | k4) != 0 ? 1u : 0u);
                        }
                        if (kc == p.nkc - 1 && !(DBG && (p.dbg_flags & 8))) {
                            // norm columns: ones x split(-||x||^2/2), 32-byte rows, 32-byte swizzle
                            mma(d_tmem, umma_desc_sw32(a_aug_addr + a_off), umma_desc_sw32(b_addr + s * SLOT_BYTES + SLOT_CHUNK), 1u);
                        }
                        commit(BAR(B_EMPTY + s));   // slot reusable once these MMAs retire
                    }
                    if (ok) commit(BAR(B_TFULL + b));
                }
                if (ok) commit(a_empty_bar(ab));     // query tile buffer reusable
            }
            TC_PROF(if (blockIdx.x < 160) {
                g_tc_prof[blockIdx.x * TC_PROF_WORDS + 1] = prof_full;
                g_tc_prof[blockIdx.x * TC_PROF_WORDS + 2] = prof_tempty;
            })
        }
    } else {
        // ------------------------------ epilogue warps --------------------------------------
        // warp = 4 * warpgroup + TMEM lane quarter; warpgroup g reads columns 128g .. 128g+127 of
        // every accumulator and keeps its own pool per query row.
        const int wg = warp >> 2, quarter = warp & 3;
        constexpr bool BIG = (MODE == TC_MODE_KNN_BIG);
        constexpr bool GS = (MODE == TC_MODE_KNN_GS);
        constexpr bool GLOB = BIG || GS;                 // pools addressed in global memory
        constexpr bool MID = (MODE == TC_MODE_KNN_MID);
        constexpr bool GP = (MODE == TC_MODE_KNN_GPOOL);
        constexpr int CAP = BIG ? TC_BIG_CAP : MID ? TC_MID_CAP : GP ? TC_GP_CAP : TC_CAP;
        constexpr int K1 = BIG ? TC_BIG_K1 : MID ? TC_MID_K1 : GP ? TC_GP_K1 : TC_K1;
        constexpr int PSTR = CAP + 1;                    // shared pools: padded stride, slot CAP is scratch
        constexpr int PUB = BIG ? TC_BIG_CAP : MID ? TC_MID_PUB : TC_CAP;   // published entries per pool
        // pool of lane 0's row and distance (elements) between the pools of consecutive rows
        float* warp_sc = pool_sc + warp * 32 * PSTR;
        uint32_t* warp_id = pool_id + warp * 32 * PSTR;
        int64_t pstride = PSTR;
        float* my_sc = warp_sc + lane * PSTR;
        uint32_t* my_id = warp_id + lane * PSTR;
        const uint32_t lane_taddr = tmem_base + (uint32_t(quarter * 32) << 16);
        uint32_t tile_no = 0;
        bool ok = true;
        TC_PROF(long long prof_tfull = 0; long long prof_rare = 0; long long prof_cc = 0;
                unsigned prof_groups = 0; unsigned prof_compact = 0; unsigned prof_append = 0;
                const long long prof_t0 = clock64();)
        // hands accumulator b back to the MMA lane (of the leader, for a pair)
        auto release_acc = [&](int b) {
            if (PAIR) mbar_arrive_cluster(BAR(B_TEMPTY + b), 0u); else mbar_arrive(BAR(B_TEMPTY + b));
        };
        for (int it = it_first; it < n_items && ok; it += it_step) {
            const int itp = p.item_order != nullptr ? __ldg(p.item_order + it) : it;
            const int split = itp / n_units, unit = itp - split * n_units;
            const int qt = PAIR ? 2 * unit + (int)cta_rank : unit;
            int t0, t1;
            tc_item_range(p, itp, split, t0, t1);
            const int64_t qrow = (int64_t)qt * TC_BM + quarter * 32 + lane;
            float tau_in = __ldcg(p.tau + qrow);
            int qidx = -1;
            if (p.row_query != nullptr) {
                // rows that belong to the same query (one per probed list) pass their thresholds on:
                // a score below what 24 rows of another probed list reach cannot be among the k best
                qidx = __ldg(p.row_query + qrow);
                if (qidx >= 0) tau_in = fmaxf(tau_in, __ldcg(p.tau_q + qidx));
            }
            if (GLOB) {
                pstride = (int64_t)p.nsplit * TC_NWG * CAP;
                const int64_t o = (((int64_t)(qt * TC_BM + quarter * 32) * p.nsplit + split) * TC_NWG + wg) * CAP;
                warp_sc = p.part_sc + o;
                warp_id = p.part_id + o;
                my_sc = warp_sc + lane * pstride;
                my_id = warp_id + lane * pstride;
            }
            float tau = tau_in;
            int cnt = 0;
            float cls[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) cls[c] = neg_inf();
            float b1 = neg_inf(), b2 = neg_inf();   // assignment mode: best / second-best packed score
            int tbest = 0;                           // tile that produced b1
            const int nt = t1 - t0;
            const int rot = (int)(((int64_t)unit * nt) / n_units);
            for (int i = 0; i < nt; ++i, ++tile_no) {
                const int t = t0 + (i + rot < nt ? i + rot : i + rot - nt);
                const int b = tile_no & 1;
                TC_PROF(const long long c0 = clock64();)
                if (!__all_sync(FULL_MASK, mbar_wait(BAR(B_TFULL + b), (tile_no >> 1) & 1, abort_flag, 2 * p.wait_ns, p.wait_hint_ns))) {
                    if (lane == 0) tc_report_timeout(p.status, warp, B_TFULL + b);
                    ok = false;
                    break;
                }
                TC_PROF(prof_tfull += clock64() - c0;)
                tc_fence_after_sync();
                // this warpgroup's half of the accumulator columns / of the tile's database rows
                const uint32_t tile_taddr = lane_taddr + b * TC_BN + wg * (TC_BN / TC_NWG);
                const uint32_t row_base = (uint32_t)t * TC_BN + wg * (TC_BN / TC_NWG);

                // Pass 1, branch free: stream the 256 scores of this thread's query row through
                // registers, 64 columns per wait, and note which groups of 8 columns hold a score
                // above the row's threshold (bit g of `hits` = columns 8g .. 8g+7).
                // tcgen05.wait::ld waits for every load in flight, so while one batch of 64
                // columns is reduced the next one is already on its way.
                uint32_t va[32], vb[32], vc[32], vd[32];
                constexpr bool SEED = (MODE == TC_MODE_SEED);
                if (MODE == TC_MODE_ASSIGN) {
                    const float b1_before = b1;
                    // column index into the low 7 mantissa bits: one three-input logic instruction per
                    // score, (v & mask) | column, with the mask held in a register
                    uint32_t idx_mask;
                    asm volatile("mov.u32 %0, 0xFFFFFF80;" : "=r"(idx_mask));
                    auto pack = [&](uint32_t v, uint32_t col) {
                        uint32_t r;
                        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(v), "r"(idx_mask), "r"(col));
                        return r;
                    };
                    auto top2 = [&](uint32_t (&v)[32], int slice) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float x = __uint_as_float(pack(v[j], (uint32_t)(slice * 32 + j)));
                            const float y = __uint_as_float(pack(v[j + 1], (uint32_t)(slice * 32 + j + 1)));
                            const float hi = fmaxf(x, y), lo = fminf(x, y);
                            b2 = fmax3(b2, lo, fminf(b1, hi));
                            b1 = fmaxf(b1, hi);
                        }
                    };
                    tmem_ld_32x32b_x32(tile_taddr, va);
                    tmem_ld_32x32b_x32(tile_taddr + 32, vb);
                    tmem_ld_wait();
                    reg_fence32(va);
                    reg_fence32(vb);
                    tmem_ld_32x32b_x32(tile_taddr + 64, vc);
                    tmem_ld_32x32b_x32(tile_taddr + 96, vd);
                    top2(va, 0);
                    top2(vb, 1);
                    tmem_ld_wait();
                    reg_fence32(vc);
                    reg_fence32(vd);
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(b);
                    top2(vc, 2);
                    top2(vd, 3);
                    if (b1 != b1_before) tbest = t;
                    continue;
                }
                if (SEED) {
                    auto fold = [&](uint32_t (&v)[32]) {
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            cls[c] = fmax3(cls[c], __uint_as_float(v[c]), __uint_as_float(v[c + 16]));
                    };
                    tmem_ld_32x32b_x32(tile_taddr, va);
                    tmem_ld_32x32b_x32(tile_taddr + 32, vb);
                    tmem_ld_wait();
                    reg_fence32(va);
                    reg_fence32(vb);
                    tmem_ld_32x32b_x32(tile_taddr + 64, vc);
                    tmem_ld_32x32b_x32(tile_taddr + 96, vd);
                    fold(va);
                    fold(vb);
                    tmem_ld_wait();
                    reg_fence32(vc);
                    reg_fence32(vd);
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(b);
                    fold(vc);
                    fold(vd);
                    continue;
                }
                if (GP) {
                    // this row's pool in global memory and the address of its next free slot
                    float2* warp_pool = p.gpool + (((int64_t)(qt * TC_BM + quarter * 32) * p.nsplit + split) * TC_NWG + wg) * CAP;
                    const int gstride = p.nsplit * TC_NWG * CAP;      // pairs between the pools of consecutive rows
                    const uint64_t my_addr = reinterpret_cast<uint64_t>(warp_pool + (int64_t)lane * gstride);
                    uint64_t waddr = my_addr + 8ull * (uint64_t)cnt;
                    const uint64_t lim = my_addr + 8ull * (uint64_t)(CAP - 8);
                    tmem_ld_32x32b_x32(tile_taddr, va);
                    tmem_ld_32x32b_x32(tile_taddr + 32, vb);
                    tmem_ld_32x32b_x32(tile_taddr + 64, vc);
                    tmem_ld_32x32b_x32(tile_taddr + 96, vd);
                    tmem_ld_wait();
                    reg_fence32(va);
                    reg_fence32(vb);
                    reg_fence32(vc);
                    reg_fence32(vd);
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(b);
                    auto dense = [&](uint32_t (&v)[32], int slice) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (__any_sync(FULL_MASK, waddr > lim)) {
                                cnt = (int)((waddr - my_addr) >> 3);
                                const unsigned need = __ballot_sync(FULL_MASK, cnt > CAP - 8);
                                TC_PROF(prof_compact += __popc(need);)
                                const float2 cr = tc_compact_rows_pairs<CAP, K1>(need, warp_pool, gstride, cnt, tau);
                                cnt = __float_as_int(cr.x);
                                tau = cr.y;
                                waddr = my_addr + 8ull * (uint64_t)cnt;
                            }
                            // the 8 comparisons first (independent), then the predicated stores: only
                            // the address increments form a chain
                            const uint32_t col0 = row_base + slice * 32 + g * 8;
                            const uint32_t* x = v + g * 8;
                            asm volatile(
                                "{\n\t.reg .pred p0, p1, p2, p3, p4, p5, p6, p7;\n\t.reg .b32 c;\n\t"
                                "setp.gt.f32 p0, %3, %1;\n\tsetp.gt.f32 p1, %4, %1;\n\tsetp.gt.f32 p2, %5, %1;\n\tsetp.gt.f32 p3, %6, %1;\n\t"
                                "setp.gt.f32 p4, %7, %1;\n\tsetp.gt.f32 p5, %8, %1;\n\tsetp.gt.f32 p6, %9, %1;\n\tsetp.gt.f32 p7, %10, %1;\n\t"
                                "@p0 st.global.v2.b32 [%0], {%11, %2};\n\t@p0 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 1;\n\t"
                                "@p1 st.global.v2.b32 [%0], {%12, c};\n\t@p1 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 2;\n\t"
                                "@p2 st.global.v2.b32 [%0], {%13, c};\n\t@p2 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 3;\n\t"
                                "@p3 st.global.v2.b32 [%0], {%14, c};\n\t@p3 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 4;\n\t"
                                "@p4 st.global.v2.b32 [%0], {%15, c};\n\t@p4 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 5;\n\t"
                                "@p5 st.global.v2.b32 [%0], {%16, c};\n\t@p5 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 6;\n\t"
                                "@p6 st.global.v2.b32 [%0], {%17, c};\n\t@p6 add.u64 %0, %0, 8;\n\tadd.u32 c, %2, 7;\n\t"
                                "@p7 st.global.v2.b32 [%0], {%18, c};\n\t@p7 add.u64 %0, %0, 8;\n\t}"
                                : "+l"(waddr)
                                : "f"(tau), "r"(col0),
                                  "f"(__uint_as_float(x[0])), "f"(__uint_as_float(x[1])), "f"(__uint_as_float(x[2])),
                                  "f"(__uint_as_float(x[3])), "f"(__uint_as_float(x[4])), "f"(__uint_as_float(x[5])),
                                  "f"(__uint_as_float(x[6])), "f"(__uint_as_float(x[7])),
                                  "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(x[4]), "r"(x[5]), "r"(x[6]), "r"(x[7])
                                : "memory");
                        }
                    };
                    dense(va, 0);
                    dense(vb, 1);
                    dense(vc, 2);
                    dense(vd, 3);
                    TC_PROF(prof_append += (int)((waddr - my_addr) >> 3) - cnt;)
                    cnt = (int)((waddr - my_addr) >> 3);
                    continue;
                }
                if (MID) {
                    // pools of this mode hold (score, row) pairs; `waddr` is the shared-memory address
                    // of this row's next free slot
                    float2* warp_pool = reinterpret_cast<float2*>(pool_sc) + warp * 32 * PSTR;
                    const uint32_t my_addr = smem_u32(warp_pool + lane * PSTR);
                    uint32_t waddr = my_addr + 8u * (uint32_t)cnt;
                    const uint32_t lim = my_addr + 8u * (uint32_t)(CAP - 8);
                    tmem_ld_32x32b_x32(tile_taddr, va);
                    tmem_ld_32x32b_x32(tile_taddr + 32, vb);
                    tmem_ld_32x32b_x32(tile_taddr + 64, vc);
                    tmem_ld_32x32b_x32(tile_taddr + 96, vd);
                    tmem_ld_wait();
                    reg_fence32(va);
                    reg_fence32(vb);
                    reg_fence32(vc);
                    reg_fence32(vd);
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(b);
                    auto dense = [&](uint32_t (&v)[32], int slice) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            // every lane's pool has room for the 8 scores of the group
                            if (__any_sync(FULL_MASK, waddr > lim)) {
                                cnt = (int)((waddr - my_addr) >> 3);
                                const unsigned need = __ballot_sync(FULL_MASK, cnt > CAP - 8);
                                TC_PROF(prof_compact += __popc(need);)
                                const float2 cr = tc_compact_rows_pairs<CAP, K1>(need, warp_pool, PSTR, cnt, tau);
                                cnt = __float_as_int(cr.x);
                                tau = cr.y;
                                waddr = my_addr + 8u * (uint32_t)cnt;
                            }
                            const uint32_t col0 = row_base + slice * 32 + g * 8;
                            const uint32_t* x = v + g * 8;
                            asm volatile(
                                "{\n\t.reg .pred p0, p1, p2, p3, p4, p5, p6, p7;\n\t.reg .b32 c;\n\t"
                                "setp.gt.f32 p0, %3, %1;\n\tsetp.gt.f32 p1, %4, %1;\n\tsetp.gt.f32 p2, %5, %1;\n\tsetp.gt.f32 p3, %6, %1;\n\t"
                                "setp.gt.f32 p4, %7, %1;\n\tsetp.gt.f32 p5, %8, %1;\n\tsetp.gt.f32 p6, %9, %1;\n\tsetp.gt.f32 p7, %10, %1;\n\t"
                                "@p0 st.shared.v2.b32 [%0], {%11, %2};\n\t@p0 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 1;\n\t"
                                "@p1 st.shared.v2.b32 [%0], {%12, c};\n\t@p1 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 2;\n\t"
                                "@p2 st.shared.v2.b32 [%0], {%13, c};\n\t@p2 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 3;\n\t"
                                "@p3 st.shared.v2.b32 [%0], {%14, c};\n\t@p3 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 4;\n\t"
                                "@p4 st.shared.v2.b32 [%0], {%15, c};\n\t@p4 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 5;\n\t"
                                "@p5 st.shared.v2.b32 [%0], {%16, c};\n\t@p5 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 6;\n\t"
                                "@p6 st.shared.v2.b32 [%0], {%17, c};\n\t@p6 add.u32 %0, %0, 8;\n\tadd.u32 c, %2, 7;\n\t"
                                "@p7 st.shared.v2.b32 [%0], {%18, c};\n\t@p7 add.u32 %0, %0, 8;\n\t}"
                                : "+r"(waddr)
                                : "f"(tau), "r"(col0),
                                  "f"(__uint_as_float(x[0])), "f"(__uint_as_float(x[1])), "f"(__uint_as_float(x[2])),
                                  "f"(__uint_as_float(x[3])), "f"(__uint_as_float(x[4])), "f"(__uint_as_float(x[5])),
                                  "f"(__uint_as_float(x[6])), "f"(__uint_as_float(x[7])),
                                  "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(x[4]), "r"(x[5]), "r"(x[6]), "r"(x[7])
                                : "memory");
                        }
                    };
                    dense(va, 0);
                    dense(vb, 1);
                    dense(vc, 2);
                    dense(vd, 3);
                    TC_PROF(prof_append += ((waddr - my_addr) >> 3) - cnt;)
                    cnt = (int)((waddr - my_addr) >> 3);
                    continue;
                }
                unsigned hits = 0;
                auto scan = [&](uint32_t (&v)[32], int slice) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float x = fmax3(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]),
                                              __uint_as_float(v[g * 8 + 2]));
                        const float y = fmax3(__uint_as_float(v[g * 8 + 3]), __uint_as_float(v[g * 8 + 4]),
                                              __uint_as_float(v[g * 8 + 5]));
                        const float z = fmax3(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]), x);
                        hits |= (fmaxf(y, z) > tau) ? (1u << (slice * 4 + g)) : 0u;
                    }
                    if (DBG) {
                        if (p.dbg_scores != nullptr && qt == 0) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                p.dbg_scores[(int64_t)(quarter * 32 + lane) * p.dbg_ld + row_base + slice * 32 + j] =
                                    __uint_as_float(v[j]);
                        }
                    }
                };
                if (!DBG || !(p.dbg_flags & 4)) {
                    tmem_ld_32x32b_x32(tile_taddr, va);
                    tmem_ld_32x32b_x32(tile_taddr + 32, vb);
                    tmem_ld_wait();
                    reg_fence32(va);
                    reg_fence32(vb);
                    tmem_ld_32x32b_x32(tile_taddr + 64, vc);
                    tmem_ld_32x32b_x32(tile_taddr + 96, vd);
                    scan(va, 0);
                    scan(vb, 1);
                    tmem_ld_wait();
                    reg_fence32(vc);
                    reg_fence32(vd);
                    scan(vc, 2);
                    scan(vd, 3);
                }
                if (DBG && (p.dbg_flags & 1)) hits = 0;

                // Pass 2, rare.  A lane seldom has more than one flagged group in a tile, so the
                // work is split in two: (a) a small loop copies every flagged group from tensor
                // memory and each flagged lane keeps the 8 scores of its first flagged group in
                // registers -- after that the accumulator goes back to the MMA warp; (b) all lanes
                // handle their kept group together in one straight-line step (a lone warp pays a
                // few cycles per instruction, so once per tile beats once per group).  Further
                // flagged groups of the same lane ("late") are handled one by one before (b).
                unsigned wm = __reduce_or_sync(FULL_MASK, hits);
                if (wm) {
                    TC_PROF(const long long cr0 = clock64();)
                    float sv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) sv[j] = neg_inf();
                    uint32_t scb = 0;
                    bool have = false;
                    unsigned late = 0;
                    do {
                        // four flagged groups per round trip: a copy from tensor memory takes a few
                        // hundred cycles and tcgen05.wait::ld waits for all copies in flight
                        int gs[4];
                        bool live[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int f = __ffs(wm) - 1;          // -1 when no group is left
                            live[k] = f >= 0;
                            gs[k] = f >= 0 ? f : 0;
                            wm &= wm - 1;                         // 0 stays 0
                        }
                        uint32_t rn[4][8];
#pragma unroll
                        for (int k = 0; k < 4; ++k) tmem_ld_32x32b_x8(tile_taddr + gs[k] * 8, rn[k]);
                        tmem_ld_wait();
#pragma unroll
                        for (int k = 0; k < 4; ++k) reg_fence8(rn[k]);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const bool mine = live[k] && ((hits >> gs[k]) & 1u);
                            const bool take = mine && !have;
#pragma unroll
                            for (int j = 0; j < 8; ++j) sv[j] = take ? __uint_as_float(rn[k][j]) : sv[j];
                            scb = take ? row_base + gs[k] * 8 : scb;
                            late |= (mine && have) ? (1u << gs[k]) : 0u;
                            have = have || mine;
                            TC_PROF(prof_groups += live[k] ? 1 : 0;)
                        }
                    } while (wm);
                    unsigned wl = __reduce_or_sync(FULL_MASK, late);
#pragma unroll 1
                    while (wl) {
                        const int g = __ffs(wl) - 1;
                        wl &= wl - 1;
                        const unsigned need = __ballot_sync(FULL_MASK, cnt > CAP - 8);
                        if (need) {
                            TC_PROF(prof_compact += __popc(need);)
                            const float2 cr = tc_compact_rows<CAP, K1>(need, warp_sc, warp_id, pstride, cnt, tau);
                            cnt = __float_as_int(cr.x);
                            tau = cr.y;
                        }
                        uint32_t r[8];
                        tmem_ld_32x32b_x8(tile_taddr + g * 8, r);
                        tmem_ld_wait();
                        reg_fence8(r);
                        unsigned pm = 0;
#pragma unroll
                        for (int j = 0; j < 8; ++j) pm |= (__uint_as_float(r[j]) > tau) ? (1u << j) : 0u;
                        pm = ((late >> g) & 1u) ? pm : 0u;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const bool pass = (pm >> j) & 1u;
                            const int pos = pass ? cnt + __popc(pm & ((1u << j) - 1u)) : CAP;
                            if (!GLOB || pass) {      // shared pools: slot CAP is the row's scratch slot
                                my_sc[pos] = __uint_as_float(r[j]);
                                my_id[pos] = row_base + g * 8 + j;
                            }
                        }
                        cnt += __popc(pm);
                        TC_PROF(prof_append += __popc(pm);)
                    }
                    // every flagged score is in registers or in a pool: hand the accumulator back
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(b);
                    // (b) all lanes at once
                    const unsigned need = __ballot_sync(FULL_MASK, cnt > CAP - 8);
                    if (need) {
                        TC_PROF(prof_compact += __popc(need); const long long cc0 = clock64();)
                        const float2 cr = tc_compact_rows<CAP, K1>(need, warp_sc, warp_id, pstride, cnt, tau);
                        TC_PROF(prof_cc += clock64() - cc0;)
                        cnt = __float_as_int(cr.x);
                        tau = cr.y;
                    }
                    unsigned pm = 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) pm |= (sv[j] > tau) ? (1u << j) : 0u;   // sv is -inf without a kept group
                    const int np = __popc(pm);
                    if (!__any_sync(FULL_MASK, np > 1)) {
                        // at most one passing score per lane: it is the maximum of the group
                        const float mx = fmaxf(fmax3(sv[0], sv[1], sv[2]), fmax3(fmax3(sv[3], sv[4], sv[5]), sv[6], sv[7]));
                        const int pos = np ? cnt : CAP;
                        if (!GLOB || np) {
                            my_sc[pos] = mx;
                            my_id[pos] = scb + (__ffs(pm) - 1);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const bool pass = (pm >> j) & 1u;
                            const int pos = pass ? cnt + __popc(pm & ((1u << j) - 1u)) : CAP;
                            if (!GLOB || pass) {
                                my_sc[pos] = sv[j];
                                my_id[pos] = scb + j;
                            }
                        }
                    }
                    cnt += np;
                    TC_PROF(prof_append += np;)
                    TC_PROF(prof_rare += clock64() - cr0;)
                } else {
                    // nothing flagged: hand the accumulator back right away
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) release_acc(b);
                }
            }
            if (!ok) break;
            if (MODE == TC_MODE_ASSIGN) {
                const int64_t o = qrow * TC_NWG + wg;
                p.asg_sc[2 * o] = b1;
                p.asg_sc[2 * o + 1] = b2;
                p.asg_id[o] = (uint32_t)tbest * TC_BN + wg * (TC_BN / TC_NWG) + (__float_as_uint(b1) & 0x7Fu);
                continue;
            }
            if (MODE == TC_MODE_SEED) {
                float4* o = reinterpret_cast<float4*>(p.seed_cls + (qrow * TC_NWG + wg) * 16);
#pragma unroll
                for (int c = 0; c < 4; ++c) o[c] = make_float4(cls[4 * c], cls[4 * c + 1], cls[4 * c + 2], cls[4 * c + 3]);
                continue;
            }
            // end of the item: publish every row's pool as it stands (up to TC_CAP entries, the rest
            // padded) and the row's threshold.  The pool is not sorted here: the finalize kernel
            // merges the published entries anyway.
            if (BIG) {
                // the pools already are the published buffers
                p.part_cnt[(qrow * p.nsplit + split) * TC_NWG + wg] = cnt;
                p.part_tau[(qrow * p.nsplit + split) * TC_NWG + wg] = tau;
                if (tau > tau_in) __stcg(p.tau + qrow, tau);
                continue;
            }
            if (GS) {
                // the pools already are the published buffers: pad the unused slots
                for (int e = cnt; e < CAP; ++e) { my_sc[e] = neg_inf(); my_id[e] = INVALID_ID; }
                p.part_tau[(qrow * p.nsplit + split) * TC_NWG + wg] = tau;
                if (tau > tau_in) __stcg(p.tau + qrow, tau);
                continue;
            }
            if (GP) {
                // the pools already are the published buffers
                p.part_cnt[(qrow * p.nsplit + split) * TC_NWG + wg] = cnt;
                p.part_tau[(qrow * p.nsplit + split) * TC_NWG + wg] = tau;
                if (tau > tau_in) __stcg(p.tau + qrow, tau);
                if (qidx >= 0 && tau > tau_in) atomic_max_f32(p.tau_q + qidx, tau);
                continue;
            }
            __syncwarp();
            if (MID) {
                const float2* warp_pool = reinterpret_cast<const float2*>(pool_sc) + warp * 32 * PSTR;
#pragma unroll 1
                for (int src = 0; src < 32; ++src) {
                    const int n = __shfl_sync(FULL_MASK, cnt, src);
                    const float2* row = warp_pool + src * PSTR;
                    const int64_t q = (int64_t)qt * TC_BM + quarter * 32 + src;
                    const int64_t o = ((q * p.nsplit + split) * TC_NWG + wg) * PUB;
#pragma unroll
                    for (int e = lane; e < PUB; e += 32) {
                        const float2 v = e < n ? row[e] : make_float2(neg_inf(), __uint_as_float(INVALID_ID));
                        p.part_sc[o + e] = v.x;
                        p.part_id[o + e] = __float_as_uint(v.y);
                    }
                }
                p.part_tau[(qrow * p.nsplit + split) * TC_NWG + wg] = tau;
                if (tau > tau_in) __stcg(p.tau + qrow, tau);
                if (qidx >= 0 && tau > tau_in) atomic_max_f32(p.tau_q + qidx, tau);
            } else {
#pragma unroll 1
            for (int src = 0; src < 32; ++src) {
                const int n = __shfl_sync(FULL_MASK, cnt, src);
                const float* rsc = warp_sc + src * PSTR;
                const uint32_t* rid = warp_id + src * PSTR;
                const int64_t q = (int64_t)qt * TC_BM + quarter * 32 + src;
                const int64_t o = ((q * p.nsplit + split) * TC_NWG + wg) * PUB;
#pragma unroll
                for (int e = lane; e < PUB; e += 32) {
                    p.part_sc[o + e] = e < n ? rsc[e] : neg_inf();
                    p.part_id[o + e] = e < n ? rid[e] : INVALID_ID;
                }
            }
            p.part_tau[(qrow * p.nsplit + split) * TC_NWG + wg] = tau;
            if (tau > tau_in) __stcg(p.tau + qrow, tau);
            if (qidx >= 0 && tau > tau_in) atomic_max_f32(p.tau_q + qidx, tau);
            }
        }
        TC_PROF(
        if (warp == 0 && lane == 0 && blockIdx.x < 160) {
            unsigned long long* pr = g_tc_prof + blockIdx.x * TC_PROF_WORDS;
            pr[3] = prof_tfull; pr[4] = prof_rare; pr[5] = prof_groups; pr[6] = prof_compact; pr[7] = prof_append;
            pr[8] = clock64() - prof_t0; pr[9] = tile_no;
            pr[10] = 0; pr[11] = prof_cc;
        }
        )
    }

    // ------------------------------ common exit ----------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) cluster_sync_all();      // neither CTA leaves while the other may still touch its memory
    if (warp == W_MMA) {
        tc_fence_after_sync();
        if (PAIR) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
    }
}

// Starting threshold of every query row from the seeding pass: the `rank`-th largest of the
// row's 32 class maxima (16 column classes x 2 warpgroups, disjoint sets of database rows).  At
// least `rank` distinct rows reach it, and being an order statistic of many classes it scatters
// far less than the smallest of a few maxima.  One warp per row, lane = class.
//
// With a margin (row-sharded databases: the class maxima are the element-wise maximum over all
// shards, so the `rank` rows may live on other shards) the threshold is lowered by twice the
// scoring error bound plus the fp32 slack: a row whose score stays at or below
//     cert = pick - 2 eps_rel ||q|| maxnorm - slack
// is at least as far from the query as each of those `rank` rows, whichever shard holds them,
// so a shard that re-scores every row above `cert` cannot miss a global neighbour.  `cert` is
// also written to mg.cert_out, where the finalisation reads it.
__global__ void __launch_bounds__(256) tc_seed_select_kernel(const float* __restrict__ seed_cls, float* __restrict__ tau,
                                                             int64_t nq_pad, int rank, const TcSeedMargin mg) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= nq_pad) return;
    const float v = __ldg(seed_cls + row * (TC_NWG * 16) + lane);
    // rank of each value among the 32 (ties broken by position): a permutation
    int r = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float o = __shfl_sync(FULL_MASK, v, j);
        r += (o > v || (o == v && j < lane)) ? 1 : 0;
    }
    const unsigned sel = __ballot_sync(FULL_MASK, r == rank - 1);
    float pick = __shfl_sync(FULL_MASK, v, __ffs(sel) - 1);
    if (mg.q != nullptr) {
        float qsq = 0.f;
        if (row < mg.nq) {
            const void* qp = row_at(mg.q, row, mg.ldq, mg.dt);
            for (int c = lane; c < mg.d; c += 32) { const float x = ld_elem(qp, c, mg.dt); qsq += x * x; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qsq += __shfl_xor_sync(FULL_MASK, qsq, o);
        const float mn = __ldg(mg.maxnorm);
        if (pick > neg_inf()) pick -= 2.f * mg.eps_rel * sqrtf(qsq) * mn + 1e-5f * (qsq + mn * mn);
        if (lane == 0 && mg.cert_out != nullptr) mg.cert_out[row] = pick;
    }
    if (lane == 0 && pick > neg_inf()) tau[row] = pick;
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D bf16 row-major tensor [rows][cols]; box = box_cols columns x box_rows rows.  box_cols is
// 64 (128-byte rows in shared memory, 128-byte swizzle) or 16 (32-byte rows, 32-byte swizzle).
static int make_map_bf16(CUtensorMap* map, const void* base, int64_t rows, int cols, int box_cols, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return FL_ECUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_32B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return FL_ECUDA; }
    return FL_OK;
}

int tc_knn_big(int k) { return k > 16 ? 1 : 0; }
int tc_pool_size(int k) { return tc_knn_big(k) ? TC_BIG_K1 : TC_K1; }
int tc_partial_len(int k) { return TC_NWG * (tc_knn_big(k) ? TC_BIG_CAP : TC_CAP); }
// Deep pools for plain k <= 16 scoring when the whole database is one range, i.e. a query ends up
// with just two pools: the larger of two 12th-best scores sits too close to the k-th neighbour
// for the proof (a quarter of the rows of a 1M x 1M self-kNN failed it).  With three ranges the
// shallow pools prove every row of the benchmark mixture and are faster.  Needs the 128-feature
// shared-memory budget.
int tc_use_deep_pools(int k, int d_pad, int nsplit, int64_t nq_pad) {
    return !tc_knn_big(k) && d_pad <= 128 && nsplit == 1 && !tc_pair_enabled(nq_pad, k);
}
int tc_deep_pool_size() { return TC_MID_K1; }
int tc_deep_partial_len() { return TC_NWG * TC_MID_PUB; }
int tc_taus_per_range() { return TC_NWG; }
int tc_pair_pool_cap() { return TC_GP_CAP; }

int tc_knn_supported(int64_t nq, int64_t m, int d, int k) {
    if (nq < 1 || m < 1) return FL_EUNSUPPORTED;
    if (k > 112) return FL_EUNSUPPORTED;            // pools keep 12 (k <= 16) or 128 entries: leave the proof a margin
    if (d > 512) return FL_EUNSUPPORTED;            // resident query tile: up to 8 chunks of 64 features (beyond 4:
                                                    // pools in global memory only, two ring slots at d = 512)
    if (round_up(m, 256) / 256 > (1 << 23)) return FL_EUNSUPPORTED;
    return FL_OK;
}

// Auto mode takes the tensor-core path once the problem is large enough to amortise it.
int tc_knn_auto(int64_t nq, int64_t m, int d, int k) {
    if (tc_knn_supported(nq, m, d, k) != FL_OK) return 0;
    return (m >= 2048 && nq * m >= (int64_t(1) << 24)) ? 1 : 0;
}

// CTA pairs (cta_group::2) for plain k <= 16 scoring.  Measured on the 1M x 128 benchmark they are
// 7 % slower than single CTAs (the leader's MMA reads half of every database tile from the peer's
// shared memory and waits for both CTAs' epilogues), so they are off unless FLASHLIB_B200_TC_PAIR=1.
int tc_pair_requested() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("FLASHLIB_B200_TC_PAIR"); on = (e && atoi(e) != 0) ? 1 : 0; }
    return on;
}
// Pairs need an even number of query tiles (tc_query_rows_padded provides it).
int tc_pair_enabled(int64_t nq_pad, int k) {
    return tc_pair_requested() && !tc_knn_big(k) && (nq_pad / TC_BM) % 2 == 0 && nq_pad / TC_BM >= 2;
}
int64_t tc_query_rows_padded(int64_t nq) { return round_up(nq, tc_pair_requested() ? 2 * TC_BM : TC_BM); }

void tc_split_plan(int64_t nq_pad, int64_t m_pad, int k, int* nsplit, int64_t* tiles_per_split) {
    const bool pair = tc_pair_enabled(nq_pad, k) != 0;
    // work units that walk a range together, and how many of them the GPU runs at once
    const int64_t n_qtiles = pair ? nq_pad / TC_BM / 2 : nq_pad / TC_BM;
    const int64_t n_tiles = m_pad / TC_BN;
    const int sms = pair ? sm_count() / 2 : sm_count();
    int64_t max_s = n_tiles / 8;
    if (max_s > 64) max_s = 64;
    if (max_s < 1) max_s = 1;
    // Estimated run time in tile units: every SM works through `waves` items of `tps` tiles plus
    // a fixed cost per item (query tile load, pipeline fill and drain, pool publication).
    constexpr int64_t ITEM_OVERHEAD_TILES = 8;
    int64_t best_cost = -1;
    int64_t best_s = 1;
    for (int64_t s = 1; s <= max_s; ++s) {
        const int64_t tps = ceil_div(n_tiles, s);
        const int64_t s_eff = ceil_div(n_tiles, tps);
        const int64_t items = n_qtiles * s_eff;
        const int64_t grid = items < sms ? items : sms;
        const int64_t waves = ceil_div(items, grid);
        const int64_t cost = waves * (tps + ITEM_OVERHEAD_TILES);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s_eff; }
    }
    *tiles_per_split = ceil_div(n_tiles, best_s);
    *nsplit = (int)ceil_div(n_tiles, *tiles_per_split);
}

// ---- experiment controls ------------------------------------------------------------------
// Timing experiments and seeding overrides.  The environment is read once, when the first
// tensor-core launch is prepared; fl_debug_tc_experiment changes the flags and the wait limit
// afterwards (tests of the bounded-wait exit).  Launches with experiment flags 1..16 set mark
// the status words (FL_EUNSUPPORTED): their neighbours are not to be used.
struct TcExperiment {
    int flags = 0;
    uint32_t hint_ns = 1000u;
    uint64_t wait_ns = TC_WAIT_DEFAULT_NS;
    int noseed = 0, seed_tiles = -1, seed_rank = -1;
};
static TcExperiment& tc_experiment() {
    static TcExperiment e = [] {
        TcExperiment x;
        if (const char* v = getenv("FLASHLIB_B200_TC_DEBUG")) x.flags = atoi(v);
        if (const char* v = getenv("FLASHLIB_B200_TC_HINT")) x.hint_ns = (uint32_t)atoi(v);
        if (const char* v = getenv("FLASHLIB_B200_TC_NOSEED")) x.noseed = atoi(v) != 0;
        if (const char* v = getenv("FLASHLIB_B200_TC_SEED_TILES")) x.seed_tiles = atoi(v);
        if (const char* v = getenv("FLASHLIB_B200_TC_SEED_RANK")) x.seed_rank = atoi(v);
        return x;
    }();
    return e;
}
void tc_debug_set(int flags, unsigned wait_us) {
    TcExperiment& e = tc_experiment();
    e.flags = flags;
    e.wait_ns = wait_us ? (uint64_t)wait_us * 1000ull : TC_WAIT_DEFAULT_NS;
}

// Tensor maps are encoded once per (buffer, shape, box) and kept in a small per-thread cache:
// a serving loop calls with the same plane and the same workspace over and over.
struct MapKey { const void* base; int64_t rows; int cols, box_cols, box_rows; };
static int cached_map_bf16(CUtensorMap* map, const void* base, int64_t rows, int cols, int box_cols, int box_rows) {
    constexpr int SLOTS = 16;
    thread_local MapKey keys[SLOTS];
    thread_local CUtensorMap maps[SLOTS];
    thread_local int used = 0, next = 0;
    for (int i = 0; i < used; ++i) {
        const MapKey& k = keys[i];
        if (k.base == base && k.rows == rows && k.cols == cols && k.box_cols == box_cols && k.box_rows == box_rows) {
            *map = maps[i];
            return FL_OK;
        }
    }
    const int rc = make_map_bf16(map, base, rows, cols, box_cols, box_rows);
    if (rc != FL_OK) return rc;
    const int slot = used < SLOTS ? used++ : (next++ % SLOTS);
    keys[slot] = MapKey{base, rows, cols, box_cols, box_rows};
    maps[slot] = *map;
    return FL_OK;
}

int tc_seed_tiles(int64_t m_pad, int k);

struct TcLaunch {
    CUtensorMap map_q, map_q_aug, map_db, map_db_aug;
    TcSmemPlan sp;
    TcKernelParams kp;
    int seed_tiles, seed_rank;
    bool big, mid, gs;
};

// Plain k <= 16 scoring with the small pools in global memory (mode KNN_GS) instead of shared memory.
// Measured on 1M rows x 10 000 queries: 8 % slower at 128 features (2.86 vs 2.65 ms: the three-slot ring
// was not what held the kernel back, and compactions through the L2 cost more), 12 % faster at 192 and
// 21 % faster at 256 features (4.83 vs 5.85 ms), where pools in shared memory leave only two ring
// slots.  So: beyond 128 features.  FLASHLIB_B200_TC_GS=0/1 overrides.
static int tc_gs_requested(int d_pad) {
    static int v = -2;
    if (v == -2) { const char* e = getenv("FLASHLIB_B200_TC_GS"); v = e ? (atoi(e) != 0 ? 1 : 0) : -1; }
    return v >= 0 ? v : (d_pad > 128 ? 1 : 0);
}

// Everything a launch needs: tensor maps, shared-memory plan, kernel parameters and the size of
// the seeding sample.
static int tc_prepare(const TcKnnParams& p, float* dbg, int64_t dbg_ld, TcLaunch* L) {
    FL_CHECK_ARG(p.qplane && p.dbrows && p.tau, "tensor-core kNN launch with a null buffer");
    L->big = tc_knn_big(p.k) != 0 || p.big_pools != 0;
    L->mid = p.deep_pools != 0;
    const TcExperiment& ex0 = tc_experiment();
    L->gs = !L->big && !L->mid && p.pair_pools == nullptr && dbg == nullptr && ex0.flags == 0 && p.row_query == nullptr &&
            p.item_t0 == nullptr && !tc_pair_enabled(p.nq_pad, p.k) && tc_gs_requested(p.d_pad) != 0;
    const int pitch = p.d_pad + PLANE_AUG_COLS;
    int rc = cached_map_bf16(&L->map_q, p.qplane, p.nq_pad, pitch, TC_BK, TC_BM);
    if (rc == FL_OK) rc = cached_map_bf16(&L->map_q_aug, p.qplane, p.nq_pad, pitch, PLANE_AUG_COLS, TC_BM);
    if (rc == FL_OK) rc = cached_map_bf16(&L->map_db, p.dbrows, p.m_pad, pitch, TC_BK, TC_BN);
    if (rc == FL_OK) rc = cached_map_bf16(&L->map_db_aug, p.dbrows, p.m_pad, pitch, PLANE_AUG_COLS, TC_BN);
    if (rc != FL_OK) return rc;
    FL_CHECK_ARG(!(L->mid && (L->big || dbg)), "tensor-core kNN launch: deep pools go with k <= 16");
    L->sp = tc_smem_plan(p.d_pad, smem_optin_bytes(), (L->big || L->gs || p.pair_pools != nullptr) ? 0 : L->mid ? TC_MID_CAP + 1 : TC_PSTR);
    if (L->sp.nstage < 2) { set_error("tensor-core kNN: feature dimension %d leaves no room for the TMA ring", p.d_pad); return FL_EUNSUPPORTED; }
    const TcExperiment& ex = tc_experiment();
    TcKernelParams& kp = L->kp;
    kp = TcKernelParams{};
    kp.n_qtiles = (int)(p.nq_pad / TC_BM);
    kp.n_tiles = (int)(p.m_pad / TC_BN);
    kp.nsplit = p.nsplit;
    kp.tiles_per_split = (int)p.tiles_per_split;
    kp.nkc = L->sp.nkc; kp.nstage = L->sp.nstage;
    kp.off_b = L->sp.off_b; kp.off_pool_sc = L->sp.off_pool_sc; kp.off_pool_id = L->sp.off_pool_id;
    kp.off_bar = L->sp.off_bar;
    kp.nq_pad = p.nq_pad; kp.part_sc = p.part_sc; kp.part_id = p.part_id;
    kp.tau = p.tau; kp.part_tau = p.part_tau; kp.status = p.status; kp.dbg_scores = dbg; kp.dbg_ld = dbg_ld;
    kp.part_cnt = p.part_cnt;
    kp.gpool = reinterpret_cast<float2*>(p.pair_pools);
    kp.seed_cls = p.seed_cls;
    kp.nq_dev = p.nq_dev; kp.item_t0 = p.item_t0; kp.item_t1 = p.item_t1; kp.item_order = p.item_order;
    kp.row_query = p.row_query; kp.tau_q = p.tau_q;
    kp.dbg_flags = ex.flags;
    kp.wait_hint_ns = ex.hint_ns;
    kp.wait_ns = ex.wait_ns;
    kp.tile_stride = 1;
    // Seeding sample.  The threshold is the seed_rank-th largest of 32 class maxima, which sits
    // near rank 32 ln(32 / (32 - seed_rank)) of the sample, hence near that figure times
    // n_tiles / seed_tiles of the whole database.
    //  k <= 16: the pools tighten the threshold quickly; one tile in 16 (at most 64 tiles, 96 for the
    //           largest databases), k + 6 rows guaranteed.
    //  large k: the pools seldom fill, so the seeded threshold is what filters.  Aim at about
    //           rank 6 k of the database: loose enough that the k-th neighbour's error band
    //           stays inside, tight enough that a few hundred rows per query are published.
    int seed_rank = p.k + 6 < 32 ? p.k + 6 : 32;
    if (L->big) seed_rank = p.k >= 64 ? 16 : 8;
    if (ex.seed_rank >= 0) seed_rank = ex.seed_rank;
    if (seed_rank < 1) seed_rank = 1;
    if (seed_rank > 32) seed_rank = 32;
    const int seed_tiles = tc_seed_tiles(p.m_pad, p.k);
    L->seed_tiles = seed_tiles;
    L->seed_rank = seed_rank;
    return FL_OK;
}

// Database tiles the seeding pass samples (0: no seeding for this shape).
int tc_seed_tiles(int64_t m_pad, int k) {
    const int n_tiles = (int)(m_pad / TC_BN);
    const TcExperiment& ex = tc_experiment();
    // one tile in 16, at most 64 -- 96 for the largest databases (measured on 3 907 tiles x 10 000
    // queries: 64 tiles 2.795 ms per step, 96 2.767, 128 2.777, 160 2.797; on 489-tile shards x 80 000
    // queries the 30 tiles of the rule beat 16 and 48)
    int seed_tiles = n_tiles >= 3072 ? 96 : n_tiles >= 1024 ? 64 : n_tiles / 16;

    if (tc_knn_big(k)) {
        const double sample_rank = k >= 64 ? 22.2 : 9.2;
        seed_tiles = (int)((double)n_tiles * sample_rank / (6.0 * k));
        if (seed_tiles > n_tiles / 8) seed_tiles = n_tiles / 8;
        if (seed_tiles > n_tiles / 2) seed_tiles = n_tiles / 2;
        if (seed_tiles < 16) seed_tiles = 0;
    } else if (n_tiles < 256) {
        // Small databases (k <= 16): a cold pool costs a fixed few dozen insertions and compactions
        // per query row, which dwarfs the scoring of a handful of tiles (the coarse probe of an
        // inverted-file search scores 4).  Sample 16 tiles, or simply all of them: the threshold
        // is then tight, so the selection lowers it by the proof's margin (tc_seed_dense).
        seed_tiles = n_tiles < 16 ? n_tiles : 16;
    }
    if (ex.seed_tiles >= 0) seed_tiles = ex.seed_tiles < n_tiles ? ex.seed_tiles : n_tiles;
    if (ex.noseed) seed_tiles = 0;
    return seed_tiles;
}
// 1 when the seeding sample is a large share of the database: a threshold that k + 6 sampled rows
// reach then cuts close to the k-th neighbour, and must be lowered by twice the scoring error bound
// for the finalisation's proof to hold (see tc_seed_select_kernel).
int tc_seed_dense(int64_t m_pad, int k) {
    const int n_tiles = (int)(m_pad / TC_BN);
    return !tc_knn_big(k) && n_tiles < 256 && tc_seed_tiles(m_pad, k) > 0;
}

// Seeding pass: class maxima of a strided sample of the database tiles into p.seed_cls
// ([nq_pad][32]).  Without a sample (database too small) the maxima are set to -inf.
int launch_knn_tc_seed(const TcKnnParams& p, cudaStream_t st) {
    FL_CHECK_ARG(p.seed_cls != nullptr, "tensor-core seeding pass without a class buffer");
    TcLaunch L;
    int rc = tc_prepare(p, nullptr, 0, &L);
    if (rc != FL_OK) return rc;
    TcKernelParams sk = L.kp;
    sk.dbg_scores = nullptr;
    sk.row_query = nullptr; sk.tau_q = nullptr;
    if (p.item_t0 != nullptr) {
        // item tables (inverted-file scan): the first item_tile_cap tiles of every item's own range
        FL_CHECK_ARG(p.item_tile_cap > 0 && p.nsplit == 1, "tensor-core seeding over item tables needs a tile cap");
        sk.item_tile_cap = p.item_tile_cap;
    } else {
        if (L.seed_tiles == 0) return launch_fill_f32(p.seed_cls, p.nq_pad * (TC_NWG * 16), -INFINITY, st);
        sk.nsplit = 1;
        sk.tiles_per_split = L.seed_tiles;
        sk.tile_stride = L.kp.n_tiles / L.seed_tiles;
        sk.n_tiles = L.seed_tiles;
        sk.nq_dev = nullptr;
    }
    // the seeding kernel keeps no pools: the ring gets the shared memory the pools would take
    const TcSmemPlan sp = L.sp;
    const int sgrid = sk.n_qtiles < sm_count() ? sk.n_qtiles : sm_count();
    FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_SEED>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
    knn_tc_kernel<false, TC_MODE_SEED><<<sgrid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, sk);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// Starting thresholds from class maxima (this shard's, or the element-wise maximum over all
// shards of a sharded database): see tc_seed_select_kernel.
int launch_knn_tc_seed_select(const TcKnnParams& p, const TcSeedMargin& mg, cudaStream_t st) {
    FL_CHECK_ARG(p.seed_cls != nullptr && p.tau != nullptr, "tensor-core threshold selection without buffers");
    TcLaunch L;
    int rc = tc_prepare(p, nullptr, 0, &L);
    if (rc != FL_OK) return rc;
    tc_seed_select_kernel<<<(unsigned)ceil_div(p.nq_pad, 8), 256, 0, st>>>(p.seed_cls, p.tau, p.nq_pad, L.seed_rank, mg);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// Main scoring launch (thresholds in p.tau as they stand).
static int launch_tc_main(const TcKnnParams& p, float* dbg, int64_t dbg_ld, cudaStream_t st) {
    const bool gp = p.pair_pools != nullptr;
    FL_CHECK_ARG(p.part_tau && (gp ? p.part_cnt != nullptr : (p.part_sc && p.part_id)), "tensor-core kNN launch with a null buffer");
    TcLaunch L;
    int rc = tc_prepare(p, dbg, dbg_ld, &L);
    if (rc != FL_OK) return rc;
    const bool big = L.big, mid = L.mid;
    FL_CHECK_ARG(!gp || (!big && !dbg && p.k <= 16), "tensor-core kNN launch: global pair pools go with k <= 16");
    FL_CHECK_ARG(!big || (p.part_cnt && !dbg), "tensor-core kNN launch (large k) without a count buffer");
    FL_CHECK_ARG((p.row_query == nullptr) == (p.tau_q == nullptr), "tensor-core kNN launch: row_query and tau_q go together");
    FL_CHECK_ARG((p.item_t0 == nullptr) == (p.item_t1 == nullptr) && (p.item_t0 == nullptr || (p.nsplit == 1 && !big)),
                 "tensor-core kNN launch: per-tile ranges need one range per query tile and k <= 16");
    const TcKernelParams& kp = L.kp;
    const TcSmemPlan& sp = L.sp;
    const int pitch = p.d_pad + PLANE_AUG_COLS;
    const int items = kp.n_qtiles * kp.nsplit;
    const int grid = items < sm_count() ? items : sm_count();
    // CTA pairs (cta_group::2): plain k <= 16 scoring over uniform ranges, an even number of query
    // tiles, at least one pair-item per cluster of a full grid.  FLASHLIB_B200_TC_PAIR=0/1 overrides.
    const bool pair = !gp && !mid && dbg == nullptr && p.item_t0 == nullptr && p.nq_dev == nullptr &&
                      tc_pair_enabled(p.nq_pad, p.k);
    if (gp) {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_KNN_GPOOL>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
        knn_tc_kernel<false, TC_MODE_KNN_GPOOL><<<grid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, kp);
    } else if (pair) {
        CUtensorMap map_db_h, map_db_aug_h;
        rc = cached_map_bf16(&map_db_h, p.dbrows, p.m_pad, pitch, TC_BK, TC_BN / 2);
        if (rc == FL_OK) rc = cached_map_bf16(&map_db_aug_h, p.dbrows, p.m_pad, pitch, PLANE_AUG_COLS, TC_BN / 2);
        if (rc != FL_OK) return rc;
        const TcSmemPlan spp = tc_smem_plan(p.d_pad, smem_optin_bytes(), TC_PSTR, TC_B_STAGE / 2);
        TcKernelParams kq = kp;
        kq.nstage = spp.nstage; kq.off_b = spp.off_b; kq.off_pool_sc = spp.off_pool_sc; kq.off_pool_id = spp.off_pool_id;
        kq.off_bar = spp.off_bar;
        const int pair_items = (kp.n_qtiles / 2) * kp.nsplit;
        int clusters = sm_count() / 2;
        if (clusters > pair_items) clusters = pair_items;
        auto kern = kp.dbg_flags != 0 ? knn_tc_kernel<true, TC_MODE_KNN, true> : knn_tc_kernel<false, TC_MODE_KNN, true>;
        FL_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, spp.bytes));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(2 * clusters));
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = (size_t)spp.bytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        FL_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, L.map_q, L.map_q_aug, map_db_h, map_db_aug_h, kq));
    } else if (mid) {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_KNN_MID>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
        knn_tc_kernel<false, TC_MODE_KNN_MID><<<grid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, kp);
    } else if (big) {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_KNN_BIG>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
        knn_tc_kernel<false, TC_MODE_KNN_BIG><<<grid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, kp);
    } else if (L.gs) {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_KNN_GS>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
        knn_tc_kernel<false, TC_MODE_KNN_GS><<<grid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, kp);
    } else if (dbg != nullptr || kp.dbg_flags != 0) {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<true, TC_MODE_KNN>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
        knn_tc_kernel<true, TC_MODE_KNN><<<grid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, kp);
    } else {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_KNN>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
        knn_tc_kernel<false, TC_MODE_KNN><<<grid, TC_THREADS, sp.bytes, st>>>(L.map_q, L.map_q_aug, L.map_db, L.map_db_aug, kp);
    }
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// Seeding (when p.seed_cls is given and the database is large enough for it to matter), threshold
// selection and the main scoring launch.
static int launch_tc_impl(const TcKnnParams& p, float* dbg, int64_t dbg_ld, cudaStream_t st) {
    if (p.seed_cls != nullptr && tc_seed_tiles(p.m_pad, p.k) > 0) {
        int rc = launch_knn_tc_seed(p, st);
        if (rc != FL_OK) return rc;
        rc = launch_knn_tc_seed_select(p, TcSeedMargin{}, st);
        if (rc != FL_OK) return rc;
    }
    return launch_tc_main(p, dbg, dbg_ld, st);
}
int launch_knn_tc_scoring(const TcKnnParams& p, cudaStream_t st) { return launch_tc_main(p, nullptr, 0, st); }

// FLASHLIB_B200_ASSIGN_SINGLE_A=1: one query-tile buffer in the assignment launches (measurements).
static int tc_assign_single_a() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("FLASHLIB_B200_ASSIGN_SINGLE_A"); v = (e && atoi(e) != 0) ? 1 : 0; }
    return v;
}

int tc_prof_read(unsigned long long* host_out, int words) {
    const size_t n = sizeof(unsigned long long) * (size_t)(words < 160 * TC_PROF_WORDS ? words : 160 * TC_PROF_WORDS);
    FL_CHECK_CUDA(cudaMemcpyFromSymbol(host_out, g_tc_prof, n));
    return FL_OK;
}

// Assignment launch: queries = sample rows, database = centroids; writes per (row, warpgroup)
// the best and second-best score and the best centroid.
int launch_assign_tc(const TcKnnParams& p, float* asg_sc, uint32_t* asg_id, const int* nq_dev, cudaStream_t st) {
    FL_CHECK_ARG(p.qplane && p.dbrows && asg_sc && asg_id && p.tau, "tensor-core assignment launch with a null buffer");
    CUtensorMap map_q, map_q_aug, map_db, map_db_aug;
    const int pitch = p.d_pad + PLANE_AUG_COLS;
    int rc = make_map_bf16(&map_q, p.qplane, p.nq_pad, pitch, TC_BK, TC_BM);
    if (rc == FL_OK) rc = make_map_bf16(&map_q_aug, p.qplane, p.nq_pad, pitch, PLANE_AUG_COLS, TC_BM);
    if (rc == FL_OK) rc = make_map_bf16(&map_db, p.dbrows, p.m_pad, pitch, TC_BK, TC_BN);
    if (rc == FL_OK) rc = make_map_bf16(&map_db_aug, p.dbrows, p.m_pad, pitch, PLANE_AUG_COLS, TC_BN);
    if (rc != FL_OK) return rc;
    // Items are short here (a query tile against a handful of centroid tiles): with room for a second
    // query-tile buffer beside a three-slot ring the next item's tile is loaded while this one is scored.
    TcSmemPlan sp = tc_smem_plan(p.d_pad, smem_optin_bytes(), 0, TC_B_STAGE, 2);
    int nabuf = 2;
    if (sp.nstage < 3 || tc_assign_single_a()) { sp = tc_smem_plan(p.d_pad, smem_optin_bytes(), 0); nabuf = 1; }
    if (sp.nstage < 2) { set_error("tensor-core assignment: feature dimension %d leaves no room for the TMA ring", p.d_pad); return FL_EUNSUPPORTED; }
    TcKernelParams kp{};
    kp.nabuf = nabuf;
    kp.n_qtiles = (int)(p.nq_pad / TC_BM);
    kp.n_tiles = (int)(p.m_pad / TC_BN);
    kp.nsplit = 1;
    kp.tiles_per_split = kp.n_tiles;
    kp.nkc = sp.nkc; kp.nstage = sp.nstage;
    kp.off_b = sp.off_b; kp.off_pool_sc = sp.off_pool_sc; kp.off_pool_id = sp.off_pool_id; kp.off_bar = sp.off_bar;
    kp.nq_pad = p.nq_pad; kp.tau = p.tau; kp.status = p.status;
    kp.asg_sc = asg_sc; kp.asg_id = asg_id;
    kp.nq_dev = nq_dev;
    kp.tile_stride = 1; kp.wait_hint_ns = 1000u;
    const int grid = kp.n_qtiles < sm_count() ? kp.n_qtiles : sm_count();
    FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel<false, TC_MODE_ASSIGN>, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
    knn_tc_kernel<false, TC_MODE_ASSIGN><<<grid, TC_THREADS, sp.bytes, st>>>(map_q, map_q_aug, map_db, map_db_aug, kp);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

int launch_knn_tc(const TcKnnParams& p, cudaStream_t st) { return launch_tc_impl(p, nullptr, 0, st); }
int launch_knn_tc_debug(const TcKnnParams& p, float* dbg, int64_t dbg_ld, cudaStream_t st) {
    return launch_tc_impl(p, dbg, dbg_ld, st);
}

}  // namespace fl
