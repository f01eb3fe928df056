// Internal launch interfaces shared by the kNN translation units.
#pragma once
#include "common.cuh"
#include "plane.h"

namespace fl {

// Exact CUDA-core scoring pass: every (slot, split) pair gets a descending pool of K1
// (score, row) entries at part[(slot*nsplit + split)*K1].
struct SimtKnnParams {
    int dt;                 // element type of the q and db rows (DT_*; leading dimensions in elements)
    const void* q; int64_t ldq;
    const int* qlist;       // optional slot -> query row map
    const int* count_dev;   // optional device-resident slot count
    int64_t count;          // slot count when count_dev is null
    const void* db; int64_t m; int64_t ldb; int d;
    const float* hnorm;     // ||x||^2 / 2 per database row
    int K1, cap, npl;       // published entries per pool, pool capacity, capacity / 32
    int keep;               // entries kept at a compaction inside the scan (<= K1; 0: K1)
    int nsplit; int64_t rows_per_split;
    float* part_sc; uint32_t* part_id;
    int vecq, vecd;
    // dyn_blocks > 0 (fallback pass, slot count only known on the device): the launch is a
    // 1-D grid of dyn_blocks blocks and the kernel spreads them over the live query blocks, so
    // a handful of slots is scanned by many short ranges instead of a few long ones
    // (simt_dyn_split); nsplit / rows_per_split are then ignored.
    int dyn_blocks; int dyn_bq;
    // Inverted-file mode (ivf != 0): block b is work item b = (list c, group g of up to BQ
    // of the (query, probe) pairs that name list c).  item_off/pair_off are exclusive scans
    // over lists (nlist+1 entries), sorted_pair lists the pair ids grouped by list, and the
    // block scans rows list_offsets[c] .. list_offsets[c+1] of db.  Pools are written at
    // part[pair_id * K1]; bq_items is the group size the item table was built for.
    int ivf; int nlist; int nprobe; int bq_items;
    const int* item_off; const int* pair_off; const int* sorted_pair;
    const int64_t* list_offsets;
    // batch > 1 (static geometry only): grid.z walks `batch` independent problems of the same shape;
    // problem b reads q + b * q_bstride and db + b * db_bstride (elements), hnorm + b * m, and
    // writes the pools of its `count` slots after those of problem b - 1.
    int batch; int64_t q_bstride, db_bstride;
    // Optional f32 [queries], -inf initialised: running threshold of every query, shared by the
    // blocks that scan its probed lists.  A block starts from it and raises it to its own
    // pool's threshold when it ends, so lists scanned later start warm.
    float* tau_q;
};
int launch_knn_simt(const SimtKnnParams& p, int64_t max_slots, cudaStream_t st);
// Range split of the dynamic mode for `count` live slots: the same figures on the device
// (scan and finalisation kernels) and on the host (buffer sizing).
struct SimtDynSplit { int nsplit; int64_t rows_per_split; };
__host__ __device__ inline SimtDynSplit simt_dyn_split(int64_t count, int bq, int blocks, int64_t m) {
    const int64_t nqb = (count + bq - 1) / bq;
    int64_t ns = nqb > 0 ? blocks / nqb : 1;
    const int64_t tiles = (m + 127) / 128;
    // ranges of at least four tiles -- or, for a database of a few tiles (k-means centroids), of one:
    // a handful of slots is then still spread over eight times as many blocks
    int64_t lim = tiles / 4;
    if (lim < 8) lim = tiles < 8 ? tiles : 8;
    if (ns > lim) ns = lim;
    if (ns > 296) ns = 296;     // two blocks per SM when a single query block is live
    if (ns < 1) ns = 1;
    const int64_t rps = ((m + ns - 1) / ns + 127) / 128 * 128;
    SimtDynSplit r;
    r.rows_per_split = rps;
    r.nsplit = (int)((m + rps - 1) / rps);
    return r;
}
// Split count / rows per split the CUDA-core pass uses for a problem.
void simt_split_plan(int64_t slots, int64_t m, int K1, int d, int* nsplit, int64_t* rows_per_split);
// Queries per block the CUDA-core pass uses for a pool of K1 entries (0: does not fit).
int simt_block_queries(int K1);

// Merge of the per-split pools, exact fp32 re-rank, top-k selection and (optionally)
// verification of the candidate pool against the scoring error bound.
struct FinalizeParams {
    int dt;                  // element type of the q and db rows (DT_*)
    const void* q; int64_t ldq;
    const int* qlist; const int* count_dev; int64_t count;
    const void* db; int64_t m; int64_t ldb; int d; int vec;
    const float* part_sc; const uint32_t* part_id; int nsplit; int K1;
    int k; int rerank; int64_t row_offset;
    float* out_dist; int32_t* out_idx;
    int verify; float eps_rel; const float* maxnorm;
    // thresholds the scoring pass published per (slot, range): every row it left out of its
    // published pool scored at most this much (nullptr: none were left out below the pool)
    const float* part_tau; int ntau;
    int dyn_blocks; int dyn_bq;   // pools written by a dynamic-mode scan: nsplit comes from simt_dyn_split
    // Optional indirections (inverted-file scan on the tensor-core kernel): pool s of slot q is
    // pool number pool_row[q * nsplit + s] (< 0: empty) instead of q * nsplit + s, and candidate
    // ids are rows of a padded operand plane that id_map turns into database rows (< 0: padding).
    const int* pool_row; const int* id_map; int64_t id_bound;
    const int* part_cnt;     // large-k finalisation: entries per published pool ([slot][ntau])
    // Optional f32 [queries] (row-sharded databases, k <= 16): a slot is also accepted when every row
    // that was not re-scored scored at most cert_tau[query] -- such rows lie at least as far from the
    // query as k rows known to exist somewhere in the database, so this shard's list may be short
    const float* cert_tau;
    int* fb_count; int* fb_list; int fb_cap;
    // Optional: unproven queries go to this list first (the split-plane stage), and to the exact-path
    // list only when it is absent or full
    int* next_count; int* next_list; int next_cap;
    // batch > 1 (slot count known at launch, no lists): grid.y walks `batch` independent problems of
    // `count` slots each; problem b reads q + b * q_bstride and db + b * db_bstride (elements), its
    // pools and its outputs follow those of problem b - 1.
    int batch; int64_t q_bstride, db_bstride;
};
// Finalisation of the large-k tensor-core pools (one block per query).
int launch_knn_finalize_big(const FinalizeParams& p, int64_t max_slots, cudaStream_t st);
int launch_knn_finalize(const FinalizeParams& p, int64_t max_slots, cudaStream_t st);

// Tensor-core (tcgen05) candidate pass over the bf16 plane.
struct TcKnnParams {
    const void* qplane;      // bf16 [nq_pad][d_pad + 16]: features zero padded, ones in the norm columns
    int64_t nq, nq_pad;
    const void* dbrows;      // bf16 [m_pad][d_pad]
    const float* hnorm;      // f32 [m_pad]
    int64_t m, m_pad; int d_pad;
    int K1;                  // entries a pool keeps (informational: fixed by the kernel mode)
    int nsplit; int64_t tiles_per_split;   // database tiles of 256 rows per split
    float* part_sc; uint32_t* part_id;     // [nq_pad][nsplit][tc_partial_len]
    float* tau;              // f32 [nq_pad], running per-query thresholds, -inf initialised
    float* part_tau;         // f32 [nq_pad][nsplit][tc_taus_per_range]: thresholds each (query, range) ended with
    int* part_cnt;           // large-k pools only: i32 [nq_pad][nsplit][tc_taus_per_range] entries per pool
    float* seed_cls;         // f32 [nq_pad][32] scratch of the threshold-seeding pass (nullptr: no seeding)
    int deep_pools;          // 1: pools keep tc_deep_pool_size() entries and publish tc_deep_partial_len() per
                             //    (query, range) (k <= 16): for queries with only a few pools each
    const int* nq_dev;       // optional: live query rows (device); query tiles beyond them are skipped
    const int* row_query;    // optional: query index of every query row (-1: none) and a running threshold
    float* tau_q;            //   per query (f32, -inf initialised) shared by the rows of that query
    const int* item_t0;      // optional, with nsplit == 1: database tile range [item_t0[t], item_t1[t]) of
    const int* item_t1;      //   query tile t instead of one uniform range (inverted-file scan)
    int item_tile_cap;       // seeding pass over item tables: tiles of every item's range it samples
    const int* item_order;   // optional, with item tables: order in which the items are dealt to the CTAs
    void* pair_pools;        // optional (k <= 16): pools kept in global memory as (score f32, row u32) pairs,
                             //   [nq_pad][nsplit][tc_taus_per_range][tc_pair_pool_cap]; entry counts go to
                             //   part_cnt, thresholds to part_tau, part_sc / part_id are not used
    int k;                   // neighbours wanted: selects the pool geometry (tc_knn_big)
    int big_pools;           // 1: the large global-memory pools whatever k is (no pool in shared memory:
                             //    room for a query tile of up to 384 feature columns)
    int32_t* status;
};
// 1 when k takes the large pools (256 entries per (query, range, warpgroup), kept in global memory).
int tc_knn_big(int k);
// Returns FL_EUNSUPPORTED when the shape is outside the tensor-core kernel's range.
int tc_knn_supported(int64_t nq, int64_t m, int d, int k);
int tc_pool_size(int k);
// Entries the tensor-core pass publishes per (query, range): a multiple of the pool size.
int tc_partial_len(int k);
int tc_deep_pool_size();
int tc_use_deep_pools(int k, int d_pad, int nsplit, int64_t nq_pad);
int tc_deep_partial_len();
// Thresholds the tensor-core pass publishes per (query, range).
int tc_taus_per_range();
// Slots of a (query row, warpgroup) pool in the global pair-pool mode.
int tc_pair_pool_cap();
// 1 when FL_KNN_AUTO should take the tensor-core path for this shape.
int tc_knn_auto(int64_t nq, int64_t m, int d, int k);
// Margin applied by the threshold selection when the class maxima cover more than this shard's rows
// (q == nullptr: none): the threshold is lowered by 2 eps_rel ||q|| *maxnorm + slack and copied to
// cert_out (f32 [nq_pad], may be null).
struct TcSeedMargin {
    const void* q; int dt; int64_t ldq; int d; int64_t nq;
    const float* maxnorm; float eps_rel;
    float* cert_out;
};
// Seeding pass alone (class maxima into p.seed_cls, -inf when the database is too small to sample),
// threshold selection alone (p.seed_cls -> p.tau), and the main scoring launch alone.
int launch_knn_tc_seed(const TcKnnParams& p, cudaStream_t st);
int launch_knn_tc_seed_select(const TcKnnParams& p, const TcSeedMargin& mg, cudaStream_t st);
int launch_knn_tc_scoring(const TcKnnParams& p, cudaStream_t st);
// 1 when thresholds seeded for this shape need the proof's margin (sample = a large share of the rows).
int tc_seed_dense(int64_t m_pad, int k);
// Experiment flags of the scoring kernel and the limit of its barrier waits (0: default).
void tc_debug_set(int flags, unsigned wait_us);
// Same as launch_knn_tc, additionally dumping the scores of query tile 0 to dbg[128][dbg_ld].
int tc_prof_read(unsigned long long* host_out, int words);
int launch_knn_tc_debug(const TcKnnParams& p, float* dbg, int64_t dbg_ld, cudaStream_t st);
void tc_split_plan(int64_t nq_pad, int64_t m_pad, int k, int* nsplit, int64_t* tiles_per_split);
int tc_pair_enabled(int64_t nq_pad, int k);
// Query rows of the bf16 query plane for nq queries: whole tiles of 128 (whole pairs of tiles when
// CTA pairs are requested).
int64_t tc_query_rows_padded(int64_t nq);
int launch_knn_tc(const TcKnnParams& p, cudaStream_t st);
// k-means assignment on the same pipeline: asg_sc [nq_pad][2][2] (best, second-best score per
// warpgroup half), asg_id [nq_pad][2] (best centroid per half).  Only qplane/nq_pad, dbrows/
// m_pad/d_pad, tau (scratch) and status of `p` are used.
// nq_dev (optional): device-resident count of live rows; query tiles beyond it are skipped.
int launch_assign_tc(const TcKnnParams& p, float* asg_sc, uint32_t* asg_id, const int* nq_dev, cudaStream_t st);

// Split (hi/lo) operand planes of the second, more precise tensor-core stage (kmeans_tc.cu).
// Database side: rows [m_pad][3 d_pad + 16] = [hi | hi | lo | norm terms] laid out by
// plane_layout(m, 3 d_pad).  Query side: the rows listed in `rows` (live count on the device, at
// most `cap`) as [hi | lo | hi | ones]; with `tau_out` the kernel also derives each listed row's
// starting threshold from the k-th distance found so far (`prev_dist` [nq][k]):
// (||q||^2 - d_k) / 2 lowered by 2 eps_rel ||q|| *maxnorm and the proof's slack.
int split_plane_supported(int d);
int launch_split_db_plane(const float* c, int64_t m, int d, int64_t ldc, void* plane, cudaStream_t st);
int launch_split_query_gather(const float* x, int64_t ldx, int d, const int* rows, const int* rows_count, int cap,
                              void* out, int d_pad, const float* prev_dist, int k, const float* maxnorm, float eps_rel,
                              float* tau_out, cudaStream_t st);

// bf16 query plane [nq_pad][d_pad + 16] (features zero padded, ones in the norm columns) from fp32 queries.
int launch_query_plane(const void* q, int64_t nq, int64_t ldq, int d, void* qplane, int64_t nq_pad,
                       int d_pad, cudaStream_t st, int dt = DT_F32);

// Small helpers shared by the entry points.
int launch_plane_build(const void* db, int64_t m, int d, int64_t ld, void* plane, cudaStream_t st, int dt = DT_F32);
int launch_fill_f32(float* p, int64_t n, float v, cudaStream_t st);
int launch_ivf_group(const int32_t* probed, int64_t npairs, int nlist, int bq, const int64_t* list_offsets, int* cnt,
                     int* pair_off, int* item_off, int* cursor, int* sorted_pair, cudaStream_t st);
int launch_fallback_fixup(int* fb_count, int fb_cap, int32_t* status, int K1, cudaStream_t st);

}  // namespace fl
