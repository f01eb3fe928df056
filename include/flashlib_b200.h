/*
 * flashlib_b200 -- C ABI of the B200 (sm_100a) fused squared-L2 distance + top-k path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*).  Nothing here allocates device memory unless the
 * comment on the entry point says otherwise: the caller passes outputs and a
 * workspace sized by the matching *_workspace_bytes() query.  All launches are
 * stream-ordered and never synchronise the host.
 *
 * The reference project (FlashML-org/flashlib) is pure Python; it has no FFI layer.
 * Each declaration therefore cites the Python function (path:line inside the reference
 * tree) whose device work it replaces.
 *
 * Return value: 0 on success, a negative FL_E* code otherwise; fl_last_error() returns
 * a thread-local human-readable message for the last failure.
 */
#ifndef FLASHLIB_B200_H_
#define FLASHLIB_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FL_OK            0
#define FL_EINVAL       -1   /* bad argument (maps to ValueError / AssertionError)      */
#define FL_EUNSUPPORTED -2   /* shape or mode outside what this build implements         */
#define FL_ECUDA        -3   /* a CUDA runtime / driver call failed                      */
#define FL_ETIMEOUT     -4   /* a bounded device-side wait gave up (see status words)    */
#define FL_EWORKSPACE   -5   /* workspace or plane buffer too small                      */

/* Element types of the caller's rows (argument `dtype` of fl_knn_rows and its helpers). */
#define FL_DTYPE_F32   0
#define FL_DTYPE_BF16  1
#define FL_DTYPE_F16   2

/* kNN modes (argument `mode` of fl_knn_f32 / fl_knn_workspace_bytes). */
#define FL_KNN_AUTO        -1  /* tensor-core path when supported, else CUDA-core path   */
#define FL_KNN_EXACT_SIMT   0  /* fp32 CUDA-core scoring + exact re-rank                 */
#define FL_KNN_BF16_RERANK  1  /* tcgen05 bf16 candidates, exact fp32 re-rank, verified  */

/* Device status words (int32[FL_STATUS_WORDS]) written by the kNN / assign kernels.     */
#define FL_STATUS_WORDS     8
#define FL_STATUS_ERROR     0  /* 0; FL_ETIMEOUT when a bounded wait expired (the results
                                  of that call are invalid); FL_EUNSUPPORTED when the call
                                  ran with timing-experiment flags (results invalid);
                                  FL_EWORKSPACE if more rows failed verification than the
                                  fallback list holds (cannot happen with a workspace of
                                  fl_knn_workspace_bytes: the list holds every query)     */
#define FL_STATUS_WHERE     1  /* which wait expired (role << 16 | barrier index)        */
#define FL_STATUS_FALLBACK  2  /* rows whose candidate pool failed verification and were
                                  recomputed on the exact CUDA-core path                 */
#define FL_STATUS_POOL      3  /* candidate-pool size per row used by the last call      */
#define FL_STATUS_STAGE2    4  /* fl_knn_staged_f32: rows the first proof rejected and the
                                  split-plane tensor-core stage scored again             */

int         fl_version(void);
const char* fl_last_error(void);

/* 1 when the running process can see an sm_100 device, 0 otherwise (never fails). */
int         fl_device_ok(void);

/* Measurement hooks; they have no counterpart in the reference (it times from Python,   */
/* knn/triton/_common.py:32-44).  fl_launch_count: kernels launched by this library since */
/* it was loaded.  fl_profile_enable(1) makes fl_knn_f32 / fl_kmeans_assign_f32 /        */
/* fl_ivf_fine_scan_f32 bracket their dominant (scoring) kernel with CUDA events on the  */
/* caller's stream, up to 256 samples; fl_profile_read_ms waits for sample i and returns */
/* its duration.  fl_profile_enable(2) instead records an event at every step of         */
/* fl_ivf_fine_scan_tc_f32's launch sequence; sample i is then the time between steps i    */
/* and i + 1.  Not thread-safe; meant for one benchmarking thread.                        */
unsigned long long fl_launch_count(void);
int         fl_profile_enable(int on);
int         fl_profile_count(void);
int         fl_profile_read_ms(int i, float* ms);

/* ---------------------------------------------------------------------------------- */
/* Row norms.  Replaces flashlib/primitives/knn/triton/_row_norm.py:59-93               */
/* (_fast_row_sq) and knn/cutedsl/blackwell_impl.py:114-124 (_row_sqnorm).              */
/* out[i] = sum_j x[i*ld + j]^2 in fp32.                                               */
int fl_rownorm_f32(const float* x, int64_t n, int d, int64_t ld, float* out, void* stream);

/* ---------------------------------------------------------------------------------- */
/* Database operand plane for the tensor-core path (index-build-time work; the          */
/* reference caches the equivalent c_sq per data_ptr: knn/triton/_row_norm.py:82-93,    */
/* and casts storage per knn/impl.py:257-261).                                          */
/* Layout of `plane` (all offsets 1024-byte aligned, see fl_knn_plane_bytes):           */
/*   bf16 [m_pad][d_pad+16] row-major, zero padded (m_pad % 256 == 0, d_pad % 64 == 0);   */
/*                        columns d_pad..d_pad+2 hold -||x||^2/2 split into three bf16     */
/*   f32  [m_pad]         half squared norms ||x||^2/2 of the fp32 rows, +inf padding   */
/*   f32  [4]             [0] = max row norm ||x|| over the plane                        */
int64_t fl_knn_plane_bytes(int64_t m, int d);
int     fl_knn_prepare_db_f32(const float* db, int64_t m, int d, int64_t ld,
                              void* plane, int64_t plane_bytes, void* stream);

/* ---------------------------------------------------------------------------------- */
/* Fused exact kNN.  Replaces flash_knn_triton/_run/_try_launch                         */
/* (knn/triton/dispatch.py:934-1178), the insert kernel (knn/triton/insert.py:30-204),  */
/* the split merge (dispatch.py:987-994), the Blackwell CuTe-DSL kernels                */
/* (knn/cutedsl/blackwell_impl.py:152-1225) and the exact distance gather               */
/* (kernels/distance/triton/knn_gather_l2sq.py:173-229) behind                          */
/* flash_knn_dispatch (knn/impl.py:199-282).                                            */
/*                                                                                      */
/* q [nq][ldq], db [m][ldb] fp32 row-major on the device.  out_dist [nq][k] fp32 true   */
/* squared L2, ascending; out_idx [nq][k] int32 = database row + row_offset (row_offset */
/* lets a row shard report global ids); ties keep the lower row.  `plane` is the buffer */
/* filled by fl_knn_prepare_db_f32 for the same db (may be NULL for FL_KNN_EXACT_SIMT). */
/* `status` is int32[FL_STATUS_WORDS] on the device (may be NULL).                      */
int64_t fl_knn_workspace_bytes(int64_t nq, int64_t m, int d, int k, int mode);
int     fl_knn_f32(const float* q, int64_t nq, int64_t ldq,
                   const float* db, int64_t m, int64_t ldb, int d, int k, int mode,
                   const void* plane, int64_t row_offset,
                   float* out_dist, int32_t* out_idx,
                   void* ws, int64_t ws_bytes, int32_t* status, void* stream);

/* A batch of independent problems of one shape in one call (the reference's kernels take  */
/* the batch on a grid axis, knn/triton/insert.py:49; its callers are many small problems, */
/* where a launch per problem is the whole cost).  Problem b reads q + b * q_bstride and    */
/* db + b * db_bstride (elements) and writes out_dist / out_idx [batch][nq][k].  Exact      */
/* CUDA-core path; large problems are better served by one fl_knn_f32 call each.            */
int64_t fl_knn_batch_workspace_bytes(int batch, int64_t nq, int64_t m, int d, int k);
int     fl_knn_batch_f32(const float* q, int batch, int64_t nq, int64_t ldq, int64_t q_bstride,
                         const float* db, int64_t m, int64_t ldb, int64_t db_bstride, int d, int k,
                         float* out_dist, int32_t* out_idx, void* ws, int64_t ws_bytes, void* stream);

/* fl_knn_f32 for rows stored as fp32, bf16 or fp16 (`dtype` = FL_DTYPE_*, the same for q and */
/* db; leading dimensions in elements).  The reference runs its kernels on 16-bit inputs as    */
/* they are, and casts fp32 inputs to 16-bit storage when the caller's `tol` allows it          */
/* (knn/impl.py:257-261, linalg/gemm/__init__.py:163-183): the database then takes half the     */
/* memory.  Here the bf16 operand plane is built straight from the 16-bit rows                  */
/* (fl_knn_prepare_db_rows; bf16 values enter it unrounded), no fp32 copy exists, and the exact */
/* re-rank and the exact pass widen the stored values to fp32 on load -- which is exact, so the */
/* result is the exact kNN of the values as stored, distances in fp32.  Workspace as for        */
/* fl_knn_f32.  No split-plane stage for 16-bit rows.                                           */
int     fl_knn_prepare_db_rows(const void* db, int dtype, int64_t m, int d, int64_t ld,
                               void* plane, int64_t plane_bytes, void* stream);
int     fl_knn_rows(const void* q, int64_t nq, int64_t ldq,
                    const void* db, int64_t m, int64_t ldb, int d, int k, int dtype, int mode,
                    const void* plane, int64_t row_offset,
                    float* out_dist, int32_t* out_idx,
                    void* ws, int64_t ws_bytes, int32_t* status, void* stream);

/* fl_knn_f32 (tensor-core mode) with a second tensor-core stage between the bf16 pass and  */
/* the exact CUDA-core pass.  Rows whose bf16 candidate pool cannot be proven complete are  */
/* scored again with every fp32 operand carried as two bf16 values (hi = bf16(v),           */
/* lo = bf16(v - hi); one product over [hi|lo|hi] x [hi|hi|lo] columns gives                */
/* hi.hi + lo.hi + hi.lo), the error-compensated split the reference uses for fp32-exact    */
/* ranking on tensor cores (linalg/gemm/bf16_x3.py:1-22 with bf16 halves, the lo.lo product  */
/* dropped and one fp32 accumulator across the three products; linalg/gemm/tf32_x3.py:9-31, */
/* linalg/gemm/triton/fused_kernels.py:222-294 with TF32 halves).  The scoring error drops from 2^-8 to about 2^-16 of          */
/* ||q|| max||x||, so the same proof accepts nearly every row; what is left takes the exact  */
/* pass as before (status[FL_STATUS_STAGE2] / [FL_STATUS_FALLBACK] count the two).  d <= 128.*/
/* `split_plane` is filled once per database by fl_knn_prepare_split_f32                    */
/* (fl_knn_split_plane_bytes = 0: no split plane for this d); NULL = no second stage.       */
int64_t fl_knn_split_plane_bytes(int64_t m, int d);
int     fl_knn_prepare_split_f32(const float* db, int64_t m, int d, int64_t ld,
                                 void* split_plane, int64_t split_plane_bytes, void* stream);
int64_t fl_knn_staged_workspace_bytes(int64_t nq, int64_t m, int d, int k);
int     fl_knn_staged_f32(const float* q, int64_t nq, int64_t ldq,
                          const float* db, int64_t m, int64_t ldb, int d, int k,
                          const void* plane, const void* split_plane, int64_t row_offset,
                          float* out_dist, int32_t* out_idx,
                          void* ws, int64_t ws_bytes, int32_t* status, void* stream);

/* Row-sharded databases (the reference has no sharded kNN; the closest is its multi-GPU   */
/* k-means, kmeans/large.py:35-280): fl_knn_f32 in two calls, so that the shards can share */
/* what the threshold-seeding pass found before the scoring pass runs.  k <= 16, tensor-    */
/* core mode only.                                                                          */
/*  1. fl_knn_seed_f32 builds the bf16 query plane in `ws` and writes, per query, the 32     */
/*     class maxima of a strided sample of this shard's rows to seed_cls                     */
/*     (f32 [fl_knn_seed_floats(nq)], 32 per padded query row; -inf when the shard is too    */
/*     small to sample).  It clears `status`.                                                */
/*  2. The caller takes the element-wise maximum of seed_cls over all shards (an all-reduce  */
/*     with MAX) and, once per database, the maximum over all shards of the f32 at byte       */
/*     offset fl_knn_plane_maxnorm_offset(m, d) of each shard's plane (largest row norm).     */
/*  3. fl_knn_seeded_f32, with the SAME ws (untouched in between), q, nq, d, k and plane,     */
/*     scores this shard from thresholds derived from the combined maxima: k + 6 rows of the  */
/*     whole database are known to reach them, and they are lowered by twice the scoring     */
/*     error bound, so a row this shard leaves out cannot be one of the database's k         */
/*     nearest.  A shard may therefore return fewer than k rows (padded +inf / -1); merging  */
/*     all shards' lists with fl_topk_merge_f32 gives the exact result.  Rows that can be     */
/*     neither proven nor ruled out are recomputed exactly, as in fl_knn_f32; status is not   */
/*     cleared, so an error of step 1 stays visible.                                          */
int64_t fl_knn_seed_floats(int64_t nq);
int     fl_knn_seed_f32(const float* q, int64_t nq, int64_t ldq, int d, int k,
                        const void* plane, int64_t m, float* seed_cls,
                        void* ws, int64_t ws_bytes, int32_t* status, void* stream);
int64_t fl_knn_plane_maxnorm_offset(int64_t m, int d);
int     fl_knn_seeded_f32(const float* q, int64_t nq, int64_t ldq,
                          const float* db, int64_t m, int64_t ldb, int d, int k,
                          const void* plane, int64_t row_offset,
                          const float* seed_cls, const float* global_maxnorm,
                          float* out_dist, int32_t* out_idx,
                          void* ws, int64_t ws_bytes, int32_t* status, void* stream);

/* Test hook without a counterpart in the reference: experiment flags of the tensor-core  */
/* scoring kernel (bit values 1..16 leave work out for timing runs and mark the status     */
/* words FL_EUNSUPPORTED; 32 makes the producer skip one operand load so that a wait runs   */
/* out) and the limit of its barrier waits in microseconds (0 = the default 2 s).           */
/* (0, 0) restores normal operation.  Process-wide; not for concurrent use.                 */
int     fl_debug_tc_experiment(int flags, unsigned wait_us);

/* Test hook without a counterpart in the reference: runs only the tensor-core scoring    */
/* pass for nq <= 128 queries and writes scores[i][j] = <q_i, x_j> - ||x_j||^2/2 (bf16      */
/* products, fp32 accumulation) for every database row j; ld_scores >= m rounded up to 256. */
/* ws is sized by fl_knn_workspace_bytes(nq, m, d, 10, FL_KNN_BF16_RERANK).                 */
int     fl_debug_knn_tc_scores(const float* q, int64_t nq, int64_t ldq, int d, const void* plane,
                               int64_t m, float* scores, int64_t ld_scores,
                               void* ws, int64_t ws_bytes, int32_t* status, void* stream);

/* Debug aid without a counterpart in the reference: per-CTA cycle counters of the last   */
/* tensor-core kNN launch (16 x uint64 for each of up to 160 CTAs: waits of the producer, */
/* MMA and epilogue roles, slow-path and compaction counts, kernel cycles, tiles).          */
int     fl_debug_tc_prof_read(unsigned long long* host_out, int words);

/* Which mode FL_KNN_AUTO resolves to for a shape (no device work). */
int     fl_knn_resolve_mode(int64_t nq, int64_t m, int d, int k);

/* ---------------------------------------------------------------------------------- */
/* k-way merge of per-shard candidates (the reference has no sharded kNN; within one    */
/* GPU its split merge is torch.topk, knn/triton/dispatch.py:987-994).                  */
/* cand_dist/cand_idx [nq][ncand]; picks the k smallest (dist, idx) per row, ascending. */
/* Entries with idx < 0 are ignored.                                                    */
int fl_topk_merge_f32(const float* cand_dist, const int32_t* cand_idx, int64_t nq, int ncand,
                      int k, float* out_dist, int32_t* out_idx, void* stream);

/* Exchange format of the row-sharded kNN (no counterpart in the reference).              */
/* fl_knn_pack_f32 writes this rank's (nq, k) candidates as int32 messages, laid end to   */
/* end in `out` (fl_knn_pack_ints elements): owner != 0 -> one message per destination    */
/* rank r holding the query rows [r*base + min(r, rem), ...) of an even split of nq over  */
/* `world` ranks (the first nq % world ranks get one more); owner == 0 -> one message     */
/* with all rows.  A message is rows x [k distance bit patterns | k row ids] followed by  */
/* the FL_STATUS_WORDS status words of the call that produced the candidates (zeros when   */
/* status is NULL).  fl_knn_merge_packed_f32 takes `world` received messages of `rows`     */
/* rows each, stored back to back, and writes the k best (distance, id) per row, ascending */
/* (ids < 0 are padding), plus the folded status: first error word in sender order, sum   */
/* of the fallback counts.                                                                */
int64_t fl_knn_pack_ints(int64_t nq, int k, int world, int owner);
int     fl_knn_pack_f32(const float* dist, const int32_t* idx, int64_t nq, int k, int world, int owner,
                        const int32_t* status, int32_t* out, void* stream);
int     fl_knn_merge_packed_f32(const int32_t* msgs, int64_t rows, int k, int world,
                                float* out_dist, int32_t* out_idx, int32_t* status, void* stream);
/* fp32 -> bf16 rounded toward -inf and back: halves the bytes of the seeding maxima that  */
/* the shards exchange; a threshold rounded down stays valid.                              */
int     fl_f32_to_bf16_down(const float* in, void* out, int64_t n, void* stream);
int     fl_bf16_to_f32(const void* in, float* out, int64_t n, void* stream);

/* ---------------------------------------------------------------------------------- */
/* Exact gather distances.  Replaces triton_knn_gather_sqdist                           */
/* (kernels/distance/triton/knn_gather_l2sq.py:173-229):                                */
/* out[i][j] = sum_d (x[i][d] - c[idx[i][j]][d])^2 ; idx < 0 gives +inf.               */
/* idx_is_i64 selects int64 or int32 index elements.                                    */
int fl_gather_l2sq_f32(const float* x, int64_t n, int64_t ldx,
                       const float* c, int64_t m, int64_t ldc, int d,
                       const void* idx, int idx_is_i64, int k, float* out, void* stream);

/* ---------------------------------------------------------------------------------- */
/* k-means.  Replaces euclid_assign_triton (kmeans/triton/assign.py:1439-1596),         */
/* triton_centroid_update_sorted_euclid / _centroid_update_chunk_kernel                 */
/* (kmeans/triton/update.py:179-259,313-384), triton_centroid_finalize                  */
/* (update.py:406-554) and the Blackwell assign kernels                                 */
/* (kmeans/cutedsl/blackwell_assign.py:77-2289).                                        */
/*                                                                                      */
/* labels[i] = argmin_j ||x_i - c_j||^2 (lowest j on exact ties), int32.                */
int64_t fl_kmeans_assign_workspace_bytes(int64_t n, int K, int d);
int     fl_kmeans_assign_f32(const float* x, int64_t n, int64_t ldx,
                             const float* c, int K, int64_t ldc, int d,
                             int32_t* labels, void* ws, int64_t ws_bytes, void* stream);
/* Tensor-core assignment (tcgen05 bf16 candidates, exact fp32 re-score, proven or recomputed */
/* on the exact path; d <= 256).  Replaces the Blackwell assign kernels of                    */
/* kmeans/cutedsl/blackwell_assign.py:77-2289 for fp32 inputs.  `xplane` is the bf16 operand   */
/* plane of the sample rows followed by their squared norms, built once per data set by       */
/* fl_kmeans_prepare_x_f32 (NULL: both are built in the workspace on every call).  Labels are  */
/* identical to fl_kmeans_assign_f32's.                                                       */
int64_t fl_kmeans_xplane_bytes(int64_t n, int d);
int     fl_kmeans_prepare_x_f32(const float* x, int64_t n, int d, int64_t ldx,
                                void* xplane, int64_t xplane_bytes, void* stream);
int64_t fl_kmeans_assign_tc_workspace_bytes(int64_t n, int K, int d, int have_xplane);
int     fl_kmeans_assign_tc_f32(const float* x, int64_t n, int64_t ldx, const void* xplane,
                                const float* c, int K, int64_t ldc, int d, int32_t* labels,
                                void* ws, int64_t ws_bytes, int32_t* status, void* stream);
/* Same assignment for callers that cannot allocate device memory or pass a workspace (a  */
/* plugin that only receives a stream and its buffers, a host whose memory pool owns the   */
/* whole GPU, a loop that must avoid cudaMalloc's synchronisation).  It has no counterpart */
/* in the reference.  The half norms go to a 64 KiB array built into the library image     */
/* (resident on every GPU that loads the library until exit), so K is limited to           */
/* FL_KMEANS_NOALLOC_MAX_K (larger K returns FL_EUNSUPPORTED) and the call never runs       */
/* cudaMalloc/cudaFree.  The first call on a device looks the array's address up; make it  */
/* before any stream capture.  All calls on a device share the array: calls that overlap   */
/* on the GPU race and must be serialised by the caller.                                   */
#define FL_KMEANS_NOALLOC_MAX_K 16384
int     fl_kmeans_assign_noalloc_f32(const float* x, int64_t n, int64_t ldx,
                                     const float* c, int K, int64_t ldc, int d,
                                     int32_t* labels, void* stream);
/* sums [K][d] fp32 and cnts [K] int32 are overwritten with the per-cluster sums/counts. */
int     fl_kmeans_update_f32(const float* x, int64_t n, int64_t ldx, int d,
                             const int32_t* labels, int K,
                             float* sums, int32_t* cnts, void* stream);
/* Incremental form for the Lloyd loop (no counterpart in the reference, which re-reads x    */
/* every iteration, kmeans/triton/update.py:313-384): sums / cnts hold the result for the   */
/* labels in prev_labels [n]; the rows of the points whose label changed are moved from the */
/* old cluster's sum to the new one's, and prev_labels is brought up to date.  Same sums up */
/* to fp32 rounding; a caller refreshes them with fl_kmeans_update_f32 now and then.        */
int     fl_kmeans_update_delta_f32(const float* x, int64_t n, int64_t ldx, int d,
                                   const int32_t* labels, int32_t* prev_labels, int K,
                                   float* sums, int32_t* cnts, void* stream);
/* Batched forms for many small problems at once (the reference's kernels take the batch  */
/* on a grid axis, kmeans/triton/assign.py:1028-1129; its IVF-PQ build runs B = m           */
/* sub-quantisers of 2-8 features each, ivf_pq/triton/build.py:41-70): `batch` problems of  */
/* n rows and K centroids each in one launch.  x is [batch][n][ldx] with x_batch_stride      */
/* elements between items, c [batch][K][ldc] back to back, labels [batch][n], sums           */
/* [batch][K][d], cnts [batch][K].  The exact CUDA-core kernels; results per item are those  */
/* of the single-problem entry points.  fl_kmeans_finalize_f32 serves a batch as K * batch   */
/* centroids (the arrays are contiguous).                                                   */
int64_t fl_kmeans_assign_batch_workspace_bytes(int batch, int64_t n, int K, int d);
int     fl_kmeans_assign_batch_f32(const float* x, int batch, int64_t n, int64_t ldx, int64_t x_batch_stride,
                                   const float* c, int K, int64_t ldc, int64_t c_batch_stride, int d,
                                   int32_t* labels, void* ws, int64_t ws_bytes, void* stream);
int     fl_kmeans_update_batch_f32(const float* x, int batch, int64_t n, int64_t ldx, int d,
                                   const int32_t* labels, int K,
                                   float* sums, int32_t* cnts, void* stream);
/* new_c = cnt ? sums/cnt : old_c ; shift[j] = ||new_c[j] - old_c[j]||_2.               */
int     fl_kmeans_finalize_f32(const float* sums, const int32_t* cnts, const float* old_c,
                               float* new_c, float* shift, int K, int d, void* stream);

/* ---------------------------------------------------------------------------------- */
/* IVF-Flat fine scan.  Replaces ivf_fine_scan_gemm + _ivf_fine_gemm_kernel             */
/* (ivf_flat/triton/fine_scan_gemm.py:41-272) and ivf_fine_scan                         */
/* (ivf_flat/triton/fine_scan.py:44-235).                                               */
/* data [m][ldd] is cell-contiguous; list c owns rows list_offsets[c]..list_offsets[c+1]*/
/* (int64[nlist+1]).  probed [nq][nprobe] int32 list ids.  out_dist [nq][k] exact       */
/* squared L2 ascending, out_pos [nq][k] int32 stored-row positions; rows with fewer    */
/* than k candidates are padded with +inf / -1.  data_hnorm is ||row||^2/2 per stored    */
/* row (fp32 [m]; what fl_rownorm_f32 returns, halved) or NULL to have it computed in    */
/* the workspace on every call.                                                         */
int64_t fl_ivf_fine_scan_workspace_bytes(int64_t nq, int nprobe, int nlist, int64_t m, int d, int k);
int     fl_ivf_fine_scan_f32(const float* q, int64_t nq, int64_t ldq,
                             const float* data, int64_t m, int64_t ldd, int d,
                             const int64_t* list_offsets, int nlist,
                             const int32_t* probed, int nprobe, int k,
                             const float* data_hnorm,
                             float* out_dist, int32_t* out_pos,
                             void* ws, int64_t ws_bytes, void* stream);

/* Cell-contiguous index layout from per-row list labels.  Replaces the torch glue of      */
/* ivf_flat_build_triton (ivf_flat/triton/build.py:59-95: bincount, cumsum, stable argsort,  */
/* index_select, .item()) with device work and no host synchronisation.                     */
/* labels [m] int32 in [0, nlist) (what fl_kmeans_assign_* returns for the coarse centroids).*/
/* data [m][d] receives the rows grouped by list, rows of one list in their original order   */
/* (a stable partition); ids [m] int64 the original row of every stored row; list_offsets   */
/* [nlist+1] int64 the exclusive scan of the list lengths; *max_list_len (device int32, may  */
/* be NULL) the longest list.                                                               */
int64_t fl_ivf_build_workspace_bytes(int64_t m, int nlist);
int     fl_ivf_build_csr_f32(const float* x, int64_t m, int64_t ldx, int d,
                             const int32_t* labels, int nlist,
                             float* data, int64_t* ids, int64_t* list_offsets, int32_t* max_list_len,
                             void* ws, int64_t ws_bytes, void* stream);
/* Stored positions (the fine scans' out_pos, -1 padded) to the caller's row ids: out[i] =  */
/* pos[i] >= 0 ? ids[pos[i]] : -1, the last line of the reference's search                  */
/* (ivf_flat/triton/search.py:104-107).                                                     */
int     fl_ivf_map_ids(const int32_t* pos, const int64_t* ids, int64_t n, int64_t m,
                       int64_t* out, void* stream);

/* The same fine scan on the tensor cores (k <= 16, d <= 256), the counterpart of the     */
/* reference's GEMM variant (ivf_flat/triton/fine_scan_gemm.py:41-272).                   */
/* fl_ivf_prepare_f32 builds, once per index, the bf16 operand plane of the stored rows    */
/* (every list padded to whole 256-row tiles) and the map back to stored rows, in a         */
/* caller buffer of fl_ivf_plane_bytes bytes.  fl_ivf_fine_scan_tc_f32 has the contract of  */
/* fl_ivf_fine_scan_f32 (same outputs, bit-for-bit the same distances for proven rows):     */
/* candidates come from bf16 scoring and are re-scored exactly; a query whose result       */
/* cannot be proven against the scoring error bound is recomputed by an exact scan of its   */
/* probed lists (status[FL_STATUS_FALLBACK] counts them).  Workspace size 0 = unsupported.  */
int64_t fl_ivf_plane_bytes(int64_t m, int nlist, int d);
int     fl_ivf_prepare_f32(const float* data, int64_t m, int64_t ldd, int d,
                           const int64_t* list_offsets, int nlist,
                           void* plane, int64_t plane_bytes, void* stream);
int64_t fl_ivf_fine_scan_tc_workspace_bytes(int64_t nq, int nprobe, int nlist, int64_t m, int d, int k);
int     fl_ivf_fine_scan_tc_f32(const float* q, int64_t nq, int64_t ldq,
                                const float* data, int64_t m, int64_t ldd, int d,
                                const int64_t* list_offsets, int nlist,
                                const int32_t* probed, int nprobe, int k,
                                const void* ivf_plane,
                                float* out_dist, int32_t* out_pos,
                                void* ws, int64_t ws_bytes, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHLIB_B200_H_ */
