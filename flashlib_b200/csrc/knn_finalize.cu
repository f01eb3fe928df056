// Pool finalisation shared by both kNN modes: merge of the published pools, exact fp32 re-rank,
// top-k selection and verification against the scoring error bound.  The warp-per-slot kernels are
// templates (knn_finalize.cuh); this file instantiates them for fp32 rows, knn_finalize_rows16.cu for
// 16-bit rows and batches.
#include "knn_finalize.cuh"

namespace fl {

int launch_knn_finalize(const FinalizeParams& p, int64_t max_slots, cudaStream_t st) {
    if (max_slots <= 0) return FL_OK;
    int64_t blocks = ceil_div(max_slots, 4);
    if (p.count_dev != nullptr && blocks > (int64_t)sm_count() * 32) blocks = (int64_t)sm_count() * 32;
    const unsigned grid = (unsigned)blocks;
    const bool indirect = p.pool_row != nullptr;
    if (p.batch > 1) {
        if (p.count_dev != nullptr || p.qlist != nullptr || indirect || p.part_tau != nullptr || p.fb_count != nullptr ||
            p.dyn_blocks > 0 || p.batch > 65535) {
            set_error("batched finalisation: plain pools of a static scan only, at most 65535 problems");
            return FL_EINVAL;
        }
        return launch_finalize_batch(p, dim3((unsigned)blocks, (unsigned)p.batch), st);
    }
    if (indirect && (p.id_map == nullptr || p.K1 != 128)) {
        set_error("finalisation: pool indirection goes with an id map and 128 published entries per pool");
        return FL_EINVAL;
    }
    if (!indirect && p.id_map != nullptr) { set_error("finalisation: id map without pool indirection"); return FL_EINVAL; }
    const bool dyn = p.dyn_blocks > 0;
    if (dyn && (indirect || p.count_dev == nullptr)) { set_error("finalisation: dynamic split goes with a device-side count"); return FL_EINVAL; }
    return p.dt == DT_F32 ? launch_finalize_rows<true>(p, grid, indirect, dyn, st) : launch_finalize_rows16(p, grid, indirect, dyn, st);
}


// ------------------------------------------------------------------------------------
// Finalisation of the large-k tensor-core pools: one block per query.
//
// The scoring pass published, per (query, range, warpgroup), a pool of up to 256 (score, row)
// entries with its entry count and final threshold; every row it did not publish scored at most
// u = the largest threshold.  The block gathers the entries scoring above u (the others can
// never satisfy the proof), sorts them by score, re-scores the best BIG_RERANK with exact fp32
// sum (q - x)^2, sorts those by (distance, row) and accepts the first k when the k-th distance
// lies below qsq - 2 (bound + eps), bound = max(u, best score that was not re-scored).
// Otherwise (or when more than BIG_CAND entries survive) the query is queued for the exact path.
// ------------------------------------------------------------------------------------
constexpr int BIG_THREADS = 256, BIG_CAND = 2048, BIG_RERANK = 256, BIG_POOL = 256;

static __device__ __forceinline__ void finalize_big_slot(const FinalizeParams& p, const int64_t slot) {
    __shared__ float s_key[BIG_CAND];
    __shared__ uint32_t s_id[BIG_CAND];
    __shared__ float s_q[512];
    __shared__ float s_red[BIG_THREADS / 32];
    __shared__ int s_n;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t qi = p.qlist != nullptr ? (int64_t)p.qlist[slot] : slot;
    const void* qp = row_at(p.q, qi, p.ldq, p.dt);

    // u and ||q||^2
    float u = neg_inf(), qs = 0.f;
    for (int i = tid; i < p.ntau; i += BIG_THREADS) u = fmaxf(u, p.part_tau[slot * p.ntau + i]);
    for (int c = tid; c < p.d; c += BIG_THREADS) { const float v = ld_elem(qp, c, p.dt); s_q[c] = v; qs += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        u = fmaxf(u, __shfl_xor_sync(FULL_MASK, u, o));
        qs += __shfl_xor_sync(FULL_MASK, qs, o);
    }
    if (lane == 0) s_red[warp] = u;
    if (tid == 0) s_n = 0;
    __syncthreads();
    u = s_red[0];
#pragma unroll
    for (int w = 1; w < BIG_THREADS / 32; ++w) u = fmaxf(u, s_red[w]);
    __syncthreads();
    if (lane == 0) s_red[warp] = qs;
    __syncthreads();
    float qsq = 0.f;
#pragma unroll
    for (int w = 0; w < BIG_THREADS / 32; ++w) qsq += s_red[w];

    // Gather the survivors (score above `cut`), one pool per warp at a time.  If more than
    // BIG_CAND survive (a loose starting threshold), the BIG_CAND that were stored -- an
    // arbitrary subset -- are sorted, the cut moves up to the score at their first quarter and
    // the gather is repeated; everything below the cut is covered by `bound`.
    float cut = u;
    int total = 0;
    for (int round = 0; round < 4; ++round) {
        __syncthreads();
        if (tid == 0) s_n = 0;
        __syncthreads();
        for (int pi = warp; pi < p.ntau; pi += BIG_THREADS / 32) {
            int cnt = p.part_cnt[slot * p.ntau + pi];
            cnt = cnt < BIG_POOL ? cnt : BIG_POOL;
            const float* psc = p.part_sc + (slot * p.ntau + pi) * (int64_t)BIG_POOL;
            const uint32_t* pid = p.part_id + (slot * p.ntau + pi) * (int64_t)BIG_POOL;
            for (int e0 = 0; e0 < cnt; e0 += 32) {
                const int e = e0 + lane;
                float sc = neg_inf();
                uint32_t cid = INVALID_ID;
                if (e < cnt) { sc = psc[e]; cid = pid[e]; }
                const bool keep = sc > cut && cid < (uint32_t)p.m;
                const unsigned mask = __ballot_sync(FULL_MASK, keep);
                if (mask) {
                    int base = 0;
                    if (lane == 0) base = atomicAdd(&s_n, __popc(mask));
                    base = __shfl_sync(FULL_MASK, base, 0);
                    const int pos = base + __popc(mask & ((1u << lane) - 1u));
                    if (keep && pos < BIG_CAND) { s_key[pos] = sc; s_id[pos] = cid; }
                }
            }
        }
        __syncthreads();
        total = s_n;
        if (total <= BIG_CAND) break;
        block_sort_desc<BIG_THREADS>(s_key, s_id, BIG_CAND);
        cut = fmaxf(cut, s_key[BIG_CAND / 4 - 1]);
    }
    const bool overflow = total > BIG_CAND;
    const int n = overflow ? BIG_CAND : total;
    int P = BIG_RERANK;
    while (P < n) P <<= 1;
    for (int i = n + tid; i < P; i += BIG_THREADS) { s_key[i] = neg_inf(); s_id[i] = INVALID_ID; }
    block_sort_desc<BIG_THREADS>(s_key, s_id, P);

    // Exact distances in rounds of 64 candidates, best scores first.  After a round the walk stops
    // when k of the exact distances seen so far lie below the lower bound that the next
    // candidate's score (and the cut) puts on every row not yet re-scored; at most BIG_RERANK.
    __shared__ float s_dist[BIG_RERANK];
    const float mn = __ldg(p.maxnorm);
    const float eps = p.eps_rel * sqrtf(qsq) * mn;
    const float slack = 1e-5f * (qsq + mn * mn);
    const int n_rr = n < BIG_RERANK ? n : BIG_RERANK;
    float bound = cut;
    int done = 0;
    __syncthreads();
    for (int r0 = 0; r0 < n_rr; r0 += 64) {
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
            const int c0 = r0 + warp * 8 + h * 4;
            uint32_t cid[4];
            float a[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) { cid[t] = s_id[c0 + t]; a[t] = 0.f; }
            if (p.vec) {
                for (int c = lane * 4; c < p.d; c += 128) {
                    const float4 qv = *reinterpret_cast<const float4*>(s_q + c);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (cid[t] != INVALID_ID) {
                            const float4 xv = ld_elem4(row_at(p.db, cid[t], p.ldb, p.dt), c, p.dt);
                            const float d0 = qv.x - xv.x, d1 = qv.y - xv.y, d2 = qv.z - xv.z, d3 = qv.w - xv.w;
                            a[t] += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
                        }
                    }
                }
            } else {
                for (int c = lane; c < p.d; c += 32) {
                    const float qv = s_q[c];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (cid[t] != INVALID_ID) {
                            const float df = qv - ld_elem(row_at(p.db, cid[t], p.ldb, p.dt), c, p.dt);
                            a[t] += df * df;
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) a[t] += __shfl_xor_sync(FULL_MASK, a[t], o);
                if (lane == 0) s_dist[c0 + t] = cid[t] != INVALID_ID ? a[t] : pos_inf();
            }
        }
        done = r0 + 64;
        // everything from position `done` on scored at most s_key[done] (sorted) or the cut
        const float nxt = done < n ? s_key[done] : neg_inf();
        bound = fmaxf(cut, nxt);
        const float T = qsq - 2.f * (bound + eps) - slack;
        __syncthreads();                                   // this round's distances are written
        const int below = __syncthreads_count(tid < done && s_dist[tid] < T);
        if (done >= p.k && below >= p.k) break;
    }
    // order the re-scored candidates by (distance, row)
    __syncthreads();
    for (int i = tid; i < BIG_RERANK; i += BIG_THREADS) {
        const bool have = i < done && i < n_rr && s_id[i] != INVALID_ID;
        s_key[i] = have ? -s_dist[i] : neg_inf();
        if (!have) s_id[i] = INVALID_ID;
    }
    block_sort_desc<BIG_THREADS>(s_key, s_id, BIG_RERANK);

    for (int e = tid; e < p.k; e += BIG_THREADS) {
        const bool ok = s_id[e] != INVALID_ID;
        p.out_dist[qi * p.k + e] = ok ? -s_key[e] : pos_inf();
        p.out_idx[qi * p.k + e] = ok ? (int32_t)((int64_t)s_id[e] + p.row_offset) : -1;
    }
    if (tid == 0) {
        bool proven = !overflow;
        if (proven && bound > neg_inf()) {
            const float dk = s_id[p.k - 1] != INVALID_ID ? -s_key[p.k - 1] : pos_inf();
            proven = dk < qsq - 2.f * (bound + eps) - slack;
        }
        if (!proven) {
            bool queued = false;
            if (p.next_count != nullptr) {
                const int i = atomicAdd(p.next_count, 1);
                if (i < p.next_cap) { p.next_list[i] = (int)qi; queued = true; }
            }
            if (!queued) {
                const int i = atomicAdd(p.fb_count, 1);
                if (i < p.fb_cap) p.fb_list[i] = (int)qi;
            }
        }
    }
}

// One block per slot; with a device-side slot count (capped by p.count) the blocks of a modest grid
// stride over the live slots instead.
__global__ void __launch_bounds__(BIG_THREADS) knn_finalize_big_kernel(FinalizeParams p) {
    int64_t count = p.count;
    if (p.count_dev != nullptr) { const int64_t c = *p.count_dev; count = c < count ? c : count; }
    for (int64_t slot = blockIdx.x; slot < count; slot += gridDim.x) {
        finalize_big_slot(p, slot);
        __syncthreads();
    }
}

int launch_knn_finalize_big(const FinalizeParams& p, int64_t max_slots, cudaStream_t st) {
    if (max_slots <= 0) return FL_OK;
    FL_CHECK_ARG(p.part_cnt && p.part_tau && p.K1 == 2 * BIG_POOL && p.d <= 512 && p.k <= BIG_RERANK && p.count == max_slots,
                 "large-k finalisation: bad parameters");
    int64_t grid = max_slots;
    if (p.count_dev != nullptr && grid > (int64_t)sm_count() * 4) grid = (int64_t)sm_count() * 4;
    knn_finalize_big_kernel<<<(unsigned)grid, BIG_THREADS, 0, st>>>(p);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

}  // namespace fl
