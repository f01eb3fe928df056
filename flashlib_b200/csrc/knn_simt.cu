// Exact CUDA-core kNN scoring pass (the pools it publishes are finalised in knn_finalize.cu).
#include "knn_internal.h"
#include "pool.cuh"
#include "simt_tile.cuh"

namespace fl {

// ------------------------------------------------------------------------------------
// Scoring pass.  grid = (ceil(slots / BQ), nsplit).  Each block keeps BQ query rows,
// streams its split of the database in tiles of 128 rows, scores every pair with
// score = <q,x> - ||x||^2/2 in fp32 FFMA and feeds the per-row pools.
// ------------------------------------------------------------------------------------
// One block's work: virtual block (vbx, vby) of the launch geometry described above.
template <int TQ>
__device__ __forceinline__ void knn_simt_block(const SimtKnnParams& p, const int vbx, const int vby, float* smem) {
    using T = SimtTile<TQ>;
    constexpr int BQ = T::BQ;
    constexpr int SSTR = 129;
    float* slab = smem;
    float* pool_sc = smem + T::SLAB_FLOATS;
    uint32_t* pool_id = reinterpret_cast<uint32_t*>(pool_sc + BQ * p.cap);
    float* tau = reinterpret_cast<float*>(pool_id + BQ * p.cap);
    int* cnt = reinterpret_cast<int*>(tau + BQ);
    int* qmap = cnt + BQ;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int tx = tid & 15, ty = tid >> 4;
    int* pslot = qmap + BQ;
    int64_t slot0, row_begin, row_end;
    int split;
    int nsplit = p.nsplit;
    if (p.ivf) {
        const int b = vbx;
        if (b >= p.item_off[p.nlist]) return;
        int lo = 0, hi = p.nlist;  // largest c with item_off[c] <= b
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.item_off[mid] <= b) lo = mid; else hi = mid;
        }
        const int c = lo;
        const int s0 = p.pair_off[c] + (b - p.item_off[c]) * BQ;
        const int s1 = min(s0 + BQ, p.pair_off[c + 1]);
        row_begin = p.list_offsets[c];
        row_end = p.list_offsets[c + 1];
        slot0 = 0;
        split = 0;
        for (int i = tid; i < BQ; i += 256) {
            const int pr = (s0 + i < s1) ? p.sorted_pair[s0 + i] : -1;
            pslot[i] = pr;
            qmap[i] = pr >= 0 ? pr / p.nprobe : -1;
            tau[i] = (pr >= 0 && p.tau_q != nullptr) ? __ldcg(p.tau_q + pr / p.nprobe) : neg_inf();
            cnt[i] = 0;
        }
    } else {
        const int64_t count = p.count_dev ? (int64_t)(*p.count_dev) : p.count;
        int64_t rps = p.rows_per_split;
        if (p.dyn_blocks > 0) {
            if (count <= 0) return;
            const SimtDynSplit ds = simt_dyn_split(count, BQ, p.dyn_blocks, p.m);
            nsplit = ds.nsplit;
            rps = ds.rows_per_split;
            const int64_t nqb = (count + BQ - 1) / BQ;
            slot0 = ((int64_t)vbx % nqb) * BQ;
            split = (int)((int64_t)vbx / nqb);
            if (split >= nsplit) return;
        } else {
            slot0 = (int64_t)vbx * BQ;
            if (slot0 >= count) return;
            split = vby;
        }
        row_begin = (int64_t)split * rps;
        row_end = min(p.m, row_begin + rps);
        for (int i = tid; i < BQ; i += 256) {
            const int64_t slot = slot0 + i;
            qmap[i] = slot < count ? (p.qlist ? p.qlist[slot] : (int)slot) : -1;
            pslot[i] = 0;
            tau[i] = neg_inf();
            cnt[i] = 0;
        }
    }
    __syncthreads();

    const void* qrow[T::QL];
#pragma unroll
    for (int i = 0; i < T::QL; ++i) {
        const int r = (i * 256 + tid) >> 3;
        qrow[i] = (r < BQ && qmap[r] >= 0) ? row_at(p.q, qmap[r], p.ldq, p.dt) : nullptr;
    }

    constexpr int RPW = BQ / 8;  // rows per warp in the pool phase
    const int keep = p.keep > 0 ? p.keep : p.K1;
    for (int64_t tile_row = row_begin; tile_row < row_end; tile_row += 128) {
        const void* drow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t gr = tile_row + ((i * 256 + tid) >> 3);
            drow[i] = gr < row_end ? row_at(p.db, gr, p.ldb, p.dt) : nullptr;
        }
        float acc[TQ][8];
        simt_cross_tile<TQ>(qrow, drow, p.d, p.vecq != 0, p.vecd != 0, slab, acc, p.dt, p.dt);

        // Scores into the tile buffer (it aliases the operand slabs, which are idle now).
        float* S = slab;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = (j < 4) ? (tx * 4 + j) : (64 + tx * 4 + (j - 4));
            const int64_t gr = tile_row + col;
            const float hv = gr < row_end ? __ldg(p.hnorm + gr) : pos_inf();
#pragma unroll
            for (int i = 0; i < TQ; ++i) S[(ty * TQ + i) * SSTR + col] = acc[i][j] - hv;
        }
        __syncthreads();

#pragma unroll 1
        for (int rr = 0; rr < RPW; ++rr) {
            const int row = warp * RPW + rr;
            if (qmap[row] < 0) continue;
            float t = tau[row];
            int c = cnt[row];
            float* sc = pool_sc + row * p.cap;
            uint32_t* idp = pool_id + row * p.cap;
#pragma unroll
            for (int sub = 0; sub < 4; ++sub) {
                const float s = S[row * SSTR + sub * 32 + lane];
                const bool pass = s > t;
                const unsigned mask = __ballot_sync(FULL_MASK, pass);
                if (mask) {
                    if (pass) {
                        const int pos = c + __popc(mask & ((1u << lane) - 1u));
                        sc[pos] = s;
                        idp[pos] = (uint32_t)(tile_row + sub * 32 + lane);
                    }
                    c += __popc(mask);
                    if (c > p.cap - 32) {
                        __syncwarp();
                        t = pool_compact_dyn(sc, idp, c, keep, p.npl);
                        c = min(c, keep);
                    }
                }
            }
            if (lane == 0) { tau[row] = t; cnt[row] = c; }
        }
        __syncthreads();
    }

#pragma unroll 1
    for (int rr = 0; rr < RPW; ++rr) {
        const int row = warp * RPW + rr;
        if (qmap[row] < 0) continue;
        float* sc = pool_sc + row * p.cap;
        uint32_t* idp = pool_id + row * p.cap;
        __syncwarp();
        pool_compact_dyn(sc, idp, cnt[row], p.K1, p.npl);
        // tau[row] came from the shared threshold or from a compaction of this pool (keep-th
        // best of rows this query probes): both hold for the query's other lists too
        if (p.ivf && p.tau_q != nullptr && lane == 0 && tau[row] > neg_inf()) atomic_max_f32(p.tau_q + qmap[row], tau[row]);
        const int64_t o = p.ivf ? (int64_t)pslot[row] * p.K1
                                : ((slot0 + row) * nsplit + split) * (int64_t)p.K1;
        for (int e = lane; e < p.K1; e += 32) {
            p.part_sc[o + e] = sc[e];
            p.part_id[o + e] = idp[e];
        }
    }
}

// The kernel proper.  Static geometries: one virtual block per block.  Dynamic mode (slot count on
// the device): the launch has a fixed, modest number of blocks and each walks the virtual blocks
// that the live slot count calls for -- a grid sized for the largest possible count would spend
// most of its time launching blocks that find nothing to do.
template <int TQ>
__global__ void __launch_bounds__(256) knn_simt_kernel(SimtKnnParams p) {
    extern __shared__ __align__(16) float smem[];
    if (p.dyn_blocks <= 0 || p.ivf) {
        knn_simt_block<TQ>(p, blockIdx.x, blockIdx.y, smem);
        return;
    }
    const int64_t count = p.count_dev ? (int64_t)(*p.count_dev) : p.count;
    if (count <= 0) return;
    const int64_t nqb = (count + SimtTile<TQ>::BQ - 1) / SimtTile<TQ>::BQ;
    const int64_t live = nqb * simt_dyn_split(count, SimtTile<TQ>::BQ, p.dyn_blocks, p.m).nsplit;
    for (int64_t vb = blockIdx.x; vb < live; vb += gridDim.x) {
        knn_simt_block<TQ>(p, (int)vb, 0, smem);
        __syncthreads();
    }
}

// Batch of independent problems of one shape (static geometry): problem blockIdx.z runs the same
// code on shifted operands and pools.
template <int TQ>
__global__ void __launch_bounds__(256) knn_simt_batch_kernel(SimtKnnParams p) {
    extern __shared__ __align__(16) float smem[];
    const int64_t b = blockIdx.z;
    p.q = static_cast<const char*>(p.q) + b * p.q_bstride * dt_size_dev(p.dt);
    p.db = static_cast<const char*>(p.db) + b * p.db_bstride * dt_size_dev(p.dt);
    p.hnorm += b * p.m;
    const int64_t pools = p.count * p.nsplit * (int64_t)p.K1;
    p.part_sc += b * pools;
    p.part_id += b * pools;
    knn_simt_block<TQ>(p, blockIdx.x, blockIdx.y, smem);
}

template <int TQ>
static size_t simt_smem_bytes(int cap) {
    using T = SimtTile<TQ>;
    return sizeof(float) * ((size_t)T::SLAB_FLOATS + (size_t)T::BQ * cap * 2 + (size_t)T::BQ * 4);
}

static int simt_pick_tq(int cap) {
    const size_t lim = (size_t)smem_optin_bytes() - 1024;
    if (simt_smem_bytes<4>(cap) <= lim) return 4;
    if (simt_smem_bytes<2>(cap) <= lim) return 2;
    if (simt_smem_bytes<1>(cap) <= lim) return 1;
    return 0;
}

int simt_block_queries(int K1) { return 16 * simt_pick_tq(simt_pool_cap(K1)); }

void simt_split_plan(int64_t slots, int64_t m, int K1, int d, int* nsplit, int64_t* rows_per_split) {
    (void)d;
    const int tq = simt_pick_tq(simt_pool_cap(K1));
    const int bq = 16 * (tq > 0 ? tq : 1);
    const int64_t qblocks = ceil_div(slots > 0 ? slots : 1, bq);
    const int64_t tiles = ceil_div(m, 128);
    int64_t want = ceil_div(2 * (int64_t)sm_count(), qblocks);
    int64_t max_split = tiles / 4 > 0 ? tiles / 4 : 1;
    if (want > max_split) want = max_split;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    int64_t rps = round_up(ceil_div(m, want), 128);
    *rows_per_split = rps;
    *nsplit = (int)ceil_div(m, rps);
}

template <int TQ>
static int launch_simt_t(const SimtKnnParams& p, int64_t max_slots, cudaStream_t st) {
    const size_t smem = simt_smem_bytes<TQ>(p.cap);
    FL_CHECK_CUDA(cudaFuncSetAttribute(knn_simt_kernel<TQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
    dim3 grid(p.ivf ? (unsigned)max_slots : (unsigned)ceil_div(max_slots, SimtTile<TQ>::BQ),
              (unsigned)p.nsplit, (unsigned)(p.batch > 1 ? p.batch : 1));
    if (p.batch > 1 && (p.ivf || p.dyn_blocks > 0 || p.count_dev != nullptr || p.qlist != nullptr || p.batch > 65535)) {
        set_error("batched CUDA-core scan: static geometry only, at most 65535 problems");
        return FL_EINVAL;
    }
    if (p.dyn_blocks > 0) {
        if (p.ivf || p.dyn_bq != SimtTile<TQ>::BQ || p.count_dev == nullptr) {
            set_error("dynamic split: plan made for %d queries per block, kernel uses %d", p.dyn_bq, SimtTile<TQ>::BQ);
            return FL_EINVAL;
        }
        // (p.dyn_blocks stays the figure the range split and the pool storage are planned with)
        const int launched = 4 * sm_count();
        grid = dim3((unsigned)(p.dyn_blocks < launched ? p.dyn_blocks : launched), 1);
    }
    if (p.batch > 1) {
        FL_CHECK_CUDA(cudaFuncSetAttribute(knn_simt_batch_kernel<TQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        knn_simt_batch_kernel<TQ><<<grid, 256, smem, st>>>(p);
        FL_CHECK_LAUNCH();
        return FL_OK;
    }
    knn_simt_kernel<TQ><<<grid, 256, smem, st>>>(p);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

int launch_knn_simt(const SimtKnnParams& p, int64_t max_slots, cudaStream_t st) {
    if (max_slots <= 0) return FL_OK;
    const int tq = simt_pick_tq(p.cap);
    if (tq == 0) {
        set_error("kNN pool of %d entries per row does not fit shared memory", p.cap);
        return FL_EUNSUPPORTED;
    }
    if (p.ivf && p.bq_items != 16 * tq) {
        set_error("inverted-file item table built for %d queries per block, kernel uses %d", p.bq_items, 16 * tq);
        return FL_EINVAL;
    }
    if (tq == 4) return launch_simt_t<4>(p, max_slots, st);
    if (tq == 2) return launch_simt_t<2>(p, max_slots, st);
    return launch_simt_t<1>(p, max_slots, st);
}

}  // namespace fl
