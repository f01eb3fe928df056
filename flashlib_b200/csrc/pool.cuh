// Per-row candidate pools: an append buffer of `cap` (score, id) entries with a
// threshold.  A row accepts a candidate only when its score beats the threshold; when
// the buffer is nearly full a warp sorts it, keeps the K1 best and raises the threshold
// to the K1-th best score.  Larger score = closer neighbour (score = <q,x> - ||x||^2/2).
#pragma once
#include "common.cuh"

namespace fl {

// Runtime-sized front end of warp_pool_compact: `npl` = capacity / 32 in {2,4,8,16,32}.
// Kept out of line: compaction is rare and the sorting networks are large.
static __device__ __noinline__ float pool_compact_dyn(float* sc, uint32_t* idv, int cnt, int K1,
                                                      int npl) {
    switch (npl) {
        case 2: return warp_pool_compact<2>(sc, idv, cnt, K1);
        case 4: return warp_pool_compact<4>(sc, idv, cnt, K1);
        case 8: return warp_pool_compact<8>(sc, idv, cnt, K1);
        case 16: return warp_pool_compact<16>(sc, idv, cnt, K1);
        default: return warp_pool_compact<32>(sc, idv, cnt, K1);
    }
}

// Pool size (a power of two >= 32) used for k neighbours on the exact CUDA-core path: room for the
// k wanted and at least 8 more, which the exact re-rank needs where fp32 scores of rows that close
// to the k-th neighbour come out in the wrong order (k > 504: what 512 entries leave).
static inline int simt_pool_size(int k) {
    int p = pow2_ceil(k + 8 < 512 ? k + 8 : 512);
    return p < 32 ? 32 : p;
}

// Pool capacity for K1 published entries: room for at least 64 appends between compactions.
static inline int simt_pool_cap(int K1) { return K1 <= 32 ? 128 : 2 * K1; }

// Entries a pool keeps at a compaction inside the scan: the k wanted plus the margin the exact
// re-rank takes (k + 8), in steps of 8.  Fewer than K1 keeps the threshold tight and leaves room
// in the pool while it is still filling.
static inline int simt_pool_keep(int K1, int k) {
    const int want = (k + 8 + 7) / 8 * 8;
    return want < K1 ? want : K1;
}

}  // namespace fl
