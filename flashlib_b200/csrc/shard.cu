// Exchange format of the row-sharded kNN: every rank packs its (nq, k) candidates into one int32
// message per destination rank -- distance bits, row ids and the call's status words -- and the
// receiving side picks the k best of world x k candidates per query straight from the received
// messages.  One kernel each way; the collective in between (NCCL all-to-all or all-gather) is
// the caller's.
#include "knn_internal.h"
#include "pool.cuh"

namespace fl {

// Rows [start, end) of `rank` when n rows are dealt to `world` ranks contiguously, the first
// n % world ranks holding one more.
__host__ __device__ inline void shard_rows(int64_t n, int world, int rank, int64_t* start, int64_t* end) {
    const int64_t base = n / world, rem = n % world;
    const int64_t s = rank * base + (rank < rem ? rank : rem);
    *start = s;
    *end = s + base + (rank < rem ? 1 : 0);
}

// Message for destination r (owner form): the rows shard_rows(nq, world, r) of
// [k distance bits | k row ids], then FL_STATUS_WORDS status words.  Messages are laid end to end.
// Replicated form (owner == 0): one message with all nq rows and one status block.
__global__ void knn_pack_kernel(const float* __restrict__ dist, const int32_t* __restrict__ idx, int64_t nq, int k,
                                int world, int owner, const int32_t* __restrict__ status, int32_t* __restrict__ out) {
    const int64_t total = nq * 2 * k;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int nmsg = owner ? world : 1;
    if (i < total) {
        const int64_t row = i / (2 * k);
        const int c = (int)(i - row * 2 * k);
        int dest = 0;
        if (owner) {
            // destination of this row: invert shard_rows
            const int64_t base = nq / world, rem = nq % world;
            const int64_t cut = rem * (base + 1);
            dest = row < cut ? (int)(row / (base + 1)) : (int)(rem + (base > 0 ? (row - cut) / base : 0));
        }
        const int32_t v = c < k ? __float_as_int(dist[row * k + c]) : idx[row * k + (c - k)];
        out[i + (int64_t)dest * FL_STATUS_WORDS] = v;
    } else if (i < total + (int64_t)nmsg * FL_STATUS_WORDS) {
        const int64_t j = i - total;
        const int msg = (int)(j / FL_STATUS_WORDS), w = (int)(j % FL_STATUS_WORDS);
        int64_t s = 0, e = nq;
        if (owner) shard_rows(nq, world, msg, &s, &e);
        out[e * 2 * k + (int64_t)msg * FL_STATUS_WORDS + w] = status ? status[w] : 0;
    }
}

// One warp per query row: streams that row's world x k candidates out of the `world` received
// messages (each `rows` x [k bits | k ids] + status words, `msg_stride` int32 apart) and keeps the
// k best (distance, id).  Thread 0 of block 0 folds the senders' status words: the first error
// word met (senders in rank order) and the sum of the fallback counts.
template <int NPL1>
__global__ void __launch_bounds__(128) knn_merge_packed_kernel(const int32_t* __restrict__ in, int64_t rows, int k,
                                                               int world, int64_t msg_stride, float* __restrict__ od,
                                                               int32_t* __restrict__ oi, int32_t* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (blockIdx.x == 0 && threadIdx.x == 0 && status != nullptr) {
        int err = 0, where = 0, fb = 0;
        for (int s = 0; s < world; ++s) {
            const int32_t* st = in + s * msg_stride + rows * 2 * k;
            if (err == 0 && st[FL_STATUS_ERROR] != 0) { err = st[FL_STATUS_ERROR]; where = st[FL_STATUS_WHERE]; }
            fb += st[FL_STATUS_FALLBACK];
        }
        for (int w = 0; w < FL_STATUS_WORDS; ++w) status[w] = 0;
        status[FL_STATUS_ERROR] = err;
        status[FL_STATUS_WHERE] = where;
        status[FL_STATUS_FALLBACK] = fb;
    }
    if (row >= rows) return;
    constexpr int N2 = 2 * NPL1;
    float key[N2];
    uint32_t id[N2];
#pragma unroll
    for (int r = 0; r < NPL1; ++r) { key[r] = neg_inf(); id[r] = INVALID_ID; }
    const int ncand = world * k;
    for (int base = 0; base < ncand; base += NPL1 * 32) {
#pragma unroll
        for (int r = 0; r < NPL1; ++r) {
            const int e = base + ((r << 5) | lane);
            bool ok = e < ncand;
            float dv = 0.f;
            int32_t iv = -1;
            if (ok) {
                const int s = e / k, j = e - s * k;
                const int32_t* p = in + s * msg_stride + row * 2 * k;
                dv = __int_as_float(p[j]);
                iv = p[k + j];
                ok = iv >= 0;
            }
            key[NPL1 + r] = ok ? -dv : neg_inf();
            id[NPL1 + r] = ok ? (uint32_t)iv : INVALID_ID;
        }
        warp_sort_desc<N2, true>(key, id);
    }
#pragma unroll
    for (int r = 0; r < NPL1; ++r) {
        const int e = (r << 5) | lane;
        if (e < k) {
            const bool ok = id[r] != INVALID_ID;
            od[row * k + e] = ok ? -key[r] : pos_inf();
            oi[row * k + e] = ok ? (int32_t)id[r] : -1;
        }
    }
}

// fp32 -> bf16 rounded toward -inf (a threshold may only get looser on the way), and back.
__global__ void f32_to_bf16_down_kernel(const float* __restrict__ in, uint16_t* __restrict__ out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t b = __float_as_uint(in[i]);
    uint32_t hi = b >> 16;
    // truncation moves toward zero: for a negative value with dropped bits step one further down
    // (-inf has no dropped bits; NaN never occurs: scores are finite or -inf)
    if ((b & 0x80000000u) && (b & 0xFFFFu)) hi += 1;
    out[i] = (uint16_t)hi;
}
__global__ void bf16_to_f32_kernel(const uint16_t* __restrict__ in, float* __restrict__ out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __uint_as_float((uint32_t)in[i] << 16);
}

}  // namespace fl

using namespace fl;

extern "C" int64_t fl_knn_pack_ints(int64_t nq, int k, int world, int owner) {
    if (nq < 0 || k < 1 || world < 1) return 0;
    return nq * 2 * k + (int64_t)(owner ? world : 1) * FL_STATUS_WORDS;
}

extern "C" int fl_knn_pack_f32(const float* dist, const int32_t* idx, int64_t nq, int k, int world, int owner,
                               const int32_t* status, int32_t* out, void* stream) {
    FL_CHECK_ARG(nq >= 0 && k >= 1 && world >= 1, "fl_knn_pack_f32: bad shape");
    FL_CHECK_ARG(out && (nq == 0 || (dist && idx)), "fl_knn_pack_f32: null pointer");
    const int64_t total = fl_knn_pack_ints(nq, k, world, owner);
    knn_pack_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, (cudaStream_t)stream>>>(dist, idx, nq, k, world, owner ? 1 : 0,
                                                                                     status, out);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_knn_merge_packed_f32(const int32_t* msgs, int64_t rows, int k, int world, float* out_dist,
                                       int32_t* out_idx, int32_t* status, void* stream) {
    FL_CHECK_ARG(rows >= 0 && k >= 1 && world >= 1, "fl_knn_merge_packed_f32: bad shape");
    if (k > 512) { set_error("fl_knn_merge_packed_f32: k=%d > 512 is not supported", k); return FL_EUNSUPPORTED; }
    FL_CHECK_ARG(msgs && (rows == 0 || (out_dist && out_idx)), "fl_knn_merge_packed_f32: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t stride = rows * 2 * k + FL_STATUS_WORDS;
    const unsigned grid = (unsigned)ceil_div(rows > 0 ? rows : 1, 4);
    const int K1 = simt_pool_size(k);
    switch (K1 / 32) {
        case 1: knn_merge_packed_kernel<1><<<grid, 128, 0, st>>>(msgs, rows, k, world, stride, out_dist, out_idx, status); break;
        case 2: knn_merge_packed_kernel<2><<<grid, 128, 0, st>>>(msgs, rows, k, world, stride, out_dist, out_idx, status); break;
        case 4: knn_merge_packed_kernel<4><<<grid, 128, 0, st>>>(msgs, rows, k, world, stride, out_dist, out_idx, status); break;
        case 8: knn_merge_packed_kernel<8><<<grid, 128, 0, st>>>(msgs, rows, k, world, stride, out_dist, out_idx, status); break;
        default: knn_merge_packed_kernel<16><<<grid, 128, 0, st>>>(msgs, rows, k, world, stride, out_dist, out_idx, status); break;
    }
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_f32_to_bf16_down(const float* in, void* out, int64_t n, void* stream) {
    FL_CHECK_ARG(n >= 0 && (n == 0 || (in && out)), "fl_f32_to_bf16_down: bad arguments");
    if (n == 0) return FL_OK;
    f32_to_bf16_down_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(in, static_cast<uint16_t*>(out), n);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_bf16_to_f32(const void* in, float* out, int64_t n, void* stream) {
    FL_CHECK_ARG(n >= 0 && (n == 0 || (in && out)), "fl_bf16_to_f32: bad arguments");
    if (n == 0) return FL_OK;
    bf16_to_f32_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(static_cast<const uint16_t*>(in), out, n);
    FL_CHECK_LAUNCH();
    return FL_OK;
}
