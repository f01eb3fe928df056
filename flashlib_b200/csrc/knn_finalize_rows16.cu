// Pool finalisation for 16-bit rows (bf16 / fp16, widened on load) and for batches of small problems:
// the same templates as knn_finalize.cu, instantiated in a translation unit of their own so that the
// two compile side by side.
#include "knn_finalize.cuh"

namespace fl {

int launch_finalize_rows16(const FinalizeParams& p, unsigned grid, bool indirect, bool dyn, cudaStream_t st) {
    return launch_finalize_rows<false>(p, grid, indirect, dyn, st);
}

int launch_finalize_batch(const FinalizeParams& p, dim3 grid, cudaStream_t st) {
    switch (p.K1 / 32) {
        case 1: knn_finalize_batch_kernel<1><<<grid, 128, 0, st>>>(p); break;
        case 2: knn_finalize_batch_kernel<2><<<grid, 128, 0, st>>>(p); break;
        case 4: knn_finalize_batch_kernel<4><<<grid, 128, 0, st>>>(p); break;
        case 8: knn_finalize_batch_kernel<8><<<grid, 128, 0, st>>>(p); break;
        case 16: knn_finalize_batch_kernel<16><<<grid, 128, 0, st>>>(p); break;
        default: set_error("unsupported pool size %d", p.K1); return FL_EUNSUPPORTED;
    }
    FL_CHECK_LAUNCH();
    return FL_OK;
}

}  // namespace fl
