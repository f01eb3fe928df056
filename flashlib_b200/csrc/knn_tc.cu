// placeholder
#include "knn_internal.h"
namespace fl {
int tc_knn_supported(int64_t, int64_t, int, int) { return FL_EUNSUPPORTED; }
int tc_pool_size(int) { return 32; }
void tc_split_plan(int64_t, int64_t, int* nsplit, int64_t* tps) { *nsplit = 1; *tps = 1; }
int launch_knn_tc(const TcKnnParams&, cudaStream_t) { set_error("tc kernel not built"); return FL_EUNSUPPORTED; }
}
