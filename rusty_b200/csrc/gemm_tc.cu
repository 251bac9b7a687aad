// placeholder until the tcgen05 kernel lands
#include "internal.h"
namespace rusty {
bool tc_supported(const rusty_cuda_ctx*, const QLinearArgs&) { return false; }
uint32_t tc_min_rows() { return 5; }
int launch_tc(rusty_cuda_ctx* ctx, const QLinearArgs&) { return fail(ctx, RUSTY_CUDA_ERR_UNSUPPORTED, "tcgen05 path not built"); }
}
