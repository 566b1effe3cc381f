// Prefill GEMM placeholder translation unit (filled in by the tcgen05 kernel).
#include "lbk_internal.cuh"

namespace lbk {

int gemm_init(Ctx *) { return LBK_OK; }

int launch_gemm(Ctx *, const GroupArgs &g, cudaStream_t) {
    return fail(LBK_ERR_UNSUPPORTED, "m = %zu token rows: the prefill GEMM kernel is not built yet", g.m);
}

}  // namespace lbk
