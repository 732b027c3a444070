// placeholder until the tcgen05 kernel lands
#include "common.cuh"
bool talos_gemm_tc_launch(talos_ctx*, int, int, int64_t, int64_t, int64_t, const float*, int64_t, const float*, int64_t,
                          float*, int64_t, int, const EpiArgs&) { return false; }
void talos_gemm_tc_release(talos_ctx*) {}
