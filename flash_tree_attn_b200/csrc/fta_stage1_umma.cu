// Stage 1, tcgen05 family (placeholder until the TMEM kernel lands): reports itself
// unavailable so that every request runs on the warp-MMA family.
#include "fta_common.cuh"

int fta_umma_supported(const FtaParams&) { return 0; }

cudaError_t fta_launch_stage1_umma(const FtaParams&, const FtaGeom&, cudaStream_t, int, int*) {
  return cudaErrorNotSupported;
}
