// placeholder replaced below by the tcgen05 evaluator
#include "frame.cuh"
namespace mlpsp {
int launch_mlp_f16(const mlpsp_scene*, const RecIn*, const int32_t*, const int2*, const int32_t*, float4*, int, int32_t*, cudaStream_t) {
  set_error("fp16 evaluator not built yet");
  return MLPSP_E_ARG;
}
}
extern "C" int64_t mlpsp_packed_weight_bytes(int32_t, int32_t) { return 0; }
extern "C" int mlpsp_pack_weights_f16(const mlpsp_scene*, void*, void*) { return MLPSP_E_ARG; }
