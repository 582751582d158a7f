// bf16 instantiations of the weight-streaming GEMM (gemm_stream.cuh).
#include "gemm_stream.cuh"

namespace mb200 {
int launch_gemm_stream_bf16(const GemmArgs& g) { return stream::launch_dtype<__nv_bfloat16>(g); }
int read_stream_status_bf16(int* value, bool reset) { return stream::read_status(value, reset); }
}  // namespace mb200

