// fp16 instantiations of the weight-streaming GEMM (gemm_stream.cuh).
#include "gemm_stream.cuh"

namespace mb200 {
int launch_gemm_stream_f16(const GemmArgs& g) { return stream::launch_dtype<__half>(g); }
int64_t gemm_stream_scratch_bytes(int64_t m, int64_t n, int64_t k) { return stream::scratch_bytes(m, n, k); }
int read_stream_status_f16(int* value, bool reset) { return stream::read_status(value, reset); }
}  // namespace mb200
