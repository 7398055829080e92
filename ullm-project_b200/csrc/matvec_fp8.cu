// FP8 instantiations of the decode matvec (kernels and design notes: matvec_impl.cuh).
#include "matvec_impl.cuh"

namespace ullm {
cudaError_t launch_matvec_fp8(const Context *ctx, cudaStream_t stream, const MatvecLaunch &l) {
  return matvec_impl::launch_enc<ULLM_CUDA_ENCODING_FP8_CHANNEL>(ctx, stream, l.p, l.m);
}
}  // namespace ullm
