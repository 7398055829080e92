// Host side of the decode matvec: shape support and dispatch to the per-encoding translation units
// (the kernels live in matvec_impl.cuh; see that file for the design).
#include "matvec_impl.cuh"

namespace ullm {

using namespace matvec_impl;

bool matvec_supports(const LinearArgs &a, const char **why) {
  if (a.m < 1 || a.m > 8) {
    *why = "the matvec kernel serves 1 <= M <= 8";
    return false;
  }
  const uint32_t kp = pad_k(a.k, a.encoding);
  if (smem_bytes(a.m, kp, a.encoding) > kSmemBudget) {
    *why = "M*K activations do not fit the matvec kernel's shared-memory staging";
    return false;
  }
  return true;
}

int launch_matvec(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err) {
  Params p;
  p.x = a.x;
  p.y = a.y;
  p.w = a.w;
  p.scales = a.scales;
  p.n = a.n;
  p.k = a.k;
  p.x_stride = a.x_stride;
  p.y_stride = a.y_stride;
  p.x_dtype = a.x_dtype;
  p.y_dtype = a.y_dtype;
  p.prologue = a.prologue;
  p.epilogue = a.epilogue;
  p.rms_eps = a.rms_eps;
  p.k_pad = pad_k(a.k, a.encoding);
  p.norm_weight = a.norm_weight;
  p.residual = a.residual;
  p.res_stride = a.res_stride;
  p.po = a.push_out;
  p.pi = a.push_in;
  p.flags = ctx->device_flags;
  p.abort_word = a.abort_word != nullptr ? a.abort_word : ctx->abort_word;
  p.wait_ns = (uint64_t)(a.wait_limit_ms != 0 ? a.wait_limit_ms : kDefaultWaitLimitMs) * 1000000ull;
  const uint64_t xe = a.x_dtype == ULLM_CUDA_DTYPE_F32 ? 4 : 2;
  const bool aligned = reinterpret_cast<uintptr_t>(a.x) % 16 == 0 && (a.x_stride * xe) % 16 == 0 &&
                       (a.k * xe) % 16 == 0 && a.k % 8 == 0;
  p.vec_ok = (a.push_in.tp != 0 || aligned) ? 1u : 0u;
  MatvecLaunch l{p, a.m};
  cudaError_t e = a.encoding == AQ4 ? launch_matvec_aq4(ctx, stream, l) : launch_matvec_fp8(ctx, stream, l);
  *err = e;
  return e == cudaSuccess ? 1 : -1;
}

}  // namespace ullm
