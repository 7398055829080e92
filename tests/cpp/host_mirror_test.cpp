// CPU-side check of the C++ host mirror (include/ullm_cuda.hpp): no GPU is needed, every device entry must
// answer CUDA_UNAVAILABLE here.  Prints "ok <n>" lines; exits non-zero on the first failed expectation.
#include <cstdio>
#include <cstdlib>

#include "ullm_cuda.hpp"

#include <cstring>
#include <vector>

using namespace ullm::cuda;

#define EXPECT(cond)                                                   \
  do {                                                                 \
    if (!(cond)) {                                                     \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      return 1;                                                        \
    }                                                                  \
  } while (0)

int main(int argc, char **argv) {
  const bool expect_gpu = argc > 1 && std::atoi(argv[1]) == 1;
  EXPECT(abi_version() == ULLM_CUDA_ABI_VERSION);
  const Version v = version();
  EXPECT(v.major + v.minor + v.patch < 1000);
  EXPECT(status_from_raw(4) == Status::CudaUnavailable);
  EXPECT(status_from_raw(16) == Status::DeviceFlagged);
  EXPECT(status_from_raw(999) == Status::Unknown);
  EXPECT(std::string(Backend::name()) == "cuda");
  EXPECT(Backend::capabilities().numerical_execution && !Backend::capabilities().metadata_only);

  const BackendProbe probe = backend_probe();  // an answer, never an exception, also without a GPU
  EXPECT(probe.available == expect_gpu);
  if (!expect_gpu) {
    EXPECT(!probe.diagnostic.empty());
    bool threw = false;
    try {
      (void)Backend::connect();
    } catch (const Error &e) {
      threw = e.status() == Status::CudaUnavailable && std::string(e.what()) == probe.diagnostic;
    }
    EXPECT(threw);
    threw = false;
    try {
      Context ctx(0);  // no CPU fallback: creating a context fails loudly
    } catch (const Error &e) {
      threw = e.status() == Status::CudaUnavailable;
    }
    EXPECT(threw);
  }

  // shape-only capability query: works without a device
  QuantLinear op;
  op.n = 256;
  op.k = 512;
  op.m = 1;
  BackendSupport s = Backend::supports(op);
  EXPECT(s.supported && s.kernel == ULLM_CUDA_KERNEL_MATVEC);
  op.m = 64;  // the same answer with or without a device: the query looks at shapes only
  s = Backend::supports(op);
  EXPECT(s.supported && s.kernel == ULLM_CUDA_KERNEL_GEMM);
  op.encoding = ULLM_CUDA_ENCODING_AQ4;
  op.k = 200;  // not a multiple of the group size
  s = Backend::supports(op);
  EXPECT(!s.supported && !s.reason.empty());
  op.encoding = ULLM_CUDA_ENCODING_NVFP4;  // served by the decode kernel only: 64 tokens are too many, one is fine
  op.k = 512;
  s = Backend::supports(op);
  EXPECT(!s.supported);
  op.m = 1;
  s = Backend::supports(op);
  EXPECT(s.supported && s.kernel == ULLM_CUDA_KERNEL_MATVEC);
  op.encoding = 77;  // not an encoding at all: an argument error or unsupported, never a crash
  bool handled = false;
  try {
    handled = !Backend::supports(op).supported;
  } catch (const Error &e) {
    handled = e.status() == Status::InvalidArgument || e.status() == Status::Unsupported;
  }
  EXPECT(handled);
  if (expect_gpu) {
    // One linear through the per-op path and the same one through a prepared command list.  FP8 weights whose codes
    // are all 0x38 (= 1.0) with scale 0.5: y[n] = 0.5 * sum_k x[k].
    const uint64_t n = 256, k = 512;
    Context ctx(0);
    Queue q(ctx);
    Buffer w(ctx, n * k), sc(ctx, 4 * n), x(ctx, 2 * k), y(ctx, 4 * n), y2(ctx, 4 * n);
    std::vector<uint8_t> codes(n * k, 0x38);
    std::vector<float> scales(n, 0.5f);
    std::vector<uint16_t> xb(k);
    float sum = 0.0f;
    for (uint64_t i = 0; i < k; ++i) {
      const float v = (float)((int)(i % 7) - 3) * 0.25f;  // exactly representable in bf16
      uint32_t bits;
      std::memcpy(&bits, &v, 4);
      xb[i] = (uint16_t)(bits >> 16);
      sum += v;
    }
    q.upload(w.at(), codes.data(), codes.size());
    q.upload(sc.at(), scales.data(), scales.size() * 4);
    q.upload(x.at(), xb.data(), xb.size() * 2);
    QuantLinear lin;
    lin.n = n;
    lin.k = k;
    lin.m = 1;
    lin.weight_values = w.at();
    lin.weight_scales = sc.at();
    lin.input = x.at();
    lin.output = y.at();
    lin.output_dtype = ULLM_CUDA_DTYPE_F32;
    const auto report = q.linear(lin).wait(std::chrono::seconds(5));
    EXPECT(report.has_value() && report->fallback_used == 0 && report->device_flags == 0 && report->dispatch_count >= 1);
    std::vector<float> out(n), out2(n);
    q.download(y.at(), out.data(), n * 4);
    for (uint64_t i = 0; i < n; ++i) EXPECT(out[i] == 0.5f * sum);
    Prepared plan(ctx, {lin});
    const Event ev = plan.submit(q, {{0, ULLM_CUDA_SLOT_WEIGHT_VALUES, ULLM_CUDA_ACCESS_READ, w.at()},
                                     {0, ULLM_CUDA_SLOT_WEIGHT_SCALES, ULLM_CUDA_ACCESS_READ, sc.at()},
                                     {0, ULLM_CUDA_SLOT_INPUT, ULLM_CUDA_ACCESS_READ, x.at()},
                                     {0, ULLM_CUDA_SLOT_OUTPUT, ULLM_CUDA_ACCESS_WRITE, y2.at()}});
    EXPECT(ev.wait(std::chrono::milliseconds(5000)));
    EXPECT(ev.query() == EventState::Success);
    q.download(y2.at(), out2.data(), n * 4);
    EXPECT(std::memcmp(out.data(), out2.data(), n * 4) == 0);
    bool refused = false;  // an output bound read-only is an argument error before anything is launched
    try {
      (void)plan.submit(q, {{0, ULLM_CUDA_SLOT_WEIGHT_VALUES, ULLM_CUDA_ACCESS_READ, w.at()},
                            {0, ULLM_CUDA_SLOT_WEIGHT_SCALES, ULLM_CUDA_ACCESS_READ, sc.at()},
                            {0, ULLM_CUDA_SLOT_INPUT, ULLM_CUDA_ACCESS_READ, x.at()},
                            {0, ULLM_CUDA_SLOT_OUTPUT, ULLM_CUDA_ACCESS_READ, y2.at()}});
    } catch (const Error &e) {
      refused = e.status() == Status::InvalidArgument;
    }
    EXPECT(refused);
  }
  std::puts("host mirror ok");
  return 0;
}
