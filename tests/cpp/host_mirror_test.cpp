// CPU-side check of the C++ host mirror (include/ullm_cuda.hpp): no GPU is needed, every device entry must
// answer CUDA_UNAVAILABLE here.  Prints "ok <n>" lines; exits non-zero on the first failed expectation.
#include <cstdio>
#include <cstdlib>

#include "ullm_cuda.hpp"

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
  std::puts("host mirror ok");
  return 0;
}
