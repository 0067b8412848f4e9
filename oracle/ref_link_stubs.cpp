// TEST INFRASTRUCTURE — link-time stand-ins used only when building oracle/_ref.
//
// The reference's CPU Adam (patrickstar/ops/csrc/adam/cpu_adam.cpp) is compiled
// unmodified from where it lies.  Its Adam_Optimizer constructor touches a
// `Context` singleton (patrickstar/ops/csrc/includes/context.h:41-52) that
// creates a cuBLAS handle and a cuRAND generator and asks torch for the current
// CUDA stream (context.h:83-90).  None of these is used by the Adam arithmetic,
// and all of them fail on a host without a GPU.  The definitions below are
// linked into the reference build (with -Wl,-Bsymbolic, so that the calls made
// inside that shared object bind here) and make those calls succeed without a
// device.  Every stream handed out is the legacy default stream (0).
#include <c10/cuda/CUDAStream.h>

extern "C" {
int cublasCreate_v2(void** handle)
{
    *handle = nullptr;
    return 0;
}
int cublasDestroy_v2(void*) { return 0; }
int curandCreateGenerator(void** gen, int)
{
    *gen = nullptr;
    return 0;
}
int curandSetPseudoRandomGeneratorSeed(void*, unsigned long long) { return 0; }
}

namespace c10 {
namespace cuda {

static CUDAStream default_stream_stand_in()
{
    return CUDAStream(CUDAStream::UNCHECKED,
                      Stream(Stream::UNSAFE, Device(DeviceType::CUDA, 0), 0));
}

CUDAStream getCurrentCUDAStream(DeviceIndex) { return default_stream_stand_in(); }
CUDAStream getStreamFromPool(const bool, DeviceIndex) { return default_stream_stand_in(); }
cudaStream_t CUDAStream::stream() const { return nullptr; }

}  // namespace cuda
}  // namespace c10
