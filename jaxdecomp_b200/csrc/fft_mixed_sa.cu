// Instantiations of the length-specialised mixed-radix pass (fft_mixed_static.h)
// for the lengths 3 * 2^k and 9 * 2^k.
#include "fft_mixed_static.h"

namespace jdb {

#define JD_MIXED_CASE(NN)                                                              \
  case NN:                                                                             \
    return d.elem_bytes == 8 ? launch_mixed_static_n<float, NN>(d, (cudaStream_t)stream) \
                             : launch_mixed_static_n<double, NN>(d, (cudaStream_t)stream);

int launch_mixed_static_a(const PassDesc& d, void* stream) {
  switch (d.M) {
    JD_MIXED_CASE(96)
    JD_MIXED_CASE(192)
    JD_MIXED_CASE(384)
    JD_MIXED_CASE(768)
    JD_MIXED_CASE(1536)
    JD_MIXED_CASE(3072)
    JD_MIXED_CASE(288)
    JD_MIXED_CASE(576)
    JD_MIXED_CASE(1152)
    JD_MIXED_CASE(2304)
    default:
      return JD_ERR_UNSUPPORTED;
  }
}

}  // namespace jdb
