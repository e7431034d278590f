// Instantiations of the length-specialised mixed-radix pass (fft_mixed_static.h)
// for the lengths 125 * 2^k, 15 * 2^k and 7 * 2^k.
#include "fft_mixed_static.h"

namespace jdb {

#define JD_MIXED_CASE(NN)                                                              \
  case NN:                                                                             \
    return d.elem_bytes == 8 ? launch_mixed_static_n<float, NN>(d, (cudaStream_t)stream) \
                             : launch_mixed_static_n<double, NN>(d, (cudaStream_t)stream);

int launch_mixed_static_c(const PassDesc& d, void* stream) {
  switch (d.M) {
    JD_MIXED_CASE(250)
    JD_MIXED_CASE(500)
    JD_MIXED_CASE(1000)
    JD_MIXED_CASE(2000)
    JD_MIXED_CASE(240)
    JD_MIXED_CASE(480)
    JD_MIXED_CASE(960)
    JD_MIXED_CASE(1920)
    JD_MIXED_CASE(448)
    JD_MIXED_CASE(896)
    JD_MIXED_CASE(1792)
    default:
      return JD_ERR_UNSUPPORTED;
  }
}

}  // namespace jdb
