// Instantiations of the length-specialised mixed-radix pass (fft_mixed_static.h)
// for the lengths 5 * 2^k and 25 * 2^k.
#include "fft_mixed_static.h"

namespace jdb {

#define JD_MIXED_CASE(NN)                                                              \
  case NN:                                                                             \
    return d.elem_bytes == 8 ? launch_mixed_static_n<float, NN>(d, (cudaStream_t)stream) \
                             : launch_mixed_static_n<double, NN>(d, (cudaStream_t)stream);

int launch_mixed_static_b(const PassDesc& d, void* stream) {
  switch (d.M) {
    JD_MIXED_CASE(160)
    JD_MIXED_CASE(320)
    JD_MIXED_CASE(640)
    JD_MIXED_CASE(1280)
    JD_MIXED_CASE(2560)
    JD_MIXED_CASE(200)
    JD_MIXED_CASE(400)
    JD_MIXED_CASE(800)
    JD_MIXED_CASE(1600)
    default:
      return JD_ERR_UNSUPPORTED;
  }
}

}  // namespace jdb
