// Instantiations of the int8 tcgen05 GEMM with 256-row CTA tiles (two 128-row accumulators that share
// every weight stage).  Kept in a translation unit of their own so that the build compiles them in
// parallel with the 128-row ones.
#include "int8_tcgen05.cuh"

namespace zt {
namespace i8tc {

int launch_mh2(int bn, const CUtensorMap &ta, const CUtensorMap &tb, const TcParams &p, int epi, bool a_signed,
               cudaStream_t st) {
  switch (bn) {
    case 128: return launch_bn<2, 128, 4, 2>(ta, tb, p, epi, a_signed, st);  // 2 x 2 x 128 = 512 TMEM columns
    case 160: return launch_bn<2, 160, 4, 1>(ta, tb, p, epi, a_signed, st);
    case 192: return launch_bn<2, 192, 3, 1>(ta, tb, p, epi, a_signed, st);
    case 256: return launch_bn<2, 256, 3, 1>(ta, tb, p, epi, a_signed, st);
    default: break;
  }
  set_error("int8_tcgen05_launch: unsupported 256-row tile width %d", bn);
  return ZT_UNSUPPORTED;
}

}  // namespace i8tc
}  // namespace zt
