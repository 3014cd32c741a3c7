// C entry points around the reference's own packed-int8 GEMM (src/tensors/cpu/mjdgemm/*), compiled from
// the reference tree where it lies (see the Makefile's _ref target).  Test infrastructure only.
//   ref_mjd_supported(N, K)      1 when the reference instantiates this weight shape (mjdgemm_tmp.h:97-121)
//   ref_mjd_gemm(...)            marian::cpu::mjdgemm::gemmInt8Packed (mjdgemm.cpp:50-77): picks the ISA itself
//   ref_mjd_pack_b(...)          the reference's packB<> (mjdgemm_utils.h:136-165) for the same shapes
//   ref_mjd_isa()                the instruction set gemmInt8Packed will use on this host (cpu_info.h:122-179)
#include "tensors/cpu/mjdgemm/mjdgemm.h"
#include "tensors/cpu/mjdgemm/mjdgemm_utils.h"

using namespace marian::cpu;
using namespace marian::cpu::mjdgemm;

namespace {
template <int N, int K>
void pack(const int8_t* b, int8_t* out) { packB<InstructionSet::AVX512, N, K>(b, out); }
}  // namespace

#define MJD_SHAPES(X) X(512, 512) X(1024, 1024) X(4096, 1024) X(3072, 1024) X(1024, 4096) X(8192, 512) X(512, 8192) X(1024, 512) X(512, 1024) X(32000, 512)

extern "C" {

int ref_mjd_supported(int N, int K) {
#define X(n, k) if(N == n && K == k) return 1;
  MJD_SHAPES(X)
#undef X
  return 0;
}

int ref_mjd_isa() { return static_cast<int>(getSupportedInstructionSet()); }

int ref_mjd_gemm(const float* A, const int8_t* packedB, const float* bias, float* C, int M, int N, int K) {
  if(!ref_mjd_supported(N, K))
    return 1;
  gemmInt8Packed(A, packedB, bias, C, M, N, K);
  return 0;
}

int ref_mjd_pack_b(const int8_t* B, int8_t* packedB, int N, int K) {
#define X(n, k) if(N == n && K == k) { pack<n, k>(B, packedB); return 0; }
  MJD_SHAPES(X)
#undef X
  return 1;
}

}  // extern "C"
