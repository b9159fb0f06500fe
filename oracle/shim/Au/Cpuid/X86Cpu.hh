// Test-only stand-in for the header of AMD's aocl-utils that the reference's common/platform_info.hpp
// includes (the library itself is a download of the reference's super-build and is not in this image).
// It answers the four ISA questions the reference asks with the compiler's CPUID builtins; vendor and
// family fields are zero.  Used only when oracle/Makefile compiles reference files for cross-checks.
#pragma once
#include <cstdlib>
namespace Au {
enum class ECpuidFlag { avx2, avx512f, avx512bw, avx512vl };
struct VendorInfo { int m_mfg = 0, m_family = 0, m_model = 0, m_uarch = 0; };
class X86Cpu {
 public:
  explicit X86Cpu(int = 0) {}
  VendorInfo getVendorInfo() const { return VendorInfo{}; }
  bool hasFlag(ECpuidFlag f) const {
    switch (f) {
    case ECpuidFlag::avx2: return __builtin_cpu_supports("avx2");
    // ORACLE_REF_SCALAR=1 makes the reference take its scalar code paths (set before the library is loaded)
    case ECpuidFlag::avx512f: return !std::getenv("ORACLE_REF_SCALAR") && __builtin_cpu_supports("avx512f");
    case ECpuidFlag::avx512bw: return __builtin_cpu_supports("avx512bw");
    case ECpuidFlag::avx512vl: return __builtin_cpu_supports("avx512vl");
    }
    return false;
  }
};
}  // namespace Au
using namespace Au;
