// Checked build (-DRA_BOUNDS_CHECK=1): the stand-in for a memory checker on machines where none can be run.
//
// Kernels wrap the logical indices behind their global-memory accesses in RA_IN_BOUNDS(index, count, limit, tag):
// "elements [index, index + count) of an object of `limit` elements". In a normal build the macro is `true` and
// costs nothing. In the checked build a violation is counted and its first occurrence recorded (tag of the
// access, index, limit) in a per-translation-unit device record, and the macro returns false so that the access
// is skipped: the kernel never traps and never touches the bad address. ra_bounds_report() sums the records
// of all translation units for the host. TMA transfers are range-checked by the hardware against their tensor
// map and need no macro.
#pragma once
#include <cuda_runtime.h>

namespace ra {

#ifdef RA_BOUNDS_CHECK
// one record per translation unit (no relocatable device code): [0] violations, [1] tag, [2] index, [3] limit
static __device__ unsigned long long g_bounds_record[4];

__device__ __forceinline__ bool in_bounds(long long idx, long long n, long long limit, int tag) {
  if (idx >= 0 && n >= 0 && idx + n <= limit) return true;
  if (atomicAdd(&g_bounds_record[0], 1ull) == 0ull) {
    g_bounds_record[1] = static_cast<unsigned long long>(tag);
    g_bounds_record[2] = static_cast<unsigned long long>(idx);
    g_bounds_record[3] = static_cast<unsigned long long>(limit);
  }
  return false;
}
#define RA_IN_BOUNDS(idx, n, limit, tag) \
  (::ra::in_bounds(static_cast<long long>(idx), static_cast<long long>(n), static_cast<long long>(limit), (tag)))

typedef int (*BoundsReader)(unsigned long long* out4, int reset);
void register_bounds_reader(BoundsReader fn);  // host_util.cu

// Put once in every .cu file that uses RA_IN_BOUNDS: registers a reader of this file's record.
#define RA_BOUNDS_TRANSLATION_UNIT()                                                                      \
  namespace {                                                                                             \
  int ra_bounds_read_this_tu(unsigned long long* out4, int reset) {                                       \
    if (cudaMemcpyFromSymbol(out4, ::ra::g_bounds_record, 4 * sizeof(unsigned long long)) != cudaSuccess) \
      return -1;                                                                                          \
    if (reset) {                                                                                          \
      const unsigned long long z[4] = {0, 0, 0, 0};                                                       \
      if (cudaMemcpyToSymbol(::ra::g_bounds_record, z, sizeof(z)) != cudaSuccess) return -1;              \
    }                                                                                                     \
    return 0;                                                                                             \
  }                                                                                                       \
  struct RaBoundsRegistrar {                                                                              \
    RaBoundsRegistrar() { ::ra::register_bounds_reader(&ra_bounds_read_this_tu); }                        \
  } ra_bounds_registrar_instance;                                                                         \
  }
#else
#define RA_IN_BOUNDS(idx, n, limit, tag) true
#define RA_BOUNDS_TRANSLATION_UNIT()
#endif

// Tags of the checked accesses (what the host prints for the first violation).
enum BoundsTag : int {
  kTagGemmStore = 1,
  kTagGemmResidual = 2,
  kTagAttnFwdOut = 10,
  kTagAttnFwdLse = 11,
  kTagAttnFwdCarry = 12,
  kTagAttnMaskBits = 13,
  kTagAttnSeg = 14,
  kTagAttnBias = 15,
  kTagAttnBwdDkv = 20,
  kTagAttnBwdPrep = 21,
  kTagRmsnorm = 30,
  kTagRope = 31,
  kTagSwiglu = 32,
  kTagEmbeddingToken = 33,
  kTagEmbeddingRow = 34,
  kTagXentTarget = 35,
  kTagXentRow = 36,
  kTagAdamw = 37,
  kTagCast = 38,
  kTagPackMask = 39,
  kTagDecodeCacheRow = 40,
  kTagDecodeMerge = 41,
  kTagDecodeMask = 42,
  kTagSmallMLinear = 43,
  kTagPeerCopy = 50,
};

}  // namespace ra
