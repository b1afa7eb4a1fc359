#include "host_util.h"

#include <stdio.h>
#include <string.h>

#include <mutex>

namespace ra {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

thread_local char g_err[512] = {0};

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, const void* base, int rank,
              const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled entry point not available");
    return kHostNoDriver;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx,
                  es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[400];
    snprintf(buf, sizeof(buf),
             "cuTensorMapEncodeTiled failed (%d): rank %d base %p dims [%llu %llu %llu %llu] "
             "stride1 %llu box [%u %u %u %u]",
             static_cast<int>(r), rank, base, (unsigned long long)dims[0],
             (unsigned long long)(rank > 1 ? dims[1] : 0), (unsigned long long)(rank > 2 ? dims[2] : 0),
             (unsigned long long)(rank > 3 ? dims[3] : 0),
             (unsigned long long)(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0,
             rank > 2 ? box[2] : 0, rank > 3 ? box[3] : 0);
    set_error(buf);
    return kHostTmapFail;
  }
  return kHostOk;
}
}  // namespace

void set_error(const char* msg) {
  strncpy(g_err, msg, sizeof(g_err) - 1);
  g_err[sizeof(g_err) - 1] = 0;
}

int make_tmap_bf16_sw128(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box);
}
int make_tmap_f32_sw128(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char buf[400];
    snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    set_error(buf);
    return kHostLaunchFail;
  }
  return kHostOk;
}

}  // namespace ra

extern "C" const char* ra_last_error() { return ra::g_err; }

// ---- checked build: sum of the per-translation-unit violation records (see common/bounds.cuh)
#ifdef RA_BOUNDS_CHECK
#include "bounds.cuh"
namespace ra {
namespace {
BoundsReader g_readers[32];
int g_n_readers = 0;
}  // namespace
void register_bounds_reader(BoundsReader fn) {
  if (g_n_readers < 32) g_readers[g_n_readers++] = fn;
}
}  // namespace ra
#endif

// out4 = {violations, tag of the first one, its index, its limit}, summed over the library for the current
// device (after a device synchronisation); reset != 0 clears the records. Returns 1 in a checked build, 0 in a
// normal build (out4 zeroed: nothing is checked), negative on a CUDA error.
extern "C" int ra_bounds_report(unsigned long long* out4, int reset) {
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
#ifdef RA_BOUNDS_CHECK
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  for (int i = 0; i < ra::g_n_readers; ++i) {
    unsigned long long r[4] = {0, 0, 0, 0};
    if (ra::g_readers[i](r, reset) != 0) return -1;
    if (r[0] && !out4[0]) {
      out4[1] = r[1];
      out4[2] = r[2];
      out4[3] = r[3];
    }
    out4[0] += r[0];
  }
  return 1;
#else
  (void)reset;
  return 0;
#endif
}
