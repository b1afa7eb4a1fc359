// Host-side helpers shared by all launchers: TMA descriptor encoding through the driver entry
// point (no link-time dependency on libcuda), launch-error capture, device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ra {

// Error codes returned by every extern "C" launcher (0 = ok).
enum HostError : int {
  kHostOk = 0,
  kHostBadArg = -1,
  kHostTmapFail = -2,
  kHostLaunchFail = -3,
  kHostNoDriver = -4,
  kHostTooLarge = -5,
};

// rank-`rank` bf16 tensor map with 128-byte swizzle and zero fill for out-of-range elements.
// dims[0] is the innermost (contiguous) extent; strides_bytes has rank-1 entries (dims 1..).
int make_tmap_bf16_sw128(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box);

// Same, element type fp32 (box inner extent 32 elements = 128 bytes).
int make_tmap_f32_sw128(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box);

int sm_count();                 // SM count of the current device (cached per device)
int check_launch(const char*);  // cudaGetLastError -> HostError, message kept for ra_last_error
void set_error(const char* msg);

}  // namespace ra

extern "C" const char* ra_last_error();
