// Attention backward without any device allocation; see attn_bwd_noalloc.h for the contract.
#include "attn_bwd_noalloc.h"

#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>

#include <mutex>

#include "attn_api.h"
#include "common/host_util.h"

namespace {

// The scratch itself: [ dQ accumulator | lse (log2 units) | delta ], all fp32. The name below is
// a host-side handle in host code, not an address a kernel could use; the device address comes
// from cudaGetSymbolAddress in scratch_for_current_device().
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocMaxDqElems + 2 * kNoAllocMaxRows];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// Device address of the array on the current device; resolved once per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ra::set_error("ra_attn_bwd_noalloc: cannot identify the current device");
    return ra::kHostLaunchFail;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      char msg[256];
      snprintf(msg, sizeof(msg), "ra_attn_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
               cudaGetErrorString(e));
      ra::set_error(msg);
      cudaGetLastError();
      return ra::kHostLaunchFail;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return ra::kHostOk;
}

}  // namespace

// Defined next to the kernels they name: make the driver load each kernel's code on the current device.
extern "C" int ra_attn_bwd_load_kernels(void);
extern "C" int ra_cast_load_kernels(void);

extern "C" int ra_attn_bwd_noalloc_prepare(void) {
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != ra::kHostOk) return rc;
  if ((rc = ra_attn_bwd_load_kernels()) != ra::kHostOk) return rc;
  return ra_cast_load_kernels();
}

extern "C" int ra_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out,
                                   const void* dout, const float* lse, void* dq, void* dk, void* dv,
                                   int B, int H, int Sq, int Sk, int D, int causal_block_size, int q_off,
                                   int k_off, int* status, void* stream) {
  using namespace ra;
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0 || (D != 64 && D != 128)) {
    set_error("ra_attn_bwd_noalloc: bad shape (head_dim must be 64 or 128)");
    return kHostBadArg;
  }
  const long long sq_pad = (static_cast<long long>(Sq) + 127) / 128 * 128;
  const long long dq_elems = static_cast<long long>(B) * Sq * H * D;
  const long long rows = static_cast<long long>(B) * H * sq_pad;
  if (dq_elems > kNoAllocMaxDqElems || rows > kNoAllocMaxRows) {
    char msg[320];
    snprintf(msg, sizeof(msg),
             "ra_attn_bwd_noalloc: problem too large for the built-in scratch: B*Sq*H*D = %lld (max %d), "
             "B*H*roundup(Sq,128) = %lld (max %d); use ra_attn_bwd with caller-provided buffers",
             dq_elems, static_cast<int>(kNoAllocMaxDqElems), rows, static_cast<int>(kNoAllocMaxRows));
    set_error(msg);
    return kHostTooLarge;
  }
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != kHostOk) return rc;
  float* dq_acc = scratch;
  float* lse2 = scratch + kNoAllocMaxDqElems;
  float* delta = lse2 + kNoAllocMaxRows;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  // The accumulator still holds the previous call's dQ: clear the part this call reduces into.
  if (cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(dq_elems) * sizeof(float), s) != cudaSuccess) {
    set_error("ra_attn_bwd_noalloc: cudaMemsetAsync failed");
    cudaGetLastError();
    return kHostLaunchFail;
  }
  const long long ss = static_cast<long long>(H) * D;  // contiguous (B, S, H, D)
  const long long sbq = ss * Sq, sbk = ss * Sk;
  rc = ra_attn_bwd_prep(out, sbq, ss, D, dout, sbq, ss, D, lse, lse2, delta, B, H, Sq,
                        static_cast<int>(sq_pad), D, stream);
  if (rc != kHostOk) return rc;

  RaAttnBwdArgs a = {};
  a.q = q; a.k = k; a.v = v; a.d_o = dout;
  a.q_sb = sbq; a.q_ss = ss; a.q_sh = D;
  a.k_sb = sbk; a.k_ss = ss; a.k_sh = D;
  a.v_sb = sbk; a.v_ss = ss; a.v_sh = D;
  a.do_sb = sbq; a.do_ss = ss; a.do_sh = D;
  a.lse2 = lse2; a.delta = delta; a.Sq_pad = static_cast<int>(sq_pad);
  a.dq_acc = dq_acc;
  a.dk = dk; a.dv = dv; a.dkv_sb = sbk; a.dkv_ss = ss; a.dkv_sh = D; a.dkv_mode = 0;
  a.B = B; a.H = H; a.Sq = Sq; a.Sk = Sk; a.D = D;
  a.softmax_scale = 1.0f / sqrtf(static_cast<float>(D));
  a.causal_block_size = causal_block_size;
  a.q_off0 = q_off; a.q_off1 = 0; a.q_half = 1 << 30;
  a.k_off0 = k_off; a.k_off1 = 0; a.k_half = 1 << 30;
  a.status = status;
  a.stream = stream;
  rc = ra_attn_bwd(&a);
  if (rc != kHostOk) return rc;
  return ra_cast_f32_bf16(dq_acc, dq, static_cast<long long>(B) * Sq, H * D, ss, ss, stream);
}
