// ra_attn_bwd_noalloc: attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (haoliuhl/ringattention has no native code
// and no notion of device scratch memory). It exists for hosts that drive this library through the
// C ABI and cannot call cudaMalloc at the moment they need a backward pass:
//   * a serving or training process that handed the whole GPU to its own memory pool at start-up,
//     so that a later cudaMalloc would simply fail;
//   * a latency-critical loop that cannot tolerate the device-wide synchronisation that
//     cudaMalloc / cudaFree imply;
//   * a plain C/C++ program without PyTorch, whose caching allocator normally provides the
//     temporaries of the regular path (ra_attn_bwd_prep + ra_attn_bwd + ra_cast_f32_bf16).
//
// The regular backward needs three temporaries: the fp32 dQ accumulator the kernel reduces into,
// and the per-row log-sum-exp (log2 units) and delta = rowsum(dO * O) vectors. Here they live in
// one array that is part of the library image: kNoAllocScratchBytes (16.5 MiB) of device memory per GPU,
// held until the process exits. With CUDA's default lazy module loading that memory, and the code of the
// three kernels involved, is placed on a GPU the first time this entry point (or
// ra_attn_bwd_noalloc_prepare) runs there, not when the library is loaded. That first use therefore does
// take device memory, implicitly, and it fails if none is left.
//
// Limits (larger problems are rejected with kHostTooLarge and a message in ra_last_error()):
//     B * Sq * H * D                      <= 4,194,304 elements   (fp32 dQ accumulator, 16 MiB)
//     B * H * roundup(Sq, 128)            <=    65,536 rows       (lse and delta, 256 KiB each)
//
// Rules for callers:
//   * Call ra_attn_bwd_noalloc_prepare() once per device, with that device current, while device memory
//     is still available: before the host hands the rest of the GPU to its own pool, and outside any
//     stream capture. It looks up the device address of the array (cudaGetSymbolAddress) and loads the
//     kernels, so that later calls of ra_attn_bwd_noalloc need nothing from the driver's allocator.
//     Without it, the first ra_attn_bwd_noalloc call on a device does the same set-up itself and is
//     subject to the same two conditions.
//   * All calls on a device share the one array. It keeps the previous call's contents; the part
//     that must start from zero (the dQ accumulator) is cleared on the stream at the start of
//     every call. Two calls whose kernels can overlap on the GPU (different streams, no ordering
//     between them) race on the array: order them, or use the allocating path for one of them.
//   * q, k, v, out, dout are contiguous (B, S, H, D) bf16; lse is (B, H, Sq) fp32 from the forward;
//     dq, dk, dv are contiguous bf16 outputs. D is 64 or 128. Masking: causal_block_size (0 = none)
//     with contiguous global offsets q_off / k_off, the same meaning as in ra_attn_bwd.
//   * Nothing is allocated or freed: no cudaMalloc, no cudaFree, no library call that allocates.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum { kNoAllocMaxDqElems = 4194304, kNoAllocMaxRows = 65536 };
enum { kNoAllocScratchBytes = (kNoAllocMaxDqElems + 2 * kNoAllocMaxRows) * 4 };

// Per-device set-up (see the rules above); returns 0 or a negative host error code. Idempotent.
int ra_attn_bwd_noalloc_prepare(void);

int ra_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                        const float* lse, void* dq, void* dk, void* dv, int B, int H, int Sq, int Sk,
                        int D, int causal_block_size, int q_off, int k_off, int* status, void* stream);

#ifdef __cplusplus
}
#endif
