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
// one array that is part of the library image, so every GPU that loads the library holds
// kNoAllocScratchBytes (16.5 MiB) until the process exits, whether or not this function is used.
//
// Limits (larger problems are rejected with kHostTooLarge and a message in ra_last_error()):
//     B * Sq * H * D                      <= 4,194,304 elements   (fp32 dQ accumulator, 16 MiB)
//     B * H * roundup(Sq, 128)            <=    65,536 rows       (lse and delta, 256 KiB each)
//
// Rules for callers:
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress,
//     with that device current) and remembers it. Make that first call outside any stream capture.
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

int ra_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                        const float* lse, void* dq, void* dk, void* dv, int B, int H, int Sq, int Sk,
                        int D, int causal_block_size, int q_off, int k_off, int* status, void* stream);

#ifdef __cplusplus
}
#endif
