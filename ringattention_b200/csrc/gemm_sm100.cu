// Persistent warp-specialised bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T (+ C).
//
//   warp 0      TMA producer: 128x64 A tile + 256x64 B tile per stage, 4-stage mbarrier ring
//   warp 1      tcgen05.mma issuer (one thread), two 128x256 fp32 accumulators in TMEM (512 cols)
//   warps 2..5  epilogue: tcgen05.ld -> bf16/fp32 -> global, overlapped with the next tile's MMAs
//
// Each operand is either K-major (contiguous along the reduction dim) or MN-major (contiguous
// along M resp. N); both are loaded with 128-byte-swizzled TMA boxes and described to the tensor
// core by shared-memory descriptors, so the forward (x W^T), dgrad (dy W) and wgrad (dy^T x)
// products of a linear layer all run through this one kernel without any transposes in memory.
#include "gemm_kernel.cuh"

RA_BOUNDS_TRANSLATION_UNIT()

namespace ra {
namespace gemm {

template <int A_MN, int B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, cudaStream_t stream,
           const CUtensorMap* tb_half = nullptr) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) {
    set_error("gemm: cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
    return kHostLaunchFail;
  }
  const int tiles_n = p.swiglu_F ? (p.swiglu_F + BN / 2 - 1) / (BN / 2) : (p.N + BN - 1) / BN;
  const int tiles = ((p.M + BM - 1) / BM) * tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  TmaSet set;
  set.m[0] = tb;
  if (tb_half) set.m[1] = *tb_half;
  GatherParams g = {};
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, set, p, g);
  return check_launch("gemm_bf16_kernel");
}

}  // namespace gemm
}  // namespace ra


// C[M,N] (ldc) = A * B^T (+ R). a_mn = 0: A is [M][lda] (K contiguous); 1: A is [K][lda] (M
// contiguous). b_mn = 0: B is [N][ldb]; 1: B is [K][ldb]. All leading dimensions in elements and
// multiples of 8; base pointers 16-byte aligned. c_fp32 selects the type of C and R. R is an
// optional addend (residual or running gradient) and may alias C for in-place accumulation.
extern "C" int ra_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N,
                            int K, long long lda, long long ldb, long long ldc, long long ldr,
                            int a_mn, int b_mn, int c_fp32, int group_m, int* status,
                            void* stream) {
  using namespace ra;
  if (M <= 0 || N <= 0 || K <= 0 || (lda % 8) || (ldb % 8) || (ldc % (c_fp32 ? 4 : 8)) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(R) & 15) ||
      (R && (ldr % (c_fp32 ? 4 : 8)))) {
    set_error("ra_gemm_bf16: bad shape/alignment");
    return kHostBadArg;
  }
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    if (a_mn) { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = gemm::BK; }
    else      { dims[0] = K; dims[1] = M; box[0] = gemm::BK; box[1] = gemm::BM; }
    str[0] = static_cast<uint64_t>(lda) * 2;
    if ((rc = make_tmap_bf16_sw128(&ta, A, 2, dims, str, box)) != 0) return rc;
    if (b_mn) { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = gemm::BK; }
    else      { dims[0] = K; dims[1] = N; box[0] = gemm::BK; box[1] = gemm::BN; }
    str[0] = static_cast<uint64_t>(ldb) * 2;
    if ((rc = make_tmap_bf16_sw128(&tb, B, 2, dims, str, box)) != 0) return rc;
  }
  gemm::Params p{C, ldc, M, N, K, c_fp32, R, ldr, group_m > 0 ? group_m : 8, status, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return gemm::launch<0, 0>(ta, tb, p, s);
  if (!a_mn && b_mn) return gemm::launch<0, 1>(ta, tb, p, s);
  if (a_mn && !b_mn) return gemm::launch<1, 0>(ta, tb, p, s);
  return gemm::launch<1, 1>(ta, tb, p, s);
}


// H[M,F] (ldh) = silu(A Wg^T) * (A Wu^T) for W = [Wg ; Wu] stored as [2F][ldb] (K contiguous): the gate/up
// projection of a SwiGLU feed-forward with the activation in the GEMM epilogue, so the (M, 2F) pre-activations
// are never written. A is [M][lda], K contiguous. F must be a multiple of 8.
extern "C" int ra_gemm_bf16_swiglu(const void* A, const void* W, void* Hout, int M, int F, int K, long long lda,
                                   long long ldb, long long ldh, int group_m, int* status, void* stream) {
  using namespace ra;
  if (M <= 0 || F <= 0 || K <= 0 || (F % 8) || (lda % 8) || (ldb % 8) || (ldh % 8) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(Hout) & 15)) {
    set_error("ra_gemm_bf16_swiglu: bad shape/alignment");
    return kHostBadArg;
  }
  CUtensorMap ta, tb, tbh;
  int rc;
  uint64_t dims[2], str[1];
  uint32_t box[2];
  dims[0] = K; dims[1] = M; box[0] = gemm::BK; box[1] = gemm::BM;
  str[0] = static_cast<uint64_t>(lda) * 2;
  if ((rc = make_tmap_bf16_sw128(&ta, A, 2, dims, str, box)) != 0) return rc;
  dims[0] = K; dims[1] = 2ull * F; box[0] = gemm::BK; box[1] = gemm::BN;
  str[0] = static_cast<uint64_t>(ldb) * 2;
  if ((rc = make_tmap_bf16_sw128(&tb, W, 2, dims, str, box)) != 0) return rc;
  box[1] = gemm::BN / 2;
  if ((rc = make_tmap_bf16_sw128(&tbh, W, 2, dims, str, box)) != 0) return rc;
  gemm::Params p{Hout, ldh, M, 2 * F, K, 0, nullptr, 0, group_m > 0 ? group_m : 8, status, F};
  return gemm::launch<0, 0>(ta, tb, p, static_cast<cudaStream_t>(stream), &tbh);
}
