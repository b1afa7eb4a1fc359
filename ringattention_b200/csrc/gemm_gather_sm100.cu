// GEMM whose weight operand is row-sharded over the GPUs of an fsdp group and gathered *inside* the
// kernel: leading CTAs pull the remote shards from their owners' memory into a local scratch while
// the remaining CTAs already run the tiles (forward) or k-blocks (dgrad) that need local rows only;
// a remote shard's tiles start as soon as its copy has landed (bounded flag wait). This replaces the
// "all-gather parameters, then matmul" pair of an FSDP step with one launch.
//
//   forward: y[M, N]  = x[M, K]  W[N, K]^T      W rows (N) sharded    -> b_mn = 0
//   dgrad  : dx[M, Kw] = dy[M, Nw] W[Nw, Kw]     W rows (Nw = reduction dim) sharded -> b_mn = 1
#include "gemm_kernel.cuh"

RA_BOUNDS_TRANSLATION_UNIT()

namespace ra {
namespace gemm {

template <int B_MN>
int launch_gather(const CUtensorMap& ta, const TmaSet& set, const Params& p, const GatherParams& g,
                  cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<0, B_MN, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
    set_error("gemm_gather: cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
    return kHostLaunchFail;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int compute = sm_count() - g.copy_ctas;  // every CTA of the grid must be resident at once
  if (compute < 1) compute = 1;
  if (tiles < compute) compute = tiles;
  kern<<<compute + g.copy_ctas, THREADS, SMEM_BYTES, stream>>>(ta, set, p, g);
  return check_launch("gemm_bf16_kernel<gather>");
}

}  // namespace gemm
}  // namespace ra

// shard_local[s]: where rows of shard s are read from on this GPU (own segment, or the scratch the
// copy CTAs fill). shard_src[s]: the owner's memory for remote shards, null for the own shard.
// For b_mn = 0, (N, K) are the GEMM dims and W is [N][ldw]; for b_mn = 1 the GEMM computes
// C[M, N] with reduction length K = number of W rows, and W is [K][ldw] with ldw >= N.
// copy_ctas == 0: the remote shards are already in `shard_local` from an earlier call whose flag target is
// passed again; nothing is copied and every CTA computes.
// pf_dst / pf_src / pf_n16 (all three or none): the copy CTAs pull these ranges (16-byte units, entry
// `my_shard` ignored) instead of this call's own remote shards, i.e. they prefetch the operand of a later
// call while this one computes on shards that are already resident; the counters advance as for any gather.
extern "C" int ra_gemm_bf16_gather(const void* A, void* C, const void* R, int M, int N, int K, long long lda,
                                   long long ldc, long long ldr, int b_mn, int c_fp32, int n_shards,
                                   int my_shard, int shard_rows, long long ldw,
                                   const void* const* shard_local, const void* const* shard_src,
                                   unsigned int* flags, unsigned int flag_target, int copy_ctas,
                                   int group_m, int* status, void* stream, const void* const* pf_dst,
                                   const void* const* pf_src, const long long* pf_n16) {
  using namespace ra;
  using namespace ra::gemm;
  const int w_rows = b_mn ? K : N;
  if (M <= 0 || N <= 0 || K <= 0 || n_shards < 1 || n_shards > MAX_SHARDS || my_shard < 0 ||
      my_shard >= n_shards || shard_rows % BN || (lda % 8) || (ldw % 8) || (ldc % (c_fp32 ? 4 : 8)) ||
      static_cast<long long>(shard_rows) * (n_shards - 1) >= w_rows + shard_rows || copy_ctas < 0) {
    set_error("ra_gemm_bf16_gather: bad shape (shard_rows must be a multiple of 256)");
    return kHostBadArg;
  }
  CUtensorMap ta;
  int rc;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {BK, BM};
    if ((rc = make_tmap_bf16_sw128(&ta, A, 2, dims, str, box)) != 0) return rc;
  }
  TmaSet set;
  GatherParams g = {};
  g.n_shards = n_shards;
  g.my_shard = my_shard;
  g.shard_rows = shard_rows;
  g.copy_ctas = n_shards > 1 ? copy_ctas : 0;
  g.flags = flags;
  g.flag_target = flag_target;
  for (int s = 0; s < n_shards; ++s) {
    long long rows = static_cast<long long>(w_rows) - static_cast<long long>(s) * shard_rows;
    if (rows > shard_rows) rows = shard_rows;
    if (rows < 0) rows = 0;
    const long long inner = b_mn ? N : K;
    if (rows > 0) {
      uint64_t dims[2] = {static_cast<uint64_t>(inner), static_cast<uint64_t>(rows)};
      uint64_t str[1] = {static_cast<uint64_t>(ldw) * 2};
      uint32_t box[2] = {64, static_cast<uint32_t>(b_mn ? BK : BN)};
      if ((rc = make_tmap_bf16_sw128(&set.m[s], shard_local[s], 2, dims, str, box)) != 0) return rc;
    } else {
      set.m[s] = set.m[0];
    }
    g.src[s] = (s == my_shard) ? nullptr : reinterpret_cast<const uint4*>(shard_src[s]);
    g.dst[s] = (s == my_shard) ? nullptr
                               : reinterpret_cast<uint4*>(const_cast<void*>(shard_local[s]));
    g.n16[s] = (s == my_shard) ? 0 : rows * ldw * 2 / 16;
    if (pf_dst && pf_src && pf_n16 && s != my_shard) {
      g.src[s] = reinterpret_cast<const uint4*>(pf_src[s]);
      g.dst[s] = reinterpret_cast<uint4*>(const_cast<void*>(pf_dst[s]));
      g.n16[s] = pf_n16[s];
    }
  }
  Params p{C, ldc, M, N, K, c_fp32, R, ldr, group_m > 0 ? group_m : 8, status};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return b_mn ? launch_gather<1>(ta, set, p, g, st) : launch_gather<0>(ta, set, p, g, st);
}
