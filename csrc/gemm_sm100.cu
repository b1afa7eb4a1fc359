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
#include "common/host_util.h"
#include "common/sm100.cuh"

namespace ra {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int NUM_ACC = 2;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_TX_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SLAB_BYTES = 64 * BK * 2;  // one 64-wide MN-major slab: 64 k-rows x 128 B
constexpr int SMEM_BYTES = STAGES * STAGE_TX_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int THREADS = 192;

struct Params {
  void* C;
  long long ldc;
  int M, N, K;
  int c_fp32;   // 1: C is fp32, 0: bf16
  const void* R;  // optional addend with C's element type: C = A B^T + R (R may alias C)
  long long ldr;
  int group_m;  // m-tiles per rasterisation group (L2 reuse of B across the group)
  int* status;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm,
                                            int& tn) {
  const int group_size = group_m * tiles_n;
  const int g = tile / group_size;
  const int first_m = g * group_m;
  const int gm = min(group_m, tiles_m - first_m);
  const int r = tile - g * group_size;
  tm = first_m + r % gm;
  tn = r / gm;
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + NUM_ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + NUM_ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, wc, kTimeoutSmemEmpty)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[stage], STAGE_TX_BYTES);
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(a_dst + i * SLAB_BYTES, &tma_a, &full[stage], m0 + 64 * i, k0);
          } else {
            tma_load_2d(a_dst, &tma_a, &full[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(b_dst + i * SLAB_BYTES, &tma_b, &full[stage], n0 + 64 * i, k0);
          } else {
            tma_load_2d(b_dst, &tma_b, &full[stage], k0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, wc, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, wc, kTimeoutSmemFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // K-major: 16 k-elements = 32 B inside the 128 B swizzle row.
            // MN-major: 16 k-rows of 128 B = 2048 B.
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + kk * 2048, SLAB_BYTES, 1024)
                                        : make_smem_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + kk * 2048, SLAB_BYTES, 1024)
                                        : make_smem_desc(b_addr + kk * 32, 16, 1024);
            umma_ss(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == NUM_ACC) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
      const int row = tm * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, wc, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          if (p.c_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (col0 + j * 4 < p.N) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (p.R) {
                  const float4 o = *reinterpret_cast<const float4*>(
                      reinterpret_cast<const float*>(p.R) + static_cast<long long>(row) * p.ldr + col0 + 4 * j);
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4*>(dst + 4 * j) = v;
              }
            }
          } else {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col0 + j * 8 < p.N) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
                if (p.R) {
                  const uint4 o = *reinterpret_cast<const uint4*>(
                      reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<long long>(row) * p.ldr + col0 + 8 * j);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 of = __bfloat1622float2(ob[e]);
                    f[2 * e] += of.x;
                    f[2 * e + 1] += of.y;
                  }
                }
                uint4 v;
                v.x = pack_bf16x2(f[0], f[1]);
                v.y = pack_bf16x2(f[2], f[3]);
                v.z = pack_bf16x2(f[4], f[5]);
                v.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst + 8 * j) = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
      if (++acc == NUM_ACC) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) bounded_drain_pause();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int A_MN, int B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) {
    set_error("gemm: cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
    return kHostLaunchFail;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
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
  gemm::Params p{C, ldc, M, N, K, c_fp32, R, ldr, group_m > 0 ? group_m : 8, status};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return gemm::launch<0, 0>(ta, tb, p, s);
  if (!a_mn && b_mn) return gemm::launch<0, 1>(ta, tb, p, s);
  if (a_mn && !b_mn) return gemm::launch<1, 0>(ta, tb, p, s);
  return gemm::launch<1, 1>(ta, tb, p, s);
}
