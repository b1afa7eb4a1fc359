// Kernel template shared by the plain GEMM (gemm_sm100.cu) and the variant whose B operand is
// row-sharded over several GPUs and gathered inside the kernel (gemm_gather_sm100.cu).
#pragma once
#include "common/bounds.cuh"
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
  // SwiGLU epilogue (forward of a gate/up projection, B = W[2F][K] K-major with rows [gate | up]): every
  // 256-column tile is made of gate columns [tn*128, tn*128+128) and the matching up columns (two 128-row
  // TMA loads, tensor map 1), and the epilogue writes silu(gate) * up, F columns of bf16, instead of the
  // 2F pre-activations. gate and up are rounded to bf16 first, so the result equals the two-pass path.
  int swiglu_F;  // 0 = off
};

constexpr int MAX_SHARDS = 8;

// B operand sharded by rows of the stored weight W[N][K]: shard s holds rows
// [s*shard_rows, (s+1)*shard_rows). The local shard is read in place; every remote shard is pulled
// from its owner's memory into a local scratch by the leading `copy_ctas` CTAs of the grid while
// the other CTAs already compute on the tiles that only need local rows. A shard becomes usable
// when its counter reaches `flag_target` (each copy CTA adds 1 after its slice has landed).
struct GatherParams {
  int n_shards, my_shard, shard_rows, copy_ctas;
  const uint4* src[MAX_SHARDS];
  uint4* dst[MAX_SHARDS];
  long long n16[MAX_SHARDS];
  unsigned int* flags;
  unsigned int flag_target;
};

struct TmaSet {
  CUtensorMap m[MAX_SHARDS];
};

__device__ __forceinline__ bool wait_shard(const GatherParams& g, int s, const WaitCtx& w) {
  const unsigned int* f = g.flags + s;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (static_cast<int>(v - g.flag_target) >= 0) break;
    if (((++it) & 63u) == 0u) {
      if (*w.abort_smem) return false;
      if (globaltimer_ns() - t0 > RA_WAIT_TIMEOUT_NS) {
        raise_abort(w, kTimeoutPeerFlag);
        return false;
      }
    }
    __nanosleep(100);
  }
  // the copy was done with ordinary stores; order them before the TMA (async proxy) reads
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}

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

template <int A_MN, int B_MN, bool GATHER>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ TmaSet tma_bs,
                 const Params p, const GatherParams g) {
  const int n_copy = GATHER ? g.copy_ctas : 0;
  if (GATHER && static_cast<int>(blockIdx.x) < n_copy) {
    // ---------------------------------------------------------------- gather CTAs
    for (int d = 1; d < g.n_shards; ++d) {
      const int s = (g.my_shard + d) % g.n_shards;
      const long long stride = static_cast<long long>(n_copy) * THREADS;
      long long i = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x;
      const uint4* src = g.src[s];
      uint4* dst = g.dst[s];
      // 16 loads of 16 bytes in flight per thread: the pull is bound by bytes in flight over the NVLink
      // round trip, so depth per thread matters more than the number of gather CTAs
      for (; i + 15 * stride < g.n16[s]; i += 16 * stride) {
        uint4 r[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) r[u] = src[i + u * stride];
#pragma unroll
        for (int u = 0; u < 16; ++u) dst[i + u * stride] = r[u];
      }
      for (; i < g.n16[s]; i += stride) dst[i] = src[i];
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) atomicAdd(g.flags + s, 1u);
    }
    return;
  }
  const int cta = static_cast<int>(blockIdx.x) - n_copy;
  const int n_cta = static_cast<int>(gridDim.x) - n_copy;
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
    tma_prefetch_desc(&tma_bs.m[0]);
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
  const int tiles_n = p.swiglu_F ? (p.swiglu_F + BN / 2 - 1) / (BN / 2) : (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  // with a sharded B the tile order (B along N) or the k-block order (B along K) is rotated so
  // that work touching only local rows comes first
  const int tn_rot = (GATHER && !B_MN) ? g.my_shard * (g.shard_rows / BN) : 0;
  // (a trailing shard can be empty: its first k-block index then equals num_kb, hence the modulo)
  const int kb_rot = (GATHER && B_MN) ? (g.my_shard * (g.shard_rows / BK)) % num_kb : 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (warp-uniform flow)
    // All 32 lanes run the loop and poll the barriers; only the elected lane arms the barrier and issues the
    // loads. With the loop inside an `if (lane == 0)` region every TMA operand had to be moved to a uniform
    // register first, which matters for dgrad/wgrad (five or six loads per k-block in ~500 cycles).
    {
      const bool leader = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      unsigned int ready_mask = 0;
      for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
        tn = (tn + tn_rot) % tiles_n;
        const int m0 = tm * BM, n0 = tn * BN;
        // Shard of the B rows and the row offset inside it, tracked incrementally: this thread issues
        // up to five TMA loads per k-block and has ~500 cycles for them, so no division may sit in
        // the k loop (two of them made the sharded dgrad 60 % slower than the plain one).
        int kb = kb_rot;
        int shard = 0, row_in_shard = 0;
        if (GATHER) {
          const int w_row = B_MN ? kb * BK : n0;
          shard = w_row / g.shard_rows;
          row_in_shard = w_row - shard * g.shard_rows;
        }
        for (int kbi = 0; kbi < num_kb; ++kbi) {
          const int k0 = kb * BK;
          if (GATHER) {
            if (shard != g.my_shard && !((ready_mask >> shard) & 1u)) {
              if (!wait_shard(g, shard, wc)) {
                ok = false;
                break;
              }
              ready_mask |= 1u << shard;
            }
          }
          const CUtensorMap* tma_b = &tma_bs.m[shard];
          if (!mbar_wait(&empty[stage], phase ^ 1u, wc, kTimeoutSmemEmpty)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
          if (leader) {
            mbar_arrive_expect_tx(&full[stage], STAGE_TX_BYTES);
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < BM / 64; ++i)
                tma_load_2d(a_dst + i * SLAB_BYTES, &tma_a, &full[stage], m0 + 64 * i, k0);
            } else {
              tma_load_2d(a_dst, &tma_a, &full[stage], k0, m0);
            }
            if (B_MN) {
              const int kr = GATHER ? row_in_shard : k0;
#pragma unroll
              for (int i = 0; i < BN / 64; ++i)
                tma_load_2d(b_dst + i * SLAB_BYTES, tma_b, &full[stage], n0 + 64 * i, kr);
            } else if (!GATHER && p.swiglu_F) {
              tma_load_2d(b_dst, &tma_bs.m[1], &full[stage], k0, tn * (BN / 2));
              tma_load_2d(b_dst + B_STAGE_BYTES / 2, &tma_bs.m[1], &full[stage], k0, p.swiglu_F + tn * (BN / 2));
            } else {
              tma_load_2d(b_dst, tma_b, &full[stage], k0, GATHER ? row_in_shard : n0);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          if (++kb == num_kb) kb = 0;
          if (GATHER && B_MN) {  // next k-block: BK rows further, possibly in the next shard, or wrapped
            row_in_shard += BK;
            if (kb == 0) {
              shard = 0;
              row_in_shard = 0;
            } else if (row_in_shard >= g.shard_rows) {
              ++shard;
              row_in_shard = 0;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform flow)
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
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
            if (leader) umma_ss(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          if (leader) umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (leader) umma_commit(&tfull[acc]);
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
    for (int tile = cta; tile < num_tiles; tile += n_cta) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
      tn = (tn + tn_rot) % tiles_n;
      const int row = tm * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, wc, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      if (p.swiglu_F) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_x32(t_row + c * 32, rg);
          tmem_ld_x32(t_row + BN / 2 + c * 32, ru);
          tmem_ld_wait();
          const int col0 = tn * (BN / 2) + c * 32;
          if (row < p.M && col0 < p.swiglu_F) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col0 + j * 8 < p.swiglu_F) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gv = __bfloat162float(__float2bfloat16(__uint_as_float(rg[8 * j + e])));
                  const float uv = __bfloat162float(__float2bfloat16(__uint_as_float(ru[8 * j + e])));
                  f[e] = gv / (1.f + __expf(-gv)) * uv;
                }
                uint4 v;
                v.x = pack_bf16x2(f[0], f[1]);
                v.y = pack_bf16x2(f[2], f[3]);
                v.z = pack_bf16x2(f[4], f[5]);
                v.w = pack_bf16x2(f[6], f[7]);
                if (RA_IN_BOUNDS(row, 1, p.M, kTagGemmStore) && RA_IN_BOUNDS(col0 + 8 * j, 8, p.swiglu_F, kTagGemmStore))
                  *reinterpret_cast<uint4*>(dst + 8 * j) = v;
              }
            }
          }
        }
      } else
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
                if (RA_IN_BOUNDS(row, 1, p.M, kTagGemmStore) && RA_IN_BOUNDS(col0 + 4 * j, 4, p.N, kTagGemmStore))
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
                if (RA_IN_BOUNDS(row, 1, p.M, kTagGemmStore) && RA_IN_BOUNDS(col0 + 8 * j, 8, p.N, kTagGemmStore))
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

}  // namespace gemm
}  // namespace ra
