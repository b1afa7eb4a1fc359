// Flash-attention backward for sm_100a: one fused kernel, five GEMMs per (q tile, kv tile) pair.
//
// One CTA owns a 128-row KV tile of one (batch, head); K and V stay resident in shared memory and
// the CTA walks the visible 128-row query tiles i:
//     S^T  = K Q_i^T            (SS)  -> TMEM [0,128)
//     dP^T = V dO_i^T           (SS)  -> TMEM [128,256)
//     P^T  = exp2(S^T*c - lse)        -> packed bf16 over S^T (TMEM)
//     dS^T = P^T (dP^T - delta)       -> bf16 in shared memory (128-byte swizzle); the 1/sqrt(D)
//                                        factor is applied when dQ and dK leave TMEM
//     dV  += P^T dO_i           (A from TMEM)        -> TMEM [256,256+D)
//     dK  += dS^T Q_i           (A = dS^T, K-major)  -> TMEM [384,384+D)
//     dQ_i = dS K               (A = dS^T read MN-major, B = K MN-major) -> TMEM over dP^T
// dQ_i is added to an fp32 buffer with bulk tensor reductions (TMA, staged through shared memory); dK/dV leave through the epilogue as
// bf16, fp32 or as fp32 reductions into (possibly a peer GPU's) accumulators, which is how the
// ring backward returns gradients to the owner of the KV block.
//
//   warps 0-3    producer group (registers trimmed): warp 0 TMA (K,V once; Q_i + lse/delta
//                double-buffered; dO_i), warp 1 tcgen05.mma issuer
//   warps 4-11   softmax/dS group: two warps per TMEM lane quadrant, 64 q-columns each
//   warps 12-15  dQ drain group (registers raised): tcgen05.ld, early release, bulk reduce-add
#include "attn_api.h"
#include "attn_common.cuh"
#include "common/host_util.h"

RA_BOUNDS_TRANSLATION_UNIT()

namespace ra {
namespace attn {

constexpr int BWD_THREADS = 512;
// Register re-balancing: the CTA owns 512 x 128 registers (launch bounds); setmaxnreg.inc blocks
// until registers are free, so the per-group budgets must fit in that allocation.
constexpr int BWD_REGS_PRODUCER = 80;  // warps 0-3
constexpr int BWD_REGS_SOFTMAX = 144;  // warps 4-11
constexpr int BWD_REGS_DRAIN = 144;    // warps 12-15
static_assert(128 * BWD_REGS_PRODUCER + 256 * BWD_REGS_SOFTMAX + 128 * BWD_REGS_DRAIN <= BWD_THREADS * 128,
              "setmaxnreg budgets exceed the registers the CTA was launched with");

struct BwdParams {
  int B, H;
  MaskParams mask;
  float scale;       // 1/sqrt(D)
  float scale_log2;  // log2(e)/sqrt(D)
  const float* lse2;   // (B, H, Sq_pad): -lse*log2(e), -inf for fully masked / padded rows
  const float* delta;  // (B, H, Sq_pad): rowsum(dO * O)
  int Sq_pad;
  float* dq_acc;       // (B, Sq, H, D) fp32 contiguous, accumulated with reductions
  void* dk; void* dv;  // (B, Sk, H, D) with strides below
  long long dkv_sb, dkv_ss, dkv_sh;
  int dkv_mode;        // 0: store bf16, 1: store fp32, 2: fp32 reduction (system scope)
  const uint4* copy_src;
  uint4* copy_dst;
  long long copy_n16;
  int copy_ctas;
  int* status;
  long long* trace;  // optional phase timestamps of the first compute CTA: [role 0..3][64 iterations][4]
};

template <int D>
struct BwdSmem {
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int SLAB_BYTES = 128 * 64 * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + TILE_BYTES;
  static constexpr int Q_OFF = V_OFF + TILE_BYTES;        // 2 stages
  static constexpr int DO_OFF = Q_OFF + 2 * TILE_BYTES;   // 1 stage
  static constexpr int DS_OFF = DO_OFF + TILE_BYTES;      // 128 x 128 bf16
  static constexpr int DQ_OFF = DS_OFF + 128 * 128 * 2;   // dQ staging: 128 rows x 32 fp32, swizzled
  static constexpr int LSE_OFF = DQ_OFF + 128 * 32 * 4;   // [2 stages][lse2 128 | delta 128]
  static constexpr int SEG_OFF = LSE_OFF + 2 * 256 * 4;   // [2][128] int
  static constexpr int BAR_OFF = SEG_OFF + 2 * 128 * 4;
  static constexpr int VIS_OFF = BAR_OFF + 256;  // [VIS_WORDS] visibility of the q tiles
  static constexpr int TOTAL = VIS_OFF + VIS_WORDS * 4 + 1024;
};

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}
__device__ __forceinline__ void red_add_v4_sys(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a),
               "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Phase timestamps (SM clock) for pipeline analysis; only the first compute CTA records, only its
// first 64 iterations, and only when the launch was given a trace buffer (RaAttnBwdArgs::trace).
__device__ __forceinline__ void trace_event(long long* trace, bool on, int role, int it, int slot) {
  if (on && it < 64) trace[(role * 64 + it) * 4 + slot] = clock64();
}

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_do,
                const __grid_constant__ CUtensorMap tma_dq, const BwdParams p) {
  using SM = BwdSmem<D>;
  constexpr int NSLAB = D / 64;

  // A failure recorded earlier on this stream (for example a ring barrier that timed out) turns
  // every later attention kernel into a no-op, so nothing touches the memory of a lost peer.
  if (p.status && *reinterpret_cast<const volatile int*>(p.status) != 0) return;

  if (static_cast<int>(blockIdx.x) < p.copy_ctas) {
    const long long stride = static_cast<long long>(p.copy_ctas) * BWD_THREADS;
    long long i = static_cast<long long>(blockIdx.x) * BWD_THREADS + threadIdx.x;
    // 16 loads of 16 bytes in flight per thread (the pull is bound by bytes in flight over NVLink)
    for (; i + 15 * stride < p.copy_n16; i += 16 * stride) {
      uint4 r[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) r[u] = p.copy_src[i + u * stride];
#pragma unroll
      for (int u = 0; u < 16; ++u) p.copy_dst[i + u * stride] = r[u];
    }
    for (; i < p.copy_n16; i += stride) p.copy_dst[i] = p.copy_src[i];
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem + SM::K_OFF;
  uint8_t* sV = smem + SM::V_OFF;
  uint8_t* sQ = smem + SM::Q_OFF;
  uint8_t* sDO = smem + SM::DO_OFF;
  uint8_t* sDS = smem + SM::DS_OFF;
  uint8_t* sDQ = smem + SM::DQ_OFF;
  float* sLse = reinterpret_cast<float*>(smem + SM::LSE_OFF);  // [stage][-lse2 128 | delta 128]
  int* sSegQ = reinterpret_cast<int*>(smem + SM::SEG_OFF);     // [buf][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* kv_full = bars;        // 1
  uint64_t* q_full = bars + 1;     // 2
  uint64_t* q_empty = bars + 3;    // 2
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;
  uint64_t* s_full = bars + 7;
  uint64_t* dp_full = bars + 8;
  uint64_t* p_ready = bars + 9;    // 256 arrivals
  uint64_t* ds_ready = bars + 10;  // 256 arrivals
  uint64_t* dq_full = bars + 11;
  uint64_t* dq_empty = bars + 12;  // 128 arrivals
  uint64_t* acc_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, p.status};
  const MaskParams& mk = p.mask;

  const int nkt = (mk.Sk + 127) / 128;
  const int nqt = (mk.Sq + 127) / 128;
  const int idx = static_cast<int>(blockIdx.x) - p.copy_ctas;
  const int bh = idx / nkt;
  const int jt = idx - bh * nkt;  // kv tile; low tiles see the most queries under a causal mask
  const int h = bh % p.H;
  const int b = bh / p.H;
  const int k0 = jt * 128;
  const bool tr = p.trace != nullptr && idx == 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(ds_ready, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 128);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
    tma_prefetch_desc(&tma_do);
    tma_prefetch_desc(&tma_dq);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // which q tiles this kv tile is seen by
  uint32_t* sVis = reinterpret_cast<uint32_t*>(smem + SM::VIS_OFF);
  const bool use_vis = nqt <= 32 * VIS_WORDS;
  if (use_vis)
    fill_visibility(sVis, nqt, static_cast<int>(threadIdx.x), BWD_THREADS,
                    [&](int i) { return tile_visible(mk, b, i * 128, k0); });
  // next q tile at or after i that sees this kv tile, or nqt; every role walks the same mask
  auto next_vis = [&](int i) -> int {
    if (use_vis) return vis_next(sVis, i, nqt);
    for (; i < nqt; ++i)
      if (tile_visible(mk, b, i * 128, k0)) break;
    return i;
  };
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;         // S^T, then packed P^T (cols 0-31 and 64-95)
  const uint32_t tDP = tmem_base + 128;  // dP^T, then dQ_i
  const uint32_t tDV = tmem_base + 256;
  const uint32_t tDK = tmem_base + 384;

  if (warp < 4) {
    // ================================================================ producer warpgroup
    setmaxnreg_dec<BWD_REGS_PRODUCER>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      mbar_arrive_expect_tx(kv_full, 2 * SM::TILE_BYTES);
#pragma unroll
      for (int s = 0; s < NSLAB; ++s) {
        tma_load_4d(sK + s * SM::SLAB_BYTES, &tma_k, kv_full, s * 64, h, k0, b);
        tma_load_4d(sV + s * SM::SLAB_BYTES, &tma_v, kv_full, s * 64, h, k0, b);
      }
      int it = 0;
      for (int i = next_vis(0); i < nqt; i = next_vis(i + 1)) {
        const int qi0 = i * 128;
        const int st = it & 1;
        if (!mbar_wait_relaxed(&q_empty[st], ((it >> 1) & 1) ^ 1u, wc, kTimeoutSmemEmpty)) break;
        mbar_arrive_expect_tx(&q_full[st], SM::TILE_BYTES + 1024);
#pragma unroll
        for (int s = 0; s < NSLAB; ++s)
          tma_load_4d(sQ + st * SM::TILE_BYTES + s * SM::SLAB_BYTES, &tma_q, &q_full[st], s * 64, h,
                      qi0, b);
        const long long row_off = (static_cast<long long>(b) * p.H + h) * p.Sq_pad + qi0;
        bulk_load_1d(sLse + st * 256, p.lse2 + row_off, 512, &q_full[st]);
        bulk_load_1d(sLse + st * 256 + 128, p.delta + row_off, 512, &q_full[st]);
        if (it > 0 && !mbar_wait_relaxed(do_empty, (it - 1) & 1, wc, kTimeoutSmemEmpty)) break;
        mbar_arrive_expect_tx(do_full, SM::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < NSLAB; ++s)
          tma_load_4d(sDO + s * SM::SLAB_BYTES, &tma_do, do_full, s * 64, h, qi0, b);
        ++it;
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer (warp-uniform flow)
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_dv = make_idesc_bf16(128, D, 0, 1);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);
      constexpr uint32_t SLAB = SM::SLAB_BYTES;
      // descriptor bases: *_k = K-major view (rows of 128 B along the reduction dim),
      // *_mn = MN-major view of the same bytes (64-wide slabs SLAB bytes apart)
      const uint64_t k_k = make_smem_desc(smem_u32(sK), 16, 1024);
      const uint64_t k_mn = make_smem_desc(smem_u32(sK), SLAB, 1024);
      const uint64_t v_k = make_smem_desc(smem_u32(sV), 16, 1024);
      const uint64_t do_k = make_smem_desc(smem_u32(sDO), 16, 1024);
      const uint64_t do_mn = make_smem_desc(smem_u32(sDO), SLAB, 1024);
      const uint64_t ds_mn = make_smem_desc(smem_u32(sDS), SLAB, 1024);
      const uint64_t q_k[2] = {make_smem_desc(smem_u32(sQ), 16, 1024),
                               make_smem_desc(smem_u32(sQ + SM::TILE_BYTES), 16, 1024)};
      const uint64_t q_mn[2] = {make_smem_desc(smem_u32(sQ), SLAB, 1024),
                                make_smem_desc(smem_u32(sQ + SM::TILE_BYTES), SLAB, 1024)};
      auto issue_st = [&](int st) {  // S^T = K Q^T
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SLAB + (kk & 3) * 32;
          if (leader)
            umma_ss(tS, desc_advance(k_k, off), desc_advance(q_k[st], off), idesc_s, kk != 0 ? 1u : 0u);
        }
        if (leader) umma_commit(s_full);
      };
      auto next_visible = [&](int i) { return next_vis(i); };
      bool ok = mbar_wait(kv_full, 0, wc, kTimeoutSmemFull);
      int i = next_visible(0);
      int it = 0;
      if (ok && i < nqt) {
        ok = mbar_wait(&q_full[0], 0, wc, kTimeoutSmemFull);
        if (ok) {
          tc_fence_after();
          issue_st(0);
        }
      }
      while (ok && i < nqt) {
        const int st = it & 1;
        const uint32_t par = it & 1;
        // dP^T = V dO^T (its region doubles as dQ: wait until the previous dQ left TMEM)
        if (!mbar_wait(do_full, par, wc, kTimeoutSmemFull)) break;
        if (it > 0 && !mbar_wait(dq_empty, (it - 1) & 1, wc, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        trace_event(p.trace, tr && leader, 0, it, 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SLAB + (kk & 3) * 32;
          if (leader)
            umma_ss(tDP, desc_advance(v_k, off), desc_advance(do_k, off), idesc_s, kk != 0 ? 1u : 0u);
        }
        if (leader) umma_commit(dp_full);
        // dV += P^T dO
        if (!mbar_wait(p_ready, par, wc, kTimeoutTmemFull)) break;
        tc_fence_after();
        trace_event(p.trace, tr && leader, 0, it, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_col = tS + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8);
          if (leader)
            umma_ts(tDV, a_col, desc_advance(do_mn, kk * 2048), idesc_dv, (it != 0 || kk != 0) ? 1u : 0u);
        }
        if (leader) umma_commit(do_empty);
        // next S^T right away (P^T was consumed by the dV MMAs just issued), so that the softmax
        // group can work on it while dK/dQ of this iteration run
        const int in = next_visible(i + 1);
        if (in < nqt) {
          const int stn = (it + 1) & 1;
          if (!mbar_wait(&q_full[stn], ((it + 1) >> 1) & 1, wc, kTimeoutSmemFull)) break;
          tc_fence_after();
          issue_st(stn);
        }
        // dK += dS^T Q ; dQ_i = dS K
        if (!mbar_wait(ds_ready, par, wc, kTimeoutTmemFull)) break;
        tc_fence_after();
        trace_event(p.trace, tr && leader, 0, it, 2);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_col = tDP + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8);  // dS^T in TMEM, laid out like P^T
          if (leader)
            umma_ts(tDK, a_col, desc_advance(q_mn[st], kk * 2048), idesc_dv, (it != 0 || kk != 0) ? 1u : 0u);
        }
        if (leader) umma_commit(&q_empty[st]);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          if (leader)
            umma_ss(tDP, desc_advance(ds_mn, kk * 2048), desc_advance(k_mn, kk * 2048), idesc_dq,
                    kk != 0 ? 1u : 0u);
        if (leader) umma_commit(dq_full);
        trace_event(p.trace, tr && leader, 0, it, 3);
        i = in;
        ++it;
      }
      if (leader) umma_commit(acc_full);
    }
    __syncwarp();
  } else if (warp < 12) {
    // ================================================================ softmax / dS group
    setmaxnreg_inc<BWD_REGS_SOFTMAX>();
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;  // which 64 q-columns
    const int sm_tid = (warp - 4) * 32 + lane;
    const int row = quad * 32 + lane;  // kv row inside the tile
    const int kj = k0 + row;
    const bool row_valid = kj < mk.Sk;
    const int kpos = mk.kmap(row_valid ? kj : mk.Sk - 1);
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int my_seg = (mk.seg_k && row_valid) ? mk.seg_k[static_cast<long long>(b) * mk.Sk + kj] : -1;
    const float my_bias2 =
        (mk.bias && row_valid) ? mk.bias[b * mk.bias_stride_b + h * mk.bias_stride_h + kj] * kLog2e : 0.f;
    const unsigned int bh_u = static_cast<unsigned int>(b * p.H + h);
    uint8_t* ds_row = sDS + half * SM::SLAB_BYTES + row * 128;
    const int swz = row & 7;
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    const uint64_t bias2 = f2_pack(my_bias2, my_bias2);

    int it = 0;
    bool alive = true;
    for (int i = next_vis(0); i < nqt && alive; i = next_vis(i + 1)) {
      const int qi0 = i * 128;
      const int st = it & 1;
      const uint32_t par = it & 1;
      const bool plain = tile_plain(mk, b, qi0, k0);
      if (mk.seg_q) {
        if (sm_tid < 128)
          sSegQ[st * 128 + sm_tid] =
              (qi0 + sm_tid) < mk.Sq ? mk.seg_q[static_cast<long long>(b) * mk.Sq + qi0 + sm_tid] : -2;
        named_bar_sync(1, 256);
      }
      // a wait that gives up must end the loop for the whole warp: the TMEM loads and stores below are
      // warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(&q_full[st], (it >> 1) & 1, wc, kTimeoutSmemFull))) { alive = false; break; }
      const float4* nl4 = reinterpret_cast<const float4*>(sLse + st * 256 + half * 64);
      const float4* dl4 = reinterpret_cast<const float4*>(sLse + st * 256 + 128 + half * 64);
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, par, wc, kTimeoutTmemFull))) { alive = false; break; }
      tc_fence_after();
      trace_event(p.trace, tr && sm_tid == 0, 1, it, 0);

      // masked iff column (q index) c < lo: causal rule transposed; everything if the row is padding
      int lo = 0;
      if (!plain) {
        if (!row_valid) {
          lo = 128;
        } else if (mk.cbs) {
          const long long kstart = static_cast<long long>(kpos / mk.cbs) * mk.cbs;
          const long long v = kstart - mk.qmap(qi0);
          lo = static_cast<int>(v < 0 ? 0 : (v > 128 ? 128 : v));
        }
      }
      const unsigned int qpos0 = static_cast<unsigned int>(mk.qmap(qi0));
      uint64_t pv[32];  // 64 probabilities of this thread's row, as fp32 pairs
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32];
        tmem_ld_x32(tS + lane_base + half * 64 + c * 32, s);
        tmem_ld_wait();
        trace_event(p.trace, tr && sm_tid == 0, 3, it, c * 2);
        uint64_t x[16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 n = nl4[c * 8 + g];
          x[2 * g] = f2_fma(f2_pack_u(s[4 * g], s[4 * g + 1]), scale2, f2_pack(n.x, n.y));
          x[2 * g + 1] = f2_fma(f2_pack_u(s[4 * g + 2], s[4 * g + 3]), scale2, f2_pack(n.z, n.w));
        }
        if (!plain) {
          // keepw bit e: column (q index) base+e survives the causal rule, padding and dropout; the hash is a
          // small rolled loop that only runs when dropout is on
          const int base = half * 64 + c * 32;
          const int n = lo - base;
          uint32_t keepw = n <= 0 ? 0xffffffffu : (n >= 32 ? 0u : ~((1u << n) - 1u));
          if (mk.keep && RA_IN_BOUNDS((qi0 + base) >> 5, 1, mk.keep_sr, kTagAttnMaskBits))
            keepw &= mk.keep[b * mk.keep_sb + h * mk.keep_sh + static_cast<long long>(row_valid ? kj : mk.Sk - 1) * mk.keep_sr +
                             ((qi0 + base) >> 5)];
          if (mk.drop_threshold) {
            uint32_t drop = 0;
#pragma unroll 1
            for (int e = 0; e < 32; ++e)
              drop |= static_cast<uint32_t>(dropout_hash(mk.seed_lo, mk.seed_hi, bh_u, qpos0 + base + e,
                                                         static_cast<unsigned int>(kpos)) < mk.drop_threshold)
                      << e;
            keepw &= ~drop;
          }
          const bool has_seg = mk.seg_q != nullptr;
          const int4* seg4 = reinterpret_cast<const int4*>(sSegQ + st * 128 + base);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int4 sg = has_seg ? seg4[g] : make_int4(my_seg, my_seg, my_seg, my_seg);
            const int se[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int e = 2 * g + h2;
              x[e] = f2_add(x[e], bias2);
              float x0, x1;
              f2_unpack(x[e], x0, x1);
              const bool m0 = (((keepw >> (2 * e)) & 1u) == 0u) || (se[2 * h2] != my_seg);
              const bool m1 = (((keepw >> (2 * e + 1)) & 1u) == 0u) || (se[2 * h2 + 1] != my_seg);
              x[e] = f2_pack(m0 ? -INFINITY : x0, m1 ? -INFINITY : x1);
            }
          }
        }
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float x0, x1;
          f2_unpack(x[e], x0, x1);
          const float p0 = exp2_approx(x0), p1 = exp2_approx(x1);
          pv[c * 16 + e] = f2_pack(p0, p1);
          pk[e] = pack_bf16x2(p0, p1);
        }
        tmem_st_x16(tS + lane_base + half * 64 + c * 16, pk);
        trace_event(p.trace, tr && sm_tid == 0, 3, it, c * 2 + 1);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready);
      trace_event(p.trace, tr && sm_tid == 0, 1, it, 1);

      if (!__all_sync(0xffffffffu, mbar_wait(dp_full, par, wc, kTimeoutTmemFull))) { alive = false; break; }
      // the dS buffer is still being read by the previous dK/dQ MMAs until dq_full fires
      if (it > 0 && !__all_sync(0xffffffffu, mbar_wait(dq_full, (it - 1) & 1, wc, kTimeoutTmemFull))) { alive = false; break; }
      tc_fence_after();
      trace_event(p.trace, tr && sm_tid == 0, 1, it, 2);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dp[32];
        uint32_t dsw[16];
        tmem_ld_x32(tDP + lane_base + half * 64 + c * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float4 d0 = dl4[c * 8 + 2 * g], d1 = dl4[c * 8 + 2 * g + 1];
          const uint64_t t0 = f2_mul(pv[c * 16 + 4 * g], f2_sub(f2_pack_u(dp[8 * g], dp[8 * g + 1]), f2_pack(d0.x, d0.y)));
          const uint64_t t1 = f2_mul(pv[c * 16 + 4 * g + 1], f2_sub(f2_pack_u(dp[8 * g + 2], dp[8 * g + 3]), f2_pack(d0.z, d0.w)));
          const uint64_t t2 = f2_mul(pv[c * 16 + 4 * g + 2], f2_sub(f2_pack_u(dp[8 * g + 4], dp[8 * g + 5]), f2_pack(d1.x, d1.y)));
          const uint64_t t3 = f2_mul(pv[c * 16 + 4 * g + 3], f2_sub(f2_pack_u(dp[8 * g + 6], dp[8 * g + 7]), f2_pack(d1.z, d1.w)));
          float a0, a1, a2, a3, a4, a5, a6, a7;
          f2_unpack(t0, a0, a1);
          f2_unpack(t1, a2, a3);
          f2_unpack(t2, a4, a5);
          f2_unpack(t3, a6, a7);
          uint4 v;
          v.x = pack_bf16x2(a0, a1);
          v.y = pack_bf16x2(a2, a3);
          v.z = pack_bf16x2(a4, a5);
          v.w = pack_bf16x2(a6, a7);
          const int chunk = c * 4 + g;  // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(ds_row + ((chunk ^ swz) << 4)) = v;
          dsw[4 * g] = v.x;
          dsw[4 * g + 1] = v.y;
          dsw[4 * g + 2] = v.z;
          dsw[4 * g + 3] = v.w;
        }
        // dS^T also goes back over the dP^T columns this thread has already read, packed like P^T, and feeds
        // the dK MMA from TMEM: one 32 KB shared-memory operand read less per iteration
        tmem_st_x16(tDP + lane_base + half * 64 + c * 16, dsw);
      }
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(ds_ready);
      trace_event(p.trace, tr && sm_tid == 0, 1, it, 3);
      ++it;
    }

    // ---- epilogue: dV (half 0) / dK (half 1) for this warp's 32 kv rows. dS carried no softmax
    // scale, so dK is scaled here.
    if (alive) alive = mbar_wait(acc_full, 0, wc, kTimeoutTmemFull);
    alive = __all_sync(0xffffffffu, alive);  // TMEM loads below are warp-collective
    tc_fence_after();
    if (alive && !(it == 0 && p.dkv_mode == 2)) {
      const uint32_t tacc = (half == 0 ? tDV : tDK) + lane_base;
      void* base = half == 0 ? p.dv : p.dk;
      const float mul = half == 0 ? 1.0f : p.scale;
      const long long off = b * p.dkv_sb + static_cast<long long>(kj) * p.dkv_ss + h * p.dkv_sh;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (it > 0) {
          tmem_ld_x32(tacc + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        if (!row_valid) continue;
        if (!(RA_IN_BOUNDS(kj, 1, mk.Sk, kTagAttnBwdDkv) && RA_IN_BOUNDS(c * 32, 32, D, kTagAttnBwdDkv))) continue;
        float f[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(r[e]) * mul;
        if (p.dkv_mode == 0) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(base) + off + c * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16x2(f[8 * g], f[8 * g + 1]);
            v.y = pack_bf16x2(f[8 * g + 2], f[8 * g + 3]);
            v.z = pack_bf16x2(f[8 * g + 4], f[8 * g + 5]);
            v.w = pack_bf16x2(f[8 * g + 6], f[8 * g + 7]);
            *reinterpret_cast<uint4*>(dst + 8 * g) = v;
          }
        } else {
          float* dst = reinterpret_cast<float*>(base) + off + c * 32;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (p.dkv_mode == 1)
              *reinterpret_cast<float4*>(dst + 4 * g) =
                  make_float4(f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3]);
            else
              red_add_v4_sys(dst + 4 * g, f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3]);
          }
        }
      }
    }
  } else {
    // ================================================================ dQ drain group
    setmaxnreg_inc<BWD_REGS_DRAIN>();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // q row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int it = 0;
    for (int i = next_vis(0); i < nqt; i = next_vis(i + 1)) {
      const int qi0 = i * 128;
      bool ok = mbar_wait_relaxed(dq_full, it & 1, wc, kTimeoutTmemFull, 32);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      trace_event(p.trace, tr && warp == 12 && lane == 0, 2, it, 0);
      // pull the whole dQ tile into registers and hand the TMEM region back at once; then move it
      // to global memory with bulk tensor reductions staged through one 16 KiB shared buffer
      uint32_t r[D];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_x32(tDP + lane_base + c * 32, r + c * 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_empty);
      trace_event(p.trace, tr && warp == 12 && lane == 0, 2, it, 1);
      uint8_t* dq_row = sDQ + row * 128;
      const int swz = row & 7;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        if (warp == 12 && lane == 0) tma_store_wait_read<0>();  // staging buffer free again
        named_bar_sync(2, 128);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 v = make_float4(__uint_as_float(r[c * 32 + 4 * g]) * p.scale,
                                       __uint_as_float(r[c * 32 + 4 * g + 1]) * p.scale,
                                       __uint_as_float(r[c * 32 + 4 * g + 2]) * p.scale,
                                       __uint_as_float(r[c * 32 + 4 * g + 3]) * p.scale);
          *reinterpret_cast<float4*>(dq_row + ((g ^ swz) << 4)) = v;
        }
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        if (warp == 12 && lane == 0) {
          tma_reduce_add_4d(&tma_dq, sDQ, c * 32, h, qi0, b);
          tma_store_commit();
        }
      }
      trace_event(p.trace, tr && warp == 12 && lane == 0, 2, it, 2);
      ++it;
    }
    if (warp == 12 && lane == 0) tma_store_wait_all<0>();  // reductions complete before the CTA retires
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

// delta[b,h,q] = sum_d dO*O ; lse2 = -lse*log2(e) (-inf where lse is -inf); padded rows get
// (-inf, 0) so that exp2(s*c + lse2) is 0 for them. One warp per (b, q, h) row.
template <int D>
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, long long o_sb, long long o_ss,
                                     long long o_sh, const __nv_bfloat16* __restrict__ d_o,
                                     long long do_sb, long long do_ss, long long do_sh,
                                     const float* __restrict__ lse, float* __restrict__ lse2,
                                     float* __restrict__ delta, int B, int H, int Sq, int Sq_pad) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * H * Sq_pad;
  if (gw >= total) return;
  const int q = static_cast<int>(gw % Sq_pad);
  const int hh = static_cast<int>((gw / Sq_pad) % H);
  const int bb = static_cast<int>(gw / (static_cast<long long>(Sq_pad) * H));
  float acc = 0.f;
  float l2 = -INFINITY;
  if (q < Sq) {
    const __nv_bfloat16* po = o + bb * o_sb + static_cast<long long>(q) * o_ss + hh * o_sh;
    const __nv_bfloat16* pd = d_o + bb * do_sb + static_cast<long long>(q) * do_ss + hh * do_sh;
    constexpr int PER = D / 32;  // 2 or 4 elements per lane
#pragma unroll
    for (int e = 0; e < PER; e += 2) {
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(po + lane * PER + e);
      const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(pd + lane * PER + e);
      const float2 af = __bfloat1622float2(a), gf = __bfloat1622float2(g);
      acc += af.x * gf.x + af.y * gf.y;
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
    const float l = lse[(static_cast<long long>(bb) * H + hh) * Sq + q];
    l2 = (l == -INFINITY) ? -INFINITY : -l * kLog2e;
  }
  if (lane == 0 && RA_IN_BOUNDS(gw, 1, total, kTagAttnBwdPrep)) {
    lse2[gw] = l2;
    delta[gw] = acc;
  }
}

}  // namespace attn
}  // namespace ra

namespace {
int make_bshd_map_bwd(CUtensorMap* m, const void* base, int B, int S, int H, int D, long long sb,
                      long long ss, long long sh) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                      static_cast<uint64_t>(B)};
  uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(ss) * 2,
                     static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return ra::make_tmap_bf16_sw128(m, base, 4, dims, str, box);
}
}  // namespace


extern "C" int ra_attn_bwd(const RaAttnBwdArgs* a) {
  using namespace ra;
  using namespace ra::attn;
  if (a->D != 128 && a->D != 64) {
    set_error("ra_attn_bwd: head_dim must be 64 or 128");
    return kHostBadArg;
  }
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Sk <= 0 || (a->Sq_pad % 128) || a->Sq_pad < a->Sq ||
      (a->q_half < a->Sq && a->q_half % 128) || (a->k_half < a->Sk && a->k_half % 128) ||
      (a->copy_bytes % 16)) {
    set_error("ra_attn_bwd: bad shape");
    return kHostBadArg;
  }
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_bshd_map_bwd(&tq, a->q, a->B, a->Sq, a->H, a->D, a->q_sb, a->q_ss, a->q_sh))) return rc;
  if ((rc = make_bshd_map_bwd(&tk, a->k, a->B, a->Sk, a->H, a->D, a->k_sb, a->k_ss, a->k_sh))) return rc;
  if ((rc = make_bshd_map_bwd(&tv, a->v, a->B, a->Sk, a->H, a->D, a->v_sb, a->v_ss, a->v_sh))) return rc;
  if ((rc = make_bshd_map_bwd(&tdo, a->d_o, a->B, a->Sq, a->H, a->D, a->do_sb, a->do_ss, a->do_sh)))
    return rc;
  CUtensorMap tdq;
  {
    if (reinterpret_cast<uintptr_t>(a->dq_acc) & 15) {
      set_error("ra_attn_bwd: dq_acc must be 16-byte aligned");
      return kHostBadArg;
    }
    uint64_t dims[4] = {static_cast<uint64_t>(a->D), static_cast<uint64_t>(a->H),
                        static_cast<uint64_t>(a->Sq), static_cast<uint64_t>(a->B)};
    uint64_t str[3] = {static_cast<uint64_t>(a->D) * 4, static_cast<uint64_t>(a->H) * a->D * 4,
                       static_cast<uint64_t>(a->Sq) * a->H * a->D * 4};
    uint32_t box[4] = {32, 1, 128, 1};
    if ((rc = make_tmap_f32_sw128(&tdq, a->dq_acc, 4, dims, str, box))) return rc;
  }
  BwdParams p;
  p.B = a->B;
  p.H = a->H;
  p.mask.Sq = a->Sq;
  p.mask.Sk = a->Sk;
  p.mask.cbs = a->causal_block_size;
  p.mask.qmap = PosMap{a->q_off0, a->q_off1, a->q_half};
  p.mask.kmap = PosMap{a->k_off0, a->k_off1, a->k_half};
  p.mask.seg_q = a->seg_q;
  p.mask.seg_k = a->seg_k;
  p.mask.seg_q_mm = a->seg_q_mm;
  p.mask.seg_k_mm = a->seg_k_mm;
  p.mask.bias = a->bias;
  p.mask.bias_stride_b = a->bias_sb;
  p.mask.bias_stride_h = a->bias_sh;
  p.mask.seed_lo = static_cast<unsigned int>(a->seed & 0xffffffffull);
  p.mask.seed_hi = static_cast<unsigned int>(a->seed >> 32);
  p.mask.drop_threshold = a->drop_threshold;
  p.mask.keep = a->keep;
  p.mask.keep_sb = a->keep_sb;
  p.mask.keep_sh = a->keep_sh;
  p.mask.keep_sr = a->keep_sr;
  p.scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * kLog2e;
  p.lse2 = a->lse2;
  p.delta = a->delta;
  p.Sq_pad = a->Sq_pad;
  p.dq_acc = a->dq_acc;
  p.dk = a->dk;
  p.dv = a->dv;
  p.dkv_sb = a->dkv_sb;
  p.dkv_ss = a->dkv_ss;
  p.dkv_sh = a->dkv_sh;
  p.dkv_mode = a->dkv_mode;
  p.copy_src = reinterpret_cast<const uint4*>(a->copy_src);
  p.copy_dst = reinterpret_cast<uint4*>(a->copy_dst);
  p.copy_n16 = a->copy_bytes / 16;
  p.copy_ctas = (a->copy_src && a->copy_bytes > 0) ? a->copy_ctas : 0;
  p.status = a->status;
  p.trace = a->trace;
  const int nkt = (a->Sk + 127) / 128;
  const long long grid = static_cast<long long>(nkt) * a->H * a->B + p.copy_ctas;
  cudaStream_t s = static_cast<cudaStream_t>(a->stream);
  if (a->D == 128) {
    auto kern = attn_bwd_kernel<128>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<128>::TOTAL) !=
        cudaSuccess) {
      set_error("attn_bwd: smem attribute");
      return kHostLaunchFail;
    }
    kern<<<static_cast<unsigned>(grid), BWD_THREADS, BwdSmem<128>::TOTAL, s>>>(tq, tk, tv, tdo, tdq, p);
  } else {
    auto kern = attn_bwd_kernel<64>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<64>::TOTAL) !=
        cudaSuccess) {
      set_error("attn_bwd: smem attribute");
      return kHostLaunchFail;
    }
    kern<<<static_cast<unsigned>(grid), BWD_THREADS, BwdSmem<64>::TOTAL, s>>>(tq, tk, tv, tdo, tdq, p);
  }
  return check_launch("attn_bwd_kernel");
}

// Touch every kernel of this file on the current device so that its code is resident before a caller that
// can no longer afford implicit device allocations launches it (CUDA loads kernels lazily by default).
extern "C" int ra_attn_bwd_load_kernels(void) {
  using namespace ra;
  using namespace ra::attn;
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, attn_bwd_kernel<128>) != cudaSuccess ||
      cudaFuncGetAttributes(&fa, attn_bwd_kernel<64>) != cudaSuccess ||
      cudaFuncGetAttributes(&fa, attn_bwd_prep_kernel<128>) != cudaSuccess ||
      cudaFuncGetAttributes(&fa, attn_bwd_prep_kernel<64>) != cudaSuccess) {
    set_error("ra_attn_bwd_load_kernels: cudaFuncGetAttributes failed");
    cudaGetLastError();
    return kHostLaunchFail;
  }
  return kHostOk;
}

// Backward preprocessing: delta and scaled lse into (B, H, Sq_pad) buffers. o / d_o are
// (B, Sq, H, D) bf16 views with element strides.
extern "C" int ra_attn_bwd_prep(const void* o, long long o_sb, long long o_ss, long long o_sh,
                                const void* d_o, long long do_sb, long long do_ss, long long do_sh,
                                const float* lse, float* lse2, float* delta, int B, int H, int Sq,
                                int Sq_pad, int D, void* stream) {
  using namespace ra;
  using namespace ra::attn;
  const long long rows = static_cast<long long>(B) * H * Sq_pad;
  const int threads = 256;
  const long long blocks = (rows * 32 + threads - 1) / threads;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128)
    attn_bwd_prep_kernel<128><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(o), o_sb, o_ss, o_sh,
        reinterpret_cast<const __nv_bfloat16*>(d_o), do_sb, do_ss, do_sh, lse, lse2, delta, B, H, Sq,
        Sq_pad);
  else if (D == 64)
    attn_bwd_prep_kernel<64><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(o), o_sb, o_ss, o_sh,
        reinterpret_cast<const __nv_bfloat16*>(d_o), do_sb, do_ss, do_sh, lse, lse2, delta, B, H, Sq,
        Sq_pad);
  else {
    set_error("ra_attn_bwd_prep: head_dim must be 64 or 128");
    return kHostBadArg;
  }
  return check_launch("attn_bwd_prep_kernel");
}
