// Flash-attention forward for sm_100a with carry-in, the per-device compute of one ring step.
//
// One CTA owns 256 query rows (two 128-row tiles) of one (batch, head) and walks the visible
// 128-row KV tiles:
//   warps 0-3   producer group (registers trimmed): warp 0 TMA (Q once, K/V through a 2-stage
//               ring each), warp 1 tcgen05.mma issuer: S_w = Q_w K^T (SS), O_w += P_w V (P in TMEM)
//   warps 4-7   softmax group for tile 0, warps 8-11 for tile 1 (registers raised): tcgen05.ld S,
//               mask, online softmax with lazy rescale of O in TMEM, P written back over S as bf16
// TMEM: S0 | S1 | O0 | O1 (4 x 128 columns). While one group runs its softmax the tensor core
// works on the other tile, so MMA and exp overlap without a third party.
//
// The epilogue normalises O, optionally merges it with the carry (o_prev, lse_prev) of earlier
// ring steps and writes fp32 (intermediate step) or bf16 (last step) plus the log-sum-exp.
// Leading CTAs of the grid can be given a copy job: they pull the next ring step's KV block from
// a peer GPU's memory into a local slab with plain 16-byte loads while the other CTAs compute.
#include "attn_common.cuh"
#include "common/host_util.h"

RA_BOUNDS_TRANSLATION_UNIT()

namespace ra {
namespace attn {

constexpr int FWD_THREADS = 384;
constexpr int KV_STAGES = 2;
// Register re-balancing: the CTA owns 384 x 168 registers (launch bounds); setmaxnreg.inc blocks
// until registers are free, so the per-group budgets must fit in that allocation.
constexpr int FWD_REGS_PRODUCER = 88;   // warps 0-3
constexpr int FWD_REGS_SOFTMAX = 208;   // warps 4-11
static_assert(128 * FWD_REGS_PRODUCER + 256 * FWD_REGS_SOFTMAX <= FWD_THREADS * 168,
              "setmaxnreg budgets exceed the registers the CTA was launched with");

struct FwdParams {
  int B, H;
  MaskParams mask;
  float scale_log2;  // log2(e) / sqrt(D)
  void* out;
  int out_fp32;
  long long o_stride_b, o_stride_s, o_stride_h;  // elements
  float* lse_out;         // (B, H, Sq)
  const float* o_prev;    // (B, Sq, H, D) fp32 contiguous, or null
  const float* lse_prev;  // (B, H, Sq), or null
  const uint4* copy_src;
  uint4* copy_dst;
  long long copy_n16;
  int copy_ctas;
  int* status;
};

template <int D>
struct FwdSmem {
  static constexpr int Q_TILE_BYTES = 128 * D * 2;
  static constexpr int KV_TILE_BYTES = 128 * D * 2;
  static constexpr int SLAB_BYTES = 128 * 64 * 2;  // one 64-wide d slab of a 128-row tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + 2 * Q_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * KV_TILE_BYTES;
  static constexpr int AUX_OFF = V_OFF + KV_STAGES * KV_TILE_BYTES;  // seg/bias staging
  static constexpr int AUX_BYTES = 2 /*wg*/ * 2 /*buf*/ * 128 * 4 * 2 /*seg+bias*/;
  static constexpr int BAR_OFF = AUX_OFF + AUX_BYTES;
  static constexpr int VIS_OFF = BAR_OFF + 256;  // [2 q tiles][VIS_WORDS] visibility of the kv tiles
  static constexpr int TOTAL = VIS_OFF + 2 * VIS_WORDS * 4 + 1024;
};

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const FwdParams p) {
  using SM = FwdSmem<D>;
  constexpr int NSLAB = D / 64;

  // A failure recorded earlier on this stream (for example a ring barrier that timed out) turns
  // every later attention kernel into a no-op, so nothing touches the memory of a lost peer.
  if (p.status && *reinterpret_cast<const volatile int*>(p.status) != 0) return;

  // ------------------------------------------------------------ copy CTAs (ring KV pull)
  if (static_cast<int>(blockIdx.x) < p.copy_ctas) {
    const long long stride = static_cast<long long>(p.copy_ctas) * FWD_THREADS;
    long long i = static_cast<long long>(blockIdx.x) * FWD_THREADS + threadIdx.x;
    // 16 loads of 16 bytes in flight per thread: the pull is bound by bytes in flight over the NVLink round
    // trip; finishing early hands the SM to a compute CTA sooner
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
  uint8_t* sQ = smem + SM::Q_OFF;
  uint8_t* sK = smem + SM::K_OFF;
  uint8_t* sV = smem + SM::V_OFF;
  int* sSeg = reinterpret_cast<int*>(smem + SM::AUX_OFF);              // [wg][buf][128]
  float* sBias = reinterpret_cast<float*>(smem + SM::AUX_OFF) + 512;   // [wg][buf][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars;             // 1
  uint64_t* k_full = bars + 1;         // KV_STAGES
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;         // 2 (per q tile)
  uint64_t* p_full = bars + 11;        // 2
  uint64_t* o_done = bars + 13;        // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, p.status};
  const MaskParams& mk = p.mask;

  // block -> (q pair, head, batch); heavy (late) q tiles first inside a head, heads outermost so
  // that concurrently running CTAs share one head's K/V in L2.
  const int n_qpairs = (mk.Sq + 255) / 256;
  const int idx = static_cast<int>(blockIdx.x) - p.copy_ctas;
  const int bh = idx / n_qpairs;
  const int qp = n_qpairs - 1 - (idx - bh * n_qpairs);
  const int h = bh % p.H;
  const int b = bh / p.H;
  const int q0 = qp * 256;
  const int nk = (mk.Sk + 127) / 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&s_full[w], 1);
      mbar_init(&p_full[w], 128);
      mbar_init(&o_done[w], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // which kv tiles each of the two q tiles sees
  uint32_t* sVis = reinterpret_cast<uint32_t*>(smem + SM::VIS_OFF);
  const bool use_vis = nk <= 32 * VIS_WORDS;
  if (use_vis) {
#pragma unroll
    for (int w = 0; w < 2; ++w)
      fill_visibility(sVis + w * VIS_WORDS, nk, static_cast<int>(threadIdx.x), FWD_THREADS,
                      [&](int j) { return tile_visible(mk, b, q0 + w * 128, j * 128); });
  }
  // next kv tile at or after j that q tile w sees, or nk
  auto next_vis = [&](int w, int j) -> int {
    if (use_vis) return vis_next(sVis + w * VIS_WORDS, j, nk);
    for (; j < nk; ++j)
      if (tile_visible(mk, b, q0 + w * 128, j * 128)) break;
    return j;
  };
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};

  if (warp < 4) setmaxnreg_dec<FWD_REGS_PRODUCER>();
  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * SM::Q_TILE_BYTES);
#pragma unroll
      for (int w = 0; w < 2; ++w)
#pragma unroll
        for (int s = 0; s < NSLAB; ++s)
          tma_load_4d(sQ + w * SM::Q_TILE_BYTES + s * SM::SLAB_BYTES, &tma_q, q_full, s * 64, h,
                      q0 + w * 128, b);
      int it = 0;
      for (int j = min(next_vis(0, 0), next_vis(1, 0)); j < nk;
           j = min(next_vis(0, j + 1), next_vis(1, j + 1))) {
        const int k0 = j * 128;
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait_relaxed(&k_empty[st], ph ^ 1u, wc, kTimeoutSmemEmpty)) break;
        mbar_arrive_expect_tx(&k_full[st], SM::KV_TILE_BYTES);
#pragma unroll
        for (int s = 0; s < NSLAB; ++s)
          tma_load_4d(sK + st * SM::KV_TILE_BYTES + s * SM::SLAB_BYTES, &tma_k, &k_full[st], s * 64,
                      h, k0, b);
        if (!mbar_wait_relaxed(&v_empty[st], ph ^ 1u, wc, kTimeoutSmemEmpty)) break;
        mbar_arrive_expect_tx(&v_full[st], SM::KV_TILE_BYTES);
#pragma unroll
        for (int s = 0; s < NSLAB; ++s)
          tma_load_4d(sV + st * SM::KV_TILE_BYTES + s * SM::SLAB_BYTES, &tma_v, &v_full[st], s * 64,
                      h, k0, b);
        ++it;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================================================ MMA issuer (warp-uniform flow)
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      const uint64_t q_desc[2] = {make_smem_desc(smem_u32(sQ), 16, 1024),
                                  make_smem_desc(smem_u32(sQ + SM::Q_TILE_BYTES), 16, 1024)};
      const uint64_t k_desc[2] = {make_smem_desc(smem_u32(sK), 16, 1024),
                                  make_smem_desc(smem_u32(sK + SM::KV_TILE_BYTES), 16, 1024)};
      const uint64_t v_desc[2] = {make_smem_desc(smem_u32(sV), SM::SLAB_BYTES, 1024),
                                  make_smem_desc(smem_u32(sV + SM::KV_TILE_BYTES), SM::SLAB_BYTES, 1024)};
      auto issue_s = [&](int w, int st) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SM::SLAB_BYTES + (kk & 3) * 32;
          if (leader)
            umma_ss(tS[w], desc_advance(q_desc[w], off), desc_advance(k_desc[st], off), idesc_s,
                    kk != 0 ? 1u : 0u);
        }
        if (leader) umma_commit(&s_full[w]);
      };
      auto issue_pv = [&](int w, int st, bool acc) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P_w in TMEM: 16 bf16 of K per step = 8 columns. B = V, MN-major: 16 kv rows = 2 KiB.
          if (leader)
            umma_ts(tO[w], tS[w] + kk * 8, desc_advance(v_desc[st], kk * 2048), idesc_o,
                    (acc || kk != 0) ? 1u : 0u);
        }
        if (leader) umma_commit(&o_done[w]);
      };
      auto next_visible = [&](int j, bool& v0, bool& v1) {
        const int a = next_vis(0, j), c = next_vis(1, j);
        const int jj = min(a, c);
        v0 = a == jj && jj < nk;
        v1 = c == jj && jj < nk;
        return jj;
      };
      bool ok = mbar_wait(q_full, 0, wc, kTimeoutSmemFull);
      bool v0, v1;
      int j = next_visible(0, v0, v1);
      int it = 0;
      int cnt[2] = {0, 0};
      if (ok && j < nk) {
        ok = mbar_wait(&k_full[0], 0, wc, kTimeoutSmemFull);
        if (ok) {
          tc_fence_after();
          if (v0) issue_s(0, 0);
          if (v1) issue_s(1, 0);
          if (leader) umma_commit(&k_empty[0]);
        }
      }
      while (ok && j < nk) {
        bool n0, n1;
        const int jn = next_visible(j + 1, n0, n1);
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int stn = (it + 1) & 1;
        const uint32_t phn = ((it + 1) >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph, wc, kTimeoutSmemFull)) break;
        bool k_ready = false;
        if (v0) {
          if (!mbar_wait(&p_full[0], cnt[0] & 1, wc, kTimeoutTmemFull)) break;
          tc_fence_after();
          issue_pv(0, st, cnt[0] != 0);
          ++cnt[0];
        }
        if (jn < nk && n0) {
          if (!mbar_wait(&k_full[stn], phn, wc, kTimeoutSmemFull)) break;
          k_ready = true;
          tc_fence_after();
          issue_s(0, stn);
        }
        if (v1) {
          if (!mbar_wait(&p_full[1], cnt[1] & 1, wc, kTimeoutTmemFull)) break;
          tc_fence_after();
          issue_pv(1, st, cnt[1] != 0);
          ++cnt[1];
        }
        if (leader) umma_commit(&v_empty[st]);
        if (jn < nk) {
          if (n1) {
            if (!k_ready && !mbar_wait(&k_full[stn], phn, wc, kTimeoutSmemFull)) break;
            tc_fence_after();
            issue_s(1, stn);
          }
          if (leader) umma_commit(&k_empty[stn]);
        }
        j = jn;
        v0 = n0;
        v1 = n1;
        ++it;
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ================================================================ softmax groups
    setmaxnreg_inc<FWD_REGS_SOFTMAX>();
    const int w = (warp - 4) >> 2;  // q tile handled by this group
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int wg_tid = quad * 32 + lane;
    const int qi0 = q0 + w * 128;
    const int qi = qi0 + row;
    const bool row_valid = qi < mk.Sq;
    const int qpos = mk.qmap(row_valid ? qi : mk.Sq - 1);
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int my_seg = (mk.seg_q && row_valid) ? mk.seg_q[static_cast<long long>(b) * mk.Sq + qi] : 0;
    const unsigned int bh_u = static_cast<unsigned int>(b * p.H + h);

    float m_ref = -INFINITY;  // running reference max (scaled log2 domain)
    float l = 0.f;
    int cnt = 0;
    bool alive = true;

    // every role walks the same visibility mask, so skips stay consistent
    for (int j = next_vis(w, 0); j < nk && alive; j = next_vis(w, j + 1)) {
      const int k0 = j * 128;
      const bool plain = tile_plain(mk, b, qi0, k0);
      if (!plain && (mk.seg_k || mk.bias)) {
        const int buf = cnt & 1;
        const int kc = k0 + wg_tid;
        if (mk.seg_k)
          sSeg[(w * 2 + buf) * 128 + wg_tid] =
              kc < mk.Sk ? mk.seg_k[static_cast<long long>(b) * mk.Sk + kc] : -1;
        if (mk.bias)
          sBias[(w * 2 + buf) * 128 + wg_tid] =
              kc < mk.Sk ? mk.bias[b * mk.bias_stride_b + h * mk.bias_stride_h + kc] * kLog2e : 0.f;
        named_bar_sync(1 + w, 128);
      }
      // A wait that gives up must end the loop for the whole warp (the TMEM loads and stores are
      // warp-collective). The lanes agree on that in the vote of the rescale check below, which exists
      // anyway; until then every lane carries on (a lane that gave up merely loads a stale tile).
      const bool s_ok = mbar_wait(&s_full[w], cnt & 1, wc, kTimeoutTmemFull);
      tc_fence_after();
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x32(tS[w] + lane_base + c * 32, sr + c * 32);
      tmem_ld_wait();

      float sc = p.scale_log2;  // multiplier still to be applied to sr[] inside the exp
      float mx = -INFINITY;
      if (plain) {
        float mc[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) mc[c] = fmaxf(__uint_as_float(sr[32 * c]), __uint_as_float(sr[32 * c + 1]));
#pragma unroll
        for (int i = 2; i < 32; i += 2) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            mc[c] = max3(mc[c], __uint_as_float(sr[32 * c + i]), __uint_as_float(sr[32 * c + i + 1]));
        }
        mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3])) * sc;
      } else {
        // keep[c] bit i: column 32c+i survives the causal rule, the sequence end and dropout. Built apart
        // from the element loop so that the (large) hash code is a small rolled loop that only runs when
        // dropout is on; the element loop itself stays a handful of instructions per column.
        const int limit = causal_col_limit(mk, qpos, k0);
        uint32_t keep[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = limit - 32 * c;
          keep[c] = n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
        }
        if (mk.keep) {
          uint4 kb = make_uint4(0u, 0u, 0u, 0u);
          if (RA_IN_BOUNDS((k0 >> 5), 4, mk.keep_sr, kTagAttnMaskBits))
            kb = *reinterpret_cast<const uint4*>(
              mk.keep + b * mk.keep_sb + h * mk.keep_sh + static_cast<long long>(row_valid ? qi : mk.Sq - 1) * mk.keep_sr +
              (k0 >> 5));
          keep[0] &= kb.x;
          keep[1] &= kb.y;
          keep[2] &= kb.z;
          keep[3] &= kb.w;
        }
        if (mk.drop_threshold) {
          const unsigned int kpos0 = static_cast<unsigned int>(mk.kmap(k0));
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t drop = 0;
#pragma unroll 1
            for (int i = 0; i < 32; ++i)
              drop |= static_cast<uint32_t>(dropout_hash(mk.seed_lo, mk.seed_hi, bh_u, static_cast<unsigned int>(qpos),
                                                         kpos0 + c * 32 + i) < mk.drop_threshold)
                      << i;
            keep[c] &= ~drop;
          }
        }
        const bool has_seg = mk.seg_k != nullptr, has_bias = mk.bias != nullptr;
        const int4* seg4 = reinterpret_cast<const int4*>(sSeg + (w * 2 + (cnt & 1)) * 128);
        const float4* bias4 = reinterpret_cast<const float4*>(sBias + (w * 2 + (cnt & 1)) * 128);
        float mc[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int g = 0; g < 32; ++g) {
          const int4 sg = has_seg ? seg4[g] : make_int4(my_seg, my_seg, my_seg, my_seg);
          const float4 bs = has_bias ? bias4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
          const int se[4] = {sg.x, sg.y, sg.z, sg.w};
          const float be[4] = {bs.x, bs.y, bs.z, bs.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = 4 * g + e;
            float x = fmaf(__uint_as_float(sr[i]), sc, be[e]);
            const bool masked = (((keep[i >> 5] >> (i & 31)) & 1u) == 0u) || (se[e] != my_seg);
            x = masked ? -INFINITY : x;
            sr[i] = __float_as_uint(x);
            mc[e] = fmaxf(mc[e], x);
          }
        }
        mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
        sc = 1.0f;
      }

      // ---- online softmax with lazy rescale of the accumulator
      const float m_new = fmaxf(m_ref, mx);
      // also true when m_ref is -inf and m_new is finite
      const bool need = cnt != 0 && m_new > m_ref + 8.0f;
      const bool rare = __any_sync(0xffffffffu, need || !s_ok);
      if (rare && __any_sync(0xffffffffu, !s_ok)) {
        alive = false;
        break;
      }
      if (cnt == 0) {
        m_ref = m_new;
      } else {
        if (rare) {
          if (!__all_sync(0xffffffffu, mbar_wait(&o_done[w], (cnt - 1) & 1, wc, kTimeoutTmemFull))) {
            alive = false;
            break;
          }
          tc_fence_after();
          const float alpha = (m_new == -INFINITY) ? 1.0f : exp2_approx(m_ref - m_new);
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_x32(tO[w] + lane_base + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tO[w] + lane_base + c * 32, o);
          }
          tmem_st_wait();
          l *= alpha;
          m_ref = m_new;
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      const uint64_t neg_m2 = f2_pack(-m_use, -m_use);
      const uint64_t sc2 = f2_pack(sc, sc);
      uint64_t sum2 = f2_pack(0.f, 0.f);
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        float x0, x1;
        f2_unpack(f2_fma(f2_pack_u(sr[2 * i], sr[2 * i + 1]), sc2, neg_m2), x0, x1);
        const float p0 = exp2_approx(x0), p1 = exp2_approx(x1);
        sum2 = f2_add(sum2, f2_pack(p0, p1));
        pk[i] = pack_bf16x2(p0, p1);
      }
      float sum, sum_hi;
      f2_unpack(sum2, sum, sum_hi);
      sum += sum_hi;
      l += sum;
      tmem_st_x32(tS[w] + lane_base, pk);
      tmem_st_x32(tS[w] + lane_base + 32, pk + 32);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[w]);
      ++cnt;
    }

    // ---- epilogue: normalise, merge with carry, store
    if (alive && cnt > 0) alive = mbar_wait(&o_done[w], (cnt - 1) & 1, wc, kTimeoutTmemFull);
    tc_fence_after();
    float inv_l = 0.f;
    float lse = -INFINITY;
    if (cnt > 0 && l > 0.f) {
      inv_l = 1.0f / l;
      lse = (m_ref + log2f(l)) * kLn2;
    }
    float w_prev = 0.f, w_this = 1.f;
    const long long lse_idx = (static_cast<long long>(b) * p.H + h) * mk.Sq + qi;
    if (p.o_prev && row_valid) {
      const float lp = p.lse_prev[lse_idx];
      const float mxl = fmaxf(lp, lse);
      if (mxl == -INFINITY) {
        w_prev = 0.f;
        w_this = 0.f;
      } else {
        const float ep = __expf(lp - mxl), et = __expf(lse - mxl);
        const float tot = ep + et;
        w_prev = ep / tot;
        w_this = et / tot;
        lse = mxl + __logf(tot);
      }
    }
    if (row_valid && RA_IN_BOUNDS(lse_idx, 1, static_cast<long long>(p.B) * p.H * mk.Sq, kTagAttnFwdLse))
      p.lse_out[lse_idx] = lse;
    const float mul = inv_l * w_this;
    const float* oprev_row =
        p.o_prev ? p.o_prev + ((static_cast<long long>(b) * mk.Sq + qi) * p.H + h) * D : nullptr;
    const long long o_off = b * p.o_stride_b + static_cast<long long>(qi) * p.o_stride_s + h * p.o_stride_h;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      if (cnt > 0) {
        tmem_ld_x32(tO[w] + lane_base + c * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (row_valid && RA_IN_BOUNDS(qi, 1, mk.Sq, kTagAttnFwdOut) && RA_IN_BOUNDS(c * 32, 32, D, kTagAttnFwdOut)) {
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(o[i]) * mul;
        if (oprev_row) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 pv = *reinterpret_cast<const float4*>(oprev_row + c * 32 + 4 * i);
            f[4 * i] += pv.x * w_prev;
            f[4 * i + 1] += pv.y * w_prev;
            f[4 * i + 2] += pv.z * w_prev;
            f[4 * i + 3] += pv.w * w_prev;
          }
        }
        if (p.out_fp32) {
          float* dst = reinterpret_cast<float*>(p.out) + o_off + c * 32;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(dst + 4 * i) =
                make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + o_off + c * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(f[8 * i], f[8 * i + 1]);
            v.y = pack_bf16x2(f[8 * i + 2], f[8 * i + 3]);
            v.z = pack_bf16x2(f[8 * i + 4], f[8 * i + 5]);
            v.w = pack_bf16x2(f[8 * i + 6], f[8 * i + 7]);
            *reinterpret_cast<uint4*>(dst + 8 * i) = v;
          }
        }
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

}  // namespace attn
}  // namespace ra

namespace {
// (B, S, H, D) bf16 view with element strides -> 4-D map (d, h, s, b), box 64 x 1 x 128 x 1.
int make_bshd_map(CUtensorMap* m, const void* base, int B, int S, int H, int D, long long sb,
                  long long ss, long long sh) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                      static_cast<uint64_t>(B)};
  uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(ss) * 2,
                     static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return ra::make_tmap_bf16_sw128(m, base, 4, dims, str, box);
}
}  // namespace

struct RaAttnFwdArgs {
  const void* q; const void* k; const void* v;
  long long q_sb, q_ss, q_sh;   // element strides of (B, Sq, H, D) views; D contiguous
  long long k_sb, k_ss, k_sh;
  long long v_sb, v_ss, v_sh;
  void* out; long long o_sb, o_ss, o_sh; int out_fp32;
  float* lse_out;
  const float* o_prev; const float* lse_prev;
  int B, H, Sq, Sk, D;
  float softmax_scale;          // 1/sqrt(D)
  int causal_block_size;
  int q_off0, q_off1, q_half;
  int k_off0, k_off1, k_half;
  const int* seg_q; const int* seg_k; const int* seg_q_mm; const int* seg_k_mm;
  const float* bias; long long bias_sb, bias_sh;
  unsigned long long seed; unsigned int drop_threshold;
  const unsigned int* keep; long long keep_sb, keep_sh, keep_sr;  // boolean mask bitmap by query row, or null
  const void* copy_src; void* copy_dst; long long copy_bytes; int copy_ctas;
  int* status;
  void* stream;
};

extern "C" int ra_attn_fwd(const RaAttnFwdArgs* a) {
  using namespace ra;
  using namespace ra::attn;
  if (a->D != 128 && a->D != 64) {
    set_error("ra_attn_fwd: head_dim must be 64 or 128");
    return kHostBadArg;
  }
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Sk <= 0 || (a->q_half < a->Sq && a->q_half % 128) ||
      (a->k_half < a->Sk && a->k_half % 128) || (a->copy_bytes % 16)) {
    set_error("ra_attn_fwd: bad shape");
    return kHostBadArg;
  }
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_bshd_map(&tq, a->q, a->B, a->Sq, a->H, a->D, a->q_sb, a->q_ss, a->q_sh))) return rc;
  if ((rc = make_bshd_map(&tk, a->k, a->B, a->Sk, a->H, a->D, a->k_sb, a->k_ss, a->k_sh))) return rc;
  if ((rc = make_bshd_map(&tv, a->v, a->B, a->Sk, a->H, a->D, a->v_sb, a->v_ss, a->v_sh))) return rc;
  FwdParams p;
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
  if (a->keep && ((a->keep_sr % 4) || (a->keep_sb % 4) || (a->keep_sh % 4) || (reinterpret_cast<uintptr_t>(a->keep) & 15))) {
    set_error("ra_attn_fwd: mask bitmap rows must be 16-byte aligned");
    return kHostBadArg;
  }
  p.scale_log2 = a->softmax_scale * kLog2e;
  p.out = a->out;
  p.out_fp32 = a->out_fp32;
  p.o_stride_b = a->o_sb;
  p.o_stride_s = a->o_ss;
  p.o_stride_h = a->o_sh;
  p.lse_out = a->lse_out;
  p.o_prev = a->o_prev;
  p.lse_prev = a->lse_prev;
  p.copy_src = reinterpret_cast<const uint4*>(a->copy_src);
  p.copy_dst = reinterpret_cast<uint4*>(a->copy_dst);
  p.copy_n16 = a->copy_bytes / 16;
  p.copy_ctas = (a->copy_src && a->copy_bytes > 0) ? a->copy_ctas : 0;
  p.status = a->status;
  const int n_qpairs = (a->Sq + 255) / 256;
  const long long grid = static_cast<long long>(n_qpairs) * a->H * a->B + p.copy_ctas;
  cudaStream_t s = static_cast<cudaStream_t>(a->stream);
  cudaError_t e;
  if (a->D == 128) {
    auto kern = attn_fwd_kernel<128>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<128>::TOTAL);
    if (e != cudaSuccess) { set_error("attn_fwd: smem attribute"); return kHostLaunchFail; }
    kern<<<static_cast<unsigned>(grid), FWD_THREADS, FwdSmem<128>::TOTAL, s>>>(tq, tk, tv, p);
  } else {
    auto kern = attn_fwd_kernel<64>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<64>::TOTAL);
    if (e != cudaSuccess) { set_error("attn_fwd: smem attribute"); return kHostLaunchFail; }
    kern<<<static_cast<unsigned>(grid), FWD_THREADS, FwdSmem<64>::TOTAL, s>>>(tq, tk, tv, p);
  }
  return check_launch("attn_fwd_kernel");
}
