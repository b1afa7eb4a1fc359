// Decode attention over a sequence-sharded KV cache that stays where it is.
//
// The reference's inference op rotates the whole KV cache around the ring for every call
// (ringattention/ringattention_inference.py:17-33). Here each GPU reads its own shard exactly once:
//   1. decode_splitkv_kernel : the shard is cut into `splits` row ranges, one CTA per (range, head,
//      batch). A few query rows (QL <= 8) are held in registers; K/V stream from HBM as 16-byte pieces
//      through a per-thread cp.async ring; online softmax in fp32; each CTA emits a partial (o, lse)
//      for its range. One query row: a batched GEMV on the CUDA cores at the speed of a plain copy.
//      decode_splitkv_mma_kernel is the same pass for 2-8 query rows (streams sharing a cache) with the
//      query rows as the M side of mma.sync m16n8k16, per-warp cp.async ring and ldmatrix.
//   2. decode_merge_kernel   : merges partials with log-sum-exp weights. decode_merge_exchange_kernel
//      does that for a ring in one launch: the merged per-GPU result is *stored into every peer's
//      inbox* (plain stores to peer memory), a per-row flag is released on every rank, and after a
//      bounded wait for the same row of every rank the N per-GPU partials are merged; every rank ends
//      up with the identical result, as the reference's rotation would give.
// The file also holds the other kernels of a decode step: the weight-streaming linears for a handful of
// rows (CUDA cores with RMSNorm / SwiGLU prologues for one row, mma.sync for 2-8 rows), RoPE + cache
// append, and the device-side step counters that make the step replayable as one CUDA graph.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/bounds.cuh"
#include "common/host_util.h"
#include "common/sm100.cuh"

RA_BOUNDS_TRANSLATION_UNIT()

namespace ra {
namespace decode {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;

struct SplitParams {
  const __nv_bfloat16* q;  // (B, QL, H, D) contiguous
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  long long k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;  // element strides of the (B, S, H, D) cache views
  float* o_part;    // (B, H, QL, splits, D) fp32, normalised partial outputs
  float* lse_part;  // (B, H, QL, splits)
  const uint8_t* mask;  // (B, Hm, QL, S) nonzero = attend, or null
  long long m_sb, m_sh, m_sq;
  int B, H, S;      // S = number of local cache rows to visit
  int splits, rows_per_split;
  float scale_log2;
  long long q_pos0;  // global position of query row 0, or < 0 for no causal rule
  long long k_pos0;  // global position of local cache row 0
  const long long* pos_ptr;  // optional: the query position lives on the device (CUDA-graph decode);
                             // then q_pos0 = *pos_ptr and the rows to visit are [0, min(S, *pos_ptr + 1 - k_pos0))
  // Striped cache (stripe_n > 0, with pos_ptr): the first stripe_base rows of every rank hold the prefilled
  // context (positions < stripe_len0, all visible); decoded token i = position - stripe_len0 lives on rank
  // i % stripe_n at row stripe_base + i / stripe_n. No causal rule is needed: every stored row is in the past.
  int stripe_n, stripe_rank;
  long long stripe_base, stripe_len0;
};

// Rows of this rank that hold tokens up to and including position `pos` in the striped layout.
__device__ __forceinline__ long long striped_rows(long long pos, int n, int rank, long long base, long long len0) {
  const long long i = pos - len0;
  return base + (i >= 0 ? (i + n - rank) / n : 0);
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// 16-byte asynchronous copy global -> shared; `bytes` = 0 writes zeros without reading the source.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int DEC_UNROLL = 4;  // cache rows per thread and loop trip

// D = head dim (64 or 128), QL = query rows held per CTA, ST = stages of the asynchronous-copy ring (0: the rows
// of a trip are loaded straight into registers). With ST > 0 every thread copies the rows of trip i + ST - 1 into
// its own shared-memory slots (cp.async, no registers held while the data is in flight) before it works on trip
// i, so memory requests are outstanding during the arithmetic too; a thread only ever reads what it copied itself,
// hence cp.async.wait_group is all the synchronisation needed. Dynamic shared memory: ST * 4 rows * 32 bytes per
// thread.
template <int D, int QL, int ST>
__global__ void __launch_bounds__(THREADS) decode_splitkv_kernel(const SplitParams p) {
  constexpr int LPR = D / 8;        // lanes per cache row (16 bytes per lane)
  constexpr int RPW = 32 / LPR;     // rows per warp step
  constexpr int UNROLL = DEC_UNROLL;  // cache rows in flight per thread (8 made it slower: 4.6 vs 5.2 TB/s, fewer CTAs per SM)
  extern __shared__ uint4 stage_buf[];  // [ST][UNROLL][k|v][THREADS]
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, dl = lane % LPR;  // which row of the step, which 8-wide slice of D

  float qf[QL][8];
#pragma unroll
  for (int i = 0; i < QL; ++i) {
    const uint4 u = *reinterpret_cast<const uint4*>(p.q + ((static_cast<long long>(b) * QL + i) * p.H + h) * D + dl * 8);
    unpack8(u, qf[i]);
#pragma unroll
    for (int e = 0; e < 8; ++e) qf[i][e] *= p.scale_log2;
  }
  float acc[QL][8];
  float m[QL], l[QL];
#pragma unroll
  for (int i = 0; i < QL; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  }

  long long q_pos0 = p.q_pos0;
  int S = p.S, rows_per_split = p.rows_per_split;
  if (p.pos_ptr) {
    q_pos0 = *p.pos_ptr;
    long long n = q_pos0 + 1 - p.k_pos0;
    if (p.stripe_n > 0) {
      n = striped_rows(q_pos0, p.stripe_n, p.stripe_rank, p.stripe_base, p.stripe_len0);
      q_pos0 = -1;
    }
    S = static_cast<int>(n < 0 ? 0 : (n > p.S ? p.S : n));
    rows_per_split = (S + p.splits - 1) / p.splits;
    if (rows_per_split < 1) rows_per_split = 1;
  }
  const int r0 = split * rows_per_split;
  const int r1 = min(S, r0 + rows_per_split);
  const __nv_bfloat16* kb = p.k + b * p.k_sb + h * p.k_sh + dl * 8;
  const __nv_bfloat16* vb = p.v + b * p.v_sb + h * p.v_sh + dl * 8;
  const int step = WARPS * RPW;

  // The trip count is the same for every lane of a warp (the loop variable ignores `sub`), so the
  // full-mask shuffles below always see all 32 lanes; rows past the end are merely masked out.
  // stage `slot` <- the rows of the trip that starts at row base_w (of this warp)
  auto issue = [&](int base_w, int slot) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int r = base_w + sub + u * step;
      const bool in = r < r1;
      const long long rr = in ? r : r0;  // r0 < r1 whenever the loop runs: a valid address, never read when !in
      uint4* dst = stage_buf + ((slot * UNROLL + u) * 2) * THREADS + threadIdx.x;
      cp_async16(dst, kb + rr * p.k_ss, in ? 16 : 0);
      cp_async16(dst + THREADS, vb + rr * p.v_ss, in ? 16 : 0);
    }
  };
  int ahead_w = r0 + warp * RPW, slot_in = 0, slot_out = 0;
  if (ST > 0) {
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
      if (ahead_w < r1) issue(ahead_w, slot_in);
      cp_async_commit();  // one group per trip, empty or not, so that the group count below is a constant
      ahead_w += step * UNROLL;
      slot_in = slot_in + 1 == ST ? 0 : slot_in + 1;
    }
  }
  for (int base_w = r0 + warp * RPW; base_w < r1; base_w += step * UNROLL) {
    const int base = base_w + sub;
    uint4 ku[UNROLL], vu[UNROLL];
    bool ok[UNROLL];
    if (ST > 0) {
      if (ahead_w < r1) issue(ahead_w, slot_in);
      cp_async_commit();
      ahead_w += step * UNROLL;
      slot_in = slot_in + 1 == ST ? 0 : slot_in + 1;
      cp_async_wait<(ST > 0 ? ST - 1 : 0)>();  // all but the newest ST - 1 groups are complete: this trip's rows are in
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        ok[u] = base + u * step < r1;
        const uint4* src = stage_buf + ((slot_out * UNROLL + u) * 2) * THREADS + threadIdx.x;
        ku[u] = src[0];
        vu[u] = src[THREADS];
      }
      slot_out = slot_out + 1 == ST ? 0 : slot_out + 1;
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int r = base + u * step;
        ok[u] = r < r1;
        if (ok[u]) {
          ku[u] = *reinterpret_cast<const uint4*>(kb + static_cast<long long>(r) * p.k_ss);
          vu[u] = *reinterpret_cast<const uint4*>(vb + static_cast<long long>(r) * p.v_ss);
        } else {
          ku[u] = make_uint4(0, 0, 0, 0);
          vu[u] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    float s[UNROLL][QL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float kf[8];
      unpack8(ku[u], kf);
      const int r = base + u * step;
#pragma unroll
      for (int i = 0; i < QL; ++i) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qf[i][e], kf[e], d);
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        bool vis = ok[u];
        if (q_pos0 >= 0) vis = vis && (p.k_pos0 + r <= q_pos0 + i);
        if (p.mask && vis)
          vis = p.mask[b * p.m_sb + h * p.m_sh + i * p.m_sq + r] != 0;
        s[u][i] = vis ? d : -INFINITY;
      }
    }
#pragma unroll
    for (int i = 0; i < QL; ++i) {
      float mx = m[i];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) mx = fmaxf(mx, s[u][i]);
      const float m_use = mx == -INFINITY ? 0.f : mx;
      const float alpha = exp2f(m[i] - m_use);  // 0 when m is -inf
      l[i] *= alpha;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] *= alpha;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const float pr = exp2f(s[u][i] - m_use);
        l[i] += pr;
        float vf[8];
        unpack8(vu[u], vf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(pr, vf[e], acc[i][e]);
      }
      m[i] = mx;
    }
  }

  if (ST > 0) cp_async_wait<0>();  // only empty groups can be left; nothing is in flight when the CTA ends
  // ---- combine the row groups of a warp, then the warps of the CTA
  __shared__ float sm_m[WARPS][QL], sm_l[WARPS][QL];
  __shared__ float sm_o[WARPS][QL][D];
#pragma unroll
  for (int i = 0; i < QL; ++i) {
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[i], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[i], o);
      const float mx = fmaxf(m[i], m2);
      const float mu = mx == -INFINITY ? 0.f : mx;
      const float a1 = exp2f(m[i] - mu), a2 = exp2f(m2 - mu);
      l[i] = l[i] * a1 + l2 * a2;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float o2 = __shfl_xor_sync(0xffffffffu, acc[i][e], o);
        acc[i][e] = acc[i][e] * a1 + o2 * a2;
      }
      m[i] = mx;
    }
    if (sub == 0) {
      if (dl == 0) {
        sm_m[warp][i] = m[i];
        sm_l[warp][i] = l[i];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sm_o[warp][i][dl * 8 + e] = acc[i][e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < QL * D; idx += THREADS) {
    const int i = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, sm_m[w][i]);
    const float mu = mx == -INFINITY ? 0.f : mx;
    float lt = 0.f, ot = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float a = exp2f(sm_m[w][i] - mu);
      lt += sm_l[w][i] * a;
      ot += sm_o[w][i][d] * a;
    }
    const long long pi = ((static_cast<long long>(b) * p.H + h) * QL + i) * p.splits + split;
    p.o_part[pi * D + d] = lt > 0.f ? ot / lt : 0.f;
    if (d == 0) p.lse_part[pi] = lt > 0.f ? (mx + log2f(lt)) * 0.6931471805599453f : -INFINITY;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same split-KV pass on the tensor cores, for calls with several query rows per cache row (shared-prefix
// streams, short speculative or multi-token steps). With q rows the CUDA-core kernel above spends q times the
// instructions per cache row and becomes bound by its instruction stream (four rows: twice the time of one).
// Here the <= 8 query rows are the M side of a 16 x 8 x 16 MMA (rows 8..15 are zero), the cache rows its N side:
//   S (16 x 16 kv)  = Q (16 x D) K_chunk^T        2 n-tiles x D/16 k-steps, B fragments by ldmatrix
//   O (16 x D)     += P (16 x 16 kv) V_chunk      D/8 n-tiles, B fragments by ldmatrix.trans, P from the S fragments
// so a chunk of 16 cache rows costs 2 * D/8 MMAs and D/8 ldmatrix whatever the number of query rows. Every warp walks
// its own chunks and stages them through its own three-stage cp.async ring in shared memory (16-byte pieces,
// XOR-swizzled by the row so that ldmatrix is conflict-free); only __syncwarp() is needed around a stage. The legacy
// mma.sync path is the right size here: the kernel is bound by HBM, a 128-row tcgen05 tile would bring nothing but a
// longer hand-off chain per tile.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
// d += a * b for m16n8k16, bf16 inputs, fp32 accumulation; rows 8..15 of a are zero (a1 = a3 = 0)
__device__ __forceinline__ void mma_16816_top(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

constexpr int MMA_ST = 3;       // stages of a warp's ring
constexpr int MMA_ROWS = 16;    // cache rows per chunk

template <int D>
__global__ void __launch_bounds__(THREADS) decode_splitkv_mma_kernel(const SplitParams p, int QL) {
  constexpr int RB = D * 2;                 // bytes per cache row
  constexpr int PPR = D / 8;                // 16-byte pieces per row
  constexpr int TILE = MMA_ROWS * RB;       // bytes of a K (or V) chunk
  constexpr int NT = D / 8;                 // n-tiles of O
  extern __shared__ uint4 mma_ring[];       // [WARPS][MMA_ST][K tile | V tile]
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;    // fragment coordinates: query row g, column pair t
  uint8_t* ring = reinterpret_cast<uint8_t*>(mma_ring) + warp * (MMA_ST * 2 * TILE);

  long long q_pos0 = p.q_pos0;
  int S = p.S, rows_per_split = p.rows_per_split;
  if (p.pos_ptr) {
    q_pos0 = *p.pos_ptr;
    long long n = q_pos0 + 1 - p.k_pos0;
    if (p.stripe_n > 0) {
      n = striped_rows(q_pos0, p.stripe_n, p.stripe_rank, p.stripe_base, p.stripe_len0);
      q_pos0 = -1;
    }
    S = static_cast<int>(n < 0 ? 0 : (n > p.S ? p.S : n));
    rows_per_split = (S + p.splits - 1) / p.splits;
    if (rows_per_split < 1) rows_per_split = 1;
  }
  const int r0 = split * rows_per_split;
  const int r1 = min(S, r0 + rows_per_split);
  const __nv_bfloat16* kb = p.k + b * p.k_sb + h * p.k_sh;
  const __nv_bfloat16* vb = p.v + b * p.v_sb + h * p.v_sh;

  // Q fragments: a0 = Q[g][16ks + 2t, +1], a2 = Q[g][16ks + 8 + 2t, +1]; rows >= QL are zero
  uint32_t qa[D / 16][2];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    qa[ks][0] = qa[ks][1] = 0u;
    if (g < QL) {
      const __nv_bfloat16* qr = p.q + ((static_cast<long long>(b) * QL + g) * p.H + h) * D + 16 * ks + 2 * t;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qr);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(qr + 8);
    }
  }
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m = -INFINITY, l = 0.f;  // of query row g; l is this lane's share of the row sum

  // chunk c of this warp starts at row r0 + (warp + WARPS * c) * 16
  auto issue = [&](int c, int slot) {
    const int base = r0 + (warp + WARPS * c) * MMA_ROWS;
    uint8_t* kt = ring + slot * 2 * TILE;
#pragma unroll
    for (int j = 0; j < MMA_ROWS * PPR / 32; ++j) {
      const int piece = lane + 32 * j;
      const int row = piece / PPR, ch = piece % PPR;
      const int r = base + row;
      const bool in = r < r1;
      const long long rr = in ? r : r0;  // a valid address; not read when !in (the piece is zero-filled)
      const int off = row * RB + ((ch ^ (row & 7)) << 4);
      cp_async16(kt + off, kb + rr * p.k_ss + ch * 8, in ? 16 : 0);
      cp_async16(kt + TILE + off, vb + rr * p.v_ss + ch * 8, in ? 16 : 0);
    }
  };
  const int my_rows = r1 - (r0 + warp * MMA_ROWS);
  const int n_chunks = my_rows <= 0 ? 0 : (my_rows + WARPS * MMA_ROWS - 1) / (WARPS * MMA_ROWS);
#pragma unroll
  for (int i = 0; i < MMA_ST - 1; ++i) {
    if (i < n_chunks) issue(i, i);
    cp_async_commit();  // one group per chunk, empty or not: the group count in the wait below is a constant
  }
  int slot = 0;
  for (int c = 0; c < n_chunks; ++c) {
    __syncwarp();  // every lane is done with the stage that is filled next
    if (c + MMA_ST - 1 < n_chunks) issue(c + MMA_ST - 1, (slot + MMA_ST - 1) % MMA_ST);
    cp_async_commit();
    cp_async_wait<MMA_ST - 1>();
    __syncwarp();  // the other lanes' pieces of chunk c are in too
    const uint8_t* kt = ring + slot * 2 * TILE;
    const uint8_t* vt = kt + TILE;
    const int base = r0 + (warp + WARPS * c) * MMA_ROWS;

    // ---- S = Q K^T: s[nt] holds row g, cache rows base + 8 nt + 2t, +1
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
    {
      const int mat = lane >> 3, rr = lane & 7;
      const int row = rr + 8 * (mat >> 1);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int ch = 2 * ks + (mat & 1);
        uint32_t bf[4];
        ldmatrix_x4(bf, kt + row * RB + ((ch ^ (row & 7)) << 4));
        mma_16816_top(s[0], qa[ks][0], qa[ks][1], bf[0], bf[1]);
        mma_16816_top(s[1], qa[ks][0], qa[ks][1], bf[2], bf[3]);
      }
    }
    // ---- mask, online softmax of row g over the 16 cache rows
    float x[2][2];
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int r = base + 8 * nt + 2 * t + e;
        bool vis = r < r1 && g < QL;
        if (q_pos0 >= 0) vis = vis && (p.k_pos0 + r <= q_pos0 + g);
        if (p.mask && vis) vis = p.mask[b * p.m_sb + h * p.m_sh + g * p.m_sq + r] != 0;
        x[nt][e] = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, x[nt][e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = exp2f(m - m_use);  // 0 when m is -inf
    float pr[2][2];
    float psum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[nt][e] = exp2f(x[nt][e] - m_use);
        psum += pr[nt][e];
      }
    l = l * alpha + psum;
    m = m_new;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= alpha;
      o[j][1] *= alpha;
    }
    // ---- O += P V: P as the A fragment (a0: cache rows 2t, 2t+1; a2: rows 8 + 2t, +1)
    __nv_bfloat162 p0 = __floats2bfloat162_rn(pr[0][0], pr[0][1]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(pr[1][0], pr[1][1]);
    const uint32_t a0 = *reinterpret_cast<uint32_t*>(&p0), a2 = *reinterpret_cast<uint32_t*>(&p1);
    {
      const int mat = lane >> 3, rr = lane & 7;
      const int row = rr + 8 * (mat & 1);
#pragma unroll
      for (int j = 0; j < NT / 2; ++j) {
        const int ch = 2 * j + (mat >> 1);
        uint32_t bf[4];
        ldmatrix_x4_trans(bf, vt + row * RB + ((ch ^ (row & 7)) << 4));
        mma_16816_top(o[2 * j], a0, a2, bf[0], bf[1]);
        mma_16816_top(o[2 * j + 1], a0, a2, bf[2], bf[3]);
      }
    }
    slot = slot + 1 == MMA_ST ? 0 : slot + 1;
  }
  cp_async_wait<0>();  // only empty groups can be left

  // ---- the row sum over the four lanes of a row, then the warps of the CTA (as in the kernel above)
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  __shared__ float sm_m[WARPS][8], sm_l[WARPS][8];
  __shared__ float sm_o[WARPS][8][D];
  if (t == 0) {
    sm_m[warp][g] = m;
    sm_l[warp][g] = l;
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    sm_o[warp][g][8 * j + 2 * t] = o[j][0];
    sm_o[warp][g][8 * j + 2 * t + 1] = o[j][1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < QL * D; idx += THREADS) {
    const int i = idx / D, d = idx % D;
    float mxw = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mxw = fmaxf(mxw, sm_m[w][i]);
    const float mu = mxw == -INFINITY ? 0.f : mxw;
    float lt = 0.f, ot = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float a = exp2f(sm_m[w][i] - mu);
      lt += sm_l[w][i] * a;
      ot += sm_o[w][i][d] * a;
    }
    const long long pi = ((static_cast<long long>(b) * p.H + h) * QL + i) * p.splits + split;
    p.o_part[pi * D + d] = lt > 0.f ? ot / lt : 0.f;
    if (d == 0) p.lse_part[pi] = lt > 0.f ? (mxw + log2f(lt)) * 0.6931471805599453f : -INFINITY;
  }
}

struct MergeParams {
  const float* o_part;    // element (row, part, d) at row*o_rs + part*o_ps + d
  const float* lse_part;  // element (row, part) at row*l_rs + part*l_ps
  long long o_rs, o_ps, l_rs, l_ps;
  int rows, nparts, D, H, QL;  // QL = 0: rows are already in output order (b, t, h)
  void* out;              // (B, QL, H, D) bf16 or fp32, or null
  int out_fp32;
  float* lse_out;         // (rows) or null
  // ring variant: store this GPU's merged partial into slot `my_rank` of every rank's inbox
  float* const* inbox_o;    // [n_ranks] pointers to (rows, n_ranks, D)
  float* const* inbox_lse;  // [n_ranks] pointers to (rows, n_ranks)
  int n_ranks, my_rank;
  // optional double-buffer selection from a device-side step counter (CUDA-graph decode): slot =
  // (*step_ptr * slot_mul + slot_add) & 1 is applied to the inbox stores (out_slot_*) and to the partials read
  // (in_slot_*): slot_mul = exchanges per decode step, slot_add = index of this exchange within the step, so
  // that consecutive exchanges always alternate slots
  const long long* step_ptr;
  long long slot_mul, slot_add;
  long long out_slot_o, out_slot_l, in_slot_o, in_slot_l;  // strides in floats
};

// One CTA per row = (b, h, i); D threads.
__global__ void decode_merge_kernel(const MergeParams p) {
  const int row = blockIdx.x, d = threadIdx.x;
  const long long slot = p.step_ptr ? ((*p.step_ptr * p.slot_mul + p.slot_add) & 1) : 0;
  const float* o_in = p.o_part + slot * p.in_slot_o;
  const float* lp = p.lse_part + slot * p.in_slot_l + static_cast<long long>(row) * p.l_rs;
  float mx = -INFINITY;
  for (int s = 0; s < p.nparts; ++s) mx = fmaxf(mx, lp[s * p.l_ps]);
  float wsum = 0.f, o = 0.f;
  if (mx != -INFINITY) {
    for (int s = 0; s < p.nparts; ++s) {
      const float w = __expf(lp[s * p.l_ps] - mx);
      wsum += w;
      o += w * o_in[static_cast<long long>(row) * p.o_rs + s * p.o_ps + d];
    }
    o /= wsum;
  }
  const float lse = mx == -INFINITY ? -INFINITY : mx + __logf(wsum);
  if (p.inbox_o) {
    for (int r = 0; r < p.n_ranks; ++r) {
      p.inbox_o[r][slot * p.out_slot_o + (static_cast<long long>(row) * p.n_ranks + p.my_rank) * p.D + d] = o;
      if (d == 0) p.inbox_lse[r][slot * p.out_slot_l + static_cast<long long>(row) * p.n_ranks + p.my_rank] = lse;
    }
    __threadfence_system();
  }
  if (p.out) {
    // row = (b*H + h)*QL + i  ->  out[b, i, h, d]
    long long oi = static_cast<long long>(row) * p.D + d;
    if (p.QL > 0) {
      const int i = row % p.QL, h = (row / p.QL) % p.H, b = row / (p.QL * p.H);
      oi = ((static_cast<long long>(b) * p.QL + i) * p.H + h) * p.D + d;
    }
    if (!RA_IN_BOUNDS(oi, 1, static_cast<long long>(gridDim.x) * p.D, kTagDecodeMerge)) {
    } else if (p.out_fp32)
      reinterpret_cast<float*>(p.out)[oi] = o;
    else
      reinterpret_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16(o);
  }
  if (p.lse_out && d == 0) {
    // like `out`: row (b, h, i) of a decode call goes to position (b, i, h), so that the merged values of calls with
    // different (B, QL) splits of the same queries line up
    long long li = row;
    if (p.QL > 0) {
      const int i = row % p.QL, h = (row / p.QL) % p.H, b = row / (p.QL * p.H);
      li = (static_cast<long long>(b) * p.QL + i) * p.H + h;
    }
    p.lse_out[li] = lse;
  }
}

// The whole cross-GPU merge of a decode step in one launch: merge this GPU's split partials of a row, store the
// result into slot `my_rank` of every rank's inbox (peer stores), tell every rank that this row has arrived, wait
// until the same row of every rank has arrived here, and merge those. Synchronisation is per row: CTA `row` of
// rank a only ever waits for CTA `row` of the other ranks, and every CTA signals before it waits, so the launch
// cannot deadlock as long as all its CTAs are resident at once (the launcher refuses larger grids). The wait is
// bounded: after `timeout_ns` the CTA records kTimeoutPeerFlag in the status word and finishes with what is there.
//   epoch    = *epoch_ptr + 1: counts the launches of this kernel on the ring (same on every rank); the last CTA to
//              finish stores it back, so a launch recorded in a CUDA graph works on every replay
//   slot     = epoch & 1: the inbox is double-buffered. A rank can be at most one exchange ahead of another (it
//              needs that rank's flag of the previous exchange to get further), so two slots are enough
//   flags[r] = rank r's (max_rows, n_ranks) words; word (row, src) holds the last epoch whose row `row` from
//              rank `src` is complete in r's inbox
struct ExchangeParams {
  MergeParams m;  // stage 1 inputs, inbox pointer tables, ranks, final `out` and its row mapping
  uint32_t* const* flags;
  uint32_t* epoch_ptr;
  unsigned int* done_ctr;
  const float* inbox_o_local;  // this rank's inbox: 2 slots of (rows, n_ranks, D) / (rows, n_ranks)
  const float* inbox_l_local;
  long long slot_rows;  // rows per inbox slot (the same for every launch on the ring, whatever its own row count)
  unsigned long long timeout_ns;
  int* status;
};

__global__ void decode_merge_exchange_kernel(const ExchangeParams e) {
  const MergeParams& p = e.m;
  const int row = blockIdx.x, d = threadIdx.x, n = p.n_ranks;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(e.epoch_ptr) + 1u;
  const long long slot = epoch & 1u;
  // ---- stage 1: this GPU's splits
  const float* lp = p.lse_part + static_cast<long long>(row) * p.l_rs;
  float mx = -INFINITY;
  for (int s = 0; s < p.nparts; ++s) mx = fmaxf(mx, lp[s * p.l_ps]);
  float wsum = 0.f, o = 0.f;
  if (mx != -INFINITY) {
    for (int s = 0; s < p.nparts; ++s) {
      const float w = __expf(lp[s * p.l_ps] - mx);
      wsum += w;
      o += w * p.o_part[static_cast<long long>(row) * p.o_rs + s * p.o_ps + d];
    }
    o /= wsum;
  }
  const float lse = mx == -INFINITY ? -INFINITY : mx + __logf(wsum);
  const long long slot_o = slot * e.slot_rows * n * p.D, slot_l = slot * e.slot_rows * n;
  for (int r = 0; r < n; ++r) {
    p.inbox_o[r][slot_o + (static_cast<long long>(row) * n + p.my_rank) * p.D + d] = o;
    if (d == 0) p.inbox_lse[r][slot_l + static_cast<long long>(row) * n + p.my_rank] = lse;
  }
  __threadfence_system();
  __syncthreads();
  // ---- signal every rank, then wait for every rank's copy of this row
  if (d < n) {
    uint32_t* remote = e.flags[d] + static_cast<long long>(row) * n + p.my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* mine = e.flags[p.my_rank] + static_cast<long long>(row) * n + d;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if (((++it) & 255u) == 0u && globaltimer_ns() - t0 > e.timeout_ns) {
        if (e.status) atomicCAS(e.status, 0, static_cast<int>(kTimeoutPeerFlag));
        break;
      }
      __nanosleep(100);
    }
    __threadfence_system();
  }
  __syncthreads();
  // ---- stage 2: the ranks' partials of this row (written by peers: read past L1)
  const float* il = e.inbox_l_local + slot_l + static_cast<long long>(row) * n;
  const float* io = e.inbox_o_local + slot_o + static_cast<long long>(row) * n * p.D;
  mx = -INFINITY;
  for (int r = 0; r < n; ++r) mx = fmaxf(mx, __ldcg(il + r));
  wsum = 0.f;
  o = 0.f;
  if (mx != -INFINITY) {
    for (int r = 0; r < n; ++r) {
      const float w = __expf(__ldcg(il + r) - mx);
      wsum += w;
      o += w * __ldcg(io + static_cast<long long>(r) * p.D + d);
    }
    o /= wsum;
  }
  long long oi = static_cast<long long>(row) * p.D + d;
  if (p.QL > 0) {  // row = (b*H + h)*QL + i  ->  out[b, i, h, d]
    const int i = row % p.QL, h = (row / p.QL) % p.H, b = row / (p.QL * p.H);
    oi = ((static_cast<long long>(b) * p.QL + i) * p.H + h) * p.D + d;
  }
  if (!RA_IN_BOUNDS(oi, 1, static_cast<long long>(gridDim.x) * p.D, kTagDecodeMerge)) {
  } else if (p.out_fp32)
    reinterpret_cast<float*>(p.out)[oi] = o;
  else
    reinterpret_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16(o);
  // ---- the last CTA to get here advances the ring's launch counter
  __syncthreads();
  if (d == 0) {
    const unsigned int prev = atomicAdd(e.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *e.done_ctr = 0u;
      *reinterpret_cast<volatile uint32_t*>(e.epoch_ptr) = epoch;
    }
  }
}

// Decode-time cache append: the new token's K and V (rows of a (B, 1, 3, H, D) qkv buffer) go to cache row
// (*pos_ptr - k0) of this rank's shard if that position is local. The cache is given as two (B, S_max, H, D) views
// with element strides (batch, row, head), so any layout of the shard works: rows-major (B, S, 2, H, D) or
// heads-major (B, 2, H, S, D), where every (k|v, head) is one contiguous stream for the decode kernel.
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                                 __nv_bfloat16* __restrict__ vc, long long sb, long long ss, long long sh,
                                 const long long* __restrict__ pos_ptr, long long k0, int S_max, int H, int D,
                                 int stripe_n, int stripe_rank, long long stripe_base, long long stripe_len0) {
  long long r = *pos_ptr - k0;
  if (stripe_n > 0) {  // striped layout: token i = pos - len0 belongs to rank i % n, row base + i / n
    const long long i = *pos_ptr - stripe_len0;
    r = (i >= 0 && i % stripe_n == stripe_rank) ? stripe_base + i / stripe_n : -1;
  }
  if (r < 0 || r >= S_max) return;
  const int b = blockIdx.x;
  const int HD = H * D, vpr = D / 8;  // 16-byte vectors per head row
  const uint4* src_k = reinterpret_cast<const uint4*>(qkv + (static_cast<long long>(b) * 3 + 1) * HD);
  const uint4* src_v = reinterpret_cast<const uint4*>(qkv + (static_cast<long long>(b) * 3 + 2) * HD);
  for (int i = threadIdx.x; i < HD / 8; i += blockDim.x) {
    const int h = i / vpr, c = i - h * vpr;
    const long long off = b * sb + r * ss + h * sh + c * 8;
    if (!RA_IN_BOUNDS(r, 1, S_max, kTagDecodeCacheRow)) continue;
    *reinterpret_cast<uint4*>(kc + off) = src_k[i];
    *reinterpret_cast<uint4*>(vc + off) = src_v[i];
  }
}

// state = {position, step}: advanced once per decoded token.
__global__ void decode_advance_kernel(long long* state) {
  state[0] += 1;
  state[1] += 1;
}

// y[M, N] = x[M, K] W[N, K]^T for a handful of rows (M <= 8): one warp per output column, the
// weight row is read once with 16-byte loads. Bandwidth-bound companion of the tcgen05 GEMM for
// decode steps, where a 128-row tile would leave most SMs idle.
template <int M>
__global__ void __launch_bounds__(256) small_m_linear_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              __nv_bfloat16* __restrict__ y,
                                                              const __nv_bfloat16* __restrict__ res, int N,
                                                              int K) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= N) return;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<long long>(warp) * K);
  auto consume = [&](const uint4& wv, int c) {
    float wf[8];
    unpack8(wv, wf);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float xf[8];
      unpack8(reinterpret_cast<const uint4*>(x + static_cast<long long>(m) * K)[c], xf);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[m] = fmaf(wf[e], xf[e], acc[m]);
    }
  };
  const int n16 = K / 8;
  int c = lane;
  for (; c + 96 < n16; c += 128) {  // four 16-byte weight loads in flight per lane
    const uint4 w0 = wr[c], w1 = wr[c + 32], w2 = wr[c + 64], w3 = wr[c + 96];
    consume(w0, c);
    consume(w1, c + 32);
    consume(w2, c + 64);
    consume(w3, c + 96);
  }
  for (; c < n16; c += 32) consume(wr[c], c);
#pragma unroll
  for (int m = 0; m < M; ++m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    if (lane == 0) {
      float v = acc[m];
      if (res) v += __bfloat162float(res[static_cast<long long>(m) * N + warp]);
      if (RA_IN_BOUNDS(warp, 1, N, kTagSmallMLinear)) y[static_cast<long long>(m) * N + warp] = __float2bfloat16(v);
    }
  }
}

// The same product with a prologue f applied to x, so that a decode step needs no separate normalisation or
// activation launch: y = f(x) W^T (+ res).
//   PRO_RMSNORM  f(x) = x * rsqrt(mean(x^2) + eps) * gain     (x is the (M, K) residual stream)
//   PRO_SWIGLU   f(x) = silu(x[:, :K]) * x[:, K:]              (x is the (M, 2K) gate/up projection)
// f(x) is built ONCE per CTA in shared memory (M * K bf16) and every warp then walks `cpw` consecutive columns
// against it; the launcher picks cpw so that the whole grid is resident at once. Each warp issues the first
// weight loads of its first column before the prologue, so the prologue's latency hides behind them. (Applying
// f inside every warp's k loop instead repeats it N times and made a 7B decode step 9 % slower.)
enum { PRO_RMSNORM = 1, PRO_SWIGLU = 2 };

template <int M, int PRO>
__global__ void __launch_bounds__(256) small_m_linear_pro_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ w,
                                                                  __nv_bfloat16* __restrict__ y,
                                                                  const __nv_bfloat16* __restrict__ res,
                                                                  const __nv_bfloat16* __restrict__ gain, float eps,
                                                                  int N, int K, int cpw) {
  extern __shared__ uint4 xs[];  // [M][K / 8] f(x) as bf16, without the rstd factor of RMSNorm
  __shared__ float red[8][M];
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int n16 = K / 8;
  const int col0 = (blockIdx.x * 8 + wid) * cpw;
  const bool full = n16 >= 128;  // the unrolled loop runs at least once
  const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<long long>(col0 < N ? col0 : 0) * K);
  uint4 w0 = {}, w1 = {}, w2 = {}, w3 = {};
  if (full && col0 < N) {
    w0 = wr[lane];
    w1 = wr[lane + 32];
    w2 = wr[lane + 64];
    w3 = wr[lane + 96];
  }
  // ---- prologue: f(x) -> shared memory
  float ss[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    ss[m] = 0.f;
    const long long ldx = PRO == PRO_SWIGLU ? 2ll * K : K;
    const uint4* xr = reinterpret_cast<const uint4*>(x + m * ldx);
    for (int c = tid; c < n16; c += 256) {
      float xf[8], of[8];
      unpack8(xr[c], xf);
      unpack8(PRO == PRO_SWIGLU ? xr[c + n16] : reinterpret_cast<const uint4*>(gain)[c], of);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (PRO == PRO_RMSNORM) {
          ss[m] = fmaf(xf[e], xf[e], ss[m]);
          xf[e] *= of[e];
        } else {
          xf[e] = xf[e] / (1.f + __expf(-xf[e])) * of[e];  // same arithmetic as the stand-alone activation kernel
        }
      }
      xs[m * n16 + c] = pack8(xf);
    }
  }
  float rstd[M];
  if (PRO == PRO_RMSNORM) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
      if (lane == 0) red[wid][m] = ss[m];
    }
  }
  __syncthreads();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    rstd[m] = 1.f;
    if (PRO == PRO_RMSNORM) {
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) t += red[i][m];
      rstd[m] = rsqrtf(t / K + eps);
    }
  }
  // ---- cpw columns per warp
  for (int j = 0; j < cpw; ++j) {
    const int col = col0 + j;
    if (col >= N) break;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    auto consume = [&](const uint4& wv, int c) {
      float wf[8];
      unpack8(wv, wf);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xf[8];
        unpack8(xs[m * n16 + c], xf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[m] = fmaf(wf[e], xf[e], acc[m]);
      }
    };
    int c = lane;
    if (full) {
      if (j > 0) {
        w0 = wr[c];
        w1 = wr[c + 32];
        w2 = wr[c + 64];
        w3 = wr[c + 96];
      }
      while (true) {
        const int cn = c + 128;
        const bool more = cn + 96 < n16;
        uint4 n0 = {}, n1 = {}, n2 = {}, n3 = {};
        if (more) {  // the next four loads leave before this group is consumed
          n0 = wr[cn];
          n1 = wr[cn + 32];
          n2 = wr[cn + 64];
          n3 = wr[cn + 96];
        }
        consume(w0, c);
        consume(w1, c + 32);
        consume(w2, c + 64);
        consume(w3, c + 96);
        c = cn;
        if (!more) break;
        w0 = n0;
        w1 = n1;
        w2 = n2;
        w3 = n3;
      }
    }
    for (; c < n16; c += 32) consume(wr[c], c);
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
      if (lane == 0) {
        float v = acc[m] * rstd[m];
        if (res) v += __bfloat162float(res[static_cast<long long>(m) * N + col]);
        if (RA_IN_BOUNDS(col, 1, N, kTagSmallMLinear)) y[static_cast<long long>(m) * N + col] = __float2bfloat16(v);
      }
    }
    wr += n16;
  }
}

// The same product on the tensor cores, for 2..8 rows (several decode streams): with M rows the kernels above spend
// M times the FMAs per weight and become bound by their instruction stream (M = 8: 189 us against 34 us for M = 1 on
// 22016 x 4096). Built like decode_splitkv_mma_kernel: the rows of x are the M side of a 16 x 8 x 16 MMA (rows >= M are
// zero), 16 weight rows (output columns) a chunk's N side, and K is walked in chunks of 128. A warp owns 16 output
// columns and a quarter of K; it stages its chunks (16 weight rows x 256 bytes, and the matching 128 elements of the
// eight x rows) through its own three-stage cp.async ring, XOR-swizzled for ldmatrix, with __syncwarp() as the only
// synchronisation in the loop; the four warps of a CTA add their accumulators through shared memory at the end.
// (Loading the B fragments straight from global memory, eight rows x 64 bytes per instruction, reached only 2.5
// TB/s; staged like this the weight stream is read in 256-byte row segments.) x is taken as it is: RMSNorm or
// SwiGLU run as their own launches before it on this path.
#ifndef RA_LM_ST
#define RA_LM_ST 3  // ring depth; measured 2 / 3 / 4 on 4 x 4096 x 11008: 26.9 / 19.5 / 19.4 us, on 4 x 22016 x 4096: 34.2 / 33.8 / 35.7 us
#endif
constexpr int LM_THREADS = 128, LM_WARPS = 4, LM_ST = RA_LM_ST, LM_KC = 128, LM_COLS = 16;
constexpr int LM_WTILE = LM_COLS * LM_KC * 2;     // bytes of a weight chunk
constexpr int LM_XTILE = 8 * LM_KC * 2;           // bytes of an x chunk (eight rows)
constexpr int LM_STAGE = LM_WTILE + LM_XTILE;

__global__ void __launch_bounds__(LM_THREADS) small_m_linear_mma_kernel(const __nv_bfloat16* __restrict__ x,
                                                                        const __nv_bfloat16* __restrict__ w,
                                                                        __nv_bfloat16* __restrict__ y,
                                                                        const __nv_bfloat16* __restrict__ res, int M,
                                                                        int N, int K) {
  extern __shared__ uint4 lm_ring[];  // [LM_WARPS][LM_ST][weights | x]
  __shared__ float red[LM_WARPS][8][LM_COLS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* ring = reinterpret_cast<uint8_t*>(lm_ring) + warp * (LM_ST * LM_STAGE);
  const int col0 = blockIdx.x * LM_COLS;
  const int n_kc = (K + LM_KC - 1) / LM_KC;  // chunks of K; warp w takes chunks w, w + 4, ... (the CTA reads 1 KB of a row at a time)
  const int my_kc = warp < n_kc ? (n_kc - warp + LM_WARPS - 1) / LM_WARPS : 0;

  auto issue = [&](int c, int slot) {
    const int k0 = (warp + LM_WARPS * c) * LM_KC;
    uint8_t* wt = ring + slot * LM_STAGE;
#pragma unroll
    for (int j = 0; j < LM_COLS * 16 / 32; ++j) {   // 16 rows x 16 pieces of 16 bytes
      const int piece = lane + 32 * j;
      const int row = piece >> 4, ch = piece & 15;
      const int col = col0 + row;
      const bool in = col < N && k0 + ch * 8 < K;
      const __nv_bfloat16* src = w + static_cast<long long>(in ? col : 0) * K + (in ? k0 + ch * 8 : 0);
      cp_async16(wt + row * (LM_KC * 2) + ((ch ^ (row & 7)) << 4), src, in ? 16 : 0);
    }
#pragma unroll
    for (int j = 0; j < 8 * 16 / 32; ++j) {         // 8 rows x 16 pieces
      const int piece = lane + 32 * j;
      const int row = piece >> 4, ch = piece & 15;
      const bool in = row < M && k0 + ch * 8 < K;
      const __nv_bfloat16* src = x + static_cast<long long>(in ? row : 0) * K + (in ? k0 + ch * 8 : 0);
      cp_async16(wt + LM_WTILE + row * (LM_KC * 2) + ((ch ^ (row & 7)) << 4), src, in ? 16 : 0);
    }
  };
#pragma unroll
  for (int i = 0; i < LM_ST - 1; ++i) {
    if (i < my_kc) issue(i, i);
    cp_async_commit();  // one group per chunk, empty or not
  }
  float acc[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
  int slot = 0;
  const int mat = lane >> 3, rr = lane & 7;
  for (int c = 0; c < my_kc; ++c) {
    __syncwarp();  // every lane is done with the stage that is filled next
    if (c + LM_ST - 1 < my_kc) issue(c + LM_ST - 1, (slot + LM_ST - 1) % LM_ST);
    cp_async_commit();
    cp_async_wait<LM_ST - 1>();
    __syncwarp();
    const uint8_t* wt = ring + slot * LM_STAGE;
    const uint8_t* xt = wt + LM_WTILE;
#pragma unroll
    for (int ks2 = 0; ks2 < LM_KC / 32; ++ks2) {  // two k-steps of 16 per round
      // A fragments of both k-steps with one ldmatrix: matrices (x rows 0-7, 16-byte piece 4 ks2 + mat)
      uint32_t af[4];
      {
        const int ch = 4 * ks2 + mat;
        ldmatrix_x4(af, xt + rr * (LM_KC * 2) + ((ch ^ (rr & 7)) << 4));
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // B fragments: (weight rows 0-7 | 8-15) x (piece 2 ks | 2 ks + 1) with ks = 2 ks2 + h
        const int row = rr + 8 * (mat >> 1);
        const int ch = 2 * (2 * ks2 + h) + (mat & 1);
        uint32_t bf[4];
        ldmatrix_x4(bf, wt + row * (LM_KC * 2) + ((ch ^ (row & 7)) << 4));
        mma_16816_top(acc[0], af[2 * h], af[2 * h + 1], bf[0], bf[1]);
        mma_16816_top(acc[1], af[2 * h], af[2 * h + 1], bf[2], bf[3]);
      }
    }
    slot = slot + 1 == LM_ST ? 0 : slot + 1;
  }
  cp_async_wait<0>();
  // ---- the four warps' sums of y[row g][col0 + 8 nt + 2t, +1]
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    red[warp][g][8 * nt + 2 * t] = acc[nt][0];
    red[warp][g][8 * nt + 2 * t + 1] = acc[nt][1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < M * LM_COLS; i += LM_THREADS) {
    const int m = i / LM_COLS, c = i % LM_COLS;
    if (col0 + c >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < LM_WARPS; ++k) v += red[k][m][c];
    const long long o = static_cast<long long>(m) * N + col0 + c;
    if (res) v += __bfloat162float(res[o]);
    if (RA_IN_BOUNDS(col0 + c, 1, N, kTagSmallMLinear)) y[o] = __float2bfloat16(v);
  }
}

// One decode token per sequence: rotate the q and k heads of the (B, 1, 3, H, D) qkv buffer in place (RoPE at the
// position in *pos_ptr) and append the rotated K and the V to the cache shard when this rank owns the position
// (same ownership rule and cache views as kv_append_kernel). One launch instead of two per layer and token.
template <int D>
__global__ void rope_append_kernel(__nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                                   __nv_bfloat16* __restrict__ vc, long long sb, long long ss, long long sh,
                                   const long long* __restrict__ pos_ptr, float log2_theta, long long k0, int S_max,
                                   int H, int stripe_n, int stripe_rank, long long stripe_base,
                                   long long stripe_len0) {
  const long long pos = *pos_ptr;
  long long r = pos - k0;
  if (stripe_n > 0) {
    const long long i = pos - stripe_len0;
    r = (i >= 0 && i % stripe_n == stripe_rank) ? stripe_base + i / stripe_n : -1;
  }
  const bool mine = r >= 0 && r < S_max;
  const int b = blockIdx.x;
  constexpr int hd2 = D / 2, VPH = hd2 / 8;  // 16-byte vectors per half head
  __nv_bfloat16* base = qkv + static_cast<long long>(b) * 3 * H * D;
  // q and k heads: 2H heads x VPH vector pairs
  for (int i = threadIdx.x; i < 2 * H * VPH; i += blockDim.x) {
    const int hh = i / VPH, v = i - hh * VPH;  // hh in [0, 2H): q heads then k heads
    __nv_bfloat16* p = base + static_cast<long long>(hh) * D + v * 8;
    float a[8], c[8];
    unpack8(*reinterpret_cast<const uint4*>(p), a);
    unpack8(*reinterpret_cast<const uint4*>(p + hd2), c);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float inv_freq = exp2f(-log2_theta * (2.0f * (v * 8 + e) / D));
      float sn, cs;
      sincosf(static_cast<int>(pos) * inv_freq, &sn, &cs);  // same arithmetic as the stand-alone RoPE kernel
      const float a2 = a[e] * cs - c[e] * sn, c2 = c[e] * cs + a[e] * sn;
      a[e] = a2;
      c[e] = c2;
    }
    const uint4 lo = pack8(a), hi = pack8(c);
    *reinterpret_cast<uint4*>(p) = lo;
    *reinterpret_cast<uint4*>(p + hd2) = hi;
    if (mine && hh >= H && RA_IN_BOUNDS(r, 1, S_max, kTagDecodeCacheRow)) {
      const long long off = b * sb + r * ss + (hh - H) * sh + v * 8;
      *reinterpret_cast<uint4*>(kc + off) = lo;
      *reinterpret_cast<uint4*>(kc + off + hd2) = hi;
    }
  }
  if (mine) {
    const uint4* src_v = reinterpret_cast<const uint4*>(base + 2ll * H * D);
    for (int i = threadIdx.x; i < H * D / 8; i += blockDim.x) {
      const int h = i / (D / 8), cidx = i - h * (D / 8);
      *reinterpret_cast<uint4*>(vc + b * sb + r * ss + h * sh + cidx * 8) = src_v[i];
    }
  }
}

}  // namespace decode
}  // namespace ra

using namespace ra;

struct RaDecodeArgs {
  const void* q; const void* k; const void* v;
  long long k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
  float* o_part; float* lse_part;
  const unsigned char* mask; long long m_sb, m_sh, m_sq;
  int B, H, QL, S, D, splits;
  float softmax_scale;
  long long q_pos0, k_pos0;
  const long long* pos_ptr;
  int stripe_n, stripe_rank;
  long long stripe_base, stripe_len0;
  void* stream;
  int stages;  // 0, 3 or 4: depth of the asynchronous-copy ring of the cache rows (0: loads into registers)
  int mma;     // 1: the tensor-core kernel (any q_len <= 8), 0: the CUDA-core kernel
};

extern "C" int ra_decode_splitkv(const RaDecodeArgs* a) {
  using namespace ra::decode;
  if ((a->D != 64 && a->D != 128) || a->QL < 1 || a->QL > 8 || a->B < 1 || a->H < 1 || a->splits < 1 ||
      a->S < 0) {
    set_error("ra_decode_splitkv: head_dim must be 64/128 and 1 <= q_len <= 8");
    return kHostBadArg;
  }
  SplitParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.k_sb = a->k_sb; p.k_ss = a->k_ss; p.k_sh = a->k_sh;
  p.v_sb = a->v_sb; p.v_ss = a->v_ss; p.v_sh = a->v_sh;
  p.o_part = a->o_part;
  p.lse_part = a->lse_part;
  p.mask = a->mask;
  p.m_sb = a->m_sb; p.m_sh = a->m_sh; p.m_sq = a->m_sq;
  p.B = a->B; p.H = a->H; p.S = a->S;
  p.splits = a->splits;
  p.rows_per_split = (a->S + a->splits - 1) / a->splits;
  if (p.rows_per_split < 1) p.rows_per_split = 1;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.q_pos0 = a->q_pos0;
  p.k_pos0 = a->k_pos0;
  p.pos_ptr = a->pos_ptr;
  p.stripe_n = a->stripe_n; p.stripe_rank = a->stripe_rank;
  p.stripe_base = a->stripe_base; p.stripe_len0 = a->stripe_len0;
  dim3 grid(a->splits, a->H, a->B);
  cudaStream_t s = static_cast<cudaStream_t>(a->stream);
  const int ql = a->QL <= 1 ? 1 : (a->QL <= 2 ? 2 : (a->QL <= 4 ? 4 : 8));
  if (ql != a->QL) {
    set_error("ra_decode_splitkv: q_len must be 1, 2, 4 or 8 (pad the query)");
    return kHostBadArg;
  }
  if (a->mma) {
    constexpr int kRing128 = WARPS * MMA_ST * 2 * MMA_ROWS * 128 * 2, kRing64 = WARPS * MMA_ST * 2 * MMA_ROWS * 64 * 2;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_done[dev]) {  // with the static arrays the 128-wide variant needs more than 48 KB
      cudaFuncSetAttribute(decode_splitkv_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing128);
      cudaFuncSetAttribute(decode_splitkv_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing64);
      attr_done[dev] = true;
    }
    if (a->D == 128)
      decode_splitkv_mma_kernel<128><<<grid, THREADS, kRing128, s>>>(p, a->QL);
    else
      decode_splitkv_mma_kernel<64><<<grid, THREADS, kRing64, s>>>(p, a->QL);
    return check_launch("decode_splitkv_mma_kernel");
  }
  if (a->stages != 0 && a->stages != 3 && a->stages != 4) {
    set_error("ra_decode_splitkv: stages must be 0, 3 or 4");
    return kHostBadArg;
  }
// (the dynamic ring plus the static arrays exceed 48 KB for every ST > 0, hence the attribute)
#define RA_LAUNCH_DEC3(DD, QQ, SS)                                                                          \
  do {                                                                                                      \
    constexpr int smem = SS * DEC_UNROLL * 2 * THREADS * 16;                                                \
    static bool attr_done[64] = {};                                                                         \
    int dev = 0;                                                                                            \
    cudaGetDevice(&dev);                                                                                    \
    if (smem > 0 && dev < 64 && !attr_done[dev]) {                                                          \
      cudaFuncSetAttribute(decode_splitkv_kernel<DD, QQ, SS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
      attr_done[dev] = true;                                                                                \
    }                                                                                                       \
    decode_splitkv_kernel<DD, QQ, SS><<<grid, THREADS, smem, s>>>(p);                                       \
  } while (0)
#define RA_LAUNCH_DEC(DD, QQ)                                                                               \
  do {                                                                                                      \
    if (a->stages == 3) RA_LAUNCH_DEC3(DD, QQ, 3);                                                          \
    else if (a->stages == 4) RA_LAUNCH_DEC3(DD, QQ, 4);                                                     \
    else RA_LAUNCH_DEC3(DD, QQ, 0);                                                                         \
  } while (0)
  if (a->D == 128) {
    if (ql == 1) RA_LAUNCH_DEC(128, 1); else if (ql == 2) RA_LAUNCH_DEC(128, 2);
    else if (ql == 4) RA_LAUNCH_DEC(128, 4); else RA_LAUNCH_DEC(128, 8);
  } else {
    if (ql == 1) RA_LAUNCH_DEC(64, 1); else if (ql == 2) RA_LAUNCH_DEC(64, 2);
    else if (ql == 4) RA_LAUNCH_DEC(64, 4); else RA_LAUNCH_DEC(64, 8);
  }
#undef RA_LAUNCH_DEC
#undef RA_LAUNCH_DEC3
  return check_launch("decode_splitkv_kernel");
}

extern "C" int ra_decode_merge(const float* o_part, const float* lse_part, long long o_rs, long long o_ps,
                               long long l_rs, long long l_ps, int rows, int nparts, int D, int H,
                               int QL, void* out, int out_fp32, float* lse_out,
                               void* const* inbox_o, void* const* inbox_lse, int n_ranks, int my_rank,
                               const long long* step_ptr, long long slot_mul, long long slot_add,
                               long long out_slot_o, long long out_slot_l,
                               long long in_slot_o, long long in_slot_l, void* stream) {
  using namespace ra::decode;
  if (rows < 1 || nparts < 1 || (D != 64 && D != 128)) {
    set_error("ra_decode_merge: bad shape");
    return kHostBadArg;
  }
  MergeParams p;
  p.o_part = o_part; p.lse_part = lse_part;
  p.o_rs = o_rs; p.o_ps = o_ps; p.l_rs = l_rs; p.l_ps = l_ps;
  p.rows = rows; p.nparts = nparts; p.D = D; p.H = H; p.QL = QL;
  p.out = out; p.out_fp32 = out_fp32; p.lse_out = lse_out;
  p.inbox_o = reinterpret_cast<float* const*>(inbox_o);
  p.inbox_lse = reinterpret_cast<float* const*>(inbox_lse);
  p.n_ranks = n_ranks; p.my_rank = my_rank;
  p.step_ptr = step_ptr;
  p.slot_mul = slot_mul; p.slot_add = slot_add;
  p.out_slot_o = out_slot_o; p.out_slot_l = out_slot_l; p.in_slot_o = in_slot_o; p.in_slot_l = in_slot_l;
  decode_merge_kernel<<<rows, D, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("decode_merge_kernel");
}

// Rows one launch of the fused exchange may have: every CTA has to be resident while it waits for its peers.
extern "C" int ra_decode_exchange_max_rows() { return 2 * sm_count(); }

// `sync` : this rank's 8-byte {epoch, done counter} words (zero-initialised, used by this kernel only).
// `flags`: device table of every rank's flag words, each (>= rows * n_ranks) u32, zero-initialised.
// `inbox_o` / `inbox_lse`: device tables of every rank's inbox, 2 slots of (slot_rows, n_ranks, D) and (slot_rows,
// n_ranks) floats; `*_local` this rank's own. Launches with different row counts may share them: the slot stride
// does not depend on `rows`.
extern "C" int ra_decode_merge_exchange(const float* o_part, const float* lse_part, long long o_rs, long long o_ps,
                                        long long l_rs, long long l_ps, int rows, int nparts, int D, int H, int QL,
                                        void* out, int out_fp32, void* const* inbox_o, void* const* inbox_lse,
                                        const float* inbox_o_local, const float* inbox_l_local, int slot_rows,
                                        void* const* flags, void* sync, int n_ranks, int my_rank, unsigned long long timeout_ns,
                                        int* status, void* stream) {
  using namespace ra::decode;
  if (rows < 1 || rows > ra_decode_exchange_max_rows() || nparts < 1 || (D != 64 && D != 128) || n_ranks < 2 ||
      n_ranks > 32 || my_rank < 0 || my_rank >= n_ranks || !out || !flags || !sync || slot_rows < rows) {
    set_error("ra_decode_merge_exchange: bad shape (rows must not exceed twice the SM count)");
    return kHostBadArg;
  }
  ExchangeParams e;
  MergeParams& p = e.m;
  p = MergeParams{};
  p.o_part = o_part; p.lse_part = lse_part;
  p.o_rs = o_rs; p.o_ps = o_ps; p.l_rs = l_rs; p.l_ps = l_ps;
  p.rows = rows; p.nparts = nparts; p.D = D; p.H = H; p.QL = QL;
  p.out = out; p.out_fp32 = out_fp32;
  p.inbox_o = reinterpret_cast<float* const*>(inbox_o);
  p.inbox_lse = reinterpret_cast<float* const*>(inbox_lse);
  p.n_ranks = n_ranks; p.my_rank = my_rank;
  e.flags = reinterpret_cast<uint32_t* const*>(flags);
  e.epoch_ptr = static_cast<uint32_t*>(sync);
  e.done_ctr = static_cast<unsigned int*>(sync) + 1;
  e.inbox_o_local = inbox_o_local;
  e.inbox_l_local = inbox_l_local;
  e.slot_rows = slot_rows;
  e.timeout_ns = timeout_ns;
  e.status = status;
  decode_merge_exchange_kernel<<<rows, D, 0, static_cast<cudaStream_t>(stream)>>>(e);
  return check_launch("decode_merge_exchange_kernel");
}

extern "C" int ra_kv_append(const void* qkv, void* k_cache, void* v_cache, long long sb, long long ss, long long sh,
                            const long long* pos_ptr, long long k0, int S_max, int B, int H, int D, int stripe_n,
                            int stripe_rank, long long stripe_base, long long stripe_len0, void* stream) {
  using namespace ra::decode;
  if (D % 8 || B < 1 || H < 1 || !pos_ptr || (sb % 8) || (ss % 8) || (sh % 8)) {
    set_error("ra_kv_append: bad arguments");
    return kHostBadArg;
  }
  kv_append_kernel<<<B, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(k_cache),
      static_cast<__nv_bfloat16*>(v_cache), sb, ss, sh, pos_ptr, k0, S_max, H, D, stripe_n, stripe_rank, stripe_base,
      stripe_len0);
  return check_launch("kv_append_kernel");
}

extern "C" int ra_decode_advance(long long* state, void* stream) {
  ra::decode::decode_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(state);
  return check_launch("decode_advance_kernel");
}

extern "C" int ra_small_m_linear(const void* x, const void* w, void* y, const void* res, int M, int N,
                                 int K, void* stream) {
  using namespace ra::decode;
  if (M < 1 || M > 8 || K % 8 || N < 1) {
    set_error("ra_small_m_linear: need 1 <= M <= 8 and K % 8 == 0");
    return kHostBadArg;
  }
  const int blocks = (N * 32 + 255) / 256;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* ww = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* yy = static_cast<__nv_bfloat16*>(y);
  const __nv_bfloat16* rr = static_cast<const __nv_bfloat16*>(res);
  switch (M) {
    case 1: small_m_linear_kernel<1><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    case 2: small_m_linear_kernel<2><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    case 3: small_m_linear_kernel<3><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    case 4: small_m_linear_kernel<4><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    case 5: small_m_linear_kernel<5><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    case 6: small_m_linear_kernel<6><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    case 7: small_m_linear_kernel<7><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
    default: small_m_linear_kernel<8><<<blocks, 256, 0, s>>>(xx, ww, yy, rr, N, K); break;
  }
  return check_launch("small_m_linear_kernel");
}

// Shared memory the prologue variant needs: M * K bf16. The Python side falls back to two launches above this.
extern "C" int ra_small_m_linear_fused_max_smem() { return 48 * 1024; }

extern "C" int ra_small_m_linear_fused(const void* x, const void* w, void* y, const void* res, const void* gain,
                                       float eps, int prologue, int M, int N, int K, void* stream) {
  using namespace ra::decode;
  const long long smem = static_cast<long long>(M) * K * 2;
  if (M < 1 || M > 8 || K % 8 || N < 1 || (prologue != PRO_RMSNORM && prologue != PRO_SWIGLU) ||
      (prologue == PRO_RMSNORM && !gain) || smem > ra_small_m_linear_fused_max_smem()) {
    set_error("ra_small_m_linear_fused: need 1 <= M <= 8, K % 8 == 0, M * K * 2 <= 48 KB, a prologue of 1 (RMSNorm, "
              "with a gain) or 2 (SwiGLU)");
    return kHostBadArg;
  }
  // columns per warp: the whole grid resident at once (four CTAs of 256 threads per SM)
  const int resident = sm_count() * 4;
  int cpw = (N + 8 * resident - 1) / (8 * resident);
  if (cpw < 1) cpw = 1;
  const int blocks = (N + 8 * cpw - 1) / (8 * cpw);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* ww = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* yy = static_cast<__nv_bfloat16*>(y);
  const __nv_bfloat16* rr = static_cast<const __nv_bfloat16*>(res);
  const __nv_bfloat16* gg = static_cast<const __nv_bfloat16*>(gain);
#define RA_SML_CASE(MM)                                                                                        \
  case MM:                                                                                                     \
    if (prologue == PRO_RMSNORM)                                                                               \
      small_m_linear_pro_kernel<MM, PRO_RMSNORM><<<blocks, 256, smem, s>>>(xx, ww, yy, rr, gg, eps, N, K, cpw); \
    else                                                                                                       \
      small_m_linear_pro_kernel<MM, PRO_SWIGLU><<<blocks, 256, smem, s>>>(xx, ww, yy, rr, gg, eps, N, K, cpw);  \
    break;
  switch (M) {
    RA_SML_CASE(1) RA_SML_CASE(2) RA_SML_CASE(3) RA_SML_CASE(4) RA_SML_CASE(5) RA_SML_CASE(6) RA_SML_CASE(7)
    RA_SML_CASE(8)
  }
#undef RA_SML_CASE
  return check_launch("small_m_linear_pro_kernel");
}

// y = x W^T (+ res) for 1 <= M <= 8 rows on the tensor cores (x as it is: no prologue on this path).
extern "C" int ra_small_m_linear_mma(const void* x, const void* w, void* y, const void* res, int M, int N, int K,
                                     void* stream) {
  using namespace ra::decode;
  if (M < 1 || M > 8 || K % 8 || N < 1) {
    set_error("ra_small_m_linear_mma: need 1 <= M <= 8 and K % 8 == 0");
    return kHostBadArg;
  }
  constexpr int smem = LM_WARPS * LM_ST * LM_STAGE;  // 72 KB
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(small_m_linear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess) {
      cudaGetLastError();
      set_error("ra_small_m_linear_mma: cannot raise the shared-memory limit");
      return kHostLaunchFail;
    }
    attr_done[dev] = true;
  }
  const int blocks = (N + LM_COLS - 1) / LM_COLS;
  small_m_linear_mma_kernel<<<blocks, LM_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
      static_cast<const __nv_bfloat16*>(res), M, N, K);
  return check_launch("small_m_linear_mma_kernel");
}

extern "C" int ra_rope_append(void* qkv, void* k_cache, void* v_cache, long long sb, long long ss, long long sh,
                              const long long* pos_ptr, float theta, long long k0, int S_max, int B, int H, int D,
                              int stripe_n, int stripe_rank, long long stripe_base, long long stripe_len0,
                              void* stream) {
  using namespace ra::decode;
  if ((D != 64 && D != 128) || B < 1 || H < 1 || !pos_ptr || (sb % 8) || (ss % 8) || (sh % 8)) {
    set_error("ra_rope_append: bad arguments");
    return kHostBadArg;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16 *q = static_cast<__nv_bfloat16*>(qkv), *kc = static_cast<__nv_bfloat16*>(k_cache),
                *vc = static_cast<__nv_bfloat16*>(v_cache);
  if (D == 128)
    rope_append_kernel<128><<<B, 256, 0, s>>>(q, kc, vc, sb, ss, sh, pos_ptr, log2f(theta), k0, S_max, H, stripe_n,
                                              stripe_rank, stripe_base, stripe_len0);
  else
    rope_append_kernel<64><<<B, 256, 0, s>>>(q, kc, vc, sb, ss, sh, pos_ptr, log2f(theta), k0, S_max, H, stripe_n,
                                             stripe_rank, stripe_base, stripe_len0);
  return check_launch("rope_append_kernel");
}
