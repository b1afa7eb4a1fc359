// Shared pieces of the attention kernels: position maps, tile visibility, dropout hash.
#pragma once
#include "common/bounds.cuh"
#include "common/sm100.cuh"

namespace ra {
namespace attn {

// Global token position of local index i. A shard is one contiguous run (half >= length) or two
// runs of `half` tokens each (zig-zag layout); `half` is a multiple of the 128-row tile.
struct PosMap {
  int off0;
  int off1;
  int half;
  __device__ __forceinline__ int operator()(int i) const {
    return i < half ? off0 + i : off1 + (i - half);
  }
};

struct MaskParams {
  int Sq, Sk;
  int cbs;  // causal block size, 0 = not causal
  PosMap qmap, kmap;
  const int* seg_q;     // (B, Sq) segment ids of the local queries, or null
  const int* seg_k;     // (B, Sk) segment ids of this KV block, or null
  const int* seg_q_mm;  // (B, ceil(Sq/128), 2) per-tile {min, max} segment id, or null
  const int* seg_k_mm;  // (B, ceil(Sk/128), 2)
  const float* bias;    // (B, Hb, Sk) additive key bias in natural-log units, or null
  long long bias_stride_b, bias_stride_h;
  unsigned int seed_lo, seed_hi;
  unsigned int drop_threshold;  // 0 = dropout off; logit dropped iff hash < threshold
  // Optional boolean mask as a bitmap (bit set = attend), rows padded to whole 128-column tiles. The forward
  // reads it by query row (word w of row q: keys 32w..32w+31 of this KV block), the backward by kv row (word w
  // of row k: queries 32w..32w+31); strides in 32-bit words, row stride a multiple of 4.
  const uint32_t* keep;
  long long keep_sb, keep_sh, keep_sr;
};

// False when every entry of the (128 q x 128 k) tile is masked by the causal rule or because the
// segment-id ranges of the two tiles are disjoint. qi0/k0 are local start indices.
__device__ __forceinline__ bool tile_visible(const MaskParams& m, int b, int qi0, int k0) {
  if (qi0 >= m.Sq || k0 >= m.Sk) return false;
  if (m.cbs == 1) {  // plain causal: no divisions on the hot path
    if (m.qmap(min(qi0 + 127, m.Sq - 1)) < m.kmap(k0)) return false;
  } else if (m.cbs) {
    const int q_hi = m.qmap(min(qi0 + 127, m.Sq - 1));
    const int k_lo = m.kmap(k0);
    if (q_hi / m.cbs < k_lo / m.cbs) return false;
  }
  if (m.seg_q_mm) {
    const int nqt = (m.Sq + 127) >> 7, nkt = (m.Sk + 127) >> 7;
    const int* qm = m.seg_q_mm + (static_cast<long long>(b) * nqt + (qi0 >> 7)) * 2;
    const int* km = m.seg_k_mm + (static_cast<long long>(b) * nkt + (k0 >> 7)) * 2;
    if (qm[1] < km[0] || km[1] < qm[0]) return false;
  }
  return true;
}

// ---- per-CTA visibility bitmask ---------------------------------------------------------------------
// With segment ids every evaluation of tile_visible costs a global-memory round trip. A CTA that walked
// its tiles one by one spent ~100 us on that walk alone (256 tiles); instead all threads of the CTA
// evaluate the predicate once, 32 tiles per warp step, into a bitmask in shared memory, and the roles
// walk the set bits.
constexpr int VIS_WORDS = 256;  // capacity: 8192 tiles (1M rows); longer launches fall back to the direct walk

// bit t of `words` = pred(t) for t < n (n <= 32 * VIS_WORDS). Call with every thread of the CTA, converged,
// `nthreads` a multiple of 32; a __syncthreads() must follow before the mask is read.
template <typename F>
__device__ __forceinline__ void fill_visibility(uint32_t* words, int n, int tid, int nthreads, F pred) {
  const int n_pad = (n + 31) & ~31;
  for (int t = tid; t < n_pad; t += nthreads) {  // a warp's 32 values of t share one word: uniform trip count
    const bool v = t < n && pred(t);
    const uint32_t bits = __ballot_sync(0xffffffffu, v);
    if ((tid & 31) == 0) words[t >> 5] = bits;
  }
}

// Smallest set bit at or after t, or n.
__device__ __forceinline__ int vis_next(const uint32_t* words, int t, int n) {
  while (t < n) {
    const uint32_t w = words[t >> 5] >> (t & 31);
    if (w) return t + __ffs(static_cast<int>(w)) - 1;  // bits at or beyond n are never set
    t = (t | 31) + 1;
  }
  return n;
}

// True when no entry of the tile needs element-wise masking or bias. With segment ids that is the case
// when both tiles lie inside one and the same segment (per-tile min == max, equal on both sides), which
// holds for most tiles of packed documents much longer than a tile.
__device__ __forceinline__ bool tile_plain(const MaskParams& m, int b, int qi0, int k0) {
  if (m.bias || m.drop_threshold || m.keep) return false;
  if (k0 + 128 > m.Sk || qi0 + 128 > m.Sq) return false;
  if (m.seg_q) {
    if (!m.seg_q_mm) return false;
    const int nqt = (m.Sq + 127) >> 7, nkt = (m.Sk + 127) >> 7;
    const int* qm = m.seg_q_mm + (static_cast<long long>(b) * nqt + (qi0 >> 7)) * 2;
    const int* km = m.seg_k_mm + (static_cast<long long>(b) * nkt + (k0 >> 7)) * 2;
    const int q_lo = qm[0], k_lo = km[0];
    if (q_lo != qm[1] || k_lo != km[1] || q_lo != k_lo) return false;
  }
  if (m.cbs == 1) {
    if (m.qmap(qi0) < m.kmap(min(k0 + 127, m.Sk - 1))) return false;
  } else if (m.cbs) {
    const int q_lo = m.qmap(qi0);
    const int k_hi = m.kmap(min(k0 + 127, m.Sk - 1));
    if (q_lo / m.cbs < k_hi / m.cbs) return false;
  }
  return true;
}

// Number of leading columns of the k tile that the causal rule and the sequence end leave
// visible to a query at global position qpos: column c is masked iff c >= limit.
__device__ __forceinline__ int causal_col_limit(const MaskParams& m, int qpos, int k0) {
  int limit = m.Sk - k0;
  if (m.cbs) {
    const int kbase = m.kmap(k0);
    const long long lim =
        (m.cbs == 1 ? static_cast<long long>(qpos) + 1 : (static_cast<long long>(qpos / m.cbs) + 1) * m.cbs) - kbase;
    limit = static_cast<int>(lim < limit ? (lim < 0 ? 0 : lim) : limit);
  }
  return limit;
}

__device__ __forceinline__ unsigned int mix32(unsigned int x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}
// Counter-based dropout hash of (seed, b*H+h, q position, k position).
__device__ __forceinline__ unsigned int dropout_hash(unsigned int seed_lo, unsigned int seed_hi,
                                                     unsigned int bh, unsigned int qpos,
                                                     unsigned int kpos) {
  unsigned int x = qpos * 0x9E3779B1u + kpos * 0x85EBCA77u + bh * 0xC2B2AE3Du + seed_lo;
  x = mix32(x);
  x = mix32((x ^ seed_hi) + kpos);
  return x;
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace attn
}  // namespace ra
