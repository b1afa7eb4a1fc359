// Memory-bound kernels of the LLaMA driver: RMSNorm fwd/bwd, RoPE (in place, forward and
// inverse), SwiGLU fwd/bwd, embedding gather / scatter-add, fused softmax-cross-entropy
// (loss + dlogits in one pass over a logits chunk), AdamW over flat buffers, squared-norm
// reduction and dtype casts. All use 16-byte vector accesses; bf16 activations, fp32 statistics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/bounds.cuh"
#include "common/host_util.h"

RA_BOUNDS_TRANSLATION_UNIT()

namespace ra {
namespace ew {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is a shared array of 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
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

// ---------------------------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w. One warp per row: the row sits in registers (MAXV 16-byte vectors per lane,
// d <= 256 * MAXV), so x is read once, the sum of squares needs only warp shuffles, and the eight warps of a CTA
// keep eight rows of loads in flight. A warp takes exactly one row (a grid-stride loop left some warps with one
// row more than others: 15 % of the time at 64K rows), and two CTAs fit on an SM.
template <int MAXV>
__global__ void __launch_bounds__(256, 2) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                          int rows, int d, float eps) {
  const int nv = d >> 3;
  const int lane = threadIdx.x & 31;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (r < rows) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * d);
    uint4 xv[MAXV];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = lane + v * 32;
      xv[v] = i < nv ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      float f[8];
      unpack8(xv[v], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / d + eps);
    if (lane == 0 && rstd) rstd[r] = rs;
    uint4* yr = reinterpret_cast<uint4*>(y + r * d);
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = lane + v * 32;
      if (i < nv) {
        float f[8], g[8];
        unpack8(xv[v], f);
        unpack8(wr[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = f[e] * rs * g[e];
        if (RA_IN_BOUNDS(r * d + i * 8, 8, static_cast<long long>(rows) * d, kTagRmsnorm)) yr[i] = pack8(f);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres) ; dw += sum_rows dy * xhat.
// A row is shared by the four warps of a half CTA (128 threads, MAXV vectors per thread, d <= 1024 * MAXV): x and
// dy are read once into registers, the gain is re-read from L1 (keeping it in registers too cost spills at two
// CTAs per SM: 0.44 of the copy bandwidth against 0.65 with one), the row's dot product is combined
// through shared memory with one 128-thread barrier, and each thread accumulates the gain gradient of its own
// columns over all rows it sees. The per-CTA partial gain gradients go to `dw_part` (gridDim.x * 2 rows of d
// floats) and a second kernel sums them: no atomics.
template <int MAXV>
__global__ void __launch_bounds__(256, 2) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const float* __restrict__ rstd,
                                                          const __nv_bfloat16* __restrict__ dres,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                                          int rows, int d) {
  __shared__ float red[2][2][4];  // [half CTA][parity][warp]
  const int nv = d >> 3;
  const int grp = threadIdx.x >> 7;   // which half of the CTA
  const int gt = threadIdx.x & 127;   // thread inside the half
  const int gw = gt >> 5, lane = gt & 31;
  float dwacc[MAXV][8];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[v][e] = 0.f;
  }
  int par = 0;
  // the row loop has the same trip count for every thread of a half CTA (the barrier below is per half)
  for (long long r = static_cast<long long>(blockIdx.x) * 2 + grp; r < rows; r += static_cast<long long>(gridDim.x) * 2) {
    const long long off = r * d;
    const uint4* xr = reinterpret_cast<const uint4*>(x + off);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + off);
    uint4 xv[MAXV], gv[MAXV];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = gt + v * 128;
      xv[v] = i < nv ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
      gv[v] = i < nv ? gr[i] : make_uint4(0u, 0u, 0u, 0u);
    }
    const float rs = rstd[r];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = gt + v * 128;
      float xf[8], gf[8], wf[8];
      unpack8(xv[v], xf);
      unpack8(gv[v], gf);
      unpack8(i < nv ? wr[i] : make_uint4(0u, 0u, 0u, 0u), wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += gf[e] * wf[e] * xf[e];
    }
    dot = warp_sum(dot);
    if (lane == 0) red[grp][par][gw] = dot;
    asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
    dot = (red[grp][par][0] + red[grp][par][1] + red[grp][par][2] + red[grp][par][3]) * rs / d;
    par ^= 1;  // the next row writes the other slot: no second barrier is needed before it
    uint4* outr = reinterpret_cast<uint4*>(dx + off);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + off) : nullptr;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = gt + v * 128;
      if (i < nv) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[v], xf);
        unpack8(gv[v], gf);
        unpack8(wr[i], wf);
        if (rr) unpack8(rr[i], o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = xf[e] * rs;
          dwacc[v][e] += gf[e] * xh;
          const float t = rs * (gf[e] * wf[e] - xh * dot);
          o[e] = rr ? o[e] + t : t;
        }
        if (RA_IN_BOUNDS(off + i * 8, 8, static_cast<long long>(rows) * d, kTagRmsnorm)) outr[i] = pack8(o);
      }
    }
  }
  float* part = dw_part + (static_cast<long long>(blockIdx.x) * 2 + grp) * d;
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
    const int i = gt + v * 128;
    if (i < nv) {
      reinterpret_cast<float4*>(part + i * 8)[0] = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
      reinterpret_cast<float4*>(part + i * 8)[1] = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
    }
  }
}

// dw[c] += sum over the `parts` partial rows; one thread per column, coalesced across the columns.
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ dw_part, float* __restrict__ dw, int parts, int d) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float acc = 0.f;
  for (int p = 0; p < parts; ++p) acc += dw_part[static_cast<long long>(p) * d + c];
  if (RA_IN_BOUNDS(c, 1, d, kTagRmsnorm)) dw[c] += acc;
}

// ---------------------------------------------------------------------------------- RoPE
// In-place rotation of a (B, S, H, D) view: pairs (i, i + D/2), angle pos * theta^(-2i/D).
// pos = two-run position map of the local token index (see attn PosMap). sign = +1 fwd, -1 bwd.
// One warp per token: a lane owns 8 frequencies (a 16-byte vector of the first half of a head and its partner in
// the second half), computes their sines and cosines once and walks the heads, 32 / (D/16) heads per warp step,
// so the transcendental work is shared by all heads of the token and the kernel runs at memory speed.
template <int D>
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, long long sb, long long ss, long long sh,
                            int B, int S, int H, int off0, int off1, int half, float log2_theta,
                            float sign, const long long* __restrict__ pos_ptr) {
  if (pos_ptr) off0 += static_cast<int>(*pos_ptr);  // position kept on the device (decode under a CUDA graph)
  constexpr int hd2 = D >> 1;
  constexpr int VPH = hd2 >> 3;    // 16-byte vectors per half head
  constexpr int HL = 32 / VPH;     // heads per warp step
  const int lane = threadIdx.x & 31;
  const int v = lane % VPH, hl = lane / VPH;
  const long long n_tok = static_cast<long long>(B) * S;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float inv_freq[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) inv_freq[e] = exp2f(-log2_theta * (2.0f * (v * 8 + e) / D));
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < n_tok; t += warps) {
    const int s = static_cast<int>(t % S);
    const int b = static_cast<int>(t / S);
    const int pos = s < half ? off0 + s : off1 + (s - half);
    float sn[8], cs[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      sincosf(pos * inv_freq[e], &sn[e], &cs[e]);
      sn[e] *= sign;
    }
    __nv_bfloat16* row = x + b * sb + static_cast<long long>(s) * ss + v * 8;
    for (int h = hl; h < H; h += HL) {
      __nv_bfloat16* p = row + h * sh;
      if (!(RA_IN_BOUNDS(b, 1, B, kTagRope) && RA_IN_BOUNDS(h, 1, H, kTagRope) && RA_IN_BOUNDS(v * 8 + hd2, 8, D, kTagRope)))
        continue;
      float a[8], c[8];
      unpack8(*reinterpret_cast<const uint4*>(p), a);
      unpack8(*reinterpret_cast<const uint4*>(p + hd2), c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a2 = a[e] * cs[e] - c[e] * sn[e];
        const float c2 = c[e] * cs[e] + a[e] * sn[e];
        a[e] = a2;
        c[e] = c2;
      }
      *reinterpret_cast<uint4*>(p) = pack8(a);
      *reinterpret_cast<uint4*>(p + hd2) = pack8(c);
    }
  }
}

// ---------------------------------------------------------------------------------- SwiGLU
// gu: (rows, 2F) = [gate | up]; h = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                                  long long rows, int F) {
  const int nv = F >> 3;
  const long long total = rows * nv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / nv;
    const int v = static_cast<int>(idx - r * nv);
    const __nv_bfloat16* g = gu + r * 2 * F + v * 8;
    float gf[8], uf[8];
    unpack8(*reinterpret_cast<const uint4*>(g), gf);
    unpack8(*reinterpret_cast<const uint4*>(g + F), uf);
#pragma unroll
    for (int e = 0; e < 8; ++e) gf[e] = gf[e] / (1.f + __expf(-gf[e])) * uf[e];
    if (RA_IN_BOUNDS(r * F + v * 8, 8, rows * F, kTagSwiglu)) *reinterpret_cast<uint4*>(h + r * F + v * 8) = pack8(gf);
  }
}
// dgu = [dh * up * silu'(gate) | dh * silu(gate)]; may run in place over gu.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* dgu, long long rows, int F) {
  const int nv = F >> 3;
  const long long total = rows * nv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / nv;
    const int v = static_cast<int>(idx - r * nv);
    const long long o = r * 2 * F + v * 8;
    float gf[8], uf[8], df[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + o), gf);
    unpack8(*reinterpret_cast<const uint4*>(gu + o + F), uf);
    unpack8(*reinterpret_cast<const uint4*>(dh + r * F + v * 8), df);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-gf[e]));
      const float silu = gf[e] * sg;
      const float dsilu = sg * (1.f + gf[e] * (1.f - sg));
      const float dg = df[e] * uf[e] * dsilu;
      uf[e] = df[e] * silu;
      gf[e] = dg;
    }
    if (RA_IN_BOUNDS(o + F, 8, rows * 2 * F, kTagSwiglu)) {
      *reinterpret_cast<uint4*>(dgu + o) = pack8(gf);
      *reinterpret_cast<uint4*>(dgu + o + F) = pack8(uf);
    }
  }
}

// ---------------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long n, int d, int vocab) {
  const int nv = d >> 3;
  const long long total = n * nv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / nv;
    const int v = static_cast<int>(idx - r * nv);
    int t = tok[r];
    (void)RA_IN_BOUNDS(t, 1, vocab, kTagEmbeddingToken);
    t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
    if (RA_IN_BOUNDS(r * d + v * 8, 8, n * d, kTagEmbeddingRow))
    reinterpret_cast<uint4*>(out + r * d)[v] =
        reinterpret_cast<const uint4*>(table + static_cast<long long>(t) * d)[v];
  }
}
__global__ void embedding_bwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ dtable, long long n, int d, int vocab) {
  const int nv = d >> 3;
  const long long total = n * nv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / nv;
    const int v = static_cast<int>(idx - r * nv);
    int t = tok[r];
    (void)RA_IN_BOUNDS(t, 1, vocab, kTagEmbeddingToken);
    t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(dy + r * d)[v], f);
    float* dst = dtable + static_cast<long long>(t) * d + v * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(dst + e, f[e]);
  }
}

// ---------------------------------------------------------------------------------- cross-entropy
// One CTA per row of a (rows, V) bf16 logits chunk (leading dim ld). Writes loss[row] (0 for
// target < 0) and overwrites the logits with dlogits = (softmax - onehot) * grad_scale.
__global__ void xent_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                                    const int* __restrict__ target, float* __restrict__ loss, int V,
                                    float grad_scale) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  __nv_bfloat16* row = logits + r * ld;
  const int nv = V >> 3;
  const int tgt = target[r];
  if (tgt >= 0) (void)RA_IN_BOUNDS(tgt, 1, V, kTagXentTarget);
  const bool valid = tgt >= 0 && tgt < V;
  const float tgt_logit = valid ? __bfloat162float(row[tgt]) : 0.f;  // read before the row is overwritten
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(row)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) mx = fmaxf(mx, f[e]);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(row)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += __expf(f[e] - mx);
  }
  sum = block_sum(sum, red);
  const float lse = mx + __logf(sum);
  if (threadIdx.x == 0) loss[r] = valid ? lse - tgt_logit : 0.f;
  const float gs = valid ? grad_scale : 0.f;
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(row)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float pr = __expf(f[e] - mx) * inv;
      if (i * 8 + e == tgt) pr -= 1.f;
      f[e] = pr * gs;
    }
    if (RA_IN_BOUNDS(i * 8, 8, V, kTagXentRow)) reinterpret_cast<uint4*>(row)[i] = pack8(f);
  }
}

// ---------------------------------------------------------------------------------- optimizer
// sum of squares of an fp32 buffer, accumulated into *out with one atomic per CTA.
__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n4 << 2; i < n; ++i) acc += g[i] * g[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// AdamW over flat fp32 master / moments with fp32 grads; writes the bf16 working copy.
// The clip coefficient is min(1, clip / (sqrt(*gnorm_sq) + 1e-6)) when clip > 0 (read on device).
// decay_mask: optional per-element-range flag is not needed: weight decay is applied to the
// half-open index range [0, decay_end) only (matrices first, norm gains last).
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n,
                             long long decay_end, float lr, float b1, float b2, float eps, float wd,
                             float bc1, float bc2, float clip, const float* __restrict__ gnorm_sq,
                             float grad_mul) {
  float coef = grad_mul;
  if (clip > 0.f && gnorm_sq) {
    const float nrm = sqrtf(*gnorm_sq) * grad_mul;
    coef *= fminf(1.f, clip / (nrm + 1e-6f));
  }
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float* pa = reinterpret_cast<float*>(&pp);
    float* ma = reinterpret_cast<float*>(&mm);
    float* va = reinterpret_cast<float*>(&vv);
    const float* ga = reinterpret_cast<const float*>(&gg);
    const float wdl = (i * 4 < decay_end) ? wd : 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float gr = ga[e] * coef;
      ma[e] = b1 * ma[e] + (1.f - b1) * gr;
      va[e] = b2 * va[e] + (1.f - b2) * gr * gr;
      const float mh = ma[e] / bc1;
      const float vh = va[e] / bc2;
      pa[e] = pa[e] - lr * (mh / (sqrtf(vh) + eps) + wdl * pa[e]);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    __nv_bfloat162 lo = __floats2bfloat162_rn(pa[0], pa[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(pa[2], pa[3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    if (RA_IN_BOUNDS(i * 4, 4, n, kTagAdamw)) reinterpret_cast<uint2*>(p16)[i] = o;
  }
}

// ---------------------------------------------------------------------------------- casts
// fp32 (rows, d) with a row stride -> bf16 view with a row stride (used for dQ into a fused dQKV buffer).
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                     long long rows, int d, long long src_ld, long long dst_ld) {
  const int nv = d >> 3;
  const long long total = rows * nv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / nv;
    const int v = static_cast<int>(idx - r * nv);
    const float4 a = reinterpret_cast<const float4*>(src + r * src_ld)[2 * v];
    const float4 b = reinterpret_cast<const float4*>(src + r * src_ld)[2 * v + 1];
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (RA_IN_BOUNDS(r, 1, rows, kTagCast) && RA_IN_BOUNDS(v * 8, 8, d, kTagCast))
      *reinterpret_cast<uint4*>(dst + r * dst_ld + v * 8) = pack8(f);
  }
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                     long long n) {
  const long long n8 = n >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(src)[i], f);
    reinterpret_cast<float4*>(dst)[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

inline unsigned grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<unsigned>(b);
}

}  // namespace ew
}  // namespace ra

using namespace ra;
using namespace ra::ew;
typedef __nv_bfloat16 bf16;

extern "C" int ra_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int d,
                              float eps, void* stream) {
  if (d % 8 || rows <= 0 || d > 8192) { set_error("rmsnorm_fwd: d must be a multiple of 8 and <= 8192"); return kHostBadArg; }
  const unsigned grid = static_cast<unsigned>((static_cast<long long>(rows) + 7) / 8);  // one warp per row
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bf16 *xp = static_cast<const bf16*>(x), *wp = static_cast<const bf16*>(w);
  bf16* yp = static_cast<bf16*>(y);
  const int nv = d / 8;
  if (nv <= 32) rmsnorm_fwd_kernel<1><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, d, eps);
  else if (nv <= 64) rmsnorm_fwd_kernel<2><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, d, eps);
  else if (nv <= 128) rmsnorm_fwd_kernel<4><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, d, eps);
  else if (nv <= 256) rmsnorm_fwd_kernel<8><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, d, eps);
  else if (nv <= 512) rmsnorm_fwd_kernel<16><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, d, eps);
  else rmsnorm_fwd_kernel<32><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, d, eps);
  return check_launch("rmsnorm_fwd");
}

// Number of partial gain-gradient rows ra_rmsnorm_bwd writes for `rows` input rows: the caller provides a scratch
// of that many rows of d floats.
extern "C" int ra_rmsnorm_bwd_parts(int rows) {
  const int ctas = rows < sm_count() * 16 ? (rows + 1) / 2 : sm_count() * 8;
  return (ctas < 1 ? 1 : ctas) * 2;
}

extern "C" int ra_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                              const void* dres, void* dx, float* dw, float* dw_part, int rows, int d, void* stream) {
  if (d % 8 || rows <= 0 || d > 8192 || !dw_part) {
    set_error("rmsnorm_bwd: d must be a multiple of 8 and <= 8192, and a scratch for the partial sums is needed");
    return kHostBadArg;
  }
  const int parts = ra_rmsnorm_bwd_parts(rows);
  const unsigned grid = parts / 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bf16 *gp = static_cast<const bf16*>(dy), *xp = static_cast<const bf16*>(x), *wp = static_cast<const bf16*>(w);
  const bf16* rp = static_cast<const bf16*>(dres);
  bf16* op = static_cast<bf16*>(dx);
  const int nv = d / 8;
  if (nv <= 128) rmsnorm_bwd_kernel<1><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_part, rows, d);
  else if (nv <= 256) rmsnorm_bwd_kernel<2><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_part, rows, d);
  else if (nv <= 512) rmsnorm_bwd_kernel<4><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_part, rows, d);
  else rmsnorm_bwd_kernel<8><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, op, dw_part, rows, d);
  int rc = check_launch("rmsnorm_bwd");
  if (rc != kHostOk) return rc;
  rmsnorm_dw_reduce_kernel<<<(d + 255) / 256, 256, 0, s>>>(dw_part, dw, parts, d);
  return check_launch("rmsnorm_dw_reduce");
}

static int launch_rope(void* x, long long sb, long long ss, long long sh, int B, int S, int H, int D, int off0,
                       int off1, int half, float theta, float sign, const long long* pos_ptr, void* stream) {
  const long long work = static_cast<long long>(B) * S * 32;  // one warp per token
  const unsigned grid = grid_for(work, 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  bf16* xp = static_cast<bf16*>(x);
  const float l2t = log2f(theta);
  if (D == 64)
    rope_kernel<64><<<grid, 256, 0, st>>>(xp, sb, ss, sh, B, S, H, off0, off1, half, l2t, sign, pos_ptr);
  else if (D == 128)
    rope_kernel<128><<<grid, 256, 0, st>>>(xp, sb, ss, sh, B, S, H, off0, off1, half, l2t, sign, pos_ptr);
  else
    rope_kernel<256><<<grid, 256, 0, st>>>(xp, sb, ss, sh, B, S, H, off0, off1, half, l2t, sign, pos_ptr);
  return check_launch("rope");
}

extern "C" int ra_rope(void* x, long long sb, long long ss, long long sh, int B, int S, int H, int D,
                       int off0, int off1, int half, float theta, int inverse, void* stream) {
  if ((D != 64 && D != 128 && D != 256) || B <= 0 || S <= 0) {
    set_error("rope: head_dim must be 64, 128 or 256");
    return kHostBadArg;
  }
  return launch_rope(x, sb, ss, sh, B, S, H, D, off0, off1, half, theta, inverse ? -1.f : 1.f, nullptr, stream);
}

// Same rotation with the position of token 0 read from device memory (off0 is added to it).
extern "C" int ra_rope_at(void* x, long long sb, long long ss, long long sh, int B, int S, int H, int D,
                          int off0, const long long* pos_ptr, float theta, void* stream) {
  if ((D != 64 && D != 128 && D != 256) || B <= 0 || S <= 0 || !pos_ptr) {
    set_error("rope_at: bad arguments");
    return kHostBadArg;
  }
  return launch_rope(x, sb, ss, sh, B, S, H, D, off0, 0, 1 << 30, theta, 1.f, pos_ptr, stream);
}

extern "C" int ra_swiglu_fwd(const void* gu, void* h, long long rows, int F, void* stream) {
  if (F % 8) { set_error("swiglu: F must be a multiple of 8"); return kHostBadArg; }
  swiglu_fwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(gu), static_cast<bf16*>(h), rows, F);
  return check_launch("swiglu_fwd");
}
extern "C" int ra_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long rows, int F,
                             void* stream) {
  if (F % 8) { set_error("swiglu: F must be a multiple of 8"); return kHostBadArg; }
  swiglu_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(gu), static_cast<const bf16*>(dh), static_cast<bf16*>(dgu), rows, F);
  return check_launch("swiglu_bwd");
}

extern "C" int ra_embedding_fwd(const int* tok, const void* table, void* out, long long n, int d,
                                int vocab, void* stream) {
  if (d % 8) { set_error("embedding: d must be a multiple of 8"); return kHostBadArg; }
  embedding_fwd_kernel<<<grid_for(n * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      tok, static_cast<const bf16*>(table), static_cast<bf16*>(out), n, d, vocab);
  return check_launch("embedding_fwd");
}
extern "C" int ra_embedding_bwd(const int* tok, const void* dy, float* dtable, long long n, int d,
                                int vocab, void* stream) {
  if (d % 8) { set_error("embedding: d must be a multiple of 8"); return kHostBadArg; }
  embedding_bwd_kernel<<<grid_for(n * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      tok, static_cast<const bf16*>(dy), dtable, n, d, vocab);
  return check_launch("embedding_bwd");
}

extern "C" int ra_xent_fwd_bwd(void* logits, long long ld, const int* target, float* loss, long long rows,
                               int V, float grad_scale, void* stream) {
  if (V % 8 || ld % 8 || rows <= 0) { set_error("xent: V and ld must be multiples of 8"); return kHostBadArg; }
  xent_fwd_bwd_kernel<<<static_cast<unsigned>(rows), 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<bf16*>(logits), ld, target, loss, V, grad_scale);
  return check_launch("xent_fwd_bwd");
}

extern "C" int ra_sumsq(const float* g, long long n, float* out, void* stream) {
  sumsq_kernel<<<grid_for(n / 4 + 1, 512), 512, 0, static_cast<cudaStream_t>(stream)>>>(g, n, out);
  return check_launch("sumsq");
}

extern "C" int ra_adamw(float* p, float* m, float* v, const float* g, void* p16, long long n,
                        long long decay_end, float lr, float b1, float b2, float eps, float wd, float bc1,
                        float bc2, float clip, const float* gnorm_sq, float grad_mul, void* stream) {
  if (n % 4 || decay_end % 4) { set_error("adamw: sizes must be multiples of 4"); return kHostBadArg; }
  adamw_kernel<<<grid_for(n / 4, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      p, m, v, g, static_cast<bf16*>(p16), n, decay_end, lr, b1, b2, eps, wd, bc1, bc2, clip, gnorm_sq,
      grad_mul);
  return check_launch("adamw");
}

extern "C" int ra_cast_f32_bf16(const float* src, void* dst, long long rows, int d, long long src_ld,
                                long long dst_ld, void* stream) {
  if (d % 8 || dst_ld % 8 || src_ld % 4) { set_error("cast: d must be a multiple of 8"); return kHostBadArg; }
  cast_f32_bf16_kernel<<<grid_for(rows * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<bf16*>(dst), rows, d, src_ld, dst_ld);
  return check_launch("cast_f32_bf16");
}
extern "C" int ra_cast_bf16_f32(const void* src, float* dst, long long n, void* stream) {
  if (n % 8) { set_error("cast: n must be a multiple of 8"); return kHostBadArg; }
  cast_bf16_f32_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(src), dst, n);
  return check_launch("cast_bf16_f32");
}
extern "C" int ra_cast_load_kernels(void) {
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, ra::ew::cast_f32_bf16_kernel) != cudaSuccess) {
    ra::set_error("ra_cast_load_kernels: cudaFuncGetAttributes failed");
    cudaGetLastError();
    return ra::kHostLaunchFail;
  }
  return ra::kHostOk;
}

// ---------------------------------------------------------------------------------------------------
// Boolean attention masks as bitmaps for the attention kernels.
//
// mask is (B, Hm, Sq, Sk) bytes (non-zero = attend) with element strides sb/sh/sq (0 = broadcast) and a
// contiguous last dim. Two bitmaps are written, both with rows padded to whole 128-column tiles:
//   by_q [B][Hm][Sq][Wk]   word w of row q  holds columns k = 32w .. 32w+31   (forward: a thread owns a q row)
//   by_k [B][Hm][Sk][Wq]   word w of row k  holds rows    q = 32w .. 32w+31   (backward: a thread owns a kv row)
// with Wk = 4*ceil(Sk/128), Wq = 4*ceil(Sq/128). Bits beyond Sq / Sk are 0. One CTA packs a 32 x 32 patch.
namespace ra {
namespace ew {
__global__ void pack_mask_kernel(const uint8_t* __restrict__ mask, long long sb, long long sh, long long sq,
                                 uint32_t* __restrict__ by_q, uint32_t* __restrict__ by_k, int Hm, int Sq,
                                 int Sk, int Wk, int Wq) {
  __shared__ uint32_t cols[32];  // cols[j] bit i = mask[q0+i][k0+j]
  const int k0 = blockIdx.x * 32, q0 = blockIdx.y * 32;
  const int bh = blockIdx.z;
  const int b = bh / Hm, h = bh - b * Hm;
  const int lane = threadIdx.x, i = threadIdx.y;  // lane: column inside the patch, i: row inside the patch
  const int q = q0 + i, k = k0 + lane;
  bool on = false;
  if (q < Sq && k < Sk) on = mask[b * sb + h * sh + static_cast<long long>(q) * sq + k] != 0;
  const uint32_t row_bits = __ballot_sync(0xffffffffu, on);
  if (lane == 0) {
    cols[i] = 0;  // reused below as the transposed patch
  }
  __syncthreads();
  if (on) atomicOr(&cols[lane], 1u << i);
  __syncthreads();
  if (by_q && lane == 0 && q < Sq && RA_IN_BOUNDS(k0 >> 5, 1, Wk, kTagPackMask))
    by_q[(static_cast<long long>(bh) * Sq + q) * Wk + (k0 >> 5)] = row_bits;
  if (by_k && i == 0 && k < Sk && RA_IN_BOUNDS(q0 >> 5, 1, Wq, kTagPackMask))
    by_k[(static_cast<long long>(bh) * Sk + k) * Wq + (q0 >> 5)] = cols[lane];
}
}  // namespace ew
}  // namespace ra

// by_q / by_k must be zero-filled by the caller (words of the padding columns are never written).
extern "C" int ra_pack_mask(const void* mask, long long sb, long long sh, long long sq, void* by_q, void* by_k,
                            int B, int Hm, int Sq, int Sk, void* stream) {
  using namespace ra;
  if (B <= 0 || Hm <= 0 || Sq <= 0 || Sk <= 0 || static_cast<long long>(B) * Hm > 65535) {
    set_error("ra_pack_mask: bad shape");
    return kHostBadArg;
  }
  const int Wk = 4 * ((Sk + 127) / 128), Wq = 4 * ((Sq + 127) / 128);
  dim3 grid((Sk + 31) / 32, (Sq + 31) / 32, B * Hm), block(32, 32);
  if (grid.y > 65535) {
    set_error("ra_pack_mask: too many query rows");
    return kHostBadArg;
  }
  ew::pack_mask_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(mask), sb, sh, sq, static_cast<uint32_t*>(by_q), static_cast<uint32_t*>(by_k),
      Hm, Sq, Sk, Wk, Wq);
  return check_launch("pack_mask");
}
