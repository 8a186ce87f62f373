// Tensor-pipe kernel of nvc_attn_paged_wide (bf16 storage, included by attn_wide.cu only): grouped-query softmax attention with
// separate key and value widths, a sliding window or a chunk mask, capped scores, a sink, a sigmoid gate and a constant factor.
//
// The M dimension of mma.sync.m16n8k16 holds 16 (token, head) rows of ONE sequence and ONE key / value head: the heads / kv_heads
// query heads that share a key head are packed beside one another, so a key / value tile is loaded once for all of them.  Every
// row has its own visible range [lo, hi] (window and causal bound).  Keys go through shared memory in tiles that start at
// multiples of 64 tokens (cp.async, 16-byte-chunk XOR swizzle), K read with ldmatrix for S = Q K^T, V with ldmatrix.trans for
// O += P V; online softmax in the log2 domain on the accumulator fragments, fp32 accumulators.
//   64 rows and more (a prompt portion): a CTA takes 64 consecutive rows, 16 per warp, and all four warps read the same 64-token
//     tiles from one ring; tiles in front of the CTA's earliest visible key are never loaded (a window costs its own length).
//   fewer rows (decode, short portions): a CTA takes one 16-row chunk, warp w owns the 16-token tiles w, w + 4, ... in a private
//     ring, and the warps merge once at the end.
// DKM / DVM: compile-time bounds of the head sizes (64 or 128 numbers); the real sizes are multiples of 16 up to them.
#pragma once
#include <algorithm>
#include <cstdlib>

#include "paged_decode_mma.cuh"
#include "typed.cuh"

namespace widemma {

using pdmma::cp_async16;
using pdmma::cp_async_commit;
using pdmma::cp_async_wait;
using pdmma::fast_exp2;
using pdmma::ldmatrix_x4;
using pdmma::ldmatrix_x4_trans;
using pdmma::mma_bf16;

constexpr int kWarps = 4;
constexpr int kCtaTok = 64;
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;

struct Args {
  const nvc_bf16 *q, *k_cache, *v_cache;
  nvc_bf16* out;
  int ldq, ldk, ldv, ldo;
  const int32_t *block_tables, *context_lens, *cu_seqlens;
  int bt_stride, block_size;
  int heads, kv_heads, dk, dv;
  float scale_log2e;
  int window;
  const float* sink;
  const float* gate;
  int ldg;
  float out_scale;
  int chunk;                 // > 0: a row sees the keys of its own chunk of that many positions only
  float cap_log2e;           // > 0: scores are cap tanh(s / cap): cap * log2(e) here and scale / cap in scale_log2e
  int gate_per_head;         // the gate holds one number per head instead of one per output number
};

// first key a row at position pos sees (both rules are monotone in pos)
__host__ __device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  return window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : (chunk > 0 ? pos - pos % chunk : 0);
}
// tanh from one exp2 and one division: absolute error of a few 1e-7, exact limits at both ends
__device__ __forceinline__ float tanh_exp2(float x) { return 1.0f - __fdividef(2.0f, fast_exp2(x * (2.0f * kLog2e)) + 1.0f); }

template <int DKM, int DVM> constexpr int smem_bytes() {
  constexpr int ring = kStages * kCtaTok * (DKM + DVM) * 2;
  constexpr int merge = (2 * kWarps * 16 + kWarps * 16 * DVM) * 4;
  return ring > merge ? ring : merge;
}

// One online-softmax step of a warp's 16 rows over NSUB consecutive 16-token sub-tiles (the first `nsub` are computed).
// stK / stV: shared-memory addresses of the tile's first key / value row; rows of DKM / DVM numbers, chunks swizzled by row & 7.
template <int DKM, int DVM, int NSUB>
__device__ __forceinline__ void softmax_step(uint32_t stK, uint32_t stV, int tok0, int nsub, int ks_n, int nt_n, const uint32_t (*qa)[4],
                                             float (*o)[4], float& m0, float& m1, float& l0, float& l1, int lo_a, int hi_a, int lo_b, int hi_b,
                                             float scale_log2e, float cap_log2e, bool all_visible, int lane) {
  constexpr int RBK = DKM * 2, RBV = DVM * 2, KS = DKM / 16, NT = DVM / 8;
  const int tq = lane & 3;
  float s[2 * NSUB][4];
  {
    const int r = (lane & 7) + ((lane >> 4) << 3);
    const int chi = (lane >> 3) & 1;
#pragma unroll
    for (int j = 0; j < 2 * NSUB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    // k-steps outside, sub-tiles inside: consecutive MMAs go to different accumulators (no back-to-back dependent pairs)
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      if (ks < ks_n) {
        const int c = 2 * ks + chi;
#pragma unroll
        for (int j = 0; j < NSUB; ++j) {
          if (j < nsub) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(stK + (j * 16 + r) * RBK + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
            mma_bf16(s[2 * j], qa[ks], b0, b1);
            mma_bf16(s[2 * j + 1], qa[ks], b2, b3);
          }
        }
      }
    }
  }
  // columns tok0 + 8 jn + 2 tq + {0, 1}; a sub-tile that was not computed lies behind every row's bound
  float mx0 = -INFINITY, mx1 = -INFINITY;
  if (cap_log2e > 0.f) {       // scale_log2e carries scale / cap: the capped score, already in the log2 domain, needs no further factor
#pragma unroll
    for (int jn = 0; jn < 2 * NSUB; ++jn) {
      s[jn][0] = cap_log2e * tanh_exp2(s[jn][0] * scale_log2e); s[jn][1] = cap_log2e * tanh_exp2(s[jn][1] * scale_log2e);
      s[jn][2] = cap_log2e * tanh_exp2(s[jn][2] * scale_log2e); s[jn][3] = cap_log2e * tanh_exp2(s[jn][3] * scale_log2e);
    }
    scale_log2e = 1.f;
  }
  if (all_visible) {
#pragma unroll
    for (int jn = 0; jn < 2 * NSUB; ++jn) {
      s[jn][0] *= scale_log2e; s[jn][1] *= scale_log2e; s[jn][2] *= scale_log2e; s[jn][3] *= scale_log2e;
      mx0 = fmaxf(mx0, fmaxf(s[jn][0], s[jn][1]));
      mx1 = fmaxf(mx1, fmaxf(s[jn][2], s[jn][3]));
    }
  } else {
#pragma unroll
    for (int jn = 0; jn < 2 * NSUB; ++jn) {
      const int t0 = tok0 + 8 * jn + 2 * tq;
      s[jn][0] = (t0 >= lo_a && t0 <= hi_a) ? s[jn][0] * scale_log2e : -INFINITY;
      s[jn][1] = (t0 + 1 >= lo_a && t0 + 1 <= hi_a) ? s[jn][1] * scale_log2e : -INFINITY;
      s[jn][2] = (t0 >= lo_b && t0 <= hi_b) ? s[jn][2] * scale_log2e : -INFINITY;
      s[jn][3] = (t0 + 1 >= lo_b && t0 + 1 <= hi_b) ? s[jn][3] * scale_log2e : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[jn][0], s[jn][1]));
      mx1 = fmaxf(mx1, fmaxf(s[jn][2], s[jn][3]));
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
  // a row that has seen no key yet keeps m = -inf: subtract 0 instead, every exponential below is then exp2(-inf) = 0
  const float mb0 = mn0 == -INFINITY ? 0.f : mn0, mb1 = mn1 == -INFINITY ? 0.f : mn1;
  const float al0 = fast_exp2(m0 - mb0), al1 = fast_exp2(m1 - mb1);
  m0 = mn0;
  m1 = mn1;
  uint32_t pa[NSUB][4];
  float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
  for (int jn = 0; jn < 2 * NSUB; ++jn) {
    const float p0 = fast_exp2(s[jn][0] - mb0), p1 = fast_exp2(s[jn][1] - mb0);
    const float p2 = fast_exp2(s[jn][2] - mb1), p3 = fast_exp2(s[jn][3] - mb1);
    ps0 += p0 + p1;
    ps1 += p2 + p3;
    pa[jn >> 1][2 * (jn & 1)] = pack_bf16(p0, p1);
    pa[jn >> 1][2 * (jn & 1) + 1] = pack_bf16(p2, p3);
  }
  l0 = l0 * al0 + ps0;
  l1 = l1 * al1 + ps1;
  if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {      // a running maximum moved: rare after the first tiles
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      o[nt][0] *= al0; o[nt][1] *= al0;
      o[nt][2] *= al1; o[nt][3] *= al1;
    }
  }
  {
    const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int cadd = lane >> 4;
#pragma unroll
    for (int j = 0; j < NSUB; ++j) {
      if (j < nsub) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          if (2 * np < nt_n) {
            const int c = 2 * np + cadd;
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(stV + (j * 16 + r) * RBV + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
            mma_bf16(o[2 * np], pa[j], b0, b1);
            mma_bf16(o[2 * np + 1], pa[j], b2, b3);
          }
        }
      }
    }
  }
}

template <int DKM, int DVM>
__global__ void __launch_bounds__(kWarps * 32) attn_wide_mma_kernel(const Args a) {
  constexpr int RBK = DKM * 2, RBV = DVM * 2, KS = DKM / 16, NT = DVM / 8;
  constexpr int kTileK = kCtaTok * RBK, kTileBytes = kCtaTok * (RBK + RBV);
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y, g = blockIdx.z;
  const int hg = a.heads / a.kv_heads;
  const int row_begin = a.cu_seqlens ? a.cu_seqlens[b] : b;
  const int qlen = a.cu_seqlens ? a.cu_seqlens[b + 1] - row_begin : 1;
  const int total = qlen * hg;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, tq = lane & 3;
  const int ctx_len = a.context_lens[b];
  const int base = ctx_len - qlen;                  // token t of the portion sits at position base + t
  const int32_t* bt = a.block_tables + (int64_t)b * a.bt_stride;
  const int ks_n = a.dk >> 4, nt_n = a.dv >> 3;     // k-steps of S and n-tiles of O that exist
  const int nck = a.dk >> 3, ncv = a.dv >> 3;       // 16-byte chunks per key / value row
  const nvc_bf16* kc = a.k_cache + (int64_t)g * a.dk;
  const nvc_bf16* vc = a.v_cache + (int64_t)g * a.dv;
  const bool many = total >= 16 * kWarps;
  int r0c;                                          // first row of the CTA
  if (many) {
    const int n64 = (total + 16 * kWarps - 1) / (16 * kWarps);
    if ((int)blockIdx.x >= n64) return;
    r0c = (n64 - 1 - (int)blockIdx.x) * (16 * kWarps);     // the rows with the most keys start first
  } else {
    r0c = blockIdx.x * 16;
    if (r0c >= total) return;
  }
  const int r0 = many ? r0c + warp * 16 : r0c;
  const int ra = r0 + quad, rb = r0 + quad + 8;
  const bool va = ra < total, vb = rb < total;
  const int ta = va ? ra / hg : 0, tb = vb ? rb / hg : 0;
  const int ha = g * hg + (va ? ra - ta * hg : 0), hb = g * hg + (vb ? rb - tb * hg : 0);
  const int hi_a = va ? base + ta : -1, hi_b = vb ? base + tb : -1;
  const int lo_a = first_visible(hi_a, a.window, a.chunk), lo_b = first_visible(hi_b, a.window, a.chunk);
  // Q as A fragments (rows past the end are zero)
  uint32_t qa[KS][4];
  {
    const nvc_bf16* qrow0 = a.q + (int64_t)(row_begin + ta) * a.ldq + (int64_t)ha * a.dk;
    const nvc_bf16* qrow1 = a.q + (int64_t)(row_begin + tb) * a.ldq + (int64_t)hb * a.dk;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + 2 * tq;
      const bool in = ks < ks_n;
      qa[ks][0] = va && in ? __ldg(reinterpret_cast<const uint32_t*>(qrow0 + d)) : 0u;
      qa[ks][1] = vb && in ? __ldg(reinterpret_cast<const uint32_t*>(qrow1 + d)) : 0u;
      qa[ks][2] = va && in ? __ldg(reinterpret_cast<const uint32_t*>(qrow0 + d + 8)) : 0u;
      qa[ks][3] = vb && in ? __ldg(reinterpret_cast<const uint32_t*>(qrow1 + d + 8)) : 0u;
    }
  }
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  // One warp loads 16 consecutive tokens' K and V rows (tok0 a multiple of 16) into a tile at stK / stV.  Every lane owns one
  // 16-byte chunk of a row - lanes [0, nck) a key chunk, lanes [nck, nck + ncv) a value chunk (nck + ncv <= 32) - so a row is one
  // cp.async per lane.  With a block size that is a multiple of 16 the tile lies in one block: one table lookup per tile.
  // Rows past kmax are zero-filled.
  const bool lane_k = lane < nck, lane_on = lane < nck + ncv;
  const int lc = lane_k ? lane : lane - nck;
  const uint8_t* lane_src = lane_k ? reinterpret_cast<const uint8_t*>(kc) + lc * 16 : reinterpret_cast<const uint8_t*>(vc) + lc * 16;
  const int64_t lane_pitch = lane_k ? (int64_t)a.ldk * 2 : (int64_t)a.ldv * 2;
  const bool one_block = (a.block_size & 15) == 0;
  auto load16 = [&](uint32_t stK, uint32_t stV, int tok0, int kmax) {
    const uint32_t dst0 = lane_k ? stK : stV;
    constexpr int RBmax = RBK > RBV ? RBK : RBV;
    const uint32_t rb = lane_k ? RBK : RBV;
    (void)RBmax;
    if (one_block) {
      const int tl = min(tok0, kmax);              // a tile wholly past kmax is zero-filled: look up a token that exists
      const int64_t slot0 = (int64_t)__ldg(bt + tl / a.block_size) * a.block_size + tl % a.block_size;
      const uint8_t* src = lane_src + slot0 * lane_pitch;
      const int nvalid = kmax - tok0 + 1;          // rows of the tile that exist
      if (lane_on) {
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const bool ok = r < nvalid;
          cp_async16(dst0 + r * rb + ((lc ^ (r & 7)) << 4), ok ? src + r * lane_pitch : src, ok ? 16u : 0u);
        }
      }
    } else {
      int64_t my_slot = 0;
      if (lane < 16) {
        const int tk = min(tok0 + lane, kmax);
        my_slot = (int64_t)__ldg(bt + tk / a.block_size) * a.block_size + tk % a.block_size;
      }
#pragma unroll 4
      for (int r = 0; r < 16; ++r) {
        const int64_t slot = __shfl_sync(0xffffffffu, my_slot, r);
        if (lane_on) cp_async16(dst0 + r * rb + ((lc ^ (r & 7)) << 4), lane_src + slot * lane_pitch, tok0 + r <= kmax ? 16u : 0u);
      }
    }
  };
  if (many) {
    const int last_c = min(r0c + 16 * kWarps - 1, total - 1);
    const int kmax_cta = base + last_c / hg;
    const int kmin_cta = first_visible(base + r0c / hg, a.window, a.chunk);
    const int kmax_w = r0 < total ? base + min(r0 + 15, total - 1) / hg : -1;    // a warp past the end only loads
    const int first_w = base + r0 / hg;                                          // position of the warp's first row
    const int kmin_w = first_visible(first_w, a.window, a.chunk);
    // a tile is wholly visible to every row of the warp when it lies in [lo of the LAST row, hi of the FIRST row]
    const int lo_last = first_visible(kmax_w, a.window, a.chunk);
    const int tile0 = kmin_cta / kCtaTok;
    const int n_tiles = kmax_cta / kCtaTok + 1 - tile0;
    const uint32_t ring = smem_u32(smem);
    auto issue = [&](int i) {
      if (i < n_tiles) {      // warp w brings rows 16 w .. 16 w + 15 of the 64-token tile
        const uint32_t st = ring + (i % kStages) * kTileBytes;
        load16(st + warp * 16 * RBK, st + kTileK + warp * 16 * RBV, (tile0 + i) * kCtaTok + warp * 16, kmax_cta);
      }
      cp_async_commit();
    };
#pragma unroll
    for (int p = 0; p < kStages - 1; ++p) issue(p);
    for (int i = 0; i < n_tiles; ++i) {
      cp_async_wait<kStages - 2>();       // tile i has landed (later tiles may be in flight)
      __syncthreads();                    // ... for every thread's part of it; and every warp is done with tile i - 1,
      issue(i + kStages - 1);             // whose stage the newly issued tile takes
      const int tok0 = (tile0 + i) * kCtaTok;
      if (tok0 > kmax_w || tok0 + kCtaTok - 1 < kmin_w) continue;    // warp-uniform: nothing of this tile is visible to the warp
      const uint32_t st = ring + (i % kStages) * kTileBytes;
      const int nsub = min(kCtaTok / 16, (kmax_w - tok0) / 16 + 1);
      const bool all_visible = tok0 >= lo_last && tok0 + kCtaTok - 1 <= first_w;     // (rows past the end have q = 0: finite, never stored)
      softmax_step<DKM, DVM, kCtaTok / 16>(st, st + kTileK, tok0, nsub, ks_n, nt_n, qa, o, m0, m1, l0, l1, lo_a, hi_a, lo_b, hi_b, a.scale_log2e,
                                           a.cap_log2e, all_visible, lane);
    }
    cp_async_wait<0>();
  } else {
    // few rows: the four warps split the KEYS of one 16-row chunk
    const int last_row = min(r0 + 15, total - 1);
    const int kmax = base + last_row / hg;
    const int kmin = first_visible(base + r0 / hg, a.window, a.chunk);
    const int first = (kmin / kCtaTok) * kCtaTok + warp * 16;       // this warp's first 16-token tile
    const int hi_first = base + r0 / hg;                            // the chunk's first row sees the least far ahead,
    const int lo_last = first_visible(kmax, a.window, a.chunk);   // its last row the least far back
    const int n_tiles = kmax >= first ? (kmax - first) / kCtaTok + 1 : 0;
    constexpr int kWarpStage = 16 * (RBK + RBV);
    const uint32_t ring = smem_u32(smem) + warp * (kStages * kWarpStage);
    auto issue = [&](int i) {
      if (i < n_tiles) load16(ring + (i % kStages) * kWarpStage, ring + (i % kStages) * kWarpStage + 16 * RBK, first + i * kCtaTok, kmax);
      cp_async_commit();
    };
#pragma unroll
    for (int p = 0; p < kStages - 1; ++p) issue(p);
    for (int i = 0; i < n_tiles; ++i) {
      issue(i + kStages - 1);
      cp_async_wait<kStages - 1>();
      __syncwarp();
      const uint32_t st = ring + (i % kStages) * kWarpStage;
      const int tok0 = first + i * kCtaTok;
      softmax_step<DKM, DVM, 1>(st, st + 16 * RBK, tok0, 1, ks_n, nt_n, qa, o, m0, m1, l0, l1, lo_a, hi_a, lo_b, hi_b, a.scale_log2e,
                                a.cap_log2e, tok0 >= lo_last && tok0 + 15 <= hi_first, lane);
      __syncwarp();
    }
    cp_async_wait<0>();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (many) {
    // this warp's rows are complete: the sink joins the denominator, then gate, factor and store (pairs of columns)
    float f0 = 1.f, f1 = 1.f;
    if (a.sink) {
      const float sa = __ldg(a.sink + ha) * kLog2e, sb = __ldg(a.sink + hb) * kLog2e;
      const float Ma = fmaxf(m0, sa), Mb = fmaxf(m1, sb);
      f0 = fast_exp2(m0 - Ma); l0 = l0 * f0 + fast_exp2(sa - Ma);
      f1 = fast_exp2(m1 - Mb); l1 = l1 * f1 + fast_exp2(sb - Mb);
    }
    const float i0 = l0 > 0.f ? f0 * a.out_scale / l0 : 0.f, i1 = l1 > 0.f ? f1 * a.out_scale / l1 : 0.f;
    nvc_bf16* o0 = a.out + (int64_t)(row_begin + ta) * a.ldo + (int64_t)ha * a.dv;
    nvc_bf16* o1 = a.out + (int64_t)(row_begin + tb) * a.ldo + (int64_t)hb * a.dv;
    const float* g0 = a.gate && !a.gate_per_head ? a.gate + (int64_t)(row_begin + ta) * a.ldg + (int64_t)ha * a.dv : nullptr;
    const float* g1 = a.gate && !a.gate_per_head ? a.gate + (int64_t)(row_begin + tb) * a.ldg + (int64_t)hb * a.dv : nullptr;
    float i0h = 1.f, i1h = 1.f;
    if (a.gate && a.gate_per_head) {
      if (va) i0h = sigmoid_f32(a.gate[(int64_t)(row_begin + ta) * a.ldg + ha]);
      if (vb) i1h = sigmoid_f32(a.gate[(int64_t)(row_begin + tb) * a.ldg + hb]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (nt < nt_n) {
        const int d = nt * 8 + 2 * tq;
        if (va) {
          float x = o[nt][0] * i0 * i0h, y = o[nt][1] * i0 * i0h;
          if (g0) { x *= sigmoid_f32(g0[d]); y *= sigmoid_f32(g0[d + 1]); }
          *reinterpret_cast<uint32_t*>(o0 + d) = pack_bf16(x, y);
        }
        if (vb) {
          float x = o[nt][2] * i1 * i1h, y = o[nt][3] * i1 * i1h;
          if (g1) { x *= sigmoid_f32(g1[d]); y *= sigmoid_f32(g1[d + 1]); }
          *reinterpret_cast<uint32_t*>(o1 + d) = pack_bf16(x, y);
        }
      }
    }
    return;
  }
  // ---- merge the warps (the rings are dead now)
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(smem);       // [kWarps][16]
  float* sm_l = sm_m + kWarps * 16;
  float* sm_o = sm_l + kWarps * 16;                   // [kWarps][16][DVM]
  if (tq == 0) {
    sm_m[warp * 16 + quad] = m0;
    sm_m[warp * 16 + quad + 8] = m1;
    sm_l[warp * 16 + quad] = l0;
    sm_l[warp * 16 + quad + 8] = l1;
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int d = nt * 8 + 2 * tq;
    float* p0 = sm_o + (warp * 16 + quad) * DVM + d;
    float* p1 = sm_o + (warp * 16 + quad + 8) * DVM + d;
    p0[0] = o[nt][0]; p0[1] = o[nt][1];
    p1[0] = o[nt][2]; p1[1] = o[nt][3];
  }
  __syncthreads();
  const int nrows = min(16, total - r0);
  for (int idx = threadIdx.x; idx < nrows * a.dv; idx += kWarps * 32) {
    const int rr = idx / a.dv, d = idx - rr * a.dv;
    const int row = r0 + rr, t = row / hg, h = g * hg + row - t * hg;
    const float sk = a.sink ? __ldg(a.sink + h) * kLog2e : -INFINITY;
    float M = sk;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sm_m[w * 16 + rr]);
    float L = a.sink ? fast_exp2(sk - M) : 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_m[w * 16 + rr];
      const float wt = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      L += sm_l[w * 16 + rr] * wt;
      O += sm_o[(w * 16 + rr) * DVM + d] * wt;
    }
    float y = L > 0.f ? O / L * a.out_scale : 0.f;
    if (a.gate) y *= sigmoid_f32(a.gate[(int64_t)(row_begin + t) * a.ldg + (a.gate_per_head ? (int64_t)h : (int64_t)h * a.dv + d)]);
    a.out[(int64_t)(row_begin + t) * a.ldo + (int64_t)h * a.dv + d] = __bfloat16_as_ushort(__float2bfloat16_rn(y));
  }
}

}  // namespace widemma

namespace {

inline bool attn_wide_mma_takes(const nvc_attn_spec& s, int ldq, int ldk, int ldv, int ldo, int block_size) {
  static const bool off = getenv("NVC_ATTN_WIDE_MMA") && atoi(getenv("NVC_ATTN_WIDE_MMA")) == 0;
  return !off && s.dim % 16 == 0 && s.vdim % 16 == 0 && s.dim <= 128 && s.vdim <= 128 && ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 &&
         ldo % 2 == 0 && block_size > 0 && (!s.gate || s.gate_per_head || s.ldg % 2 == 0);
}

template <int DKM, int DVM>
inline int attn_wide_mma_launch_t(nvc_ctx* ctx, const widemma::Args& a, dim3 grid, cudaStream_t stream) {
  constexpr int smem = widemma::smem_bytes<DKM, DVM>();
  static bool attr_set = false;
  if (!attr_set) {
    NVC_CUDA_CHECK(ctx, cudaFuncSetAttribute(widemma::attn_wide_mma_kernel<DKM, DVM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, widemma::attn_wide_mma_kernel<DKM, DVM>, grid, dim3(widemma::kWarps * 32), (size_t)smem, stream, a));
  ctx->launches++;
  return NVC_OK;
}

inline int attn_wide_mma_launch(nvc_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, void* out, int ldq, int ldk, int ldv, int ldo,
                                const int32_t* block_tables, const int32_t* context_lens, const int32_t* cu_seqlens, int bt_stride, int B, int rows,
                                int max_qlen, int block_size, const nvc_attn_spec& s, cudaStream_t stream) {
  const int hg = s.heads / s.kv_heads;
  const int max_total = (cu_seqlens ? max_qlen : 1) * hg;
  const int gx = max_total >= 64 ? std::max((max_total + 63) / 64, 4) : (max_total + 15) / 16;
  if (s.kv_heads > 65535 || B > 65535) return NVC_ENOTIMPL;
  widemma::Args a{reinterpret_cast<const nvc_bf16*>(q), reinterpret_cast<const nvc_bf16*>(k_cache), reinterpret_cast<const nvc_bf16*>(v_cache),
                  reinterpret_cast<nvc_bf16*>(out), ldq, ldk, ldv, ldo, block_tables, context_lens, cu_seqlens, bt_stride, block_size,
                  s.heads, s.kv_heads, s.dim, s.vdim, s.softcap > 0.f ? s.scale / s.softcap : s.scale * widemma::kLog2e, s.window, s.sink, s.gate, s.ldg,
                  s.out_scale, s.chunk, s.softcap * widemma::kLog2e, s.gate_per_head};
  const dim3 grid(gx, B, s.kv_heads);
  const bool k64 = s.dim <= 64, v64 = s.vdim <= 64;
  if (k64 && v64) return attn_wide_mma_launch_t<64, 64>(ctx, a, grid, stream);
  if (k64) return attn_wide_mma_launch_t<64, 128>(ctx, a, grid, stream);
  if (v64) return attn_wide_mma_launch_t<128, 64>(ctx, a, grid, stream);
  return attn_wide_mma_launch_t<128, 128>(ctx, a, grid, stream);
}

}  // namespace
