// The gated delta rule: a linear-attention mixer whose per-head state S [dim, vdim] is decayed, corrected towards the new value
// and read in every token,
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q,
// with q, k, v taken through a short causal convolution over time per channel.  Three kernels:
//   delta_prep_kernel   one warp per (token, unit), the sequence from the block index: convolution + silu of a q / k / v head (the taps - 1 inputs in front of a
//                       portion come from the sequence's convolution state), unit length for q and k, q scale; one more unit per token
//                       for the per-head decay g = exp(-exp(A_log) softplus(a + dt_bias)) and beta = sigmoid(b)
//   delta_scan_kernel   one CTA per (sequence, head, slice of 32 value columns); thread (column v, row group r) keeps rows
//                       [r DPT, (r + 1) DPT) of column v of the state in registers and walks the sequence's new tokens.  One pass over
//                       the state per token: with a = S^T k, c = S^T q of the state BEFORE the token and kq = k . q,
//                           u = beta (v - g a),   o = g c + kq u,   S <- g S + k u^T
//                       (the same sums as the four steps above, regrouped so that a token needs one reduction over row groups).
//                       The CTAs of a sequence also advance its convolution state, a share of the channels each.
//   delta_chunk_kernel  the same recurrence 32 tokens at a time for prompt portions (see there).
// Both states live in fp32 in pools of state slots; a sequence whose first new token sits at position 0 starts from zeros.
// Everything here is plain fp32 FMA code.
#include <cooperative_groups.h>

#include "typed.cuh"

namespace {

struct DeltaArgs {
  nvc_delta_prep p;
  int N;
  int vec;                       // sizes, strides and pointers allow 16-byte accesses
  float* o;
  int ldo;
  float* state;
};

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// grid (token tiles of the longest portion, units, sequences): the sequence comes from the block index, so a warp's first loads are
// its sequence's bounds and nothing has to be searched; CTAs behind a sequence's last token leave at once
__global__ void __launch_bounds__(128, 8) delta_prep_kernel(const DeltaArgs a) {
  pdl_trigger();
  pdl_wait();
  const nvc_delta_prep& p = a.p;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = 2 * p.kv_heads + p.heads + 1;
  const int b = blockIdx.z, uu = blockIdx.y;
  const int r0 = p.cu_seqlens ? p.cu_seqlens[b] : b;
  const int r1 = p.cu_seqlens ? p.cu_seqlens[b + 1] : b + 1;
  const int n = r0 + blockIdx.x * (blockDim.x >> 5) + wid;
  if (n >= r1) return;
  const float* in = p.in + (int64_t)n * p.ldi;
  if (uu == units - 1) {
    // ---- decay and beta of every head
    for (int h = lane; h < p.heads; h += 32) {
      const float dt = softplus_f32(in[p.a_off + h] + __ldg(p.dt_bias + h));
      p.gb_out[(int64_t)n * 2 * p.heads + 2 * h] = -expf(__ldg(p.A_log + h)) * dt;       // log of the decay
      p.gb_out[(int64_t)n * 2 * p.heads + 2 * h + 1] = sigmoid_f32(in[p.b_off + h]);
    }
    return;
  }
  const int t = n - r0;                                 // index inside the portion
  const bool fresh = p.positions[r0] == 0;
  const int C = 2 * p.kv_heads * p.dim + p.heads * p.vdim;
  const float* cs = p.conv_state + (int64_t)p.state_slots[b] * (p.taps - 1) * C;
  // which head: q heads, then k heads, then v heads
  int kind, h;
  if (uu < p.kv_heads) { kind = 0; h = uu; }
  else if (uu < 2 * p.kv_heads) { kind = 1; h = uu - p.kv_heads; }
  else { kind = 2; h = uu - 2 * p.kv_heads; }
  const int width = kind == 2 ? p.vdim : p.dim;
  const int col = (kind == 0 ? p.q_off : (kind == 1 ? p.k_off : p.v_off)) + h * width;            // column of the projection row
  const int ch = (kind == 0 ? 0 : (kind == 1 ? p.kv_heads * p.dim : 2 * p.kv_heads * p.dim)) + h * width;   // channel
  float* out = kind == 0 ? p.q_out + (int64_t)n * p.ldq : (kind == 1 ? p.k_out + (int64_t)n * p.ldk : p.v_out + (int64_t)n * p.ldv);
  out += h * width;
  if (a.vec && width <= 512) {
    // four channels per lane, 16-byte accesses, the head stays in registers between the convolution and the unit length
    float4 y[4];
    float ss4 = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = 4 * lane + 128 * k;
      y[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < width) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < p.taps; ++i) {
          const int src = t - (p.taps - 1) + i;
          float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
          if (src >= 0) x = *reinterpret_cast<const float4*>(in + (int64_t)(src - t) * p.ldi + col + j);
          else if (!fresh) x = *reinterpret_cast<const float4*>(cs + (int64_t)(p.taps - 1 + src) * C + ch + j);
          const float4 w = __ldg(reinterpret_cast<const float4*>(p.conv_w + (int64_t)i * C + ch + j));      // tap-major: lanes read side by side
          acc.x = fmaf(w.x, x.x, acc.x);
          acc.y = fmaf(w.y, x.y, acc.y);
          acc.z = fmaf(w.z, x.z, acc.z);
          acc.w = fmaf(w.w, x.w, acc.w);
        }
        y[k] = make_float4(acc.x * sigmoid_f32(acc.x), acc.y * sigmoid_f32(acc.y), acc.z * sigmoid_f32(acc.z), acc.w * sigmoid_f32(acc.w));
        ss4 += y[k].x * y[k].x + y[k].y * y[k].y + y[k].z * y[k].z + y[k].w * y[k].w;
      }
    }
    float r = 1.f;
    if (kind != 2) r = (kind == 0 ? p.q_scale : 1.f) / sqrtf(warp_sum(ss4) + p.unit_eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = 4 * lane + 128 * k;
      if (j < width) *reinterpret_cast<float4*>(out + j) = make_float4(y[k].x * r, y[k].y * r, y[k].z * r, y[k].w * r);
    }
    return;
  }
  float ss = 0.f;
  for (int j = lane; j < width; j += 32) {
    float acc = 0.f;
    for (int i = 0; i < p.taps; ++i) {
      const int src = t - (p.taps - 1) + i;             // portion index of the input under tap i
      float x;
      if (src >= 0) x = in[(int64_t)(src - t) * p.ldi + col + j];
      else x = fresh ? 0.f : cs[(int64_t)(p.taps - 1 + src) * C + ch + j];
      acc = fmaf(__ldg(p.conv_w + (int64_t)i * C + ch + j), x, acc);
    }
    const float y = acc * sigmoid_f32(acc);
    out[j] = y;
    ss += y * y;
  }
  if (kind == 2) return;
  ss = warp_sum(ss);
  const float r = (kind == 0 ? p.q_scale : 1.f) / sqrtf(ss + p.unit_eps);
  __syncwarp();
  for (int j = lane; j < width; j += 32) out[j] *= r;
}


// The convolution state of a sequence after a portion: the last taps - 1 inputs of (what it held, this portion).  Slot i reads slot
// i + len or the portion, never a slot below itself, so one thread per channel shifts in place.  The channels are spread over the
// CTAs (head, value slice) of the sequence; nothing else in a scan kernel reads this state.
__device__ __forceinline__ void advance_conv_state(const nvc_delta_prep& p, int r0, int r1, bool fresh, int slot) {
  const int C = 2 * p.kv_heads * p.dim + p.heads * p.vdim, len = r1 - r0, keep = p.taps - 1;
  if (keep == 0) return;
  float* cs = p.conv_state + (int64_t)slot * keep * C;
  const int part = blockIdx.y * gridDim.z + blockIdx.z, parts = gridDim.y * gridDim.z;
  const int qk = p.kv_heads * p.dim;
  for (int c = part * blockDim.x + threadIdx.x; c < C; c += parts * blockDim.x) {
    const int col = c < qk ? p.q_off + c : (c < 2 * qk ? p.k_off + c - qk : p.v_off + c - 2 * qk);
    for (int i = 0; i < keep; ++i) {
      const int src = len - keep + i;                 // portion index
      float x;
      if (src >= 0) x = p.in[(int64_t)(r0 + src) * p.ldi + col];
      else x = fresh ? 0.f : cs[(int64_t)(keep + src) * C + c];
      cs[(int64_t)i * C + c] = x;
    }
  }
}

template <int DPT>
__global__ void delta_scan_kernel(const DeltaArgs a) {
  extern __shared__ float sm[];
  pdl_trigger();
  const nvc_delta_prep& p = a.p;
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * 32;
  const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5, groups = blockDim.x >> 5;
  const int v = v0 + lane;
  const bool vok = v < p.vdim;
  const int hk = h / (p.heads / p.kv_heads);
  float* q_s = sm;                    // [2][dim]
  float* k_s = sm + 2 * p.dim;        // [2][dim]
  float* red = sm + 4 * p.dim;        // [3][groups][32]
  pdl_wait();
  const int r0 = p.cu_seqlens ? p.cu_seqlens[b] : b;
  const int r1 = p.cu_seqlens ? p.cu_seqlens[b + 1] : b + 1;
  const bool fresh = p.positions[r0] == 0;
  const int slot = p.state_slots[b];
  advance_conv_state(p, r0, r1, fresh, slot);
  const int d0 = rg * DPT;
  float S[DPT];
  float* sp = a.state + (((int64_t)slot * p.heads + h) * p.dim) * p.vdim;
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = (!fresh && vok && d0 + i < p.dim) ? sp[(int64_t)(d0 + i) * p.vdim + v] : 0.f;
  for (int d = threadIdx.x; d < p.dim; d += blockDim.x) {
    q_s[d] = p.q_out[(int64_t)r0 * p.ldq + hk * p.dim + d];
    k_s[d] = p.k_out[(int64_t)r0 * p.ldk + hk * p.dim + d];
  }
  float vt = vok ? p.v_out[(int64_t)r0 * p.ldv + h * p.vdim + v] : 0.f;
  float gt = expf(p.gb_out[(int64_t)r0 * 2 * p.heads + 2 * h]), bt = p.gb_out[(int64_t)r0 * 2 * p.heads + 2 * h + 1];
  __syncthreads();
  for (int t = r0; t < r1; ++t) {
    const int cur = (t - r0) & 1;
    const float* qc = q_s + cur * p.dim;
    const float* kc = k_s + cur * p.dim;
    float vn = 0.f, gn = 0.f, bn = 0.f;
    if (t + 1 < r1) {       // fetch the next token into the other buffer
      for (int d = threadIdx.x; d < p.dim; d += blockDim.x) {
        q_s[(cur ^ 1) * p.dim + d] = p.q_out[(int64_t)(t + 1) * p.ldq + hk * p.dim + d];
        k_s[(cur ^ 1) * p.dim + d] = p.k_out[(int64_t)(t + 1) * p.ldk + hk * p.dim + d];
      }
      vn = vok ? p.v_out[(int64_t)(t + 1) * p.ldv + h * p.vdim + v] : 0.f;
      gn = expf(p.gb_out[(int64_t)(t + 1) * 2 * p.heads + 2 * h]);
      bn = p.gb_out[(int64_t)(t + 1) * 2 * p.heads + 2 * h + 1];
    }
    float sk = 0.f, sq = 0.f, kq = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      if (d0 + i < p.dim) {
        const float kv = kc[d0 + i], qv = qc[d0 + i];
        sk = fmaf(S[i], kv, sk);
        sq = fmaf(S[i], qv, sq);
        kq = fmaf(kv, qv, kq);
      }
    }
    if (groups > 1) {
      red[(0 * groups + rg) * 32 + lane] = sk;
      red[(1 * groups + rg) * 32 + lane] = sq;
      red[(2 * groups + rg) * 32 + lane] = kq;
      __syncthreads();
      sk = sq = kq = 0.f;
      for (int g = 0; g < groups; ++g) {
        sk += red[(0 * groups + g) * 32 + lane];
        sq += red[(1 * groups + g) * 32 + lane];
        kq += red[(2 * groups + g) * 32 + lane];
      }
    }
    const float u = bt * (vt - gt * sk);
    if (vok && rg == 0) a.o[(int64_t)t * a.ldo + h * p.vdim + v] = fmaf(kq, u, gt * sq);
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < p.dim) S[i] = fmaf(gt, S[i], kc[d0 + i] * u);
    vt = vn; gt = gn; bt = bn;
    __syncthreads();
  }
  if (vok)
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < p.dim) sp[(int64_t)(d0 + i) * p.vdim + v] = S[i];
}


// ---- prompt portions: 32 tokens at a time.  Within a chunk that starts from the state S0, with L_t the running sum of log g up to
// token t (so exp(L_t - L_j) is the decay between tokens j and t),
//   u_t = beta_t (v_t - exp(L_t) S0^T k_t - sum_{j<t} exp(L_t - L_j) (k_j . k_t) u_j)        a triangular system, solved forwards
//   o_t = exp(L_t) S0^T q_t + sum_{j<=t} exp(L_t - L_j) (k_j . q_t) u_j
//   S   = exp(L_n) S0 + sum_j exp(L_n - L_j) k_j u_j^T
// which are the four steps of the recurrence written out over the chunk; only differences L_t - L_j <= 0 are exponentiated, so a
// decay that underflows over a chunk stays a plain zero.  One CTA of four warps per (sequence, head, 32 value columns); thread
// (column v, warp w) keeps rows [w DPT, (w + 1) DPT) of column v of the state in registers.  Tokens behind a portion's end are
// padded with g = 1, beta = 0, k = q = v = 0, which leaves state and outputs alone.
constexpr int kDC = 32;
constexpr int kDW = 4;
constexpr int kDAs = kDC + 4;            // row stride of the token-by-token matrices (16-byte rows)

// staged key / query rows: 4 DPT numbers and more (zeros behind `dim`), 16-byte aligned, rows 4 banks apart
__host__ __device__ inline int delta_chunk_row(int dim, int dpt) { return max((dim + 3) / 4 * 4, kDW * dpt) + 4; }
__host__ __device__ inline size_t delta_chunk_smem_floats(int dim, int dpt) {
  return (size_t)2 * kDC * delta_chunk_row(dim, dpt) + 2 * kDC * kDAs + 3 * kDC * 32 + (size_t)kDW * kDC * 32 + 2 * kDC + 8;
}

__device__ __forceinline__ float fma4(const float4& x, const float4& y, float acc) {
  acc = fmaf(x.x, y.x, acc);
  acc = fmaf(x.y, y.y, acc);
  acc = fmaf(x.z, y.z, acc);
  return fmaf(x.w, y.w, acc);
}

// Forward substitution of the chunk's triangular system, one value column per lane of one warp: Us holds v_t on entry and u_t on
// return.  Fully unrolled (the u_t live in registers); not inlined, so that it is compiled once and not once per kernel variant.
__device__ __noinline__ void delta_chunk_solve(const float* Am, float* Us, const float* W1, const float* Ls, const float* Bs, int lane) {
  constexpr int as = kDAs;
  float u[kDC];
#pragma unroll
  for (int t = 0; t < kDC; ++t) {
    float x = Bs[t] * (Us[t * 32 + lane] - expf(Ls[t]) * W1[t * 32 + lane]);
#pragma unroll
    for (int j4 = 0; j4 < t; j4 += 4) {       // entries at and behind the diagonal are zero
      const float4 am = *reinterpret_cast<const float4*>(Am + t * as + j4);
      x = fmaf(-am.x, u[j4], x);
      if (j4 + 1 < t) x = fmaf(-am.y, u[j4 + 1], x);
      if (j4 + 2 < t) x = fmaf(-am.z, u[j4 + 2], x);
      if (j4 + 3 < t) x = fmaf(-am.w, u[j4 + 3], x);
    }
    u[t] = x;
  }
#pragma unroll
  for (int t = 0; t < kDC; ++t) Us[t * 32 + lane] = u[t];
}

// kCluster: the CTAs of one (sequence, head) - its slices of 32 value columns - form a thread-block cluster, split the rows of the two
// token-by-token matrices among themselves and write them into one another's shared memory: the products that do not depend on the
// value column are computed once per (sequence, head), not once per slice.
template <int DPT, bool kCluster>
__global__ void __launch_bounds__(kDW * 32) delta_chunk_kernel(const DeltaArgs a) {
  namespace cg = cooperative_groups;
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  const nvc_delta_prep& p = a.p;
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * 32;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int v = v0 + lane;
  const bool vok = v < p.vdim;
  const int hk = h / (p.heads / p.kv_heads);
  const int dim = p.dim, ds = delta_chunk_row(dim, DPT), dz = ds - 4;      // dz: numbers of a row that the products read
  constexpr int as = kDAs;
  float* Ks = sm;                          // [kDC][ds]
  float* Qs = Ks + kDC * ds;               // [kDC][ds]
  float* Am = Qs + kDC * ds;               // [kDC][as]  beta_t exp(L_t - L_j) (k_t . k_j), j < t
  float* Pm = Am + kDC * as;               // [kDC][as]  exp(L_t - L_j) (q_t . k_j), j <= t
  float* Us = Pm + kDC * as;               // [kDC][32]  v_t, then u_t
  float* W1 = Us + kDC * 32;               // [kDC][32]  S0^T k_t
  float* W2 = W1 + kDC * 32;               // [kDC][32]  S0^T q_t
  float* Wp = W2 + kDC * 32;               // [kDW][kDC][32] partial sums of the row groups
  float* Ls = Wp + kDW * kDC * 32;         // [kDC]
  float* Bs = Ls + kDC;                    // [kDC]
  pdl_wait();
  const int r0 = p.cu_seqlens ? p.cu_seqlens[b] : b;
  const int r1 = p.cu_seqlens ? p.cu_seqlens[b + 1] : b + 1;
  const bool fresh = p.positions[r0] == 0;
  const int slot = p.state_slots[b];
  advance_conv_state(p, r0, r1, fresh, slot);
  const int d0 = w * DPT;
  float S[DPT];                            // rows behind `dim` stay zero: the staged rows are zero there
  float* sp = a.state + (((int64_t)slot * p.heads + h) * dim) * p.vdim;
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = (!fresh && vok && d0 + i < dim) ? sp[(int64_t)(d0 + i) * p.vdim + v] : 0.f;
  for (int c0 = r0; c0 < r1; c0 += kDC) {
    const int n = min(kDC, r1 - c0);
    // ---- stage the chunk (a row per warp and pass: no division, coalesced)
    for (int t = w; t < kDC; t += kDW) {
      const float* kg = p.k_out + (int64_t)(c0 + t) * p.ldk + hk * dim;
      const float* qg = p.q_out + (int64_t)(c0 + t) * p.ldq + hk * dim;
      for (int c = lane; c < dz; c += 32) {
        const bool in = t < n && c < dim;
        Ks[t * ds + c] = in ? kg[c] : 0.f;
        Qs[t * ds + c] = in ? qg[c] : 0.f;
      }
      Us[t * 32 + lane] = (t < n && vok) ? p.v_out[(int64_t)(c0 + t) * p.ldv + h * p.vdim + v] : 0.f;
    }
    if (w == 0) {
      float lg = lane < n ? p.gb_out[(int64_t)(c0 + lane) * 2 * p.heads + 2 * h] : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, lg, o);
        if (lane >= o) lg += up;
      }
      Ls[lane] = lg;
      Bs[lane] = lane < n ? p.gb_out[(int64_t)(c0 + lane) * 2 * p.heads + 2 * h + 1] : 0.f;
    }
    __syncthreads();
    // ---- products between the chunk's tokens: two rows t per warp and pass, column j per lane, 16-byte operands
    {
      const int Z = kCluster ? (int)gridDim.z : 1, zr = kCluster ? (int)blockIdx.z : 0;
      for (int t = 2 * (zr + Z * w); t < kDC; t += 2 * Z * kDW) {
        float kk0 = 0.f, qk0 = 0.f, kk1 = 0.f, qk1 = 0.f;
        if (lane <= t + 1) {
          const float4* kt0 = reinterpret_cast<const float4*>(Ks + t * ds);
          const float4* qt0 = reinterpret_cast<const float4*>(Qs + t * ds);
          const float4* kt1 = reinterpret_cast<const float4*>(Ks + (t + 1) * ds);
          const float4* qt1 = reinterpret_cast<const float4*>(Qs + (t + 1) * ds);
          const float4* kj = reinterpret_cast<const float4*>(Ks + lane * ds);
#pragma unroll 2
          for (int c = 0; c < dz / 4; ++c) {
            const float4 x = kj[c];
            kk0 = fma4(kt0[c], x, kk0);
            qk0 = fma4(qt0[c], x, qk0);
            kk1 = fma4(kt1[c], x, kk1);
            qk1 = fma4(qt1[c], x, qk1);
          }
          const float e0 = expf(fminf(Ls[t] - Ls[lane], 0.f)), e1 = expf(fminf(Ls[t + 1] - Ls[lane], 0.f));
          kk0 *= e0 * Bs[t];
          qk0 *= e0;
          kk1 *= e1 * Bs[t + 1];
          qk1 *= e1;
        }
        const float a0 = lane < t ? kk0 : 0.f, p0 = lane <= t ? qk0 : 0.f, a1 = lane < t + 1 ? kk1 : 0.f, p1 = lane <= t + 1 ? qk1 : 0.f;
        if constexpr (kCluster) {
          cg::cluster_group cl = cg::this_cluster();
          for (int r = 0; r < Z; ++r) {
            float* am = cl.map_shared_rank(Am, r);
            float* pm = cl.map_shared_rank(Pm, r);
            am[t * as + lane] = a0;
            pm[t * as + lane] = p0;
            am[(t + 1) * as + lane] = a1;
            pm[(t + 1) * as + lane] = p1;
          }
        } else {
          Am[t * as + lane] = a0;
          Pm[t * as + lane] = p0;
          Am[(t + 1) * as + lane] = a1;
          Pm[(t + 1) * as + lane] = p1;
        }
      }
    }
    // ---- what the state before the chunk says to every key and query: partial sums over this warp's rows, then over the warps
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const float* X = pass == 0 ? Ks : Qs;
      float* Wd = pass == 0 ? W1 : W2;
#pragma unroll 1
      for (int t0 = 0; t0 < kDC; t0 += 8) {
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float4 x = *reinterpret_cast<const float4*>(X + (t0 + u) * ds + d0 + i);
            acc[u] = fmaf(S[i], x.x, acc[u]);
            acc[u] = fmaf(S[i + 1], x.y, acc[u]);
            acc[u] = fmaf(S[i + 2], x.z, acc[u]);
            acc[u] = fmaf(S[i + 3], x.w, acc[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) Wp[(w * kDC + t0 + u) * 32 + lane] = acc[u];
      }
      __syncthreads();
      for (int t = w; t < kDC; t += kDW) {
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < kDW; ++g) s += Wp[(g * kDC + t) * 32 + lane];
        Wd[t * 32 + lane] = s;
      }
      __syncthreads();
    }
    if constexpr (kCluster) cg::this_cluster().sync();      // every slice's rows of the two matrices have arrived
    // ---- the triangular system, one value column per lane of warp 0
    if (w == 0) delta_chunk_solve(Am, Us, W1, Ls, Bs, lane);
    __syncthreads();
    // ---- outputs and the state behind the chunk
    {
      float uu[kDC];
#pragma unroll
      for (int j = 0; j < kDC; ++j) uu[j] = Us[j * 32 + lane];
      for (int t = w; t < n; t += kDW) {
        float o = expf(Ls[t]) * W2[t * 32 + lane];
#pragma unroll
        for (int j4 = 0; j4 < kDC; j4 += 4) {     // entries behind the diagonal are zero
          const float4 pm = *reinterpret_cast<const float4*>(Pm + t * as + j4);
          o = fmaf(pm.x, uu[j4], o);
          o = fmaf(pm.y, uu[j4 + 1], o);
          o = fmaf(pm.z, uu[j4 + 2], o);
          o = fmaf(pm.w, uu[j4 + 3], o);
        }
        if (vok) a.o[(int64_t)(c0 + t) * a.ldo + h * p.vdim + v] = o;
      }
      const float Ln = Ls[kDC - 1];
      const float gn = expf(Ln);
#pragma unroll
      for (int i = 0; i < DPT; ++i) S[i] *= gn;
#pragma unroll 4
      for (int j = 0; j < kDC; ++j) {             // a loop over the tokens around an unrolled pass over this thread's rows: short code
        const float uj = Us[j * 32 + lane] * expf(Ln - Ls[j]);
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 x = *reinterpret_cast<const float4*>(Ks + j * ds + d0 + i);
          S[i] = fmaf(x.x, uj, S[i]);
          S[i + 1] = fmaf(x.y, uj, S[i + 1]);
          S[i + 2] = fmaf(x.z, uj, S[i + 2]);
          S[i + 3] = fmaf(x.w, uj, S[i + 3]);
        }
      }
    }
    if constexpr (kCluster) cg::this_cluster().sync();      // no slice writes the next chunk's rows into a neighbour that still reads these
    else __syncthreads();
  }
  if (vok)
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < dim) sp[(int64_t)(d0 + i) * p.vdim + v] = S[i];
}

template <int DPT>
cudaError_t launch_delta_chunk(nvc_ctx* ctx, const DeltaArgs& a, dim3 grid, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_chunk_kernel<DPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(delta_chunk_kernel<DPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  static const bool no_cluster = getenv("NVC_DELTA_CLUSTER") && atoi(getenv("NVC_DELTA_CLUSTER")) == 0;
  if (grid.z >= 2 && grid.z <= 8 && !no_cluster)       // the value slices of a (sequence, head) as one cluster
    return nvc_launch_cluster3(ctx, delta_chunk_kernel<DPT, true>, grid, dim3(kDW * 32), smem, st, dim3(1, 1, grid.z), a);
  return nvc_launch(ctx, delta_chunk_kernel<DPT, false>, grid, dim3(kDW * 32), smem, st, a);
}

int check_prep(nvc_ctx* ctx, const nvc_delta_prep* p) {
  NVC_REQUIRE(ctx, ctx && p && p->in && p->conv_w && p->conv_state && p->state_slots && p->positions && p->A_log && p->dt_bias && p->q_out &&
                       p->k_out && p->v_out && p->gb_out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, p->heads > 0 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->dim > 0 && p->vdim > 0 && p->taps >= 1 && p->B > 0 &&
                       p->dim <= 1024 && p->heads <= 65535, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, p->ldq >= p->kv_heads * p->dim && p->ldk >= p->kv_heads * p->dim && p->ldv >= p->heads * p->vdim, NVC_EINVAL, "bad strides");
  return NVC_OK;
}

}  // namespace

extern "C" int nvc_delta_prep_run(nvc_ctx* ctx, const nvc_delta_prep* p, int N, int max_qlen, void* stream) {
  int rc = check_prep(ctx, p);
  if (rc) return rc;
  NVC_REQUIRE(ctx, p->cu_seqlens || N == p->B, NVC_EINVAL, "rows without cu_seqlens: one per sequence");
  if (N == 0) return NVC_OK;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const int vec = p->dim % 4 == 0 && p->vdim % 4 == 0 && p->ldi % 4 == 0 && p->q_off % 4 == 0 && p->k_off % 4 == 0 && p->v_off % 4 == 0 && p->ldq % 4 == 0 &&
                  p->ldk % 4 == 0 && p->ldv % 4 == 0 && al16(p->in) && al16(p->conv_state) && al16(p->conv_w) && al16(p->q_out) && al16(p->k_out) && al16(p->v_out);
  DeltaArgs a{*p, N, vec, nullptr, 0, nullptr};
  const int units = 2 * p->kv_heads + p->heads + 1;
  const int longest = p->cu_seqlens ? std::min(N, std::max(max_qlen, 1)) : 1;
  NVC_REQUIRE(ctx, units <= 65535 && p->B <= 65535, NVC_ESHAPE, "more than 65 535 heads or sequences");
  const int warps = longest >= 4 ? 4 : 1;
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, delta_prep_kernel, dim3((unsigned)((longest + warps - 1) / warps), units, p->B), dim3(32 * warps), 0,
                                 nvc_stream(stream), a));
  ctx->launches++;
  return NVC_OK;
}

extern "C" int nvc_delta_rule_scan(nvc_ctx* ctx, const nvc_delta_prep* p, float* o, int ldo, float* state, int max_qlen, void* stream) {
  int rc = check_prep(ctx, p);
  if (rc) return rc;
  NVC_REQUIRE(ctx, o && state && ldo >= p->heads * p->vdim && max_qlen >= 1, NVC_EINVAL, "bad output / state");
  DeltaArgs a{*p, 0, 0, o, ldo, state};
  const int dim = p->dim;
  if (p->cu_seqlens && max_qlen >= 8 && dim <= 256) {
    // prompt portions: 32 tokens at a time (keys of more than 256 numbers stay token by token)
    const int per = (dim + kDW - 1) / kDW;     // rows of the state per warp
    const int cd = per <= 8 ? 8 : (per <= 16 ? 16 : (per <= 32 ? 32 : 64));
    const dim3 grid(p->B, p->heads, (p->vdim + 31) / 32);
    const size_t smem = delta_chunk_smem_floats(dim, cd) * sizeof(float);
    cudaError_t ce;
    if (cd == 8) ce = launch_delta_chunk<8>(ctx, a, grid, smem, nvc_stream(stream));
    else if (cd == 16) ce = launch_delta_chunk<16>(ctx, a, grid, smem, nvc_stream(stream));
    else if (cd == 32) ce = launch_delta_chunk<32>(ctx, a, grid, smem, nvc_stream(stream));
    else ce = launch_delta_chunk<64>(ctx, a, grid, smem, nvc_stream(stream));
    NVC_CUDA_CHECK(ctx, ce);
    ctx->launches++;
    return NVC_OK;
  }
  // about four row groups per value column: four times the warps - and loads in flight - of one thread per whole column, at the price
  // of one shared-memory reduction of three numbers per token
  const int dpt = dim <= 64 ? 16 : (dim <= 128 ? 32 : (dim <= 256 ? 64 : 128));
  const int groups = (dim + dpt - 1) / dpt;
  const dim3 grid(p->B, p->heads, (p->vdim + 31) / 32), block(32 * groups);
  const size_t smem = ((size_t)4 * dim + (size_t)3 * groups * 32) * sizeof(float);
  cudaError_t ce;
  switch (dpt) {
    case 16: ce = nvc_launch(ctx, delta_scan_kernel<16>, grid, block, smem, nvc_stream(stream), a); break;
    case 32: ce = nvc_launch(ctx, delta_scan_kernel<32>, grid, block, smem, nvc_stream(stream), a); break;
    case 64: ce = nvc_launch(ctx, delta_scan_kernel<64>, grid, block, smem, nvc_stream(stream), a); break;
    default: ce = nvc_launch(ctx, delta_scan_kernel<128>, grid, block, smem, nvc_stream(stream), a); break;
  }
  NVC_CUDA_CHECK(ctx, ce);
  ctx->launches++;
  return NVC_OK;
}
