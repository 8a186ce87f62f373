// The gated delta rule: a linear-attention mixer whose per-head state S [dim, vdim] is decayed, corrected towards the new value
// and read in every token,
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q,
// with q, k, v taken through a short causal convolution over time per channel.  Two kernels:
//   delta_prep_kernel   one warp per (token, unit): convolution + silu of a q / k / v head (the taps - 1 inputs in front of a
//                       portion come from the sequence's convolution state), unit length for q and k, q scale; one more unit per token
//                       for the per-head decay g = exp(-exp(A_log) softplus(a + dt_bias)) and beta = sigmoid(b)
//   delta_scan_kernel   one CTA per (sequence, head, slice of 32 value columns); thread (column v, row group r) keeps rows
//                       [r DPT, (r + 1) DPT) of column v of the state in registers and walks the sequence's new tokens.  One pass over
//                       the state per token: with a = S^T k, c = S^T q of the state BEFORE the token and kq = k . q,
//                           u = beta (v - g a),   o = g c + kq u,   S <- g S + k u^T
//                       (the same sums as the four steps above, regrouped so that a token needs one reduction over row groups).
//                       The CTAs of head 0, slice 0 also advance the convolution state of their sequence.
// Both states live in fp32 in pools of state slots; a sequence whose first new token sits at position 0 starts from zeros.
// Everything here is plain fp32 FMA code.
#include "typed.cuh"

namespace {

struct DeltaArgs {
  nvc_delta_prep p;
  int N;
  float* o;
  int ldo;
  float* state;
};

__device__ __forceinline__ int delta_find_seq(const int32_t* cu, int B, int row) {
  int lo = 0, hi = B - 1;      // largest b with cu[b] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__global__ void delta_prep_kernel(const DeltaArgs a) {
  pdl_trigger();
  pdl_wait();
  const nvc_delta_prep& p = a.p;
  const int warps = blockDim.x >> 5, wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = 2 * p.kv_heads + p.heads + 1;
  const int64_t u = (int64_t)blockIdx.x * warps + wid;
  if (u >= (int64_t)a.N * units) return;
  const int n = (int)(u / units), uu = (int)(u % units);
  const float* in = p.in + (int64_t)n * p.ldi;
  if (uu == units - 1) {
    // ---- decay and beta of every head
    for (int h = lane; h < p.heads; h += 32) {
      const float dt = softplus_f32(in[p.a_off + h] + __ldg(p.dt_bias + h));
      p.gb_out[(int64_t)n * 2 * p.heads + 2 * h] = expf(-expf(__ldg(p.A_log + h)) * dt);
      p.gb_out[(int64_t)n * 2 * p.heads + 2 * h + 1] = sigmoid_f32(in[p.b_off + h]);
    }
    return;
  }
  int b = n, r0 = n;
  if (p.cu_seqlens) {
    b = delta_find_seq(p.cu_seqlens, p.B, n);
    r0 = p.cu_seqlens[b];
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
  float ss = 0.f;
  for (int j = lane; j < width; j += 32) {
    const float* w = p.conv_w + (int64_t)(ch + j) * p.taps;
    float acc = 0.f;
    for (int i = 0; i < p.taps; ++i) {
      const int src = t - (p.taps - 1) + i;             // portion index of the input under tap i
      float x;
      if (src >= 0) x = in[(int64_t)(src - t) * p.ldi + col + j];
      else x = fresh ? 0.f : cs[(int64_t)(p.taps - 1 + src) * C + ch + j];
      acc = fmaf(__ldg(w + i), x, acc);
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
  if (h == 0 && blockIdx.z == 0) {
    // ---- the convolution state of this sequence: the last taps - 1 inputs of (what it held, this portion); slot i reads slot
    // i + len or the portion, never a slot below itself, so one thread per channel can shift in place
    const int C = 2 * p.kv_heads * p.dim + p.heads * p.vdim, len = r1 - r0, keep = p.taps - 1;
    float* cs = p.conv_state + (int64_t)slot * keep * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const int qk = p.kv_heads * p.dim;
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
  float gt = p.gb_out[(int64_t)r0 * 2 * p.heads + 2 * h], bt = p.gb_out[(int64_t)r0 * 2 * p.heads + 2 * h + 1];
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
      gn = p.gb_out[(int64_t)(t + 1) * 2 * p.heads + 2 * h];
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

int check_prep(nvc_ctx* ctx, const nvc_delta_prep* p) {
  NVC_REQUIRE(ctx, ctx && p && p->in && p->conv_w && p->conv_state && p->state_slots && p->positions && p->A_log && p->dt_bias && p->q_out &&
                       p->k_out && p->v_out && p->gb_out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, p->heads > 0 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->dim > 0 && p->vdim > 0 && p->taps >= 1 && p->B > 0 &&
                       p->dim <= 1024 && p->heads <= 65535, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, p->ldq >= p->kv_heads * p->dim && p->ldk >= p->kv_heads * p->dim && p->ldv >= p->heads * p->vdim, NVC_EINVAL, "bad strides");
  return NVC_OK;
}

}  // namespace

extern "C" int nvc_delta_prep_run(nvc_ctx* ctx, const nvc_delta_prep* p, int N, void* stream) {
  int rc = check_prep(ctx, p);
  if (rc) return rc;
  NVC_REQUIRE(ctx, p->cu_seqlens || N == p->B, NVC_EINVAL, "rows without cu_seqlens: one per sequence");
  if (N == 0) return NVC_OK;
  DeltaArgs a{*p, N, nullptr, 0, nullptr};
  const int64_t units = (int64_t)N * (2 * p->kv_heads + p->heads + 1);
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, delta_prep_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, nvc_stream(stream), a));
  ctx->launches++;
  return NVC_OK;
}

extern "C" int nvc_delta_rule_scan(nvc_ctx* ctx, const nvc_delta_prep* p, float* o, int ldo, float* state, int max_qlen, void* stream) {
  int rc = check_prep(ctx, p);
  if (rc) return rc;
  NVC_REQUIRE(ctx, o && state && ldo >= p->heads * p->vdim && max_qlen >= 1, NVC_EINVAL, "bad output / state");
  DeltaArgs a{*p, 0, o, ldo, state};
  const int dim = p->dim;
  const int dpt = dim <= 16 ? 16 : (dim <= 32 ? 32 : (dim <= 64 ? 64 : 128));
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
