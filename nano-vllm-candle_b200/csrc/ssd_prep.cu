// nvc_ssd_prep: a selective state space layer between its fused projection and its recurrence, over the new tokens of every sequence
// of a step (fp32 throughout):
//   channels [x | B | C]     causal convolution over time per channel with a bias, then silu.  The taps - 1 inputs in front of a
//                            portion come from the sequence's convolution state (zeros for a sequence that starts at position 0)
//   dt_h                     softplus(projection + dt_bias_h), no clamp
//   outputs                  x, v = dt x (what the recurrence adds to the state, with B as its key), B, C,
//                            log decay = -exp(A_log_h) dt   (the recurrence multiplies the state by its exponential)
// nvc_ssd_conv_advance then writes every sequence's last taps - 1 inputs into its state slot (a portion shorter than that keeps the
// tail of what the slot held).  It runs behind the first kernel on the same stream, which still reads the old state.
// The recurrence itself is nvc_decay_scan (retention.cu) with q = C, k = B, a decay per token and head and the skip term D x.
#include "typed.cuh"

namespace {

constexpr int kMaxTaps = 16;

struct SsdArgs {
  nvc_ssd_prep p;
  int N;
};

__device__ __forceinline__ int ssd_find_seq(const int32_t* cu, int B, int row) {
  int lo = 0, hi = B - 1;      // largest b with cu[b] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float softplus_f32(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

constexpr int kPrepThreads = 256;

// CTA = (token, block of 256 x CW channels): the token's sequence is looked up once, and the step sizes of the heads whose channels
// the CTA holds are computed once (a softplus per channel would cost more than the convolution).  A thread takes CW neighbouring
// channels - 4 with 16-byte accesses when every width, offset and stride is a multiple of 4 (a head never ends inside a thread's
// four), else 1 - and a warp reads neighbouring columns of a projection row.
template <int CW>
__global__ void __launch_bounds__(kPrepThreads) ssd_prep_kernel(const SsdArgs a) {
  constexpr int kSpan = kPrepThreads * CW;
  __shared__ int s_r0, s_fresh, s_slot;
  __shared__ float s_dt[kSpan];
  pdl_trigger();
  pdl_wait();
  const nvc_ssd_prep& p = a.p;
  const int inner = p.heads * p.vdim, gn = p.groups * p.state, C = inner + 2 * gn;
  const int n = blockIdx.x, c0 = blockIdx.y * kSpan, c = c0 + CW * threadIdx.x;
  if (threadIdx.x == 0) {
    int b = n, r0 = n;
    if (p.cu_seqlens) {
      b = ssd_find_seq(p.cu_seqlens, p.B, n);
      r0 = p.cu_seqlens[b];
    }
    s_r0 = r0;
    s_fresh = p.positions[r0] == 0;
    s_slot = p.state_slots[b];
  }
  const int h_first = c0 / p.vdim;                       // the first head with channels in this CTA
  if (c0 < inner) {
    for (int h = h_first + threadIdx.x; h < p.heads && h * p.vdim < c0 + kSpan; h += kPrepThreads) {
      const float dt = softplus_f32(p.in[(int64_t)n * p.ldi + p.dt_off + h] + __ldg(p.dt_bias + h));
      s_dt[h - h_first] = dt;
      if (h * p.vdim >= c0) p.log_decay[(int64_t)n * p.ldl + h] = -expf(__ldg(p.A_log + h)) * dt;     // the CTA with the head's first channel
    }
  }
  __syncthreads();
  if (c >= C) return;
  const int r0 = s_r0;
  const int t = n - r0;                                  // index inside the portion
  const bool fresh = s_fresh != 0;
  const float* st = p.conv_state + (int64_t)s_slot * (p.taps - 1) * C;
  float acc[CW], y[CW];
  if (CW == 4) {
    const float4 b4 = *reinterpret_cast<const float4*>(p.conv_b + c);
    acc[0] = b4.x; acc[1 % CW] = b4.y; acc[2 % CW] = b4.z; acc[3 % CW] = b4.w;
  } else {
    acc[0] = __ldg(p.conv_b + c);
  }
  for (int i2 = 0; i2 < p.taps; ++i2) {
    const int idx = t - (p.taps - 1) + i2;               // the input's index inside the portion; negative: in front of it
    const float* xp = idx >= 0 ? p.in + (int64_t)(r0 + idx) * p.ldi + p.xbc_off + c : st + (int64_t)(p.taps - 1 + idx) * C + c;
    const float* wp = p.conv_w + (int64_t)i2 * C + c;
    const bool zero = idx < 0 && fresh;
    if (CW == 4) {
      const float4 x4 = zero ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(xp);
      const float4 w4 = *reinterpret_cast<const float4*>(wp);
      acc[0] = fmaf(w4.x, x4.x, acc[0]); acc[1 % CW] = fmaf(w4.y, x4.y, acc[1 % CW]);
      acc[2 % CW] = fmaf(w4.z, x4.z, acc[2 % CW]); acc[3 % CW] = fmaf(w4.w, x4.w, acc[3 % CW]);
    } else {
      acc[0] = fmaf(__ldg(wp), zero ? 0.f : *xp, acc[0]);
    }
  }
#pragma unroll
  for (int u = 0; u < CW; ++u) y[u] = acc[u] * sigmoid_f32(acc[u]);
  float* out;
  if (c < inner) {
    const float dt = s_dt[c / p.vdim - h_first];
    out = p.x_out + (int64_t)n * p.ldx + c;
    float* vo = p.v_out + (int64_t)n * p.ldx + c;
    if (CW == 4) *reinterpret_cast<float4*>(vo) = make_float4(dt * y[0], dt * y[1 % CW], dt * y[2 % CW], dt * y[3 % CW]);
    else vo[0] = dt * y[0];
  } else if (c < inner + gn) {
    out = p.b_out + (int64_t)n * p.ldbc + c - inner;
  } else {
    out = p.c_out + (int64_t)n * p.ldbc + c - inner - gn;
  }
  if (CW == 4) *reinterpret_cast<float4*>(out) = make_float4(y[0], y[1 % CW], y[2 % CW], y[3 % CW]);
  else out[0] = y[0];
}

// thread = (sequence, channel): reads the taps - 1 inputs that end the sequence so far, then writes them
__global__ void ssd_conv_advance_kernel(const SsdArgs a) {
  pdl_trigger();
  pdl_wait();
  const nvc_ssd_prep& p = a.p;
  const int C = p.heads * p.vdim + 2 * p.groups * p.state, keep = p.taps - 1;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)p.B * C) return;
  const int b = (int)(i / C), c = (int)(i % C);
  const int r0 = p.cu_seqlens ? p.cu_seqlens[b] : b;
  const int r1 = p.cu_seqlens ? p.cu_seqlens[b + 1] : b + 1;
  const int qlen = r1 - r0;
  const bool fresh = p.positions[r0] == 0;
  float* st = p.conv_state + (int64_t)p.state_slots[b] * keep * C;
  float v[kMaxTaps];
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) {
    if (j < keep) {
      const int idx = qlen - keep + j;
      if (idx >= 0) v[j] = p.in[(int64_t)(r0 + idx) * p.ldi + p.xbc_off + c];
      else v[j] = fresh ? 0.f : st[(int64_t)(keep + idx) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j)
    if (j < keep) st[(int64_t)j * C + c] = v[j];
}

int check(nvc_ctx* ctx, const nvc_ssd_prep* p) {
  NVC_REQUIRE(ctx, ctx && p && p->in && p->conv_w && p->conv_b && p->conv_state && p->state_slots && p->positions, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, p->heads > 0 && p->vdim > 0 && p->groups > 0 && p->heads % p->groups == 0 && p->state > 0 && p->taps >= 1 && p->taps <= kMaxTaps &&
                       p->B > 0,
              NVC_EINVAL, "bad sizes (up to 16 taps)");
  const int C = p->heads * p->vdim + 2 * p->groups * p->state;
  NVC_REQUIRE(ctx, p->xbc_off >= 0 && p->dt_off >= 0 && p->ldi >= p->xbc_off + C && p->ldi >= p->dt_off + p->heads, NVC_EINVAL, "bad columns");
  return NVC_OK;
}

}  // namespace

extern "C" int nvc_ssd_prep_run(nvc_ctx* ctx, const nvc_ssd_prep* p, int N, void* stream) {
  int rc = check(ctx, p);
  if (rc) return rc;
  NVC_REQUIRE(ctx, p->A_log && p->dt_bias && p->x_out && p->v_out && p->b_out && p->c_out && p->log_decay, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= p->B && p->ldx >= p->heads * p->vdim && p->ldbc >= p->groups * p->state && p->ldl >= p->heads, NVC_EINVAL, "bad strides");
  const int C = p->heads * p->vdim + 2 * p->groups * p->state;
  SsdArgs a{*p, N};
  if (N == 0) return NVC_OK;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const int gn = p->groups * p->state;
  const bool vec = ((p->vdim | gn | p->ldi | p->xbc_off | p->ldx | p->ldbc) & 3) == 0 && al16(p->in) && al16(p->conv_w) && al16(p->conv_b) &&
                   al16(p->conv_state) && al16(p->x_out) && al16(p->v_out) && al16(p->b_out) && al16(p->c_out);
  if (vec) {
    NVC_CUDA_CHECK(ctx, nvc_launch(ctx, ssd_prep_kernel<4>, dim3((unsigned)N, (unsigned)((C + 4 * kPrepThreads - 1) / (4 * kPrepThreads))),
                                   dim3(kPrepThreads), 0, nvc_stream(stream), a));
  } else {
    NVC_CUDA_CHECK(ctx, nvc_launch(ctx, ssd_prep_kernel<1>, dim3((unsigned)N, (unsigned)((C + kPrepThreads - 1) / kPrepThreads)), dim3(kPrepThreads), 0,
                                   nvc_stream(stream), a));
  }
  ctx->launches++;
  return NVC_OK;
}

extern "C" int nvc_ssd_conv_advance(nvc_ctx* ctx, const nvc_ssd_prep* p, void* stream) {
  int rc = check(ctx, p);
  if (rc) return rc;
  if (p->taps == 1) return NVC_OK;
  const int C = p->heads * p->vdim + 2 * p->groups * p->state;
  SsdArgs a{*p, 0};
  const int64_t total = (int64_t)p->B * C;
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, ssd_conv_advance_kernel, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, nvc_stream(stream), a));
  ctx->launches++;
  return NVC_OK;
}
