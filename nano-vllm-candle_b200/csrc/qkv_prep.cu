// nvc_qkv_prep: everything between the fused q / k / v projection of a mixer and its attention or recurrence, in one pass
// over the fp32 projection rows:
//   + bias                                   (optional)
//   silu                                     (optional, on q, k and v)
//   per-head RMS norm of q and k             (optional; one weight vector of `dim` numbers shared by the heads, or no weight)
//   rotary positions on the first rot_dims numbers of every q / k head, pairs (2i, 2i + 1) or (i, i + rot_dims / 2),
//                                            angles from a table of (cos, sin) per position
//   k *= k_scale                             (after the rotation)
//   value blending                           v <- (1 - lambda) v + lambda v_first, or v_first <- v in the layer that provides it
//   v *= v_scale                             (a constant weight of the mixer, so that every attention kernel can leave it out)
//   stores                                   q to its buffer; k and v to rows of a paged cache (slot mapping) or to plain rows
// One warp per (token, head) of q, k or v; a head is staged in shared memory so that any pairing reads its partner.  The purely
// element-wise case (bias and silu only, plain fp32 rows out) runs a flat kernel with 16-byte accesses instead.
#include "typed.cuh"

namespace {

struct PrepArgs {
  nvc_qkv_prep p;
  int N;
};

template <typename TQ, typename TKV>
__global__ void qkv_prep_kernel(const PrepArgs a) {
  extern __shared__ float stage[];
  pdl_trigger();
  pdl_wait();
  const nvc_qkv_prep& p = a.p;
  const int warps = blockDim.x >> 5, wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = p.q_heads + 2 * p.kv_heads;
  const int64_t u = (int64_t)blockIdx.x * warps + wid;
  if (u >= (int64_t)a.N * units) return;
  const int n = (int)(u / units), uu = (int)(u % units);
  const int wmax = p.dim > p.vdim ? p.dim : p.vdim;
  float* x = stage + (size_t)wid * wmax;
  const float* in = p.in + (int64_t)n * p.ldi;
  if (uu >= p.q_heads + p.kv_heads) {
    // ---- a value head
    const int h = uu - p.q_heads - p.kv_heads;
    const int col = p.v_off + h * p.vdim;
    const int64_t orow = p.slot_mapping ? p.slot_mapping[n] : n;
    const float lam = p.blend == NVC_BLEND_MIX ? __ldg(p.lambda) : 0.f;
    for (int j = lane; j < p.vdim; j += 32) {
      float v = in[col + j] + (p.bias ? __ldg(p.bias + col + j) : 0.f);
      if (p.act == NVC_PREP_ACT_SILU) v = v * sigmoid_f32(v);
      if (p.blend == NVC_BLEND_PROVIDE) p.v_first[(int64_t)n * p.ldvf + h * p.vdim + j] = v;
      else if (p.blend == NVC_BLEND_MIX) v = (1.0f - lam) * v + lam * p.v_first[(int64_t)n * p.ldvf + h * p.vdim + j];
      v *= p.v_scale;
      if (orow >= 0) st_f(reinterpret_cast<TKV*>(p.v_out) + orow * p.ldv + h * p.vdim + j, v);
    }
    return;
  }
  const bool is_q = uu < p.q_heads;
  const int h = is_q ? uu : uu - p.q_heads;
  const int col = (is_q ? p.q_off : p.k_off) + h * p.dim;
  const int64_t orow = is_q ? n : (p.slot_mapping ? p.slot_mapping[n] : n);
  if (orow < 0) return;
  float ss = 0.f;
  for (int j = lane; j < p.dim; j += 32) {
    float v = in[col + j] + (p.bias ? __ldg(p.bias + col + j) : 0.f);
    if (p.act == NVC_PREP_ACT_SILU) v = v * sigmoid_f32(v);
    x[j] = v;
    ss += v * v;
  }
  const float* nw = is_q ? p.q_norm : p.k_norm;
  float r = 1.f;
  if (nw || p.unit_norm) {
    ss = warp_sum(ss);
    r = 1.0f / sqrtf(ss / (float)p.dim + p.eps);
  }
  __syncwarp();
  const int half = p.rot_dims >> 1;
  const float2* tab = reinterpret_cast<const float2*>(p.rot_table) + (int64_t)(p.rot_dims ? p.positions[n] : 0) * half;
  const float post = is_q ? 1.f : p.k_scale;
  for (int j = lane; j < p.dim; j += 32) {
    float y = x[j] * r * (nw ? __ldg(nw + j) : 1.f);
    if (j < p.rot_dims) {
      int i, partner;
      float sign;
      if (p.rot_half) { i = j < half ? j : j - half; partner = j < half ? j + half : j - half; sign = j < half ? -1.f : 1.f; }
      else { i = j >> 1; partner = j ^ 1; sign = (j & 1) ? 1.f : -1.f; }
      const float2 cs = __ldg(tab + i);
      const float z = x[partner] * r * (nw ? __ldg(nw + partner) : 1.f);
      y = y * cs.x + sign * z * cs.y;
    }
    y *= post;
    if (is_q) st_f(reinterpret_cast<TQ*>(p.q_out) + orow * p.ldq + h * p.dim + j, y);
    else st_f(reinterpret_cast<TKV*>(p.k_out) + orow * p.ldk + h * p.dim + j, y);
  }
}


// The element-wise case (no norm, no rotation, no blending, no scale, plain fp32 rows out): q, k, v = act(in + bias), four numbers per
// thread.  CTA = (token, block of 256 x 4 columns of [q | k | v]).
__global__ void __launch_bounds__(256) prep_flat_kernel(const PrepArgs a) {
  pdl_trigger();
  pdl_wait();
  const nvc_qkv_prep& p = a.p;
  const int qw = p.q_heads * p.dim, kw = p.kv_heads * p.dim, vw = p.kv_heads * p.vdim;
  const int64_t n = blockIdx.x;
  const int j = 4 * (blockIdx.y * blockDim.x + threadIdx.x);          // column of [q | k | v]
  if (j >= qw + kw + vw) return;
  int col;
  float* out;
  if (j < qw) { col = p.q_off + j; out = reinterpret_cast<float*>(p.q_out) + n * p.ldq + j; }
  else if (j < qw + kw) { col = p.k_off + j - qw; out = reinterpret_cast<float*>(p.k_out) + n * p.ldk + j - qw; }
  else { col = p.v_off + j - qw - kw; out = reinterpret_cast<float*>(p.v_out) + n * p.ldv + j - qw - kw; }
  float4 v = *reinterpret_cast<const float4*>(p.in + n * p.ldi + col);
  if (p.bias) {
    const float4 b = *reinterpret_cast<const float4*>(p.bias + col);
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  if (p.act == NVC_PREP_ACT_SILU) { v.x *= sigmoid_f32(v.x); v.y *= sigmoid_f32(v.y); v.z *= sigmoid_f32(v.z); v.w *= sigmoid_f32(v.w); }
  *reinterpret_cast<float4*>(out) = v;
}

// one warp per (token, head) of a query projection laid out [heads][dim | rot_dim]: the unrotated part goes to out_a, the rotated
// part (turned by the token's position) to out_b
template <typename T>
__global__ void head_split_rot_kernel(const float* __restrict__ in, int ldi, int heads, int dim, int rot_dim, int rot_dims, int rot_half,
                                      const float* __restrict__ rot_table, const int32_t* __restrict__ positions, T* __restrict__ out_a,
                                      int ld_a, int hs_a, T* __restrict__ out_b, int ld_b, int hs_b, int off_b, int N) {
  pdl_trigger();
  pdl_wait();
  const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (u >= (int64_t)N * heads) return;
  const int n = (int)(u / heads), h = (int)(u % heads);
  const float* x = in + (int64_t)n * ldi + (int64_t)h * (dim + rot_dim);
  T* a = out_a + (int64_t)n * ld_a + (int64_t)h * hs_a;
  for (int j = lane; j < dim; j += 32) st_f(a + j, x[j]);
  const float* xr = x + dim;
  T* b = out_b + (int64_t)n * ld_b + (int64_t)h * hs_b + off_b;
  const int half = rot_dims >> 1;
  const float2* tab = reinterpret_cast<const float2*>(rot_table) + (int64_t)(rot_dims ? positions[n] : 0) * half;
  for (int j = lane; j < rot_dim; j += 32) {
    float y = xr[j];
    if (j < rot_dims) {
      int i, partner;
      float sign;
      if (rot_half) { i = j < half ? j : j - half; partner = j < half ? j + half : j - half; sign = j < half ? -1.f : 1.f; }
      else { i = j >> 1; partner = j ^ 1; sign = (j & 1) ? 1.f : -1.f; }
      const float2 cs = __ldg(tab + i);
      y = y * cs.x + sign * xr[partner] * cs.y;
    }
    st_f(b + j, y);
  }
}

template <typename TQ, typename TKV>
int launch_prep(nvc_ctx* ctx, const nvc_qkv_prep* p, int N, void* stream) {
  PrepArgs a{*p, N};
  const int64_t units = (int64_t)N * (p->q_heads + 2 * p->kv_heads);
  const int wmax = p->dim > p->vdim ? p->dim : p->vdim;
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, qkv_prep_kernel<TQ, TKV>, dim3((unsigned)((units + 3) / 4)), dim3(128), (size_t)4 * wmax * sizeof(float),
                                 nvc_stream(stream), a));
  ctx->launches++;
  return NVC_OK;
}

}  // namespace

extern "C" int nvc_qkv_prep_run(nvc_ctx* ctx, const nvc_qkv_prep* p, int N, void* stream) {
  NVC_REQUIRE(ctx, ctx && p && p->in && p->q_out && p->k_out && p->v_out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && p->q_heads > 0 && p->kv_heads > 0 && p->dim > 0 && p->vdim > 0 && p->dim <= 2048 && p->vdim <= 2048,
              NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, p->rot_dims >= 0 && p->rot_dims % 2 == 0 && p->rot_dims <= p->dim && (p->rot_dims == 0 || (p->rot_table && p->positions)),
              NVC_EINVAL, "bad rotary arguments");
  NVC_REQUIRE(ctx, (p->q_norm == nullptr) == (p->k_norm == nullptr) && !(p->unit_norm && p->q_norm), NVC_EINVAL,
              "q and k norms come together, with a weight or without");
  NVC_REQUIRE(ctx, p->blend == NVC_BLEND_NONE || (p->v_first && p->ldvf >= p->kv_heads * p->vdim && (p->blend != NVC_BLEND_MIX || p->lambda)),
              NVC_EINVAL, "value blending needs its buffer and weight");
  NVC_REQUIRE(ctx, p->ldq >= p->q_heads * p->dim && p->ldk >= p->kv_heads * p->dim && p->ldv >= p->kv_heads * p->vdim, NVC_EINVAL,
              "bad strides");
  if (N == 0) return NVC_OK;
  {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    const int qw = p->q_heads * p->dim, kw = p->kv_heads * p->dim, vw = p->kv_heads * p->vdim;
    const bool flat = p->q_dtype == NVC_DT_F32 && p->kv_dtype == NVC_DT_F32 && !p->q_norm && !p->unit_norm && p->rot_dims == 0 &&
                      p->blend == NVC_BLEND_NONE && !p->slot_mapping && p->k_scale == 1.f && p->v_scale == 1.f &&
                      ((qw | kw | vw | p->q_off | p->k_off | p->v_off | p->ldi | p->ldq | p->ldk | p->ldv) & 3) == 0 && al16(p->in) &&
                      al16(p->bias) && al16(p->q_out) && al16(p->k_out) && al16(p->v_out);
    if (flat) {
      PrepArgs a{*p, N};
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, prep_flat_kernel, dim3((unsigned)N, (unsigned)(((qw + kw + vw) / 4 + 255) / 256)), dim3(256), 0,
                                     nvc_stream(stream), a));
      ctx->launches++;
      return NVC_OK;
    }
  }
  if (p->q_dtype == NVC_DT_F32 && p->kv_dtype == NVC_DT_F32) return launch_prep<float, float>(ctx, p, N, stream);
  if (p->q_dtype == NVC_DT_BF16 && p->kv_dtype == NVC_DT_BF16) return launch_prep<__nv_bfloat16, __nv_bfloat16>(ctx, p, N, stream);
  if (p->q_dtype == NVC_DT_BF16 && p->kv_dtype == NVC_DT_F32) return launch_prep<__nv_bfloat16, float>(ctx, p, N, stream);
  return launch_prep<float, __nv_bfloat16>(ctx, p, N, stream);
}

extern "C" int nvc_head_split_rot(nvc_ctx* ctx, const float* in, int ldi, int heads, int dim, int rot_dim, int rot_dims, int rot_half,
                                  const float* rot_table, const int32_t* positions, void* out_a, int ld_a, int hs_a, void* out_b, int ld_b,
                                  int hs_b, int off_b, int dtype, int N, void* stream) {
  NVC_REQUIRE(ctx, ctx && in && out_a && out_b, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && heads > 0 && dim > 0 && rot_dim >= 0 && ldi >= heads * (dim + rot_dim) && hs_a >= dim &&
                       ld_a >= (heads - 1) * hs_a + dim && off_b >= 0 && hs_b >= off_b + rot_dim && ld_b >= (heads - 1) * hs_b + off_b + rot_dim,
              NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim && (rot_dims == 0 || (rot_table && positions)), NVC_EINVAL,
              "bad rotary arguments");
  if (N == 0) return NVC_OK;
  const int64_t units = (int64_t)N * heads;
  NVC_DISPATCH_DT(dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, head_split_rot_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, nvc_stream(stream),
                                                 in, ldi, heads, dim, rot_dim, rot_dims, rot_half, rot_table, positions,
                                                 reinterpret_cast<T*>(out_a), ld_a, hs_a, reinterpret_cast<T*>(out_b), ld_b, hs_b, off_b, N)));
  ctx->launches++;
  return NVC_OK;
}

// (cos, sin) of position * base^(-2 i / dims) for every position below max_pos and i < dims / 2, angles in double precision.
// Synchronous (called once, when a model is built).
extern "C" int nvc_rotary_table_init_sync(nvc_ctx* ctx, float base, int dims, int max_pos, float* out) {
  NVC_REQUIRE(ctx, ctx && out && dims > 0 && dims % 2 == 0 && max_pos > 0 && base > 0.f, NVC_EINVAL, "bad arguments");
  const int half = dims / 2;
  std::string buf((size_t)max_pos * half * 2 * sizeof(float), '\0');
  float* h = reinterpret_cast<float*>(&buf[0]);
  for (int i = 0; i < half; ++i) {
    const double f = pow((double)base, -2.0 * (double)i / (double)dims);
    for (int p = 0; p < max_pos; ++p) {
      const double ang = (double)p * f;
      h[((size_t)p * half + i) * 2] = (float)cos(ang);
      h[((size_t)p * half + i) * 2 + 1] = (float)sin(ang);
    }
  }
  NVC_CUDA_CHECK(ctx, cudaMemcpy(out, h, buf.size(), cudaMemcpyHostToDevice));
  return NVC_OK;
}
