// Norms and row operations of the models whose residual stream and norms are fp32 end to end:
//   nvc_embed_gather_f32    token rows of the embedding table as fp32
//   nvc_dyt_norm            Dynamic Tanh norm (no mean, no variance) fused with the residual accumulation
//   nvc_latent_norm_store   plain-weight RMS norms of the two low-rank latents of latent attention, the key / value
//                           latent scattered into the paged cache in the same pass
//   nvc_act_mul             gated / plain feed-forward activations (tanh-gelu gate, squared relu)
// Every kernel exists for bf16 and fp32 storage; arithmetic is fp32.
#include "typed.cuh"

namespace {

template <typename T>
__global__ void embed_gather_f32_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table, int ldt,
                                        float* __restrict__ out, int ldo, int N, int H) {
  pdl_trigger();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)N * H) return;
  const int n = (int)(i / H), j = (int)(i % H);
  out[(int64_t)n * ldo + j] = ld_f(table + (int64_t)ids[n] * ldt + j);
}

// one CTA per output row
template <typename T>
__global__ void dyt_norm_kernel(const float* __restrict__ res_in, const float* __restrict__ a0, const float* __restrict__ a1,
                                const float* __restrict__ a2, float* __restrict__ res_out, int ld, const float* __restrict__ w,
                                const float* __restrict__ b, const float* __restrict__ alpha, T* __restrict__ out, int ldo,
                                const int32_t* __restrict__ rows, int H) {
  pdl_trigger();
  const float al = w ? __ldg(alpha) : 0.f;
  pdl_wait();
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const int64_t k = src * ld + j;
    float s = res_in ? res_in[k] : 0.f;
    if (a0) s += a0[k];
    if (a1) s += a1[k];
    if (a2) s += a2[k];
    if (res_out) res_out[k] = s;
    if (w) st_f(out + (int64_t)blockIdx.x * ldo + j, tanh_f32(al * s) * __ldg(w + j) + __ldg(b + j));
  }
}

// one warp per row: segment 0 = columns [0, n0) -> out0; segment 1 = columns [off1, off1 + n1) -> the cache row of the slot
template <typename T>
__global__ void latent_norm_store_kernel(const float* __restrict__ in, int ldi, int n0, int off1, int n1,
                                         const float* __restrict__ w0, const float* __restrict__ w1, float eps,
                                         T* __restrict__ out0, int ld0, T* __restrict__ cache, int ldc,
                                         const int32_t* __restrict__ slots, int rot_dim, int rot_dims, int rot_half,
                                         const float* __restrict__ rot_table, const int32_t* __restrict__ positions, int N) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= N) return;
  const float* x = in + (int64_t)row * ldi;
  float ss = 0.f;
  for (int j = lane; j < n0; j += 32) ss += x[j] * x[j];
  ss = warp_sum(ss);
  float r = 1.0f / sqrtf(ss / (float)n0 + eps);
  for (int j = lane; j < n0; j += 32) st_f(out0 + (int64_t)row * ld0 + j, x[j] * r * __ldg(w0 + j));
  const int slot = slots ? slots[row] : -1;
  if (slot < 0 || !cache) return;
  ss = 0.f;
  for (int j = lane; j < n1; j += 32) ss += x[off1 + j] * x[off1 + j];
  ss = warp_sum(ss);
  r = 1.0f / sqrtf(ss / (float)n1 + eps);
  for (int j = lane; j < n1; j += 32) st_f(cache + (int64_t)slot * ldc + j, x[off1 + j] * r * __ldg(w1 + j));
  // the key part that all heads share, behind the latent: turned by the token's position, not normed
  const float* kr = x + off1 + n1;
  const int half = rot_dims >> 1;
  const float2* tab = reinterpret_cast<const float2*>(rot_table) + (int64_t)(rot_dims ? positions[row] : 0) * half;
  for (int j = lane; j < rot_dim; j += 32) {
    float y = kr[j];
    if (j < rot_dims) {
      int i, partner;
      float sign;
      if (rot_half) { i = j < half ? j : j - half; partner = j < half ? j + half : j - half; sign = j < half ? -1.f : 1.f; }
      else { i = j >> 1; partner = j ^ 1; sign = (j & 1) ? 1.f : -1.f; }
      const float2 cs = __ldg(tab + i);
      y = y * cs.x + sign * kr[partner] * cs.y;
    }
    st_f(cache + (int64_t)slot * ldc + n1 + j, y);
  }
}

// NVC_ACT_GELU_TANH_MUL: out[n, j] = gelu_tanh(in[n, j]) * in[n, Fp + j];  NVC_ACT_RELU2: out[n, j] = relu(in[n, j])^2;
// NVC_ACT_SILU_MUL: silu(in[n, j]) * in[n, Fp + j];  NVC_ACT_GELU_TANH: gelu_tanh(in[n, j]);  NVC_ACT_GLU_CLAMP: g sigmoid(p1 g) (u + 1), g = min(in[n, j], p0), u = clamp(in[n, Fp + j], +-p0)
__device__ __forceinline__ float act_unit(int kind, float g, float u, float p0, float p1) {
  if (kind == NVC_ACT_GELU_TANH_MUL) return gelu_tanh_f32(g) * u;
  if (kind == NVC_ACT_GELU_TANH) return gelu_tanh_f32(g);
  if (kind == NVC_ACT_SILU_MUL) return g * sigmoid_f32(g) * u;
  if (kind == NVC_ACT_GLU_CLAMP) {
    const float gc = fminf(g, p0);
    return gc * sigmoid_f32(p1 * gc) * (fminf(fmaxf(u, -p0), p0) + 1.0f);
  }
  const float t = fmaxf(g, 0.f);
  return t * t;
}

// rows_per_cta rows per CTA, the threads walk along a row: no division per element.  V: numbers per access (8 when every
// row start is 16-byte aligned in both buffers and F, Fp are multiples of 8; else 1)
template <typename T, int V>
__global__ void act_mul_kernel(const T* __restrict__ in, int ldi, T* __restrict__ out, int ldo, int N, int F, int Fp, int kind, float p0,
                               float p1, int rows_per_cta) {
  pdl_trigger();
  pdl_wait();
  const bool two = kind == NVC_ACT_GELU_TANH_MUL || kind == NVC_ACT_GLU_CLAMP || kind == NVC_ACT_SILU_MUL;
  for (int rr = 0; rr < rows_per_cta; ++rr) {
    const int64_t n = (int64_t)blockIdx.x * rows_per_cta + rr;
    if (n >= N) return;
    const T* x = in + n * ldi;
    T* y = out + n * ldo;
    if constexpr (V == 1) {
      for (int j = threadIdx.x; j < F; j += blockDim.x) st_f(y + j, act_unit(kind, ld_f(x + j), two ? ld_f(x + Fp + j) : 0.f, p0, p1));
    } else {
      constexpr int PER = 16 / sizeof(T);          // numbers per 16-byte access
      for (int j = threadIdx.x * PER; j < F; j += blockDim.x * PER) {
        __align__(16) T g[PER];
        __align__(16) T u[PER];
        __align__(16) T o[PER];
        *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(x + j);
        if (two) *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(x + Fp + j);
#pragma unroll
        for (int k = 0; k < PER; ++k) st_f(o + k, act_unit(kind, ld_f(g + k), two ? ld_f(u + k) : 0.f, p0, p1));
        *reinterpret_cast<uint4*>(y + j) = *reinterpret_cast<const uint4*>(o);
      }
    }
  }
}

}  // namespace

extern "C" {

int nvc_embed_gather_f32(nvc_ctx* ctx, const int32_t* ids, const void* table, int table_dtype, int ldt, float* out, int ldo,
                         int N, int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && ids && table && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && ldt >= H && ldo >= H, NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  const int64_t total = (int64_t)N * H;
  NVC_DISPATCH_DT(table_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, embed_gather_f32_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                                 nvc_stream(stream), ids, reinterpret_cast<const T*>(table), ldt, out, ldo, N, H)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_dyt_norm(nvc_ctx* ctx, const float* res_in, const float* a0, const float* a1, const float* a2, float* res_out, int ld,
                 const float* w, const float* b, const float* alpha, void* out, int out_dtype, int ldo, const int32_t* rows,
                 int N, int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && (res_in || a0), NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, (w == nullptr) == (out == nullptr) && (!w || (b && alpha)), NVC_EINVAL, "norm needs weight, bias, alpha and an output");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && ld >= H && (!w || ldo >= H), NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, !(rows && res_out), NVC_EINVAL, "a gathering call does not write the residual back");
  if (N == 0) return NVC_OK;
  const int threads = H >= 1024 ? 512 : (H >= 256 ? 256 : 128);
  NVC_DISPATCH_DT(out_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, dyt_norm_kernel<T>, dim3(N), dim3(threads), 0, nvc_stream(stream), res_in, a0, a1, a2,
                                                 res_out, ld, w, b, alpha, reinterpret_cast<T*>(out), ldo, rows, H)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_latent_norm_store(nvc_ctx* ctx, const float* in, int ldi, int n0, int off1, int n1, const float* w0, const float* w1,
                          float eps, void* out0, int ld0, void* cache, int ldc, const int32_t* slot_mapping, int dtype, int N,
                          void* stream) {
  return nvc_latent_norm_store_rot(ctx, in, ldi, n0, off1, n1, w0, w1, eps, out0, ld0, cache, ldc, slot_mapping, 0, 0, 0, nullptr, nullptr,
                                   dtype, N, stream);
}

int nvc_latent_norm_store_rot(nvc_ctx* ctx, const float* in, int ldi, int n0, int off1, int n1, const float* w0, const float* w1,
                              float eps, void* out0, int ld0, void* cache, int ldc, const int32_t* slot_mapping, int rot_dim,
                              int rot_dims, int rot_half, const float* rot_table, const int32_t* positions, int dtype, int N,
                              void* stream) {
  NVC_REQUIRE(ctx, ctx && in && w0 && out0, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, rot_dim >= 0 && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim && (rot_dims == 0 || (rot_table && positions)),
              NVC_EINVAL, "bad rotary arguments");
  if (!cache) rot_dim = rot_dims = 0;
  NVC_REQUIRE(ctx, !cache || (w1 && slot_mapping), NVC_EINVAL, "a cache needs its norm weight and the slot mapping");
  NVC_REQUIRE(ctx, N >= 0 && n0 > 0 && n1 >= 0 && off1 >= n0 && ldi >= off1 + n1 + rot_dim && ld0 >= n0 && (!cache || ldc >= n1 + rot_dim),
              NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  NVC_DISPATCH_DT(dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, latent_norm_store_kernel<T>, dim3((N + 3) / 4), dim3(128), 0, nvc_stream(stream), in,
                                                 ldi, n0, off1, n1, w0, w1, eps, reinterpret_cast<T*>(out0), ld0,
                                                 reinterpret_cast<T*>(cache), ldc, slot_mapping, rot_dim, rot_dims, rot_half, rot_table,
                                                 positions, N)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_act_mul(nvc_ctx* ctx, const void* in, int ldi, void* out, int ldo, int dtype, int N, int F, int Fp, int kind, void* stream) {
  NVC_REQUIRE(ctx, kind == NVC_ACT_GELU_TANH_MUL || kind == NVC_ACT_RELU2, NVC_EINVAL, "bad arguments");
  return nvc_act_mul_p(ctx, in, ldi, out, ldo, dtype, N, F, Fp, kind, 0.f, 0.f, stream);
}

int nvc_act_mul_p(nvc_ctx* ctx, const void* in, int ldi, void* out, int ldo, int dtype, int N, int F, int Fp, int kind, float p0, float p1,
                  void* stream) {
  NVC_REQUIRE(ctx, ctx && in && out, NVC_EINVAL, "null pointer");
  const bool two = kind == NVC_ACT_GELU_TANH_MUL || kind == NVC_ACT_GLU_CLAMP || kind == NVC_ACT_SILU_MUL;
  NVC_REQUIRE(ctx, N >= 0 && F > 0 && (two || kind == NVC_ACT_RELU2 || kind == NVC_ACT_GELU_TANH), NVC_EINVAL, "bad arguments");
  NVC_REQUIRE(ctx, ldo >= F && ldi >= (two ? Fp + F : F), NVC_EINVAL, "bad strides");
  if (N == 0) return NVC_OK;
  const int per = dtype == NVC_DT_F32 ? 4 : 8;
  const bool vec = F % per == 0 && Fp % per == 0 && ldi % per == 0 && ldo % per == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const int lanes = vec ? F / per : F;                       // accesses per row
  const int threads = lanes >= 256 ? 256 : (lanes >= 128 ? 128 : 64);
  const int rows_per_cta = lanes >= 64 ? 1 : (64 / (lanes > 0 ? lanes : 1));
  const unsigned grid = (unsigned)((N + rows_per_cta - 1) / rows_per_cta);
  NVC_DISPATCH_DT(dtype, T, {
    auto k1 = act_mul_kernel<T, 1>;
    auto k8 = act_mul_kernel<T, 8>;
    NVC_CUDA_CHECK(ctx, nvc_launch(ctx, vec ? k8 : k1, dim3(grid), dim3(threads), 0, nvc_stream(stream), reinterpret_cast<const T*>(in), ldi,
                                   reinterpret_cast<T*>(out), ldo, N, F, Fp, kind, p0, p1, rows_per_cta));
  });
  ctx->launches++;
  return NVC_OK;
}

}  // extern "C"
