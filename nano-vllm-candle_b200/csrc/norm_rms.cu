// Row operations of the models whose fp32 residual stream goes through RMS norms:
//   nvc_embed_gather_scaled_f32   token rows of the embedding table as fp32, times a constant
//   nvc_rms_norm_pair             the residual accumulation fused with up to two RMS norms of the same sum (a parallel layer
//                                 whose mixer and feed-forward have a norm each), optional row gather for the head
//   nvc_rms_norm_sandwich         the norm behind a sublayer, the residual sum and the norm in front of the next sublayer in one pass
//   nvc_head_gate                 per-head output stage of a mixer: optional division by the head's root mean square, times a
//                                 sigmoid or silu gate, times a constant
// Every kernel exists for bf16 and fp32 storage; arithmetic is fp32.
#include "typed.cuh"

namespace {

template <typename T>
__global__ void embed_gather_scaled_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table, int ldt, float scale,
                                           float* __restrict__ out, int ldo, int N, int H) {
  pdl_trigger();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)N * H) return;
  const int n = (int)(i / H), j = (int)(i % H);
  out[(int64_t)n * ldo + j] = ld_f(table + (int64_t)ids[n] * ldt + j) * scale;
}

// one CTA per output row; the summed row stays in shared memory between the two passes
template <typename T>
__global__ void rms_norm_pair_kernel(const float* __restrict__ res_in, const float* __restrict__ a0, const float* __restrict__ a1,
                                     float* __restrict__ res_out, int ld, const float* __restrict__ w0, T* __restrict__ out0,
                                     const float* __restrict__ w1, T* __restrict__ out1, int ldo, float eps,
                                     const int32_t* __restrict__ rows, int H) {
  extern __shared__ float row[];
  __shared__ float part[32];
  pdl_trigger();
  pdl_wait();
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const int64_t k = src * ld + j;
    float s = res_in ? res_in[k] : 0.f;
    if (a0) s += a0[k];
    if (a1) s += a1[k];
    if (res_out) res_out[k] = s;
    row[j] = s;
    ss += s * s;
  }
  if (!w0) return;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) part[0] = 1.0f / sqrtf(t / (float)H + eps);
  }
  __syncthreads();
  const float r = part[0];
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float y = row[j] * r;
    st_f(out0 + (int64_t)blockIdx.x * ldo + j, y * __ldg(w0 + j));
    if (w1) st_f(out1 + (int64_t)blockIdx.x * ldo + j, y * __ldg(w1 + j));
  }
}


// one CTA per output row: y is normed and added to the residual row, the sum is normed again; the row stays in shared memory
template <typename T>
__global__ void rms_norm_sandwich_kernel(const float* __restrict__ res_in, const float* __restrict__ y, const float* __restrict__ wy,
                                         float* __restrict__ res_out, int ld, const float* __restrict__ w, T* __restrict__ out, int ldo,
                                         float eps, float woff, const int32_t* __restrict__ rows, int H) {
  extern __shared__ float row[];
  __shared__ float part[33];
  pdl_trigger();
  pdl_wait();
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  const int warps = blockDim.x >> 5;
  float ry = 0.f;
  if (y) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      const float v = y[src * ld + j];
      row[j] = v;
      ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < warps ? part[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) part[32] = 1.0f / sqrtf(t / (float)H + eps);
    }
    __syncthreads();
    ry = part[32];
  }
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const int64_t k = src * ld + j;
    float s = res_in[k];
    if (y) s += row[j] * ry * (__ldg(wy + j) + woff);
    if (res_out) res_out[k] = s;
    row[j] = s;
    ss += s * s;
  }
  if (!w) return;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < warps ? part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) part[32] = 1.0f / sqrtf(t / (float)H + eps);
  }
  __syncthreads();
  const float r = part[32];
  for (int j = threadIdx.x; j < H; j += blockDim.x) st_f(out + (int64_t)blockIdx.x * ldo + j, row[j] * r * (__ldg(w + j) + woff));
}

// one warp per (row, head)
template <typename T>
__global__ void head_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ g, int ldg,
                                 const float* __restrict__ wgt, T* __restrict__ out, int ldout, int heads, int vdim, int norm, float eps, int act, float out_scale, int N) {
  pdl_trigger();
  pdl_wait();
  const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (u >= (int64_t)N * heads) return;
  const int n = (int)(u / heads), h = (int)(u % heads);
  const float* x = o + (int64_t)n * ldo + (int64_t)h * vdim;
  float r = 1.f;
  if (norm) {
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss += x[j] * x[j];
    ss = warp_sum(ss);
    r = 1.0f / sqrtf(ss / (float)vdim + eps);
  }
  for (int j = lane; j < vdim; j += 32) {
    float y = x[j] * r;
    if (wgt) y *= __ldg(wgt + j);
    if (g) {
      const float z = g[(int64_t)n * ldg + (int64_t)h * vdim + j];
      y *= act == NVC_GATE_SILU ? z * sigmoid_f32(z) : sigmoid_f32(z);
    }
    st_f(out + (int64_t)n * ldout + (int64_t)h * vdim + j, y * out_scale);
  }
}

}  // namespace

extern "C" {

int nvc_embed_gather_scaled_f32(nvc_ctx* ctx, const int32_t* ids, const void* table, int table_dtype, int ldt, float scale, float* out,
                                int ldo, int N, int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && ids && table && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && ldt >= H && ldo >= H, NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  const int64_t total = (int64_t)N * H;
  NVC_DISPATCH_DT(table_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, embed_gather_scaled_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                                 nvc_stream(stream), ids, reinterpret_cast<const T*>(table), ldt, scale, out, ldo, N, H)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_rms_norm_pair(nvc_ctx* ctx, const float* res_in, const float* a0, const float* a1, float* res_out, int ld, const float* w0,
                      void* out0, const float* w1, void* out1, int out_dtype, int ldo, float eps, const int32_t* rows, int N, int H,
                      void* stream) {
  NVC_REQUIRE(ctx, ctx && (res_in || a0), NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, (w0 == nullptr) == (out0 == nullptr) && (w1 == nullptr) == (out1 == nullptr) && (w0 || !w1), NVC_EINVAL,
              "every norm needs its weight and its output; the second norm needs the first");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && H <= 12288 && ld >= H && (!w0 || ldo >= H), NVC_EINVAL, "bad sizes (rows of up to 12 288 numbers)");
  NVC_REQUIRE(ctx, !(rows && res_out), NVC_EINVAL, "a gathering call does not write the residual back");
  if (N == 0) return NVC_OK;
  const int threads = H >= 1024 ? 512 : (H >= 256 ? 256 : 128);
  NVC_DISPATCH_DT(out_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, rms_norm_pair_kernel<T>, dim3(N), dim3(threads), (size_t)H * sizeof(float),
                                                 nvc_stream(stream), res_in, a0, a1, res_out, ld, w0, reinterpret_cast<T*>(out0), w1,
                                                 reinterpret_cast<T*>(out1), ldo, eps, rows, H)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_rms_norm_sandwich(nvc_ctx* ctx, const float* res_in, const float* y, const float* wy, float* res_out, int ld, const float* w,
                          void* out, int out_dtype, int ldo, float eps, float weight_offset, const int32_t* rows, int N, int H,
                          void* stream) {
  NVC_REQUIRE(ctx, ctx && res_in, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, (y == nullptr) == (wy == nullptr) && (w == nullptr) == (out == nullptr), NVC_EINVAL,
              "every norm needs its weight and its input or output");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && H <= 12288 && ld >= H && (!w || ldo >= H), NVC_EINVAL, "bad sizes (rows of up to 12 288 numbers)");
  NVC_REQUIRE(ctx, !(rows && res_out), NVC_EINVAL, "a gathering call does not write the residual back");
  if (N == 0) return NVC_OK;
  const int threads = H >= 1024 ? 512 : (H >= 256 ? 256 : 128);
  NVC_DISPATCH_DT(out_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, rms_norm_sandwich_kernel<T>, dim3(N), dim3(threads), (size_t)H * sizeof(float),
                                                 nvc_stream(stream), res_in, y, wy, res_out, ld, w, reinterpret_cast<T*>(out), ldo, eps,
                                                 weight_offset, rows, H)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_head_gate(nvc_ctx* ctx, const float* o, int ldo, const float* gate, int ldg, void* out, int ldout, int out_dtype, int heads,
                  int vdim, int norm, float eps, int act, float out_scale, int N, void* stream) {
  return nvc_head_gate_w(ctx, o, ldo, gate, ldg, nullptr, out, ldout, out_dtype, heads, vdim, norm, eps, act, out_scale, N, stream);
}

int nvc_head_gate_w(nvc_ctx* ctx, const float* o, int ldo, const float* gate, int ldg, const float* weight, void* out, int ldout,
                    int out_dtype, int heads, int vdim, int norm, float eps, int act, float out_scale, int N, void* stream) {
  NVC_REQUIRE(ctx, ctx && o && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && heads > 0 && vdim > 0 && ldo >= heads * vdim && ldout >= heads * vdim && (!gate || ldg >= heads * vdim),
              NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, act == NVC_GATE_SIGMOID || act == NVC_GATE_SILU, NVC_EINVAL, "unknown gate");
  if (N == 0) return NVC_OK;
  const int64_t units = (int64_t)N * heads;
  NVC_DISPATCH_DT(out_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, head_gate_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0,
                                                 nvc_stream(stream), o, ldo, gate, ldg, weight, reinterpret_cast<T*>(out), ldout, heads, vdim, norm,
                                                 eps, act, out_scale, N)));
  ctx->launches++;
  return NVC_OK;
}

}  // extern "C"
