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

// the same with rows of 4 V numbers per thread kept in registers and 16-byte accesses (H a multiple of 4, H <= 4 V blockDim.x)
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float4& v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float block_sum(float v, float* part) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) part[32] = t;
  }
  __syncthreads();
  t = part[32];
  __syncthreads();
  return t;
}

template <typename T, int V>
__global__ void rms_norm_sandwich_vec_kernel(const float* __restrict__ res_in, const float* __restrict__ y, const float* __restrict__ wy,
                                             float* __restrict__ res_out, int ld, const float* __restrict__ w, T* __restrict__ out, int ldo,
                                             float eps, float woff, const int32_t* __restrict__ rows, int H) {
  __shared__ float part[33];
  pdl_trigger();
  pdl_wait();
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  const int H4 = H >> 2;
  float4 s[V];
  float4 yy[V];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int j = threadIdx.x + k * blockDim.x;
    s[k] = j < H4 ? *reinterpret_cast<const float4*>(res_in + src * ld + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (y) {
      yy[k] = j < H4 ? *reinterpret_cast<const float4*>(y + src * ld + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss += yy[k].x * yy[k].x + yy[k].y * yy[k].y + yy[k].z * yy[k].z + yy[k].w * yy[k].w;
    }
  }
  if (y) {
    const float ry = 1.0f / sqrtf(block_sum(ss, part) / (float)H + eps);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int j = threadIdx.x + k * blockDim.x;
      if (j < H4) {
        const float4 g = *reinterpret_cast<const float4*>(wy + 4 * j);
        s[k].x += yy[k].x * ry * (g.x + woff);
        s[k].y += yy[k].y * ry * (g.y + woff);
        s[k].z += yy[k].z * ry * (g.z + woff);
        s[k].w += yy[k].w * ry * (g.w + woff);
      }
    }
  }
  ss = 0.f;
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int j = threadIdx.x + k * blockDim.x;
    if (j < H4) {
      if (res_out) *reinterpret_cast<float4*>(res_out + src * ld + 4 * j) = s[k];
      ss += s[k].x * s[k].x + s[k].y * s[k].y + s[k].z * s[k].z + s[k].w * s[k].w;
    }
  }
  if (!w) return;
  const float r = 1.0f / sqrtf(block_sum(ss, part) / (float)H + eps);
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int j = threadIdx.x + k * blockDim.x;
    if (j < H4) {
      const float4 g = *reinterpret_cast<const float4*>(w + 4 * j);
      st4(out + (int64_t)blockIdx.x * ldo + 4 * j,
          make_float4(s[k].x * r * (g.x + woff), s[k].y * r * (g.y + woff), s[k].z * r * (g.z + woff), s[k].w * r * (g.w + woff)));
    }
  }
}

// one warp per (row, head); vec: vdim and every stride are multiples of 4 and the pointers 16-byte aligned (16-byte accesses)
template <typename T>
__global__ void head_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ g, int ldg,
                                 const float* __restrict__ wgt, T* __restrict__ out, int ldout, int heads, int vdim, int norm, float eps, int act,
                                 float out_scale, int N, int vec) {
  pdl_trigger();
  pdl_wait();
  const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (u >= (int64_t)N * heads) return;
  const int n = (int)(u / heads), h = (int)(u % heads);
  const float* x = o + (int64_t)n * ldo + (int64_t)h * vdim;
  const float* z = g ? g + (int64_t)n * ldg + (int64_t)h * vdim : nullptr;
  T* dst = out + (int64_t)n * ldout + (int64_t)h * vdim;
  if (vec) {
    const int v4 = vdim >> 2;
    float r = 1.f;
    if (norm) {
      float ss = 0.f;
      for (int j = lane; j < v4; j += 32) {
        const float4 a = *reinterpret_cast<const float4*>(x + 4 * j);
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      }
      ss = warp_sum(ss);
      r = 1.0f / sqrtf(ss / (float)vdim + eps);
    }
    r *= out_scale;
    for (int j = lane; j < v4; j += 32) {
      float4 a = *reinterpret_cast<const float4*>(x + 4 * j);
      a.x *= r; a.y *= r; a.z *= r; a.w *= r;
      if (wgt) {
        const float4 c = *reinterpret_cast<const float4*>(wgt + 4 * j);
        a.x *= c.x; a.y *= c.y; a.z *= c.z; a.w *= c.w;
      }
      if (z) {
        const float4 c = *reinterpret_cast<const float4*>(z + 4 * j);
        if (act == NVC_GATE_SILU) { a.x *= c.x * sigmoid_f32(c.x); a.y *= c.y * sigmoid_f32(c.y); a.z *= c.z * sigmoid_f32(c.z); a.w *= c.w * sigmoid_f32(c.w); }
        else { a.x *= sigmoid_f32(c.x); a.y *= sigmoid_f32(c.y); a.z *= sigmoid_f32(c.z); a.w *= sigmoid_f32(c.w); }
      }
      st4(dst + 4 * j, a);
    }
    return;
  }
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
    if (z) y *= act == NVC_GATE_SILU ? z[j] * sigmoid_f32(z[j]) : sigmoid_f32(z[j]);
    st_f(dst + j, y * out_scale);
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
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (H % 4 == 0 && ld % 4 == 0 && (!w || ldo % 4 == 0) && H <= 8192 && al16(res_in) && al16(y) && al16(wy) && al16(res_out) && al16(w) && al16(out)) {
    // rows in registers, 16-byte accesses: one float4 per thread up to 1024 numbers, two up to 4096 (256 and 512 threads), then four
    const int H4 = H / 4;
    const int threads = H4 <= 64 ? 64 : (H4 <= 128 ? 128 : (H4 <= 256 ? 256 : 512));
    const int V = (H4 + threads - 1) / threads;
    NVC_DISPATCH_DT(out_dtype, T, {
      auto k1 = rms_norm_sandwich_vec_kernel<T, 1>;
      auto k2 = rms_norm_sandwich_vec_kernel<T, 2>;
      auto k4 = rms_norm_sandwich_vec_kernel<T, 4>;
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, V <= 1 ? k1 : (V <= 2 ? k2 : k4), dim3(N), dim3(threads), 0, nvc_stream(stream), res_in, y, wy, res_out, ld, w,
                                     reinterpret_cast<T*>(out), ldo, eps, weight_offset, rows, H));
    });
    ctx->launches++;
    return NVC_OK;
  }
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
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const int vec = vdim % 4 == 0 && ldo % 4 == 0 && ldout % 4 == 0 && (!gate || ldg % 4 == 0) && al16(o) && al16(gate) && al16(weight) && al16(out);
  NVC_DISPATCH_DT(out_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, head_gate_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0,
                                                 nvc_stream(stream), o, ldo, gate, ldg, weight, reinterpret_cast<T*>(out), ldout, heads, vdim, norm,
                                                 eps, act, out_scale, N, vec)));
  ctx->launches++;
  return NVC_OK;
}

}  // extern "C"
