// Row operations of the models whose sublayer outputs enter the fp32 residual stream with constant factors, plain or through a
// weighted RMS norm of their own, and whose mixers norm their output in groups of columns:
//   nvc_rms_norm_blend     s = res + bias + c0 f(y0) + c1 f(y1), f = identity or a weighted RMS norm; res_out = s; out = norm(s) w
//                          (or s itself in the storage format): the residual sums of a layer, the merge of two mixers that run side
//                          by side and the norm in front of the next sublayer in ONE pass over the row; optional row gather
//   nvc_group_norm_gate    a mixer's output stage: RMS norm over equal groups of columns with a full-width weight and a sigmoid or
//                          silu gate in front of or behind the norm
// Both exist for bf16 and fp32 storage; arithmetic is fp32, every reduction has a fixed order.
#include "typed.cuh"

namespace {

// sum over the CTA; part: 33 floats of shared memory; every thread gets the result
__device__ __forceinline__ float cta_sum(float v, float* part) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) part[32] = t;
  }
  __syncthreads();
  const float t = part[32];
  __syncthreads();
  return t;
}

// four neighbouring numbers in the storage format with one store (p 16-byte aligned for fp32, 8-byte aligned for bf16)
__device__ __forceinline__ void st_f4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st_f4(__nv_bfloat16* p, const float4& v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float sq4(const float4& v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }

// one CTA per output row; the branch rows and the summed row stay in shared memory between the passes
// VEC: H, ld and ldo are multiples of 4 and every pointer is 16-byte aligned: four numbers per access
template <typename T, bool VEC>
__global__ void rms_norm_blend_kernel(const float* __restrict__ res_in, const float* __restrict__ bias, const float* __restrict__ y0,
                                      const float* __restrict__ w0, float c0, const float* __restrict__ y1, const float* __restrict__ w1,
                                      float c1, float* __restrict__ res_out, int ld, const float* __restrict__ w, T* __restrict__ out, int ldo,
                                      float eps, const int32_t* __restrict__ rows, int H) {
  extern __shared__ __align__(16) float sm[];          // [3][H]: y0, y1, s
  __shared__ float part[33];
  pdl_trigger();
  pdl_wait();
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r0 = sm;
  float* r1 = sm + H;
  float* rs = sm + 2 * H;
  float f0 = c0, f1 = c1;
  if (VEC) {
    const int H4 = H >> 2;
    float4* r0v = reinterpret_cast<float4*>(r0);
    float4* r1v = reinterpret_cast<float4*>(r1);
    float4* rsv = reinterpret_cast<float4*>(rs);
    if (y0) {
      float ss = 0.f;
      for (int j = threadIdx.x; j < H4; j += blockDim.x) {
        const float4 v = ld4(y0 + src * ld + 4 * j);
        r0v[j] = v;
        ss += sq4(v);
      }
      if (w0) f0 = c0 / sqrtf(cta_sum(ss, part) / (float)H + eps);
    }
    if (y1) {
      float ss = 0.f;
      for (int j = threadIdx.x; j < H4; j += blockDim.x) {
        const float4 v = ld4(y1 + src * ld + 4 * j);
        r1v[j] = v;
        ss += sq4(v);
      }
      if (w1) f1 = c1 / sqrtf(cta_sum(ss, part) / (float)H + eps);
    }
    float ss = 0.f;
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    for (int j = threadIdx.x; j < H4; j += blockDim.x) {
      const int64_t k = src * ld + 4 * j;
      float4 sv = res_in ? ld4(res_in + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (bias) { const float4 b = ld4(bias + 4 * j); sv.x += b.x; sv.y += b.y; sv.z += b.z; sv.w += b.w; }
      if (y0) {
        const float4 a = r0v[j], ww = w0 ? ld4(w0 + 4 * j) : one;
        sv.x += a.x * f0 * ww.x; sv.y += a.y * f0 * ww.y; sv.z += a.z * f0 * ww.z; sv.w += a.w * f0 * ww.w;
      }
      if (y1) {
        const float4 a = r1v[j], ww = w1 ? ld4(w1 + 4 * j) : one;
        sv.x += a.x * f1 * ww.x; sv.y += a.y * f1 * ww.y; sv.z += a.z * f1 * ww.z; sv.w += a.w * f1 * ww.w;
      }
      if (res_out) st_f4(res_out + k, sv);
      rsv[j] = sv;
      ss += sq4(sv);
    }
    if (!out) return;
    float r = 1.f;
    if (w) r = 1.0f / sqrtf(cta_sum(ss, part) / (float)H + eps);
    for (int j = threadIdx.x; j < H4; j += blockDim.x) {
      float4 sv = rsv[j];
      if (w) { const float4 ww = ld4(w + 4 * j); sv.x = sv.x * r * ww.x; sv.y = sv.y * r * ww.y; sv.z = sv.z * r * ww.z; sv.w = sv.w * r * ww.w; }
      st_f4(out + (int64_t)blockIdx.x * ldo + 4 * j, sv);
    }
    return;
  }
  if (y0) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      const float v = y0[src * ld + j];
      r0[j] = v;
      ss += v * v;
    }
    if (w0) f0 = c0 / sqrtf(cta_sum(ss, part) / (float)H + eps);
  }
  if (y1) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      const float v = y1[src * ld + j];
      r1[j] = v;
      ss += v * v;
    }
    if (w1) f1 = c1 / sqrtf(cta_sum(ss, part) / (float)H + eps);
  }
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const int64_t k = src * ld + j;
    float s = res_in ? res_in[k] : 0.f;
    if (bias) s += __ldg(bias + j);
    if (y0) s += r0[j] * f0 * (w0 ? __ldg(w0 + j) : 1.f);
    if (y1) s += r1[j] * f1 * (w1 ? __ldg(w1 + j) : 1.f);
    if (res_out) res_out[k] = s;
    rs[j] = s;
    ss += s * s;
  }
  if (!out) return;
  float r = 1.f;
  if (w) r = 1.0f / sqrtf(cta_sum(ss, part) / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) st_f(out + (int64_t)blockIdx.x * ldo + j, w ? rs[j] * r * __ldg(w + j) : rs[j]);
}

// one CTA per (row, group).  VEC: gsize and the three row strides are multiples of 4 and every pointer is 16-byte aligned (out: 8 bytes in
// bf16): four numbers per access
template <typename T, bool VEC>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg,
                                       const float* __restrict__ weight, T* __restrict__ out, int ldout, int gsize, int gate_first, float eps,
                                       int act) {
  extern __shared__ __align__(16) float sm[];          // [gsize]
  __shared__ float part[33];
  pdl_trigger();
  pdl_wait();
  const int64_t n = blockIdx.x;
  const int c0 = blockIdx.y * gsize;
  if (VEC) {
    const int g4 = gsize >> 2;
    float4* smv = reinterpret_cast<float4*>(sm);
    auto gated = [&](float4 v, const float4& z) {
      if (act == NVC_GATE_SILU) { v.x *= z.x * sigmoid_f32(z.x); v.y *= z.y * sigmoid_f32(z.y); v.z *= z.z * sigmoid_f32(z.z); v.w *= z.w * sigmoid_f32(z.w); }
      else { v.x *= sigmoid_f32(z.x); v.y *= sigmoid_f32(z.y); v.z *= sigmoid_f32(z.z); v.w *= sigmoid_f32(z.w); }
      return v;
    };
    float ss = 0.f;
    for (int j = threadIdx.x; j < g4; j += blockDim.x) {
      float4 v = ld4(o + n * ldo + c0 + 4 * j);
      if (gate && gate_first) v = gated(v, ld4(gate + n * ldg + c0 + 4 * j));
      smv[j] = v;
      ss += sq4(v);
    }
    const float r = 1.0f / sqrtf(cta_sum(ss, part) / (float)gsize + eps);
    for (int j = threadIdx.x; j < g4; j += blockDim.x) {
      float4 y = smv[j];
      const float4 ww = weight ? ld4(weight + c0 + 4 * j) : make_float4(1.f, 1.f, 1.f, 1.f);
      y.x = y.x * r * ww.x; y.y = y.y * r * ww.y; y.z = y.z * r * ww.z; y.w = y.w * r * ww.w;
      if (gate && !gate_first) y = gated(y, ld4(gate + n * ldg + c0 + 4 * j));
      st_f4(out + n * ldout + c0 + 4 * j, y);
    }
    return;
  }
  float ss = 0.f;
  for (int j = threadIdx.x; j < gsize; j += blockDim.x) {
    float v = o[n * ldo + c0 + j];
    if (gate && gate_first) {
      const float z = gate[n * ldg + c0 + j];
      v *= act == NVC_GATE_SILU ? z * sigmoid_f32(z) : sigmoid_f32(z);
    }
    sm[j] = v;
    ss += v * v;
  }
  const float r = 1.0f / sqrtf(cta_sum(ss, part) / (float)gsize + eps);
  for (int j = threadIdx.x; j < gsize; j += blockDim.x) {
    float y = sm[j] * r * (weight ? __ldg(weight + c0 + j) : 1.f);
    if (gate && !gate_first) {
      const float z = gate[n * ldg + c0 + j];
      y *= act == NVC_GATE_SILU ? z * sigmoid_f32(z) : sigmoid_f32(z);
    }
    st_f(out + n * ldout + c0 + j, y);
  }
}

}  // namespace

extern "C" {

int nvc_rms_norm_blend(nvc_ctx* ctx, const float* res_in, const float* bias, const float* y0, const float* w0, float c0, const float* y1,
                       const float* w1, float c1, float* res_out, int ld, const float* w, void* out, int out_dtype, int ldo, float eps,
                       const int32_t* rows, int N, int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && (res_in || y0), NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, (y0 || !w0) && (y1 || !w1) && (out || !w), NVC_EINVAL, "a weight without its input or output");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && H <= 16384 && ld >= H && (!out || ldo >= H), NVC_EINVAL, "bad sizes (rows of up to 16 384 numbers)");
  NVC_REQUIRE(ctx, !(rows && res_out), NVC_EINVAL, "a gathering call does not write the residual back");
  if (N == 0) return NVC_OK;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = (size_t)3 * H * sizeof(float);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (H & 3) == 0 && (ld & 3) == 0 && (!out || ((ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0 &&
                                                              (out_dtype != NVC_DT_F32 || al16(out)))) &&
                   al16(res_in) && al16(bias) && al16(y0) && al16(w0) && al16(y1) && al16(w1) && al16(res_out) && al16(w);
  NVC_DISPATCH_DT(out_dtype, T, {
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
      NVC_CUDA_CHECK(ctx, cudaFuncSetAttribute(rms_norm_blend_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384 * 4));
      NVC_CUDA_CHECK(ctx, cudaFuncSetAttribute(rms_norm_blend_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384 * 4));
      attr_set = true;
    }
    if (vec) {
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, rms_norm_blend_kernel<T, true>, dim3(N), dim3(threads), smem, nvc_stream(stream), res_in, bias, y0, w0, c0, y1,
                                     w1, c1, res_out, ld, w, reinterpret_cast<T*>(out), ldo, eps, rows, H));
    } else {
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, rms_norm_blend_kernel<T, false>, dim3(N), dim3(threads), smem, nvc_stream(stream), res_in, bias, y0, w0, c0, y1,
                                     w1, c1, res_out, ld, w, reinterpret_cast<T*>(out), ldo, eps, rows, H));
    }
  });
  ctx->launches++;
  return NVC_OK;
}

int nvc_group_norm_gate(nvc_ctx* ctx, const float* o, int ldo, const float* gate, int ldg, const float* weight, void* out, int ldout,
                        int out_dtype, int groups, int gsize, int gate_first, float eps, int act, int N, void* stream) {
  NVC_REQUIRE(ctx, ctx && o && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && groups > 0 && groups <= 65535 && gsize > 0 && gsize <= 12288 && ldo >= groups * gsize && ldout >= groups * gsize &&
                       (!gate || ldg >= groups * gsize),
              NVC_EINVAL, "bad sizes (groups of up to 12 288 numbers)");
  NVC_REQUIRE(ctx, act == NVC_GATE_SIGMOID || act == NVC_GATE_SILU, NVC_EINVAL, "unknown gate");
  if (N == 0) return NVC_OK;
  const int threads = gsize >= 2048 ? 512 : (gsize >= 512 ? 256 : 128);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (gsize & 3) == 0 && (ldo & 3) == 0 && (ldout & 3) == 0 && (!gate || ((ldg & 3) == 0 && al16(gate))) && al16(o) && al16(weight) &&
                   (reinterpret_cast<uintptr_t>(out) & (out_dtype == NVC_DT_F32 ? 15 : 7)) == 0;
  NVC_DISPATCH_DT(out_dtype, T, {
    if (vec) {
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, group_norm_gate_kernel<T, true>, dim3(N, groups), dim3(threads), (size_t)gsize * sizeof(float),
                                     nvc_stream(stream), o, ldo, gate, ldg, weight, reinterpret_cast<T*>(out), ldout, gsize, gate_first, eps, act));
    } else {
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, group_norm_gate_kernel<T, false>, dim3(N, groups), dim3(threads), (size_t)gsize * sizeof(float),
                                     nvc_stream(stream), o, ldo, gate, ldg, weight, reinterpret_cast<T*>(out), ldout, gsize, gate_first, eps, act));
    }
  });
  ctx->launches++;
  return NVC_OK;
}

}  // extern "C"
