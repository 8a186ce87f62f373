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

// one CTA per output row; the branch rows and the summed row stay in shared memory between the passes
template <typename T>
__global__ void rms_norm_blend_kernel(const float* __restrict__ res_in, const float* __restrict__ bias, const float* __restrict__ y0,
                                      const float* __restrict__ w0, float c0, const float* __restrict__ y1, const float* __restrict__ w1,
                                      float c1, float* __restrict__ res_out, int ld, const float* __restrict__ w, T* __restrict__ out, int ldo,
                                      float eps, const int32_t* __restrict__ rows, int H) {
  extern __shared__ float sm[];          // [3][H]: y0, y1, s
  __shared__ float part[33];
  pdl_trigger();
  pdl_wait();
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r0 = sm;
  float* r1 = sm + H;
  float* rs = sm + 2 * H;
  float f0 = c0, f1 = c1;
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

// one CTA per (row, group)
template <typename T>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg,
                                       const float* __restrict__ weight, T* __restrict__ out, int ldout, int gsize, int gate_first, float eps,
                                       int act) {
  extern __shared__ float sm[];          // [gsize]
  __shared__ float part[33];
  pdl_trigger();
  pdl_wait();
  const int64_t n = blockIdx.x;
  const int c0 = blockIdx.y * gsize;
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
  NVC_DISPATCH_DT(out_dtype, T, {
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
      NVC_CUDA_CHECK(ctx, cudaFuncSetAttribute(rms_norm_blend_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384 * 4));
      attr_set = true;
    }
    NVC_CUDA_CHECK(ctx, nvc_launch(ctx, rms_norm_blend_kernel<T>, dim3(N), dim3(threads), smem, nvc_stream(stream), res_in, bias, y0, w0, c0, y1, w1,
                                   c1, res_out, ld, w, reinterpret_cast<T*>(out), ldo, eps, rows, H));
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
  NVC_DISPATCH_DT(out_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, group_norm_gate_kernel<T>, dim3(N, groups), dim3(threads), (size_t)gsize * sizeof(float),
                                                 nvc_stream(stream), o, ldo, gate, ldg, weight, reinterpret_cast<T*>(out), ldout, gsize, gate_first,
                                                 eps, act)));
  ctx->launches++;
  return NVC_OK;
}

}  // extern "C"
