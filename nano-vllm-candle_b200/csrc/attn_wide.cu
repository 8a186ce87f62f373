// nvc_attn_paged_wide: grouped-query softmax attention over a paged cache whose keys and values have their own widths
// (dim, vdim), with an optional sliding window or chunk mask, an optional cap on the scores (cap tanh(s / cap)), an optional sink
// term in the denominator, an optional sigmoid gate (per output number or per head) and a constant factor on the output.  Rows of
// sequence b are the LAST q_len positions of its context; row at position i sees keys max(0, i - window + 1) .. i (window), the
// keys of its own chunk i - i % chunk .. i (chunk), or 0 .. i (neither).
//
// Two kernels:
//   attn_wide_mma_kernel (attn_wide_mma.cuh)  bf16 storage, dim and vdim multiples of 16 up to 256: tensor pipe
//   attn_wide_simt_kernel                      any sizes, both storage formats, plain fp32 FMA: the exact mode
// Both take the keys of a row in tiles that start at the row's own first visible key, so the order of every sum depends on
// the row's position alone - not on how the prompt was cut, on the batch or on the pages.
#include "typed.cuh"
#include "attn_wide_mma.cuh"

namespace {

constexpr int kSimtWarps = 4;
constexpr int kMaxVPL = 16;     // value columns per lane: vdim <= 512

struct WideArgs {
  const void *q, *k_cache, *v_cache;
  void* out;
  int ldq, ldk, ldv, ldo;
  const int32_t *block_tables, *context_lens, *cu_seqlens;
  int bt_stride, B, block_size;
  nvc_attn_spec s;
};

__device__ __forceinline__ int find_seq(const int32_t* cu, int B, int row) {
  int lo = 0, hi = B - 1;      // largest b with cu[b] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// one CTA of 4 warps per (row, head): warp w takes the 32-key tiles w, w + 4, ... of the row's key range
template <typename T>
__global__ void __launch_bounds__(kSimtWarps * 32) attn_wide_simt_kernel(const WideArgs a) {
  extern __shared__ float sm[];
  pdl_trigger();
  const nvc_attn_spec& s = a.s;
  const int row = blockIdx.x, h = blockIdx.y;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = sm;                                   // [dim]
  float* acc_s = sm + s.dim;                         // [warps][vdim]
  float* ml_s = acc_s + kSimtWarps * s.vdim;         // [warps][2]
  pdl_wait();
  int b = row, qlen = 1, r0 = row;
  if (a.cu_seqlens) {
    b = find_seq(a.cu_seqlens, a.B, row);
    r0 = a.cu_seqlens[b];
    qlen = a.cu_seqlens[b + 1] - r0;
  }
  const int pos = a.context_lens[b] - qlen + (row - r0);
  const int lo = widemma::first_visible(pos, s.window, s.chunk);
  const int g = h / (s.heads / s.kv_heads);
  const T* qp = reinterpret_cast<const T*>(a.q) + (int64_t)row * a.ldq + (int64_t)h * s.dim;
  for (int d = threadIdx.x; d < s.dim; d += blockDim.x) q_s[d] = ld_f(qp + d);
  __syncthreads();
  const int32_t* bt = a.block_tables + (int64_t)b * a.bt_stride;
  const T* K = reinterpret_cast<const T*>(a.k_cache) + (int64_t)g * s.dim;
  const T* V = reinterpret_cast<const T*>(a.v_cache) + (int64_t)g * s.vdim;
  const int vpl = (s.vdim + 31) >> 5;
  float acc[kMaxVPL];
#pragma unroll
  for (int c = 0; c < kMaxVPL; ++c) acc[c] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int t = lo + 32 * wid; t <= pos; t += 32 * kSimtWarps) {
    const int j = t + lane;
    const bool valid = j <= pos;
    int64_t slot = 0;
    float sc = -INFINITY;
    if (valid) {
      slot = (int64_t)bt[j / a.block_size] * a.block_size + j % a.block_size;
      const T* kp = K + slot * a.ldk;
      float dot = 0.f;
      for (int d = 0; d < s.dim; ++d) dot = fmaf(q_s[d], ld_f(kp + d), dot);
      sc = dot * s.scale;
      if (s.softcap > 0.f) sc = s.softcap * tanhf(sc / s.softcap);
    }
    const float mn = fmaxf(m, warp_max(sc));     // finite: the tile's first key is visible
    const float p = valid ? expf(sc - mn) : 0.f;
    const float corr = expf(m - mn);             // m == -inf: 0
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int c = 0; c < kMaxVPL; ++c) acc[c] *= corr;
    const int nk = min(32, pos - t + 1);
    for (int jj = 0; jj < nk; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t sj = __shfl_sync(0xffffffffu, slot, jj);
      const T* vp = V + sj * a.ldv;
#pragma unroll
      for (int c = 0; c < kMaxVPL; ++c)
        if (c < vpl && lane + 32 * c < s.vdim) acc[c] = fmaf(pj, ld_f(vp + lane + 32 * c), acc[c]);
    }
  }
#pragma unroll
  for (int c = 0; c < kMaxVPL; ++c)
    if (c < vpl && lane + 32 * c < s.vdim) acc_s[wid * s.vdim + lane + 32 * c] = acc[c];
  if (lane == 0) { ml_s[2 * wid] = m; ml_s[2 * wid + 1] = l; }
  __syncthreads();
  float M = s.sink ? __ldg(s.sink + h) : -INFINITY;
#pragma unroll
  for (int w = 0; w < kSimtWarps; ++w) M = fmaxf(M, ml_s[2 * w]);
  float L = s.sink ? expf(__ldg(s.sink + h) - M) : 0.f;
  float f[kSimtWarps];
#pragma unroll
  for (int w = 0; w < kSimtWarps; ++w) {
    f[w] = expf(ml_s[2 * w] - M);       // a warp without keys has m = -inf: factor 0
    L += ml_s[2 * w + 1] * f[w];
  }
  const float inv = 1.0f / L;
  T* op = reinterpret_cast<T*>(a.out) + (int64_t)row * a.ldo + (int64_t)h * s.vdim;
  for (int c = threadIdx.x; c < s.vdim; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kSimtWarps; ++w) o += acc_s[w * s.vdim + c] * f[w];
    o *= inv;
    if (s.gate) o *= sigmoid_f32(s.gate[(int64_t)row * s.ldg + (s.gate_per_head ? (int64_t)h : (int64_t)h * s.vdim + c)]);
    st_f(op + c, o * s.out_scale);
  }
}

}  // namespace

extern "C" int nvc_attn_paged_wide(nvc_ctx* ctx, const void* q, int ldq, const void* k_cache, int ldk, const void* v_cache, int ldv,
                                   const int32_t* block_tables, int bt_stride, const int32_t* context_lens, const int32_t* cu_seqlens,
                                   int B, int rows, int max_qlen, int block_size, const nvc_attn_spec* spec, void* out, int ldo, int dtype,
                                   void* stream) {
  NVC_REQUIRE(ctx, ctx && q && k_cache && v_cache && block_tables && context_lens && spec && out, NVC_EINVAL, "null pointer");
  const nvc_attn_spec& s = *spec;
  NVC_REQUIRE(ctx, B > 0 && rows >= B && block_size > 0 && bt_stride > 0 && max_qlen >= 1, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, cu_seqlens || rows == B, NVC_EINVAL, "rows without cu_seqlens: one per sequence");
  NVC_REQUIRE(ctx, s.heads > 0 && s.kv_heads > 0 && s.heads % s.kv_heads == 0 && s.dim > 0 && s.vdim > 0 && s.dim <= 512 && s.vdim <= 512,
              NVC_ESHAPE, "heads / kv_heads / dim / vdim (dim, vdim <= 512)");
  NVC_REQUIRE(ctx, s.window >= 0 && s.chunk >= 0 && !(s.window > 0 && s.chunk > 0) && s.softcap >= 0.f &&
                       (!s.gate || s.ldg >= (s.gate_per_head ? s.heads : s.heads * s.vdim)),
              NVC_EINVAL, "bad window / chunk / cap / gate");
  NVC_REQUIRE(ctx, ldq >= s.heads * s.dim && ldk >= s.kv_heads * s.dim && ldv >= s.kv_heads * s.vdim && ldo >= s.heads * s.vdim, NVC_EINVAL,
              "bad strides");
  WideArgs a{q, k_cache, v_cache, out, ldq, ldk, ldv, ldo, block_tables, context_lens, cu_seqlens, bt_stride, B, block_size, s};
  if (dtype == NVC_DT_BF16 && attn_wide_mma_takes(s, ldq, ldk, ldv, ldo, block_size)) {
    int rc = attn_wide_mma_launch(ctx, a.q, a.k_cache, a.v_cache, a.out, ldq, ldk, ldv, ldo, block_tables, context_lens, cu_seqlens, bt_stride,
                                  B, rows, max_qlen, block_size, s, nvc_stream(stream));
    if (rc != NVC_ENOTIMPL) return rc;
  }
  const size_t smem = ((size_t)s.dim + (size_t)kSimtWarps * s.vdim + 2 * kSimtWarps) * sizeof(float);
  NVC_DISPATCH_DT(dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, attn_wide_simt_kernel<T>, dim3(rows, s.heads), dim3(kSimtWarps * 32), smem,
                                                 nvc_stream(stream), a)));
  ctx->launches++;
  return NVC_OK;
}
