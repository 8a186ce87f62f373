// Mixture-of-experts routing around the grouped matrix products (linear_generic.cu, moe_gemm): everything is sized
// by device-resident counts, so a step needs no host round trip and replays inside a CUDA graph.
//   nvc_moe_route    router logits in fp32, sigmoid scores, biased top-k choice, normalised weights, shared-expert gate
//   nvc_moe_sort     counting sort of the (token, choice) pairs by expert: group offsets, source rows, positions
//   nvc_moe_combine  weighted sum of a token's expert rows plus the gated shared expert, fp32
#include "typed.cuh"

namespace {

// one warp per token.  Scores of up to 32 * kPerLane experts live in registers.
constexpr int kMaxPerLane = 8;   // experts <= 256

// top-k by repeated arg-max over the choice scores c (ties -> the lower expert index); expert e lives in lane e % 32,
// slot e / 32.  Writes idx / weights of token n: s_chosen / (sum of the chosen s + 1e-20) * scale.
__device__ __forceinline__ void topk_write(float (&s)[kMaxPerLane], float (&c)[kMaxPerLane], int lane, int E, int top, float scale,
                                           int32_t* __restrict__ idx, float* __restrict__ wout, int64_t n, bool normalize = true) {
  // top-k by repeated arg-max over the choice scores (ties -> the lower expert index)
  float sel_sum = 0.f, my_w = 0.f;
  int my_e = 0;
  for (int t = 0; t < top; ++t) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (c[i] > bv || (c[i] == bv && e < be))) { bv = c[i]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    // the owner lane publishes the unbiased score and retires the expert
    float sv = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (lane + 32 * i == be) { sv = s[i]; c[i] = -INFINITY; }
    sv = __shfl_sync(0xffffffffu, sv, be & 31);
    sel_sum += sv;
    if (lane == t % 32) { my_w = sv; my_e = be; }
    if (t % 32 == 31 || t == top - 1) {
      // flush up to 32 choices (weights are scaled after the loop: keep raw scores for now)
      const int t0 = t - (t % 32);
      if (t0 + lane <= t) { idx[(int64_t)n * top + t0 + lane] = my_e; wout[(int64_t)n * top + t0 + lane] = my_w; }
    }
  }
  __syncwarp();
  const float inv = normalize ? scale / (sel_sum + 1e-20f) : scale;
  for (int t = lane; t < top; t += 32) wout[(int64_t)n * top + t] *= inv;
}

// scores from logits that a matrix product has already taken: z [N, ldz] fp32, column gate_col (if >= 0) = the shared gate
__global__ void moe_topk_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ corr, int E, int top, float scale,
                                int gate_col, int score, int normalize, int32_t* __restrict__ idx, float* __restrict__ wout,
                                float* __restrict__ gate, int N) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const float* zr = z + (int64_t)n * ldz;
  float s[kMaxPerLane], c[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    s[i] = 0.f;
    c[i] = -INFINITY;
    if (e < E) s[i] = zr[e];
  }
  if (score == NVC_ROUTE_SOFTMAX) {       // over all E columns, fp32
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (lane + 32 * i < E) mx = fmaxf(mx, s[i]);
    mx = warp_max(mx);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (lane + 32 * i < E) { s[i] = expf(s[i] - mx); den += s[i]; }
    den = warp_sum(den);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) s[i] = s[i] / den;
  } else {
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (lane + 32 * i < E) s[i] = sigmoid_f32(s[i]);
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i)
    if (lane + 32 * i < E) c[i] = s[i] + __ldg(corr + lane + 32 * i);
  if (gate_col >= 0 && gate && lane == 0) gate[n] = sigmoid_f32(zr[gate_col]);
  topk_write(s, c, lane, E, top, scale, idx, wout, n, normalize != 0);
}

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ wr, const float* __restrict__ corr,
                                 const float* __restrict__ wsg, int E, int top, float scale, int32_t* __restrict__ idx,
                                 float* __restrict__ wout, float* __restrict__ gate, int N, int H) {
  extern __shared__ float hs[];   // [warps][H]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  float* x = hs + (size_t)warp * H;
  for (int j = lane; j < H; j += 32) x[j] = ld_f(h + (int64_t)n * ldh + j);
  __syncwarp();
  // expert e's score lives in lane e % 32, slot e / 32; every dot product is taken by the whole warp (coalesced weight rows)
  float s[kMaxPerLane], c[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) { s[i] = 0.f; c[i] = -INFINITY; }
  for (int e0 = 0; e0 < E; e0 += 4) {           // four experts at a time: independent loads and sums
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    const float* w0 = wr + (int64_t)e0 * H;
#pragma unroll 4
    for (int j = lane; j < H; j += 32) {
      const float xv = x[j];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (e0 + u < E) z[u] = fmaf(xv, __ldg(w0 + (int64_t)u * H + j), z[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = e0 + u;
      const float zu = warp_sum(z[u]);
      if (e < E && lane == (e & 31)) {
        const float sv = sigmoid_f32(zu), cv = sv + __ldg(corr + e);
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i)
          if (i == (e >> 5)) { s[i] = sv; c[i] = cv; }
      }
    }
  }
  if (wsg && gate) {
    float z = 0.f;
    for (int j = lane; j < H; j += 32) z = fmaf(x[j], __ldg(wsg + j), z);
    z = warp_sum(z);
    if (lane == 0) gate[n] = sigmoid_f32(z);
  }
  topk_write(s, c, lane, E, top, scale, idx, wout, n);
}

// Stable counting sort by expert in one CTA of 32 warps (pairs = N * top).  Warp w owns the contiguous segment w of the
// pairs: it counts its pairs per expert, a prefix over (expert, warp) gives every warp its first position in every
// expert's group, and the warp then places its pairs in order (__match_any_sync ranks equal experts inside a batch of
// 32).  Within an expert the pairs keep token order, so the layout - and every sum downstream - is deterministic.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int32_t* __restrict__ idx, int P, int top, int E, int E_real, int align, int32_t* __restrict__ offsets,
                int32_t* __restrict__ src_rows, int32_t* __restrict__ pos, int32_t* __restrict__ tile_group, int tiles_cap) {
  extern __shared__ int32_t sm[];   // [32][E] counts -> starts, then [E + 1] offsets, then [E] sizes
  int32_t* cnt = sm;
  int32_t* off = sm + 32 * E;
  int32_t* size = off + E + 1;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const int seg = ((P + 31) / 32 + 31) / 32 * 32;      // pairs per warp, a multiple of 32
  const int p_begin = warp * seg, p_end = min(P, p_begin + seg);
  for (int p = p_begin + lane; p < p_end; p += 32) atomicAdd(&cnt[warp * E + idx[p]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int total = 0;
    for (int w = 0; w < 32; ++w) total += cnt[w * E + e];
    size[e] = total;
  }
  __syncthreads();
  if (threadIdx.x == 0) {                                // every group starts at a multiple of `align` rows
    off[0] = 0;
    for (int e = 0; e < E; ++e) off[e + 1] = off[e] + (size[e] + align - 1) / align * align;
  }
  __syncthreads();
  if (align > 1) {
    // rows between a group's last pair and the next group's start have no source; tiles of `align` rows -> their group
    for (int e = warp; e < E; e += blockDim.x >> 5) {
      for (int r = off[e] + size[e] + lane; r < off[e + 1]; r += 32) src_rows[r] = -1;
      if (tile_group)
        for (int t = off[e] / align + lane; t < off[e + 1] / align; t += 32) tile_group[t] = e < E_real ? e : -1;   // no product behind an identity expert
    }
    if (tile_group)
      for (int t = off[E] / align + threadIdx.x; t < tiles_cap; t += blockDim.x) tile_group[t] = -1;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) {    // counts -> first position of (warp, expert)
    int a = off[e];
    for (int w = 0; w < 32; ++w) {
      const int n = cnt[w * E + e];
      cnt[w * E + e] = a;
      a += n;
    }
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  __syncthreads();
  for (int p0 = p_begin; p0 < p_end; p0 += 32) {
    const int p = p0 + lane;
    const bool have = p < p_end;
    const int e = have ? idx[p] : -1 - lane;             // absent lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (have) {
      const int at = cnt[warp * E + e] + __popc(peers & ((1u << lane) - 1));
      src_rows[at] = p / top;
      pos[p] = at;
    }
    __syncwarp();
    if (have && lane == 31 - __clz(peers)) cnt[warp * E + e] += __popc(peers);   // the last peer advances the group
    __syncwarp();
  }
}

// out[r] = in[src_rows[r]] for r < *num_rows (a device count), zeros where src_rows[r] < 0; 16 bytes per thread
__global__ void gather_rows_kernel(const uint4* __restrict__ in, int ld_in, const int32_t* __restrict__ src_rows,
                                   const int32_t* __restrict__ num_rows, uint4* __restrict__ out, int ld_out, int rows_cap, int per_row,
                                   int rows_per_cta) {
  pdl_trigger();
  pdl_wait();
  const int n = min(rows_cap, *num_rows);
  for (int i = threadIdx.x; i < rows_per_cta * per_row; i += blockDim.x) {
    const int r = blockIdx.x * rows_per_cta + i / per_row, c = i % per_row;
    if (r >= n) break;
    const int src = src_rows[r];
    out[(int64_t)r * ld_out + c] = src >= 0 ? in[(int64_t)src * ld_in + c] : make_uint4(0u, 0u, 0u, 0u);
  }
}

// experts from E_real on are identity experts: their pairs read the token's own row x[n] instead of a row of y
template <typename TY, typename TX>
__global__ void moe_combine_identity_kernel(const TY* __restrict__ y, int ldy, const int32_t* __restrict__ pos, const float* __restrict__ w,
                                            const int32_t* __restrict__ idx, int top, int E_real, const TX* __restrict__ x, int ldx,
                                            float* __restrict__ out, int ldo, int H) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float a = 0.f;
    for (int t = 0; t < top; ++t) {
      const int64_t p = (int64_t)n * top + t;
      const float v = idx[p] < E_real ? ld_f(y + (int64_t)pos[p] * ldy + j) : ld_f(x + (int64_t)n * ldx + j);
      a = fmaf(w[p], v, a);
    }
    out[(int64_t)n * ldo + j] = a;
  }
}

template <typename TY, typename TS>
__global__ void moe_combine_kernel(const TY* __restrict__ y, int ldy, const int32_t* __restrict__ pos, const float* __restrict__ w,
                                   int top, const TS* __restrict__ shared, int lds, const float* __restrict__ gate,
                                   float* __restrict__ out, int ldo, int H) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float a = 0.f;
    for (int t = 0; t < top; ++t) a = fmaf(w[(int64_t)n * top + t], ld_f(y + (int64_t)pos[(int64_t)n * top + t] * ldy + j), a);
    if (shared) a += ld_f(shared + (int64_t)n * lds + j) * (gate ? gate[n] : 1.0f);
    out[(int64_t)n * ldo + j] = a;
  }
}

// the same sum on fp32 rows whose width and strides are multiples of 4: 16-byte loads and stores, same order of additions
__global__ void moe_combine_f4_kernel(const float4* __restrict__ y, int ldy4, const int32_t* __restrict__ pos, const float* __restrict__ w,
                                      int top, const float4* __restrict__ shared, int lds4, const float* __restrict__ gate,
                                      float4* __restrict__ out, int ldo4, int H4) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const float g = shared ? (gate ? gate[n] : 1.0f) : 0.f;
  for (int j = threadIdx.x; j < H4; j += blockDim.x) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = 0; t < top; ++t) {
      const float wt = w[(int64_t)n * top + t];
      const float4 v = y[(int64_t)pos[(int64_t)n * top + t] * ldy4 + j];
      a.x = fmaf(wt, v.x, a.x); a.y = fmaf(wt, v.y, a.y); a.z = fmaf(wt, v.z, a.z); a.w = fmaf(wt, v.w, a.w);
    }
    if (shared) {
      const float4 v = shared[(int64_t)n * lds4 + j];
      a.x += v.x * g; a.y += v.y * g; a.z += v.z * g; a.w += v.w * g;
    }
    out[(int64_t)n * ldo4 + j] = a;
  }
}

// one CTA per (token, choice): the token's row times the pair's router weight, written where the sort put the pair
template <typename T>
__global__ void moe_scatter_scaled_kernel(const T* __restrict__ h, int ldh, const int32_t* __restrict__ pos, const float* __restrict__ topk_w,
                                          T* __restrict__ out, int ldo, int top, int H) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x, n = pair / top;
  const float w = topk_w[pair];
  const T* x = h + (int64_t)n * ldh;
  T* y = out + (int64_t)pos[pair] * ldo;
  for (int j = threadIdx.x; j < H; j += blockDim.x) st_f(y + j, w * ld_f(x + j));
}

}  // namespace

extern "C" {

int nvc_moe_route(nvc_ctx* ctx, const void* h, int h_dtype, int ldh, const float* w_router, const float* correction,
                  const float* w_shared_gate, int E, int top, float scale, int32_t* topk_idx, float* topk_w, float* gate, int N,
                  int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && h && w_router && correction && topk_idx && topk_w, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, (w_shared_gate == nullptr) == (gate == nullptr), NVC_EINVAL, "the shared gate needs its weight and its output");
  NVC_REQUIRE(ctx, E > 0 && E <= 32 * kMaxPerLane && top > 0 && top <= E, NVC_ESHAPE, "experts must be in [1, 256], top in [1, experts]");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && ldh >= H && H <= 12288, NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  const int warps = H <= 3072 ? 4 : 1;
  const size_t smem = (size_t)warps * H * sizeof(float);
  NVC_DISPATCH_DT(h_dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_route_kernel<T>, dim3((N + warps - 1) / warps), dim3(32 * warps), smem,
                                                 nvc_stream(stream), reinterpret_cast<const T*>(h), ldh, w_router, correction,
                                                 w_shared_gate, E, top, scale, topk_idx, topk_w, gate, N, H)));
  ctx->launches++;
  return NVC_OK;
}

int nvc_moe_route_logits(nvc_ctx* ctx, const float* z, int ldz, const float* correction, int E, int top, float scale, int gate_col,
                         int32_t* topk_idx, float* topk_w, float* gate, int N, void* stream) {
  return nvc_moe_route_logits_ex(ctx, z, ldz, correction, E, top, scale, gate_col, NVC_ROUTE_SIGMOID, 1, topk_idx, topk_w, gate, N, stream);
}

int nvc_moe_route_logits_ex(nvc_ctx* ctx, const float* z, int ldz, const float* correction, int E, int top, float scale, int gate_col,
                            int score, int normalize, int32_t* topk_idx, float* topk_w, float* gate, int N, void* stream) {
  NVC_REQUIRE(ctx, ctx && z && correction && topk_idx && topk_w, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, score == NVC_ROUTE_SIGMOID || score == NVC_ROUTE_SOFTMAX, NVC_EINVAL, "unknown score function");
  NVC_REQUIRE(ctx, E > 0 && E <= 32 * kMaxPerLane && top > 0 && top <= E, NVC_ESHAPE, "experts must be in [1, 256], top in [1, experts]");
  NVC_REQUIRE(ctx, N >= 0 && ldz >= E && gate_col < ldz && (gate_col < 0 || gate), NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_topk_kernel, dim3((N + 3) / 4), dim3(128), 0, nvc_stream(stream), z, ldz, correction, E, top, scale,
                                 gate_col, score, normalize, topk_idx, topk_w, gate, N));
  ctx->launches++;
  return NVC_OK;
}

int nvc_moe_sort(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int32_t* offsets, int32_t* src_rows, int32_t* pos,
                 void* stream) {
  return nvc_moe_sort_padded(ctx, topk_idx, N, top, E, 1, offsets, src_rows, pos, nullptr, 0, stream);
}

int nvc_moe_sort_padded(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int align, int32_t* offsets, int32_t* src_rows,
                        int32_t* pos, int32_t* tile_group, int tiles_cap, void* stream) {
  return nvc_moe_sort_padded_ex(ctx, topk_idx, N, top, E, E, align, offsets, src_rows, pos, tile_group, tiles_cap, stream);
}

int nvc_moe_sort_padded_ex(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int E_real, int align, int32_t* offsets,
                           int32_t* src_rows, int32_t* pos, int32_t* tile_group, int tiles_cap, void* stream) {
  NVC_REQUIRE(ctx, ctx && topk_idx && offsets && src_rows && pos, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, E_real >= 0 && E_real <= E, NVC_EINVAL, "E_real must be in [0, E]");
  NVC_REQUIRE(ctx, N >= 0 && top > 0 && E > 0 && E <= 320 && align >= 1, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, !tile_group || (align > 1 && (int64_t)tiles_cap * align >= (int64_t)N * top + (int64_t)E * (align - 1)), NVC_EINVAL,
              "tile_group needs align > 1 and room for every group's padding");
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_sort_kernel, dim3(1), dim3(1024), (size_t)(34 * E + 1) * sizeof(int32_t), nvc_stream(stream),
                                 topk_idx, N * top, top, E, E_real, align, offsets, src_rows, pos, tile_group, tiles_cap));
  ctx->launches++;
  return NVC_OK;
}

int nvc_gather_rows_bf16(nvc_ctx* ctx, const nvc_bf16* in, int ld_in, const int32_t* src_rows, const int32_t* num_rows, nvc_bf16* out,
                         int ld_out, int rows_cap, int width, void* stream) {
  NVC_REQUIRE(ctx, ctx && in && src_rows && num_rows && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, rows_cap >= 0 && width > 0 && width % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && ld_in >= width && ld_out >= width,
              NVC_ESHAPE, "width and row strides must be multiples of 8");
  NVC_REQUIRE(ctx, ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0, NVC_EINVAL, "pointers must be 16-byte aligned");
  if (rows_cap == 0) return NVC_OK;
  const int per_row = width / 8;                                   // 16-byte chunks per row
  const int rows_per_cta = std::max(1, 256 / per_row);
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, gather_rows_kernel, dim3((rows_cap + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, nvc_stream(stream),
                                 reinterpret_cast<const uint4*>(in), ld_in / 8, src_rows, num_rows, reinterpret_cast<uint4*>(out), ld_out / 8,
                                 rows_cap, per_row, rows_per_cta));
  ctx->launches++;
  return NVC_OK;
}

int nvc_moe_combine(nvc_ctx* ctx, const void* y, int y_dtype, int ldy, const int32_t* pos, const float* topk_w, int top,
                    const void* shared, int shared_dtype, int lds, const float* gate, float* out, int ldo, int N, int H,
                    void* stream) {
  NVC_REQUIRE(ctx, ctx && y && pos && topk_w && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && top > 0 && ldy >= H && ldo >= H && (!shared || lds >= H), NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  if (y_dtype == NVC_DT_F32 && (!shared || shared_dtype == NVC_DT_F32) && H % 4 == 0 && ldy % 4 == 0 && ldo % 4 == 0 &&
      (!shared || lds % 4 == 0) && ((uintptr_t)y % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)shared % 16) == 0) {
    NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_combine_f4_kernel, dim3(N), dim3(H / 4 >= 256 ? 256 : (H / 4 > 32 ? 128 : 32)), 0, nvc_stream(stream),
                                   reinterpret_cast<const float4*>(y), ldy / 4, pos, topk_w, top, reinterpret_cast<const float4*>(shared), lds / 4,
                                   gate, reinterpret_cast<float4*>(out), ldo / 4, H / 4));
    ctx->launches++;
    return NVC_OK;
  }
  const dim3 grid(N), block(H >= 1024 ? 512 : 128);
#define NVC_COMBINE(TY, TS)                                                                                                        \
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_combine_kernel<TY, TS>, grid, block, 0, nvc_stream(stream), reinterpret_cast<const TY*>(y), \
                                 ldy, pos, topk_w, top, reinterpret_cast<const TS*>(shared), lds, gate, out, ldo, H))
  if (y_dtype == NVC_DT_F32 && shared_dtype == NVC_DT_F32) NVC_COMBINE(float, float);
  else if (y_dtype == NVC_DT_F32) NVC_COMBINE(float, __nv_bfloat16);
  else if (shared_dtype == NVC_DT_F32) NVC_COMBINE(__nv_bfloat16, float);
  else NVC_COMBINE(__nv_bfloat16, __nv_bfloat16);
#undef NVC_COMBINE
  ctx->launches++;
  return NVC_OK;
}

int nvc_moe_combine_identity(nvc_ctx* ctx, const void* y, int y_dtype, int ldy, const int32_t* pos, const float* topk_w,
                             const int32_t* topk_idx, int top, int E_real, const void* x, int x_dtype, int ldx, float* out, int ldo,
                             int N, int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && y && pos && topk_w && topk_idx && x && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && top > 0 && E_real >= 0 && ldy >= H && ldo >= H && ldx >= H, NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  const dim3 grid(N), block(H >= 1024 ? 512 : 128);
#define NVC_COMBINE(TY, TX)                                                                                                                  \
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_combine_identity_kernel<TY, TX>, grid, block, 0, nvc_stream(stream), reinterpret_cast<const TY*>(y), \
                                 ldy, pos, topk_w, topk_idx, top, E_real, reinterpret_cast<const TX*>(x), ldx, out, ldo, H))
  if (y_dtype == NVC_DT_F32 && x_dtype == NVC_DT_F32) NVC_COMBINE(float, float);
  else if (y_dtype == NVC_DT_F32) NVC_COMBINE(float, __nv_bfloat16);
  else if (x_dtype == NVC_DT_F32) NVC_COMBINE(__nv_bfloat16, float);
  else NVC_COMBINE(__nv_bfloat16, __nv_bfloat16);
#undef NVC_COMBINE
  ctx->launches++;
  return NVC_OK;
}

int nvc_moe_scatter_scaled(nvc_ctx* ctx, const void* h, int dtype, int ldh, const int32_t* pos, const float* topk_w, int top, void* out,
                           int ldo, int N, int H, void* stream) {
  NVC_REQUIRE(ctx, ctx && h && pos && topk_w && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && top > 0 && ldh >= H && ldo >= H, NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
  NVC_DISPATCH_DT(dtype, T,
                  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_scatter_scaled_kernel<T>, dim3(N * top), dim3(H >= 1024 ? 256 : 128), 0, nvc_stream(stream),
                                                 reinterpret_cast<const T*>(h), ldh, pos, topk_w, reinterpret_cast<T*>(out), ldo, top, H)));
  ctx->launches++;
  return NVC_OK;
}

}  // extern "C"
