// nvc_retention_scan: linear attention with a fixed decay per head and no softmax or denominator,
//   S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
// over the new tokens of every sequence of a step, token by token.  The state S [dim, vdim] of every (sequence, head) lives in
// fp32 in a pool of state slots: a sequence whose first new token sits at position 0 starts from zeros, every other one from what
// its slot holds, and the slot is written back after the last token.  q, k, v, o are fp32 rows (the caller has already rotated q and
// k and scaled k).
//
// Two kernels, both with one CTA per (sequence, head, slice of 32 value columns) whose threads (column v, row group r) keep rows
// [r DPT, (r + 1) DPT) of column v of the state in registers (token by token: 32 rows per warp, up to 32 warps):
//   retention_scan_kernel    token by token (decode steps and very short portions): 2 DPT FMAs per thread and token and, when the
//                            rows are split, one shared-memory reduction; the next token's q / k / v are fetched meanwhile.
//   retention_chunk_kernel   32 tokens at a time (prompt portions), the same recurrence regrouped:
//                              A[t][j] = decay^(t - j) (q_t . k_j), j <= t            inside the chunk
//                              o_t     = sum_j A[t][j] v_j + decay^(t + 1) S^T q_t     S: the state before the chunk
//                              S      <- decay^n S + sum_j decay^(n - 1 - j) k_j v_j^T n: tokens of the chunk
//                            Powers of the decay come from a table built by repeated multiplication (exact for 0 and 1).
// Both are plain fp32 FMA code; they differ from one another by rounding only.
//
// nvc_decay_scan is the same pair of kernels with what other linear recurrences of this shape need (VAR = true):
//   a decay per token and head, given as its logarithm: S_t = exp(l_t) S_(t-1) + k_t v_t^T.  Inside a chunk only differences of the
//     running sums L_t = l_0 + .. + l_t are exponentiated (all <= 0): A[t][j] carries exp(L_t - L_j), the state's share exp(L_t), the
//     state update exp(L_(n-1) - L_j); a decay that underflows stays a plain zero;
//   q and k heads shared by groups of value heads (head h reads q / k head h / (heads / qk_heads));
//   a skip term o_t += skip_w[h] * skip_t.
// A selective state space layer in its dual form is this recurrence with q = C, k = B, v = dt x, l = -exp(A_log) dt, skip = x.
#include "typed.cuh"

namespace {

struct RetArgs {
  const float *q, *k, *v;
  float* o;
  int ldq, ldk, ldv, ldo;
  float* state;                  // [slots, heads, dim, vdim]
  const int32_t *state_slots, *cu_seqlens, *positions;
  const float* decay;            // [heads]                       (VAR = false)
  int heads, dim, vdim;
  int qk_heads;                  // q / k heads (a divisor of heads)
  const float* log_decay;        // [rows, ldl], one per head       (VAR = true)
  int ldl;
  const float* skip;             // [rows, lds] like v, or NULL
  const float* skip_w;           // [heads]
  int lds;
};

template <int DPT, bool VAR>
__global__ void retention_scan_kernel(const RetArgs a) {
  extern __shared__ float sm[];
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * 32;
  const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5, groups = blockDim.x >> 5;
  const int v = v0 + lane;
  const bool vok = v < a.vdim;
  float* q_s = sm;                    // [2][dim]
  float* k_s = sm + 2 * a.dim;        // [2][dim]
  float* red = sm + 4 * a.dim;        // [groups][32]
  const int hq = h / (a.heads / a.qk_heads);
  float dec = VAR ? 0.f : __ldg(a.decay + h);
  const float sw = a.skip ? __ldg(a.skip_w + h) : 0.f;
  pdl_wait();
  const int r0 = a.cu_seqlens ? a.cu_seqlens[b] : b;
  const int r1 = a.cu_seqlens ? a.cu_seqlens[b + 1] : b + 1;
  const int d0 = rg * DPT;
  float S[DPT];
  float* sp = a.state + (((int64_t)a.state_slots[b] * a.heads + h) * a.dim) * a.vdim;
  const bool fresh = a.positions[r0] == 0;
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = (!fresh && vok && d0 + i < a.dim) ? sp[(int64_t)(d0 + i) * a.vdim + v] : 0.f;
  // stage token r0
  for (int d = threadIdx.x; d < a.dim; d += blockDim.x) {
    q_s[d] = a.q[(int64_t)r0 * a.ldq + hq * a.dim + d];
    k_s[d] = a.k[(int64_t)r0 * a.ldk + hq * a.dim + d];
  }
  float vt = vok ? a.v[(int64_t)r0 * a.ldv + h * a.vdim + v] : 0.f;
  float ln = VAR ? a.log_decay[(int64_t)r0 * a.ldl + h] : 0.f;
  __syncthreads();
  for (int t = r0; t < r1; ++t) {
    const int cur = (t - r0) & 1;
    const float* qc = q_s + cur * a.dim;
    const float* kc = k_s + cur * a.dim;
    float vn = 0.f;
    if (t + 1 < r1) {       // fetch the next token into the other buffer
      for (int d = threadIdx.x; d < a.dim; d += blockDim.x) {
        q_s[(cur ^ 1) * a.dim + d] = a.q[(int64_t)(t + 1) * a.ldq + hq * a.dim + d];
        k_s[(cur ^ 1) * a.dim + d] = a.k[(int64_t)(t + 1) * a.ldk + hq * a.dim + d];
      }
      vn = vok ? a.v[(int64_t)(t + 1) * a.ldv + h * a.vdim + v] : 0.f;
    }
    if (VAR) {
      dec = expf(ln);
      if (t + 1 < r1) ln = a.log_decay[(int64_t)(t + 1) * a.ldl + h];
    }
    const float sk = (a.skip && vok) ? sw * a.skip[(int64_t)t * a.lds + h * a.vdim + v] : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      if (d0 + i < a.dim) {
        S[i] = fmaf(dec, S[i], kc[d0 + i] * vt);
        acc = fmaf(S[i], qc[d0 + i], acc);
      }
    }
    if (groups > 1) {
      red[rg * 32 + lane] = acc;
      __syncthreads();
      if (rg == 0) {
        float s = 0.f;
        for (int g = 0; g < groups; ++g) s += red[g * 32 + lane];
        if (vok) a.o[(int64_t)t * a.ldo + h * a.vdim + v] = s + sk;
      }
    } else if (vok) {
      a.o[(int64_t)t * a.ldo + h * a.vdim + v] = acc + sk;
    }
    vt = vn;
    __syncthreads();
  }
  if (vok)
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < a.dim) sp[(int64_t)(d0 + i) * a.vdim + v] = S[i];
}

constexpr int kChunk = 32;          // tokens per chunk
constexpr int kChunkWarps = 8;         // a divisor of 8: the chunk's 8 groups of four keys are dealt out to the warps
constexpr int kKeyGroups = 8 / kChunkWarps;

__device__ __forceinline__ float dot4(const float4& x, const float4& y, float acc) {
  acc = fmaf(x.x, y.x, acc);
  acc = fmaf(x.y, y.y, acc);
  acc = fmaf(x.z, y.z, acc);
  return fmaf(x.w, y.w, acc);
}

// float4 units per staged q row: odd, so that the 8 lanes of a 128-bit shared-memory phase (lane = token) hit distinct banks
__host__ __device__ inline int chunk_q_stride4(int dim) { const int q4 = (dim + 3) / 4; return (q4 & 1) ? q4 : q4 + 1; }

// Shared-memory operands are read as float4 (one load per four FMAs) and reused across a register tile: the kernel is bound
// by the FMA pipe, not by shared-memory loads.
// The variant with per-token decays at up to 16 rows per warp is capped at 85 registers (a few spilled words) so that three CTAs -
// what shared memory allows - fit an SM; the fixed-decay variant needs 80 as it is.
template <int DPT, bool VAR>
__global__ void __launch_bounds__(kChunkWarps * 32, DPT <= 16 ? 3 : 0) retention_chunk_kernel(const RetArgs a) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * 32;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int v = v0 + lane;
  const bool vok = v < a.vdim;
  const int dim = a.dim, q4 = (dim + 3) / 4, dim4 = 4 * q4, RS = chunk_q_stride4(dim);
  float4* q_s = reinterpret_cast<float4*>(sm);                 // [32][RS]   rows padded with zeros
  float4* k_s = q_s + kChunk * RS;                             // [32][q4]   (read as broadcasts)
  float* v_s = reinterpret_cast<float*>(k_s + kChunk * q4);    // [32][32]
  float4* a_s = reinterpret_cast<float4*>(v_s + kChunk * 32);  // [32][9]    A[t][j], j in fours, zero above the diagonal
  float* part = reinterpret_cast<float*>(a_s + kChunk * 9);    // [warps][32][32]
  float* gp = part + kChunkWarps * kChunk * 32;                // decay^0 .. decay^32;  VAR: the running sums L_0 .. L_31 of the chunk
  const int hq = h / (a.heads / a.qk_heads);
  const float sw = a.skip ? __ldg(a.skip_w + h) : 0.f;
  if (!VAR && threadIdx.x == 0) {
    const float dec = __ldg(a.decay + h);
    float p = 1.f;
    for (int i = 0; i <= kChunk; ++i) { gp[i] = p; p *= dec; }
  }
  pdl_wait();
  const int r0 = a.cu_seqlens ? a.cu_seqlens[b] : b;
  const int r1 = a.cu_seqlens ? a.cu_seqlens[b + 1] : b + 1;
  const int d0 = w * DPT;                                      // this warp's rows of the state (DPT is a multiple of 4)
  float S[DPT];
  float* sp = a.state + (((int64_t)a.state_slots[b] * a.heads + h) * dim) * a.vdim;
  const bool fresh = a.positions[r0] == 0;
#pragma unroll
  for (int i = 0; i < DPT; ++i) S[i] = (!fresh && vok && d0 + i < dim) ? sp[(int64_t)(d0 + i) * a.vdim + v] : 0.f;
  float* q_sf = reinterpret_cast<float*>(q_s);
  float* k_sf = reinterpret_cast<float*>(k_s);
  const bool vec = (dim & 3) == 0 && (a.ldq & 3) == 0 && (a.ldk & 3) == 0 && ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k)) & 15) == 0;
  for (int c0 = r0; c0 < r1; c0 += kChunk) {
    const int n = min(kChunk, r1 - c0);
    __syncthreads();                                   // the previous chunk is done with the staged rows
    // a warp stages whole rows (t = w, w + warps, ...), lanes along the row: no index division, 16-byte loads where the layout allows
    for (int t = w; t < kChunk; t += kChunkWarps) {
      const bool tin = t < n;
      const float* qrow = a.q + (int64_t)(c0 + t) * a.ldq + hq * dim;
      const float* krow = a.k + (int64_t)(c0 + t) * a.ldk + hq * dim;
      if (vec) {
        for (int d4 = lane; d4 < q4; d4 += 32) {
          const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
          q_s[t * RS + d4] = tin ? *reinterpret_cast<const float4*>(qrow + 4 * d4) : z;
          k_s[t * q4 + d4] = tin ? *reinterpret_cast<const float4*>(krow + 4 * d4) : z;
        }
      } else {
        for (int d = lane; d < dim4; d += 32) {
          const bool in = tin && d < dim;
          q_sf[t * 4 * RS + d] = in ? qrow[d] : 0.f;
          k_sf[t * dim4 + d] = in ? krow[d] : 0.f;
        }
      }
    }
    if (VAR && threadIdx.x < 32) {        // inclusive running sums of the chunk's log decays (a fixed order: lane by lane)
      float l = lane < n ? a.log_decay[(int64_t)(c0 + lane) * a.ldl + h] : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, l, o);
        if (lane >= o) l += up;
      }
      gp[lane] = l;
    }
    for (int idx = threadIdx.x; idx < kChunk * 32; idx += blockDim.x) {
      const int t = idx >> 5, c = idx & 31;
      v_s[idx] = (t < n && v0 + c < a.vdim) ? a.v[(int64_t)(c0 + t) * a.ldv + h * a.vdim + v0 + c] : 0.f;
    }
    __syncthreads();
    // ---- A[t][j]: lane = t; warp w takes the groups of four keys jg = w, w + warps, ... (j = 4 jg + u)
    {
      float acc[kKeyGroups][4];
#pragma unroll
      for (int g = 0; g < kKeyGroups; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
      for (int d4 = 0; d4 < q4; ++d4) {
        const float4 qv = q_s[lane * RS + d4];
#pragma unroll
        for (int g = 0; g < kKeyGroups; ++g)
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[g][u] = dot4(qv, k_s[(4 * (w + kChunkWarps * g) + u) * q4 + d4], acc[g][u]);
      }
#pragma unroll
      for (int g = 0; g < kKeyGroups; ++g) {
        const int j0 = 4 * (w + kChunkWarps * g);
        float4 r;
        if (VAR) {
          const float Lt = gp[lane];
          r.x = j0 <= lane ? acc[g][0] * expf(Lt - gp[j0]) : 0.f;
          r.y = j0 + 1 <= lane ? acc[g][1] * expf(Lt - gp[j0 + 1]) : 0.f;
          r.z = j0 + 2 <= lane ? acc[g][2] * expf(Lt - gp[j0 + 2]) : 0.f;
          r.w = j0 + 3 <= lane ? acc[g][3] * expf(Lt - gp[j0 + 3]) : 0.f;
        } else {
          r.x = j0 <= lane ? acc[g][0] * gp[lane - j0] : 0.f;
          r.y = j0 + 1 <= lane ? acc[g][1] * gp[lane - j0 - 1] : 0.f;
          r.z = j0 + 2 <= lane ? acc[g][2] * gp[lane - j0 - 2] : 0.f;
          r.w = j0 + 3 <= lane ? acc[g][3] * gp[lane - j0 - 3] : 0.f;
        }
        a_s[lane * 9 + w + kChunkWarps * g] = r;
      }
    }
    // ---- the state's share of every output: this warp's rows of S against q_t, lane = value column
    for (int t = 0; t < n; ++t) {
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; ++i4) {
        if (d0 + 4 * i4 < dim4) {
          const float4 qv = q_s[t * RS + (d0 >> 2) + i4];
          acc = fmaf(S[4 * i4], qv.x, acc);
          acc = fmaf(S[4 * i4 + 1], qv.y, acc);
          acc = fmaf(S[4 * i4 + 2], qv.z, acc);
          acc = fmaf(S[4 * i4 + 3], qv.w, acc);
        }
      }
      part[(w * kChunk + t) * 32 + lane] = acc;
    }
    __syncthreads();
    // ---- o_t for this warp's tokens t = w, w + warps, ... (a register tile of tokens against four value rows at a time)
    {
      float acc[kChunk / kChunkWarps];
#pragma unroll
      for (int tt = 0; tt < kChunk / kChunkWarps; ++tt) acc[tt] = 0.f;
      const int j4n = (n + 3) >> 2;
      for (int j4 = 0; j4 < j4n; ++j4) {
        float4 vv;
        vv.x = v_s[(4 * j4) * 32 + lane];
        vv.y = v_s[(4 * j4 + 1) * 32 + lane];
        vv.z = v_s[(4 * j4 + 2) * 32 + lane];
        vv.w = v_s[(4 * j4 + 3) * 32 + lane];
#pragma unroll
        for (int tt = 0; tt < kChunk / kChunkWarps; ++tt) acc[tt] = dot4(a_s[(w + kChunkWarps * tt) * 9 + j4], vv, acc[tt]);
      }
#pragma unroll
      for (int tt = 0; tt < kChunk / kChunkWarps; ++tt) {
        const int t = w + kChunkWarps * tt;
        if (t < n) {
          float cross = 0.f;
#pragma unroll
          for (int g = 0; g < kChunkWarps; ++g) cross += part[(g * kChunk + t) * 32 + lane];
          const float sk = (a.skip && vok) ? sw * a.skip[(int64_t)(c0 + t) * a.lds + h * a.vdim + v] : 0.f;
          if (vok) a.o[(int64_t)(c0 + t) * a.ldo + h * a.vdim + v] = fmaf(VAR ? expf(gp[t]) : gp[t + 1], cross, acc[tt]) + sk;
        }
      }
    }
    // ---- the state after the chunk
    {
      const float gn = VAR ? expf(gp[n - 1]) : gp[n];
#pragma unroll
      for (int i = 0; i < DPT; ++i) S[i] *= gn;
      for (int j = 0; j < n; ++j) {
        const float vv = v_s[j * 32 + lane] * (VAR ? expf(gp[n - 1] - gp[j]) : gp[n - 1 - j]);
#pragma unroll
        for (int i4 = 0; i4 < DPT / 4; ++i4) {
          if (d0 + 4 * i4 < dim4) {
            const float4 kv = k_s[j * q4 + (d0 >> 2) + i4];
            S[4 * i4] = fmaf(kv.x, vv, S[4 * i4]);
            S[4 * i4 + 1] = fmaf(kv.y, vv, S[4 * i4 + 1]);
            S[4 * i4 + 2] = fmaf(kv.z, vv, S[4 * i4 + 2]);
            S[4 * i4 + 3] = fmaf(kv.w, vv, S[4 * i4 + 3]);
          }
        }
      }
    }
  }
  if (vok)
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < dim) sp[(int64_t)(d0 + i) * a.vdim + v] = S[i];
}

template <int DPT, bool VAR>
cudaError_t launch_chunk(nvc_ctx* ctx, const RetArgs& a, dim3 grid, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(retention_chunk_kernel<DPT, VAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  return nvc_launch(ctx, retention_chunk_kernel<DPT, VAR>, grid, dim3(kChunkWarps * 32), smem, st, a);
}

template <bool VAR>
int run_scan(nvc_ctx* ctx, const RetArgs& a, int B, int max_qlen, void* stream) {
  const int heads = a.heads, dim = a.dim, vdim = a.vdim;
  if (a.cu_seqlens && max_qlen > 4 && dim <= 512) {
    // prompt portions: 32 tokens at a time
    const int per = ((dim + 3) / 4 * 4 + kChunkWarps - 1) / kChunkWarps;     // rows of the state per warp
    const dim3 grid(B, heads, (vdim + 31) / 32);
    const size_t smem = ((size_t)kChunk * 4 * chunk_q_stride4(dim) + (size_t)kChunk * 4 * ((dim + 3) / 4) + kChunk * 32 + kChunk * 36 +
                         kChunkWarps * kChunk * 32 + kChunk + 4) * sizeof(float);
    cudaError_t ce;
    if (per <= 8) ce = launch_chunk<8, VAR>(ctx, a, grid, smem, nvc_stream(stream));
    else if (per <= 16) ce = launch_chunk<16, VAR>(ctx, a, grid, smem, nvc_stream(stream));
    else if (per <= 32) ce = launch_chunk<32, VAR>(ctx, a, grid, smem, nvc_stream(stream));
    else ce = launch_chunk<64, VAR>(ctx, a, grid, smem, nvc_stream(stream));      // dim <= 512: at most 64 rows per warp
    NVC_CUDA_CHECK(ctx, ce);
    ctx->launches++;
    return NVC_OK;
  }
  // rows of a state column are split over warps of the CTA, 32 (16) rows each: a decode step is bound by reading and writing the
  // state once, and a CTA of one warp holding whole columns of 128 numbers leaves too few loads in flight
  const int dpt = dim <= 16 ? 16 : 32;
  const int groups = (dim + dpt - 1) / dpt;
  const dim3 grid(B, heads, (vdim + 31) / 32), block(32 * groups);
  const size_t smem = ((size_t)4 * dim + (size_t)groups * 32) * sizeof(float);
  cudaError_t ce;
  if (dpt == 16) ce = nvc_launch(ctx, retention_scan_kernel<16, VAR>, grid, block, smem, nvc_stream(stream), a);
  else ce = nvc_launch(ctx, retention_scan_kernel<32, VAR>, grid, block, smem, nvc_stream(stream), a);
  NVC_CUDA_CHECK(ctx, ce);
  ctx->launches++;
  return NVC_OK;
}

}  // namespace

extern "C" int nvc_retention_scan(nvc_ctx* ctx, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, float* o, int ldo,
                                  float* state, const int32_t* state_slots, const int32_t* cu_seqlens, const int32_t* positions,
                                  const float* decay, int B, int max_qlen, int heads, int dim, int vdim, void* stream) {
  NVC_REQUIRE(ctx, ctx && q && k && v && o && state && state_slots && positions && decay, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, B > 0 && heads > 0 && dim > 0 && vdim > 0 && dim <= 1024 && heads <= 65535, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, ldq >= heads * dim && ldk >= heads * dim && ldv >= heads * vdim && ldo >= heads * vdim, NVC_EINVAL, "bad strides");
  RetArgs a{q, k, v, o, ldq, ldk, ldv, ldo, state, state_slots, cu_seqlens, positions, decay, heads, dim, vdim, heads, nullptr, 0, nullptr, nullptr, 0};
  return run_scan<false>(ctx, a, B, max_qlen, stream);
}

extern "C" int nvc_decay_scan(nvc_ctx* ctx, const nvc_decay_scan_args* p, int B, int max_qlen, void* stream) {
  NVC_REQUIRE(ctx, ctx && p && p->q && p->k && p->v && p->o && p->state && p->state_slots && p->positions, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, (p->decay != nullptr) != (p->log_decay != nullptr), NVC_EINVAL, "one of decay and log_decay");
  NVC_REQUIRE(ctx, B > 0 && p->heads > 0 && p->qk_heads > 0 && p->heads % p->qk_heads == 0 && p->dim > 0 && p->vdim > 0 && p->dim <= 1024 &&
                       p->heads <= 65535,
              NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, p->ldq >= p->qk_heads * p->dim && p->ldk >= p->qk_heads * p->dim && p->ldv >= p->heads * p->vdim && p->ldo >= p->heads * p->vdim &&
                       (!p->log_decay || p->ldl >= p->heads) && (!p->skip || (p->skip_w && p->lds >= p->heads * p->vdim)),
              NVC_EINVAL, "bad strides");
  RetArgs a{p->q, p->k, p->v, p->o, p->ldq, p->ldk, p->ldv, p->ldo, p->state, p->state_slots, p->cu_seqlens, p->positions, p->decay,
            p->heads, p->dim, p->vdim, p->qk_heads, p->log_decay, p->ldl, p->skip, p->skip_w, p->lds};
  return p->log_decay ? run_scan<true>(ctx, a, B, max_qlen, stream) : run_scan<false>(ctx, a, B, max_qlen, stream);
}
