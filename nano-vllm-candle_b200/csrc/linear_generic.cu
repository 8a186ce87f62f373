// C = act(A . W^T) for any sizes and both storage formats.  fp32 operands run on the FMA pipe (plain IEEE products and
// sums: the matrix product of the exact mode); bf16 operands whose rows are 16-byte aligned run on the tensor pipe
// (mma.sync m16n8k16, fp32 accumulators, cp.async double buffering) - the small per-head and per-expert products that the
// tcgen05 GEMMs (one dense product per launch, K % 64) do not take.
// Three forms share each kernel:
//   plain      C[M, N] = A[M, K] . W[N, K]^T
//   batched    blockIdx.z = b: A + b * sa, W + b * sw, C + b * sc  (one small product per attention head)
//   grouped    rows [offsets[g], offsets[g + 1]) of C use W + g * sw; row r of A is a_rows[r] (mixture of experts:
//              the rows of one expert are contiguous after the sort, offsets live in device memory)
// 64 x 64 output tile per CTA, 16-deep k-slices through shared memory, 4 x 4 outputs per thread.
#include <cstdlib>

#include "typed.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T, typename TC>
__global__ void __launch_bounds__(256)
linear_kernel(const T* __restrict__ A, int lda, int64_t sa, const int32_t* __restrict__ a_rows, const T* __restrict__ W, int ldw,
              int64_t sw, TC* __restrict__ C, int ldc, int64_t sc, const int32_t* __restrict__ offsets, int groups, int M, int N,
              int K, int act) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Ws[TK][TN + 4];
  pdl_trigger();
  pdl_wait();
  int row0, row_end;
  if (offsets) {
    // tile blockIdx.x of the concatenated per-group tile lists
    int t = blockIdx.x, g = 0, base = 0;
    for (; g < groups; ++g) {
      base = offsets[g];
      const int n = offsets[g + 1] - base;
      const int tiles = (n + TM - 1) / TM;
      if (t < tiles) break;
      t -= tiles;
    }
    if (g == groups) return;
    row0 = base + t * TM;
    row_end = offsets[g + 1];
    W += (int64_t)g * sw;
  } else {
    row0 = blockIdx.x * TM;
    row_end = M;
    A += (int64_t)blockIdx.z * sa;
    W += (int64_t)blockIdx.z * sw;
    C += (int64_t)blockIdx.z * sc;
  }
  const int col0 = blockIdx.y * TN;
  const int tid = threadIdx.x;
  const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
  float acc[4][4] = {};
  // loader: thread -> (row of the tile, 4 consecutive k)
  const int lr = tid / 4, lk = (tid % 4) * 4;
  const int ar = row0 + lr;
  const int64_t a_src = ar < row_end ? (a_rows ? (int64_t)a_rows[ar] : (int64_t)ar) : -1;
  const int wr = col0 + lr;
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_src >= 0 && k < K) ? ld_f(A + a_src * lda + k) : 0.f;
      Ws[lk + i][lr] = (wr < N && k < K) ? ld_f(W + (int64_t)wr * ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][tr + i]; w[i] = Ws[k][tc + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + tr + i;
    if (r >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tc + j;
      if (c >= N) continue;
      float v = acc[i][j];
      if (act == NVC_ACT_RELU2) { v = fmaxf(v, 0.f); v *= v; }
      else if (act == NVC_ACT_GELU_TANH) v = gelu_tanh_f32(v);
      st_f(C + (int64_t)r * ldc + c, v);
    }
  }
}

// ---- bf16 on the tensor pipe: 64 x 64 tile, 4 warps of 32 x 32, k-slices of 32 --------------------------------------
constexpr int MK = 32;                 // k per stage
constexpr int MROW = (MK + 8) * 2;     // bytes per padded smem row (80: the 8 rows of an ldmatrix hit 8 different 16-byte segments)

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// BT x BT output tile, 2 * BT threads: BT / 32 x 2 warps of 32 x BT / 2
template <typename TC, int BT>
__global__ void __launch_bounds__(2 * BT)
linear_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, int64_t sa, const int32_t* __restrict__ a_rows,
                  const __nv_bfloat16* __restrict__ W, int ldw, int64_t sw, TC* __restrict__ C, int ldc, int64_t sc,
                  const int32_t* __restrict__ offsets, int groups, int M, int N, int K, int act) {
  __shared__ __align__(128) uint8_t sA[2][BT * MROW];
  __shared__ __align__(128) uint8_t sW[2][BT * MROW];
  pdl_trigger();
  pdl_wait();
  int row0, row_end;
  if (offsets) {
    int t = blockIdx.x, g = 0, base = 0;
    for (; g < groups; ++g) {
      base = offsets[g];
      const int tiles = (offsets[g + 1] - base + BT - 1) / BT;
      if (t < tiles) break;
      t -= tiles;
    }
    if (g == groups) return;
    row0 = base + t * BT;
    row_end = offsets[g + 1];
    W += (int64_t)g * sw;
  } else {
    row0 = blockIdx.x * BT;
    row_end = M;
    A += (int64_t)blockIdx.z * sa;
    W += (int64_t)blockIdx.z * sw;
    C += (int64_t)blockIdx.z * sc;
  }
  const int col0 = blockIdx.y * BT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int WNT = BT / 2, NP = WNT / 16, NT = WNT / 8;   // warp tile 32 x WNT
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * WNT;
  // loader: BT rows x 4 chunks of 16 bytes per operand and stage; thread -> rows (tid / 4) and (tid / 4 + BT / 2), chunk tid % 4
  const int lc = tid & 3;
  const __nv_bfloat16* a_src[2];
  const __nv_bfloat16* w_src[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (tid >> 2) + (BT / 2) * i;
    const int ar = row0 + r;
    a_src[i] = ar < row_end ? A + (int64_t)(a_rows ? a_rows[ar] : ar) * lda : nullptr;
    w_src[i] = col0 + r < N ? W + (int64_t)(col0 + r) * ldw : nullptr;
  }
  auto load = [&](int kb, int stage) {
    const int k = kb * MK + lc * 8;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (tid >> 2) + (BT / 2) * i;
      const uint32_t off = r * MROW + lc * 16;
      // K is a multiple of 8: a chunk is inside the row or entirely past its end (zero-filled)
      cp16(smem_u32(sA[stage]) + off, a_src[i] && k < K ? (const void*)(a_src[i] + k) : (const void*)A, a_src[i] && k < K ? 16u : 0u);
      cp16(smem_u32(sW[stage]) + off, w_src[i] && k < K ? (const void*)(w_src[i] + k) : (const void*)W, w_src[i] && k < K ? 16u : 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[2][NT][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  const int nkb = (K + MK - 1) / MK;
  load(0, 0);
  for (int kb = 0; kb < nkb; ++kb) {
    if (kb + 1 < nkb) load(kb + 1, (kb + 1) & 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const uint32_t a_base = smem_u32(sA[kb & 1]), w_base = smem_u32(sW[kb & 1]);
#pragma unroll
    for (int ks = 0; ks < MK / 16; ++ks) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldsm4(a_base + (wm + mt * 16 + (lane & 15)) * MROW + (ks * 2 + (lane >> 4)) * 16, af[mt][0], af[mt][1], af[mt][2], af[mt][3]);
#pragma unroll
      for (int np = 0; np < NP; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm4(w_base + (wn + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * MROW + (ks * 2 + ((lane >> 3) & 1)) * 16, b0, b1, b2, b3);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma16816(acc[mt][2 * np], af[mt], b0, b1);
          mma16816(acc[mt][2 * np + 1], af[mt], b2, b3);
        }
      }
    }
    __syncthreads();
  }
  const int quad = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = row0 + wm + mt * 16 + quad + 8 * hf;
      if (r >= row_end) continue;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int c = col0 + wn + nt * 8 + 2 * tq;
        float v0 = acc[mt][nt][2 * hf], v1 = acc[mt][nt][2 * hf + 1];
        if (act == NVC_ACT_RELU2) { v0 = fmaxf(v0, 0.f); v0 *= v0; v1 = fmaxf(v1, 0.f); v1 *= v1; }
        else if (act == NVC_ACT_GELU_TANH) { v0 = gelu_tanh_f32(v0); v1 = gelu_tanh_f32(v1); }
        TC* dst = C + (int64_t)r * ldc + c;
        if (c + 1 < N && (reinterpret_cast<uintptr_t>(dst) % (2 * sizeof(TC))) == 0) {     // the pair in one store
          if constexpr (sizeof(TC) == 2) *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v0, v1);
          else *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
        } else {
          if (c < N) st_f(dst, v0);
          if (c + 1 < N) st_f(dst + 1, v1);
        }
      }
    }
}

bool mma_ok(int in_dtype, const void* A, int lda, int64_t sa, const void* W, int ldw, int64_t sw, int K) {
  static const bool env = !(getenv("NVC_LINEAR_MMA") && atoi(getenv("NVC_LINEAR_MMA")) == 0);
  return env && in_dtype == NVC_DT_BF16 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && sa % 8 == 0 && sw % 8 == 0 &&
         ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0;
}

template <typename TC, int BT>
int launch_mma_t(nvc_ctx* ctx, dim3 grid, void* stream, const void* A, int lda, int64_t sa, const int32_t* a_rows, const void* W, int ldw,
                 int64_t sw, void* C, int ldc, int64_t sc, const int32_t* offsets, int groups, int M, int N, int K, int act) {
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, linear_mma_kernel<TC, BT>, grid, dim3(2 * BT), 0, nvc_stream(stream),
                                 reinterpret_cast<const __nv_bfloat16*>(A), lda, sa, a_rows, reinterpret_cast<const __nv_bfloat16*>(W), ldw,
                                 sw, reinterpret_cast<TC*>(C), ldc, sc, offsets, groups, M, N, K, act));
  ctx->launches++;
  return NVC_OK;
}

// 128 x 128 tiles when there are enough rows and columns to fill the GPU with them (prefill-sized products), else 64 x 64;
// `batch` is the z extent of a plain / batched launch (1 for a grouped one)
template <typename TC>
int launch_mma(nvc_ctx* ctx, int batch, void* stream, const void* A, int lda, int64_t sa, const int32_t* a_rows, const void* W, int ldw,
               int64_t sw, void* C, int ldc, int64_t sc, const int32_t* offsets, int groups, int M, int N, int K, int act) {
  const bool big = N >= 128 && (int64_t)(M / 128 + groups) * ((N + 127) / 128) * batch >= ctx->num_sms;
  const int BT = big ? 128 : 64;
  const int mt = offsets ? M / BT + groups : (M + BT - 1) / BT;     // grouped: every group may end with a partial tile
  const dim3 grid(mt, (N + BT - 1) / BT, batch);
  if (big) return launch_mma_t<TC, 128>(ctx, grid, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K, act);
  return launch_mma_t<TC, 64>(ctx, grid, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K, act);
}

template <typename T, typename TC>
int launch(nvc_ctx* ctx, dim3 grid, void* stream, const void* A, int lda, int64_t sa, const int32_t* a_rows, const void* W, int ldw,
           int64_t sw, void* C, int ldc, int64_t sc, const int32_t* offsets, int groups, int M, int N, int K, int act) {
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, linear_kernel<T, TC>, grid, dim3(256), 0, nvc_stream(stream), reinterpret_cast<const T*>(A), lda,
                                 sa, a_rows, reinterpret_cast<const T*>(W), ldw, sw, reinterpret_cast<TC*>(C), ldc, sc, offsets, groups,
                                 M, N, K, act));
  ctx->launches++;
  return NVC_OK;
}

int dispatch(nvc_ctx* ctx, dim3 grid, void* stream, int in_dtype, int out_dtype, const void* A, int lda, int64_t sa,
             const int32_t* a_rows, const void* W, int ldw, int64_t sw, void* C, int ldc, int64_t sc, const int32_t* offsets,
             int groups, int M, int N, int K, int act) {
  if (mma_ok(in_dtype, A, lda, sa, W, ldw, sw, K)) {
    if (out_dtype == NVC_DT_F32)
      return launch_mma<float>(ctx, (int)grid.z, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K, act);
    return launch_mma<__nv_bfloat16>(ctx, (int)grid.z, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K, act);
  }
  if (in_dtype == NVC_DT_F32) {
    NVC_REQUIRE(ctx, out_dtype == NVC_DT_F32, NVC_EINVAL, "fp32 operands give an fp32 result");
    return launch<float, float>(ctx, grid, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K, act);
  }
  if (out_dtype == NVC_DT_F32)
    return launch<__nv_bfloat16, float>(ctx, grid, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K, act);
  return launch<__nv_bfloat16, __nv_bfloat16>(ctx, grid, stream, A, lda, sa, a_rows, W, ldw, sw, C, ldc, sc, offsets, groups, M, N, K,
                                              act);
}

}  // namespace

extern "C" {

int nvc_linear(nvc_ctx* ctx, const void* A, int lda, int64_t sa, const void* W, int ldw, int64_t sw, void* C, int ldc, int64_t sc,
               int in_dtype, int out_dtype, int M, int N, int K, int batch, int act, void* stream) {
  NVC_REQUIRE(ctx, ctx && A && W && C, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, M >= 0 && N > 0 && K > 0 && batch > 0 && batch <= 65535 && lda >= K && ldw >= K && ldc >= N, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, act == NVC_ACT_NONE || act == NVC_ACT_RELU2 || act == NVC_ACT_GELU_TANH, NVC_EINVAL, "bad activation");
  if (M == 0) return NVC_OK;
  return dispatch(ctx, dim3((M + TM - 1) / TM, (N + TN - 1) / TN, batch), stream, in_dtype, out_dtype, A, lda, sa, nullptr, W, ldw, sw,
                  C, ldc, sc, nullptr, 0, M, N, K, act);
}

int nvc_linear_grouped(nvc_ctx* ctx, const void* A, int lda, const int32_t* a_rows, const void* W, int ldw, int64_t sw, void* C,
                       int ldc, const int32_t* offsets, int groups, int max_rows, int in_dtype, int out_dtype, int N, int K, int act,
                       void* stream) {
  NVC_REQUIRE(ctx, ctx && A && W && C && offsets, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, max_rows >= 0 && groups > 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, act == NVC_ACT_NONE || act == NVC_ACT_RELU2 || act == NVC_ACT_GELU_TANH, NVC_EINVAL, "bad activation");
  if (max_rows == 0) return NVC_OK;
  // every group may end with a partial tile: at most max_rows / TM + groups tiles exist
  const int tiles = max_rows / TM + groups;
  return dispatch(ctx, dim3(tiles, (N + TN - 1) / TN, 1), stream, in_dtype, out_dtype, A, lda, 0, a_rows, W, ldw, sw, C, ldc, 0, offsets,
                  groups, max_rows, N, K, act);
}

}  // extern "C"
