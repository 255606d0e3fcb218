// C = act(A . W^T) for any sizes and both storage formats, on the fp32 FMA pipe (plain IEEE products and sums:
// this is the matrix product of the exact fp32 mode, and of bf16 shapes the tcgen05 kernels do not take).
// Three forms share one kernel:
//   plain      C[M, N] = A[M, K] . W[N, K]^T
//   batched    blockIdx.z = b: A + b * sa, W + b * sw, C + b * sc  (one small product per attention head)
//   grouped    rows [offsets[g], offsets[g + 1]) of C use W + g * sw; row r of A is a_rows[r] (mixture of experts:
//              the rows of one expert are contiguous after the sort, offsets live in device memory)
// 64 x 64 output tile per CTA, 16-deep k-slices through shared memory, 4 x 4 outputs per thread.
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
      st_f(C + (int64_t)r * ldc + c, v);
    }
  }
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
  NVC_REQUIRE(ctx, act == NVC_ACT_NONE || act == NVC_ACT_RELU2, NVC_EINVAL, "bad activation");
  if (M == 0) return NVC_OK;
  return dispatch(ctx, dim3((M + TM - 1) / TM, (N + TN - 1) / TN, batch), stream, in_dtype, out_dtype, A, lda, sa, nullptr, W, ldw, sw,
                  C, ldc, sc, nullptr, 0, M, N, K, act);
}

int nvc_linear_grouped(nvc_ctx* ctx, const void* A, int lda, const int32_t* a_rows, const void* W, int ldw, int64_t sw, void* C,
                       int ldc, const int32_t* offsets, int groups, int max_rows, int in_dtype, int out_dtype, int N, int K, int act,
                       void* stream) {
  NVC_REQUIRE(ctx, ctx && A && W && C && offsets, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, max_rows >= 0 && groups > 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, act == NVC_ACT_NONE || act == NVC_ACT_RELU2, NVC_EINVAL, "bad activation");
  if (max_rows == 0) return NVC_OK;
  // every group may end with a partial tile: at most max_rows / TM + groups tiles exist
  const int tiles = max_rows / TM + groups;
  return dispatch(ctx, dim3(tiles, (N + TN - 1) / TN, 1), stream, in_dtype, out_dtype, A, lda, 0, a_rows, W, ldw, sw, C, ldc, 0, offsets,
                  groups, max_rows, N, K, act);
}

}  // extern "C"
