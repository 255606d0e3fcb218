// Latent attention over a paged cache of shared latents (multi-head latent attention in its absorbed form, without a
// positional part): every head of a token scores the SAME cached row c_j of D numbers and sums the SAME rows,
//   out[i, h, :] = sum_{j <= pos_i} softmax_j(scale * q[i, h, :] . c_j) * c_j ,
// where q has already been carried into the latent space by the key up-projection and the caller applies the value
// up-projection to `out`.  One cache row per token serves keys and values of all heads.
// A sequence contributes q_len >= 1 query tokens that are the LAST positions of its context (q_len = 1: decode; more: a
// prompt or a portion of one behind an already cached prefix); all sequences of a step run in one launch.
//
// nvc_latent_attn_paged: the tensor-pipe kernel (latent_attn_mma.cuh) for bf16 rows of 64 or 128 numbers, else the fp32 FMA
// kernel below (the exact mode, and any other width).
#include <algorithm>
#include <cstdlib>

#include "typed.cuh"
#include "latent_attn_mma.cuh"

namespace {

constexpr int kKeys = 32;      // keys per shared-memory tile: one per lane
constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 4;
constexpr int kRows = kRowsPerWarp * kWarps;   // query rows (token, head) per CTA
constexpr int kMaxDPerLane = 16;               // D <= 512

template <typename T>
__global__ void __launch_bounds__(32 * kWarps)
latent_attn_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ cache, int ldc, const int32_t* __restrict__ block_tables,
                   int bt_stride, const int32_t* __restrict__ context_lens, const int32_t* __restrict__ cu_seqlens, int heads, int D,
                   int head_stride, int block_size, float scale, T* __restrict__ out, int ldo) {
  extern __shared__ float sm[];
  const int Dp = D + 1;                 // padded row: lane l reads row l, bank (l * Dp + d) % 32 differs per lane
  float* ks = sm;                       // [kKeys][Dp]
  float* qs = sm + kKeys * Dp;          // [kRows][D]
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int row_begin = cu_seqlens ? cu_seqlens[b] : b;
  const int qlen = cu_seqlens ? cu_seqlens[b + 1] - row_begin : 1;
  const int r0 = blockIdx.x * kRows;    // first (token, head) row of this CTA within the sequence
  if (r0 >= qlen * heads) return;
  const int ctx = context_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nrows = min(kRows, qlen * heads - r0);
  // the queries, pre-multiplied by the scale
  for (int i = threadIdx.x; i < nrows * D; i += blockDim.x) {
    const int r = r0 + i / D, d = i % D;
    const int t = r / heads, h = r % heads;
    qs[(i / D) * D + d] = ld_f(q + (int64_t)(row_begin + t) * ldq + (int64_t)h * head_stride + d) * scale;
  }
  const int last_tok = (r0 + nrows - 1) / heads;
  const int max_pos = ctx - qlen + last_tok;             // the farthest key any row of the CTA sees
  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][kMaxDPerLane];
  int pos[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
    const int r = warp * kRowsPerWarp + i;
    pos[i] = r < nrows ? ctx - qlen + (r0 + r) / heads : -1;
#pragma unroll
    for (int k = 0; k < kMaxDPerLane; ++k) acc[i][k] = 0.f;
  }
  const int32_t* bt = block_tables + (int64_t)b * bt_stride;
  for (int j0 = 0; j0 <= max_pos; j0 += kKeys) {
    __syncthreads();
    const int nk = min(kKeys, max_pos + 1 - j0);
    for (int i = threadIdx.x; i < nk * D; i += blockDim.x) {
      const int j = j0 + i / D, d = i % D;
      const int64_t slot = (int64_t)bt[j / block_size] * block_size + j % block_size;
      ks[(i / D) * Dp + d] = ld_f(cache + slot * ldc + d);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      if (pos[i] < j0) continue;                          // warp-uniform: nothing of this tile is visible
      const float* qr = qs + (warp * kRowsPerWarp + i) * D;
      const float* kr = ks + lane * Dp;
      float s = 0.f;
      if (lane < nk)
        for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      const bool vis = lane < nk && j0 + lane <= pos[i];
      s = vis ? s : -INFINITY;
      const float mn = fmaxf(m[i], warp_max(s));
      const float p = vis ? expf(s - mn) : 0.f;
      const float corr = expf(m[i] - mn);                 // first tile: exp(-inf) = 0
      l[i] = l[i] * corr + warp_sum(p);
      m[i] = mn;
#pragma unroll
      for (int k = 0; k < kMaxDPerLane; ++k) acc[i][k] *= corr;
      for (int jj = 0; jj < nk; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const float* kj = ks + jj * Dp;
#pragma unroll
        for (int k = 0; k < kMaxDPerLane; ++k) {
          const int d = lane + 32 * k;
          if (d < D) acc[i][k] = fmaf(pj, kj[d], acc[i][k]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int r = warp * kRowsPerWarp + i;
    if (r >= nrows) continue;
    const int t = (r0 + r) / heads, h = (r0 + r) % heads;
    const float inv = 1.0f / l[i];
#pragma unroll
    for (int k = 0; k < kMaxDPerLane; ++k) {
      const int d = lane + 32 * k;
      if (d < D) st_f(out + (int64_t)(row_begin + t) * ldo + (int64_t)h * head_stride + d, acc[i][k] * inv);
    }
  }
}

}  // namespace

extern "C" int nvc_latent_attn_paged(nvc_ctx* ctx, const void* q, int ldq, const void* cache, int ldc, const int32_t* block_tables,
                                     int bt_stride, const int32_t* context_lens, const int32_t* cu_seqlens, int B, int max_qlen,
                                     int heads, int D, int head_stride, int block_size, float scale, void* out, int ldo, int dtype,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  NVC_REQUIRE(ctx, ctx && q && cache && block_tables && context_lens && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, B >= 0 && max_qlen > 0 && heads > 0 && D > 0 && block_size > 0 && bt_stride > 0, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, D <= 32 * kMaxDPerLane, NVC_ESHAPE, "latent size above 512");
  NVC_REQUIRE(ctx, head_stride >= D && ldq >= heads * head_stride && ldo >= heads * head_stride && ldc >= D, NVC_EINVAL, "bad strides");
  if (B == 0) return NVC_OK;
  static const bool mma_env = !(getenv("NVC_LATENT_ATTN_MMA") && atoi(getenv("NVC_LATENT_ATTN_MMA")) == 0);
  if (dtype == NVC_DT_BF16 && mma_env && (head_stride == 64 || head_stride == 128) && ldc >= head_stride && ldc % 8 == 0 &&
      ldq % 2 == 0 && ldo % 2 == 0 && ((uintptr_t)cache % 16) == 0 && ((uintptr_t)q % 4) == 0 && ((uintptr_t)out % 4) == 0) {
    // padding columns [D, head_stride) of q and of the cache rows are zero (the caller guarantees it)
    const int chunks = (int)(((size_t)max_qlen * heads + 15) / 16);
    // a decode launch that would leave most SMs idle splits every sequence's keys over several CTAs (partials in the
    // caller's workspace, merged by a second kernel)
    int S = 1;
    if (max_qlen == 1 && workspace && heads < 16 * latmma::kWarps) {     // (more heads: every warp owns a chunk, no split)
      S = std::min(8, std::max(1, (2 * ctx->num_sms) / (chunks * B)));
      while (S > 1 && (size_t)B * chunks * 16 * S * (2 + head_stride) * sizeof(float) > workspace_bytes) --S;
    }
    const dim3 grid(chunks, B, S);
    const float sl2 = scale * 1.4426950408889634f;
    float* part = reinterpret_cast<float*>(workspace);
    if (head_stride == 64) {
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, latmma::latent_attn_mma_kernel<64>, grid, dim3(latmma::kWarps * 32), latmma::smem_bytes<64>(),
                                     nvc_stream(stream), reinterpret_cast<const nvc_bf16*>(q), ldq, reinterpret_cast<const nvc_bf16*>(cache),
                                     ldc, block_tables, bt_stride, context_lens, cu_seqlens, heads, head_stride, block_size, sl2,
                                     reinterpret_cast<nvc_bf16*>(out), ldo, part, S));
      if (S > 1)
        NVC_CUDA_CHECK(ctx, nvc_launch(ctx, latmma::latent_attn_combine_kernel<64>, dim3(B * chunks * 16), dim3(64), 0, nvc_stream(stream),
                                       (const float*)part, S, chunks, cu_seqlens, heads, head_stride, reinterpret_cast<nvc_bf16*>(out), ldo));
    } else {
      NVC_CUDA_CHECK(ctx, nvc_launch(ctx, latmma::latent_attn_mma_kernel<128>, grid, dim3(latmma::kWarps * 32), latmma::smem_bytes<128>(),
                                     nvc_stream(stream), reinterpret_cast<const nvc_bf16*>(q), ldq, reinterpret_cast<const nvc_bf16*>(cache),
                                     ldc, block_tables, bt_stride, context_lens, cu_seqlens, heads, head_stride, block_size, sl2,
                                     reinterpret_cast<nvc_bf16*>(out), ldo, part, S));
      if (S > 1)
        NVC_CUDA_CHECK(ctx, nvc_launch(ctx, latmma::latent_attn_combine_kernel<128>, dim3(B * chunks * 16), dim3(128), 0, nvc_stream(stream),
                                       (const float*)part, S, chunks, cu_seqlens, heads, head_stride, reinterpret_cast<nvc_bf16*>(out), ldo));
    }
    if (S > 1) ctx->launches++;
    ctx->launches++;
    return NVC_OK;
  }
  const size_t smem = ((size_t)kKeys * (D + 1) + (size_t)kRows * D) * sizeof(float);
  const dim3 grid(((size_t)max_qlen * heads + kRows - 1) / kRows, B);
  NVC_DISPATCH_DT(dtype, T, {
    if (smem > 48 * 1024)
      NVC_CUDA_CHECK(ctx, cudaFuncSetAttribute(latent_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NVC_CUDA_CHECK(ctx, nvc_launch(ctx, latent_attn_kernel<T>, grid, dim3(32 * kWarps), smem, nvc_stream(stream),
                                   reinterpret_cast<const T*>(q), ldq, reinterpret_cast<const T*>(cache), ldc, block_tables, bt_stride,
                                   context_lens, cu_seqlens, heads, D, head_stride, block_size, scale, reinterpret_cast<T*>(out), ldo));
  });
  ctx->launches++;
  return NVC_OK;
}
