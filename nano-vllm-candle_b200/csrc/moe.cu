// Mixture-of-experts routing around the grouped matrix products (linear_generic.cu, moe_gemm): everything is sized
// by device-resident counts, so a step needs no host round trip and replays inside a CUDA graph.
//   nvc_moe_route    router logits in fp32, sigmoid scores, biased top-k choice, normalised weights, shared-expert gate
//   nvc_moe_sort     counting sort of the (token, choice) pairs by expert: group offsets, source rows, positions
//   nvc_moe_combine  weighted sum of a token's expert rows plus the gated shared expert, fp32
#include "typed.cuh"

namespace {

// one warp per token.  Scores of up to 32 * kPerLane experts live in registers.
constexpr int kMaxPerLane = 8;   // experts <= 256

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
  float s[kMaxPerLane], c[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    s[i] = 0.f;
    c[i] = -INFINITY;
    if (e < E) {
      float z = 0.f;
      const float* w = wr + (int64_t)e * H;
      for (int j = 0; j < H; ++j) z = fmaf(x[j], __ldg(w + j), z);
      s[i] = sigmoid_f32(z);
      c[i] = s[i] + __ldg(corr + e);
    }
  }
  if (wsg && gate) {
    float z = 0.f;
    for (int j = lane; j < H; j += 32) z = fmaf(x[j], __ldg(wsg + j), z);
    z = warp_sum(z);
    if (lane == 0) gate[n] = sigmoid_f32(z);
  }
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
  const float inv = scale / (sel_sum + 1e-20f);
  for (int t = lane; t < top; t += 32) wout[(int64_t)n * top + t] *= inv;
}

// Counting sort by expert in one CTA (pairs = N * top).  Within an expert the pairs keep token order, so the
// layout - and with it every sum downstream - does not depend on thread timing.
__global__ void moe_sort_kernel(const int32_t* __restrict__ idx, int P, int top, int E, int32_t* __restrict__ offsets,
                                int32_t* __restrict__ src_rows, int32_t* __restrict__ pos) {
  extern __shared__ int32_t sm[];   // [E] counts, then [E + 1] offsets
  int32_t* cnt = sm;
  int32_t* off = sm + E;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0;
    for (int e = 0; e < E; ++e) { off[e] = a; a += cnt[e]; }
    off[E] = a;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  // expert e is filled by one warp at a time walking the pairs in order: stable
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int e = warp; e < E; e += warps) {
    int fill = off[e];
    for (int p0 = 0; p0 < P; p0 += 32) {
      const int p = p0 + lane;
      const bool mine = p < P && idx[p] == e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int at = fill + __popc(m & ((1u << lane) - 1));
        src_rows[at] = p / top;
        pos[p] = at;
      }
      fill += __popc(m);
    }
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

int nvc_moe_sort(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int32_t* offsets, int32_t* src_rows, int32_t* pos,
                 void* stream) {
  NVC_REQUIRE(ctx, ctx && topk_idx && offsets && src_rows && pos, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && top > 0 && E > 0 && E <= 4096, NVC_EINVAL, "bad sizes");
  NVC_CUDA_CHECK(ctx, nvc_launch(ctx, moe_sort_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int32_t), nvc_stream(stream),
                                 topk_idx, N * top, top, E, offsets, src_rows, pos));
  ctx->launches++;
  return NVC_OK;
}

int nvc_moe_combine(nvc_ctx* ctx, const void* y, int y_dtype, int ldy, const int32_t* pos, const float* topk_w, int top,
                    const void* shared, int shared_dtype, int lds, const float* gate, float* out, int ldo, int N, int H,
                    void* stream) {
  NVC_REQUIRE(ctx, ctx && y && pos && topk_w && out, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, N >= 0 && H > 0 && top > 0 && ldy >= H && ldo >= H && (!shared || lds >= H), NVC_EINVAL, "bad sizes");
  if (N == 0) return NVC_OK;
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

}  // extern "C"
