// nvc_retention_scan: linear attention with a fixed decay per head and no softmax or denominator,
//   S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
// over the new tokens of every sequence of a step, token by token.  The state S [dim, vdim] of every (sequence, head) lives in
// fp32 in a pool of state slots: a sequence whose first new token sits at position 0 starts from zeros, every other one from what
// its slot holds, and the slot is written back after the last token.  q, k, v, o are fp32 rows (the caller has already rotated q and
// k and scaled k).
//
// One CTA per (sequence, head, slice of 32 value columns): thread (column v, row group r) keeps rows [r DPT, (r + 1) DPT) of column v
// in registers; a token costs 2 DPT FMAs per thread and, when the rows are split, one shared-memory reduction.  The next token's q / k / v
// are fetched while the current one is computed.
#include "typed.cuh"

namespace {

struct RetArgs {
  const float *q, *k, *v;
  float* o;
  int ldq, ldk, ldv, ldo;
  float* state;                  // [slots, heads, dim, vdim]
  const int32_t *state_slots, *cu_seqlens, *positions;
  const float* decay;            // [heads]
  int heads, dim, vdim;
};

template <int DPT>
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
  const float dec = __ldg(a.decay + h);
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
    q_s[d] = a.q[(int64_t)r0 * a.ldq + h * a.dim + d];
    k_s[d] = a.k[(int64_t)r0 * a.ldk + h * a.dim + d];
  }
  float vt = vok ? a.v[(int64_t)r0 * a.ldv + h * a.vdim + v] : 0.f;
  __syncthreads();
  for (int t = r0; t < r1; ++t) {
    const int cur = (t - r0) & 1;
    const float* qc = q_s + cur * a.dim;
    const float* kc = k_s + cur * a.dim;
    float vn = 0.f;
    if (t + 1 < r1) {       // fetch the next token into the other buffer
      for (int d = threadIdx.x; d < a.dim; d += blockDim.x) {
        q_s[(cur ^ 1) * a.dim + d] = a.q[(int64_t)(t + 1) * a.ldq + h * a.dim + d];
        k_s[(cur ^ 1) * a.dim + d] = a.k[(int64_t)(t + 1) * a.ldk + h * a.dim + d];
      }
      vn = vok ? a.v[(int64_t)(t + 1) * a.ldv + h * a.vdim + v] : 0.f;
    }
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
        if (vok) a.o[(int64_t)t * a.ldo + h * a.vdim + v] = s;
      }
    } else if (vok) {
      a.o[(int64_t)t * a.ldo + h * a.vdim + v] = acc;
    }
    vt = vn;
    __syncthreads();
  }
  if (vok)
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < a.dim) sp[(int64_t)(d0 + i) * a.vdim + v] = S[i];
}

}  // namespace

extern "C" int nvc_retention_scan(nvc_ctx* ctx, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, float* o, int ldo,
                                  float* state, const int32_t* state_slots, const int32_t* cu_seqlens, const int32_t* positions,
                                  const float* decay, int B, int heads, int dim, int vdim, void* stream) {
  NVC_REQUIRE(ctx, ctx && q && k && v && o && state && state_slots && positions && decay, NVC_EINVAL, "null pointer");
  NVC_REQUIRE(ctx, B > 0 && heads > 0 && dim > 0 && vdim > 0 && dim <= 1024 && heads <= 65535, NVC_EINVAL, "bad sizes");
  NVC_REQUIRE(ctx, ldq >= heads * dim && ldk >= heads * dim && ldv >= heads * vdim && ldo >= heads * vdim, NVC_EINVAL, "bad strides");
  RetArgs a{q, k, v, o, ldq, ldk, ldv, ldo, state, state_slots, cu_seqlens, positions, decay, heads, dim, vdim};
  const int dpt = dim <= 16 ? 16 : (dim <= 32 ? 32 : (dim <= 64 ? 64 : 128));
  const int groups = (dim + dpt - 1) / dpt;
  const dim3 grid(B, heads, (vdim + 31) / 32), block(32 * groups);
  const size_t smem = ((size_t)4 * dim + (size_t)groups * 32) * sizeof(float);
  cudaError_t ce;
  switch (dpt) {
    case 16: ce = nvc_launch(ctx, retention_scan_kernel<16>, grid, block, smem, nvc_stream(stream), a); break;
    case 32: ce = nvc_launch(ctx, retention_scan_kernel<32>, grid, block, smem, nvc_stream(stream), a); break;
    case 64: ce = nvc_launch(ctx, retention_scan_kernel<64>, grid, block, smem, nvc_stream(stream), a); break;
    default: ce = nvc_launch(ctx, retention_scan_kernel<128>, grid, block, smem, nvc_stream(stream), a); break;
  }
  NVC_CUDA_CHECK(ctx, ce);
  ctx->launches++;
  return NVC_OK;
}
