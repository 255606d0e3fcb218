// Latent attention on the tensor pipe (bf16 storage): 16 query rows - any (token, head) pairs of ONE sequence, each with
// its own causal bound - are the M dimension of mma.sync.m16n8k16, the shared latent row of a token is both the key (read
// with ldmatrix) and the value (the SAME shared-memory tile read with ldmatrix.trans), so one 16-token tile is loaded
// once for S = Q C^T and O += P C.  Online softmax in the log2 domain on the accumulator fragments, fp32 accumulators.
// Fewer than 64 rows (decode, q_len = 1: `heads` rows per sequence; short portions): the CTA's 4 warps work on one 16-row chunk, warp w owns the
// 16-token tiles w, w + 4, ... of the keys (private 3-stage cp.async ring, 16-byte-chunk XOR swizzle) and the warps meet once,
// in the final merge.  Many rows (a prompt portion, q_len * heads >= 64): the CTA takes 64 consecutive rows, 16 per warp,
// and all warps read the same 64-token tiles from one ring of the CTA.  Both in one launch, chosen per sequence.
// DP = padded latent width (64 or 128 numbers per row; padding columns of q and of the cache rows are zero).
#pragma once
#include "paged_decode_mma.cuh"

namespace latmma {

using pdmma::cp_async16;
using pdmma::cp_async_commit;
using pdmma::cp_async_wait;
using pdmma::fast_exp2;
using pdmma::ldmatrix_x4;
using pdmma::ldmatrix_x4_trans;
using pdmma::mma_bf16;

constexpr int kWarps = 4;
constexpr int kTileTok = 16;
constexpr int kStages = 3;
template <int DP> constexpr int stage_bytes() { return kTileTok * DP * 2; }
template <int DP> constexpr int smem_bytes() {
  return kWarps * kStages * stage_bytes<DP>() > (2 * kWarps * 16 + kWarps * 16 * DP) * 4 ? kWarps * kStages * stage_bytes<DP>()
                                                                                         : (2 * kWarps * 16 + kWarps * 16 * DP) * 4;
}

template <int DP>
__global__ void __launch_bounds__(kWarps * 32)
latent_attn_mma_kernel(const nvc_bf16* __restrict__ q, int ldq, const nvc_bf16* __restrict__ cache, int ldc,
                       const int32_t* __restrict__ block_tables, int bt_stride, const int32_t* __restrict__ context_lens,
                       const int32_t* __restrict__ cu_seqlens, int heads, int head_stride, int block_size, float scale_log2e,
                       nvc_bf16* __restrict__ out, int ldo, float* __restrict__ part, int num_splits) {
  constexpr int RB = DP * 2;               // bytes per latent row
  constexpr int NC = DP / 8;               // 16-byte chunks per row
  constexpr int KS = DP / 16;              // k-steps of S
  constexpr int NT = DP / 8;               // n-tiles of O
  constexpr int kCtaTok = kWarps * kTileTok;
  constexpr int kStageBytes = kTileTok * DP * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int row_begin = cu_seqlens ? cu_seqlens[b] : b;
  const int qlen = cu_seqlens ? cu_seqlens[b + 1] - row_begin : 1;
  const int total = qlen * heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, tq = lane & 3;
  const int ctx_len = context_lens[b];
  const int32_t* bt = block_tables + (int64_t)b * bt_stride;
  // Two ways to spend the four warps.  Many rows (a prompt portion): the CTA takes 64 consecutive rows, 16 per warp, and
  // walks their keys in 64-token tiles that the four warps share (one ring for the CTA, one barrier per tile, one softmax
  // update per 64 keys).  Few rows (decode: one chunk of `heads` rows per sequence): see below.
  if (total >= 16 * kWarps) {
    constexpr int kTileBytes = kCtaTok * RB;
    const int n64 = (total + 16 * kWarps - 1) / (16 * kWarps);
    if ((int)blockIdx.x >= n64 || blockIdx.z != 0) return;
    const int r0c = (n64 - 1 - (int)blockIdx.x) * (16 * kWarps);   // the rows with the most keys start first
    const int r0 = r0c + warp * 16;
    const int base = ctx_len - qlen;                               // token t of the portion sees keys 0 .. base + t
    const int ra = r0 + quad, rb = r0 + quad + 8;
    const bool va = ra < total, vb = rb < total;
    const int ta = va ? ra / heads : 0, tb = vb ? rb / heads : 0;
    const int ha = va ? ra - ta * heads : 0, hb = vb ? rb - tb * heads : 0;
    const int pa_ = va ? base + ta : -1, pb_ = vb ? base + tb : -1;
    const int kmax_cta = base + min(r0c + 16 * kWarps - 1, total - 1) / heads;
    const int kmax_w = r0 < total ? base + min(r0 + 15, total - 1) / heads : -1;   // a warp past the end only loads
    const int kmin_w = base + r0 / heads;                          // every valid row of the warp sees at least this far
    const int n_tiles = kmax_cta / kCtaTok + 1;
    const uint32_t ring = smem_u32(smem);
    auto issue = [&](int i) {
      if (i < n_tiles) {
        const int tok0 = i * kCtaTok;
        const uint32_t st = ring + (i % kStages) * kTileBytes;
#pragma unroll
        for (int k = 0; k < kCtaTok * NC / (kWarps * 32); ++k) {
          const int idx = k * (kWarps * 32) + threadIdx.x;
          const int r = idx / NC, c = idx % NC;
          const int tok = tok0 + r;
          const uint32_t ok = tok <= kmax_cta ? 16u : 0u;
          const int tk = ok ? tok : tok0;
          const int64_t slot = (int64_t)__ldg(bt + tk / block_size) * block_size + tk % block_size;
          cp_async16(st + r * RB + ((c ^ (r & 7)) << 4), reinterpret_cast<const uint8_t*>(cache + slot * ldc) + c * 16, ok);
        }
      }
      cp_async_commit();
    };
    issue(0);
    issue(1);
    uint32_t qa[KS][4];
    {
      const nvc_bf16* qrow0 = q + (int64_t)(row_begin + ta) * ldq + (int64_t)ha * head_stride;
      const nvc_bf16* qrow1 = q + (int64_t)(row_begin + tb) * ldq + (int64_t)hb * head_stride;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int d = ks * 16 + 2 * tq;
        qa[ks][0] = va ? __ldg(reinterpret_cast<const uint32_t*>(qrow0 + d)) : 0u;
        qa[ks][1] = vb ? __ldg(reinterpret_cast<const uint32_t*>(qrow1 + d)) : 0u;
        qa[ks][2] = va ? __ldg(reinterpret_cast<const uint32_t*>(qrow0 + d + 8)) : 0u;
        qa[ks][3] = vb ? __ldg(reinterpret_cast<const uint32_t*>(qrow1 + d + 8)) : 0u;
      }
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    for (int i = 0; i < n_tiles; ++i) {
      cp_async_wait<1>();                 // tile i has landed (tile i + 1 may be in flight)
      __syncthreads();                    // ... for every thread's part of it; and every warp is done with tile i - 1,
      issue(i + 2);                       // whose stage tile i + 2 takes
      const int tok0 = i * kCtaTok;
      if (tok0 > kmax_w) continue;        // warp-uniform: the later rows of the CTA see farther than this warp's
      const uint32_t st = ring + (i % kStages) * kTileBytes;
      const int nsub = min(kCtaTok / 16, (kmax_w - tok0) / 16 + 1);   // 16-token sub-tiles any row of the warp sees
      float s[kCtaTok / 8][4];
      {
        const int r = (lane & 7) + ((lane >> 4) << 3);
        const int chi = (lane >> 3) & 1;
#pragma unroll
        for (int j = 0; j < kCtaTok / 16; ++j) {
          s[2 * j][0] = s[2 * j][1] = s[2 * j][2] = s[2 * j][3] = 0.f;
          s[2 * j + 1][0] = s[2 * j + 1][1] = s[2 * j + 1][2] = s[2 * j + 1][3] = 0.f;
          if (j < nsub) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
              const int c = 2 * ks + chi;
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4(st + (j * 16 + r) * RB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
              mma_bf16(s[2 * j], qa[ks], b0, b1);
              mma_bf16(s[2 * j + 1], qa[ks], b2, b3);
            }
          }
        }
      }
      // ---- one online-softmax update for the 64 keys; columns tok0 + 8 jn + 2 tq + {0, 1}; row bounds pa_ / pb_
      float mx0 = -INFINITY, mx1 = -INFINITY;
      if (tok0 + kCtaTok - 1 <= kmin_w) {            // every row of the warp sees the whole tile
#pragma unroll
        for (int jn = 0; jn < kCtaTok / 8; ++jn) {
          s[jn][0] *= scale_log2e; s[jn][1] *= scale_log2e; s[jn][2] *= scale_log2e; s[jn][3] *= scale_log2e;
          mx0 = fmaxf(mx0, fmaxf(s[jn][0], s[jn][1]));
          mx1 = fmaxf(mx1, fmaxf(s[jn][2], s[jn][3]));
        }
      } else {
#pragma unroll
        for (int jn = 0; jn < kCtaTok / 8; ++jn) {
          const int t0 = tok0 + 8 * jn + 2 * tq;
          s[jn][0] = t0 <= pa_ ? s[jn][0] * scale_log2e : -INFINITY;
          s[jn][1] = t0 + 1 <= pa_ ? s[jn][1] * scale_log2e : -INFINITY;
          s[jn][2] = t0 <= pb_ ? s[jn][2] * scale_log2e : -INFINITY;
          s[jn][3] = t0 + 1 <= pb_ ? s[jn][3] * scale_log2e : -INFINITY;
          mx0 = fmaxf(mx0, fmaxf(s[jn][0], s[jn][1]));
          mx1 = fmaxf(mx1, fmaxf(s[jn][2], s[jn][3]));
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // a row that has seen no key yet keeps m = -inf: subtract 0 instead, every exponential below is then exp2(-inf) = 0
      const float mb0 = mn0 == -INFINITY ? 0.f : mn0, mb1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = fast_exp2(m0 - mb0), al1 = fast_exp2(m1 - mb1);
      m0 = mn0;
      m1 = mn1;
      uint32_t pa[kCtaTok / 16][4];
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int jn = 0; jn < kCtaTok / 8; ++jn) {
        const float p0 = fast_exp2(s[jn][0] - mb0), p1 = fast_exp2(s[jn][1] - mb0);
        const float p2 = fast_exp2(s[jn][2] - mb1), p3 = fast_exp2(s[jn][3] - mb1);
        ps0 += p0 + p1;
        ps1 += p2 + p3;
        pa[jn >> 1][2 * (jn & 1)] = pack_bf16(p0, p1);
        pa[jn >> 1][2 * (jn & 1) + 1] = pack_bf16(p2, p3);
      }
      l0 = l0 * al0 + ps0;
      l1 = l1 * al1 + ps1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        o[nt][0] *= al0; o[nt][1] *= al0;
        o[nt][2] *= al1; o[nt][3] *= al1;
      }
      // ---- O += P C: the same tile, transposed on the way out of shared memory
      {
        const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int cadd = lane >> 4;
#pragma unroll
        for (int j = 0; j < kCtaTok / 16; ++j) {
          if (j < nsub) {
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
              const int c = 2 * np + cadd;
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4_trans(st + (j * 16 + r) * RB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
              mma_bf16(o[2 * np], pa[j], b0, b1);
              mma_bf16(o[2 * np + 1], pa[j], b2, b3);
            }
          }
        }
      }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // ---- this warp's rows are complete: normalise and store the fragments (pairs of columns)
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    nvc_bf16* o0 = out + (int64_t)(row_begin + ta) * ldo + (int64_t)ha * head_stride;
    nvc_bf16* o1 = out + (int64_t)(row_begin + tb) * ldo + (int64_t)hb * head_stride;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int d = nt * 8 + 2 * tq;
      if (va) *reinterpret_cast<uint32_t*>(o0 + d) = pack_bf16(o[nt][0] * i0, o[nt][1] * i0);
      if (vb) *reinterpret_cast<uint32_t*>(o1 + d) = pack_bf16(o[nt][2] * i1, o[nt][3] * i1);
    }
    return;
  }
  // Few rows: the four warps split the KEYS of one 16-row chunk (warp w owns the 16-token tiles w, w + 4, ... in a
  // private ring) and merge at the end.
  const int chunk = blockIdx.x;
  const int r0 = chunk * 16;
  if (r0 >= total) return;                 // CTA-uniform
  // key split over CTAs (decode launches of small batches): CTA z takes the 64-token tiles z, z + S, z + 2S, ...
  const int S = num_splits, split = blockIdx.z;
  const int tile_stride = kCtaTok * S;
  const int tile_first = split * kCtaTok + warp * kTileTok;
  // rows of this thread's accumulator fragments
  const int ra = r0 + quad, rb = r0 + quad + 8;
  const bool va = ra < total, vb = rb < total;
  const int ta = va ? ra / heads : 0, tb = vb ? rb / heads : 0;
  const int ha = va ? ra - ta * heads : 0, hb = vb ? rb - tb * heads : 0;
  const int pa_ = va ? ctx_len - qlen + ta : -1, pb_ = vb ? ctx_len - qlen + tb : -1;   // last visible key
  const int last_row = min(r0 + 15, total - 1);
  const int kmax = ctx_len - qlen + last_row / heads;       // the farthest key any row of the chunk sees
  const int n_tiles = ((kmax + 1 + kCtaTok - 1) / kCtaTok - split + S - 1) / S;   // 64-token tiles of this split (may be <= 0)

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const uint32_t ring = smem_u32(smem) + warp * (kStages * kStageBytes);

  auto issue = [&](int i) {
    if (i < n_tiles) {
      const int tok0 = i * tile_stride + tile_first;
      if (tok0 <= kmax) {
        const uint32_t st = ring + (i % kStages) * kStageBytes;
        // 32 lanes cover 16 rows x NC chunks in 16 * NC / 32 rounds
        constexpr int kRowsPerRound = 32 / NC;       // NC = 8: 4 rows per round; NC = 16: 2 rows
        const int c = lane % NC;
        // tiles start at multiples of 16: with a block size that is a multiple of 16 a tile lies in one block
        const bool one_block = (block_size & 15) == 0;
        const int64_t slot0 = (int64_t)__ldg(bt + tok0 / block_size) * block_size + tok0 % block_size;
#pragma unroll
        for (int rr = 0; rr < 16 / kRowsPerRound; ++rr) {
          const int r = rr * kRowsPerRound + lane / NC;
          const int tok = tok0 + r;
          const uint32_t ok = tok <= kmax ? 16u : 0u;
          const int tk = ok ? tok : tok0;
          const int64_t slot = one_block ? slot0 + (tk - tok0) : (int64_t)__ldg(bt + tk / block_size) * block_size + tk % block_size;
          cp_async16(st + r * RB + ((c ^ (r & 7)) << 4), reinterpret_cast<const uint8_t*>(cache + slot * ldc) + c * 16, ok);
        }
      }
    }
    cp_async_commit();
  };
  issue(0);
  issue(1);
  // ---- Q as A fragments (rows past the chunk's end are zero)
  uint32_t qa[KS][4];
  {
    const nvc_bf16* qrow0 = q + (int64_t)(row_begin + ta) * ldq + (int64_t)ha * head_stride;
    const nvc_bf16* qrow1 = q + (int64_t)(row_begin + tb) * ldq + (int64_t)hb * head_stride;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + 2 * tq;
      qa[ks][0] = va ? __ldg(reinterpret_cast<const uint32_t*>(qrow0 + d)) : 0u;
      qa[ks][1] = vb ? __ldg(reinterpret_cast<const uint32_t*>(qrow1 + d)) : 0u;
      qa[ks][2] = va ? __ldg(reinterpret_cast<const uint32_t*>(qrow0 + d + 8)) : 0u;
      qa[ks][3] = vb ? __ldg(reinterpret_cast<const uint32_t*>(qrow1 + d + 8)) : 0u;
    }
  }
  for (int i = 0; i < n_tiles; ++i) {
    issue(i + 2);
    cp_async_wait<2>();
    __syncwarp();
    const int tok0 = i * tile_stride + tile_first;
    if (tok0 <= kmax) {                                // warp-uniform
      const uint32_t st = ring + (i % kStages) * kStageBytes;
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      {
        const int r = (lane & 7) + ((lane >> 4) << 3);
        const int chi = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int c = 2 * ks + chi;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(st + r * RB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
          mma_bf16(s[0], qa[ks], b0, b1);
          mma_bf16(s[1], qa[ks], b2, b3);
        }
      }
      // ---- online softmax; columns tok0 + 8j + 2tq + {0, 1}; row bounds pa_ / pb_
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int t0 = tok0 + 8 * j + 2 * tq;
        s[j][0] = t0 <= pa_ ? s[j][0] * scale_log2e : -INFINITY;
        s[j][1] = t0 + 1 <= pa_ ? s[j][1] * scale_log2e : -INFINITY;
        s[j][2] = t0 <= pb_ ? s[j][2] * scale_log2e : -INFINITY;
        s[j][3] = t0 + 1 <= pb_ ? s[j][3] * scale_log2e : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // a row that has seen no key yet keeps m = -inf: subtract 0 instead, every exponential below is then exp2(-inf) = 0
      const float mb0 = mn0 == -INFINITY ? 0.f : mn0, mb1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = fast_exp2(m0 - mb0), al1 = fast_exp2(m1 - mb1);
      m0 = mn0;
      m1 = mn1;
      uint32_t pa[4];
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = fast_exp2(s[j][0] - mb0), p1 = fast_exp2(s[j][1] - mb0);
        const float p2 = fast_exp2(s[j][2] - mb1), p3 = fast_exp2(s[j][3] - mb1);
        ps0 += p0 + p1;
        ps1 += p2 + p3;
        pa[2 * j] = pack_bf16(p0, p1);
        pa[2 * j + 1] = pack_bf16(p2, p3);
      }
      l0 = l0 * al0 + ps0;
      l1 = l1 * al1 + ps1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        o[nt][0] *= al0; o[nt][1] *= al0;
        o[nt][2] *= al1; o[nt][3] *= al1;
      }
      // ---- O += P C: the same tile, transposed on the way out of shared memory
      {
        const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int cadd = lane >> 4;
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          const int c = 2 * np + cadd;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(st + r * RB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
          mma_bf16(o[2 * np], pa, b0, b1);
          mma_bf16(o[2 * np + 1], pa, b2, b3);
        }
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // ---- merge the warps (the rings are dead now)
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(smem);       // [kWarps][16]
  float* sm_l = sm_m + kWarps * 16;
  float* sm_o = sm_l + kWarps * 16;                   // [kWarps][16][DP]
  if (tq == 0) {
    sm_m[warp * 16 + quad] = m0;
    sm_m[warp * 16 + quad + 8] = m1;
    sm_l[warp * 16 + quad] = l0;
    sm_l[warp * 16 + quad + 8] = l1;
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int d = nt * 8 + 2 * tq;
    float* p0 = sm_o + (warp * 16 + quad) * DP + d;
    float* p1 = sm_o + (warp * 16 + quad + 8) * DP + d;
    p0[0] = o[nt][0]; p0[1] = o[nt][1];
    p1[0] = o[nt][2]; p1[1] = o[nt][3];
  }
  __syncthreads();
  const int nrows = min(16, total - r0);
  for (int idx = threadIdx.x; idx < nrows * DP; idx += kWarps * 32) {
    const int g = idx / DP, d = idx % DP;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sm_m[w * 16 + g]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_m[w * 16 + g];
      const float wt = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      L += sm_l[w * 16 + g] * wt;
      O += sm_o[(w * 16 + g) * DP + d] * wt;
    }
    if (S == 1) {
      const int rr = r0 + g, t = rr / heads, h = rr - t * heads;
      out[(int64_t)(row_begin + t) * ldo + (int64_t)h * head_stride + d] = __bfloat16_as_ushort(__float2bfloat16_rn(L > 0.f ? O / L : 0.f));
    } else {
      // partial (max, sum, un-normalised row) of this split: [b][chunk][row][split][2 + DP]
      float* p = part + ((((int64_t)b * gridDim.x + chunk) * 16 + g) * S + split) * (2 + DP);
      if (d == 0) { __stcg(p, M); __stcg(p + 1, L); }
      __stcg(p + 2 + d, O);
    }
  }
}

// merges the splits of every row: out = sum_s O_s 2^(M_s - M) / sum_s L_s 2^(M_s - M)
template <int DP>
__global__ void latent_attn_combine_kernel(const float* __restrict__ part, int S, int chunks, const int32_t* __restrict__ cu_seqlens,
                                           int heads, int head_stride, nvc_bf16* __restrict__ out, int ldo) {
  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.x & 15, chunk = (blockIdx.x >> 4) % chunks, b = (blockIdx.x >> 4) / chunks;
  const int row_begin = cu_seqlens ? cu_seqlens[b] : b;
  const int qlen = cu_seqlens ? cu_seqlens[b + 1] - row_begin : 1;
  const int rr = chunk * 16 + g;
  if (rr >= qlen * heads) return;
  const float* p = part + (((int64_t)b * chunks + chunk) * 16 + g) * S * (2 + DP);
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, p[s * (2 + DP)]);
  const int t = rr / heads, h = rr - t * heads;
  for (int d = threadIdx.x; d < DP; d += blockDim.x) {
    float L = 0.f, O = 0.f;
    for (int s = 0; s < S; ++s) {
      const float ms = p[s * (2 + DP)];
      const float wt = ms == -INFINITY ? 0.f : fast_exp2(ms - M);
      L += p[s * (2 + DP) + 1] * wt;
      O += p[s * (2 + DP) + 2 + d] * wt;
    }
    out[(int64_t)(row_begin + t) * ldo + (int64_t)h * head_stride + d] = __bfloat16_as_ushort(__float2bfloat16_rn(L > 0.f ? O / L : 0.f));
  }
}

}  // namespace latmma
