// What the model bodies behind the step executor share: number formats of checkpoint tensors, zeroed device allocations,
// matrices written into padded device layouts, the plain product (tcgen05 GEMM when it takes the shape, the generic kernel
// otherwise) and the per-op event profile of a step.
#pragma once
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "runner.h"

namespace {

inline int pad64(int v) { return (v + 63) / 64 * 64; }

inline float bf16_bits_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
inline float f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) { u = sign; }
    else { int e = -1; do { ++e; man <<= 1; } while (!(man & 0x400u)); u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13); }
  } else if (exp == 31) { u = sign | 0x7f800000u | (man << 13); }
  else { u = sign | ((exp + 112u) << 23) | (man << 13); }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// a checkpoint tensor (NVC_ST_*) as fp32; false for a format no body takes
inline bool tensor_to_f32(const void* data, int st_dtype, size_t n, std::vector<float>& v) {
  v.resize(n);
  if (st_dtype == NVC_ST_F32) { memcpy(v.data(), data, n * 4); return true; }
  if (st_dtype != NVC_ST_BF16 && st_dtype != NVC_ST_F16) return false;
  const uint16_t* s = reinterpret_cast<const uint16_t*>(data);
  for (size_t i = 0; i < n; ++i) {
    uint16_t b;
    memcpy(&b, s + i, 2);
    v[i] = st_dtype == NVC_ST_BF16 ? bf16_bits_to_f32(b) : f16_bits_to_f32(b);
  }
  return true;
}

struct nvc_body_base : nvc_model_body {
  int dt = NVC_DT_BF16;                // storage format of weights and activations
  size_t esz = 2;
  bool use_tc = true;                  // tcgen05 GEMMs for the plain products of the bf16 mode
  bool prof_armed = false, prof_on = false;
  std::vector<std::pair<const char*, cudaEvent_t>> marks;
  std::string prof_json = "{}";

  int arm_profile() override { prof_armed = true; return NVC_OK; }
  bool profile_armed() const override { return prof_armed; }
  const char* profile_json() const override { return prof_json.c_str(); }
  // names the op(s) launched since the previous mark
  void mark(nvc_runner* r, const char* name) {
    if (!prof_on) return;
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    cudaEventRecord(e, r->stream);
    marks.emplace_back(name, e);
  }
  void finish_profile(nvc_runner* r) {
    if (!prof_on) return;
    prof_on = false;
    cudaStreamSynchronize(r->stream);
    std::map<std::string, double> us;
    std::vector<std::string> order;
    for (size_t i = 1; i < marks.size(); ++i) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, marks[i - 1].second, marks[i].second);
      if (!us.count(marks[i].first)) order.push_back(marks[i].first);
      us[marks[i].first] += ms * 1e3;
    }
    for (auto& m : marks) cudaEventDestroy(m.second);
    marks.clear();
    prof_json = "{";
    for (size_t i = 0; i < order.size(); ++i)
      prof_json += (i ? ", \"" : "\"") + order[i] + "\": " + std::to_string(us[order[i]]);
    prof_json += "}";
  }

  template <typename P>
  int zalloc(nvc_runner* r, P** p, size_t bytes) {
    uint8_t* q = nullptr;
    int rc = dev_alloc_bytes(r, &q, bytes);
    if (rc) return rc;
    *p = reinterpret_cast<P*>(q);
    return NVC_OK;
  }
  int dev_alloc_bytes(nvc_runner* r, uint8_t** p, size_t bytes) {
    void* q = nullptr;
    bytes = std::max<size_t>(bytes, 256);
    NVC_CUDA_CHECK(r->ctx, cudaMalloc(&q, bytes));
    r->allocs.push_back(q);
    NVC_CUDA_CHECK(r->ctx, cudaMemset(q, 0, bytes));
    *p = reinterpret_cast<uint8_t*>(q);
    return NVC_OK;
  }

  // dst[(r0 + i) * ld + c0 + j] = src[i * scols + j] converted to the storage format (dst: device, T)
  int put_matrix(nvc_runner* r, void* dst, size_t ld, size_t r0, size_t c0, const float* src, size_t rows, size_t cols, size_t src_rs,
                 size_t src_cs) {
    std::vector<uint8_t> stage(rows * cols * esz);
    for (size_t i = 0; i < rows; ++i)
      for (size_t j = 0; j < cols; ++j) {
        const float v = src[i * src_rs + j * src_cs];
        if (dt == NVC_DT_F32) memcpy(&stage[(i * cols + j) * 4], &v, 4);
        else { const uint16_t b = f32_to_bf16_bits(v); memcpy(&stage[(i * cols + j) * 2], &b, 2); }
      }
    NVC_CUDA_CHECK(r->ctx, cudaMemcpy2D(reinterpret_cast<uint8_t*>(dst) + (r0 * ld + c0) * esz, ld * esz, stage.data(), cols * esz,
                                        cols * esz, rows, cudaMemcpyHostToDevice));
    return NVC_OK;
  }
  int put_f32(nvc_runner* r, float* dst, const float* src, size_t n) {
    NVC_CUDA_CHECK(r->ctx, cudaMemcpy(dst, src, n * 4, cudaMemcpyHostToDevice));
    return NVC_OK;
  }

  // C = A . W^T on padded shapes: the tcgen05 GEMM when it takes the shape, the FMA kernel otherwise
  int linear(nvc_runner* r, const void* A, int lda, const void* Wt, void* C, int ldc, int out_dt, int M, int N, int K, int act = NVC_ACT_NONE) {
    if (use_tc && act == NVC_ACT_NONE && K % 64 == 0 && N % 16 == 0 && lda % 8 == 0 && ldc % 8 == 0)
      return nvc_gemm_bf16(r->ctx, reinterpret_cast<const nvc_bf16*>(A), lda, reinterpret_cast<const nvc_bf16*>(Wt), C, ldc, out_dt, M, N, K,
                           r->stream);
    return nvc_linear(r->ctx, A, lda, 0, Wt, K, 0, C, ldc, 0, dt, dt == NVC_DT_F32 ? NVC_DT_F32 : out_dt, M, N, K, 1, act, r->stream);
  }
};

}  // namespace
