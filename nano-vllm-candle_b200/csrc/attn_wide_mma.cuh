// Tensor-pipe kernel of nvc_attn_paged_wide (bf16 storage): declared here, included by attn_wide.cu only.
#pragma once
#include "typed.cuh"

namespace {

inline bool attn_wide_mma_takes(const nvc_attn_spec&, int, int, int, int, int) { return false; }

inline int attn_wide_mma_launch(nvc_ctx*, const void*, const void*, const void*, void*, int, int, int, int, const int32_t*, const int32_t*,
                                const int32_t*, int, int, int, int, int, const nvc_attn_spec&, cudaStream_t) {
  return NVC_ENOTIMPL;
}

}  // namespace
