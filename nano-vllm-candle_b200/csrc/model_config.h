// Parsed model configurations of the registered architectures (model_config.cpp).
#pragma once
#include <string>
#include <vector>

#include "../../include/nvc_b200_engine.h"

// Karuzen: a stack of parallel layers (one Dynamic-Tanh norm feeds the mixer and the feed-forward, both added to the fp32
// residual stream), latent attention without positions, dense gated-gelu or sigmoid-routed mixture-of-experts
// feed-forward, an optional block of layers that is run several times with the same weights and its own cache per pass.
struct nvc_karuzen_mixer {
  std::string type;          // "latent_attention"
  int heads = 0, dim = 0, vdim = 0, kv_rank = 0, q_rank = 0;
  float scale = 0.f;
};
struct nvc_karuzen_mlp {
  enum Kind { None, Dense, Moe } kind = None;
  int ff = 0;                                   // dense
  int experts = 0, top = 0, expert_ff = 0;      // moe
  float router_scale = 1.f;
  int shared_ff = 0;                            // moe: 0 = no shared expert
};
struct nvc_karuzen_layer {
  nvc_karuzen_mixer mixer;
  nvc_karuzen_mlp mlp;
};
struct nvc_karuzen_config {
  int vocab = 0, width = 0;
  float eps = 1e-5f;
  std::vector<nvc_karuzen_layer> layers;
  int loop_start = 0, loop_stop = 0, loop_times = 1;
  // the order in which layers run: (layer, pass); first_of_later_pass marks where the embedding is added again
  struct Run { int layer; int pass; bool readd_embedding; };
  std::vector<Run> runs() const;
};

struct nvc_model_config {
  std::string architecture;   // "Qwen3ForCausalLM" or "Karuzen"
  nvc_qwen3_config qwen3{};
  int qwen3_tied = 0;
  nvc_karuzen_config karuzen;
};
