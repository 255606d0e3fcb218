// The step executor's state, shared by the model families that run behind it.
//
// nvc_runner owns what every model needs - stream, step inputs and their pinned staging, logits, sampling state, decode
// graphs - and runs one engine step from flat step inputs (runner.cu).  The transformer body is either the built-in
// Qwen3 one (the Layer fields below) or a ModelBody from the registry (model_registry.cpp), which owns its weights and its
// paged cache pools and is called for the embedding + layers + head of a step.
#pragma once
#include "common.cuh"
#include "internal.h"

#include <map>
#include <set>
#include <string>
#include <vector>

struct nvc_runner;

// What a step looks like to a model body: N query rows of B sequences, already uploaded to the runner's device inputs
// (d_ids, d_pos, d_slots, d_cu, d_bt, d_ctx).  Sequences are the last q_len positions of their contexts.
struct nvc_step_shape {
  int N = 0, B = 0;
  int max_seqlen = 1;     // longest q_len of the step
  bool decode = false;    // every sequence has one query row and d_cu was not uploaded
  int rows = 0;           // rows whose logits are computed (d_last_rows holds their indices; decode: rows == B, identity)
  // mixed step: the first num_decode sequences have one query row each; d_cu2 holds the cu_seqlens of the others relative to
  // their first row (when 0 < num_decode < B), and max_chunk is the longest q_len among them
  int num_decode = 0;
  int max_chunk = 1;
};

// A model family behind the runner.  Implementations: model_karuzen.cu, model_ranilix.cu.
struct nvc_model_body {
  virtual ~nvc_model_body() {}
  // one tensor of the checkpoint, in its own dtype (NVC_ST_*), host memory; shape has ndim entries
  virtual int load_tensor(nvc_runner* r, const char* name, const void* data, int st_dtype, const int64_t* shape, int ndim) = 0;
  virtual int finalize(nvc_runner* r) = 0;
  // embedding, layers, head: fp32 logits [rows, ld = logits_ld] in r->logits
  virtual int forward(nvc_runner* r, const nvc_step_shape& s) = 0;
  virtual int64_t cache_bytes_per_token() const = 0;
  virtual int vocab() const = 0;
  virtual int logits_ld() const = 0;
  // optional: residual stream after every layer run of the next step, [runs, N, width] fp32 into host memory
  virtual int set_residual_tap(float* /*host*/, size_t /*capacity_floats*/) { return NVC_ENOTIMPL; }
  // optional: the next (non-graph) step records CUDA events around every op; profile_json() = {"op": microseconds summed
  // over layer runs, ...} of that step
  virtual int arm_profile() { return NVC_ENOTIMPL; }
  virtual bool profile_armed() const { return false; }
  virtual const char* profile_json() const { return "{}"; }
  virtual int layer_runs() const { return 0; }
  virtual int width() const { return 0; }
  // > 0: the body keeps per-sequence recurrent state in that many slots; every step then names the slot of each of its
  // sequences (r->d_state_slots [B], armed with nvc_runner_set_state_slots), and a sequence whose first token of a step sits
  // at position 0 starts from an empty state
  virtual int num_state_slots() const { return 0; }
};

struct nvc_qwen3_layer {
  nvc_bf16 *w_qkv = nullptr, *w_o = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  nvc_bf16 *w_gu = nullptr, *w_down = nullptr, *ln1 = nullptr, *ln2 = nullptr;
  nvc_bf16 *k_cache = nullptr, *v_cache = nullptr;
};

struct nvc_arg_pair { float val; int32_t idx; };

struct nvc_runner {
  nvc_ctx* ctx = nullptr;
  nvc_qwen3_config cfg{};
  nvc_runner_options opt{};
  int tp = 1, rank = 0;
  int nh_l = 0, kv_l = 0, I_l = 0, V_l = 0, qkv_l = 0, max_blocks_cap = 0;
  bool finalized = false;
  nvc_model_body* body = nullptr;   // a registry model; NULL = the built-in Qwen3 body
  int dtype = NVC_DT_BF16;          // storage format of a registry model's weights and activations
  int max_logit_rows = 0;           // rows of r->logits
  int logit_rows_armed = 0;         // > 0: the next step computes logits for these rows (nvc_runner_set_logit_rows)
  std::vector<int32_t> armed_rows;
  cudaStream_t stream = nullptr;
  std::vector<nvc_qwen3_layer> layers;
  nvc_bf16 *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr;
  float* rope = nullptr;
  std::set<std::string> loaded;
  int64_t weight_bytes = 0;
  std::vector<void*> allocs;
  // activations
  nvc_bf16 *x = nullptr, *xn = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr;
  float* residual = nullptr;
  nvc_bf16 *x_last = nullptr, *xn_last = nullptr;
  float *res_last = nullptr, *logits = nullptr;
  void* decode_ws = nullptr;
  size_t decode_ws_bytes = 0;
  // step inputs on device + pinned staging
  int32_t* d_state_slots = nullptr;   // state slot of every sequence of the step (bodies with recurrent state)
  std::vector<int32_t> armed_state_slots;
  int state_slots_armed = 0;          // > 0: nvc_runner_set_state_slots named the slots of the next step's sequences
  int32_t* d_cu2 = nullptr;     // mixed step: cu_seqlens of the prompt chunks, relative to their first token
  int32_t *d_ids = nullptr, *d_pos = nullptr, *d_cu = nullptr, *d_slots = nullptr, *d_bt = nullptr, *d_ctx = nullptr,
          *d_last_rows = nullptr, *d_tok = nullptr;
  float* d_tok_val = nullptr;
  nvc_arg_pair* d_pairs = nullptr;
  int32_t* h_stage = nullptr;   // pinned
  size_t h_stage_ints = 0;
  size_t in_pitch = 0;             // ints between d_ids / d_pos / d_slots / d_ctx (one block, d_state_slots behind them: a decode step uploads them in ONE 2-D copy)
  std::vector<int32_t> bt_mirror;  // the padded block table the device holds (decode steps re-upload it only when it changed)
  int bt_mirror_B = -1;            // rows of bt_mirror that are valid; -1: unknown (a prefill / mixed step wrote d_bt)
  nvc_arg_pair* h_pairs = nullptr;   // pinned
  int32_t* h_tok = nullptr;     // pinned
  int last_B = 0;
  // on-device temperature sampling (K8s), armed per step by nvc_runner_set_sampling
  float* d_temps = nullptr;
  uint64_t* d_streams = nullptr;
  float* h_temps = nullptr;        // pinned
  uint64_t* h_streams = nullptr;   // pinned
  bool sampling_armed = false;
  int last_sampling_B = 0;
  uint64_t sampling_seed = 0;
  // decode graphs keyed by (B, 2 * blocks hint + sampling)
  std::map<std::pair<int, int>, cudaGraphExec_t> graphs;
  int launches_per_decode = 0;
  int64_t last_h2d_bytes = 0;      // host-to-device bytes of the last step's inputs
  bool x_nvls = false;             // r->x is the context's NVLS slot: all-reduces go through the switch
  int last_decode_hint = 0;
  int last_decode_key2 = 0;
};

