// Ranilix model body behind the step executor (runner.cu): weights, per-layer paged key / value pools, per-layer recurrent
// state slots, the layer loop.
//
// One layer over the N query rows of a step (h1 = rms(x) w1, h2 = rms(x) w2; x <- x + mixer(h1) + ff(h2)):
//   nvc_rms_norm_pair       x += pending sums of the previous layer; h1 and h2 from one pass over the row
//   linear w_in             ONE fused projection of everything the mixer reads from h1, fp32 out:
//                             attention: [q | k | v | gate]      parallel: [left q | left k | left v | right q | k | v | gate]
//   nvc_qkv_prep_run        bias, q / k head norms, rotary, value blending, k / v into this layer's paged pools
//   nvc_attn_paged_wide     softmax attention (window, sink, sigmoid gate and the mixer's constant factor in its epilogue)
//   parallel only:          nvc_qkv_prep_run (rotate-half, k scaled; fp32 rows) -> nvc_retention_scan over the state slots of the
//                           step's sequences -> nvc_head_gate (per-head root mean square, silu gate, constant factor)
//   linear w_o              ONE output projection over [left heads | right heads] -> fp32 mixer output
//   linear up (+ relu^2) -> linear down (fp32)
// The residual sum itself happens in the NEXT nvc_rms_norm_pair (or the final one), in fp32.
//
// Feature dimensions that a matrix product sums over or produces are padded to multiples of 64 in the weight and activation
// buffers (zeros), so that the tcgen05 GEMMs (K % 64, N % 16) take every product of the bf16 mode; heads are NOT padded: q, the
// caches and the attention kernels use the logical head sizes.
#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "body_common.h"
#include "model_config.h"
#include "runner.h"

namespace {

struct RLayerW {
  float *n1 = nullptr, *n2 = nullptr;
  void* w_in = nullptr;                 // [np, Wp]
  float* bias = nullptr;                // [np] (attention; zero under the gate columns)
  int np = 0;
  int q_off = 0, k_off = 0, v_off = 0, g_off = 0;        // attention / left half
  int rq_off = 0, rk_off = 0, rv_off = 0, rg_off = 0;    // right half
  float *q_norm = nullptr, *k_norm = nullptr, *lambda = nullptr, *sink = nullptr, *decay = nullptr;
  void* w_o = nullptr;                  // [Wp, ow]
  int lwp = 0, ow = 0;                  // padded width of the (left) heads' outputs; K of the output projection
  void *w_up = nullptr, *w_down = nullptr;
  int ffp = 0;
  void *k_cache = nullptr, *v_cache = nullptr;
  float* state = nullptr;               // [state slots, heads, dim, vdim]
  const float *rot = nullptr, *rrot = nullptr;
};

struct RanilixBody : nvc_body_base {
  nvc_ranilix_config cfg;
  int Wp = 0, Vp = 0;
  int first_blend = -1;
  int state_slots = 0;
  bool use_flash = true;               // tcgen05 paged-prefill kernel for long portions of plain causal attention with 128-wide heads
  std::vector<RLayerW> L;
  void *embed = nullptr, *head = nullptr;
  float* fw = nullptr;
  std::map<std::string, bool> want;
  std::map<std::pair<int, uint32_t>, float*> rot_tables;   // (dims, bits of base) -> [max_model_len, dims / 2, 2]
  // activations
  float *x0 = nullptr, *res = nullptr, *proj = nullptr, *mix = nullptr, *ffo = nullptr, *v_first = nullptr;
  float *rq = nullptr, *rk = nullptr, *rv = nullptr, *ro = nullptr;
  void *h1 = nullptr, *h2 = nullptr, *q = nullptr, *ao = nullptr, *act = nullptr, *hn = nullptr;
  int blend_w = 0;
  float* tap_host = nullptr;
  size_t tap_cap = 0;

  int vocab() const override { return cfg.vocab; }
  int logits_ld() const override { return Vp; }
  int layer_runs() const override { return (int)cfg.layers.size(); }
  int width() const override { return cfg.width; }
  int num_state_slots() const override { return state_slots; }
  int64_t cache_bytes_per_token() const override {
    int64_t b = 0;
    for (auto& ly : cfg.layers) b += (int64_t)ly.attn.kv_heads * (ly.attn.dim + ly.attn.vdim) * (int64_t)esz;
    return b;
  }
  int set_residual_tap(float* host, size_t cap) override {
    tap_host = host;
    tap_cap = host ? cap : 0;
    return NVC_OK;
  }

  int rotary_table(nvc_runner* r, const nvc_rotary_spec& rs, const float** out) {
    *out = nullptr;
    if (rs.dims == 0) return NVC_OK;
    uint32_t bits;
    memcpy(&bits, &rs.base, 4);
    auto key = std::make_pair(rs.dims, bits);
    auto it = rot_tables.find(key);
    if (it == rot_tables.end()) {
      float* t = nullptr;
      int rc = zalloc(r, &t, (size_t)r->opt.max_model_len * rs.dims * sizeof(float));
      if (rc) return rc;
      if ((rc = nvc_rotary_table_init_sync(r->ctx, rs.base, rs.dims, r->opt.max_model_len, t))) return rc;
      it = rot_tables.emplace(key, t).first;
    }
    *out = it->second;
    return NVC_OK;
  }

  int init(nvc_runner* r) {
    nvc_ctx* ctx = r->ctx;
    dt = r->dtype;
    esz = dt == NVC_DT_F32 ? 4 : 2;
    use_tc = dt == NVC_DT_BF16 && !(getenv("NVC_RANILIX_TC") && atoi(getenv("NVC_RANILIX_TC")) == 0);
    use_flash = use_tc && !(getenv("NVC_RANILIX_FLASH") && atoi(getenv("NVC_RANILIX_FLASH")) == 0);
    Wp = pad64(cfg.width);
    Vp = pad64(cfg.vocab);
    first_blend = cfg.first_blend_layer();
    state_slots = cfg.has_state() ? r->opt.max_num_seqs : 0;
    const size_t T = (size_t)std::max(r->opt.max_num_batched_tokens, r->opt.max_num_seqs);
    const size_t slots = (size_t)r->opt.num_kvcache_blocks * r->opt.kvcache_block_size;
    int rc;
    L.resize(cfg.layers.size());
    size_t m_np = 0, m_q = 0, m_ow = 0, m_ff = 0, m_rqk = 0, m_rv = 0;
    int64_t wbytes = 0;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
      const auto& ly = cfg.layers[i];
      const auto& a = ly.attn;
      RLayerW& w = L[i];
      const std::string p = "l" + std::to_string(i) + ".";
      NVC_REQUIRE(ctx, a.dim <= 512 && a.vdim <= 512, NVC_ESHAPE, "head sizes above 512");
      if ((rc = zalloc(r, &w.n1, cfg.width * 4)) || (rc = zalloc(r, &w.n2, cfg.width * 4))) return rc;
      want[p + "norm1"] = false;
      want[p + "norm2"] = false;
      const int qw = a.heads * a.dim, kw = a.kv_heads * a.dim, vw = a.kv_heads * a.vdim, hw = a.heads * a.vdim;
      w.q_off = 0; w.k_off = qw; w.v_off = qw + kw;
      int total = qw + kw + vw;
      w.lwp = pad64(hw);
      if (ly.kind == nvc_ranilix_layer::Attention) {
        w.g_off = total;
        total += hw;
        w.ow = w.lwp;
        if ((rc = zalloc(r, &w.q_norm, a.dim * 4)) || (rc = zalloc(r, &w.k_norm, a.dim * 4)) || (rc = zalloc(r, &w.lambda, 4)) ||
            (rc = zalloc(r, &w.sink, a.heads * 4)))
          return rc;
        for (const char* n : {"mix.q", "mix.q.b", "mix.k", "mix.k.b", "mix.v", "mix.v.b", "mix.q.norm", "mix.k.norm", "mix.sink", "mix.g", "mix.o"})
          want[p + n] = false;
        if (a.blend_values && (int)i != first_blend) want[p + "mix.vmix"] = false;
        if (a.blend_values) blend_w = vw;
        wbytes += (int64_t)esz * ((int64_t)(qw + kw + vw + hw) * cfg.width + (int64_t)cfg.width * hw);
      } else {
        const auto& rt = ly.ret;
        NVC_REQUIRE(ctx, rt.dim <= 512, NVC_ESHAPE, "retention key size above 512");
        const int rqw = rt.heads * rt.dim, rvw = rt.heads * rt.vdim;
        w.rq_off = total; w.rk_off = total + rqw; w.rv_off = total + 2 * rqw; w.rg_off = total + 2 * rqw + rvw;
        total += 2 * rqw + 2 * rvw;
        w.ow = w.lwp + pad64(rvw);
        if ((rc = zalloc(r, &w.decay, rt.heads * 4))) return rc;
        NVC_CUDA_CHECK(ctx, cudaMemcpy(w.decay, rt.decay.data(), rt.heads * 4, cudaMemcpyHostToDevice));
        if ((rc = zalloc(r, &w.state, (size_t)state_slots * rt.heads * rt.dim * rt.vdim * 4))) return rc;
        if ((rc = rotary_table(r, rt.rot, &w.rrot))) return rc;
        for (const char* n : {"mix.left.q", "mix.left.k", "mix.left.v", "mix.left.o", "mix.right.q", "mix.right.k", "mix.right.v",
                              "mix.right.g", "mix.right.o"})
          want[p + n] = false;
        m_rqk = std::max(m_rqk, (size_t)rqw);
        m_rv = std::max(m_rv, (size_t)rvw);
        wbytes += (int64_t)esz * ((int64_t)(qw + kw + vw + 2 * rqw + 2 * rvw) * cfg.width + (int64_t)cfg.width * (hw + rvw));
      }
      if ((rc = rotary_table(r, a.rot, &w.rot))) return rc;
      w.np = pad64(total);
      if ((rc = zalloc(r, &w.w_in, (size_t)w.np * Wp * esz)) || (rc = zalloc(r, &w.bias, (size_t)w.np * 4)) ||
          (rc = zalloc(r, &w.w_o, (size_t)Wp * w.ow * esz)))
        return rc;
      if ((rc = zalloc(r, &w.k_cache, slots * kw * esz)) || (rc = zalloc(r, &w.v_cache, slots * vw * esz))) return rc;
      if (ly.ff > 0) {
        w.ffp = pad64(ly.ff);
        if ((rc = zalloc(r, &w.w_up, (size_t)w.ffp * Wp * esz)) || (rc = zalloc(r, &w.w_down, (size_t)Wp * w.ffp * esz))) return rc;
        want[p + "mlp.up"] = false;
        want[p + "mlp.down"] = false;
        wbytes += (int64_t)esz * 2 * ly.ff * cfg.width;
        m_ff = std::max(m_ff, (size_t)w.ffp);
      }
      m_np = std::max(m_np, (size_t)w.np);
      m_q = std::max(m_q, (size_t)qw);
      m_ow = std::max(m_ow, (size_t)w.ow);
    }
    if ((rc = zalloc(r, &embed, (size_t)Vp * Wp * esz)) || (rc = zalloc(r, &head, (size_t)Vp * Wp * esz)) || (rc = zalloc(r, &fw, cfg.width * 4)))
      return rc;
    for (const char* n : {"embed", "head", "final.norm"}) want[n] = false;
    r->weight_bytes = wbytes + (int64_t)esz * 2 * cfg.vocab * cfg.width;
    // activations (zeroed once: padding columns are never written)
    if ((rc = zalloc(r, &x0, T * Wp * 4)) || (rc = zalloc(r, &res, T * Wp * 4)) || (rc = zalloc(r, &mix, T * Wp * 4)) ||
        (rc = zalloc(r, &ffo, T * Wp * 4)) || (rc = zalloc(r, &proj, T * m_np * 4)))
      return rc;
    if ((rc = zalloc(r, &h1, T * Wp * esz)) || (rc = zalloc(r, &h2, T * Wp * esz)) || (rc = zalloc(r, &q, T * m_q * esz)) ||
        (rc = zalloc(r, &ao, T * m_ow * esz)))
      return rc;
    if (m_ff && (rc = zalloc(r, &act, T * m_ff * esz))) return rc;
    if (blend_w && (rc = zalloc(r, &v_first, T * blend_w * 4))) return rc;
    if (m_rqk && ((rc = zalloc(r, &rq, T * m_rqk * 4)) || (rc = zalloc(r, &rk, T * m_rqk * 4)) || (rc = zalloc(r, &rv, T * m_rv * 4)) ||
                  (rc = zalloc(r, &ro, T * m_rv * 4))))
      return rc;
    if ((rc = zalloc(r, &hn, (size_t)r->max_logit_rows * Wp * esz))) return rc;
    return NVC_OK;
  }

  int load_tensor(nvc_runner* r, const char* cname, const void* data, int st_dtype, const int64_t* shape, int ndim) override {
    nvc_ctx* ctx = r->ctx;
    const std::string name(cname);
    auto it = want.find(name);
    if (it == want.end()) return NVC_OK;    // not a tensor of this configuration: ignored
    size_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= (size_t)shape[i];
    std::vector<float> v;
    NVC_REQUIRE(ctx, tensor_to_f32(data, st_dtype, n, v), NVC_EINVAL, "unsupported dtype for " + name);
    const int64_t d0 = ndim > 0 ? shape[0] : 1, d1 = ndim > 1 ? shape[1] : 1;
    auto shape_is = [&](int64_t a, int64_t b) { return (ndim <= 2) && d0 == a && d1 == b && (ndim == 2 || b == 1); };
    auto bad = [&]() {
      nvc_set_error(ctx, "unexpected shape for " + name);
      return NVC_ESHAPE;
    };
    const int W = cfg.width;
    int rc = NVC_OK;
    if (name == "embed") { if (!shape_is(cfg.vocab, W)) return bad(); rc = put_matrix(r, embed, Wp, 0, 0, v.data(), cfg.vocab, W, W, 1); }
    else if (name == "head") { if (!shape_is(cfg.vocab, W)) return bad(); rc = put_matrix(r, head, Wp, 0, 0, v.data(), cfg.vocab, W, W, 1); }
    else if (name == "final.norm") { if (n != (size_t)W) return bad(); rc = put_f32(r, fw, v.data(), W); }
    else {
      const size_t dot = name.find('.');
      const int li = atoi(name.substr(1, dot - 1).c_str());
      const std::string sub = name.substr(dot + 1);
      const auto& ly = cfg.layers[li];
      const auto& a = ly.attn;
      const auto& rt = ly.ret;
      RLayerW& w = L[li];
      // rows [off, off + rows) of the fused input projection
      auto in_rows = [&](int off, int rows) { return shape_is(rows, W) ? put_matrix(r, w.w_in, Wp, off, 0, v.data(), rows, W, W, 1) : bad(); };
      auto in_bias = [&](int off, int rows) { return n == (size_t)rows ? put_f32(r, w.bias + off, v.data(), rows) : bad(); };
      // columns [off, off + cols) of the output projection
      auto out_cols = [&](int off, int cols) { return shape_is(W, cols) ? put_matrix(r, w.w_o, w.ow, 0, off, v.data(), W, cols, cols, 1) : bad(); };
      const int qw = a.heads * a.dim, kw = a.kv_heads * a.dim, vw = a.kv_heads * a.vdim, hw = a.heads * a.vdim;
      const int rqw = rt.heads * rt.dim, rvw = rt.heads * rt.vdim;
      if (sub == "norm1") { if (n != (size_t)W) return bad(); rc = put_f32(r, w.n1, v.data(), W); }
      else if (sub == "norm2") { if (n != (size_t)W) return bad(); rc = put_f32(r, w.n2, v.data(), W); }
      else if (sub == "mix.q" || sub == "mix.left.q") rc = in_rows(w.q_off, qw);
      else if (sub == "mix.k" || sub == "mix.left.k") rc = in_rows(w.k_off, kw);
      else if (sub == "mix.v" || sub == "mix.left.v") rc = in_rows(w.v_off, vw);
      else if (sub == "mix.g") rc = in_rows(w.g_off, hw);
      else if (sub == "mix.q.b") rc = in_bias(w.q_off, qw);
      else if (sub == "mix.k.b") rc = in_bias(w.k_off, kw);
      else if (sub == "mix.v.b") rc = in_bias(w.v_off, vw);
      else if (sub == "mix.q.norm") { if (n != (size_t)a.dim) return bad(); rc = put_f32(r, w.q_norm, v.data(), n); }
      else if (sub == "mix.k.norm") { if (n != (size_t)a.dim) return bad(); rc = put_f32(r, w.k_norm, v.data(), n); }
      else if (sub == "mix.vmix") { if (n != 1) return bad(); rc = put_f32(r, w.lambda, v.data(), 1); }
      else if (sub == "mix.sink") { if (n != (size_t)a.heads) return bad(); rc = put_f32(r, w.sink, v.data(), n); }
      else if (sub == "mix.o" || sub == "mix.left.o") rc = out_cols(0, hw);
      else if (sub == "mix.right.q") rc = in_rows(w.rq_off, rqw);
      else if (sub == "mix.right.k") rc = in_rows(w.rk_off, rqw);
      else if (sub == "mix.right.v") rc = in_rows(w.rv_off, rvw);
      else if (sub == "mix.right.g") rc = in_rows(w.rg_off, rvw);
      else if (sub == "mix.right.o") rc = out_cols(w.lwp, rvw);
      else if (sub == "mlp.up") { if (!shape_is(ly.ff, W)) return bad(); rc = put_matrix(r, w.w_up, Wp, 0, 0, v.data(), ly.ff, W, W, 1); }
      else if (sub == "mlp.down") { if (!shape_is(W, ly.ff)) return bad(); rc = put_matrix(r, w.w_down, w.ffp, 0, 0, v.data(), W, ly.ff, ly.ff, 1); }
    }
    if (rc == NVC_OK) it->second = true;
    return rc;
  }

  int finalize(nvc_runner* r) override {
    std::string missing;
    int n = 0;
    for (auto& kv : want)
      if (!kv.second && ++n <= 4) missing += kv.first + " ";
    NVC_REQUIRE(r->ctx, n == 0, NVC_ESTATE, "missing " + std::to_string(n) + " tensors: " + missing);
    return NVC_OK;
  }

  int tap(nvc_runner* r, int run, int N) {
    const size_t need = (size_t)(run + 1) * N * cfg.width;
    NVC_REQUIRE(r->ctx, need <= tap_cap, NVC_ENOMEM, "residual tap buffer too small");
    NVC_CUDA_CHECK(r->ctx, cudaMemcpy2DAsync(tap_host + (size_t)run * N * cfg.width, (size_t)cfg.width * 4, res, (size_t)Wp * 4,
                                             (size_t)cfg.width * 4, N, cudaMemcpyDeviceToHost, r->stream));
    return NVC_OK;
  }

  static constexpr int kFlashMinChunk = 64;
  bool flash_portions(const nvc_runner* r, const nvc_step_shape& s, const nvc_softmax_attn_spec& a, bool is_attention_layer) const {
    const int bs = r->opt.kvcache_block_size;
    return use_flash && !is_attention_layer && a.window == 0 && a.dim == 128 && a.vdim == 128 && !s.decode && s.num_decode < s.B &&
           s.max_chunk >= kFlashMinChunk && (bs == 16 || bs == 32 || bs == 64 || bs % 128 == 0);
  }

  // bias / norms / rotary / blending / cache store of a softmax-attention mixer, then the attention itself into ao[:, :heads * vdim]
  int softmax_mixer(nvc_runner* r, const nvc_step_shape& s, int li, bool is_attention_layer, float out_scale) {
    nvc_ctx* ctx = r->ctx;
    const auto& a = cfg.layers[li].attn;
    RLayerW& w = L[li];
    nvc_qkv_prep p{};
    p.in = proj; p.ldi = w.np;
    p.bias = is_attention_layer ? w.bias : nullptr;
    p.q_off = w.q_off; p.k_off = w.k_off; p.v_off = w.v_off;
    p.q_heads = a.heads; p.kv_heads = a.kv_heads; p.dim = a.dim; p.vdim = a.vdim;
    p.q_norm = is_attention_layer ? w.q_norm : nullptr;
    p.k_norm = is_attention_layer ? w.k_norm : nullptr;
    p.eps = cfg.eps;
    p.rot_dims = a.rot.dims; p.rot_half = 0; p.rot_table = w.rot; p.positions = r->d_pos;
    p.k_scale = 1.f;
    p.v_scale = out_scale;             // the mixer's constant weight rides on the cached values: no attention kernel needs to know it
    p.blend = !a.blend_values ? NVC_BLEND_NONE : (li == first_blend ? NVC_BLEND_PROVIDE : NVC_BLEND_MIX);
    p.lambda = w.lambda; p.v_first = v_first; p.ldvf = blend_w;
    p.q_out = q; p.ldq = a.heads * a.dim;
    p.k_out = w.k_cache; p.v_out = w.v_cache; p.ldk = a.kv_heads * a.dim; p.ldv = a.kv_heads * a.vdim;
    p.slot_mapping = r->d_slots;
    p.q_dtype = dt; p.kv_dtype = dt;
    int rc = nvc_qkv_prep_run(ctx, &p, s.N, r->stream);
    if (rc) return rc;
    mark(r, "qkv_prep");
    nvc_attn_spec sp{};
    sp.heads = a.heads; sp.kv_heads = a.kv_heads; sp.dim = a.dim; sp.vdim = a.vdim;
    sp.scale = a.scale;
    sp.window = a.window;
    sp.sink = is_attention_layer ? w.sink : nullptr;
    sp.gate = is_attention_layer ? proj + w.g_off : nullptr;
    sp.ldg = w.np;
    sp.out_scale = 1.f;
    const int bs = r->opt.kvcache_block_size, cap = r->max_blocks_cap;
    if (flash_portions(r, s, a, is_attention_layer)) {
      // Plain causal attention with 128-wide keys and values is what the tcgen05 paged-prefill kernel of the Qwen3 family
      // computes: long prompt portions go there (it writes the left part of the output projection's input through its row
      // stride); the one-token sequences of a mixed step come first in the batch and keep the decode path of the wide kernel.
      const int nd = s.num_decode;
      const nvc_bf16* qb = reinterpret_cast<const nvc_bf16*>(q);
      nvc_bf16* ob = reinterpret_cast<nvc_bf16*>(ao);
      if (nd > 0 && (rc = nvc_attn_paged_wide(ctx, q, p.ldq, w.k_cache, p.ldk, w.v_cache, p.ldv, r->d_bt, cap, r->d_ctx, nullptr, nd, nd, 1, bs,
                                              &sp, ao, w.ow, dt, r->stream)))
        return rc;
      rc = nvc_prefill_attn_paged_ld(ctx, qb + (size_t)nd * p.ldq, p.ldq, reinterpret_cast<const nvc_bf16*>(w.k_cache),
                                     reinterpret_cast<const nvc_bf16*>(w.v_cache), r->d_bt + (size_t)nd * cap, cap, r->d_ctx + nd,
                                     nd ? r->d_cu2 : r->d_cu, s.B - nd, s.N - nd, s.max_chunk, a.heads, a.kv_heads, a.dim, bs,
                                     r->opt.num_kvcache_blocks, a.scale, ob + (size_t)nd * w.ow, w.ow, r->stream);
    } else {
      rc = nvc_attn_paged_wide(ctx, q, p.ldq, w.k_cache, p.ldk, w.v_cache, p.ldv, r->d_bt, cap, r->d_ctx, s.decode ? nullptr : r->d_cu, s.B,
                               s.N, s.decode ? 1 : s.max_seqlen, bs, &sp, ao, w.ow, dt, r->stream);
    }
    mark(r, "attention");
    return rc;
  }

  int retention_mixer(nvc_runner* r, const nvc_step_shape& s, int li, float out_scale) {
    nvc_ctx* ctx = r->ctx;
    const auto& rt = cfg.layers[li].ret;
    RLayerW& w = L[li];
    const int qw = rt.heads * rt.dim, vw = rt.heads * rt.vdim;
    nvc_qkv_prep p{};
    p.in = proj; p.ldi = w.np;
    p.q_off = w.rq_off; p.k_off = w.rk_off; p.v_off = w.rv_off;
    p.q_heads = rt.heads; p.kv_heads = rt.heads; p.dim = rt.dim; p.vdim = rt.vdim;
    p.eps = cfg.eps;
    p.rot_dims = rt.rot.dims; p.rot_half = 1; p.rot_table = w.rrot; p.positions = r->d_pos;
    p.k_scale = 1.0f / sqrtf((float)rt.dim);
    p.v_scale = 1.f;
    p.blend = NVC_BLEND_NONE;
    p.q_out = rq; p.ldq = qw;
    p.k_out = rk; p.v_out = rv; p.ldk = qw; p.ldv = vw;
    p.slot_mapping = nullptr;
    p.q_dtype = NVC_DT_F32; p.kv_dtype = NVC_DT_F32;
    int rc = nvc_qkv_prep_run(ctx, &p, s.N, r->stream);
    if (rc) return rc;
    mark(r, "retention_prep");
    if ((rc = nvc_retention_scan(ctx, rq, qw, rk, qw, rv, vw, ro, vw, w.state, r->d_state_slots, s.decode ? nullptr : r->d_cu, r->d_pos, w.decay,
                                 s.B, s.decode ? 1 : s.max_seqlen, rt.heads, rt.dim, rt.vdim, r->stream)))
      return rc;
    mark(r, "retention_scan");
    uint8_t* dst = reinterpret_cast<uint8_t*>(ao) + (size_t)w.lwp * esz;
    rc = nvc_head_gate(ctx, ro, vw, proj + w.rg_off, w.np, dst, w.ow, dt, rt.heads, rt.vdim, 1, cfg.eps, NVC_GATE_SILU, out_scale, s.N, r->stream);
    mark(r, "retention_gate");
    return rc;
  }

  int forward(nvc_runner* r, const nvc_step_shape& s) override {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const int N = s.N, W = cfg.width;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(r->stream, &cap);
    prof_on = prof_armed && cap == cudaStreamCaptureStatusNone;
    if (prof_on) prof_armed = false;
    mark(r, "start");
    int rc = nvc_embed_gather_scaled_f32(ctx, r->d_ids, embed, dt, Wp, cfg.embedding_scale, x0, Wp, N, W, st);
    if (rc) return rc;
    mark(r, "embed");
    const float *a0 = nullptr, *a1 = nullptr;     // sums not yet added to the residual stream
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
      const auto& ly = cfg.layers[i];
      RLayerW& w = L[i];
      const bool first = i == 0;
      if (tap_host && !first) {
        // debug: land the previous layer's sums first, copy the stream out, then open this layer
        if ((rc = nvc_rms_norm_pair(ctx, res, a0, a1, res, Wp, nullptr, nullptr, nullptr, nullptr, dt, 0, cfg.eps, nullptr, N, W, st))) return rc;
        if ((rc = tap(r, (int)i - 1, N))) return rc;
        a0 = a1 = nullptr;
      }
      rc = nvc_rms_norm_pair(ctx, first ? x0 : res, a0, a1, res, Wp, w.n1, h1, ly.ff > 0 ? w.n2 : nullptr, ly.ff > 0 ? h2 : nullptr, dt, Wp, cfg.eps,
                             nullptr, N, W, st);
      if (rc) return rc;
      mark(r, "rms_norm_pair");
      // ---- mixer
      if ((rc = linear(r, h1, Wp, w.w_in, proj, w.np, NVC_DT_F32, N, w.np, Wp))) return rc;
      mark(r, "gemm_in");
      if (ly.kind == nvc_ranilix_layer::Attention) {
        if ((rc = softmax_mixer(r, s, (int)i, true, 1.f))) return rc;
      } else {
        if ((rc = softmax_mixer(r, s, (int)i, false, ly.left_scale))) return rc;
        if ((rc = retention_mixer(r, s, (int)i, ly.right_scale))) return rc;
      }
      if ((rc = linear(r, ao, w.ow, w.w_o, mix, Wp, NVC_DT_F32, N, Wp, w.ow))) return rc;
      mark(r, "gemm_o");
      a0 = mix;
      a1 = nullptr;
      // ---- feed-forward
      if (ly.ff > 0) {
        if (use_tc) {        // squared relu in the epilogue of the up-projection
          if ((rc = nvc_gemm_bf16_act(ctx, reinterpret_cast<const nvc_bf16*>(h2), Wp, reinterpret_cast<const nvc_bf16*>(w.w_up), act, w.ffp,
                                      NVC_DT_BF16, N, w.ffp, Wp, NVC_ACT_RELU2, st)))
            return rc;
        } else if ((rc = linear(r, h2, Wp, w.w_up, act, w.ffp, dt, N, w.ffp, Wp, NVC_ACT_RELU2))) {
          return rc;
        }
        mark(r, "gemm_up");
        if ((rc = linear(r, act, w.ffp, w.w_down, ffo, Wp, NVC_DT_F32, N, Wp, w.ffp))) return rc;
        mark(r, "gemm_down");
        a1 = ffo;
      }
    }
    if (tap_host) {
      if ((rc = nvc_rms_norm_pair(ctx, res, a0, a1, res, Wp, nullptr, nullptr, nullptr, nullptr, dt, 0, cfg.eps, nullptr, N, W, st))) return rc;
      if ((rc = tap(r, (int)cfg.layers.size() - 1, N))) return rc;
      a0 = a1 = nullptr;
      tap_host = nullptr;      // one step only
    }
    // ---- head: final norm of the wanted rows (the last layer's sums are added on the way), logits
    rc = nvc_rms_norm_pair(ctx, res, a0, a1, nullptr, Wp, fw, hn, nullptr, nullptr, dt, Wp, cfg.eps, s.decode ? nullptr : r->d_last_rows, s.rows, W, st);
    if (rc) return rc;
    mark(r, "final_norm");
    rc = linear(r, hn, Wp, head, r->logits, Vp, NVC_DT_F32, s.rows, Vp, Wp);
    mark(r, "lm_head");
    finish_profile(r);
    return rc;
  }
};

}  // namespace

nvc_model_body* nvc_make_ranilix_body(nvc_runner* r, const nvc_ranilix_config& cfg, int* status) {
  RanilixBody* b = new RanilixBody();
  b->cfg = cfg;
  *status = b->init(r);
  return b;
}
