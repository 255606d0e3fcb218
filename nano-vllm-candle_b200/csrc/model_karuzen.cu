// Karuzen model body behind the step executor (runner.cu): weights, per-run latent cache pools, the layer loop.
//
// One layer run over the N query rows of a step (h = DyT(x); x <- x + mixer(h) + ff(h), both read the same h):
//   nvc_dyt_norm            x += pending sums of the previous run (+ the embedding at the start of a later pass); h
//   linear [dq; dkv]        one fused down-projection, fp32 out
//   nvc_latent_norm_store   RMS norms of both latents; the key / value latent goes into this run's paged cache
//   linear uq               queries per head
//   linear uk^T (per head)  queries carried into the latent space (absorbed key up-projection)
//   nvc_latent_attn*        softmax over the cached latents, one cache row per token for all heads
//   linear uv (per head)    value up-projection of the attended latent;  linear o -> fp32 mixer output
//   dense:  linear [gate; up] -> gelu_tanh(gate) * up -> linear down (fp32)
//   moe:    route -> sort -> grouped up (relu^2) -> grouped down (fp32) -> shared expert -> combine (fp32)
// The residual sum itself happens in the NEXT nvc_dyt_norm (or the final one), in fp32.
//
// Every feature dimension is padded to a multiple of 64 in the weight and activation buffers (zeros), so that the
// tcgen05 GEMMs (K % 64, N % 16) take every product of the bf16 mode; norms divide by the logical width.
// Each pass over the looped block has its own cache pool; block ids and slots are the engine's, shared by all pools.
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "body_common.h"
#include "model_config.h"
#include "runner.h"

namespace {

struct LayerW {
  // norm
  float *nw = nullptr, *nb = nullptr, *nalpha = nullptr;
  // mixer
  void *w_down = nullptr;              // [qrp + kvp, Wp]: rows [0, q_rank) = dq, rows [qrp, qrp + kv_rank) = dkv
  float *dq_norm = nullptr, *dkv_norm = nullptr;
  void *w_uq = nullptr;                // [heads * dimp, qrp]
  void *w_ukT = nullptr;               // [heads][kvp, dimp]
  void *w_uv = nullptr;                // [heads][vdp, kvp]
  void *w_o = nullptr;                 // [Wp, heads * vdp]
  // dense ff
  void *w_gu = nullptr, *w_fdown = nullptr;   // [2 ffp, Wp] (gate rows, then up rows at ffp), [Wp, ffp]
  // moe
  void* router = nullptr;              // [Ep, Wp]: rows [0, E) = router, row E = the shared expert's gate vector
  float* corr = nullptr;
  int Ep = 0;
  void *w_eup = nullptr, *w_edown = nullptr;  // [E][effp, Wp], [E][Wp, effp]
  void *w_sup = nullptr, *w_sdown = nullptr;  // [sfp, Wp], [Wp, sfp]
  int qrp = 0, kvp = 0, dimp = 0, vdp = 0, ffp = 0, effp = 0, sfp = 0;
  bool moe_tc = false;                        // experts through the grouped tcgen05 product (groups padded to 128 rows)
};

struct KaruzenBody : nvc_body_base {
  nvc_karuzen_config cfg;
  std::vector<nvc_karuzen_config::Run> runs;
  int Wp = 0, Vp = 0;
  bool use_moe_tc = true;              // grouped tcgen05 products for the experts (bf16, padded expert size of 128 and more)
  bool use_flash = true;               // tcgen05 paged-prefill kernel for long prompt portions (bf16, padded latent of 128)
  std::vector<LayerW> L;
  std::vector<void*> cache;            // per run: [slots, kvp]
  int kvp_max = 0;
  void* embed = nullptr;               // [Vp, Wp]
  float *fw = nullptr, *fb = nullptr, *falpha = nullptr;
  std::map<std::string, bool> want;    // tensor name -> loaded
  // activations
  float *x0 = nullptr, *res = nullptr, *down = nullptr, *mix = nullptr, *ffo = nullptr, *y = nullptr, *sd = nullptr;
  void *h = nullptr, *cq = nullptr, *q = nullptr, *qabs = nullptr, *olat = nullptr, *ao = nullptr, *gu = nullptr, *act = nullptr,
       *hid = nullptr, *su = nullptr, *hn = nullptr;
  int32_t *tk_idx = nullptr, *offsets = nullptr, *src_rows = nullptr, *pos = nullptr, *tile_group = nullptr;
  void* xs = nullptr;                  // rows of h gathered into the experts' padded groups
  float *tk_w = nullptr, *gate = nullptr, *zlog = nullptr;
  void* attn_ws = nullptr;             // key-split partials of small decode batches
  size_t attn_ws_bytes = 0;
  float* tap_host = nullptr;
  size_t tap_cap = 0;


  int vocab() const override { return cfg.vocab; }
  int logits_ld() const override { return Vp; }
  int layer_runs() const override { return (int)runs.size(); }
  int width() const override { return cfg.width; }
  int64_t cache_bytes_per_token() const override {
    int64_t b = 0;
    for (auto& rn : runs) b += (int64_t)cfg.layers[rn.layer].mixer.kv_rank * (int64_t)esz;
    return b;
  }
  int set_residual_tap(float* host, size_t cap) override {
    tap_host = host;
    tap_cap = host ? cap : 0;
    return NVC_OK;
  }


  int init(nvc_runner* r) {
    nvc_ctx* ctx = r->ctx;
    dt = r->dtype;
    esz = dt == NVC_DT_F32 ? 4 : 2;
    use_tc = dt == NVC_DT_BF16 && !(getenv("NVC_KARUZEN_TC") && atoi(getenv("NVC_KARUZEN_TC")) == 0);
    use_flash = use_tc && !(getenv("NVC_KARUZEN_FLASH") && atoi(getenv("NVC_KARUZEN_FLASH")) == 0);
    use_moe_tc = use_tc && !(getenv("NVC_KARUZEN_MOE_TC") && atoi(getenv("NVC_KARUZEN_MOE_TC")) == 0);
    runs = cfg.runs();
    Wp = pad64(cfg.width);
    Vp = pad64(cfg.vocab);
    const size_t T = (size_t)std::max(r->opt.max_num_batched_tokens, r->opt.max_num_seqs);
    const size_t slots = (size_t)r->opt.num_kvcache_blocks * r->opt.kvcache_block_size;
    int rc;
    L.resize(cfg.layers.size());
    size_t m_down = 0, m_cq = 0, m_q = 0, m_qabs = 0, m_ao = 0, m_gu = 0, m_act = 0, m_hid = 0, m_su = 0, m_top = 0, m_E = 0, m_Ep = 0;
    size_t m_prow = 0, m_effp = 0, m_tcrow = 0;     // rows of the sorted (token, choice) layout, padded where the groups are
    int64_t wbytes = 0;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
      const auto& m = cfg.layers[i].mixer;
      const auto& f = cfg.layers[i].mlp;
      LayerW& w = L[i];
      const std::string p = "l" + std::to_string(i) + ".";
      NVC_REQUIRE(ctx, m.kv_rank <= 512, NVC_ESHAPE, "kv_rank above 512");
      w.qrp = pad64(m.q_rank); w.kvp = pad64(m.kv_rank); w.dimp = pad64(m.dim); w.vdp = pad64(m.vdim);
      kvp_max = std::max(kvp_max, w.kvp);
      if ((rc = zalloc(r, &w.nw, cfg.width * 4)) || (rc = zalloc(r, &w.nb, cfg.width * 4)) || (rc = zalloc(r, &w.nalpha, 4))) return rc;
      if ((rc = zalloc(r, &w.w_down, (size_t)(w.qrp + w.kvp) * Wp * esz))) return rc;
      if ((rc = zalloc(r, &w.dq_norm, m.q_rank * 4)) || (rc = zalloc(r, &w.dkv_norm, m.kv_rank * 4))) return rc;
      if ((rc = zalloc(r, &w.w_uq, (size_t)m.heads * w.dimp * w.qrp * esz))) return rc;
      if ((rc = zalloc(r, &w.w_ukT, (size_t)m.heads * w.kvp * w.dimp * esz))) return rc;
      if ((rc = zalloc(r, &w.w_uv, (size_t)m.heads * w.vdp * w.kvp * esz))) return rc;
      if ((rc = zalloc(r, &w.w_o, (size_t)Wp * m.heads * w.vdp * esz))) return rc;
      wbytes += (int64_t)esz * ((int64_t)(m.q_rank + m.kv_rank) * cfg.width + (int64_t)m.heads * m.dim * (m.q_rank + m.kv_rank) +
                                (int64_t)m.heads * m.vdim * (m.kv_rank + cfg.width));
      for (const char* n : {"norm1", "norm1.b", "norm1.alpha", "mix.dq", "mix.dq.norm", "mix.uq", "mix.dkv", "mix.dkv.norm", "mix.uk",
                            "mix.uv", "mix.o"})
        want[p + n] = false;
      m_down = std::max(m_down, (size_t)w.qrp + w.kvp);
      m_cq = std::max(m_cq, (size_t)w.qrp);
      m_q = std::max(m_q, (size_t)m.heads * w.dimp);
      m_qabs = std::max(m_qabs, (size_t)m.heads * w.kvp);
      m_ao = std::max(m_ao, (size_t)m.heads * w.vdp);
      if (f.kind == nvc_karuzen_mlp::Dense) {
        w.ffp = pad64(f.ff);
        if ((rc = zalloc(r, &w.w_gu, (size_t)2 * w.ffp * Wp * esz)) || (rc = zalloc(r, &w.w_fdown, (size_t)Wp * w.ffp * esz))) return rc;
        wbytes += (int64_t)esz * 3 * f.ff * cfg.width;
        for (const char* n : {"mlp.gate", "mlp.up", "mlp.down"}) want[p + n] = false;
        m_gu = std::max(m_gu, (size_t)2 * w.ffp);
        m_act = std::max(m_act, (size_t)w.ffp);
      } else if (f.kind == nvc_karuzen_mlp::Moe) {
        w.effp = pad64(f.expert_ff);
        w.Ep = pad64(f.experts + 1);
        if ((rc = zalloc(r, &w.router, (size_t)w.Ep * Wp * esz)) || (rc = zalloc(r, &w.corr, f.experts * 4))) return rc;
        m_Ep = std::max(m_Ep, (size_t)w.Ep);
        if ((rc = zalloc(r, &w.w_eup, (size_t)f.experts * w.effp * Wp * esz)) ||
            (rc = zalloc(r, &w.w_edown, (size_t)f.experts * Wp * w.effp * esz)))
          return rc;
        wbytes += (int64_t)esz * 2 * f.experts * f.expert_ff * cfg.width;
        want[p + "mlp.router"] = false;
        want[p + "mlp.correction"] = false;
        for (int e = 0; e < f.experts; ++e) {
          want[p + "mlp.e" + std::to_string(e) + ".up"] = false;
          want[p + "mlp.e" + std::to_string(e) + ".down"] = false;
        }
        if (f.shared_ff > 0) {
          w.sfp = pad64(f.shared_ff);
          if ((rc = zalloc(r, &w.w_sup, (size_t)w.sfp * Wp * esz)) || (rc = zalloc(r, &w.w_sdown, (size_t)Wp * w.sfp * esz))) return rc;
          wbytes += (int64_t)esz * 2 * f.shared_ff * cfg.width;
          for (const char* n : {"mlp.shared.up", "mlp.shared.down", "mlp.shared.sg"}) want[p + n] = false;
          m_su = std::max(m_su, (size_t)w.sfp);
        }
        m_hid = std::max(m_hid, (size_t)f.top * w.effp);
        // The tcgen05 tile is 128 rows: experts narrower than that (after padding) stay with the mma.sync product.
        w.moe_tc = use_moe_tc && w.effp >= 128 && Wp >= 128;
        const size_t rows = w.moe_tc ? moe_tiles((int)std::min<size_t>(T * f.top, 0x3fffffff), f.experts) * (size_t)128 : T * f.top;
        m_prow = std::max(m_prow, rows);
        if (w.moe_tc) m_tcrow = std::max(m_tcrow, rows);
        m_effp = std::max(m_effp, (size_t)w.effp);
        m_top = std::max(m_top, (size_t)f.top);
        m_E = std::max(m_E, (size_t)f.experts);
      }
    }
    if ((rc = zalloc(r, &embed, (size_t)Vp * Wp * esz))) return rc;
    if ((rc = zalloc(r, &fw, cfg.width * 4)) || (rc = zalloc(r, &fb, cfg.width * 4)) || (rc = zalloc(r, &falpha, 4))) return rc;
    for (const char* n : {"embed", "final.norm", "final.norm.b", "final.norm.alpha"}) want[n] = false;
    r->weight_bytes = wbytes + (int64_t)esz * cfg.vocab * cfg.width;
    cache.resize(runs.size());
    for (size_t k = 0; k < runs.size(); ++k)
      if ((rc = zalloc(r, &cache[k], slots * L[runs[k].layer].kvp * esz))) return rc;
    // activations (zeroed once: padding columns are never written)
    if ((rc = zalloc(r, &x0, T * Wp * 4)) || (rc = zalloc(r, &res, T * Wp * 4)) || (rc = zalloc(r, &mix, T * Wp * 4)) ||
        (rc = zalloc(r, &ffo, T * Wp * 4)) || (rc = zalloc(r, &down, T * m_down * 4)))
      return rc;
    if ((rc = zalloc(r, &h, T * Wp * esz)) || (rc = zalloc(r, &cq, T * m_cq * esz)) || (rc = zalloc(r, &q, T * m_q * esz)) ||
        (rc = zalloc(r, &qabs, T * m_qabs * esz)) || (rc = zalloc(r, &olat, T * m_qabs * esz)) || (rc = zalloc(r, &ao, T * m_ao * esz)))
      return rc;
    if (m_gu && ((rc = zalloc(r, &gu, T * m_gu * esz)) || (rc = zalloc(r, &act, T * m_act * esz)))) return rc;
    if (m_top) {
      if ((rc = zalloc(r, &tk_idx, T * m_top * 4)) || (rc = zalloc(r, &tk_w, T * m_top * 4)) || (rc = zalloc(r, &gate, T * 4)) || (rc = zalloc(r, &zlog, T * m_Ep * 4)) ||
          (rc = zalloc(r, &offsets, (m_E + 1) * 4)) || (rc = zalloc(r, &src_rows, m_prow * 4)) || (rc = zalloc(r, &pos, T * m_top * 4)) ||
          (rc = zalloc(r, &hid, m_prow * m_effp * esz)) || (rc = zalloc(r, &y, m_prow * Wp * 4)))
        return rc;
      if (m_tcrow && ((rc = zalloc(r, &xs, m_tcrow * Wp * esz)) || (rc = zalloc(r, &tile_group, (m_tcrow / 128 + 1) * 4)))) return rc;
      if (m_su && ((rc = zalloc(r, &su, T * m_su * esz)) || (rc = zalloc(r, &sd, T * Wp * 4)))) return rc;
    }
    if ((rc = zalloc(r, &hn, (size_t)r->max_logit_rows * Wp * esz))) return rc;
    {
      size_t chunks = 1;
      for (auto& ly : cfg.layers) chunks = std::max(chunks, (size_t)(ly.mixer.heads + 15) / 16);
      attn_ws_bytes = std::min<size_t>((size_t)r->opt.max_num_seqs, (size_t)2 * ctx->num_sms) * chunks * 16 * 8 * (2 + 128) * sizeof(float);
      if ((rc = zalloc(r, &attn_ws, attn_ws_bytes))) return rc;
    }
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
    if (name == "embed") {
      if (!shape_is(cfg.vocab, W)) return bad();
      rc = put_matrix(r, embed, Wp, 0, 0, v.data(), cfg.vocab, W, W, 1);
    } else if (name == "final.norm") { if (n != (size_t)W) return bad(); rc = put_f32(r, fw, v.data(), W); }
    else if (name == "final.norm.b") { if (n != (size_t)W) return bad(); rc = put_f32(r, fb, v.data(), W); }
    else if (name == "final.norm.alpha") { if (n != 1) return bad(); rc = put_f32(r, falpha, v.data(), 1); }
    else {
      const size_t dot = name.find('.');
      const int li = atoi(name.substr(1, dot - 1).c_str());
      const std::string sub = name.substr(dot + 1);
      const auto& m = cfg.layers[li].mixer;
      const auto& f = cfg.layers[li].mlp;
      LayerW& w = L[li];
      if (sub == "norm1") { if (n != (size_t)W) return bad(); rc = put_f32(r, w.nw, v.data(), W); }
      else if (sub == "norm1.b") { if (n != (size_t)W) return bad(); rc = put_f32(r, w.nb, v.data(), W); }
      else if (sub == "norm1.alpha") { if (n != 1) return bad(); rc = put_f32(r, w.nalpha, v.data(), 1); }
      else if (sub == "mix.dq") { if (!shape_is(m.q_rank, W)) return bad(); rc = put_matrix(r, w.w_down, Wp, 0, 0, v.data(), m.q_rank, W, W, 1); }
      else if (sub == "mix.dkv") { if (!shape_is(m.kv_rank, W)) return bad(); rc = put_matrix(r, w.w_down, Wp, w.qrp, 0, v.data(), m.kv_rank, W, W, 1); }
      else if (sub == "mix.dq.norm") { if (n != (size_t)m.q_rank) return bad(); rc = put_f32(r, w.dq_norm, v.data(), n); }
      else if (sub == "mix.dkv.norm") { if (n != (size_t)m.kv_rank) return bad(); rc = put_f32(r, w.dkv_norm, v.data(), n); }
      else if (sub == "mix.uq") {
        if (!shape_is((int64_t)m.heads * m.dim, m.q_rank)) return bad();
        for (int hh = 0; hh < m.heads && !rc; ++hh)
          rc = put_matrix(r, w.w_uq, w.qrp, (size_t)hh * w.dimp, 0, v.data() + (size_t)hh * m.dim * m.q_rank, m.dim, m.q_rank, m.q_rank, 1);
      } else if (sub == "mix.uk") {      // stored transposed per head: ukT[h][c][d] = uk[h * dim + d][c]
        if (!shape_is((int64_t)m.heads * m.dim, m.kv_rank)) return bad();
        for (int hh = 0; hh < m.heads && !rc; ++hh)
          rc = put_matrix(r, w.w_ukT, w.dimp, (size_t)hh * w.kvp, 0, v.data() + (size_t)hh * m.dim * m.kv_rank, m.kv_rank, m.dim, 1, m.kv_rank);
      } else if (sub == "mix.uv") {
        if (!shape_is((int64_t)m.heads * m.vdim, m.kv_rank)) return bad();
        for (int hh = 0; hh < m.heads && !rc; ++hh)
          rc = put_matrix(r, w.w_uv, w.kvp, (size_t)hh * w.vdp, 0, v.data() + (size_t)hh * m.vdim * m.kv_rank, m.vdim, m.kv_rank, m.kv_rank, 1);
      } else if (sub == "mix.o") {
        if (!shape_is(W, (int64_t)m.heads * m.vdim)) return bad();
        for (int hh = 0; hh < m.heads && !rc; ++hh)
          rc = put_matrix(r, w.w_o, (size_t)m.heads * w.vdp, 0, (size_t)hh * w.vdp, v.data() + (size_t)hh * m.vdim, W, m.vdim,
                          (size_t)m.heads * m.vdim, 1);
      } else if (sub == "mlp.gate" || sub == "mlp.up") {
        if (!shape_is(f.ff, W)) return bad();
        const bool up = sub == "mlp.up";
        if (!use_tc) {                   // [gate rows; up rows at ffp]: two halves for the stand-alone activation kernel
          rc = put_matrix(r, w.w_gu, Wp, up ? w.ffp : 0, 0, v.data(), f.ff, W, W, 1);
        } else {                         // groups of 16 rows, gate group then up group: the fused epilogue meets both in one thread
          for (int g0 = 0; g0 < f.ff && !rc; g0 += 16)
            rc = put_matrix(r, w.w_gu, Wp, (size_t)2 * g0 + (up ? 16 : 0), 0, v.data() + (size_t)g0 * W, std::min(16, f.ff - g0), W, W, 1);
        }
      }
      else if (sub == "mlp.down") { if (!shape_is(W, f.ff)) return bad(); rc = put_matrix(r, w.w_fdown, w.ffp, 0, 0, v.data(), W, f.ff, f.ff, 1); }
      else if (sub == "mlp.router") { if (!shape_is(f.experts, W)) return bad(); rc = put_matrix(r, w.router, Wp, 0, 0, v.data(), f.experts, W, W, 1); }
      else if (sub == "mlp.correction") { if (n != (size_t)f.experts) return bad(); rc = put_f32(r, w.corr, v.data(), n); }
      else if (sub == "mlp.shared.up") { if (!shape_is(f.shared_ff, W)) return bad(); rc = put_matrix(r, w.w_sup, Wp, 0, 0, v.data(), f.shared_ff, W, W, 1); }
      else if (sub == "mlp.shared.down") { if (!shape_is(W, f.shared_ff)) return bad(); rc = put_matrix(r, w.w_sdown, w.sfp, 0, 0, v.data(), W, f.shared_ff, f.shared_ff, 1); }
      else if (sub == "mlp.shared.sg") { if (n != (size_t)W) return bad(); rc = put_matrix(r, w.router, Wp, f.experts, 0, v.data(), 1, W, W, 1); }
      else if (sub.rfind("mlp.e", 0) == 0) {
        const size_t d2 = sub.find('.', 5);
        const int e = atoi(sub.substr(5, d2 - 5).c_str());
        const std::string part = sub.substr(d2 + 1);
        if (part == "up") {
          if (!shape_is(f.expert_ff, W)) return bad();
          rc = put_matrix(r, w.w_eup, Wp, (size_t)e * w.effp, 0, v.data(), f.expert_ff, W, W, 1);
        } else {
          if (!shape_is(W, f.expert_ff)) return bad();
          rc = put_matrix(r, w.w_edown, w.effp, (size_t)e * Wp, 0, v.data(), W, f.expert_ff, f.expert_ff, 1);
        }
      }
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

  // Prompt portions of this step go through the tcgen05 paged-prefill kernel when the storage is bf16, the padded latent is
  // that kernel's head size and the block size is one it tiles; shorter portions stay with the latent kernel (a 128-row
  // query tile per head would be mostly empty).
  // 128-row tiles that P sorted pairs of E groups can take when every group is padded to a multiple of 128
  static int moe_tiles(int P, int E) { return (int)(((int64_t)P + (int64_t)E * 127 + 127) / 128); }
  static constexpr int kFlashMinChunk = 64;
  bool flash_portions(const nvc_runner* r, const nvc_step_shape& s, int kvp) const {
    const int bs = r->opt.kvcache_block_size;
    return use_flash && !s.decode && kvp == 128 && s.num_decode < s.B && s.max_chunk >= kFlashMinChunk &&
           (bs == 16 || bs == 32 || bs == 64 || bs % 128 == 0);
  }

  int tap(nvc_runner* r, int run, int N) {
    const size_t need = (size_t)(run + 1) * N * cfg.width;
    NVC_REQUIRE(r->ctx, need <= tap_cap, NVC_ENOMEM, "residual tap buffer too small");
    NVC_CUDA_CHECK(r->ctx, cudaMemcpy2DAsync(tap_host + (size_t)run * N * cfg.width, (size_t)cfg.width * 4, res, (size_t)Wp * 4,
                                             (size_t)cfg.width * 4, N, cudaMemcpyDeviceToHost, r->stream));
    return NVC_OK;
  }

  int forward(nvc_runner* r, const nvc_step_shape& s) override {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const int N = s.N, W = cfg.width;
    const int odt = dt;   // storage format of activations
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(r->stream, &cap);
    prof_on = prof_armed && cap == cudaStreamCaptureStatusNone;
    if (prof_on) prof_armed = false;
    mark(r, "start");
    int rc = nvc_embed_gather_f32(ctx, r->d_ids, embed, dt, Wp, x0, Wp, N, W, st);
    if (rc) return rc;
    mark(r, "embed");
    const float *a0 = nullptr, *a1 = nullptr;     // sums not yet added to the residual stream
    bool first = true;
    for (size_t k = 0; k < runs.size(); ++k) {
      const int li = runs[k].layer;
      const auto& m = cfg.layers[li].mixer;
      const auto& f = cfg.layers[li].mlp;
      LayerW& w = L[li];
      if (tap_host && !first) {
        // debug: land the previous run's sums first, copy the stream out, then open this run
        if ((rc = nvc_dyt_norm(ctx, res, a0, a1, nullptr, res, Wp, nullptr, nullptr, nullptr, nullptr, odt, 0, nullptr, N, W, st))) return rc;
        if ((rc = tap(r, (int)k - 1, N))) return rc;
        a0 = a1 = nullptr;
      }
      rc = nvc_dyt_norm(ctx, first ? x0 : res, a0, a1, runs[k].readd_embedding ? x0 : nullptr, res, Wp, w.nw, w.nb, w.nalpha, h, odt, Wp,
                        nullptr, N, W, st);
      if (rc) return rc;
      first = false;
      mark(r, "dyt_norm");
      // ---- mixer
      const int dl = w.qrp + w.kvp;
      if ((rc = linear(r, h, Wp, w.w_down, down, dl, NVC_DT_F32, N, dl, Wp))) return rc;
      mark(r, "gemm_down_latents");
      if ((rc = nvc_latent_norm_store(ctx, down, dl, m.q_rank, w.qrp, m.kv_rank, w.dq_norm, w.dkv_norm, cfg.eps, cq, w.qrp, cache[k],
                                      w.kvp, r->d_slots, dt, N, st)))
        return rc;
      mark(r, "latent_norm_store");
      const int qw = m.heads * w.dimp, lw = m.heads * w.kvp, vw = m.heads * w.vdp;
      if ((rc = linear(r, cq, w.qrp, w.w_uq, q, qw, odt, N, qw, w.qrp))) return rc;
      mark(r, "gemm_uq");
      if ((rc = nvc_linear(ctx, q, qw, w.dimp, w.w_ukT, w.dimp, (int64_t)w.kvp * w.dimp, qabs, lw, w.kvp, dt, odt, N, w.kvp, w.dimp,
                           m.heads, NVC_ACT_NONE, st)))
        return rc;
      mark(r, "absorb_uk");
      if (flash_portions(r, s, w.kvp)) {
        // Long prompt portions: in the absorbed form a layer is multi-query attention with ONE key / value head whose
        // key and value are both the cached latent row, so the tcgen05 paged-prefill kernel runs it unchanged (k = v =
        // this run's pool, head size = the padded latent width).  One-token sequences of a mixed step come first in the
        // batch and keep the decode path of the latent kernel.
        const int nd = s.num_decode, cap = r->max_blocks_cap;
        const nvc_bf16* qb = reinterpret_cast<const nvc_bf16*>(qabs);
        nvc_bf16* ob = reinterpret_cast<nvc_bf16*>(olat);
        const nvc_bf16* pool = reinterpret_cast<const nvc_bf16*>(cache[k]);
        if (nd > 0 && (rc = nvc_latent_attn_paged(ctx, qabs, lw, cache[k], w.kvp, r->d_bt, cap, r->d_ctx, nullptr, nd, 1, m.heads, m.kv_rank,
                                                  w.kvp, r->opt.kvcache_block_size, m.scale, olat, lw, dt, attn_ws, attn_ws_bytes, st)))
          return rc;
        if ((rc = nvc_prefill_attn_paged(ctx, qb + (size_t)nd * lw, lw, pool, pool, r->d_bt + (size_t)nd * cap, cap, r->d_ctx + nd,
                                         nd ? r->d_cu2 : r->d_cu, s.B - nd, s.N - nd, s.max_chunk, m.heads, 1, w.kvp,
                                         r->opt.kvcache_block_size, r->opt.num_kvcache_blocks, m.scale, ob + (size_t)nd * lw, st)))
          return rc;
      } else if ((rc = nvc_latent_attn_paged(ctx, qabs, lw, cache[k], w.kvp, r->d_bt, r->max_blocks_cap, r->d_ctx,
                                             s.decode ? nullptr : r->d_cu, s.B, s.decode ? 1 : s.max_seqlen, m.heads, m.kv_rank, w.kvp,
                                             r->opt.kvcache_block_size, m.scale, olat, lw, dt, attn_ws, attn_ws_bytes, st))) {
        return rc;
      }
      mark(r, "latent_attn");
      if ((rc = nvc_linear(ctx, olat, lw, w.kvp, w.w_uv, w.kvp, (int64_t)w.vdp * w.kvp, ao, vw, w.vdp, dt, odt, N, w.vdp, w.kvp, m.heads,
                           NVC_ACT_NONE, st)))
        return rc;
      mark(r, "absorb_uv");
      if ((rc = linear(r, ao, vw, w.w_o, mix, Wp, NVC_DT_F32, N, Wp, vw))) return rc;
      mark(r, "gemm_o");
      a0 = mix;
      a1 = nullptr;
      // ---- feed-forward
      if (f.kind == nvc_karuzen_mlp::Dense) {
        if (use_tc) {                    // gate_up projection with the gated gelu in the GEMM's epilogue
          if ((rc = nvc_gemm_bf16_gelu_mul(ctx, reinterpret_cast<const nvc_bf16*>(h), Wp, reinterpret_cast<const nvc_bf16*>(w.w_gu),
                                           reinterpret_cast<nvc_bf16*>(act), w.ffp, N, w.ffp, Wp, st)))
            return rc;
          mark(r, "gemm_gate_up");
        } else {
          if ((rc = linear(r, h, Wp, w.w_gu, gu, 2 * w.ffp, odt, N, 2 * w.ffp, Wp))) return rc;
          mark(r, "gemm_gate_up");
          if ((rc = nvc_act_mul(ctx, gu, 2 * w.ffp, act, w.ffp, dt, N, f.ff, w.ffp, NVC_ACT_GELU_TANH_MUL, st))) return rc;
          mark(r, "gelu_mul");
        }
        if ((rc = linear(r, act, w.ffp, w.w_fdown, ffo, Wp, NVC_DT_F32, N, Wp, w.ffp))) return rc;
        mark(r, "gemm_ff_down");
        a1 = ffo;
      } else if (f.kind == nvc_karuzen_mlp::Moe) {
        const int P = N * f.top;
        // router logits (and the shared gate's, one more row) as one product with fp32 accumulation and output
        // (all Ep padded columns on the tcgen05 kernel - the padding rows of the matrix are zero - or the logical ones on the FMA kernel)
        if (use_tc) {
          if ((rc = linear(r, h, Wp, w.router, zlog, w.Ep, NVC_DT_F32, N, w.Ep, Wp))) return rc;
        } else if ((rc = nvc_linear(ctx, h, Wp, 0, w.router, Wp, 0, zlog, w.Ep, 0, dt, NVC_DT_F32, N, f.experts + 1, Wp, 1, NVC_ACT_NONE, st))) {
          return rc;
        }
        if ((rc = nvc_moe_route_logits(ctx, zlog, w.Ep, w.corr, f.experts, f.top, f.router_scale, w.w_sup ? f.experts : -1, tk_idx, tk_w,
                                       w.w_sup ? gate : nullptr, N, st)))
          return rc;
        mark(r, "moe_route");
        if (w.moe_tc) {
          // groups padded to the 128-row tile of the tcgen05 kernel; which tiles exist is a device table (no host round trip)
          const int tiles = moe_tiles(P, f.experts), mcap = tiles * 128;
          if ((rc = nvc_moe_sort_padded(ctx, tk_idx, N, f.top, f.experts, 128, offsets, src_rows, pos, tile_group, tiles, st))) return rc;
          mark(r, "moe_sort");
          if ((rc = nvc_gather_rows_bf16(ctx, reinterpret_cast<const nvc_bf16*>(h), Wp, src_rows, offsets + f.experts,
                                         reinterpret_cast<nvc_bf16*>(xs), Wp, mcap, Wp, st)))
            return rc;
          mark(r, "moe_gather");
          if ((rc = nvc_gemm_bf16_grouped(ctx, reinterpret_cast<const nvc_bf16*>(xs), Wp, reinterpret_cast<const nvc_bf16*>(w.w_eup), hid,
                                          w.effp, NVC_DT_BF16, mcap, w.effp, Wp, tile_group, f.experts, NVC_ACT_RELU2, st)))
            return rc;
          mark(r, "moe_up");
          if ((rc = nvc_gemm_bf16_grouped(ctx, reinterpret_cast<const nvc_bf16*>(hid), w.effp, reinterpret_cast<const nvc_bf16*>(w.w_edown), y,
                                          Wp, NVC_DT_F32, mcap, Wp, w.effp, tile_group, f.experts, NVC_ACT_NONE, st)))
            return rc;
          mark(r, "moe_down");
        } else {
        if ((rc = nvc_moe_sort(ctx, tk_idx, N, f.top, f.experts, offsets, src_rows, pos, st))) return rc;
        mark(r, "moe_sort");
        if ((rc = nvc_linear_grouped(ctx, h, Wp, src_rows, w.w_eup, Wp, (int64_t)w.effp * Wp, hid, w.effp, offsets, f.experts, P, dt, odt,
                                     w.effp, Wp, NVC_ACT_RELU2, st)))
          return rc;
        mark(r, "moe_up");
        if ((rc = nvc_linear_grouped(ctx, hid, w.effp, nullptr, w.w_edown, w.effp, (int64_t)Wp * w.effp, y, Wp, offsets, f.experts, P, dt,
                                     NVC_DT_F32, Wp, w.effp, NVC_ACT_NONE, st)))
          return rc;
        mark(r, "moe_down");
        }
        if (w.w_sup) {
          if (use_tc) {      // squared relu in the epilogue of the up-projection
            if ((rc = nvc_gemm_bf16_act(ctx, reinterpret_cast<const nvc_bf16*>(h), Wp, reinterpret_cast<const nvc_bf16*>(w.w_sup), su, w.sfp,
                                        NVC_DT_BF16, N, w.sfp, Wp, NVC_ACT_RELU2, st)))
              return rc;
          } else {
            if ((rc = linear(r, h, Wp, w.w_sup, su, w.sfp, odt, N, w.sfp, Wp))) return rc;
            if ((rc = nvc_act_mul(ctx, su, w.sfp, su, w.sfp, dt, N, f.shared_ff, w.sfp, NVC_ACT_RELU2, st))) return rc;
          }
          if ((rc = linear(r, su, w.sfp, w.w_sdown, sd, Wp, NVC_DT_F32, N, Wp, w.sfp))) return rc;
          mark(r, "shared_expert");
        }
        if ((rc = nvc_moe_combine(ctx, y, NVC_DT_F32, Wp, pos, tk_w, f.top, w.w_sup ? sd : nullptr, NVC_DT_F32, Wp, w.w_sup ? gate : nullptr,
                                  ffo, Wp, N, W, st)))
          return rc;
        mark(r, "moe_combine");
        a1 = ffo;
      }
    }
    if (tap_host) {
      if ((rc = nvc_dyt_norm(ctx, res, a0, a1, nullptr, res, Wp, nullptr, nullptr, nullptr, nullptr, odt, 0, nullptr, N, W, st))) return rc;
      if ((rc = tap(r, (int)runs.size() - 1, N))) return rc;
      a0 = a1 = nullptr;
      tap_host = nullptr;      // one step only
    }
    // ---- head: final norm of the wanted rows (the last run's sums are added on the way), logits against the embedding
    rc = nvc_dyt_norm(ctx, res, a0, a1, nullptr, nullptr, Wp, fw, fb, falpha, hn, odt, Wp, s.decode ? nullptr : r->d_last_rows, s.rows, W, st);
    if (rc) return rc;
    mark(r, "final_norm");
    rc = linear(r, hn, Wp, embed, r->logits, Vp, NVC_DT_F32, s.rows, Vp, Wp);
    mark(r, "lm_head");
    finish_profile(r);
    return rc;
  }
};

}  // namespace

nvc_model_body* nvc_make_karuzen_body(nvc_runner* r, const nvc_karuzen_config& cfg, int* status) {
  KaruzenBody* b = new KaruzenBody();
  b->cfg = cfg;
  *status = b->init(r);
  return b;
}
