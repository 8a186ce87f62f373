// Fefozen model body behind the step executor (runner.cu): weights, paged latent pools, recurrent state slots, the layer loop.
//
// One layer over the N query rows of a step (x <- x + n1b(mixer(n1(x))); x <- x + n2b(ff(n2(x))); norm weights stored around zero):
//   nvc_rms_norm_sandwich     x += norm-behind(previous sublayer's output); h = norm-in-front(x): one pass over the row
//   latent attention:
//     linear w_in             ONE fused projection of everything the mixer reads from h, fp32 out: [dq | dkv | gate]
//     nvc_latent_norm_store_rot  RMS norms of both latents; the token's cache row [normed latent | rotated shared key part] goes
//                             into this layer's paged pool (a layer with kv_from reads the named layer's pool and stores nothing)
//     linear uq (fp32 out) -> nvc_head_split_rot: unrotated query parts, rotated parts straight into the absorbed queries
//     linear uk^T per head    unrotated query parts carried into the latent space (absorbed key up-projection)
//     attention               softmax over the cached rows: in the absorbed form a layer is multi-query attention with ONE key /
//                             value head - key = the whole row (kv_rank + rot_dim numbers), value = its first kv_rank numbers.
//                             nvc_attn_paged_wide (sink in its epilogue), or the tcgen05 paged-prefill kernel for long portions
//                             when the row has 128 numbers (the sink joins the denominator in its epilogue; the rotated part
//                             rides along as value columns that the value up-projection never reads)
//     linear uv per head (fp32 out) -> nvc_head_gate (sigmoid gate of h) -> linear o
//   delta:
//     linear w_in             [q | k | v | beta | a | gate], fp32 out
//     nvc_delta_prep_run      short convolutions + silu, unit q / k, decay and beta;  nvc_delta_rule_scan: the recurrence over the
//                             state slots of the step's sequences (and the convolution state);  nvc_head_gate_w: per-head root mean
//                             square, weight, silu gate;  linear o
//   dense ff:  linear up with the tanh-gelu in its epilogue -> linear down (fp32)
//   moe ff:    router product (fp32) -> softmax scores, biased top-k -> sort -> grouped [gate; up] -> clamped gated unit ->
//              grouped down (fp32) -> combine (identity experts add the token's own h)
// The residual sum itself happens in the NEXT nvc_rms_norm_sandwich (or the final one), in fp32.
//
// Feature dimensions that a dense matrix product sums over or produces are padded to multiples of 64 in the weight and activation
// buffers (zeros), so that the tcgen05 GEMMs (K % 64, N % 16) take every such product of the bf16 mode; heads are not padded.
#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "body_common.h"
#include "model_config.h"
#include "runner.h"

namespace {

inline int pad8(int v) { return (v + 7) / 8 * 8; }

constexpr float kGluAlpha = 1.702f;      // g * sigmoid(alpha g) of the experts' gated unit
constexpr float kUnitEps = 1e-6f;        // inside the root of the delta rule's unit vectors

struct FLayerW {
  float *n1 = nullptr, *n1b = nullptr, *n2 = nullptr, *n2b = nullptr;
  void* w_in = nullptr;                 // [np, Wp]
  int np = 0;
  int g_off = 0;
  // latent attention
  int kv_off = 0;                       // first column of the key / value down-projection in a projection row
  float *dq_norm = nullptr, *dkv_norm = nullptr, *sink = nullptr;
  void* w_uq = nullptr;                 // [uqn, qrp]
  void* w_ukT = nullptr;                // [heads][kv_rank, dimp]
  void* w_uv = nullptr;                 // [heads][vdim, kvp]
  int qrp = 0, uqn = 0, dimp = 0, kvp = 0, Dk = 0, ldpool = 0, ldqa = 0, ldol = 0;
  void* pool = nullptr;                 // [slots, ldpool]: [normed latent | rotated key part] per token (own layers)
  const float* rot = nullptr;
  // delta
  int q_off = 0, k_off = 0, v_off = 0, b_off = 0, a_off = 0;
  float *conv_w = nullptr, *conv_state = nullptr, *A_log = nullptr, *dt_bias = nullptr, *onorm = nullptr, *state = nullptr;
  // both
  void* w_o = nullptr;                  // [Wp, owp]
  int owp = 0;
  // dense ff
  void *w_up = nullptr, *w_down = nullptr;
  int ffp = 0;
  // moe
  void* router = nullptr;               // [Ep, Wp]
  float* corr = nullptr;
  int Ep = 0, effp = 0;
  void *w_egu = nullptr, *w_edown = nullptr;   // [E][2 effp, Wp] (gate rows, then up rows at effp), [E][Wp, effp]
  bool moe_tc = false;
};

struct FefozenBody : nvc_body_base {
  nvc_fefozen_config cfg;
  int Wp = 0, Vp = 0;
  int state_slots = 0;
  bool use_flash = true, use_moe_tc = true;
  std::vector<FLayerW> L;
  void* embed = nullptr;
  float* fw = nullptr;
  std::map<std::string, bool> want;
  std::map<std::pair<int, uint32_t>, float*> rot_tables;
  // activations
  float *x0 = nullptr, *res = nullptr, *proj = nullptr, *mix = nullptr, *ffo = nullptr, *qf = nullptr, *hv = nullptr;
  float *rq = nullptr, *rk = nullptr, *rv = nullptr, *ro = nullptr, *gb = nullptr, *zlog = nullptr, *tk_w = nullptr, *y = nullptr;
  void *h = nullptr, *cq = nullptr, *qn = nullptr, *qabs = nullptr, *olat = nullptr, *ao = nullptr, *act = nullptr, *hn = nullptr;
  void *hid2 = nullptr, *hid = nullptr, *xs = nullptr;
  int32_t *tk_idx = nullptr, *offsets = nullptr, *src_rows = nullptr, *pos = nullptr, *tile_group = nullptr;
  float* tap_host = nullptr;
  size_t tap_cap = 0;

  int vocab() const override { return cfg.vocab; }
  int logits_ld() const override { return Vp; }
  int layer_runs() const override { return (int)cfg.layers.size(); }
  int width() const override { return cfg.width; }
  int num_state_slots() const override { return state_slots; }
  int64_t cache_bytes_per_token() const override {
    int64_t b = 0;
    for (size_t i = 0; i < cfg.layers.size(); ++i)
      if (cfg.layers[i].kind == nvc_fefozen_layer::Latent && cfg.layers[i].lat.kv_from < 0) b += (int64_t)L[i].ldpool * (int64_t)esz;
    return b;
  }
  int set_residual_tap(float* host, size_t cap) override {
    tap_host = host;
    tap_cap = host ? cap : 0;
    return NVC_OK;
  }

  static int moe_tiles(int pairs, int experts) { return (pairs + experts * 127 + 127) / 128; }

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
    use_tc = dt == NVC_DT_BF16 && !(getenv("NVC_FEFOZEN_TC") && atoi(getenv("NVC_FEFOZEN_TC")) == 0);
    use_flash = use_tc && !(getenv("NVC_FEFOZEN_FLASH") && atoi(getenv("NVC_FEFOZEN_FLASH")) == 0);
    use_moe_tc = use_tc && !(getenv("NVC_FEFOZEN_MOE_TC") && atoi(getenv("NVC_FEFOZEN_MOE_TC")) == 0);
    Wp = pad64(cfg.width);
    Vp = pad64(cfg.vocab);
    state_slots = cfg.has_state() ? r->opt.max_num_seqs : 0;
    const size_t T = (size_t)std::max(r->opt.max_num_batched_tokens, r->opt.max_num_seqs);
    const size_t slots = (size_t)r->opt.num_kvcache_blocks * r->opt.kvcache_block_size;
    int rc;
    L.resize(cfg.layers.size());
    size_t m_np = 0, m_qrp = 0, m_uqn = 0, m_qn = 0, m_qa = 0, m_ol = 0, m_hv = 0, m_ow = 0, m_ff = 0, m_dqk = 0, m_dv = 0, m_gb = 0;
    size_t m_Ep = 0, m_top = 0, m_E = 0, m_hid = 0, m_pairs_rows = 0, m_tiles = 0;
    int64_t wbytes = 0;
    const int W = cfg.width;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
      const auto& ly = cfg.layers[i];
      FLayerW& w = L[i];
      const std::string p = "l" + std::to_string(i) + ".";
      if ((rc = zalloc(r, &w.n1, W * 4)) || (rc = zalloc(r, &w.n1b, W * 4))) return rc;
      want[p + "norm1"] = false;
      want[p + "norm1b"] = false;
      int ow = 0;
      if (ly.kind == nvc_fefozen_layer::Latent) {
        const auto& a = ly.lat;
        const bool own = a.kv_from < 0;
        w.Dk = a.kv_rank + a.rot_dim;
        NVC_REQUIRE(ctx, w.Dk <= 512, NVC_ESHAPE, "kv_rank + rot_dim above 512");
        w.kv_off = a.q_rank;
        w.g_off = a.q_rank + (own ? w.Dk : 0);
        ow = a.heads * a.vdim;
        w.np = pad64(w.g_off + ow);
        w.qrp = pad64(a.q_rank);
        w.uqn = pad64(a.heads * (a.dim + a.rot_dim));
        w.dimp = pad8(a.dim);
        w.kvp = pad8(a.kv_rank);
        w.ldpool = pad8(w.Dk);
        w.ldqa = pad8(a.heads * w.Dk);
        w.ldol = pad8(a.heads * w.Dk);          // room for value columns as wide as the key (the tcgen05 route)
        if ((rc = zalloc(r, &w.dq_norm, a.q_rank * 4)) || (rc = zalloc(r, &w.w_uq, (size_t)w.uqn * w.qrp * esz)) ||
            (rc = zalloc(r, &w.w_ukT, (size_t)a.heads * a.kv_rank * w.dimp * esz)) || (rc = zalloc(r, &w.w_uv, (size_t)a.heads * a.vdim * w.kvp * esz)))
          return rc;
        for (const char* n : {"mix.dq", "mix.dq.norm", "mix.uq", "mix.uk", "mix.uv", "mix.g", "mix.o"}) want[p + n] = false;
        if (own) {
          if ((rc = zalloc(r, &w.dkv_norm, a.kv_rank * 4)) || (rc = zalloc(r, &w.pool, slots * w.ldpool * esz))) return rc;
          want[p + "mix.dkv"] = false;
          want[p + "mix.dkv.norm"] = false;
        }
        if (a.sink) {
          if ((rc = zalloc(r, &w.sink, a.heads * 4))) return rc;
          want[p + "mix.sink"] = false;
        }
        if ((rc = rotary_table(r, a.rot, &w.rot))) return rc;
        wbytes += (int64_t)esz * ((int64_t)(a.q_rank + (own ? w.Dk : 0) + ow) * W + (int64_t)a.heads * (a.dim + a.rot_dim) * a.q_rank +
                                  (int64_t)a.heads * (a.dim + a.vdim) * a.kv_rank + (int64_t)W * ow);
        m_qrp = std::max(m_qrp, (size_t)w.qrp);
        m_uqn = std::max(m_uqn, (size_t)w.uqn);
        m_qn = std::max(m_qn, (size_t)a.heads * w.dimp);
        m_qa = std::max(m_qa, (size_t)w.ldqa);
        m_ol = std::max(m_ol, (size_t)w.ldol);
        m_hv = std::max(m_hv, (size_t)ow);
      } else {
        const auto& d = ly.delta;
        const int qk = d.kv_heads * d.dim, vw = d.heads * d.vdim, C = 2 * qk + vw;
        w.q_off = 0; w.k_off = qk; w.v_off = 2 * qk; w.b_off = C; w.a_off = C + d.heads; w.g_off = C + 2 * d.heads;
        ow = vw;
        w.np = pad64(w.g_off + vw);
        if ((rc = zalloc(r, &w.conv_w, (size_t)C * d.taps * 4)) || (rc = zalloc(r, &w.conv_state, (size_t)state_slots * std::max(d.taps - 1, 1) * C * 4)) ||
            (rc = zalloc(r, &w.A_log, d.heads * 4)) || (rc = zalloc(r, &w.dt_bias, d.heads * 4)) || (rc = zalloc(r, &w.onorm, d.vdim * 4)) ||
            (rc = zalloc(r, &w.state, (size_t)state_slots * d.heads * d.dim * d.vdim * 4)))
          return rc;
        for (const char* n : {"mix.q", "mix.q.conv", "mix.k", "mix.k.conv", "mix.v", "mix.v.conv", "mix.b", "mix.a", "mix.A_log", "mix.dt_bias",
                              "mix.norm", "mix.g", "mix.o"})
          want[p + n] = false;
        wbytes += (int64_t)esz * ((int64_t)(C + 2 * d.heads + vw) * W + (int64_t)W * vw);
        m_dqk = std::max(m_dqk, (size_t)qk);
        m_dv = std::max(m_dv, (size_t)vw);
        m_gb = std::max(m_gb, (size_t)2 * d.heads);
      }
      w.owp = pad64(ow);
      if ((rc = zalloc(r, &w.w_in, (size_t)w.np * Wp * esz)) || (rc = zalloc(r, &w.w_o, (size_t)Wp * w.owp * esz))) return rc;
      m_np = std::max(m_np, (size_t)w.np);
      m_ow = std::max(m_ow, (size_t)w.owp);
      const auto& f = ly.mlp;
      if (f.kind != nvc_routed_mlp_spec::None) {
        if ((rc = zalloc(r, &w.n2, W * 4)) || (rc = zalloc(r, &w.n2b, W * 4))) return rc;
        want[p + "norm2"] = false;
        want[p + "norm2b"] = false;
      }
      if (f.kind == nvc_routed_mlp_spec::Dense) {
        w.ffp = pad64(f.ff);
        if ((rc = zalloc(r, &w.w_up, (size_t)w.ffp * Wp * esz)) || (rc = zalloc(r, &w.w_down, (size_t)Wp * w.ffp * esz))) return rc;
        want[p + "mlp.up"] = false;
        want[p + "mlp.down"] = false;
        wbytes += (int64_t)esz * 2 * f.ff * W;
        m_ff = std::max(m_ff, (size_t)w.ffp);
      } else if (f.kind == nvc_routed_mlp_spec::Moe) {
        const int Et = f.experts + f.identity;
        w.Ep = pad64(Et);
        w.effp = pad64(f.expert_ff);
        w.moe_tc = use_moe_tc && f.experts > 0 && w.effp >= 128;
        if ((rc = zalloc(r, &w.router, (size_t)w.Ep * Wp * esz)) || (rc = zalloc(r, &w.corr, Et * 4))) return rc;
        want[p + "mlp.router"] = false;
        want[p + "mlp.correction"] = false;
        if (f.experts > 0 &&
            ((rc = zalloc(r, &w.w_egu, (size_t)f.experts * 2 * w.effp * Wp * esz)) || (rc = zalloc(r, &w.w_edown, (size_t)f.experts * Wp * w.effp * esz))))
          return rc;
        for (int e = 0; e < f.experts; ++e)
          for (const char* n : {"gate", "up", "down"}) want[p + "mlp.e" + std::to_string(e) + "." + n] = false;
        wbytes += (int64_t)esz * ((int64_t)Et * W + (int64_t)f.experts * 3 * f.expert_ff * W);
        m_Ep = std::max(m_Ep, (size_t)w.Ep);
        m_top = std::max(m_top, (size_t)f.top);
        m_E = std::max(m_E, (size_t)Et);
        m_hid = std::max(m_hid, (size_t)w.effp);
        const size_t rows = w.moe_tc ? (size_t)moe_tiles((int)T * f.top, Et) * 128 : T * f.top;
        m_pairs_rows = std::max(m_pairs_rows, rows);
        if (w.moe_tc) m_tiles = std::max(m_tiles, (size_t)moe_tiles((int)T * f.top, Et));
      }
    }
    if ((rc = zalloc(r, &embed, (size_t)Vp * Wp * esz)) || (rc = zalloc(r, &fw, W * 4))) return rc;
    want["embed"] = false;
    want["final.norm"] = false;
    r->weight_bytes = wbytes + (int64_t)esz * cfg.vocab * W;
    // activations (zeroed once: padding columns are never written)
    if ((rc = zalloc(r, &x0, T * Wp * 4)) || (rc = zalloc(r, &res, T * Wp * 4)) || (rc = zalloc(r, &mix, T * Wp * 4)) ||
        (rc = zalloc(r, &ffo, T * Wp * 4)) || (rc = zalloc(r, &proj, T * m_np * 4)) || (rc = zalloc(r, &h, T * Wp * esz)) ||
        (rc = zalloc(r, &ao, T * m_ow * esz)) || (rc = zalloc(r, &hn, (size_t)r->max_logit_rows * Wp * esz)))
      return rc;
    if (m_uqn && ((rc = zalloc(r, &cq, T * m_qrp * esz)) || (rc = zalloc(r, &qf, T * m_uqn * 4)) || (rc = zalloc(r, &qn, T * m_qn * esz)) ||
                  (rc = zalloc(r, &qabs, T * m_qa * esz)) || (rc = zalloc(r, &olat, T * m_ol * esz)) || (rc = zalloc(r, &hv, T * m_hv * 4))))
      return rc;
    if (m_dv && ((rc = zalloc(r, &rq, T * m_dqk * 4)) || (rc = zalloc(r, &rk, T * m_dqk * 4)) || (rc = zalloc(r, &rv, T * m_dv * 4)) ||
                 (rc = zalloc(r, &ro, T * m_dv * 4)) || (rc = zalloc(r, &gb, T * m_gb * 4))))
      return rc;
    if (m_ff && (rc = zalloc(r, &act, T * m_ff * esz))) return rc;
    if (m_E) {
      if ((rc = zalloc(r, &zlog, T * m_Ep * 4)) || (rc = zalloc(r, &tk_idx, T * m_top * 4)) || (rc = zalloc(r, &tk_w, T * m_top * 4)) ||
          (rc = zalloc(r, &offsets, (m_E + 1) * 4)) || (rc = zalloc(r, &src_rows, m_pairs_rows * 4)) || (rc = zalloc(r, &pos, T * m_top * 4)) ||
          (rc = zalloc(r, &hid2, m_pairs_rows * 2 * m_hid * esz)) || (rc = zalloc(r, &hid, m_pairs_rows * m_hid * esz)) ||
          (rc = zalloc(r, &y, m_pairs_rows * Wp * 4)))
        return rc;
      if (m_tiles && ((rc = zalloc(r, &tile_group, m_tiles * 4)) || (rc = zalloc(r, &xs, m_pairs_rows * Wp * esz)))) return rc;
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
    auto vec = [&](float* dst, size_t len) { return n == len ? put_f32(r, dst, v.data(), len) : bad(); };
    int rc = NVC_OK;
    if (name == "embed") { if (!shape_is(cfg.vocab, W)) return bad(); rc = put_matrix(r, embed, Wp, 0, 0, v.data(), cfg.vocab, W, W, 1); }
    else if (name == "final.norm") rc = vec(fw, W);
    else {
      const size_t dot = name.find('.');
      const int li = atoi(name.substr(1, dot - 1).c_str());
      const std::string sub = name.substr(dot + 1);
      const auto& ly = cfg.layers[li];
      const auto& a = ly.lat;
      const auto& d = ly.delta;
      const auto& f = ly.mlp;
      FLayerW& w = L[li];
      const bool latent = ly.kind == nvc_fefozen_layer::Latent;
      auto in_rows = [&](int off, int rows) { return shape_is(rows, W) ? put_matrix(r, w.w_in, Wp, off, 0, v.data(), rows, W, W, 1) : bad(); };
      const int ow = latent ? a.heads * a.vdim : d.heads * d.vdim;
      const int qk = d.kv_heads * d.dim;
      if (sub == "norm1") rc = vec(w.n1, W);
      else if (sub == "norm1b") rc = vec(w.n1b, W);
      else if (sub == "norm2") rc = vec(w.n2, W);
      else if (sub == "norm2b") rc = vec(w.n2b, W);
      else if (sub == "mix.g") rc = in_rows(w.g_off, ow);
      else if (sub == "mix.o") { if (!shape_is(W, ow)) return bad(); rc = put_matrix(r, w.w_o, w.owp, 0, 0, v.data(), W, ow, ow, 1); }
      else if (latent && sub == "mix.dq") rc = in_rows(0, a.q_rank);
      else if (latent && sub == "mix.dkv") rc = in_rows(w.kv_off, w.Dk);
      else if (latent && sub == "mix.dq.norm") rc = vec(w.dq_norm, a.q_rank);
      else if (latent && sub == "mix.dkv.norm") rc = vec(w.dkv_norm, a.kv_rank);
      else if (latent && sub == "mix.sink") rc = vec(w.sink, a.heads);
      else if (latent && sub == "mix.uq") {
        if (!shape_is(a.heads * (a.dim + a.rot_dim), a.q_rank)) return bad();
        rc = put_matrix(r, w.w_uq, w.qrp, 0, 0, v.data(), a.heads * (a.dim + a.rot_dim), a.q_rank, a.q_rank, 1);
      } else if (latent && sub == "mix.uk") {
        // [heads * dim, kv_rank] -> per head the transposed block [kv_rank, dimp]: q' = W_uk,h^T q
        if (!shape_is(a.heads * a.dim, a.kv_rank)) return bad();
        for (int hh = 0; hh < a.heads && rc == NVC_OK; ++hh)
          rc = put_matrix(r, reinterpret_cast<uint8_t*>(w.w_ukT) + (size_t)hh * a.kv_rank * w.dimp * esz, w.dimp, 0, 0,
                          v.data() + (size_t)hh * a.dim * a.kv_rank, a.kv_rank, a.dim, 1, a.kv_rank);
      } else if (latent && sub == "mix.uv") {
        if (!shape_is(a.heads * a.vdim, a.kv_rank)) return bad();
        for (int hh = 0; hh < a.heads && rc == NVC_OK; ++hh)
          rc = put_matrix(r, reinterpret_cast<uint8_t*>(w.w_uv) + (size_t)hh * a.vdim * w.kvp * esz, w.kvp, 0, 0,
                          v.data() + (size_t)hh * a.vdim * a.kv_rank, a.vdim, a.kv_rank, a.kv_rank, 1);
      }
      else if (!latent && sub == "mix.q") rc = in_rows(w.q_off, qk);
      else if (!latent && sub == "mix.k") rc = in_rows(w.k_off, qk);
      else if (!latent && sub == "mix.v") rc = in_rows(w.v_off, ow);
      else if (!latent && sub == "mix.b") rc = in_rows(w.b_off, d.heads);
      else if (!latent && sub == "mix.a") rc = in_rows(w.a_off, d.heads);
      else if (!latent && (sub == "mix.q.conv" || sub == "mix.k.conv" || sub == "mix.v.conv")) {
        // [channels, taps] of the checkpoint -> tap-major [taps, all channels] (q, k, v side by side): a warp's lanes read neighbours
        const int rows = sub == "mix.v.conv" ? ow : qk, ch0 = sub == "mix.q.conv" ? 0 : (sub == "mix.k.conv" ? qk : 2 * qk), C = 2 * qk + ow;
        if (!shape_is(rows, d.taps)) return bad();
        std::vector<float> col(rows);
        for (int i = 0; i < d.taps && rc == NVC_OK; ++i) {
          for (int c = 0; c < rows; ++c) col[c] = v[(size_t)c * d.taps + i];
          rc = put_f32(r, w.conv_w + (size_t)i * C + ch0, col.data(), rows);
        }
      }
      else if (!latent && sub == "mix.A_log") rc = vec(w.A_log, d.heads);
      else if (!latent && sub == "mix.dt_bias") rc = vec(w.dt_bias, d.heads);
      else if (!latent && sub == "mix.norm") rc = vec(w.onorm, d.vdim);
      else if (sub == "mlp.up") { if (!shape_is(f.ff, W)) return bad(); rc = put_matrix(r, w.w_up, Wp, 0, 0, v.data(), f.ff, W, W, 1); }
      else if (sub == "mlp.down") { if (!shape_is(W, f.ff)) return bad(); rc = put_matrix(r, w.w_down, w.ffp, 0, 0, v.data(), W, f.ff, f.ff, 1); }
      else if (sub == "mlp.router") { if (!shape_is(f.experts + f.identity, W)) return bad(); rc = put_matrix(r, w.router, Wp, 0, 0, v.data(), f.experts + f.identity, W, W, 1); }
      else if (sub == "mlp.correction") rc = vec(w.corr, f.experts + f.identity);
      else if (sub.rfind("mlp.e", 0) == 0) {
        const size_t d2 = sub.find('.', 5);
        const int e = atoi(sub.substr(5, d2 - 5).c_str());
        const std::string part = sub.substr(d2 + 1);
        uint8_t* gu = reinterpret_cast<uint8_t*>(w.w_egu) + (size_t)e * 2 * w.effp * Wp * esz;
        if (part == "gate") { if (!shape_is(f.expert_ff, W)) return bad(); rc = put_matrix(r, gu, Wp, 0, 0, v.data(), f.expert_ff, W, W, 1); }
        else if (part == "up") { if (!shape_is(f.expert_ff, W)) return bad(); rc = put_matrix(r, gu, Wp, w.effp, 0, v.data(), f.expert_ff, W, W, 1); }
        else if (part == "down") {
          if (!shape_is(W, f.expert_ff)) return bad();
          rc = put_matrix(r, reinterpret_cast<uint8_t*>(w.w_edown) + (size_t)e * Wp * w.effp * esz, w.effp, 0, 0, v.data(), W, f.expert_ff, f.expert_ff, 1);
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

  int tap(nvc_runner* r, int run, int N) {
    const size_t need = (size_t)(run + 1) * N * cfg.width;
    NVC_REQUIRE(r->ctx, need <= tap_cap, NVC_ENOMEM, "residual tap buffer too small");
    NVC_CUDA_CHECK(r->ctx, cudaMemcpy2DAsync(tap_host + (size_t)run * N * cfg.width, (size_t)cfg.width * 4, res, (size_t)Wp * 4,
                                             (size_t)cfg.width * 4, N, cudaMemcpyDeviceToHost, r->stream));
    return NVC_OK;
  }

  static constexpr int kFlashMinChunk = 64;
  bool flash_portions(const nvc_runner* r, const nvc_step_shape& s, const FLayerW& w, const nvc_latent_attn_spec& a) const {
    const int bs = r->opt.kvcache_block_size;
    return use_flash && w.Dk == 128 && w.ldpool == 128 && !s.decode && s.num_decode < s.B && s.max_chunk >= kFlashMinChunk &&
           (bs == 16 || bs == 32 || bs == 64 || bs % 128 == 0);
  }

  int latent_mixer(nvc_runner* r, const nvc_step_shape& s, int li) {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const auto& a = cfg.layers[li].lat;
    FLayerW& w = L[li];
    const int N = s.N;
    const bool own = a.kv_from < 0;
    const void* pool = own ? w.pool : L[a.kv_from].pool;
    int rc;
    if ((rc = nvc_latent_norm_store_rot(ctx, proj, w.np, a.q_rank, w.kv_off, own ? a.kv_rank : 0, w.dq_norm, w.dkv_norm, cfg.eps, cq, w.qrp, own ? w.pool : nullptr,
                                        w.ldpool, r->d_slots, a.rot_dim, a.rot.dims, a.rot_half ? 1 : 0, w.rot, r->d_pos, dt, N, st)))
      return rc;
    mark(r, "latent_norm_store");
    if ((rc = linear(r, cq, w.qrp, w.w_uq, qf, w.uqn, NVC_DT_F32, N, w.uqn, w.qrp))) return rc;
    mark(r, "gemm_uq");
    const int hd = a.heads * w.dimp;
    if ((rc = nvc_head_split_rot(ctx, qf, w.uqn, a.heads, a.dim, a.rot_dim, a.rot.dims, a.rot_half ? 1 : 0, w.rot, r->d_pos, qn, hd, w.dimp, qabs, w.ldqa,
                                 w.Dk, a.kv_rank, dt, N, st)))
      return rc;
    mark(r, "q_split_rot");
    if ((rc = nvc_linear(ctx, qn, hd, w.dimp, w.w_ukT, w.dimp, (int64_t)a.kv_rank * w.dimp, qabs, w.ldqa, w.Dk, dt, dt, N, a.kv_rank, w.dimp, a.heads,
                         NVC_ACT_NONE, st)))
      return rc;
    mark(r, "absorb_uk");
    const int bs = r->opt.kvcache_block_size, cap = r->max_blocks_cap;
    nvc_attn_spec sp{};
    sp.heads = a.heads; sp.kv_heads = 1; sp.dim = w.Dk; sp.vdim = a.kv_rank;
    sp.scale = a.scale;
    sp.window = 0;
    sp.sink = a.sink ? w.sink : nullptr;
    sp.gate = nullptr; sp.ldg = 0;
    sp.out_scale = 1.f;
    int ohs = a.kv_rank;                 // numbers per head in olat
    if (flash_portions(r, s, w, a)) {
      // key = value = the whole 128-number row: the value columns behind the latent come out as a weighted sum of rotated key parts,
      // which the value up-projection below never reads.  One-token sequences of a mixed step come first in the batch and keep the
      // decode path of the wide kernel (same output layout: value width = key width).
      const int nd = s.num_decode;
      ohs = w.Dk;
      sp.vdim = w.Dk;
      if (nd > 0 && (rc = nvc_attn_paged_wide(ctx, qabs, w.ldqa, pool, w.ldpool, pool, w.ldpool, r->d_bt, cap, r->d_ctx, nullptr, nd, nd, 1, bs, &sp, olat,
                                              w.ldol, dt, st)))
        return rc;
      const nvc_bf16* qb = reinterpret_cast<const nvc_bf16*>(qabs);
      nvc_bf16* ob = reinterpret_cast<nvc_bf16*>(olat);
      const nvc_bf16* pb = reinterpret_cast<const nvc_bf16*>(pool);
      if ((rc = nvc_prefill_attn_paged_sink(ctx, qb + (size_t)nd * w.ldqa, w.ldqa, pb, pb, r->d_bt + (size_t)nd * cap, cap, r->d_ctx + nd,
                                            nd ? r->d_cu2 : r->d_cu, s.B - nd, s.N - nd, s.max_chunk, a.heads, 1, w.Dk, bs, r->opt.num_kvcache_blocks,
                                            a.scale, sp.sink, ob + (size_t)nd * w.ldol, w.ldol, st)))
        return rc;
    } else if ((rc = nvc_attn_paged_wide(ctx, qabs, w.ldqa, pool, w.ldpool, pool, w.ldpool, r->d_bt, cap, r->d_ctx, s.decode ? nullptr : r->d_cu, s.B,
                                         s.N, s.decode ? 1 : s.max_seqlen, bs, &sp, olat, w.ldol, dt, st))) {
      return rc;
    }
    mark(r, "attention");
    const int vw = a.heads * a.vdim;
    if ((rc = nvc_linear(ctx, olat, w.ldol, ohs, w.w_uv, w.kvp, (int64_t)a.vdim * w.kvp, hv, vw, a.vdim, dt, NVC_DT_F32, N, a.vdim,
                         ohs % 8 == 0 ? w.kvp : a.kv_rank, a.heads, NVC_ACT_NONE, st)))
      return rc;
    mark(r, "absorb_uv");
    if ((rc = nvc_head_gate(ctx, hv, vw, proj + w.g_off, w.np, ao, w.owp, dt, a.heads, a.vdim, 0, cfg.eps, NVC_GATE_SIGMOID, 1.f, N, st))) return rc;
    mark(r, "head_gate");
    return NVC_OK;
  }

  int delta_mixer(nvc_runner* r, const nvc_step_shape& s, int li) {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const auto& d = cfg.layers[li].delta;
    FLayerW& w = L[li];
    nvc_delta_prep p{};
    p.in = proj; p.ldi = w.np;
    p.q_off = w.q_off; p.k_off = w.k_off; p.v_off = w.v_off; p.b_off = w.b_off; p.a_off = w.a_off;
    p.heads = d.heads; p.kv_heads = d.kv_heads; p.dim = d.dim; p.vdim = d.vdim; p.taps = d.taps;
    p.conv_w = w.conv_w; p.conv_state = w.conv_state;
    p.state_slots = r->d_state_slots; p.cu_seqlens = s.decode ? nullptr : r->d_cu; p.positions = r->d_pos;
    p.A_log = w.A_log; p.dt_bias = w.dt_bias;
    p.unit_eps = kUnitEps; p.q_scale = 1.0f / sqrtf((float)d.dim);
    p.q_out = rq; p.k_out = rk; p.v_out = rv; p.ldq = p.ldk = d.kv_heads * d.dim; p.ldv = d.heads * d.vdim;
    p.gb_out = gb;
    p.B = s.B;
    int rc = nvc_delta_prep_run(ctx, &p, s.N, s.decode ? 1 : s.max_seqlen, st);
    if (rc) return rc;
    mark(r, "delta_prep");
    if ((rc = nvc_delta_rule_scan(ctx, &p, ro, p.ldv, w.state, s.decode ? 1 : s.max_seqlen, st))) return rc;
    mark(r, "delta_scan");
    rc = nvc_head_gate_w(ctx, ro, p.ldv, proj + w.g_off, w.np, w.onorm, ao, w.owp, dt, d.heads, d.vdim, 1, cfg.eps, NVC_GATE_SILU, 1.f, s.N, st);
    mark(r, "head_gate");
    return rc;
  }

  int moe_ff(nvc_runner* r, const nvc_step_shape& s, int li) {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const auto& f = cfg.layers[li].mlp;
    FLayerW& w = L[li];
    const int N = s.N, W = cfg.width, Et = f.experts + f.identity, P = N * f.top;
    int rc;
    if (use_tc) {
      if ((rc = linear(r, h, Wp, w.router, zlog, w.Ep, NVC_DT_F32, N, w.Ep, Wp))) return rc;
    } else if ((rc = nvc_linear(ctx, h, Wp, 0, w.router, Wp, 0, zlog, w.Ep, 0, dt, NVC_DT_F32, N, Et, Wp, 1, NVC_ACT_NONE, st))) {
      return rc;
    }
    if ((rc = nvc_moe_route_logits_ex(ctx, zlog, w.Ep, w.corr, Et, f.top, 1.f, -1, NVC_ROUTE_SOFTMAX, 0, tk_idx, tk_w, nullptr, N, st))) return rc;
    mark(r, "moe_route");
    if (f.experts > 0 && w.moe_tc) {
      const int tiles = moe_tiles(P, Et), mcap = tiles * 128;
      if ((rc = nvc_moe_sort_padded_ex(ctx, tk_idx, N, f.top, Et, f.experts, 128, offsets, src_rows, pos, tile_group, tiles, st))) return rc;
      mark(r, "moe_sort");
      if ((rc = nvc_gather_rows_bf16(ctx, reinterpret_cast<const nvc_bf16*>(h), Wp, src_rows, offsets + f.experts, reinterpret_cast<nvc_bf16*>(xs), Wp,
                                     mcap, Wp, st)))
        return rc;
      mark(r, "moe_gather");
      if ((rc = nvc_gemm_bf16_grouped(ctx, reinterpret_cast<const nvc_bf16*>(xs), Wp, reinterpret_cast<const nvc_bf16*>(w.w_egu), hid2, 2 * w.effp,
                                      NVC_DT_BF16, mcap, 2 * w.effp, Wp, tile_group, f.experts, NVC_ACT_NONE, st)))
        return rc;
      mark(r, "moe_gate_up");
      if ((rc = nvc_act_mul_p(ctx, hid2, 2 * w.effp, hid, w.effp, dt, mcap, f.expert_ff, w.effp, NVC_ACT_GLU_CLAMP, f.limit, kGluAlpha, st))) return rc;
      mark(r, "moe_glu");
      if ((rc = nvc_gemm_bf16_grouped(ctx, reinterpret_cast<const nvc_bf16*>(hid), w.effp, reinterpret_cast<const nvc_bf16*>(w.w_edown), y, Wp, NVC_DT_F32,
                                      mcap, Wp, w.effp, tile_group, f.experts, NVC_ACT_NONE, st)))
        return rc;
      mark(r, "moe_down");
    } else {
      if ((rc = nvc_moe_sort(ctx, tk_idx, N, f.top, Et, offsets, src_rows, pos, st))) return rc;
      mark(r, "moe_sort");
      if (f.experts > 0) {
        if ((rc = nvc_linear_grouped(ctx, h, Wp, src_rows, w.w_egu, Wp, (int64_t)2 * w.effp * Wp, hid2, 2 * w.effp, offsets, f.experts, P, dt, dt,
                                     2 * w.effp, Wp, NVC_ACT_NONE, st)))
          return rc;
        mark(r, "moe_gate_up");
        if ((rc = nvc_act_mul_p(ctx, hid2, 2 * w.effp, hid, w.effp, dt, P, f.expert_ff, w.effp, NVC_ACT_GLU_CLAMP, f.limit, kGluAlpha, st))) return rc;
        mark(r, "moe_glu");
        if ((rc = nvc_linear_grouped(ctx, hid, w.effp, nullptr, w.w_edown, w.effp, (int64_t)Wp * w.effp, y, Wp, offsets, f.experts, P, dt, NVC_DT_F32, Wp,
                                     w.effp, NVC_ACT_NONE, st)))
          return rc;
        mark(r, "moe_down");
      }
    }
    rc = nvc_moe_combine_identity(ctx, y, NVC_DT_F32, Wp, pos, tk_w, tk_idx, f.top, f.experts, h, dt, Wp, ffo, Wp, N, W, st);
    mark(r, "moe_combine");
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
    int rc = nvc_embed_gather_f32(ctx, r->d_ids, embed, dt, Wp, x0, Wp, N, W, st);
    if (rc) return rc;
    mark(r, "embed");
    const float* pend = nullptr;       // a sublayer's output whose norm and residual sum are still to come
    const float* pend_w = nullptr;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
      const auto& ly = cfg.layers[i];
      FLayerW& w = L[i];
      const bool first = i == 0;
      if (tap_host && !first) {
        // debug: land the previous layer's last sum first, copy the stream out, then open this layer
        if ((rc = nvc_rms_norm_sandwich(ctx, res, pend, pend_w, res, Wp, nullptr, nullptr, dt, 0, cfg.eps, 1.f, nullptr, N, W, st))) return rc;
        if ((rc = tap(r, (int)i - 1, N))) return rc;
        pend = pend_w = nullptr;
      }
      if ((rc = nvc_rms_norm_sandwich(ctx, first ? x0 : res, pend, pend_w, res, Wp, w.n1, h, dt, Wp, cfg.eps, 1.f, nullptr, N, W, st))) return rc;
      mark(r, "norm");
      // ---- mixer
      if ((rc = linear(r, h, Wp, w.w_in, proj, w.np, NVC_DT_F32, N, w.np, Wp))) return rc;
      mark(r, "gemm_in");
      if ((rc = ly.kind == nvc_fefozen_layer::Latent ? latent_mixer(r, s, (int)i) : delta_mixer(r, s, (int)i))) return rc;
      if ((rc = linear(r, ao, w.owp, w.w_o, mix, Wp, NVC_DT_F32, N, Wp, w.owp))) return rc;
      mark(r, "gemm_o");
      pend = mix;
      pend_w = w.n1b;
      // ---- feed-forward
      const auto& f = ly.mlp;
      if (f.kind == nvc_routed_mlp_spec::None) continue;
      if ((rc = nvc_rms_norm_sandwich(ctx, res, pend, pend_w, res, Wp, w.n2, h, dt, Wp, cfg.eps, 1.f, nullptr, N, W, st))) return rc;
      mark(r, "norm");
      if (f.kind == nvc_routed_mlp_spec::Dense) {
        if (use_tc) {        // tanh-gelu in the epilogue of the up-projection
          if ((rc = nvc_gemm_bf16_act(ctx, reinterpret_cast<const nvc_bf16*>(h), Wp, reinterpret_cast<const nvc_bf16*>(w.w_up), act, w.ffp, NVC_DT_BF16,
                                      N, w.ffp, Wp, NVC_ACT_GELU_TANH, st)))
            return rc;
        } else if ((rc = linear(r, h, Wp, w.w_up, act, w.ffp, dt, N, w.ffp, Wp, NVC_ACT_GELU_TANH))) {
          return rc;
        }
        mark(r, "gemm_up");
        if ((rc = linear(r, act, w.ffp, w.w_down, ffo, Wp, NVC_DT_F32, N, Wp, w.ffp))) return rc;
        mark(r, "gemm_down");
      } else if ((rc = moe_ff(r, s, (int)i))) {
        return rc;
      }
      pend = ffo;
      pend_w = w.n2b;
    }
    if (tap_host) {
      if ((rc = nvc_rms_norm_sandwich(ctx, res, pend, pend_w, res, Wp, nullptr, nullptr, dt, 0, cfg.eps, 1.f, nullptr, N, W, st))) return rc;
      if ((rc = tap(r, (int)cfg.layers.size() - 1, N))) return rc;
      pend = pend_w = nullptr;
      tap_host = nullptr;      // one step only
    }
    // ---- head: the last sum and the final norm of the wanted rows, logits against the embedding table
    rc = nvc_rms_norm_sandwich(ctx, res, pend, pend_w, nullptr, Wp, fw, hn, dt, Wp, cfg.eps, 1.f, s.decode ? nullptr : r->d_last_rows, s.rows, W, st);
    if (rc) return rc;
    mark(r, "final_norm");
    rc = linear(r, hn, Wp, embed, r->logits, Vp, NVC_DT_F32, s.rows, Vp, Wp);
    mark(r, "lm_head");
    finish_profile(r);
    return rc;
  }
};

}  // namespace

nvc_model_body* nvc_make_fefozen_body(nvc_runner* r, const nvc_fefozen_config& cfg, int* status) {
  FefozenBody* b = new FefozenBody();
  b->cfg = cfg;
  *status = b->init(r);
  return b;
}
