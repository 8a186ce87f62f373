// Batatar model body behind the step executor (runner.cu): weights, per-run paged key / value pools and recurrent state slots, the
// layer loop.
//
// One layer over the N query rows of a step (x <- x + m mixer(n1(x)); x <- x + m ff(n2(x)), fp32 residual stream):
//   nvc_rms_norm_blend       x += m * (what the previous sublayer left: a plain output, or two outputs that are normed over the
//                            width, weighted, halved and summed); h = n(x): one pass over the row
//   parallel:
//     linear w_in            ONE fused projection of everything both mixers read from h, fp32 out:
//                            [q | k | v | head gates | z | x B C | dt]
//     nvc_qkv_prep_run       biases, q and k heads divided by their root mean square, k / v into this run's paged pools
//     nvc_attn_paged_wide    capped scores, keys of the row's own chunk, sink of score zero, one sigmoid gate per head
//     nvc_ssd_prep_run       short convolution + silu, step sizes, log decays;  nvc_decay_scan: S <- exp(l) S + B (dt x)^T, y = S^T C + D x;
//     nvc_ssd_conv_advance   the convolution state;  nvc_group_norm_gate: y silu(z), RMS norm in groups, weight
//     linear o (left), linear o (right)   two outputs, merged by the next nvc_rms_norm_blend
//   lightning:
//     linear w_in            [q | k | v | gate], fp32 out
//     nvc_qkv_prep_run       silu on q, k, v;  nvc_retention_scan: S <- decay S + k v^T, o = S^T q
//     nvc_group_norm_gate    one RMS norm over all heads, weight, sigmoid gate;  linear o
//   experts:                 router logits as a product with fp32 output, nvc_moe_route_logits_ex (sigmoid scores, not renormalised),
//                            sort, nvc_moe_scatter_scaled (score x input row), grouped gate / up product, silu(g) u, grouped down
//                            product, combine with unit weights
// A pass of the looped block opens with the residual row and the embedding row side by side in the storage format, one product
// with loop.in and the pass's vector as a bias of the next norm.  Every run of a layer (layer x pass) has pools and state of its
// own; block ids, slots and state slots are the engine's, shared by all of them.
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "body_common.h"
#include "model_config.h"
#include "runner.h"

namespace {

struct BLayerW {
  float *n1 = nullptr, *n2 = nullptr;
  void* w_in = nullptr;                 // [np, Wp]
  int np = 0;
  // parallel, left
  int q_off = 0, k_off = 0, v_off = 0, g_off = 0;
  float *bias = nullptr, *sink = nullptr, *out_l = nullptr, *out_r = nullptr;
  // parallel, right
  int z_off = 0, xbc_off = 0, dt_off = 0;
  float *conv_w = nullptr, *conv_b = nullptr, *A_log = nullptr, *dt_bias = nullptr, *D = nullptr, *ssd_norm = nullptr;
  void* w_o2 = nullptr;                 // [Wp, owp2]
  int owp2 = 0;
  // lightning
  float *decay = nullptr, *lin_norm = nullptr;
  // both
  void* w_o = nullptr;                  // [Wp, owp]
  int owp = 0;
  // experts
  void* router = nullptr;               // [Ep, Wp]
  float* corr = nullptr;                // zeros: the router has no correction
  int Ep = 0, effp = 0;
  void *w_egu = nullptr, *w_edown = nullptr;   // [E][2 effp, Wp] (gate rows, then up rows at effp), [E][Wp, effp]
  bool moe_tc = false;
};

struct BRunState {                      // what one run of a layer keeps between steps
  void *k_cache = nullptr, *v_cache = nullptr;     // [slots, kv_heads * dim], [slots, kv_heads * vdim]
  float *state = nullptr, *conv_state = nullptr;   // [state slots, heads, rows, vdim], [state slots, taps - 1, channels]
};

struct BatatarBody : nvc_body_base {
  nvc_batatar_config cfg;
  std::vector<nvc_batatar_config::Run> runs;
  int Wp = 0, Vp = 0;
  int state_slots = 0;
  bool use_moe_tc = true;
  std::vector<BLayerW> L;
  std::vector<BRunState> R;
  void *embed = nullptr, *head = nullptr, *w_loop = nullptr;   // w_loop [Wp, 2 Wp]: columns [0, W) take x, [Wp, Wp + W) the embedding
  float *fw = nullptr, *loop_step = nullptr;                   // loop_step [times, W]
  std::map<std::string, bool> want;
  // activations
  float *x0 = nullptr, *res = nullptr, *proj = nullptr, *mix = nullptr, *mix2 = nullptr, *ffo = nullptr;
  float *sq = nullptr, *sk = nullptr, *sv = nullptr, *sx = nullptr, *so = nullptr, *sld = nullptr;   // recurrence operands, fp32 rows
  float *zlog = nullptr, *tk_w = nullptr, *ones = nullptr, *y = nullptr;
  void *h = nullptr, *q = nullptr, *ao = nullptr, *ao2 = nullptr, *hn = nullptr, *cat = nullptr, *hid2 = nullptr, *hid = nullptr, *xs = nullptr;
  int32_t *tk_idx = nullptr, *offsets = nullptr, *src_rows = nullptr, *pos = nullptr, *tile_group = nullptr;
  float* tap_host = nullptr;
  size_t tap_cap = 0;

  int vocab() const override { return cfg.vocab; }
  int logits_ld() const override { return Vp; }
  int layer_runs() const override { return (int)runs.size(); }
  int width() const override { return cfg.width; }
  int num_state_slots() const override { return state_slots; }
  int64_t cache_bytes_per_token() const override {
    int64_t b = 0;
    for (auto& run : runs) {
      const auto& ly = cfg.layers[run.layer];
      if (ly.kind == nvc_batatar_layer::Parallel) b += (int64_t)ly.attn.kv_heads * (ly.attn.dim + ly.attn.vdim) * (int64_t)esz;
    }
    return b;
  }
  int set_residual_tap(float* host, size_t cap) override {
    tap_host = host;
    tap_cap = host ? cap : 0;
    return NVC_OK;
  }

  static int moe_tiles(int pairs, int experts) { return (pairs + experts * 127 + 127) / 128; }

  int init(nvc_runner* r) {
    dt = r->dtype;
    esz = dt == NVC_DT_F32 ? 4 : 2;
    use_tc = dt == NVC_DT_BF16 && !(getenv("NVC_BATATAR_TC") && atoi(getenv("NVC_BATATAR_TC")) == 0);
    use_moe_tc = use_tc && !(getenv("NVC_BATATAR_MOE_TC") && atoi(getenv("NVC_BATATAR_MOE_TC")) == 0);
    Wp = pad64(cfg.width);
    Vp = pad64(cfg.vocab);
    runs = cfg.runs();
    state_slots = r->opt.max_num_seqs;
    const size_t T = (size_t)std::max(r->opt.max_num_batched_tokens, r->opt.max_num_seqs);
    const size_t slots = (size_t)r->opt.num_kvcache_blocks * r->opt.kvcache_block_size;
    int rc;
    L.resize(cfg.layers.size());
    R.resize(runs.size());
    size_t m_np = 0, m_q = 0, m_ow = 0, m_ow2 = 0, m_rq = 0, m_rv = 0, m_h = 0;
    size_t m_Ep = 0, m_top = 0, m_E = 0, m_hid = 0, m_pairs_rows = 0, m_tiles = 0;
    int64_t wbytes = 0;
    const int W = cfg.width;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
      const auto& ly = cfg.layers[i];
      BLayerW& w = L[i];
      const std::string p = "l" + std::to_string(i) + ".";
      if ((rc = zalloc(r, &w.n1, W * 4))) return rc;
      want[p + "norm1"] = false;
      int ow = 0;
      if (ly.kind == nvc_batatar_layer::Parallel) {
        const auto& a = ly.attn;
        const auto& d = ly.ssd;
        const int inner = d.heads * d.vdim, C = inner + 2 * d.groups * d.state;
        w.q_off = 0; w.k_off = a.heads * a.dim; w.v_off = w.k_off + a.kv_heads * a.dim; w.g_off = w.v_off + a.kv_heads * a.vdim;
        w.z_off = w.g_off + a.heads; w.xbc_off = w.z_off + inner; w.dt_off = w.xbc_off + C;
        w.np = pad64(w.dt_off + d.heads);
        ow = a.heads * a.vdim;
        w.owp2 = pad64(inner);
        if ((rc = zalloc(r, &w.bias, (size_t)w.np * 4)) || (rc = zalloc(r, &w.sink, a.heads * 4)) || (rc = zalloc(r, &w.out_l, W * 4)) ||
            (rc = zalloc(r, &w.out_r, W * 4)) || (rc = zalloc(r, &w.conv_w, (size_t)C * d.taps * 4)) || (rc = zalloc(r, &w.conv_b, (size_t)C * 4)) ||
            (rc = zalloc(r, &w.A_log, d.heads * 4)) || (rc = zalloc(r, &w.dt_bias, d.heads * 4)) || (rc = zalloc(r, &w.D, d.heads * 4)) ||
            (rc = zalloc(r, &w.ssd_norm, (size_t)inner * 4)) || (rc = zalloc(r, &w.w_o2, (size_t)Wp * w.owp2 * esz)))
          return rc;
        for (const char* n : {"mix.left.q", "mix.left.q.b", "mix.left.k", "mix.left.k.b", "mix.left.v", "mix.left.v.b", "mix.left.g", "mix.left.o",
                              "mix.left.out", "mix.right.in", "mix.right.conv", "mix.right.conv.b", "mix.right.dt_bias", "mix.right.A_log",
                              "mix.right.D", "mix.right.norm", "mix.right.o", "mix.right.out"})
          want[p + n] = false;
        wbytes += (int64_t)esz * ((int64_t)(w.dt_off + d.heads) * W + (int64_t)W * (ow + inner));
        m_q = std::max(m_q, (size_t)a.heads * a.dim);
        m_ow2 = std::max(m_ow2, (size_t)w.owp2);
        m_rq = std::max(m_rq, (size_t)d.groups * d.state);
        m_rv = std::max(m_rv, (size_t)inner);
        m_h = std::max(m_h, (size_t)d.heads);
      } else {
        const auto& a = ly.lin;
        const int qw = a.heads * a.dim, vw = a.heads * a.vdim;
        w.q_off = 0; w.k_off = qw; w.v_off = 2 * qw; w.g_off = 2 * qw + vw;
        w.np = pad64(w.g_off + vw);
        ow = vw;
        if ((rc = zalloc(r, &w.decay, a.heads * 4)) || (rc = zalloc(r, &w.lin_norm, (size_t)vw * 4))) return rc;
        if ((rc = put_f32(r, w.decay, a.decay.data(), a.heads))) return rc;
        for (const char* n : {"mix.q", "mix.k", "mix.v", "mix.g", "mix.o", "mix.norm"}) want[p + n] = false;
        wbytes += (int64_t)esz * ((int64_t)(w.g_off + vw) * W + (int64_t)W * vw);
        m_rq = std::max(m_rq, (size_t)qw);
        m_rv = std::max(m_rv, (size_t)vw);
      }
      w.owp = pad64(ow);
      if ((rc = zalloc(r, &w.w_in, (size_t)w.np * Wp * esz)) || (rc = zalloc(r, &w.w_o, (size_t)Wp * w.owp * esz))) return rc;
      m_np = std::max(m_np, (size_t)w.np);
      m_ow = std::max(m_ow, (size_t)w.owp);
      const auto& f = ly.mlp;
      if (f.kind == nvc_routed_mlp_spec::Moe) {
        if ((rc = zalloc(r, &w.n2, W * 4))) return rc;
        want[p + "norm2"] = false;
        w.Ep = pad64(f.experts);
        w.effp = pad64(f.expert_ff);
        w.moe_tc = use_moe_tc && w.effp >= 128;
        if ((rc = zalloc(r, &w.router, (size_t)w.Ep * Wp * esz)) || (rc = zalloc(r, &w.corr, f.experts * 4)) ||
            (rc = zalloc(r, &w.w_egu, (size_t)f.experts * 2 * w.effp * Wp * esz)) || (rc = zalloc(r, &w.w_edown, (size_t)f.experts * Wp * w.effp * esz)))
          return rc;
        want[p + "mlp.router"] = false;
        for (int e = 0; e < f.experts; ++e)
          for (const char* n : {"gate", "up", "down"}) want[p + "mlp.e" + std::to_string(e) + "." + n] = false;
        wbytes += (int64_t)esz * ((int64_t)f.experts * W + (int64_t)f.experts * 3 * f.expert_ff * W);
        m_Ep = std::max(m_Ep, (size_t)w.Ep);
        m_top = std::max(m_top, (size_t)f.top);
        m_E = std::max(m_E, (size_t)f.experts);
        m_hid = std::max(m_hid, (size_t)w.effp);
        const size_t rows = w.moe_tc ? (size_t)moe_tiles((int)T * f.top, f.experts) * 128 : T * f.top;
        m_pairs_rows = std::max(m_pairs_rows, rows);
        if (w.moe_tc) m_tiles = std::max(m_tiles, (size_t)moe_tiles((int)T * f.top, f.experts));
      }
    }
    // pools and state of every run
    for (size_t k = 0; k < runs.size(); ++k) {
      const auto& ly = cfg.layers[runs[k].layer];
      BRunState& s = R[k];
      if (ly.kind == nvc_batatar_layer::Parallel) {
        const auto& a = ly.attn;
        const auto& d = ly.ssd;
        const size_t C = (size_t)d.heads * d.vdim + 2 * (size_t)d.groups * d.state;
        if ((rc = zalloc(r, &s.k_cache, slots * a.kv_heads * a.dim * esz)) || (rc = zalloc(r, &s.v_cache, slots * a.kv_heads * a.vdim * esz)) ||
            (rc = zalloc(r, &s.state, (size_t)state_slots * d.heads * d.state * d.vdim * 4)) ||
            (rc = zalloc(r, &s.conv_state, (size_t)state_slots * std::max(d.taps - 1, 1) * C * 4)))
          return rc;
      } else if ((rc = zalloc(r, &s.state, (size_t)state_slots * ly.lin.heads * ly.lin.dim * ly.lin.vdim * 4))) {
        return rc;
      }
    }
    if ((rc = zalloc(r, &embed, (size_t)Vp * Wp * esz)) || (rc = zalloc(r, &head, (size_t)Vp * Wp * esz)) || (rc = zalloc(r, &fw, W * 4))) return rc;
    want["embed"] = false;
    want["head"] = false;
    want["final.norm"] = false;
    wbytes += (int64_t)esz * 2 * cfg.vocab * W;
    if (cfg.looped) {
      if ((rc = zalloc(r, &w_loop, (size_t)Wp * 2 * Wp * esz)) || (rc = zalloc(r, &loop_step, (size_t)cfg.loop_times * W * 4)) ||
          (rc = zalloc(r, &cat, T * 2 * Wp * esz)))
        return rc;
      want["loop.in"] = false;
      want["loop.step"] = false;
      wbytes += (int64_t)esz * 2 * W * W;
    }
    r->weight_bytes = wbytes;
    // activations (zeroed once: padding columns are never written)
    if ((rc = zalloc(r, &x0, T * Wp * 4)) || (rc = zalloc(r, &res, T * Wp * 4)) || (rc = zalloc(r, &mix, T * Wp * 4)) ||
        (rc = zalloc(r, &mix2, T * Wp * 4)) || (rc = zalloc(r, &ffo, T * Wp * 4)) || (rc = zalloc(r, &proj, T * m_np * 4)) ||
        (rc = zalloc(r, &h, T * Wp * esz)) || (rc = zalloc(r, &ao, T * m_ow * esz)) || (rc = zalloc(r, &hn, (size_t)r->max_logit_rows * Wp * esz)) ||
        (rc = zalloc(r, &sq, T * m_rq * 4)) || (rc = zalloc(r, &sk, T * m_rq * 4)) || (rc = zalloc(r, &sv, T * m_rv * 4)) ||
        (rc = zalloc(r, &so, T * m_rv * 4)))
      return rc;
    if (m_q && ((rc = zalloc(r, &q, T * m_q * esz)) || (rc = zalloc(r, &ao2, T * m_ow2 * esz)) || (rc = zalloc(r, &sx, T * m_rv * 4)) ||
                (rc = zalloc(r, &sld, T * m_h * 4))))
      return rc;
    if (m_E) {
      if ((rc = zalloc(r, &zlog, T * m_Ep * 4)) || (rc = zalloc(r, &tk_idx, T * m_top * 4)) || (rc = zalloc(r, &tk_w, T * m_top * 4)) ||
          (rc = zalloc(r, &ones, T * m_top * 4)) || (rc = zalloc(r, &offsets, (m_E + 1) * 4)) || (rc = zalloc(r, &src_rows, m_pairs_rows * 4)) ||
          (rc = zalloc(r, &pos, T * m_top * 4)) || (rc = zalloc(r, &hid2, m_pairs_rows * 2 * m_hid * esz)) ||
          (rc = zalloc(r, &hid, m_pairs_rows * m_hid * esz)) || (rc = zalloc(r, &y, m_pairs_rows * Wp * 4)) ||
          (rc = zalloc(r, &xs, m_pairs_rows * Wp * esz)))
        return rc;
      if (m_tiles && (rc = zalloc(r, &tile_group, m_tiles * 4))) return rc;
      std::vector<float> one(T * m_top, 1.0f);
      if ((rc = put_f32(r, ones, one.data(), one.size()))) return rc;
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
    else if (name == "head") { if (!shape_is(cfg.vocab, W)) return bad(); rc = put_matrix(r, head, Wp, 0, 0, v.data(), cfg.vocab, W, W, 1); }
    else if (name == "final.norm") rc = vec(fw, W);
    else if (name == "loop.in") {
      // [W, 2 W] -> [Wp, 2 Wp]: the half that reads the embedding starts at column Wp
      if (!shape_is(W, 2 * W)) return bad();
      if ((rc = put_matrix(r, w_loop, 2 * (size_t)Wp, 0, 0, v.data(), W, W, 2 * (size_t)W, 1))) return rc;
      rc = put_matrix(r, w_loop, 2 * (size_t)Wp, 0, Wp, v.data() + W, W, W, 2 * (size_t)W, 1);
    }
    else if (name == "loop.step") { if (!shape_is(cfg.loop_times, W)) return bad(); rc = put_f32(r, loop_step, v.data(), n); }
    else {
      const size_t dot = name.find('.');
      const int li = atoi(name.substr(1, dot - 1).c_str());
      const std::string sub = name.substr(dot + 1);
      const auto& ly = cfg.layers[li];
      const auto& a = ly.attn;
      const auto& d = ly.ssd;
      const auto& ln = ly.lin;
      const auto& f = ly.mlp;
      BLayerW& w = L[li];
      const bool par = ly.kind == nvc_batatar_layer::Parallel;
      auto in_rows = [&](int off, int rows) { return shape_is(rows, W) ? put_matrix(r, w.w_in, Wp, off, 0, v.data(), rows, W, W, 1) : bad(); };
      auto bias_at = [&](int off, size_t len) { return n == len ? put_f32(r, w.bias + off, v.data(), len) : bad(); };
      const int inner = d.heads * d.vdim, C = inner + 2 * d.groups * d.state;
      const int low = par ? a.heads * a.vdim : ln.heads * ln.vdim;
      if (sub == "norm1") rc = vec(w.n1, W);
      else if (sub == "norm2") rc = vec(w.n2, W);
      else if (par && sub == "mix.left.q") rc = in_rows(w.q_off, a.heads * a.dim);
      else if (par && sub == "mix.left.k") rc = in_rows(w.k_off, a.kv_heads * a.dim);
      else if (par && sub == "mix.left.v") rc = in_rows(w.v_off, a.kv_heads * a.vdim);
      else if (par && sub == "mix.left.g") rc = in_rows(w.g_off, a.heads);
      else if (par && sub == "mix.left.q.b") rc = bias_at(w.q_off, (size_t)a.heads * a.dim);
      else if (par && sub == "mix.left.k.b") rc = bias_at(w.k_off, (size_t)a.kv_heads * a.dim);
      else if (par && sub == "mix.left.v.b") rc = bias_at(w.v_off, (size_t)a.kv_heads * a.vdim);
      else if (par && sub == "mix.left.o") { if (!shape_is(W, low)) return bad(); rc = put_matrix(r, w.w_o, w.owp, 0, 0, v.data(), W, low, low, 1); }
      else if (par && sub == "mix.left.out") rc = vec(w.out_l, W);
      else if (par && sub == "mix.right.out") rc = vec(w.out_r, W);
      else if (par && sub == "mix.right.in") rc = in_rows(w.z_off, 2 * inner + 2 * d.groups * d.state + d.heads);
      else if (par && sub == "mix.right.conv") {
        // [channels, taps] of the checkpoint -> tap-major [taps, channels]: a warp's lanes read neighbours
        if (!shape_is(C, d.taps)) return bad();
        std::vector<float> tm((size_t)C * d.taps);
        for (int c = 0; c < C; ++c)
          for (int i = 0; i < d.taps; ++i) tm[(size_t)i * C + c] = v[(size_t)c * d.taps + i];
        rc = put_f32(r, w.conv_w, tm.data(), tm.size());
      }
      else if (par && sub == "mix.right.conv.b") rc = vec(w.conv_b, C);
      else if (par && sub == "mix.right.dt_bias") rc = vec(w.dt_bias, d.heads);
      else if (par && sub == "mix.right.A_log") rc = vec(w.A_log, d.heads);
      else if (par && sub == "mix.right.D") rc = vec(w.D, d.heads);
      else if (par && sub == "mix.right.norm") rc = vec(w.ssd_norm, inner);
      else if (par && sub == "mix.right.o") { if (!shape_is(W, inner)) return bad(); rc = put_matrix(r, w.w_o2, w.owp2, 0, 0, v.data(), W, inner, inner, 1); }
      else if (!par && sub == "mix.q") rc = in_rows(w.q_off, ln.heads * ln.dim);
      else if (!par && sub == "mix.k") rc = in_rows(w.k_off, ln.heads * ln.dim);
      else if (!par && sub == "mix.v") rc = in_rows(w.v_off, low);
      else if (!par && sub == "mix.g") rc = in_rows(w.g_off, low);
      else if (!par && sub == "mix.norm") rc = vec(w.lin_norm, low);
      else if (!par && sub == "mix.o") { if (!shape_is(W, low)) return bad(); rc = put_matrix(r, w.w_o, w.owp, 0, 0, v.data(), W, low, low, 1); }
      else if (sub == "mlp.router") { if (!shape_is(f.experts, W)) return bad(); rc = put_matrix(r, w.router, Wp, 0, 0, v.data(), f.experts, W, W, 1); }
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

  // left half of a parallel mixer into ao[:, :heads * vdim]
  int chunk_attention(nvc_runner* r, const nvc_step_shape& s, int li, int run) {
    nvc_ctx* ctx = r->ctx;
    const auto& a = cfg.layers[li].attn;
    BLayerW& w = L[li];
    BRunState& rs = R[run];
    nvc_qkv_prep p{};
    p.in = proj; p.ldi = w.np;
    p.bias = w.bias;
    p.q_off = w.q_off; p.k_off = w.k_off; p.v_off = w.v_off;
    p.q_heads = a.heads; p.kv_heads = a.kv_heads; p.dim = a.dim; p.vdim = a.vdim;
    p.unit_norm = 1;
    p.eps = cfg.eps;
    p.k_scale = 1.f; p.v_scale = 1.f;
    p.blend = NVC_BLEND_NONE;
    p.q_out = q; p.ldq = a.heads * a.dim;
    p.k_out = rs.k_cache; p.v_out = rs.v_cache; p.ldk = a.kv_heads * a.dim; p.ldv = a.kv_heads * a.vdim;
    p.slot_mapping = r->d_slots;
    p.q_dtype = dt; p.kv_dtype = dt;
    int rc = nvc_qkv_prep_run(ctx, &p, s.N, r->stream);
    if (rc) return rc;
    mark(r, "qkv_prep");
    nvc_attn_spec sp{};
    sp.heads = a.heads; sp.kv_heads = a.kv_heads; sp.dim = a.dim; sp.vdim = a.vdim;
    sp.scale = a.scale;
    sp.softcap = a.softcap;
    sp.chunk = a.chunk;
    sp.sink = w.sink;                  // zeros: one more term exp(0) in every denominator
    sp.gate = proj + w.g_off; sp.ldg = w.np; sp.gate_per_head = 1;
    sp.out_scale = 1.f;
    rc = nvc_attn_paged_wide(ctx, q, p.ldq, rs.k_cache, p.ldk, rs.v_cache, p.ldv, r->d_bt, r->max_blocks_cap, r->d_ctx, s.decode ? nullptr : r->d_cu,
                             s.B, s.N, s.decode ? 1 : s.max_seqlen, r->opt.kvcache_block_size, &sp, ao, w.owp, dt, r->stream);
    mark(r, "attention");
    return rc;
  }

  // right half of a parallel mixer into ao2[:, :heads * vdim]
  int ssd_mixer(nvc_runner* r, const nvc_step_shape& s, int li, int run) {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const auto& d = cfg.layers[li].ssd;
    BLayerW& w = L[li];
    BRunState& rs = R[run];
    const int inner = d.heads * d.vdim, gn = d.groups * d.state;
    nvc_ssd_prep p{};
    p.in = proj; p.ldi = w.np;
    p.xbc_off = w.xbc_off; p.dt_off = w.dt_off;
    p.heads = d.heads; p.vdim = d.vdim; p.groups = d.groups; p.state = d.state; p.taps = d.taps;
    p.conv_w = w.conv_w; p.conv_b = w.conv_b; p.conv_state = rs.conv_state;
    p.state_slots = r->d_state_slots; p.cu_seqlens = s.decode ? nullptr : r->d_cu; p.positions = r->d_pos;
    p.A_log = w.A_log; p.dt_bias = w.dt_bias;
    p.x_out = sx; p.v_out = sv; p.ldx = inner;
    p.b_out = sk; p.c_out = sq; p.ldbc = gn;
    p.log_decay = sld; p.ldl = d.heads;
    p.B = s.B;
    int rc = nvc_ssd_prep_run(ctx, &p, s.N, st);
    if (rc) return rc;
    if ((rc = nvc_ssd_conv_advance(ctx, &p, st))) return rc;
    mark(r, "ssd_prep");
    nvc_decay_scan_args sc{};
    sc.q = sq; sc.k = sk; sc.v = sv; sc.ldq = gn; sc.ldk = gn; sc.ldv = inner;
    sc.o = so; sc.ldo = inner;
    sc.state = rs.state; sc.state_slots = r->d_state_slots; sc.cu_seqlens = p.cu_seqlens; sc.positions = r->d_pos;
    sc.log_decay = sld; sc.ldl = d.heads;
    sc.skip = sx; sc.skip_w = w.D; sc.lds = inner;
    sc.heads = d.heads; sc.qk_heads = d.groups; sc.dim = d.state; sc.vdim = d.vdim;
    if ((rc = nvc_decay_scan(ctx, &sc, s.B, s.decode ? 1 : s.max_seqlen, st))) return rc;
    mark(r, "ssd_scan");
    rc = nvc_group_norm_gate(ctx, so, inner, proj + w.z_off, w.np, w.ssd_norm, ao2, w.owp2, dt, d.norm_groups, inner / d.norm_groups, 1, cfg.eps,
                             NVC_GATE_SILU, s.N, st);
    mark(r, "ssd_gate_norm");
    return rc;
  }

  int lightning_mixer(nvc_runner* r, const nvc_step_shape& s, int li, int run) {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const auto& a = cfg.layers[li].lin;
    BLayerW& w = L[li];
    const int qw = a.heads * a.dim, vw = a.heads * a.vdim;
    nvc_qkv_prep p{};
    p.in = proj; p.ldi = w.np;
    p.q_off = w.q_off; p.k_off = w.k_off; p.v_off = w.v_off;
    p.q_heads = a.heads; p.kv_heads = a.heads; p.dim = a.dim; p.vdim = a.vdim;
    p.act = NVC_PREP_ACT_SILU;
    p.eps = cfg.eps;
    p.k_scale = 1.f; p.v_scale = 1.f;
    p.blend = NVC_BLEND_NONE;
    p.q_out = sq; p.ldq = qw;
    p.k_out = sk; p.v_out = sv; p.ldk = qw; p.ldv = vw;
    p.slot_mapping = nullptr;
    p.q_dtype = NVC_DT_F32; p.kv_dtype = NVC_DT_F32;
    int rc = nvc_qkv_prep_run(ctx, &p, s.N, st);
    if (rc) return rc;
    mark(r, "lightning_prep");
    if ((rc = nvc_retention_scan(ctx, sq, qw, sk, qw, sv, vw, so, vw, R[run].state, r->d_state_slots, s.decode ? nullptr : r->d_cu, r->d_pos, w.decay,
                                 s.B, s.decode ? 1 : s.max_seqlen, a.heads, a.dim, a.vdim, st)))
      return rc;
    mark(r, "lightning_scan");
    rc = nvc_group_norm_gate(ctx, so, vw, proj + w.g_off, w.np, w.lin_norm, ao, w.owp, dt, 1, vw, 0, cfg.eps, NVC_GATE_SIGMOID, s.N, st);
    mark(r, "lightning_norm_gate");
    return rc;
  }

  int moe_ff(nvc_runner* r, const nvc_step_shape& s, int li) {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const auto& f = cfg.layers[li].mlp;
    BLayerW& w = L[li];
    const int N = s.N, W = cfg.width, E = f.experts, P = N * f.top;
    int rc;
    if (use_tc) {
      if ((rc = linear(r, h, Wp, w.router, zlog, w.Ep, NVC_DT_F32, N, w.Ep, Wp))) return rc;
    } else if ((rc = nvc_linear(ctx, h, Wp, 0, w.router, Wp, 0, zlog, w.Ep, 0, dt, NVC_DT_F32, N, E, Wp, 1, NVC_ACT_NONE, st))) {
      return rc;
    }
    if ((rc = nvc_moe_route_logits_ex(ctx, zlog, w.Ep, w.corr, E, f.top, 1.f, -1, NVC_ROUTE_SIGMOID, 0, tk_idx, tk_w, nullptr, N, st))) return rc;
    mark(r, "moe_route");
    int mcap = P;
    if (w.moe_tc) {
      const int tiles = moe_tiles(P, E);
      mcap = tiles * 128;
      if ((rc = nvc_moe_sort_padded_ex(ctx, tk_idx, N, f.top, E, E, 128, offsets, src_rows, pos, tile_group, tiles, st))) return rc;
    } else if ((rc = nvc_moe_sort(ctx, tk_idx, N, f.top, E, offsets, src_rows, pos, st))) {
      return rc;
    }
    mark(r, "moe_sort");
    // the router's score multiplies the expert's INPUT: every (token, choice) pair gets its own scaled copy of the row
    if ((rc = nvc_moe_scatter_scaled(ctx, h, dt, Wp, pos, tk_w, f.top, xs, Wp, N, W, st))) return rc;
    mark(r, "moe_scatter");
    if (w.moe_tc) {
      if ((rc = nvc_gemm_bf16_grouped(ctx, reinterpret_cast<const nvc_bf16*>(xs), Wp, reinterpret_cast<const nvc_bf16*>(w.w_egu), hid2, 2 * w.effp,
                                      NVC_DT_BF16, mcap, 2 * w.effp, Wp, tile_group, E, NVC_ACT_NONE, st)))
        return rc;
    } else if ((rc = nvc_linear_grouped(ctx, xs, Wp, nullptr, w.w_egu, Wp, (int64_t)2 * w.effp * Wp, hid2, 2 * w.effp, offsets, E, P, dt, dt, 2 * w.effp, Wp,
                                        NVC_ACT_NONE, st))) {
      return rc;
    }
    mark(r, "moe_gate_up");
    if ((rc = nvc_act_mul_p(ctx, hid2, 2 * w.effp, hid, w.effp, dt, mcap, f.expert_ff, w.effp, NVC_ACT_SILU_MUL, 0.f, 0.f, st))) return rc;
    mark(r, "moe_glu");
    if (w.moe_tc) {
      if ((rc = nvc_gemm_bf16_grouped(ctx, reinterpret_cast<const nvc_bf16*>(hid), w.effp, reinterpret_cast<const nvc_bf16*>(w.w_edown), y, Wp, NVC_DT_F32,
                                      mcap, Wp, w.effp, tile_group, E, NVC_ACT_NONE, st)))
        return rc;
    } else if ((rc = nvc_linear_grouped(ctx, hid, w.effp, nullptr, w.w_edown, w.effp, (int64_t)Wp * w.effp, y, Wp, offsets, E, P, dt, NVC_DT_F32, Wp,
                                        w.effp, NVC_ACT_NONE, st))) {
      return rc;
    }
    mark(r, "moe_down");
    rc = nvc_moe_combine(ctx, y, NVC_DT_F32, Wp, pos, ones, f.top, nullptr, NVC_DT_F32, 0, nullptr, ffo, Wp, N, W, st);
    mark(r, "moe_combine");
    return rc;
  }

  // what a sublayer left for the next pass over the residual rows: x += c0 f(y0, w0) + c1 f(y1, w1)
  struct Pending {
    const float *y0 = nullptr, *w0 = nullptr, *y1 = nullptr, *w1 = nullptr;
    float c0 = 0.f, c1 = 0.f;
  };
  // x (+ bias) (+ pending) -> res; out = norm(x) w, x itself (w == NULL, out != NULL) or nothing
  int land(nvc_runner* r, const float* x_in, const float* bias, Pending& pd, float* res_out, const float* w, void* out, int ldo, const int32_t* rows,
           int n) {
    int rc = nvc_rms_norm_blend(r->ctx, x_in, bias, pd.y0, pd.w0, pd.c0, pd.y1, pd.w1, pd.c1, res_out, Wp, w, out, dt, ldo, cfg.eps, rows, n, cfg.width,
                                r->stream);
    pd = Pending();
    return rc;
  }

  int forward(nvc_runner* r, const nvc_step_shape& s) override {
    nvc_ctx* ctx = r->ctx;
    void* st = r->stream;
    const int N = s.N, W = cfg.width;
    const float m = cfg.residual_mult;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(r->stream, &cap);
    prof_on = prof_armed && cap == cudaStreamCaptureStatusNone;
    if (prof_on) prof_armed = false;
    mark(r, "start");
    int rc = nvc_embed_gather_f32(ctx, r->d_ids, embed, dt, Wp, x0, Wp, N, W, st);
    if (rc) return rc;
    mark(r, "embed");
    Pending pd;
    const float* cur = x0;             // where the residual rows live: the embedding until the first pass over them writes `res`
    bool x0_in_cat = false;
    for (size_t k = 0; k < runs.size(); ++k) {
      const int li = runs[k].layer;
      const auto& ly = cfg.layers[li];
      BLayerW& w = L[li];
      const float* bias = nullptr;
      if (runs[k].opens_pass) {
        // x <- loop.in [x ; x0] + step_t: both halves side by side in the storage format, one product, the vector rides on the next norm
        if ((rc = land(r, cur, nullptr, pd, res, nullptr, cat, 2 * Wp, nullptr, N))) return rc;
        if (!x0_in_cat) {
          Pending none;
          if ((rc = land(r, x0, nullptr, none, nullptr, nullptr, reinterpret_cast<uint8_t*>(cat) + (size_t)Wp * esz, 2 * Wp, nullptr, N))) return rc;
          x0_in_cat = true;
        }
        mark(r, "loop_concat");
        if ((rc = linear(r, cat, 2 * Wp, w_loop, res, Wp, NVC_DT_F32, N, Wp, 2 * Wp))) return rc;
        mark(r, "gemm_loop");
        cur = res;
        bias = loop_step + (size_t)runs[k].pass * W;
      }
      if ((rc = land(r, cur, bias, pd, res, w.n1, h, Wp, nullptr, N))) return rc;
      cur = res;
      mark(r, "norm");
      // ---- mixer
      if ((rc = linear(r, h, Wp, w.w_in, proj, w.np, NVC_DT_F32, N, w.np, Wp))) return rc;
      mark(r, "gemm_in");
      if (ly.kind == nvc_batatar_layer::Parallel) {
        if ((rc = chunk_attention(r, s, li, (int)k))) return rc;
        if ((rc = ssd_mixer(r, s, li, (int)k))) return rc;
        if ((rc = linear(r, ao, w.owp, w.w_o, mix, Wp, NVC_DT_F32, N, Wp, w.owp))) return rc;
        if ((rc = linear(r, ao2, w.owp2, w.w_o2, mix2, Wp, NVC_DT_F32, N, Wp, w.owp2))) return rc;
        mark(r, "gemm_o");
        pd.y0 = mix; pd.w0 = w.out_l; pd.c0 = 0.5f * m;
        pd.y1 = mix2; pd.w1 = w.out_r; pd.c1 = 0.5f * m;
      } else {
        if ((rc = lightning_mixer(r, s, li, (int)k))) return rc;
        if ((rc = linear(r, ao, w.owp, w.w_o, mix, Wp, NVC_DT_F32, N, Wp, w.owp))) return rc;
        mark(r, "gemm_o");
        pd.y0 = mix; pd.c0 = m;
      }
      // ---- feed-forward
      if (ly.mlp.kind == nvc_routed_mlp_spec::Moe) {
        if ((rc = land(r, res, nullptr, pd, res, w.n2, h, Wp, nullptr, N))) return rc;
        mark(r, "norm");
        if ((rc = moe_ff(r, s, li))) return rc;
        pd.y0 = ffo; pd.c0 = m;
      }
      if (tap_host) {
        // debug: land this run's last sum and copy the stream out
        if ((rc = land(r, res, nullptr, pd, res, nullptr, nullptr, 0, nullptr, N))) return rc;
        if ((rc = tap(r, (int)k, N))) return rc;
      }
    }
    tap_host = nullptr;      // one step only
    // ---- head: the last sum and the final norm of the wanted rows, logits
    rc = land(r, cur, nullptr, pd, nullptr, fw, hn, Wp, s.decode ? nullptr : r->d_last_rows, s.rows);
    if (rc) return rc;
    mark(r, "final_norm");
    rc = linear(r, hn, Wp, head, r->logits, Vp, NVC_DT_F32, s.rows, Vp, Wp);
    mark(r, "lm_head");
    finish_profile(r);
    return rc;
  }
};

}  // namespace

nvc_model_body* nvc_make_batatar_body(nvc_runner* r, const nvc_batatar_config& cfg, int* status) {
  BatatarBody* b = new BatatarBody();
  b->cfg = cfg;
  *status = b->init(r);
  return b;
}
