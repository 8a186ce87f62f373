// Model registry, configuration side: config.json -> nvc_model_config.  The architecture is taken from config.json
// ("architecture": "<name>", or the first entry of HF's "architectures" list); each registered family parses its own keys.
// Plain host C++ (also built without CUDA by the sanitizer tests).
#include "model_config.h"

#include "json.h"

using namespace nvcjson;

namespace {

thread_local std::string g_cfg_error;

int cfg_fail(const std::string& m) {
  g_cfg_error = m;
  return NVC_EINVAL;
}

bool get_int(const JValue* o, const char* key, int& out, int lo, std::string& err) {
  const JValue* v = o ? o->get(key) : nullptr;
  if (!v || v->kind != JValue::Num || v->num != (double)(int64_t)v->num || v->num < lo || v->num > 2147483647.0) {
    err = std::string("missing or invalid integer `") + key + "`";
    return false;
  }
  out = (int)v->num;
  return true;
}
bool get_float(const JValue* o, const char* key, float& out, std::string& err) {
  const JValue* v = o ? o->get(key) : nullptr;
  if (!v || v->kind != JValue::Num) {
    err = std::string("missing or invalid number `") + key + "`";
    return false;
  }
  out = (float)v->num;
  return true;
}

int parse_karuzen(const JValue& root, nvc_karuzen_config& c) {
  std::string err;
  if (!get_int(&root, "vocab", c.vocab, 1, err) || !get_int(&root, "width", c.width, 1, err)) return cfg_fail(err);
  const JValue* norm = root.get("norm");
  if (!norm || norm->kind != JValue::Obj || !get_float(norm, "eps", c.eps, err)) return cfg_fail("norm.eps: " + err);
  const JValue* layers = root.get("layers");
  if (!layers || layers->kind != JValue::Arr || layers->arr.empty()) return cfg_fail("`layers` must be a non-empty list");
  for (size_t i = 0; i < layers->arr.size(); ++i) {
    const JValue& jl = layers->arr[i];
    const std::string where = "layers[" + std::to_string(i) + "]: ";
    if (jl.kind != JValue::Obj) return cfg_fail(where + "not an object");
    nvc_karuzen_layer L;
    const JValue* type = jl.get("type");
    if (!type || type->kind != JValue::Str) return cfg_fail(where + "missing `type`");
    L.mixer.type = type->str;
    if (L.mixer.type != "latent_attention") return cfg_fail(where + "mixer type `" + L.mixer.type + "` is not supported");
    const JValue* m = jl.get("mixer");
    if (!m || m->kind != JValue::Obj) return cfg_fail(where + "missing `mixer`");
    if (!get_int(m, "heads", L.mixer.heads, 1, err) || !get_int(m, "dim", L.mixer.dim, 1, err) ||
        !get_int(m, "vdim", L.mixer.vdim, 1, err) || !get_int(m, "kv_rank", L.mixer.kv_rank, 1, err) ||
        !get_int(m, "q_rank", L.mixer.q_rank, 1, err) || !get_float(m, "scale", L.mixer.scale, err))
      return cfg_fail(where + "mixer: " + err);
    const JValue* mlp = jl.get("mlp");
    if (mlp && mlp->kind == JValue::Obj) {
      const JValue* kind = mlp->get("kind");
      if (!kind || kind->kind != JValue::Str) return cfg_fail(where + "mlp: missing `kind`");
      if (kind->str == "dense") {
        L.mlp.kind = nvc_karuzen_mlp::Dense;
        if (!get_int(mlp, "ff", L.mlp.ff, 1, err)) return cfg_fail(where + "mlp: " + err);
      } else if (kind->str == "moe") {
        L.mlp.kind = nvc_karuzen_mlp::Moe;
        const JValue* r = mlp->get("router");
        const JValue* e = mlp->get("expert");
        if (!r || !e) return cfg_fail(where + "mlp: a mixture of experts needs `router` and `expert`");
        if (!get_int(r, "experts", L.mlp.experts, 1, err) || !get_int(r, "top", L.mlp.top, 1, err) ||
            !get_float(r, "scale", L.mlp.router_scale, err) || !get_int(e, "ff", L.mlp.expert_ff, 1, err))
          return cfg_fail(where + "mlp: " + err);
        if (L.mlp.top > L.mlp.experts) return cfg_fail(where + "mlp: top exceeds experts");
        const JValue* sh = mlp->get("shared");
        if (sh && sh->kind == JValue::Obj && !get_int(sh, "ff", L.mlp.shared_ff, 1, err)) return cfg_fail(where + "mlp.shared: " + err);
      } else {
        return cfg_fail(where + "mlp kind `" + kind->str + "` is not supported");
      }
    } else if (mlp && mlp->kind != JValue::Null) {
      return cfg_fail(where + "`mlp` must be an object or null");
    }
    c.layers.push_back(L);
  }
  const int n = (int)c.layers.size();
  c.loop_start = c.loop_stop = 0;
  c.loop_times = 1;
  const JValue* loop = root.get("loop");
  if (loop && loop->kind == JValue::Obj) {
    if (!get_int(loop, "start", c.loop_start, 0, err) || !get_int(loop, "stop", c.loop_stop, 0, err) ||
        !get_int(loop, "times", c.loop_times, 1, err))
      return cfg_fail("loop: " + err);
    if (c.loop_start > c.loop_stop || c.loop_stop > n) return cfg_fail("loop: start <= stop <= number of layers is required");
  } else if (loop && loop->kind != JValue::Null) {
    return cfg_fail("`loop` must be an object or null");
  }
  return NVC_OK;
}

bool parse_rotary(const JValue* m, nvc_rotary_spec& r, int dim, std::string& err) {
  const JValue* rot = m->get("rot");
  if (!rot || rot->kind == JValue::Null) { r.dims = 0; return true; }
  if (rot->kind != JValue::Obj || !get_int(rot, "dims", r.dims, 0, err) || !get_float(rot, "base", r.base, err)) {
    if (err.empty()) err = "`rot` must be an object";
    return false;
  }
  if (r.dims % 2 != 0 || r.dims > dim) { err = "rot.dims must be even and at most dim"; return false; }
  if (!(r.base > 0.f)) { err = "rot.base must be positive"; return false; }
  return true;
}

bool parse_softmax_attn(const JValue* m, nvc_softmax_attn_spec& a, std::string& err) {
  if (!get_int(m, "heads", a.heads, 1, err) || !get_int(m, "kv_heads", a.kv_heads, 1, err) || !get_int(m, "dim", a.dim, 1, err) ||
      !get_int(m, "vdim", a.vdim, 1, err) || !get_float(m, "scale", a.scale, err) || !parse_rotary(m, a.rot, a.dim, err))
    return false;
  if (a.heads % a.kv_heads != 0) { err = "heads must be a multiple of kv_heads"; return false; }
  return true;
}

int parse_ranilix(const JValue& root, nvc_ranilix_config& c) {
  std::string err;
  if (!get_int(&root, "vocab", c.vocab, 1, err) || !get_int(&root, "width", c.width, 1, err)) return cfg_fail(err);
  const JValue* norm = root.get("norm");
  if (!norm || norm->kind != JValue::Obj || !get_float(norm, "eps", c.eps, err)) return cfg_fail("norm.eps: " + err);
  const JValue* emb = root.get("embedding");
  c.embedding_scale = 1.f;
  if (emb && emb->kind == JValue::Obj && emb->get("scale") && !get_float(emb, "scale", c.embedding_scale, err))
    return cfg_fail("embedding.scale: " + err);
  const JValue* layers = root.get("layers");
  if (!layers || layers->kind != JValue::Arr || layers->arr.empty()) return cfg_fail("`layers` must be a non-empty list");
  int blend_width = -1;
  for (size_t i = 0; i < layers->arr.size(); ++i) {
    const JValue& jl = layers->arr[i];
    const std::string where = "layers[" + std::to_string(i) + "]: ";
    if (jl.kind != JValue::Obj) return cfg_fail(where + "not an object");
    nvc_ranilix_layer L;
    const JValue* type = jl.get("type");
    const JValue* m = jl.get("mixer");
    if (!type || type->kind != JValue::Str) return cfg_fail(where + "missing `type`");
    if (!m || m->kind != JValue::Obj) return cfg_fail(where + "missing `mixer`");
    if (type->str == "attention") {
      L.kind = nvc_ranilix_layer::Attention;
      if (!parse_softmax_attn(m, L.attn, err)) return cfg_fail(where + "mixer: " + err);
      const JValue* mask = m->get("mask");
      if (mask && mask->kind == JValue::Obj) {
        if (!get_int(mask, "size", L.attn.window, 1, err)) return cfg_fail(where + "mixer.mask: " + err);
      } else if (mask && mask->kind != JValue::Null) {
        return cfg_fail(where + "mixer.mask must be an object or null");
      }
      const JValue* vm = m->get("v_mix");
      if (vm && vm->kind == JValue::Bool) L.attn.blend_values = vm->b;
      else if (vm && vm->kind != JValue::Null) return cfg_fail(where + "mixer.v_mix must be true or false");
      if (L.attn.blend_values) {
        const int wv = L.attn.kv_heads * L.attn.vdim;
        if (blend_width >= 0 && wv != blend_width) return cfg_fail(where + "layers that blend values must have equal kv_heads * vdim");
        blend_width = wv;
      }
    } else if (type->str == "parallel") {
      L.kind = nvc_ranilix_layer::Parallel;
      const JValue* left = m->get("left");
      const JValue* right = m->get("right");
      if (!left || left->kind != JValue::Obj || !right || right->kind != JValue::Obj) return cfg_fail(where + "mixer needs `left` and `right`");
      if (!parse_softmax_attn(left, L.attn, err)) return cfg_fail(where + "mixer.left: " + err);
      if (!get_int(right, "heads", L.ret.heads, 1, err) || !get_int(right, "dim", L.ret.dim, 1, err) ||
          !get_int(right, "vdim", L.ret.vdim, 1, err) || !parse_rotary(right, L.ret.rot, L.ret.dim, err))
        return cfg_fail(where + "mixer.right: " + err);
      const JValue* dec = right->get("decay");
      if (!dec || dec->kind != JValue::Arr || (int)dec->arr.size() != L.ret.heads) return cfg_fail(where + "mixer.right.decay must list one number per head");
      for (auto& d : dec->arr) {
        if (d.kind != JValue::Num) return cfg_fail(where + "mixer.right.decay must list numbers");
        L.ret.decay.push_back((float)d.num);
      }
      if (!get_float(m, "left_scale", L.left_scale, err) || !get_float(m, "right_scale", L.right_scale, err)) return cfg_fail(where + "mixer: " + err);
    } else {
      return cfg_fail(where + "mixer type `" + type->str + "` is not supported");
    }
    const JValue* mlp = jl.get("mlp");
    if (mlp && mlp->kind == JValue::Obj) {
      const JValue* kind = mlp->get("kind");
      if (!kind || kind->kind != JValue::Str || kind->str != "dense") return cfg_fail(where + "mlp: only kind `dense` is supported");
      if (!get_int(mlp, "ff", L.ff, 1, err)) return cfg_fail(where + "mlp: " + err);
    } else if (mlp && mlp->kind != JValue::Null) {
      return cfg_fail(where + "`mlp` must be an object or null");
    }
    c.layers.push_back(L);
  }
  return NVC_OK;
}


int parse_fefozen(const JValue& root, nvc_fefozen_config& c) {
  std::string err;
  if (!get_int(&root, "vocab", c.vocab, 1, err) || !get_int(&root, "width", c.width, 1, err)) return cfg_fail(err);
  const JValue* norm = root.get("norm");
  if (!norm || norm->kind != JValue::Obj || !get_float(norm, "eps", c.eps, err)) return cfg_fail("norm.eps: " + err);
  const JValue* layers = root.get("layers");
  if (!layers || layers->kind != JValue::Arr || layers->arr.empty()) return cfg_fail("`layers` must be a non-empty list");
  for (size_t i = 0; i < layers->arr.size(); ++i) {
    const JValue& jl = layers->arr[i];
    const std::string where = "layers[" + std::to_string(i) + "]: ";
    if (jl.kind != JValue::Obj) return cfg_fail(where + "not an object");
    nvc_fefozen_layer L;
    const JValue* type = jl.get("type");
    const JValue* m = jl.get("mixer");
    if (!type || type->kind != JValue::Str) return cfg_fail(where + "missing `type`");
    if (!m || m->kind != JValue::Obj) return cfg_fail(where + "missing `mixer`");
    if (type->str == "latent_attention" || type->str == "latent_attention_2") {
      L.kind = nvc_fefozen_layer::Latent;
      auto& a = L.lat;
      a.rot_half = type->str == "latent_attention_2";
      a.sink = !a.rot_half;
      if (!get_int(m, "heads", a.heads, 1, err) || !get_int(m, "dim", a.dim, 1, err) || !get_int(m, "rot_dim", a.rot_dim, 0, err) ||
          !get_int(m, "vdim", a.vdim, 1, err) || !get_int(m, "kv_rank", a.kv_rank, 1, err) || !get_int(m, "q_rank", a.q_rank, 1, err) ||
          !get_float(m, "scale", a.scale, err) || !parse_rotary(m, a.rot, a.rot_dim, err))
        return cfg_fail(where + "mixer: " + err);
      const JValue* from = m->get("kv_from");
      if (from && from->kind != JValue::Null) {
        if (!get_int(m, "kv_from", a.kv_from, 0, err)) return cfg_fail(where + "mixer: " + err);
        if (a.kv_from >= (int)i) return cfg_fail(where + "mixer.kv_from must name an earlier layer");
        const auto& src = c.layers[a.kv_from];
        if (src.kind != nvc_fefozen_layer::Latent || src.lat.kv_from >= 0) return cfg_fail(where + "mixer.kv_from must name a latent-attention layer with a cache of its own");
        if (src.lat.kv_rank != a.kv_rank || src.lat.rot_dim != a.rot_dim || src.lat.rot.dims != a.rot.dims || src.lat.rot.base != a.rot.base ||
            src.lat.rot_half != a.rot_half)
          return cfg_fail(where + "mixer.kv_from: kv_rank, rot_dim and the rotation must equal the named layer's");
      }
    } else if (type->str == "delta") {
      L.kind = nvc_fefozen_layer::Delta;
      auto& d = L.delta;
      if (!get_int(m, "heads", d.heads, 1, err) || !get_int(m, "kv_heads", d.kv_heads, 1, err) || !get_int(m, "dim", d.dim, 1, err) ||
          !get_int(m, "vdim", d.vdim, 1, err) || !get_int(m, "conv", d.taps, 1, err))
        return cfg_fail(where + "mixer: " + err);
      if (d.heads % d.kv_heads != 0) return cfg_fail(where + "mixer: heads must be a multiple of kv_heads");
    } else {
      return cfg_fail(where + "mixer type `" + type->str + "` is not supported");
    }
    const JValue* mlp = jl.get("mlp");
    if (mlp && mlp->kind == JValue::Obj) {
      const JValue* kind = mlp->get("kind");
      if (!kind || kind->kind != JValue::Str) return cfg_fail(where + "mlp: missing `kind`");
      if (kind->str == "dense") {
        L.mlp.kind = nvc_routed_mlp_spec::Dense;
        if (!get_int(mlp, "ff", L.mlp.ff, 1, err)) return cfg_fail(where + "mlp: " + err);
      } else if (kind->str == "moe") {
        L.mlp.kind = nvc_routed_mlp_spec::Moe;
        const JValue* r = mlp->get("router");
        const JValue* e = mlp->get("expert");
        if (!r || !e) return cfg_fail(where + "mlp: a mixture of experts needs `router` and `expert`");
        if (!get_int(r, "experts", L.mlp.experts, 0, err) || !get_int(r, "top", L.mlp.top, 1, err) || !get_int(e, "ff", L.mlp.expert_ff, 1, err) ||
            !get_float(e, "limit", L.mlp.limit, err))
          return cfg_fail(where + "mlp: " + err);
        if (r->get("identity") && r->get("identity")->kind != JValue::Null && !get_int(r, "identity", L.mlp.identity, 0, err))
          return cfg_fail(where + "mlp: " + err);
        if (L.mlp.experts + L.mlp.identity < 1 || L.mlp.top > L.mlp.experts + L.mlp.identity) return cfg_fail(where + "mlp: top exceeds the experts");
        if (L.mlp.experts + L.mlp.identity > 256) return cfg_fail(where + "mlp: at most 256 experts, identity experts included");
      } else {
        return cfg_fail(where + "mlp kind `" + kind->str + "` is not supported");
      }
    } else if (mlp && mlp->kind != JValue::Null) {
      return cfg_fail(where + "`mlp` must be an object or null");
    }
    c.layers.push_back(L);
  }
  return NVC_OK;
}

int parse_batatar(const JValue& root, nvc_batatar_config& c) {
  std::string err;
  if (!get_int(&root, "vocab", c.vocab, 1, err) || !get_int(&root, "width", c.width, 1, err) ||
      !get_float(&root, "residual_mult", c.residual_mult, err))
    return cfg_fail(err);
  const JValue* norm = root.get("norm");
  if (!norm || norm->kind != JValue::Obj || !get_float(norm, "eps", c.eps, err)) return cfg_fail("norm.eps: " + err);
  const JValue* layers = root.get("layers");
  if (!layers || layers->kind != JValue::Arr || layers->arr.empty()) return cfg_fail("`layers` must be a non-empty list");
  for (size_t i = 0; i < layers->arr.size(); ++i) {
    const JValue& jl = layers->arr[i];
    const std::string where = "layers[" + std::to_string(i) + "]: ";
    if (jl.kind != JValue::Obj) return cfg_fail(where + "not an object");
    nvc_batatar_layer L;
    const JValue* type = jl.get("type");
    const JValue* m = jl.get("mixer");
    if (!type || type->kind != JValue::Str) return cfg_fail(where + "missing `type`");
    if (!m || m->kind != JValue::Obj) return cfg_fail(where + "missing `mixer`");
    if (type->str == "parallel") {
      L.kind = nvc_batatar_layer::Parallel;
      const JValue* l = m->get("left");
      const JValue* r = m->get("right");
      if (!l || l->kind != JValue::Obj || !r || r->kind != JValue::Obj) return cfg_fail(where + "a parallel mixer needs `left` and `right`");
      auto& a = L.attn;
      if (!get_int(l, "heads", a.heads, 1, err) || !get_int(l, "kv_heads", a.kv_heads, 1, err) || !get_int(l, "dim", a.dim, 1, err) ||
          !get_int(l, "vdim", a.vdim, 1, err) || !get_float(l, "scale", a.scale, err))
        return cfg_fail(where + "mixer.left: " + err);
      if (a.heads % a.kv_heads != 0) return cfg_fail(where + "mixer.left: heads must be a multiple of kv_heads");
      if (const JValue* cap = l->get("softcap"); cap && cap->kind != JValue::Null) {
        if (!get_float(l, "softcap", a.softcap, err) || !(a.softcap > 0.f)) return cfg_fail(where + "mixer.left: softcap must be a positive number");
      }
      if (const JValue* mask = l->get("mask"); mask && mask->kind != JValue::Null) {
        if (mask->kind != JValue::Obj || !get_int(mask, "size", a.chunk, 1, err)) return cfg_fail(where + "mixer.left.mask: " + err);
      }
      auto& d = L.ssd;
      if (!get_int(r, "heads", d.heads, 1, err) || !get_int(r, "vdim", d.vdim, 1, err) || !get_int(r, "state", d.state, 1, err) ||
          !get_int(r, "groups", d.groups, 1, err) || !get_int(r, "conv", d.taps, 1, err) || !get_int(r, "norm_groups", d.norm_groups, 1, err))
        return cfg_fail(where + "mixer.right: " + err);
      if (d.heads % d.groups != 0) return cfg_fail(where + "mixer.right: heads must be a multiple of groups");
      if ((d.heads * d.vdim) % d.norm_groups != 0) return cfg_fail(where + "mixer.right: heads * vdim must be a multiple of norm_groups");
      if (d.taps > 16) return cfg_fail(where + "mixer.right: at most 16 taps");
    } else if (type->str == "lightning") {
      L.kind = nvc_batatar_layer::Lightning;
      auto& a = L.lin;
      if (!get_int(m, "heads", a.heads, 1, err) || !get_int(m, "dim", a.dim, 1, err) || !get_int(m, "vdim", a.vdim, 1, err))
        return cfg_fail(where + "mixer: " + err);
      const JValue* dec = m->get("decay");
      if (!dec || dec->kind != JValue::Arr || (int)dec->arr.size() != a.heads) return cfg_fail(where + "mixer.decay must list one number per head");
      for (const JValue& v : dec->arr) {
        if (v.kind != JValue::Num || v.num < 0.0 || v.num > 1.0) return cfg_fail(where + "mixer.decay: numbers in [0, 1]");
        a.decay.push_back((float)v.num);
      }
    } else {
      return cfg_fail(where + "mixer type `" + type->str + "` is not supported");
    }
    const JValue* mlp = jl.get("mlp");
    if (mlp && mlp->kind == JValue::Obj) {
      const JValue* kind = mlp->get("kind");
      if (!kind || kind->kind != JValue::Str) return cfg_fail(where + "mlp: missing `kind`");
      if (kind->str != "moe") return cfg_fail(where + "mlp kind `" + kind->str + "` is not supported");
      L.mlp.kind = nvc_routed_mlp_spec::Moe;
      const JValue* r = mlp->get("router");
      const JValue* e = mlp->get("expert");
      if (!r || !e) return cfg_fail(where + "mlp: a mixture of experts needs `router` and `expert`");
      if (!get_int(r, "experts", L.mlp.experts, 1, err) || !get_int(r, "top", L.mlp.top, 1, err) || !get_int(e, "ff", L.mlp.expert_ff, 1, err))
        return cfg_fail(where + "mlp: " + err);
      if (L.mlp.top > L.mlp.experts) return cfg_fail(where + "mlp: top exceeds the experts");
      if (L.mlp.experts > 256) return cfg_fail(where + "mlp: at most 256 experts");
    } else if (mlp && mlp->kind != JValue::Null) {
      return cfg_fail(where + "`mlp` must be an object or null");
    }
    c.layers.push_back(L);
  }
  const JValue* loop = root.get("loop");
  if (loop && loop->kind == JValue::Obj) {
    c.looped = true;
    if (!get_int(loop, "start", c.loop_start, 0, err) || !get_int(loop, "stop", c.loop_stop, 0, err) || !get_int(loop, "times", c.loop_times, 1, err))
      return cfg_fail("loop: " + err);
    if (c.loop_start >= c.loop_stop || c.loop_stop > (int)c.layers.size()) return cfg_fail("loop: 0 <= start < stop <= number of layers");
  } else if (loop && loop->kind != JValue::Null) {
    return cfg_fail("`loop` must be an object or null");
  }
  return NVC_OK;
}

}  // namespace

std::vector<nvc_karuzen_config::Run> nvc_karuzen_config::runs() const {
  std::vector<Run> out;
  for (int i = 0; i < loop_start; ++i) out.push_back({i, 0, false});
  for (int t = 0; t < (loop_stop > loop_start ? loop_times : 0); ++t)
    for (int i = loop_start; i < loop_stop; ++i) out.push_back({i, t, t > 0 && i == loop_start});
  for (int i = loop_stop; i < (int)layers.size(); ++i) out.push_back({i, 0, false});
  return out;
}

std::vector<nvc_batatar_config::Run> nvc_batatar_config::runs() const {
  std::vector<Run> out;
  const int n = (int)layers.size();
  if (!looped) {
    for (int i = 0; i < n; ++i) out.push_back({i, 0, false});
    return out;
  }
  for (int i = 0; i < loop_start; ++i) out.push_back({i, 0, false});
  for (int t = 0; t < loop_times; ++t)
    for (int i = loop_start; i < loop_stop; ++i) out.push_back({i, t, i == loop_start});
  for (int i = loop_stop; i < n; ++i) out.push_back({i, 0, false});
  return out;
}

extern "C" {

const char* nvc_model_config_last_error(void) { return g_cfg_error.c_str(); }

int nvc_model_config_from_json(const char* text, nvc_model_config** out) {
  if (!text || !out) return cfg_fail("null pointer");
  *out = nullptr;
  JValue root;
  std::string err;
  if (!parse_json(text, strlen(text), root, err) || root.kind != JValue::Obj) return cfg_fail("config is not a JSON object: " + err);
  std::string arch;
  if (const JValue* a = root.get("architecture"); a && a->kind == JValue::Str) arch = a->str;
  if (arch.empty())
    if (const JValue* a = root.get("architectures"); a && a->kind == JValue::Arr && !a->arr.empty() && a->arr[0].kind == JValue::Str)
      arch = a->arr[0].str;
  if (arch.empty())
    if (const JValue* a = root.get("model_type"); a && a->kind == JValue::Str && a->str == "qwen3") arch = "Qwen3ForCausalLM";
  auto* c = new nvc_model_config();
  c->architecture = arch;
  int rc = NVC_OK;
  if (arch == "Karuzen") {
    rc = parse_karuzen(root, c->karuzen);
  } else if (arch == "Ranilix") {
    rc = parse_ranilix(root, c->ranilix);
  } else if (arch == "Fefozen") {
    rc = parse_fefozen(root, c->fefozen);
  } else if (arch == "Batatar") {
    rc = parse_batatar(root, c->batatar);
  } else if (arch == "Qwen3ForCausalLM") {
    // parsed by nvc_qwen3_config_from_hf_dir (hf_loader.cpp) when loaded from a directory
  } else {
    rc = cfg_fail("architecture `" + arch + "` is not registered (known: Qwen3ForCausalLM, Karuzen, Ranilix, Fefozen, Batatar)");
  }
  if (rc) { delete c; return rc; }
  *out = c;
  return NVC_OK;
}

int nvc_model_config_load(const char* model_dir, nvc_model_config** out) {
  if (!model_dir || !out) return cfg_fail("null pointer");
  std::string text;
  if (!read_file(std::string(model_dir) + "/config.json", text)) return cfg_fail(std::string("cannot read ") + model_dir + "/config.json");
  int rc = nvc_model_config_from_json(text.c_str(), out);
  if (rc) return rc;
  if ((*out)->architecture == "Qwen3ForCausalLM") {
    rc = nvc_qwen3_config_from_hf_dir(model_dir, &(*out)->qwen3, &(*out)->qwen3_tied);
    if (rc) { g_cfg_error = nvc_hf_last_error(); delete *out; *out = nullptr; }
  }
  return rc;
}

void nvc_model_config_free(nvc_model_config* c) { delete c; }
const char* nvc_model_config_architecture(const nvc_model_config* c) { return c ? c->architecture.c_str() : ""; }
int nvc_model_config_vocab(const nvc_model_config* c) {
  if (!c) return 0;
  if (c->architecture == "Ranilix") return c->ranilix.vocab;
  if (c->architecture == "Fefozen") return c->fefozen.vocab;
  if (c->architecture == "Batatar") return c->batatar.vocab;
  return c->architecture == "Karuzen" ? c->karuzen.vocab : c->qwen3.vocab_size;
}
int nvc_model_config_layer_runs(const nvc_model_config* c, int32_t* layers, int32_t* passes, int32_t* readd, int capacity) {
  if (c && (c->architecture == "Ranilix" || c->architecture == "Fefozen")) {      // no looped block: every layer runs once
    const int n = (int)(c->architecture == "Ranilix" ? c->ranilix.layers.size() : c->fefozen.layers.size());
    for (int i = 0; i < n && i < capacity; ++i) {
      if (layers) layers[i] = i;
      if (passes) passes[i] = 0;
      if (readd) readd[i] = 0;
    }
    return n;
  }
  if (c && c->architecture == "Batatar") {      // readd = 1 where a pass of the looped block opens
    const auto runs = c->batatar.runs();
    for (int i = 0; i < (int)runs.size() && i < capacity; ++i) {
      if (layers) layers[i] = runs[i].layer;
      if (passes) passes[i] = runs[i].pass;
      if (readd) readd[i] = runs[i].opens_pass ? 1 : 0;
    }
    return (int)runs.size();
  }
  if (!c || c->architecture != "Karuzen") return NVC_EINVAL;
  const auto runs = c->karuzen.runs();
  for (int i = 0; i < (int)runs.size() && i < capacity; ++i) {
    if (layers) layers[i] = runs[i].layer;
    if (passes) passes[i] = runs[i].pass;
    if (readd) readd[i] = runs[i].readd_embedding ? 1 : 0;
  }
  return (int)runs.size();
}
int nvc_model_config_qwen3(const nvc_model_config* c, nvc_qwen3_config* out, int* tied) {
  if (!c || !out || c->architecture != "Qwen3ForCausalLM") return NVC_EINVAL;
  *out = c->qwen3;
  if (tied) *tied = c->qwen3_tied;
  return NVC_OK;
}

}  // extern "C"
