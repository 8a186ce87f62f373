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

// Ranilix: a stack of parallel layers with two RMS norms of the same fp32 residual stream (one feeds the mixer, one the
// squared-relu feed-forward).  Two kinds of mixer: "attention" (grouped-query attention with biases, per-head q / k norms,
// partial interleaved rotary, a sliding window, a sink term in the softmax denominator, values blended with those of the
// first blending layer, a sigmoid output gate) and "parallel" (plain causal grouped-query attention beside retention - a
// per-head recurrent state with a fixed decay - summed with two constant weights).
struct nvc_rotary_spec {
  int dims = 0;              // leading numbers of a head that are rotated (0: none)
  float base = 10000.f;
};
struct nvc_softmax_attn_spec {     // grouped-query softmax attention
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
  float scale = 0.f;
  nvc_rotary_spec rot;       // interleaved pairs (2i, 2i + 1)
  int window = 0;            // 0: every earlier token is visible; n: the token itself and the n - 1 before it
  bool blend_values = false; // v <- (1 - lambda) v + lambda v_first
};
struct nvc_retention_spec {
  int heads = 0, dim = 0, vdim = 0;
  nvc_rotary_spec rot;       // rotate-half pairs (i, i + dims / 2)
  std::vector<float> decay;  // per head
};
struct nvc_ranilix_layer {
  enum Kind { Attention, Parallel } kind = Attention;
  nvc_softmax_attn_spec attn;      // the "attention" mixer, or the left half of "parallel"
  nvc_retention_spec ret;          // the right half of "parallel"
  float left_scale = 1.f, right_scale = 1.f;
  int ff = 0;                      // 0: no feed-forward
};
struct nvc_ranilix_config {
  int vocab = 0, width = 0;
  float eps = 1e-5f;
  float embedding_scale = 1.f;
  std::vector<nvc_ranilix_layer> layers;
  int first_blend_layer() const {
    for (size_t i = 0; i < layers.size(); ++i)
      if (layers[i].kind == nvc_ranilix_layer::Attention && layers[i].attn.blend_values) return (int)i;
    return -1;
  }
  bool has_state() const {
    for (auto& l : layers)
      if (l.kind == nvc_ranilix_layer::Parallel) return true;
    return false;
  }
};

// Fefozen: a stack of sequential layers with a norm in front of and behind each sublayer (RMS norms whose weights are stored
// around zero), x <- x + n1b(mixer(n1(x))), x <- x + n2b(ff(n2(x))).  Mixers: latent attention with a rotated key part that all
// heads share (a token leaves [normed latent | rotated part] in the cache; optional sink; sigmoid output gate; a layer may read
// another layer's rows), or the gated delta rule (short convolutions, a per-head recurrent state).  Feed-forward: dense tanh-gelu
// or softmax-routed experts with identity experts and clamped gated units.  Tied logits.
struct nvc_latent_attn_spec {
  int heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, q_rank = 0;
  float scale = 0.f;
  nvc_rotary_spec rot;       // on the rot_dim part of queries and of the shared key part
  bool rot_half = false;     // pairs (i, i + dims / 2) instead of (2i, 2i + 1)
  bool sink = false;         // one more term exp(sink_h) in the softmax denominator
  int kv_from = -1;          // >= 0: no key / value down-projection of its own, reads that layer's cache rows
};
struct nvc_delta_spec {
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, taps = 1;
};
struct nvc_routed_mlp_spec {
  enum Kind { None, Dense, Moe } kind = None;
  int ff = 0;                                       // dense
  int experts = 0, identity = 0, top = 0, expert_ff = 0;   // moe: `identity` pass-through experts behind the real ones
  float limit = 0.f;                                // clamp of the gated units
};
struct nvc_fefozen_layer {
  enum Kind { Latent, Delta } kind = Latent;
  nvc_latent_attn_spec lat;
  nvc_delta_spec delta;
  nvc_routed_mlp_spec mlp;
};
struct nvc_fefozen_config {
  int vocab = 0, width = 0;
  float eps = 1e-5f;
  std::vector<nvc_fefozen_layer> layers;
  bool has_state() const {
    for (auto& l : layers)
      if (l.kind == nvc_fefozen_layer::Delta) return true;
    return false;
  }
};

// Batatar: a stack of sequential pre-normed layers on an fp32 residual stream with one constant factor on both branches,
// x <- x + m mixer(n1(x)), x <- x + m ff(n2(x)).  Mixers: "parallel" - grouped-query attention without positions (biases, unit-rms
// q and k heads, capped scores, keys of the query's own chunk only, a sink of score zero, one sigmoid gate per head) beside a
// selective state space layer (short convolution, a decay per token and head, a grouped gated norm), each side normed over the
// width, halved and summed - or "lightning" (linear attention with a constant decay per head, one norm over all heads, a sigmoid
// gate).  Feed-forward: sigmoid-routed experts whose router weight multiplies their input.  A block of layers may run several
// passes with the same weights; every pass has its own cache and state and opens with a projection of [x ; embedding] and a
// vector of its own.
struct nvc_chunk_attn_spec {
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
  float scale = 0.f;
  float softcap = 0.f;       // 0: scores are not capped
  int chunk = 0;             // 0: every earlier token is visible; n: position i sees j <= i with floor(i / n) = floor(j / n)
};
struct nvc_ssd_spec {
  int heads = 0, vdim = 0, state = 0, groups = 1, taps = 1, norm_groups = 1;
};
struct nvc_lightning_spec {
  int heads = 0, dim = 0, vdim = 0;
  std::vector<float> decay;  // per head
};
struct nvc_batatar_layer {
  enum Kind { Parallel, Lightning } kind = Parallel;
  nvc_chunk_attn_spec attn;        // left half of "parallel"
  nvc_ssd_spec ssd;                // right half of "parallel"
  nvc_lightning_spec lin;
  nvc_routed_mlp_spec mlp;         // None or Moe (no identity experts, no clamp)
};
struct nvc_batatar_config {
  int vocab = 0, width = 0;
  float eps = 1e-5f;
  float residual_mult = 1.f;
  std::vector<nvc_batatar_layer> layers;
  bool looped = false;             // config.json has `loop`: layers [loop_start, loop_stop) run loop_times passes
  int loop_start = 0, loop_stop = 0, loop_times = 1;
  struct Run { int layer; int pass; bool opens_pass; };
  std::vector<Run> runs() const;
  bool has_state() const { return !layers.empty(); }     // every mixer of the design keeps a recurrent state
};

struct nvc_model_config {
  std::string architecture;   // "Qwen3ForCausalLM", "Karuzen", "Ranilix", "Fefozen" or "Batatar"
  nvc_qwen3_config qwen3{};
  int qwen3_tied = 0;
  nvc_karuzen_config karuzen;
  nvc_ranilix_config ranilix;
  nvc_fefozen_config fefozen;
  nvc_batatar_config batatar;
};
