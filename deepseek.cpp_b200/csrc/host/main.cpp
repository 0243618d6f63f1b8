// main.cpp — `main <checkpoint_dir> [options]`: the reference's CLI surface (src/main.cpp:18-43, 594-691) over libdsk.so.
// Host side in C++ calling CUDA through the thin C-ABI (include/dsk.h): .dseek loader, trie tokenizer
// (src/tokenizer.cpp:3-94), completion + perplexity modes.  The forward pass is dsk_forward(); sampling (greedy, temperature /
// top-p, perplexity probabilities) runs on the device through dsk_sample / dsk_sample_prob, so no logits cross PCIe.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/dsk.h"
#include "dseek_loader.h"
#include "json_min.h"

static void error_usage() {
  fprintf(stderr, "Usage:   main <checkpoint_dir> [options]\n");
  fprintf(stderr, "Example: main model_weights_dir/ -i \"Q: What is the meaning of life?\"\n");
  fprintf(stderr, "Options:\n");
  fprintf(stderr, "  -h Display this help message\n");
  fprintf(stderr, "  -L Locks model weights to RAM while they are uploaded\n");
  fprintf(stderr, "  -m [completion,perplexity] which mode to run in (default - completion)\n");
  fprintf(stderr, "  -T <int> sliding window context length (0 - max)\n");
  fprintf(stderr, "  -g <int> CUDA device (default 0)\n");
  fprintf(stderr, "  -q [bf16,fp32] matrix type of config.json checkpoints (layer-list models; default bf16)\n");
  fprintf(stderr, "  -I <ids> prompt as comma-separated token ids (checkpoints without a tokenizer)\n");
  fprintf(stderr, "Completion mode options:\n");
  fprintf(stderr, "  -n <int>    number of steps to run for in completion mode, default 256. 0 = max_seq_len, -1 = infinite\n");
  fprintf(stderr, "  -i <string> input prompt | -f <filepath> input file with prompt\n");
  fprintf(stderr, "  -t <float> temperature (default - 1.0; 0 = greedy)   -p <float> p for top-p sampling (default - 0.95)\n");
  fprintf(stderr, "Perplexity mode options:  -i <string> | -f <filepath>\n");
  exit(1);
}

static double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

// ---- tokenizer: greedy longest-match over a trie, byte fallback (src/tokenizer.cpp:3-94) ----------------------------
struct TokenTrie { std::unordered_map<char, std::unique_ptr<TokenTrie>> children; int token_id = -1; };
struct Tokenizer {
  std::vector<std::string> vocab;
  TokenTrie root;
  int bos_id = -1, eos_id = -1, eot_id = -1, byte_fallback_start = -1;
  Tokenizer(const DseekData& d) {
    bos_id = std::stoi(d.metadata.at("bos_token_id"));
    eos_id = std::stoi(d.metadata.at("eos_token_id"));
    const DseekTensor& t = d.tensors.at("tokenizer.tokens");
    const char* p = (const char*)t.data; const char* end = p + t.size;
    for (; p < end; p++) { const char* s = p; while (p < end && *p != '\0') p++; vocab.emplace_back(s, p - s); }
    for (size_t i = 0; i < vocab.size(); i++) {
      if (vocab[i] == "<0x00>") byte_fallback_start = (int)i;
      else if (vocab[i] == "<|eot_id|>" || vocab[i] == "<|end|>" || vocab[i] == "<|im_end|>") eot_id = (int)i;
      TokenTrie* n = &root;
      for (char c : vocab[i]) { auto& ch = n->children[c]; if (!ch) ch = std::make_unique<TokenTrie>(); n = ch.get(); }
      n->token_id = (int)i;
    }
  }
  std::vector<int> encode(const std::string& text, bool bos) const {
    std::vector<int> out;
    if (bos) out.push_back(bos_id);
    for (size_t i = 0; i < text.size();) {
      size_t l = 0, valid_l = 0; const TokenTrie* n = &root; const TokenTrie* valid = nullptr;
      while (i + l < text.size()) {
        auto it = n->children.find(text[i + l]);
        if (it == n->children.end()) break;
        n = it->second.get(); l++;
        if (n->token_id >= 0) { valid = n; valid_l = l; }
      }
      if (!valid) { if (byte_fallback_start >= 0) out.push_back((unsigned char)text[i] + byte_fallback_start); i++; }
      else { out.push_back(valid->token_id); i += valid_l; }
    }
    return out;
  }
  std::string decode_one(int prev, int tok) const {
    const std::string& piece = vocab[tok];
    if (prev == bos_id && !piece.empty() && piece[0] == ' ') return piece.substr(1);
    if (byte_fallback_start >= 0 && tok >= byte_fallback_start && tok - byte_fallback_start < 256) return std::string(1, (char)(tok - byte_fallback_start));
    return piece;
  }
};

// Sampling runs on the device (dsk_sample / dsk_sample_prob: Sampler::sample / sample_prob, src/sampler.cpp:12-75); the host
// only draws the random number, with the reference's generator and seed policy (std::srand / std::rand, src/sampler.cpp:7-10,65).
static int meta_i(const DseekData& d, const char* k, int def, bool required = false) {
  auto it = d.metadata.find(k);
  if (it == d.metadata.end()) { if (required) { fprintf(stderr, "FATAL: missing metadata %s\n", k); exit(1); } return def; }
  return std::stoi(it->second);
}
static float meta_f(const DseekData& d, const char* k, float def) { auto it = d.metadata.find(k); return it == d.metadata.end() ? def : std::stof(it->second); }
static std::string meta_s(const DseekData& d, const char* k, const char* def) { auto it = d.metadata.find(k); return it == d.metadata.end() ? def : it->second; }

// Config::from_yalm (src/model.cpp:22-127)
static dsk_config config_from(const DseekData& d, int context) {
  dsk_config c{};
  c.dim = meta_i(d, "dim", 0, true); c.hidden_dim = meta_i(d, "hidden_dim", 0, true); c.n_layers = meta_i(d, "n_layers", 0, true);
  c.n_heads = meta_i(d, "n_heads", 0, true); c.vocab_size = meta_i(d, "vocab_size", 0, true); c.max_seq_len = meta_i(d, "max_seq_len", 0, true);
  if (context) c.max_seq_len = std::min(c.max_seq_len, context);
  c.rope_theta = meta_f(d, "rope_theta", 10000.f); c.norm_eps = meta_f(d, "norm_eps", 1e-5f);
  c.act_silu = meta_s(d, "act_type", "gelu") == "silu";
  c.first_k_dense_replace = meta_i(d, "first_k_dense_replace", 0);
  c.n_shared_experts = meta_i(d, "n_shared_experts", 0); c.n_routed_experts = meta_i(d, "n_routed_experts", 0);
  c.n_active_routed = meta_i(d, "n_active_routed", 0); c.moe_intermediate_size = meta_i(d, "moe_intermediate_size", 0);
  c.routed_scaling_factor = meta_f(d, "routed_scaling_factor", 1.0f); c.n_group = meta_i(d, "n_group", 1);
  c.norm_topk_prob = meta_s(d, "norm_topk_prob", "False") == "True";
  c.scoring_sigmoid = meta_s(d, "scoring_func", "softmax") == "sigmoid";
  c.topk_group = meta_i(d, "topk_group", 0);
  std::string tm = meta_s(d, "topk_method", "");
  if (tm == "noaux_tc") { fprintf(stderr, "FATAL: topk_method noaux_tc unsupported (src/model.cpp:51-53)\n"); exit(1); }
  c.topk_method = tm == "group_limited_greedy";
  c.is_v3 = meta_s(d, "arch", "") == "DeepseekV3ForCausalLM";
  c.kv_lora_rank = meta_i(d, "kv_lora_rank", 0); c.q_lora_rank = meta_i(d, "q_lora_rank", 0);
  c.qk_nope_head_dim = meta_i(d, "qk_nope_head_dim", 0); c.qk_rope_head_dim = meta_i(d, "qk_rope_head_dim", 0); c.v_head_dim = meta_i(d, "v_head_dim", 0);
  std::string q = meta_s(d, "quant", "");
  if (q == "fp32") c.quant = DSK_F32; else if (q == "fp16") c.quant = DSK_F16; else if (q == "f8e5m2") c.quant = DSK_F8E5M2;
  else if (q == "q2_k") c.quant = DSK_Q2_K; else if (q == "q3_k") c.quant = DSK_Q3_K;
  else { fprintf(stderr, "FATAL: unsupported quant: %s\n", q.c_str()); exit(1); }
  c.bs0 = meta_i(d, "quantization_block_size_0", 0); c.bs1 = meta_i(d, "quantization_block_size_1", 0);
  c.original_max_position = meta_i(d, "rope_scaling_original_max_position_embeddings", 4096);
  c.use_mla = meta_i(d, "use_mla", 0) ? 1 : 0;
  return c;
}

#define DSK_OK(call) do { if ((call) != 0) { fprintf(stderr, "FATAL: %s: %s\n", #call, dsk_last_error()); exit(1); } } while (0)

static bool file_exists(const std::string& p) { std::ifstream f(p); return f.good(); }

// ---- layer-list checkpoints: config.json ("architecture" picks the family) + model.safetensors --------------------------------------
// Mixer "type" strings -> mixer kernels; two names may denote one mechanism.
static int mixer_of(const std::string& type) {
  if (type == "mamba2" || type == "mamba2_2") return DSK_MIX_SSD;
  if (type == "latent_attention") return DSK_MIX_LATENT_SWA;
  return -1;
}
static bool hybrid_config_from(const JValue& j, const std::string& quant, int context, dsk_hybrid_config* hc, std::vector<dsk_layer_spec>* specs) {
  const JValue& layers = j.at("layers");
  if (layers.kind != JValue::Arr || layers.arr.empty()) { fprintf(stderr, "FATAL: config.json has no layers\n"); return false; }
  *hc = dsk_hybrid_config{};
  hc->dim = j.integer("width", 0); hc->vocab_size = j.integer("vocab", 0); hc->n_layers = (int)layers.arr.size();
  hc->max_seq_len = context > 0 ? context : 1 << 30;
  hc->quant = quant == "fp32" ? DSK_F32 : DSK_BF16;
  hc->chunk = context > 0 ? std::min(256, context) : 256;
  hc->norm_eps = (float)j.at("norm").number("eps", 1e-5); hc->norm_groups = j.at("norm").integer("groups", 1);
  hc->residual_mult = (float)j.number("residual_mult", 1.0); hc->logit_scale = (float)j.number("logit_scale", 1.0);
  hc->side_dim = j.at("token_side").integer("dim", 0);
  hc->block = DSK_BLOCK_PARALLEL; hc->norm_kind = DSK_NORM_RMS; hc->tie_head = 1;
  for (size_t i = 0; i < layers.arr.size(); i++) {
    const JValue& lc = layers.arr[i];
    const JValue& mx = lc.at("mixer");
    dsk_layer_spec sp{};
    sp.mixer = mixer_of(lc.at("type").str);
    sp.att_kv_from = -1; sp.att_mask = DSK_MASK_WINDOW;
    if (sp.mixer == DSK_MIX_SSD) {
      sp.ssm_heads = mx.integer("heads", 0); sp.ssm_vdim = mx.integer("vdim", 0); sp.ssm_state = mx.integer("state", 0);
      sp.ssm_groups = mx.integer("groups", 1); sp.ssm_conv = mx.integer("conv", 0); sp.ssm_norm_groups = mx.integer("norm_groups", 1);
    } else if (sp.mixer == DSK_MIX_LATENT_SWA) {
      sp.att_heads = mx.integer("heads", 0); sp.att_dim = mx.integer("dim", 0); sp.att_vdim = mx.integer("vdim", 0);
      sp.att_kv_rank = mx.integer("kv_rank", 0); sp.att_scale = (float)mx.number("scale", 1.0);
      sp.att_window = mx.at("mask").integer("size", 1 << 30); sp.att_kv_from = mx.integer("kv_from", -1);
    } else { fprintf(stderr, "FATAL: layer %zu: unknown mixer type %s\n", i, lc.at("type").str.c_str()); return false; }
    if (lc.has("mlp")) {
      const JValue& ff = lc.at("mlp");
      if (ff.has("kind") && ff.at("kind").str != "moe") { fprintf(stderr, "FATAL: layer %zu: unknown feed-forward kind %s\n", i, ff.at("kind").str.c_str()); return false; }
      sp.ff_kind = DSK_FF_MOE;
      sp.ff_experts = ff.at("router").integer("experts", 0); sp.ff_top = ff.at("router").integer("top", 0);
      sp.ff_router_scale = (float)ff.at("router").number("scale", 1.0);
      sp.ff_hidden = ff.at("expert").integer("ff", 0); sp.ff_limit = (float)ff.at("expert").number("limit", 0.0);
    }
    specs->push_back(sp);
  }
  return true;
}

// The Rutulix design: sandwich blocks with layer norms, grouped-query attention (values = key projection, whole-projection
// query / key norm, partial rotation with YaRN scaling, head mixing, chunk mask), dense xIELU feed-forwards, untied head, layer loop.
static bool rutulix_config_from(const JValue& j, const std::string& quant, int context, dsk_hybrid_config* hc, std::vector<dsk_layer_spec>* specs) {
  const JValue& layers = j.at("layers");
  if (layers.kind != JValue::Arr || layers.arr.empty()) { fprintf(stderr, "FATAL: config.json has no layers\n"); return false; }
  *hc = dsk_hybrid_config{};
  hc->dim = j.integer("width", 0); hc->vocab_size = j.integer("vocab", 0); hc->n_layers = (int)layers.arr.size();
  hc->max_seq_len = context > 0 ? context : 1 << 30;
  hc->quant = quant == "fp32" ? DSK_F32 : DSK_BF16;
  hc->chunk = context > 0 ? std::min(256, context) : 256;
  hc->norm_eps = (float)j.at("norm").number("eps", 1e-5); hc->norm_groups = 1;
  hc->residual_mult = 1.f; hc->logit_scale = 1.f;
  hc->block = DSK_BLOCK_SANDWICH; hc->norm_kind = DSK_NORM_LAYER; hc->tie_head = 0;
  const JValue& loop = j.at("loop");
  if (j.has("loop")) { hc->loop_start = loop.integer("start", 0); hc->loop_stop = loop.integer("stop", 0); hc->loop_times = loop.integer("times", 0); }
  for (size_t i = 0; i < layers.arr.size(); i++) {
    const JValue& lc = layers.arr[i];
    const JValue& mx = lc.at("mixer");
    if (lc.at("type").str != "attention") { fprintf(stderr, "FATAL: layer %zu: unknown mixer type %s\n", i, lc.at("type").str.c_str()); return false; }
    dsk_layer_spec sp{};
    sp.mixer = DSK_MIX_GQA; sp.att_kv_from = -1;
    sp.att_heads = mx.integer("heads", 0); sp.att_kv_heads = mx.integer("kv_heads", sp.att_heads);
    sp.att_dim = mx.integer("dim", 0); sp.att_vdim = mx.integer("vdim", 0); sp.att_scale = (float)mx.number("scale", 1.0);
    sp.att_mask = DSK_MASK_CHUNK; sp.att_window = mx.at("mask").integer("size", 1 << 30); sp.att_talk = 1;
    const JValue& rot = mx.at("rot");
    sp.rot_dims = rot.integer("dims", 0); sp.rot_base = (float)rot.number("base", 10000.0);
    if (rot.has("scaling")) {
      const JValue& sc = rot.at("scaling");
      sp.rot_factor = (float)sc.number("factor", 0.0); sp.rot_original = sc.integer("original", 0);
      sp.rot_fast = (float)sc.number("fast", 0.0); sp.rot_slow = (float)sc.number("slow", 0.0);
      if (!(sp.rot_factor > 0.f)) { fprintf(stderr, "FATAL: layer %zu: rotation scaling factor must be positive\n", i); return false; }
    }
    if (lc.has("mlp")) {
      const JValue& ff = lc.at("mlp");
      if (ff.at("kind").str != "dense") { fprintf(stderr, "FATAL: layer %zu: unknown feed-forward kind %s\n", i, ff.at("kind").str.c_str()); return false; }
      sp.ff_kind = DSK_FF_DENSE; sp.ff_hidden = ff.integer("ff", 0); sp.ff_act = DSK_ACT_XIELU;
    }
    specs->push_back(sp);
  }
  return true;
}

// The Sakusun design: post-norm blocks (input convolution, gated sublayer results, single-number RMS norms, layer scale), a scaled
// token embedding plus a bigram table, grouped-query attention with its switches on (value matrix, biases, score cap, distance-bucket
// bias, window with kept first positions, sink, value mixing) or latent attention with a query latent, a shared rotated key part and
// an output gate, gated GELU feed-forwards, an untied head.
static bool sakusun_config_from(const JValue& j, const std::string& quant, int context, dsk_hybrid_config* hc, std::vector<dsk_layer_spec>* specs) {
  const JValue& layers = j.at("layers");
  if (layers.kind != JValue::Arr || layers.arr.empty()) { fprintf(stderr, "FATAL: config.json has no layers\n"); return false; }
  *hc = dsk_hybrid_config{};
  hc->dim = j.integer("width", 0); hc->vocab_size = j.integer("vocab", 0); hc->n_layers = (int)layers.arr.size();
  hc->max_seq_len = context > 0 ? context : 1 << 30;
  hc->quant = quant == "fp32" ? DSK_F32 : DSK_BF16;
  hc->chunk = context > 0 ? std::min(256, context) : 256;
  hc->norm_eps = (float)j.at("norm").number("eps", 1e-5); hc->norm_groups = 1;
  hc->residual_mult = 1.f; hc->logit_scale = 1.f;
  hc->block = DSK_BLOCK_POST; hc->norm_kind = DSK_NORM_RMS; hc->tie_head = 0; hc->norm_scalar = 1;
  const JValue& emb = j.at("embedding");
  hc->embed_scale = (float)emb.number("scale", 1.0);
  if (emb.has("bigram")) {
    const JValue& bg = emb.at("bigram");
    hc->bigram_buckets = bg.integer("buckets", 0); hc->bigram_mul_prev = bg.integer("mul_prev", 0); hc->bigram_mul_cur = bg.integer("mul_cur", 0);
  }
  hc->canon_taps = j.at("canon").integer("taps", 0);
  hc->res_gate = 1; hc->layer_scale = 1;
  for (size_t i = 0; i < layers.arr.size(); i++) {
    const JValue& lc = layers.arr[i];
    const JValue& mx = lc.at("mixer");
    const JValue& mask = mx.at("mask");
    const std::string type = lc.at("type").str;
    dsk_layer_spec sp{};
    sp.att_kv_from = -1; sp.att_mask = DSK_MASK_WINDOW; sp.att_window = mask.integer("size", 1 << 30);
    sp.att_heads = mx.integer("heads", 0); sp.att_dim = mx.integer("dim", 0); sp.att_vdim = mx.integer("vdim", 0); sp.att_scale = (float)mx.number("scale", 1.0);
    if (type == "attention") {
      sp.mixer = DSK_MIX_GQA;
      sp.att_kv_heads = mx.integer("kv_heads", sp.att_heads);
      sp.att_value_proj = 1; sp.att_bias = 1; sp.att_sink = 1;
      sp.att_keep_first = mask.has("size") ? mask.integer("keep_first", 0) : 0;
      sp.att_softcap = (float)mx.number("softcap", 0.0); sp.att_rel_max = mx.integer("bias_max", 0);
      sp.att_vmix = mx.has("v_mix") && mx.at("v_mix").kind == JValue::Bool && mx.at("v_mix").b;
    } else if (type == "latent_attention") {
      sp.mixer = DSK_MIX_MLA;
      sp.att_kv_rank = mx.integer("kv_rank", 0); sp.att_q_rank = mx.integer("q_rank", 0); sp.att_rot_dim = mx.integer("rot_dim", 0); sp.att_out_gate = 1;
      sp.rot_dims = mx.at("rot").integer("dims", 0); sp.rot_base = (float)mx.at("rot").number("base", 10000.0);
    } else { fprintf(stderr, "FATAL: layer %zu: unknown mixer type %s\n", i, type.c_str()); return false; }
    if (lc.has("mlp")) {
      const JValue& ff = lc.at("mlp");
      if (ff.at("kind").str != "dense") { fprintf(stderr, "FATAL: layer %zu: unknown feed-forward kind %s\n", i, ff.at("kind").str.c_str()); return false; }
      sp.ff_kind = DSK_FF_DENSE; sp.ff_hidden = ff.integer("ff", 0); sp.ff_act = DSK_ACT_GEGLU;
    }
    specs->push_back(sp);
  }
  return true;
}

// The Nalizen design: post-norm blocks whose layer norms carry a bias, a token shift in front of every mixer, a scaled embedding that
// is also the head, the per-layer token input; grouped-query attention (half-split rotation with wavelength-band scaling, per-head
// query / key norm after the rotation, sliding window, output gate, optionally another layer's keys and values) or the HGRN2
// recurrence; gated dense feed-forwards or routed ones (largest logits, softmax over the chosen, squared-ReLU experts).
static bool nalizen_config_from(const JValue& j, const std::string& quant, int context, dsk_hybrid_config* hc, std::vector<dsk_layer_spec>* specs) {
  const JValue& layers = j.at("layers");
  if (layers.kind != JValue::Arr || layers.arr.empty()) { fprintf(stderr, "FATAL: config.json has no layers\n"); return false; }
  *hc = dsk_hybrid_config{};
  hc->dim = j.integer("width", 0); hc->vocab_size = j.integer("vocab", 0); hc->n_layers = (int)layers.arr.size();
  hc->max_seq_len = context > 0 ? context : 1 << 30;
  hc->quant = quant == "fp32" ? DSK_F32 : DSK_BF16;
  hc->chunk = context > 0 ? std::min(256, context) : 256;
  hc->norm_eps = (float)j.at("norm").number("eps", 1e-5); hc->norm_groups = 1;
  hc->residual_mult = 1.f; hc->logit_scale = 1.f;
  hc->side_dim = j.at("token_side").integer("dim", 0);
  hc->block = DSK_BLOCK_POST; hc->norm_kind = DSK_NORM_LAYER; hc->norm_bias = 1; hc->tie_head = 1; hc->token_shift = 1;
  hc->embed_scale = (float)j.at("embedding").number("scale", 1.0);
  for (size_t i = 0; i < layers.arr.size(); i++) {
    const JValue& lc = layers.arr[i];
    const JValue& mx = lc.at("mixer");
    const std::string type = lc.at("type").str;
    dsk_layer_spec sp{};
    sp.att_kv_from = -1;
    if (type == "attention") {
      sp.mixer = DSK_MIX_GQA;
      sp.att_heads = mx.integer("heads", 0); sp.att_kv_heads = mx.integer("kv_heads", sp.att_heads);
      sp.att_dim = mx.integer("dim", 0); sp.att_vdim = mx.integer("vdim", 0); sp.att_scale = (float)mx.number("scale", 1.0);
      sp.att_mask = DSK_MASK_WINDOW; sp.att_window = mx.at("mask").integer("size", 1 << 30);
      sp.att_value_proj = 1; sp.att_out_gate = 1; sp.att_qk_norm = DSK_QKNORM_HEAD;
      sp.att_kv_from = mx.integer("kv_from", -1);
      const JValue& rot = mx.at("rot");
      sp.rot_dims = rot.integer("dims", 0); sp.rot_base = (float)rot.number("base", 10000.0); sp.rot_layout = DSK_ROT_HALF;
      if (rot.has("scaling")) {
        const JValue& sc = rot.at("scaling");
        sp.rot_scale = DSK_ROTSCALE_BANDS; sp.rot_factor = (float)sc.number("factor", 0.0); sp.rot_original = sc.integer("original", 0);
        sp.rot_fast = (float)sc.number("high", 0.0); sp.rot_slow = (float)sc.number("low", 0.0);
        if (!(sp.rot_factor > 0.f)) { fprintf(stderr, "FATAL: layer %zu: rotation scaling factor must be positive\n", i); return false; }
      }
    } else if (type == "hgrn2") {
      sp.mixer = DSK_MIX_HGRN2;
      sp.lin_heads = mx.integer("heads", 0); sp.lin_dim = mx.integer("dim", 0); sp.lin_vdim = mx.integer("vdim", 0);
    } else { fprintf(stderr, "FATAL: layer %zu: unknown mixer type %s\n", i, type.c_str()); return false; }
    if (lc.has("mlp")) {
      const JValue& ff = lc.at("mlp");
      const std::string kind = ff.at("kind").str;
      if (kind == "dense") { sp.ff_kind = DSK_FF_DENSE; sp.ff_hidden = ff.integer("ff", 0); sp.ff_act = DSK_ACT_GEGLU; }
      else if (kind == "moe") {
        sp.ff_kind = DSK_FF_MOE; sp.ff_router = DSK_ROUTER_TOP_SOFTMAX; sp.ff_expert = DSK_EXPERT_RELU2; sp.ff_router_scale = 1.f;
        sp.ff_experts = ff.at("router").integer("experts", 0); sp.ff_top = ff.at("router").integer("top", 0); sp.ff_hidden = ff.at("expert").integer("ff", 0);
      } else { fprintf(stderr, "FATAL: layer %zu: unknown feed-forward kind %s\n", i, kind.c_str()); return false; }
    }
    specs->push_back(sp);
  }
  return true;
}

// config.json "architecture" -> builder of the C-ABI model description
typedef bool (*ArchBuilder)(const JValue&, const std::string&, int, dsk_hybrid_config*, std::vector<dsk_layer_spec>*);
static const struct { const char* name; ArchBuilder build; } kArchitectures[] = {{"Desarax", hybrid_config_from}, {"Rutulix", rutulix_config_from},
                                                                                {"Sakusun", sakusun_config_from}, {"Nalizen", nalizen_config_from}};

// completion over token ids: the prompt goes through dsk_forward_chunk (prefill in portions), then the usual
// dsk_sample -> dsk_forward loop; the ids are printed (these checkpoints carry no tokenizer).
static int run_layer_list(const std::string& dir, const std::string& quant, const std::string& prompt_ids, int context, int device, int num_steps,
                          float temperature, float top_p, bool lock) {
  std::ifstream fs(dir + "/config.json");
  std::stringstream ss; ss << fs.rdbuf();
  const std::string text = ss.str();
  JValue cfg; JReader jr{text.data(), text.data() + text.size(), ""};
  if (!jr.parse(cfg) || cfg.kind != JValue::Obj) { fprintf(stderr, "FATAL: config.json: %s\n", jr.err.c_str()); return 1; }
  const std::string arch = cfg.at("architecture").str;
  ArchBuilder builder = nullptr;
  for (const auto& a : kArchitectures) if (arch == a.name) builder = a.build;
  if (!builder) { fprintf(stderr, "FATAL: unknown architecture '%s' (known: Desarax, Rutulix, Sakusun, Nalizen)\n", arch.c_str()); return 1; }
  if (quant != "bf16" && quant != "fp32") { fprintf(stderr, "FATAL: -q must be bf16 or fp32\n"); return 1; }
  std::vector<int> enc;
  for (size_t i = 0; i < prompt_ids.size();) {
    size_t j = prompt_ids.find(',', i); if (j == std::string::npos) j = prompt_ids.size();
    if (j > i) enc.push_back(atoi(prompt_ids.substr(i, j - i).c_str()));
    i = j + 1;
  }
  if (enc.empty()) { fprintf(stderr, "No prompt provided (-I <ids>)\n"); return 1; }
  dsk_hybrid_config hc; std::vector<dsk_layer_spec> specs;
  if (!builder(cfg, quant, context, &hc, &specs)) return 1;
  DseekData data;
  std::string err = data.load_shard(dir + "/model.safetensors", lock);
  if (!err.empty()) { fprintf(stderr, "failed to load checkpoint: %s\n", err.c_str()); return 1; }
  std::cout << "loading " << arch << " model with quant: " << quant << std::endl;
  DSK_OK(dsk_init(device));
  double t0 = now_s();
  dsk_model* model = dsk_model_create_hybrid(&hc, specs.data(), 0, 1);
  if (!model) { fprintf(stderr, "FATAL: %s\n", dsk_last_error()); return 1; }
  static const char* names[] = {"F32", "F16", "BF16", "F8_E5M2", "F8_E4M3", "I32", "I16", "I8", "U8"};   // CodecDType order
  for (auto& kv : data.tensors) {
    const DseekTensor& t = kv.second;
    int dt = -1;
    for (int k = 0; k < 9; k++) if (t.dtype == names[k]) dt = k;
    DSK_OK(dsk_upload_tensor(model, t.name.c_str(), dt, t.shape, t.data, t.size, 0));
  }
  DSK_OK(dsk_model_finalize(model));
  dsk_state* state = dsk_state_create(model);
  if (!state) { fprintf(stderr, "FATAL: %s\n", dsk_last_error()); return 1; }
  std::cout << "uploaded in " << now_s() - t0 << " s (" << dsk_model_resident_bytes(model) / 1e9 << " GB resident)" << std::endl;
  srand((unsigned)(uint64_t)(now_s() * 1000));
  if (num_steps <= 0) num_steps = 256;
  const double start = now_s();
  const int32_t last = (int32_t)enc.size() - 1;
  DSK_OK(dsk_forward_chunk(model, state, enc.data(), (int)enc.size(), 0, &last, 1, nullptr, nullptr));
  const double end_hydrate = now_s();
  const size_t n_prompt = enc.size();
  for (int i = 0; i < num_steps; i++) {
    int tok = -1;
    const float coin = temperature == 0.0f ? 0.f : rand() / (float)RAND_MAX;
    DSK_OK(dsk_sample(model, state, temperature, top_p, coin, &tok));
    enc.push_back(tok);
    if (i + 1 < num_steps) DSK_OK(dsk_forward(model, state, tok, (int)enc.size() - 1, DSK_OUTPUT_LOGITS, nullptr, nullptr));
  }
  const double elapsed = now_s() - start;
  std::cout << "\nGeneration stats:\n  " << enc.size() << " tokens\n  prefill: " << n_prompt / (end_hydrate - start) << "tok/s\n  decode: "
            << (enc.size() - n_prompt) / (elapsed - (end_hydrate - start)) << "tok/s\n  total: " << elapsed << "s\n" << std::endl;
  std::cout << "generated ids:";
  for (size_t i = 0; i < enc.size(); i++) std::cout << " " << enc[i];
  std::cout << std::endl;
  dsk_state_destroy(state);
  dsk_model_destroy(model);
  return 0;
}

int main(int argc, char* argv[]) {
  if (argc < 2) error_usage();
  std::string dir = argv[1], mode = "completion", prompt, prompt_path, prompt_ids, hquant = "bf16";
  bool lock = false; int context = 0, device = 0, num_steps = 256; float temperature = 1.0f, top_p = 0.95f;
  for (int i = 2; i < argc;) {
    if (argv[i][0] != '-' || strlen(argv[i]) != 2) error_usage();
    char f = argv[i][1];
    if (f == 'h') error_usage();
    if (f == 'L') { lock = true; i++; continue; }
    if (i + 1 >= argc) error_usage();
    const char* v = argv[i + 1];
    switch (f) {
      case 'm': if (std::string("completion").rfind(v, 0) == 0) mode = "completion"; else if (std::string("perplexity").rfind(v, 0) == 0) mode = "perplexity"; else error_usage(); break;
      case 'T': context = atoi(v); break; case 'g': device = atoi(v); break; case 'n': num_steps = atoi(v); break;
      case 'q': hquant = v; break; case 'I': prompt_ids = v; break;
      case 'i': prompt = v; break; case 'f': prompt_path = v; break; case 't': temperature = (float)atof(v); break; case 'p': top_p = (float)atof(v); break;
      default: error_usage();
    }
    i += 2;
  }
  if (!prompt_path.empty()) { std::ifstream fs(prompt_path); std::stringstream ss; ss << fs.rdbuf(); prompt = ss.str(); }
  if (file_exists(dir + "/config.json"))
    return run_layer_list(dir, hquant, prompt_ids, context, device, num_steps, temperature, top_p, lock);
  if (prompt.empty()) { fprintf(stderr, "No prompt provided\n"); error_usage(); }

  DseekData data;
  std::string err = data.load(dir, lock);
  if (!err.empty()) { fprintf(stderr, "failed to load checkpoint: %s\n", err.c_str()); return 1; }
  dsk_config cfg = config_from(data, context);
  std::cout << "loading model with quant: " << data.metadata["quant"] << std::endl;
  DSK_OK(dsk_init(device));
  double t0 = now_s();
  dsk_model* model = dsk_model_create(&cfg, 0, 1);
  if (!model) { fprintf(stderr, "FATAL: %s\n", dsk_last_error()); return 1; }
  size_t up = 0;
  for (auto& kv : data.tensors) {
    const DseekTensor& t = kv.second;
    static const char* names[] = {"F32", "F16", "BF16", "F8_E5M2", "F8_E4M3", "I32", "I16", "I8", "U8"};   // CodecDType order
    int dt = -1;
    for (int k = 0; k < 9; k++) if (t.dtype == names[k]) dt = k;
    if (dt < 0) { fprintf(stderr, "FATAL: tensor %s has unknown dtype %s\n", t.name.c_str(), t.dtype.c_str()); return 1; }
    DSK_OK(dsk_upload_tensor(model, t.name.c_str(), dt, t.shape, t.data, t.size, 0));
    up += t.size;
  }
  DSK_OK(dsk_model_finalize(model));
  dsk_state* state = dsk_state_create(model);
  if (!state) { fprintf(stderr, "FATAL: %s\n", dsk_last_error()); return 1; }
  std::cout << "uploaded " << up / 1e9 << " GB in " << now_s() - t0 << " s (" << dsk_model_resident_bytes(model) / 1e9 << " GB resident)" << std::endl;
  std::cout << "Model active bytes per token (algorithmic): " << dsk_model_active_bytes_per_token(model) << std::endl;

  Tokenizer tokenizer(data);
  srand((unsigned)(uint64_t)(now_s() * 1000));
  if (num_steps == 0) num_steps = cfg.max_seq_len;
  DSK_OK(dsk_forward(model, state, 0, 0, DSK_OUTPUT_LOGITS, nullptr, nullptr));   // warm-up (graph capture), like src/main.cpp:299-303
  std::vector<int> enc = tokenizer.encode(prompt, true);
  std::cout << "[";
  for (size_t i = 0; i < enc.size(); i++) std::cout << (i ? "," : "") << enc[i];
  std::cout << "]" << std::endl;

  if (mode == "perplexity") {  // src/main.cpp:371-431
    double sum_nll = 0, ss = 0; size_t n = 0;
    for (size_t pos = 0; pos + 1 < enc.size(); pos++) {
      DSK_OK(dsk_forward(model, state, enc[pos], (int)pos, DSK_OUTPUT_LOGITS, nullptr, nullptr));
      float pr = 0.f;
      DSK_OK(dsk_sample_prob(model, state, enc[pos + 1], &pr));
      double lp = std::log((double)pr);
      sum_nll += -lp; ss += lp * lp; n++;
    }
    double mean = sum_nll / n, var = ss / n - mean * mean;
    std::cout << "perplexity: " << std::exp(mean) << " ± " << std::exp(mean) * std::sqrt(std::max(0.0, var) / n) << " over " << n << " tokens" << std::endl;
    return 0;
  }
  double start = now_s();
  for (size_t pos = 0; pos < enc.size(); pos++) {   // hydrate (src/main.cpp:312-319)
    bool last = pos + 1 == enc.size();
    DSK_OK(dsk_forward(model, state, enc[pos], (int)pos, last ? DSK_OUTPUT_LOGITS : DSK_HYDRATE_KV_CACHE, nullptr, nullptr));
  }
  double end_hydrate = now_s();
  for (int i = 0; i < num_steps || num_steps == -1; i++) {   // src/main.cpp:324-335
    int tok = -1;
    const float coin = temperature == 0.0f ? 0.f : rand() / (float)RAND_MAX;
    DSK_OK(dsk_sample(model, state, temperature, top_p, coin, &tok));
    std::cout << tokenizer.decode_one(enc.back(), tok) << std::flush;
    enc.push_back(tok);
    if (tok == tokenizer.eos_id || tok == tokenizer.eot_id) break;
    if ((int)enc.size() - 1 >= cfg.max_seq_len && cfg.original_max_position > cfg.max_seq_len) break;
    DSK_OK(dsk_forward(model, state, tok, (int)enc.size() - 1, DSK_OUTPUT_LOGITS, nullptr, nullptr));
  }
  double elapsed = now_s() - start;
  std::cout << "\n\nGeneration stats:\n  " << enc.size() << " tokens\n  throughput: " << enc.size() / elapsed << "tok/s\n  latency: " << elapsed / enc.size()
            << "s/tok\n  hydrate: " << end_hydrate - start << "s\n  bandwidth: " << dsk_model_active_bytes_per_token(model) * enc.size() / 1e9 / elapsed
            << "GB/s\n  total: " << elapsed << "s\n" << std::endl;
  std::cout << "generated ids:";
  for (size_t i = 0; i < enc.size(); i++) std::cout << " " << enc[i];
  std::cout << std::endl;
  dsk_state_destroy(state);
  dsk_model_destroy(model);
  return 0;
}
