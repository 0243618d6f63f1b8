// dsk_hybrid_host.cuh — host side of the layer-list ("hybrid") model family inside libdsk: model description, tensor upload by
// name, the per-sequence state (recurrent states, convolution histories, latent ring caches) and the chunk step that
// dsk_forward / dsk_forward_chunk / dsk_decode_greedy drive.  Included at the end of dsk_engine.cu (it uses that file's error,
// allocation and sampling helpers); dsk_model::hy / dsk_state::hy point at the structures below.
//
// Tensor names (safetensors, [out, in] matrices):  embed, side.embed, final.norm, head (untied LM head), loop.step (layer loop),
// and per layer i ("l<i>."):
//   norm1 (and norm1b, norm2, norm2b in sandwich blocks)
//         | mix.in, mix.conv, mix.conv.b, mix.dt_bias, mix.A_log, mix.D, mix.norm, mix.o              (state-space mixer)
//         | mix.q, mix.dkv, mix.dkv.norm, mix.uk, mix.uv, mix.o                                        (latent attention)
//         | mix.q, mix.k, mix.q.norm, mix.k.norm, mix.talk, mix.o                                      (grouped-query attention)
//   mlp.router, mlp.correction, mlp.e<j>.gate|up|down                                                 (routed feed-forward)
//   mlp.up, mlp.up.b, mlp.down, mlp.down.b, mlp.act                                                   (dense feed-forward)
//   side.gate, side.proj, side.norm                                                                   (per-layer token input)
//   shift (token shift), norm1.b / norm2.b / final.norm.b (layer norms with a bias)
//         | mix.q, mix.f, mix.f.b, mix.lower, mix.v, mix.norm, mix.o                                   (gated linear recurrence)
//   mlp.router, mlp.router.b, mlp.e<j>.up|down                                                        (routed feed-forward, top-softmax router)
// Grouped-query attention with its switches on adds mix.v, mix.q.b / k.b / v.b, mix.rel, mix.sink, mix.vmix; latent attention with a
// rotated key part (DSK_MIX_MLA) has mix.dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o; a gated dense feed-forward mlp.gate / up / down;
// DSK_BLOCK_POST layers norm1 / norm2, ls1 / ls2, canon1 / canon2, rg1 / rg2 (+ .b); the model "bigram" beside "embed".
// A parallel block computes, with h = norm1(x):  x += m (mixer(h) + ff(h));  a sandwich block  x += norm1b(mixer(norm1(x))),
// x += norm2b(ff(norm2(x))).  Then, when the model has a per-layer token table,
// g = gelu_tanh(side.gate x) * side.embed[token][i*sd : (i+1)*sd],  y = side.proj g,  x += m * rmsnorm(y) * side.norm.
// A layer loop repeats a range of layers with the same weights; each repetition ("layer run") keeps a separate cache / state.
#pragma once

namespace hyb {
using namespace dsk;
using namespace dsk::hy;

struct HTensor {
  void* p = nullptr;       // model quant type (float | bf16)
  long long rows = 0, cols = 0;
  bool present = false;
};

struct HLayer {
  dsk_layer_spec sp;
  float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr;
  // state-space mixer
  HTensor in, o;
  float *conv_w = nullptr, *conv_b = nullptr, *dt_bias = nullptr, *A_log = nullptr, *D = nullptr, *mnorm = nullptr;
  // latent attention
  HTensor q, dkv, ukT, uk, uv;      // ukT: [heads][kv_rank][dim], the transposed key up-projection (absorbed into the query);
                                    // uk: the same matrix as stored, for portions that up-project the keys instead
  float* dkv_norm = nullptr;
  int owner = -1;                   // layer whose latent cache this layer reads (itself unless kv_from)
  int ring = 0;                     // rows of this layer's own ring cache (owners only)
  // grouped-query attention (with q, o above): key projection, whole-projection norm weights, score mixing, rotation table
  HTensor kproj;
  float *q_norm = nullptr, *k_norm = nullptr, *talk = nullptr, *rot_freq = nullptr;
  float rot_mag = 1.f;
  // grouped-query attention with a value matrix: q, k and v rows (and the output gate's rows, when there is one) stacked into one
  // matrix (one product per step) with their biases; a layer that reads another layer's keys and values stacks [q | gate]
  HTensor qkv;
  float *qkv_b = nullptr, *rel = nullptr, *sink = nullptr;
  int* rel_bucket = nullptr;        // distance (0 .. att_rel_max) -> row of rel
  int rel_rows = 0;
  float vmix = 0.f;                 // value-mixing weight (mix.vmix), read once at upload
  char have_qkv[4] = {0, 0, 0, 0}, have_qkvb[3] = {0, 0, 0}, have_vmix = 0;   // have_qkv[3]: the output gate's rows behind q / k / v
  // latent attention with a rotated key part: the two down-projections stacked [q_rank | kv_rank + rot_dim], query up-projection, output gate
  HTensor in2, uq, gmat;
  float* dq_norm = nullptr;
  char have_in2[2] = {0, 0};
  // DSK_BLOCK_POST: input convolutions, residual gates, closing norm weights (norm weight x layer scale, folded when the model is finalised)
  HTensor rg1, rg2;
  float *rg1_b = nullptr, *rg2_b = nullptr, *canon1 = nullptr, *canon2 = nullptr, *ls1 = nullptr, *ls2 = nullptr, *close1 = nullptr, *close2 = nullptr;
  float norm1_s = 1.f, norm2_s = 1.f;   // single-number norm weights
  char have_n1 = 0, have_n2 = 0;
  // dense feed-forward (gate_d: the gate matrix of a gated one)
  HTensor up, down, gate_d;
  float *up_b = nullptr, *down_b = nullptr, *act = nullptr;
  float act_a = 0.f, act_b = 0.f;
  // routed feed-forward
  HTensor gate_s, up_s, down_s;     // expert stacks [E][ff][width], [E][ff][width], [E][width][ff]
  std::vector<char> have;           // 3 E flags
  float *router = nullptr, *correction = nullptr;
  // per-layer token input
  HTensor sgate, sproj;
  float* snorm = nullptr;
  // token shift weight; biases of the layer norms; bias of a top-softmax router
  float *shift = nullptr, *norm1_bias = nullptr, *norm2_bias = nullptr, *router_b = nullptr;
  // gated linear recurrence: [q | f | v] rows stacked into one matrix, the forget gate's bias at the f rows of a stacked bias
  // (zeros elsewhere), lower bounds, and the output norm's weight (one vector for all heads)
  HTensor lin_in;
  float *lin_bias = nullptr, *lower = nullptr, *lin_norm = nullptr;
  char have_lin[3] = {0, 0, 0}, have_linb = 0;
};

// one execution of a layer: layers inside the loop range run once per pass, each time with a state of their own
struct Run {
  int layer;
  int pass;        // >= 0: this run opens pass `pass` of the loop (loop.step[pass] is added to the residual stream first)
  int owner_run;   // latent attention: the run whose latent cache this run reads (itself unless kv_from)
};

struct Model {
  dsk_hybrid_config c;
  std::vector<HLayer> L;
  std::vector<Run> runs;
  HTensor embed, side_embed, head, bigram;
  float *final_norm = nullptr, *final_norm_b = nullptr, *loop_step = nullptr;
  int vmix_first = -1;              // the first layer whose values later value-mixing layers blend in
  size_t wsize = 4;                 // bytes per matrix element
};

struct LayerState {
  float* ssm = nullptr;             // [heads][vdim][state]
  float* hist = nullptr;            // [conv - 1][channels]
  void* cache = nullptr;            // [ring][kv_rank] (owner layers); grouped-query attention: keys [ring][kv_heads * dim]
  void* vcache = nullptr;           // grouped-query attention: values [ring][kv_heads * vdim]
  float* canon = nullptr;           // DSK_BLOCK_POST: [2][taps - 1][width] rings of the two input convolutions
  float* shift = nullptr;           // token shift: the mixer input of the sequence's last token [width]
  float* lin = nullptr;             // gated linear recurrence: [heads][dim][vdim]
  size_t ssm_bytes = 0, hist_bytes = 0, cache_bytes = 0, vcache_bytes = 0, canon_bytes = 0, shift_bytes = 0, lin_bytes = 0;
};

struct State {
  std::vector<LayerState> L;
  int chunk = 0;
  int next_pos = 0;
  int *d_tok = nullptr, *d_want = nullptr, *d_ctl = nullptr, *d_idx = nullptr, *d_perm = nullptr, *d_ntiles = nullptr;
  int4* d_tiles = nullptr;
  int max_tiles = 0;
  int head_rows = 0;                         // rows of the logits buffer: the LM head runs over the wanted rows in groups of this size
  float* part = nullptr;                     // partial softmax results of key-split attention (decode-sized chunks)
  // prefill attention as matrix products (blocks of kPrefillQ queries): up-projected keys / values, their per-head packing, scores
  float *kf = nullptr, *vf = nullptr, *sc = nullptr, *sc2 = nullptr;   // sc2: scores after the heads were mixed
  void *kb = nullptr, *vt = nullptr;
  int* d_rows = nullptr;
  int prefill_keys = 0;                      // keys a block of queries can see at most; 0: the matrix path is off
  float* y = nullptr;                        // a sublayer's output before its closing norm (sandwich and post blocks)
  float* hs = nullptr;                       // the token-shifted mixer input of the step
  float* vfirst = nullptr;                   // [chunk][kv_heads * vdim] values of the step's tokens in the first value-mixing layer
  int* d_prev = nullptr;                     // the sequence's last token (bigram embedding)
  float *x = nullptr, *h = nullptr, *b0 = nullptr, *b1 = nullptr, *b2 = nullptr, *b3 = nullptr, *wgt = nullptr, *logits = nullptr;
  int *h_tok = nullptr, *h_want = nullptr;   // pinned staging of a chunk's token ids / wanted rows
  std::vector<void*> allocs;
  cudaGraphExec_t step_graph = nullptr;      // captured greedy decode step (arg-max -> token -> one-token chunk)
  // DSK_HY_TIMELINE=1: CUDA events between the groups of launches of every step, summed per label and printed to stderr
  bool timeline = false;
  std::vector<cudaEvent_t> tl_events;
  std::vector<const char*> tl_labels;
  size_t tl_used = 0;
  long long launches = 0;
};

static constexpr int kPrefillQ = 256, kPrefillMin = 32;   // prefill attention: queries per block / smallest portion that takes the matrix path
static constexpr int kAttnSplitMax = 64, kAttnSplitTokens = 4;   // decode-sized chunks split a window over up to 64 CTAs

static bool is_ssd(const dsk_layer_spec& s) { return s.mixer == DSK_MIX_SSD; }
static long long ssd_inner(const dsk_layer_spec& s) { return (long long)s.ssm_heads * s.ssm_vdim; }
static long long ssd_channels(const dsk_layer_spec& s) { return ssd_inner(s) + 2LL * s.ssm_groups * s.ssm_state; }
static long long ssd_proj(const dsk_layer_spec& s) { return ssd_inner(s) + ssd_channels(s) + s.ssm_heads; }

static int validate(const dsk_hybrid_config& c, const dsk_layer_spec* L) {
  if (c.dim <= 0 || c.vocab_size <= 0 || c.n_layers <= 0 || c.max_seq_len <= 0) return fail(-1, "hybrid model: bad dimensions");
  if (c.quant != DSK_F32 && c.quant != DSK_BF16) return fail(-1, "hybrid models run with quant fp32 or bf16");
  if (c.norm_groups <= 0 || c.dim % c.norm_groups != 0) return fail(-1, "norm groups %d do not divide width %d", c.norm_groups, c.dim);
  if (c.chunk < 1 || c.chunk > 4096) return fail(-1, "chunk %d out of range (1..4096)", c.chunk);
  if (c.side_dim < 0) return fail(-1, "negative side_dim");
  if (c.block != DSK_BLOCK_PARALLEL && c.block != DSK_BLOCK_SANDWICH && c.block != DSK_BLOCK_POST) return fail(-1, "unknown block kind %d", c.block);
  if (c.block == DSK_BLOCK_POST && (c.norm_groups != 1 || c.loop_times >= 1))
    return fail(-1, "post-norm blocks run with ungrouped norms and without a layer loop");
  if (c.block == DSK_BLOCK_POST && c.norm_kind == DSK_NORM_LAYER && c.norm_scalar) return fail(-1, "single-number norm weights belong to RMS norms");
  if (c.norm_bias && c.norm_kind != DSK_NORM_LAYER) return fail(-1, "norm biases belong to layer norms");
  if (c.norm_bias && c.block == DSK_BLOCK_SANDWICH) return fail(-1, "sandwich blocks run their layer norms without a bias");
  if (c.block != DSK_BLOCK_POST && (c.canon_taps || c.res_gate || c.layer_scale || c.norm_scalar))
    return fail(-1, "input convolutions, gated residuals, layer scales and single-number norm weights belong to post-norm blocks");
  if (c.canon_taps < 0 || c.canon_taps > kCanonMaxTaps) return fail(-1, "input convolution of %d taps unsupported (at most %d)", c.canon_taps, kCanonMaxTaps);
  if (c.bigram_buckets < 0) return fail(-1, "negative bigram table size");
  if (c.norm_kind != DSK_NORM_RMS && c.norm_kind != DSK_NORM_LAYER) return fail(-1, "unknown norm kind %d", c.norm_kind);
  if (c.loop_times >= 1 && (c.loop_start < 0 || c.loop_stop > c.n_layers || c.loop_start > c.loop_stop))
    return fail(-1, "layer loop %d..%d outside the %d layers", c.loop_start, c.loop_stop, c.n_layers);
  for (int i = 0; i < c.n_layers; i++) {
    const dsk_layer_spec& s = L[i];
    if (s.mixer == DSK_MIX_SSD) {
      if (s.ssm_heads <= 0 || s.ssm_vdim <= 0 || s.ssm_state <= 0 || s.ssm_groups <= 0 || s.ssm_conv < 1 || s.ssm_norm_groups <= 0)
        return fail(-1, "layer %d: bad state-space mixer sizes", i);
      if (s.ssm_heads % s.ssm_groups != 0) return fail(-1, "layer %d: heads %d not a multiple of groups %d", i, s.ssm_heads, s.ssm_groups);
      if ((s.ssm_heads * s.ssm_vdim) % s.ssm_norm_groups != 0) return fail(-1, "layer %d: norm_groups does not divide the inner width", i);
      if (s.ssm_state > 256) return fail(-1, "layer %d: state size %d > 256 unsupported (the scan keeps the state in registers)", i, s.ssm_state);
    } else if (s.mixer == DSK_MIX_LATENT_SWA) {
      if (s.att_heads <= 0 || s.att_dim <= 0 || s.att_vdim <= 0 || s.att_kv_rank <= 0 || s.att_window <= 0)
        return fail(-1, "layer %d: bad latent-attention sizes", i);
      if (s.att_kv_rank > 1024) return fail(-1, "layer %d: kv_rank %d > 1024 unsupported", i, s.att_kv_rank);
      if (s.att_kv_from >= 0) {
        const int j = s.att_kv_from;
        if (j >= i || L[j].mixer != DSK_MIX_LATENT_SWA || L[j].att_kv_from >= 0 || L[j].att_kv_rank != s.att_kv_rank)
          return fail(-1, "layer %d: kv_from %d must name an earlier latent-attention layer that projects its own latent of the same rank", i, j);
      }
    } else if (s.mixer == DSK_MIX_GQA) {
      if (s.att_heads <= 0 || s.att_kv_heads <= 0 || s.att_dim <= 0 || s.att_vdim <= 0 || s.att_window <= 0) return fail(-1, "layer %d: bad attention sizes", i);
      if (s.att_heads % s.att_kv_heads != 0) return fail(-1, "layer %d: heads %d not a multiple of kv_heads %d", i, s.att_heads, s.att_kv_heads);
      if (!s.att_value_proj && s.att_vdim != s.att_dim) return fail(-1, "layer %d: values come out of the key matrix, so vdim %d must equal dim %d", i, s.att_vdim, s.att_dim);
      if (s.att_bias && !s.att_value_proj) return fail(-1, "layer %d: projection biases need the stacked q / k / v projection (att_value_proj)", i);
      if (s.att_talk && (s.att_softcap > 0.f || s.att_rel_max > 0)) return fail(-1, "layer %d: head mixing together with a score cap or distance bias is undefined", i);
      if (s.att_keep_first < 0 || (s.att_keep_first > 0 && s.att_mask != DSK_MASK_WINDOW)) return fail(-1, "layer %d: kept first positions belong to a window mask", i);
      if (s.att_rel_max < 0 || s.att_softcap < 0.f) return fail(-1, "layer %d: negative score cap or distance limit", i);
      if (s.rot_dims < 0 || s.rot_dims > s.att_dim || s.rot_dims % 2 != 0) return fail(-1, "layer %d: rot dims %d must be even and at most dim %d", i, s.rot_dims, s.att_dim);
      if (s.rot_dims > 0 && !(s.rot_base > 0.f)) return fail(-1, "layer %d: bad rotation base", i);
      if ((s.rot_layout != DSK_ROT_PAIRS && s.rot_layout != DSK_ROT_HALF) || (s.rot_scale != DSK_ROTSCALE_YARN && s.rot_scale != DSK_ROTSCALE_BANDS) ||
          (s.att_qk_norm != DSK_QKNORM_WHOLE && s.att_qk_norm != DSK_QKNORM_HEAD))
        return fail(-1, "layer %d: unknown rotation layout, rotation scaling or query / key norm", i);
      if (s.rot_scale == DSK_ROTSCALE_BANDS && s.rot_factor > 0.f && (!(s.rot_fast > s.rot_slow) || s.rot_original <= 0))
        return fail(-1, "layer %d: wavelength-band rotation scaling needs high > low and a positive original length", i);
      if (s.att_out_gate && !s.att_value_proj) return fail(-1, "layer %d: the output gate's rows ride in the stacked q / k / v projection (att_value_proj)", i);
      if (s.att_kv_from >= 0) {
        const int j = s.att_kv_from;
        if (j >= i || L[j].mixer != DSK_MIX_GQA || L[j].att_kv_from >= 0)
          return fail(-1, "layer %d: kv_from %d must name an earlier attention layer that projects its own keys and values", i, j);
        const dsk_layer_spec& o = L[j];
        if (o.att_kv_heads != s.att_kv_heads || o.att_dim != s.att_dim || o.att_vdim != s.att_vdim || o.att_keep_first != s.att_keep_first || !o.att_value_proj ||
            !s.att_value_proj || s.att_vmix || s.att_bias)
          return fail(-1, "layer %d: a layer that reads layer %d's keys and values needs its key heads, sizes and kept positions, a value matrix there, and no biases or value mixing of its own", i, j);
      }
      if (gqa_attn_smem_floats(s.att_heads, s.att_kv_heads, s.att_dim, s.att_vdim) * 4 > 200 * 1024)
        return fail(-1, "layer %d: %d heads x %d with %d key heads do not fit the attention kernel's shared memory", i, s.att_heads, s.att_dim, s.att_kv_heads);
    } else if (s.mixer == DSK_MIX_MLA) {
      if (s.att_heads <= 0 || s.att_dim <= 0 || s.att_rot_dim < 0 || s.att_vdim <= 0 || s.att_kv_rank <= 0 || s.att_q_rank <= 0 || s.att_window <= 0)
        return fail(-1, "layer %d: bad latent-attention sizes", i);
      if (s.att_kv_rank + s.att_rot_dim > 1024) return fail(-1, "layer %d: kv_rank + rot_dim %d > 1024 unsupported", i, s.att_kv_rank + s.att_rot_dim);
      if (s.rot_dims < 0 || s.rot_dims > s.att_rot_dim || s.rot_dims % 2 != 0) return fail(-1, "layer %d: rot dims %d must be even and at most rot_dim %d", i, s.rot_dims, s.att_rot_dim);
      if (s.rot_dims > 0 && !(s.rot_base > 0.f)) return fail(-1, "layer %d: bad rotation base", i);
    } else if (s.mixer == DSK_MIX_HGRN2) {
      if (s.lin_heads <= 0 || s.lin_dim <= 0 || s.lin_vdim <= 0) return fail(-1, "layer %d: bad linear-recurrence sizes", i);
      if (s.lin_dim > 256) return fail(-1, "layer %d: key size %d > 256 unsupported (the recurrence keeps the state in registers)", i, s.lin_dim);
    } else return fail(-1, "layer %d: unknown mixer %d", i, s.mixer);
    if (s.mixer != DSK_MIX_SSD && s.mixer != DSK_MIX_HGRN2 && s.att_mask != DSK_MASK_WINDOW && s.att_mask != DSK_MASK_CHUNK) return fail(-1, "layer %d: unknown mask %d", i, s.att_mask);
    if (s.ff_kind == DSK_FF_DENSE) {
      if (s.ff_hidden <= 0) return fail(-1, "layer %d: bad feed-forward size", i);
      if (s.ff_act != DSK_ACT_XIELU && s.ff_act != DSK_ACT_GEGLU) return fail(-1, "layer %d: unknown activation %d", i, s.ff_act);
    } else if (s.ff_kind == DSK_FF_MOE) {
      if (s.ff_experts <= 0 || s.ff_top <= 0 || s.ff_top > s.ff_experts || s.ff_hidden <= 0) return fail(-1, "layer %d: bad routed feed-forward sizes", i);
      if (s.ff_experts > 4096) return fail(-1, "layer %d: more than 4096 experts unsupported", i);
      if ((s.ff_router != DSK_ROUTER_SIGMOID && s.ff_router != DSK_ROUTER_TOP_SOFTMAX) || (s.ff_expert != DSK_EXPERT_GLU_CLAMPED && s.ff_expert != DSK_EXPERT_RELU2))
        return fail(-1, "layer %d: unknown router or expert kind", i);
    } else if (s.ff_kind != DSK_FF_NONE) return fail(-1, "layer %d: unknown feed-forward kind %d", i, s.ff_kind);
  }
  return 0;
}

static void set_kernel_attrs() {
  static bool done = false;
  if (done) return;
  const int big = 200 * 1024;
  cudaFuncSetAttribute(latent_swa_attn<float, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(latent_swa_attn<float, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(latent_swa_attn<float, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(latent_swa_attn<float, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(ssd_scan<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(ssd_scan<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(ssd_scan<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(ssd_scan<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(ssd_scan<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(ssd_scan<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(gemm_mma<HEPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_GELU_MUL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_XIELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_GEGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_SIGMUL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_RELU2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(gemm_mma<HEPI_LINGATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmem);
  cudaFuncSetAttribute(hgrn2_scan<1, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(hgrn2_scan<2, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(hgrn2_scan<3, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(hgrn2_scan<4, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(hgrn2_scan<6, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(hgrn2_scan<8, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(hgrn2_scan<1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(hgrn2_scan<2, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(hgrn2_scan<3, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(hgrn2_scan<4, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(hgrn2_scan<1, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, big); cudaFuncSetAttribute(hgrn2_scan<2, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(gqa_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  cudaFuncSetAttribute(mix_heads, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
  done = true;
}

static dsk_model* model_create(const dsk_hybrid_config* cfg, const dsk_layer_spec* layers, int rank, int n_ranks) {
  if (need_device()) return nullptr;
  if (!cfg || !layers) { fail(-1, "bad arguments"); return nullptr; }
  if (n_ranks != 1 || rank != 0) { fail(-1, "hybrid models run on one GPU (n_ranks must be 1)"); return nullptr; }
  if (validate(*cfg, layers)) return nullptr;
  set_kernel_attrs();
  dsk_model* m = new dsk_model();
  Model* M = new Model();
  m->hy = M;
  M->c = *cfg;
  M->wsize = cfg->quant == DSK_BF16 ? 2 : 4;
  m->c = dsk_config{};
  m->c.dim = cfg->dim; m->c.vocab_size = cfg->vocab_size; m->c.n_layers = cfg->n_layers; m->c.max_seq_len = cfg->max_seq_len;
  m->c.quant = cfg->quant; m->c.norm_eps = cfg->norm_eps;
  M->L.resize(cfg->n_layers);
  for (int i = 0; i < cfg->n_layers; i++) {
    HLayer& L = M->L[i];
    L.sp = layers[i];
    if (L.sp.ff_kind == DSK_FF_MOE) L.have.assign(3 * (size_t)L.sp.ff_experts, 0);
    if (L.sp.mixer == DSK_MIX_LATENT_SWA) L.owner = L.sp.att_kv_from >= 0 ? L.sp.att_kv_from : i;
    if (L.sp.mixer == DSK_MIX_GQA) L.owner = L.sp.att_kv_from >= 0 ? L.sp.att_kv_from : i;
    if (L.sp.mixer == DSK_MIX_MLA) L.owner = i;
    if (L.sp.mixer == DSK_MIX_GQA && L.sp.att_vmix) {
      if (M->vmix_first < 0) M->vmix_first = i;
      else if ((long long)L.sp.att_kv_heads * L.sp.att_vdim != (long long)M->L[M->vmix_first].sp.att_kv_heads * M->L[M->vmix_first].sp.att_vdim) {
        fail(-1, "layer %d: value mixing needs as many value entries per token as layer %d has", i, M->vmix_first); dsk_model_destroy(m); return nullptr;
      }
    }
  }
  // ring caches: the owner keeps the widest window (or chunk of the mask) among its readers plus one step, capped by the sequence limit
  for (int i = 0; i < cfg->n_layers; i++) {
    const HLayer& L = M->L[i];
    if (L.owner < 0) continue;
    HLayer& O = M->L[L.owner];
    const long long need = (long long)L.sp.att_window - 1 + cfg->chunk;
    O.ring = (int)std::max<long long>(O.ring, std::min<long long>(need, (long long)cfg->max_seq_len));
  }
  // the order of layer runs: layers before the loop, the loop's passes, the layers after it
  const bool looped = cfg->loop_times >= 1 && cfg->loop_stop > cfg->loop_start;   // one pass is a loop too: it has its pass vector
  const int ls = looped ? cfg->loop_start : 0, le = looped ? cfg->loop_stop : 0, lt = looped ? cfg->loop_times : 0;
  for (int i = 0; i < ls; i++) M->runs.push_back(Run{i, -1, -1});
  for (int t = 0; t < lt; t++)
    for (int i = ls; i < le; i++) M->runs.push_back(Run{i, i == ls ? t : -1, -1});
  for (int i = le; i < cfg->n_layers; i++) M->runs.push_back(Run{i, -1, -1});
  for (size_t r = 0; r < M->runs.size(); r++) {   // a reader of another layer's latent cache reads that layer's latest run
    const int o = M->L[M->runs[r].layer].owner;
    if (o < 0) continue;
    for (int q = (int)r; q >= 0; q--)
      if (M->runs[q].layer == o) { M->runs[r].owner_run = q; break; }
    if (M->runs[r].owner_run < 0) { fail(-1, "layer %d reads the latent cache of layer %d, which has not run before it", M->runs[r].layer, o); dsk_model_destroy(m); return nullptr; }
  }
  // rotation tables of the attention layers that rotate: frequency per pair, in double, rounded once to fp32
  for (int i = 0; i < cfg->n_layers; i++) {
    HLayer& L = M->L[i];
    const dsk_layer_spec& s = L.sp;
    if ((s.mixer != DSK_MIX_GQA && s.mixer != DSK_MIX_MLA) || s.rot_dims <= 0) continue;
    const int half = s.rot_dims / 2;
    std::vector<float> f((size_t)half);
    const double base = s.rot_base, dims = s.rot_dims;
    const bool yarn = s.rot_factor > 0.f && (s.mixer != DSK_MIX_GQA || s.rot_scale == DSK_ROTSCALE_YARN);
    const bool bands = s.rot_factor > 0.f && s.mixer == DSK_MIX_GQA && s.rot_scale == DSK_ROTSCALE_BANDS;
    double lo = 0, hi = 0;
    if (yarn) {   // the pair index at which `original` positions hold t turns
      auto at = [&](double t) { return dims * std::log((double)s.rot_original / (2.0 * M_PI * t)) / (2.0 * std::log(base)); };
      lo = std::max(std::floor(at(s.rot_fast)), 0.0);
      hi = std::min(std::ceil(at(s.rot_slow)), dims - 1.0);
      L.rot_mag = (float)(0.1 * std::log((double)s.rot_factor) + 1.0);
    }
    for (int k = 0; k < half; k++) {
      double fr = std::pow(base, -2.0 * k / dims);
      if (yarn) {
        const double ramp = std::min(1.0, std::max(0.0, (k - lo) / std::max(hi - lo, 0.001)));
        fr = fr / s.rot_factor * ramp + fr * (1.0 - ramp);
      }
      if (bands) {   // by wavelength: short ones keep their frequency, long ones are slowed by the factor, a linear blend between
        const double wl = 2.0 * M_PI / fr, orig = s.rot_original;
        if (wl > orig / s.rot_slow) fr = fr / s.rot_factor;
        else if (!(wl < orig / s.rot_fast)) {
          const double sm = (orig / wl - s.rot_slow) / ((double)s.rot_fast - s.rot_slow);
          fr = (1.0 - sm) * fr / s.rot_factor + sm * fr;
        }
      }
      f[k] = (float)fr;
    }
    if (dmalloc(m, (void**)&L.rot_freq, (size_t)half * 4) || cudaMemcpy(L.rot_freq, f.data(), (size_t)half * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
      fail(-2, "rotation table allocation failed"); dsk_model_destroy(m); return nullptr;
    }
  }
  return m;
}

static void model_free(dsk_model* m) { delete m->hy; m->hy = nullptr; }

template <typename ST>
static void launch_convert(const void* src, void* dst, long long rows, long long cols, int tr, bool to_bf16) {
  const long long n = rows * cols;
  const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>((n + 255) / 256, 1 << 16));
  if (to_bf16) convert_kernel<ST, __nv_bfloat16><<<grid, 256>>>((const ST*)src, (__nv_bfloat16*)dst, rows, cols, tr);
  else convert_kernel<ST, float><<<grid, 256>>>((const ST*)src, (float*)dst, rows, cols, tr);
}

// payload (BF16 or F32; host or device) of logical shape rows x cols (cols == 0: a vector) -> dst (fp32 or bf16), optionally
// transposed per head (tr)
static int put(const char* name, int dtype, const int64_t shape[4], const void* data, size_t nbytes, int on_dev, long long rows,
               long long cols, void* dst, bool to_bf16, int tr) {
  if (dtype != DSK_DT_BF16 && dtype != DSK_DT_F32) return fail(-4, "tensor %s: dtype %s unsupported (BF16 or F32)", name, dtype_name(dtype));
  const size_t es = dtype == DSK_DT_BF16 ? 2 : 4;
  const long long n = rows * std::max<long long>(cols, 1);
  if (shape[0] != rows || shape[1] != cols || shape[2] != 0 || nbytes != (size_t)n * es)
    return fail(-4, "tensor mismatch for %s: expected shape=[%lld,%lld], got shape=[%lld,%lld,%lld] (%zu bytes)", name, rows, cols,
                (long long)shape[0], (long long)shape[1], (long long)shape[2], nbytes);
  const void* src = data;
  void* staging = nullptr;
  if (!on_dev) {
    CK(cudaMalloc(&staging, nbytes ? nbytes : 16));
    CK(cudaMemcpy(staging, data, nbytes, cudaMemcpyHostToDevice));
    src = staging;
  }
  if (dtype == DSK_DT_BF16) launch_convert<__nv_bfloat16>(src, dst, rows, std::max<long long>(cols, 1), tr, to_bf16);
  else launch_convert<float>(src, dst, rows, std::max<long long>(cols, 1), tr, to_bf16);
  CK(cudaGetLastError());
  if (staging) { CK(cudaDeviceSynchronize()); CK(cudaFree(staging)); }
  return 0;
}

static int upload(dsk_model* m, const char* name, int dtype, const int64_t shape[4], const void* data, size_t nbytes, int on_dev) {
  Model* M = m->hy;
  const dsk_hybrid_config& c = M->c;
  const bool bf = c.quant == DSK_BF16;
  const std::string nm(name);
  // matrix in the model's quant type
  auto MAT = [&](HTensor& t, long long rows, long long cols, int tr = 0) -> int {
    if (t.present) return fail(-4, "tensor %s uploaded twice", name);
    if (dmalloc(m, &t.p, (size_t)rows * cols * M->wsize + 16)) return -2;
    t.rows = rows; t.cols = cols; t.present = true;
    return put(name, dtype, shape, data, nbytes, on_dev, rows, cols, t.p, bf, tr);
  };
  // fp32 side tensor (norm weights, biases, decays, router)
  auto F32 = [&](float** dst, long long rows, long long cols) -> int {
    if (*dst) return fail(-4, "tensor %s uploaded twice", name);
    if (dmalloc(m, (void**)dst, (size_t)rows * std::max<long long>(cols, 1) * 4)) return -2;
    return put(name, dtype, shape, data, nbytes, on_dev, rows, cols, *dst, false, 0);
  };
  // rows [row0, row0 + rows) of a matrix that stacks several checkpoint tensors (one product instead of several per step)
  auto STACK = [&](HTensor& st, long long total, long long cols, long long row0, long long rows, char* have) -> int {
    if (*have) return fail(-4, "tensor %s uploaded twice", name);
    if (!st.p) {
      if (dmalloc(m, &st.p, (size_t)total * cols * M->wsize + 16)) return -2;
      st.rows = total; st.cols = cols;
    }
    *have = 1;
    return put(name, dtype, shape, data, nbytes, on_dev, rows, cols, (char*)st.p + (size_t)row0 * cols * M->wsize, bf, 0);
  };
  auto STACKV = [&](float** dst, long long total, long long off, long long n, char* have) -> int {   // the same for fp32 vectors
    if (*have) return fail(-4, "tensor %s uploaded twice", name);
    if (!*dst) { if (dmalloc(m, (void**)dst, (size_t)total * 4)) return -2; }
    *have = 1;
    return put(name, dtype, shape, data, nbytes, on_dev, n, 0, *dst + off, false, 0);
  };
  // a single number (shape []) -> host float
  auto SCALAR = [&](float* dst, char* have) -> int {
    if (*have) return fail(-4, "tensor %s uploaded twice", name);
    if (dtype != DSK_DT_BF16 && dtype != DSK_DT_F32) return fail(-4, "tensor %s: dtype %s unsupported (BF16 or F32)", name, dtype_name(dtype));
    const size_t es = dtype == DSK_DT_BF16 ? 2 : 4;
    if (shape[0] > 1 || shape[1] != 0 || nbytes != es) return fail(-4, "tensor mismatch for %s: expected a single number, got shape=[%lld,%lld] (%zu bytes)", name, (long long)shape[0], (long long)shape[1], nbytes);
    unsigned char raw[4] = {0, 0, 0, 0};
    if (on_dev) CK(cudaMemcpy(raw, data, es, cudaMemcpyDeviceToHost)); else memcpy(raw, data, es);
    uint32_t bits;
    if (es == 2) bits = ((uint32_t)raw[0] | ((uint32_t)raw[1] << 8)) << 16; else memcpy(&bits, raw, 4);
    memcpy(dst, &bits, 4);
    *have = 1;
    return 0;
  };
  if (nm == "embed") return MAT(M->embed, c.vocab_size, c.dim);
  if (nm == "bigram" && c.bigram_buckets > 0) return MAT(M->bigram, (long long)c.bigram_buckets + 1, c.dim);
  if (nm == "final.norm" && c.norm_scalar) {   // one number for all coordinates: kept as a constant vector, so every norm kernel takes it
    if (M->final_norm) return fail(-4, "tensor %s uploaded twice", name);
    float g = 0.f; char have = 0;
    if (int rc = SCALAR(&g, &have)) return rc;
    std::vector<float> v((size_t)c.dim, g);
    if (dmalloc(m, (void**)&M->final_norm, (size_t)c.dim * 4)) return -2;
    CK(cudaMemcpy(M->final_norm, v.data(), (size_t)c.dim * 4, cudaMemcpyHostToDevice));
    return 0;
  }
  if (nm == "final.norm") return F32(&M->final_norm, c.dim, 0);
  if (nm == "final.norm.b" && c.norm_bias) return F32(&M->final_norm_b, c.dim, 0);
  if (nm == "head") {
    if (c.tie_head) return fail(-4, "tensor %s: this model's LM head is its embedding table", name);
    return MAT(M->head, c.vocab_size, c.dim);
  }
  if (nm == "loop.step") {
    if (c.loop_times < 1) return fail(-4, "tensor %s: the model has no layer loop", name);
    return F32(&M->loop_step, c.loop_times, c.dim);
  }
  if (nm == "side.embed") {
    if (c.side_dim <= 0) return fail(-4, "tensor %s: the model has no per-layer token input", name);
    return MAT(M->side_embed, c.vocab_size, (long long)c.side_dim * c.n_layers);
  }
  if (nm.size() < 3 || nm[0] != 'l') return fail(-4, "unknown tensor name %s", name);
  char* end = nullptr;
  const long li = strtol(name + 1, &end, 10);
  if (end == name + 1 || *end != '.' || li < 0 || li >= c.n_layers) return fail(-4, "unknown tensor name %s", name);
  HLayer& L = M->L[li];
  const dsk_layer_spec& s = L.sp;
  const std::string rest(end + 1);
  if (rest == "shift" && c.token_shift) return F32(&L.shift, c.dim, 0);
  if (c.norm_bias) {
    if (rest == "norm1.b") return F32(&L.norm1_bias, c.dim, 0);
    if (rest == "norm2.b" && s.ff_kind != DSK_FF_NONE) return F32(&L.norm2_bias, c.dim, 0);
  }
  if (c.block == DSK_BLOCK_POST) {
    const bool ff = s.ff_kind != DSK_FF_NONE;
    if (rest == "norm1") return c.norm_scalar ? SCALAR(&L.norm1_s, &L.have_n1) : F32(&L.norm1, c.dim, 0);
    if (rest == "norm2" && ff) return c.norm_scalar ? SCALAR(&L.norm2_s, &L.have_n2) : F32(&L.norm2, c.dim, 0);
    if (c.layer_scale) {
      if (rest == "ls1") return F32(&L.ls1, c.dim, 0);
      if (rest == "ls2" && ff) return F32(&L.ls2, c.dim, 0);
    }
    if (c.canon_taps > 0) {
      if (rest == "canon1") return F32(&L.canon1, c.dim, c.canon_taps);
      if (rest == "canon2" && ff) return F32(&L.canon2, c.dim, c.canon_taps);
    }
    if (c.res_gate) {
      if (rest == "rg1") return MAT(L.rg1, c.dim, c.dim);
      if (rest == "rg1.b") return F32(&L.rg1_b, c.dim, 0);
      if (rest == "rg2" && ff) return MAT(L.rg2, c.dim, c.dim);
      if (rest == "rg2.b" && ff) return F32(&L.rg2_b, c.dim, 0);
    }
  } else if (rest == "norm1") return F32(&L.norm1, c.dim, 0);
  if (c.block == DSK_BLOCK_SANDWICH) {
    if (rest == "norm1b") return F32(&L.norm1b, c.dim, 0);
    if (rest == "norm2" && s.ff_kind != DSK_FF_NONE) return F32(&L.norm2, c.dim, 0);
    if (rest == "norm2b" && s.ff_kind != DSK_FF_NONE) return F32(&L.norm2b, c.dim, 0);
  }
  if (rest.rfind("mix.", 0) == 0) {
    const std::string k = rest.substr(4);
    if (is_ssd(s)) {
      const long long inner = ssd_inner(s), ch = ssd_channels(s);
      if (k == "in") return MAT(L.in, ssd_proj(s), c.dim);
      if (k == "conv") return F32(&L.conv_w, ch, s.ssm_conv);
      if (k == "conv.b") return F32(&L.conv_b, ch, 0);
      if (k == "dt_bias") return F32(&L.dt_bias, s.ssm_heads, 0);
      if (k == "A_log") return F32(&L.A_log, s.ssm_heads, 0);
      if (k == "D") return F32(&L.D, s.ssm_heads, 0);
      if (k == "norm") return F32(&L.mnorm, inner, 0);
      if (k == "o") return MAT(L.o, c.dim, inner);
    } else if (s.mixer == DSK_MIX_HGRN2) {
      const long long HN = (long long)s.lin_heads * s.lin_dim, HP = (long long)s.lin_heads * s.lin_vdim, tot = 2 * HN + HP;
      if (k == "q") return STACK(L.lin_in, tot, c.dim, 0, HN, &L.have_lin[0]);
      if (k == "f") return STACK(L.lin_in, tot, c.dim, HN, HN, &L.have_lin[1]);
      if (k == "v") return STACK(L.lin_in, tot, c.dim, 2 * HN, HP, &L.have_lin[2]);
      if (k == "f.b") {   // the bias of the stacked product: zeros at the q and v rows
        if (!L.lin_bias) { if (dmalloc(m, (void**)&L.lin_bias, (size_t)tot * 4)) return -2; CK(cudaMemset(L.lin_bias, 0, (size_t)tot * 4)); }
        return STACKV(&L.lin_bias, tot, HN, HN, &L.have_linb);
      }
      if (k == "lower") return F32(&L.lower, HN, 0);
      if (k == "o") return MAT(L.o, c.dim, HP);
      if (k == "norm") return F32(&L.lin_norm, s.lin_vdim, 0);   // one weight vector for all heads
    } else if (s.mixer == DSK_MIX_MLA) {
      const long long H = s.att_heads, DK = s.att_dim + s.att_rot_dim, R = s.att_kv_rank, Q = s.att_q_rank, tot = Q + R + s.att_rot_dim;
      if (k == "dq") return STACK(L.in2, tot, c.dim, 0, Q, &L.have_in2[0]);
      if (k == "dkv") return STACK(L.in2, tot, c.dim, Q, R + s.att_rot_dim, &L.have_in2[1]);
      if (k == "dq.norm") return F32(&L.dq_norm, Q, 0);
      if (k == "dkv.norm") return F32(&L.dkv_norm, R, 0);
      if (k == "uq") return MAT(L.uq, H * DK, Q);
      if (k == "uk") { if (int rc = MAT(L.ukT, H * s.att_dim, R, s.att_dim)) return rc; return MAT(L.uk, H * s.att_dim, R); }
      if (k == "uv") return MAT(L.uv, H * s.att_vdim, R);
      if (k == "g" && s.att_out_gate) return MAT(L.gmat, H * s.att_vdim, c.dim);
      if (k == "o") return MAT(L.o, c.dim, H * s.att_vdim);
    } else if (s.mixer == DSK_MIX_GQA) {
      const long long HD = (long long)s.att_heads * s.att_dim, GD = (long long)s.att_kv_heads * s.att_dim, GV = (long long)s.att_kv_heads * s.att_vdim;
      const long long HV = s.att_out_gate ? (long long)s.att_heads * s.att_vdim : 0;
      if (s.att_kv_from >= 0) {   // reads another layer's keys and values: only the query projection (and gate) of its own
        if (k == "q") return STACK(L.qkv, HD + HV, c.dim, 0, HD, &L.have_qkv[0]);
        if (k == "g" && s.att_out_gate) return STACK(L.qkv, HD + HV, c.dim, HD, HV, &L.have_qkv[3]);
      } else if (s.att_value_proj) {
        const long long tot = HD + GD + GV + HV;
        if (k == "g" && s.att_out_gate) return STACK(L.qkv, tot, c.dim, HD + GD + GV, HV, &L.have_qkv[3]);
        if (k == "q") return STACK(L.qkv, tot, c.dim, 0, HD, &L.have_qkv[0]);
        if (k == "k") return STACK(L.qkv, tot, c.dim, HD, GD, &L.have_qkv[1]);
        if (k == "v") return STACK(L.qkv, tot, c.dim, HD + GD, GV, &L.have_qkv[2]);
        if (s.att_bias) {
          if (!L.qkv_b && HV > 0) { if (dmalloc(m, (void**)&L.qkv_b, (size_t)tot * 4)) return -2; CK(cudaMemset(L.qkv_b, 0, (size_t)tot * 4)); }   // no bias on the gate's rows
          if (k == "q.b") return STACKV(&L.qkv_b, tot, 0, HD, &L.have_qkvb[0]);
          if (k == "k.b") return STACKV(&L.qkv_b, tot, HD, GD, &L.have_qkvb[1]);
          if (k == "v.b") return STACKV(&L.qkv_b, tot, HD + GD, GV, &L.have_qkvb[2]);
        }
      }
      if (k == "rel" && s.att_rel_max > 0) {   // the number of distance buckets is the tensor's first size
        if (shape[0] < 2 || shape[0] > (1 << 20)) return fail(-4, "tensor %s: %lld distance buckets", name, (long long)shape[0]);
        L.rel_rows = (int)shape[0];
        return F32(&L.rel, shape[0], s.att_heads);
      }
      if (k == "sink" && s.att_sink) return F32(&L.sink, s.att_heads, 0);
      if (k == "vmix" && s.att_vmix) return SCALAR(&L.vmix, &L.have_vmix);
      if (k == "vmix" || (k == "rel" && s.att_rel_max <= 0)) return 0;   // a checkpoint may carry them for layers that do not use them
      if (k == "q" && !s.att_value_proj) return MAT(L.q, HD, c.dim);
      if (k == "k" && !s.att_value_proj) return MAT(L.kproj, GD, c.dim);
      if (k == "q.norm" && s.att_qk_norm == DSK_QKNORM_WHOLE) return F32(&L.q_norm, HD, 0);
      if (k == "k.norm" && s.att_qk_norm == DSK_QKNORM_WHOLE) return F32(&L.k_norm, GD, 0);
      if (k == "talk" && s.att_talk) return F32(&L.talk, s.att_heads, s.att_heads);
      if (k == "o") return MAT(L.o, c.dim, (long long)s.att_heads * s.att_vdim);
    } else {
      const long long H = s.att_heads;
      if (k == "q") return MAT(L.q, H * s.att_dim, c.dim);
      if (k == "uk") { if (int rc = MAT(L.ukT, H * s.att_dim, s.att_kv_rank, s.att_dim)) return rc; return MAT(L.uk, H * s.att_dim, s.att_kv_rank); }
      if (k == "uv") return MAT(L.uv, H * s.att_vdim, s.att_kv_rank);
      if (k == "o") return MAT(L.o, c.dim, H * s.att_vdim);
      if (s.att_kv_from < 0) {
        if (k == "dkv") return MAT(L.dkv, s.att_kv_rank, c.dim);
        if (k == "dkv.norm") return F32(&L.dkv_norm, s.att_kv_rank, 0);
      }
    }
    return fail(-4, "unknown tensor name %s for this layer's mixer", name);
  }
  if (rest.rfind("mlp.", 0) == 0 && s.ff_kind == DSK_FF_DENSE && s.ff_act == DSK_ACT_GEGLU) {
    const std::string k = rest.substr(4);
    if (k == "gate") return MAT(L.gate_d, s.ff_hidden, c.dim);
    if (k == "up") return MAT(L.up, s.ff_hidden, c.dim);
    if (k == "down") return MAT(L.down, c.dim, s.ff_hidden);
    return fail(-4, "unknown tensor name %s", name);
  }
  if (rest.rfind("mlp.", 0) == 0 && s.ff_kind == DSK_FF_DENSE) {
    const std::string k = rest.substr(4);
    if (k == "up") return MAT(L.up, s.ff_hidden, c.dim);
    if (k == "up.b") return F32(&L.up_b, s.ff_hidden, 0);
    if (k == "down") return MAT(L.down, c.dim, s.ff_hidden);
    if (k == "down.b") return F32(&L.down_b, c.dim, 0);
    if (k == "act") {   // the activation's two numbers enter as softplus(p) and 1/2 + softplus(q), in fp32
      if (int rc = F32(&L.act, 2, 0)) return rc;
      float pq[2];
      CK(cudaMemcpy(pq, L.act, sizeof(pq), cudaMemcpyDeviceToHost));
      auto softplus = [](float v) { return v > 20.f ? v : log1pf(expf(v)); };
      L.act_a = softplus(pq[0]);
      L.act_b = 0.5f + softplus(pq[1]);
      return 0;
    }
    return fail(-4, "unknown tensor name %s", name);
  }
  if (rest.rfind("mlp.", 0) == 0 && s.ff_kind == DSK_FF_MOE) {
    const std::string k = rest.substr(4);
    const long long E = s.ff_experts, ff = s.ff_hidden;
    if (k == "router") return F32(&L.router, E, c.dim);
    if (k == "correction" && s.ff_router == DSK_ROUTER_SIGMOID) return F32(&L.correction, E, 0);
    if (k == "router.b" && s.ff_router == DSK_ROUTER_TOP_SOFTMAX) return F32(&L.router_b, E, 0);
    if (k.size() > 1 && k[0] == 'e') {
      char* e2 = nullptr;
      const long e = strtol(k.c_str() + 1, &e2, 10);
      if (e2 != k.c_str() + 1 && *e2 == '.' && e >= 0 && e < E) {
        const std::string part(e2 + 1);
        const int which = part == "gate" ? 0 : part == "up" ? 1 : part == "down" ? 2 : -1;
        if (which >= (s.ff_expert == DSK_EXPERT_RELU2 ? 1 : 0)) {
          HTensor& st = which == 0 ? L.gate_s : which == 1 ? L.up_s : L.down_s;
          if (!st.p) {
            if (dmalloc(m, &st.p, (size_t)E * ff * c.dim * M->wsize + 16)) return -2;
            st.rows = which == 2 ? c.dim : ff; st.cols = which == 2 ? ff : c.dim;
          }
          if (L.have[(size_t)which * E + e]) return fail(-4, "tensor %s uploaded twice", name);
          L.have[(size_t)which * E + e] = 1;
          return put(name, dtype, shape, data, nbytes, on_dev, st.rows, st.cols, (char*)st.p + (size_t)e * ff * c.dim * M->wsize, bf, 0);
        }
      }
    }
    return fail(-4, "unknown tensor name %s", name);
  }
  if (rest.rfind("side.", 0) == 0 && c.side_dim > 0) {
    const std::string k = rest.substr(5);
    if (k == "gate") return MAT(L.sgate, c.side_dim, c.dim);
    if (k == "proj") return MAT(L.sproj, c.dim, c.side_dim);
    if (k == "norm") return F32(&L.snorm, c.dim, 0);
  }
  return fail(-4, "unknown tensor name %s", name);
}

static int finalize(dsk_model* m) {
  Model* M = m->hy;
  const dsk_hybrid_config& c = M->c;
  if (!M->embed.present) return fail(-5, "missing tensor embed");
  if (!M->final_norm) return fail(-5, "missing tensor final.norm");
  if (c.norm_bias && !M->final_norm_b) return fail(-5, "missing tensor final.norm.b");
  if (c.side_dim > 0 && !M->side_embed.present) return fail(-5, "missing tensor side.embed");
  if (!c.tie_head && !M->head.present) return fail(-5, "missing tensor head");
  if (c.bigram_buckets > 0 && !M->bigram.present) return fail(-5, "missing tensor bigram");
  // closing norm weight of a post-norm sublayer: (norm weight, a vector or one number) x (layer scale), folded once in fp32
  auto fold = [&](const float* normv, float norm_s, const float* ls, float** out) -> int {
    std::vector<float> a((size_t)c.dim, norm_s), b((size_t)c.dim, 1.f);
    if (normv) CK(cudaMemcpy(a.data(), normv, (size_t)c.dim * 4, cudaMemcpyDeviceToHost));
    if (ls) CK(cudaMemcpy(b.data(), ls, (size_t)c.dim * 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < c.dim; i++) a[i] *= b[i];
    if (!*out && dmalloc(m, (void**)out, (size_t)c.dim * 4)) return -2;
    CK(cudaMemcpy(*out, a.data(), (size_t)c.dim * 4, cudaMemcpyHostToDevice));
    return 0;
  };
  CK(cudaDeviceSynchronize());
  if (c.loop_times >= 1 && c.loop_stop > c.loop_start && !M->loop_step) return fail(-5, "missing tensor loop.step");
  for (int i = 0; i < c.n_layers; i++) {
    HLayer& L = M->L[i];
    const dsk_layer_spec& s = L.sp;
    if (c.block == DSK_BLOCK_POST) {
      const bool ff = s.ff_kind != DSK_FF_NONE;
      if (c.norm_scalar ? (!L.have_n1 || (ff && !L.have_n2)) : (!L.norm1 || (ff && !L.norm2))) return fail(-5, "layer %d: missing norm tensors (norm1, norm2)", i);
      if (c.layer_scale && (!L.ls1 || (ff && !L.ls2))) return fail(-5, "layer %d: missing layer scale tensors (ls1, ls2)", i);
      if (c.canon_taps > 0 && (!L.canon1 || (ff && !L.canon2))) return fail(-5, "layer %d: missing input convolution tensors (canon1, canon2)", i);
      if (c.res_gate && (!L.rg1.present || !L.rg1_b || (ff && (!L.rg2.present || !L.rg2_b)))) return fail(-5, "layer %d: missing residual gate tensors (rg1, rg1.b, rg2, rg2.b)", i);
      if (fold(L.norm1, L.norm1_s, L.ls1, &L.close1) || (ff && fold(L.norm2, L.norm2_s, L.ls2, &L.close2))) return -2;
    } else if (!L.norm1) return fail(-5, "missing tensor l%d.norm1", i);
    if (c.token_shift && !L.shift) return fail(-5, "missing tensor l%d.shift", i);
    if (c.norm_bias && (!L.norm1_bias || (s.ff_kind != DSK_FF_NONE && !L.norm2_bias))) return fail(-5, "layer %d: missing norm biases (norm1.b, norm2.b)", i);
    if (c.block == DSK_BLOCK_SANDWICH && (!L.norm1b || (s.ff_kind != DSK_FF_NONE && (!L.norm2 || !L.norm2b))))
      return fail(-5, "layer %d: missing norm tensors (norm1b, norm2, norm2b)", i);
    if (s.mixer == DSK_MIX_HGRN2) {
      L.lin_in.present = L.have_lin[0] && L.have_lin[1] && L.have_lin[2];
      if (!L.lin_in.present || !L.have_linb || !L.lower || !L.lin_norm || !L.o.present)
        return fail(-5, "layer %d: missing linear-recurrence tensors (mix.q, f, f.b, lower, v, norm, o)", i);
    } else if (s.mixer == DSK_MIX_GQA) {
      if (s.att_out_gate && !L.have_qkv[3]) return fail(-5, "layer %d: missing tensor mix.g", i);
      if (s.att_kv_from >= 0) {
        L.qkv.present = L.have_qkv[0];
        if (!L.qkv.present) return fail(-5, "layer %d: missing tensor mix.q", i);
      } else if (s.att_value_proj) {
        L.qkv.present = L.have_qkv[0] && L.have_qkv[1] && L.have_qkv[2];
        if (!L.qkv.present || (s.att_bias && !(L.have_qkvb[0] && L.have_qkvb[1] && L.have_qkvb[2]))) return fail(-5, "layer %d: missing attention projections (mix.q, k, v and their biases)", i);
      } else if (!L.q.present || !L.kproj.present) return fail(-5, "layer %d: missing attention tensors (mix.q, k)", i);
      if (!L.o.present || (s.att_qk_norm == DSK_QKNORM_WHOLE && (!L.q_norm || !L.k_norm)) || (s.att_talk && !L.talk))
        return fail(-5, "layer %d: missing attention tensors (mix.q.norm, k.norm, talk, o)", i);
      if ((s.att_sink && !L.sink) || (s.att_rel_max > 0 && !L.rel) || (s.att_vmix && !L.have_vmix && i != M->vmix_first))
        return fail(-5, "layer %d: missing attention tensors (mix.sink, rel, vmix)", i);
      if (s.att_rel_max > 0) {   // distance -> bucket, in double: below half the buckets one distance each, then logarithmic steps up to att_rel_max
        const int B = L.rel_rows, half = B / 2, D = s.att_rel_max;
        if (D <= half) return fail(-5, "layer %d: distance limit %d must exceed half of the %d distance buckets", i, D, B);
        std::vector<int> bk((size_t)D + 1);
        for (int n = 0; n <= D; n++)
          bk[n] = n < half ? n : std::min(B - 1, half + (int)std::floor(std::log((double)n / half) / std::log((double)D / half) * (B - half)));
        if (!L.rel_bucket && dmalloc(m, (void**)&L.rel_bucket, bk.size() * 4)) return -2;
        CK(cudaMemcpy(L.rel_bucket, bk.data(), bk.size() * 4, cudaMemcpyHostToDevice));
      }
    } else if (s.mixer == DSK_MIX_MLA) {
      L.in2.present = L.have_in2[0] && L.have_in2[1];
      if (!L.in2.present || !L.dq_norm || !L.dkv_norm || !L.uq.present || !L.ukT.present || !L.uk.present || !L.uv.present || !L.o.present || (s.att_out_gate && !L.gmat.present))
        return fail(-5, "layer %d: missing latent-attention tensors (mix.dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o)", i);
    } else if (is_ssd(s)) {
      if (!L.in.present || !L.o.present || !L.conv_w || !L.conv_b || !L.dt_bias || !L.A_log || !L.D || !L.mnorm)
        return fail(-5, "layer %d: missing state-space mixer tensors (mix.in, conv, conv.b, dt_bias, A_log, D, norm, o)", i);
    } else {
      if (!L.q.present || !L.ukT.present || !L.uk.present || !L.uv.present || !L.o.present) return fail(-5, "layer %d: missing latent-attention tensors (mix.q, uk, uv, o)", i);
      if (s.att_kv_from < 0 && (!L.dkv.present || !L.dkv_norm)) return fail(-5, "layer %d: missing mix.dkv / mix.dkv.norm", i);
    }
    if (s.ff_kind == DSK_FF_DENSE && s.ff_act == DSK_ACT_GEGLU) {
      if (!L.gate_d.present || !L.up.present || !L.down.present) return fail(-5, "layer %d: missing feed-forward tensors (mlp.gate, up, down)", i);
    } else if (s.ff_kind == DSK_FF_DENSE && (!L.up.present || !L.down.present || !L.up_b || !L.down_b || !L.act))
      return fail(-5, "layer %d: missing feed-forward tensors (mlp.up, up.b, down, down.b, act)", i);
    if (s.ff_kind == DSK_FF_MOE) {
      if (!L.router || (s.ff_router == DSK_ROUTER_SIGMOID ? !L.correction : !L.router_b)) return fail(-5, "layer %d: missing mlp.router / mlp.correction / mlp.router.b", i);
      for (size_t k = s.ff_expert == DSK_EXPERT_RELU2 ? (size_t)s.ff_experts : 0; k < L.have.size(); k++)
        if (!L.have[k]) return fail(-5, "layer %d: missing expert tensor mlp.e%zu.%s", i, k % s.ff_experts, k / s.ff_experts == 0 ? "gate" : k / s.ff_experts == 1 ? "up" : "down");
    }
    if (c.side_dim > 0 && (!L.sgate.present || !L.sproj.present || !L.snorm)) return fail(-5, "layer %d: missing side.gate / side.proj / side.norm", i);
  }
  CK(cudaDeviceSynchronize());
  return 0;
}

// algorithmic weight bytes one decoded token streams
static double active_bytes(const dsk_model* m) {
  const Model* M = m->hy;
  const dsk_hybrid_config& c = M->c;
  const double ws = (double)M->wsize, W = c.dim;
  double tot = W * ws * (c.bigram_buckets > 0 ? 2 : 1) + (double)c.vocab_size * W * ws + W * 4;
  for (const Run& R : M->runs) {
    const HLayer& L = M->L[R.layer];
    const dsk_layer_spec& s = L.sp;
    double mat = 0, f32 = W;
    if (R.pass >= 0) f32 += W;
    if (c.block == DSK_BLOCK_SANDWICH) f32 += W * (s.ff_kind != DSK_FF_NONE ? 3 : 1);
    if (c.block == DSK_BLOCK_POST) {   // per sublayer: convolution taps, gate matrix and bias (the closing weight is the W counted above)
      const double subs = s.ff_kind != DSK_FF_NONE ? 2 : 1;
      f32 += subs * (W * c.canon_taps + (c.res_gate ? W : 0)) + (subs - 1) * W;
      if (c.res_gate) mat += subs * W * W;
    }
    if (c.token_shift) f32 += W;
    if (c.norm_bias) f32 += W * (s.ff_kind != DSK_FF_NONE ? 2 : 1);
    if (s.mixer == DSK_MIX_HGRN2) {
      const double HN = (double)s.lin_heads * s.lin_dim, HP = (double)s.lin_heads * s.lin_vdim;
      mat += (2 * HN + HP) * W + W * HP;
      f32 += 3 * HN + 2 * HP;
    } else if (s.mixer == DSK_MIX_GQA) {
      const bool reads = s.att_kv_from >= 0;
      const double HD = (double)s.att_heads * s.att_dim, GD = reads ? 0.0 : (double)s.att_kv_heads * s.att_dim, GV = s.att_value_proj && !reads ? (double)s.att_kv_heads * s.att_vdim : 0.0;
      mat += (HD + GD + GV) * W + W * s.att_heads * s.att_vdim * (s.att_out_gate ? 2 : 1);
      f32 += (s.att_qk_norm == DSK_QKNORM_WHOLE ? HD + GD : 0.0) + (s.att_talk ? (double)s.att_heads * s.att_heads : 0.0) + (s.att_bias ? HD + GD + GV : 0.0) + (s.att_sink ? s.att_heads : 0);
    } else if (s.mixer == DSK_MIX_MLA) {
      const double H = s.att_heads, DK = s.att_dim + s.att_rot_dim, Rr = s.att_kv_rank, Q = s.att_q_rank;
      mat += (Q + Rr + s.att_rot_dim) * W + H * DK * Q + H * (s.att_dim + s.att_vdim) * Rr + (s.att_out_gate ? H * s.att_vdim * W : 0.0) + W * H * s.att_vdim;
      f32 += Q + Rr;
    } else if (is_ssd(s)) { mat += (double)ssd_proj(s) * W + W * ssd_inner(s); f32 += (double)ssd_channels(s) * (s.ssm_conv + 1) + 3.0 * s.ssm_heads + ssd_inner(s); }
    else {
      mat += (double)s.att_heads * s.att_dim * W + (double)s.att_heads * (s.att_dim + s.att_vdim) * s.att_kv_rank + W * s.att_heads * s.att_vdim;
      if (s.att_kv_from < 0) { mat += (double)s.att_kv_rank * W; f32 += s.att_kv_rank; }
    }
    if (s.ff_kind == DSK_FF_MOE) { mat += (s.ff_expert == DSK_EXPERT_RELU2 ? 2.0 : 3.0) * s.ff_top * s.ff_hidden * W; f32 += (double)s.ff_experts * (W + 1); }
    if (s.ff_kind == DSK_FF_DENSE && s.ff_act == DSK_ACT_GEGLU) mat += 3.0 * s.ff_hidden * W;
    else if (s.ff_kind == DSK_FF_DENSE) { mat += 2.0 * s.ff_hidden * W; f32 += s.ff_hidden + W; }
    if (c.side_dim > 0) { mat += 2.0 * c.side_dim * W + c.side_dim; f32 += W; }
    tot += mat * ws + f32 * 4;
  }
  return tot;
}

// kernels one decoded token launches (embedding + layers + final norm + LM head + arg-max)
static bool fused_norms(const dsk_hybrid_config& c);
static int launches_per_token(const dsk_model* m) {
  const Model* M = m->hy;
  int n = fused_norms(M->c) ? 3 : 4;
  if (M->c.bigram_buckets > 0) n += 1;
  const bool sandwich = M->c.block == DSK_BLOCK_SANDWICH, post = M->c.block == DSK_BLOCK_POST;
  for (const Run& R : M->runs) {
    const HLayer& L = M->L[R.layer];
    const dsk_layer_spec& s = L.sp;
    if (M->c.token_shift && (&R == &M->runs[0] || !(post && M->c.side_dim > 0 && M->c.canon_taps <= 0))) n += 1;   // later runs: shifted by the previous run's last kernel
    if (post && M->c.canon_taps <= 0) n += (s.ff_kind != DSK_FF_NONE ? 2 : 1) * (1 + (M->c.res_gate ? 1 : 0));   // gate, closing norm
    else if (post) n += (s.ff_kind != DSK_FF_NONE ? 2 : 1) * (1 + (M->c.res_gate ? 1 : 0)) + (&R == &M->runs[0] && M->c.canon_taps > 0 ? 1 : 0);   // gate, closing norm + next convolution in one
    else if (fused_norms(M->c)) n += 1 + (s.ff_kind != DSK_FF_NONE ? 1 : 0) + (&R == &M->runs[0] ? 1 + (R.pass >= 0 ? 1 : 0) : 0);
    else n += 1 + (R.pass >= 0 ? 1 : 0) + (sandwich ? 1 + (s.ff_kind != DSK_FF_NONE ? 2 : 0) : 0);
    if (s.mixer == DSK_MIX_HGRN2) n += 4;   // stacked projection, recurrence, head norm, o
    else if (s.mixer == DSK_MIX_GQA) n += s.att_value_proj ? 5 : 6;   // q, k (or one stacked q / k / v (/ gate) product), norm + rotation, attention, merge, o
    else if (s.mixer == DSK_MIX_MLA) n += 10 + (s.att_out_gate ? 1 : 0);   // down-projections, query norm, query up, latent preparation, absorbed query, attention, merge, value up, (gate,) o
    else if (s.mixer != DSK_MIX_MLA && s.mixer != DSK_MIX_HGRN2 && s.mixer != DSK_MIX_GQA) n += is_ssd(s) ? 5 + (s.ssm_conv > 1 ? 1 : 0) : 5 + (s.att_kv_from < 0 ? 2 : 0);
    if (s.ff_kind == DSK_FF_MOE) n += post && M->c.norm_kind == DSK_NORM_LAYER && !M->c.res_gate && M->c.dim <= 256 * kLnRegs ? 4 : 5;
    if (s.ff_kind == DSK_FF_DENSE) n += 2;
    if (M->c.side_dim > 0) n += 3;
  }
  return n;
}

// ---------------------------------------------------------------------------------------------------------------------
// state
// ---------------------------------------------------------------------------------------------------------------------
static int salloc(State* S, void** p, size_t bytes) {
  CK(cudaMalloc(p, bytes ? bytes : 16));
  CK(cudaMemset(*p, 0, bytes ? bytes : 16));
  S->allocs.push_back(*p);
  return 0;
}

static int state_reset(dsk_state* s) {
  State* S = s->hy;
  for (LayerState& l : S->L) {
    if (l.ssm) CK(cudaMemsetAsync(l.ssm, 0, l.ssm_bytes, s->stream));
    if (l.hist) CK(cudaMemsetAsync(l.hist, 0, l.hist_bytes, s->stream));
    if (l.cache) CK(cudaMemsetAsync(l.cache, 0, l.cache_bytes, s->stream));
    if (l.vcache) CK(cudaMemsetAsync(l.vcache, 0, l.vcache_bytes, s->stream));
    if (l.canon) CK(cudaMemsetAsync(l.canon, 0, l.canon_bytes, s->stream));
    if (l.shift) CK(cudaMemsetAsync(l.shift, 0, l.shift_bytes, s->stream));
    if (l.lin) CK(cudaMemsetAsync(l.lin, 0, l.lin_bytes, s->stream));
  }
  S->next_pos = 0;
  s->last_pos = -1;
  s->have_logits = false;
  return 0;
}

static dsk_state* state_create(dsk_model* m) {
  Model* M = m->hy;
  const dsk_hybrid_config& c = M->c;
  dsk_state* s = new dsk_state();
  State* S = new State();
  s->m = m;
  s->hy = S;
  S->chunk = c.chunk;
  S->timeline = getenv("DSK_HY_TIMELINE") != nullptr;
  const size_t Tc = c.chunk;
  // the pieces the shared sampling / arg-max code reads
  cudaMalloc((void**)&s->ctrl, sizeof(Ctrl)); cudaMemset(s->ctrl, 0, sizeof(Ctrl));
  cudaMallocHost((void**)&s->h_ctrl, sizeof(Ctrl)); memset(s->h_ctrl, 0, sizeof(Ctrl));
  s->token_log_cap = 1 << 16;
  cudaMalloc((void**)&s->token_log, s->token_log_cap * sizeof(int));
  cudaMalloc((void**)&s->step, sizeof(int));
  cudaMalloc((void**)&s->sample_out, 4 * sizeof(float)); cudaMemset(s->sample_out, 0, 4 * sizeof(float));
  cudaMalloc((void**)&s->logits, (size_t)c.vocab_size * 4); cudaMemset(s->logits, 0, (size_t)c.vocab_size * 4);
  s->logits_src = s->logits;
  cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking);
  cudaEventCreate(&s->ev0); cudaEventCreate(&s->ev1);
  if (cudaGetLastError() != cudaSuccess) { fail(-2, "state allocation failed"); return nullptr; }
  size_t mx0 = c.dim, mx1 = c.dim, mx2 = c.dim, mx3 = c.dim, mxE = 1, mxTop = 1;
  S->L.resize(M->runs.size());   // one state per layer run
  bool any_talk = false;
  size_t mxGV = 0;
  for (size_t r = 0; r < M->runs.size(); r++) {
    const int i = M->runs[r].layer;
    const HLayer& L = M->L[i];
    const dsk_layer_spec& sp = L.sp;
    LayerState& ls = S->L[r];
    if (c.block == DSK_BLOCK_POST && c.canon_taps > 1) {
      ls.canon_bytes = (size_t)2 * (c.canon_taps - 1) * c.dim * 4;
      if (salloc(S, (void**)&ls.canon, ls.canon_bytes)) return nullptr;
    }
    if (c.token_shift) {
      ls.shift_bytes = (size_t)c.dim * 4;
      if (salloc(S, (void**)&ls.shift, ls.shift_bytes)) return nullptr;
    }
    if (sp.mixer == DSK_MIX_HGRN2) {
      const size_t HN = (size_t)sp.lin_heads * sp.lin_dim, HP = (size_t)sp.lin_heads * sp.lin_vdim;
      ls.lin_bytes = HN * sp.lin_vdim * 4;
      if (salloc(S, (void**)&ls.lin, ls.lin_bytes)) return nullptr;
      mx0 = std::max<size_t>(mx0, 2 * HN + HP); mx2 = std::max<size_t>(mx2, HP); mx3 = std::max<size_t>(mx3, HP);
    } else if (sp.mixer == DSK_MIX_GQA) {
      const size_t HD = (size_t)sp.att_heads * sp.att_dim, GD = (size_t)sp.att_kv_heads * sp.att_dim, GV = (size_t)sp.att_kv_heads * sp.att_vdim;
      if (M->runs[r].owner_run == (int)r) {   // a layer that reads another layer's keys and values caches nothing
        const size_t rows = (size_t)sp.att_keep_first + L.ring;   // the kept first positions have rows of their own in front of the ring
        ls.cache_bytes = rows * GD * 4;
        ls.vcache_bytes = rows * GV * 4;
        if (salloc(S, &ls.cache, ls.cache_bytes) || salloc(S, &ls.vcache, ls.vcache_bytes)) return nullptr;
      }
      mx0 = std::max<size_t>(mx0, (sp.att_value_proj ? HD + GD + GV : HD) + (sp.att_out_gate ? (size_t)sp.att_heads * sp.att_vdim : 0)); mx1 = std::max<size_t>(mx1, GD); mx2 = std::max<size_t>(mx2, HD);
      mx3 = std::max<size_t>(mx3, (size_t)sp.att_heads * sp.att_vdim);
      any_talk |= sp.att_talk != 0;
      if (sp.att_vmix) mxGV = std::max(mxGV, GV);
    } else if (sp.mixer == DSK_MIX_MLA) {
      const size_t H = sp.att_heads, RW = (size_t)sp.att_kv_rank + sp.att_rot_dim;
      ls.cache_bytes = (size_t)L.ring * RW * 4;
      if (salloc(S, &ls.cache, ls.cache_bytes)) return nullptr;
      mx0 = std::max<size_t>(mx0, std::max(H * (sp.att_dim + sp.att_rot_dim), H * sp.att_vdim));
      mx1 = std::max<size_t>(mx1, sp.att_q_rank + RW);
      mx2 = std::max<size_t>(mx2, std::max<size_t>(sp.att_q_rank, H * RW));
      mx3 = std::max<size_t>(mx3, std::max(H * RW, H * sp.att_vdim));
    } else if (is_ssd(sp)) {
      ls.ssm_bytes = (size_t)sp.ssm_heads * sp.ssm_vdim * sp.ssm_state * 4;
      ls.hist_bytes = (size_t)std::max(1, sp.ssm_conv - 1) * ssd_channels(sp) * 4;
      if (salloc(S, (void**)&ls.ssm, ls.ssm_bytes) || salloc(S, (void**)&ls.hist, ls.hist_bytes)) return nullptr;
      mx0 = std::max<size_t>(mx0, ssd_proj(sp)); mx1 = std::max<size_t>(mx1, ssd_channels(sp));
      mx2 = std::max<size_t>(mx2, ssd_inner(sp)); mx3 = std::max<size_t>(mx3, ssd_inner(sp));
    } else {
      if (M->runs[r].owner_run == (int)r) {
        ls.cache_bytes = (size_t)L.ring * sp.att_kv_rank * 4;
        if (salloc(S, &ls.cache, ls.cache_bytes)) return nullptr;
      }
      mx0 = std::max<size_t>(mx0, std::max((size_t)sp.att_heads * sp.att_dim, (size_t)sp.att_heads * sp.att_vdim));
      mx1 = std::max<size_t>(mx1, sp.att_kv_rank);
      mx2 = std::max<size_t>(mx2, (size_t)sp.att_heads * sp.att_kv_rank);
      mx3 = std::max<size_t>(mx3, std::max((size_t)sp.att_heads * sp.att_kv_rank, (size_t)sp.att_heads * sp.att_vdim));
    }
    if (sp.ff_kind == DSK_FF_MOE) {
      mxE = std::max<size_t>(mxE, sp.ff_experts); mxTop = std::max<size_t>(mxTop, sp.ff_top);
      mx0 = std::max<size_t>(mx0, sp.ff_experts);
      mx2 = std::max<size_t>(mx2, (size_t)sp.ff_top * sp.ff_hidden); mx3 = std::max<size_t>(mx3, (size_t)sp.ff_top * c.dim);
    }
    if (sp.ff_kind == DSK_FF_DENSE) mx2 = std::max<size_t>(mx2, sp.ff_hidden);
    mx1 = std::max<size_t>(mx1, c.side_dim);
  }
  S->max_tiles = (int)(Tc * mxTop / 64 + mxE + 1);
  int rc = 0;
  size_t mxPart = 0;
  for (const HLayer& L : M->L) {
    if (L.sp.mixer == DSK_MIX_LATENT_SWA) mxPart = std::max(mxPart, (size_t)kAttnSplitTokens * L.sp.att_heads * kAttnSplitMax * (L.sp.att_kv_rank + 2));
    if (L.sp.mixer == DSK_MIX_GQA) mxPart = std::max(mxPart, (size_t)kAttnSplitTokens * L.sp.att_heads * kAttnSplitMax * (L.sp.att_vdim + 2));
    if (L.sp.mixer == DSK_MIX_MLA) mxPart = std::max(mxPart, (size_t)kAttnSplitTokens * L.sp.att_heads * kAttnSplitMax * (L.sp.att_kv_rank + L.sp.att_rot_dim + 2));
  }
  rc |= salloc(S, (void**)&S->part, mxPart * 4);
  if ((int)Tc >= kPrefillMin) {   // buffers of the matrix-product attention path, unless a window is too long for them
    // latent attention up-projects keys and values of all heads (fp32, then packed in the matrix type); grouped-query
    // attention packs its cached key / value heads in fp32 (kf / vf) and needs a second score array when it mixes heads
    // (latent attention with a rotated key part packs in fp32: its scores are 32-bit products)
    size_t keys = 0, hd = 0, hv = 0, heads = 0, pack_es = 0;
    bool latent = false;
    for (const HLayer& L : M->L) {
      if (L.sp.mixer == DSK_MIX_SSD || L.sp.mixer == DSK_MIX_HGRN2) continue;
      const size_t kh = L.sp.mixer == DSK_MIX_GQA ? L.sp.att_kv_heads : L.sp.att_heads;
      latent |= L.sp.mixer == DSK_MIX_LATENT_SWA || L.sp.mixer == DSK_MIX_MLA;
      if (L.sp.mixer == DSK_MIX_LATENT_SWA) pack_es = std::max(pack_es, M->wsize);
      if (L.sp.mixer == DSK_MIX_MLA) pack_es = 4;
      keys = std::max<size_t>(keys, (size_t)std::min<long long>((long long)L.sp.att_window - 1, (long long)c.max_seq_len) + std::min<size_t>(Tc, kPrefillQ) +
                                        (L.sp.mixer == DSK_MIX_GQA ? L.sp.att_keep_first : 0));
      hd = std::max<size_t>(hd, kh * (L.sp.att_dim + (L.sp.mixer == DSK_MIX_MLA ? L.sp.att_rot_dim : 0))); hv = std::max<size_t>(hv, kh * L.sp.att_vdim);
      heads = std::max<size_t>(heads, L.sp.att_heads);
    }
    const size_t bytes = keys * (hd + hv) * (4 + (latent ? pack_es : 0)) + heads * kPrefillQ * keys * 4 * (any_talk ? 2 : 1);
    if (keys > 0 && bytes <= ((size_t)4 << 30)) {
      S->prefill_keys = (int)keys;
      rc |= salloc(S, (void**)&S->kf, keys * hd * 4) | salloc(S, (void**)&S->vf, keys * hv * 4);
      if (latent) rc |= salloc(S, &S->kb, keys * hd * pack_es) | salloc(S, &S->vt, keys * hv * pack_es);
      rc |= salloc(S, (void**)&S->sc, heads * kPrefillQ * keys * 4) | salloc(S, (void**)&S->d_rows, keys * 4);
      if (any_talk) rc |= salloc(S, (void**)&S->sc2, heads * kPrefillQ * keys * 4);
    }
  }
  rc |= salloc(S, (void**)&S->x, Tc * c.dim * 4) | salloc(S, (void**)&S->h, Tc * c.dim * 4);
  if (c.block != DSK_BLOCK_PARALLEL) rc |= salloc(S, (void**)&S->y, Tc * c.dim * 4);
  if (c.token_shift) rc |= salloc(S, (void**)&S->hs, Tc * c.dim * 4);
  if (mxGV) rc |= salloc(S, (void**)&S->vfirst, Tc * mxGV * 4);
  rc |= salloc(S, (void**)&S->d_prev, 16);
  rc |= salloc(S, (void**)&S->b0, Tc * mx0 * 4) | salloc(S, (void**)&S->b1, Tc * mx1 * 4) | salloc(S, (void**)&S->b2, Tc * mx2 * 4) | salloc(S, (void**)&S->b3, Tc * mx3 * 4);
  rc |= salloc(S, (void**)&S->wgt, Tc * mxTop * 4) | salloc(S, (void**)&S->d_idx, Tc * mxTop * 4) | salloc(S, (void**)&S->d_perm, Tc * mxTop * 4);
  rc |= salloc(S, (void**)&S->d_tiles, (size_t)S->max_tiles * sizeof(int4)) | salloc(S, (void**)&S->d_ntiles, 16);
  rc |= salloc(S, (void**)&S->d_tok, Tc * 4) | salloc(S, (void**)&S->d_want, Tc * 4) | salloc(S, (void**)&S->d_ctl, 16);
  S->head_rows = (int)std::min<size_t>(Tc, 256);
  rc |= salloc(S, (void**)&S->logits, (size_t)S->head_rows * c.vocab_size * 4);
  if (rc) { fail(-2, "state allocation failed"); return nullptr; }
  if (cudaMallocHost((void**)&S->h_tok, Tc * 4) != cudaSuccess || cudaMallocHost((void**)&S->h_want, Tc * 4) != cudaSuccess) { fail(-2, "pinned allocation failed"); return nullptr; }
  m->n_states++;
  return s;
}

static void state_free(dsk_state* s) {
  State* S = s->hy;
  if (!S) return;
  if (S->step_graph) cudaGraphExecDestroy(S->step_graph);
  for (cudaEvent_t e : S->tl_events) cudaEventDestroy(e);
  for (void* p : S->allocs) cudaFree(p);
  cudaFreeHost(S->h_tok); cudaFreeHost(S->h_want);
  delete S;
  s->hy = nullptr;
}

// ---------------------------------------------------------------------------------------------------------------------
// the chunk step
// ---------------------------------------------------------------------------------------------------------------------
// marks the end of a group of launches (timeline mode only; never inside a captured step)
static void mark(State* S, const char* label, cudaStream_t st) {
  if (!S->timeline) return;
  if (S->tl_used == S->tl_events.size()) { cudaEvent_t e; cudaEventCreate(&e); S->tl_events.push_back(e); S->tl_labels.push_back(label); }
  S->tl_labels[S->tl_used] = label;
  cudaEventRecord(S->tl_events[S->tl_used++], st);
}
static void timeline_report(State* S, int T) {
  if (!S->timeline || S->tl_used < 2) { S->tl_used = 0; return; }
  cudaEventSynchronize(S->tl_events[S->tl_used - 1]);
  std::map<std::string, double> sum;
  double tot = 0;
  for (size_t i = 1; i < S->tl_used; i++) {
    float ms = 0;
    cudaEventElapsedTime(&ms, S->tl_events[i - 1], S->tl_events[i]);
    sum[S->tl_labels[i]] += ms; tot += ms;
  }
  fprintf(stderr, "[dsk timeline] step of %d tokens: %.3f ms |", T, tot);
  for (auto& kv : sum) fprintf(stderr, " %s %.3f", kv.first.c_str(), kv.second);
  fprintf(stderr, "\n");
  S->tl_used = 0;
}

static GemmP gp(const float* A, int lda, const void* W, int ldw, float* C, int ldc, int M, int N, int K) {
  GemmP P{};
  P.A = A; P.lda = lda; P.W = W; P.ldw = ldw; P.C = C; P.ldc = ldc; P.M = M; P.N = N; P.K = K;
  P.a_div = 1; P.z_adiv = 1; P.z_wdiv = 1; P.alpha = 1.f;
  return P;
}

static void launch_gemm_mma(int epi, const GemmP& P, int Z, int tile_cap, cudaStream_t st) {
  const int bn = epi_dual(epi) ? 64 : 128;
  const dim3 grid((unsigned)((P.N + bn - 1) / bn), (unsigned)(P.tiles ? tile_cap : (P.M + 127) / 128), (unsigned)Z);
  switch (epi) {
    case HEPI_STORE: gemm_mma<HEPI_STORE><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_ADD: gemm_mma<HEPI_ADD><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_GLU: gemm_mma<HEPI_GLU><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_XIELU: gemm_mma<HEPI_XIELU><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_GEGLU: gemm_mma<HEPI_GEGLU><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_SIGMUL: gemm_mma<HEPI_SIGMUL><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_RELU2: gemm_mma<HEPI_RELU2><<<grid, 256, kMmaSmem, st>>>(P); break;
    case HEPI_LINGATE: gemm_mma<HEPI_LINGATE><<<grid, 256, kMmaSmem, st>>>(P); break;
    default: gemm_mma<HEPI_GELU_MUL><<<grid, 256, kMmaSmem, st>>>(P); break;
  }
}

template <typename WT>
static void launch_gemm_t(int epi, const GemmP& P, int Z, bool small, int tile_cap, cudaStream_t st) {
  if (small) {
    const dim3 grid((unsigned)std::max(1, std::min((P.N + 7) / 8, 148 * 8)), (unsigned)Z);
    switch (epi) {
      case HEPI_STORE: gemv_rows<WT, HEPI_STORE><<<grid, 256, 0, st>>>(P); break;
      case HEPI_ADD: gemv_rows<WT, HEPI_ADD><<<grid, 256, 0, st>>>(P); break;
      case HEPI_GLU: gemv_rows<WT, HEPI_GLU><<<grid, 256, 0, st>>>(P); break;
      case HEPI_XIELU: gemv_rows<WT, HEPI_XIELU><<<grid, 256, 0, st>>>(P); break;
      case HEPI_GEGLU: gemv_rows<WT, HEPI_GEGLU><<<grid, 256, 0, st>>>(P); break;
      case HEPI_SIGMUL: gemv_rows<WT, HEPI_SIGMUL><<<grid, 256, 0, st>>>(P); break;
      case HEPI_RELU2: gemv_rows<WT, HEPI_RELU2><<<grid, 256, 0, st>>>(P); break;
      case HEPI_LINGATE: gemv_rows<WT, HEPI_LINGATE><<<grid, 256, 0, st>>>(P); break;
      default: gemv_rows<WT, HEPI_GELU_MUL><<<grid, 256, 0, st>>>(P); break;
    }
  } else {
    const dim3 grid((unsigned)((P.N + 63) / 64), (unsigned)(P.tiles ? tile_cap : (P.M + 63) / 64), (unsigned)Z);
    switch (epi) {
      case HEPI_STORE: gemm_tiled<WT, HEPI_STORE><<<grid, 256, 0, st>>>(P); break;
      case HEPI_ADD: gemm_tiled<WT, HEPI_ADD><<<grid, 256, 0, st>>>(P); break;
      case HEPI_GLU: gemm_tiled<WT, HEPI_GLU><<<grid, 256, 0, st>>>(P); break;
      case HEPI_XIELU: gemm_tiled<WT, HEPI_XIELU><<<grid, 256, 0, st>>>(P); break;
      case HEPI_GEGLU: gemm_tiled<WT, HEPI_GEGLU><<<grid, 256, 0, st>>>(P); break;
      case HEPI_SIGMUL: gemm_tiled<WT, HEPI_SIGMUL><<<grid, 256, 0, st>>>(P); break;
      case HEPI_RELU2: gemm_tiled<WT, HEPI_RELU2><<<grid, 256, 0, st>>>(P); break;
      case HEPI_LINGATE: gemm_tiled<WT, HEPI_LINGATE><<<grid, 256, 0, st>>>(P); break;
      default: gemm_tiled<WT, HEPI_GELU_MUL><<<grid, 256, 0, st>>>(P); break;
    }
  }
}
// C = A W^T (+ epilogue).  Z > 1: per-head batches or (gemv) one batch per routed (token, slot) pair.
static void linear(State* S, bool bf16, int epi, const GemmP& P, int Z, cudaStream_t st, int tile_cap = 0) {
  const bool small = P.z_expert != nullptr || (!P.tiles && P.M <= 4);
  if (!small && !P.tiles && Z == 1 && P.N <= 64) {   // narrow output (router, token-input gate): warp-per-row products over batches of 4 rows
    GemmP Q = P;
    Q.z_rows = P.M;
    const int zb = (P.M + 3) / 4;
    if (bf16) launch_gemm_t<__nv_bfloat16>(epi, Q, zb, true, 0, st);
    else launch_gemm_t<float>(epi, Q, zb, true, 0, st);
    S->launches++;
    return;
  }
  if (bf16 && !small) launch_gemm_mma(epi, P, Z, tile_cap, st);
  else if (bf16) launch_gemm_t<__nv_bfloat16>(epi, P, Z, small, tile_cap, st);
  else launch_gemm_t<float>(epi, P, Z, small, tile_cap, st);
  S->launches++;
}

static void launch_scan(const dsk_layer_spec& sp, const float* proj, int ld_proj, const float* xbc, int ld_xbc, const HLayer& L,
                        float* state, float* out, int T, cudaStream_t st) {
  const int H = sp.ssm_heads, P = sp.ssm_vdim, N = sp.ssm_state, G = sp.ssm_groups;
  const int inner = H * P;
  int PB = std::min(P, 64);   // value channels per CTA: fewer when the heads alone would leave most SMs idle
  while (PB > 32 && H * ((P + PB - 1) / PB) < 148) PB /= 2;   // (measured: 32 channels per CTA is the best split at 64 heads x 64)
  if (const char* e = getenv("DSK_SCAN_PB")) PB = std::max(1, std::min(std::min(P, 64), atoi(e)));   // A/B switch
  const dim3 grid((unsigned)H, (unsigned)((P + PB - 1) / PB));
  const int threads = ((PB * 8 + 31) / 32) * 32;
  const int TB = T >= 64 ? 64 : 16;   // tokens staged per round
  const int NP = (N + 3) & ~3;
  const size_t smem = (size_t)TB * (2 + 2 * NP + 2 * PB) * 4;
  const int need = (N + 31) / 32;     // float4 groups of state per thread
#define DSK_SCAN(RQ) ssd_scan<RQ><<<grid, threads, smem, st>>>(proj, ld_proj, 0, inner + (int)ssd_channels(sp), xbc, ld_xbc, 0, inner, inner + G * N, \
                                                               L.dt_bias, L.A_log, L.D, state, out, inner, T, H, P, N, G, PB, TB)
  if (need <= 1) DSK_SCAN(1); else if (need <= 2) DSK_SCAN(2); else if (need <= 3) DSK_SCAN(3); else if (need <= 4) DSK_SCAN(4);
  else if (need <= 6) DSK_SCAN(6); else DSK_SCAN(8);
#undef DSK_SCAN
}

static void launch_hgrn2(const dsk_layer_spec& sp, const float* proj, int ld, float* state, float* out, int T, cudaStream_t st) {
  const int H = sp.lin_heads, N = sp.lin_dim, P = sp.lin_vdim;
  // threads per value channel (measured at 16 heads x 128 x 128 and x 64 x 64: 16 threads and 16 channels per CTA are the best split; fewer
  // channels per CTA repeat the staging of a head's gates and queries in more CTAs, more leave SMs idle)
  int TPC = N >= 256 ? 32 : N >= 64 ? 16 : 8;
  if (const char* e = getenv("DSK_LIN_TPC")) { const int v = atoi(e); if ((v == 8 || v == 16 || v == 32) && N >= 4 * v) TPC = v; }   // A/B switch
  int PB = std::min(P, 512 / TPC);   // value channels per CTA
  while (PB > 16 && H * ((P + PB - 1) / PB) < 148) PB /= 2;
  if (PB == 16 && H * ((P + 15) / 16) < 74) PB = 8;
  if (const char* e = getenv("DSK_LIN_PB")) PB = std::max(1, std::min(std::min(P, 512 / TPC), atoi(e)));   // A/B switch
  const dim3 grid((unsigned)H, (unsigned)((P + PB - 1) / PB));
  const int threads = ((PB * TPC + 31) / 32) * 32;
  const int NP = (N + 3) & ~3;
  int TB = T >= 64 ? 64 : 16;         // tokens staged per round, in two buffers
  while (TB > 16 && (size_t)2 * TB * (2 * NP + PB) * 4 > 160 * 1024) TB /= 2;
  const size_t smem = (size_t)2 * TB * (2 * NP + PB) * 4;
  const int need = (N + 4 * TPC - 1) / (4 * TPC);     // float4 groups of state per thread
#define DSK_LIN(RQ, C) hgrn2_scan<RQ, C><<<grid, threads, smem, st>>>(proj, ld, 0, H * N, 2 * H * N, state, out, H * P, T, H, N, P, PB, TB)
  if (TPC == 32) { if (need <= 1) DSK_LIN(1, 32); else DSK_LIN(2, 32); }
  else if (TPC == 16) { if (need <= 1) DSK_LIN(1, 16); else if (need <= 2) DSK_LIN(2, 16); else if (need <= 3) DSK_LIN(3, 16); else DSK_LIN(4, 16); }
  else if (need <= 1) DSK_LIN(1, 8); else if (need <= 2) DSK_LIN(2, 8); else if (need <= 3) DSK_LIN(3, 8); else if (need <= 4) DSK_LIN(4, 8);
  else if (need <= 6) DSK_LIN(6, 8); else DSK_LIN(8, 8);
#undef DSK_LIN
}

static int R0(const Model* M, size_t ri) { return M->runs[ri].owner_run; }

static void launch_attn(const float* qa, const float* cache, float* out, int T, int H, int R, const int* ctl, int mask, int window, int ring,
                        float scale, float* part, cudaStream_t st) {
  const int TQ = T >= 8 ? 8 : T >= 4 ? 4 : T >= 2 ? 2 : 1, HB = 8 / TQ;
  int NS = 1;
  if (T <= kAttnSplitTokens) {   // the widest key range a CTA can meet is window + TQ - 1 keys
    const int tiles = (std::min(window, ring) + TQ - 1 + 31) / 32;
    NS = std::max(1, std::min(tiles, kAttnSplitMax));
  }
  const dim3 grid((unsigned)((T + TQ - 1) / TQ), (unsigned)((H + HB - 1) / HB), (unsigned)NS);
  const size_t smem = ((size_t)8 * R + (size_t)32 * (R + 1)) * 4;
  if (R <= 128) latent_swa_attn<float, 4><<<grid, 256, smem, st>>>(qa, cache, out, T, H, R, ctl, mask, window, ring, scale, TQ, NS, part);
  else if (R <= 256) latent_swa_attn<float, 8><<<grid, 256, smem, st>>>(qa, cache, out, T, H, R, ctl, mask, window, ring, scale, TQ, NS, part);
  else if (R <= 512) latent_swa_attn<float, 16><<<grid, 256, smem, st>>>(qa, cache, out, T, H, R, ctl, mask, window, ring, scale, TQ, NS, part);
  else latent_swa_attn<float, 32><<<grid, 256, smem, st>>>(qa, cache, out, T, H, R, ctl, mask, window, ring, scale, TQ, NS, part);
  if (NS > 1) latent_swa_merge<<<dim3((unsigned)(T * H), (unsigned)((R + 127) / 128)), 128, 0, st>>>(part, out, R, NS);
}

// LM head on the wanted rows [first, first + count) of the chunk whose normalised rows are in S->h -> S->logits [count][vocab]
static void enqueue_head(dsk_model* m, dsk_state* s, int first, int count, cudaStream_t st) {
  Model* M = m->hy;
  State* S = s->hy;
  const dsk_hybrid_config& c = M->c;
  GemmP P = gp(S->h, c.dim, c.tie_head ? M->embed.p : M->head.p, c.dim, S->logits, c.vocab_size, count, c.vocab_size, c.dim);
  P.a_map = S->d_want + first; P.alpha = c.logit_scale;
  linear(S, c.quant == DSK_BF16, HEPI_STORE, P, 1, st);
}

// the model's norm over the T rows of `in` (width values each): stored into `out`, or added into it times alpha (mode 1)
static void norm_rows(const dsk_hybrid_config& c, State* S, const float* in, const float* w, const float* b, float* out, int T, int mode, float alpha, cudaStream_t st) {
  if (c.norm_kind == DSK_NORM_LAYER) layer_norm<<<T, 256, 0, st>>>(in, c.dim, w, b, out, c.dim, c.dim, c.norm_eps, mode, alpha, nullptr, 0);
  else group_rmsnorm<float><<<T, 256, 0, st>>>(in, c.dim, w, out, c.dim, c.dim, c.norm_groups, c.norm_eps, mode, alpha, nullptr, 0);
  S->launches++;
}

static bool fused_norms(const dsk_hybrid_config& c) {
  return c.block == DSK_BLOCK_SANDWICH && c.norm_kind == DSK_NORM_LAYER && c.dim <= 256 * kLnRegs && c.side_dim == 0;
}

// where a sublayer's last product goes: added into the residual stream (parallel blocks), or stored for the closing norm
struct Sink { int epi; float* C; float alpha; };

// Enqueues the kernels of one chunk of T <= chunk tokens (ids in S->d_tok, first position in S->d_ctl) on `st`.
// n_want > 0: the LM head runs on the rows listed in S->d_want -> S->logits [n_want][vocab].  trace (device, nullable):
// [layer runs][T][width] copies of the residual stream after every layer run.
// pos0 >= 0: the first position as the host knows it (portions may then take the matrix-product attention path); -1 inside a
// captured step, where positions live in device memory only.
static int enqueue_chunk(dsk_model* m, dsk_state* s, int T, int n_want, float* trace, cudaStream_t st, int pos0 = -1) {
  Model* M = m->hy;
  State* S = s->hy;
  const dsk_hybrid_config& c = M->c;
  const bool bf = c.quant == DSK_BF16;
  const bool sandwich = c.block == DSK_BLOCK_SANDWICH, post = c.block == DSK_BLOCK_POST;
  const int W = c.dim;
  const float mult = c.residual_mult;
  const float es = c.embed_scale != 0.f ? c.embed_scale : 1.f;
  const int nb = c.bigram_buckets;
  if (bf) embed_rows<__nv_bfloat16><<<T, 256, 0, st>>>(S->d_tok, (const __nv_bfloat16*)M->embed.p, W, S->x, es, nb > 0 ? (const __nv_bfloat16*)M->bigram.p : nullptr,
                                                       nb, c.bigram_mul_prev, c.bigram_mul_cur, S->d_ctl, S->d_prev);
  else embed_rows<float><<<T, 256, 0, st>>>(S->d_tok, (const float*)M->embed.p, W, S->x, es, nb > 0 ? (const float*)M->bigram.p : nullptr, nb, c.bigram_mul_prev,
                                            c.bigram_mul_cur, S->d_ctl, S->d_prev);
  S->launches++;
  if (nb > 0) { carry_token<<<1, 1, 0, st>>>(S->d_tok, T, S->d_prev); S->launches++; }   // the next step's first token pairs with this step's last
  if (pos0 < 0) S->tl_used = 0;   // a captured step records no events
  const bool tl = S->timeline && pos0 >= 0;
  auto MK = [&](const char* label) { if (tl) mark(S, label, st); };
  MK("embed");
  const Sink to_x{HEPI_ADD, S->x, mult}, to_y{HEPI_STORE, S->y, 1.f};
  // sandwich blocks of layer norms: "x += ln(y); h = ln(x)" runs as one kernel (not while the residual stream is being recorded)
  const bool fuse = fused_norms(c) && !trace;
  bool h_ready = false;   // S->h already holds the norm that opens the coming run (or the final norm)
  bool hs_ready = false;  // S->hs already holds the token-shifted input of the coming run's mixer
  for (size_t ri = 0; ri < M->runs.size(); ri++) {
    const Run& run = M->runs[ri];
    const int li = run.layer;
    const HLayer& L = M->L[li];
    const dsk_layer_spec& sp = L.sp;
    LayerState& ls = S->L[ri];
    // post-norm blocks: a sublayer reads u = x + conv(x) (S->h; the stream itself without a convolution); afterwards its result y is gated
    // by sigmoid(rg x + b), normalised with the folded weight (norm x layer scale) and added to the stream
    auto open_post = [&](const float* taps, int which) -> const float* {
      if (c.canon_taps <= 0) return S->x;
      float* ring = ls.canon ? ls.canon + (size_t)which * (c.canon_taps - 1) * W : nullptr;
      const int ty = (T + kCanonTokens - 1) / kCanonTokens;
      canon_conv<<<dim3((unsigned)((W + 127) / 128), (unsigned)ty), 128, 0, st>>>(S->x, W, taps, ring, S->h, W, T, W, c.canon_taps, S->d_ctl);
      S->launches++;
      if (ty > 1 && c.canon_taps > 1) { canon_history<<<(W + 127) / 128, 128, 0, st>>>(S->x, W, ring, T, W, c.canon_taps, S->d_ctl); S->launches++; }
      return S->h;
    };
    auto close_post = [&](const HTensor& rg, const float* rg_b, const float* close_w, const float* close_b) {
      if (c.res_gate) {
        GemmP G = gp(S->x, W, rg.p, W, S->y, W, T, W, W);
        G.bias = rg_b;
        linear(S, bf, HEPI_SIGMUL, G, 1, st);
      }
      norm_rows(c, S, S->y, close_w, close_b, S->x, T, 1, mult, st);
    };
    // decode-sized steps: the closing norm and the next sublayer's input convolution as one kernel (not while the stream is recorded);
    // next_taps / next_ring: the convolution that follows (the feed-forward's, or the next layer's mixer's)
    const bool small_post = post && c.canon_taps > 0 && T <= kCloseOpenTokens && !trace;
    auto close_open = [&](const HTensor& rg, const float* rg_b, const float* close_w, const float* next_taps, float* next_ring) {
      if (c.res_gate) {
        GemmP G = gp(S->x, W, rg.p, W, S->y, W, T, W, W);
        G.bias = rg_b;
        linear(S, bf, HEPI_SIGMUL, G, 1, st);
      }
      close_open_small<<<(W + 127) / 128, 128, 0, st>>>(S->y, close_w, mult, c.norm_eps, S->x, W, next_taps, next_ring, S->h, T, W, c.canon_taps, S->d_ctl);
      S->launches++;
    };
    auto ring_of = [&](size_t run_i, int which) { return S->L[run_i].canon ? S->L[run_i].canon + (size_t)which * (c.canon_taps - 1) * W : nullptr; };
    const bool has_next = ri + 1 < M->runs.size();
    const float* hin = S->h;   // what the mixer reads
    if (post) { if (!h_ready) hin = open_post(L.canon1, 0); }
    else if (!h_ready) {
      if (run.pass >= 0) {   // a pass of the layer loop opens with its own vector added to the residual stream
        add_row<<<T, 256, 0, st>>>(S->x, W, M->loop_step + (size_t)run.pass * W, W);
        S->launches++;
      }
      norm_rows(c, S, S->x, L.norm1, L.norm1_bias, S->h, T, 0, 0.f, st);
    }
    h_ready = false;
    const float* hff = hin;   // what a feed-forward of a parallel block reads: the mixer's input ahead of the token shift
    if (c.token_shift && hs_ready) { hin = S->hs; hs_ready = false; }   // the previous run's last kernel shifted already
    else if (c.token_shift) {      // the mixer reads its input blended with the previous token's; the step's last row is carried on
      const int ty = (T + kCanonTokens - 1) / kCanonTokens;
      token_shift<<<dim3((unsigned)((W + 127) / 128), (unsigned)ty), 128, 0, st>>>(hin, W, L.shift, ls.shift, S->hs, W, T, W, S->d_ctl);
      S->launches++;
      if (ty > 1) { shift_carry<<<(W + 127) / 128, 128, 0, st>>>(hin, W, ls.shift, T, W); S->launches++; }
      hin = S->hs;
    }
    // the closing norm of this run's last sublayer, fused with what opens the next run (its pass vector and first norm) or the head
    auto close_run = [&](const float* wb) {
      if (!fuse) { norm_rows(c, S, S->y, wb, nullptr, S->x, T, 1, mult, st); return; }
      const Run* next = ri + 1 < M->runs.size() ? &M->runs[ri + 1] : nullptr;
      const float* row = next && next->pass >= 0 ? M->loop_step + (size_t)next->pass * W : nullptr;
      layer_norm_add_norm<<<T, 256, 0, st>>>(S->y, wb, S->x, row, next ? M->L[next->layer].norm1 : M->final_norm, S->h, W, c.norm_eps, mult);
      S->launches++;
      h_ready = true;
    };
    const Sink sink = (sandwich || post) ? to_y : to_x;
    // a routed feed-forward that closes with a layer norm and no gate: no separate pass for the weighted sum of the experts' outputs
    const bool combine_in_norm = post && sp.ff_kind == DSK_FF_MOE && c.norm_kind == DSK_NORM_LAYER && !c.res_gate && W <= 256 * kLnRegs;
    if (sp.mixer == DSK_MIX_GQA) {
      const int H = sp.att_heads, G = sp.att_kv_heads, D = sp.att_dim, V = sp.att_vdim, HD = H * D, GD = G * D, GV = G * V, rep = H / G;
      const int keep = sp.att_keep_first;
      const bool reads = sp.att_kv_from >= 0;   // keys and values of another layer: its caches, written earlier in this step
      const int ring = M->L[L.owner].ring;
      float *kc = (float*)S->L[R0(M, ri)].cache, *vc = (float*)S->L[R0(M, ri)].vcache;
      const ScoreMods sm{sp.att_softcap, sp.att_rel_max > 0 ? L.rel : nullptr, L.rel_bucket, sp.att_rel_max, sp.att_sink ? L.sink : nullptr, keep};
      MK("norm");
      const int HV = sp.att_out_gate ? H * V : 0;   // the output gate's raw values come out of the stacked product, behind q / k / v
      const int ldp = reads ? HD + HV : HD + GD + GV + HV;
      const float* gate = HV ? S->b0 + (ldp - HV) : nullptr;
      if (reads) {
        linear(S, bf, HEPI_STORE, gp(hin, W, L.qkv.p, W, S->b0, ldp, T, ldp, W), 1, st);
        MK("att.qk");
        qk_norm_rope<<<T, 256, 0, st>>>(S->b0, S->b2, HD, nullptr, nullptr, GD, GV, ldp, 0, 0, L.q_norm, nullptr, c.norm_eps, D, sp.rot_dims, L.rot_freq,
                                        L.rot_mag, S->d_ctl, nullptr, nullptr, ring, keep, nullptr, 0.f, nullptr, sp.rot_layout, sp.att_qk_norm);
      } else if (sp.att_value_proj) {   // one product for the stacked q / k / v rows; the first value-mixing layer keeps its values for the later ones
        const int ld = ldp;
        GemmP P = gp(hin, W, L.qkv.p, W, S->b0, ld, T, ld, W);
        P.bias = sp.att_bias ? L.qkv_b : nullptr;
        linear(S, bf, HEPI_STORE, P, 1, st);
        MK("att.qk");
        const bool blend = sp.att_vmix && li != M->vmix_first;
        qk_norm_rope<<<T, 256, 0, st>>>(S->b0, S->b2, HD, S->b0 + HD, S->b0 + HD + GD, GD, GV, ld, ld, ld, L.q_norm, L.k_norm, c.norm_eps, D, sp.rot_dims,
                                        L.rot_freq, L.rot_mag, S->d_ctl, kc, vc, ring, keep, blend ? S->vfirst : nullptr, L.vmix,
                                        sp.att_vmix && li == M->vmix_first ? S->vfirst : nullptr, sp.rot_layout, sp.att_qk_norm);
      } else {
        linear(S, bf, HEPI_STORE, gp(hin, W, L.q.p, W, S->b0, HD, T, HD, W), 1, st);
        linear(S, bf, HEPI_STORE, gp(hin, W, L.kproj.p, W, S->b1, GD, T, GD, W), 1, st);
        MK("att.qk");
        qk_norm_rope<<<T, 256, 0, st>>>(S->b0, S->b2, HD, S->b1, nullptr, GD, GV, HD, GD, GD, L.q_norm, L.k_norm, c.norm_eps, D, sp.rot_dims, L.rot_freq,
                                        L.rot_mag, S->d_ctl, kc, vc, ring, keep, nullptr, 0.f, nullptr, sp.rot_layout, sp.att_qk_norm);
      }
      S->launches++;
      MK("att.norm+rot");
      if (pos0 >= 0 && T >= kPrefillMin && S->prefill_keys > 0) {
        // a portion: blocks of kPrefillQ queries, each as  scores = q k^T per head (fp32);  mixing of the heads;  masked softmax;  o = P v
        for (int t0 = 0; t0 < T; t0 += kPrefillQ) {
          const int Tq = std::min(kPrefillQ, T - t0), qpos0 = pos0 + t0;
          const int first = mask_first(sp.att_mask, sp.att_window, qpos0), nk = std::min(keep, first), Lk = nk + qpos0 + Tq - first;
          pack_ring_kv<float><<<Lk, 256, 0, st>>>(kc, vc, S->kf, S->vf, first, Lk, ring, G, D, V, nk, keep);
          S->launches++;
          MK("att.pack");
          GemmP Sc = gp(S->b2 + (size_t)t0 * HD, HD, S->kf, D, S->sc, Lk, Tq, Lk, D);
          Sc.sA = D; Sc.sW = (long long)Lk * D; Sc.z_wdiv = rep; Sc.sC = (long long)Tq * Lk; Sc.alpha = sp.att_scale;
          linear(S, false, HEPI_STORE, Sc, H, st);
          MK("att.scores");
          float* pr = S->sc;
          if (sp.att_talk) {
            const long long n = (long long)Tq * Lk;
            mix_heads<<<(unsigned)((n + 127) / 128), 128, (size_t)(H * H + H * 128) * 4, st>>>(S->sc, S->sc2, L.talk, H, n);
            S->launches++;
            pr = S->sc2;
          }
          softmax_band<<<dim3((unsigned)Tq, (unsigned)H), 128, 0, st>>>(pr, Tq, Lk, first, qpos0, sp.att_mask, sp.att_window, nk, sm);
          S->launches++;
          MK("att.softmax");
          GemmP Ov = gp(pr, Lk, S->vf, Lk, S->b3 + (size_t)t0 * H * V, H * V, Tq, V, Lk);
          Ov.sA = (long long)Tq * Lk; Ov.sW = (long long)V * Lk; Ov.z_wdiv = rep; Ov.sC = V;
          linear(S, false, HEPI_STORE, Ov, H, st);
          MK("att.pv");
        }
        if (gate) { gate_rows<<<T, 256, 0, st>>>(S->b3, H * V, gate, ldp, H * V); S->launches++; }   // heads *= sigmoid(g h)
      } else {
        int NS = 1;
        if (T <= kAttnSplitTokens) NS = std::max(1, std::min((std::min(sp.att_window, ring) + keep + 31) / 32, kAttnSplitMax));
        // without score mixing the key heads are dealt over CTAs, as few per CTA as keep four query heads (half the warps) busy
        int GL = G;
        if (!sp.att_talk)
          for (int d = G; d >= 1; d--) if (G % d == 0 && d * rep >= 4) GL = d;
        gqa_attn<<<dim3((unsigned)T, (unsigned)NS, (unsigned)(G / GL)), 256, gqa_attn_smem_floats(H, G, D, V) * 4, st>>>(
            S->b2, kc, vc, S->b3, sp.att_talk ? L.talk : nullptr, T, H, G, D, V, S->d_ctl, sp.att_mask, sp.att_window, ring, sp.att_scale, NS, S->part, sm,
            NS > 1 ? nullptr : gate, ldp);
        if (NS > 1) latent_swa_merge<<<dim3((unsigned)(T * H), (unsigned)((V + 127) / 128)), 128, 0, st>>>(S->part, S->b3, V, NS, gate, ldp, H);
        S->launches += NS > 1 ? 2 : 1;
        MK("att.decode");
      }
      GemmP P = gp(S->b3, H * V, L.o.p, H * V, sink.C, W, T, W, H * V);
      P.alpha = sink.alpha;
      linear(S, bf, sink.epi, P, 1, st);
      MK("att.o");
    } else if (sp.mixer == DSK_MIX_MLA) {
      const int H = sp.att_heads, D = sp.att_dim, Rd = sp.att_rot_dim, DK = D + Rd, V = sp.att_vdim, R = sp.att_kv_rank, RW = R + Rd, Q = sp.att_q_rank;
      float* cache = (float*)ls.cache;
      const int ldi = Q + RW;
      MK("norm");
      linear(S, bf, HEPI_STORE, gp(hin, W, L.in2.p, W, S->b1, ldi, T, ldi, W), 1, st);              // [query latent | key / value latent | rotated key part]
      group_rmsnorm<float><<<T, 256, 0, st>>>(S->b1, ldi, L.dq_norm, S->b2, Q, Q, 1, c.norm_eps, 0, 0.f, nullptr, 0);
      S->launches++;
      linear(S, bf, HEPI_STORE, gp(S->b2, Q, L.uq.p, Q, S->b0, H * DK, T, H * DK, Q), 1, st);       // q [T][H][D | Rd]
      const bool portion = pos0 >= 0 && T >= kPrefillMin && S->prefill_keys > 0;
      mla_prepare<<<T, 256, 0, st>>>(S->b1 + Q, ldi, L.dkv_norm, c.norm_eps, S->b0, portion ? nullptr : S->b2, H, D, Rd, R, sp.rot_dims, L.rot_freq,
                                     S->d_ctl, cache, L.ring);
      S->launches++;
      MK("att.q+latent");
      float* ov = S->b3;   // [T][H*V] heads' outputs
      if (portion) {
        // blocks of kPrefillQ queries: plain keys and values up-projected from the visible latents, the rotated key part appended to every
        // head's keys; scores, softmax and the value product in fp32
        for (int t0 = 0; t0 < T; t0 += kPrefillQ) {
          const int Tq = std::min(kPrefillQ, T - t0), qpos0 = pos0 + t0;
          const int first = mask_first(sp.att_mask, sp.att_window, qpos0), Lk = qpos0 + Tq - first;
          ring_rows<<<(Lk + 255) / 256, 256, 0, st>>>(first, Lk, L.ring, S->d_rows);
          GemmP K = gp(cache, RW, L.uk.p, R, S->kf, H * D, Lk, H * D, R);
          K.a_map = S->d_rows;
          linear(S, bf, HEPI_STORE, K, 1, st);
          GemmP Vp = gp(cache, RW, L.uv.p, R, S->vf, H * V, Lk, H * V, R);
          Vp.a_map = S->d_rows;
          linear(S, bf, HEPI_STORE, Vp, 1, st);
          MK("att.kv_up");
          pack_mla_kv<<<Lk, 256, 0, st>>>(S->kf, S->vf, cache, S->d_rows, (float*)S->kb, (float*)S->vt, Lk, H, D, Rd, R, V);
          MK("att.pack");
          GemmP Sc = gp(S->b0 + (size_t)t0 * H * DK, H * DK, S->kb, DK, S->sc, Lk, Tq, Lk, DK);
          Sc.sA = DK; Sc.sW = (long long)Lk * DK; Sc.sC = (long long)Tq * Lk; Sc.alpha = sp.att_scale;
          linear(S, false, HEPI_STORE, Sc, H, st);
          MK("att.scores");
          softmax_band<<<dim3((unsigned)Tq, (unsigned)H), 128, 0, st>>>(S->sc, Tq, Lk, first, qpos0, sp.att_mask, sp.att_window, 0, ScoreMods{});
          MK("att.softmax");
          GemmP Ov = gp(S->sc, Lk, S->vt, Lk, S->b3 + (size_t)t0 * H * V, H * V, Tq, V, Lk);
          Ov.sA = (long long)Tq * Lk; Ov.sW = (long long)V * Lk; Ov.sC = V;
          linear(S, false, HEPI_STORE, Ov, H, st);
          MK("att.pv");
          S->launches += 3;
        }
      } else {
        {   // absorbed query: qa[t][h][0:R] = W_uk[h]^T q_plain[t][h]  (mla_prepare put the rotated part behind it)
          GemmP P = gp(S->b0, H * DK, L.ukT.p, D, S->b2, H * RW, T, R, D);
          P.sA = DK; P.sW = (long long)R * D; P.sC = RW;
          linear(S, bf, HEPI_STORE, P, H, st);
        }
        launch_attn(S->b2, cache, S->b3, T, H, RW, S->d_ctl, sp.att_mask, sp.att_window, L.ring, sp.att_scale, S->part, st);
        S->launches++;
        {  // value up-projection per head from the first R entries of the weighted cache rows
          GemmP P = gp(S->b3, H * RW, L.uv.p, R, S->b0, H * V, T, V, R);
          P.sA = RW; P.sW = (long long)V * R; P.sC = V;
          linear(S, bf, HEPI_STORE, P, H, st);
        }
        ov = S->b0;
        MK("att.absorbed");
      }
      if (sp.att_out_gate) linear(S, bf, HEPI_SIGMUL, gp(hin, W, L.gmat.p, W, ov, H * V, T, H * V, W), 1, st);   // heads *= sigmoid(g u)
      GemmP P = gp(ov, H * V, L.o.p, H * V, sink.C, W, T, W, H * V);
      P.alpha = sink.alpha;
      linear(S, bf, sink.epi, P, 1, st);
      MK("att.o");
    } else if (sp.mixer == DSK_MIX_HGRN2) {
      const int H = sp.lin_heads, HN = H * sp.lin_dim, HP = H * sp.lin_vdim, pw = 2 * HN + HP;
      MK("norm");
      GemmP In = gp(hin, W, L.lin_in.p, W, S->b0, pw, T, pw, W);   // [silu(q) | forget gate | v]: the activations run in the product's epilogue, in fp32
      In.bias = L.lin_bias; In.aux = L.lower; In.aux_off = HN;
      linear(S, bf, HEPI_LINGATE, In, 1, st);
      MK("lin.in");
      launch_hgrn2(sp, S->b0, pw, ls.lin, S->b2, T, st);
      MK("lin.scan");
      head_rmsnorm<<<(unsigned)(((long long)T * H + 7) / 8), 256, 0, st>>>(S->b2, HP, L.lin_norm, S->b3, HP, T, H, sp.lin_vdim, c.norm_eps);
      S->launches += 2;
      MK("lin.norm");
      GemmP P = gp(S->b3, HP, L.o.p, HP, sink.C, W, T, W, HP);
      P.alpha = sink.alpha;
      linear(S, bf, sink.epi, P, 1, st);
      MK("lin.o");
    } else if (is_ssd(sp)) {
      const int inner = (int)ssd_inner(sp), ch = (int)ssd_channels(sp), pw = (int)ssd_proj(sp);
      MK("norm");
      linear(S, bf, HEPI_STORE, gp(hin, W, L.in.p, W, S->b0, pw, T, pw, W), 1, st);
      MK("ssd.in");
      causal_conv_silu<<<dim3((unsigned)((ch + 127) / 128), (unsigned)T), 128, 0, st>>>(S->b0 + inner, pw, L.conv_w, L.conv_b, ls.hist, S->b1, ch, T, ch, sp.ssm_conv);
      if (sp.ssm_conv > 1) conv_history_update<<<(ch + 127) / 128, 128, 0, st>>>(S->b0 + inner, pw, ls.hist, T, ch, sp.ssm_conv);
      MK("ssd.conv");
      launch_scan(sp, S->b0, pw, S->b1, ch, L, ls.ssm, S->b2, T, st);
      MK("ssd.scan");
      group_rmsnorm<float><<<T, 256, 0, st>>>(S->b2, inner, L.mnorm, S->b3, inner, inner, sp.ssm_norm_groups, c.norm_eps, 0, 0.f, nullptr, 0);
      S->launches += 4;
      MK("ssd.norm");
      GemmP P = gp(S->b3, inner, L.o.p, inner, sink.C, W, T, W, inner);
      P.alpha = sink.alpha;
      linear(S, bf, sink.epi, P, 1, st);
      MK("ssd.o");
    } else {
      const int H = sp.att_heads, D = sp.att_dim, V = sp.att_vdim, R = sp.att_kv_rank;
      const HLayer& O = M->L[L.owner];
      float* cache = (float*)S->L[R0(M, ri)].cache;
      MK("norm");
      linear(S, bf, HEPI_STORE, gp(hin, W, L.q.p, W, S->b0, H * D, T, H * D, W), 1, st);
      if (L.owner == li) {
        linear(S, bf, HEPI_STORE, gp(hin, W, L.dkv.p, W, S->b1, R, T, R, W), 1, st);
        group_rmsnorm<float><<<T, 256, 0, st>>>(S->b1, R, L.dkv_norm, cache, R, R, 1, c.norm_eps, 0, 0.f, S->d_ctl, O.ring);
        S->launches++;
      }
      MK("att.q+latent");
      const float* ov = S->b0;   // [T][H*V] heads' outputs
      if (pos0 >= 0 && T >= kPrefillMin && S->prefill_keys > 0) {
        // a portion: blocks of kPrefillQ queries, each as  k, v = up-projections of the visible latents;  P = softmax_band(q k^T);  o = P v
        ov = S->b3;
        for (int t0 = 0; t0 < T; t0 += kPrefillQ) {
          const int Tq = std::min(kPrefillQ, T - t0), qpos0 = pos0 + t0;
          const int first = mask_first(sp.att_mask, sp.att_window, qpos0), Lk = qpos0 + Tq - first;
          ring_rows<<<(Lk + 255) / 256, 256, 0, st>>>(first, Lk, O.ring, S->d_rows);
          GemmP K = gp(cache, R, L.uk.p, R, S->kf, H * D, Lk, H * D, R);
          K.a_map = S->d_rows;
          linear(S, bf, HEPI_STORE, K, 1, st);
          GemmP Vp = gp(cache, R, L.uv.p, R, S->vf, H * V, Lk, H * V, R);
          Vp.a_map = S->d_rows;
          linear(S, bf, HEPI_STORE, Vp, 1, st);
          MK("att.kv_up");
          if (bf) pack_keys_values<__nv_bfloat16><<<Lk, 256, 0, st>>>(S->kf, S->vf, (__nv_bfloat16*)S->kb, (__nv_bfloat16*)S->vt, Lk, H, D, V);
          else pack_keys_values<float><<<Lk, 256, 0, st>>>(S->kf, S->vf, (float*)S->kb, (float*)S->vt, Lk, H, D, V);
          GemmP Sc = gp(S->b0 + (size_t)t0 * H * D, H * D, S->kb, D, S->sc, Lk, Tq, Lk, D);
          Sc.sA = D; Sc.sW = (long long)Lk * D; Sc.sC = (long long)Tq * Lk; Sc.alpha = sp.att_scale;
          MK("att.pack");
          linear(S, bf, HEPI_STORE, Sc, H, st);
          MK("att.scores");
          softmax_band<<<dim3((unsigned)Tq, (unsigned)H), 128, 0, st>>>(S->sc, Tq, Lk, first, qpos0, sp.att_mask, sp.att_window, 0, ScoreMods{});
          GemmP Ov = gp(S->sc, Lk, S->vt, Lk, S->b3 + (size_t)t0 * H * V, H * V, Tq, V, Lk);
          Ov.sA = (long long)Tq * Lk; Ov.sW = (long long)V * Lk; Ov.sC = V;
          MK("att.softmax");
          linear(S, bf, HEPI_STORE, Ov, H, st);
          MK("att.pv");
          S->launches += 3;
        }
      } else {
        {  // absorbed query: qa[t][h][:] = W_uk[h]^T q[t][h][:]
          GemmP P = gp(S->b0, H * D, L.ukT.p, D, S->b2, H * R, T, R, D);
          P.sA = D; P.sW = (long long)R * D; P.sC = R;
          linear(S, bf, HEPI_STORE, P, H, st);
        }
        launch_attn(S->b2, cache, S->b3, T, H, R, S->d_ctl, sp.att_mask, sp.att_window, O.ring, sp.att_scale, S->part, st);
        S->launches++;
        {  // value up-projection per head: ov[t][h][:] = W_uv[h] o[t][h][:]
          GemmP P = gp(S->b3, H * R, L.uv.p, R, S->b0, H * V, T, V, R);
          P.sA = R; P.sW = (long long)V * R; P.sC = V;
          linear(S, bf, HEPI_STORE, P, H, st);
        }
      }
      MK("att.absorbed");
      GemmP P = gp(ov, H * V, L.o.p, H * V, sink.C, W, T, W, H * V);
      P.alpha = sink.alpha;
      linear(S, bf, sink.epi, P, 1, st);
      MK("att.o");
    }
    if (!post) hin = hff;
    if (post) {   // the mixer's result closes; the feed-forward (or, without one, the next layer's mixer) opens on the new stream
      if (small_post && sp.ff_kind != DSK_FF_NONE) { close_open(L.rg1, L.rg1_b, L.close1, L.canon2, ring_of(ri, 1)); hin = S->h; }
      else if (small_post && has_next) { close_open(L.rg1, L.rg1_b, L.close1, M->L[M->runs[ri + 1].layer].canon1, ring_of(ri + 1, 0)); h_ready = true; }
      else {
        close_post(L.rg1, L.rg1_b, L.close1, L.norm1_bias);
        if (sp.ff_kind != DSK_FF_NONE) hin = open_post(L.canon2, 1);
      }
      MK("norm");
    }
    if (sandwich) {   // x += norm1b(mixer output); the feed-forward then reads norm2 of the new x
      if (sp.ff_kind == DSK_FF_NONE) close_run(L.norm1b);
      else if (fuse) {
        layer_norm_add_norm<<<T, 256, 0, st>>>(S->y, L.norm1b, S->x, nullptr, L.norm2, S->h, W, c.norm_eps, mult);
        S->launches++;
      } else {
        norm_rows(c, S, S->y, L.norm1b, nullptr, S->x, T, 1, mult, st);
        norm_rows(c, S, S->x, L.norm2, nullptr, S->h, T, 0, 0.f, st);
      }
      MK("norm");
    }
    if (sp.ff_kind == DSK_FF_DENSE && sp.ff_act == DSK_ACT_GEGLU) {
      const int ff = sp.ff_hidden;
      GemmP U = gp(hin, W, L.gate_d.p, W, S->b2, ff, T, ff, W);
      U.W2 = L.up.p;
      linear(S, bf, HEPI_GEGLU, U, 1, st);
      MK("ff.up");
      GemmP Dn = gp(S->b2, ff, L.down.p, ff, sink.C, W, T, W, ff);
      Dn.alpha = sink.alpha;
      linear(S, bf, sink.epi, Dn, 1, st);
      MK("ff.down");
    } else if (sp.ff_kind == DSK_FF_DENSE) {
      const int ff = sp.ff_hidden;
      GemmP U = gp(hin, W, L.up.p, W, S->b2, ff, T, ff, W);
      U.bias = L.up_b; U.act_a = L.act_a; U.act_b = L.act_b;
      linear(S, bf, HEPI_XIELU, U, 1, st);
      MK("ff.up");
      GemmP Dn = gp(S->b2, ff, L.down.p, ff, sink.C, W, T, W, ff);
      Dn.bias = L.down_b; Dn.alpha = sink.alpha;
      linear(S, bf, sink.epi, Dn, 1, st);
      MK("ff.down");
    }
    if (sp.ff_kind == DSK_FF_MOE) {
      const int E = sp.ff_experts, top = sp.ff_top, ff = sp.ff_hidden, pairs = T * top;
      GemmP Rt = gp(hin, W, L.router, W, S->b0, E, T, E, W);   // router: fp32 weights in every mode
      Rt.bias = sp.ff_router == DSK_ROUTER_TOP_SOFTMAX ? L.router_b : nullptr;
      linear(S, false, HEPI_STORE, Rt, 1, st);
      moe_route<<<T, 128, (size_t)(2 * E + top) * 4, st>>>(S->b0, sp.ff_router == DSK_ROUTER_SIGMOID ? L.correction : nullptr, E, top, sp.ff_router_scale, S->d_idx,
                                                           S->wgt, sp.ff_router == DSK_ROUTER_TOP_SOFTMAX ? 1 : 0);
      S->launches++;
      MK("moe.router");
      const bool relu2 = sp.ff_expert == DSK_EXPERT_RELU2;   // one up matrix per expert instead of a gated pair
      const int epi_up = relu2 ? HEPI_RELU2 : HEPI_GLU;
      GemmP G = gp(hin, W, relu2 ? L.up_s.p : L.gate_s.p, W, S->b2, ff, pairs, ff, W);
      G.W2 = relu2 ? nullptr : L.up_s.p; G.sW = (long long)ff * W; G.lim = sp.ff_limit;
      GemmP Dn = gp(S->b2, ff, L.down_s.p, ff, S->b3, W, pairs, W, ff);
      Dn.sW = (long long)ff * W;
      if (T <= 4) {
        G.z_expert = S->d_idx; G.z_adiv = top; Dn.z_expert = S->d_idx; Dn.z_adiv = 1;
        linear(S, bf, epi_up, G, pairs, st);
        MK("moe.glu");
        linear(S, bf, HEPI_STORE, Dn, pairs, st);
        MK("moe.down");
      } else {
        const int bm = bf ? 128 : 64;   // rows per tile of the product kernel that follows (gemm_mma / gemm_tiled)
        moe_plan<<<1, 1024, (size_t)2 * E * 4, st>>>(S->d_idx, pairs, E, bm, S->d_perm, S->d_tiles, S->d_ntiles);
        S->launches++;
        G.tiles = S->d_tiles; G.n_tiles = S->d_ntiles; G.a_map = S->d_perm; G.a_div = top; G.c_map = S->d_perm;
        Dn.tiles = S->d_tiles; Dn.n_tiles = S->d_ntiles; Dn.a_map = S->d_perm; Dn.a_div = 1; Dn.c_map = S->d_perm;
        const int cap = std::min(S->max_tiles, pairs / bm + E + 1);
        MK("moe.plan");
        linear(S, bf, epi_up, G, 1, st, cap);
        MK("moe.glu");
        linear(S, bf, HEPI_STORE, Dn, 1, st, cap);
        MK("moe.down");
      }
      if (combine_in_norm) {   // x += ln(sum_k w_k y_k): the weighted sum of the experts' outputs is taken by the closing layer norm as it reads its row
        layer_norm<<<T, 256, 0, st>>>(S->b3, W, L.close2, L.norm2_bias, S->x, W, W, c.norm_eps, 1, mult, S->wgt, top);
      } else moe_combine<<<T, 256, 0, st>>>(sink.C, W, S->b3, S->wgt, top, W, sink.alpha, sink.epi == HEPI_ADD ? 1 : 0);
      S->launches++;
      MK("moe.combine");
    }
    if (sandwich && sp.ff_kind != DSK_FF_NONE) {
      close_run(L.norm2b);
      MK("norm");
    }
    if (post && sp.ff_kind != DSK_FF_NONE && !combine_in_norm) {
      if (small_post && has_next) { close_open(L.rg2, L.rg2_b, L.close2, M->L[M->runs[ri + 1].layer].canon1, ring_of(ri + 1, 0)); h_ready = true; }
      else close_post(L.rg2, L.rg2_b, L.close2, L.norm2_bias);
      MK("norm");
    }
    if (c.side_dim > 0) {
      const int sd = c.side_dim;
      GemmP P = gp(S->x, W, L.sgate.p, W, S->b1, sd, T, sd, W);
      P.aux = M->side_embed.p; P.aux_row = S->d_tok; P.aux_ld = sd * c.n_layers; P.aux_off = li * sd;
      linear(S, bf, HEPI_GELU_MUL, P, 1, st);
      linear(S, bf, HEPI_STORE, gp(S->b1, sd, L.sproj.p, sd, S->h, W, T, W, sd), 1, st);
      // decode-sized steps of post-norm blocks: the normed addition and the next layer's token shift in one launch over 128-channel CTAs
      if (post && c.canon_taps <= 0 && T <= kCloseOpenTokens && !trace) {
        const bool next_shift = c.token_shift && has_next;
        rms_add_shift_small<<<(W + 127) / 128, 128, 0, st>>>(S->h, L.snorm, mult, c.norm_eps, S->x, W, next_shift ? M->L[M->runs[ri + 1].layer].shift : nullptr,
                                                             next_shift ? S->L[ri + 1].shift : nullptr, S->hs, T, W, S->d_ctl);
        hs_ready = next_shift;
      } else group_rmsnorm<float><<<T, 256, 0, st>>>(S->h, W, L.snorm, S->x, W, W, 1, c.norm_eps, 1, mult, nullptr, 0);
      S->launches++;
      MK("side");
    }
    if (trace) CKL(cudaMemcpyAsync(trace + ri * (size_t)T * W, S->x, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st));
  }
  if (n_want > 0) {   // final norm of every row, LM head on the first group of wanted rows (enqueue_head does the others)
    if (!h_ready) norm_rows(c, S, S->x, M->final_norm, M->final_norm_b, S->h, T, 0, 0.f, st);
    enqueue_head(m, s, 0, std::min(n_want, S->head_rows), st);
    MK("head");
  }
  CKL(cudaGetLastError());
  return 0;
}

// tokens [n] at positions pos0.. of the state's sequence; want: ascending indices into tokens whose logits go to host_logits
// [n_want][vocab]; host_layers (nullable): [layers][n][width] residual stream after every layer.
static int forward_chunk(dsk_model* m, dsk_state* s, const int32_t* tokens, int n, int pos0, const int32_t* want, int n_want,
                         float* host_logits, float* host_layers) {
  Model* M = m->hy;
  State* S = s->hy;
  const dsk_hybrid_config& c = M->c;
  if (n <= 0) return fail(-4, "empty chunk");
  if (pos0 == 0) { if (state_reset(s)) return -2; }
  else if (pos0 != S->next_pos) return fail(-4, "chunk starts at position %d but the state's sequence is at %d (recurrent state cannot be rewound; position 0 starts a new sequence)", pos0, S->next_pos);
  for (int i = 0; i < n; i++) if (tokens[i] < 0 || tokens[i] >= c.vocab_size) return fail(-4, "token %d out of range", tokens[i]);
  for (int i = 0; i < n_want; i++) if (want[i] < 0 || want[i] >= n || (i && want[i] <= want[i - 1])) return fail(-4, "wanted rows must be ascending indices into the chunk");
  for (const HLayer& L : M->L)   // a ring cache shortened to max_seq_len holds no position beyond it
    if (L.owner >= 0 && M->L[L.owner].ring < L.sp.att_window - 1 + S->chunk && pos0 + n > M->L[L.owner].ring)
      return fail(-4, "position %d does not fit the attention cache (max_seq_len %d)", pos0 + n - 1, c.max_seq_len);
  float* d_trace = nullptr;
  int wi = 0;
  for (int o = 0; o < n; o += S->chunk) {
    const int T = std::min(S->chunk, n - o);
    CK(cudaStreamSynchronize(s->stream));   // the pinned staging buffers are reused
    memcpy(S->h_tok, tokens + o, (size_t)T * 4);
    int nw = 0;
    while (wi + nw < n_want && want[wi + nw] < o + T) { S->h_want[nw] = want[wi + nw] - o; nw++; }
    CK(cudaMemcpyAsync(S->d_tok, S->h_tok, (size_t)T * 4, cudaMemcpyHostToDevice, s->stream));
    if (nw) CK(cudaMemcpyAsync(S->d_want, S->h_want, (size_t)nw * 4, cudaMemcpyHostToDevice, s->stream));
    set_ctl<<<1, 1, 0, s->stream>>>(S->d_ctl, pos0 + o);
    if (host_layers) { CK(cudaMalloc((void**)&d_trace, M->runs.size() * (size_t)T * c.dim * 4)); }
    if (enqueue_chunk(m, s, T, nw, d_trace, s->stream, pos0 + o)) { if (d_trace) cudaFree(d_trace); return -2; }
    for (int g0 = 0; g0 < nw; g0 += S->head_rows) {   // the LM head in groups of head_rows wanted rows
      const int gn = std::min(S->head_rows, nw - g0);
      if (g0 > 0) enqueue_head(m, s, g0, gn, s->stream);
      if (host_logits) CK(cudaMemcpyAsync(host_logits + (size_t)(wi + g0) * c.vocab_size, S->logits, (size_t)gn * c.vocab_size * 4, cudaMemcpyDeviceToHost, s->stream));
    }
    if (nw) {   // the last wanted row stays in the state for the samplers
      CK(cudaMemcpyAsync(s->logits, S->logits + (size_t)((nw - 1) % S->head_rows) * c.vocab_size, (size_t)c.vocab_size * 4, cudaMemcpyDeviceToDevice, s->stream));
      argmax_row<<<1, 1024, 0, s->stream>>>(s->logits, c.vocab_size, s->ctrl, nullptr, nullptr, 0);
    }
    timeline_report(S, T);
    if (host_layers) {
      CK(cudaStreamSynchronize(s->stream));
      for (size_t l = 0; l < M->runs.size(); l++)
        CK(cudaMemcpy(host_layers + ((size_t)l * n + o) * c.dim, d_trace + (size_t)l * T * c.dim, (size_t)T * c.dim * 4, cudaMemcpyDeviceToHost));
      cudaFree(d_trace); d_trace = nullptr;
    }
    wi += nw;
  }
  CK(cudaStreamSynchronize(s->stream));
  CK(cudaGetLastError());
  S->next_pos = pos0 + n;
  s->last_pos = pos0 + n - 1;
  s->have_logits = n_want > 0 && want[n_want - 1] == n - 1;
  return 0;
}

// greedy loop on the device: arg-max of the logits in the state -> next token -> one-token chunk -> logits, n_steps times,
// without a host round trip.  The step is captured once per state as a CUDA graph (positions advance in device memory).
static int decode_greedy(dsk_model* m, dsk_state* s, int start_pos, int n_steps, int32_t* out_tokens, float* elapsed_ms) {
  Model* M = m->hy;
  State* S = s->hy;
  const dsk_hybrid_config& c = M->c;
  if (start_pos != S->next_pos) return fail(-4, "dsk_decode_greedy: start_pos %d must follow the state's sequence (at %d)", start_pos, S->next_pos);
  const int one = 0;
  CK(cudaMemcpyAsync(S->d_want, &one, 4, cudaMemcpyHostToDevice, s->stream));
  set_ctl<<<1, 1, 0, s->stream>>>(S->d_ctl, start_pos);
  CK(cudaMemsetAsync(s->step, 0, sizeof(int), s->stream));
  CK(cudaStreamSynchronize(s->stream));
  if (!S->step_graph) {
    cudaGraph_t g = nullptr;
    CK(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    greedy_feed<<<1, 1, 0, s->stream>>>(s->ctrl, S->d_tok, s->token_log, s->step);
    int rc = enqueue_chunk(m, s, 1, 1, nullptr, s->stream);
    cudaMemcpyAsync(s->logits, S->logits, (size_t)c.vocab_size * 4, cudaMemcpyDeviceToDevice, s->stream);
    argmax_row<<<1, 1024, 0, s->stream>>>(s->logits, c.vocab_size, s->ctrl, nullptr, nullptr, 0);
    advance_ctl<<<1, 1, 0, s->stream>>>(S->d_ctl, 1);
    cudaError_t e = cudaStreamEndCapture(s->stream, &g);
    if (rc || e != cudaSuccess) return fail(-2, "capturing the decode step failed: %s", cudaGetErrorString(e));
    CK(cudaGraphInstantiate(&S->step_graph, g, 0));
    cudaGraphDestroy(g);
  }
  CK(cudaEventRecord(s->ev0, s->stream));
  for (int i = 0; i < n_steps; i++) CK(cudaGraphLaunch(S->step_graph, s->stream));
  CK(cudaEventRecord(s->ev1, s->stream));
  CK(cudaStreamSynchronize(s->stream));
  if (elapsed_ms) CK(cudaEventElapsedTime(elapsed_ms, s->ev0, s->ev1));
  if (out_tokens) CK(cudaMemcpy(out_tokens, s->token_log, (size_t)n_steps * 4, cudaMemcpyDeviceToHost));
  S->next_pos = start_pos + n_steps;
  s->last_pos = S->next_pos - 1;
  s->have_logits = true;
  return 0;
}

}  // namespace hyb
