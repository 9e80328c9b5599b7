// zudatar_model.cu — the Zudatar architecture on the runner's model interface (model.hpp).
//
// Zudatar is a decoder-only model on an f32 residual stream with an RMS norm before AND after every sublayer,
//     x <- x + rms(mixer(rms(x) w1)) w1b;   x <- x + rms(ff(rms(x) w2)) w2b        (a layer may have no feed-forward),
// an embedding that adds a hashed bigram row (previous token, current token) to the scaled token row, and a tied output head
// (logits = E rms(x) w * logit_scale).  Three kinds of mixer, in any order:
//   "attention"         grouped-query softmax attention in a sliding window (capped_attn.cu): biased q and k, the VALUES are
//                       the keys as projected; rotary on neighbouring pairs of the first rot.dims values of q and k, then a
//                       weightless RMS norm per head; one sigmoid gate per head on the output; keys and values in the paged cache;
//   "latent_attention"  latent attention without positions in a sliding window (latent_attn.cu): queries through an RMS-normed
//                       latent, keys and values linear maps of ONE cached RMS-normed latent per token (the key map is folded
//                       into the query, the value map applied after the softmax); a learned sink per head in the softmax
//                       denominator; one sigmoid gate per head; a layer may read the latents another layer cached (`kv_from`);
//   "channel_delta"     the gated delta rule with a decay per key channel (recurrence.cu): q, k, v through a short causal
//                       convolution + SiLU, q and k made unit vectors, beta = sigmoid, decay and output gate through two-step
//                       (low-rank) projections; per-head RMS norm with a shared weight and a sigmoid gate.  Its state matrices
//                       and the convolution's last inputs live in per-sequence state slots that the scheduler hands out, as
//                       does the previous token of the bigram embedding.
// Feed-forward: dense SiLU-gated.  Every size, constant and the layer order come from the configuration; the inner size of
// the two-step projections comes from the tensors' shapes.
//
// configuration keys read here: architecture, vocab, width, norm.eps, logit_scale, embedding.scale,
// embedding.bigram.{buckets,mul_prev,mul_cur}, layers[i].type, layers[i].mixer (attention: heads, kv_heads, dim, vdim,
// scale, mask.size, rot.{base,dims}; latent_attention: heads, dim, vdim, q_rank, kv_rank, scale, mask.size, kv_from;
// channel_delta: heads, kv_heads, dim, vdim, conv, low_rank (synthetic weights only)), layers[i].mlp (null | kind "dense", ff).
// tensors: embed, bigram, final.norm, l<i>.norm{1,1b,2,2b}, l<i>.mix.{q,k,g,o}, l<i>.mix.{q,k}.b (attention);
// l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o} (latent); l<i>.mix.{q,k,v}{,.conv}, l<i>.mix.{b,A_log,norm,a1,a2,
// dt_bias,g1,g2,o} (delta); l<i>.mlp.{gate,up,down}.
#include <algorithm>
#include <cmath>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../common.cuh"
#include "model.hpp"

namespace nvllm {
namespace {

#define RUN(expr)                   \
  do {                              \
    int _rc = (expr);               \
    if (_rc != 0) return _rc;       \
  } while (0)

inline int pad8(int n) { return (n + 7) / 8 * 8; }

enum MixKind { kAttention = 0, kLatent = 1, kDelta = 2 };

struct Layer {
  int mix = kAttention;
  bool has_mlp = false;
  int H = 0, G = 0, D = 0, V = 0, window = 0;
  float scale = 1.f;
  // attention
  int rot_dims = 0;
  double rot_base = 10000.0;
  const float* rope = nullptr;
  // latent attention
  int q_rank = 0, kv_rank = 0, kv_from = -1;
  // delta rule
  int taps = 1, ra = 0, rg = 0, low_rank_cfg = 0;   // ra / rg: inner sizes of the decay and gate projections (from the tensors)
  // feed-forward
  int ff = 0;
  // weights: projections in the operand type (bf16 | f32), vectors f32
  float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr;
  void *in = nullptr, *o = nullptr;              // packed input projection, output projection
  float *qb = nullptr, *kb = nullptr;            // attention biases
  float *dq_norm = nullptr, *dkv_norm = nullptr, *sink = nullptr;
  void *uq = nullptr, *ukT = nullptr, *uv = nullptr;   // ukT: per head [kv_rank, dim]
  void* ukv = nullptr;                                 // [uk | uv] as stored, [H * (dim + vdim), kv_rank]: keys and values of whole prompts
  float *conv_w = nullptr, *a_log = nullptr, *dt_bias = nullptr, *o_norm = nullptr;
  void *a1 = nullptr, *g1 = nullptr, *lr = nullptr, *a2 = nullptr, *g2 = nullptr;   // lr: [a1 | g1] packed once both are known
  void *gu = nullptr, *down = nullptr;
  // packed projection layouts (f32 output rows, padded to 8 columns)
  bool own_latent() const { return kv_from < 0; }
  int a_cols() const { return H * D + G * D + H; }                                  // [q | k | g]
  int l_cols() const { return q_rank + (own_latent() ? kv_rank : 0) + H; }          // [dq | dkv | g]
  int d_ch() const { return 2 * G * D + H * V; }                                    // convolved channels [q | k | v]
  int d_cols() const { return d_ch() + H; }                                         // [q | k | v | b]
  int lr_cols() const { return pad8(ra) + pad8(rg); }
  int cache_row() const { return pad8(kv_rank); }
};

struct LayerState {
  void *kc = nullptr, *vc = nullptr;          // attention cache
  void* lat = nullptr;                        // latent cache [rows, cache_row]
  float *S = nullptr, *conv = nullptr;        // [slots, H, D, V], [slots, taps - 1, channels]
};

class Zudatar : public ModelImpl {
 public:
  int vocab_ = 0, width_ = 0, buckets_ = 1, mul_prev_ = 0, mul_cur_ = 0;
  float eps_ = 1e-5f, embed_scale_ = 1.f, logit_scale_ = 1.f;
  std::vector<Layer> layers_;
  std::vector<LayerState> state_;
  int32_t* last_token_ = nullptr;             // [slots]: the token before the next one, for the bigram row
  ModelLimits lim_{};
  int dt_ = NVLLM_BF16;
  size_t esz_ = 2;
  void *embed_ = nullptr, *bigram_ = nullptr;
  float* final_norm_ = nullptr;
  std::map<std::pair<double, int>, float*> rope_tables_;
  // activations
  float *h_ = nullptr, *proj_ = nullptr, *q_abs_ = nullptr, *conv_out_ = nullptr, *decay_ = nullptr, *gate_ = nullptr, *y_ = nullptr;
  float* lat_ws_ = nullptr; size_t lat_ws_bytes_ = 0;   // partial softmaxes of single tokens whose keys are split over CTAs
  void *kv_ = nullptr, *c_dense_ = nullptr;   // whole prompts of a latent layer: the step's latents and their keys / values per head
  void *sub_out_ = nullptr;   // a sublayer's output in the operand type; its norm and the residual sum are f32
  void *normed_ = nullptr, *q_ = nullptr, *cq_ = nullptr, *o_lat_ = nullptr, *mix_in_ = nullptr, *lr_out_ = nullptr, *gu_buf_ = nullptr, *act_ = nullptr,
       *head_in_ = nullptr;
  int head_rows_ = 0;
  std::vector<void*> allocs_;
  std::set<std::string> needed_, loaded_;
  bool ready_ = false;

  ~Zudatar() override { for (void* p : allocs_) cudaFree(p); }
  int vocab() const override { return vocab_; }
  int hidden() const override { return width_; }
  int layer_runs() const override { return static_cast<int>(layers_.size()); }
  bool recurrent_state() const override { return true; }   // the previous token (bigram row) is per-sequence state in every model
  bool weights_ready() const override { return ready_; }

  int parse(const json::Value& c) {
    vocab_ = c["vocab"].need_int("vocab");
    width_ = c["width"].need_int("width");
    eps_ = static_cast<float>(c["norm"]["eps"].as_double(1e-5));
    logit_scale_ = static_cast<float>(c["logit_scale"].as_double(1.0));
    embed_scale_ = static_cast<float>(c["embedding"]["scale"].as_double(1.0));
    const json::Value& bg = c["embedding"]["bigram"];
    buckets_ = bg["buckets"].need_int("embedding.bigram.buckets");
    mul_prev_ = bg["mul_prev"].need_int("embedding.bigram.mul_prev");
    mul_cur_ = bg["mul_cur"].need_int("embedding.bigram.mul_cur");
    const json::Value& ls = c["layers"];
    NVLLM_CHECK_ARG(ls.is_array() && ls.size() > 0 && vocab_ > 0 && width_ > 0 && buckets_ > 0 && mul_prev_ >= 0 && mul_cur_ >= 0, NVLLM_ERR_ARG,
                    "Zudatar config: layers / vocab / width / bigram");
    for (size_t i = 0; i < ls.size(); ++i) {
      const json::Value& l = ls[i];
      Layer L;
      const std::string type = l["type"].as_string();
      const json::Value& m = l["mixer"];
      L.H = m["heads"].need_int("mixer.heads");
      L.D = m["dim"].need_int("mixer.dim");
      L.V = m["vdim"].as_int(L.D);
      NVLLM_CHECK_ARG(L.H > 0 && L.D > 0 && L.V > 0, NVLLM_ERR_ARG, "Zudatar config: layer %zu heads / dim / vdim", i);
      if (type == "attention") {
        L.mix = kAttention;
        L.G = m["kv_heads"].as_int(L.H);
        L.scale = static_cast<float>(m["scale"].need_double("mixer.scale"));
        L.window = m["mask"]["size"].as_int(0);
        L.rot_dims = m["rot"]["dims"].as_int(0);
        L.rot_base = m["rot"]["base"].as_double(10000.0);
        NVLLM_CHECK_ARG(L.G > 0 && L.H % L.G == 0 && L.V == L.D && L.V <= 512 && L.window >= 0 && L.rot_dims >= 0 && L.rot_dims % 2 == 0 &&
                            L.rot_dims <= L.D && L.rot_base > 0, NVLLM_ERR_ARG,
                        "Zudatar config: layer %zu attention (heads %d / %d, dim %d = vdim %d <= 512: the values are the keys; rot dims %d even)", i,
                        L.H, L.G, L.D, L.V, L.rot_dims);
      } else if (type == "latent_attention") {
        L.mix = kLatent;
        L.G = 1;
        L.scale = static_cast<float>(m["scale"].need_double("mixer.scale"));
        L.window = m["mask"]["size"].as_int(0);
        L.q_rank = m["q_rank"].need_int("mixer.q_rank");
        L.kv_rank = m["kv_rank"].need_int("mixer.kv_rank");
        L.kv_from = m["kv_from"].is_null() ? -1 : m["kv_from"].as_int(-1);
        NVLLM_CHECK_ARG(L.q_rank > 0 && L.kv_rank > 0 && L.kv_rank <= 1024 && L.window >= 0, NVLLM_ERR_ARG,
                        "Zudatar config: layer %zu latent attention (q_rank %d, kv_rank %d <= 1024)", i, L.q_rank, L.kv_rank);
        if (L.kv_from >= 0) {
          NVLLM_CHECK_ARG(L.kv_from < static_cast<int>(i) && layers_[L.kv_from].mix == kLatent && layers_[L.kv_from].own_latent() &&
                              layers_[L.kv_from].kv_rank == L.kv_rank, NVLLM_ERR_ARG,
                          "Zudatar config: layer %zu reads the latents of layer %d, which must be an earlier latent_attention layer with "
                          "latents of its own and the same kv_rank", i, L.kv_from);
        }
      } else if (type == "channel_delta") {
        L.mix = kDelta;
        L.G = m["kv_heads"].as_int(L.H);
        L.taps = m["conv"].as_int(1);
        L.low_rank_cfg = m["low_rank"].as_int(0);
        NVLLM_CHECK_ARG(L.G > 0 && L.H % L.G == 0 && L.D <= 512 && L.taps >= 1 && L.taps <= 16, NVLLM_ERR_ARG,
                        "Zudatar config: layer %zu delta rule (heads %d / %d, dim %d <= 512, conv %d <= 16)", i, L.H, L.G, L.D, L.taps);
      } else {
        NVLLM_CHECK_ARG(false, NVLLM_ERR_ARG, "Zudatar config: layer %zu has mixer type '%s' (known: attention, latent_attention, channel_delta)", i,
                        type.c_str());
      }
      const json::Value& f = l["mlp"];
      if (!f.is_null()) {
        const std::string kind = f["kind"].as_string("dense");
        NVLLM_CHECK_ARG(kind == "dense", NVLLM_ERR_ARG, "Zudatar config: layer %zu feed-forward kind '%s' (known: dense)", i, kind.c_str());
        L.has_mlp = true;
        L.ff = f["ff"].need_int("mlp.ff");
        NVLLM_CHECK_ARG(L.ff > 0, NVLLM_ERR_ARG, "Zudatar config: layer %zu feed-forward size", i);
      }
      layers_.push_back(L);
    }
    return 0;
  }

  template <typename T>
  int dalloc(T** p, size_t count, size_t elt = sizeof(T), bool zero = false) {
    void* q = nullptr;
    const size_t bytes = (count * elt + 255) & ~static_cast<size_t>(255);
    cudaError_t e = cudaMalloc(&q, bytes ? bytes : 256);
    if (e != cudaSuccess) { set_error("cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e)); return static_cast<int>(e); }
    allocs_.push_back(q);
    if (zero) cudaMemset(q, 0, bytes ? bytes : 256);
    *p = static_cast<T*>(q);
    return 0;
  }
  int oalloc(void** p, size_t count, bool zero = false) { return dalloc(p, count, esz_, zero); }  // operand-typed buffer
  int valloc(float** p, size_t count, const std::string& name) { needed_.insert(name); return dalloc(p, count); }

  int create(const ModelLimits& lim, cudaStream_t stream) override {
    lim_ = lim;
    dt_ = lim.dtype;
    esz_ = dt_ == NVLLM_F32 ? 4 : 2;
    const size_t W = width_, T = lim.max_tokens, S = lim.max_seqs;
    RUN(oalloc(&embed_, static_cast<size_t>(vocab_) * W)); needed_.insert("embed");
    RUN(oalloc(&bigram_, static_cast<size_t>(buckets_ + 1) * W)); needed_.insert("bigram");
    RUN(valloc(&final_norm_, W, "final.norm"));
    RUN(dalloc(&last_token_, S, sizeof(int32_t), true));
    size_t m_kv = 0, m_cd = 0;
    size_t m_proj = 8, m_q = 8, m_cq = 8, m_lat = 8, m_mix = 8, m_ch = 1, m_hd = 1, m_hv = 1, m_ff = 0;
    state_.resize(layers_.size());
    const size_t rows = static_cast<size_t>(lim.num_blocks) * lim.block_size;
    for (size_t i = 0; i < layers_.size(); ++i) {
      Layer& L = layers_[i];
      LayerState& st = state_[i];
      const std::string p = "l" + std::to_string(i) + ".", a = p + "mix.";
      RUN(valloc(&L.norm1, W, p + "norm1")); RUN(valloc(&L.norm1b, W, p + "norm1b"));
      const size_t HV = static_cast<size_t>(L.H) * L.V, HD = static_cast<size_t>(L.H) * L.D;
      RUN(oalloc(&L.o, W * HV)); needed_.insert(a + "o");
      m_mix = std::max(m_mix, HV);
      if (L.mix == kAttention) {
        RUN(oalloc(&L.in, static_cast<size_t>(pad8(L.a_cols())) * W, true));
        for (const char* t : {"q", "k", "g"}) needed_.insert(a + t);
        RUN(valloc(&L.qb, HD, a + "q.b")); RUN(valloc(&L.kb, static_cast<size_t>(L.G) * L.D, a + "k.b"));
        if (L.rot_dims > 0) {  // rotary table shared by the layers that agree on (base, dims)
          const auto key = std::make_pair(L.rot_base, L.rot_dims);
          auto it = rope_tables_.find(key);
          if (it == rope_tables_.end()) {
            float* tab = nullptr;
            RUN(dalloc(&tab, static_cast<size_t>(lim.max_positions) * L.rot_dims));
            RUN(nvllm_rope_table_interleaved(tab, lim.max_positions, L.rot_dims, L.rot_base, stream));
            it = rope_tables_.emplace(key, tab).first;
          }
          L.rope = it->second;
        }
        RUN(oalloc(&st.kc, rows * L.G * L.D, true)); RUN(oalloc(&st.vc, rows * L.G * L.V, true));
        m_proj = std::max<size_t>(m_proj, pad8(L.a_cols()));
        m_q = std::max(m_q, HD);
      } else if (L.mix == kLatent) {
        RUN(oalloc(&L.in, static_cast<size_t>(pad8(L.l_cols())) * W, true));
        needed_.insert(a + "dq"); needed_.insert(a + "g");
        RUN(valloc(&L.dq_norm, L.q_rank, a + "dq.norm"));
        RUN(oalloc(&L.uq, HD * L.q_rank)); needed_.insert(a + "uq");
        RUN(oalloc(&L.ukT, HD * L.kv_rank)); needed_.insert(a + "uk");
        RUN(oalloc(&L.uv, HV * L.kv_rank)); needed_.insert(a + "uv");
        RUN(oalloc(&L.ukv, (HD + HV) * L.kv_rank));
        m_kv = std::max(m_kv, HD + HV); m_cd = std::max<size_t>(m_cd, L.cache_row());
        RUN(valloc(&L.sink, L.H, a + "sink"));
        if (L.own_latent()) {
          needed_.insert(a + "dkv");
          RUN(valloc(&L.dkv_norm, L.kv_rank, a + "dkv.norm"));
          RUN(oalloc(&st.lat, rows * L.cache_row(), true));
        }
        m_proj = std::max<size_t>(m_proj, pad8(L.l_cols()));
        m_q = std::max(m_q, HD);
        m_cq = std::max<size_t>(m_cq, L.q_rank);
        m_lat = std::max(m_lat, static_cast<size_t>(L.H) * L.kv_rank);
      } else {
        RUN(oalloc(&L.in, static_cast<size_t>(pad8(L.d_cols())) * W, true));
        for (const char* t : {"q", "k", "v", "b", "a1", "a2", "g1", "g2"}) needed_.insert(a + t);
        RUN(dalloc(&L.conv_w, static_cast<size_t>(L.d_ch()) * L.taps));
        for (const char* t : {"q.conv", "k.conv", "v.conv"}) needed_.insert(a + t);
        RUN(valloc(&L.a_log, L.H, a + "A_log")); RUN(valloc(&L.dt_bias, HD, a + "dt_bias")); RUN(valloc(&L.o_norm, L.V, a + "norm"));
        RUN(dalloc(&st.S, S * HD * L.V, sizeof(float), true));
        RUN(dalloc(&st.conv, S * std::max(1, L.taps - 1) * L.d_ch(), sizeof(float), true));
        m_proj = std::max<size_t>(m_proj, pad8(L.d_cols()));
        m_ch = std::max<size_t>(m_ch, L.d_ch()); m_hd = std::max(m_hd, HD); m_hv = std::max(m_hv, HV);
      }
      if (L.has_mlp) {
        RUN(valloc(&L.norm2, W, p + "norm2")); RUN(valloc(&L.norm2b, W, p + "norm2b"));
        RUN(oalloc(&L.gu, static_cast<size_t>(2) * L.ff * W)); RUN(oalloc(&L.down, W * L.ff));
        for (const char* t : {"gate", "up", "down"}) needed_.insert(p + "mlp." + t);
        m_ff = std::max<size_t>(m_ff, L.ff);
      }
    }
    RUN(dalloc(&h_, T * W)); RUN(oalloc(&normed_, T * W)); RUN(dalloc(&proj_, T * m_proj)); RUN(oalloc(&sub_out_, T * W));
    RUN(oalloc(&q_, T * m_q)); RUN(oalloc(&cq_, T * m_cq)); RUN(dalloc(&q_abs_, T * m_lat)); RUN(oalloc(&o_lat_, T * m_lat));
    RUN(oalloc(&mix_in_, T * m_mix)); RUN(dalloc(&conv_out_, T * m_ch)); RUN(dalloc(&decay_, T * m_hd)); RUN(dalloc(&gate_, T * m_hv));
    RUN(dalloc(&y_, T * m_hv));
    if (m_ff > 0) { RUN(oalloc(&gu_buf_, T * 2 * m_ff)); RUN(oalloc(&act_, T * m_ff)); }
    if (m_kv > 0) {
      RUN(oalloc(&kv_, T * m_kv)); RUN(oalloc(&c_dense_, T * m_cd, true));
      lat_ws_bytes_ = std::min<size_t>(T, 256) * 4 * (m_lat + 2 * 64) * sizeof(float);   // (tokens <= 256) x heads x 4 splits x (kv_rank + 2)
      RUN(dalloc(&lat_ws_, lat_ws_bytes_ / sizeof(float)));
    }
    NVLLM_CUDA(cudaStreamSynchronize(stream));
    return 0;
  }

  // ---- weights ---------------------------------------------------------------------------------------------------
  static float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
  }
  // host bf16 [rows, cols] -> device operand tensor at ELEMENT offset `off`
  int put(void* dst, size_t off, const uint16_t* src, int64_t rows, int64_t cols, cudaStream_t st) {
    const size_t n = static_cast<size_t>(rows) * cols;
    const void* from = src;
    std::vector<float> tmp;
    if (esz_ == 4) {
      tmp.resize(n);
      for (size_t i = 0; i < n; ++i) tmp[i] = bf16_bits_to_f32(src[i]);
      from = tmp.data();
    }
    NVLLM_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(dst) + off * esz_, from, n * esz_, cudaMemcpyHostToDevice, st));
    NVLLM_CUDA(cudaStreamSynchronize(st));
    return 0;
  }
  int putf(float* dst, const uint16_t* src, int64_t n, float scale, cudaStream_t st) {
    std::vector<float> tmp(n);
    for (int64_t i = 0; i < n; ++i) tmp[i] = bf16_bits_to_f32(src[i]) * scale;
    NVLLM_CUDA(cudaMemcpyAsync(dst, tmp.data(), n * 4, cudaMemcpyHostToDevice, st));
    NVLLM_CUDA(cudaStreamSynchronize(st));
    return 0;
  }

  // The tensor's shape and where it goes.  kind: 0 operand matrix at (dst, element offset); 1 f32 vector; 2 the key map of a
  // latent layer (stored per head transposed); 3 a two-step projection, whose inner size the tensor itself decides (rows < 0
  // or cols < 0: taken from the tensor); 4 a convolution's taps, written into the packed [channels, taps] table at row `off`.
  struct Target { int kind = -1; void* dst = nullptr; size_t off = 0; int64_t rows = 0, cols = 0; float scale = 1.f; };
  Target target_of(const std::string& name) const {
    const int64_t W = width_;
    Target t;
    auto mat = [&](void* d, size_t off, int64_t r, int64_t c) { t.kind = 0; t.dst = d; t.off = off; t.rows = r; t.cols = c; return t; };
    auto vec = [&](float* d, int64_t n) { t.kind = 1; t.dst = d; t.rows = 1; t.cols = n; return t; };
    if (name == "embed") return mat(embed_, 0, vocab_, W);
    if (name == "bigram") return mat(bigram_, 0, buckets_ + 1, W);
    if (name == "final.norm") { t = vec(final_norm_, W); t.scale = logit_scale_; return t; }   // the logits' scale rides in the last norm's weight
    if (name.size() < 4 || name[0] != 'l') return t;
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return t;
    const int li = atoi(name.substr(1, dot - 1).c_str());
    if (li < 0 || li >= static_cast<int>(layers_.size())) return t;
    const Layer& L = layers_[li];
    const std::string rest = name.substr(dot + 1);
    const int64_t HD = static_cast<int64_t>(L.H) * L.D, HV = static_cast<int64_t>(L.H) * L.V, GD = static_cast<int64_t>(L.G) * L.D;
    if (rest == "norm1") return vec(L.norm1, W);
    if (rest == "norm1b") return vec(L.norm1b, W);
    if (rest == "norm2") return vec(L.norm2, W);
    if (rest == "norm2b") return vec(L.norm2b, W);
    if (rest == "mix.o") return mat(L.o, 0, W, HV);
    if (L.mix == kAttention) {
      if (rest == "mix.q") return mat(L.in, 0, HD, W);
      if (rest == "mix.k") return mat(L.in, HD * W, GD, W);
      if (rest == "mix.g") return mat(L.in, (HD + GD) * W, L.H, W);
      if (rest == "mix.q.b") return vec(L.qb, HD);
      if (rest == "mix.k.b") return vec(L.kb, GD);
    } else if (L.mix == kLatent) {
      const int64_t own = L.own_latent() ? L.kv_rank : 0;
      if (rest == "mix.dq") return mat(L.in, 0, L.q_rank, W);
      if (rest == "mix.dkv") return mat(L.in, static_cast<int64_t>(L.q_rank) * W, L.kv_rank, W);
      if (rest == "mix.g") return mat(L.in, (L.q_rank + own) * W, L.H, W);
      if (rest == "mix.dq.norm") return vec(L.dq_norm, L.q_rank);
      if (rest == "mix.dkv.norm") return vec(L.dkv_norm, L.kv_rank);
      if (rest == "mix.uq") return mat(L.uq, 0, HD, L.q_rank);
      if (rest == "mix.uk") { t = mat(L.ukT, 0, HD, L.kv_rank); t.kind = 2; return t; }
      if (rest == "mix.uv") return mat(L.uv, 0, HV, L.kv_rank);
      if (rest == "mix.sink") return vec(L.sink, L.H);
    } else {
      if (rest == "mix.q") return mat(L.in, 0, GD, W);
      if (rest == "mix.k") return mat(L.in, GD * W, GD, W);
      if (rest == "mix.v") return mat(L.in, 2 * GD * W, HV, W);
      if (rest == "mix.b") return mat(L.in, (2 * GD + HV) * W, L.H, W);
      if (rest == "mix.q.conv") { t.kind = 4; t.dst = L.conv_w; t.off = 0; t.rows = GD; t.cols = L.taps; return t; }
      if (rest == "mix.k.conv") { t.kind = 4; t.dst = L.conv_w; t.off = GD; t.rows = GD; t.cols = L.taps; return t; }
      if (rest == "mix.v.conv") { t.kind = 4; t.dst = L.conv_w; t.off = 2 * GD; t.rows = HV; t.cols = L.taps; return t; }
      if (rest == "mix.A_log") return vec(L.a_log, L.H);
      if (rest == "mix.dt_bias") return vec(L.dt_bias, HD);
      if (rest == "mix.norm") return vec(L.o_norm, L.V);
      if (rest == "mix.a1") { t.kind = 3; t.off = 0; t.rows = -1; t.cols = W; return t; }
      if (rest == "mix.g1") { t.kind = 3; t.off = 1; t.rows = -1; t.cols = W; return t; }
      if (rest == "mix.a2") { t.kind = 3; t.off = 2; t.rows = HD; t.cols = -1; return t; }
      if (rest == "mix.g2") { t.kind = 3; t.off = 3; t.rows = HV; t.cols = -1; return t; }
    }
    if (L.has_mlp) {
      if (rest == "mlp.gate") return mat(L.gu, 0, L.ff, W);
      if (rest == "mlp.up") return mat(L.gu, static_cast<size_t>(L.ff) * W, L.ff, W);
      if (rest == "mlp.down") return mat(L.down, 0, W, L.ff);
    }
    return t;
  }

  // Operand matrices and f32 vectors arrive as bf16 bit patterns.
  int load_weight(const char* name_c, const void* src_v, int64_t rows, int64_t cols, cudaStream_t st) override {
    NVLLM_CHECK_ARG(name_c && src_v, NVLLM_ERR_ARG, "load_weight: NULL");
    const std::string name(name_c);
    NVLLM_CHECK_ARG(needed_.count(name), NVLLM_ERR_ARG, "load_weight: tensor '%s' is not part of this model", name_c);
    Target t = target_of(name);
    NVLLM_CHECK_ARG(t.kind >= 0, NVLLM_ERR_ARG, "load_weight: unknown tensor '%s'", name_c);
    const uint16_t* src = static_cast<const uint16_t*>(src_v);
    if (t.kind == 3) {  // a two-step projection: the tensor decides the inner size; both steps must agree
      Layer& L = layers_[atoi(name.substr(1).c_str())];
      const bool first = t.off < 2, decay = (t.off & 1) == 0;
      const int64_t inner = first ? rows : cols;
      NVLLM_CHECK_ARG(inner > 0 && (first ? cols == t.cols : rows == t.rows), NVLLM_ERR_ARG, "load_weight(%s): got [%lld, %lld]", name_c,
                      (long long)rows, (long long)cols);
      int& have = decay ? L.ra : L.rg;
      NVLLM_CHECK_ARG(have == 0 || have == inner, NVLLM_ERR_ARG, "load_weight(%s): inner size %lld, its other step has %d", name_c, (long long)inner, have);
      have = static_cast<int>(inner);
      void** dst = t.off == 0 ? &L.a1 : t.off == 1 ? &L.g1 : t.off == 2 ? &L.a2 : &L.g2;
      if (*dst == nullptr) RUN(oalloc(dst, static_cast<size_t>(rows) * cols));
      RUN(put(*dst, 0, src, rows, cols, st));
    } else {
      NVLLM_CHECK_ARG(rows * cols == t.rows * t.cols && (t.kind == 1 || (rows == t.rows && cols == t.cols)), NVLLM_ERR_ARG,
                      "load_weight(%s): expected [%lld, %lld], got [%lld, %lld]", name_c, (long long)t.rows, (long long)t.cols, (long long)rows,
                      (long long)cols);
      if (t.kind == 0) {
        RUN(put(t.dst, t.off, src, rows, cols, st));
        const Layer& L0 = name[0] == 'l' ? layers_[atoi(name.substr(1).c_str())] : layers_[0];
        if (name[0] == 'l' && L0.mix == kLatent && t.dst == L0.uv)   // the value map also sits below the key map
          RUN(put(L0.ukv, static_cast<size_t>(L0.H) * L0.D * L0.kv_rank, src, rows, cols, st));
      }
      else if (t.kind == 1) RUN(putf(static_cast<float*>(t.dst), src, rows * cols, t.scale, st));
      else if (t.kind == 4) RUN(putf(static_cast<float*>(t.dst) + t.off * cols, src, rows * cols, 1.f, st));
      else {  // key map [H * D, R] -> per head [R, D]: the query is folded through it, q_abs_h = Uk_h^T q_h
        const Layer& L = layers_[atoi(name.substr(1).c_str())];
        std::vector<uint16_t> tr(static_cast<size_t>(rows) * cols);
        for (int h = 0; h < L.H; ++h)
          for (int d = 0; d < L.D; ++d)
            for (int r = 0; r < L.kv_rank; ++r)
              tr[(static_cast<size_t>(h) * L.kv_rank + r) * L.D + d] = src[(static_cast<size_t>(h) * L.D + d) * L.kv_rank + r];
        RUN(put(t.dst, 0, tr.data(), rows, cols, st));
        RUN(put(L.ukv, 0, src, rows, cols, st));           // and as stored, above the value map
      }
    }
    loaded_.insert(name);
    if (loaded_.size() == needed_.size() && !ready_) RUN(finish_load(st));
    return 0;
  }

  // Once every tensor is there: pack the first steps of the delta layers' two-step projections side by side ([a1 | g1], each
  // padded to 8 rows) so that one product serves both, and size the buffer that holds their output.
  int finish_load(cudaStream_t st) {
    size_t m_lr = 0;
    for (Layer& L : layers_) {
      if (L.mix != kDelta) continue;
      const size_t W = width_;
      if (L.lr == nullptr) RUN(oalloc(&L.lr, static_cast<size_t>(L.lr_cols()) * W, true));
      NVLLM_CUDA(cudaMemcpyAsync(L.lr, L.a1, static_cast<size_t>(L.ra) * W * esz_, cudaMemcpyDeviceToDevice, st));
      NVLLM_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(L.lr) + static_cast<size_t>(pad8(L.ra)) * W * esz_, L.g1, static_cast<size_t>(L.rg) * W * esz_,
                                 cudaMemcpyDeviceToDevice, st));
      m_lr = std::max<size_t>(m_lr, L.lr_cols());
    }
    if (m_lr > 0 && lr_out_ == nullptr) RUN(oalloc(&lr_out_, static_cast<size_t>(lim_.max_tokens) * m_lr, true));
    NVLLM_CUDA(cudaStreamSynchronize(st));
    ready_ = true;
    return 0;
  }

  // Seeded synthetic weights (benchmarks, smoke runs): every needed tensor drawn on the host from a counter-based generator
  // and sent through load_weight, so that synthetic and checkpoint weights take the same path.
  int init_weights(uint64_t seed, float std, cudaStream_t st) override {
    auto mix = [](uint64_t x) {
      x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
      x ^= x >> 27; x *= 0x94D049BB133111EBull;
      x ^= x >> 31;
      return x;
    };
    auto to_bf16 = [](float f) {
      uint32_t u;
      memcpy(&u, &f, 4);
      return static_cast<uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
    };
    auto ends = [](const std::string& s, const char* suf) { const size_t n = strlen(suf); return s.size() >= n && s.compare(s.size() - n, n, suf) == 0; };
    std::vector<uint16_t> buf;
    uint64_t tid = 0;
    for (const std::string& name : needed_) {
      ++tid;
      Target t = target_of(name);
      NVLLM_CHECK_ARG(t.kind >= 0, NVLLM_ERR_STATE, "init_weights: no target for '%s'", name.c_str());
      if (t.kind == 3) {  // inner size of a two-step projection: the configuration's `low_rank`, else an eighth of the width
        const Layer& L = layers_[atoi(name.substr(1).c_str())];
        const int r = L.low_rank_cfg > 0 ? L.low_rank_cfg : std::max(8, pad8(width_ / 8));
        if (t.rows < 0) t.rows = r;
        if (t.cols < 0) t.cols = r;
      }
      buf.resize(static_cast<size_t>(t.rows) * t.cols);
      const bool norm_w = name.find("norm") != std::string::npos, is_alog = ends(name, ".A_log"), is_dtb = ends(name, ".dt_bias");
      const bool is_conv = ends(name, ".conv"), is_table = name == "embed" || name == "bigram";
      for (size_t i = 0; i < buf.size(); ++i) {
        const uint64_t hsh = mix(seed ^ (tid << 40) ^ (i + 1) * 0x9E3779B97F4A7C15ull);
        const int s = static_cast<int>((hsh & 0xffff) + ((hsh >> 16) & 0xffff) + ((hsh >> 32) & 0xffff) + (hsh >> 48)) - 131070;
        const float g = static_cast<float>(s) * 2.6428998e-05f;  // ~N(0, 1)
        float v = g * std;
        if (norm_w) v = 1.0f + 0.1f * g;
        else if (is_alog) v = -1.0f + 0.5f * g;
        else if (is_dtb) v = -1.0f + 0.5f * g;
        else if (is_conv) v = 0.5f * g;
        else if (is_table) v = 0.5f * g;
        buf[i] = to_bf16(v);
      }
      RUN(load_weight(name.c_str(), buf.data(), t.rows, t.cols, st));
    }
    return 0;
  }

  // ---- forward ---------------------------------------------------------------------------------------------------
  int forward(const StepView& v) override {
    void* st = v.stream;
    const int N = v.n_tokens, W = width_, S = v.n_seqs;
    launches = 0;
    NVLLM_CHECK_ARG(ready_, NVLLM_ERR_STATE, "Zudatar forward: weights are not loaded");
    NVLLM_CHECK_ARG(v.cu_tokens && v.seq_slots && v.tables, NVLLM_ERR_ARG, "Zudatar forward: the step carries no token ranges / state slots / block tables");
    auto mk = [&](const char* name) { if (v.mark) v.mark(v.mark_ctx, name); };
    auto lin = [&](void* y, const void* x, const void* w, int n, int k, int64_t ldx, int64_t ldy, int out_dt, const char* name) {
      ++launches;
      const int rc = nvllm_linear(y, x, w, N, n, k, ldx, k, ldy, 1, 0, 0, 0, dt_, out_dt, st);
      mk(name);
      return rc;
    };
    // h += rms(y) * post;  normed = rms(h) * pre
    auto norm = [&](const void* y, const float* post, const float* pre) {
      ++launches;
      const int rc = nvllm_rms_residual_norm(normed_, h_, y, dt_, post, pre, N, W, eps_, dt_, st);
      mk("rms_residual_norm");
      return rc;
    };
    auto off = [&](void* p, size_t elems) { return static_cast<void*>(static_cast<uint8_t*>(p) + elems * esz_); };
    RUN(nvllm_embedding_bigram(h_, embed_, bigram_, v.ids, v.positions, v.tok_seq, v.cu_tokens, v.seq_slots, last_token_, N, W, vocab_, buckets_,
                               mul_prev_, mul_cur_, embed_scale_, dt_, st)); ++launches; mk("embedding_bigram");
    RUN(norm(nullptr, nullptr, layers_[0].norm1));
    for (size_t i = 0; i < layers_.size(); ++i) {
      const Layer& L = layers_[i];
      const LayerState& ls = state_[i];
      const float* next = i + 1 < layers_.size() ? layers_[i + 1].norm1 : final_norm_;
      const int HD = L.H * L.D, HV = L.H * L.V, GD = L.G * L.D;
      if (L.mix == kAttention) {
        // [q | k | g] in one projection (f32 rows); biases, rotary, per-head norm and the cache store; windowed attention with
        // the head gate fused; Wo
        const int lda = pad8(L.a_cols());
        RUN(lin(proj_, normed_, L.in, lda, W, W, lda, NVLLM_F32, "attention q k g projection"));
        RUN(nvllm_attn_rope_norm_store(q_, HD, ls.kc, ls.vc, GD, GD, proj_, lda, L.qb, L.kb, nullptr, v.positions, L.rope, L.rot_dims,
                                       lim_.max_positions, eps_, v.slots, N, L.H, L.G, L.D, L.V, 1, dt_, st)); ++launches; mk("attn_rope_norm_store");
        RUN(nvllm_window_attention(mix_in_, HV, q_, HD, proj_ + HD + GD, lda, 1, ls.kc, ls.vc, GD, GD, v.tok_seq, v.positions, v.tables,
                                   v.table_cap, lim_.block_size, N, L.H, L.G, L.D, L.V, L.scale, 0.f, 0.f, 1, L.window, nullptr, v.cu_tokens, S,
                                   dt_, st)); ++launches; mk("window_attention");
      } else if (L.mix == kLatent) {
        // [dq | dkv | g] in one projection; both latents RMS-normed (the kv latent straight into its cache rows); q = Wuq cq;
        // the key map folded into the query per head; attention over the cached latents; the value map per head; Wo
        const int ldl = pad8(L.l_cols()), R = L.kv_rank, HR = L.H * R;
        const int own = L.own_latent() ? R : 0;
        void* cache = L.own_latent() ? ls.lat : state_[L.kv_from].lat;
        RUN(lin(proj_, normed_, L.in, ldl, W, W, ldl, NVLLM_F32, "latent dq dkv g projection"));
        RUN(nvllm_rms_norm_rows(cq_, L.q_rank, proj_, ldl, L.dq_norm, nullptr, N, L.q_rank, eps_, dt_, st)); ++launches; mk("rms_norm_rows (query latent)");
        if (own) {
          RUN(nvllm_rms_norm_rows(cache, L.cache_row(), proj_ + L.q_rank, ldl, L.dkv_norm, v.slots, N, R, eps_, dt_, st)); ++launches;
          mk("rms_norm_rows (kv latent -> cache)");
        }
        RUN(lin(q_, cq_, L.uq, HD, L.q_rank, L.q_rank, HD, dt_, "query up-projection"));
        // Whole prompts (every sequence starts at position 0, so all keys are the step's own tokens): keys and values per head
        // are computed from the step's latents and the layer runs as ordinary windowed attention over them — a fraction of the
        // folded form's work (a key costs dim + vdim multiply-adds per head instead of 2 kv_rank).  Portions and single tokens
        // take the folded form below, which reads nothing but the cached latents.
        const bool unfolded = v.whole_prompts && dt_ == NVLLM_BF16 && knobs().latent_unfold && N >= 256 && L.D % 8 == 0 && L.V % 8 == 0 &&
                              L.D <= 128 && L.V <= 128;
        // Per-head projections of the folded form: with many tokens every head is a tensor-core GEMM of its own; with few
        // (decoding) one batched launch of the mma.sync tile kernel beats `heads` launch latencies.
        const bool head_gemms = dt_ == NVLLM_BF16 && N >= 512 && L.D % 64 == 0 && R % 64 == 0 && L.V % 8 == 0 && HD % 8 == 0 && L.D % 8 == 0;
        if (unfolded) {
          const int row = L.cache_row(), kvn = HD + HV;
          if (own) {
            RUN(nvllm_rms_norm_rows(c_dense_, row, proj_ + L.q_rank, ldl, L.dkv_norm, nullptr, N, R, eps_, dt_, st)); ++launches; mk("rms_norm_rows (kv latent, dense)");
          } else {
            RUN(nvllm_gather_rows(c_dense_, cache, v.slots, N, row, lim_.num_blocks * lim_.block_size, dt_, st)); ++launches; mk("gather_rows (cached latents)");
          }
          RUN(lin(kv_, c_dense_, L.ukv, kvn, R, row, kvn, dt_, "key / value up-projection"));
          RUN(nvllm_window_attention(mix_in_, HV, q_, HD, proj_ + L.q_rank + own, ldl, 1, kv_, off(kv_, HD), kvn, kvn, v.tok_seq, v.positions, nullptr,
                                     v.table_cap, lim_.block_size, N, L.H, L.H, L.D, L.V, L.scale, 0.f, 0.f, 1, L.window, L.sink, v.cu_tokens, S, dt_, st));
          ++launches; mk("window_attention (latent layer, whole prompts)");
        } else {
          if (head_gemms) {
            for (int hh = 0; hh < L.H; ++hh) {
              RUN(nvllm_gemm_bf16(q_abs_ + static_cast<size_t>(hh) * R, off(q_, static_cast<size_t>(hh) * L.D), off(L.ukT, static_cast<size_t>(hh) * R * L.D),
                                  N, R, L.D, HD, L.D, HR, NVLLM_F32, nullptr, 0, st)); ++launches;
            }
            mk("q absorb (per-head GEMMs)");
          } else {
            RUN(nvllm_linear(q_abs_, q_, L.ukT, N, R, L.D, HD, L.D, HR, L.H, L.D, static_cast<int64_t>(R) * L.D, R, dt_, NVLLM_F32, st)); ++launches;
            mk("q absorb (per-head linear)");
          }
          RUN(nvllm_latent_window_attention(o_lat_, HR, q_abs_, HR, nullptr, 0, v.tok_seq, v.positions, v.tables, v.table_cap, lim_.block_size, cache,
                                            L.cache_row(), N, L.H, L.D, 0, R, L.scale, L.window, L.sink, proj_ + L.q_rank + own, ldl, lat_ws_, lat_ws_bytes_,
                                            dt_, st));
          ++launches; mk("latent_window_attention");
          if (head_gemms) {
            for (int hh = 0; hh < L.H; ++hh) {
              RUN(nvllm_gemm_bf16(off(mix_in_, static_cast<size_t>(hh) * L.V), off(o_lat_, static_cast<size_t>(hh) * R),
                                  off(L.uv, static_cast<size_t>(hh) * L.V * R), N, L.V, R, HR, R, HV, NVLLM_BF16, nullptr, 0, st)); ++launches;
            }
            mk("value up-projection (per-head GEMMs)");
          } else {
            RUN(nvllm_linear(mix_in_, o_lat_, L.uv, N, L.V, R, HR, R, HV, L.H, R, static_cast<int64_t>(L.V) * R, L.V, dt_, dt_, st)); ++launches;
            mk("value up-projection (per-head linear)");
          }
        }
      } else {
        // [q | k | v | b] in one projection (f32 rows) and the first steps [a1 | g1] in another; the second steps; the
        // convolution + SiLU over (q, k, v); unit vectors, beta, decay; the recurrence; gated per-head norm; Wo
        const int ldd = pad8(L.d_cols()), ch = L.d_ch(), ldlr = L.lr_cols();
        RUN(lin(proj_, normed_, L.in, ldd, W, W, ldd, NVLLM_F32, "delta q k v b projection"));
        RUN(lin(lr_out_, normed_, L.lr, ldlr, W, W, ldlr, dt_, "delta decay / gate first step"));
        RUN(lin(decay_, lr_out_, L.a2, HD, L.ra, ldlr, HD, NVLLM_F32, "delta decay second step"));
        RUN(lin(gate_, off(lr_out_, pad8(L.ra)), L.g2, HV, L.rg, ldlr, HV, NVLLM_F32, "delta gate second step"));
        RUN(nvllm_causal_conv(conv_out_, ch, proj_, ldd, L.conv_w, nullptr, ls.conv, v.tok_seq, v.seq_slots, v.cu_tokens, v.positions, N, S, ch,
                              L.taps, 1, st)); launches += L.taps > 1 ? 2 : 1; mk("causal_conv");
        RUN(nvllm_delta_prepare(conv_out_, ch, conv_out_ + GD, ch, proj_ + ch, ldd, decay_, HD, L.a_log, L.dt_bias, N, L.H, L.G, L.D,
                                1.0f / sqrtf(static_cast<float>(L.D)), 1e-6f, st)); ++launches; mk("delta_prepare");
        RUN(nvllm_gated_delta_recurrence(y_, HV, conv_out_, ch, conv_out_ + GD, ch, conv_out_ + 2 * GD, ch, decay_, HD, proj_ + ch, ldd, ls.S,
                                         v.seq_slots, v.cu_tokens, v.positions, S, L.H, L.G, L.D, L.V, st)); ++launches; mk("gated_delta_recurrence");
        RUN(nvllm_gated_group_norm_act(mix_in_, HV, y_, HV, gate_, HV, L.o_norm, 1, N, HV, L.H, eps_, 0, 1, dt_, st)); ++launches; mk("gated_group_norm");
      }
      RUN(lin(sub_out_, mix_in_, L.o, W, HV, HV, W, dt_, "mixer output projection"));
      if (L.has_mlp) {
        RUN(norm(sub_out_, L.norm1b, L.norm2));
        if (dt_ == NVLLM_BF16 && L.ff % 128 == 0 && W % 64 == 0) {  // SiLU gate in the GEMM's epilogue: [N, 2 ff] never reaches HBM
          RUN(nvllm_gemm_silu_mul_bf16(act_, normed_, L.gu, N, L.ff, W, W, W, L.ff, nullptr, 0, st)); ++launches; mk("gate_up projection + SiLU gate");
        } else {
          RUN(lin(gu_buf_, normed_, L.gu, 2 * L.ff, W, W, 2 * L.ff, dt_, "gate_up projection"));
          RUN(nvllm_ff_activation(act_, gu_buf_, N, L.ff, 0, dt_, st)); ++launches; mk("ff_activation (silu gate)");
        }
        RUN(lin(sub_out_, act_, L.down, W, L.ff, L.ff, W, dt_, "down projection"));
        RUN(norm(sub_out_, L.norm2b, next));
      } else {
        RUN(norm(sub_out_, L.norm1b, next));
      }
      if (v.layer_tap != nullptr && !v.capturing)
        NVLLM_CUDA(cudaMemcpyAsync(v.layer_tap + i * static_cast<size_t>(N) * W, h_, static_cast<size_t>(N) * W * 4, cudaMemcpyDeviceToHost,
                                   static_cast<cudaStream_t>(st)));
    }
    if (v.n_logit_rows > 0) {
      if (v.n_logit_rows > head_rows_) {
        NVLLM_CHECK_ARG(!v.capturing, NVLLM_ERR_STATE, "forward: logit rows grew inside a graph capture");
        NVLLM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(st)));
        head_rows_ = std::max(v.n_logit_rows, lim_.max_seqs);
        RUN(oalloc(&head_in_, static_cast<size_t>(head_rows_) * W));
      }
      RUN(nvllm_gather_rows(head_in_, normed_, v.logit_rows, v.n_logit_rows, W, N, dt_, st)); ++launches; mk("gather_rows");
      ++launches;
      RUN(nvllm_linear(v.logits, head_in_, embed_, v.n_logit_rows, vocab_, W, W, W, vocab_, 1, 0, 0, 0, dt_, NVLLM_F32, st));
      mk("head projection (tied embedding)");
    }
    return 0;
  }
};

}  // namespace

ModelImpl* make_zudatar(const json::Value& cfg) {
  Zudatar* m = new Zudatar();
  if (m->parse(cfg) != 0) { delete m; return nullptr; }
  return m;
}

}  // namespace nvllm
