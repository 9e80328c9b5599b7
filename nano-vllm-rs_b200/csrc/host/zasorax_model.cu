// zasorax_model.cu — the Zasorax architecture on the runner's model interface (model.hpp).
//
// Zasorax is a decoder-only model on an f32 residual stream whose blocks carry a norm on the sublayer's OUTPUT only,
//     x <- x + rms(mixer(x)) w1;   x <- x + rms(ff(x)) w2        (a layer may have no feed-forward),
// so every sublayer reads the stream itself (in the operand type).  Scaled embedding, a final RMS norm and an output head of
// its own.  Two kinds of mixer, in any order (both grouped-query softmax attention over the paged cache, capped_attn.cu):
//   "attention"    no rotation; queries and keys RMS-normed over the WHOLE projection (all heads at once, one weight per
//                  column); score = q.k * scale * temp_h + rel[bucket(i - j), h] with a learned table of distance buckets
//                  (one row per distance below half the table, logarithmic steps up to bias_max above); position i sees the
//                  j <= i of its own chunk (chunks of mask.size positions counted from the sequence's start); a learned sink
//                  per head joins the softmax denominator.  A layer with `kv_from: j` has no key / value tensors: it reads
//                  the cache rows layer j wrote, with queries, table, temperatures and sinks of its own.
//   "attention_2"  rotary on the first rot.dims values of every query and key head (value i paired with i + dims / 2), then a
//                  weightless RMS norm per head; the VALUES are rotated by their position over all of vdim before they are
//                  cached, and every head's output is turned back by the query's position; causal; softmax denominator
//                  1 + sum over the keys (a zero sink); one sigmoid gate per head.
// Feed-forward: dense, W_down xielu(W_up x) with two learned numbers; or a mixture of experts routed on the logits
// (z = W_r x + b in f32, the `top` largest, softmax over the chosen alone), experts SiLU-gated.
// Every size, constant and the layer order come from the configuration; the rows of a distance table come from its tensor.
//
// configuration keys read here: architecture, vocab, width, norm.eps, embedding.scale, layers[i].type, layers[i].mixer
// (heads, kv_heads, dim, vdim, scale; attention: mask.size, bias_max, kv_from, bias_rows (synthetic weights only);
// attention_2: rot.{base,dims}), layers[i].mlp (null | kind "dense", ff | kind "moe", expert.ff, router.{experts,top}).
// tensors: embed, head, final.norm, l<i>.norm{1,2}, l<i>.mix.{q,k,v,o}, l<i>.mix.{q.norm,k.norm,rel,temp,sink} (attention),
// l<i>.mix.g (attention_2), l<i>.mlp.{up,down,act} (dense), l<i>.mlp.{router,router.b}, l<i>.mlp.e<k>.{gate,up,down} (experts).
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

enum MixKind { kChunked = 0, kRotary = 1 };
enum FfKind { kNone = 0, kDense = 1, kExperts = 2 };

struct Layer {
  int mix = kChunked, ffk = kNone;
  int H = 0, G = 0, D = 0, V = 0;
  float scale = 1.f;
  // chunked attention with a distance bias
  int chunk = 0, bias_max = 0, bias_rows_cfg = 0, kv_from = -1;
  int dist_rows = 0;
  int rel_rows = 0;                     // rows of the table as stored (the tensor decides); dist: one row per distance
  float *qn = nullptr, *kn = nullptr, *temp = nullptr, *sink = nullptr, *dist = nullptr;
  // rotary attention
  int rot_dims = 0;
  double rot_base = 10000.0;
  const float *rope = nullptr, *vrope = nullptr;
  // feed-forward
  int ff = 0, experts = 0, top = 0, tile_rows = 32;
  float *norm1 = nullptr, *norm2 = nullptr, *act = nullptr, *router_b = nullptr;
  void *in = nullptr, *o = nullptr;                 // packed input projection [q | k | v (| g)], output projection
  void *up = nullptr, *down = nullptr;              // dense feed-forward
  void *router = nullptr, *egu = nullptr, *edown = nullptr;   // experts: [E][gate rows | up rows][W], [E][W][ff]
  bool own_kv() const { return kv_from < 0; }
  int q_cols() const { return H * D; }
  int k_cols() const { return own_kv() ? G * D : 0; }
  int v_cols() const { return own_kv() ? G * V : 0; }
  int in_cols() const { return q_cols() + k_cols() + v_cols() + (mix == kRotary ? H : 0); }
};

struct LayerCache { void *kc = nullptr, *vc = nullptr; };

class Zasorax : public ModelImpl {
 public:
  int vocab_ = 0, width_ = 0;
  float eps_ = 1e-5f, embed_scale_ = 1.f;
  std::vector<Layer> layers_;
  std::vector<LayerCache> cache_;
  ModelLimits lim_{};
  int dt_ = NVLLM_BF16;
  size_t esz_ = 2;
  void *embed_ = nullptr, *head_ = nullptr;
  float *final_norm_ = nullptr, *zero_sink_ = nullptr;
  std::map<std::pair<double, int>, float*> rope_tables_;
  // activations
  float *h_ = nullptr, *proj_ = nullptr, *route_ = nullptr, *topk_w_ = nullptr;
  int32_t *topk_idx_ = nullptr, *row_token_ = nullptr, *tile_expert_ = nullptr, *slot_row_ = nullptr;
  void *x_ = nullptr, *q_ = nullptr, *mix_in_ = nullptr, *sub_out_ = nullptr, *up_buf_ = nullptr, *act_ = nullptr, *xg_ = nullptr, *egu_buf_ = nullptr,
       *eout_ = nullptr, *head_in_ = nullptr;
  int head_rows_ = 0, max_rows_ = 0;
  std::vector<void*> allocs_;
  std::set<std::string> needed_, loaded_;
  bool ready_ = false;

  ~Zasorax() override { for (void* p : allocs_) cudaFree(p); }
  int vocab() const override { return vocab_; }
  int hidden() const override { return width_; }
  int layer_runs() const override { return static_cast<int>(layers_.size()); }
  bool weights_ready() const override { return ready_; }

  int parse(const json::Value& c) {
    vocab_ = c["vocab"].need_int("vocab");
    width_ = c["width"].need_int("width");
    eps_ = static_cast<float>(c["norm"]["eps"].as_double(1e-5));
    embed_scale_ = static_cast<float>(c["embedding"]["scale"].as_double(1.0));
    const json::Value& ls = c["layers"];
    NVLLM_CHECK_ARG(ls.is_array() && ls.size() > 0 && vocab_ > 0 && width_ > 0, NVLLM_ERR_ARG, "Zasorax config: layers / vocab / width");
    for (size_t i = 0; i < ls.size(); ++i) {
      const json::Value& l = ls[i];
      Layer L;
      const std::string type = l["type"].as_string();
      const json::Value& m = l["mixer"];
      L.H = m["heads"].need_int("mixer.heads");
      L.G = m["kv_heads"].as_int(L.H);
      L.D = m["dim"].need_int("mixer.dim");
      L.V = m["vdim"].as_int(L.D);
      L.scale = static_cast<float>(m["scale"].need_double("mixer.scale"));
      NVLLM_CHECK_ARG(L.H > 0 && L.G > 0 && L.H % L.G == 0 && L.D > 0 && L.V > 0 && L.V <= 512 && L.D <= 2048, NVLLM_ERR_ARG,
                      "Zasorax config: layer %zu heads %d / %d, dim %d, vdim %d (<= 512)", i, L.H, L.G, L.D, L.V);
      if (type == "attention") {
        L.mix = kChunked;
        L.chunk = m["mask"]["size"].as_int(0);
        L.bias_max = m["bias_max"].need_int("mixer.bias_max");
        L.bias_rows_cfg = m["bias_rows"].as_int(0);
        L.kv_from = m["kv_from"].is_null() ? -1 : m["kv_from"].as_int(-1);
        NVLLM_CHECK_ARG(L.chunk >= 0 && L.bias_max > 0, NVLLM_ERR_ARG, "Zasorax config: layer %zu mask.size %d, bias_max %d", i, L.chunk, L.bias_max);
        if (L.kv_from >= 0) {
          NVLLM_CHECK_ARG(L.kv_from < static_cast<int>(i) && layers_[L.kv_from].own_kv() && layers_[L.kv_from].G == L.G &&
                              layers_[L.kv_from].D == L.D && layers_[L.kv_from].V == L.V && layers_[L.kv_from].mix == L.mix, NVLLM_ERR_ARG,
                          "Zasorax config: layer %zu reads the keys and values of layer %d, which must be an earlier layer of the same kind with "
                          "keys of its own and the same kv_heads / dim / vdim", i, L.kv_from);
        }
      } else if (type == "attention_2") {
        L.mix = kRotary;
        L.rot_dims = m["rot"]["dims"].as_int(0);
        L.rot_base = m["rot"]["base"].need_double("mixer.rot.base");
        NVLLM_CHECK_ARG(L.rot_dims >= 0 && L.rot_dims % 2 == 0 && L.rot_dims <= L.D && L.rot_base > 0 && L.V % 2 == 0, NVLLM_ERR_ARG,
                        "Zasorax config: layer %zu rot dims %d (even, <= dim %d), vdim %d (even: the values are rotated in pairs)", i, L.rot_dims,
                        L.D, L.V);
      } else {
        NVLLM_CHECK_ARG(false, NVLLM_ERR_ARG, "Zasorax config: layer %zu has mixer type '%s' (known: attention, attention_2)", i, type.c_str());
      }
      const json::Value& f = l["mlp"];
      if (!f.is_null()) {
        const std::string kind = f["kind"].as_string("dense");
        if (kind == "dense") {
          L.ffk = kDense;
          L.ff = f["ff"].need_int("mlp.ff");
          NVLLM_CHECK_ARG(L.ff > 0, NVLLM_ERR_ARG, "Zasorax config: layer %zu feed-forward size", i);
        } else if (kind == "moe") {
          L.ffk = kExperts;
          L.ff = f["expert"]["ff"].need_int("mlp.expert.ff");
          L.experts = f["router"]["experts"].need_int("mlp.router.experts");
          L.top = f["router"]["top"].need_int("mlp.router.top");
          NVLLM_CHECK_ARG(L.ff > 0 && L.experts > 0 && L.experts <= 3072 && L.top > 0 && L.top <= L.experts, NVLLM_ERR_ARG,
                          "Zasorax config: layer %zu experts %d (<= 3072), top %d, expert size %d", i, L.experts, L.top, L.ff);
        } else {
          NVLLM_CHECK_ARG(false, NVLLM_ERR_ARG, "Zasorax config: layer %zu feed-forward kind '%s' (known: dense, moe)", i, kind.c_str());
        }
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

  // rotary table shared by everything that agrees on (base, dims): [max_pos, dims / 2] of (cos, sin), angles in f64
  int rope_table(const float** out, double base, int dims, cudaStream_t stream) {
    const auto key = std::make_pair(base, dims);
    auto it = rope_tables_.find(key);
    if (it == rope_tables_.end()) {
      float* tab = nullptr;
      RUN(dalloc(&tab, static_cast<size_t>(lim_.max_positions) * dims));
      RUN(nvllm_rope_table_interleaved(tab, lim_.max_positions, dims, base, stream));
      it = rope_tables_.emplace(key, tab).first;
    }
    *out = it->second;
    return 0;
  }

  int create(const ModelLimits& lim, cudaStream_t stream) override {
    lim_ = lim;
    dt_ = lim.dtype;
    esz_ = dt_ == NVLLM_F32 ? 4 : 2;
    const size_t W = width_, T = lim.max_tokens;
    RUN(oalloc(&embed_, static_cast<size_t>(vocab_) * W)); needed_.insert("embed");
    RUN(oalloc(&head_, static_cast<size_t>(vocab_) * W)); needed_.insert("head");
    RUN(valloc(&final_norm_, W, "final.norm"));
    size_t m_proj = 8, m_q = 8, m_mix = 8, m_ff = 0, m_eff = 0, m_exp = 0, m_top = 0, m_h = 1;
    cache_.resize(layers_.size());
    const size_t rows = static_cast<size_t>(lim.num_blocks) * lim.block_size;
    for (size_t i = 0; i < layers_.size(); ++i) {
      Layer& L = layers_[i];
      const std::string p = "l" + std::to_string(i) + ".", a = p + "mix.";
      const size_t HD = static_cast<size_t>(L.H) * L.D, HV = static_cast<size_t>(L.H) * L.V;
      RUN(valloc(&L.norm1, W, p + "norm1"));
      RUN(oalloc(&L.in, static_cast<size_t>(pad8(L.in_cols())) * W, true)); needed_.insert(a + "q");
      RUN(oalloc(&L.o, W * HV)); needed_.insert(a + "o");
      if (L.own_kv()) {
        needed_.insert(a + "k"); needed_.insert(a + "v");
        RUN(oalloc(&cache_[i].kc, rows * L.G * L.D, true)); RUN(oalloc(&cache_[i].vc, rows * L.G * L.V, true));
      }
      if (L.mix == kChunked) {
        RUN(valloc(&L.qn, HD, a + "q.norm"));
        if (L.own_kv()) RUN(valloc(&L.kn, static_cast<size_t>(L.G) * L.D, a + "k.norm"));
        RUN(valloc(&L.temp, L.H, a + "temp")); RUN(valloc(&L.sink, L.H, a + "sink"));
        needed_.insert(a + "rel");
      } else {
        needed_.insert(a + "g");
        if (L.rot_dims > 0) RUN(rope_table(&L.rope, L.rot_base, L.rot_dims, stream));
        RUN(rope_table(&L.vrope, L.rot_base, L.V, stream));
      }
      m_proj = std::max<size_t>(m_proj, pad8(L.in_cols())); m_q = std::max(m_q, HD); m_mix = std::max(m_mix, HV); m_h = std::max<size_t>(m_h, L.H);
      if (L.ffk != kNone) RUN(valloc(&L.norm2, W, p + "norm2"));
      if (L.ffk == kDense) {
        RUN(oalloc(&L.up, static_cast<size_t>(L.ff) * W)); RUN(oalloc(&L.down, W * L.ff)); RUN(valloc(&L.act, 2, p + "mlp.act"));
        needed_.insert(p + "mlp.up"); needed_.insert(p + "mlp.down");
        m_ff = std::max<size_t>(m_ff, L.ff);
      } else if (L.ffk == kExperts) {
        const size_t E = L.experts;
        RUN(oalloc(&L.router, static_cast<size_t>(pad8(L.experts)) * W, true)); needed_.insert(p + "mlp.router");
        RUN(valloc(&L.router_b, E, p + "mlp.router.b"));
        RUN(oalloc(&L.egu, E * 2 * L.ff * W)); RUN(oalloc(&L.edown, E * W * L.ff));
        for (int e = 0; e < L.experts; ++e)
          for (const char* t : {"gate", "up", "down"}) needed_.insert(p + "mlp.e" + std::to_string(e) + "." + t);
        if (dt_ == NVLLM_BF16 && W % 64 == 0 && L.ff % 64 == 0) L.tile_rows = 128;  // experts on the tensor-core grouped GEMM
        max_rows_ = std::max(max_rows_, nvllm_moe_max_rows(lim.max_tokens, L.top, L.experts, L.tile_rows));
        m_eff = std::max<size_t>(m_eff, L.ff); m_exp = std::max<size_t>(m_exp, pad8(L.experts)); m_top = std::max<size_t>(m_top, L.top);
      }
    }
    RUN(dalloc(&zero_sink_, m_h, sizeof(float), true));
    RUN(dalloc(&h_, T * W)); RUN(oalloc(&x_, T * W)); RUN(dalloc(&proj_, T * m_proj)); RUN(oalloc(&sub_out_, T * W));
    RUN(oalloc(&q_, T * m_q)); RUN(oalloc(&mix_in_, T * m_mix));
    if (m_ff > 0) RUN(oalloc(&up_buf_, T * m_ff));
    const size_t R = max_rows_;
    if (std::max(m_ff, m_eff) > 0) RUN(oalloc(&act_, std::max(T * m_ff, R * m_eff)));
    if (m_eff > 0) {
      RUN(dalloc(&route_, T * m_exp)); RUN(dalloc(&topk_idx_, T * m_top)); RUN(dalloc(&topk_w_, T * m_top));
      RUN(dalloc(&row_token_, R)); RUN(dalloc(&tile_expert_, R / 32 + 1)); RUN(dalloc(&slot_row_, T * m_top));
      RUN(oalloc(&xg_, R * W)); RUN(oalloc(&egu_buf_, R * 2 * m_eff)); RUN(oalloc(&eout_, R * W));
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
  int putf(float* dst, const uint16_t* src, int64_t n, cudaStream_t st) {
    std::vector<float> tmp(n);
    for (int64_t i = 0; i < n; ++i) tmp[i] = bf16_bits_to_f32(src[i]);
    NVLLM_CUDA(cudaMemcpyAsync(dst, tmp.data(), n * 4, cudaMemcpyHostToDevice, st));
    NVLLM_CUDA(cudaStreamSynchronize(st));
    return 0;
  }

  // The tensor's shape and where it goes.  kind: 0 operand matrix at (dst, element offset); 1 f32 vector; 2 a distance-bias
  // table, whose row count the tensor itself decides (rows < 0) and which is expanded per distance on the host.
  struct Target { int kind = -1; void* dst = nullptr; size_t off = 0; int64_t rows = 0, cols = 0; int layer = -1; };
  Target target_of(const std::string& name) const {
    const int64_t W = width_;
    Target t;
    auto mat = [&](void* d, size_t off, int64_t r, int64_t c) { t.kind = 0; t.dst = d; t.off = off; t.rows = r; t.cols = c; return t; };
    auto vec = [&](float* d, int64_t n) { t.kind = 1; t.dst = d; t.rows = 1; t.cols = n; return t; };
    if (name == "embed") return mat(embed_, 0, vocab_, W);
    if (name == "head") return mat(head_, 0, vocab_, W);
    if (name == "final.norm") return vec(final_norm_, W);
    if (name.size() < 4 || name[0] != 'l') return t;
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return t;
    const int li = atoi(name.substr(1, dot - 1).c_str());
    if (li < 0 || li >= static_cast<int>(layers_.size())) return t;
    const Layer& L = layers_[li];
    t.layer = li;
    const std::string rest = name.substr(dot + 1);
    const int64_t HD = static_cast<int64_t>(L.H) * L.D, HV = static_cast<int64_t>(L.H) * L.V, GD = static_cast<int64_t>(L.G) * L.D,
                  GV = static_cast<int64_t>(L.G) * L.V;
    if (rest == "norm1") return vec(L.norm1, W);
    if (rest == "norm2" && L.ffk != kNone) return vec(L.norm2, W);
    if (rest == "mix.q") return mat(L.in, 0, HD, W);
    if (rest == "mix.o") return mat(L.o, 0, W, HV);
    if (L.own_kv()) {
      if (rest == "mix.k") return mat(L.in, HD * W, GD, W);
      if (rest == "mix.v") return mat(L.in, (HD + GD) * W, GV, W);
    }
    if (L.mix == kChunked) {
      if (rest == "mix.q.norm") return vec(L.qn, HD);
      if (rest == "mix.k.norm" && L.own_kv()) return vec(L.kn, GD);
      if (rest == "mix.temp") return vec(L.temp, L.H);
      if (rest == "mix.sink") return vec(L.sink, L.H);
      if (rest == "mix.rel") { t.kind = 2; t.rows = -1; t.cols = L.H; return t; }
    } else {
      if (rest == "mix.g") return mat(L.in, (HD + GD + GV) * W, L.H, W);
    }
    if (L.ffk == kDense) {
      if (rest == "mlp.up") return mat(L.up, 0, L.ff, W);
      if (rest == "mlp.down") return mat(L.down, 0, W, L.ff);
      if (rest == "mlp.act") return vec(L.act, 2);
    } else if (L.ffk == kExperts) {
      if (rest == "mlp.router") return mat(L.router, 0, L.experts, W);
      if (rest == "mlp.router.b") return vec(L.router_b, L.experts);
      if (rest.compare(0, 5, "mlp.e") == 0) {
        const size_t d2 = rest.find('.', 5);
        if (d2 == std::string::npos) return t;
        const int e = atoi(rest.substr(5, d2 - 5).c_str());
        if (e < 0 || e >= L.experts || rest.substr(5, d2 - 5) != std::to_string(e)) return t;
        const std::string part = rest.substr(d2 + 1);
        const size_t gu = static_cast<size_t>(e) * 2 * L.ff * W;
        if (part == "gate") return mat(L.egu, gu, L.ff, W);
        if (part == "up") return mat(L.egu, gu + static_cast<size_t>(L.ff) * W, L.ff, W);
        if (part == "down") return mat(L.edown, static_cast<size_t>(e) * W * L.ff, W, L.ff);
      }
    }
    return t;
  }

  // Row of a distance table with `rows` rows for the distance n: one row per distance below half the table, above it
  // logarithmic steps that reach the last row at the distance `far`.  Computed in f64, once per table.
  static int distance_bucket(int n, int rows, int far) {
    const int half = rows / 2;
    if (n < half) return n;
    if (half <= 0 || far <= half) return rows - 1;
    const double r = std::log(static_cast<double>(n) / half) / std::log(static_cast<double>(far) / half) * (rows - half);
    return std::min<int64_t>(rows - 1, half + static_cast<int64_t>(std::floor(r)));
  }

  // Operand matrices and f32 vectors arrive as bf16 bit patterns.
  int load_weight(const char* name_c, const void* src_v, int64_t rows, int64_t cols, cudaStream_t st) override {
    NVLLM_CHECK_ARG(name_c && src_v, NVLLM_ERR_ARG, "load_weight: NULL");
    const std::string name(name_c);
    NVLLM_CHECK_ARG(needed_.count(name), NVLLM_ERR_ARG, "load_weight: tensor '%s' is not part of this model", name_c);
    Target t = target_of(name);
    NVLLM_CHECK_ARG(t.kind >= 0, NVLLM_ERR_ARG, "load_weight: unknown tensor '%s'", name_c);
    const uint16_t* src = static_cast<const uint16_t*>(src_v);
    if (t.kind == 2) {
      // the table as stored is [buckets, heads]; what the kernel reads is, per head, one value per distance 0 .. far (every
      // larger distance reads the last one, and inside a chunk no distance reaches the chunk's size)
      Layer& L = layers_[t.layer];
      NVLLM_CHECK_ARG(rows > 0 && cols == L.H, NVLLM_ERR_ARG, "load_weight(%s): expected [rows, %d], got [%lld, %lld]", name_c, L.H, (long long)rows,
                      (long long)cols);
      L.rel_rows = static_cast<int>(rows);
      int dr = std::max(L.bias_max, L.rel_rows / 2) + 1;
      if (L.chunk > 0) dr = std::min(dr, L.chunk);
      std::vector<float> ex(static_cast<size_t>(dr) * L.H);
      for (int n = 0; n < dr; ++n) {
        const int b = distance_bucket(n, L.rel_rows, L.bias_max);
        for (int h = 0; h < L.H; ++h) ex[static_cast<size_t>(h) * dr + n] = bf16_bits_to_f32(src[static_cast<size_t>(b) * L.H + h]);
      }
      if (L.dist == nullptr || dr > L.dist_rows) RUN(dalloc(&L.dist, ex.size()));
      L.dist_rows = dr;
      NVLLM_CUDA(cudaMemcpyAsync(L.dist, ex.data(), ex.size() * 4, cudaMemcpyHostToDevice, st));
      NVLLM_CUDA(cudaStreamSynchronize(st));
    } else {
      NVLLM_CHECK_ARG(rows * cols == t.rows * t.cols && (t.kind == 1 || (rows == t.rows && cols == t.cols)), NVLLM_ERR_ARG,
                      "load_weight(%s): expected [%lld, %lld], got [%lld, %lld]", name_c, (long long)t.rows, (long long)t.cols, (long long)rows,
                      (long long)cols);
      if (t.kind == 0) RUN(put(t.dst, t.off, src, rows, cols, st));
      else RUN(putf(static_cast<float*>(t.dst), src, rows * cols, st));
    }
    loaded_.insert(name);
    if (loaded_.size() == needed_.size()) ready_ = true;
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
      if (t.kind == 2) {  // rows of a distance table: the configuration's `bias_rows`, else 32
        const Layer& L = layers_[t.layer];
        t.rows = L.bias_rows_cfg > 0 ? L.bias_rows_cfg : 32;
      }
      buf.resize(static_cast<size_t>(t.rows) * t.cols);
      const bool norm_w = name.find("norm") != std::string::npos, is_temp = ends(name, ".temp"), is_table = name == "embed";
      const bool unit = ends(name, ".sink") || ends(name, ".rel") || ends(name, ".act") || ends(name, ".router.b");
      for (size_t i = 0; i < buf.size(); ++i) {
        const uint64_t hsh = mix(seed ^ (tid << 40) ^ (i + 1) * 0x9E3779B97F4A7C15ull);
        const int s = static_cast<int>((hsh & 0xffff) + ((hsh >> 16) & 0xffff) + ((hsh >> 32) & 0xffff) + (hsh >> 48)) - 131070;
        const float g = static_cast<float>(s) * 2.6428998e-05f;  // ~N(0, 1)
        float v = g * std;
        if (norm_w) v = 1.0f + 0.1f * g;
        else if (is_temp) v = 1.0f + 0.2f * g;
        else if (unit) v = 0.5f * g;
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
    NVLLM_CHECK_ARG(ready_, NVLLM_ERR_STATE, "Zasorax forward: weights are not loaded");
    NVLLM_CHECK_ARG(v.cu_tokens && v.tables, NVLLM_ERR_ARG, "Zasorax forward: the step carries no token ranges / block tables");
    auto mk = [&](const char* name) { if (v.mark) v.mark(v.mark_ctx, name); };
    auto lin = [&](void* y, const void* x, const void* w, int n, int k, int64_t ldx, int64_t ldy, int out_dt, const char* name) {
      ++launches;
      const int rc = nvllm_linear(y, x, w, N, n, k, ldx, k, ldy, 1, 0, 0, 0, dt_, out_dt, st);
      mk(name);
      return rc;
    };
    // h += rms(y) * post;  then the operand of what reads the stream next: the stream itself (x_), or at the very end the
    // model's last norm
    auto add = [&](const void* y, const float* post, const float* last) {
      ++launches;
      const int rc = nvllm_rms_residual_norm(x_, h_, y, dt_, post, last, N, W, eps_, dt_, st);
      mk(last ? "rms_residual_norm (+ final norm)" : "rms_residual_norm");
      return rc;
    };
    const float norm_eps = eps_ > 0.f ? eps_ : 1e-30f;
    RUN(nvllm_embedding_stream(h_, x_, dt_, embed_, v.ids, N, W, vocab_, embed_scale_, dt_, st)); ++launches; mk("embedding_stream");
    for (size_t i = 0; i < layers_.size(); ++i) {
      const Layer& L = layers_[i];
      const LayerCache& kv = L.own_kv() ? cache_[i] : cache_[L.kv_from];
      const bool last_layer = i + 1 == layers_.size();
      const int HD = L.H * L.D, HV = L.H * L.V, GD = L.G * L.D, GV = L.G * L.V, ld = pad8(L.in_cols());
      RUN(lin(proj_, x_, L.in, ld, W, W, ld, NVLLM_F32, L.mix == kChunked ? "attention q k v projection" : "attention q k v g projection"));
      if (L.mix == kChunked) {
        // RMS norm of q and of k over the whole projection, the cache store; chunked attention with the head temperature, the
        // distance bias and the sink
        RUN(nvllm_attn_wide_norm_store(q_, HD, kv.kc, kv.vc, GD, GV, proj_, ld, L.qn, L.kn, eps_, v.slots, N, HD, L.k_cols(), L.v_cols(), dt_, st));
        ++launches; mk("attn_wide_norm_store");
        RUN(nvllm_biased_attention(mix_in_, HV, q_, HD, nullptr, 0, 0, kv.kc, kv.vc, GD, GV, v.tok_seq, v.positions, v.tables, v.table_cap,
                                   lim_.block_size, N, L.H, L.G, L.D, L.V, L.scale, 0.f, 0.f, 1, 0, L.sink, L.chunk, L.temp, L.dist, L.dist_rows,
                                   nullptr, 0, v.cu_tokens, S, dt_, st)); ++launches; mk("biased_attention (chunked)");
      } else {
        // rotary on q and k (halves), weightless per-head norm, the values rotated over vdim, the cache store; causal attention
        // with a zero sink, the output turned back and gated per head
        RUN(nvllm_attn_rotary_store(q_, HD, kv.kc, kv.vc, GD, GV, proj_, ld, nullptr, nullptr, nullptr, v.positions, L.rope, L.rot_dims, 1, L.vrope,
                                    lim_.max_positions, norm_eps, v.slots, N, L.H, L.G, L.D, L.V, 0, dt_, st)); ++launches; mk("attn_rotary_store");
        RUN(nvllm_biased_attention(mix_in_, HV, q_, HD, proj_ + HD + GD + GV, ld, 1, kv.kc, kv.vc, GD, GV, v.tok_seq, v.positions, v.tables,
                                   v.table_cap, lim_.block_size, N, L.H, L.G, L.D, L.V, L.scale, 0.f, 0.f, 1, 0, zero_sink_, 0, nullptr, nullptr, 0,
                                   L.vrope, lim_.max_positions, v.cu_tokens, S, dt_, st)); ++launches; mk("biased_attention (rotated values)");
      }
      RUN(lin(sub_out_, mix_in_, L.o, W, HV, HV, W, dt_, "mixer output projection"));
      RUN(add(sub_out_, L.norm1, (last_layer && L.ffk == kNone) ? final_norm_ : nullptr));
      if (L.ffk == kDense) {
        RUN(lin(up_buf_, x_, L.up, L.ff, W, W, L.ff, dt_, "up projection"));
        RUN(nvllm_ff_activation_params(act_, up_buf_, N, L.ff, 2, L.act, dt_, st)); ++launches; mk("ff_activation (xielu)");
        RUN(lin(sub_out_, act_, L.down, W, L.ff, L.ff, W, dt_, "down projection"));
      } else if (L.ffk == kExperts) {
        const int E = L.experts, lde = pad8(E);
        RUN(lin(route_, x_, L.router, lde, W, W, lde, NVLLM_F32, "router projection"));
        RUN(nvllm_moe_route_logits(topk_idx_, topk_w_, route_, lde, L.router_b, N, E, L.top, st)); ++launches; mk("moe_route_logits");
        const int rows = nvllm_moe_max_rows(N, L.top, E, L.tile_rows);
        RUN(nvllm_moe_sort(row_token_, tile_expert_, slot_row_, topk_idx_, N, L.top, E, rows, L.tile_rows, st)); ++launches; mk("moe_sort");
        if (L.tile_rows == 128) {
          RUN(nvllm_gather_rows(xg_, x_, row_token_, rows, W, N, dt_, st)); ++launches; mk("expert row gather");
          RUN(nvllm_gemm_bf16_grouped(egu_buf_, xg_, L.egu, rows, 2 * L.ff, W, E, W, W, 2 * L.ff, tile_expert_, st)); ++launches; mk("expert gate / up grouped GEMM");
          RUN(nvllm_ff_activation(act_, egu_buf_, rows, L.ff, 0, dt_, st)); ++launches; mk("ff_activation (silu gate)");
          RUN(nvllm_gemm_bf16_grouped(eout_, act_, L.edown, rows, W, L.ff, E, L.ff, L.ff, W, tile_expert_, st)); ++launches; mk("expert down grouped GEMM");
        } else {
          RUN(nvllm_linear_grouped(act_, x_, L.egu, rows, L.ff, W, W, W, L.ff, static_cast<int64_t>(2) * L.ff * W, row_token_, tile_expert_, 3, 0.f,
                                   dt_, dt_, st)); ++launches; mk("expert gate / up + silu gate grouped tile kernel");
          RUN(nvllm_linear_grouped(eout_, act_, L.edown, rows, W, L.ff, L.ff, L.ff, W, static_cast<int64_t>(W) * L.ff, nullptr, tile_expert_, 0, 0.f,
                                   dt_, dt_, st)); ++launches; mk("expert down grouped tile kernel");
        }
        RUN(nvllm_moe_combine(sub_out_, eout_, x_, nullptr, topk_idx_, topk_w_, slot_row_, N, W, L.top, E, dt_, st)); ++launches; mk("moe_combine");
      }
      if (L.ffk != kNone) RUN(add(sub_out_, L.norm2, last_layer ? final_norm_ : nullptr));
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
      RUN(nvllm_gather_rows(head_in_, x_, v.logit_rows, v.n_logit_rows, W, N, dt_, st)); ++launches; mk("gather_rows");
      ++launches;
      RUN(nvllm_linear(v.logits, head_in_, head_, v.n_logit_rows, vocab_, W, W, W, vocab_, 1, 0, 0, 0, dt_, NVLLM_F32, st));
      mk("head projection");
    }
    return 0;
  }
};

}  // namespace

ModelImpl* make_zasorax(const json::Value& cfg) {
  Zasorax* m = new Zasorax();
  if (m->parse(cfg) != 0) { delete m; return nullptr; }
  return m;
}

}  // namespace nvllm
