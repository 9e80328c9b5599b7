// kosazen_model.cu — the Kosazen architecture on the runner's model interface (model.hpp).
//
// Kosazen is a decoder-only model whose blocks are sandwich-normed with Dynamic Tanh (dyt_norm.cu) around an f32 residual
// stream:  h += dyt1b(mixer(dyt1(h)));  h += dyt2b(ff(dyt2(h))).  The mixer is latent attention (latent_attn.cu): the cache
// holds one normalised latent and one shared rotated key part per token.  The feed-forward is a mixture of experts
// (moe.cu, linear_any.cu) with identity experts, a selection bias and an always-on shared expert; a layer may have no
// feed-forward.  A contiguous range of layers may be run several times with the same weights (`loop`); every run has its
// own cache region.  Every size, constant and the layer order come from the configuration; nothing is assumed equal.
//
// configuration keys read here: architecture, vocab, width, norm.eps, loop.{start,stop,times}, layers[i].type ("latent_attention"),
// layers[i].mixer.{heads,dim,rot_dim,vdim,kv_rank,scale,rot.{base,dims}}, layers[i].mlp (null | kind "moe",
// expert.{ff,limit}, router.{experts,identity,top,scale}, shared.{ff,limit}).
// tensors: embed, head, final.norm{,.alpha,.b}, l<i>.norm{1,1b,2,2b}{,.alpha,.b}, l<i>.mix.{q,dkv,dkv.norm,uk,uv,o},
// l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down}}.
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

struct Dyt { float *alpha = nullptr, *w = nullptr, *b = nullptr; };

struct Layer {
  // mixer
  int heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, rot_dims = 0;
  double rot_base = 10000.0;
  float scale = 1.f;
  // feed-forward
  bool has_mlp = false, has_shared = false;
  int experts = 0, identity = 0, top = 0, ff = 0, sff = 0;
  float router_scale = 1.f, limit = 0.f, slimit = 0.f;
  // weights; operand tensors are bf16 or f32 (model dtype), norm / bias vectors are f32
  Dyt n1, n1b, n2, n2b;
  void *qdkv = nullptr, *ukT = nullptr, *uv = nullptr, *o = nullptr;
  float* c_norm = nullptr;
  void *router = nullptr, *egu = nullptr, *edown = nullptr, *sgu = nullptr, *sdown = nullptr;
  float* correction = nullptr;
  const float* rope = nullptr;
  int tile_rows = 32;  // 128: experts run on the tensor-core grouped GEMM (bf16, aligned sizes), else the tile kernel
  int qdim() const { return heads * (dim + rot_dim); }
  int qd_n() const { return qdim() + kv_rank + rot_dim; }
  int cache_row() const { return (kv_rank + rot_dim + 7) / 8 * 8; }
};

class Kosazen : public ModelImpl {
 public:
  int vocab_ = 0, width_ = 0;
  float eps_ = 1e-5f;
  std::vector<Layer> layers_;
  std::vector<int> runs_;  // layer index of every layer run, in execution order
  ModelLimits lim_{};
  int dt_ = NVLLM_BF16;
  size_t esz_ = 2;
  void *embed_ = nullptr, *head_ = nullptr;
  Dyt final_;
  std::vector<void*> cache_;  // per run
  std::map<std::pair<double, int>, float*> rope_tables_;
  // activations
  float *h_ = nullptr, *q_abs_ = nullptr, *router_logits_ = nullptr, *topk_w_ = nullptr;
  void *normed_ = nullptr, *qd_ = nullptr, *o_lat_ = nullptr, *attn_ = nullptr, *proj_ = nullptr, *act_ = nullptr,
       *eout_ = nullptr, *xg_ = nullptr, *egu_buf_ = nullptr, *sgu_buf_ = nullptr, *sact_ = nullptr, *sout_ = nullptr, *moe_out_ = nullptr, *head_in_ = nullptr;
  int32_t *topk_idx_ = nullptr, *row_token_ = nullptr, *tile_expert_ = nullptr, *slot_row_ = nullptr;
  int max_rows_ = 0, head_rows_ = 0;
  std::vector<void*> allocs_;
  std::set<std::string> needed_, loaded_;
  bool ready_ = false;

  ~Kosazen() override { for (void* p : allocs_) cudaFree(p); }
  int vocab() const override { return vocab_; }
  int hidden() const override { return width_; }
  int layer_runs() const override { return static_cast<int>(runs_.size()); }
  bool weights_ready() const override { return ready_; }

  int parse(const json::Value& c) {
    vocab_ = c["vocab"].need_int("vocab");
    width_ = c["width"].need_int("width");
    eps_ = static_cast<float>(c["norm"]["eps"].as_double(1e-5));
    const json::Value& ls = c["layers"];
    NVLLM_CHECK_ARG(ls.is_array() && ls.size() > 0 && vocab_ > 0 && width_ > 0, NVLLM_ERR_ARG, "Kosazen config: layers / vocab / width");
    for (size_t i = 0; i < ls.size(); ++i) {
      const json::Value& l = ls[i];
      Layer L;
      const std::string type = l["type"].as_string();
      NVLLM_CHECK_ARG(type == "latent_attention", NVLLM_ERR_ARG, "Kosazen config: layer %zu has mixer type '%s' (known: latent_attention)", i, type.c_str());
      const json::Value& m = l["mixer"];
      L.heads = m["heads"].need_int("mixer.heads"); L.dim = m["dim"].need_int("mixer.dim");
      L.rot_dim = m["rot_dim"].need_int("mixer.rot_dim"); L.vdim = m["vdim"].need_int("mixer.vdim");
      L.kv_rank = m["kv_rank"].need_int("mixer.kv_rank");
      L.scale = static_cast<float>(m["scale"].need_double("mixer.scale"));
      L.rot_dims = m["rot"]["dims"].as_int(L.rot_dim);
      L.rot_base = m["rot"]["base"].as_double(10000.0);
      NVLLM_CHECK_ARG(L.heads > 0 && L.dim >= 0 && L.rot_dim >= 0 && L.dim + L.rot_dim > 0 && L.vdim > 0 && L.kv_rank > 0 &&
                          L.kv_rank <= 1024 && L.rot_dims >= 0 && L.rot_dims % 2 == 0 && L.rot_dims <= L.rot_dim && L.rot_base > 0,
                      NVLLM_ERR_ARG, "Kosazen config: layer %zu mixer sizes", i);
      const json::Value& f = l["mlp"];
      if (!f.is_null()) {
        const std::string kind = f["kind"].as_string("moe");
        NVLLM_CHECK_ARG(kind == "moe", NVLLM_ERR_ARG, "Kosazen config: layer %zu feed-forward kind '%s' (known: moe)", i, kind.c_str());
        L.has_mlp = true;
        L.experts = f["router"]["experts"].need_int("router.experts");
        L.identity = f["router"]["identity"].as_int(0);
        L.top = f["router"]["top"].need_int("router.top");
        L.router_scale = static_cast<float>(f["router"]["scale"].as_double(1.0));
        L.ff = f["expert"]["ff"].as_int(0);
        L.limit = static_cast<float>(f["expert"]["limit"].as_double(INFINITY));
        if (!f["shared"].is_null()) {
          L.has_shared = true;
          L.sff = f["shared"]["ff"].need_int("shared.ff");
          L.slimit = static_cast<float>(f["shared"]["limit"].as_double(INFINITY));
        }
        NVLLM_CHECK_ARG(L.experts >= 0 && L.identity >= 0 && L.top > 0 && L.top <= L.experts + L.identity &&
                            L.experts + L.identity <= 1536 && (L.experts == 0 || L.ff > 0) && (!L.has_shared || L.sff > 0),
                        NVLLM_ERR_ARG, "Kosazen config: layer %zu router / expert sizes", i);
      }
      layers_.push_back(L);
    }
    const int n = static_cast<int>(layers_.size());
    int start = 0, stop = 0, times = 1;
    if (c["loop"].is_object()) {
      start = c["loop"]["start"].as_int(0); stop = c["loop"]["stop"].as_int(0); times = c["loop"]["times"].as_int(1);
      NVLLM_CHECK_ARG(0 <= start && start <= stop && stop <= n && times >= 0, NVLLM_ERR_ARG, "Kosazen config: loop %d..%d x %d", start, stop, times);
    }
    for (int i = 0; i < start; ++i) runs_.push_back(i);
    for (int t = 0; t < times; ++t) for (int i = start; i < stop; ++i) runs_.push_back(i);
    for (int i = stop; i < n; ++i) runs_.push_back(i);
    NVLLM_CHECK_ARG(!runs_.empty(), NVLLM_ERR_ARG, "Kosazen config: no layer runs");
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
  int oalloc(void** p, size_t count) { return dalloc(p, count, esz_); }  // operand-typed buffer
  int dyt_alloc(Dyt& d, const std::string& name) {
    RUN(dalloc(&d.alpha, 1)); RUN(dalloc(&d.w, width_)); RUN(dalloc(&d.b, width_));
    needed_.insert(name); needed_.insert(name + ".alpha"); needed_.insert(name + ".b");
    return 0;
  }

  int create(const ModelLimits& lim, cudaStream_t stream) override {
    lim_ = lim;
    dt_ = lim.dtype;
    esz_ = dt_ == NVLLM_F32 ? 4 : 2;
    const size_t W = width_, T = lim.max_tokens;
    RUN(oalloc(&embed_, static_cast<size_t>(vocab_) * W)); RUN(oalloc(&head_, static_cast<size_t>(vocab_) * W));
    needed_.insert("embed"); needed_.insert("head");
    RUN(dyt_alloc(final_, "final.norm"));
    size_t m_qd = 0, m_hr = 0, m_hv = 0, m_et = 0, m_ff = 0, m_sff = 0, m_top = 1;
    for (size_t i = 0; i < layers_.size(); ++i) {
      Layer& L = layers_[i];
      const std::string p = "l" + std::to_string(i) + ".";
      RUN(dyt_alloc(L.n1, p + "norm1")); RUN(dyt_alloc(L.n1b, p + "norm1b"));
      if (L.has_mlp) { RUN(dyt_alloc(L.n2, p + "norm2")); RUN(dyt_alloc(L.n2b, p + "norm2b")); }
      RUN(oalloc(&L.qdkv, static_cast<size_t>(L.qd_n()) * W));
      RUN(oalloc(&L.ukT, static_cast<size_t>(L.heads) * L.kv_rank * (L.dim > 0 ? L.dim : 1)));
      RUN(oalloc(&L.uv, static_cast<size_t>(L.heads) * L.vdim * L.kv_rank));
      RUN(oalloc(&L.o, W * L.heads * L.vdim));
      RUN(dalloc(&L.c_norm, L.kv_rank));
      for (const char* t : {"q", "dkv", "dkv.norm", "uv", "o"}) needed_.insert(p + "mix." + t);
      if (L.dim > 0) needed_.insert(p + "mix.uk");
      if (L.has_mlp) {
        const size_t et = L.experts + L.identity;
        RUN(oalloc(&L.router, et * W)); RUN(dalloc(&L.correction, et, sizeof(float), true));
        needed_.insert(p + "mlp.router"); needed_.insert(p + "mlp.correction");
        if (L.experts > 0) {
          RUN(oalloc(&L.egu, static_cast<size_t>(L.experts) * 2 * L.ff * W));
          RUN(oalloc(&L.edown, static_cast<size_t>(L.experts) * W * L.ff));
          for (int e = 0; e < L.experts; ++e)
            for (const char* t : {"gate", "up", "down"}) needed_.insert(p + "mlp.e" + std::to_string(e) + "." + t);
        }
        if (L.has_shared) {
          RUN(oalloc(&L.sgu, static_cast<size_t>(2) * L.sff * W)); RUN(oalloc(&L.sdown, W * L.sff));
          for (const char* t : {"gate", "up", "down"}) needed_.insert(p + "mlp.shared." + t);
        }
        m_et = std::max(m_et, et); m_ff = std::max<size_t>(m_ff, L.ff); m_sff = std::max<size_t>(m_sff, L.sff);
        m_top = std::max<size_t>(m_top, L.top);
        if (dt_ == NVLLM_BF16 && L.experts > 0 && W % 64 == 0 && L.ff % 64 == 0) L.tile_rows = 128;
        max_rows_ = std::max(max_rows_, nvllm_moe_max_rows(lim.max_tokens, L.top, L.experts, L.tile_rows));
      }
      m_qd = std::max<size_t>(m_qd, L.qd_n()); m_hr = std::max<size_t>(m_hr, static_cast<size_t>(L.heads) * L.kv_rank);
      m_hv = std::max<size_t>(m_hv, static_cast<size_t>(L.heads) * L.vdim);
      // rotary table shared by the layers that agree on (base, dims)
      if (L.rot_dims > 0) {
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
    }
    // one cache region per layer run: [num_blocks * block_size, kv_rank + rot_dim] rows, zero-initialised
    cache_.resize(runs_.size());
    for (size_t r = 0; r < runs_.size(); ++r) {
      const Layer& L = layers_[runs_[r]];
      const size_t n = static_cast<size_t>(lim.num_blocks) * lim.block_size * L.cache_row();
      RUN(oalloc(&cache_[r], n));
      NVLLM_CUDA(cudaMemsetAsync(cache_[r], 0, n * esz_, stream));
    }
    RUN(dalloc(&h_, T * W)); RUN(oalloc(&normed_, T * W)); RUN(oalloc(&qd_, T * m_qd));
    RUN(dalloc(&q_abs_, T * m_hr)); RUN(oalloc(&o_lat_, T * m_hr)); RUN(oalloc(&attn_, T * m_hv)); RUN(oalloc(&proj_, T * W));
    if (m_et > 0) {
      RUN(dalloc(&router_logits_, T * m_et)); RUN(dalloc(&topk_w_, T * m_top)); RUN(dalloc(&topk_idx_, T * m_top));
      RUN(dalloc(&slot_row_, T * m_top)); RUN(dalloc(&row_token_, static_cast<size_t>(max_rows_) + 32));
      RUN(dalloc(&tile_expert_, static_cast<size_t>(max_rows_) / 32 + 1));
      RUN(oalloc(&act_, static_cast<size_t>(max_rows_) * (m_ff ? m_ff : 1))); RUN(oalloc(&eout_, static_cast<size_t>(max_rows_) * W));
      RUN(oalloc(&xg_, static_cast<size_t>(max_rows_) * W)); RUN(oalloc(&egu_buf_, static_cast<size_t>(max_rows_) * 2 * (m_ff ? m_ff : 1)));
      RUN(oalloc(&sgu_buf_, T * 2 * (m_sff ? m_sff : 1))); RUN(oalloc(&sact_, T * (m_sff ? m_sff : 1))); RUN(oalloc(&sout_, T * W));
      RUN(oalloc(&moe_out_, T * W));
    }
    return 0;
  }

  // ---- weights -----------------------------------------------------------------------------------------------
  static float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
  }
  // host bf16 [rows, cols] -> device operand tensor at element offset `off` (row pitch cols), optionally transposed
  int put(void* dst, size_t off, const uint16_t* src, int64_t rows, int64_t cols, bool transpose, cudaStream_t st) {
    const size_t n = static_cast<size_t>(rows) * cols;
    std::vector<uint8_t> tmp(n * esz_);
    for (int64_t r = 0; r < rows; ++r)
      for (int64_t c = 0; c < cols; ++c) {
        const size_t o = transpose ? static_cast<size_t>(c) * rows + r : static_cast<size_t>(r) * cols + c;
        const uint16_t v = src[r * cols + c];
        if (esz_ == 2) reinterpret_cast<uint16_t*>(tmp.data())[o] = v;
        else reinterpret_cast<float*>(tmp.data())[o] = bf16_bits_to_f32(v);
      }
    NVLLM_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(dst) + off * esz_, tmp.data(), n * esz_, cudaMemcpyHostToDevice, st));
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
#define SHAPE(er, ec)                                                                                                       \
  NVLLM_CHECK_ARG(rows == (er) && cols == (ec), NVLLM_ERR_ARG, "load_weight(%s): expected [%lld, %lld], got [%lld, %lld]", name_c, \
                  (long long)(er), (long long)(ec), (long long)rows, (long long)cols)

  int load_weight(const char* name_c, const void* src_v, int64_t rows, int64_t cols, cudaStream_t st) override {
    NVLLM_CHECK_ARG(name_c && src_v, NVLLM_ERR_ARG, "load_weight: NULL");
    const std::string name(name_c);
    const uint16_t* src = static_cast<const uint16_t*>(src_v);
    NVLLM_CHECK_ARG(needed_.count(name), NVLLM_ERR_ARG, "load_weight: tensor '%s' is not part of this model", name_c);
    const int64_t W = width_;
    auto done = [&](int rc) {
      if (rc == 0) { loaded_.insert(name); ready_ = loaded_.size() == needed_.size(); }
      return rc;
    };
    auto dyt = [&](Dyt& d, const std::string& base) -> int {
      if (name == base) { SHAPE(1, W); return done(putf(d.w, src, W, st)); }
      if (name == base + ".b") { SHAPE(1, W); return done(putf(d.b, src, W, st)); }
      SHAPE(1, 1);
      return done(putf(d.alpha, src, 1, st));
    };
    if (name == "embed") { SHAPE(vocab_, W); return done(put(embed_, 0, src, rows, cols, false, st)); }
    if (name == "head") { SHAPE(vocab_, W); return done(put(head_, 0, src, rows, cols, false, st)); }
    if (name.compare(0, 10, "final.norm") == 0) return dyt(final_, "final.norm");
    NVLLM_CHECK_ARG(name[0] == 'l', NVLLM_ERR_ARG, "load_weight: unknown tensor '%s'", name_c);
    const size_t dot = name.find('.');
    const int li = atoi(name.substr(1, dot - 1).c_str());
    NVLLM_CHECK_ARG(li >= 0 && li < static_cast<int>(layers_.size()), NVLLM_ERR_ARG, "load_weight: layer %d out of range", li);
    Layer& L = layers_[li];
    const std::string p = name.substr(0, dot + 1), rest = name.substr(dot + 1);
    if (rest.compare(0, 6, "norm1b") == 0) return dyt(L.n1b, p + "norm1b");
    if (rest.compare(0, 5, "norm1") == 0) return dyt(L.n1, p + "norm1");
    if (rest.compare(0, 6, "norm2b") == 0) return dyt(L.n2b, p + "norm2b");
    if (rest.compare(0, 5, "norm2") == 0) return dyt(L.n2, p + "norm2");
    const int64_t H = L.heads, R = L.kv_rank;
    if (rest == "mix.q") { SHAPE(L.qdim(), W); return done(put(L.qdkv, 0, src, rows, cols, false, st)); }
    if (rest == "mix.dkv") { SHAPE(R + L.rot_dim, W); return done(put(L.qdkv, static_cast<size_t>(L.qdim()) * W, src, rows, cols, false, st)); }
    if (rest == "mix.dkv.norm") { SHAPE(1, R); return done(putf(L.c_norm, src, R, st)); }
    if (rest == "mix.uk") {  // [H * dim, R] -> per head the transpose [R, dim], so that the key map folds into the query
      SHAPE(H * L.dim, R);
      for (int64_t h = 0; h < H; ++h)
        RUN(put(L.ukT, static_cast<size_t>(h) * R * L.dim, src + h * L.dim * R, L.dim, R, true, st));
      return done(0);
    }
    if (rest == "mix.uv") { SHAPE(H * L.vdim, R); return done(put(L.uv, 0, src, rows, cols, false, st)); }
    if (rest == "mix.o") { SHAPE(W, H * L.vdim); return done(put(L.o, 0, src, rows, cols, false, st)); }
    if (rest == "mlp.router") { SHAPE(L.experts + L.identity, W); return done(put(L.router, 0, src, rows, cols, false, st)); }
    if (rest == "mlp.correction") { SHAPE(1, L.experts + L.identity); return done(putf(L.correction, src, cols, st)); }
    if (rest == "mlp.shared.gate") { SHAPE(L.sff, W); return done(put(L.sgu, 0, src, rows, cols, false, st)); }
    if (rest == "mlp.shared.up") { SHAPE(L.sff, W); return done(put(L.sgu, static_cast<size_t>(L.sff) * W, src, rows, cols, false, st)); }
    if (rest == "mlp.shared.down") { SHAPE(W, L.sff); return done(put(L.sdown, 0, src, rows, cols, false, st)); }
    if (rest.compare(0, 5, "mlp.e") == 0) {
      const size_t d2 = rest.find('.', 5);
      const int e = atoi(rest.substr(5, d2 - 5).c_str());
      const std::string t = rest.substr(d2 + 1);
      NVLLM_CHECK_ARG(e >= 0 && e < L.experts, NVLLM_ERR_ARG, "load_weight(%s): expert out of range", name_c);
      const size_t gu = static_cast<size_t>(e) * 2 * L.ff * W;
      if (t == "gate") { SHAPE(L.ff, W); return done(put(L.egu, gu, src, rows, cols, false, st)); }
      if (t == "up") { SHAPE(L.ff, W); return done(put(L.egu, gu + static_cast<size_t>(L.ff) * W, src, rows, cols, false, st)); }
      if (t == "down") { SHAPE(W, L.ff); return done(put(L.edown, static_cast<size_t>(e) * W * L.ff, src, rows, cols, false, st)); }
    }
    NVLLM_CHECK_ARG(false, NVLLM_ERR_ARG, "load_weight: unknown tensor '%s'", name_c);
  }

  // Seeded synthetic weights (benchmarks, smoke runs): every needed tensor drawn on the host from a counter-based
  // generator and sent through load_weight, so that synthetic and checkpoint weights take the same path.
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
    std::vector<uint16_t> buf;
    uint64_t tid = 0;
    for (const std::string& name : needed_) {
      ++tid;
      int64_t rows = 1, cols = 1;
      RUN(shape_of(name, &rows, &cols));
      buf.resize(static_cast<size_t>(rows) * cols);
      const bool is_alpha = name.size() > 6 && name.compare(name.size() - 6, 6, ".alpha") == 0;
      const bool is_norm_w = !is_alpha && (name.find("norm") != std::string::npos) && name.compare(name.size() - 2, 2, ".b") != 0;
      for (size_t i = 0; i < buf.size(); ++i) {
        const uint64_t hsh = mix(seed ^ (tid << 40) ^ (i + 1) * 0x9E3779B97F4A7C15ull);
        const int s = static_cast<int>((hsh & 0xffff) + ((hsh >> 16) & 0xffff) + ((hsh >> 32) & 0xffff) + (hsh >> 48)) - 131070;
        const float g = static_cast<float>(s) * 2.6428998e-05f;  // ~N(0, 1)
        float v = g * std;
        if (is_alpha) v = 1.0f + 0.1f * g;
        else if (is_norm_w) v = 1.0f + 0.1f * g;
        buf[i] = to_bf16(v);
      }
      RUN(load_weight(name.c_str(), buf.data(), rows, cols, st));
    }
    return 0;
  }
  int shape_of(const std::string& name, int64_t* rows, int64_t* cols) const {
    const int64_t W = width_;
    auto set = [&](int64_t r, int64_t c) { *rows = r; *cols = c; return 0; };
    if (name.size() > 6 && name.compare(name.size() - 6, 6, ".alpha") == 0) return set(1, 1);
    if (name == "embed" || name == "head") return set(vocab_, W);
    if (name.find("norm") != std::string::npos && name.find("dkv") == std::string::npos) return set(1, W);
    const size_t dot = name.find('.');
    const Layer& L = layers_[atoi(name.substr(1, dot - 1).c_str())];
    const std::string rest = name.substr(dot + 1);
    if (rest == "mix.q") return set(L.qdim(), W);
    if (rest == "mix.dkv") return set(L.kv_rank + L.rot_dim, W);
    if (rest == "mix.dkv.norm") return set(1, L.kv_rank);
    if (rest == "mix.uk") return set(static_cast<int64_t>(L.heads) * L.dim, L.kv_rank);
    if (rest == "mix.uv") return set(static_cast<int64_t>(L.heads) * L.vdim, L.kv_rank);
    if (rest == "mix.o") return set(W, static_cast<int64_t>(L.heads) * L.vdim);
    if (rest == "mlp.router") return set(L.experts + L.identity, W);
    if (rest == "mlp.correction") return set(1, L.experts + L.identity);
    if (rest == "mlp.shared.gate" || rest == "mlp.shared.up") return set(L.sff, W);
    if (rest == "mlp.shared.down") return set(W, L.sff);
    if (rest.size() > 5 && rest.compare(rest.size() - 5, 5, ".down") == 0) return set(W, L.ff);
    return set(L.ff, W);
  }

  // ---- forward ---------------------------------------------------------------------------------------------------
  int forward(const StepView& v) override {
    void* st = v.stream;
    const int N = v.n_tokens, W = width_;
    launches = 0;
    auto mk = [&](const char* name) { if (v.mark) v.mark(v.mark_ctx, name); };
    auto lin = [&](void* y, const void* x, const void* w, int n, int k, int64_t ldx, int64_t ldy, int out_dt, const char* name) {
      ++launches;
      const int rc = nvllm_linear(y, x, w, N, n, k, ldx, k, ldy, 1, 0, 0, 0, dt_, out_dt, st);
      mk(name);
      return rc;
    };
    const int act_dt = dt_;  // activations follow the model dtype
    RUN(nvllm_embedding_gather_f32(h_, embed_, v.ids, N, W, vocab_, dt_, st)); ++launches; mk("embedding_gather_f32");
    const Layer& first = layers_[runs_[0]];
    RUN(nvllm_dyt_residual_norm(normed_, h_, nullptr, nullptr, nullptr, nullptr, first.n1.alpha, first.n1.w, first.n1.b, N, W, dt_, st)); ++launches; mk("dyt_residual_norm");
    for (size_t r = 0; r < runs_.size(); ++r) {
      const Layer& L = layers_[runs_[r]];
      const Dyt& next = r + 1 < runs_.size() ? layers_[runs_[r + 1]].n1 : final_;
      const int64_t ldqd = L.qd_n(), HR = static_cast<int64_t>(L.heads) * L.kv_rank, HV = static_cast<int64_t>(L.heads) * L.vdim;
      const int qh = L.dim + L.rot_dim;
      uint8_t* qd = static_cast<uint8_t*>(qd_);
      // q and the compressed kv in one projection: rows [q heads | latent | shared rotated key]
      RUN(lin(qd_, normed_, L.qdkv, L.qd_n(), W, W, ldqd, act_dt, "q + compressed kv projection"));
      RUN(nvllm_latent_prepare(qd_, ldqd, qd + static_cast<size_t>(L.qdim()) * esz_, ldqd, L.c_norm, eps_, v.positions, L.rope,
                               L.rot_dims, lim_.max_positions, N, L.heads, L.dim, L.rot_dim, L.kv_rank, cache_[r], L.cache_row(),
                               v.slots, dt_, st)); ++launches; mk("latent_prepare");
      // fold the key up-projection into the query: qa[t, h, :] = Uk_h^T q[t, h, :dim]  (f32)
      // Per-head projections: with many tokens every head is a tensor-core GEMM of its own (views into the packed
      // activations); with few (decoding) one batched launch of the tile kernel beats `heads` launch latencies.
      const bool head_gemms = dt_ == NVLLM_BF16 && N >= 512 && L.dim % 64 == 0 && L.kv_rank % 64 == 0 && L.vdim % 8 == 0 &&
                              qh % 8 == 0 && ldqd % 8 == 0;
      if (L.dim > 0 && head_gemms) {
        for (int hh = 0; hh < L.heads; ++hh) {
          RUN(nvllm_gemm_bf16(q_abs_ + static_cast<size_t>(hh) * L.kv_rank, qd + static_cast<size_t>(hh) * qh * 2,
                              static_cast<uint8_t*>(L.ukT) + static_cast<size_t>(hh) * L.kv_rank * L.dim * 2, N, L.kv_rank, L.dim, ldqd,
                              L.dim, HR, NVLLM_F32, nullptr, 0, st)); ++launches;
        }
        mk("q absorb (per-head GEMMs)");
      } else if (L.dim > 0) {
        RUN(nvllm_linear(q_abs_, qd_, L.ukT, N, L.kv_rank, L.dim, ldqd, L.dim, HR, L.heads, qh, static_cast<int64_t>(L.kv_rank) * L.dim,
                         L.kv_rank, dt_, NVLLM_F32, st)); ++launches; mk("q absorb (per-head linear)");
      } else {
        NVLLM_CUDA(cudaMemsetAsync(q_abs_, 0, static_cast<size_t>(N) * HR * 4, static_cast<cudaStream_t>(st)));
      }
      RUN(nvllm_latent_attention(o_lat_, HR, q_abs_, HR, qd_, ldqd, v.tok_seq, v.positions, v.tables, v.table_cap, lim_.block_size,
                                 cache_[r], L.cache_row(), N, L.heads, L.dim, L.rot_dim, L.kv_rank, L.scale, dt_, st)); ++launches; mk("latent_attention");
      // values: per head Uv_h applied to the attended latent, then the output projection
      if (head_gemms) {
        for (int hh = 0; hh < L.heads; ++hh) {
          RUN(nvllm_gemm_bf16(static_cast<uint8_t*>(attn_) + static_cast<size_t>(hh) * L.vdim * 2,
                              static_cast<uint8_t*>(o_lat_) + static_cast<size_t>(hh) * L.kv_rank * 2,
                              static_cast<uint8_t*>(L.uv) + static_cast<size_t>(hh) * L.vdim * L.kv_rank * 2, N, L.vdim, L.kv_rank, HR,
                              L.kv_rank, HV, NVLLM_BF16, nullptr, 0, st)); ++launches;
        }
        mk("value up-projection (per-head GEMMs)");
      } else {
        RUN(nvllm_linear(attn_, o_lat_, L.uv, N, L.vdim, L.kv_rank, HR, L.kv_rank, HV, L.heads, L.kv_rank,
                         static_cast<int64_t>(L.vdim) * L.kv_rank, L.vdim, dt_, act_dt, st)); ++launches; mk("value up-projection (per-head linear)");
      }
      RUN(lin(proj_, attn_, L.o, W, static_cast<int>(HV), HV, W, act_dt, "attention output projection"));
      if (!L.has_mlp) {
        RUN(nvllm_dyt_residual_norm(normed_, h_, proj_, L.n1b.alpha, L.n1b.w, L.n1b.b, next.alpha, next.w, next.b, N, W, dt_, st)); ++launches; mk("dyt_residual_norm");
      } else {
        RUN(nvllm_dyt_residual_norm(normed_, h_, proj_, L.n1b.alpha, L.n1b.w, L.n1b.b, L.n2.alpha, L.n2.w, L.n2.b, N, W, dt_, st)); ++launches; mk("dyt_residual_norm");
        const int et = L.experts + L.identity;
        RUN(lin(router_logits_, normed_, L.router, et, W, W, et, NVLLM_F32, "router logits"));
        RUN(nvllm_moe_route(topk_idx_, topk_w_, router_logits_, L.correction, N, et, L.top, L.router_scale, st)); ++launches; mk("moe_route");
        const int rows = nvllm_moe_max_rows(N, L.top, L.experts, L.tile_rows);
        RUN(nvllm_moe_sort(row_token_, tile_expert_, slot_row_, topk_idx_, N, L.top, L.experts, rows, L.tile_rows, st)); ++launches; mk("moe_sort");
        if (L.experts > 0 && L.tile_rows == 128) {
          // tensor cores: gather the rows by expert, [gate | up] in one grouped GEMM, activation, grouped down projection
          RUN(nvllm_gather_rows(xg_, normed_, row_token_, rows, W, N, dt_, st)); ++launches; mk("expert row gather");
          RUN(nvllm_gemm_bf16_grouped(egu_buf_, xg_, L.egu, rows, 2 * L.ff, W, L.experts, W, W, 2 * L.ff, tile_expert_, st)); ++launches; mk("expert gate_up grouped GEMM");
          RUN(nvllm_glu_clamped(act_, egu_buf_, rows, L.ff, L.limit, dt_, st)); ++launches; mk("expert glu_clamped");
          RUN(nvllm_gemm_bf16_grouped(eout_, act_, L.edown, rows, W, L.ff, L.experts, L.ff, L.ff, W, tile_expert_, st)); ++launches; mk("expert down grouped GEMM");
        } else if (L.experts > 0) {
          RUN(nvllm_linear_grouped(act_, normed_, L.egu, rows, L.ff, W, W, W, L.ff, static_cast<int64_t>(2) * L.ff * W, row_token_,
                                   tile_expert_, 1, L.limit, dt_, act_dt, st)); ++launches; mk("expert gate_up+glu grouped tile kernel");
          RUN(nvllm_linear_grouped(eout_, act_, L.edown, rows, W, L.ff, L.ff, L.ff, W, static_cast<int64_t>(W) * L.ff, nullptr,
                                   tile_expert_, 0, 0.f, dt_, act_dt, st)); ++launches; mk("expert down grouped tile kernel");
        }
        if (L.has_shared) {
          RUN(lin(sgu_buf_, normed_, L.sgu, 2 * L.sff, W, W, 2 * L.sff, act_dt, "shared gate_up projection"));
          RUN(nvllm_glu_clamped(sact_, sgu_buf_, N, L.sff, L.slimit, dt_, st)); ++launches; mk("shared glu_clamped");
          RUN(lin(sout_, sact_, L.sdown, W, L.sff, L.sff, W, act_dt, "shared down projection"));
        }
        RUN(nvllm_moe_combine(moe_out_, eout_, normed_, L.has_shared ? sout_ : nullptr, topk_idx_, topk_w_, slot_row_, N, W, L.top,
                              L.experts, dt_, st)); ++launches; mk("moe_combine");
        RUN(nvllm_dyt_residual_norm(normed_, h_, moe_out_, L.n2b.alpha, L.n2b.w, L.n2b.b, next.alpha, next.w, next.b, N, W, dt_, st)); ++launches; mk("dyt_residual_norm");
      }
      if (v.layer_tap != nullptr && !v.capturing)
        NVLLM_CUDA(cudaMemcpyAsync(v.layer_tap + r * static_cast<size_t>(N) * W, h_, static_cast<size_t>(N) * W * 4, cudaMemcpyDeviceToHost,
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
      RUN(nvllm_linear(v.logits, head_in_, head_, v.n_logit_rows, vocab_, W, W, W, vocab_, 1, 0, 0, 0, dt_, NVLLM_F32, st));
      mk("head projection");
    }
    return 0;
  }
};

}  // namespace

ModelImpl* make_kosazen(const json::Value& cfg) {
  Kosazen* m = new Kosazen();
  if (m->parse(cfg) != 0) { delete m; return nullptr; }
  return m;
}

// ---- registry --------------------------------------------------------------------------------------------------
namespace {
struct Entry { const char* name; ModelImpl* (*make)(const json::Value&); };
const Entry kRegistry[] = {{"Kosazen", make_kosazen}, {"Talapel", make_talapel}, {"Zudatar", make_zudatar}, {"Zasorax", make_zasorax}};
}  // namespace

const char* registered_architectures() { return "Qwen3 (built in: qwen3-0.6b, qwen3-8b, qwen3-32b, ...), Kosazen, Talapel, Zudatar, Zasorax"; }

ModelImpl* make_model(const json::Value& cfg) {
  const std::string arch = cfg["architecture"].as_string();
  for (const Entry& e : kRegistry)
    if (arch == e.name) {
      try {
        return e.make(cfg);
      } catch (const std::exception& ex) {
        set_error("%s", ex.what());
        return nullptr;
      }
    }
  set_error("no model registered for architecture '%s' (known: %s)", arch.c_str(), registered_architectures());
  return nullptr;
}

}  // namespace nvllm
