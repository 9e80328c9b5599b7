// model.hpp — what the runner needs from a model architecture, and the registry that maps the `architecture` string of a
// model's config.json to an implementation.  The runner owns the stream, the step metadata (ids, positions, slots, block
// tables, the sequence of every token), the logits, sampling and CUDA-graph capture; a model owns its weights, its cache
// (one region per layer run, addressed through the runner's block tables) and its activation buffers.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "json.hpp"
#include "../../../include/nvllm_engine.h"

namespace nvllm {

struct ModelLimits {
  int max_tokens = 0;   // tokens of one step
  int max_seqs = 0;
  int num_blocks = 0, block_size = 0, table_cap = 0;
  int max_positions = 0;
  int dtype = 0;        // NVLLM_BF16: bf16 operands, f32 where the architecture says so; NVLLM_F32: everything in f32
};

// One step as the runner uploaded it (device pointers).  Every token carries its own sequence index and position, so a
// step may hold whole prompts, portions of prompts and single decoded tokens side by side.
struct StepView {
  cudaStream_t stream = nullptr;
  int n_tokens = 0, n_seqs = 0;
  const int64_t* ids = nullptr;
  const int64_t* positions = nullptr;
  const int32_t* slots = nullptr;     // cache slot of every token (< 0: padding row of a captured graph, nothing stored)
  const int32_t* tok_seq = nullptr;   // row of `tables` of every token
  const int32_t* tables = nullptr;    // [n_seqs, table_cap]
  int table_cap = 0;
  const int32_t* cu_tokens = nullptr;   // [n_seqs + 1] token range of every sequence in the step (tokens in order of position)
  const int32_t* seq_slots = nullptr;   // [n_seqs] recurrent-state slot of every sequence (< 0: padding sequence), or null
  const int32_t* logit_rows = nullptr;  // tokens whose logits are wanted
  int n_logit_rows = 0;
  float* logits = nullptr;            // [n_logit_rows, vocab]
  float* layer_tap = nullptr;         // host memory, or null: the f32 residual stream after every layer run, [runs, n_tokens, width]
  bool capturing = false;
  bool whole_prompts = false;         // every sequence of the step starts at position 0 (known on the host): its keys are the step's own rows
  // per-launch profile of eager steps (nvllm_runner_profile): called after every launch with the kernel's name
  void (*mark)(void* ctx, const char* name) = nullptr;
  void* mark_ctx = nullptr;
};

class ModelImpl {
 public:
  virtual ~ModelImpl() {}
  virtual int vocab() const = 0;
  virtual int hidden() const = 0;
  virtual int layer_runs() const = 0;
  // true: the model keeps a fixed-size state per sequence in one of ModelLimits::max_seqs slots (StepView::seq_slots)
  virtual bool recurrent_state() const { return false; }
  virtual int create(const ModelLimits& lim, cudaStream_t stream) = 0;
  virtual int init_weights(uint64_t seed, float std, cudaStream_t stream) = 0;
  virtual int load_weight(const char* name, const void* h_bf16, int64_t rows, int64_t cols, cudaStream_t stream) = 0;
  virtual bool weights_ready() const = 0;
  virtual int forward(const StepView& v) = 0;
  int64_t launches = 0;
};

// Returns a new model for the `architecture` named in the configuration, or nullptr (with nvllm_last_error set) when no
// implementation is registered under that name or the configuration is malformed.
ModelImpl* make_model(const json::Value& cfg);
// Architectures the registry knows, comma-separated (error messages, command line help).
const char* registered_architectures();

ModelImpl* make_kosazen(const json::Value& cfg);  // kosazen_model.cu
ModelImpl* make_talapel(const json::Value& cfg);  // talapel_model.cu
ModelImpl* make_zudatar(const json::Value& cfg);  // zudatar_model.cu
ModelImpl* make_zasorax(const json::Value& cfg);  // zasorax_model.cu

}  // namespace nvllm
