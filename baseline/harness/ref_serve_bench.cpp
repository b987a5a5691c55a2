// Benchmark harness around the UNMODIFIED reference library (Scifan/Tesseract): continuous batching of N
// requests through the reference's own models::ContinuousBatchingScheduler, the loop its examples/llama_serve.cpp
// drives (add_request ... while has_pending(): step()), with the model shape, request mix and engine limits taken
// from the command line instead of the example's tiny synthetic ones. Nothing of tesseract_b200 is linked.
//
// Timing is wall clock around step() (every step ends with the scheduler's own device-to-host logit reads, so the
// device is idle when it returns). Requests are admitted first-in first-out inside step(), and a request emits its
// first token in the step that admits it, so time-to-first-token of a request is the end time of that step; the
// number admitted per step is read from num_waiting(). Steps that admitted nothing are pure decode steps: the
// decode rate is taken over those.
//
// Prints one JSON line; {"ok": false, "error": ...} when the reference throws. Exit code 0 either way.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <exception>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "tesseract/core/Tensor.hpp"
#include "tesseract/models/Llama.hpp"
#include "tesseract/models/Scheduler.hpp"

using namespace tesseract;
using namespace tesseract::models;

namespace {

struct Args {
  int64_t requests = 256, layers = 32, max_batch = 256;
  int64_t vocab = 128256, hidden = 4096, heads = 32, kv_heads = 8, ffn = 14336;
  int64_t prompt_lo = 128, prompt_hi = 2048, out_lo = 64, out_hi = 512;
  double rope_theta = 500000.0, top_p = 1.0, temperature = 0.0, time_limit_s = 0.0;
  int kv_int8 = 0;
  std::string dtype = "bf16", device = "cuda";   // "cpu" only for a smoke test of the harness itself
};

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (c == '\n' || c == '\r' || c == '\t') o += ' ';
    else o += c;
  }
  return o;
}

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int run(const Args& a) {
  const bool on_gpu = a.device != "cpu";
  const Device dev = on_gpu ? Device{DeviceType::CUDA, 0} : cpu_device();
  const int64_t max_seq = a.prompt_hi + a.out_hi;
  LlamaConfig cfg;
  cfg.vocab_size = a.vocab;
  cfg.hidden_size = a.hidden;
  cfg.num_hidden_layers = a.layers;
  cfg.num_attention_heads = a.heads;
  cfg.num_key_value_heads = a.kv_heads;
  cfg.intermediate_size = a.ffn;
  cfg.max_position_embeddings = max_seq;
  cfg.rope_theta = a.rope_theta;
  cfg.dtype = a.dtype == "bf16" ? DType::BFloat16 : a.dtype == "f16" ? DType::Float16 : DType::Float32;
  auto model = std::make_shared<LlamaModel>(cfg);
  model->to(dev);
  model->eval();

  std::mt19937_64 rng(0);
  auto uni = [&](int64_t lo, int64_t hi) { return lo + static_cast<int64_t>(rng() % static_cast<uint64_t>(hi - lo + 1)); };
  std::vector<std::vector<int32_t>> prompts;
  std::vector<int64_t> outs;
  int64_t total_tokens = 0, prompt_tokens = 0, gen_tokens = 0;
  for (int64_t r = 0; r < a.requests; ++r) {
    const int64_t p = uni(a.prompt_lo, a.prompt_hi), o = uni(a.out_lo, a.out_hi);
    std::vector<int32_t> ids(static_cast<size_t>(p));
    for (auto& t : ids) t = static_cast<int32_t>(rng() % static_cast<uint64_t>(a.vocab));
    prompts.push_back(std::move(ids));
    outs.push_back(o);
    total_tokens += p + o;
    prompt_tokens += p;
    gen_tokens += o;
  }

  EngineConfig ec;
  ec.block_size = 16;
  ec.num_blocks = total_tokens / 16 + a.requests + 64;   // every request can be resident at once
  ec.max_seq_len = max_seq;
  ec.max_batch_size = a.max_batch;
  ec.kv_int8 = a.kv_int8 != 0;
  ContinuousBatchingScheduler sched(model, ec);

  auto gen_cfg = [&](int64_t max_new, uint64_t seed) {
    LlamaModel::GenerateConfig g;
    g.max_new_tokens = max_new;
    g.eos_token_id = -1;
    if (a.temperature > 0.0) {
      g.do_sample = true;
      g.seed = seed;
      g.sampling.temperature = a.temperature;
      g.sampling.top_p = a.top_p;
    }
    return g;
  };

  // warm-up: one short request end to end (cuBLASLt heuristics, allocator buckets)
  {
    std::vector<int32_t> w(prompts[0].begin(), prompts[0].begin() + std::min<int64_t>(64, static_cast<int64_t>(prompts[0].size())));
    sched.add_request(w, gen_cfg(4, 0));
    sched.run();
  }
  for (int64_t r = 0; r < a.requests; ++r) sched.add_request(prompts[static_cast<size_t>(r)], gen_cfg(outs[static_cast<size_t>(r)], static_cast<uint64_t>(r)));

  if (on_gpu) cudaDeviceSynchronize();
  const double t0 = now_s();
  std::vector<double> ttft;
  double decode_s = 0.0, admit_s = 0.0;
  int64_t decode_tokens = 0, steps = 0, admitted_total = 0;
  bool cut_short = false;
  while (sched.has_pending()) {
    const int64_t waiting_before = sched.num_waiting();
    const int64_t running_before = sched.num_running();
    const double s0 = now_s();
    sched.step();
    const double s1 = now_s();
    const int64_t admitted = waiting_before - sched.num_waiting();
    for (int64_t i = 0; i < admitted; ++i) ttft.push_back(s1 - t0);
    admitted_total += admitted;
    if (admitted == 0) {
      decode_s += s1 - s0;
      decode_tokens += running_before;      // one token per running request in a pure decode step
    } else {
      admit_s += s1 - s0;
    }
    ++steps;
    if (a.time_limit_s > 0.0 && s1 - t0 > a.time_limit_s) { cut_short = true; break; }
  }
  if (on_gpu) cudaDeviceSynchronize();
  const double wall = now_s() - t0;
  std::sort(ttft.begin(), ttft.end());
  const double ttft_p50 = ttft.empty() ? -1.0 : ttft[ttft.size() / 2];
  size_t free_b = 0, total_b = 0;
  if (on_gpu) cudaMemGetInfo(&free_b, &total_b);
  std::printf(
      "{\"ok\": true, \"requests\": %lld, \"kv\": \"%s\", \"sampling\": \"%s\", \"dtype\": \"%s\", \"layers\": %lld, "
      "\"max_batch\": %lld, \"block_size\": 16, \"end_to_end_s\": %.3f, \"steps\": %lld, \"cut_short\": %s, "
      "\"admitted\": %lld, \"prompt_tokens\": %lld, \"generated_tokens\": %lld, \"total_tok_s\": %.2f, "
      "\"decode_tok_s\": %.2f, \"decode_steps_s\": %.3f, \"decode_tokens_counted\": %lld, \"admit_steps_s\": %.3f, "
      "\"ttft_p50_ms\": %.2f, \"device_mem_used_gb\": %.1f}\n",
      static_cast<long long>(a.requests), a.kv_int8 ? "int8" : a.dtype.c_str(),
      a.temperature > 0.0 ? "top_p" : "greedy", a.dtype.c_str(), static_cast<long long>(a.layers),
      static_cast<long long>(a.max_batch), wall, static_cast<long long>(steps), cut_short ? "true" : "false",
      static_cast<long long>(admitted_total), static_cast<long long>(prompt_tokens), static_cast<long long>(gen_tokens),
      cut_short ? 0.0 : static_cast<double>(total_tokens) / wall,
      decode_s > 0.0 ? static_cast<double>(decode_tokens) / decode_s : 0.0, decode_s,
      static_cast<long long>(decode_tokens), admit_s, ttft_p50 * 1e3, static_cast<double>(total_b - free_b) / 1e9);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  Args a;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i];
    const char* v = argv[i + 1];
    if (k == "--requests") a.requests = std::atoll(v);
    else if (k == "--layers") a.layers = std::atoll(v);
    else if (k == "--max-batch") a.max_batch = std::atoll(v);
    else if (k == "--vocab") a.vocab = std::atoll(v);
    else if (k == "--hidden") a.hidden = std::atoll(v);
    else if (k == "--heads") a.heads = std::atoll(v);
    else if (k == "--kv-heads") a.kv_heads = std::atoll(v);
    else if (k == "--ffn") a.ffn = std::atoll(v);
    else if (k == "--prompt-lo") a.prompt_lo = std::atoll(v);
    else if (k == "--prompt-hi") a.prompt_hi = std::atoll(v);
    else if (k == "--out-lo") a.out_lo = std::atoll(v);
    else if (k == "--out-hi") a.out_hi = std::atoll(v);
    else if (k == "--kv-int8") a.kv_int8 = std::atoi(v);
    else if (k == "--top-p") a.top_p = std::atof(v);
    else if (k == "--temperature") a.temperature = std::atof(v);
    else if (k == "--time-limit") a.time_limit_s = std::atof(v);
    else if (k == "--dtype") a.dtype = v;
    else if (k == "--device") a.device = v;
    else { std::fprintf(stderr, "unknown flag %s\n", k.c_str()); return 2; }
  }
  try {
    return run(a);
  } catch (const std::exception& e) {
    std::printf("{\"ok\": false, \"error\": \"%s\"}\n", json_escape(e.what()).c_str());
    return 0;
  }
}
