// Benchmark harness around the UNMODIFIED reference library (Scifan/Tesseract): one Llama training step
// (forward + cross-entropy + backward + Adam) timed on the device, driven only through the reference's own
// public C++ API -- the same calls its examples/llama_train.cpp makes (LlamaModel, ops::cross_entropy_with_logits,
// Engine::backward, optim::Adam), with the model shape taken from the command line instead of the example's
// hard-coded tiny one. Nothing of tesseract_b200 is linked.
//
// Prints one JSON line: {"ok": true, "ms_per_step": ..., "e2e_ms_per_step": ..., "loss": ..., ...} or
// {"ok": false, "error": "<exception text>"}; exit code 0 in both cases so the caller can read the line.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <memory>
#include <string>
#include <vector>

#include "tesseract/autograd/Engine.hpp"
#include "tesseract/core/Stream.hpp"
#include "tesseract/core/Tensor.hpp"
#include "tesseract/models/Llama.hpp"
#include "tesseract/ops/Loss.hpp"
#include "tesseract/ops/View.hpp"
#include "tesseract/optim/Adam.hpp"

using namespace tesseract;
using namespace tesseract::models;

namespace {

struct Args {
  int64_t steps = 4, warmup = 3, batch = 8, seq = 4096, micro = 1, layers = 32;
  int64_t vocab = 128256, hidden = 4096, heads = 32, kv_heads = 8, ffn = 14336;
  double rope_theta = 500000.0, lr = 1e-4, time_limit_s = 0.0;   // 0 = time exactly --steps steps
  std::string dtype = "bf16", device = "cuda";   // "cpu" only for a smoke test of the harness itself
  int e2e = 1;
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

uint64_t lcg_next(uint64_t& s) {
  s = s * 6364136223846793005ULL + 1442695040888963407ULL;
  return s >> 33;
}

float loss_value(const Tensor& loss) {
  Tensor h = loss.device().is_cpu() ? loss : loss.to(cpu_device());   // the per-step host read of the example
  switch (h.dtype()) {
    case DType::Float32: return *h.data_ptr<float>();
    case DType::Float64: return static_cast<float>(*h.data_ptr<double>());
    case DType::BFloat16: {
      uint16_t b; std::memcpy(&b, h.raw_data(), 2);
      uint32_t u = static_cast<uint32_t>(b) << 16; float f; std::memcpy(&f, &u, 4); return f;
    }
    default: return 0.f;   // fp16: value is not needed for the timing
  }
}

int run(const Args& a) {
  const bool on_gpu = a.device != "cpu";
  const Device dev = on_gpu ? Device{DeviceType::CUDA, 0} : cpu_device();
  LlamaConfig cfg;
  cfg.vocab_size = a.vocab;
  cfg.hidden_size = a.hidden;
  cfg.num_hidden_layers = a.layers;
  cfg.num_attention_heads = a.heads;
  cfg.num_key_value_heads = a.kv_heads;
  cfg.intermediate_size = a.ffn;
  cfg.max_position_embeddings = a.seq;
  cfg.rope_theta = a.rope_theta;
  cfg.dtype = a.dtype == "bf16" ? DType::BFloat16 : a.dtype == "f16" ? DType::Float16 : DType::Float32;

  auto t_init0 = std::chrono::steady_clock::now();
  auto model = std::make_shared<LlamaModel>(cfg);
  model->to(dev);
  optim::Adam opt(model->parameters(), a.lr);
  const double init_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_init0).count();

  // two synthetic batches of uniform random ids, [B, S+1]: inputs = [:, :-1], targets = [:, 1:]
  const int64_t B = a.batch, S = a.seq, mb = a.micro, n_micro = B / mb;
  std::vector<Tensor> host_in[2], host_tg[2], dev_in[2], dev_tg[2];
  uint64_t seed = 1000;
  for (int k = 0; k < 2; ++k) {
    for (int64_t m = 0; m < n_micro; ++m) {
      Tensor in = on_gpu ? Tensor::empty_pinned(Shape({mb, S}), DType::Int64) : Tensor::empty(Shape({mb, S}), DType::Int64);
      Tensor tg = on_gpu ? Tensor::empty_pinned(Shape(std::vector<int64_t>{mb * S}), DType::Int64)
                         : Tensor::empty(Shape(std::vector<int64_t>{mb * S}), DType::Int64);
      int64_t* pi = in.data_ptr<int64_t>();
      int64_t* pt = tg.data_ptr<int64_t>();
      for (int64_t b = 0; b < mb; ++b) {
        int64_t prev = static_cast<int64_t>(lcg_next(seed) % static_cast<uint64_t>(a.vocab));
        for (int64_t s = 0; s < S; ++s) {
          const int64_t nxt = static_cast<int64_t>(lcg_next(seed) % static_cast<uint64_t>(a.vocab));
          pi[b * S + s] = prev;
          pt[b * S + s] = nxt;
          prev = nxt;
        }
      }
      host_in[k].push_back(in);
      host_tg[k].push_back(tg);
      dev_in[k].push_back(in.to(dev));
      dev_tg[k].push_back(tg.to(dev));
    }
  }

  float last_loss = 0.f;
  auto step = [&](int k, bool from_host) {
    opt.zero_grad();
    float acc = 0.f;
    for (int64_t m = 0; m < n_micro; ++m) {
      Tensor in = from_host && on_gpu ? host_in[k][m].to(dev) : dev_in[k][m];
      Tensor tg = from_host && on_gpu ? host_tg[k][m].to(dev) : dev_tg[k][m];
      Tensor logits = model->forward(in);                                    // [mb, S, V]
      Tensor flat = ops::reshape(logits, Shape({mb * S, cfg.vocab_size}));
      Tensor loss = ops::cross_entropy_with_logits(flat, tg);
      if (n_micro == 1) {
        Engine::backward(loss);
      } else {
        Engine::backward(loss, Tensor::full(loss.shape(), 1.0 / static_cast<double>(n_micro), loss.dtype(), dev));
      }
      acc += loss_value(loss) / static_cast<float>(n_micro);
    }
    opt.step();
    last_loss = acc;
  };

  cudaStream_t stream = on_gpu ? static_cast<cudaStream_t>(current_stream(dev).native_handle()) : nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (on_gpu) {
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
  }
  auto timed = [&](bool from_host, int64_t steps) -> double {
    if (!on_gpu) {
      auto t0 = std::chrono::steady_clock::now();
      for (int64_t i = 0; i < steps; ++i) step(static_cast<int>(i % 2), from_host);
      return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    }
    cudaDeviceSynchronize();
    cudaEventRecord(e0, stream);
    for (int64_t i = 0; i < steps; ++i) step(static_cast<int>(i % 2), from_host);
    cudaEventRecord(e1, stream);
    cudaDeviceSynchronize();
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    return static_cast<double>(ms);
  };

  auto t_w0 = std::chrono::steady_clock::now();
  for (int64_t i = 0; i < a.warmup; ++i) step(static_cast<int>(i % 2), false);
  if (on_gpu) cudaDeviceSynchronize();
  const double warm_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_w0).count();
  const float first_loss = last_loss;

  // With a time limit the number of timed steps shrinks (never below 3) so that both timed regions end inside it;
  // the JSON line reports the number that was timed.
  int64_t steps = a.steps;
  if (a.time_limit_s > 0.0 && a.warmup > 0) {
    const double elapsed = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_init0).count();
    const double per_step = warm_s / static_cast<double>(a.warmup);
    const double regions = a.e2e ? 2.0 : 1.0;
    const int64_t fit = static_cast<int64_t>((a.time_limit_s - elapsed - per_step) / (regions * per_step));
    steps = std::max<int64_t>(3, std::min<int64_t>(a.steps, fit));
  }
  const double ms_dev = timed(false, steps);
  double ms_e2e = -1.0;
  if (a.e2e) {
    step(0, true);
    ms_e2e = timed(true, steps);
  }
  size_t free_b = 0, total_b = 0;
  if (on_gpu) cudaMemGetInfo(&free_b, &total_b);
  std::printf(
      "{\"ok\": true, \"ms_per_step\": %.4f, \"e2e_ms_per_step\": %.4f, \"steps\": %lld, \"warmup\": %lld, "
      "\"global_batch\": %lld, \"seq_len\": %lld, \"micro_batch\": %lld, \"layers\": %lld, \"dtype\": \"%s\", "
      "\"first_loss\": %.6f, \"loss\": %.6f, \"init_s\": %.1f, \"warmup_s\": %.1f, \"device_mem_used_gb\": %.1f, "
      "\"h2d_bytes_per_step\": %lld, \"d2h_bytes_per_step\": %lld}\n",
      ms_dev / static_cast<double>(steps), a.e2e ? ms_e2e / static_cast<double>(steps) : -1.0,
      static_cast<long long>(steps), static_cast<long long>(a.warmup), static_cast<long long>(B),
      static_cast<long long>(S), static_cast<long long>(mb), static_cast<long long>(a.layers), a.dtype.c_str(),
      first_loss, last_loss, init_s, warm_s, static_cast<double>(total_b - free_b) / 1e9,
      static_cast<long long>(B * S * 8 * 2), static_cast<long long>(n_micro * (cfg.dtype == DType::Float32 ? 4 : 2)));
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  Args a;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i];
    const char* v = argv[i + 1];
    if (k == "--steps") a.steps = std::atoll(v);
    else if (k == "--warmup") a.warmup = std::atoll(v);
    else if (k == "--batch") a.batch = std::atoll(v);
    else if (k == "--seq") a.seq = std::atoll(v);
    else if (k == "--micro") a.micro = std::atoll(v);
    else if (k == "--layers") a.layers = std::atoll(v);
    else if (k == "--vocab") a.vocab = std::atoll(v);
    else if (k == "--hidden") a.hidden = std::atoll(v);
    else if (k == "--heads") a.heads = std::atoll(v);
    else if (k == "--kv-heads") a.kv_heads = std::atoll(v);
    else if (k == "--ffn") a.ffn = std::atoll(v);
    else if (k == "--dtype") a.dtype = v;
    else if (k == "--device") a.device = v;
    else if (k == "--time-limit") a.time_limit_s = std::atof(v);
    else if (k == "--rope-theta") a.rope_theta = std::atof(v);
    else if (k == "--e2e") a.e2e = std::atoi(v);
    else { std::fprintf(stderr, "unknown flag %s\n", k.c_str()); return 2; }
  }
  if (a.batch % a.micro != 0) { std::fprintf(stderr, "--batch must be a multiple of --micro\n"); return 2; }
  try {
    return run(a);
  } catch (const std::exception& e) {
    std::printf("{\"ok\": false, \"error\": \"%s\"}\n", json_escape(e.what()).c_str());
    return 0;
  }
}
