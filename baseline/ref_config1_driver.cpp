// Times the UNMODIFIED reference (xprimesamx/MYTHOS.cpp) on the tiny byte-level configuration:
// 4 layers, d_model 256, 4 heads of 64, SwiGLU FFN 1024, vocab 256, context 128, batch 16, AdamW
// lr 3e-4, seeded Zipf(1.1) byte ids. It links the reference's own static libraries (built by
// baseline/build_reference.py from the reference's CMake project) and calls its stock public API:
// oil::DenseModel, oil::AdamW, oil::Trainer::compile and oil::Trainer::train_step
// (src/trainer.cpp:583-606). The reference trains in FP32 on the CPU and does not wire the
// straight-through quantiser into this loop (include/oil/trainer.h:32 is unused), so this is its
// FP32 number. Prints one JSON line: tokens per second over the timed steps and the last loss.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "oil/model.h"
#include "oil/optimizer.h"
#include "oil/trainer.h"

int main(int argc, char** argv) {
  const int steps = argc > 1 ? std::atoi(argv[1]) : 20;
  const int warmup = argc > 2 ? std::atoi(argv[2]) : 2;
  const int64_t B = 16, S = 128, V = 256;
  oil::TransformerConfig cfg;
  cfg.vocab_size = V;
  cfg.hidden_size = 256;
  cfg.num_layers = 4;
  cfg.num_heads = 4;
  cfg.head_dim = 64;
  cfg.ffn_hidden_size = 1024;
  cfg.max_seq_len = S;
  oil::DenseModel model(cfg);
  oil::AdamW opt(3e-4f);
  oil::Trainer trainer(&model, nullptr);
  oil::TrainConfig tc;
  tc.batch_size = B;
  tc.seq_length = S;
  tc.learning_rate = 3e-4f;
  tc.warmup_steps = 0;
  tc.schedule = oil::AdamW::Schedule::CONSTANT;
  trainer.compile(&opt, tc);

  // Zipf(1.1) over 256 byte ids, seeded
  std::vector<double> cdf(V);
  double z = 0;
  for (int i = 0; i < V; ++i) z += 1.0 / std::pow(i + 1.0, 1.1);
  double acc = 0;
  for (int i = 0; i < V; ++i) { acc += 1.0 / std::pow(i + 1.0, 1.1) / z; cdf[i] = acc; }
  std::mt19937_64 rng(1234);
  std::uniform_real_distribution<double> uni(0.0, 1.0);
  auto draw = [&]() {
    const double u = uni(rng);
    int lo = 0, hi = V - 1;
    while (lo < hi) { const int mid = (lo + hi) / 2; if (cdf[mid] < u) lo = mid + 1; else hi = mid; }
    return (float)lo;
  };
  oil::Tensor ids(oil::Shape{B, S}, oil::DType::F32), labels(oil::Shape{B, S}, oil::DType::F32);
  auto fill = [&]() {
    float* a = ids.data<float>();
    float* t = labels.data<float>();
    for (int64_t b = 0; b < B; ++b) {
      float prev = draw();
      for (int64_t s = 0; s < S; ++s) { const float nx = draw(); a[b * S + s] = prev; t[b * S + s] = nx; prev = nx; }
    }
  };
  float loss = 0;
  for (int i = 0; i < warmup; ++i) { fill(); loss = trainer.train_step(ids, labels); }
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < steps; ++i) { fill(); loss = trainer.train_step(ids, labels); }
  const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  std::printf("{\"impl\": \"reference\", \"config\": \"tiny-byte 4L d256 4h ffn1024 v256 ctx128 batch16 fp32 cpu\", "
              "\"steps\": %d, \"tokens_per_s\": %.1f, \"ms_per_step\": %.2f, \"last_loss\": %.4f}\n",
              steps, steps * (double)(B * S) / sec, sec / steps * 1e3, loss);
  return 0;
}
