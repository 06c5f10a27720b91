// Throughput benchmark over the C ABI: `batch` concurrent requests of `prompt_len` tokens, `output_len` greedy tokens each.
// Prints the time to the first token of every request (prefill) and the decode rate after it.
// (The reference's counterpart: example/benchmark/benchmark.cpp.)
//
//   fastllm_benchmark -p <model folder> [-b 16] [--prompt_len 128 | -f prompt.txt] [-l 128] [--dtype D] [--device DEV] [--options JSON]
#include <chrono>
#include <fstream>
#include <random>
#include <sstream>
#include <vector>

#include "app_common.h"

static double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

int main(int argc, char** argv) {
  auto a = app::parse_args(argc, argv, {{"p", "path"}, {"b", "batch"}, {"l", "output_len"}, {"f", "file"}, {"d", "dtype"}});
  if (a.count("help") || a.count("h")) {
    printf("usage: %s -p <model folder> [-b batch] [--prompt_len N | -f prompt.txt] [-l output tokens] [--dtype D] [--device DEV] [--options JSON]\n", argv[0]);
    return 0;
  }
  const int model = app::load_model(a);
  const int batch = atoi(app::get(a, "batch", "16").c_str());
  const int out_len = atoi(app::get(a, "output_len", "128").c_str());
  int prompt_len = atoi(app::get(a, "prompt_len", "128").c_str());

  char* info = get_info_llm_model(model);
  int vocab = 32000;
  if (info) {
    if (const char* v = strstr(info, "\"vocab_size\": ")) vocab = atoi(v + 14);
    fastllm_free(info);
  }
  std::vector<std::vector<int>> prompts(batch);
  if (a.count("file")) {
    std::ifstream f(a["file"]);
    std::stringstream ss;
    ss << f.rdbuf();
    std::vector<int> ids(1 << 20);
    const int n = token_encode_string(model, ss.str().c_str(), (int)ids.size(), ids.data());
    if (n <= 0) { fprintf(stderr, "empty prompt file or tokeniser error: %s\n", fastllm_last_error()); return 1; }
    ids.resize(n < (int)ids.size() ? n : ids.size());
    for (auto& p : prompts) p = ids;
    prompt_len = (int)ids.size();
  } else {
    std::mt19937 rng(1);
    for (auto& p : prompts) {
      p.resize(prompt_len);
      for (int& t : p) t = (int)(rng() % (unsigned)vocab);      // different prompts: no prefix-cache hits between requests
    }
  }

  fastllm_generation_config cfg = {};
  cfg.max_length = out_len; cfg.min_length = out_len; cfg.do_sample = 0; cfg.top_k = 1;
  // warm-up: one short request (kernel loading, graph capture)
  {
    const int h = launch_response_llm_model(model, prompt_len < 16 ? prompt_len : 16, prompts[0].data(), &cfg);
    if (h < 0) { fprintf(stderr, "warm-up failed: %s\n", fastllm_last_error()); return 1; }
    for (int i = 0; i < 4 && fetch_response_llm_model(model, h) >= 0; ++i) {}
    abort_response_llm_model(model, h);
  }

  std::vector<int> handles(batch);
  const double t0 = now_s();
  for (int i = 0; i < batch; ++i) {
    handles[i] = launch_response_llm_model(model, prompt_len, prompts[i].data(), &cfg);
    if (handles[i] < 0) { fprintf(stderr, "launch failed: %s\n", fastllm_last_error()); return 1; }
  }
  long total = 0;
  std::vector<bool> live(batch, true);
  for (int i = 0; i < batch; ++i) {                         // first token of every request
    if (fetch_response_llm_model(model, handles[i]) < 0) live[i] = false; else ++total;
  }
  const double t1 = now_s();
  int alive = batch;
  long decoded = 0;
  while (alive > 0) {
    alive = 0;
    for (int i = 0; i < batch; ++i) {
      if (!live[i]) continue;
      if (fetch_response_llm_model(model, handles[i]) < 0) live[i] = false; else { ++decoded; ++alive; }
    }
  }
  const double t2 = now_s();
  printf("batch %d, prompt %d tokens, output up to %d tokens\n", batch, prompt_len, out_len);
  printf("prefill: %.3f s (%.1f prompt tokens/s)\n", t1 - t0, (double)batch * prompt_len / (t1 - t0));
  printf("decode: %ld tokens in %.3f s (%.1f tokens/s)\n", decoded, t2 - t1, decoded > 0 ? decoded / (t2 - t1) : 0.0);
  printf("total: %ld output tokens in %.3f s (%.1f tokens/s)\n", total + decoded, t2 - t0, (total + decoded) / (t2 - t0));
  release_memory(model);
  return 0;
}
