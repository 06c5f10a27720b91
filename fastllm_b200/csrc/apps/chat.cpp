// Command-line chat over the C ABI: reads one user turn per line, streams the reply, keeps the conversation.
// "reset" starts over, "stop" / "exit" / end of input leaves.  (The reference's counterpart: main.cpp, its CLI chat.)
//
//   fastllm_chat -p <model folder> [--dtype auto] [--device cuda|cpu] [--options JSON] [--system TEXT]
//                [--max_tokens 512] [--temperature T] [--top_p P] [--top_k K] [--repeat_penalty R]
#include <unistd.h>

#include <iostream>
#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  auto a = app::parse_args(argc, argv, {{"p", "path"}, {"t", "threads"}, {"d", "dtype"}});
  if (a.count("help") || a.count("h")) {
    printf("usage: %s -p <model folder> [--dtype D] [--device DEV] [--options JSON] [--system TEXT] [--max_tokens N] [--temperature T] "
           "[--top_p P] [--top_k K] [--repeat_penalty R]\n", argv[0]);
    return 0;
  }
  const int model = app::load_model(a);
  const std::string system = app::get(a, "system", "");
  std::string sampling = "\"max_tokens\": " + app::get(a, "max_tokens", "512");
  for (const char* k : {"temperature", "top_p", "top_k"})
    if (a.count(k)) sampling += std::string(", \"") + k + "\": " + a[k];
  if (a.count("repeat_penalty")) sampling += ", \"repetition_penalty\": " + a["repeat_penalty"];

  std::vector<std::pair<std::string, std::string>> turns;      // (role, content)
  auto reset = [&] { turns.clear(); if (!system.empty()) turns.push_back({"system", system}); };
  reset();
  const bool tty = isatty(0);
  std::string line;
  while (true) {
    if (tty) { printf("user: "); fflush(stdout); }
    if (!std::getline(std::cin, line)) break;
    if (line == "stop" || line == "exit") break;
    if (line == "reset") { reset(); continue; }
    if (line.empty()) continue;
    turns.push_back({"user", line});
    std::string body = "{\"messages\": [";
    for (size_t i = 0; i < turns.size(); ++i)
      body += std::string(i ? ", " : "") + "{\"role\": \"" + turns[i].first + "\", \"content\": \"" + app::json_escape(turns[i].second) + "\"}";
    body += "], " + sampling + "}";
    const int h = launch_request_json_llm_model(model, body.c_str());
    if (h < 0) { fprintf(stderr, "request failed: %s\n", fastllm_last_error()); turns.pop_back(); continue; }
    printf("assistant: ");
    std::string reply;
    while (char* piece = fetch_response_str_llm_model(model, h)) {
      fputs(piece, stdout);
      fflush(stdout);
      reply += piece;
      fastllm_free(piece);
    }
    printf("\n");
    turns.push_back({"assistant", reply});
  }
  release_memory(model);
  return 0;
}
