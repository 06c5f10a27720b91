// Shared helpers of the native command-line hosts (chat, benchmark, apiserver) over the C ABI (../capi/fastllm_b200.h).
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

#include "../capi/fastllm_b200.h"

namespace app {

// "--name value" / "-n value" pairs and bare "--flag"s; `alias` maps short to long names.
inline std::map<std::string, std::string> parse_args(int argc, char** argv, const std::map<std::string, std::string>& alias) {
  std::map<std::string, std::string> out;
  for (int i = 1; i < argc; ++i) {
    std::string k = argv[i];
    if (k.rfind("--", 0) == 0) k = k.substr(2);
    else if (k.rfind("-", 0) == 0) { auto it = alias.find(k.substr(1)); k = it == alias.end() ? k.substr(1) : it->second; }
    else { out["_"] = k; continue; }
    if (i + 1 < argc && (argv[i + 1][0] != '-' || (argv[i + 1][1] >= '0' && argv[i + 1][1] <= '9') || argv[i + 1][1] == 0)) out[k] = argv[++i];
    else out[k] = "1";
  }
  return out;
}

inline std::string get(const std::map<std::string, std::string>& a, const char* k, const char* dflt) {
  auto it = a.find(k);
  return it == a.end() ? dflt : it->second;
}

inline std::string json_escape(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 8);
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += (char)c;
    }
  }
  return o;
}

// Load the model named by -p / --path with --dtype and --options (JSON); exits with a message on failure.
inline int load_model(const std::map<std::string, std::string>& a) {
  const std::string path = get(a, "path", get(a, "_", "").c_str());
  if (path.empty()) { fprintf(stderr, "missing -p <model folder>\n"); exit(2); }
  std::string opts = get(a, "options", "");
  const std::string device = get(a, "device", "");
  if (opts.empty() && !device.empty()) opts = "{\"device\": \"" + json_escape(device) + "\"}";
  const int m = create_llm_model_fromhf(path.c_str(), get(a, "dtype", "auto").c_str(), opts.c_str());
  if (m < 0) { fprintf(stderr, "loading %s failed: %s\n", path.c_str(), fastllm_last_error()); exit(1); }
  return m;
}

}  // namespace app
