// C ABI of fastllm_b200 for hosts that are not Python (C, C++, anything with a C foreign-function interface).
//
// The library embeds the interpreter that runs the engine's scheduling thread; the calls below are safe from any host thread.
// Models and requests are named by small integers.  Functions that return `char*` hand out malloc'd, NUL-terminated UTF-8
// that the caller releases with fastllm_free; a NULL / negative result means failure and fastllm_last_error() tells why
// (per thread).  Counterpart in the reference: tools/src/pytools.cpp (the C ABI under its Python package).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Start the embedded interpreter.  `python_executable`: the interpreter whose environment (site-packages) holds torch;
// NULL takes $FASTLLM_PYTHON, else the first `python3` on PATH.  Called implicitly by the first create_* call.
int fastllm_init(const char* python_executable);
const char* fastllm_last_error(void);
void fastllm_free(void* p);

// dtype: "auto", "float16", "bfloat16", "int8", "int4g128", "fp8", "nvfp4" ...; options_json: "" or a JSON object of further
// model / engine options ({"device": "cpu", "kv_cache_dtype": "fp8_e4m3", "max_batch": 64, "tp": 2, ...}).
int create_llm_model_fromhf(const char* path, const char* dtype, const char* options_json);
void release_memory(int model);
int set_option_llm_model(int model, const char* name, const char* value);
char* get_info_llm_model(int model);            // JSON: type, vocab_size, max_input_len, kv_cache_token_limit, max_batch

struct fastllm_generation_config {              // zero / negative fields take the model's defaults
  int max_length, min_length, do_sample, top_k;
  float top_p, temperature, repeat_penalty;
  int stop_token_cnt;
  const int* stop_token_ids;
};

int launch_response_llm_model(int model, int len, const int* token_ids, const struct fastllm_generation_config* cfg);
int launch_response_str_llm_model(int model, const char* content, int as_chat, const struct fastllm_generation_config* cfg);
int launch_request_json_llm_model(int model, const char* chat_completions_body);
int request_wants_stream(const char* chat_completions_body);  // 1 when the body asks for "stream": true
int can_fetch_response_llm_model(int model, int handle);
int fetch_response_llm_model(int model, int handle);          // next token id (blocking); -1 ended; -2 error
char* fetch_response_str_llm_model(int model, int handle);    // next text piece (may be ""); NULL ended (or error: see last_error)
void abort_response_llm_model(int model, int handle);
char* response_str_llm_model(int model, const char* content, int as_chat, const struct fastllm_generation_config* cfg);
char* get_response_statistics_llm_model(int model, int handle);   // JSON

int token_encode_string(int model, const char* content, int capacity, int* out_ids);   // number of ids (may exceed capacity)
int token_decode(int model, int token_id, int capacity, char* out_bytes);               // number of bytes (may exceed capacity)
char* apply_chat_template(int model, const char* messages_json);

#ifdef __cplusplus
}
#endif
