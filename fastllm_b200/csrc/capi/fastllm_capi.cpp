// C ABI host library: embeds CPython and forwards to fastllm_b200/capi.py (see fastllm_b200.h).
//
// Threading: the interpreter is started once; the starting thread then gives up the GIL, and every exported call takes it
// for the duration of the forwarded call (PyGILState).  The engine's scheduling thread is a Python thread and runs whenever
// the callers are blocked or outside the library.  Loaded into a process that already runs Python (ctypes), the library
// uses that interpreter.
#include <Python.h>

#include <climits>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include <dlfcn.h>
#include <unistd.h>

#include "fastllm_b200.h"

namespace {

thread_local std::string t_error;
std::mutex g_init_mu;
bool g_ready = false;
PyObject* g_mod = nullptr;      // fastllm_b200.capi

std::string find_python(const char* given) {
  if (given && *given) return given;
  if (const char* e = getenv("FASTLLM_PYTHON")) return e;
  std::string path = getenv("PATH") ? getenv("PATH") : "";
  size_t pos = 0;
  while (pos <= path.size()) {
    size_t end = path.find(':', pos);
    if (end == std::string::npos) end = path.size();
    std::string cand = path.substr(pos, end - pos) + "/python3";
    if (access(cand.c_str(), X_OK) == 0) return cand;
    pos = end + 1;
  }
  return "python3";
}

// the package root: this library sits in <root>/fastllm_b200/lib/
std::string package_root() {
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&package_root), &info) == 0 || info.dli_fname == nullptr) return ".";
  char resolved[PATH_MAX];
  std::string p = realpath(info.dli_fname, resolved) ? resolved : info.dli_fname;       // "bin/../lib/..." when found through an rpath
  for (int up = 0; up < 3; ++up) {
    size_t s = p.find_last_of('/');
    if (s == std::string::npos) return ".";
    p.erase(s);
  }
  return p.empty() ? "/" : p;
}

void set_error_from_python() {
  PyObject *type = nullptr, *value = nullptr, *tb = nullptr;
  PyErr_Fetch(&type, &value, &tb);
  PyErr_NormalizeException(&type, &value, &tb);
  t_error = "python error";
  if (value) {
    PyObject* s = PyObject_Str(value);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) t_error = c;
      Py_DECREF(s);
    }
    if (type) {
      PyObject* n = PyObject_GetAttrString(type, "__name__");
      if (n) {
        const char* c = PyUnicode_AsUTF8(n);
        if (c) t_error = std::string(c) + ": " + t_error;
        Py_DECREF(n);
      }
    }
  }
  PyErr_Clear();
  Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(tb);
}

bool ensure_init(const char* exe) {
  std::lock_guard<std::mutex> lk(g_init_mu);
  if (g_ready) return true;
  const bool own = !Py_IsInitialized();
  if (own) {
    PyConfig config;
    PyConfig_InitPythonConfig(&config);
    const std::string py = find_python(exe);
    PyStatus st = PyConfig_SetBytesString(&config, &config.program_name, py.c_str());
    if (!PyStatus_Exception(st)) st = PyConfig_SetBytesString(&config, &config.executable, py.c_str());
    config.install_signal_handlers = 0;
    if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
    PyConfig_Clear(&config);
    if (PyStatus_Exception(st)) {
      t_error = std::string("interpreter start failed: ") + (st.err_msg ? st.err_msg : "?");
      return false;
    }
  }
  PyGILState_STATE gs = own ? PyGILState_UNLOCKED : PyGILState_Ensure();
  bool ok = false;
  {
    PyObject* sys_path = PySys_GetObject("path");      // borrowed
    PyObject* root = PyUnicode_FromString(package_root().c_str());
    if (sys_path && root && PySequence_Contains(sys_path, root) == 0) PyList_Insert(sys_path, 0, root);
    Py_XDECREF(root);
    g_mod = PyImport_ImportModule("fastllm_b200.capi");
    if (g_mod == nullptr) set_error_from_python(); else ok = true;
  }
  if (own) PyEval_SaveThread();            // hand the GIL to whoever calls next (and to the engine thread)
  else PyGILState_Release(gs);
  g_ready = ok;
  return ok;
}

struct Gil {
  PyGILState_STATE s;
  Gil() : s(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(s); }
};

PyObject* int_list(const int* v, int n) {
  PyObject* l = PyList_New(n > 0 ? n : 0);
  for (int i = 0; i < n; ++i) PyList_SET_ITEM(l, i, PyLong_FromLong(v[i]));
  return l;
}

// call capi.<fn>(*args); args is a new reference to a tuple (stolen)
PyObject* call(const char* fn, PyObject* args) {
  PyObject* f = PyObject_GetAttrString(g_mod, fn);
  PyObject* r = f && args ? PyObject_CallObject(f, args) : nullptr;
  Py_XDECREF(f);
  Py_XDECREF(args);
  if (r == nullptr) set_error_from_python();
  return r;
}

char* dup_utf8(PyObject* s) {
  Py_ssize_t n = 0;
  const char* c = PyUnicode_AsUTF8AndSize(s, &n);
  if (c == nullptr) { set_error_from_python(); return nullptr; }
  char* out = static_cast<char*>(malloc((size_t)n + 1));
  if (out == nullptr) { t_error = "out of memory"; return nullptr; }
  memcpy(out, c, (size_t)n);
  out[n] = 0;
  return out;
}

PyObject* gen_args(const fastllm_generation_config* c) {      // the eight trailing arguments of capi.launch_*
  static const fastllm_generation_config zero = {};
  if (c == nullptr) c = &zero;
  return Py_BuildValue("(iiidifdN)", c->max_length, c->min_length, c->do_sample, (double)c->top_p, c->top_k, (double)c->temperature,
                       (double)c->repeat_penalty, int_list(c->stop_token_ids, c->stop_token_ids ? c->stop_token_cnt : 0));
}

PyObject* concat(PyObject* head, PyObject* tail) {            // both stolen
  PyObject* r = head && tail ? PySequence_Concat(head, tail) : nullptr;
  Py_XDECREF(head);
  Py_XDECREF(tail);
  return r;
}

long as_long(PyObject* r, long fail) {
  if (r == nullptr) return fail;
  const long v = PyLong_AsLong(r);
  Py_DECREF(r);
  if (v == -1 && PyErr_Occurred()) { set_error_from_python(); return fail; }
  return v;
}

}  // namespace

extern "C" {

int fastllm_init(const char* python_executable) { return ensure_init(python_executable) ? 0 : -1; }
const char* fastllm_last_error(void) { return t_error.c_str(); }
void fastllm_free(void* p) { free(p); }

int create_llm_model_fromhf(const char* path, const char* dtype, const char* options_json) {
  if (!ensure_init(nullptr)) return -1;
  Gil g;
  return (int)as_long(call("create_model", Py_BuildValue("(sss)", path, dtype ? dtype : "auto", options_json ? options_json : "")), -1);
}

void release_memory(int model) {
  if (!g_ready) return;
  Gil g;
  Py_XDECREF(call("release", Py_BuildValue("(i)", model)));
}

int set_option_llm_model(int model, const char* name, const char* value) {
  if (!g_ready) return -1;
  Gil g;
  PyObject* r = call("set_option", Py_BuildValue("(iss)", model, name, value));
  if (r == nullptr) return -1;
  Py_DECREF(r);
  return 0;
}

static char* str_call(const char* fn, PyObject* args) {
  PyObject* r = call(fn, args);
  if (r == nullptr) return nullptr;
  char* out = nullptr;
  if (r == Py_None) t_error.clear(); else out = dup_utf8(r);
  Py_DECREF(r);
  return out;
}

char* get_info_llm_model(int model) {
  if (!g_ready) return nullptr;
  Gil g;
  return str_call("info_json", Py_BuildValue("(i)", model));
}

int launch_response_llm_model(int model, int len, const int* token_ids, const fastllm_generation_config* cfg) {
  if (!g_ready) return -1;
  Gil g;
  return (int)as_long(call("launch_tokens", concat(Py_BuildValue("(iN)", model, int_list(token_ids, len)), gen_args(cfg))), -1);
}

int launch_response_str_llm_model(int model, const char* content, int as_chat, const fastllm_generation_config* cfg) {
  if (!g_ready) return -1;
  Gil g;
  return (int)as_long(call("launch_text", concat(Py_BuildValue("(isi)", model, content, as_chat), gen_args(cfg))), -1);
}

int launch_request_json_llm_model(int model, const char* body) {
  if (!g_ready) return -1;
  Gil g;
  return (int)as_long(call("launch_request_json", Py_BuildValue("(is)", model, body)), -1);
}

int request_wants_stream(const char* body) {
  if (!ensure_init(nullptr)) return 0;
  Gil g;
  return (int)as_long(call("request_wants_stream", Py_BuildValue("(s)", body)), 0);
}

int can_fetch_response_llm_model(int model, int handle) {
  if (!g_ready) return 0;
  Gil g;
  return (int)as_long(call("can_fetch", Py_BuildValue("(ii)", model, handle)), 0);
}

int fetch_response_llm_model(int model, int handle) {
  if (!g_ready) return -2;
  Gil g;
  return (int)as_long(call("fetch_token", Py_BuildValue("(ii)", model, handle)), -2);
}

char* fetch_response_str_llm_model(int model, int handle) {
  if (!g_ready) return nullptr;
  Gil g;
  return str_call("fetch_text", Py_BuildValue("(ii)", model, handle));
}

void abort_response_llm_model(int model, int handle) {
  if (!g_ready) return;
  Gil g;
  Py_XDECREF(call("abort", Py_BuildValue("(ii)", model, handle)));
}

char* response_str_llm_model(int model, const char* content, int as_chat, const fastllm_generation_config* cfg) {
  if (!g_ready) return nullptr;
  Gil g;
  return str_call("response_text", concat(Py_BuildValue("(isi)", model, content, as_chat), gen_args(cfg)));
}

char* get_response_statistics_llm_model(int model, int handle) {
  if (!g_ready) return nullptr;
  Gil g;
  return str_call("stats_json", Py_BuildValue("(ii)", model, handle));
}

int token_encode_string(int model, const char* content, int capacity, int* out_ids) {
  if (!g_ready) return -1;
  Gil g;
  PyObject* r = call("encode", Py_BuildValue("(is)", model, content));
  if (r == nullptr) return -1;
  const Py_ssize_t n = PyList_Size(r);
  for (Py_ssize_t i = 0; i < n && i < capacity; ++i) out_ids[i] = (int)PyLong_AsLong(PyList_GET_ITEM(r, i));
  Py_DECREF(r);
  return (int)n;
}

int token_decode(int model, int token_id, int capacity, char* out_bytes) {
  if (!g_ready) return -1;
  Gil g;
  PyObject* r = call("decode_token", Py_BuildValue("(ii)", model, token_id));
  if (r == nullptr) return -1;
  char* buf = nullptr;
  Py_ssize_t n = 0;
  if (PyBytes_AsStringAndSize(r, &buf, &n) != 0) { set_error_from_python(); Py_DECREF(r); return -1; }
  if (capacity > 0) memcpy(out_bytes, buf, (size_t)(n < capacity ? n : capacity));
  Py_DECREF(r);
  return (int)n;
}

char* apply_chat_template(int model, const char* messages_json) {
  if (!g_ready) return nullptr;
  Gil g;
  return str_call("apply_chat_template", Py_BuildValue("(is)", model, messages_json));
}

}  // extern "C"
