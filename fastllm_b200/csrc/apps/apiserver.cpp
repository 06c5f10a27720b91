// OpenAI-style HTTP server over the C ABI, plus a one-page chat UI at "/".  Plain POSIX sockets, one thread per connection;
// the engine batches the concurrent requests.  Request bodies go to the library unparsed (it reads `messages`, `prompt`,
// `max_tokens`, `temperature`, `top_p`, `top_k`, `stream`); this file does HTTP, server-sent events and the response envelopes.
// (The reference's counterparts: example/apiserver/apiserver.cpp and example/webui/webui.cpp.)
//
//   fastllm_apiserver -p <model folder> [--host 127.0.0.1] [--port 8080] [--model_name NAME] [--api_key KEY]
//                     [--dtype D] [--device DEV] [--options JSON]
//
// Routes: POST /v1/chat/completions, POST /v1/completions, GET /v1/models, GET /health, GET / (chat page).
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <thread>

#include "app_common.h"

namespace {

int g_model = -1;
std::string g_name = "fastllm_b200", g_key;
std::atomic<long> g_seq{0};

const char* kPage =
    "<!doctype html><meta charset=utf-8><title>fastllm_b200</title>"
    "<style>body{font-family:sans-serif;max-width:48em;margin:2em auto}#log div{margin:.5em 0;white-space:pre-wrap}"
    ".u{color:#246}.a{color:#222}textarea{width:100%;height:4em}</style>"
    "<h3>fastllm_b200</h3><div id=log></div><textarea id=q placeholder='message, Ctrl+Enter to send'></textarea>"
    "<button id=send>send</button> <button id=reset>reset</button><script>"
    "let msgs=[];const log=document.getElementById('log'),q=document.getElementById('q');"
    "function add(c,t){const d=document.createElement('div');d.className=c;d.textContent=t;log.appendChild(d);return d}"
    "async function send(){const t=q.value.trim();if(!t)return;q.value='';msgs.push({role:'user',content:t});add('u','user: '+t);"
    "const d=add('a','assistant: ');let out='';"
    "const r=await fetch('/v1/chat/completions',{method:'POST',headers:{'Content-Type':'application/json'},"
    "body:JSON.stringify({messages:msgs,stream:true,max_tokens:1024})});"
    "const rd=r.body.getReader(),dec=new TextDecoder();let buf='';"
    "for(;;){const {done,value}=await rd.read();if(done)break;buf+=dec.decode(value,{stream:true});"
    "let i;while((i=buf.indexOf('\\n\\n'))>=0){const ev=buf.slice(0,i);buf=buf.slice(i+2);"
    "if(!ev.startsWith('data: ')||ev=='data: [DONE]')continue;"
    "const c=JSON.parse(ev.slice(6)).choices[0].delta.content;if(c){out+=c;d.textContent='assistant: '+out}}}"
    "msgs.push({role:'assistant',content:out})}"
    "document.getElementById('send').onclick=send;document.getElementById('reset').onclick=()=>{msgs=[];log.textContent=''};"
    "q.onkeydown=e=>{if(e.key=='Enter'&&e.ctrlKey)send()}</script>";

bool send_all(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    const ssize_t n = send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
    if (n <= 0) return false;
    off += (size_t)n;
  }
  return true;
}

void reply(int fd, int code, const char* ctype, const std::string& body) {
  const char* what = code == 200 ? "OK" : code == 400 ? "Bad Request" : code == 401 ? "Unauthorized" : code == 404 ? "Not Found" : "Internal Server Error";
  send_all(fd, "HTTP/1.1 " + std::to_string(code) + " " + what + "\r\nContent-Type: " + ctype + "\r\nContent-Length: " +
                   std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body);
}

std::string error_json(const std::string& msg) { return "{\"error\": {\"message\": \"" + app::json_escape(msg) + "\"}}"; }

std::string header_value(const std::string& head, const char* name) {     // case-insensitive header lookup
  const size_t nl = strlen(name);
  size_t pos = 0;
  while ((pos = head.find("\r\n", pos)) != std::string::npos) {
    pos += 2;
    if (head.size() >= pos + nl + 1 && strncasecmp(head.c_str() + pos, name, nl) == 0 && head[pos + nl] == ':') {
      size_t b = pos + nl + 1, e = head.find("\r\n", b);
      while (b < head.size() && head[b] == ' ') ++b;
      return head.substr(b, e == std::string::npos ? std::string::npos : e - b);
    }
  }
  return "";
}

long json_int(const char* json, const char* key) {
  const char* p = json ? strstr(json, key) : nullptr;
  return p ? atol(p + strlen(key)) : 0;
}

void completions(int fd, const std::string& body, bool chat) {
  const bool stream = request_wants_stream(body.c_str()) != 0;
  const int h = launch_request_json_llm_model(g_model, body.c_str());
  if (h < 0) { reply(fd, 400, "application/json", error_json(fastllm_last_error())); return; }
  const std::string id = std::string(chat ? "chatcmpl-" : "cmpl-") + std::to_string(++g_seq);
  const long created = (long)std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count();
  const std::string head = "{\"id\": \"" + id + "\", \"object\": \"" + (chat ? (stream ? "chat.completion.chunk" : "chat.completion") : "text_completion") +
                           "\", \"created\": " + std::to_string(created) + ", \"model\": \"" + app::json_escape(g_name) + "\", \"choices\": [{\"index\": 0, ";
  if (stream) {
    if (!send_all(fd, "HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nConnection: close\r\n\r\n")) {
      abort_response_llm_model(g_model, h);
      return;
    }
    if (chat) send_all(fd, "data: " + head + "\"delta\": {\"role\": \"assistant\", \"content\": \"\"}, \"finish_reason\": null}]}\n\n");
    while (char* piece = fetch_response_str_llm_model(g_model, h)) {
      const std::string text = piece;
      fastllm_free(piece);
      if (text.empty()) continue;
      const std::string ev = "data: " + head + (chat ? "\"delta\": {\"content\": \"" + app::json_escape(text) + "\"}" : "\"text\": \"" + app::json_escape(text) + "\"") +
                             ", \"finish_reason\": null}]}\n\n";
      if (!send_all(fd, ev)) { abort_response_llm_model(g_model, h); return; }      // the client went away
    }
    send_all(fd, "data: " + head + (chat ? "\"delta\": {}" : "\"text\": \"\"") + ", \"finish_reason\": \"stop\"}]}\n\ndata: [DONE]\n\n");
    return;
  }
  std::string text;
  while (char* piece = fetch_response_str_llm_model(g_model, h)) { text += piece; fastllm_free(piece); }
  char* st = get_response_statistics_llm_model(g_model, h);
  const long pt = json_int(st, "\"prompt_tokens\": "), ct = json_int(st, "\"output_tokens\": ");
  fastllm_free(st);
  reply(fd, 200, "application/json",
        head + (chat ? "\"message\": {\"role\": \"assistant\", \"content\": \"" + app::json_escape(text) + "\"}" : "\"text\": \"" + app::json_escape(text) + "\"") +
            ", \"finish_reason\": \"stop\"}], \"usage\": {\"prompt_tokens\": " + std::to_string(pt) + ", \"completion_tokens\": " + std::to_string(ct) +
            ", \"total_tokens\": " + std::to_string(pt + ct) + "}}");
}

void serve(int fd) {
  std::string buf;
  char tmp[8192];
  size_t head_end = std::string::npos;
  while (head_end == std::string::npos && buf.size() < (1u << 20)) {
    const ssize_t n = recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) { close(fd); return; }
    buf.append(tmp, (size_t)n);
    head_end = buf.find("\r\n\r\n");
  }
  if (head_end == std::string::npos) { reply(fd, 400, "application/json", error_json("header too large")); close(fd); return; }
  const std::string head = buf.substr(0, head_end + 2);
  std::string body = buf.substr(head_end + 4);
  const size_t want = (size_t)atol(header_value(head, "Content-Length").c_str());
  while (body.size() < want && want < (256u << 20)) {
    const ssize_t n = recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) break;
    body.append(tmp, (size_t)n);
  }
  const size_t sp1 = head.find(' '), sp2 = head.find(' ', sp1 + 1);
  const std::string method = head.substr(0, sp1);
  std::string path = sp2 == std::string::npos ? "" : head.substr(sp1 + 1, sp2 - sp1 - 1);
  const size_t qm = path.find('?');
  if (qm != std::string::npos) path.erase(qm);

  if (!g_key.empty() && path.rfind("/v1/", 0) == 0 && header_value(head, "Authorization") != "Bearer " + g_key) {
    reply(fd, 401, "application/json", error_json("invalid API key"));
  } else if (method == "POST" && path == "/v1/chat/completions") {
    completions(fd, body, true);
  } else if (method == "POST" && path == "/v1/completions") {
    completions(fd, body, false);
  } else if (method == "GET" && path == "/v1/models") {
    reply(fd, 200, "application/json", "{\"object\": \"list\", \"data\": [{\"id\": \"" + app::json_escape(g_name) + "\", \"object\": \"model\", \"owned_by\": \"fastllm_b200\"}]}");
  } else if (method == "GET" && path == "/health") {
    reply(fd, 200, "application/json", "{\"status\": \"ok\"}");
  } else if (method == "GET" && (path == "/" || path == "/index.html")) {
    reply(fd, 200, "text/html; charset=utf-8", kPage);
  } else {
    reply(fd, 404, "application/json", error_json("no such route: " + method + " " + path));
  }
  shutdown(fd, SHUT_RDWR);
  close(fd);
}

}  // namespace

int main(int argc, char** argv) {
  auto a = app::parse_args(argc, argv, {{"p", "path"}, {"d", "dtype"}});
  if (a.count("help") || a.count("h")) {
    printf("usage: %s -p <model folder> [--host H] [--port N] [--model_name NAME] [--api_key KEY] [--dtype D] [--device DEV] [--options JSON]\n", argv[0]);
    return 0;
  }
  signal(SIGPIPE, SIG_IGN);
  g_model = app::load_model(a);
  g_name = app::get(a, "model_name", g_name.c_str());
  g_key = app::get(a, "api_key", "");
  const std::string host = app::get(a, "host", "127.0.0.1");
  const int port = atoi(app::get(a, "port", "8080").c_str());

  const int ls = socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr = {};
  addr.sin_family = AF_INET;
  addr.sin_port = htons((uint16_t)port);
  if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) { fprintf(stderr, "bad --host %s (an IPv4 address)\n", host.c_str()); return 2; }
  if (bind(ls, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || listen(ls, 128) != 0) { perror("bind / listen"); return 1; }
  socklen_t len = sizeof addr;
  getsockname(ls, reinterpret_cast<sockaddr*>(&addr), &len);
  printf("listening on http://%s:%d\n", host.c_str(), (int)ntohs(addr.sin_port));
  fflush(stdout);
  while (true) {
    const int fd = accept(ls, nullptr, nullptr);
    if (fd < 0) continue;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    std::thread(serve, fd).detach();
  }
}
