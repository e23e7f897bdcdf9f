// libtfb_serve: OpenAI-compatible HTTP/SSE front end over raw sockets.
//
//   accept thread (select, 1 s tick) -> connection queue -> worker pool (default 4 threads)
//   one request per connection, Content-Length bodies only (chunked -> 501)
//   limits: request line 8 KB (414), headers 64 KB (431), body 4 MiB (413), 30 s receive timeout (408)
//   per-IP token-bucket rate limit (429), Bearer auth on /v1/* (401), max_concurrent admission (503),
//   415 for non-JSON POST bodies, CORS + security headers, OPTIONS -> 204
//   routes: GET /health, GET /metrics, GET /v1/models, POST /v1/completions, POST /v1/chat/completions,
//           POST /v1/embeddings, POST /v1/models/load, POST /v1/models/unload;  streaming = "data: {json}\n\n" ... "data: [DONE]\n\n"
//   errors: {"error":{"code","message","type"}}
// Generation and embeddings are callbacks (C function pointers) so the engine can live in Python or C++.
//
// Contract parity: reference src/server/http_server.cpp (limits :749-769, rate limiter :116-152, auth
// :254-275, admission :277-305, routes :931-1425, error shape :210-222) and tests/test_server_contract.cpp.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/select.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#define TFB_EXPORT extern "C" __attribute__((visibility("default")))

extern "C" {
typedef void (*tfb_emit_fn)(void* emit_ctx, const char* piece);
// returns 0 on success; fills usage counters; calls emit for every generated piece of text
typedef int (*tfb_generate_fn)(void* user, const char* prompt, int max_tokens, float temperature, float top_p, int top_k,
                               int stream, tfb_emit_fn emit, void* emit_ctx, int* prompt_tokens, int* completion_tokens);
// writes up to cap floats, returns the embedding dimension (<= 0 on error)
typedef int (*tfb_embed_fn)(void* user, const char* text, float* out, int cap);
typedef int (*tfb_load_model_fn)(void* user, const char* path);   // non-zero = the model at `path` is now the served one
typedef void (*tfb_unload_model_fn)(void* user);
}

namespace {

// ------------------------------------------------------------------------------------------------
// minimal JSON
// ------------------------------------------------------------------------------------------------
struct Json {
  enum T { NUL, BOOL, NUM, STR, ARR, OBJ } t = NUL;
  bool b = false;
  double n = 0;
  std::string s;
  std::vector<Json> a;
  std::map<std::string, Json> o;
  bool has(const std::string& k) const { return t == OBJ && o.count(k); }
  const Json& at(const std::string& k) const { static Json nul; auto it = o.find(k); return it == o.end() ? nul : it->second; }
};
struct JsonParser {
  const std::string& s;
  size_t i = 0;
  bool ok = true;
  int depth = 0;
  explicit JsonParser(const std::string& str) : s(str) {}
  void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  Json parse() { Json v = value(); ws(); if (i != s.size()) ok = false; return v; }
  Json value() {
    Json v;
    ws();
    if (i >= s.size() || ++depth > 64) { ok = false; return v; }
    const char c = s[i];
    if (c == '{') {
      v.t = Json::OBJ; ++i; ws();
      if (i < s.size() && s[i] == '}') { ++i; --depth; return v; }
      while (ok) {
        ws();
        Json k = str();
        ws();
        if (!ok || i >= s.size() || s[i] != ':') { ok = false; break; }
        ++i;
        v.o[k.s] = value();
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; break; }
        ok = false;
      }
    } else if (c == '[') {
      v.t = Json::ARR; ++i; ws();
      if (i < s.size() && s[i] == ']') { ++i; --depth; return v; }
      while (ok) {
        v.a.push_back(value());
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; break; }
        ok = false;
      }
    } else if (c == '"') v = str();
    else if (!s.compare(i, 4, "true")) { v.t = Json::BOOL; v.b = true; i += 4; }
    else if (!s.compare(i, 5, "false")) { v.t = Json::BOOL; i += 5; }
    else if (!s.compare(i, 4, "null")) { i += 4; }
    else {
      char* end = nullptr;
      v.n = strtod(s.c_str() + i, &end);
      if (end == s.c_str() + i) ok = false;
      v.t = Json::NUM;
      i = size_t(end - s.c_str());
    }
    --depth;
    return v;
  }
  Json str() {
    Json v;
    v.t = Json::STR;
    if (i >= s.size() || s[i] != '"') { ok = false; return v; }
    ++i;
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) {
        const char c = s[++i];
        switch (c) {
          case 'n': v.s.push_back('\n'); break;
          case 't': v.s.push_back('\t'); break;
          case 'r': v.s.push_back('\r'); break;
          case 'b': v.s.push_back('\b'); break;
          case 'f': v.s.push_back('\f'); break;
          case 'u': {
            if (i + 4 >= s.size()) { ok = false; return v; }
            unsigned cp = unsigned(strtoul(s.substr(i + 1, 4).c_str(), nullptr, 16));
            i += 4;
            if (cp < 0x80) v.s.push_back(char(cp));
            else if (cp < 0x800) { v.s.push_back(char(0xC0 | (cp >> 6))); v.s.push_back(char(0x80 | (cp & 0x3F))); }
            else { v.s.push_back(char(0xE0 | (cp >> 12))); v.s.push_back(char(0x80 | ((cp >> 6) & 0x3F))); v.s.push_back(char(0x80 | (cp & 0x3F))); }
            break;
          }
          default: v.s.push_back(c);
        }
        ++i;
      } else v.s.push_back(s[i++]);
    }
    if (i >= s.size()) { ok = false; return v; }
    ++i;
    return v;
  }
};
std::string jstr(const std::string& s) {
  std::string o = "\"";
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o.push_back(char(c));
    }
  }
  return o + "\"";
}

std::string error_json(const std::string& msg, const std::string& type, const std::string& code) {
  return "{\"error\":{\"code\":" + jstr(code) + ",\"message\":" + jstr(msg) + ",\"type\":" +
         jstr(type.empty() ? "invalid_request_error" : type) + "}}";
}

const char* status_text(int c) {
  switch (c) {
    case 200: return "OK"; case 204: return "No Content"; case 400: return "Bad Request"; case 401: return "Unauthorized";
    case 404: return "Not Found"; case 405: return "Method Not Allowed"; case 408: return "Request Timeout";
    case 413: return "Payload Too Large"; case 414: return "URI Too Long"; case 415: return "Unsupported Media Type";
    case 429: return "Too Many Requests"; case 431: return "Request Header Fields Too Large";
    case 500: return "Internal Server Error"; case 501: return "Not Implemented"; case 503: return "Service Unavailable";
    default: return "Unknown";
  }
}

struct Request {
  std::string method, path, body;
  std::map<std::string, std::string> headers;  // lower-case names
};

struct Histogram {
  std::mutex mu;
  std::vector<double> samples;
  void add(double ms) { std::lock_guard<std::mutex> l(mu); if (samples.size() >= 65536) samples.erase(samples.begin(), samples.begin() + 32768); samples.push_back(ms); }
  double pct(double p) { std::lock_guard<std::mutex> l(mu); if (samples.empty()) return 0; std::vector<double> v = samples; std::sort(v.begin(), v.end()); return v[std::min(v.size() - 1, size_t(p * v.size()))]; }
};

struct Server {
  int port = 8080, bound_port = 0, listen_fd = -1;
  int workers = 4, timeout_s = 30, max_header = 64 * 1024, max_concurrent = 0;
  size_t max_body = 4u << 20, max_line = 8 * 1024;
  double rate_rps = 0, rate_burst = 0;
  std::string auth_token, model_name = "tfb-model";
  tfb_generate_fn gen = nullptr;
  void* gen_user = nullptr;
  tfb_embed_fn emb = nullptr;
  void* emb_user = nullptr;
  tfb_load_model_fn load_model = nullptr;      // POST /v1/models/load {"path": ..., "name": ...}
  tfb_unload_model_fn unload_model = nullptr;  // POST /v1/models/unload
  void* model_user = nullptr;
  std::mutex model_mu;                         // one load / unload at a time
  std::atomic<bool> model_loaded{true};
  std::atomic<bool> running{false};
  std::atomic<int> current{0};
  std::atomic<long long> total{0}, errors{0}, tokens_out{0};
  std::thread accept_thread;
  std::vector<std::thread> pool;
  std::mutex qmu;
  std::condition_variable qcv;
  std::deque<std::pair<int, std::string>> queue;  // fd, peer ip
  std::mutex rmu;
  std::map<std::string, std::pair<double, double>> buckets;  // ip -> (tokens, last time)
  Histogram latency, ttft;
  std::chrono::steady_clock::time_point started;
};

double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

bool send_all(int fd, const char* p, size_t n) {
  while (n) {
    const ssize_t k = send(fd, p, n, MSG_NOSIGNAL);
    if (k <= 0) return false;
    p += k;
    n -= size_t(k);
  }
  return true;
}
std::string common_headers() {
  return "Access-Control-Allow-Origin: *\r\nAccess-Control-Allow-Headers: Content-Type, Authorization\r\n"
         "Access-Control-Allow-Methods: GET, POST, OPTIONS\r\nX-Content-Type-Options: nosniff\r\n"
         "X-Frame-Options: DENY\r\nCache-Control: no-store\r\nConnection: close\r\n";
}
void respond(int fd, int code, const std::string& ctype, const std::string& body) {
  std::ostringstream h;
  h << "HTTP/1.1 " << code << " " << status_text(code) << "\r\nContent-Type: " << ctype << "\r\nContent-Length: " << body.size()
    << "\r\n" << common_headers() << "\r\n";
  const std::string hs = h.str();
  if (send_all(fd, hs.data(), hs.size())) send_all(fd, body.data(), body.size());
}
void respond_err(Server& s, int fd, int code, const std::string& msg, const std::string& type, const std::string& ecode) {
  ++s.errors;
  respond(fd, code, "application/json", error_json(msg, type, ecode));
}

// returns 0 ok, else the HTTP status to answer with
int read_request(Server& s, int fd, Request& rq) {
  std::string buf;
  char tmp[8192];
  size_t hdr_end = std::string::npos;
  while (hdr_end == std::string::npos) {
    const ssize_t k = recv(fd, tmp, sizeof tmp, 0);
    if (k == 0) return 400;
    if (k < 0) return 408;
    buf.append(tmp, size_t(k));
    const size_t eol = buf.find("\r\n");
    if (eol == std::string::npos ? buf.size() > s.max_line : eol > s.max_line) return 414;
    hdr_end = buf.find("\r\n\r\n");
    if (hdr_end == std::string::npos && buf.size() > size_t(s.max_header)) return 431;
  }
  if (hdr_end > size_t(s.max_header)) return 431;
  std::istringstream hs(buf.substr(0, hdr_end));
  std::string line;
  std::getline(hs, line);
  if (!line.empty() && line.back() == '\r') line.pop_back();
  {
    std::istringstream ls(line);
    std::string ver;
    if (!(ls >> rq.method >> rq.path >> ver) || ver.compare(0, 5, "HTTP/") != 0) return 400;
  }
  const size_t q = rq.path.find('?');
  if (q != std::string::npos) rq.path.resize(q);
  while (std::getline(hs, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    const size_t c = line.find(':');
    if (c == std::string::npos) continue;
    std::string k = line.substr(0, c), v = line.substr(c + 1);
    std::transform(k.begin(), k.end(), k.begin(), ::tolower);
    while (!v.empty() && v.front() == ' ') v.erase(v.begin());
    rq.headers[k] = v;
  }
  if (rq.headers.count("transfer-encoding")) return 501;
  size_t clen = 0;
  if (rq.headers.count("content-length")) {
    const std::string& v = rq.headers["content-length"];
    if (v.empty() || v.find_first_not_of("0123456789") != std::string::npos || v.size() > 12) return 400;
    clen = size_t(strtoull(v.c_str(), nullptr, 10));
  }
  if (clen > s.max_body) return 413;
  rq.body = buf.substr(hdr_end + 4);
  while (rq.body.size() < clen) {
    const ssize_t k = recv(fd, tmp, std::min(sizeof tmp, clen - rq.body.size()), 0);
    if (k == 0) return 400;
    if (k < 0) return 408;
    rq.body.append(tmp, size_t(k));
  }
  rq.body.resize(std::min(rq.body.size(), clen));
  return 0;
}

bool rate_ok(Server& s, const std::string& ip) {
  if (s.rate_rps <= 0) return true;
  std::lock_guard<std::mutex> l(s.rmu);
  const double t = now_s();
  auto it = s.buckets.find(ip);
  if (it == s.buckets.end()) it = s.buckets.emplace(ip, std::make_pair(std::max(1.0, s.rate_burst), t)).first;
  auto& b = it->second;
  b.first = std::min(std::max(1.0, s.rate_burst), b.first + (t - b.second) * s.rate_rps);
  b.second = t;
  if (b.first < 1.0) return false;
  b.first -= 1.0;
  return true;
}

struct EmitCtx {
  Server* s;
  int fd;
  bool stream, chat, first = true, broken = false;
  std::string id, text;
  long long created;
  double t0;
};
void emit_piece(void* ctx, const char* piece) {
  EmitCtx* e = static_cast<EmitCtx*>(ctx);
  if (e->first) { e->s->ttft.add((now_s() - e->t0) * 1e3); e->first = false; }
  if (!e->stream) { e->text += piece; return; }
  if (e->broken) return;
  std::string j;
  if (e->chat)
    j = "{\"id\":" + jstr(e->id) + ",\"object\":\"chat.completion.chunk\",\"created\":" + std::to_string(e->created) +
        ",\"model\":" + jstr(e->s->model_name) + ",\"choices\":[{\"index\":0,\"delta\":{\"content\":" + jstr(piece) +
        "},\"finish_reason\":null}]}";
  else
    j = "{\"id\":" + jstr(e->id) + ",\"object\":\"text_completion\",\"created\":" + std::to_string(e->created) +
        ",\"model\":" + jstr(e->s->model_name) + ",\"choices\":[{\"index\":0,\"text\":" + jstr(piece) +
        ",\"finish_reason\":null}]}";
  const std::string f = "data: " + j + "\n\n";
  if (!send_all(e->fd, f.data(), f.size())) e->broken = true;
}

std::string chat_prompt(const Json& messages) {
  std::string p;
  for (const Json& m : messages.a)
    p += "<|im_start|>" + m.at("role").s + "\n" + m.at("content").s + "<|im_end|>\n";
  return p + "<|im_start|>assistant\n";
}

void handle_generate(Server& s, int fd, const Request& rq, bool chat) {
  if (!s.model_loaded) return respond_err(s, fd, 503, "no model is loaded", "server_error", "model_not_loaded");
  JsonParser jp(rq.body);
  Json j = jp.parse();
  if (!jp.ok || j.t != Json::OBJ) return respond_err(s, fd, 400, "request body is not valid JSON", "invalid_request_error", "invalid_json");
  std::vector<std::string> prompts;
  if (chat) {
    if (!j.has("messages") || j.at("messages").t != Json::ARR || j.at("messages").a.empty())
      return respond_err(s, fd, 400, "'messages' must be a non-empty array", "invalid_request_error", "missing_messages");
    prompts.push_back(chat_prompt(j.at("messages")));
  } else {
    const Json& p = j.at("prompt");
    if (p.t == Json::STR) prompts.push_back(p.s);
    else if (p.t == Json::ARR) { for (const Json& x : p.a) if (x.t == Json::STR) prompts.push_back(x.s); }
    if (prompts.empty()) return respond_err(s, fd, 400, "'prompt' must be a string or an array of strings", "invalid_request_error", "missing_prompt");
  }
  int max_tokens = j.has("max_tokens") && j.at("max_tokens").t == Json::NUM ? int(j.at("max_tokens").n) : 64;
  max_tokens = std::max(1, std::min(4096, max_tokens));
  const float temperature = j.has("temperature") && j.at("temperature").t == Json::NUM ? float(j.at("temperature").n) : 0.7f;
  const float top_p = j.has("top_p") && j.at("top_p").t == Json::NUM ? float(j.at("top_p").n) : 0.9f;
  const int top_k = j.has("top_k") && j.at("top_k").t == Json::NUM ? int(j.at("top_k").n) : 40;
  const bool stream = j.has("stream") && j.at("stream").t == Json::BOOL && j.at("stream").b;
  const long long created = (long long)time(nullptr);
  const std::string id = std::string(chat ? "chatcmpl-" : "cmpl-") + std::to_string(s.total.load());

  if (stream) {
    const std::string h = std::string("HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\n") + common_headers() + "\r\n";
    if (!send_all(fd, h.data(), h.size())) return;
    if (!s.gen) {
      const std::string f = "data: " + error_json("No generate callback registered", "server_error", "no_generate_callback") + "\n\ndata: [DONE]\n\n";
      send_all(fd, f.data(), f.size());
      return;
    }
    EmitCtx e{&s, fd, true, chat};
    e.id = id; e.created = created; e.t0 = now_s();
    if (chat) {
      const std::string f = "data: {\"id\":" + jstr(id) + ",\"object\":\"chat.completion.chunk\",\"created\":" + std::to_string(created) +
                            ",\"model\":" + jstr(s.model_name) + ",\"choices\":[{\"index\":0,\"delta\":{\"role\":\"assistant\"},\"finish_reason\":null}]}\n\n";
      send_all(fd, f.data(), f.size());
    }
    int pt = 0, ct = 0;
    s.gen(s.gen_user, prompts[0].c_str(), max_tokens, temperature, top_p, top_k, 1, emit_piece, &e, &pt, &ct);
    s.tokens_out += ct;
    const std::string fin = chat
        ? "data: {\"id\":" + jstr(id) + ",\"object\":\"chat.completion.chunk\",\"created\":" + std::to_string(created) + ",\"model\":" + jstr(s.model_name) +
              ",\"choices\":[{\"index\":0,\"delta\":{},\"finish_reason\":\"stop\"}]}\n\ndata: [DONE]\n\n"
        : "data: {\"id\":" + jstr(id) + ",\"object\":\"text_completion\",\"created\":" + std::to_string(created) + ",\"model\":" + jstr(s.model_name) +
              ",\"choices\":[{\"index\":0,\"text\":\"\",\"finish_reason\":\"stop\"}]}\n\ndata: [DONE]\n\n";
    send_all(fd, fin.data(), fin.size());
    return;
  }
  if (!s.gen) return respond_err(s, fd, 503, "No generate callback registered", "server_error", "no_generate_callback");
  std::string choices;
  int pt_total = 0, ct_total = 0;
  for (size_t i = 0; i < prompts.size(); ++i) {
    EmitCtx e{&s, fd, false, chat};
    e.t0 = now_s();
    int pt = 0, ct = 0;
    const int rc = s.gen(s.gen_user, prompts[i].c_str(), max_tokens, temperature, top_p, top_k, 0, emit_piece, &e, &pt, &ct);
    if (rc != 0) return respond_err(s, fd, 500, "generation failed", "server_error", "generation_failed");
    if (pt == 0) pt = int(prompts[i].size() / 4);
    if (ct == 0) ct = int(e.text.size() / 4);
    pt_total += pt;
    ct_total += ct;
    if (i) choices += ",";
    if (chat)
      choices += "{\"index\":" + std::to_string(i) + ",\"message\":{\"role\":\"assistant\",\"content\":" + jstr(e.text) + "},\"finish_reason\":\"stop\"}";
    else
      choices += "{\"index\":" + std::to_string(i) + ",\"text\":" + jstr(e.text) + ",\"logprobs\":null,\"finish_reason\":\"stop\"}";
  }
  s.tokens_out += ct_total;
  const std::string body = "{\"id\":" + jstr(id) + ",\"object\":" + (chat ? "\"chat.completion\"" : "\"text_completion\"") + ",\"created\":" +
                           std::to_string(created) + ",\"model\":" + jstr(s.model_name) + ",\"choices\":[" + choices + "],\"usage\":{\"prompt_tokens\":" +
                           std::to_string(pt_total) + ",\"completion_tokens\":" + std::to_string(ct_total) + ",\"total_tokens\":" +
                           std::to_string(pt_total + ct_total) + "}}";
  respond(fd, 200, "application/json", body);
}

void handle_embeddings(Server& s, int fd, const Request& rq) {
  JsonParser jp(rq.body);
  Json j = jp.parse();
  if (!jp.ok || j.t != Json::OBJ) return respond_err(s, fd, 400, "request body is not valid JSON", "invalid_request_error", "invalid_json");
  std::vector<std::string> inputs;
  const Json& in = j.at("input");
  if (in.t == Json::STR) inputs.push_back(in.s);
  else if (in.t == Json::ARR) for (const Json& x : in.a) if (x.t == Json::STR) inputs.push_back(x.s);
  if (inputs.empty()) return respond_err(s, fd, 400, "'input' must be a string or an array of strings", "invalid_request_error", "missing_input");
  if (inputs.size() > 256) return respond_err(s, fd, 400, "at most 256 inputs per request", "invalid_request_error", "too_many_inputs");
  if (!s.emb) return respond_err(s, fd, 503, "No embeddings callback registered", "server_error", "no_embeddings_callback");
  std::string data;
  std::vector<float> buf(16384);
  int toks = 0;
  for (size_t i = 0; i < inputs.size(); ++i) {
    const int dim = s.emb(s.emb_user, inputs[i].c_str(), buf.data(), int(buf.size()));
    if (dim <= 0) return respond_err(s, fd, 500, "embedding failed", "server_error", "embedding_failed");
    if (i) data += ",";
    data += "{\"object\":\"embedding\",\"index\":" + std::to_string(i) + ",\"embedding\":[";
    for (int d = 0; d < dim; ++d) { char t[32]; snprintf(t, sizeof t, d ? ",%.6g" : "%.6g", buf[d]); data += t; }
    data += "]}";
    toks += int(inputs[i].size() / 4) + 1;
  }
  respond(fd, 200, "application/json", "{\"object\":\"list\",\"data\":[" + data + "],\"model\":" + jstr(s.model_name) +
                                           ",\"usage\":{\"prompt_tokens\":" + std::to_string(toks) + ",\"total_tokens\":" + std::to_string(toks) + "}}");
}

// POST /v1/models/load and /v1/models/unload: hand the request to the registered callbacks (the engine lives behind them);
// the served model name follows a successful load.
void handle_model_admin(Server& s, int fd, const Request& rq, bool load) {
  if (load) {
    JsonParser jp(rq.body);
    Json j = jp.parse();
    if (!jp.ok || j.t != Json::OBJ) return respond_err(s, fd, 400, "request body is not valid JSON", "invalid_request_error", "invalid_json");
    const Json& pth = j.at("path");
    if (pth.t != Json::STR || pth.s.empty()) return respond_err(s, fd, 400, "'path' must be a non-empty string", "invalid_request_error", "missing_path");
    if (!s.load_model) return respond_err(s, fd, 503, "No model-load callback registered", "server_error", "no_load_callback");
    std::lock_guard<std::mutex> l(s.model_mu);
    if (!s.load_model(s.model_user, pth.s.c_str())) return respond_err(s, fd, 500, "model could not be loaded from " + pth.s, "server_error", "load_failed");
    const Json& nm = j.at("name");
    if (nm.t == Json::STR && !nm.s.empty()) s.model_name = nm.s;
    s.model_loaded = true;
    return respond(fd, 200, "application/json", "{\"status\":\"loaded\",\"model\":" + jstr(s.model_name) + ",\"path\":" + jstr(pth.s) + "}");
  }
  if (!s.unload_model) return respond_err(s, fd, 503, "No model-unload callback registered", "server_error", "no_unload_callback");
  std::lock_guard<std::mutex> l(s.model_mu);
  s.unload_model(s.model_user);
  s.model_loaded = false;
  respond(fd, 200, "application/json", "{\"status\":\"unloaded\"}");
}

void handle(Server& s, int fd, const std::string& ip) {
  timeval tv{s.timeout_s, 0};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
  Request rq;
  const double t0 = now_s();
  ++s.total;
  const int st = read_request(s, fd, rq);
  if (st) {
    const char* msg = st == 408 ? "request timed out" : st == 413 ? "request body too large" : st == 414 ? "request line too long"
                      : st == 431 ? "request headers too large" : st == 501 ? "chunked transfer encoding is not supported" : "malformed request";
    return respond_err(s, fd, st, msg, "invalid_request_error", "bad_request");
  }
  if (rq.method == "OPTIONS") return respond(fd, 204, "text/plain", "");
  if (!rate_ok(s, ip)) return respond_err(s, fd, 429, "rate limit exceeded", "rate_limit_error", "rate_limited");
  const bool v1 = rq.path.compare(0, 4, "/v1/") == 0;
  if (v1 && !s.auth_token.empty()) {
    const std::string want = "Bearer " + s.auth_token;
    auto it = rq.headers.find("authorization");
    if (it == rq.headers.end() || it->second != want) return respond_err(s, fd, 401, "missing or invalid bearer token", "authentication_error", "invalid_api_key");
  }
  struct Admit {
    Server& s; bool ok;
    explicit Admit(Server& sv) : s(sv) { const int c = ++s.current; ok = s.max_concurrent <= 0 || c <= s.max_concurrent; }
    ~Admit() { --s.current; }
  } admit(s);
  if (!admit.ok) return respond_err(s, fd, 503, "server is at capacity", "server_error", "overloaded");
  if (rq.method == "GET" && rq.path == "/health") {
    const double up = std::chrono::duration<double>(std::chrono::steady_clock::now() - s.started).count();
    return respond(fd, 200, "application/json", "{\"status\":\"ok\",\"model\":" + jstr(s.model_name) + ",\"uptime_s\":" + std::to_string(up) +
                                                    ",\"total_requests\":" + std::to_string(s.total.load()) + ",\"active_requests\":" +
                                                    std::to_string(s.current.load()) + ",\"errors\":" + std::to_string(s.errors.load()) + "}");
  }
  if (rq.method == "GET" && rq.path == "/metrics") {
    std::ostringstream m;
    m << "tfb_requests_total " << s.total.load() << "\ntfb_errors_total " << s.errors.load() << "\ntfb_active_requests " << s.current.load()
      << "\ntfb_generated_tokens_total " << s.tokens_out.load() << "\ntfb_latency_ms{quantile=\"0.5\"} " << s.latency.pct(0.5)
      << "\ntfb_latency_ms{quantile=\"0.95\"} " << s.latency.pct(0.95) << "\ntfb_latency_ms{quantile=\"0.99\"} " << s.latency.pct(0.99)
      << "\ntfb_ttft_ms{quantile=\"0.5\"} " << s.ttft.pct(0.5) << "\ntfb_ttft_ms{quantile=\"0.99\"} " << s.ttft.pct(0.99) << "\n";
    return respond(fd, 200, "text/plain; version=0.0.4", m.str());
  }
  if (rq.method == "GET" && rq.path == "/v1/models") {
    if (!s.model_loaded) return respond(fd, 200, "application/json", "{\"object\":\"list\",\"data\":[]}");
    return respond(fd, 200, "application/json", "{\"object\":\"list\",\"data\":[{\"id\":" + jstr(s.model_name) + ",\"object\":\"model\",\"owned_by\":\"tfb\"}]}");
  }
  if (rq.method == "POST") {
    auto ct = rq.headers.find("content-type");
    if (ct == rq.headers.end() || ct->second.find("application/json") == std::string::npos)
      return respond_err(s, fd, 415, "Content-Type must be application/json", "invalid_request_error", "unsupported_media_type");
    if (rq.path == "/v1/completions") { handle_generate(s, fd, rq, false); s.latency.add((now_s() - t0) * 1e3); return; }
    if (rq.path == "/v1/chat/completions") { handle_generate(s, fd, rq, true); s.latency.add((now_s() - t0) * 1e3); return; }
    if (rq.path == "/v1/embeddings") { handle_embeddings(s, fd, rq); s.latency.add((now_s() - t0) * 1e3); return; }
    if (rq.path == "/v1/models/load") return handle_model_admin(s, fd, rq, true);
    if (rq.path == "/v1/models/unload") return handle_model_admin(s, fd, rq, false);
  }
  if (rq.path == "/v1/models/load" || rq.path == "/v1/models/unload" || rq.path == "/health" || rq.path == "/v1/models" || rq.path == "/v1/completions" || rq.path == "/v1/chat/completions" || rq.path == "/v1/embeddings")
    return respond_err(s, fd, 405, "method not allowed", "invalid_request_error", "method_not_allowed");
  respond_err(s, fd, 404, "unknown route " + rq.path, "invalid_request_error", "not_found");
}

void worker_loop(Server* s) {
  while (true) {
    std::pair<int, std::string> job;
    {
      std::unique_lock<std::mutex> l(s->qmu);
      s->qcv.wait(l, [&] { return !s->queue.empty() || !s->running; });
      if (s->queue.empty()) return;
      job = s->queue.front();
      s->queue.pop_front();
    }
    handle(*s, job.first, job.second);
    shutdown(job.first, SHUT_RDWR);
    close(job.first);
  }
}
void accept_loop(Server* s) {
  while (s->running) {
    fd_set fds;
    FD_ZERO(&fds);
    FD_SET(s->listen_fd, &fds);
    timeval tv{1, 0};
    if (select(s->listen_fd + 1, &fds, nullptr, nullptr, &tv) <= 0) continue;
    sockaddr_in peer{};
    socklen_t pl = sizeof peer;
    const int fd = accept(s->listen_fd, reinterpret_cast<sockaddr*>(&peer), &pl);
    if (fd < 0) continue;
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    char ip[64] = "?";
    inet_ntop(AF_INET, &peer.sin_addr, ip, sizeof ip);
    {
      std::lock_guard<std::mutex> l(s->qmu);
      s->queue.emplace_back(fd, ip);
    }
    s->qcv.notify_one();
  }
}

}  // namespace

TFB_EXPORT void* tfb_server_new(int port) { Server* s = new Server(); s->port = port; return s; }
TFB_EXPORT void tfb_server_free(void* h) { delete static_cast<Server*>(h); }
TFB_EXPORT void tfb_server_set_workers(void* h, int n) { static_cast<Server*>(h)->workers = n > 0 ? n : 4; }
TFB_EXPORT void tfb_server_set_timeout(void* h, int sec) { static_cast<Server*>(h)->timeout_s = sec > 0 ? sec : 30; }
TFB_EXPORT void tfb_server_set_max_body(void* h, long long n) { static_cast<Server*>(h)->max_body = n > 0 ? size_t(n) : (4u << 20); }
TFB_EXPORT void tfb_server_set_max_header(void* h, int n) { static_cast<Server*>(h)->max_header = n > 0 ? n : 64 * 1024; }
TFB_EXPORT int tfb_server_max_header(void* h) { return static_cast<Server*>(h)->max_header; }
TFB_EXPORT void tfb_server_set_max_concurrent(void* h, int n) { static_cast<Server*>(h)->max_concurrent = n > 0 ? n : 0; }
TFB_EXPORT int tfb_server_max_concurrent(void* h) { return static_cast<Server*>(h)->max_concurrent; }
TFB_EXPORT void tfb_server_set_rate_limit(void* h, double rps, double burst) { Server* s = static_cast<Server*>(h); s->rate_rps = rps; s->rate_burst = burst; }
TFB_EXPORT void tfb_server_set_auth_token(void* h, const char* t) { static_cast<Server*>(h)->auth_token = t ? t : ""; }
TFB_EXPORT void tfb_server_set_model_name(void* h, const char* n) { static_cast<Server*>(h)->model_name = n ? n : ""; }
TFB_EXPORT void tfb_server_set_generate(void* h, tfb_generate_fn fn, void* user) { Server* s = static_cast<Server*>(h); s->gen = fn; s->gen_user = user; }
TFB_EXPORT void tfb_server_set_embeddings(void* h, tfb_embed_fn fn, void* user) { Server* s = static_cast<Server*>(h); s->emb = fn; s->emb_user = user; }
TFB_EXPORT void tfb_server_set_model_callbacks(void* h, tfb_load_model_fn load, tfb_unload_model_fn unload, void* user) {
  Server* s = static_cast<Server*>(h);
  s->load_model = load; s->unload_model = unload; s->model_user = user;
}
TFB_EXPORT int tfb_server_is_running(void* h) { return static_cast<Server*>(h)->running ? 1 : 0; }
TFB_EXPORT int tfb_server_current_requests(void* h) { return static_cast<Server*>(h)->current.load(); }
TFB_EXPORT long long tfb_server_total_requests(void* h) { return static_cast<Server*>(h)->total.load(); }
TFB_EXPORT long long tfb_server_total_errors(void* h) { return static_cast<Server*>(h)->errors.load(); }
TFB_EXPORT long long tfb_server_total_tokens(void* h) { return static_cast<Server*>(h)->tokens_out.load(); }
TFB_EXPORT int tfb_server_model_name(void* h, char* out, int cap) {
  const std::string& n = static_cast<Server*>(h)->model_name;
  if (out && cap > 0) { int k = (int)n.size() < cap - 1 ? (int)n.size() : cap - 1; memcpy(out, n.data(), k); out[k] = 0; }
  return (int)n.size();
}
TFB_EXPORT int tfb_server_port(void* h) { return static_cast<Server*>(h)->bound_port; }
TFB_EXPORT double tfb_server_latency_pct(void* h, double p) { return static_cast<Server*>(h)->latency.pct(p); }
TFB_EXPORT double tfb_server_ttft_pct(void* h, double p) { return static_cast<Server*>(h)->ttft.pct(p); }

TFB_EXPORT int tfb_server_start(void* h) {
  Server* s = static_cast<Server*>(h);
  if (s->running) return 0;
  s->listen_fd = socket(AF_INET, SOCK_STREAM, 0);
  if (s->listen_fd < 0) return -1;
  int one = 1;
  setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_ANY);
  a.sin_port = htons(uint16_t(s->port));
  if (bind(s->listen_fd, reinterpret_cast<sockaddr*>(&a), sizeof a) != 0 || listen(s->listen_fd, 256) != 0) {
    close(s->listen_fd);
    s->listen_fd = -1;
    return -1;
  }
  socklen_t al = sizeof a;
  getsockname(s->listen_fd, reinterpret_cast<sockaddr*>(&a), &al);
  s->bound_port = ntohs(a.sin_port);
  s->running = true;
  s->started = std::chrono::steady_clock::now();
  s->accept_thread = std::thread(accept_loop, s);
  for (int i = 0; i < s->workers; ++i) s->pool.emplace_back(worker_loop, s);
  return 0;
}
TFB_EXPORT void tfb_server_stop(void* h) {
  Server* s = static_cast<Server*>(h);
  if (!s->running) return;
  s->running = false;
  s->qcv.notify_all();
  if (s->accept_thread.joinable()) s->accept_thread.join();
  for (auto& t : s->pool) if (t.joinable()) t.join();
  s->pool.clear();
  if (s->listen_fd >= 0) close(s->listen_fd);
  s->listen_fd = -1;
}
// exact-bytes helpers (wire contract)
TFB_EXPORT int tfb_openai_error_json(const char* msg, const char* type, const char* code, char* out, int cap) {
  const std::string j = error_json(msg ? msg : "", type ? type : "", code ? code : "");
  snprintf(out, size_t(cap), "%s", j.c_str());
  return int(j.size());
}
TFB_EXPORT int tfb_sse_data_frame(const char* json, char* out, int cap) {
  const std::string f = std::string("data: ") + json + "\n\n";
  snprintf(out, size_t(cap), "%s", f.c_str());
  return int(f.size());
}
TFB_EXPORT const char* tfb_sse_done_frame() { return "data: [DONE]\n\n"; }
