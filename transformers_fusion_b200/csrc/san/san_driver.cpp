// Sanitizer harness for the host-side native code: the block codec and the .quant container, the tokenizers and the
// HTTP server are compiled together with this driver under -fsanitize=address,undefined (or -fsanitize=thread) and
// exercised with the inputs most likely to index out of range or race: every format at ragged block sizes, truncated and
// random payloads, truncated / corrupted container and tokenizer files, and a server under concurrent well-formed and
// malformed requests.  Exit code 0 = every section ran and its own checks held; the sanitizer aborts with its own report
// otherwise.  Built by `python -m transformers_fusion_b200.build --sanitize asan|tsan` into lib/bin/tfb_san_<kind>.
//
// Reference counterpart: the QUANT_SANITIZE build (cmake/compiler.cmake:8-11, -fsanitize=address,undefined); the reference
// has no thread-sanitizer configuration.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "../codec/tfb_codec.h"

extern "C" {
typedef void (*tfb_emit_fn)(void* emit_ctx, const char* piece);
typedef int (*tfb_generate_fn)(void* user, const char* prompt, int max_tokens, float temperature, float top_p, int top_k, int stream,
                               tfb_emit_fn emit, void* emit_ctx, int* prompt_tokens, int* completion_tokens);
void* tfb_server_new(int port);
void tfb_server_free(void* h);
void tfb_server_set_workers(void* h, int n);
void tfb_server_set_timeout(void* h, int sec);
void tfb_server_set_max_body(void* h, long long n);
void tfb_server_set_max_header(void* h, int n);
void tfb_server_set_generate(void* h, tfb_generate_fn fn, void* user);
int tfb_server_start(void* h);
void tfb_server_stop(void* h);
int tfb_server_port(void* h);
void* tfb_tok_new(int kind);
void tfb_tok_free(void* h);
int tfb_tok_train(void* h, const char* text, long long n, int vocab_size);
int tfb_tok_vocab_size(void* h);
long long tfb_tok_encode(void* h, const char* text, long long n, int* out, long long cap);
long long tfb_tok_decode(void* h, const int* ids, int n, char* out, long long cap);
int tfb_tok_save(void* h, const char* path);
int tfb_tok_load(void* h, const char* path);
}

static int g_fail = 0;
#define CHECK(cond, what)                                             \
  do {                                                                \
    if (!(cond)) {                                                    \
      std::fprintf(stderr, "san_driver: check failed: %s (%s:%d)\n", what, __FILE__, __LINE__); \
      ++g_fail;                                                       \
    }                                                                 \
  } while (0)

static std::string tmp_path(const char* dir, const char* name) { return std::string(dir) + "/" + name; }

static std::vector<uint8_t> slurp(const std::string& p) {
  std::vector<uint8_t> v;
  if (FILE* f = std::fopen(p.c_str(), "rb")) {
    uint8_t buf[4096];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) v.insert(v.end(), buf, buf + n);
    std::fclose(f);
  }
  return v;
}
static void spit(const std::string& p, const uint8_t* d, size_t n) {
  if (FILE* f = std::fopen(p.c_str(), "wb")) {
    if (n) std::fwrite(d, 1, n, f);
    std::fclose(f);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
static void section_codec() {
  std::mt19937 rng(7);
  std::normal_distribution<float> nd(0.f, 0.05f);
  const uint32_t sizes[] = {1, 5, 31, 32, 33, 96, 255, 256, 257, 1000};
  for (int fmt = 0; fmt < TFB_FORMAT_COUNT; ++fmt) {
    CHECK(tfb_format_name(fmt) != nullptr, "format name");
    CHECK(tfb_format_parse(tfb_format_name(fmt)) == fmt, "format name round trip");
    for (uint32_t n : sizes) {
      std::vector<float> w(n), out(n, 123.f);
      for (float& x : w) x = nd(rng);
      const size_t cap = tfb_block_claimed_bytes(fmt, n);
      std::vector<uint8_t> payload(cap ? cap : 1);
      const long wrote = tfb_quantize_block(fmt, w.data(), n, payload.data(), cap);
      CHECK(wrote >= 0 && size_t(wrote) <= cap, "payload within the claimed size");
      if (wrote < 0) continue;
      tfb_dequantize_block(fmt, payload.data(), size_t(wrote), nullptr, 0, n, out.data());
      // a payload cut short and a payload of noise must decode without reading past their ends (values are arbitrary)
      for (size_t cut : {size_t(0), size_t(wrote) / 2, size_t(wrote) > 0 ? size_t(wrote) - 1 : 0}) {
        std::vector<uint8_t> part(payload.begin(), payload.begin() + cut);   // exact-size heap block: overreads are caught
        tfb_dequantize_block(fmt, part.data(), part.size(), nullptr, 0, n, out.data());
      }
      std::vector<uint8_t> noise(static_cast<size_t>(wrote), uint8_t(0));
      for (uint8_t& b : noise) b = uint8_t(rng());
      tfb_dequantize_block(fmt, noise.data(), noise.size(), nullptr, 0, n, out.data());
    }
  }
  // an encode buffer that is too small is refused, never overrun
  std::vector<float> w(256, 0.01f);
  std::vector<uint8_t> small(3);
  CHECK(tfb_quantize_block(TFB_FMT_Q32, w.data(), 256, small.data(), small.size()) < 0, "short encode buffer refused");
  uint8_t h[32];
  tfb_sha256(reinterpret_cast<const uint8_t*>("abc"), 3, h);
  CHECK(h[0] == 0xba && h[31] == 0xad, "sha256 known answer");
}

static void section_container(const char* dir) {
  std::mt19937 rng(11);
  std::normal_distribution<float> nd(0.f, 0.05f);
  const std::string path = tmp_path(dir, "san.quant");
  std::vector<float> a(5000), b(300);
  for (float& x : a) x = nd(rng);
  for (float& x : b) x = nd(rng);
  const uint8_t cfg[5] = {1, 2, 3, 4, 5};
  tfb_writer* w = tfb_writer_open(path.c_str(), 1, 0, cfg, sizeof cfg);
  CHECK(w != nullptr, "writer opens");
  if (!w) return;
  CHECK(tfb_writer_add_tensor(w, "a.weight", a.data(), (long long)a.size(), tfb_format_parse("Q_8"), 256) == 0, "add tensor");
  CHECK(tfb_writer_add_tensor(w, "b.weight", b.data(), (long long)b.size(), TFB_FMT_Q32, 32768) == 0, "add tensor");
  std::vector<uint8_t> fm(20);
  for (size_t i = 0; i < fm.size(); ++i) fm[i] = uint8_t(i % 2 ? tfb_format_parse("Q_4") : tfb_format_parse("Q_G_4"));
  CHECK(tfb_writer_add_tensor_mixed(w, "c.weight", a.data(), (long long)a.size(), fm.data(), uint32_t(fm.size()), 256) == 0, "add mixed tensor");
  CHECK(tfb_writer_close(w, 1) == 0, "writer closes");
  tfb_reader* r = tfb_reader_open(path.c_str());
  CHECK(r && tfb_reader_valid(r), "reader accepts its own file");
  if (r) {
    CHECK(tfb_reader_num_tensors(r) == 3, "tensor count");
    std::vector<float> out(b.size());
    CHECK(tfb_reader_read_tensor(r, "b.weight", out.data(), (long long)out.size()) == (long long)b.size(), "exact tensor length");
    CHECK(std::memcmp(out.data(), b.data(), b.size() * 4) == 0, "raw tensor is bit-exact");
    CHECK(tfb_reader_read_tensor(r, "a.weight", out.data(), 10) < 0, "short output buffer refused");
    CHECK(tfb_reader_tensor_numel(r, "nope") < 0, "unknown tensor");
    uint8_t small_cfg[2];
    CHECK(tfb_reader_config(r, small_cfg, sizeof small_cfg) == sizeof cfg, "config size reported");
    tfb_reader_close(r);
  }
  // truncations at many offsets and single-byte corruptions: the reader says "invalid" or fails the read; it never walks
  // out of the file image
  const std::vector<uint8_t> img = slurp(path);
  CHECK(img.size() > 64, "file written");
  if (img.size() <= 64) return;
  const std::string bad = tmp_path(dir, "san_bad.quant");
  std::vector<float> out(a.size());
  for (size_t cut = 0; cut < img.size(); cut += (cut < 256 ? 7 : 509)) {
    spit(bad, img.data(), cut);
    if (tfb_reader* rb = tfb_reader_open(bad.c_str())) {
      if (tfb_reader_valid(rb))
        for (uint32_t i = 0; i < tfb_reader_num_tensors(rb); ++i)
          if (const char* nm = tfb_reader_tensor_name(rb, i)) (void)tfb_reader_read_tensor(rb, nm, out.data(), (long long)out.size());
      tfb_reader_close(rb);
    }
  }
  for (int trial = 0; trial < 200; ++trial) {
    std::vector<uint8_t> c = img;
    const size_t pos = rng() % std::min<size_t>(c.size(), 600);      // header, tables and the first block headers
    c[pos] = uint8_t(rng());
    if (trial % 3 == 0) c[(pos + 1) % c.size()] = 0xff;
    spit(bad, c.data(), c.size());
    if (tfb_reader* rb = tfb_reader_open(bad.c_str())) {
      if (tfb_reader_valid(rb))
        for (uint32_t i = 0; i < tfb_reader_num_tensors(rb); ++i)
          if (const char* nm = tfb_reader_tensor_name(rb, i)) (void)tfb_reader_read_tensor(rb, nm, out.data(), (long long)out.size());
      tfb_reader_close(rb);
    }
  }
  // optimizer state
  const std::string op = tmp_path(dir, "san.opt");
  const long long sizes[2] = {100, 7};
  std::vector<float> m0(100, 1.f), m1(7, 2.f), v0(100, 3.f), v1(7, 4.f);
  const float* ms[2] = {m0.data(), m1.data()};
  const float* vs[2] = {v0.data(), v1.data()};
  CHECK(tfb_opt_write(op.c_str(), 5, 1e-3f, 2, sizes, ms, vs) == 0, "opt write");
  int step = 0, np = 0;
  float lr = 0;
  CHECK(tfb_opt_read_header(op.c_str(), &step, &lr, &np) == 0 && step == 5 && np == 2, "opt header");
  std::vector<float> rm0(100), rm1(7), rv0(100), rv1(7);
  float* rms[2] = {rm0.data(), rm1.data()};
  float* rvs[2] = {rv0.data(), rv1.data()};
  CHECK(tfb_opt_read(op.c_str(), 2, sizes, rms, rvs) == 0 && rv1[6] == 4.f, "opt read");
  const std::vector<uint8_t> oimg = slurp(op);
  for (size_t cut = 0; cut < oimg.size(); cut += 37) {
    spit(bad, oimg.data(), cut);
    (void)tfb_opt_read(bad.c_str(), 2, sizes, rms, rvs);
  }
}

static void section_tokenizer(const char* dir) {
  std::string text;
  const char* words[] = {"the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "naïve", "café", "日本語", "🙂"};
  std::mt19937 rng(3);
  for (int i = 0; i < 4000; ++i) {
    text += words[rng() % 12];
    text += (i % 11 == 10) ? "\n" : " ";
  }
  for (int kind = 0; kind < 2; ++kind) {
    void* t = tfb_tok_new(kind);
    CHECK(tfb_tok_train(t, text.data(), (long long)text.size(), 300) == 0, "tokenizer trains");
    CHECK(tfb_tok_vocab_size(t) > 10, "vocabulary built");
    const std::string probe = "the naïve fox 🙂 jumps over 日本語 \xff\xfe broken utf8";
    std::vector<int> ids(4 * probe.size() + 8);
    const long long n = tfb_tok_encode(t, probe.data(), (long long)probe.size(), ids.data(), (long long)ids.size());
    CHECK(n > 0 && n <= (long long)ids.size(), "encode");
    int tiny[2];
    (void)tfb_tok_encode(t, probe.data(), (long long)probe.size(), tiny, 2);           // short output buffer
    std::vector<char> outc(8 * probe.size());
    const long long m = tfb_tok_decode(t, ids.data(), int(n > 0 ? n : 0), outc.data(), (long long)outc.size());
    CHECK(m >= 0, "decode");
    char tinyc[3];
    (void)tfb_tok_decode(t, ids.data(), int(n > 0 ? n : 0), tinyc, 3);                   // short output buffer
    const int wild[4] = {-5, 1 << 30, 0, tfb_tok_vocab_size(t)};
    (void)tfb_tok_decode(t, wild, 4, outc.data(), (long long)outc.size());               // ids out of range
    const std::string p = tmp_path(dir, kind == 0 ? "san.bpe" : "san.tsv");
    CHECK(tfb_tok_save(t, p.c_str()) == 0, "tokenizer saves");
    void* t2 = tfb_tok_new(kind);
    CHECK(tfb_tok_load(t2, p.c_str()) == 0 && tfb_tok_vocab_size(t2) == tfb_tok_vocab_size(t), "tokenizer loads");
    const std::vector<uint8_t> img = slurp(p);
    const std::string bad = tmp_path(dir, "san_bad.tok");
    for (size_t cut = 0; cut < img.size(); cut += 211) {
      spit(bad, img.data(), cut);
      void* t3 = tfb_tok_new(kind);
      if (tfb_tok_load(t3, bad.c_str()) == 0) (void)tfb_tok_encode(t3, probe.data(), (long long)probe.size(), ids.data(), (long long)ids.size());
      tfb_tok_free(t3);
    }
    tfb_tok_free(t2);
    tfb_tok_free(t);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
static std::atomic<int> g_generated{0};
static int gen_cb(void*, const char* prompt, int max_tokens, float, float, int, int, tfb_emit_fn emit, void* ctx, int* pt, int* ct) {
  const int n = max_tokens > 0 && max_tokens < 8 ? max_tokens : 4;
  for (int i = 0; i < n; ++i) emit(ctx, i ? " tok" : "tok");
  *pt = int(std::strlen(prompt));
  *ct = n;
  g_generated.fetch_add(n);
  return 0;
}

static std::string http(int port, const std::string& req, bool half_close_early = false) {
  const int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return "";
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  a.sin_port = htons(uint16_t(port));
  timeval tv{5, 0};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  std::string out;
  if (connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof a) == 0) {
    size_t off = 0;
    while (off < req.size()) {
      const ssize_t k = send(fd, req.data() + off, req.size() - off, MSG_NOSIGNAL);
      if (k <= 0) break;
      off += size_t(k);
    }
    if (half_close_early) shutdown(fd, SHUT_WR);
    char buf[4096];
    ssize_t k;
    while ((k = recv(fd, buf, sizeof buf, 0)) > 0) out.append(buf, size_t(k));
  }
  close(fd);
  return out;
}

static std::string post(const char* path, const std::string& body) {
  return std::string("POST ") + path + " HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nConnection: close\r\nContent-Length: " +
         std::to_string(body.size()) + "\r\n\r\n" + body;
}

static void section_server() {
  void* s = tfb_server_new(0);
  tfb_server_set_workers(s, 4);
  tfb_server_set_timeout(s, 2);
  tfb_server_set_max_body(s, 4096);
  tfb_server_set_max_header(s, 2048);
  tfb_server_set_generate(s, gen_cb, nullptr);
  CHECK(tfb_server_start(s) == 0, "server starts");
  const int port = tfb_server_port(s);
  CHECK(port > 0, "server bound a port");
  std::vector<std::thread> clients;
  std::atomic<int> ok{0};
  for (int c = 0; c < 8; ++c) {
    clients.emplace_back([&, c] {
      for (int i = 0; i < 6; ++i) {
        std::string r;
        switch ((c + i) % 8) {
          case 0: r = http(port, "GET /health HTTP/1.1\r\nHost: x\r\nConnection: close\r\n\r\n"); break;
          case 1: r = http(port, post("/v1/completions", "{\"prompt\": \"hello\", \"max_tokens\": 3}")); break;
          case 2: r = http(port, post("/v1/chat/completions", "{\"messages\": [{\"role\": \"user\", \"content\": \"hi\"}], \"stream\": true}")); break;
          case 3: r = http(port, post("/v1/completions", "{\"prompt\": [1, 2, {\"deep\": [[[[\"x\"]]]]}], \"max_tokens\": \"many\"")); break;   // cut-off JSON
          case 4: r = http(port, post("/v1/completions", std::string(9000, 'a'))); break;                                          // body over the limit
          case 5: r = http(port, "GET /" + std::string(5000, 'b') + " HTTP/1.1\r\n\r\n"); break;                                   // header over the limit
          case 6: r = http(port, "POST /v1/completions HTTP/1.1\r\nContent-Length: 500\r\n\r\n{\"prompt\":", true); break;          // short body, peer closes
          default: r = http(port, "\x16\x03\x01 garbage \r\n\r\n"); break;                                                         // not HTTP
        }
        if (r.compare(0, 9, "HTTP/1.1 ") == 0) ok.fetch_add(1);
      }
    });
  }
  for (auto& t : clients) t.join();
  CHECK(ok.load() >= 24, "well-formed and malformed requests are answered");
  CHECK(g_generated.load() > 0, "the generate callback ran");
  tfb_server_stop(s);
  tfb_server_free(s);
}

int main(int argc, char** argv) {
  const char* dir = argc > 1 ? argv[1] : "/tmp";
  const std::string only = argc > 2 ? argv[2] : "all";
  if (only == "all" || only == "codec") section_codec();
  if (only == "all" || only == "container") section_container(dir);
  if (only == "all" || only == "tokenizer") section_tokenizer(dir);
  if (only == "all" || only == "server") section_server();
  std::printf("san_driver: %s, %d failed check(s)\n", only.c_str(), g_fail);
  return g_fail ? 1 : 0;
}
