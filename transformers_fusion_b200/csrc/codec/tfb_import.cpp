// Foreign checkpoint readers for libtfb_codec: GGUF (v1-v3; F32, F16, BF16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0),
// safetensors (F64/F32/F16/BF16/ints/BOOL/F8_E4M3/F8_E5M2, plus block-scaled FP8 pairs) and headerless raw fp32.
// Every tensor is delivered as fp32; the caller re-encodes it into a .quant container.
//
// Reference counterparts: tools/convert.cpp:58-349 (GGUF subset F32/F16/Q4_0/Q4_1/Q8_0),
// src/adapters/include/adapters/safetensors_bridge.h:28-45 (dtype table, load_block_fp8_pair).
// The GGUF block layouts here follow the GGML file format (low nibbles are elements 0..15 of a block, high
// nibbles elements 16..31), and tensor data offsets are relative to the aligned end of the tensor table.
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "tfb_codec.h"

#define TFB_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_err;

struct Ten {
  std::string name, dtype;
  std::vector<long long> shape;   // outermost first
  long long numel = 0;
  uint64_t off = 0, bytes = 0;    // absolute file range
  int ggml = -1;                  // GGML type id, or -1 for safetensors / raw
};

float half_to_float(uint16_t h) {
  const uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
  uint32_t bits;
  if (e == 0) {
    if (m == 0) bits = s << 31;
    else {
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 1024)) { mm <<= 1; ++sh; }
      bits = (s << 31) | ((127 - 15 - sh + 1) << 23) | ((mm & 1023) << 13);
    }
  } else if (e == 31) bits = (s << 31) | 0x7F800000u | (m << 13);
  else bits = (s << 31) | ((e - 15 + 127) << 23) | (m << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
float bf16_to_float(uint16_t h) {
  const uint32_t bits = uint32_t(h) << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
float e4m3_to_float(uint8_t v) {   // "fn" flavour: no infinities, S.1111.111 is NaN
  const int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
  float f;
  if (e == 15 && m == 7) f = NAN;
  else if (e == 0) f = ldexpf(float(m), -9);
  else f = ldexpf(float(8 + m), e - 10);
  return s ? -f : f;
}
float e5m2_to_float(uint8_t v) { return half_to_float(uint16_t(v) << 8); }

// ---- minimal JSON reader (safetensors header) --------------------------------------------------
struct Json {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string str() {
    std::string s;
    ws();
    if (p >= e || *p != '"') { ok = false; return s; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) {
          case 'n': s += '\n'; break;
          case 't': s += '\t'; break;
          case 'u': if (p + 4 < e) { s += '?'; p += 4; } break;
          default: s += *p;
        }
        ++p;
      } else s += *p++;
    }
    if (p >= e) { ok = false; return s; }
    ++p;
    return s;
  }
  double num() {
    ws();
    char* q = nullptr;
    const double v = strtod(p, &q);
    if (q == p) ok = false;
    p = q;
    return v;
  }
  void skip() {   // any value
    ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return;
      do {
        if (open == '{') { str(); if (!eat(':')) { ok = false; return; } }
        skip();
        if (!ok) return;
      } while (eat(','));
      if (!eat(close)) ok = false;
      return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

}  // namespace

struct tfb_import {
  FILE* f = nullptr;
  uint64_t size = 0;
  std::vector<Ten> tensors;
  std::map<std::string, int> by_name;
  std::map<std::string, std::string> meta;
  std::string kind;

  bool read_at(uint64_t off, void* dst, size_t n) const {
    if (off > size || n > size - off) return false;
    if (fseeko(f, off_t(off), SEEK_SET) != 0) return false;
    return fread(dst, 1, n, f) == n;
  }
};

namespace {

// ---- GGUF ----------------------------------------------------------------------------------------
struct Cursor {
  tfb_import* h;
  uint64_t pos;
  bool ok = true;
  bool v1 = false;
  template <class T> T get() {
    T v{};
    if (!ok || !h->read_at(pos, &v, sizeof(T))) { ok = false; return v; }
    pos += sizeof(T);
    return v;
  }
  uint64_t len() { return v1 ? uint64_t(get<uint32_t>()) : get<uint64_t>(); }
  std::string str() {
    const uint64_t n = len();
    if (!ok || n > (1u << 24)) { ok = false; return ""; }   // names and metadata strings are small; vocab entries too
    std::string s(size_t(n), '\0');
    if (n && !h->read_at(pos, &s[0], size_t(n))) { ok = false; return ""; }
    pos += n;
    return s;
  }
};

const size_t kScalarSize[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};

std::string gguf_scalar(Cursor& c, uint32_t t) {
  char buf[64];
  switch (t) {
    case 0: snprintf(buf, 64, "%u", unsigned(c.get<uint8_t>())); break;
    case 1: snprintf(buf, 64, "%d", int(c.get<int8_t>())); break;
    case 2: snprintf(buf, 64, "%u", unsigned(c.get<uint16_t>())); break;
    case 3: snprintf(buf, 64, "%d", int(c.get<int16_t>())); break;
    case 4: snprintf(buf, 64, "%u", c.get<uint32_t>()); break;
    case 5: snprintf(buf, 64, "%d", c.get<int32_t>()); break;
    case 6: snprintf(buf, 64, "%.9g", double(c.get<float>())); break;
    case 7: snprintf(buf, 64, "%d", int(c.get<uint8_t>() != 0)); break;
    case 10: snprintf(buf, 64, "%llu", (unsigned long long)c.get<uint64_t>()); break;
    case 11: snprintf(buf, 64, "%lld", (long long)c.get<int64_t>()); break;
    case 12: snprintf(buf, 64, "%.17g", c.get<double>()); break;
    default: c.ok = false; buf[0] = 0;
  }
  return buf;
}

bool ggml_block(int type, int* elems, int* bytes) {
  switch (type) {
    case 0: *elems = 1; *bytes = 4; return true;     // F32
    case 1: *elems = 1; *bytes = 2; return true;     // F16
    case 30: *elems = 1; *bytes = 2; return true;    // BF16
    case 2: *elems = 32; *bytes = 18; return true;   // Q4_0
    case 3: *elems = 32; *bytes = 20; return true;   // Q4_1
    case 6: *elems = 32; *bytes = 22; return true;   // Q5_0
    case 7: *elems = 32; *bytes = 24; return true;   // Q5_1
    case 8: *elems = 32; *bytes = 34; return true;   // Q8_0
  }
  return false;
}
const char* ggml_name(int t) {
  switch (t) {
    case 0: return "F32"; case 1: return "F16"; case 30: return "BF16"; case 2: return "Q4_0"; case 3: return "Q4_1";
    case 6: return "Q5_0"; case 7: return "Q5_1"; case 8: return "Q8_0";
  }
  return "unsupported";
}

bool parse_gguf(tfb_import* h) {
  Cursor c{h, 0};
  char magic[4];
  if (!h->read_at(0, magic, 4) || memcmp(magic, "GGUF", 4) != 0) { g_err = "not a GGUF file"; return false; }
  c.pos = 4;
  const uint32_t version = c.get<uint32_t>();
  if (version < 1 || version > 3) { g_err = "unsupported GGUF version " + std::to_string(version); return false; }
  c.v1 = version == 1;
  const uint64_t nt = c.len(), nkv = c.len();
  if (!c.ok || nt > (1u << 20) || nkv > (1u << 20)) { g_err = "corrupt GGUF header"; return false; }
  h->meta["gguf.version"] = std::to_string(version);
  for (uint64_t i = 0; i < nkv && c.ok; ++i) {
    const std::string key = c.str();
    const uint32_t t = c.get<uint32_t>();
    if (t == 8) h->meta[key] = c.str();
    else if (t == 9) {
      const uint32_t at = c.get<uint32_t>();
      const uint64_t n = c.len();
      if (at == 8) { for (uint64_t j = 0; j < n && c.ok; ++j) c.str(); }
      else if (at < 13 && kScalarSize[at]) {
        if (n > h->size / kScalarSize[at]) c.ok = false; else c.pos += n * kScalarSize[at];
      } else c.ok = false;    // nested arrays do not occur in model files
      h->meta[key] = "[" + std::to_string(n) + "]";
    } else if (t < 13) h->meta[key] = gguf_scalar(c, t);
    else c.ok = false;
  }
  if (!c.ok) { g_err = "corrupt GGUF metadata"; return false; }
  std::vector<uint64_t> rel(nt);
  h->tensors.resize(nt);
  for (uint64_t i = 0; i < nt && c.ok; ++i) {
    Ten& t = h->tensors[i];
    t.name = c.str();
    const uint32_t nd = c.get<uint32_t>();
    if (!c.ok || nd > 4) { g_err = "bad tensor rank in GGUF"; return false; }
    t.numel = 1;
    std::vector<long long> ne(nd);
    for (uint32_t d = 0; d < nd; ++d) {
      const uint64_t v = c.v1 ? uint64_t(c.get<uint32_t>()) : c.get<uint64_t>();
      if (v == 0 || v > (1ull << 40) || t.numel > (1ll << 50) / (long long)std::max<uint64_t>(v, 1)) { c.ok = false; break; }
      ne[d] = (long long)v;
      t.numel *= (long long)v;
    }
    t.shape.assign(ne.rbegin(), ne.rend());       // GGML lists the fastest dimension first
    t.ggml = int(c.get<uint32_t>());
    rel[i] = c.get<uint64_t>();
    t.dtype = ggml_name(t.ggml);
  }
  if (!c.ok) { g_err = "corrupt GGUF tensor table"; return false; }
  uint64_t align = 32;
  auto it = h->meta.find("general.alignment");
  if (it != h->meta.end()) align = std::max<uint64_t>(1, strtoull(it->second.c_str(), nullptr, 10));
  const uint64_t base = (c.pos + align - 1) / align * align;
  for (uint64_t i = 0; i < nt; ++i) {
    Ten& t = h->tensors[i];
    int el = 0, by = 0;
    t.off = base + rel[i];
    if (ggml_block(t.ggml, &el, &by)) t.bytes = uint64_t((t.numel + el - 1) / el) * by;
    h->by_name[t.name] = int(i);
  }
  return true;
}

long long read_ggml(const tfb_import* h, const Ten& t, float* out) {
  int el = 0, by = 0;
  if (!ggml_block(t.ggml, &el, &by)) { g_err = "unsupported GGML type " + std::to_string(t.ggml) + " (" + t.name + ")"; return -1; }
  std::vector<uint8_t> buf(t.bytes);
  if (!h->read_at(t.off, buf.data(), buf.size())) { g_err = "truncated tensor " + t.name; return -1; }
  const long long n = t.numel;
  auto h16 = [&](const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return half_to_float(v); };
  if (t.ggml == 0) memcpy(out, buf.data(), size_t(n) * 4);
  else if (t.ggml == 1) for (long long i = 0; i < n; ++i) out[i] = h16(&buf[i * 2]);
  else if (t.ggml == 30) for (long long i = 0; i < n; ++i) { uint16_t v; memcpy(&v, &buf[i * 2], 2); out[i] = bf16_to_float(v); }
  else {
    const long long nb = (n + 31) / 32;
    for (long long b = 0; b < nb; ++b) {
      const uint8_t* p = &buf[size_t(b) * by];
      float v[32];
      const float d = h16(p);
      if (t.ggml == 2) for (int j = 0; j < 16; ++j) { v[j] = (float(p[2 + j] & 15) - 8) * d; v[j + 16] = (float(p[2 + j] >> 4) - 8) * d; }
      else if (t.ggml == 3) { const float m = h16(p + 2); for (int j = 0; j < 16; ++j) { v[j] = float(p[4 + j] & 15) * d + m; v[j + 16] = float(p[4 + j] >> 4) * d + m; } }
      else if (t.ggml == 6) {
        uint32_t qh; memcpy(&qh, p + 2, 4);
        for (int j = 0; j < 16; ++j) {
          v[j] = (float((p[6 + j] & 15) | (((qh >> j) & 1) << 4)) - 16) * d;
          v[j + 16] = (float((p[6 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4)) - 16) * d;
        }
      } else if (t.ggml == 7) {
        const float m = h16(p + 2);
        uint32_t qh; memcpy(&qh, p + 4, 4);
        for (int j = 0; j < 16; ++j) {
          v[j] = float((p[8 + j] & 15) | (((qh >> j) & 1) << 4)) * d + m;
          v[j + 16] = float((p[8 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4)) * d + m;
        }
      } else for (int j = 0; j < 32; ++j) v[j] = float(int8_t(p[2 + j])) * d;
      const long long cnt = std::min<long long>(32, n - b * 32);
      memcpy(out + b * 32, v, size_t(cnt) * 4);
    }
  }
  return n;
}

// ---- safetensors ------------------------------------------------------------------------------------
int st_elem_size(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  return 0;
}

bool parse_safetensors(tfb_import* h) {
  uint64_t hl = 0;
  if (!h->read_at(0, &hl, 8) || hl < 2 || hl > h->size - 8 || hl > (1ull << 30)) { g_err = "bad safetensors header length"; return false; }
  std::string hdr(size_t(hl), '\0');
  if (!h->read_at(8, &hdr[0], size_t(hl))) { g_err = "truncated safetensors header"; return false; }
  const uint64_t base = 8 + hl;
  Json j{hdr.data(), hdr.data() + hdr.size()};
  if (!j.eat('{')) { g_err = "safetensors header is not a JSON object"; return false; }
  if (!j.eat('}')) {
    do {
      const std::string name = j.str();
      if (!j.ok || !j.eat(':')) { g_err = "malformed safetensors header"; return false; }
      if (name == "__metadata__") {
        if (j.eat('{') && !j.eat('}')) {
          do {
            const std::string k = j.str();
            if (!j.eat(':')) { j.ok = false; break; }
            j.ws();
            if (j.p < j.e && *j.p == '"') h->meta[k] = j.str(); else j.skip();
          } while (j.ok && j.eat(','));
          if (!j.eat('}')) j.ok = false;
        }
      } else {
        Ten t;
        t.name = name;
        uint64_t a = 0, b = 0;
        if (!j.eat('{')) { g_err = "malformed tensor entry " + name; return false; }
        do {
          const std::string k = j.str();
          if (!j.eat(':')) { j.ok = false; break; }
          if (k == "dtype") t.dtype = j.str();
          else if (k == "shape") {
            if (!j.eat('[')) { j.ok = false; break; }
            if (!j.eat(']')) { do { t.shape.push_back((long long)j.num()); } while (j.ok && j.eat(',')); if (!j.eat(']')) j.ok = false; }
          } else if (k == "data_offsets") {
            if (!j.eat('[')) { j.ok = false; break; }
            a = uint64_t(j.num()); j.eat(','); b = uint64_t(j.num());
            if (!j.eat(']')) j.ok = false;
          } else j.skip();
        } while (j.ok && j.eat(','));
        if (!j.ok || !j.eat('}')) { g_err = "malformed tensor entry " + name; return false; }
        t.numel = 1;
        for (long long d : t.shape) {
          if (d < 0 || (d > 0 && t.numel > (1ll << 50) / d)) { g_err = "bad shape for " + name; return false; }
          t.numel *= d;
        }
        const int es = st_elem_size(t.dtype);
        if (!es) { g_err = "unsupported safetensors dtype " + t.dtype + " (" + name + ")"; return false; }
        if (b < a || b - a != uint64_t(t.numel) * es || base + b > h->size) { g_err = "data range of " + name + " does not match its shape"; return false; }
        t.off = base + a;
        t.bytes = b - a;
        h->by_name[t.name] = int(h->tensors.size());
        h->tensors.push_back(std::move(t));
      }
    } while (j.ok && j.eat(','));
  }
  if (!j.ok) { g_err = "malformed safetensors header"; return false; }
  return true;
}

long long read_st(const tfb_import* h, const Ten& t, float* out) {
  std::vector<uint8_t> buf(t.bytes);
  if (t.bytes && !h->read_at(t.off, buf.data(), buf.size())) { g_err = "truncated tensor " + t.name; return -1; }
  const long long n = t.numel;
  const uint8_t* p = buf.data();
  const std::string& d = t.dtype;
#define CONV(T) for (long long i = 0; i < n; ++i) { T v; memcpy(&v, p + i * sizeof(T), sizeof(T)); out[i] = float(v); }
  if (d == "F32") memcpy(out, p, size_t(n) * 4);
  else if (d == "F64") CONV(double)
  else if (d == "F16") for (long long i = 0; i < n; ++i) { uint16_t v; memcpy(&v, p + i * 2, 2); out[i] = half_to_float(v); }
  else if (d == "BF16") for (long long i = 0; i < n; ++i) { uint16_t v; memcpy(&v, p + i * 2, 2); out[i] = bf16_to_float(v); }
  else if (d == "I64") CONV(int64_t) else if (d == "U64") CONV(uint64_t)
  else if (d == "I32") CONV(int32_t) else if (d == "U32") CONV(uint32_t)
  else if (d == "I16") CONV(int16_t) else if (d == "U16") CONV(uint16_t)
  else if (d == "I8") CONV(int8_t) else if (d == "U8") CONV(uint8_t)
  else if (d == "BOOL") for (long long i = 0; i < n; ++i) out[i] = p[i] ? 1.f : 0.f;
  else if (d == "F8_E4M3") for (long long i = 0; i < n; ++i) out[i] = e4m3_to_float(p[i]);
  else if (d == "F8_E5M2") for (long long i = 0; i < n; ++i) out[i] = e5m2_to_float(p[i]);
  else { g_err = "unsupported dtype " + d; return -1; }
#undef CONV
  return n;
}

long long read_any(const tfb_import* h, int i, float* out, long long cap) {
  if (!h || i < 0 || i >= int(h->tensors.size())) { g_err = "tensor index out of range"; return -1; }
  const Ten& t = h->tensors[i];
  if (t.numel > cap) { g_err = "output buffer too small"; return -1; }
  if (h->kind == "gguf") return read_ggml(h, t, out);
  return read_st(h, t, out);
}

}  // namespace

TFB_EXPORT const char* tfb_import_error() { return g_err.c_str(); }

TFB_EXPORT tfb_import* tfb_import_open(const char* path, const char* kind) {
  g_err.clear();
  FILE* f = fopen(path, "rb");
  if (!f) { g_err = std::string("cannot open ") + path; return nullptr; }
  tfb_import* h = new tfb_import();
  h->f = f;
  fseeko(f, 0, SEEK_END);
  h->size = uint64_t(ftello(f));
  std::string k = kind ? kind : "auto";
  if (k == "auto") {
    char m[4] = {0, 0, 0, 0};
    h->read_at(0, m, 4);
    const std::string p = path;
    if (memcmp(m, "GGUF", 4) == 0) k = "gguf";
    else if (p.size() > 12 && p.compare(p.size() - 12, 12, ".safetensors") == 0) k = "safetensors";
    else k = "rawfp32";
  }
  h->kind = k;
  bool ok = false;
  if (k == "gguf") ok = parse_gguf(h);
  else if (k == "safetensors") ok = parse_safetensors(h);
  else if (k == "rawfp32") {
    if (h->size == 0 || h->size % 4) g_err = "raw fp32 input must be a non-empty multiple of 4 bytes";
    else {
      Ten t;
      t.name = "weights";
      t.dtype = "F32";
      t.numel = (long long)(h->size / 4);
      t.shape = {t.numel};
      t.off = 0;
      t.bytes = h->size;
      h->by_name[t.name] = 0;
      h->tensors.push_back(t);
      ok = true;
    }
  } else g_err = "unknown input format " + k;
  if (!ok) { fclose(f); delete h; return nullptr; }
  return h;
}
TFB_EXPORT void tfb_import_close(tfb_import* h) { if (h) { if (h->f) fclose(h->f); delete h; } }
TFB_EXPORT const char* tfb_import_kind(const tfb_import* h) { return h->kind.c_str(); }
TFB_EXPORT int tfb_import_num_tensors(const tfb_import* h) { return int(h->tensors.size()); }
TFB_EXPORT const char* tfb_import_name(const tfb_import* h, int i) { return (i < 0 || i >= int(h->tensors.size())) ? nullptr : h->tensors[i].name.c_str(); }
TFB_EXPORT const char* tfb_import_dtype(const tfb_import* h, int i) { return (i < 0 || i >= int(h->tensors.size())) ? nullptr : h->tensors[i].dtype.c_str(); }
TFB_EXPORT int tfb_import_ndim(const tfb_import* h, int i) { return (i < 0 || i >= int(h->tensors.size())) ? -1 : int(h->tensors[i].shape.size()); }
TFB_EXPORT long long tfb_import_dim(const tfb_import* h, int i, int d) {
  if (i < 0 || i >= int(h->tensors.size()) || d < 0 || d >= int(h->tensors[i].shape.size())) return -1;
  return h->tensors[i].shape[d];
}
TFB_EXPORT long long tfb_import_numel(const tfb_import* h, int i) { return (i < 0 || i >= int(h->tensors.size())) ? -1 : h->tensors[i].numel; }
TFB_EXPORT int tfb_import_find(const tfb_import* h, const char* name) {
  auto it = h->by_name.find(name);
  return it == h->by_name.end() ? -1 : it->second;
}
TFB_EXPORT long long tfb_import_read(const tfb_import* h, int i, float* out, long long cap) { g_err.clear(); return read_any(h, i, out, cap); }

// FP8 weight + fp32/bf16 scales.  Two scale layouts are accepted: one scale per `block` consecutive elements
// (scale count == ceil(numel / block)), or one per block x block tile of a 2-D weight (scale shape
// [ceil(R / block), ceil(C / block)]).  out = fp8 value * scale.
TFB_EXPORT long long tfb_import_read_block_fp8(const tfb_import* h, int wi, int si, int block, float* out, long long cap) {
  g_err.clear();
  if (!h || wi < 0 || si < 0 || wi >= int(h->tensors.size()) || si >= int(h->tensors.size()) || block <= 0) { g_err = "bad arguments"; return -1; }
  const Ten& w = h->tensors[wi];
  const Ten& s = h->tensors[si];
  if (w.dtype != "F8_E4M3" && w.dtype != "F8_E5M2") { g_err = w.name + " is not an FP8 tensor"; return -1; }
  if (read_any(h, wi, out, cap) < 0) return -1;
  std::vector<float> sc(size_t(std::max<long long>(1, s.numel)));
  if (read_any(h, si, sc.data(), s.numel) < 0) return -1;
  const long long n = w.numel;
  if (s.numel == (n + block - 1) / block && !(w.shape.size() == 2 && s.shape.size() == 2)) {
    for (long long i = 0; i < n; ++i) out[i] *= sc[size_t(i / block)];
    return n;
  }
  if (w.shape.size() == 2) {
    const long long R = w.shape[0], C = w.shape[1], br = (R + block - 1) / block, bc = (C + block - 1) / block;
    if (s.numel == br * bc) {
      for (long long r = 0; r < R; ++r)
        for (long long c = 0; c < C; ++c) out[r * C + c] *= sc[size_t((r / block) * bc + c / block)];
      return n;
    }
    if (s.numel == (n + block - 1) / block) {
      for (long long i = 0; i < n; ++i) out[i] *= sc[size_t(i / block)];
      return n;
    }
  }
  g_err = "scale tensor " + s.name + " does not match " + w.name + " for block " + std::to_string(block);
  return -1;
}
TFB_EXPORT int tfb_import_num_meta(const tfb_import* h) { return int(h->meta.size()); }
TFB_EXPORT const char* tfb_import_meta_key(const tfb_import* h, int i) {
  if (i < 0 || i >= int(h->meta.size())) return nullptr;
  auto it = h->meta.begin();
  std::advance(it, i);
  return it->first.c_str();
}
TFB_EXPORT const char* tfb_import_meta(const tfb_import* h, const char* key) {
  auto it = h->meta.find(key);
  return it == h->meta.end() ? nullptr : it->second.c_str();
}
