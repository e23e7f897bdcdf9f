// ".quant" container reader / writer, ".quant.idx" side-car, SHA-256 and the ".opt" optimizer file.
// Layouts follow the reference (src/codec/quant_format.cpp:175-397,624-721; src/trainer/trainer_core.cpp:865-932);
// deliberate differences: the writer always emits tables before blocks (the order the reference reader
// requires) and the full 22-byte index magic.
#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "tfb_codec.h"

#define TFB_EXPORT extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------------------------------------
// SHA-256
// ------------------------------------------------------------------------------------------------
namespace {
const uint32_t K256[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
void sha_block(uint32_t h[8], const uint8_t* p) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i) w[i] = uint32_t(p[i * 4]) << 24 | uint32_t(p[i * 4 + 1]) << 16 | uint32_t(p[i * 4 + 2]) << 8 | p[i * 4 + 3];
  for (int i = 16; i < 64; ++i) {
    const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
  for (int i = 0; i < 64; ++i) {
    const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
    const uint32_t t1 = hh + S1 + ch + K256[i] + w[i];
    const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
    const uint32_t t2 = S0 + mj;
    hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}
}  // namespace

TFB_EXPORT void tfb_sha256(const uint8_t* data, size_t n, uint8_t out[32]) {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  size_t i = 0;
  for (; i + 64 <= n; i += 64) sha_block(h, data + i);
  uint8_t tail[128] = {0};
  const size_t rem = n - i;
  if (rem) memcpy(tail, data + i, rem);
  tail[rem] = 0x80;
  const size_t total = rem + 1 + 8 <= 64 ? 64 : 128;
  const uint64_t bits = uint64_t(n) * 8;
  for (int k = 0; k < 8; ++k) tail[total - 1 - k] = uint8_t(bits >> (8 * k));
  sha_block(h, tail);
  if (total == 128) sha_block(h, tail + 64);
  for (int k = 0; k < 8; ++k) {
    out[k * 4] = uint8_t(h[k] >> 24); out[k * 4 + 1] = uint8_t(h[k] >> 16);
    out[k * 4 + 2] = uint8_t(h[k] >> 8); out[k * 4 + 3] = uint8_t(h[k]);
  }
}

// ------------------------------------------------------------------------------------------------
// reader
// ------------------------------------------------------------------------------------------------
struct tfb_reader {
  std::vector<uint8_t> data;
  bool valid = false;
  uint32_t version = 0, flags = 0, config_size = 0;
  size_t config_off = 0;
  struct Fmt { uint32_t id; uint8_t fmt; uint32_t cb; };
  std::vector<Fmt> fmts;
  struct Ten { std::string name; uint32_t start, count; };
  std::vector<Ten> tensors;
  std::map<std::string, size_t> by_name;
  std::vector<size_t> block_off;
};

namespace {
template <typename T>
bool rd(const std::vector<uint8_t>& d, size_t& off, T* v) {
  if (off + sizeof(T) > d.size()) return false;
  memcpy(v, d.data() + off, sizeof(T));
  off += sizeof(T);
  return true;
}
const uint64_t kMaxFile = 64ull << 30;
const uint32_t kMaxTensorWeights = 256u << 20;
}  // namespace

TFB_EXPORT tfb_reader* tfb_reader_open(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) return nullptr;
  tfb_reader* r = new tfb_reader();
  fseek(f, 0, SEEK_END);
  const long long sz = ftell(f);
  fseek(f, 0, SEEK_SET);
  if (sz < 16 || uint64_t(sz) > kMaxFile) { fclose(f); return r; }
  r->data.resize(size_t(sz));
  if (fread(r->data.data(), 1, size_t(sz), f) != size_t(sz)) { fclose(f); return r; }
  fclose(f);
  const auto& d = r->data;
  if (memcmp(d.data(), "QUA1", 4) != 0) return r;
  size_t off = 4;
  if (!rd(d, off, &r->version) || !rd(d, off, &r->flags) || !rd(d, off, &r->config_size)) return r;
  if (off + r->config_size > d.size()) return r;
  r->config_off = off;
  off += r->config_size;
  uint32_t nf = 0;
  if (!rd(d, off, &nf) || uint64_t(nf) * 9 > d.size()) return r;
  r->fmts.resize(nf);
  for (uint32_t i = 0; i < nf; ++i)
    if (!rd(d, off, &r->fmts[i].id) || !rd(d, off, &r->fmts[i].fmt) || !rd(d, off, &r->fmts[i].cb)) return r;
  uint32_t nt = 0;
  if (!rd(d, off, &nt) || uint64_t(nt) * 10 > d.size()) return r;
  r->tensors.resize(nt);
  for (uint32_t i = 0; i < nt; ++i) {
    uint16_t len = 0;
    if (!rd(d, off, &len) || off + len > d.size()) return r;
    r->tensors[i].name.assign(reinterpret_cast<const char*>(d.data() + off), len);
    off += len;
    if (!rd(d, off, &r->tensors[i].start) || !rd(d, off, &r->tensors[i].count)) return r;
    const uint64_t end = uint64_t(r->tensors[i].start) + r->tensors[i].count;
    if (end > nf) return r;
    r->by_name[r->tensors[i].name] = i;
  }
  r->block_off.resize(nf);
  for (uint32_t b = 0; b < nf; ++b) {
    r->block_off[b] = off;
    uint32_t nw = 0, cb = 0, ib = 0;
    if (!rd(d, off, &nw) || !rd(d, off, &cb) || off + cb > d.size()) return r;
    off += cb;
    if (!rd(d, off, &ib) || off + ib > d.size()) return r;
    off += ib;
  }
  r->valid = true;
  return r;
}
TFB_EXPORT int tfb_reader_valid(const tfb_reader* r) { return r && r->valid; }
TFB_EXPORT void tfb_reader_close(tfb_reader* r) { delete r; }
TFB_EXPORT uint32_t tfb_reader_version(const tfb_reader* r) { return r->version; }
TFB_EXPORT uint32_t tfb_reader_flags(const tfb_reader* r) { return r->flags; }
TFB_EXPORT uint32_t tfb_reader_config(const tfb_reader* r, uint8_t* out, uint32_t cap) {
  if (r->valid && out) memcpy(out, r->data.data() + r->config_off, std::min(cap, r->config_size));
  return r->config_size;
}
TFB_EXPORT uint32_t tfb_reader_num_tensors(const tfb_reader* r) { return uint32_t(r->tensors.size()); }
TFB_EXPORT uint32_t tfb_reader_num_blocks(const tfb_reader* r) { return uint32_t(r->fmts.size()); }
TFB_EXPORT const char* tfb_reader_tensor_name(const tfb_reader* r, uint32_t i) {
  return i < r->tensors.size() ? r->tensors[i].name.c_str() : nullptr;
}
TFB_EXPORT long long tfb_reader_tensor_numel(const tfb_reader* r, const char* name) {
  if (!r->valid) return -1;
  auto it = r->by_name.find(name);
  if (it == r->by_name.end()) return -1;
  const auto& t = r->tensors[it->second];
  uint64_t total = 0;
  for (uint32_t b = t.start; b < t.start + t.count; ++b) {
    uint32_t nw;
    memcpy(&nw, r->data.data() + r->block_off[b], 4);
    total += nw;
    if (total > kMaxTensorWeights) return -1;
  }
  return (long long)total;
}
TFB_EXPORT int tfb_reader_tensor_format(const tfb_reader* r, const char* name) {
  auto it = r->by_name.find(name);
  if (!r->valid || it == r->by_name.end() || r->tensors[it->second].count == 0) return -1;
  return r->fmts[r->tensors[it->second].start].fmt;
}
// Format bytes of every block of a tensor; returns the block count (or -1), writes at most cap entries.
TFB_EXPORT long tfb_reader_tensor_block_formats(const tfb_reader* r, const char* name, uint8_t* out, long cap) {
  auto it = r->by_name.find(name);
  if (!r->valid || it == r->by_name.end()) return -1;
  const auto& t = r->tensors[it->second];
  for (uint32_t b = 0; b < t.count && long(b) < cap; ++b) out[b] = r->fmts[t.start + b].fmt;
  return long(t.count);
}
// ---- block-level access (reference: QUANTReader::read_block / tensor_blocks / block_sizes, include/quant/quant_format.h:90-140)
// First block and block count of a tensor; returns 0, or -1 for an unknown name.
TFB_EXPORT int tfb_reader_tensor_range(const tfb_reader* r, const char* name, uint32_t* start, uint32_t* count) {
  auto it = r->by_name.find(name);
  if (!r->valid || it == r->by_name.end()) return -1;
  *start = r->tensors[it->second].start;
  *count = r->tensors[it->second].count;
  return 0;
}
// Table entry and payload sizes of block b: {table id, format byte, table codebook bytes, weights, codebook bytes, index bytes}.
TFB_EXPORT int tfb_reader_block_info(const tfb_reader* r, uint32_t b, uint32_t out[6]) {
  if (!r->valid || b >= r->fmts.size()) return -1;
  const uint8_t* p = r->data.data() + r->block_off[b];
  uint32_t nw, cb, ib;
  memcpy(&nw, p, 4);
  memcpy(&cb, p + 4, 4);
  memcpy(&ib, p + 8 + cb, 4);
  out[0] = r->fmts[b].id; out[1] = r->fmts[b].fmt; out[2] = r->fmts[b].cb; out[3] = nw; out[4] = cb; out[5] = ib;
  return 0;
}
// Byte offset of block b's record from the start of the file; -1 for a block that does not exist.
TFB_EXPORT long long tfb_reader_block_offset(const tfb_reader* r, uint32_t b) {
  if (!r->valid || b >= r->block_off.size()) return -1;
  return (long long)r->block_off[b];
}
// Copies the codebook and index bytes of block b (either pointer may be null); returns 0 or -1.
TFB_EXPORT int tfb_reader_block_payload(const tfb_reader* r, uint32_t b, uint8_t* codebook, uint8_t* indices) {
  uint32_t info[6];
  if (tfb_reader_block_info(r, b, info) != 0) return -1;
  const uint8_t* p = r->data.data() + r->block_off[b];
  if (codebook && info[4]) memcpy(codebook, p + 8, info[4]);
  if (indices && info[5]) memcpy(indices, p + 8 + info[4] + 4, info[5]);
  return 0;
}
// Decodes block b alone into out[nw]; returns the weight count, -1 on a bad id, -2 for a foreign stream (see read_tensor).
TFB_EXPORT long long tfb_reader_decode_block(const tfb_reader* r, uint32_t b, float* out, long long cap) {
  uint32_t info[6];
  if (tfb_reader_block_info(r, b, info) != 0 || (long long)info[3] > cap) return -1;
  int fmt = info[1];
  if (fmt >= TFB_FORMAT_COUNT) fmt = TFB_FMT_Q32;
  if (!tfb_format_is_wire_exact(fmt) && !(r->flags & TFB_FLAG_OWN_STREAMS)) return -2;
  const uint8_t* p = r->data.data() + r->block_off[b];
  tfb_dequantize_block(fmt, p + 8 + info[4] + 4, info[5], p + 8, info[4], info[3], out);
  return info[3];
}

TFB_EXPORT long long tfb_reader_read_tensor(const tfb_reader* r, const char* name, float* out, long long cap) {
  const long long numel = tfb_reader_tensor_numel(r, name);
  if (numel < 0 || numel > cap) return -1;
  const auto& t = r->tensors[r->by_name.find(name)->second];
  long long pos = 0;
  for (uint32_t b = t.start; b < t.start + t.count; ++b) {
    const uint8_t* p = r->data.data() + r->block_off[b];
    uint32_t nw, cb, ib;
    memcpy(&nw, p, 4);
    memcpy(&cb, p + 4, 4);
    const uint8_t* cbp = p + 8;
    memcpy(&ib, cbp + cb, 4);
    const uint8_t* ip = cbp + cb + 4;
    int fmt = r->fmts[b].fmt;
    if (fmt >= TFB_FORMAT_COUNT || fmt == 19 + 1000) fmt = TFB_FMT_Q32;  // out-of-range wire bytes decode as raw fp32
    // A format whose block stream this library encodes in its own way can only be decoded when this library wrote the
    // file (the writer marks such files); the same format written by another encoder has a different stream, and
    // decoding it here would return wrong weights without any sign of trouble.
    if (!tfb_format_is_wire_exact(fmt) && !(r->flags & TFB_FLAG_OWN_STREAMS)) return -2;
    tfb_dequantize_block(fmt, ip, ib, cbp, cb, nw, out + pos);
    pos += nw;
  }
  return pos;
}

// ------------------------------------------------------------------------------------------------
// writer
// ------------------------------------------------------------------------------------------------
struct tfb_writer {
  void note_format(int fmt) { if (!tfb_format_is_wire_exact(fmt)) flags |= TFB_FLAG_OWN_STREAMS; }
  std::string path;
  uint32_t version, flags;
  std::vector<uint8_t> config;
  struct Block { uint8_t fmt; uint32_t nw; std::vector<uint8_t> idx; };
  std::vector<Block> blocks;
  struct Ten { std::string name; uint32_t start, count; };
  std::vector<Ten> tensors;
};

TFB_EXPORT tfb_writer* tfb_writer_open(const char* path, uint32_t version, uint32_t flags, const uint8_t* config,
                                       uint32_t config_size) {
  tfb_writer* w = new tfb_writer();
  w->path = path;
  w->version = version;
  w->flags = flags;
  if (config && config_size) w->config.assign(config, config + config_size);
  return w;
}
TFB_EXPORT int tfb_writer_add_tensor(tfb_writer* w, const char* name, const float* data, long long numel, int fmt,
                                     uint32_t block) {
  if (!w || !name || !data || numel <= 0 || fmt < 0 || fmt >= TFB_FORMAT_COUNT || block == 0) return -1;
  tfb_writer::Ten t{name, uint32_t(w->blocks.size()), 0};
  for (long long off = 0; off < numel; off += block) {
    const uint32_t n = uint32_t(std::min<long long>(block, numel - off));
    tfb_writer::Block b;
    b.fmt = uint8_t(fmt);
    w->note_format(fmt);
    b.nw = n;
    b.idx.resize(std::max<size_t>(tfb_block_claimed_bytes(fmt, n), size_t(n) * 4 * (fmt == TFB_FMT_Q32)) + 8 + size_t(n) * 2);
    const long got = tfb_quantize_block(fmt, data + off, n, b.idx.data(), b.idx.size());
    if (got < 0) return -1;
    b.idx.resize(size_t(got));
    w->blocks.push_back(std::move(b));
    ++t.count;
  }
  w->tensors.push_back(std::move(t));
  return 0;
}
// Per-block formats (a planner's mix): fmts[i] encodes weights [i * block, (i + 1) * block).
TFB_EXPORT int tfb_writer_add_tensor_mixed(tfb_writer* w, const char* name, const float* data, long long numel,
                                           const uint8_t* fmts, uint32_t nfmts, uint32_t block) {
  if (!w || !name || !data || !fmts || numel <= 0 || block == 0) return -1;
  if ((numel + block - 1) / block != (long long)nfmts) return -1;
  tfb_writer::Ten t{name, uint32_t(w->blocks.size()), 0};
  for (uint32_t i = 0; i < nfmts; ++i) {
    const long long off = (long long)i * block;
    const uint32_t n = uint32_t(std::min<long long>(block, numel - off));
    const int fmt = fmts[i];
    if (fmt >= TFB_FORMAT_COUNT) return -1;
    tfb_writer::Block b;
    b.fmt = uint8_t(fmt);
    w->note_format(fmt);
    b.nw = n;
    b.idx.resize(std::max<size_t>(tfb_block_claimed_bytes(fmt, n), size_t(n) * 4 * (fmt == TFB_FMT_Q32)) + 8 + size_t(n) * 2);
    const long got = tfb_quantize_block(fmt, data + off, n, b.idx.data(), b.idx.size());
    if (got < 0) return -1;
    b.idx.resize(size_t(got));
    w->blocks.push_back(std::move(b));
    ++t.count;
  }
  w->tensors.push_back(std::move(t));
  return 0;
}
TFB_EXPORT int tfb_writer_close(tfb_writer* w, int write_idx) {
  if (!w) return -1;
  FILE* f = fopen(w->path.c_str(), "wb");
  if (!f) { delete w; return -1; }
  const uint32_t cs = uint32_t(w->config.size());
  fwrite("QUA1", 1, 4, f);
  fwrite(&w->version, 4, 1, f);
  fwrite(&w->flags, 4, 1, f);
  fwrite(&cs, 4, 1, f);
  if (cs) fwrite(w->config.data(), 1, cs, f);
  const uint32_t nf = uint32_t(w->blocks.size());
  fwrite(&nf, 4, 1, f);
  for (uint32_t i = 0; i < nf; ++i) {
    const uint32_t cb = 0;
    fwrite(&i, 4, 1, f);
    fwrite(&w->blocks[i].fmt, 1, 1, f);
    fwrite(&cb, 4, 1, f);
  }
  const uint32_t nt = uint32_t(w->tensors.size());
  fwrite(&nt, 4, 1, f);
  for (const auto& t : w->tensors) {
    const uint16_t len = uint16_t(t.name.size());
    fwrite(&len, 2, 1, f);
    fwrite(t.name.data(), 1, len, f);
    fwrite(&t.start, 4, 1, f);
    fwrite(&t.count, 4, 1, f);
  }
  for (const auto& b : w->blocks) {
    const uint32_t cb = 0, ib = uint32_t(b.idx.size());
    fwrite(&b.nw, 4, 1, f);
    fwrite(&cb, 4, 1, f);
    fwrite(&ib, 4, 1, f);
    if (ib) fwrite(b.idx.data(), 1, ib, f);
  }
  const bool ok = !ferror(f);
  fclose(f);
  if (ok && write_idx) {
    // "<path>.idx": magic (22 bytes) | u32 version | u32 n | per tensor {u16 len, name, sha256(name)}
    FILE* g = fopen((w->path + ".idx").c_str(), "wb");
    if (g) {
      const char magic[] = "TransFormers-FusionIDX";
      const uint32_t ver = 1;
      fwrite(magic, 1, 22, g);
      fwrite(&ver, 4, 1, g);
      fwrite(&nt, 4, 1, g);
      for (const auto& t : w->tensors) {
        const uint16_t len = uint16_t(t.name.size());
        uint8_t h[32];
        tfb_sha256(reinterpret_cast<const uint8_t*>(t.name.data()), t.name.size(), h);
        fwrite(&len, 2, 1, g);
        fwrite(t.name.data(), 1, len, g);
        fwrite(h, 1, 32, g);
      }
      fclose(g);
    }
  }
  delete w;
  return ok ? 0 : -1;
}

// ------------------------------------------------------------------------------------------------
// ".opt"
// ------------------------------------------------------------------------------------------------
TFB_EXPORT int tfb_opt_write(const char* path, int step, float lr, int num_params, const long long* sizes,
                             const float* const* m, const float* const* v) {
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  fwrite(&step, 4, 1, f);
  fwrite(&lr, 4, 1, f);
  fwrite(&num_params, 4, 1, f);
  for (int i = 0; i < num_params; ++i) {
    const int64_t n = sizes[i];
    fwrite(&n, 8, 1, f);
    fwrite(m[i], 4, size_t(n), f);
    fwrite(&n, 8, 1, f);
    fwrite(v[i], 4, size_t(n), f);
  }
  const bool ok = !ferror(f);
  fclose(f);
  return ok ? 0 : -1;
}
TFB_EXPORT int tfb_opt_read_header(const char* path, int* step, float* lr, int* num_params) {
  FILE* f = fopen(path, "rb");
  if (!f) return -1;
  const bool ok = fread(step, 4, 1, f) == 1 && fread(lr, 4, 1, f) == 1 && fread(num_params, 4, 1, f) == 1;
  fclose(f);
  return ok ? 0 : -1;
}
TFB_EXPORT int tfb_opt_read(const char* path, int num_params, const long long* sizes, float* const* m, float* const* v) {
  FILE* f = fopen(path, "rb");
  if (!f) return -1;
  int step, np;
  float lr;
  bool ok = fread(&step, 4, 1, f) == 1 && fread(&lr, 4, 1, f) == 1 && fread(&np, 4, 1, f) == 1 && np == num_params;
  for (int i = 0; ok && i < num_params; ++i) {
    int64_t n = 0;
    ok = fread(&n, 8, 1, f) == 1 && n == sizes[i] && fread(m[i], 4, size_t(n), f) == size_t(n);
    ok = ok && fread(&n, 8, 1, f) == 1 && n == sizes[i] && fread(v[i], 4, size_t(n), f) == size_t(n);
  }
  fclose(f);
  return ok ? 0 : -1;
}
