// Format registry + block codec.  See tfb_codec.h for the compatibility statement.
#include "tfb_codec.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#define TFB_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// ------------------------------------------------------------------------------------------------
// registry: ids follow the reference enum (include/quant/types.h:22-150), bpw = wire truth table
// (include/quant/types.h format_bpw)
// ------------------------------------------------------------------------------------------------
struct FormatInfo {
  std::string name;
  double bpw;
  int bits;     // element width of the family (1,2,3,4,6,8,12,16,24,32)
  int grouped;  // Q_G_* family
  int half;     // *_5 family
  int mix;      // Q_MX / Q_G_MX
  int tier;     // 0 none, 1 L, 2 M, 3 H
};

const int kBits[9] = {1, 2, 3, 4, 6, 8, 12, 16, 24};

std::vector<FormatInfo> build_registry() {
  std::vector<FormatInfo> r(TFB_FORMAT_COUNT);
  const char* tiers[3] = {"_K_L", "_K_M", "_K_H"};
  int id = 0;
  const int base_bits[10] = {1, 2, 3, 4, 6, 8, 12, 16, 24, 32};
  for (int i = 0; i < 10; ++i, ++id) r[id] = {"Q_" + std::to_string(base_bits[i]), double(base_bits[i]), base_bits[i], 0, 0, 0, 0};
  for (int i = 0; i < 9; ++i)
    for (int t = 0; t < 3; ++t, ++id) r[id] = {"Q_" + std::to_string(kBits[i]) + tiers[t], double(kBits[i]), kBits[i], 0, 0, 0, t + 1};
  const double g_bpw[9] = {1.0, 2.625, 3.5, 4.5, 6.5625, 8.5, 12.5, 16.5, 24.5};
  for (int i = 0; i < 9; ++i, ++id) r[id] = {"Q_G_" + std::to_string(kBits[i]), g_bpw[i], kBits[i], 1, 0, 0, 0};
  const double gk_bpw[9] = {1.0, 2.4375, 3.4375, 4.4375, 6.5625, 8.5, 12.5, 16.0, 24.0};
  for (int i = 0; i < 9; ++i)
    for (int t = 0; t < 3; ++t, ++id) r[id] = {"Q_G_" + std::to_string(kBits[i]) + tiers[t], gk_bpw[i], kBits[i], 1, 0, 0, t + 1};
  const double h_bpw[9] = {1.5, 2.4375, 3.5, 4.5, 6.4375, 8.5, 12.5, 16.5, 24.5};
  for (int i = 0; i < 9; ++i, ++id) r[id] = {"Q_" + std::to_string(kBits[i]) + "_5", h_bpw[i], kBits[i], 0, 1, 0, 0};
  for (int i = 0; i < 9; ++i, ++id) r[id] = {"Q_G_" + std::to_string(kBits[i]) + "_5", h_bpw[i], kBits[i], 1, 1, 0, 0};
  const int mx_bits[7] = {3, 4, 6, 8, 12, 16, 24};
  for (int i = 0; i < 7; ++i, ++id) r[id] = {"Q_MX_" + std::to_string(mx_bits[i]) + "_5", mx_bits[i] + 0.5, mx_bits[i], 0, 1, 1, 0};
  for (int i = 0; i < 7; ++i, ++id)
    r[id] = {"Q_G_MX_" + std::to_string(mx_bits[i]) + "_5", i == 0 ? 3.78125 : mx_bits[i] + 0.5, mx_bits[i], 1, 1, 1, 0};
  return r;
}
const std::vector<FormatInfo>& registry() {
  static const std::vector<FormatInfo> r = build_registry();
  return r;
}

std::string canon(const char* s) {
  std::string o;
  for (; *s; ++s) {
    char c = *s;
    if (c == '_' || c == '-' || c == '.' || c == ' ') continue;
    o.push_back(char(c >= 'a' && c <= 'z' ? c - 32 : c));
  }
  return o;
}

// ------------------------------------------------------------------------------------------------
// bit I/O (LSB first), fp16
// ------------------------------------------------------------------------------------------------
struct BitWriter {
  uint8_t* bytes;
  size_t cap, bit = 0;
  BitWriter(uint8_t* b, size_t c) : bytes(b), cap(c) {}
  void put(uint64_t v, int count) {
    for (int i = 0; i < count; ++i, ++bit) {
      if (bit >= cap * 8) return;
      if ((v >> i) & 1) bytes[bit >> 3] |= uint8_t(1u << (bit & 7));
    }
  }
};
struct BitReader {
  const uint8_t* bytes;
  size_t size, bit = 0;
  BitReader(const uint8_t* b, size_t s) : bytes(b), size(s) {}
  uint32_t get(int count) {
    if (bit >= size * 8) return 0;
    const size_t byte = bit >> 3;
    const int off = int(bit & 7);
    uint64_t window = 0;
    const size_t avail = size - byte;
    memcpy(&window, bytes + byte, avail >= 8 ? 8 : avail);
    const uint64_t mask = count >= 64 ? ~0ull : ((1ull << count) - 1ull);
    const uint32_t r = uint32_t((window >> off) & mask);
    const size_t end = bit + size_t(count);
    bit = end <= size * 8 ? end : size * 8;
    return r;
  }
};

uint16_t f32_to_f16(float v) {
  uint32_t b;
  memcpy(&b, &v, 4);
  const uint32_t sign = (b >> 16) & 0x8000u;
  int exp = int((b >> 23) & 0xFF) - 127;
  uint32_t mant = b & 0x7FFFFFu;
  if (exp > 15) return uint16_t(sign | 0x7C00u);
  if (exp >= -14) {
    uint32_t m = (mant >> 13) | 0x400u;
    const uint32_t round_bit = (mant >> 12) & 1u, sticky = (mant & 0xFFFu) ? 1u : 0u;
    if (round_bit && (sticky || (m & 1u))) m += 1;
    if (m >= 0x800u) { m >>= 1; exp += 1; if (exp > 15) return uint16_t(sign | 0x7C00u); }
    return uint16_t(sign | uint32_t(exp + 15) << 10 | (m & 0x3FFu));
  }
  if (exp < -24) return uint16_t(sign);
  const uint32_t m = mant | 0x800000u;
  const int shift = -exp - 1;
  uint32_t mf = m >> shift;
  const uint32_t round_bit = (m >> (shift - 1)) & 1u, sticky = (m & ((1u << (shift - 1)) - 1u)) ? 1u : 0u;
  if (round_bit && (sticky || (mf & 1u))) mf += 1;
  return uint16_t(sign | mf);
}
float f16_to_f32(uint16_t h) {
  const uint32_t sign = uint32_t(h >> 15) << 31;
  const int exp = (h >> 10) & 0x1F;
  uint32_t mant = h & 0x3FFu, bits;
  if (exp == 0) {
    if (!mant) bits = sign;
    else {
      int e = -14;
      while (!(mant & 0x400u)) { mant <<= 1; --e; }
      bits = sign | uint32_t(e + 127) << 23 | (mant & 0x3FFu) << 13;
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | mant << 13;
  else bits = sign | uint32_t(exp - 15 + 127) << 23 | mant << 13;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

// slot positions: `slots` evenly spread weights per block carry one bit less and fund the in-band header
bool is_slot(long long i, long long n, int slots) {
  if (slots <= 0 || n <= 0) return false;
  return ((i + 1) * slots) / n != (i * slots) / n;
}

// ------------------------------------------------------------------------------------------------
// exact families
// ------------------------------------------------------------------------------------------------
const float kQ2Levels[4] = {-1.5104f, -0.4528f, 0.4528f, 1.5104f};
const float kQ4Levels[16] = {-2.7178f, -2.0522f, -1.5995f, -1.2392f, -0.9275f, -0.6508f, -0.3976f, -0.1260f,
                             0.1260f,  0.3976f,  0.6508f,  0.9275f,  1.2392f,  1.5995f,  2.0522f,  2.7178f};
const float* comp8_levels() {  // tanh-companded 8-bit grid, k = 0.02
  static float t[256];
  static bool init = false;
  if (!init) {
    const float k = 0.02f;
    // correctly rounded single-precision tanh (via double): the reference's optimised build carries
    // compile-time-evaluated, correctly rounded table entries, which libm's tanhf misses by one ulp
    // for about a quarter of the grid
    const float den = float(tanh(double(k)));
    for (int j = 0; j < 256; ++j) t[j] = float(tanh(double(k * (float(j) / 127.5f - 1.0f)))) / den;
    init = true;
  }
  return t;
}
float lattice_level(int bits, uint32_t idx) {
  if (bits == 2) return kQ2Levels[idx > 3 ? 3 : idx];
  if (bits == 4) return kQ4Levels[idx > 15 ? 15 : idx];
  return comp8_levels()[idx > 255 ? 255 : idx];
}
uint32_t lattice_nearest(int bits, float v) {
  const int count = 1 << bits;
  if (bits == 8) {
    const float* t = comp8_levels();
    if (v <= t[0]) return 0;
    if (v >= t[255]) return 255;
    int lo = 0, hi = 255;
    while (hi - lo > 1) {
      const int mid = (lo + hi) / 2;
      if (t[mid] <= v) lo = mid; else hi = mid;
    }
    return (v - t[lo] <= t[hi] - v) ? lo : hi;
  }
  uint32_t best = 0;
  float bd = fabsf(v - lattice_level(bits, 0));
  for (int i = 1; i < count; ++i) {
    const float d = fabsf(v - lattice_level(bits, i));
    if (d < bd) { bd = d; best = i; }
  }
  return best;
}
// raw-grid levels used when a block is too small to carry a scale (n < 16): uniform on [-8, 8] for 8 bits
float small_level(int bits, uint32_t idx) {
  if (bits == 2 || bits == 4) return lattice_level(bits, idx);
  return -8.0f + 16.0f * float(idx) / 255.0f;
}
uint32_t small_nearest(int bits, float v) {
  if (bits == 2 || bits == 4) return lattice_nearest(bits, v);
  const float c = std::max(-8.0f, std::min(8.0f, v));
  return uint32_t(lroundf((c + 8.0f) * 255.0f / 16.0f));
}

void enc_lattice(const float* w, int n, int bits, uint8_t* out, size_t cap, int iters) {
  BitWriter bw(out, cap);
  if (n < 16) {
    for (int i = 0; i < n; ++i) bw.put(small_nearest(bits, w[i]), bits);
    return;
  }
  const float R = bits == 2 ? 1.5104f : bits == 4 ? 2.7178f : 1.0f;
  float maxa = 0.f;
  for (int i = 0; i < n; ++i) maxa = std::max(maxa, fabsf(w[i]));
  float s = maxa > 1e-30f ? maxa / R : 0.f;
  // least-squares refinement of the scale against the chosen levels; candidates must survive fp16 rounding
  float best_s = s;
  double best_err = 1e300;
  if (s > 0.f) {
    // coarse scan of the scale (true error including clipping), then least-squares polish from the best
    float scan_best = s;
    double scan_err = 1e300;
    for (int c = 0; c < 8 + 8 * iters; ++c) {
      const float cand = f16_to_f32(f32_to_f16(s * (0.35f + 0.9f * float(c) / float(8 + 8 * iters - 1))));
      if (!(cand > 0.f)) continue;
      double err = 0;
      for (int i = 0; i < n; ++i) {
        uint32_t idx = lattice_nearest(bits, w[i] / cand);
        if (is_slot(i, n, 16)) idx &= ~1u;
        const double d = double(w[i]) - double(lattice_level(bits, idx)) * cand;
        err += d * d;
      }
      if (err < scan_err) { scan_err = err; scan_best = cand; }
    }
    s = scan_best;
  }
  for (int it = 0; it <= iters && s > 0.f; ++it) {
    const float sh = f16_to_f32(f32_to_f16(s));
    double num = 0, den = 0, err = 0;
    for (int i = 0; i < n; ++i) {
      uint32_t idx = lattice_nearest(bits, sh > 0 ? w[i] / sh : 0.f);
      if (is_slot(i, n, 16)) idx &= ~1u;
      const float l = lattice_level(bits, idx);
      num += double(w[i]) * l;
      den += double(l) * l;
      const double d = double(w[i]) - double(l) * sh;
      err += d * d;
    }
    if (err < best_err) { best_err = err; best_s = sh; }
    if (den > 1e-20) s = float(num / den);
    if (!(s > 0.f)) break;
  }
  s = best_s;
  bw.put(f32_to_f16(s), 16);
  const float sh = f16_to_f32(f32_to_f16(s));
  for (int i = 0; i < n; ++i) {
    const bool sl = is_slot(i, n, 16);
    uint32_t idx = lattice_nearest(bits, sh > 0.f ? w[i] / sh : 0.f);
    if (sl) idx &= ~1u;
    bw.put(sl ? (idx >> 1) : idx, bits - (sl ? 1 : 0));
  }
}
void dec_lattice(const uint8_t* b, size_t size, int n, int bits, float* out) {
  BitReader br(b, size);
  if (n < 16) {
    for (int i = 0; i < n; ++i) out[i] = small_level(bits, br.get(bits));
    return;
  }
  const float scale = f16_to_f32(uint16_t(br.get(16)));
  for (int i = 0; i < n; ++i) {
    const bool sl = is_slot(i, n, 16);
    uint32_t idx = br.get(bits - (sl ? 1 : 0));
    if (sl) idx <<= 1;
    out[i] = bits == 8 ? scale * lattice_level(8, idx) : lattice_level(bits, idx) * scale;
  }
}

void enc_q24(const float* w, int n, uint8_t* out) {
  for (int i = 0; i < n; ++i) {
    uint32_t bits;
    memcpy(&bits, &w[i], 4);
    bits >>= 8;
    out[i * 3] = uint8_t(bits);
    out[i * 3 + 1] = uint8_t(bits >> 8);
    out[i * 3 + 2] = uint8_t(bits >> 16);
  }
}
void dec_q24(const uint8_t* b, size_t size, int n, float* out) {
  for (int i = 0; i < n; ++i) {
    uint32_t bits = 0;
    for (int k = 0; k < 3; ++k)
      if (size_t(i) * 3 + k < size) bits |= uint32_t(b[size_t(i) * 3 + k]) << (8 * (k + 1));
    memcpy(&out[i], &bits, 4);
  }
}

size_t q16_packed_bytes(int n) {
  size_t packed = 0;
  for (int start = 0; start < n; start += 256) {
    const int end = std::min(start + 256, n);
    const size_t ng = size_t((end - start + 3) / 4);
    packed += 8 + (ng * 63 + 7) / 8;
  }
  return packed;
}
void enc_q16(const float* w, int n, uint8_t* out) {  // out: 2n bytes, zeroed
  if (q16_packed_bytes(n) > size_t(n) * 2) {
    for (int i = 0; i < n; ++i) {
      const uint16_t h = f32_to_f16(w[i]);
      out[i * 2] = uint8_t(h);
      out[i * 2 + 1] = uint8_t(h >> 8);
    }
    return;
  }
  BitWriter bw(out, size_t(n) * 2);
  for (int start = 0; start < n; start += 256) {
    const int end = std::min(start + 256, n);
    float vmin = 1e30f, vmax = -1e30f;
    for (int i = start; i < end; ++i) { vmin = std::min(vmin, w[i]); vmax = std::max(vmax, w[i]); }
    if (vmin > vmax) vmin = vmax = 0;
    uint32_t imin, imax;
    memcpy(&imin, &vmin, 4);
    memcpy(&imax, &vmax, 4);
    bw.put(imin, 32);
    bw.put(imax, 32);
    const float range = vmax - vmin;
    const float s16 = range > 0 ? 65535.0f / range : 0.f, s15 = range > 0 ? 32767.0f / range : 0.f;
    for (int i = start; i < end; i += 4) {
      uint64_t group = 0;
      for (int k = 0; k < 4; ++k) {
        const int idx = i + k;
        if (idx >= end) continue;
        if (k == 3) {
          long q = lroundf((w[idx] - vmin) * s15);
          q = std::max(0l, std::min(32767l, q));
          group |= uint64_t(q) << 48;
        } else {
          long q = lroundf((w[idx] - vmin) * s16);
          q = std::max(0l, std::min(65535l, q));
          group |= uint64_t(q) << (16 * k);
        }
      }
      bw.put(uint32_t(group & 0xFFFFFFFFu), 32);
      bw.put(uint32_t(group >> 32), 31);
    }
  }
}
void dec_q16(const uint8_t* b, size_t size, int n, float* out) {
  if (q16_packed_bytes(n) > size_t(n) * 2) {
    const size_t avail = std::min(size, size_t(n) * 2);
    for (int i = 0; i < n; ++i) {
      uint16_t h = 0;
      if (size_t(i) * 2 + 1 < avail) h = uint16_t(b[i * 2]) | uint16_t(b[i * 2 + 1]) << 8;
      else if (size_t(i) * 2 < avail) h = b[i * 2];
      out[i] = f16_to_f32(h);
    }
    return;
  }
  BitReader br(b, size);
  for (int start = 0; start < n; start += 256) {
    const int end = std::min(start + 256, n);
    const uint32_t imin = br.get(32), imax = br.get(32);
    float vmin, vmax;
    memcpy(&vmin, &imin, 4);
    memcpy(&vmax, &imax, 4);
    const float range = vmax - vmin;
    const float s16 = range > 0 ? range / 65535.0f : 0.f, s15 = range > 0 ? range / 32767.0f : 0.f;
    for (int i = start; i < end; i += 4) {
      const uint64_t group = uint64_t(br.get(32)) | (uint64_t(br.get(31)) << 32);
      for (int k = 0; k < 4; ++k) {
        const int idx = i + k;
        if (idx >= end) break;
        // single rounding (fused multiply-add), as the reference's FMA-enabled build evaluates it
        if (k == 3) out[idx] = fmaf(float(uint32_t((group >> 48) & 0x7FFFu)), s15, vmin);
        else out[idx] = fmaf(float(uint32_t((group >> (16 * k)) & 0xFFFFu)), s16, vmin);
      }
    }
  }
}

// residual-mean tail shared by the grouped 16 / 24-bit forms: fp16 mean of (w - decoded) per 32 weights
void enc_mean_tail(const float* w, const float* plain, int n, uint8_t* p) {
  for (int g = 0; g < n / 32; ++g) {
    double mean = 0;
    for (int i = 0; i < 32; ++i) mean += double(w[g * 32 + i]) - plain[g * 32 + i];
    const uint16_t h = f32_to_f16(float(mean / 32.0));
    p[0] = uint8_t(h);
    p[1] = uint8_t(h >> 8);
    p += 2;
  }
}
void dec_mean_tail(const uint8_t* p, int n, float* out) {
  for (int g = 0; g < n / 32; ++g) {
    const float m = f16_to_f32(uint16_t(p[0]) | uint16_t(p[1]) << 8);
    p += 2;
    for (int i = 0; i < 32; ++i) out[g * 32 + i] += m;
  }
}

// 1-bit sign family: [fp16 rms scale][sign per kept weight]; 16 slot weights decode to zero
void enc_q1(const float* w, int n, uint8_t* out, size_t cap) {
  BitWriter bw(out, cap);
  if (n < 32) {
    for (int i = 0; i < n; ++i) bw.put(w[i] >= 0.f ? 1 : 0, 1);
    return;
  }
  double s = 0;
  for (int i = 0; i < n; ++i) s += double(w[i]) * w[i];
  bw.put(f32_to_f16(float(sqrt(s / n))), 16);
  for (int i = 0; i < n; ++i)
    if (!is_slot(i, n, 16)) bw.put(w[i] >= 0.f ? 1 : 0, 1);
}
void dec_q1(const uint8_t* b, size_t size, int n, float* out) {
  BitReader br(b, size);
  if (n < 32) {
    for (int i = 0; i < n; ++i) out[i] = br.get(1) ? 1.f : -1.f;
    return;
  }
  const float s = f16_to_f32(uint16_t(br.get(16)));
  for (int i = 0; i < n; ++i) out[i] = is_slot(i, n, 16) ? 0.f : (br.get(1) ? s : -s);
}

// ------------------------------------------------------------------------------------------------
// this library's own budgeted codec for the remaining formats:
//   payload = [per-group fp16 scale, fp16 offset]* then b-bit uniform indices, group size chosen as the
//   smallest power of two >= 16 whose headers fit ceil(bpw * n / 8) bytes; when even one group does
//   not fit (integer-bpw plain formats) `slots` weights give up their low bit to fund the header.
// ------------------------------------------------------------------------------------------------
struct OwnLayout {
  int bits, group, slots;
};
OwnLayout own_layout(int bits, double bpw, int n) {
  const long long budget = (long long)ceil(bpw * n / 8.0) * 8;
  for (int g = 16; g < 2 * n; g <<= 1) {
    const int gg = std::min(g, n);
    const long long groups = (n + gg - 1) / gg;
    if ((long long)n * bits + groups * 32 <= budget) return {bits, gg, 0};
    if (gg == n) break;
  }
  long long need = (long long)n * bits + 32 - budget;  // one group: header funded by slots
  int slots = int(std::max(0ll, need));
  if (slots > n) return {bits, n, -1};  // block too small for any header: raw grid on [-8, 8]
  return {bits, n, slots};
}
void enc_own(const float* w, int n, int bits, double bpw, uint8_t* out, size_t cap) {
  const OwnLayout L = own_layout(bits, bpw, n);
  BitWriter bw(out, cap);
  const uint32_t maxq = bits >= 31 ? 0x7FFFFFFFu : ((1u << bits) - 1u);
  if (L.slots < 0) {
    for (int i = 0; i < n; ++i) {
      const float c = std::max(-8.f, std::min(8.f, w[i]));
      bw.put(uint32_t(llround((c + 8.0) * maxq / 16.0)), bits);
    }
    return;
  }
  const int groups = (n + L.group - 1) / L.group;
  std::vector<float> lo(groups), sc(groups);
  for (int g = 0; g < groups; ++g) {
    const int a = g * L.group, b = std::min(n, a + L.group);
    float mn = w[a], mx = w[a];
    for (int i = a; i < b; ++i) { mn = std::min(mn, w[i]); mx = std::max(mx, w[i]); }
    if (bits <= 6 && mx > mn) {
      // few levels: clipping the tails beats covering the full range; pick the clip that minimises the error
      const float mid = 0.5f * (mn + mx), half = 0.5f * (mx - mn);
      double best = 1e300;
      float best_c = 1.f;
      for (int c = 20; c >= 7; --c) {
        const float h = half * c / 20.f, l0 = mid - h, st = 2.f * h / float(maxq);
        double err = 0;
        for (int i = a; i < b; ++i) {
          const float r = std::max(0.f, std::min(float(maxq), floorf((w[i] - l0) / st + 0.5f)));
          const double d = double(w[i]) - (l0 + r * st);
          err += d * d;
        }
        if (err < best) { best = err; best_c = c / 20.f; }
      }
      mn = mid - half * best_c;
      mx = mid + half * best_c;
    }
    const uint16_t hlo = f32_to_f16(mn);
    float flo = f16_to_f32(hlo);
    if (flo > mn) flo = f16_to_f32(uint16_t(hlo + ((hlo & 0x8000) ? 1 : -1)));  // keep the offset below the minimum
    float s = (mx - flo) / float(maxq);
    uint16_t hs = f32_to_f16(s);
    if (f16_to_f32(hs) * maxq < mx - flo) hs = uint16_t(hs + 1);  // and the range above the maximum
    lo[g] = flo;
    sc[g] = f16_to_f32(hs);
    bw.put(f32_to_f16(flo), 16);
    bw.put(hs, 16);
  }
  for (int i = 0; i < n; ++i) {
    const int g = i / L.group;
    uint32_t q = 0;
    if (sc[g] > 0.f) {
      const double r = (double(w[i]) - lo[g]) / sc[g];
      q = uint32_t(std::max(0.0, std::min(double(maxq), floor(r + 0.5))));
    }
    const bool sl = is_slot(i, n, L.slots);
    if (sl) q &= ~1u;  // slot weights keep the even sub-grid
    bw.put(sl ? (q >> 1) : q, bits - (sl ? 1 : 0));
  }
}
void dec_own(const uint8_t* b, size_t size, int n, int bits, double bpw, float* out) {
  const OwnLayout L = own_layout(bits, bpw, n);
  BitReader br(b, size);
  const uint32_t maxq = bits >= 31 ? 0x7FFFFFFFu : ((1u << bits) - 1u);
  if (L.slots < 0) {
    for (int i = 0; i < n; ++i) out[i] = -8.0f + 16.0f * float(br.get(bits)) / float(maxq);
    return;
  }
  const int groups = (n + L.group - 1) / L.group;
  std::vector<float> lo(groups), sc(groups);
  for (int g = 0; g < groups; ++g) {
    lo[g] = f16_to_f32(uint16_t(br.get(16)));
    sc[g] = f16_to_f32(uint16_t(br.get(16)));
  }
  for (int i = 0; i < n; ++i) {
    const bool sl = is_slot(i, n, L.slots);
    uint32_t q = br.get(bits - (sl ? 1 : 0));
    if (sl) q <<= 1;
    out[i] = lo[i / L.group] + sc[i / L.group] * float(q);
  }
}


// ------------------------------------------------------------------------------------------------
// Families whose wire is shared with files written elsewhere: fixed quantile codebooks (3 / 6 / 12 bit), grouped affine
// lattices with signed per-group offsets, the 6-bit scaled-integer form, the compound 8 / 12 bit forms with one fp16
// scale per 32 weights, the 8-weight-group fallback that small blocks use, and the four-tier mixes.  The decoders follow
// the wire statements of the format (bit order, field order, level tables); the encoders are this library's own fits and
// only have to produce streams those decoders read.
// Reference wire statements: src/codec/block_codec.cpp:360-427 (compound 8), :538-724 (fixed codebooks), :726-945 (8-weight
// groups), :961-1038 (compound 12), :1046-1303 (6-bit scaled integers), :1305-1687 (affine), :1875-2379 (mixes).
// ------------------------------------------------------------------------------------------------
const float kQ3Levels[8] = {-3.0776f, -2.1479f, -1.2879f, -0.4240f, 0.4240f, 1.2879f, 2.1479f, 3.0776f};

// complementary-error-function fit (Chebyshev, fractional error < 1.2e-7) and its inverse by Newton steps: the 6- and 12-bit
// codebooks are the N(0,1) quantile midpoints computed with exactly this arithmetic
double erf_fit(double x) {
  const double t = 1.0 / (1.0 + 0.5 * fabs(x));
  const double tau = t * exp(-x * x - 1.26551223 + t * (1.00002368 + t * (0.37409196 + t * (0.09678418 + t * (-0.18628806 +
                     t * (0.27886807 + t * (-1.13520398 + t * (1.48851587 + t * (-0.82215223 + t * 0.17087277)))))))));
  return x >= 0.0 ? 1.0 - tau : tau - 1.0;
}
double erfinv_fit(double y) {
  if (y <= -0.999999) return -6.0;
  if (y >= 0.999999) return 6.0;
  double z = 0.0;
  for (int it = 0; it < 24; ++it) {
    const double e = erf_fit(z) - y;
    z -= e / (1.1283791670955126 * exp(-z * z));
    if (fabs(e) < 1e-13) break;
  }
  return z;
}
const std::vector<float>& quantile_table(int bits) {   // 6 or 12: ascending negatives then ascending positives mirrored
  static std::vector<float> t6, t12;
  std::vector<float>& t = bits == 6 ? t6 : t12;
  if (t.empty()) {
    const int n = 1 << bits, half = n / 2;
    t.resize(n);
    for (int j = 0; j < half; ++j) {
      const float q = float(erfinv_fit(2.0 * (double(j) + 0.5) / double(n) - 1.0) * sqrt(2.0));
      t[j] = q;
      t[n - 1 - j] = -q;
    }
  }
  return t;
}
float fixed_level(int bits, uint32_t idx) {
  if (bits == 3) return kQ3Levels[idx & 7u];
  const std::vector<float>& t = quantile_table(bits);
  return t[std::min<size_t>(idx, t.size() - 1)];
}
uint32_t fixed_nearest(int bits, float v) {
  if (bits == 3) {
    uint32_t best = 0;
    float bd = fabsf(v - kQ3Levels[0]);
    for (int i = 1; i < 8; ++i) {
      const float d = fabsf(v - kQ3Levels[i]);
      if (d < bd) { bd = d; best = uint32_t(i); }
    }
    return best;
  }
  // the table is antisymmetric: search the positive half for |v|, mirror the index for negative values
  const std::vector<float>& t = quantile_table(bits);
  const int half = int(t.size() / 2);
  const float a = fabsf(v);
  int lo = half, hi = int(t.size()) - 1;
  while (lo < hi) {
    const int mid = (lo + hi) / 2;
    if (t[mid] < a) lo = mid + 1; else hi = mid;
  }
  if (lo > half && (t[lo] - a) >= (a - t[lo - 1])) --lo;
  return v >= 0.0f ? uint32_t(lo) : uint32_t(half - 1 - (lo - half));
}
// uniform grid on [-8, 8] for widths without a shaped table
float uniform_level(int bits, uint32_t idx) {
  if (bits == 2 || bits == 4) return lattice_level(bits, idx);
  const uint32_t maxq = bits >= 24 ? 16777215u : ((1u << bits) - 1u);
  return -8.0f + 16.0f * float(idx) / float(maxq);
}
uint32_t uniform_nearest(int bits, float v) {
  if (bits == 2 || bits == 4) return lattice_nearest(bits, v);
  const uint32_t maxq = bits >= 24 ? 16777215u : ((1u << bits) - 1u);
  const float c = std::max(-8.0f, std::min(8.0f, v));
  return uint32_t(lroundf((c + 8.0f) * float(maxq) / 16.0f));
}
float uniform_max(int bits) { return bits == 2 ? 1.5104f : bits == 4 ? 2.7178f : 8.0f; }

// least-squares scale of w against a level function, a few assign / refit rounds
template <class Near, class Level>
float fit_scale(const float* w, int n, float max_level, Near nearest, Level level, int iters = 3) {
  float maxa = 0.0f;
  for (int i = 0; i < n; ++i) maxa = std::max(maxa, fabsf(w[i]));
  float s = maxa > 1e-30f ? maxa / max_level : 0.0f;
  for (int it = 0; it < iters && s > 0.0f; ++it) {
    double num = 0.0, den = 0.0;
    for (int i = 0; i < n; ++i) {
      const float l = level(nearest(w[i] / s));
      num += double(w[i]) * l;
      den += double(l) * l;
    }
    if (den > 1e-20) s = float(num / den);
  }
  return s > 0.0f ? s : 0.0f;
}

// the decoder multiplies by the fp16-rounded scale: pick, among the fp16 neighbours of a fitted scale, the one with the
// smallest squared error (`sse(c)` = error of the block encoded with scale c)
template <class Sse>
float polish_f16_by(float s, Sse sse, int radius = 2) {
  if (!(s > 0.0f)) return 0.0f;
  const uint16_t h0 = f32_to_f16(s);
  float best = f16_to_f32(h0);
  double best_e = 1e300;
  for (int dlt = -radius; dlt <= radius; ++dlt) {
    const int hc = int(h0) + dlt;
    if (hc <= 0 || hc >= 0x7C00) continue;
    const float c = f16_to_f32(uint16_t(hc));
    const double e = sse(c);
    if (e < best_e) { best_e = e; best = c; }
  }
  return best;
}
template <class Near, class Level>
float polish_f16_scale(const float* w, int n, float s, Near nearest, Level level, int radius = 2) {
  return polish_f16_by(s, [&](float c) {
    double e = 0.0;
    for (int i = 0; i < n; ++i) { const double d = double(level(nearest(w[i] / c))) * c - w[i]; e += d * d; }
    return e;
  }, radius);
}

// Scale search for shaped (non-uniform) codebooks: the least-squares fit started from max|w| / top level can sit in a poor
// local optimum, because a smaller scale moves the bulk of the weights into the dense centre of the table at the price of
// clipping a few outliers, and a larger one trades the sparse tails for the centre.  `effort` > 0 (the K tiers) also tries
// a geometric ladder of scales and keeps the best by `sse`, the exact error of the stream the encoder would write.
template <class Near, class Level, class Sse>
float search_scale_by(const float* w, int n, float max_level, Near nearest, Level level, int effort, Sse sse) {
  float best = polish_f16_by(fit_scale(w, n, max_level, nearest, level, 4), sse, 3);
  if (!(best > 0.0f) || effort <= 0) return best;
  double best_e = sse(best);
  float maxa = 0.0f;
  for (int i = 0; i < n; ++i) maxa = std::max(maxa, fabsf(w[i]));
  const int steps = 8 * effort;
  for (int k = -steps; k <= steps; ++k) {
    if (k == 0) continue;
    const float c = polish_f16_by((maxa / max_level) * powf(3.0f, float(k) / float(steps)), sse, 2);
    if (!(c > 0.0f)) continue;
    const double e = sse(c);
    if (e < best_e) { best_e = e; best = c; }
  }
  return best;
}
template <class Near, class Level>
float search_scale(const float* w, int n, float max_level, Near nearest, Level level, int effort) {
  return search_scale_by(w, n, max_level, nearest, level, effort, [&](float c) {
    double e = 0.0;
    for (int i = 0; i < n; ++i) { const double d = double(level(nearest(w[i] / c))) * c - w[i]; e += d * d; }
    return e;
  });
}

// ---- fixed codebooks: [fp16 scale][indices; 16 evenly spread positions carry bits-1 (the even half of the table)] ----
void enc_fixed(int bits, const float* w, int n, uint8_t* out, size_t cap, int effort = 0) {
  BitWriter bw(out, cap);
  if (n < 16) {
    for (int i = 0; i < n; ++i) bw.put(fixed_nearest(bits, w[i]), bits);
    return;
  }
  auto near = [&](float v) { return fixed_nearest(bits, v); };
  auto lvl = [&](uint32_t i) { return fixed_level(bits, i); };
  // exact error of the stream: the 16 slot positions keep only the even half of the table
  auto sse = [&](float c) {
    double e = 0.0;
    for (int i = 0; i < n; ++i) {
      uint32_t idx = fixed_nearest(bits, w[i] / c);
      if (is_slot(i, n, 16)) idx &= ~1u;
      const double d = double(fixed_level(bits, idx)) * c - w[i];
      e += d * d;
    }
    return e;
  };
  const float s = search_scale_by(w, n, fixed_level(bits, (1u << bits) - 1u), near, lvl, effort, sse);
  bw.put(f32_to_f16(s), 16);
  for (int i = 0; i < n; ++i) {
    const bool sl = is_slot(i, n, 16);
    uint32_t idx = fixed_nearest(bits, s == 0.0f ? 0.0f : w[i] / s);
    if (sl) idx &= ~1u;
    bw.put(sl ? (idx >> 1) : idx, bits - (sl ? 1 : 0));
  }
}
void dec_fixed(int bits, const uint8_t* b, size_t size, int n, float* out) {
  BitReader br(b, size);
  if (n < 16) {
    for (int i = 0; i < n; ++i) out[i] = fixed_level(bits, br.get(bits));
    return;
  }
  const float scale = f16_to_f32(uint16_t(br.get(16)));
  for (int i = 0; i < n; ++i) {
    const bool sl = is_slot(i, n, 16);
    uint32_t idx = br.get(bits - (sl ? 1 : 0));
    if (sl) idx <<= 1;
    out[i] = fixed_level(bits, idx) * scale;
  }
}

// ---- 8-weight groups (what small blocks of the grouped formats fall back to):
//      [levels][3-bit scale code per 8 weights][fp16 d], or [levels][fp16 d], or bare levels, by what the budget affords ----
struct SmallLayout { size_t levels_bytes, sc_bytes; int ng; bool scales, d_only; };
SmallLayout small_layout_enc(int bits, int n, double claimed) {
  SmallLayout L;
  L.levels_bytes = (size_t(n) * bits + 7) / 8;
  L.ng = n >= 8 ? n / 8 : 0;
  L.sc_bytes = size_t((L.ng * 3 + 7) / 8);
  const size_t budget = size_t(ceil(claimed * double(n) / 8.0));
  L.scales = n == 256 || (n >= 8 && L.levels_bytes + L.sc_bytes + 2 <= budget);
  L.d_only = !L.scales && n >= 8 && L.levels_bytes + 2 <= budget;
  return L;
}
size_t enc_small_groups(int bits, const float* w, int n, double claimed, uint8_t* out, size_t cap) {
  const SmallLayout L = small_layout_enc(bits, n, claimed);
  const size_t total = L.levels_bytes + (L.scales ? L.sc_bytes : 0) + ((L.scales || L.d_only) ? 2 : 0);
  BitWriter bw(out, std::min(cap, total));
  auto near = [&](float v) { return uniform_nearest(bits, v); };
  auto lvl = [&](uint32_t i) { return uniform_level(bits, i); };
  if (!L.scales && !L.d_only) {
    for (int i = 0; i < n; ++i) bw.put(near(w[i]), bits);
    return total;
  }
  if (!L.scales) {
    const float d = f16_to_f32(f32_to_f16(fit_scale(w, n, uniform_max(bits), near, lvl)));
    for (int i = 0; i < n; ++i) bw.put(d == 0.0f ? 0u : near(w[i] / d), bits);
    const uint16_t dh = f32_to_f16(d);
    if (L.levels_bytes + 1 < cap) { out[L.levels_bytes] = uint8_t(dh & 0xFF); out[L.levels_bytes + 1] = uint8_t(dh >> 8); }
    return total;
  }
  std::vector<float> s(L.ng);
  float maxs = 0.0f;
  for (int g = 0; g < L.ng; ++g) {
    s[g] = fit_scale(w + g * 8, 8, uniform_max(bits), near, lvl);
    maxs = std::max(maxs, s[g]);
  }
  const float d = maxs > 1e-15f ? f16_to_f32(f32_to_f16(maxs / 7.0f)) : 0.0f;
  std::vector<int> sc(std::max(L.ng, 1), 0);
  for (int g = 0; g < L.ng; ++g) {
    if (d == 0.0f || s[g] == 0.0f) continue;
    const int c0 = std::max(0, std::min(7, int(lroundf(s[g] / d))));
    const int hi_w = (g == L.ng - 1) ? n : g * 8 + 8;          // the last code also serves a ragged tail
    double best_e = 1e300;
    for (int c = std::max(1, c0 - 1); c <= std::min(7, c0 + 1); ++c) {
      const float eff = d * float(c);
      double e = 0.0;
      for (int i = g * 8; i < hi_w; ++i) { const double r = double(lvl(near(w[i] / eff))) * eff - w[i]; e += r * r; }
      if (e < best_e) { best_e = e; sc[g] = c; }
    }
  }
  for (int i = 0; i < n; ++i) {
    const float eff = d * float(sc[std::min(i / 8, std::max(L.ng - 1, 0))]);
    bw.put(eff == 0.0f ? 0u : near(w[i] / eff), bits);
  }
  for (int g = 0; g < L.ng; ++g) bw.put(uint32_t(sc[g]), 3);
  bw.put(f32_to_f16(d), 16);
  return total;
}
void dec_small_groups(int bits, const uint8_t* b, size_t size, int n, float* out) {
  const size_t levels_bytes = (size_t(n) * bits + 7) / 8;
  const int ng = n >= 8 ? n / 8 : 0;
  const size_t sc_bytes = size_t((ng * 3 + 7) / 8);
  float d = 1.0f;
  std::vector<float> sc(std::max(ng, 1), 1.0f);
  if (n >= 8 && size >= levels_bytes + sc_bytes + 2) {
    BitReader br(b, size);
    for (int i = 0; i < n; ++i) br.get(bits);
    for (int g = 0; g < ng; ++g) sc[g] = float(br.get(3));
    d = f16_to_f32(uint16_t(br.get(16)));
  } else if (n >= 8 && size >= levels_bytes + 2) {
    d = f16_to_f32(uint16_t(b[size - 2] | (uint16_t(b[size - 1]) << 8)));
  }
  BitReader br(b, size);
  const int last = std::max(ng - 1, 0);
  for (int i = 0; i < n; ++i) out[i] = uniform_level(bits, br.get(bits)) * d * sc[std::min(i / 8, last)];
}

// ---- grouped affine: w ~ (d * sc_g) * level - dm * mc_g, levels uniform on [0, 1];
//      [levels][sc codes][biased signed offset codes][fp16 d][fp16 dm]; blocks that cannot afford the header use the
//      8-weight-group form ----
float affine_level(int bits, uint32_t idx) {
  const uint32_t maxq = bits == 1 ? 1u : bits == 2 ? 3u : bits == 3 ? 7u : bits == 6 ? 63u : bits == 8 ? 255u : 15u;
  switch (bits) {
    case 1: return float(std::min(idx, 1u));
    case 2: return float(std::min(idx, 3u)) * (1.0f / 3.0f);
    case 3: return float(std::min(idx, 7u)) * (1.0f / 7.0f);
    case 6: return float(std::min(idx, 63u)) * (1.0f / 63.0f);
    case 8: return float(std::min(idx, 255u)) * (1.0f / 255.0f);
    default: (void)maxq; return float(std::min(idx, 15u)) * (1.0f / 15.0f);
  }
}
uint32_t affine_nearest(int bits, float v) {
  const float c = std::max(0.0f, std::min(1.0f, v));
  const float top = bits == 1 ? 1.0f : bits == 4 ? 15.0f : bits == 3 ? 7.0f : bits == 6 ? 63.0f : bits == 8 ? 255.0f : 3.0f;
  return uint32_t(lroundf(c * top));
}
bool affine_fits(int bits, int n, int gsz, int scb, int mb, double claimed, size_t* sc_bytes, size_t* min_bytes) {
  const size_t levels_bytes = (size_t(n) * bits + 7) / 8;
  const int ng = n >= gsz ? n / gsz : 0;
  *sc_bytes = size_t((ng * scb + 7) / 8);
  *min_bytes = size_t((ng * mb + 7) / 8);
  const size_t budget = size_t(ceil(claimed * double(n) / 8.0));
  return ng > 0 && levels_bytes + *sc_bytes + *min_bytes + 4 <= budget;
}
size_t enc_affine(int bits, const float* w, int n, int gsz, int scb, int mb, double claimed, uint8_t* out, size_t cap) {
  size_t scB, mnB;
  if (!affine_fits(bits, n, gsz, scb, mb, claimed, &scB, &mnB)) return enc_small_groups(bits, w, n, claimed, out, cap);
  const int ng = n / gsz, scq = (1 << scb) - 1, mq = (1 << mb) - 1, bias = (mq + 1) / 2;
  const size_t total = (size_t(n) * bits + 7) / 8 + scB + mnB + 4;
  std::vector<float> s(ng), m(ng);
  float max_s = 0.0f, max_m = 0.0f;
  for (int g = 0; g < ng; ++g) {
    // range fit, then two least-squares refits of (scale, offset) against the assigned levels
    float lo = 1e30f, hi = -1e30f;
    for (int i = 0; i < gsz; ++i) { lo = std::min(lo, w[g * gsz + i]); hi = std::max(hi, w[g * gsz + i]); }
    float sg = hi - lo, mg = lo;
    for (int it = 0; it < 2 && fabsf(sg) > 1e-30f; ++it) {
      double sw = 0, sl = 0, sl2 = 0, sx = 0, sxl = 0;
      for (int i = 0; i < gsz; ++i) {
        const double l = affine_level(bits, affine_nearest(bits, (w[g * gsz + i] - mg) / sg));
        sw += 1.0; sl += l; sl2 += l * l; sx += w[g * gsz + i]; sxl += double(w[g * gsz + i]) * l;
      }
      const double D = sw * sl2 - sl * sl;
      if (D > 1e-20) { sg = float((sw * sxl - sx * sl) / D); mg = float((sl2 * sx - sl * sxl) / D); }
    }
    if (!(fabsf(sg) > 1e-30f)) { sg = 0.0f; mg = fabsf(hi) > 1e-30f ? lo : 0.0f; }
    s[g] = sg; m[g] = mg;
    max_s = std::max(max_s, fabsf(sg));
    max_m = std::max(max_m, fabsf(mg));
  }
  const float d = max_s > 1e-15f ? f16_to_f32(f32_to_f16(max_s / float(scq))) : 0.0f;
  const float dm = max_m > 1e-15f ? f16_to_f32(f32_to_f16(max_m / float(bias))) : 0.0f;
  BitWriter bw(out, std::min(cap, total));
  std::vector<int> sc(ng, 0), mc(ng, 0);
  for (int g = 0; g < ng; ++g) {
    sc[g] = (d == 0.0f || s[g] <= 0.0f) ? 0 : std::max(0, std::min(scq, int(lroundf(s[g] / d))));
    mc[g] = dm == 0.0f ? 0 : std::max(-bias, std::min(mq - bias, int(lroundf(-m[g] / dm))));
    if (sc[g] == 0) continue;
    // the fit above ignored the snapping of (scale, offset) to their code grids: refit against the snapped values and
    // search the neighbouring codes for the pair with the smallest error
    auto sse = [&](int c, int o) {
      const float es = d * float(c), em = -dm * float(o);
      double e = 0.0;
      for (int i = 0; i < gsz; ++i) {
        const float x = w[g * gsz + i];
        const double r = double(fmaf(es, affine_level(bits, affine_nearest(bits, (x - em) / es)), em)) - x;
        e += r * r;
      }
      return e;
    };
    for (int round = 0; round < 3; ++round) {
      int bc = sc[g], bo = mc[g];
      double be = sse(bc, bo);
      for (int dc = -1; dc <= 1; ++dc)
        for (int dof = -1; dof <= 1; ++dof) {
          const int c = sc[g] + dc, o = mc[g] + dof;
          if (c < 1 || c > scq || o < -bias || o > mq - bias || (dm == 0.0f && o != 0)) continue;
          const double e = sse(c, o);
          if (e < be) { be = e; bc = c; bo = o; }
        }
      if (bc == sc[g] && bo == mc[g]) break;
      sc[g] = bc; mc[g] = bo;
    }
  }
  for (int g = 0; g < ng; ++g) {
    const float es = d * float(sc[g]), em = -dm * float(mc[g]);
    for (int i = 0; i < gsz; ++i) bw.put(es == 0.0f ? 0u : affine_nearest(bits, (w[g * gsz + i] - em) / es), bits);
  }
  for (int i = ng * gsz; i < n; ++i) bw.put(0u, bits);      // a ragged tail decodes to zero
  for (int g = 0; g < ng; ++g) bw.put(uint32_t(sc[g]), scb);
  for (int g = 0; g < ng; ++g) bw.put(uint32_t(mc[g] + bias), mb);
  bw.put(f32_to_f16(d), 16);
  bw.put(f32_to_f16(dm), 16);
  return total;
}
void dec_affine(int bits, const uint8_t* b, size_t size, int n, int gsz, int scb, int mb, double claimed, float* out) {
  size_t scB, mnB;
  if (!affine_fits(bits, n, gsz, scb, mb, claimed, &scB, &mnB)) { dec_small_groups(bits, b, size, n, out); return; }
  const int ng = n / gsz, mq = (1 << mb) - 1, bias = (mq + 1) / 2;
  BitReader br(b, size);
  std::vector<uint8_t> idx(n);
  for (int i = 0; i < n; ++i) idx[i] = uint8_t(br.get(bits));
  std::vector<float> sc(ng), mc(ng);
  for (int g = 0; g < ng; ++g) sc[g] = float(br.get(scb));
  for (int g = 0; g < ng; ++g) mc[g] = float(br.get(mb)) - float(bias);
  const float d = f16_to_f32(uint16_t(br.get(16)));
  const float dm = f16_to_f32(uint16_t(br.get(16)));
  for (int g = 0; g < ng; ++g) {
    const float es = d * sc[g], neg = -(dm * mc[g]);
    for (int k = 0; k < gsz; ++k) out[g * gsz + k] = fmaf(es, affine_level(bits, idx[g * gsz + k]), neg);   // one rounding
  }
}

// ---- 6-bit scaled integers: w ~ d * sc_g * (code - 32), int8 scale per 16 weights: [levels][int8 scales][fp16 d] ----
int round_to_level6(float r) {
  r = std::max(-4000.0f, std::min(4000.0f, r));
  return std::max(-32, std::min(31, int(lrintf(r))));
}
size_t enc_6s(const float* w, int n, uint8_t* out, size_t cap) {
  const bool has_d = n >= 8;
  const int scn = n >= 32 ? n / 16 : 0;
  const size_t levels_bytes = (size_t(n) * 6 + 7) / 8;
  const size_t budget = size_t(ceil(6.5625 * double(n) / 8.0));
  const bool scales = n == 256 || (n >= 32 && levels_bytes + size_t(scn) + 2 <= budget);
  const size_t total = levels_bytes + (scales ? size_t(scn) : 0) + (has_d ? 2 : 0);
  BitWriter bw(out, std::min(cap, total));
  if (!has_d) {
    for (int i = 0; i < n; ++i) bw.put(uint32_t(round_to_level6(w[i]) + 32), 6);
    return total;
  }
  float maxa = 0.0f;
  for (int i = 0; i < n; ++i) maxa = std::max(maxa, fabsf(w[i]));
  if (!scales) {
    const float d = f16_to_f32(f32_to_f16(maxa / 31.0f));
    for (int i = 0; i < n; ++i) bw.put(uint32_t((d == 0.0f ? 0 : round_to_level6(w[i] / d)) + 32), 6);
    const uint16_t dh = f32_to_f16(d);
    out[total - 2] = uint8_t(dh & 0xFF); out[total - 1] = uint8_t(dh >> 8);
    return total;
  }
  // per-group real scale = group max / 31; the int8 codes share one fp16 step d
  std::vector<float> gs((n + 15) / 16, 0.0f);
  float maxg = 0.0f;
  for (int g = 0; g < int(gs.size()); ++g) {
    float ma = 0.0f;
    for (int i = g * 16; i < std::min(n, g * 16 + 16); ++i) ma = std::max(ma, fabsf(w[i]));
    gs[g] = ma / 31.0f;
    maxg = std::max(maxg, gs[g]);
  }
  const float d = f16_to_f32(f32_to_f16(maxg / 127.0f));
  std::vector<int> sc(gs.size(), 0);
  for (size_t g = 0; g < gs.size(); ++g) sc[g] = d == 0.0f ? 0 : std::max(0, std::min(127, int(ceilf(gs[g] / d))));
  for (int g = scn; g < int(sc.size()); ++g) sc[g] = sc[scn - 1];           // a partial last group shares the last code
  for (int i = 0; i < n; ++i) {
    const float eff = d * float(sc[i / 16]);
    bw.put(uint32_t((eff == 0.0f ? 0 : round_to_level6(w[i] / eff)) + 32), 6);
  }
  for (int g = 0; g < scn; ++g) out[levels_bytes + g] = uint8_t(int8_t(sc[g]));
  const uint16_t dh = f32_to_f16(d);
  out[total - 2] = uint8_t(dh & 0xFF); out[total - 1] = uint8_t(dh >> 8);
  return total;
}
void dec_6s(const uint8_t* b, size_t size, int n, float* out) {
  const bool has_d = n >= 8;
  const int scn = n >= 32 ? n / 16 : 0;
  const size_t levels_bytes = (size_t(n) * 6 + 7) / 8;
  float d = 1.0f;
  std::vector<float> sc((n + 15) / 16, 1.0f);
  if (has_d && size >= levels_bytes + 2) {
    d = f16_to_f32(uint16_t(b[size - 2] | (uint16_t(b[size - 1]) << 8)));
    const size_t have = size >= levels_bytes + 2 + size_t(scn) ? size_t(scn) : 0;
    for (size_t g = 0; g < have; ++g) sc[g] = float(int8_t(b[size - 2 - have + g]));
    if (have > 0) for (size_t g = have; g < sc.size(); ++g) sc[g] = sc[have - 1];
  }
  BitReader br(b, size);
  for (int i = 0; i < n; ++i) {
    const float e = d * sc[i / 16];
    out[i] = e * float(int(br.get(6) & 63u) - 32);
  }
}

// ---- compound forms: plain codes followed by one fp16 scale per 32 weights ----
bool compound_fits(int bits, int n) {
  return n >= 32 && n % 32 == 0 && size_t(n) * bits + size_t(n / 32) * 16 == size_t(ceil((bits + 0.5) * double(n)));
}
size_t enc_compound8(const float* w, int n, uint8_t* out, size_t cap) {
  const int ng = n / 32;
  const size_t total = size_t(n) + size_t(ng) * 2;
  if (cap < total) return total;
  for (int g = 0; g < ng; ++g) {
    const float s = f16_to_f32(f32_to_f16(fit_scale(w + g * 32, 32, 1.0f, [&](float v) { return lattice_nearest(8, v); },
                                                    [&](uint32_t i) { return lattice_level(8, i); })));
    for (int i = 0; i < 32; ++i) out[g * 32 + i] = uint8_t(s > 0.0f ? lattice_nearest(8, w[g * 32 + i] / s) : 0u);
    const uint16_t h = f32_to_f16(s);
    out[n + g * 2] = uint8_t(h & 0xFF); out[n + g * 2 + 1] = uint8_t(h >> 8);
  }
  return total;
}
void dec_compound8(const uint8_t* b, size_t size, int n, float* out) {
  const int ng = n / 32;
  if (size < size_t(n) + size_t(ng) * 2) return;
  for (int i = 0; i < n; ++i) {
    const uint8_t* sp = b + n + size_t(i >> 5) * 2;
    out[i] = f16_to_f32(uint16_t(sp[0] | (uint16_t(sp[1]) << 8))) * lattice_level(8, b[i]);
  }
}
size_t enc_compound12(const float* w, int n, uint8_t* out, size_t cap, int effort = 0) {
  const int ng = n / 32;
  const size_t total = (size_t(n) * 12 + size_t(ng) * 16 + 7) / 8;
  BitWriter bw(out, std::min(cap, total));
  std::vector<float> s(ng);
  for (int g = 0; g < ng; ++g)
    s[g] = search_scale(w + g * 32, 32, fixed_level(12, 4095), [&](float v) { return fixed_nearest(12, v); },
                        [&](uint32_t i) { return fixed_level(12, i); }, effort);
  for (int g = 0; g < ng; ++g)
    for (int i = 0; i < 32; ++i) bw.put(s[g] > 0.0f ? fixed_nearest(12, w[g * 32 + i] / s[g]) : 0u, 12);
  for (int g = 0; g < ng; ++g) bw.put(f32_to_f16(s[g]), 16);
  return total;
}
void dec_compound12(const uint8_t* b, size_t size, int n, float* out) {
  const int ng = n / 32;
  if (size * 8 < size_t(n) * 12 + size_t(ng) * 16) return;
  BitReader br(b, size);
  std::vector<uint32_t> code(n);
  for (int i = 0; i < n; ++i) code[i] = br.get(12);
  std::vector<float> sc(ng);
  for (int g = 0; g < ng; ++g) sc[g] = f16_to_f32(uint16_t(br.get(16)));
  for (int i = 0; i < n; ++i) out[i] = sc[i / 32] * fixed_level(12, code[i]);
}

// ---- four-tier mixes: a 2-bit tier per weight, then each tier's values at its own width, then the tiers' fp16 scales
//      (one per tier; the most populated tier of the grouped formats carries one per 32 of its weights) ----
struct MixTier { int bits; float percent; };
void mix_config(int fmt, MixTier c[4], bool* grouped) {
  static const MixTier plain[7][4] = {{{1, 92.0f}, {2, 1.5f}, {4, 6.0f}, {32, 0.5f}},  {{1, 58.5f}, {2, 2.0f}, {4, 39.0f}, {32, 0.5f}},
                                      {{1, 1.5f}, {2, 4.0f}, {4, 93.0f}, {32, 1.5f}},  {{1, 2.5f}, {2, 1.0f}, {4, 88.0f}, {32, 8.5f}},
                                      {{1, 0.5f}, {3, 2.0f}, {8, 87.5f}, {32, 10.0f}}, {{1, 4.5f}, {2, 7.0f}, {16, 88.0f}, {32, 0.5f}},
                                      {{1, 2.5f}, {2, 5.0f}, {24, 92.0f}, {32, 0.5f}}};
  static const MixTier grp[7][4] = {{{1, 92.0f}, {2, 4.0f}, {4, 3.0f}, {32, 1.0f}},   {{1, 58.5f}, {2, 1.0f}, {4, 39.5f}, {32, 1.0f}},
                                    {{1, 0.5f}, {3, 5.0f}, {4, 93.0f}, {32, 1.5f}},   {{1, 0.5f}, {3, 2.0f}, {4, 89.0f}, {32, 8.5f}},
                                    {{1, 1.5f}, {2, 2.5f}, {8, 85.0f}, {32, 11.0f}},  {{1, 10.0f}, {2, 1.0f}, {16, 88.0f}, {32, 1.0f}},
                                    {{1, 2.5f}, {2, 5.0f}, {24, 91.5f}, {32, 1.0f}}};
  const FormatInfo& f = registry()[fmt];
  int k = 0;
  const int mb[7] = {3, 4, 6, 8, 12, 16, 24};
  for (int i = 0; i < 7; ++i) if (mb[i] == f.bits) k = i;
  *grouped = f.grouped != 0;
  for (int t = 0; t < 4; ++t) c[t] = f.grouped ? grp[k][t] : plain[k][t];
}
struct MixPlan { int c[4], nsc[4], dom; bool collapsed; size_t payload_bytes, scale_bytes; };
MixPlan mix_plan(int fmt, int n, const MixTier cfg[4], bool grouped) {
  MixPlan P;
  int* c = P.c;
  for (int i = 0; i < 3; ++i) c[i] = std::max(1, int(lround(cfg[i].percent * 0.01 * double(n))));
  c[3] = n - c[0] - c[1] - c[2];
  if (c[3] < 1) {
    c[3] = 1;
    int excess = c[0] + c[1] + c[2] + 1 - n;
    for (int i = 0; i < 3 && excess > 0; ++i) { const int rem = std::min(c[i] - 1, excess); c[i] -= rem; excess -= rem; }
  }
  for (int i = 0; i < 4; ++i) c[i] = std::max(0, std::min(n, c[i]));
  int sum = c[0] + c[1] + c[2] + c[3];
  for (int i = 0; i < 4 && sum > n; ++i) { const int rem = std::min(c[i], sum - n); c[i] -= rem; sum -= rem; }
  const size_t budget_bits = size_t(ceil(float(registry()[fmt].bpw) * double(n)));
  auto dominant = [&]() { int d = 0; for (int t = 1; t < 4; ++t) if (c[t] > c[d]) d = t; return d; };
  // shrink the widest tiers until the stream fits the claimed size
  for (int guard = 0; guard < 4 * n; ++guard) {
    size_t total = size_t(2) * n;
    for (int t = 0; t < 4; ++t) total += size_t(c[t]) * cfg[t].bits;
    const int dom = dominant();
    for (int t = 0; t < 4; ++t)
      if (cfg[t].bits < 16) total += (grouped && t == dom) ? size_t(16) * ((c[t] + 31) / 32) : 16;
    if (total <= budget_bits) break;
    bool moved = false;
    for (int t = 3; t >= 1; --t)
      if (c[t] > 1 && cfg[t].bits > cfg[t - 1].bits) { --c[t]; ++c[t - 1]; moved = true; break; }
    if (!moved) break;
  }
  P.dom = dominant();
  size_t payload = size_t(2) * n, scales = 0;
  for (int t = 0; t < 4; ++t) payload += size_t(c[t]) * cfg[t].bits;
  for (int t = 0; t < 4; ++t)
    if (cfg[t].bits < 16 && c[t] > 0) scales += size_t((grouped && t == P.dom) ? (c[t] + 31) / 32 : 1) * 2;
  P.collapsed = (payload + 7) / 8 + scales > (budget_bits + 7) / 8;
  if (P.collapsed) { c[0] = n; c[1] = c[2] = c[3] = 0; }
  P.scale_bytes = 0;
  for (int t = 0; t < 4; ++t) {
    P.nsc[t] = 0;
    if (P.collapsed || cfg[t].bits >= 16 || c[t] == 0) continue;
    P.nsc[t] = (grouped && t == P.dom) ? (c[t] + 31) / 32 : 1;
    P.scale_bytes += size_t(P.nsc[t]) * 2;
  }
  size_t bits = size_t(2) * n;
  for (int t = 0; t < 4; ++t) bits += size_t(c[t]) * cfg[t].bits;
  P.payload_bytes = (bits + 7) / 8;
  return P;
}
float mix_level(int bits, uint32_t code) {
  switch (bits) {
    case 1: return code ? 1.0f : -1.0f;
    case 2: return kQ2Levels[code & 3u];
    case 3: return kQ3Levels[code & 7u];
    case 4: return kQ4Levels[code & 15u];
    case 6: return fixed_level(6, code);
    case 12: return fixed_level(12, code);
    default: return uniform_level(8, code);
  }
}
uint32_t mix_nearest(int bits, float v) {
  switch (bits) {
    case 1: return v >= 0.0f ? 1u : 0u;
    case 2: case 4: case 8: return uniform_nearest(bits, v);
    default: return fixed_nearest(bits, v);
  }
}
float mix_max(int bits) {
  switch (bits) {
    case 1: return 1.0f;
    case 2: return 1.5104f;
    case 3: return kQ3Levels[7];
    case 4: return 2.7178f;
    case 6: return fixed_level(6, 63);
    case 8: return 8.0f;
    default: return fixed_level(12, 4095);
  }
}
size_t enc_mix(int fmt, const float* w, int n, uint8_t* out, size_t cap) {
  MixTier cfg[4];
  bool grouped;
  mix_config(fmt, cfg, &grouped);
  const MixPlan P = mix_plan(fmt, n, cfg, grouped);
  const size_t total = P.payload_bytes + P.scale_bytes;
  if (cap < total) return total;
  // the widest tiers take the largest magnitudes
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return fabsf(w[a]) > fabsf(w[b]); });
  std::vector<uint8_t> tier(n, 0);
  int pos = 0;
  for (int t = 3; t >= 0; --t)
    for (int k = 0; k < P.c[t]; ++k) tier[order[pos++]] = uint8_t(t);
  std::vector<std::vector<int>> members(4);
  for (int i = 0; i < n; ++i) members[tier[i]].push_back(i);
  BitWriter bw(out, P.payload_bytes);
  for (int i = 0; i < n; ++i) bw.put(tier[i], 2);
  std::vector<std::vector<float>> sc(4);
  for (int t = 0; t < 4; ++t) {
    const int bits = cfg[t].bits, cnt = int(members[t].size());
    sc[t].assign(std::max(P.nsc[t], 0), 0.0f);
    for (int base = 0; base < cnt; base += 32) {
      const int len = std::min(32, cnt - base);
      float s = 1.0f;
      if (P.nsc[t] > 0) {
        const int g = std::min(base / 32, P.nsc[t] - 1);
        if (P.nsc[t] == 1 ? base == 0 : true) {
          // scale of this run (whole tier when it has a single scale): mean magnitude for signs, max / top level otherwise
          const int lo = P.nsc[t] == 1 ? 0 : base, hi = P.nsc[t] == 1 ? cnt : base + len;
          double acc = 0.0;
          float ma = 0.0f;
          for (int k = lo; k < hi; ++k) { acc += fabsf(w[members[t][k]]); ma = std::max(ma, fabsf(w[members[t][k]])); }
          if (bits == 1) sc[t][g] = f16_to_f32(f32_to_f16(float(acc / std::max(1, hi - lo))));
          else {
            std::vector<float> run(hi - lo);
            for (int k = lo; k < hi; ++k) run[k - lo] = w[members[t][k]];
            auto near = [&](float v) { return mix_nearest(bits, v); };
            auto lvl = [&](uint32_t i) { return mix_level(bits, i); };
            sc[t][g] = polish_f16_scale(run.data(), hi - lo, fit_scale(run.data(), hi - lo, mix_max(bits), near, lvl, 4), near, lvl);
          }
          (void)ma;
        }
        s = sc[t][g];
      }
      for (int k = 0; k < len; ++k) {
        const float v = w[members[t][base + k]];
        if (bits == 16) bw.put(f32_to_f16(v), 16);
        else if (bits == 24 || bits == 32) {
          uint32_t u;
          memcpy(&u, &v, 4);
          bw.put(bits == 24 ? (u >> 8) : u, bits);
        } else bw.put(mix_nearest(bits, s == 0.0f ? 0.0f : v / s), bits);
      }
    }
  }
  uint8_t* sp = out + P.payload_bytes;
  for (int t = 0; t < 4; ++t)
    for (int g = 0; g < P.nsc[t]; ++g) { const uint16_t h = f32_to_f16(sc[t][g]); *sp++ = uint8_t(h & 0xFF); *sp++ = uint8_t(h >> 8); }
  return total;
}
void dec_mix(int fmt, const uint8_t* b, size_t size, int n, float* out) {
  MixTier cfg[4];
  bool grouped;
  mix_config(fmt, cfg, &grouped);
  const MixPlan P = mix_plan(fmt, n, cfg, grouped);
  if (size < P.payload_bytes + P.scale_bytes) return;
  std::vector<std::vector<float>> sc(4);
  const uint8_t* sp = b + P.payload_bytes;
  for (int t = 0; t < 4; ++t)
    for (int g = 0; g < P.nsc[t]; ++g, sp += 2) sc[t].push_back(f16_to_f32(uint16_t(sp[0] | (uint16_t(sp[1]) << 8))));
  BitReader br(b, P.payload_bytes);
  std::vector<std::vector<int>> members(4);
  for (int i = 0; i < n; ++i) members[br.get(2)].push_back(i);
  for (int t = 0; t < 4; ++t) {
    const int bits = cfg[t].bits;
    const int cnt = std::min(P.c[t], int(members[t].size()));
    for (int k = 0; k < cnt; ++k) {
      float v;
      if (bits == 16) v = f16_to_f32(uint16_t(br.get(16)));
      else if (bits == 24 || bits == 32) {
        const uint32_t u = bits == 24 ? (br.get(24) << 8) : br.get(32);
        memcpy(&v, &u, 4);
      } else {
        const float s = P.nsc[t] > 0 ? sc[t][std::min(k / 32, P.nsc[t] - 1)] : 1.0f;
        v = mix_level(bits, br.get(bits)) * s;
      }
      out[members[t][k]] = v;
    }
  }
}

enum Family { F_RAW32, F_Q24, F_Q16, F_LATTICE, F_Q1, F_G16, F_G24, F_FIXED, F_AFFINE, F_6S, F_C8, F_C12, F_MIX, F_OWN };
// Parameters of the grouped-affine wire of a format: element bits, group size, scale-code bits, offset-code bits and the
// bits-per-weight figure its header budget is checked against (which for a few formats differs from the registry's figure).
struct AffineSpec { int bits, gsz, scb, mb; double claimed; };

Family family_of(int fmt, int* bits_out, AffineSpec* aff = nullptr) {
  const FormatInfo& f = registry()[fmt];
  *bits_out = f.bits;
  AffineSpec a{f.bits, 32, 6, 6, f.bpw};
  Family fam = F_OWN;
  if (fmt == TFB_FMT_Q32) fam = F_RAW32;
  else if (f.mix) fam = F_MIX;
  else if (!f.grouped && !f.half) {
    if (f.bits == 24) fam = F_Q24;
    else if (f.bits == 16) fam = F_Q16;
    else if (f.bits == 8 || f.bits == 4 || f.bits == 2) fam = F_LATTICE;
    else if (f.bits == 1) fam = F_Q1;
    else fam = F_FIXED;                                          // 3, 6, 12 bit quantile codebooks and their K tiers
  } else if (f.bits == 1 && !f.half) fam = F_Q1;                 // Q_G_1 and its K tiers share the sign wire
  else if (f.bits == 16) fam = fmt == 44 ? F_G16 : F_Q16;        // only Q_G_16 / Q_G_24 carry the residual-mean tail
  else if (f.bits == 24) fam = fmt == 45 ? F_G24 : F_Q24;
  else if (f.bits == 12) fam = F_C12;                            // compound when the block is whole 32-groups, else fallback
  else if (f.bits == 8) { fam = F_C8; a = AffineSpec{8, 32, 6, 6, (f.tier && !f.half) ? 8.0 : 8.5}; }
  else if (f.bits == 6 && !f.half) fam = F_6S;
  else {
    fam = F_AFFINE;
    if (f.bits == 6) a = AffineSpec{6, 32, 8, 8, 6.5};
    else if (f.bits == 2) a = AffineSpec{2, 16, 4, 4, f.half ? 2.5 : (f.tier ? 2.4375 : 2.625)};
    else if (f.bits == 1) a = AffineSpec{1, 32, 6, 6, 1.5};
    else a = AffineSpec{f.bits, 32, 6, 6, f.half ? f.bits + 0.5 : (f.tier ? f.bits + 0.4375 : f.bits + 0.5)};
  }
  if (aff) *aff = a;
  return fam;
}

}  // namespace

// =================================================================================================
// C API
// =================================================================================================
TFB_EXPORT const char* tfb_format_name(int fmt) {
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT) return nullptr;
  return registry()[fmt].name.c_str();
}
TFB_EXPORT int tfb_format_parse(const char* name) {
  if (!name) return -1;
  std::string c = canon(name);
  // legacy spellings: QG8 -> Q_G_8, QGMX45 -> Q_G_MX_4_5, Q4KM -> Q_4_K_M
  for (int i = 0; i < TFB_FORMAT_COUNT; ++i)
    if (canon(registry()[i].name.c_str()) == c) return i;
  if (c == "FP32" || c == "F32" || c == "RAWFP32") return TFB_FMT_Q32;
  if (c == "FP16" || c == "F16") return 7;
  if (c == "TERNARY" || c == "Q15") return 73;
  return -1;
}
TFB_EXPORT double tfb_format_bpw(int fmt) { return (fmt < 0 || fmt >= TFB_FORMAT_COUNT) ? 0.0 : registry()[fmt].bpw; }
TFB_EXPORT int tfb_format_is_grouped(int fmt) { return (fmt < 0 || fmt >= TFB_FORMAT_COUNT) ? 0 : registry()[fmt].grouped; }
TFB_EXPORT int tfb_format_is_mix(int fmt) { return (fmt < 0 || fmt >= TFB_FORMAT_COUNT) ? 0 : registry()[fmt].mix; }
TFB_EXPORT int tfb_format_k_tier(int fmt) { return (fmt < 0 || fmt >= TFB_FORMAT_COUNT) ? 0 : registry()[fmt].tier; }
TFB_EXPORT int tfb_format_is_wire_exact(int fmt) {
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT) return 0;
  int bits;
  return family_of(fmt, &bits) != F_OWN;
}
static size_t formula_bytes(int fmt, uint32_t n) { return size_t(ceil(float(registry()[fmt].bpw) * float(n) / 8.0f)); }
static long encode_block(int fmt, const float* w, uint32_t n, uint8_t* out, size_t cap);

// Bytes an encoder of this library writes for a block of n weights.  The wire layouts of the grouped / half-step formats
// carry whole header bytes, so at ragged block sizes a stream can be a byte longer than bpw * n / 8: the layout, not the
// formula, is what a caller's buffer has to hold.  The length depends on (format, n) only; it is taken from a dry run on
// a zero block and remembered per thread.
static size_t stream_bytes(int fmt, uint32_t n) {
  static thread_local std::vector<std::pair<uint64_t, size_t>> memo;
  const uint64_t key = (uint64_t(uint32_t(fmt)) << 32) | n;
  for (const auto& kv : memo)
    if (kv.first == key) return kv.second;
  std::vector<float> zeros(n, 0.0f);
  std::vector<uint8_t> scratch(size_t(n) * 4 + 64);
  const long got = encode_block(fmt, zeros.data(), n, scratch.data(), scratch.size());
  const size_t len = got > 0 ? size_t(got) : formula_bytes(fmt, n);
  if (memo.size() >= 256) memo.clear();
  memo.emplace_back(key, len);
  return len;
}

TFB_EXPORT size_t tfb_block_claimed_bytes(int fmt, uint32_t n) {
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT) return 0;
  const size_t f = formula_bytes(fmt, n);
  if (n == 0 || n > (1u << 20)) return f;
  return std::max(f, stream_bytes(fmt, n));
}

// Encodes into `out` when the stream fits into `cap` bytes; the encoders themselves always work in a scratch buffer with
// room for any layout (4 bytes per weight + headers), so a short `cap` is an error return, never an overrun.
TFB_EXPORT long tfb_quantize_block(int fmt, const float* w, uint32_t n, uint8_t* out, size_t cap) {
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT || !w || !out || n == 0) return -1;
  static thread_local std::vector<uint8_t> scratch;
  const size_t room = size_t(n) * 4 + 64;
  if (scratch.size() < room) scratch.resize(room);
  const long got = encode_block(fmt, w, n, scratch.data(), room);
  if (got < 0 || size_t(got) > cap) return -1;
  memcpy(out, scratch.data(), size_t(got));
  if (size_t(got) < cap) memset(out + got, 0, cap - size_t(got));   // the rest of the caller's buffer reads as zeros, as before
  return got;
}

static long encode_block(int fmt, const float* w, uint32_t n, uint8_t* out, size_t cap) {
  int bits;
  const Family fam = family_of(fmt, &bits);
  const FormatInfo& f = registry()[fmt];
  size_t need = formula_bytes(fmt, n);
  if (fam == F_Q16) need = std::max(need, size_t(n) * 2);
  if (fam == F_Q1) need = std::max(need, size_t(n + 7) / 8);
  if (cap < need) return -1;
  memset(out, 0, cap);
  const int iters = 2 + f.tier;  // K tiers spend more refinement passes on the same wire
  AffineSpec a;
  family_of(fmt, &bits, &a);
  switch (fam) {
    // families whose stream length follows from the wire layout (it may differ from the claimed figure by a few bytes)
    case F_FIXED: enc_fixed(bits, w, int(n), out, need, f.tier); break;
    case F_AFFINE: return long(enc_affine(a.bits, w, int(n), a.gsz, a.scb, a.mb, a.claimed, out, cap));
    case F_6S: return long(enc_6s(w, int(n), out, cap));
    case F_C8:
      if (compound_fits(8, int(n))) return long(enc_compound8(w, int(n), out, cap));
      return long(enc_affine(8, w, int(n), a.gsz, a.scb, a.mb, a.claimed, out, cap));
    case F_C12:
      if (compound_fits(12, int(n))) return long(enc_compound12(w, int(n), out, cap, f.tier));
      if (f.grouped && !f.half && !f.tier) return long(enc_small_groups(12, w, int(n), 12.5, out, cap));
      need = (size_t(ceil(12.0 * double(n))) + 7) / 8;
      enc_fixed(12, w, int(n), out, need, f.tier);
      break;
    case F_MIX: return long(enc_mix(fmt, w, int(n), out, cap));
    case F_RAW32: memcpy(out, w, size_t(n) * 4); break;
    case F_Q24: enc_q24(w, n, out); break;
    case F_Q16: enc_q16(w, n, out); break;
    case F_LATTICE: enc_lattice(w, n, bits, out, need, iters); break;
    case F_Q1: enc_q1(w, n, out, need); break;
    case F_G16:
    case F_G24: {
      const size_t plain = size_t(n) * (fam == F_G16 ? 2 : 3);
      if (fam == F_G16) enc_q16(w, n, out); else enc_q24(w, n, out);
      if (need > plain && n % 32 == 0) {
        std::vector<float> dec(n);
        if (fam == F_G16) dec_q16(out, plain, n, dec.data()); else dec_q24(out, plain, n, dec.data());
        enc_mean_tail(w, dec.data(), n, out + plain);
      }
      break;
    }
    case F_OWN: enc_own(w, n, bits, f.bpw, out, need); break;
  }
  return long(need);
}

TFB_EXPORT void tfb_dequantize_block(int fmt, const uint8_t* idx, size_t idx_bytes, const uint8_t* cb, size_t cb_bytes,
                                     uint32_t nw, float* out) {
  (void)cb; (void)cb_bytes;
  if (!out || nw == 0) return;
  std::fill(out, out + nw, 0.0f);
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT || !idx) return;
  const int n = int(std::min<uint32_t>(nw, 1u << 24));
  int bits;
  const Family fam = family_of(fmt, &bits);
  const FormatInfo& f = registry()[fmt];
  AffineSpec a;
  family_of(fmt, &bits, &a);
  switch (fam) {
    case F_FIXED: dec_fixed(bits, idx, idx_bytes, n, out); break;
    case F_AFFINE: dec_affine(a.bits, idx, idx_bytes, n, a.gsz, a.scb, a.mb, a.claimed, out); break;
    case F_6S: dec_6s(idx, idx_bytes, n, out); break;
    case F_C8:
      if (compound_fits(8, n)) dec_compound8(idx, idx_bytes, n, out);
      else dec_affine(8, idx, idx_bytes, n, a.gsz, a.scb, a.mb, a.claimed, out);
      break;
    case F_C12:
      if (compound_fits(12, n)) dec_compound12(idx, idx_bytes, n, out);
      else if (f.grouped && !f.half && !f.tier) dec_small_groups(12, idx, idx_bytes, n, out);
      else dec_fixed(12, idx, idx_bytes, n, out);
      break;
    case F_MIX: dec_mix(fmt, idx, idx_bytes, n, out); break;
    case F_RAW32: if (idx_bytes >= size_t(n) * 4) memcpy(out, idx, size_t(n) * 4); break;
    case F_Q24: dec_q24(idx, idx_bytes, n, out); break;
    case F_Q16: dec_q16(idx, idx_bytes, n, out); break;
    case F_LATTICE: dec_lattice(idx, idx_bytes, n, bits, out); break;
    case F_Q1: dec_q1(idx, idx_bytes, n, out); break;
    case F_G16:
    case F_G24: {
      const size_t plain = size_t(n) * (fam == F_G16 ? 2 : 3);
      const size_t claimed = formula_bytes(fmt, n);
      const bool tail = n % 32 == 0 && idx_bytes >= claimed && claimed > plain;
      if (fam == F_G16) dec_q16(idx, tail ? plain : idx_bytes, n, out); else dec_q24(idx, tail ? plain : idx_bytes, n, out);
      if (tail) dec_mean_tail(idx + plain, n, out);
      break;
    }
    case F_OWN: dec_own(idx, idx_bytes, n, bits, f.bpw, out); break;
  }
}
