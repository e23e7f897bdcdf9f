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

enum Family { F_RAW32, F_Q24, F_Q16, F_LATTICE, F_Q1, F_G16, F_G24, F_OWN };
Family family_of(int fmt, int* bits_out) {
  const FormatInfo& f = registry()[fmt];
  *bits_out = f.bits;
  if (fmt == TFB_FMT_Q32) return F_RAW32;
  if (f.mix) return F_OWN;
  if (!f.grouped && !f.half) {
    if (f.bits == 24) return F_Q24;
    if (f.bits == 16) return F_Q16;
    if (f.bits == 8 || f.bits == 4 || f.bits == 2) return F_LATTICE;
    if (f.bits == 1) return F_Q1;
    return F_OWN;
  }
  if (f.bits == 1 && !f.half) return F_Q1;           // Q_G_1 and its K tiers share the sign wire
  if (f.bits == 16) return fmt == 44 ? F_G16 : F_Q16;  // only Q_G_16 / Q_G_24 carry the residual-mean tail
  if (f.bits == 24) return fmt == 45 ? F_G24 : F_Q24;
  return F_OWN;
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
TFB_EXPORT size_t tfb_block_claimed_bytes(int fmt, uint32_t n) {
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT) return 0;
  return size_t(ceil(float(registry()[fmt].bpw) * float(n) / 8.0f));
}

TFB_EXPORT long tfb_quantize_block(int fmt, const float* w, uint32_t n, uint8_t* out, size_t cap) {
  if (fmt < 0 || fmt >= TFB_FORMAT_COUNT || !w || !out || n == 0) return -1;
  int bits;
  const Family fam = family_of(fmt, &bits);
  const FormatInfo& f = registry()[fmt];
  size_t need = tfb_block_claimed_bytes(fmt, n);
  if (fam == F_Q16) need = std::max(need, size_t(n) * 2);
  if (fam == F_Q1) need = std::max(need, size_t(n + 7) / 8);
  if (cap < need) return -1;
  memset(out, 0, need);
  const int iters = 2 + f.tier;  // K tiers spend more refinement passes on the same wire
  switch (fam) {
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
  switch (fam) {
    case F_RAW32: if (idx_bytes >= size_t(n) * 4) memcpy(out, idx, size_t(n) * 4); break;
    case F_Q24: dec_q24(idx, idx_bytes, n, out); break;
    case F_Q16: dec_q16(idx, idx_bytes, n, out); break;
    case F_LATTICE: dec_lattice(idx, idx_bytes, n, bits, out); break;
    case F_Q1: dec_q1(idx, idx_bytes, n, out); break;
    case F_G16:
    case F_G24: {
      const size_t plain = size_t(n) * (fam == F_G16 ? 2 : 3);
      const size_t claimed = tfb_block_claimed_bytes(fmt, n);
      const bool tail = n % 32 == 0 && idx_bytes >= claimed && claimed > plain;
      if (fam == F_G16) dec_q16(idx, tail ? plain : idx_bytes, n, out); else dec_q24(idx, tail ? plain : idx_bytes, n, out);
      if (tail) dec_mean_tail(idx + plain, n, out);
      break;
    }
    case F_OWN: dec_own(idx, idx_bytes, n, bits, f.bpw, out); break;
  }
}
