// libtfb_tokenizer: byte-pair (trainable), unigram (Viterbi / EM, SentencePiece TSV interchange) and
// byte-level BPE driven by a Hugging Face vocab.json + merges.txt (Qwen-style, with the ChatML
// template).  C ABI for the Python binding and the native tools.
//
// Parity: Tokenizer interface {encode, decode, vocab_size, bos_id = 1, eos_id = 2} and BPETokenizer
// train / save / load (reference include/quant/tokenizer.h:10-57), UnigramTokenizer incl. U+2581
// handling (include/quant/bpe_tokenizer.h:17-94), Qwen35Tokenizer (include/quant/qwen35_tokenizer.h:16-53).
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <fstream>
#include <map>
#include <queue>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#define TFB_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct PairHash {
  size_t operator()(const std::pair<int, int>& p) const { return (size_t(uint32_t(p.first)) << 32) ^ uint32_t(p.second); }
};

std::string hex_escape(const std::string& s) {
  static const char* hx = "0123456789abcdef";
  std::string o;
  for (unsigned char c : s) { o.push_back(hx[c >> 4]); o.push_back(hx[c & 15]); }
  return o;
}
std::string hex_unescape(const std::string& s) {
  std::string o;
  auto v = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
  for (size_t i = 0; i + 1 < s.size(); i += 2) o.push_back(char(v(s[i]) << 4 | v(s[i + 1])));
  return o;
}

// split into words: a run of spaces attaches to the following word (GPT-2 style " word")
std::vector<std::string> pretokenize(const std::string& text) {
  std::vector<std::string> out;
  size_t i = 0;
  const size_t n = text.size();
  auto cls = [](unsigned char c) {
    if (c == ' ') return 0;
    if (c == '\n' || c == '\t' || c == '\r') return 1;
    if ((c >= '0' && c <= '9')) return 2;
    if ((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c >= 128 || c == '\'' ) return 3;
    return 4;
  };
  while (i < n) {
    size_t j = i;
    std::string w;
    if (text[j] == ' ' && j + 1 < n && cls(text[j + 1]) >= 2) { w.push_back(' '); ++j; }
    const int c = cls(text[j]);
    size_t k = j;
    while (k < n && cls(text[k]) == c && (c != 4 || k == j) && (c != 2 || k - j < 3)) ++k;
    if (k == j) k = j + 1;
    w.append(text, j, k - j);
    out.push_back(w);
    i = k;
  }
  return out;
}

// ------------------------------------------------------------------------------------------------
// BPE over bytes
// ------------------------------------------------------------------------------------------------
struct Bpe {
  std::vector<std::string> vocab;  // id -> bytes
  std::unordered_map<std::pair<int, int>, int, PairHash> merges;  // pair -> merged id (rank = id)
  std::unordered_map<std::string, int> special;
  int unk = 0, bos = 1, eos = 2;
  static const int kBase = 3;  // specials before the 256 byte tokens

  Bpe() { reset(); }
  void reset() {
    vocab.clear();
    merges.clear();
    vocab = {"<unk>", "<s>", "</s>"};
    for (int b = 0; b < 256; ++b) vocab.push_back(std::string(1, char(b)));
  }
  void train(const std::string& text, int target) {
    reset();
    std::unordered_map<std::string, long long> wf;
    for (auto& w : pretokenize(text)) ++wf[w];
    std::vector<std::vector<int>> words;
    std::vector<long long> freq;
    for (auto& kv : wf) {
      std::vector<int> ids;
      for (unsigned char c : kv.first) ids.push_back(kBase + c);
      words.push_back(ids);
      freq.push_back(kv.second);
    }
    while (int(vocab.size()) < target) {
      std::unordered_map<std::pair<int, int>, long long, PairHash> cnt;
      for (size_t w = 0; w < words.size(); ++w)
        for (size_t i = 0; i + 1 < words[w].size(); ++i) cnt[{words[w][i], words[w][i + 1]}] += freq[w];
      std::pair<int, int> best{-1, -1};
      long long bc = 1;
      for (auto& kv : cnt)
        if (kv.second > bc || (kv.second == bc && best.first >= 0 && kv.first < best)) { bc = kv.second; best = kv.first; }
      if (best.first < 0) break;
      const int id = int(vocab.size());
      vocab.push_back(vocab[best.first] + vocab[best.second]);
      merges[best] = id;
      for (auto& w : words) {
        std::vector<int> o;
        for (size_t i = 0; i < w.size(); ++i) {
          if (i + 1 < w.size() && w[i] == best.first && w[i + 1] == best.second) { o.push_back(id); ++i; }
          else o.push_back(w[i]);
        }
        w.swap(o);
      }
    }
  }
  void encode_word(const std::string& w, std::vector<int>& out) const {
    std::vector<int> ids;
    for (unsigned char c : w) ids.push_back(kBase + c);
    while (ids.size() > 1) {
      int best_rank = INT32_MAX, best_i = -1;
      for (size_t i = 0; i + 1 < ids.size(); ++i) {
        auto it = merges.find({ids[i], ids[i + 1]});
        if (it != merges.end() && it->second < best_rank) { best_rank = it->second; best_i = int(i); }
      }
      if (best_i < 0) break;
      ids[best_i] = best_rank;
      ids.erase(ids.begin() + best_i + 1);
    }
    out.insert(out.end(), ids.begin(), ids.end());
  }
  std::vector<int> encode(const std::string& text) const {
    std::vector<int> out;
    for (auto& w : pretokenize(text)) encode_word(w, out);
    return out;
  }
  std::string decode(const int* ids, int n) const {
    std::string o;
    for (int i = 0; i < n; ++i)
      if (ids[i] >= kBase && ids[i] < int(vocab.size())) o += vocab[ids[i]];
    return o;
  }
  bool save(const char* path) const {
    std::ofstream f(path);
    if (!f) return false;
    f << "TFBBPE1 " << vocab.size() << " " << merges.size() << "\n";
    std::vector<std::pair<int, std::pair<int, int>>> m;
    for (auto& kv : merges) m.push_back({kv.second, kv.first});
    std::sort(m.begin(), m.end());
    for (auto& e : m) f << e.second.first << " " << e.second.second << "\n";
    return bool(f);
  }
  bool load(const char* path) {
    std::ifstream f(path);
    std::string magic;
    size_t nv, nm;
    if (!(f >> magic >> nv >> nm) || magic != "TFBBPE1") return false;
    reset();
    for (size_t i = 0; i < nm; ++i) {
      int a, b;
      if (!(f >> a >> b) || a < 0 || b < 0 || a >= int(vocab.size()) || b >= int(vocab.size())) return false;
      merges[{a, b}] = int(vocab.size());
      vocab.push_back(vocab[a] + vocab[b]);
    }
    return vocab.size() == nv;
  }
};

// ------------------------------------------------------------------------------------------------
// Unigram (Viterbi segmentation over UTF-8 pieces; U+2581 marks word starts)
// ------------------------------------------------------------------------------------------------
const char kMark[] = "\xE2\x96\x81";
size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1; }

struct Unigram {
  std::vector<std::string> pieces;
  std::vector<double> logp;
  std::unordered_map<std::string, int> index;
  int unk = 0, bos = 1, eos = 2;
  size_t max_len = 1;

  void rebuild() {
    index.clear();
    max_len = 1;
    for (size_t i = 0; i < pieces.size(); ++i) { index[pieces[i]] = int(i); max_len = std::max(max_len, pieces[i].size()); }
  }
  static std::string normalize(const std::string& t) {
    std::string o = kMark;
    bool prev_space = true;
    for (char c : t) {
      if (c == ' ' || c == '\t' || c == '\n' || c == '\r') { if (!prev_space) o += kMark; prev_space = true; }
      else { o.push_back(c); prev_space = false; }
    }
    if (prev_space && o.size() >= 3) o.resize(o.size() - 3);
    return o;
  }
  std::vector<int> viterbi(const std::string& s, std::vector<double>* lp = nullptr) const {
    const size_t n = s.size();
    std::vector<double> best(n + 1, -1e300);
    std::vector<int> back(n + 1, -1), piece(n + 1, -1);
    best[0] = 0;
    for (size_t i = 0; i < n; ++i) {
      if (best[i] <= -1e299) continue;
      if ((s[i] & 0xC0) == 0x80) continue;  // only start pieces on character boundaries
      const size_t cl = utf8_len((unsigned char)s[i]);
      bool any = false;
      for (size_t l = cl; l <= max_len && i + l <= n; ++l) {
        if (i + l < n && (s[i + l] & 0xC0) == 0x80) continue;
        auto it = index.find(s.substr(i, l));
        if (it == index.end()) continue;
        any = true;
        const double sc = best[i] + logp[it->second];
        if (sc > best[i + l]) { best[i + l] = sc; back[i + l] = int(i); piece[i + l] = it->second; }
      }
      if (!any || best[i + cl] <= -1e299) {  // unknown character
        const double sc = best[i] - 20.0;
        if (i + cl <= n && sc > best[i + cl]) { best[i + cl] = sc; back[i + cl] = int(i); piece[i + cl] = unk; }
      }
    }
    std::vector<int> out;
    for (int p = int(n); p > 0 && back[p] >= 0; p = back[p]) {
      out.push_back(piece[p]);
      if (lp) lp->push_back(piece[p] == unk ? -20.0 : logp[piece[p]]);
    }
    std::reverse(out.begin(), out.end());
    if (lp) std::reverse(lp->begin(), lp->end());
    return out;
  }
  void train(const std::string& text, int target) {
    const std::string norm = normalize(text);
    // seed: all substrings up to 8 characters that occur at least twice, plus every single character
    std::unordered_map<std::string, long long> cnt;
    std::vector<size_t> starts;
    for (size_t i = 0; i < norm.size(); i += utf8_len((unsigned char)norm[i])) starts.push_back(i);
    starts.push_back(norm.size());
    for (size_t a = 0; a + 1 < starts.size(); ++a)
      for (size_t b = a + 1; b < starts.size() && b - a <= 8; ++b) {
        if (b - a > 1 && norm.compare(starts[b - 1], 3, kMark) == 0) break;  // pieces do not span word starts
        ++cnt[norm.substr(starts[a], starts[b] - starts[a])];
      }
    std::vector<std::pair<double, std::string>> cand;
    for (auto& kv : cnt) {
      const size_t chars = std::count_if(kv.first.begin(), kv.first.end(), [](char c) { return (c & 0xC0) != 0x80; });
      if (chars == 1 || kv.second >= 2) cand.push_back({double(kv.second) * double(chars), kv.first});
    }
    std::sort(cand.rbegin(), cand.rend());
    pieces = {"<unk>", "<s>", "</s>"};
    logp = {-20, -20, -20};
    std::vector<long long> freq = {1, 1, 1};
    const size_t seed = std::min(cand.size(), size_t(std::max(target * 4, 64)));
    for (size_t i = 0; i < cand.size(); ++i) {
      const size_t chars = std::count_if(cand[i].second.begin(), cand[i].second.end(), [](char c) { return (c & 0xC0) != 0x80; });
      if (i < seed || chars == 1) { pieces.push_back(cand[i].second); freq.push_back(cnt[cand[i].second]); }
    }
    auto set_probs = [&](const std::vector<double>& f) {
      double tot = 0;
      for (double x : f) tot += x;
      logp.resize(pieces.size());
      for (size_t i = 0; i < pieces.size(); ++i) logp[i] = log(std::max(f[i], 0.5) / tot);
    };
    set_probs(std::vector<double>(freq.begin(), freq.end()));
    rebuild();
    // hard-EM rounds: segment, recount, drop the least used multi-character pieces until the target size
    for (int round = 0; round < 8; ++round) {
      std::vector<double> used(pieces.size(), 0.0);
      size_t pos = 0;
      while (pos < norm.size()) {
        size_t end = norm.find(kMark, pos + 3);
        if (end == std::string::npos) end = norm.size();
        for (int id : viterbi(norm.substr(pos, end - pos))) used[id] += 1;
        pos = end;
      }
      if (int(pieces.size()) > target) {
        std::vector<std::pair<double, int>> order;
        for (size_t i = 3; i < pieces.size(); ++i) {
          const size_t chars = std::count_if(pieces[i].begin(), pieces[i].end(), [](char c) { return (c & 0xC0) != 0x80; });
          if (chars > 1) order.push_back({used[i], int(i)});
        }
        std::sort(order.begin(), order.end());
        const size_t drop = std::min(order.size(), std::max<size_t>((pieces.size() - target + 1) / 2, pieces.size() - target > 16 ? 0 : pieces.size() - target));
        std::vector<char> dead(pieces.size(), 0);
        for (size_t i = 0; i < drop; ++i) dead[order[i].second] = 1;
        std::vector<std::string> np;
        std::vector<double> nu;
        for (size_t i = 0; i < pieces.size(); ++i)
          if (!dead[i]) { np.push_back(pieces[i]); nu.push_back(used[i]); }
        pieces.swap(np);
        used.swap(nu);
      }
      set_probs(used);
      rebuild();
    }
  }
  bool save_tsv(const char* path) const {
    std::ofstream f(path);
    if (!f) return false;
    for (size_t i = 0; i < pieces.size(); ++i) f << pieces[i] << "\t" << logp[i] << "\n";
    return bool(f);
  }
  bool load_tsv(const char* path) {
    std::ifstream f(path);
    if (!f) return false;
    pieces.clear();
    logp.clear();
    std::string line;
    while (std::getline(f, line)) {
      const size_t tab = line.rfind('\t');
      if (tab == std::string::npos) continue;
      pieces.push_back(line.substr(0, tab));
      logp.push_back(atof(line.c_str() + tab + 1));
    }
    rebuild();
    return !pieces.empty();
  }
  std::string decode(const int* ids, int n) const {
    std::string o;
    for (int i = 0; i < n; ++i)
      if (ids[i] > 2 && ids[i] < int(pieces.size())) o += pieces[ids[i]];
    std::string r;
    for (size_t i = 0; i < o.size();) {
      if (o.compare(i, 3, kMark) == 0) { if (!r.empty()) r.push_back(' '); i += 3; }
      else r.push_back(o[i++]);
    }
    return r;
  }
};

// ------------------------------------------------------------------------------------------------
// byte-level BPE from vocab.json + merges.txt
// ------------------------------------------------------------------------------------------------
struct HfBpe {
  std::unordered_map<std::string, int> tok2id;
  std::vector<std::string> id2tok;
  std::unordered_map<std::string, int> rank;  // "a b" -> rank
  std::vector<std::pair<std::string, int>> specials;
  std::string byte_enc[256];
  std::unordered_map<std::string, unsigned char> byte_dec;
  int bos = -1, eos = -1;

  HfBpe() {
    // GPT-2 printable-byte alphabet
    std::vector<int> bs, cs;
    for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
    for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
    for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
    cs = bs;
    int n = 0;
    for (int b = 0; b < 256; ++b)
      if (std::find(bs.begin(), bs.end(), b) == bs.end()) { bs.push_back(b); cs.push_back(256 + n++); }
    for (size_t i = 0; i < bs.size(); ++i) {
      const int cp = cs[i];
      std::string u;
      if (cp < 0x80) u.push_back(char(cp));
      else { u.push_back(char(0xC0 | (cp >> 6))); u.push_back(char(0x80 | (cp & 0x3F))); }
      byte_enc[bs[i]] = u;
      byte_dec[u] = (unsigned char)bs[i];
    }
  }
  static bool parse_json_string(const std::string& s, size_t& i, std::string& out) {
    if (s[i] != '"') return false;
    ++i;
    out.clear();
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) {
        const char c = s[++i];
        if (c == 'n') out.push_back('\n');
        else if (c == 't') out.push_back('\t');
        else if (c == 'r') out.push_back('\r');
        else if (c == 'b') out.push_back('\b');
        else if (c == 'f') out.push_back('\f');
        else if (c == 'u' && i + 4 < s.size()) {
          int cp = int(strtol(s.substr(i + 1, 4).c_str(), nullptr, 16));
          i += 4;
          if (cp < 0x80) out.push_back(char(cp));
          else if (cp < 0x800) { out.push_back(char(0xC0 | (cp >> 6))); out.push_back(char(0x80 | (cp & 0x3F))); }
          else { out.push_back(char(0xE0 | (cp >> 12))); out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F))); }
        } else out.push_back(c);
        ++i;
      } else out.push_back(s[i++]);
    }
    ++i;
    return true;
  }
  bool load(const std::string& dir) {
    std::ifstream vf(dir + "/vocab.json");
    if (!vf) return false;
    std::stringstream ss;
    ss << vf.rdbuf();
    const std::string s = ss.str();
    size_t i = s.find('{');
    if (i == std::string::npos) return false;
    ++i;
    while (i < s.size()) {
      while (i < s.size() && s[i] != '"' && s[i] != '}') ++i;
      if (i >= s.size() || s[i] == '}') break;
      std::string key;
      if (!parse_json_string(s, i, key)) return false;
      while (i < s.size() && (s[i] == ':' || s[i] == ' ')) ++i;
      const int id = atoi(s.c_str() + i);
      while (i < s.size() && s[i] != ',' && s[i] != '}') ++i;
      tok2id[key] = id;
      if (id >= int(id2tok.size())) id2tok.resize(id + 1);
      id2tok[id] = key;
    }
    std::ifstream mf(dir + "/merges.txt");
    std::string line;
    int r = 0;
    while (mf && std::getline(mf, line)) {
      if (line.empty() || line[0] == '#') continue;
      rank[line] = r++;
    }
    for (const char* sp : {"<|endoftext|>", "<|im_start|>", "<|im_end|>"}) add_special(sp);
    auto it = tok2id.find("<|endoftext|>");
    if (it != tok2id.end()) eos = it->second;
    return !tok2id.empty();
  }
  void add_special(const std::string& t) {
    auto it = tok2id.find(t);
    int id;
    if (it == tok2id.end()) { id = int(id2tok.size()); tok2id[t] = id; id2tok.push_back(t); }
    else id = it->second;
    specials.push_back({t, id});
  }
  void encode_piece(const std::string& piece, std::vector<int>& out) const {
    std::vector<std::string> syms;
    for (unsigned char c : piece) syms.push_back(byte_enc[c]);
    while (syms.size() > 1) {
      int best = INT32_MAX, bi = -1;
      for (size_t i = 0; i + 1 < syms.size(); ++i) {
        auto it = rank.find(syms[i] + " " + syms[i + 1]);
        if (it != rank.end() && it->second < best) { best = it->second; bi = int(i); }
      }
      if (bi < 0) break;
      syms[bi] += syms[bi + 1];
      syms.erase(syms.begin() + bi + 1);
    }
    for (auto& sy : syms) {
      auto it = tok2id.find(sy);
      if (it != tok2id.end()) out.push_back(it->second);
    }
  }
  std::vector<int> encode(const std::string& text) const {
    std::vector<int> out;
    size_t pos = 0;
    while (pos < text.size()) {
      size_t next = std::string::npos;
      int sid = -1;
      size_t slen = 0;
      for (auto& sp : specials) {
        const size_t f = text.find(sp.first, pos);
        if (f != std::string::npos && f < next) { next = f; sid = sp.second; slen = sp.first.size(); }
      }
      const std::string chunk = text.substr(pos, next == std::string::npos ? std::string::npos : next - pos);
      for (auto& w : pretokenize(chunk)) encode_piece(w, out);
      if (next == std::string::npos) break;
      out.push_back(sid);
      pos = next + slen;
    }
    return out;
  }
  std::string decode(const int* ids, int n) const {
    std::string o;
    for (int i = 0; i < n; ++i) {
      if (ids[i] < 0 || ids[i] >= int(id2tok.size())) continue;
      const std::string& t = id2tok[ids[i]];
      bool special = false;
      for (auto& sp : specials) special |= sp.second == ids[i];
      if (special) { o += t; continue; }
      for (size_t k = 0; k < t.size();) {
        const size_t l = utf8_len((unsigned char)t[k]);
        auto it = byte_dec.find(t.substr(k, l));
        if (it != byte_dec.end()) o.push_back(char(it->second));
        k += l;
      }
    }
    return o;
  }
};

struct Tok {
  int kind;  // 0 bpe, 1 unigram, 2 hf byte-level bpe
  Bpe bpe;
  Unigram uni;
  HfBpe hf;
  std::string scratch;
};

}  // namespace

TFB_EXPORT void* tfb_tok_new(int kind) {
  Tok* t = new Tok();
  t->kind = kind;
  if (kind == 1) { t->uni.pieces = {"<unk>", "<s>", "</s>"}; t->uni.logp = {-20, -20, -20}; t->uni.rebuild(); }
  return t;
}
TFB_EXPORT void tfb_tok_free(void* h) { delete static_cast<Tok*>(h); }
TFB_EXPORT int tfb_tok_train(void* h, const char* text, long long n, int vocab_size) {
  Tok* t = static_cast<Tok*>(h);
  const std::string s(text, size_t(n));
  if (t->kind == 0) t->bpe.train(s, vocab_size);
  else if (t->kind == 1) t->uni.train(s, vocab_size);
  else return -1;
  return 0;
}
TFB_EXPORT int tfb_tok_vocab_size(void* h) {
  Tok* t = static_cast<Tok*>(h);
  return t->kind == 0 ? int(t->bpe.vocab.size()) : t->kind == 1 ? int(t->uni.pieces.size()) : int(t->hf.id2tok.size());
}
TFB_EXPORT int tfb_tok_bos(void* h) { Tok* t = static_cast<Tok*>(h); return t->kind == 2 ? t->hf.bos : 1; }
TFB_EXPORT int tfb_tok_eos(void* h) { Tok* t = static_cast<Tok*>(h); return t->kind == 2 ? t->hf.eos : 2; }
// returns the number of ids; writes at most cap of them
TFB_EXPORT long long tfb_tok_encode(void* h, const char* text, long long n, int* out, long long cap) {
  Tok* t = static_cast<Tok*>(h);
  const std::string s(text, size_t(n));
  std::vector<int> ids = t->kind == 0 ? t->bpe.encode(s) : t->kind == 1 ? t->uni.viterbi(Unigram::normalize(s)) : t->hf.encode(s);
  for (long long i = 0; i < (long long)ids.size() && i < cap; ++i) out[i] = ids[i];
  return (long long)ids.size();
}
// returns the byte length of the decoded text; writes at most cap bytes
TFB_EXPORT long long tfb_tok_decode(void* h, const int* ids, int n, char* out, long long cap) {
  Tok* t = static_cast<Tok*>(h);
  const std::string s = t->kind == 0 ? t->bpe.decode(ids, n) : t->kind == 1 ? t->uni.decode(ids, n) : t->hf.decode(ids, n);
  memcpy(out, s.data(), size_t(std::min<long long>(cap, (long long)s.size())));
  return (long long)s.size();
}
TFB_EXPORT int tfb_tok_save(void* h, const char* path) {
  Tok* t = static_cast<Tok*>(h);
  if (t->kind == 0) return t->bpe.save(path) ? 0 : -1;
  if (t->kind == 1) return t->uni.save_tsv(path) ? 0 : -1;
  return -1;
}
TFB_EXPORT int tfb_tok_load(void* h, const char* path) {
  Tok* t = static_cast<Tok*>(h);
  if (t->kind == 0) return t->bpe.load(path) ? 0 : -1;
  if (t->kind == 1) return t->uni.load_tsv(path) ? 0 : -1;
  return t->hf.load(path) ? 0 : -1;
}
// Text of piece `id` (Unigram pieces / BPE vocabulary / byte-level BPE tokens); returns its byte length or -1.
TFB_EXPORT long long tfb_tok_id_to_token(void* h, int id, char* out, long long cap) {
  Tok* t = static_cast<Tok*>(h);
  const std::vector<std::string>& v = t->kind == 0 ? t->bpe.vocab : t->kind == 1 ? t->uni.pieces : t->hf.id2tok;
  if (id < 0 || size_t(id) >= v.size()) return -1;
  memcpy(out, v[size_t(id)].data(), size_t(std::min<long long>(cap, (long long)v[size_t(id)].size())));
  return (long long)v[size_t(id)].size();
}
// Log-probability of a Unigram piece (0 for the other kinds).
TFB_EXPORT double tfb_tok_piece_score(void* h, int id) {
  Tok* t = static_cast<Tok*>(h);
  return (t->kind == 1 && id >= 0 && size_t(id) < t->uni.logp.size()) ? t->uni.logp[size_t(id)] : 0.0;
}
// Unigram special ids: which = 0 unknown, 1 begin, 2 end.
TFB_EXPORT void tfb_tok_set_special(void* h, int which, int id) {
  Tok* t = static_cast<Tok*>(h);
  if (t->kind != 1) return;
  (which == 0 ? t->uni.unk : which == 1 ? t->uni.bos : t->uni.eos) = id;
}
// Encode with the per-piece log-probabilities of the best segmentation (Unigram only; others get zeros).
TFB_EXPORT long long tfb_tok_encode_scores(void* h, const char* text, long long n, int* out, double* scores, long long cap) {
  Tok* t = static_cast<Tok*>(h);
  if (t->kind != 1) return -1;
  std::vector<double> lp;
  const std::vector<int> ids = t->uni.viterbi(Unigram::normalize(std::string(text, size_t(n))), &lp);
  for (long long i = 0; i < (long long)ids.size() && i < cap; ++i) { out[i] = ids[size_t(i)]; scores[i] = lp[size_t(i)]; }
  return (long long)ids.size();
}
// 1 when `id` is one of the byte-level tokenizer's added special tokens.
TFB_EXPORT int tfb_tok_is_special(void* h, int id) {
  Tok* t = static_cast<Tok*>(h);
  if (t->kind != 2) return id >= 0 && id <= 2;
  for (const auto& sp : t->hf.specials) if (sp.second == id) return 1;
  return 0;
}
TFB_EXPORT int tfb_tok_token_to_id(void* h, const char* tok) {
  Tok* t = static_cast<Tok*>(h);
  if (t->kind == 2) { auto it = t->hf.tok2id.find(tok); return it == t->hf.tok2id.end() ? -1 : it->second; }
  if (t->kind == 1) { auto it = t->uni.index.find(tok); return it == t->uni.index.end() ? -1 : it->second; }
  for (size_t i = 0; i < t->bpe.vocab.size(); ++i) if (t->bpe.vocab[i] == tok) return int(i);
  return -1;
}
